"""Optional bridge to PyKEEN interaction models (``--model Pykeen_<Name>``).

PyKEEN is not a dependency; the wrapper resolves the model class lazily and raises a clear error when the
package is missing (reference ``dicee/models/pykeen_models.py:8-138``).  The wrapped module lives under the
``model.`` prefix of the state dict, like in the reference.
"""
from __future__ import annotations

import torch

from .base import BaseKGE


class PykeenKGE(BaseKGE):
    def __init__(self, args: dict):
        super().__init__(args)
        try:
            from pykeen.models import model_resolver
            from pykeen.triples.triples_factory import CoreTriplesFactory
        except ModuleNotFoundError as e:
            raise ModuleNotFoundError("Pykeen_* models need the optional 'pykeen' package") from e
        kw = dict(self.args.get("pykeen_model_kwargs") or {})
        kw.setdefault("embedding_dim", self.embedding_dim)
        name = self.args["model"].split("_", 1)[1]
        if name in ("QuatE",):
            kw["embedding_dim"] = max(1, self.embedding_dim // 4)
        elif name in ("ComplEx", "RotatE"):
            kw["embedding_dim"] = max(1, self.embedding_dim // 2)
        self.name = self.args["model"]
        factory = CoreTriplesFactory(mapped_triples=torch.zeros(1, 3, dtype=torch.long),
                                     num_entities=self.num_entities, num_relations=self.num_relations,
                                     create_inverse_triples=False)
        self.model = model_resolver.make(name, kw, triples_factory=factory, random_seed=self.args.get("random_seed", 0))
        # the PyKEEN module owns the embeddings
        del self.entity_embeddings, self.relation_embeddings

    def get_embeddings(self):
        ent = self.model.entity_representations[0](indices=None).detach()
        rel = self.model.relation_representations[0](indices=None).detach()
        return ent.reshape(ent.shape[0], -1), rel.reshape(rel.shape[0], -1)

    def forward_k_vs_all(self, x: torch.Tensor):
        return self.model.score_t(x)

    def forward_triples(self, x: torch.Tensor) -> torch.Tensor:
        return self.model.score_hrt(hrt_batch=x, mode=None).flatten()

    def forward_k_vs_sample(self, x, target_entity_idx):
        raise NotImplementedError("Pykeen models do not support sampled candidates")
