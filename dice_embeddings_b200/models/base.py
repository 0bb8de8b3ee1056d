"""Base class of all embedding models.

State-dict keys, constructor argument dictionary and the input-shape dispatch of
``forward`` follow the reference (``dicee/models/base_model.py:121-438``) so that a
``model.pt`` written by either implementation loads in the other.  The class is a plain
``torch.nn.Module`` (no Lightning); the optimiser factory and the loss live here as in the
reference (``base_model.py:86-118,138``).

Bilinear models implement one method, :meth:`compose`, returning the query vector ``q`` and an
optional per-query bias; the three scoring modes (all entities, given triples, sampled
candidates) are derived from it here, which is also the contract the fused CUDA kernels
implement (gather → compose → GEMM).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple, Union

import torch
from torch import nn


class IdentityClass(nn.Module):
    """No-op stand-in for a normaliser / initialiser."""

    def __init__(self, args=None):
        super().__init__()
        self.args = args

    def __call__(self, x):
        return x

    @staticmethod
    def forward(x):
        return x


class BaseKGE(nn.Module):
    #: True when scoring factorises as ``compose(h, r) · t + bias`` (enables the fused kernels)
    bilinear = False

    def __init__(self, args: dict):
        super().__init__()
        self.args = args
        self.name = type(self).__name__
        a = args.get
        self.embedding_dim = a("embedding_dim") or 1
        self.num_entities = a("num_entities", None)
        self.num_relations = a("num_relations", None)
        self.num_tokens = a("num_tokens", None)
        self.learning_rate = a("learning_rate") or 0.1
        self.weight_decay = a("weight_decay") or 0.0
        self.input_dropout_rate = a("input_dropout_rate") or 0.0
        self.hidden_dropout_rate = a("hidden_dropout_rate") or 0.0
        self.feature_map_dropout_rate = a("feature_map_dropout_rate") or 0.0
        self.kernel_size = a("kernel_size") or 3
        self.num_of_output_channels = a("num_of_output_channels") or 3
        self.optimizer_name = a("optim", None)
        self.apply_unit_norm = None
        self.selected_optimizer = None
        self.loss = nn.BCEWithLogitsLoss()
        self.loss_history = []
        self.training_step_outputs = []

        self.normalize_head_entity_embeddings = IdentityClass()
        self.normalize_relation_embeddings = IdentityClass()
        self.normalize_tail_entity_embeddings = IdentityClass()
        self.hidden_normalizer = IdentityClass()
        norm = a("normalization")
        with_tail = a("scoring_technique") in ("NegSample", "KvsSample")
        if norm == "LayerNorm":
            self.normalizer_class = nn.LayerNorm
            self.normalize_head_entity_embeddings = nn.LayerNorm(self.embedding_dim)
            self.normalize_relation_embeddings = nn.LayerNorm(self.embedding_dim)
            if with_tail:
                self.normalize_tail_entity_embeddings = nn.LayerNorm(self.embedding_dim)
        elif norm == "BatchNorm1d":
            self.normalizer_class = nn.BatchNorm1d
            self.normalize_head_entity_embeddings = nn.BatchNorm1d(self.embedding_dim, affine=False)
            self.normalize_relation_embeddings = nn.BatchNorm1d(self.embedding_dim, affine=False)
            if with_tail:
                self.normalize_tail_entity_embeddings = nn.BatchNorm1d(self.embedding_dim, affine=False)
        elif norm is None or norm == "None":
            self.normalizer_class = IdentityClass
        else:
            raise NotImplementedError(norm)

        init = a("init_param")
        if init is None or init == "None":
            self.param_init = IdentityClass()
        elif init == "xavier_normal":
            self.param_init = nn.init.xavier_normal_
        else:
            raise ValueError(f"--init_param (***{init}***) not found")

        self.input_dp_ent_real = nn.Dropout(self.input_dropout_rate)
        self.input_dp_rel_real = nn.Dropout(self.input_dropout_rate)
        # the reference builds the "hidden" dropout from the *input* rate (base_model.py:151)
        self.hidden_dropout = nn.Dropout(self.input_dropout_rate)

        self.byte_pair_encoding = a("byte_pair_encoding", False)
        self.max_length_subword_tokens = a("max_length_subword_tokens", None)
        self.block_size = a("block_size", None)
        if self.byte_pair_encoding and a("model") != "BytE":
            self.token_embeddings = nn.Embedding(self.num_tokens, self.embedding_dim)
            self.param_init(self.token_embeddings.weight.data)
            self.lf = nn.Sequential(nn.Linear(self.embedding_dim * self.max_length_subword_tokens,
                                              self.embedding_dim, bias=False))
            if a("scoring_technique") in ("AllvsAll", "KvsAll") and a("ordered_bpe_entities"):
                shaped = [s for (_, _, s) in a("ordered_bpe_entities")]
                self.register_buffer("ordered_bpe_entities", torch.tensor(shaped, dtype=torch.long),
                                     persistent=False)
        elif self.byte_pair_encoding:
            pass  # BytE owns its token embeddings
        else:
            self.entity_embeddings = nn.Embedding(self.num_entities, self.embedding_dim)
            self.relation_embeddings = nn.Embedding(self.num_relations, self.embedding_dim)
            self.param_init(self.entity_embeddings.weight.data)
            self.param_init(self.relation_embeddings.weight.data)

    # ------------------------------------------------------------------ bookkeeping
    @property
    def device(self) -> torch.device:
        try:
            return next(self.parameters()).device
        except StopIteration:
            return torch.device("cpu")

    def mem_of_model(self) -> Dict:
        """Size in MB (fp32 element count / 2^20, as the reference reports it) and parameter count."""
        num_params = sum(p.numel() for p in self.parameters())
        buffer_size = sum(b.nelement() * b.element_size() for b in self.buffers())
        return {"EstimatedSizeMB": (num_params + buffer_size) / 1024 ** 2, "NumParam": num_params}

    def get_embeddings(self) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        return self.entity_embeddings.weight.data.detach(), self.relation_embeddings.weight.data.detach()

    # ------------------------------------------------------------------ optimiser / loss
    def configure_optimizers(self, parameters=None):
        if parameters is None:
            parameters = self.parameters()
        name, lr, wd = self.optimizer_name, self.learning_rate, self.weight_decay
        if name == "SGD":
            opt = torch.optim.SGD(parameters, lr=lr, momentum=0, dampening=0, weight_decay=wd, nesterov=False)
        elif name == "Adam":
            opt = torch.optim.Adam(parameters, lr=lr, weight_decay=wd)
        elif name == "Adopt":
            from ..optim.adopt import ADOPT
            opt = ADOPT(parameters, lr=lr)
        elif name == "AdamW":
            opt = torch.optim.AdamW(parameters, lr=lr, weight_decay=wd)
        elif name == "NAdam":
            opt = torch.optim.NAdam(parameters, lr=lr, betas=(0.9, 0.999), eps=1e-08, weight_decay=wd,
                                    momentum_decay=0.004)
        elif name == "Adagrad":
            opt = torch.optim.Adagrad(parameters, lr=lr, eps=1e-10, weight_decay=wd)
        elif name == "ASGD":
            opt = torch.optim.ASGD(parameters, lr=lr, lambd=0.0001, alpha=0.75, weight_decay=wd)
        else:
            raise KeyError(f"{name} is not found!")
        self.selected_optimizer = opt
        return opt

    def loss_function(self, yhat_batch: torch.Tensor, y_batch: torch.Tensor) -> torch.Tensor:
        return self.loss(yhat_batch, y_batch)

    def training_step(self, batch, batch_idx=None) -> torch.Tensor:
        if len(batch) == 2:
            x, y = batch
            yhat = self.forward(x)
        elif len(batch) == 3:
            x, y_select, y = batch
            yhat = self.forward((x, y_select))
        else:
            raise RuntimeError("Invalid batch received.")
        return self.loss_function(yhat, y)

    # ------------------------------------------------------------------ representations
    def get_triple_representation(self, idx_hrt: torch.Tensor):
        h_idx, r_idx, t_idx = idx_hrt[:, 0], idx_hrt[:, 1], idx_hrt[:, 2]
        h = self.normalize_head_entity_embeddings(self.input_dp_ent_real(self.entity_embeddings(h_idx)))
        r = self.normalize_relation_embeddings(self.input_dp_rel_real(self.relation_embeddings(r_idx)))
        t = self.normalize_tail_entity_embeddings(self.entity_embeddings(t_idx))
        return h, r, t

    def get_head_relation_representation(self, indexed_triple: torch.Tensor):
        h_idx, r_idx = indexed_triple[:, 0], indexed_triple[:, 1]
        h = self.normalize_head_entity_embeddings(self.input_dp_ent_real(self.entity_embeddings(h_idx)))
        r = self.normalize_relation_embeddings(self.input_dp_rel_real(self.relation_embeddings(r_idx)))
        return h, r

    def get_sentence_representation(self, x: torch.Tensor):
        return (self.token_embeddings(x[:, 0, :]), self.token_embeddings(x[:, 1, :]),
                self.token_embeddings(x[:, 2, :]))

    def get_bpe_head_and_relation_representation(self, x: torch.Tensor):
        h = self.token_embeddings(x[:, 0, :])
        r = self.token_embeddings(x[:, 1, :])
        h = torch.nn.functional.normalize(h, p=2, dim=(1, 2))
        r = torch.nn.functional.normalize(r, p=2, dim=(1, 2))
        return h, r

    # ------------------------------------------------------------------ scoring contract
    def compose(self, h: torch.Tensor, r: torch.Tensor) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """Return ``(q [B, d], bias [B] or None)`` with ``score(h, r, t) = q·t + bias``."""
        raise NotImplementedError(f"MODEL:{self.name} is not bilinear")

    def score(self, h: torch.Tensor, r: torch.Tensor, t: torch.Tensor) -> torch.Tensor:
        q, bias = self.compose(h, r)
        s = (q * t).sum(dim=1)
        return s if bias is None else s + bias

    def k_vs_all_score(self, emb_h: torch.Tensor, emb_r: torch.Tensor, emb_E: torch.Tensor) -> torch.Tensor:
        q, bias = self.compose(emb_h, emb_r)
        s = q @ emb_E.transpose(0, 1)
        return s if bias is None else s + bias.unsqueeze(1)

    def forward_triples(self, x: torch.Tensor) -> torch.Tensor:
        h, r, t = self.get_triple_representation(x)
        return self.score(h, r, t)

    def forward_k_vs_all(self, x: torch.Tensor) -> torch.Tensor:
        if not self.bilinear:
            raise ValueError(f"MODEL:{self.name} does not have forward_k_vs_all function")
        h, r = self.get_head_relation_representation(x)
        return self.k_vs_all_score(h, r, self.entity_embeddings.weight)

    def forward_k_vs_sample(self, x: torch.Tensor, target_entity_idx: torch.Tensor) -> torch.Tensor:
        if not self.bilinear:
            raise ValueError(f"MODEL:{self.name} does not have forward_k_vs_sample function")
        h, r = self.get_head_relation_representation(x)
        q, bias = self.compose(h, r)
        t = self.normalize_tail_entity_embeddings(self.entity_embeddings(target_entity_idx)) \
            if getattr(self, "_normalize_sampled_tails", False) else self.entity_embeddings(target_entity_idx)
        s = torch.einsum("bd,bkd->bk", q, t)
        return s if bias is None else s + bias.unsqueeze(1)

    # byte-pair-encoded variants (reference base_model.py:178-240)
    def forward_byte_pair_encoded_k_vs_all(self, x: torch.Tensor) -> torch.Tensor:
        h, r = self.get_bpe_head_and_relation_representation(x)
        B, T, D = h.shape
        E = self.token_embeddings(self.ordered_bpe_entities.to(h.device)).reshape(-1, T * D)
        h = self.lf(self.input_dp_ent_real(h.reshape(B, T * D)))
        r = self.lf(self.input_dp_rel_real(r.reshape(B, T * D)))
        return self.k_vs_all_score(h, r, self.lf(E))

    def forward_byte_pair_encoded_triple(self, x: torch.Tensor) -> torch.Tensor:
        h, r, t = self.get_sentence_representation(x)
        B, T, C = h.shape
        return self.score(self.lf(h.reshape(B, T * C)), self.lf(r.reshape(B, T * C)), self.lf(t.reshape(B, T * C)))

    # ------------------------------------------------------------------ dispatch
    def forward(self, x: Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]], y_idx: torch.Tensor = None):
        """``(x, y_idx)`` tuple → sampled candidates; ``[B, 3]`` → triple scores; ``[B, 2]`` → scores of all
        entities; 3-D tensors → the byte-pair-encoded variants (reference ``base_model.py:310-344``)."""
        if isinstance(x, tuple):
            x, y_idx = x
            return self.forward_k_vs_sample(x=x, target_entity_idx=y_idx)
        if x.dim() == 2:
            if x.shape[1] == 3:
                return self.forward_triples(x)
            if x.shape[1] == 2:
                return self.forward_k_vs_all(x=x)
            raise ValueError(f"Unexpected input shape {tuple(x.shape)}")
        if x.shape[1] == 3:
            return self.forward_byte_pair_encoded_triple(x=x)
        if x.shape[1] == 2:
            return self.forward_byte_pair_encoded_k_vs_all(x)
        raise ValueError(f"Unexpected input shape {tuple(x.shape)}")
