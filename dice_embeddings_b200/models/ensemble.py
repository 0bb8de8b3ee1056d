"""Embedding-dimension parallel ("TP") model: one full-size replica per device, logits averaged.

Because every multiplicative score is a sum over embedding-dimension blocks, ``k`` independently seeded
``d``-dimensional replicas act like one ``k·d``-dimensional model whose logits are the mean of the parts
(reference ``dicee/models/ensemble.py:4-141``).  The reference drives all replicas from one Python thread and
copies each ``[B, |E|]`` logit matrix to GPU 0; here every replica runs on its own CUDA stream so the GPUs
overlap, the partial logits are reduced on the first device, and the class also works with CPU replicas
(devices are a constructor argument, not hard-wired ``cuda:i``).  Checkpoints are ``model_partial_{i}.pt``;
exported embeddings are concatenated along dim 1.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.nn as nn


class EnsembleKGE:
    def __init__(self, models: Optional[list] = None, seed_model=None, pretrained_models: Optional[List] = None,
                 devices: Optional[Sequence] = None):
        mods = models if models is not None else pretrained_models
        assert mods is not None and len(mods) > 0
        if devices is None:
            n_gpu = torch.cuda.device_count()
            devices = [torch.device(f"cuda:{i % n_gpu}") if n_gpu else torch.device("cpu") for i in range(len(mods))]
        self.devices = [torch.device(d) for d in devices]
        self.models = nn.ModuleList()
        self.optimizers = []
        self.loss_history = []
        for m, d in zip(mods, self.devices):
            m.to(d)
            self.optimizers.append(m.configure_optimizers())
            self.models.append(m)
        self.name = self.models[0].name
        self.train_mode = True
        self.args = self.models[0].args
        self._streams = [torch.cuda.Stream(device=d) if d.type == "cuda" else None for d in self.devices]

    # container protocol ----------------------------------------------------------------
    def named_children(self):
        return self.models[0].named_children()

    def parameters(self):
        return [p for m in self.models for p in m.parameters()]

    def modules(self):
        return [x for m in self.models for x in m.modules()]

    def __iter__(self):
        return iter(self.models)

    def __len__(self):
        return len(self.models)

    def eval(self):
        for m in self.models:
            m.eval()
        self.train_mode = False
        return self

    def train(self, mode: bool = True):
        for m in self.models:
            m.train(mode)
        self.train_mode = mode
        return self

    def to(self, device):
        if str(device) == "cpu":
            for m in self.models:
                m.cpu()
            self.devices = [torch.device("cpu")] * len(self.models)
            self._streams = [None] * len(self.models)
            return self
        raise NotImplementedError("EnsembleKGE can only be moved to cpu as a whole")

    @property
    def device(self):
        return self.devices[0]

    def state_dict(self):
        return self.models.state_dict()

    def load_state_dict(self, state_dict, strict=True):
        return self.models.load_state_dict(state_dict, strict=strict)

    def mem_of_model(self):
        out = {"EstimatedSizeMB": 0, "NumParam": 0}
        for m in self.models:
            for k, v in m.mem_of_model().items():
                out[k] += v
        return out

    # forward / step --------------------------------------------------------------------
    def _move(self, x, d):
        if isinstance(x, tuple):
            return tuple(t.to(d, non_blocking=True) for t in x)
        return x.to(d, non_blocking=True)

    def __call__(self, x_batch):
        if self.train_mode:
            for opt in self.optimizers:
                opt.zero_grad(set_to_none=True)
        d0 = self.devices[0]
        parts = []
        for m, d, s in zip(self.models, self.devices, self._streams):
            if s is not None:
                s.wait_stream(torch.cuda.current_stream(d))
                with torch.cuda.stream(s):
                    parts.append(m(self._move(x_batch, d)))
            else:
                parts.append(m(self._move(x_batch, d)))
        yhat = None
        for p, d, s in zip(parts, self.devices, self._streams):
            if s is not None:
                torch.cuda.current_stream(d).wait_stream(s)
            p0 = p.to(d0)
            yhat = p0 if yhat is None else yhat + p0
        return yhat / len(self.models)

    def step(self):
        for opt in self.optimizers:
            opt.step()

    def get_embeddings(self):
        ents, rels = [], []
        for m in self.models:
            e, r = m.get_embeddings()
            ents.append(e.cpu())
            if r is not None:
                rels.append(r.cpu())
        return torch.cat(ents, dim=1), (torch.cat(rels, dim=1) if rels else None)

    def __str__(self):
        return f"EnsembleKGE of {len(self.models)} {self.models[0]}"
