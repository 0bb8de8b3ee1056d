"""Scoring techniques as *batch-vectorised* datasets.

Every ``--scoring_technique`` of the reference is a ``torch.utils.data.Dataset`` that builds
one data point per ``__getitem__`` call in Python (reference ``dicee/dataset_classes.py``);
for KvsAll that means one dense ``|E|``-float label per item, stacked and copied to the
device every step.  Here each technique keeps its index arrays as tensors (optionally
resident on the GPU) and produces a whole batch with a handful of tensor ops —
``make_batch(idx)`` — so a training step moves only the ``[B]`` index tensor.  The label
semantics of the reference are kept exactly:

* KvsAll / AllvsAll: multi-hot over all entities, smoothing ``y·(1-ε) + 1/|E|``
  (reference ``dataset_classes.py:354-361``);
* 1vsAll: one-hot, no smoothing (``:261-264``);
* NegSample: one coin per batch decides whether all heads or all tails are corrupted with
  uniform ids, ``neg_ratio`` negatives per positive appended after the positives, labels
  ``1-ε`` / ``ε`` (``:717-745``);
* 1vsSample: true tail followed by ``neg_ratio`` distinct negatives ≠ tail (``:528-541``);
* KvsSample: all positives of the pair followed by negatives drawn with replacement outside
  the positives, padded to ``max_positives + neg_ratio`` columns (``:593-613``).

``__getitem__`` / ``collate_fn`` are still provided, so the classes also work inside a stock
``DataLoader``.
"""
from __future__ import annotations

from typing import Iterator, List, Optional, Tuple

import numpy as np
import torch

from .vocab import PairCSR


class BatchedDataset(torch.utils.data.Dataset):
    """Base: a set of ``len(self)`` data points addressable by an index tensor."""

    collate_fn = None

    def __init__(self):
        self.device = torch.device("cpu")

    def to(self, device) -> "BatchedDataset":
        self.device = torch.device(device)
        for k, v in list(self.__dict__.items()):
            if isinstance(v, torch.Tensor):
                setattr(self, k, v.to(self.device))
        return self

    def make_batch(self, idx: torch.Tensor, generator: Optional[torch.Generator] = None):
        raise NotImplementedError

    def __getitem__(self, i):
        batch = self.make_batch(torch.as_tensor([int(i)], device=self.device))
        return tuple(b[0] for b in batch)

    def batches(self, batch_size: int, shuffle: bool = True, generator: Optional[torch.Generator] = None,
                rank: int = 0, world_size: int = 1, drop_last: bool = False, pad_last: bool = False) -> Iterator[tuple]:
        """Yield batches; with ``world_size > 1`` every rank takes a strided slice of one
        shared permutation (same ``generator`` seed on every rank), padded by wrap-around so
        that all ranks see the same number of batches.  ``pad_last`` fills a short final batch up to ``batch_size``
        by wrapping around to the start of the rank's slice (for engines that need full batches; no item is
        dropped); ``drop_last`` skips it instead."""
        n = len(self)
        if shuffle:
            perm = torch.randperm(n, generator=generator)
        else:
            perm = torch.arange(n)
        if world_size > 1:
            per = -(-n // world_size)
            pad = per * world_size - n
            if pad:
                perm = torch.cat([perm, perm[:pad]])
            perm = perm[rank::world_size]
        perm = perm.to(self.device)
        for s in range(0, perm.numel(), batch_size):
            idx = perm[s:s + batch_size]
            if idx.numel() < batch_size:
                if pad_last:
                    reps = -(-(batch_size - idx.numel()) // max(perm.numel(), 1))
                    idx = torch.cat([idx] + [perm] * reps)[:batch_size]
                elif drop_last:
                    break
            yield self.make_batch(idx, generator)

    def dense_batch(self, idx: torch.Tensor, generator: Optional[torch.Generator] = None):
        """``make_batch`` with dense labels even while a fused engine has switched the dataset to id-only batches."""
        sparse = getattr(self, "sparse_labels", False)
        self.sparse_labels = False
        try:
            return self.make_batch(idx, generator)
        finally:
            self.sparse_labels = sparse

    def num_batches(self, batch_size: int, world_size: int = 1, drop_last: bool = False) -> int:
        per = -(-len(self) // world_size)
        return per // batch_size if drop_last else -(-per // batch_size)


def multihot_from_csr(rows: torch.Tensor, cols: torch.Tensor, batch: int, width: int,
                      pos_value: float, base_value: float) -> torch.Tensor:
    """Dense ``[batch, width]`` label matrix: ``base_value`` everywhere, ``pos_value`` at (rows, cols)."""
    y = torch.full((batch, width), base_value, dtype=torch.float32, device=rows.device)
    if rows.numel():
        y[rows, cols] = pos_value
    return y


class KvsAll(BatchedDataset):
    """Unique ``(h, r)`` pairs (sorted) with the multi-hot vector of their known tails.

    With ``form == 'RelationPrediction'`` the pairs are ``(h, t)`` and the label runs over
    relations (reference ``dataset_classes.py:317-322``).
    """

    def __init__(self, train_set_idx: np.ndarray, entity_idxs, relation_idxs, form: str = "EntityPrediction",
                 label_smoothing_rate: float = 0.0):
        super().__init__()
        ts = np.asarray(train_set_idx).astype(np.int64)
        assert len(ts) > 0
        self.num_entities = len(entity_idxs) if not isinstance(entity_idxs, int) else entity_idxs
        self.num_relations = len(relation_idxs) if not isinstance(relation_idxs, int) else relation_idxs
        self.form = form
        self.label_smoothing_rate = float(label_smoothing_rate)
        if form == "RelationPrediction":
            self.csr = PairCSR.build(ts[:, 0], ts[:, 2], ts[:, 1], self.num_entities)
            self.target_dim = self.num_relations
        elif form == "EntityPrediction":
            self.csr = PairCSR.build(ts[:, 0], ts[:, 1], ts[:, 2], self.num_relations)
            self.target_dim = self.num_entities
        else:
            raise NotImplementedError(form)
        self.train_data = torch.from_numpy(self.csr.pairs.copy())
        self.offsets = torch.from_numpy(self.csr.offsets.copy())
        self.values = torch.from_numpy(self.csr.values.copy())

    def __len__(self) -> int:
        return int(self.train_data.shape[0])

    def positives(self, idx: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """(row, col) coordinates of every positive label of the data points ``idx``."""
        start = self.offsets[idx]
        count = self.offsets[idx + 1] - start
        total = int(count.sum())
        rows = torch.repeat_interleave(torch.arange(idx.numel(), device=idx.device), count)
        first = torch.cumsum(count, 0) - count
        within = torch.arange(total, device=idx.device) - torch.repeat_interleave(first, count)
        cols = self.values[torch.repeat_interleave(start, count) + within]
        return rows, cols

    def label_constants(self) -> Tuple[float, float]:
        """(value at positives, value elsewhere) after the reference's smoothing rule."""
        eps = self.label_smoothing_rate
        if eps:
            base = 1.0 / self.target_dim
            return 1.0 * (1.0 - eps) + base, base
        return 1.0, 0.0

    def make_batch(self, idx, generator=None):
        x = self.train_data[idx]
        if getattr(self, "sparse_labels", False):
            # consumers that hold the CSR themselves (the fused engine) only need the data-point ids
            return x, idx
        rows, cols = self.positives(idx)
        pos, base = self.label_constants()
        y = multihot_from_csr(rows, cols, idx.numel(), self.target_dim, pos, base)
        return x, y


class AllvsAll(KvsAll):
    """Every ``(e, r)`` of ``E × R`` is a data point; unseen pairs have an all-zero label
    (reference ``dataset_classes.py:364-449``)."""

    def __init__(self, train_set_idx, entity_idxs, relation_idxs, label_smoothing_rate: float = 0.0):
        super().__init__(train_set_idx, entity_idxs, relation_idxs, "EntityPrediction", label_smoothing_rate)
        seen = self.csr
        E, R = self.num_entities, self.num_relations
        all_keys = np.arange(E * R, dtype=np.int64)
        counts = np.zeros(E * R, dtype=np.int64)
        counts[seen.keys] = seen.counts()
        offsets = np.concatenate([[0], np.cumsum(counts)])
        self.train_data = torch.from_numpy(np.stack([all_keys // R, all_keys % R], axis=1))
        self.offsets = torch.from_numpy(offsets)


class OnevsAllDataset(BatchedDataset):
    """Each triple is a data point ``x = (h, r)`` with a one-hot tail label."""

    def __init__(self, train_set_idx: np.ndarray, entity_idxs):
        super().__init__()
        ts = np.asarray(train_set_idx).astype(np.int64)
        ts = ts[np.lexsort((ts[:, 2], ts[:, 1], ts[:, 0]))]
        self.train_data = torch.from_numpy(ts)
        self.target_dim = len(entity_idxs) if not isinstance(entity_idxs, int) else entity_idxs
        self.num_entities = self.target_dim

    def __len__(self):
        return int(self.train_data.shape[0])

    def make_batch(self, idx, generator=None):
        tr = self.train_data[idx]
        if getattr(self, "sparse_labels", False):
            return tr[:, :2], idx
        y = torch.zeros(idx.numel(), self.target_dim, device=tr.device)
        y[torch.arange(idx.numel(), device=tr.device), tr[:, 2]] = 1.0
        return tr[:, :2], y


def _rand_int(high: int, size, generator, device) -> torch.Tensor:
    if device.type == "cpu":
        return torch.randint(0, high, size, generator=generator)
    # device-side sampling: CPU generators cannot drive CUDA RNG, draw a seed from it instead
    from ..ops import sampling
    seed = int(torch.randint(0, 2 ** 31 - 1, (1,), generator=generator)) if generator is not None else None
    return sampling.uniform_int(high, size, device=device, seed=seed)


class TriplePredictionDataset(BatchedDataset):
    """Negative sampling: positives followed by ``neg_ratio`` corrupted copies each."""

    def __init__(self, train_set: np.ndarray, num_entities: int, num_relations: int, neg_sample_ratio: int = 1,
                 label_smoothing_rate: float = 0.0):
        super().__init__()
        ts = np.asarray(train_set).astype(np.int64)
        ts = ts[np.lexsort((ts[:, 2], ts[:, 1], ts[:, 0]))]
        self.train_set = torch.from_numpy(ts)
        self.num_entities = int(num_entities)
        self.num_relations = int(num_relations)
        self.neg_sample_ratio = int(neg_sample_ratio)
        self.label_smoothing_rate = float(label_smoothing_rate)
        self._generator = None
        #: set by the fused training engine: batches then carry only the positives and the corruptions are drawn
        #: by the device-side generator inside the step
        self.defer_sampling = False

    def __len__(self):
        return int(self.train_set.shape[0])

    def __getitem__(self, i):
        return self.train_set[i]

    def collate_fn(self, batch: List[torch.Tensor]):
        return self.corrupt(torch.stack(batch, dim=0), self._generator)

    def corrupt(self, pos: torch.Tensor, generator=None):
        B = pos.shape[0]
        k = self.neg_sample_ratio
        eps = self.label_smoothing_rate
        h, r, t = pos[:, 0], pos[:, 1], pos[:, 2]
        label = torch.full((B,), 1.0 - eps, device=pos.device)
        if k <= 0:
            return pos, label
        corr = _rand_int(self.num_entities, (B * k,), generator, pos.device)
        coin = float(torch.rand(1, generator=generator))
        if coin >= 0.5:   # corrupt heads
            neg = torch.stack((corr, r.repeat(k), t.repeat(k)), dim=1)
        else:             # corrupt tails
            neg = torch.stack((h.repeat(k), r.repeat(k), corr), dim=1)
        x = torch.cat((pos, neg), 0)
        label = torch.cat((label, torch.full((B * k,), eps, device=pos.device)), 0)
        return x, label

    def make_batch(self, idx, generator=None):
        if self.defer_sampling:
            return self.train_set[idx], None
        return self.corrupt(self.train_set[idx], generator)


class OnevsSample(BatchedDataset):
    """Triple → ``(x=(h,r), y_idx=[t, negatives…], y_vec)`` with distinct negatives ≠ t."""

    def __init__(self, train_set: np.ndarray, num_entities, num_relations, neg_sample_ratio: int = None,
                 label_smoothing_rate: float = 0.0):
        super().__init__()
        assert isinstance(neg_sample_ratio, int) and neg_sample_ratio > 0
        assert neg_sample_ratio < num_entities
        ts = np.asarray(train_set).astype(np.int64)
        ts = ts[np.lexsort((ts[:, 2], ts[:, 1], ts[:, 0]))]
        self.train_data = torch.from_numpy(ts)
        self.num_entities = int(num_entities)
        self.num_relations = int(num_relations)
        self.neg_sample_ratio = int(neg_sample_ratio)
        self.label_smoothing_rate = float(label_smoothing_rate)

    def __len__(self):
        return int(self.train_data.shape[0])

    def make_batch(self, idx, generator=None):
        tr = self.train_data[idx]
        B, k, E = tr.shape[0], self.neg_sample_ratio, self.num_entities
        dev = tr.device
        # k distinct ids in [0, E-1) per row via random keys, then skip over the true tail
        if E - 1 <= 4096 or k * 4 > E:
            keys = torch.rand(B, E - 1, generator=generator if dev.type == "cpu" else None, device=dev)
            neg = keys.topk(k, dim=1).indices
        else:
            neg = _rand_int(E - 1, (B, k), generator, dev)
            for _ in range(8):  # resample duplicates inside a row (rare for k << E)
                s, _i = neg.sort(dim=1)
                dup = torch.zeros_like(s, dtype=torch.bool)
                dup[:, 1:] = s[:, 1:] == s[:, :-1]
                if not bool(dup.any()):
                    break
                s[dup] = _rand_int(E - 1, (int(dup.sum()),), generator, dev)
                neg = s
        neg = neg + (neg >= tr[:, 2:3]).long()
        y_idx = torch.cat((tr[:, 2:3], neg), dim=1)
        eps = self.label_smoothing_rate
        y_vec = torch.cat((torch.full((B, 1), 1.0 - eps, device=dev), torch.full((B, k), eps, device=dev)), dim=1)
        return tr[:, :2], y_idx, y_vec


class KvsSampleDataset(KvsAll):
    """Unique ``(h, r)`` → all positives then negatives (with replacement, outside the positives)
    up to ``max_positives + neg_ratio`` columns."""

    def __init__(self, train_set_idx, entity_idxs, relation_idxs, form="EntityPrediction", store=None,
                 neg_ratio: int = None, label_smoothing_rate: float = 0.0):
        super().__init__(train_set_idx, entity_idxs, relation_idxs, form, label_smoothing_rate)
        assert neg_ratio is not None
        self.neg_ratio = int(neg_ratio)
        self.max_num_of_classes = int(self.csr.counts().max()) + self.neg_ratio

    def make_batch(self, idx, generator=None):
        x = self.train_data[idx]
        dev = x.device
        B, K, E = idx.numel(), self.max_num_of_classes, self.num_entities
        start = self.offsets[idx]
        count = self.offsets[idx + 1] - start
        col = torch.arange(K, device=dev).unsqueeze(0)
        is_pos = col < count.unsqueeze(1)
        gather = (start.unsqueeze(1) + col).clamp_(max=self.values.numel() - 1)
        pos_ids = self.values[gather]
        # negatives: rejection-free draw of the j-th non-positive id.  u ~ U[0, E - count); the
        # id is u shifted past every positive ≤ it (positives are sorted ascending per pair).
        u = (torch.rand(B, K, generator=generator if dev.type == "cpu" else None, device=dev)
             * (E - count).unsqueeze(1).float()).long()
        u = torch.minimum(u, (E - count - 1).clamp_(min=0).unsqueeze(1))
        maxc = int(count.max())
        pcol = torch.arange(maxc, device=dev).unsqueeze(0)
        pvalid = pcol < count.unsqueeze(1)
        pg = (start.unsqueeze(1) + pcol).clamp_(max=self.values.numel() - 1)
        pvals = torch.where(pvalid, self.values[pg], torch.full_like(pg, E + K + 1))  # [B, maxc], ascending
        # shifted[j] = pvals[j] - j is non-decreasing: number of positives p with p - rank(p) <= u
        shifted = pvals - pcol
        nshift = (shifted.unsqueeze(1) <= u.unsqueeze(2)).sum(-1) if maxc * K * B <= 1 << 26 else \
            torch.searchsorted(shifted.contiguous(), u.contiguous(), right=True)
        neg_ids = u + nshift
        y_idx = torch.where(is_pos, pos_ids, neg_ids)
        y_vec = is_pos.float()
        return x, y_idx, y_vec


class NegSampleDataset(BatchedDataset):
    """Pre-drawn (positive, one negative) pairs (reference ``dataset_classes.py:618-657``;
    not wired into ``construct_dataset`` there either)."""

    def __init__(self, train_set: np.ndarray, num_entities: int, num_relations: int, neg_sample_ratio: int = 1):
        super().__init__()
        self.train_set = torch.from_numpy(np.asarray(train_set).astype(np.int64))
        self.num_entities = int(num_entities)
        self.num_relations = int(num_relations)
        self.neg_sample_ratio = int(neg_sample_ratio)

    def __len__(self):
        return int(self.train_set.shape[0])

    def make_batch(self, idx, generator=None):
        pos = self.train_set[idx]
        corr = _rand_int(self.num_entities, (pos.shape[0],), generator, pos.device)
        neg = torch.stack((pos[:, 0], pos[:, 1], corr), dim=1)
        x = torch.stack((pos, neg), dim=1)
        y = torch.tensor([1.0, 0.0], device=pos.device).expand(pos.shape[0], 2)
        return x, y


# ------------------------------------------------------------------ byte-pair-encoded variants
class BPE_NegativeSamplingDataset(BatchedDataset):
    """Token-id triples ``[N, 3, T]``; negatives replace head or tail by a random known entity's
    token sequence (reference ``dataset_classes.py:107-149``)."""

    def __init__(self, train_set: torch.LongTensor, ordered_shaped_bpe_entities: torch.LongTensor, neg_ratio: int):
        super().__init__()
        self.train_set = torch.as_tensor(train_set, dtype=torch.long)
        self.ordered_bpe_entities = torch.as_tensor(ordered_shaped_bpe_entities, dtype=torch.long)
        self.num_bpe_entities = int(self.ordered_bpe_entities.shape[0])
        self.neg_ratio = int(neg_ratio)
        self.num_datapoints = int(self.train_set.shape[0])

    def __len__(self):
        return self.num_datapoints

    def __getitem__(self, i):
        return self.train_set[i]

    def collate_fn(self, batch):
        return self._corrupt(torch.stack(batch, dim=0), None)

    def _corrupt(self, pos, generator):
        B = pos.shape[0]
        dev = pos.device
        k = max(self.neg_ratio, 1)
        rep = pos.repeat(k, 1, 1).clone()
        ids = _rand_int(self.num_bpe_entities, (B * k,), generator, dev)
        corr = self.ordered_bpe_entities[ids]
        head = torch.rand(B * k, generator=generator if dev.type == "cpu" else None, device=dev) >= 0.5
        rep[head, 0, :] = corr[head]
        rep[~head, 2, :] = corr[~head]
        x = torch.cat((pos, rep), 0)
        y = torch.cat((torch.ones(B, device=dev), torch.zeros(B * k, device=dev)), 0)
        return x, y

    def make_batch(self, idx, generator=None):
        return self._corrupt(self.train_set[idx], generator)


class MultiLabelDataset(BatchedDataset):
    """BPE KvsAll / AllvsAll: ``x = (bpe_h, bpe_r)`` ``[2, T]``, multi-hot over the ordered BPE entities
    (reference ``dataset_classes.py:152-177``)."""

    def __init__(self, train_set: torch.LongTensor, train_indices_target, target_dim: int,
                 torch_ordered_shaped_bpe_entities: torch.LongTensor):
        super().__init__()
        self.train_set = torch.as_tensor(train_set, dtype=torch.long)
        counts = np.array([len(v) for v in train_indices_target], dtype=np.int64)
        self.offsets = torch.from_numpy(np.concatenate([[0], np.cumsum(counts)]))
        flat = [int(i) for v in train_indices_target for i in v]
        self.values = torch.tensor(flat, dtype=torch.long)
        self.target_dim = int(target_dim)
        self.torch_ordered_shaped_bpe_entities = torch.as_tensor(torch_ordered_shaped_bpe_entities)

    def __len__(self):
        return int(self.train_set.shape[0])

    def make_batch(self, idx, generator=None):
        x = self.train_set[idx]
        start = self.offsets[idx]
        count = self.offsets[idx + 1] - start
        total = int(count.sum())
        rows = torch.repeat_interleave(torch.arange(idx.numel(), device=idx.device), count)
        first = torch.cumsum(count, 0) - count
        within = torch.arange(total, device=idx.device) - torch.repeat_interleave(first, count)
        cols = self.values[torch.repeat_interleave(start, count) + within] if total else rows
        return x, multihot_from_csr(rows, cols, idx.numel(), self.target_dim, 1.0, 0.0)


class MultiClassClassificationDataset(BatchedDataset):
    """Sliding windows of ``block_size`` tokens with next-token targets (BytE;
    reference ``dataset_classes.py:180-219``)."""

    def __init__(self, subword_units: np.ndarray, block_size: int = 8):
        super().__init__()
        self.train_data = torch.as_tensor(np.asarray(subword_units), dtype=torch.long)
        assert self.train_data.dim() == 1
        self.block_size = int(block_size)
        self.num_of_data_points = len(self.train_data) - self.block_size
        assert self.num_of_data_points > 0, "token stream shorter than block_size"

    def __len__(self):
        return self.num_of_data_points

    def make_batch(self, idx, generator=None):
        win = idx.unsqueeze(1) + torch.arange(self.block_size + 1, device=idx.device).unsqueeze(0)
        tok = self.train_data[win]
        return tok[:, :-1], tok[:, 1:]


class LiteralDataset(BatchedDataset):
    """``(entity, attribute) → normalised numeric value`` triples for literal regression
    (reference ``dataset_classes.py:776-996``).  ``normalization`` is ``z-norm``, ``min-max`` or None,
    applied per attribute."""

    def __init__(self, file_path: str = None, ent_idx: dict = None, normalization_type: str = "z-norm",
                 sampling_ratio: float = None, loader_backend: str = "pandas", df=None):
        super().__init__()
        import pandas as pd
        self.normalization_type = normalization_type
        self.ent_idx = ent_idx
        if df is None:
            df = self.load_and_validate_literal_data(file_path, loader_backend)
        df = df[df["head"].isin(ent_idx)].reset_index(drop=True)
        assert len(df) > 0, "No literal triple refers to a known entity"
        if sampling_ratio is not None and 0 < sampling_ratio < 1:
            df = df.groupby("attribute", group_keys=False).apply(
                lambda g: g.sample(frac=sampling_ratio, random_state=42)).reset_index(drop=True)
        attrs = sorted(df["attribute"].unique())
        self.data_property_to_idx = {a: i for i, a in enumerate(attrs)}
        self.num_data_properties = len(attrs)
        df = df.copy()
        df["head_idx"] = df["head"].map(ent_idx)
        df["attr_idx"] = df["attribute"].map(self.data_property_to_idx)
        self.normalization_params = {}
        vals = df["value"].astype(float)
        if normalization_type == "z-norm":
            st = df.groupby("attribute")["value"].agg(["mean", "std"])
            st["std"] = st["std"].fillna(1.0).replace(0.0, 1.0)
            self.normalization_params = {a: {"mean": float(r["mean"]), "std": float(r["std"])} for a, r in st.iterrows()}
            vals = (vals - df["attribute"].map(st["mean"])) / df["attribute"].map(st["std"])
        elif normalization_type == "min-max":
            st = df.groupby("attribute")["value"].agg(["min", "max"])
            rng = (st["max"] - st["min"]).replace(0.0, 1.0)
            self.normalization_params = {a: {"min": float(st.loc[a, "min"]), "max": float(st.loc[a, "max"])} for a in st.index}
            vals = (vals - df["attribute"].map(st["min"])) / df["attribute"].map(rng)
        elif normalization_type is None:
            pass
        else:
            raise ValueError(f"Unsupported normalization type: {normalization_type}")
        self.normalization_params["type"] = normalization_type
        self.triples = torch.tensor(np.stack([df["head_idx"].values, df["attr_idx"].values], 1), dtype=torch.long)
        self.values = torch.tensor(df["value"].astype(float).values, dtype=torch.float32)
        self.values_norm = torch.tensor(vals.values, dtype=torch.float32)
        self.train_df = df

    @staticmethod
    def load_and_validate_literal_data(file_path: str, loader_backend: str = "pandas"):
        import os
        import pandas as pd
        if not os.path.exists(file_path):
            raise FileNotFoundError(f"Data file not found at {file_path}")
        ext = os.path.splitext(file_path)[1].lower()
        if loader_backend == "rdflib" or ext in (".ttl", ".owl", ".rdf"):
            from rdflib import Graph, Literal
            g = Graph().parse(file_path)
            rows = [(str(s), str(p), float(o)) for s, p, o in g if isinstance(o, Literal) and _is_number(o)]
            df = pd.DataFrame(rows, columns=["head", "attribute", "value"])
        else:
            df = pd.read_csv(file_path, sep=r"\s+|,", engine="python", header=None, names=["head", "attribute", "value"])
        df["value"] = pd.to_numeric(df["value"], errors="coerce")
        df = df.dropna(subset=["value"]).reset_index(drop=True)
        if df.empty:
            raise ValueError("Literal file contains no numeric triples")
        return df

    @staticmethod
    def denormalize(preds_norm, attributes, normalization_params) -> np.ndarray:
        kind = normalization_params.get("type")
        preds = np.asarray(preds_norm, dtype=np.float64)
        if kind == "z-norm":
            m = np.array([normalization_params[a]["mean"] for a in attributes])
            s = np.array([normalization_params[a]["std"] for a in attributes])
            return preds * s + m
        if kind == "min-max":
            lo = np.array([normalization_params[a]["min"] for a in attributes])
            hi = np.array([normalization_params[a]["max"] for a in attributes])
            rng = np.where(hi - lo == 0, 1.0, hi - lo)
            return preds * rng + lo
        return preds

    def __len__(self):
        return int(self.triples.shape[0])

    def make_batch(self, idx, generator=None):
        return self.triples[idx], self.values_norm[idx]

    def __getitem__(self, i):
        return self.triples[i], self.values_norm[i]


def _is_number(x) -> bool:
    try:
        float(x)
        return True
    except (TypeError, ValueError):
        return False


def construct_dataset(*, train_set, valid_set=None, test_set=None, ordered_bpe_entities=None,
                      train_target_indices=None, target_dim: int = None, entity_to_idx: dict,
                      relation_to_idx: dict, form_of_labelling: str, scoring_technique: str, neg_ratio: int,
                      label_smoothing_rate: float, byte_pair_encoding=None, block_size: int = None) -> BatchedDataset:
    """Pick the dataset class for a scoring technique (reference ``dataset_classes.py:25-104``)."""
    if ordered_bpe_entities and byte_pair_encoding and scoring_technique == "NegSample":
        ds = BPE_NegativeSamplingDataset(
            torch.tensor(np.asarray(train_set), dtype=torch.long),
            torch.tensor([shaped for (_, _, shaped) in ordered_bpe_entities]), neg_ratio)
    elif ordered_bpe_entities and byte_pair_encoding and scoring_technique in ("KvsAll", "AllvsAll"):
        ds = MultiLabelDataset(torch.tensor(np.asarray(train_set), dtype=torch.long), train_target_indices,
                               target_dim, torch.tensor([shaped for (_, _, shaped) in ordered_bpe_entities]))
    elif byte_pair_encoding:
        ds = MultiClassClassificationDataset(train_set, block_size=block_size)
    elif scoring_technique == "NegSample":
        ds = TriplePredictionDataset(train_set, len(entity_to_idx), len(relation_to_idx), neg_ratio,
                                     label_smoothing_rate)
    elif form_of_labelling == "EntityPrediction":
        if scoring_technique == "1vsAll":
            ds = OnevsAllDataset(train_set, entity_to_idx)
        elif scoring_technique == "1vsSample":
            ds = OnevsSample(train_set, len(entity_to_idx), len(relation_to_idx), neg_ratio, label_smoothing_rate)
        elif scoring_technique == "KvsAll":
            ds = KvsAll(train_set, entity_to_idx, relation_to_idx, form_of_labelling, label_smoothing_rate)
        elif scoring_technique == "AllvsAll":
            ds = AllvsAll(train_set, entity_to_idx, relation_to_idx, label_smoothing_rate)
        elif scoring_technique == "KvsSample":
            ds = KvsSampleDataset(train_set, entity_to_idx, relation_to_idx, form_of_labelling,
                                  neg_ratio=neg_ratio, label_smoothing_rate=label_smoothing_rate)
        else:
            raise ValueError(f"Invalid scoring technique : {scoring_technique}")
    elif form_of_labelling == "RelationPrediction":
        ds = KvsAll(train_set, entity_to_idx, relation_to_idx, form_of_labelling, label_smoothing_rate)
    else:
        raise KeyError("Illegal input.")
    return ds
