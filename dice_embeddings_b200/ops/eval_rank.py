"""Filtered ranking and top-k over an entity table without materialising the score matrix.

``rank = 1 + #{j : s_j > s_target} − #{j ∈ known answers, j ≠ target : s_j > s_target}``: the dense count comes
from the tcgen05 kernel ``dice_eval_rank`` (GEMM tiles in TMEM, counting epilogue), the target score and the
filtered count from gather-dots (``dice_eval_sparse``).  With a process group every rank holds a row shard of the
table (contiguous or cyclic); target scores, counts and top-k candidates are merged across ranks by merge kernels that
read the ranks' buffers in a symmetric heap through peer loads, ordered by the bounded device barrier: the hot loop
holds no library collective and no host round trip.

The reference sorts a dense ``[B, |E|]`` matrix per batch (``dicee/evaluation/evaluator.py:484-508``) and uses
``torch.topk`` over all scores for ``predict_topk`` (``dicee/knowledge_graph_embeddings.py:533-607``).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import kernels

SUPPORTED_D = (64, 128, 256)


def pad_dim(d: int) -> Optional[int]:
    for s in SUPPORTED_D:
        if d <= s:
            return s
    return None


def to_kernel_operand(x: torch.Tensor, d_pad: int) -> torch.Tensor:
    """bf16, contiguous, zero-padded to ``d_pad`` columns."""
    x = x.detach()
    if x.shape[1] == d_pad:
        return x.to(torch.bfloat16).contiguous()
    out = torch.zeros(x.shape[0], d_pad, dtype=torch.bfloat16, device=x.device)
    out[:, :x.shape[1]] = x
    return out


class FusedRanker:
    """Holds one (shard of an) entity table in kernel layout and answers rank / top-k queries against it.

    ``table`` rows are entities ``y_offset + c * y_stride``; ``col_bias`` (fp32, per local row) is added to every
    score of that entity.  ``group``: process group over which the table is sharded (``None`` = whole table here).
    """

    def __init__(self, table: torch.Tensor, col_bias: Optional[torch.Tensor] = None, y_offset: int = 0,
                 y_stride: int = 1, group=None, exact: bool = False, band_capacity: int = 1 << 24):
        """``exact``: ranks equal those of an fp32 scoring of the same operands.  The tensor cores still do the bulk
        of the work on bf16-rounded operands; a score can differ from its fp32 value by at most
        ``2^-8 · ‖q‖ · ‖e‖``, so only entities whose bf16 score lies within that margin of the target are undecided,
        and exactly those (typically a fraction of a percent) are re-scored in fp32 by a second, sparse pass."""
        assert table.is_cuda, "the fused ranker runs on a CUDA device"
        self.d = table.shape[1]
        self.d_pad = pad_dim(self.d)
        if self.d_pad is None:
            raise ValueError(f"embedding width {self.d} exceeds the kernel's limit of {SUPPORTED_D[-1]}")
        self.table = to_kernel_operand(table, self.d_pad)
        self.exact = bool(exact)
        if self.exact:
            t32 = table.detach().float()
            if self.d != self.d_pad:
                t32 = torch.nn.functional.pad(t32, (0, self.d_pad - self.d))
            self.table_f32 = t32.contiguous()
            self.row_norm_max = float(self.table_f32.norm(dim=1).max()) if table.shape[0] else 0.0
            self.band_rows = torch.empty(band_capacity, dtype=torch.int32, device=table.device)
            self.band_cols = torch.empty(band_capacity, dtype=torch.int32, device=table.device)
            self.band_count = torch.zeros(1, dtype=torch.int64, device=table.device)
        self.col_bias = None if col_bias is None else col_bias.detach().float().contiguous()
        self.y_offset, self.y_stride, self.group = int(y_offset), int(y_stride), group
        self.device = table.device
        self._flags = torch.zeros(2, dtype=torch.int32, device=self.device)
        self.status = self._flags[0:1]      # kernel status word
        self.overflow = self._flags[1:2]    # set when a top-k candidate list ran full
        self.W, self.rank = 1, 0
        self._heap = None
        if group is not None:
            import torch.distributed as dist
            self.W, self.rank = dist.get_world_size(group), dist.get_rank(group)
            if self.W == 1:
                self.group = None
            elif self.exact:   # the margin of the band mode needs the largest row norm over all shards: once, here
                emax = torch.tensor([self.row_norm_max], device=self.device)
                dist.all_reduce(emax, op=dist.ReduceOp.MAX, group=group)
                self.row_norm_max = float(emax.item())

    # ------------------------------------------------------------------ cross-rank merge (symmetric heap + barrier)
    K_CAP = 32

    def _merge_buffers(self, B: int):
        """Symmetric buffers for ``B`` queries (collective when they have to grow: every rank calls with the same
        ``B``).  Two candidate sets alternate between top-k calls, so one barrier per call is enough."""
        if self._heap is None or self._heap_rows < B:
            from ..parallel.symm import SymmetricHeap
            rows = max(B, 1024)
            heap = SymmetricHeap(self.group, self.device, multicast=False)
            heap.plan("tgt", (rows,), torch.float32)
            heap.plan("greater", (rows,), torch.int32)
            heap.plan("filtered", (rows,), torch.int32)
            for par in (0, 1):
                heap.plan(f"cs{par}", (rows, self.K_CAP), torch.float32)
                heap.plan(f"ci{par}", (rows, self.K_CAP), torch.int64)
            heap.plan("sig", (64,), torch.int32)
            heap.commit()
            self._heap, self._heap_rows = heap, rows
            self._tab = {n: heap.table(n) for n in ("tgt", "greater", "filtered", "cs0", "ci0", "cs1", "ci1", "sig")}
            self._bar_count = torch.zeros(1, dtype=torch.int32, device=self.device)
            self._topk_parity = 0
            heap.host_barrier()
        return self._heap

    def _barrier(self) -> None:
        kernels.p2p_barrier(self._tab["sig"], self.rank, self.W, self._bar_count, self.status)

    def check(self) -> None:
        """Raise if a kernel reported a failure or a candidate list overflowed.  This is the one place where the ranker
        waits for the GPU: :meth:`ranks` and :meth:`topk` only queue work."""
        code, over = self._flags.tolist()
        if code != 0 or over != 0:
            self._flags.zero_()
        if code != 0:
            raise kernels.KernelError(f"kernel status {code} ({kernels.STATUS_TEXT.get(code, '?')}) in the fused ranker"
                                      " (band list full: raise band_capacity or use smaller batches)")
        if over != 0:
            raise kernels.KernelError("a top-k candidate list ran full: the table prefix used for the threshold was "
                                      "not representative; call topk again with a smaller batch")

    @torch.no_grad()
    def ranks(self, q: torch.Tensor, target: torch.Tensor, filt_ptr: Optional[torch.Tensor] = None,
              filt_cols: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Filtered ranks ``[B]`` (int64) of entity ``target[i]`` for query vector ``q[i]``.  The filter of query
        ``i`` is ``filt_cols[filt_ptr[i]:filt_ptr[i+1]]`` (global entity ids; the target itself is ignored)."""
        B = q.shape[0]
        qk = to_kernel_operand(q, self.d_pad)
        tgt_idx = target.to(torch.int32).contiguous()
        sharded = self.group is not None
        if sharded:   # partial results live in the symmetric heap, where the merge kernels of every rank read them
            heap = self._merge_buffers(B)
            tgt_part, greater, filtered = heap.local("tgt")[:B], heap.local("greater")[:B], heap.local("filtered")[:B]
            tgt_part.zero_()   # the count buffers are cleared behind the first barrier: a slower rank may still be
            tgt_score = torch.empty(B, dtype=torch.float32, device=self.device)   # merging the previous call's counts
        else:
            tgt_part = tgt_score = torch.zeros(B, dtype=torch.float32, device=self.device)
            greater = torch.zeros(B, dtype=torch.int32, device=self.device)
            filtered = torch.zeros(B, dtype=torch.int32, device=self.device)
        if filt_ptr is not None:
            filt_ptr = filt_ptr.to(torch.int64).contiguous()
            filt_cols = filt_cols.to(torch.int32).contiguous()
        if self.exact:
            return self._ranks_exact(q, qk, tgt_idx, tgt_part, tgt_score, greater, filtered, filt_ptr, filt_cols)
        if sharded:  # phase 1: owners score their targets, phase 2: everybody counts against the merged scores
            kernels.eval_sparse(qk, self.table, tgt_idx, tgt_part, None, col_bias=self.col_bias,
                                y_offset=self.y_offset, y_stride=self.y_stride)
            self._barrier()
            kernels.peer_sum_f32(self._tab["tgt"], self.W, tgt_score, B, self.status)
            greater.zero_()
            filtered.zero_()
            if filt_ptr is not None:
                kernels.eval_sparse(qk, self.table, tgt_idx, None, filtered, filt_ptr, filt_cols,
                                    col_bias=self.col_bias, target_in=tgt_score, y_offset=self.y_offset,
                                    y_stride=self.y_stride)
        else:
            kernels.eval_sparse(qk, self.table, tgt_idx, tgt_score, filtered if filt_ptr is not None else None,
                                filt_ptr, filt_cols, col_bias=self.col_bias)
        kernels.eval_rank(qk, self.table, tgt_score, tgt_idx, greater, self.status, col_bias=self.col_bias,
                          y_offset=self.y_offset, y_stride=self.y_stride)
        return self._finish_ranks(greater, filtered, B)

    def _finish_ranks(self, greater, filtered, B: int) -> torch.Tensor:
        if self.group is None:
            return (1 + greater - filtered).long()
        out = torch.empty(B, dtype=torch.int64, device=self.device)
        self._barrier()                       # every rank's counts are complete
        kernels.merge_ranks(self._tab["greater"], self._tab["filtered"], self.W, out, B, self.status)
        return out

    #: tables with more rows than this are searched in two stages (threshold from a prefix, then one collecting pass)
    TWO_STAGE_ROWS = 131072
    SAMPLE_ROWS = 32768

    def _running_topk(self, qk: torch.Tensor, table: torch.Tensor, kk: int, col_bias):
        """Per-segment running top-k lists in the kernel + merge: right for small tables (every thread keeps its own
        list, which costs a warm-up per segment)."""
        B = qk.shape[0]
        cap = kernels.eval_rank_cand_cap(B, table.shape[0], self.d_pad, kk)
        cs = torch.full((B, cap), float("-inf"), dtype=torch.float32, device=self.device)
        ci = torch.full((B, cap), -1, dtype=torch.int32, device=self.device)
        cc = torch.zeros(B, dtype=torch.int32, device=self.device)
        floor = torch.full((B,), float("-inf"), dtype=torch.float32, device=self.device)
        kernels.eval_rank(qk, table, None, None, None, self.status, col_bias=col_bias, y_offset=self.y_offset,
                          y_stride=self.y_stride, k=kk, cand_score=cs, cand_idx=ci, cand_count=cc, row_floor=floor)
        sc, pos = torch.topk(cs, kk, dim=1)
        return sc, torch.gather(ci, 1, pos).long()

    def _topk_local(self, qk: torch.Tensor, kk: int):
        n_local = self.table.shape[0]
        if n_local <= self.TWO_STAGE_ROWS:
            return self._running_topk(qk, self.table, kk, self.col_bias)
        # stage 1: the k-th best score over a sample of the table is a lower bound of the k-th best overall.  The
        # sample takes every (n / S)-th row, so it is representative whatever the order of the rows (a prefix of a
        # table sorted by norm would not be); it is copied once per ranker.
        S = self.SAMPLE_ROWS
        if getattr(self, "_sample", None) is None:
            step = max(n_local // S, 1)
            self._sample = self.table[::step][:S].contiguous()
            self._sample_bias = None if self.col_bias is None else self.col_bias[::step][:S].contiguous()
        sc_s, _ = self._running_topk(qk, self._sample, kk, self._sample_bias)
        floor = sc_s[:, kk - 1].contiguous()
        # stage 2: one pass over the whole table that appends every score >= floor (few per row) to the row's list
        B = qk.shape[0]
        cap = int(8 * kk * (n_local / S) + 64)
        cs = torch.full((B, cap), float("-inf"), dtype=torch.float32, device=self.device)
        ci = torch.full((B, cap), -1, dtype=torch.int32, device=self.device)
        cc = torch.zeros(B, dtype=torch.int32, device=self.device)
        kernels.eval_rank(qk, self.table, None, None, None, self.status, col_bias=self.col_bias,
                          y_offset=self.y_offset, y_stride=self.y_stride, k=-1, cand_score=cs, cand_idx=ci,
                          cand_count=cc, row_floor=floor)
        # a list that ran full (prefix not representative of the table, e.g. rows sorted by norm) is recorded on the
        # device and reported by check(); nothing here waits for the GPU
        self.overflow.logical_or_((cc > cap).any().view(1))
        sc, pos = torch.topk(cs, kk, dim=1)
        return sc, torch.gather(ci, 1, pos).long()

    def _ranks_exact(self, q, qk, tgt_idx, tgt_part, tgt_score, greater, filtered, filt_ptr, filt_cols) -> torch.Tensor:
        q32 = q.detach().float()
        if self.d != self.d_pad:
            q32 = torch.nn.functional.pad(q32, (0, self.d_pad - self.d))
        q32 = q32.contiguous()
        kw = dict(col_bias=self.col_bias, y_offset=self.y_offset, y_stride=self.y_stride)
        sharded = self.group is not None
        # exact target scores and exact filtered counts from the fp32 operands
        kernels.eval_sparse(q32, self.table_f32, tgt_idx, tgt_part, None if sharded else
                            (filtered if filt_ptr is not None else None), None if sharded else filt_ptr,
                            None if sharded else filt_cols, **kw)
        emax = self.row_norm_max
        if sharded:
            self._barrier()
            kernels.peer_sum_f32(self._tab["tgt"], self.W, tgt_score, q.shape[0], self.status)
            greater.zero_()
            filtered.zero_()
            if filt_ptr is not None:
                kernels.eval_sparse(q32, self.table_f32, tgt_idx, None, filtered, filt_ptr, filt_cols,
                                    target_in=tgt_score, **kw)
        # |bf16 score - fp32 score| <= 2^-8 (1 + 2^-9) |q| |e|; a little head room for the fp32 accumulation orders
        margin = (q32.norm(dim=1) * (emax * 2.0 ** -8 * 1.01) + 1e-30).contiguous()
        self.band_count.zero_()
        kernels.eval_rank(qk, self.table, tgt_score, tgt_idx, greater, self.status, margin=margin,
                          band_rows=self.band_rows, band_cols=self.band_cols, band_count=self.band_count, **kw)
        kernels.eval_band_exact(q32, self.table_f32, self.band_rows, self.band_cols, self.band_count, tgt_score,
                                greater, **kw)
        return self._finish_ranks(greater, filtered, q.shape[0])

    @torch.no_grad()
    def topk(self, q: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """``(scores [B, k], entity ids [B, k])`` of the best entities per query, best first."""
        B = q.shape[0]
        n_local = self.table.shape[0]
        qk = to_kernel_operand(q, self.d_pad)
        if k > 32:  # beyond the in-kernel list: plain matmul in slices (rare; interactive use)
            s = qk.float() @ self.table.float().t()
            if self.col_bias is not None:
                s = s + self.col_bias
            sc, ix = torch.topk(s, min(k, n_local), dim=1)
            ix = ix * self.y_stride + self.y_offset
        else:
            kk = min(k, n_local)
            sc, ix = self._topk_local(qk, kk)
        if self.group is not None:
            sc, ix = self._merge_topk(sc, ix, k)
        return sc, ix

    def _merge_topk(self, sc: torch.Tensor, ix: torch.Tensor, k: int):
        """Every rank publishes its local best ``k`` in the symmetric heap; after one barrier a merge kernel picks the
        best ``k`` of the ``W · k`` candidates per query by peer loads.  The candidate buffers alternate between calls,
        so the next call's writes cannot meet a slower rank's reads of this one."""
        B = sc.shape[0]
        if k > self.K_CAP or self.W * k > 256:   # beyond the merge kernel: library path (interactive use only)
            import torch.distributed as dist
            all_s = [torch.empty_like(sc) for _ in range(self.W)]
            all_i = [torch.empty_like(ix) for _ in range(self.W)]
            dist.all_gather(all_s, sc.contiguous(), group=self.group)
            dist.all_gather(all_i, ix.contiguous(), group=self.group)
            cat_s, cat_i = torch.cat(all_s, 1), torch.cat(all_i, 1)
            s2, pos = torch.topk(cat_s, min(k, cat_s.shape[1]), dim=1)
            return s2, torch.gather(cat_i, 1, pos)
        heap = self._merge_buffers(B)
        par = self._topk_parity
        self._topk_parity ^= 1
        cs, ci = heap.local(f"cs{par}")[:B], heap.local(f"ci{par}")[:B]
        cs.fill_(float("-inf"))
        ci.fill_(-1)
        cs[:, :sc.shape[1]].copy_(sc)
        ci[:, :ix.shape[1]].copy_(ix)
        out_s = torch.empty(B, k, dtype=torch.float32, device=self.device)
        out_i = torch.empty(B, k, dtype=torch.int64, device=self.device)
        self._barrier()
        kernels.merge_topk(self._tab[f"cs{par}"], self._tab[f"ci{par}"], self.W, k, self.K_CAP, out_s, out_i, B,
                           self.status)
        return out_s, out_i


def supports(model) -> bool:
    """True when ``model`` can be ranked by the fused path: bilinear contract, CUDA parameters, width ≤ 256."""
    try:
        w = model.entity_embeddings.weight
    except AttributeError:
        return False
    return bool(getattr(model, "bilinear", False)) and w.is_cuda and pad_dim(w.shape[1]) is not None \
        and kernels._lib.available()


def ranker_for_model(model, exact: bool = True) -> FusedRanker:
    """Ranker over the model's entity table; ``exact`` (default) gives the ranks of an fp32 evaluation."""
    return FusedRanker(model.entity_embeddings.weight, exact=exact)


@torch.no_grad()
def model_queries(model, hr: torch.Tensor) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """``(q, bias)`` of the model's bilinear form for index pairs ``hr [B, 2]``."""
    h, r = model.get_head_relation_representation(hr)
    return model.compose(h, r)
