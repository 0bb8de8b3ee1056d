"""The tcgen05 ranking / top-k kernel and the evaluator path built on it, against fp32 PyTorch references."""
import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("CUDA device required", allow_module_level=True)

from dice_embeddings_b200.ops import kernels as K
from dice_embeddings_b200.ops.eval_rank import FusedRanker

DEV = torch.device("cuda:0")


def _operands(nx, ny, D, seed):
    torch.manual_seed(seed)
    x = (torch.randn(nx, D, device=DEV) * 0.3).to(torch.bfloat16)
    y = (torch.randn(ny, D, device=DEV) * 0.3).to(torch.bfloat16)
    return x, y


def _random_filter(nx, ny, per_row, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    counts = torch.randint(0, per_row + 1, (nx,), generator=g)
    ptr = torch.zeros(nx + 1, dtype=torch.int64)
    ptr[1:] = torch.cumsum(counts, 0)
    cols = torch.randint(0, ny, (int(ptr[-1]),), generator=g, dtype=torch.int32)
    return ptr.to(DEV), cols.to(DEV)


def _ref_ranks(scores, tgt_idx, tgt_score, ptr, cols):
    nx = scores.shape[0]
    ar = torch.arange(nx, device=DEV)
    beats = scores > tgt_score[:, None]
    beats[ar, tgt_idx.long()] = False
    greater = beats.sum(1)
    rows = torch.repeat_interleave(ar, ptr[1:] - ptr[:-1])
    mask = torch.zeros_like(beats)
    mask[rows, cols.long()] = True          # duplicates in the filter list count once here ...
    mask[ar, tgt_idx.long()] = False
    filt_unique = (beats & mask).sum(1)
    return greater, filt_unique


@pytest.mark.parametrize("nx,ny,D", [(128, 128, 64), (300, 5000, 128), (257, 1300, 256), (1000, 20000, 256)])
def test_eval_rank_counts_and_filter(nx, ny, D):
    x, y = _operands(nx, ny, D, nx + ny)
    tgt = torch.randint(0, ny, (nx,), device=DEV, dtype=torch.int32)
    ptr, cols = _random_filter(nx, ny, 6, 1)
    # the CSR of a knowledge graph has no duplicates inside a row: make the rows unique
    key = torch.repeat_interleave(torch.arange(nx, device=DEV), ptr[1:] - ptr[:-1]) * ny + cols.long()
    key = torch.unique(key)
    rows_u, cols = key // ny, (key % ny).to(torch.int32)
    ptr = torch.zeros(nx + 1, dtype=torch.int64, device=DEV)
    ptr[1:] = torch.cumsum(torch.bincount(rows_u, minlength=nx), 0)
    r = FusedRanker(y)
    ranks = r.ranks(x, tgt, ptr, cols)
    scores = x.float() @ y.float().t()
    tgt_score = scores[torch.arange(nx, device=DEV), tgt.long()]
    greater, filt = _ref_ranks(scores, tgt, tgt_score, ptr, cols)
    ref = 1 + greater - filt
    diff = (ranks - ref).abs()
    assert diff.max() <= 2, diff.max()          # only scores within rounding of the target may flip
    assert (diff > 0).float().mean() < 0.02


def test_eval_sparse_target_scores():
    x, y = _operands(500, 3000, 256, 3)
    tgt = torch.randint(0, 3000, (500,), device=DEV, dtype=torch.int32)
    out = torch.zeros(500, device=DEV)
    K.eval_sparse(x, y, tgt, out, None)
    ref = (x.float() * y.float()[tgt.long()]).sum(1)
    assert torch.allclose(out, ref, atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("nx,ny,D,k", [(5, 4000, 64, 10), (200, 30000, 128, 10), (130, 3000, 256, 32), (1, 100000, 256, 3)])
def test_eval_topk(nx, ny, D, k):
    x, y = _operands(nx, ny, D, k + nx)
    r = FusedRanker(y)
    sc, ix = r.topk(x, k)
    ref_s, ref_i = torch.topk(x.float() @ y.float().t(), k, dim=1)
    assert torch.allclose(sc, ref_s, atol=2e-3, rtol=1e-3)
    same = (ix == ref_i).float().mean()
    assert same > 0.97, same                     # swaps only between entities whose scores tie within rounding
    assert (torch.sort(sc, dim=1, descending=True).values == sc).all()


def test_eval_rank_bias_and_cyclic_shards_add_up():
    """Two cyclic row shards with a per-entity bias give the same counts and top-k as the whole table."""
    nx, ny, D = 300, 7001, 128
    x, y = _operands(nx, ny, D, 11)
    bias = torch.randn(ny, device=DEV) * 0.5
    tgt = torch.randint(0, ny, (nx,), device=DEV, dtype=torch.int32)
    scores = x.float() @ y.float().t() + bias
    tgt_score = scores[torch.arange(nx, device=DEV), tgt.long()].contiguous()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    greater = torch.zeros(nx, dtype=torch.int32, device=DEV)
    cands = []
    for rank in range(2):
        ys, bs = y[rank::2].contiguous(), bias[rank::2].contiguous()
        cap = K.eval_rank_cand_cap(nx, ys.shape[0], D, 5)
        cs = torch.full((nx, cap), float("-inf"), device=DEV)
        ci = torch.full((nx, cap), -1, dtype=torch.int32, device=DEV)
        cc = torch.zeros(nx, dtype=torch.int32, device=DEV)
        K.eval_rank(x, ys, tgt_score, tgt, greater, status, col_bias=bs, y_offset=rank, y_stride=2, k=5,
                    cand_score=cs, cand_idx=ci, cand_count=cc)
        cands.append((cs, ci))
    torch.cuda.synchronize()
    K.check_status(status)
    beats = scores > tgt_score[:, None]
    beats[torch.arange(nx, device=DEV), tgt.long()] = False
    diff = (greater.long() - beats.sum(1)).abs()
    assert diff.max() <= 2 and (diff > 0).float().mean() < 0.02
    cs = torch.cat([c[0] for c in cands], 1)
    ci = torch.cat([c[1] for c in cands], 1)
    top_s, pos = torch.topk(cs, 5, dim=1)
    top_i = torch.gather(ci, 1, pos).long()
    ref_s, ref_i = torch.topk(scores, 5, dim=1)
    assert torch.allclose(top_s, ref_s, atol=2e-3, rtol=1e-3)
    assert (top_i == ref_i).float().mean() > 0.97


def test_evaluator_fused_path_agrees_with_torch_path(tmp_path):
    from dice_embeddings_b200.data.synthetic import zipf_kg
    from dice_embeddings_b200.data.vocab import er_csr
    from dice_embeddings_b200.evaluation.ranking import metrics_from_ranks, tail_ranks
    from dice_embeddings_b200.models import initialize_model
    triples = zipf_kg(2000, 20, 30000, seed=5)
    model, _ = initialize_model({"model": "ComplEx", "embedding_dim": 96, "num_entities": 2000, "num_relations": 20,
                                 "scoring_technique": "KvsAll"})
    model = model.to(DEV).eval()
    csr = er_csr(triples, 20)
    test = torch.as_tensor(triples[:3000])
    slow = tail_ranks(model, test, csr, 1024, fused=False)
    fast = tail_ranks(model, test, csr, 1024, fused=True)
    # the evaluator's fused path re-scores the undecided band in fp32: same ranks as the fp32 path
    assert (slow == fast).float().mean() > 0.999 and (slow - fast).abs().max() <= 1
    a, b = metrics_from_ranks(slow), metrics_from_ranks(fast)
    assert abs(a["MRR"] - b["MRR"]) < 1e-5


@pytest.mark.parametrize("nx,ny,D", [(300, 5000, 128), (1000, 20000, 256), (64, 3000, 96)])
def test_exact_mode_reproduces_fp32_ranks(nx, ny, D):
    """fp32 operands that are *not* bf16-representable: the band re-scoring must undo the rounding of the GEMM."""
    torch.manual_seed(nx)
    x = torch.randn(nx, D, device=DEV) * 0.3
    y = torch.randn(ny, D, device=DEV) * 0.3
    tgt = torch.randint(0, ny, (nx,), device=DEV, dtype=torch.int32)
    ptr, cols = _random_filter(nx, ny, 5, 2)
    key = torch.unique(torch.repeat_interleave(torch.arange(nx, device=DEV), ptr[1:] - ptr[:-1]) * ny + cols.long())
    rows_u, cols = key // ny, (key % ny).to(torch.int32)
    ptr = torch.zeros(nx + 1, dtype=torch.int64, device=DEV)
    ptr[1:] = torch.cumsum(torch.bincount(rows_u, minlength=nx), 0)
    scores = x.double() @ y.double().t()                     # oracle in fp64
    tgt_score = scores[torch.arange(nx, device=DEV), tgt.long()]
    greater, filt = _ref_ranks(scores, tgt, tgt_score, ptr, cols)
    ref = 1 + greater - filt
    exact = FusedRanker(y, exact=True).ranks(x, tgt, ptr, cols)
    rough = FusedRanker(y, exact=False).ranks(x, tgt, ptr, cols)
    assert (exact == ref).float().mean() > 0.998 and (exact - ref).abs().max() <= 1   # fp32 vs fp64 ties only
    assert (rough == ref).float().mean() < (exact == ref).float().mean()            # the band pass is what fixes them


@pytest.mark.parametrize("adversarial", [False, True])
def test_two_stage_topk_over_a_large_table(adversarial):
    """Tables above the two-stage limit: threshold from a strided sample of the rows, then one collecting pass; the
    sample stays representative when the rows are sorted by norm, and nothing in the call waits for the GPU."""
    nx, ny, D, k = 70, 300000, 128, 10
    x, y = _operands(nx, ny, D, 9)
    if adversarial:
        scale = torch.linspace(0.05, 3.0, ny, device=DEV)[:, None]
        y = (y.float() * scale).to(torch.bfloat16)
    r = FusedRanker(y)
    assert ny > r.TWO_STAGE_ROWS
    sc, ix = r.topk(x, k)
    ref_s, ref_i = torch.topk(x.float() @ y.float().t(), k, dim=1)
    assert torch.allclose(sc, ref_s, atol=5e-3, rtol=2e-3)
    assert (ix == ref_i).float().mean() > 0.97
