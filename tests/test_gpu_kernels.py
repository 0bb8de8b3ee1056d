"""Numerics of the sm_100a kernels against plain PyTorch fp32 references of the same ops."""
import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("CUDA device required", allow_module_level=True)

from dice_embeddings_b200.models import algebra
from dice_embeddings_b200.ops import kernels as K

DEV = torch.device("cuda:0")


def _ref_fused(x, y, base, scale):
    s = x.float() @ y.float().t()
    loss = (torch.nn.functional.softplus(s) - base * s).double().sum()
    ds = torch.sigmoid(s) - base
    out = scale * (ds @ y.float())          # plain fp32: the kernel's bf16 rounding of dS is part of what is tested
    return loss, out


@pytest.mark.parametrize("nx,ny,D", [(128, 128, 64), (300, 200, 64), (257, 130, 128), (300, 520, 256), (1000, 777, 256)])
@pytest.mark.parametrize("with_loss", [True, False])
def test_kvsall_fused_matches_reference(nx, ny, D, with_loss):
    torch.manual_seed(nx + ny + D)
    x = (torch.randn(nx, D, device=DEV) * 0.3).to(torch.bfloat16)
    y = (torch.randn(ny, D, device=DEV) * 0.3).to(torch.bfloat16)
    base, scale = 0.01, 1.0 / 64
    out = torch.zeros(nx, D, device=DEV)
    loss = torch.zeros(1, dtype=torch.float64, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    K.kvsall_fused(x, y, out, loss if with_loss else None, status, base, scale, with_loss)
    torch.cuda.synchronize()
    K.check_status(status)
    ref_loss, ref_out = _ref_fused(x, y, base, scale)
    denom = ref_out.abs().max().clamp_min(1e-6)
    assert (out - ref_out).abs().max() / denom < 2e-2
    if with_loss:
        assert abs(loss.item() - ref_loss.item()) / abs(ref_loss.item()) < 2e-3


def _masked_reference(x, y, mask_bits, base, pos, scale):
    """fp32 statement of the masked step: labels = pos where the bit is set, base elsewhere."""
    s = x.float() @ y.float().t()
    labels = torch.where(mask_bits, torch.full_like(s, pos), torch.full_like(s, base))
    loss = (torch.nn.functional.softplus(s) - labels * s).double().sum()
    ds = torch.sigmoid(s) - labels
    return loss, scale * (ds @ y.float())


def _pack_mask(bits):
    """[nx, ny] bool -> int32 words, one bit per column, rows padded as the kernels expect."""
    nx, ny = bits.shape
    stride = K.mask_stride(ny)
    padded = torch.zeros(nx, stride * 32, dtype=torch.bool, device=bits.device)
    padded[:, :ny] = bits
    w = padded.view(nx, stride, 32).to(torch.int64)
    weights = (2 ** torch.arange(32, device=bits.device, dtype=torch.int64))
    words = (w * weights).sum(-1)
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words)
    return words.to(torch.int32).contiguous()


@pytest.mark.parametrize("nx,ny,ctas", [(256, 128, 0), (1000, 777, 0), (3000, 1500, 4), (2049, 4100, 6), (130, 260, 2),
                                        (4096, 14541, 0)])
@pytest.mark.parametrize("with_loss,masked", [(True, True), (False, True), (True, False)])
def test_pair_kernel_matches_reference_and_one_cta_kernel(nx, ny, ctas, with_loss, masked, monkeypatch):
    """The CTA-pair kernel (d = 256) against the fp32 reference, with label masks, ragged edges in both dimensions
    and few CTA pairs, so that one pair walks many segments (x super-tiles); and against the one-CTA kernel."""
    torch.manual_seed(nx * 7 + ny)
    D = 256
    x = (torch.randn(nx, D, device=DEV) * 0.25).to(torch.bfloat16)
    y = (torch.randn(ny, D, device=DEV) * 0.25).to(torch.bfloat16)
    base, pos, scale = 0.002, 0.9, 1.0 / 128
    bits = torch.rand(nx, ny, device=DEV) < 0.03
    mask = _pack_mask(bits) if masked else None
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    res = {}
    for flavour in ("1", "0"):
        monkeypatch.setenv("DICE_B200_PAIR", flavour)
        out = torch.zeros(nx, D, device=DEV)
        loss = torch.zeros(1, dtype=torch.float64, device=DEV)
        K.kvsall_fused(x, y, out, loss if with_loss else None, status, base, scale, with_loss, num_ctas=ctas,
                       mask=mask, pos_delta=pos - base)
        torch.cuda.synchronize()
        K.check_status(status)
        res[flavour] = (out, loss.item())
    ref_loss, ref_out = _masked_reference(x, y, bits if masked else torch.zeros_like(bits), base, pos, scale)
    denom = ref_out.abs().max().clamp_min(1e-6)
    for flavour in ("1", "0"):
        out, loss = res[flavour]
        assert (out - ref_out).abs().max() / denom < 2e-2, flavour
        if with_loss:
            assert abs(loss - ref_loss.item()) / abs(ref_loss.item()) < 2e-3, flavour
    assert (res["1"][0] - res["0"][0]).abs().max() / denom < 1e-2


def test_pair_kernel_loss_split_between_the_two_roles_adds_up(monkeypatch):
    """The two launches of a step (roles of x and y swapped) each add the loss of one half of the (x, y) plane."""
    monkeypatch.setenv("DICE_B200_PAIR", "1")
    torch.manual_seed(5)
    nx, ny, D = 1500, 700, 256
    x = (torch.randn(nx, D, device=DEV) * 0.25).to(torch.bfloat16)
    y = (torch.randn(ny, D, device=DEV) * 0.25).to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    full = torch.zeros(1, dtype=torch.float64, device=DEV)
    halves = torch.zeros(1, dtype=torch.float64, device=DEV)
    ox, oy = torch.zeros(nx, D, device=DEV), torch.zeros(ny, D, device=DEV)
    K.kvsall_fused(x, y, ox, full, status, 0.01, 1.0, True)
    ox2, oy2 = torch.zeros(nx, D, device=DEV), torch.zeros(ny, D, device=DEV)
    K.kvsall_fused(x, y, ox2, halves, status, 0.01, 1.0, True, loss_share=0)
    part = halves.item()
    K.kvsall_fused(y, x, oy2, halves, status, 0.01, 1.0, True, loss_share=1)
    torch.cuda.synchronize()
    K.check_status(status)
    assert 0.2 * full.item() < part < 0.8 * full.item()
    assert abs(halves.item() - full.item()) < 1e-6 * abs(full.item())
    assert (ox - ox2).abs().max() <= 2e-2 * ox.abs().max()


def _pad128(v):
    out = torch.zeros(K.padded_rows(v.numel()), device=v.device)
    out[: v.numel()] = v
    return out


@pytest.mark.parametrize("nx,ny,D,ctas", [(300, 200, 64, 0), (257, 515, 128, 0), (1000, 777, 256, 0), (1500, 900, 256, 3)])
@pytest.mark.parametrize("with_loss", [True, False])
def test_kvsall_fused_with_row_and_column_bias(nx, ny, D, ctas, with_loss):
    """score_mode 1: logit = x·y + bx[x] + by[y]; loss, out and the gradient of bx against fp32 autograd."""
    torch.manual_seed(nx + ny + D)
    x = (torch.randn(nx, D, device=DEV) * 0.3).to(torch.bfloat16)
    y = (torch.randn(ny, D, device=DEV) * 0.3).to(torch.bfloat16)
    bx = torch.randn(nx, device=DEV) * 0.5
    by = torch.randn(ny, device=DEV) * 0.5
    bits = torch.rand(nx, ny, device=DEV) < 0.05
    base, pos, scale = 0.01, 0.92, 1.0 / 64
    xf = x.float().requires_grad_(True)
    bxf = bx.clone().requires_grad_(True)
    s = xf @ y.float().t() + bxf[:, None] + by[None, :]
    labels = torch.where(bits, torch.full_like(s, pos), torch.full_like(s, base))
    ref_loss = (torch.nn.functional.softplus(s) - labels * s).double().sum()
    (ref_loss * scale).backward()
    out = torch.zeros(nx, D, device=DEV)
    dsum = torch.zeros(nx, device=DEV)
    loss = torch.zeros(1, dtype=torch.float64, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    K.kvsall_fused(x, y, out, loss if with_loss else None, status, base, scale, with_loss, num_ctas=ctas,
                   mask=_pack_mask(bits), pos_delta=pos - base, score_mode=1, x_bias=_pad128(bx), y_bias=_pad128(by),
                   x_dsum=dsum)
    torch.cuda.synchronize()
    K.check_status(status)
    assert (out - xf.grad).abs().max() / xf.grad.abs().max() < 2e-2
    assert (dsum - bxf.grad).abs().max() / bxf.grad.abs().max() < 1e-2
    if with_loss:
        assert abs(loss.item() - ref_loss.item()) / abs(ref_loss.item()) < 2e-3


@pytest.mark.parametrize("nx,ny,D,ctas", [(300, 200, 64, 0), (257, 515, 128, 0), (1000, 777, 256, 0), (1500, 900, 256, 3)])
@pytest.mark.parametrize("with_loss", [True, False])
def test_kvsall_fused_distance_score(nx, ny, D, ctas, with_loss):
    """score_mode 2: logit = margin − ‖x − y‖; gradient with respect to x = out − dsum · x against fp32 autograd."""
    torch.manual_seed(nx * 3 + ny + D)
    x = (torch.randn(nx, D, device=DEV) * 0.3).to(torch.bfloat16)
    y = (torch.randn(ny, D, device=DEV) * 0.3).to(torch.bfloat16)
    bits = torch.rand(nx, ny, device=DEV) < 0.05
    base, pos, scale, margin = 0.01, 0.92, 1.0 / 64, 4.0
    xf = x.float().requires_grad_(True)
    s = margin - torch.cdist(xf, y.float())
    labels = torch.where(bits, torch.full_like(s, pos), torch.full_like(s, base))
    ref_loss = (torch.nn.functional.softplus(s) - labels * s).double().sum()
    (ref_loss * scale).backward()
    out = torch.zeros(nx, D, device=DEV)
    dsum = torch.zeros(nx, device=DEV)
    loss = torch.zeros(1, dtype=torch.float64, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    K.kvsall_fused(x, y, out, loss if with_loss else None, status, base, scale, with_loss, num_ctas=ctas,
                   mask=_pack_mask(bits), pos_delta=pos - base, score_mode=2,
                   x_bias=_pad128((x.float() ** 2).sum(1)), y_bias=_pad128((y.float() ** 2).sum(1)), x_dsum=dsum,
                   margin=margin)
    torch.cuda.synchronize()
    K.check_status(status)
    grad = out - dsum[:, None] * x.float()
    assert (grad - xf.grad).abs().max() / xf.grad.abs().max() < 2e-2
    if with_loss:
        assert abs(loss.item() - ref_loss.item()) / abs(ref_loss.item()) < 2e-3


@pytest.mark.parametrize("kind", [0, 1, 2, 3])
@pytest.mark.parametrize("nx,ny,D,ctas", [(300, 200, 64, 0), (1000, 777, 256, 0), (1500, 2100, 256, 5), (700, 900, 128, 148)])
def test_fused_entity_update_equals_scoring_then_optimizer(kind, nx, ny, D, ctas):
    """The optimiser applied inside the scoring launch (by the CTA that completes a 128-row tile of the gradient)
    against the same launch followed by the optimiser sweep: two steps, each starting from the same state in both
    paths (the gradient sums come from atomics, and over several steps that rounding noise grows through the bf16
    rounding of the operand), with a gradient buffer that already holds other contributions."""
    torch.manual_seed(kind * 100 + nx)
    y = (torch.randn(ny, D, device=DEV) * 0.3).to(torch.bfloat16)
    mask = _pack_mask(torch.rand(nx, ny, device=DEV) < 0.05)
    lr, b1, b2, eps, wd = 0.05, 0.9, 0.999, 1e-3, 0.01
    P = torch.randn(nx, D, device=DEV) * 0.3
    m, v = torch.zeros_like(P), torch.zeros_like(P)
    step = torch.zeros(1, dtype=torch.int64, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    count = torch.zeros((nx + 127) // 128, dtype=torch.int32, device=DEV)
    for it in range(2):
        g0 = torch.randn_like(P) * 1e-3                      # e.g. the row gradients of the lookups
        res = []
        for fused in (False, True):
            Pi, mi, vi, gi = P.clone(), m.clone(), v.clone(), g0.clone()
            Xi = Pi.to(torch.bfloat16)
            loss = torch.zeros(1, dtype=torch.float64, device=DEV)
            opt = K.fused_optimizer_args(kind, Pi, mi, vi, Xi, count, step, lr, b1, b2, eps, wd) if fused else None
            K.kvsall_fused(Xi, y, gi, loss, status, 0.01, 1.0 / 64, True, num_ctas=ctas, mask=mask, pos_delta=0.9,
                           opt=opt)
            if not fused:
                K.optimizer_step(kind, Pi, gi, mi, vi, Xi, step, lr, b1, b2, eps, wd)
            torch.cuda.synchronize()
            K.check_status(status)
            assert float(gi.abs().max()) == 0.0 and int(count.abs().max()) == 0
            assert torch.equal(Xi, Pi.to(torch.bfloat16))
            res.append((Pi, mi, vi, loss))
        for a, b in zip(*res):
            assert (a - b).abs().max() <= 2e-5 * a.abs().max().clamp_min(1e-6) + 1e-7
        P, m, v = res[0][:3]
        step += 1


def test_kvsall_fused_accumulates_and_splits_work():
    """Two launches add up; any CTA count gives the same sums (work ranges are arbitrary cuts of the tile grid)."""
    torch.manual_seed(0)
    nx, ny, D = 700, 900, 128
    x = (torch.randn(nx, D, device=DEV) * 0.2).to(torch.bfloat16)
    y = (torch.randn(ny, D, device=DEV) * 0.2).to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    outs = []
    for ctas in (1, 7, 148):
        out = torch.zeros(nx, D, device=DEV)
        loss = torch.zeros(1, dtype=torch.float64, device=DEV)
        K.kvsall_fused(x, y, out, loss, status, 0.0, 1.0, True, num_ctas=ctas)
        outs.append((out, loss.item()))
    torch.cuda.synchronize()
    K.check_status(status)
    for o, l in outs[1:]:
        assert (o - outs[0][0]).abs().max() < 1e-2 * outs[0][0].abs().max()
        assert abs(l - outs[0][1]) < 1e-6 * abs(outs[0][1])


@pytest.mark.parametrize("name,code,norm", [("DistMult", 0, False), ("ComplEx", 1, False), ("QMult", 2, True),
                                             ("OMult", 3, True), ("Keci", 4, False)])
def test_lookup_compose_and_backward(name, code, norm):
    torch.manual_seed(1)
    NE, NR, B, D = 500, 20, 333, 64
    E = torch.randn(NE, D, device=DEV, requires_grad=True)
    R = torch.randn(NR, D, device=DEV, requires_grad=True)
    c = torch.tensor([[0.7]], device=DEV, requires_grad=True) if code == 4 else None
    h = torch.randint(0, NE, (B,), device=DEV)
    r = torch.randint(0, NR, (B,), device=DEV)
    hv, rv = E[h], R[r]
    if code == 0:
        q = algebra.compose_distmult(hv, rv)
    elif code == 1:
        q = algebra.compose_complex(hv, rv)
    elif code == 2:
        q = algebra.compose_quaternion(hv, algebra.quaternion_normalizer(rv))
    elif code == 3:
        q = algebra.compose_octonion(hv, rv, True)
    else:
        q, _ = algebra.compose_clifford(hv, rv, D // 2, 0, 1, 0, None, c)
    Q = torch.zeros(B, D, dtype=torch.bfloat16, device=DEV)
    Qf = torch.zeros(B, D, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    Ed, Rd = E.detach().contiguous(), R.detach().contiguous()
    ent_tab = K.pointer_table([Ed], DEV)
    K.lookup_compose(code, norm, h, r, ent_tab, 1, NE, Rd, None if c is None else c.detach(), K.pointer_table([Q], DEV),
                     1, 0, Qf, B, D, status)
    torch.cuda.synchronize()
    K.check_status(status)
    assert torch.allclose(Qf, q.detach(), atol=1e-4, rtol=1e-4)
    assert torch.allclose(Q.float(), q.detach(), atol=3e-2, rtol=2e-2)
    dq = torch.randn(B, D, device=DEV)
    q.backward(dq)
    gE, gR = torch.zeros_like(Ed), torch.zeros_like(Rd)
    gC = torch.zeros(1, 1, device=DEV) if c is not None else None
    K.compose_backward(code, norm, h, r, ent_tab, 1, Rd, None if c is None else c.detach(), dq, K.pointer_table([gE], DEV),
                       gR, gC, B, D)
    torch.cuda.synchronize()
    assert torch.allclose(gE, E.grad, atol=2e-3, rtol=1e-3)
    assert torch.allclose(gR, R.grad, atol=2e-3, rtol=1e-3)
    if c is not None:
        assert torch.allclose(gC, c.grad, atol=1e-2, rtol=1e-3)


def test_positive_correction_matches_dense():
    torch.manual_seed(2)
    NE, B, D, P = 400, 96, 128, 300
    q = (torch.randn(B, D, device=DEV) * 0.3).to(torch.bfloat16)
    e = (torch.randn(NE, D, device=DEV) * 0.3).to(torch.bfloat16)
    counts = torch.randint(0, 9, (P,))
    counts[5] = 130  # one heavy data point spanning several chunks
    offsets = torch.cat([torch.zeros(1, dtype=torch.long), counts.cumsum(0)]).to(DEV)
    values = torch.cat([torch.randperm(NE)[:int(c)] for c in counts]).to(DEV)
    dp = torch.randint(0, P, (B,), device=DEV)
    dp[0] = 5
    first = torch.zeros(B + 1, dtype=torch.int32, device=DEV)
    K.positive_scan(dp, offsets, B, first)
    dq, de = torch.zeros(B, D, device=DEV), torch.zeros(NE, D, device=DEV)
    loss = torch.zeros(1, dtype=torch.float64, device=DEV)
    w, scale = 0.9, 1.0 / 37
    K.positive_correction(dp, offsets, values, first, q, e, dq, de, loss, w, scale, B, D)
    torch.cuda.synchronize()
    Y = torch.zeros(B, NE, device=DEV)
    for i in range(B):
        d = int(dp[i])
        Y[i, values[offsets[d]:offsets[d + 1]]] = 1.0
    assert int(first[-1]) == int(Y.sum())
    s = q.float() @ e.float().t()
    assert abs(loss.item() + w * (Y * s).sum().item()) < 1e-3 * (1 + abs(loss.item()))
    assert torch.allclose(dq, -w * scale * (Y @ e.float()), atol=1e-4, rtol=1e-3)
    assert torch.allclose(de, -w * scale * (Y.t() @ q.float()), atol=1e-4, rtol=1e-3)


@pytest.mark.parametrize("name,code,norm", [("DistMult", 0, False), ("ComplEx", 1, False), ("QMult", 2, True),
                                             ("OMult", 3, True), ("Keci", 4, False)])
@pytest.mark.parametrize("D", [64, 256])
def test_vectorised_lookup_and_owner_backward(name, code, norm, D):
    """The 16-byte-per-thread lookup and the owner-side backward against autograd.  The backward is run as W = 3
    emulated ranks on one device (one launch per rank over the same batch, each keeping the rows it owns), which
    must add up to the single-table gradient."""
    torch.manual_seed(1)
    NE, NR, B, W = 500, 20, 333, 3
    E = torch.randn(NE, D, device=DEV, requires_grad=True)
    R = torch.randn(NR, D, device=DEV, requires_grad=True)
    c = torch.tensor([[0.7]], device=DEV, requires_grad=True) if code == 4 else None
    h = torch.randint(0, NE, (B,), device=DEV)
    r = torch.randint(0, NR, (B,), device=DEV)
    hv, rv = E[h], R[r]
    if code == 0:
        q = algebra.compose_distmult(hv, rv)
    elif code == 1:
        q = algebra.compose_complex(hv, rv)
    elif code == 2:
        q = algebra.compose_quaternion(hv, algebra.quaternion_normalizer(rv))
    elif code == 3:
        q = algebra.compose_octonion(hv, rv, True)
    else:
        q, _ = algebra.compose_clifford(hv, rv, D // 2, 0, 1, 0, None, c)
    assert K.lookup_vec_supported(code, D)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    Ed, Rd = E.detach().contiguous(), R.detach().contiguous()
    cd = None if c is None else c.detach()
    # rows sharded cyclically over W tables on the same device
    rows = (NE + W - 1) // W
    shards = [torch.zeros(rows, D, device=DEV) for _ in range(W)]
    for k in range(W):
        shards[k][: len(range(k, NE, W))] = Ed[k::W]
    Q = [torch.zeros(B + 5, D, dtype=torch.bfloat16, device=DEV) for _ in range(2)]
    ids = [torch.zeros(3, B + 5, dtype=torch.int64, device=DEV) for _ in range(2)]
    Qf = torch.zeros(B, D, device=DEV)
    dp = torch.arange(B, device=DEV) * 7
    K.lookup_compose_vec(code, norm, h, r, dp, K.pointer_table(shards, DEV), W, NE, NR, Rd, cd,
                         K.pointer_table(Q, DEV), 2, 0, 5, Qf, K.pointer_table(ids, DEV), B + 5, B, D, status)
    torch.cuda.synchronize()
    K.check_status(status)
    assert torch.allclose(Qf, q.detach(), atol=1e-4, rtol=1e-4)
    for k in range(2):   # both destinations, at the row offset
        assert torch.allclose(Q[k][5:].float(), q.detach(), atol=3e-2, rtol=2e-2)
        assert torch.equal(ids[k][0, 5:], h) and torch.equal(ids[k][1, 5:], r) and torch.equal(ids[k][2, 5:], dp)
    dq = torch.randn(B, D, device=DEV)
    q.backward(dq)
    gR = torch.zeros_like(Rd)
    gC = torch.zeros(1, 1, device=DEV) if c is not None else None
    gshards = [torch.zeros(rows, D, device=DEV) for _ in range(W)]
    half = [0.25 * dq, 0.75 * dq]   # two partial-gradient buffers summed by the kernel
    for k in range(W):
        K.compose_backward_owner(code, norm, h, r, shards[k], W, k, NE, NR, Rd, cd, None, K.pointer_table(half, DEV),
                                 2, 0, gshards[k], gR, gC, B, D, status)
    torch.cuda.synchronize()
    K.check_status(status)
    gE = torch.zeros_like(Ed)
    for k in range(W):
        gE[k::W] = gshards[k][: len(range(k, NE, W))]
    assert torch.allclose(gE, E.grad, atol=2e-3, rtol=1e-3)
    assert torch.allclose(gR, R.grad, atol=2e-3, rtol=1e-3)
    if c is not None:
        assert torch.allclose(gC, c.grad, atol=1e-2, rtol=1e-3)
    # a bad relation id is reported through the status word, and later launches return at once
    r_bad = r.clone()
    r_bad[7] = NR
    K.lookup_compose_vec(code, norm, h, r_bad, None, K.pointer_table(shards, DEV), W, NE, NR, Rd, cd,
                         K.pointer_table(Q, DEV), 1, 0, 0, None, None, 0, B, D, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 5
    before = gR.clone()
    K.compose_backward_owner(code, norm, h, r, shards[0], W, 0, NE, NR, Rd, cd, dq, None, 0, 0, gshards[0], gR, gC, B,
                             D, status)
    torch.cuda.synchronize()
    assert torch.equal(before, gR)


@pytest.mark.parametrize("kind,name", [(0, "Adam"), (1, "AdamW"), (2, "SGD"), (3, "Adopt")])
def test_optimizer_kernels_match_torch(kind, name):
    torch.manual_seed(3)
    from dice_embeddings_b200.optim import ADOPT
    n = 10_000
    p_ref = torch.nn.Parameter(torch.randn(n, device=DEV))
    p = p_ref.detach().clone()
    wd = 0.01 if kind != 3 else 0.0
    opt = {0: lambda: torch.optim.Adam([p_ref], lr=0.05, weight_decay=wd),
           1: lambda: torch.optim.AdamW([p_ref], lr=0.05, weight_decay=wd),
           2: lambda: torch.optim.SGD([p_ref], lr=0.05, weight_decay=wd),
           3: lambda: ADOPT([p_ref], lr=0.05)}[kind]()
    m, v, g = torch.zeros_like(p), torch.zeros_like(p), torch.zeros_like(p)
    shadow = torch.zeros(n, dtype=torch.bfloat16, device=DEV)
    step = torch.zeros(1, dtype=torch.int64, device=DEV)
    b1, b2, eps = (0.9, 0.9999, 1e-6) if kind == 3 else (0.9, 0.999, 1e-8)
    for _ in range(4):
        grad = torch.randn(n, device=DEV)
        p_ref.grad = grad.clone()
        opt.step()
        g.copy_(grad)
        K.optimizer_step(kind, p, g, m, v, shadow, step, 0.05, b1, b2, eps, wd)
        step += 1
    torch.cuda.synchronize()
    assert torch.allclose(p, p_ref.detach(), atol=1e-5, rtol=1e-4)
    assert float(g.abs().max()) == 0.0
    assert torch.allclose(shadow.float(), p, atol=2e-2, rtol=1e-2)


def test_p2p_barrier_wait_is_bounded():
    """A barrier whose peer never signals gives up after its spin limit and reports it; the context stays usable."""
    sig0 = torch.zeros(2, dtype=torch.int32, device=DEV)
    sig1 = torch.zeros(2, dtype=torch.int32, device=DEV)
    table = K.pointer_table([sig0, sig1], DEV)
    count = torch.zeros(1, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    K.p2p_barrier(table, 0, 2, count, status, spin_limit=2000)
    torch.cuda.synchronize()
    assert int(status.item()) == 4                     # peer wait timed out
    assert int(sig1[0].item()) == 1                    # our own signal was delivered
    with pytest.raises(K.KernelError):
        K.check_status(status)
    # the peer "arrives": the next barrier of the pair completes
    sig0[1] = 2
    K.p2p_barrier(table, 0, 2, count, status, spin_limit=2000)
    torch.cuda.synchronize()
    K.check_status(status)
    assert (torch.ones(4, device=DEV) * 2).sum().item() == 8.0


def test_label_mask_kernels_agree():
    """The three mask builders (one warp per data point; count / scan / one thread per positive; one launch with
    block-local prefix sums) build the same masks (two shards; a graph with a few very heavy data points)."""
    from dice_embeddings_b200.data.datasets import KvsAll
    from dice_embeddings_b200.data.synthetic import zipf_kg
    NE, NR = 900, 9
    ds = KvsAll(zipf_kg(NE, NR, 20000, seed=4), NE, NR).to(DEV)
    offsets, values = ds.offsets.to(DEV).contiguous(), ds.values.to(DEV).contiguous()
    n = 700
    dp = torch.randperm(len(ds), device=DEV)[:n].contiguous()
    for W, rank in ((1, 0), (2, 1)):
        rows = (NE - rank + W - 1) // W
        masks = []
        for variant in ("warp", "scan", "block"):
            mq = torch.zeros(n, K.mask_stride(rows), dtype=torch.int32, device=DEV)
            me = torch.zeros(rows, K.mask_stride(n), dtype=torch.int32, device=DEV)
            first = torch.zeros(n + 1, dtype=torch.int32, device=DEV)
            K.build_label_masks(dp, offsets, values, n, W, rank, mq, me, first=first, variant=variant)
            masks.append((mq, me))
        for k in (1, 2):
            assert torch.equal(masks[0][0], masks[k][0]) and torch.equal(masks[0][1], masks[k][1])
        assert int(masks[0][0].ne(0).sum()) > 0


@pytest.mark.parametrize("n", [1, 31, 700, 4096, 5000, 32768, 65536])
def test_positive_scan_equals_cumsum(n):
    torch.manual_seed(n)
    n_dp = 5000
    counts = torch.randint(0, 9, (n_dp,), device=DEV)
    counts[::97] = 400                                         # a few data points own many positives
    offsets = torch.cat((torch.zeros(1, dtype=torch.int64, device=DEV), counts.cumsum(0))).contiguous()
    dp = torch.randint(0, n_dp, (n,), device=DEV)
    first = torch.full((n + 1,), -1, dtype=torch.int32, device=DEV)
    K.positive_scan(dp, offsets, n, first)
    want = torch.cat((torch.zeros(1, dtype=torch.int64, device=DEV), counts[dp].cumsum(0)))
    assert torch.equal(first.long(), want)


@pytest.mark.parametrize("W,rank,n,D", [(2, 1, 1000, 64), (4, 2, 4096, 256), (8, 5, 3001, 128)])
def test_owned_row_list_and_dq_pull(W, rank, n, D):
    """Reduce-scatter of the partial query gradients as a kernel of its own, with the W ranks' buffers emulated by W
    local tensors: the rows whose head this rank owns are listed exactly once, their partial rows are summed in place
    in this rank's buffer, and every other row of that buffer stays as it was."""
    torch.manual_seed(W * 100 + rank)
    NE = 5000
    h = torch.randint(0, NE, (n,), device=DEV)
    parts = [torch.randn(n, D, device=DEV) for _ in range(W)]
    table = K.pointer_table(parts, DEV)
    rows = torch.zeros(n, dtype=torch.int32, device=DEV)
    count = torch.zeros(1, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    expect = parts[rank].clone()
    owned = (h % W) == rank
    expect[owned] = sum(p[owned] for p in parts)
    K.owned_rows(h, n, W, rank, NE, rows, count, status)
    K.dq_pull_owner(rows, count, table, W, parts[rank], D, status)
    torch.cuda.synchronize()
    K.check_status(status)
    c = int(count)
    assert c == int(owned.sum())
    assert torch.equal(torch.sort(rows[:c].long()).values, owned.nonzero().flatten())
    assert (parts[rank] - expect).abs().max() < 1e-5
    bad = h.clone()
    bad[7] = NE + 3                                      # an id outside the table is reported, not followed
    count.zero_()
    K.owned_rows(bad, n, W, rank, NE, rows, count, status)
    torch.cuda.synchronize()
    assert int(status) != 0
