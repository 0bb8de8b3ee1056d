"""Allocation-free positive-correction entry point, called through its exported C symbol.

Callers that cannot allocate device memory (code inside a stream capture, plug-ins without access to the host
framework's allocator, thin foreign-language bindings) use ``dice_positive_correction_noalloc``: its prefix-sum
scratch is a fixed array inside the library.  The test checks it against the regular two-call entry point
(``dice_positive_scan`` + ``dice_positive_correction`` with a caller-allocated scratch) on two consecutive calls,
because the built-in scratch keeps the previous call's contents.  This file sorts last so that a failure here
cannot hide other tests under ``pytest -x``.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("CUDA device required", allow_module_level=True)

from dice_embeddings_b200.ops import _lib
from dice_embeddings_b200.ops import kernels as K

DEV = torch.device("cuda:0")


def _noalloc_symbol():
    lib = _lib.lib()   # builds the library first when the tree is fresh; the symbol is then taken from that handle
    fn = lib.dice_positive_correction_noalloc
    p, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.restype = ctypes.c_int
    fn.argtypes = [p, p, p, p, p, p, p, p, f, f, i, i, i, i, p]
    return fn


def _case(seed, B, NE=600, D=128, P=500):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(B, D, generator=g) * 0.3).to(torch.bfloat16).to(DEV)
    e = (torch.randn(NE, D, generator=g) * 0.3).to(torch.bfloat16).to(DEV)
    counts = torch.randint(0, 7, (P,), generator=g)
    counts[3] = 90
    offsets = torch.cat([torch.zeros(1, dtype=torch.long), counts.cumsum(0)]).to(DEV)
    values = torch.cat([torch.randperm(NE, generator=g)[: int(c)] for c in counts]).to(DEV)
    dp = torch.randint(0, P, (B,), generator=g).to(DEV)
    return q, e, offsets, values, dp


def test_noalloc_matches_regular_entry_point_twice():
    fn = _noalloc_symbol()
    stream = torch.cuda.current_stream().cuda_stream
    # two different problems back to back: the second call finds the first call's prefix sums in the scratch
    for seed, B in ((11, 257), (12, 96)):
        q, e, offsets, values, dp = _case(seed, B)
        NE, D = e.shape
        w, scale = 0.9, 1.0 / 41
        dq_ref, de_ref = torch.zeros(B, D, device=DEV), torch.zeros(NE, D, device=DEV)
        loss_ref = torch.zeros(1, dtype=torch.float64, device=DEV)
        first = torch.zeros(B + 1, dtype=torch.int32, device=DEV)
        K.positive_scan(dp, offsets, B, first)
        K.positive_correction(dp, offsets, values, first, q, e, dq_ref, de_ref, loss_ref, w, scale, B, D)
        dq, de = torch.zeros(B, D, device=DEV), torch.zeros(NE, D, device=DEV)
        loss = torch.zeros(1, dtype=torch.float64, device=DEV)
        rc = fn(dp.data_ptr(), offsets.data_ptr(), values.data_ptr(), q.data_ptr(), e.data_ptr(), dq.data_ptr(),
                de.data_ptr(), loss.data_ptr(), w, scale, B, D, 1, 0, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.allclose(dq, dq_ref, atol=1e-4, rtol=1e-3)
        assert torch.allclose(de, de_ref, atol=1e-4, rtol=1e-3)
        assert abs(loss.item() - loss_ref.item()) < 1e-3 * (1 + abs(loss_ref.item()))
        # and against the dense fp32 statement of the same correction
        Y = torch.zeros(B, NE, device=DEV)
        for i in range(B):
            d = int(dp[i])
            Y[i, values[offsets[d]:offsets[d + 1]]] = 1.0
        s = q.float() @ e.float().t()
        assert abs(loss.item() + w * (Y * s).sum().item()) < 1e-3 * (1 + abs(loss.item()))
        assert torch.allclose(dq, -w * scale * (Y @ e.float()), atol=1e-4, rtol=1e-3)
        assert torch.allclose(de, -w * scale * (Y.t() @ q.float()), atol=1e-4, rtol=1e-3)


def test_noalloc_rejects_oversized_batches():
    fn = _noalloc_symbol()
    q, e, offsets, values, dp = _case(13, 8)
    z = torch.zeros(8, e.shape[1], device=DEV)
    loss = torch.zeros(1, dtype=torch.float64, device=DEV)
    rc = fn(dp.data_ptr(), offsets.data_ptr(), values.data_ptr(), q.data_ptr(), e.data_ptr(), z.data_ptr(),
            z.data_ptr(), loss.data_ptr(), 1.0, 1.0, 65537, e.shape[1], 1, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == -7
