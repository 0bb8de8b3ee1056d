"""Build and load the sm_100a kernel library.

All CUDA sources under ``csrc/`` are compiled by ``nvcc`` into one shared object that sits next to this file
(``libdice_b200.so``) and is loaded with :mod:`ctypes`.  The exported entry points are plain ``extern "C"``
functions taking raw device pointers and a stream handle, so no PyTorch headers are needed to build
(a full rebuild takes seconds) and non-Python callers can link the same library.  The only supported target is
``sm_100a``; there is no fallback build for other architectures.
"""
from __future__ import annotations

import ctypes
import glob
import os
import subprocess
from typing import Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(os.path.dirname(_HERE))
CSRC = os.path.join(_ROOT, "csrc")
LIB_PATH = os.path.join(_HERE, "libdice_b200.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared",
              "-Xcompiler", "-fPIC"]

_lib: Optional[ctypes.CDLL] = None


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def needs_build() -> bool:
    if not os.path.isfile(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h"))
    return any(os.path.getmtime(s) > t for s in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile ``csrc/*.cu`` for sm_100a into ``libdice_b200.so`` (no-op when up to date).

    Several processes may call this at once (every rank of a ``torchrun`` job on a fresh checkout): the build runs
    under an exclusive file lock, into a file of the process's own, and is published with an atomic rename; a process
    that waited for the lock finds the library up to date and does not compile again."""
    if not force and not needs_build():
        return LIB_PATH
    import fcntl
    with open(LIB_PATH + ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and not needs_build():   # another process built it while this one waited
                return LIB_PATH
            nvcc = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
            if not os.path.isfile(nvcc):
                nvcc = "nvcc"
            tmp = f"{LIB_PATH}.{os.getpid()}.tmp"
            cmd = [nvcc, *NVCC_FLAGS, *sources(), "-o", tmp]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                if os.path.exists(tmp):
                    os.remove(tmp)
                raise RuntimeError(f"nvcc failed:\n{' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
            if verbose:
                print(res.stderr)
            os.replace(tmp, LIB_PATH)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return LIB_PATH


def available() -> bool:
    """True when the library file exists (it may still need a B200 to run)."""
    return os.path.isfile(LIB_PATH)


def lib() -> ctypes.CDLL:
    """Load (building first if the sources are newer and a compiler is present)."""
    global _lib
    if _lib is None:
        if needs_build():
            try:
                build()
            except (RuntimeError, FileNotFoundError):
                if not os.path.isfile(LIB_PATH):
                    raise
        _lib = ctypes.CDLL(LIB_PATH)
        for name in dir(_Sigs):
            if name.startswith("dice_"):
                fn = getattr(_lib, name)
                fn.restype = ctypes.c_int
                fn.argtypes = getattr(_Sigs, name)
    return _lib


_p = ctypes.c_void_p
_i = ctypes.c_int
_l = ctypes.c_longlong
_f = ctypes.c_float
_d = ctypes.c_double


class _Sigs:
    dice_kvsall_fused = [_p, _i, _p, _i, _i, _p, _p, _f, _f, _i, _p, _i, _p, _i, _f, _p, _i, _p, _p, _p, _f, _p, _p]
    dice_kvsall_pair = [_p, _i, _p, _i, _i, _p, _p, _f, _f, _i, _p, _i, _p, _i, _f, _i, _p, _p]
    dice_build_label_masks = [_p, _p, _p, _i, _i, _i, _p, _i, _p, _i, _p]
    dice_build_label_masks_flat = [_p, _p, _p, _p, _i, _i, _i, _p, _i, _p, _i, _l, _l, _p, _p]
    dice_lookup_vec_supported = [_i, _i]
    dice_lookup_compose_vec = [_i, _i, _p, _p, _i, _p, _p, _i, _l, _i, _p, _p, _p, _i, _p, _l, _p, _p, _l, _i, _i, _p, _p]
    dice_compose_backward_owner = [_i, _i, _p, _p, _i, _p, _i, _i, _l, _i, _p, _p, _p, _p, _i, _p, _p, _p, _p, _i, _i, _p, _p]
    dice_owned_rows = [_p, _i, _i, _i, _i, _l, _p, _p, _p, _p]
    dice_dq_pull_owner = [_p, _p, _p, _i, _p, _i, _p, _p]
    dice_bucket_reduce_update = [_i, _p, _p, _p, _p, _p, _p, _p, _p, _l, _l, _i, _f, _f, _f, _f, _f, _f, _p, _p]
    dice_step_tail = [_i, _i, _p, _p, _p, _p, _p, _p, _p, _p, _i, _p, _f, _f, _f, _f, _f, _p, _p, _d, _p, _i, _p, _p, _p]
    dice_positive_correction_noalloc = [_p, _p, _p, _p, _p, _p, _p, _p, _f, _f, _i, _i, _i, _i, _p]
    dice_lookup_compose = [_i, _i, _p, _p, _p, _i, _l, _p, _p, _p, _i, _l, _p, _i, _i, _p, _p, _p, _p]
    dice_compose_backward = [_i, _i, _p, _p, _p, _i, _p, _p, _p, _p, _p, _p, _i, _i, _p, _p, _i, _l, _p]
    dice_positive_scan = [_p, _p, _i, _p, _p]
    dice_positive_correction = [_p, _p, _p, _p, _p, _p, _p, _p, _p, _f, _f, _i, _i, _i, _i, _p, _i, _p]
    dice_optimizer_step = [_i, _p, _p, _p, _p, _p, _p, _l, _f, _f, _f, _f, _f, _p, _i, _p, _p, _p]
    dice_cast_bf16 = [_p, _p, _l, _p]
    dice_finish_step = [_p, _p, _d, _p, _p, _i, _p, _p]
    dice_p2p_barrier = [_p, _i, _i, _p, _p, ctypes.c_uint, _p]
    dice_timestamp = [_p, _p]
    dice_uniform_int = [_p, _l, _l, ctypes.c_ulonglong, ctypes.c_ulonglong, _p, _l, _l, _p]
    dice_neg_sample = [_p, _i, _i, _l, ctypes.c_ulonglong, ctypes.c_ulonglong, _p, _i, _f, _f, _p, _p, _p, _p, _p, _p]
    dice_candidate_bce = [_p, _p, _l, _l, _i, _p, _p, _p, _p, _p, _p, _f, _i, _f, _f, _i, _i, _i, _p, _l, _p, _p]
    dice_sparse_rows_optimizer = [_i, _p, _p, _p, _p, _p, _p, _l, _i, _p, _f, _f, _f, _f, _f, _p]
    dice_eval_rank = [_p, _i, _p, _i, _i, _p, _p, _p, _i, _i, _p, _i, _i, _p, _p, _p, _p, _i, _p, _p, _p, _p, _l, _p, _p]
    dice_eval_rank_cand_cap = [_i, _i, _i, _i, _i]
    dice_conv_gate_supported = [_i, _i, _i, _i]
    dice_conv_gate_forward = [_i, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p, _p, _f, _f, _p, _p, _p, _p]
    dice_conv_gate_backward = [_i, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p, _p, _p, _p]
    dice_peer_sum_f32 = [_p, _i, _p, _i, _p, _p]
    dice_merge_ranks = [_p, _p, _i, _p, _i, _p, _p]
    dice_merge_topk = [_p, _p, _i, _i, _l, _p, _p, _i, _p, _p]
    dice_eval_sparse = [_p, _p, _i, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p, _p, _i, _p]
    dice_eval_band_exact = [_p, _p, _i, _i, _i, _i, _p, _p, _p, _p, _l, _p, _p, _p]
