"""ctypes binding of libvexact_b200.so (the C ABI in include/vexact_b200.h).

The product path never falls back to another implementation: if the library is
missing `load()` raises, and every wrapper raises `B200Error` on a non-zero
return code.
"""
from __future__ import annotations

import ctypes as C
import threading
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "_C" / "libvexact_b200.so"
_lock = threading.Lock()
_lib = None

P, LL, I, F = C.c_void_p, C.c_longlong, C.c_int, C.c_float

# name -> argument types (return type is always int).  Mirrors include/vexact_b200.h.
SIGNATURES = {
    "b200_abi_version": [],
    "b200_status_read": [C.POINTER(C.c_int), P],
    "b200_gemm_bf16": [P, P, P, P, LL, I, I, LL, LL, LL, I, P],
    "b200_gemm_f16": [P, P, P, P, LL, I, I, LL, LL, LL, I, P],
    "b200_gemm_f32": [P, P, P, P, LL, I, I, LL, LL, LL, P],
    "b200_gemm_f32_from_bf16": [P, P, P, LL, I, I, LL, LL, LL, P],
    "b200_rmsnorm": [P, P, P, LL, I, LL, LL, F, I, P],
    "b200_rmsnorm_backward": [P, P, P, P, P, P, LL, I, F, P],
    "b200_add_rmsnorm": [P, P, P, P, P, LL, I, F, I, P],
    "b200_mean_lastdim": [P, P, LL, I, LL, I, P],
    "b200_log_softmax_f32": [P, P, LL, I, LL, LL, P],
    "b200_gather_logprob": [P, P, P, LL, I, LL, I, LL, P],
    "b200_gather_logprob_backward": [P, P, P, P, LL, I, LL, LL, I, LL, P],
    "b200_greedy_logprob": [P, P, P, LL, I, LL, I, P],
    "b200_lm_head_greedy": [P, P, P, P, P, LL, I, I, LL, LL, P],
    "b200_sample_token": [P, P, P, P, LL, I, LL, LL, I, F, I, F, P],
    "b200_apply_top_k_top_p": [P, P, LL, I, LL, LL, I, F, I, F, P],
    "b200_seeded_exponential": [P, P, P, LL, I, LL, P],
    "b200_gather_rows": [P, LL, LL, P, P, P, LL, I, P],
    "b200_moe_route_plan_softmax_topk": [P, I, LL, P, P, P, P, P, P, P, LL, I, I, I, I, I, P],
    "b200_moe_scatter_ranked": [P, LL, P, P, P, P, P, P, P, LL, I, I, I, P],
    "b200_selftest_wait_expiry": [I, P, P],
    "b200_prepare_step": [P, P, P, P, P, P, I, I, I, I, I, P, P, P, P, P, P, P, P],
    "b200_kv_store": [P, P, P, P, P, LL, I, I, I, LL, LL, LL, P],
    "b200_qknorm_rope_store": [P, LL, P, P, P, P, P, P, P, P, LL, I, I, I, LL, F, P],
    "b200_mla_rope_store": [P, LL, P, LL, P, LL, P, P, P, P, P, P, LL, I, I, I, I, LL, P],
    "b200_paged_attn_fwd": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, LL, LL, LL, LL, LL, LL, LL, LL, LL,
                            LL, LL, F, P],
    "b200_paged_attn_fwd_ordered": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, LL, LL, LL, LL, LL, LL, LL, LL, LL,
                            LL, LL, F, P, LL, P],
    "b200_moe_route_softmax_topk": [P, I, LL, P, P, P, P, LL, I, I, I, P],
    "b200_moe_route_sigmoid_group_topk": [P, LL, P, P, P, P, LL, I, I, I, I, I, F, P],
    "b200_moe_permute": [P, I, P, P, LL, P, P, P, P, P, P, LL, I, I, I, I, I, P],
    "b200_moe_grouped_gemm": [P, P, P, P, P, P, LL, I, I, I, LL, I, I, I, P],
    "b200_moe_permute_index": [P, I, P, P, P, P, P, P, P, LL, I, I, I, I, P],
    "b200_moe_grouped_gemm_gather": [P, LL, LL, P, P, P, P, P, P, I, I, I, LL, I, I, I, P],
    "b200_moe_grouped_gemm_noalloc": [P, P, P, P, P, LL, I, I, I, LL, I, P],
    "b200_swiglu_scale": [P, P, P, P, LL, I, P],
    "b200_swiglu_scale_strided": [P, P, P, P, LL, I, LL, P],
    "b200_moe_unpermute_reduce": [P, P, P, P, LL, I, I, P],
    "b200_moe_scatter": [P, LL, P, LL, LL, P, LL, LL, I, I, P],
    "b200_moe_gather": [P, LL, P, LL, LL, P, LL, I, I, P],
    "b200_moe_grouped_wgrad": [P, P, P, P, LL, I, I, I, P],
    "b200_transpose_last2": [P, P, I, I, I, P],
    "b200_varlen_attn_backward": [P, P, P, P, P, P, P, P, P, P, P, P, I, I, I, LL, LL, I, I, I, I, F, P],
    "b200_moe_unpermute_add_rmsnorm": [P, P, P, P, P, P, P, LL, I, I, F, I, P],
}

_ERRORS = {
    -1: "invalid argument",
    -2: "unsupported shape",
    -3: "CUDA launch error",
    -4: "driver entry point (tensor-map encoder) unavailable",
}


class B200Error(RuntimeError):
    pass


ABI_VERSION = 4


def _check_fresh(lib) -> None:
    """Refuse a library built from other sources than the ones beside this file: its entry points
    may take other argument lists than SIGNATURES declares."""
    from . import build

    if not build.sources_present():
        return
    try:
        fn = lib.b200_source_hash
    except AttributeError:
        raise B200Error(f"{_LIB_PATH} predates the source-hash check: rebuild it with "
                        "`python -m vexact_b200.build --force`") from None
    fn.restype = C.c_char_p
    have, want = fn().decode(), build._source_hash()
    if have != want:
        raise B200Error(f"{_LIB_PATH} was built from other sources (hash {have[:12]}, sources {want[:12]}): "
                        "rebuild it with `python -m vexact_b200.build`")


def lib_path() -> Path:
    return _LIB_PATH


def load() -> C.CDLL:
    """Load the shared library (built by `vexact_b200.build.build()`); raises if it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not _LIB_PATH.exists():
                raise B200Error(
                    f"{_LIB_PATH} not found: build it with `python -m vexact_b200.build` "
                    "(there is no fallback implementation)"
                )
            lib = C.CDLL(str(_LIB_PATH))
            _check_fresh(lib)
            for name, argtypes in SIGNATURES.items():
                fn = getattr(lib, name)
                fn.argtypes = argtypes
                fn.restype = C.c_int
            if lib.b200_abi_version() != ABI_VERSION:
                raise B200Error(f"{_LIB_PATH} has ABI version {lib.b200_abi_version()}, this binding needs "
                                f"{ABI_VERSION}: rebuild it with `python -m vexact_b200.build --force`")
            _lib = lib
    return _lib


# Kernels launched by one successful call of each entry point (for launch accounting).
_KERNELS_PER_CALL = {"b200_moe_permute": 2, "b200_lm_head_greedy": 2, "b200_rmsnorm_backward": 3, "b200_status_read": 0, "b200_abi_version": 0}
_launches = 0


def check(rc: int, what: str) -> None:
    global _launches
    if rc != 0:
        raise B200Error(f"{what} failed: {_ERRORS.get(rc, rc)}")
    _launches += _KERNELS_PER_CALL.get(what, 1)


def reset_launch_count() -> None:
    global _launches
    _launches = 0


def launch_count() -> int:
    """Kernels of this library launched (or captured) since the last reset."""
    return _launches


def ptr(t) -> int | None:
    """Device pointer of a torch tensor (None passes NULL)."""
    return None if t is None else t.data_ptr()


def current_stream() -> int:
    import torch

    return torch.cuda.current_stream().cuda_stream


def read_status() -> tuple[int, int, int, int]:
    out = (C.c_int * 4)()
    check(load().b200_status_read(out, current_stream()), "b200_status_read")
    return tuple(out)
