"""ctypes binding of libdlblas_b200.so (declarations mirror include/dlblas_b200.h).

There is no fallback: if the shared library is missing, or a call fails, an
exception is raised.  `python -m dlcompiler_b200.build` builds the library.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p

import torch

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libdlblas_b200.so")

DTYPE_F16, DTYPE_BF16, DTYPE_F32 = 0, 1, 2
SCORE_SIGMOID, SCORE_SOFTMAX = 0, 1
GEMM_FUSE_SILU, GEMM_WEIGHT, GEMM_SCATTER, GEMM_PEER = 1, 2, 4, 8

_DTYPES = {torch.float16: DTYPE_F16, torch.bfloat16: DTYPE_BF16, torch.float32: DTYPE_F32}

# name -> (restype, argtypes); the order of arguments is the one in include/dlblas_b200.h
SIGNATURES = {
    "dlb_version": (c_int, []),
    "dlb_last_error": (c_char_p, []),
    "dlb_set_wait_budget_ms": (c_int, [c_int64]),
    "dlb_moe_start_end": (c_int, [c_void_p, c_int, c_int64, c_int, c_void_p, c_void_p, c_int, c_void_p]),
    "dlb_silu_and_mul": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "dlb_grouped_topk_gating": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int64, c_int,
                                        c_int, c_int, c_int, c_int, c_float, c_void_p]),
    "dlb_gshard_gate": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "dlb_gshard_assign": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int64, c_void_p,
                                  c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_void_p]),
    "dlb_gshard_gate_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "dlb_gshard_gate_bwd_weights": (c_int, [c_void_p] * 7 + [c_int64, c_int, c_int, c_int64, c_void_p]),
    "dlb_moe_align_block_size": (c_int, [c_void_p, c_int, c_int64, c_int, c_int, c_void_p, c_int64, c_void_p,
                                         c_int64, c_void_p, c_void_p, c_void_p]),
    "dlb_moe_permute_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int64, c_int64,
                                     c_int64, c_int, c_void_p]),
    "dlb_moe_grouped_gemm": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int, c_int64, c_int64, c_int64,
                                     c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int,
                                     c_int, c_void_p, c_void_p]),
    "dlb_moe_grouped_gemm_sync": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int, c_int64, c_int64, c_int64,
                                          c_void_p, c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                          c_void_p, c_void_p]),
    "dlb_ep_route": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_int, c_int, c_int, c_int64, c_int, c_void_p, c_void_p]),
    "dlb_ep_send": (c_int, [c_void_p, c_int64, c_int64, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                            c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int64,
                            c_int, c_void_p]),
    "dlb_ep_combine": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int64, c_int64, c_int, c_void_p, c_int, c_int,
                               c_void_p, c_void_p, c_void_p]),
    "dlb_ep_combine_pull": (c_int, [c_void_p, c_int64, c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int, c_int64,
                                    c_int64, c_int, c_void_p, c_int, c_int, c_int64, c_int, c_void_p, c_void_p]),
    "dlb_ep_barrier": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "dlb_moe_combine": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int64, c_int64, c_int, c_void_p, c_int,
                                c_int64, c_int64, c_void_p]),
    "dlb_flash_prefill_varlen": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                                         c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                                         c_float, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "dlb_flash_prefill_paged": (c_int, [c_void_p] * 9 + [c_int64] * 21 + [c_int, c_int64, c_float, c_float, c_int, c_void_p,
                                                                      c_void_p, c_int, c_void_p, c_void_p]),
    "dlb_paged_decode_workspace_floats": (c_int64, [c_int64, c_int64, c_int64, c_int64]),
    "dlb_paged_decode": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                                 c_int64, c_int64, c_int64, c_int64,
                                 c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                                 c_int64, c_int, c_int, c_int64, c_int64, c_int64, c_float, c_float, c_int,
                                 c_void_p, c_void_p]),
    "dlb_rms_norm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                             c_int64, c_float, c_int, c_int, c_void_p]),
    "dlb_apply_rotary": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int,
                                 c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int,
                                 c_void_p]),
    "dlb_fill_kv_cache": (c_int, [c_void_p] * 8 + [c_int64] * 19 + [c_int] * 5 + [c_void_p, c_void_p, c_int, c_void_p]),
    "dlb_paged_decode_static": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                                        c_int64, c_int64, c_int64, c_int64,
                                        c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                                        c_int64, c_int, c_int, c_int64, c_int64, c_int64, c_float, c_float, c_int,
                                        c_void_p, c_void_p]),
}

DECODE_STATIC_FLOATS = 8 * 1024 * 1024

_lib = None


class DlblasError(RuntimeError):
    """A libdlblas_b200 entry point returned a non-zero status."""


def load() -> ctypes.CDLL:
    """Load the shared library (once) and attach the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise DlblasError(
            f"{LIB_PATH} is missing: build it with `python -m dlcompiler_b200.build` "
            "(there is no CPU or PyTorch fallback for these ops)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def is_built() -> bool:
    return os.path.exists(LIB_PATH)


def check(rc: int, what: str) -> None:
    """Turn a status code into an exception: negative codes are argument errors."""
    if rc == 0:
        return
    msg = load().dlb_last_error().decode(errors="replace")
    if rc < 0:
        raise AssertionError(f"{what}: {msg} (status {rc})")
    raise DlblasError(f"{what}: {msg} (cudaError {rc})")


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise AssertionError(f"unsupported dtype {t.dtype}") from None


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def stream_ptr(device=None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise AssertionError("dlcompiler_b200 ops run on CUDA tensors only (no CPU fallback)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise AssertionError("all tensors must be on the same CUDA device")
    return dev


_status_words: dict[int, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32[4] the tensor-core kernels write when a bounded wait gives up."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status_words.get(idx)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=device)
        _status_words[idx] = t
    return t


def existing_status_word(device: torch.device):
    """The device's status word if some earlier call created it, else None (the kernels take NULL).
    For call paths that must not allocate."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    return _status_words.get(idx)


def set_wait_budget_ms(ms: int) -> None:
    """Limit, in milliseconds, of every wait on a flag raised by another GPU (default 2000)."""
    check(load().dlb_set_wait_budget_ms(int(ms)), "set_wait_budget_ms")


def check_device_status(device=None) -> None:
    """Synchronise and raise if any kernel recorded a timed-out wait since the last check."""
    devs = list(_status_words) if device is None else [torch.device(device).index or 0]
    for idx in devs:
        t = _status_words.get(idx)
        if t is None:
            continue
        vals = t.cpu().tolist()
        if vals[0] != 0:
            t.zero_()
            raise DlblasError(
                f"device status on cuda:{idx}: code={vals[0]} wait_site={vals[1]} block={vals[2]} aux={vals[3]}")
