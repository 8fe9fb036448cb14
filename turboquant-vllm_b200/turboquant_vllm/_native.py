"""ctypes binding of libtq4_sm100a.so (the C ABI declared in include/tq4.h).

There is no CPU or Triton fallback: if the library is missing, or a tensor is not on a CUDA
device, the call raises.  The library is built in-tree by ``turboquant-vllm_b200/build.py``.
"""

from __future__ import annotations

import contextlib
import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p

import torch

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libtq4_sm100a.so")
_lib = None

F32, F16, BF16 = 0, 1, 2
_DTYPE_CODE = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}

DEV_BAD_SLOT, DEV_BAD_BLOCK, DEV_TIMEOUT, DEV_WRITE_ORDER = 1, 2, 4, 8
STATIC_SCRATCH_BYTES = 32 << 20

# name -> (restype, argtypes); must list every symbol of include/tq4.h
_SIGNATURES = {
    "tq4_version": (c_char_p, []),
    "tq4_status_string": (c_char_p, [c_int]),
    "tq4_compress_rows": (c_int, [c_void_p, c_int, c_int64, c_int, c_int, c_int64, c_int64,
                                  c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "tq4_pack_rotated_rows": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_int, c_void_p, c_void_p]),
    "tq4_write_paged": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int, c_int,
                                c_int64, c_int64, c_int64, c_int64, c_void_p, c_int64,
                                c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "tq4_decompress_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int,
                                    c_void_p, c_int, c_void_p]),
    "tq4_decompress_cache": (c_int, [c_void_p, c_int64, c_int64, c_int, c_int, c_void_p, c_int,
                                     c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p]),
    "tq4_attention_workspace_bytes": (c_size_t, [c_int64, c_int, c_int, c_int]),
    "tq4_paged_attention": (c_int, [c_void_p, c_int, c_int64, c_int, c_int, c_int, c_int,
                                    c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64, c_int,
                                    c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int,
                                    c_void_p, c_int, c_void_p, c_float, c_int, c_int,
                                    c_void_p, c_int, c_int64, c_int64, c_void_p, c_int,
                                    c_void_p, c_size_t, c_int, c_void_p, c_void_p]),
    "tq4_write_and_attention": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int64,
                                        c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                        c_void_p, c_int, c_int64, c_int, c_int, c_int, c_int,
                                        c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64, c_int,
                                        c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int,
                                        c_void_p, c_int, c_void_p, c_float, c_int, c_int,
                                        c_void_p, c_int, c_int64, c_int64, c_void_p, c_int,
                                        c_void_p, c_size_t, c_int, c_void_p, c_void_p]),
    "tq4_combine_partials": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_void_p,
                                     c_void_p, c_int, c_int64, c_int64, c_void_p]),
    "tq4_paged_attention_static": (c_int, [c_void_p, c_int, c_int64, c_int, c_int, c_int, c_int,
                                           c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64, c_int,
                                           c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int,
                                           c_void_p, c_int, c_void_p, c_float, c_int, c_int,
                                           c_void_p, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "tq4_profile_start": (c_int, [c_int]),
    "tq4_profile_stop": (c_int, []),
    "tq4_profile_read": (c_int, [c_int, c_void_p, c_int]),
}

PROF_WRITE, PROF_PROLOGUE, PROF_ATTENTION, PROF_COMBINE, PROF_COMPRESS = range(5)


def profile_start(max_samples: int) -> None:
    check(lib().tq4_profile_start(max_samples), "tq4_profile_start")


def profile_stop() -> None:
    lib().tq4_profile_stop()


def profile_read(kind: int, max_samples: int) -> list[float]:
    buf = (c_float * max_samples)()
    n = lib().tq4_profile_read(kind, ctypes.cast(buf, c_void_p), max_samples)
    if n < 0:
        raise RuntimeError("tq4_profile_read failed")
    return [float(buf[i]) for i in range(n)]


def library_path() -> str:
    return _LIB_PATH


def exported_symbols() -> list[str]:
    return sorted(_SIGNATURES)


def lib() -> ctypes.CDLL:
    """Load the CUDA library once; raise loudly when it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise RuntimeError(
                f"TQ4 CUDA library not found at {_LIB_PATH}. Build it with "
                "`python turboquant-vllm_b200/build.py` (needs nvcc, targets sm_100a). "
                "There is no CPU or Triton fallback."
            )
        handle = ctypes.CDLL(_LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the .so is stale
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status: int, what: str) -> None:
    if status != 0:
        msg = lib().tq4_status_string(status).decode()
        if status == 2:
            raise NotImplementedError(f"{what}: {msg}")
        if status == 5:
            raise ValueError(f"{what}: {msg}")
        raise RuntimeError(f"{what}: {msg} (tq4 status {status})")


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dt]
    except KeyError:
        raise TypeError(f"TQ4 kernels support float32/float16/bfloat16, got {dt}") from None


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "TQ4 kernels run on CUDA tensors only (sm_100a); got a tensor on "
                f"{t.device}. There is no CPU fallback in this package."
            )


_NO_GUARD = contextlib.nullcontext()


def device_guard(device: torch.device):
    """Context that makes ``device`` the current CUDA device for the duration of a library call.

    The C entry points launch on the current device (kernel attributes, the SM count and the
    built-in scratch are looked up for it), so tensors on ``cuda:1`` need ``cuda:1`` current even
    when the caller left ``cuda:0`` selected, as HuggingFace models spread with ``device_map`` do.
    """
    idx = device.index
    if idx is None or idx == torch.cuda.current_device():
        return _NO_GUARD
    return torch.cuda.device(idx)


def call(device: torch.device, name: str, *args):
    """Call entry point ``name`` with ``device`` current."""
    with device_guard(device):
        return getattr(lib(), name)(*args)


_DEV_BITS = ((DEV_BAD_SLOT, "slot_mapping entry outside the cache (TQ4_DEV_BAD_SLOT)"),
             (DEV_BAD_BLOCK, "block_table entry outside [0, num_blocks) or sequence longer than its "
                             "block-table row (TQ4_DEV_BAD_BLOCK)"),
             (DEV_TIMEOUT, "a bounded device-side wait gave up (TQ4_DEV_TIMEOUT)"),
             (DEV_WRITE_ORDER, "a fused decode step wrote a token to a slot that is not the last position of "
                               "its sequence (TQ4_DEV_WRITE_ORDER)"))


def describe_device_errors(flag: int) -> str:
    """Text for the TQ4_DEV_* bits a kernel OR-ed into the device error flag."""
    parts = [text for bit, text in _DEV_BITS if flag & bit]
    rest = flag & ~(DEV_BAD_SLOT | DEV_BAD_BLOCK | DEV_TIMEOUT | DEV_WRITE_ORDER)
    if rest:
        parts.append(f"unknown bits {rest:#x}")
    return "; ".join(parts) if parts else "no error"


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()
