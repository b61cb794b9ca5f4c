"""Loads the sm_100a kernel library and declares its C entry points.

There is no fallback: a missing library, a missing CUDA device or a device
that is not sm_100 raises `KernelLibraryError` on the first use of any
kernel. The library is built on first use (see `csrc/build.py`).
"""
from __future__ import annotations

import ctypes
from ctypes import c_double, c_float, c_int, c_longlong, c_void_p

import torch

from ..csrc import build as _build


class KernelLibraryError(RuntimeError):
    pass


class KernelError(RuntimeError):
    """A launcher refused its arguments or a launch failed."""


_lib: ctypes.CDLL | None = None

P = c_void_p
_SIGNATURES: dict[str, list] = {
    "mynah_embed_gather": [P, c_int, P, P, c_int, c_int, c_int, P],
    "mynah_rmsnorm": [P, P, P, c_int, P, P, c_int, c_int, c_int, c_float, P],
    "mynah_residual_add": [P, P, c_int, c_longlong, P],
    "mynah_swiglu": [P, P, c_int, c_int, c_int, P],
    "mynah_gemm_f32": [P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, P],
    "mynah_rope_table": [P, P, c_int, c_int, c_double, P],
    "mynah_qk_norm_rope_store": [P, c_int, c_int, c_int, c_int, c_int, c_int,
                                 P, P, c_int, c_float,
                                 P, P, c_int, c_int,
                                 P, P,
                                 P, P, P, c_int,
                                 P, P, P, P],
    "mynah_attn_prefill_generic": [P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                   P, P, P, P,
                                   P, P, P, c_int,
                                   c_int, P, P],
    "mynah_attn_decode": [P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                          P, P, P,
                          P, P, P, c_int,
                          c_int, c_int, P, P, P],
    "mynah_attn_prefill_tc": [P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                              P, P, P, P,
                              P, P, P, c_int,
                              c_int, P, P],
    "mynah_attn_decode_tc": [P, P, c_int, c_int, c_int, c_int, c_int, c_int,
                             P, P, P,
                             P, P, P, c_int,
                             c_int, c_int, P, P, P, P],
    "mynah_gemm_qkv_rope": [P, P, c_int, c_int, c_int, c_int, c_int,
                            P, P, c_int, c_float,
                            P, P, c_int,
                            P, P,
                            P, P, P, c_int,
                            P, c_int, P, P,
                            c_int, P, P],
    "mynah_attn_prefill_tcgen05": [P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                   P, P, P, P,
                                   P, P, P, c_int,
                                   c_int, P, P],
    "mynah_attn_decode_fused": [P, P, c_int, c_int, c_int, c_int, c_int, c_int,
                                P, P, c_int, c_float,
                                P, P, c_int, P,
                                P, P, c_int, P,
                                P, P, P, c_int,
                                c_int, c_int, P, P, P, P],
    "mynah_gemv_decode": [P, c_int, c_int, c_int, P, P, P, P, P, c_int, c_float, P, c_int, c_int, c_int, P],
    "mynah_gemm_tcgen05": [P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, P, P],
    "mynah_argmax": [P, c_int, c_int, c_int, P, P],
    "mynah_set_pdl": [c_int],
    "mynah_gemm_tcgen05_reset": [P],
    "mynah_sample": [P, c_int, c_int, c_int, P, P, P, P, P, P, P],
    "mynah_apply_penalties": [P, c_int, c_int, c_int, P, P, c_int, P, P, P],
    "mynah_decode_advance": [P, P, P, P, P, c_int, P],
    "mynah_sampler_accept": [P, c_int, P, P, P, c_int, P, P, P],
    "mynah_l2_prefetch": [P, P, c_int, P],
    "mynah_attn_prefill_tcgen05_stages": [c_int],
    "mynah_wait_probe": [P, P, ctypes.c_ulonglong, P],
    "mynah_read_probe": [P, P, c_int, c_int, c_int, P, P, P],
    "mynah_randn_fill": [P, c_int, c_longlong, ctypes.c_ulonglong, ctypes.c_ulonglong, c_double, c_double, P],
}


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not torch.cuda.is_available():
        raise KernelLibraryError("mynah_slm_b200 runs on a CUDA device of compute capability 10.0 (B200); "
                                 "no CUDA device is available and there is no CPU fallback")
    path = _build.library_path()
    try:
        lib = ctypes.CDLL(path)
    except OSError as e:
        raise KernelLibraryError(f"cannot load the kernel library {path}: {e}") from None
    lib.mynah_last_error.restype = ctypes.c_char_p
    lib.mynah_last_error.argtypes = []
    lib.mynah_device_arch.restype = c_int
    lib.mynah_device_arch.argtypes = []
    lib.mynah_attn_decode_scratch_floats.restype = c_longlong
    lib.mynah_attn_decode_scratch_floats.argtypes = [c_int, c_int, c_int, c_int]
    lib.mynah_gemv_decode_mode.restype = c_int
    lib.mynah_gemv_decode_mode.argtypes = [c_int]
    lib.mynah_attn_decode_stream_mode.restype = c_int
    lib.mynah_attn_decode_stream_mode.argtypes = [c_int]
    lib.mynah_attn_decode_tc_supported.restype = c_int
    lib.mynah_attn_decode_tc_supported.argtypes = [c_int, c_int, c_int]
    lib.mynah_gemm_qkv_rope_supported.restype = c_int
    lib.mynah_gemm_qkv_rope_supported.argtypes = [c_int, c_int, c_int, c_int, c_int]
    lib.mynah_argmax_parts.restype = c_int
    lib.mynah_argmax_parts.argtypes = []
    lib.mynah_attn_prefill_tc_supported.restype = c_int
    lib.mynah_attn_prefill_tc_supported.argtypes = [c_int, c_int, c_int]
    lib.mynah_attn_prefill_tcgen05_supported.restype = c_int
    lib.mynah_attn_prefill_tcgen05_supported.argtypes = [c_int, c_int, c_int]
    lib.mynah_gemm_tcgen05_supported.restype = c_int
    lib.mynah_gemm_tcgen05_supported.argtypes = [c_int, c_int, c_int]
    lib.mynah_gemm_tcgen05_splits_k.restype = c_int
    lib.mynah_gemm_tcgen05_splits_k.argtypes = [c_int, c_int, c_int, c_int]
    lib.mynah_gemv_decode_supported.restype = c_int
    lib.mynah_gemv_decode_supported.argtypes = [c_int, c_int, c_int]
    for name, args in _SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            raise KernelLibraryError(f"the kernel library {path} has no symbol {name}; rebuild it") from None
        fn.restype = c_int
        fn.argtypes = args
    arch = lib.mynah_device_arch()
    if arch != 100:
        raise KernelLibraryError(f"the kernels are built for sm_100a only; the current device reports sm_{arch}")
    import os
    global _pdl
    _pdl = os.environ.get("MYNAH_PDL", "0") == "1"     # programmatic dependent launch of every kernel launched from here on
    lib.mynah_set_pdl(1 if _pdl else 0)
    _lib = lib
    return lib


_pdl = False


def set_pdl(on: bool) -> bool:
    """Launch the kernels from now on with (or without) the programmatic-serialization attribute, which lets a
    kernel start while the one before it on the stream still runs, up to its `griddepcontrol.wait`. A captured
    graph keeps what was set while it was captured. Returns the setting before."""
    global _pdl
    before = _pdl
    load().mynah_set_pdl(1 if on else 0)
    _pdl = bool(on)
    return before


def register(name: str, argtypes: list, restype=c_int) -> None:
    """Declare a further entry point (used by kernels added in other modules)."""
    _SIGNATURES[name] = argtypes
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.restype = restype
        fn.argtypes = argtypes


_launches = 0


def launch_count() -> int:
    """Kernel launchers of this library called so far (graph replays are added by the engine)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


def call(name: str, *args) -> None:
    global _launches
    lib = load()
    _launches += 1
    rc = getattr(lib, name)(*args)
    if rc != 0:
        raise KernelError(lib.mynah_last_error().decode(errors="replace"))


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


def code(dtype: torch.dtype) -> int:
    try:
        return DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"unsupported dtype {dtype}; the kernels take float32 and bfloat16") from None


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()
