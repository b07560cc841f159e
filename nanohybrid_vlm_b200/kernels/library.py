"""Loads the compiled CUDA library with ctypes and declares its entry points.

There is no other implementation behind these names: if the library cannot be built or
loaded the engine stops with an error rather than compute on the CPU or through a
framework op.
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import c_float, c_int, c_size_t, c_void_p

_lib = None
_lock = threading.Lock()
LAUNCHES = 0    # entry points called since the counter was last reset (each launches at least one kernel)

P, I, F = c_void_p, c_int, c_float

_SIGNATURES = {
    # name: argtypes (all return int)
    "nhv_embed": [I, P, P, P, I, I, I, P],
    "nhv_feed_tokens": [P, P, P, I, I, I, P],
    "nhv_rmsnorm": [I, P, P, P, P, P, I, I, F, I, F, P],
    "nhv_silu_mul": [I, P, P, I, I, P],
    "nhv_to_f32": [I, P, P, c_size_t, P],
    "nhv_qk_norm_rope_store": [I, P, I, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, F, P],
    "nhv_attention_simt": [I, P, I, P, I, P, P, I, P, P, I, I, I, I, I, I, I, I, F, P],
    "nhv_gemm_nt_simt": [I, P, P, P, I, I, I, I, I, I, I, P],
    "nhv_sample": [P, P, I, P, P, P, I, I, P, P, P, I, P, P],
    "nhv_gemm_small_m": [P, P, P, I, I, I, I, I, I, I, P],
    "nhv_gemm_stream_k": [P, P, P, I, I, I, I, I, I, I, P, P, I, I, P],
    "nhv_gemm_slab": [P, P, P, I, I, I, I, I, I, I, P],
    "nhv_gemm_slab_hint": [P, P, P, I, I, I, I, I, I, I, P, ctypes.c_longlong, I, I, P],
    "nhv_gemm_slab_geometry": [I, I, I, I, P, P, P, P, P],
    "nhv_gemm_tcgen05": [P, P, P, I, I, I, I, I, I, I, P, P, I, I, P],
}


class KernelError(RuntimeError):
    pass


def load_library() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                from ..csrc.build import ensure_built
                path = ensure_built()
                lib = ctypes.CDLL(path)
                lib.nhv_last_error.restype = ctypes.c_char_p
                lib.nhv_last_error.argtypes = []
                for name, argtypes in _SIGNATURES.items():
                    fn = getattr(lib, name)
                    fn.argtypes = argtypes
                    fn.restype = c_int
                _lib = lib
    return _lib


def declare(name: str, argtypes) -> None:
    """Declare one more entry point (used by kernels added in their own files)."""
    _SIGNATURES[name] = argtypes
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int


def call(name: str, *args) -> None:
    global LAUNCHES
    LAUNCHES += 1
    lib = load_library()
    rc = getattr(lib, name)(*args)
    if rc != 0:
        raise KernelError(lib.nhv_last_error().decode(errors="replace"))
