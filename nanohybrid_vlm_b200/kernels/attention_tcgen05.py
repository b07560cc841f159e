"""The tcgen05 attention kernel for prompt portions, one compiled library per head size.

``get(head_dim)`` compiles (once) and loads ``csrc/variants/attention_tcgen05.cu`` for that head
size; ``supports`` says which shapes it takes: head sizes that are multiples of 64 and pages whose
size is a multiple of the 64-key tile.  Everything else stays with the mma.sync kernels.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p

from .library import KernelError

_libs: dict[int, tuple] = {}

P, I, F = c_void_p, c_int, c_float
TILE = 64


def supports(head_dim: int, nq: int, nkv: int, page_size: int) -> bool:
    return (head_dim % 64 == 0 and 64 <= head_dim <= 256 and nq % nkv == 0 and nq // nkv <= 64
            and page_size % TILE == 0)


def get(head_dim: int):
    """(launch function, function that reads and clears the error word) for this head size.  The error word is
    also registered with the step's health word (``ops.register_wait_error_source``)."""
    if head_dim not in _libs:
        from ..csrc.build import ensure_variant
        lib = ctypes.CDLL(ensure_variant("attention_tcgen05.cu", {"NHV_ATTN_D": head_dim}))
        fn = getattr(lib, f"nhv_attn_tcgen05_d{head_dim}")
        fn.argtypes = [P, I, P, I, P, P, I, P, P, I, I, I, I, I, I, I, I, F, P]
        fn.restype = c_int
        err = getattr(lib, f"nhv_attn_tcgen05_last_error_d{head_dim}")
        err.restype = ctypes.c_char_p
        word = getattr(lib, f"nhv_attn_tcgen05_error_d{head_dim}")
        word.restype = c_int
        address = getattr(lib, f"nhv_attn_tcgen05_error_word_d{head_dim}")
        address.restype, address.argtypes = c_void_p, []
        from . import ops
        ops.register_wait_error_source(f"attention_tcgen05 (head size {head_dim})", address, word)

        def launch(*args, _fn=fn, _err=err):
            if _fn(*args) != 0:
                raise KernelError(_err().decode(errors="replace"))

        _libs[head_dim] = (launch, word)
    return _libs[head_dim]
