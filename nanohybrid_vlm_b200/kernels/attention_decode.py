"""The decode attention kernel that streams the cache with TMA, one compiled library per head size.

``get(head_dim)`` compiles (once) and loads ``csrc/variants/attention_decode.cu`` for that head size;
``supports`` says which shapes it takes: head sizes that are multiples of 64, pages whose size is a
multiple of the 64-key tile, groups of up to 64 query heads, up to 512 requests in a step.  Everything
else stays with the decode kernel of ``attention_mma``.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p

from .library import KernelError

_libs: dict[int, tuple] = {}

P, I, F = c_void_p, c_int, c_float
TILE = 64
MAX_SEQS = 512


def supports(head_dim: int, nq: int, nkv: int, page_size: int, n_seqs: int = 1) -> bool:
    return (head_dim % 64 == 0 and 64 <= head_dim <= 256 and nq % nkv == 0 and nq // nkv <= 64
            and page_size % TILE == 0 and n_seqs <= MAX_SEQS)


def get(head_dim: int):
    """(launch function, blocks of a launch) for this head size.  The kernel's error word is registered with
    the step's health word (``ops.register_wait_error_source``)."""
    if head_dim not in _libs:
        from ..csrc.build import ensure_variant
        lib = ctypes.CDLL(ensure_variant("attention_decode.cu", {"NHV_ATTN_D": head_dim}))
        fn = getattr(lib, f"nhv_attn_decode_d{head_dim}")
        fn.argtypes = [P, I, P, I, P, I, P, P, I, P, P, I, I, I, I, I, I, F, P, P, P, P, P, P, P, P, I, I, I, F, F, P]
        fn.restype = c_int
        err = getattr(lib, f"nhv_attn_decode_last_error_d{head_dim}")
        err.restype = ctypes.c_char_p
        take = getattr(lib, f"nhv_attn_decode_error_d{head_dim}")
        take.restype = c_int
        address = getattr(lib, f"nhv_attn_decode_error_word_d{head_dim}")
        address.restype, address.argtypes = c_void_p, []
        blocks = getattr(lib, f"nhv_attn_decode_blocks_d{head_dim}")
        blocks.restype = c_int
        from . import ops
        ops.register_wait_error_source(f"attention_decode (head size {head_dim})", address, take)

        def launch(*args, _fn=fn, _err=err):
            if _fn(*args) != 0:
                raise KernelError(_err().decode(errors="replace"))

        _libs[head_dim] = (launch, blocks())
    return _libs[head_dim]
