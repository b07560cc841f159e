"""The tensor-core attention kernels, one compiled library per head size.

``get(head_dim)`` compiles (once) and loads ``csrc/variants/attention_mma.cu`` for that head
size and returns a callable; ``supports`` says which shapes the kernels take, the rest goes
to the CUDA-core kernel.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p

from .library import KernelError

_libs: dict[int, tuple] = {}

P, I, F = c_void_p, c_int, c_float


MAX_SEQS = 512      # requests of one step that the kernels plan for (MAX_DECODE_SEQS in the source)


def supports(head_dim: int, nq: int, nkv: int, n_seqs: int = 1) -> bool:
    return (head_dim % 16 == 0 and 16 <= head_dim <= 256 and nq % nkv == 0 and nq // nkv <= 64
            and n_seqs <= MAX_SEQS)


def get(head_dim: int):
    """(launch function, keys per tile, launch function of the decode form that works from the projection's
    output, or None) for this head size."""
    if head_dim not in _libs:
        from ..csrc.build import ensure_variant
        lib = ctypes.CDLL(ensure_variant("attention_mma.cu", {"NHV_ATTN_D": head_dim}))
        fn = getattr(lib, f"nhv_attn_mma_d{head_dim}")
        fn.argtypes = [P, I, P, I, P, P, I, P, P, I, I, I, I, I, I, I, I, I, F, P, P, P, I, I, P]
        fn.restype = c_int
        err = getattr(lib, f"nhv_attn_mma_last_error_d{head_dim}")
        err.restype = ctypes.c_char_p
        split = getattr(lib, f"nhv_attn_mma_tile_d{head_dim}")
        split.restype = c_int

        fused = getattr(lib, f"nhv_attn_mma_decode_fused_d{head_dim}")
        fused.argtypes = [P, I, P, I, P, P, I, P, P, I, I, I, I, I, I, F, P, P, P, I, P, P, P, P, P, I, I, I, F, F, P]
        fused.restype = c_int
        can_fuse = getattr(lib, f"nhv_attn_mma_can_fuse_d{head_dim}")
        can_fuse.restype = c_int

        def launch(*args, _fn=fn, _err=err):
            if _fn(*args) != 0:
                raise KernelError(_err().decode(errors="replace"))

        def launch_fused(*args, _fn=fused, _err=err):
            if _fn(*args) != 0:
                raise KernelError(_err().decode(errors="replace"))

        _libs[head_dim] = (launch, split(), launch_fused if can_fuse() else None)
    return _libs[head_dim]
