"""Tensor-level wrappers of the CUDA entry points.

Each wrapper checks what its kernel assumes (device, dtype, contiguity, sizes) and then
launches on the current CUDA stream.  Outputs are passed in by the caller, so a step can
run from preallocated buffers.  bfloat16 matrix products go to cuBLAS through
``torch.mm`` (the reference's own projections are library calls too,
nanovllm/layers/linear.py:66); float32 products use this library's fixed-order kernel so
that the 32-bit path never sees a reduced-precision matrix mode.
"""
from __future__ import annotations

import os
import weakref

import torch

from . import attention_decode, attention_mma, attention_tcgen05, library
from .library import KernelError, call

F32, BF16 = 0, 1


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, not {t.dtype}")


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("this engine computes on the GPU only: got a CPU tensor (there is no CPU fallback)")


def _contig(name: str, t: torch.Tensor) -> None:
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def _ptr(t):
    return None if t is None else t.data_ptr()


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def embed(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor) -> None:
    _need_cuda(out, table, ids)
    _contig("out", out); _contig("table", table)
    assert ids.dtype == torch.int32 and out.dtype == table.dtype and out.shape[1] == table.shape[1]
    call("nhv_embed", dtype_code(out), out.data_ptr(), table.data_ptr(), ids.data_ptr(), ids.numel(),
         table.shape[1], table.shape[0], stream_ptr())


def feed_tokens(token_ids, feed_src, chosen, vocab: int) -> None:
    """token_ids[t] = chosen[feed_src[t]] where feed_src[t] >= 0 (tokens that the step before chose, taken on the
    device); the other entries keep what the host wrote."""
    _need_cuda(token_ids, feed_src, chosen)
    assert token_ids.dtype == feed_src.dtype == chosen.dtype == torch.int32 and feed_src.numel() >= token_ids.numel()
    call("nhv_feed_tokens", token_ids.data_ptr(), feed_src.data_ptr(), chosen.data_ptr(), token_ids.numel(), chosen.numel(),
         int(vocab), stream_ptr())


def rmsnorm(out, x, weight, eps: float, residual=None, rows=None, write_residual: bool = True,
            weight_offset: float = 0.0) -> None:
    """out[r] = norm(x[src] (+ residual[src])) * (weight + weight_offset), src = rows[r] or r.
    With a residual and write_residual the rounded sum replaces residual[src]."""
    _need_cuda(out, x, weight, residual, rows)
    _contig("out", out); _contig("x", x)
    width = x.shape[-1]
    assert weight.numel() == width and weight.dtype == x.dtype and out.dtype == x.dtype
    n_rows = rows.numel() if rows is not None else x.numel() // width
    assert out.numel() == n_rows * width
    if residual is not None:
        _contig("residual", residual)
        assert residual.shape == x.shape and residual.dtype == x.dtype
    if rows is not None:
        assert rows.dtype == torch.int32
    call("nhv_rmsnorm", dtype_code(x), out.data_ptr(), x.data_ptr(), _ptr(residual), weight.data_ptr(), _ptr(rows),
         n_rows, width, float(eps), int(bool(write_residual and residual is not None and rows is None)),
         float(weight_offset), stream_ptr())


def silu_mul(out, gate_up) -> None:
    _need_cuda(out, gate_up)
    _contig("out", out); _contig("gate_up", gate_up)
    inter = gate_up.shape[-1] // 2
    assert gate_up.shape[-1] == 2 * inter and out.shape[-1] == inter and out.dtype == gate_up.dtype
    call("nhv_silu_mul", dtype_code(out), out.data_ptr(), gate_up.data_ptr(), out.numel() // inter, inter, stream_ptr())


def to_f32(out, x) -> None:
    _need_cuda(out, x)
    _contig("out", out); _contig("x", x)
    assert out.dtype == torch.float32 and out.numel() == x.numel()
    call("nhv_to_f32", dtype_code(x), out.data_ptr(), x.data_ptr(), x.numel(), stream_ptr())


def qk_norm_rope_store(qkv, q_out, kv_pages, slot_mapping, positions, q_weight, k_weight, cos_sin, rotary_dim: int,
                       nq: int, nkv: int, head_dim: int, eps: float, weight_offset: float = 0.0) -> None:
    """qkv [T, (nq+2nkv)*d] -> q_out [T, nq*d] (normed, rotated) and K/V rows in kv_pages
    [pages, 2, nkv, page_size, d] at slot_mapping.  kv_pages None: queries only."""
    _need_cuda(qkv, q_out, kv_pages, slot_mapping, positions, q_weight, k_weight, cos_sin)
    assert qkv.stride(-1) == 1 and q_out.stride(-1) == 1 and qkv.dim() == 2 and q_out.dim() == 2
    n_tokens = qkv.shape[0]
    if kv_pages is not None:
        _contig("kv_pages", kv_pages)
        n_pages, two, h, page_size, d = kv_pages.shape
        assert two == 2 and h == nkv and d == head_dim and kv_pages.dtype == qkv.dtype
        assert slot_mapping.dtype == torch.int32 and slot_mapping.numel() >= n_tokens
    else:
        n_pages, page_size = 0, 0
    if cos_sin is not None:
        assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[1] == rotary_dim
        assert positions.dtype == torch.int32
    call("nhv_qk_norm_rope_store", dtype_code(qkv), qkv.data_ptr(), qkv.stride(0), q_out.data_ptr(), q_out.stride(0),
         _ptr(kv_pages), _ptr(slot_mapping), _ptr(positions), _ptr(q_weight), _ptr(k_weight), _ptr(cos_sin),
         int(rotary_dim), 0 if cos_sin is None else cos_sin.shape[0], n_tokens, nq, nkv, head_dim, page_size, n_pages,
         float(eps), float(weight_offset), stream_ptr())


def attention_simt(out, q, kv_pages, block_table, cu_q, kv_len, n_seqs: int, n_tokens: int, nq: int, nkv: int,
                   head_dim: int, scale: float, window: int = 0) -> None:
    """Causal attention of this step's tokens over the pages: q [T, nq*d] -> out [T, nq*d]."""
    _need_cuda(out, q, kv_pages, block_table, cu_q, kv_len)
    _contig("kv_pages", kv_pages)
    assert q.stride(-1) == 1 and out.stride(-1) == 1 and out.dtype == q.dtype == kv_pages.dtype
    n_pages, two, h, page_size, d = kv_pages.shape
    assert two == 2 and h == nkv and d == head_dim
    assert block_table.dtype == torch.int32 and block_table.stride(-1) == 1
    assert cu_q.dtype == torch.int32 and kv_len.dtype == torch.int32
    call("nhv_attention_simt", dtype_code(q), q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0),
         kv_pages.data_ptr(), block_table.data_ptr(), block_table.stride(0), cu_q.data_ptr(), kv_len.data_ptr(),
         n_seqs, n_tokens, nq, nkv, head_dim, page_size, n_pages, int(window), float(scale), stream_ptr())


def attention(out, q, kv_pages, tables, batch, nq: int, nkv: int, head_dim: int, scale: float, window: int = 0) -> None:
    """Attention of the step's tokens over the cache: picks the kernel for the dtype and sizes.
    bfloat16 with a head size in steps of 16 runs on the tensor cores; everything else (float32, other
    head sizes, groups of more than 64 heads, more than 512 requests in the step) on the CUDA cores."""
    if q.dtype == torch.bfloat16 and attention_mma.supports(head_dim, nq, nkv, batch.n_seqs):
        attention_tensor_core(out, q, kv_pages, tables.block_tables, batch.cu_q, batch.kv_len, batch.n_seqs,
                              batch.n_prefill_tokens, batch.n_prefill_seqs, batch.n_decode_seqs, batch.max_kv_len,
                              nq, nkv, head_dim, scale, window)
    else:
        attention_simt(out, q, kv_pages, tables.block_tables, batch.cu_q, batch.kv_len, batch.n_seqs, batch.n_tokens,
                       nq, nkv, head_dim, scale, window)


FUSE_DECODE_QK = True             # tests switch it off to compare with the two-kernel form
USE_TMA_DECODE = True             # tests switch it off to reach the mma.sync decode kernel at the same shapes

_decode_scratch: dict = {}


def _tma_decode_scratch(device, head_dim: int, blocks: int):
    """Partial results of the decode kernel's split requests: two slots per block, kept for the life of the
    process (every launch writes a slot before any block reads it)."""
    key = (device, head_dim)
    st = _decode_scratch.get(key)
    if st is None:
        st = _decode_scratch[key] = (torch.empty(blocks * 2 * 16 * head_dim, dtype=torch.float32, device=device),
                                     torch.empty(blocks * 2 * 16 * 2, dtype=torch.float32, device=device))
    return st


def _attention_decode_tma(out, q, qkv, kv_pages, block_table, batch_cu_q, batch_kv_len, n_seqs: int, nq: int, nkv: int,
                          head_dim: int, scale: float, window: int, q_weight=None, k_weight=None, cos_sin=None,
                          positions=None, slot_mapping=None, rotary_dim: int = 0, eps: float = 0.0,
                          weight_offset: float = 0.0, store: bool = False) -> None:
    launch, blocks = attention_decode.get(head_dim)
    n_pages, two, h, page_size, d = kv_pages.shape
    group = nq // nkv
    head_blocks = nkv * -(-group // 16)
    part_o, part_ml = _tma_decode_scratch(out.device, head_dim, blocks)
    counters = _decode_counters(out.device, n_seqs * head_blocks)
    library.LAUNCHES += 1
    launch(_ptr(q), 0 if q is None else q.stride(0), _ptr(qkv), 0 if qkv is None else qkv.stride(0), out.data_ptr(),
           out.stride(0), kv_pages.data_ptr(), block_table.data_ptr(), block_table.stride(0), batch_cu_q.data_ptr(),
           batch_kv_len.data_ptr(), n_seqs, nq, nkv, page_size, n_pages, int(window), float(scale), part_o.data_ptr(),
           part_ml.data_ptr(), counters.data_ptr(), _ptr(q_weight), _ptr(k_weight), _ptr(cos_sin), _ptr(positions),
           _ptr(slot_mapping), int(rotary_dim), 0 if cos_sin is None else cos_sin.shape[0], 1 if store else 0, float(eps),
           float(weight_offset), stream_ptr())


def attention_decode_fused(out, qkv, kv_pages, tables, batch, nq: int, nkv: int, head_dim: int, scale: float,
                           window: int, q_weight, k_weight, cos_sin, rotary_dim: int, eps: float,
                           weight_offset: float, store: bool) -> bool:
    """A step of single tokens only, in bfloat16: attention straight from the projection's output.  The decode
    kernel norms and rotates the new query and key heads itself and stores the new keys and values (what
    ``qk_norm_rope_store`` does otherwise, in a launch of its own).  Returns False, having done nothing, when
    the step or the shapes do not allow it."""
    if not (FUSE_DECODE_QK and qkv.dtype == torch.bfloat16 and batch.n_prefill_seqs == 0 and batch.n_decode_seqs > 0
            and attention_mma.supports(head_dim, nq, nkv, batch.n_seqs)):
        return False
    if qkv.stride(0) % 8 or qkv.data_ptr() % 16:
        return False
    vec = head_dim // 32
    if head_dim % 32 or (cos_sin is not None and (rotary_dim <= 0 or rotary_dim % (2 * vec))):
        return False
    _need_cuda(out, qkv, kv_pages, q_weight, k_weight, cos_sin)
    _contig("kv_pages", kv_pages)
    n_pages, two, h, page_size, d = kv_pages.shape
    assert two == 2 and h == nkv and d == head_dim and kv_pages.dtype == qkv.dtype and out.stride(-1) == 1
    block_table = tables.block_tables
    assert block_table.dtype == torch.int32 and block_table.stride(-1) == 1
    n_seqs = batch.n_seqs
    if USE_TMA_DECODE and attention_decode.supports(head_dim, nq, nkv, page_size, n_seqs):
        _attention_decode_tma(out, None, qkv, kv_pages, block_table, batch.cu_q, batch.kv_len, n_seqs, nq, nkv, head_dim,
                              scale, window, q_weight, k_weight, cos_sin, batch.positions, tables.slot_mapping, rotary_dim,
                              eps, weight_offset, store)
        return True
    launch_fused = attention_mma.get(head_dim)[2]
    if launch_fused is None:
        return False
    tile = attention_mma.get(head_dim)[1]
    group = nq // nkv
    rows, head_blocks = min(group, 16), nkv * -(-group // 16)
    max_pieces = -(-batch.max_kv_len // tile) + 1
    scratch_o = torch.empty(n_seqs * head_blocks * max_pieces * rows * head_dim, dtype=torch.float32, device=qkv.device)
    scratch_ml = torch.empty(n_seqs * head_blocks * max_pieces * rows * 2, dtype=torch.float32, device=qkv.device)
    counters = _decode_counters(qkv.device, n_seqs * head_blocks)
    library.LAUNCHES += 1
    launch_fused(qkv.data_ptr(), qkv.stride(0), out.data_ptr(), out.stride(0), kv_pages.data_ptr(), block_table.data_ptr(),
                 block_table.stride(0), batch.cu_q.data_ptr(), batch.kv_len.data_ptr(), n_seqs, nq, nkv, page_size,
                 n_pages, int(window), float(scale), scratch_o.data_ptr(), scratch_ml.data_ptr(), counters.data_ptr(),
                 max_pieces, _ptr(q_weight), _ptr(k_weight), _ptr(cos_sin), batch.positions.data_ptr(),
                 tables.slot_mapping.data_ptr(), int(rotary_dim), 0 if cos_sin is None else cos_sin.shape[0],
                 1 if store else 0, float(eps), float(weight_offset), stream_ptr())
    return True


USE_TCGEN05_ATTENTION = True      # tests switch it off to reach the mma.sync prompt kernel at the same shapes


def attention_tcgen05_error(head_dim: int) -> int:
    """The error word of the tcgen05 attention kernel's bounded waits (0 = none)."""
    return attention_tcgen05.get(head_dim)[1]()


def attention_tensor_core(out, q, kv_pages, block_table, cu_q, kv_len, n_seqs: int, n_prefill_tokens: int,
                          n_prefill_seqs: int, n_decode_seqs: int, max_kv_len: int, nq: int, nkv: int, head_dim: int,
                          scale: float, window: int = 0) -> None:
    """bfloat16 attention on the tensor cores.  Prompt portions go to the tcgen05 kernel, requests with
    one new token to the kernel that streams the cache with TMA, each where its shape is supported; what
    neither takes runs in the mma.sync kernel, whose single-token path shares a request's tiles between
    blocks and merges them (scratch: one partial result per piece of a request and head block)."""
    _need_cuda(out, q, kv_pages, block_table, cu_q, kv_len)
    _contig("kv_pages", kv_pages)
    assert q.dtype == out.dtype == kv_pages.dtype == torch.bfloat16 and q.stride(-1) == 1 and out.stride(-1) == 1
    n_pages, two, h, page_size, d = kv_pages.shape
    assert two == 2 and h == nkv and d == head_dim
    assert block_table.dtype == torch.int32 and block_table.stride(-1) == 1
    launch, tile = attention_mma.get(head_dim)[:2]
    if n_prefill_tokens > 0 and USE_TCGEN05_ATTENTION and attention_tcgen05.supports(head_dim, nq, nkv, page_size):
        # prompt portions on the 5th-generation tensor cores; single tokens stay with the split kernel below
        library.LAUNCHES += 1
        attention_tcgen05.get(head_dim)[0](
            q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), kv_pages.data_ptr(), block_table.data_ptr(),
            block_table.stride(0), cu_q.data_ptr(), kv_len.data_ptr(), n_seqs, n_prefill_tokens, n_prefill_seqs,
            nq, nkv, page_size, n_pages, int(window), float(scale), stream_ptr())
        if n_decode_seqs == 0:
            return
        n_prefill_tokens = n_prefill_seqs = 0
    if n_decode_seqs > 0 and USE_TMA_DECODE and attention_decode.supports(head_dim, nq, nkv, page_size, n_seqs):
        # single tokens: the kernel that streams the cache with TMA; what is left for the launch below are the
        # prompt portions (if the tcgen05 kernel did not take them)
        _attention_decode_tma(out, q, None, kv_pages, block_table, cu_q, kv_len, n_seqs, nq, nkv, head_dim, scale, window)
        if n_prefill_tokens == 0:
            return
        n_decode_seqs = 0
    scratch_o = scratch_ml = counters = None
    max_pieces = blocks = 0
    if n_decode_seqs > 0:
        # scratch for requests whose tiles are shared between blocks: one partial result per piece, and a
        # zeroed arrival counter per (request, head block) that the kernel leaves zeroed
        group = nq // nkv
        rows, head_blocks = min(group, 16), nkv * -(-group // 16)
        max_pieces = -(-max_kv_len // tile) + 1
        blocks = 3 * _sm_count(q.device)
        scratch_o = torch.empty(n_seqs * head_blocks * max_pieces * rows * head_dim, dtype=torch.float32, device=q.device)
        scratch_ml = torch.empty(n_seqs * head_blocks * max_pieces * rows * 2, dtype=torch.float32, device=q.device)
        counters = _decode_counters(q.device, n_seqs * head_blocks)
    library.LAUNCHES += 1
    launch(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), kv_pages.data_ptr(), block_table.data_ptr(),
           block_table.stride(0), cu_q.data_ptr(), kv_len.data_ptr(), n_seqs, n_prefill_tokens, n_prefill_seqs,
           n_decode_seqs, nq, nkv, page_size, n_pages, int(window), float(scale), _ptr(scratch_o), _ptr(scratch_ml),
           _ptr(counters), max_pieces, blocks, stream_ptr())


_sm_counts: dict = {}
_counter_buffers: dict = {}


def _sm_count(device) -> int:
    if device not in _sm_counts:
        _sm_counts[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return _sm_counts[device]


def _decode_counters(device, n: int) -> torch.Tensor:
    """Zeroed ints that outlive the step (the decode kernel returns them to zero)."""
    buf = _counter_buffers.get(device)
    if buf is None or buf.numel() < n:
        buf = _counter_buffers[device] = torch.zeros(max(n, 16384), dtype=torch.int32, device=device)
    return buf


def linear(out, x, weight) -> None:
    """out[M,N] = x[M,K] @ weight[N,K]^T.  out may be float32 while x and weight are bfloat16."""
    _need_cuda(out, x, weight)
    _contig("out", out); _contig("weight", weight)
    assert x.dim() == 2 and weight.dim() == 2 and x.stride(1) == 1 and x.dtype == weight.dtype
    M, K = x.shape
    N = weight.shape[0]
    assert weight.shape[1] == K and out.shape == (M, N)
    if x.dtype == torch.float32:
        assert out.dtype == torch.float32
        call("nhv_gemm_nt_simt", F32, out.data_ptr(), x.data_ptr(), weight.data_ptr(), M, N, K, x.stride(0), K, N, 0,
             stream_ptr())
    elif small_m_ok(x, weight):
        _small_m(out, x, weight, M, N, K, int(out.dtype == torch.float32), 0)
    elif out.dtype == torch.float32:
        # the product is rounded to bfloat16 and then widened, as the reference's head does
        # (nanovllm/layers/embed_head.py:61, nanovllm/layers/sampler.py:12)
        tmp = torch.empty(M, N, dtype=x.dtype, device=x.device)
        torch.mm(x, weight.t(), out=tmp)
        to_f32(out, tmp)
    else:
        torch.mm(x, weight.t(), out=out)


SMALL_M = 8     # up to this many tokens the weight-streaming kernel runs instead of the library product
                # (measured on B200: it is ahead up to 8 tokens, the library from 9 on; the kernel itself takes 16)


def small_m_ok(x, weight) -> bool:
    return (x.dtype == torch.bfloat16 and x.shape[0] <= SMALL_M and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def swiglu_first_half(act, x, gate_up_weight) -> bool:
    """act[M, I] = silu(x Wg^T) * (x Wu^T) in one kernel when the batch is small enough for the
    weight-streaming kernel (gate_up_weight [2 I, K], gate rows first).  Returns False if it did not run."""
    if not small_m_ok(x, gate_up_weight):
        return False
    _need_cuda(act, x, gate_up_weight)
    _contig("act", act); _contig("gate_up_weight", gate_up_weight)
    M, K = x.shape
    inter = gate_up_weight.shape[0] // 2
    assert act.shape == (M, inter) and act.dtype == torch.bfloat16 and gate_up_weight.shape[1] == K
    _small_m(act, x, gate_up_weight, M, inter, K, 2, inter)
    return True


_stream_k_state: dict = {}
STREAM_K_COUNTERS = 8192


def _small_m(out, x, weight, M: int, N: int, K: int, mode: int, up_row_offset: int) -> None:
    """The weight-streaming product for up to 16 tokens: the persistent TMA kernel, one block per SM, with
    its scratch (partial sums of tiles that two blocks share, and the tiles' arrival counters)."""
    dev = x.device
    st = _stream_k_state.get(dev)
    if st is None:
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        st = _stream_k_state[dev] = (sms, torch.zeros(sms * 2 * 64 * 16, dtype=torch.float32, device=dev),
                                     torch.zeros(STREAM_K_COUNTERS, dtype=torch.int32, device=dev))
    sms, scratch, counters = st
    tiles = -(-N // (32 if mode == 2 else 64))
    slab = _slabs.get(weight.data_ptr())
    if slab is not None and slab[0]() is weight and slab[2] == mode and M <= SLAB_MAX_M:
        _slab_product(out, x, slab[1], M, N, K, mode, sms)
        return
    if tiles > STREAM_K_COUNTERS:
        call("nhv_gemm_small_m", out.data_ptr(), x.data_ptr(), weight.data_ptr(), M, N, K, x.stride(0), N, mode,
             up_row_offset, stream_ptr())
        return
    call("nhv_gemm_stream_k", out.data_ptr(), x.data_ptr(), weight.data_ptr(), M, N, K, x.stride(0), N, mode,
         up_row_offset, scratch.data_ptr(), counters.data_ptr(), STREAM_K_COUNTERS, sms, stream_ptr())


def _slab_product(out, x, copy, M: int, N: int, K: int, mode: int, sms: int) -> None:
    """The product from the per-SM copy, with a hint for the one after it.  A decode step runs the same products in
    the same order every time, so each remembers which copy was read right after its own last time; its blocks then
    ask the first bytes of that copy into L2 as they send for their own last stage, and the next product's ring
    fills from L2 instead of HBM (measured on B200 over the four products of an 8B-sized layer: 72.1 -> 70.1 us).
    Only a hint, and only between copies that were made together (``new_slab_family``: one model's copies live and
    die together, so a captured launch never names memory that has been given back); a copy that is gone or unknown
    gets none."""
    global _slab_last
    key = copy.data_ptr()
    family = _slab_family.get(key)
    if (_slab_last is not None and _slab_last != key and SLAB_HINT_BYTES and family is not None
            and _slab_family.get(_slab_last) == family):
        _slab_after[_slab_last] = (weakref.ref(copy), key, copy.numel() * copy.element_size())
    _slab_last = key
    hint = _slab_after.get(key)
    nxt = hint[0]() if hint is not None else None
    if nxt is not None and nxt.data_ptr() == hint[1] and nxt.numel() * nxt.element_size() == hint[2] and SLAB_HINT_BYTES:
        blocks = min(sms, _slab_blocks.get(hint[1], 0))
        if blocks > 0:
            call("nhv_gemm_slab_hint", out.data_ptr(), x.data_ptr(), key, M, N, K, x.stride(0), N, mode, sms, hint[1],
                 hint[2] // blocks, SLAB_HINT_BYTES, blocks, stream_ptr())
            return
    call("nhv_gemm_slab", out.data_ptr(), x.data_ptr(), key, M, N, K, x.stride(0), N, mode, sms, stream_ptr())


# of the next product's copy, per block, asked into L2 ahead (0: no hints; NHV_SLAB_HINT_BYTES overrides it)
SLAB_HINT_BYTES = int(os.environ.get("NHV_SLAB_HINT_BYTES", "65536"))
_slab_after: dict = {}  # data pointer of a copy -> (weak reference to the copy read after it last time, its pointer, its bytes)
_slab_blocks: dict = {} # data pointer of a copy -> the blocks that share it
_slab_family: dict = {} # data pointer of a copy -> the family it was made in
_family = 0


def new_slab_family() -> None:
    """The copies made from here on belong together (a model's: the runner says so before it makes them)."""
    global _family
    _family += 1


_slab_last = None       # data pointer of the copy that the last product read
SLAB_MAX_M = 8          # tokens that csrc/gemm_slab.cu takes
_slabs: dict = {}       # data pointer of a weight matrix -> (weak reference to it, its copy for gemm_slab.cu, mode)


def slab_copy_bytes(weight: torch.Tensor, mode: int) -> int:
    n, k = weight.shape
    geo = slab_geometry(n // 2 if mode == 2 else n, k, mode, _sm_count(weight.device))
    return geo["blocks"] * geo["slab_bytes"]


def can_stream_slabs(weight: torch.Tensor, mode: int) -> bool:
    return (weight.is_cuda and weight.dtype == torch.bfloat16 and weight.dim() == 2 and weight.shape[1] % 8 == 0
            and weight.shape[0] >= (2 if mode == 2 else 1))


def prepare_streaming(weight: torch.Tensor, mode: int) -> int:
    """Keep a second copy of ``weight`` laid out for ``csrc/gemm_slab.cu`` (``slab_weight``); products of up to 8
    tokens with this matrix in this mode then read the copy: one share of rows per SM, every stage of the kernel's
    ring one contiguous copy of up to 32 KB, no sums across blocks.  Measured on B200 for the four matrices of an
    8B-sized layer: 73 us, against 87 us for the stream-K kernel on the row-major matrix (64 pieces of 512 bytes a
    row apart per stage, and a fix-up of shared tiles at the end of every launch).  The copy lives as long as the
    matrix.  Returns the bytes it takes (0 if the matrix cannot be streamed this way)."""
    if not can_stream_slabs(weight, mode):
        return 0
    key = weight.data_ptr()
    old = _slabs.get(key)
    if old is not None and old[0]() is weight and old[2] == mode:
        return 0
    copy = slab_weight(weight, mode, _sm_count(weight.device))
    n = weight.shape[0] // 2 if mode == 2 else weight.shape[0]
    _slab_blocks[copy.data_ptr()] = slab_geometry(n, weight.shape[1], mode, _sm_count(weight.device))["blocks"]
    _slab_family[copy.data_ptr()] = _family
    _slabs[key] = (weakref.ref(weight), copy, mode)
    weakref.finalize(weight, _drop_slab, key, copy.data_ptr())
    return copy.numel() * copy.element_size()


def _drop_slab(key: int, copy_ptr: int) -> None:
    entry = _slabs.get(key)
    if entry is not None and entry[1].data_ptr() == copy_ptr:
        del _slabs[key]
    _slab_blocks.pop(copy_ptr, None)
    _slab_after.pop(copy_ptr, None)
    _slab_family.pop(copy_ptr, None)


def slab_geometry(N: int, K: int, mode: int, sms: int) -> dict:
    """How ``csrc/gemm_slab.cu`` cuts a matrix with N result columns and K columns on a device with ``sms`` SMs."""
    import ctypes
    blocks, rpb, nb, ks = (ctypes.c_int() for _ in range(4))
    slab_bytes = ctypes.c_longlong()
    call("nhv_gemm_slab_geometry", N, K, mode, sms, ctypes.addressof(blocks), ctypes.addressof(rpb), ctypes.addressof(nb),
         ctypes.addressof(ks), ctypes.addressof(slab_bytes))
    return dict(blocks=blocks.value, rpb=rpb.value, nb=nb.value, ks=ks.value, slab_bytes=slab_bytes.value)


def slab_weight(weight: torch.Tensor, mode: int, sms: int) -> torch.Tensor:
    """The copy of a weight matrix [N, K] (mode 2: [gate rows; up rows]) that ``linear_slab`` reads: one share of
    rows per block, walked in sub-tiles of up to 64 rows over stages of nb * 64 columns; the bytes of a stage lie
    together, box by box (64 columns), row by row (128 bytes; mode 2: a sub-tile's gate rows, then its up rows), the
    16-byte chunks of row r of a box exchanged by c ^ (r & 7).  Rows and columns beyond the matrix are zeros."""
    assert weight.dtype == torch.bfloat16 and weight.dim() == 2
    rows, K = weight.shape
    N = rows // 2 if mode == 2 else rows
    geo = slab_geometry(N, K, mode, sms)
    G, r, nb, ks = geo["blocks"], geo["rpb"], geo["nb"], geo["ks"]
    th = 32 if mode == 2 else 64
    k_pad = ks * nb * 64

    def padded(part):                                    # [N, K] -> [G, r, ks, nb, 8 chunks, 8 elements]
        w = torch.zeros(G * r, k_pad, dtype=weight.dtype, device=weight.device)
        w[:N, :K] = part
        return w.view(G, r, ks, nb, 8, 8)

    kinds = [padded(weight[:N]), padded(weight[N:])] if mode == 2 else [padded(weight)]
    chunk = torch.arange(8, device=weight.device)
    pieces = []
    for t0 in range(0, r, th):
        h = min(th, r - t0)
        sub = torch.cat([kind[:, t0:t0 + h] for kind in kinds], 1)                           # [G, rows of the box, ks, nb, 8, 8]
        rows_t = sub.shape[1]
        src = chunk[None, :] ^ (torch.arange(rows_t, device=weight.device)[:, None] & 7)     # [rows, 8]: where chunk c' comes from
        sub = torch.gather(sub, 4, src[None, :, None, None, :, None].expand(G, rows_t, ks, nb, 8, 8))
        pieces.append(sub.permute(0, 2, 3, 1, 4, 5).reshape(G, -1))                          # [G, ks, nb, rows, 64]
    out = torch.cat(pieces, 1).contiguous()
    assert out.shape[1] * 2 == geo["slab_bytes"], (out.shape, geo)
    return out.view(-1)


def linear_slab(out, x, slabs, N: int, mode: int, sms: int) -> None:
    """out [M, N] = x [M, K] @ W^T for up to 8 tokens from the copy made by ``slab_weight`` (mode 2: silu(gate) * up)."""
    _need_cuda(out, x, slabs)
    M, K = x.shape
    call("nhv_gemm_slab", out.data_ptr(), x.data_ptr(), slabs.data_ptr(), M, N, K, x.stride(0), out.stride(0), mode, sms,
         stream_ptr())


def slab_error() -> int:
    """0 unless a bounded wait inside the slab product ever ran out (synchronises the device)."""
    from .library import load_library
    return load_library().nhv_gemm_slab_error()


_tcgen05_state: dict = {}


def linear_tcgen05(out, x, weight, mode: int = 0, up_row_offset: int = 0) -> None:
    """out = x @ weight^T for 1 to 128 tokens with tcgen05.mma and tensor-memory accumulators
    (csrc/gemm_tcgen05.cu).  mode 0: out bfloat16; 1: out float32 through bfloat16; 2: weight = [gate; up] rows,
    out = silu(gate) * up.  Not on the default path: measured on B200 at the 8B layer sizes the library product is
    still 1.2 to 5 times faster for 32 to 128 tokens; the kernel is kept tested and callable."""
    _need_cuda(out, x, weight)
    _contig("out", out); _contig("weight", weight)
    assert x.dtype == weight.dtype == torch.bfloat16 and x.stride(1) == 1
    M, K = x.shape
    N = out.shape[1]
    dev = x.device
    st = _tcgen05_state.get(dev)
    if st is None:
        sms = _sm_count(dev)
        st = _tcgen05_state[dev] = (sms, torch.zeros(sms * 2 * 128 * 128, dtype=torch.float32, device=dev),
                                    torch.zeros(STREAM_K_COUNTERS, dtype=torch.int32, device=dev))
    sms, scratch, counters = st
    call("nhv_gemm_tcgen05", out.data_ptr(), x.data_ptr(), weight.data_ptr(), M, N, K, x.stride(0), N, mode, up_row_offset,
         scratch.data_ptr(), counters.data_ptr(), STREAM_K_COUNTERS, sms, stream_ptr())


def tcgen05_error() -> int:
    """0 unless a bounded wait inside the tcgen05 product ever ran out (synchronises the device)."""
    from .library import load_library
    return load_library().nhv_gemm_tcgen05_error()


def linear_stream_k(out, x, weight, mode: int = 0, up_row_offset: int = 0) -> None:
    """The weight-streaming product for 1 to 16 tokens, whatever `SMALL_M` says (tests, experiments).
    mode 0: out bfloat16; out float32 selects mode 1; mode 2: weight = [gate; up], out = silu(gate) * up."""
    _need_cuda(out, x, weight)
    _contig("out", out); _contig("weight", weight)
    M, K = x.shape
    if mode == 0 and out.dtype == torch.float32:
        mode = 1
    _small_m(out, x, weight, M, out.shape[1], K, mode, up_row_offset)


def stream_k_error() -> int:
    """0 unless a bounded wait inside the streaming product ever ran out (synchronises the device)."""
    from .library import load_library
    return load_library().nhv_gemm_stream_k_error()


def linear_simt(out, x, weight) -> None:
    """The fixed-order CUDA-core product for any storage type (tests, and sizes a fast kernel refuses)."""
    _need_cuda(out, x, weight)
    M, K = x.shape
    N = weight.shape[0]
    call("nhv_gemm_nt_simt", dtype_code(x), out.data_ptr(), x.data_ptr(), weight.data_ptr(), M, N, K, x.stride(0), K,
         N, int(out.dtype == torch.float32 and x.dtype != torch.float32), stream_ptr())


# ---------------------------------------------------------------- bounded waits that ran out
# Kernels that wait on mbarriers bound their waits; one that runs out sets its file's error word and the kernel
# leaves with whatever it has, so the step's results are not valid.  The words reach the host with the step's
# tokens: the sampler folds them into one more int behind the tokens (``sample`` below), and callers that read
# logits instead ask ``take_wait_errors`` once per step.
ERROR_WORD_SLOTS = 16
_wait_error_sources: list = []          # (name, function giving the word's device address, function that reads and clears it)
_error_word_arrays: dict = {}           # device -> (int64 tensor [ERROR_WORD_SLOTS] of addresses, sources filled in)


def register_wait_error_source(name: str, address_fn, take_fn) -> None:
    if all(n != name for n, _, _ in _wait_error_sources):
        if len(_wait_error_sources) >= ERROR_WORD_SLOTS:
            raise KernelError("more kernels with error words than the step's health word has bits")
        _wait_error_sources.append((name, address_fn, take_fn))


def _register_library_sources() -> None:
    import ctypes
    from .library import load_library
    lib = load_library()
    for name in ("gemm_slab", "gemm_stream_k", "gemm_tcgen05"):
        word = getattr(lib, f"nhv_{name}_error_word")
        word.restype, word.argtypes = ctypes.c_void_p, []
        take = getattr(lib, f"nhv_{name}_error")
        take.restype, take.argtypes = ctypes.c_int, []
        register_wait_error_source(name, word, take)


def error_word_array(device) -> torch.Tensor:
    """Device array of the addresses of all error words known so far (zeros where there is none yet).  The
    array's own address never changes, so a captured step sees words registered after its capture too."""
    _register_library_sources()
    device = torch.device(device)
    entry = _error_word_arrays.get(device)
    if entry is None:
        entry = _error_word_arrays[device] = [torch.zeros(ERROR_WORD_SLOTS, dtype=torch.int64, device=device), 0]
    arr, filled = entry
    if filled < len(_wait_error_sources):
        with torch.cuda.device(device):
            addresses = [fn() or 0 for _, fn, _ in _wait_error_sources[filled:]]
        arr[filled:len(_wait_error_sources)] = torch.tensor(addresses, dtype=torch.int64)
        entry[1] = len(_wait_error_sources)
    return arr


def take_wait_errors() -> list[tuple[str, int]]:
    """(kernel, code) of every bounded wait that ran out since the last call; the words are cleared.
    Synchronises the device."""
    _register_library_sources()
    out = []
    for name, _, take in _wait_error_sources:
        code = take()
        if code != 0:
            out.append((name, code))
    return out


def raise_wait_errors() -> None:
    """Raise ``KernelError`` naming the kernels whose bounded waits ran out, if any did."""
    bad = take_wait_errors()
    if bad:
        raise KernelError("a bounded wait ran out in " + ", ".join(f"{n} (code {c})" for n, c in bad) +
                          ": the kernel gave up and left, and the results of the step are not valid")


def sample(out, logits, temperatures, seeds, positions) -> None:
    """out[r] = the token chosen from logits[r] (float32): argmax if temperatures[r] == 0, else the
    exponential race with noise keyed by (seeds[r], positions[r]).  ``out`` may have one element more than
    ``logits`` has rows: it receives the step's health word (bit i set: the i-th registered error word of a
    kernel with bounded waits is not zero; 0 means that all is well), which the host reads with the tokens."""
    _need_cuda(out, logits, temperatures, seeds, positions)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    assert temperatures.dtype == torch.float32 and seeds.dtype == torch.int64 and positions.dtype == torch.int32
    rows = logits.shape[0]
    st = _sampler_scratch.get(logits.device)
    if st is None or st[0].numel() < rows:
        # where the blocks that share a row meet: zero, and left zero by every launch
        n = max(rows, 512)
        if st is not None:
            _sampler_retired.append(st)      # a captured step may still point at the smaller ones
        st = _sampler_scratch[logits.device] = (torch.zeros(n, dtype=torch.int64, device=logits.device),
                                                torch.zeros(n, dtype=torch.int32, device=logits.device))
    words = status = None
    if out.numel() == rows + 1:
        words, status = error_word_array(logits.device).data_ptr(), out.data_ptr() + 4 * rows
    else:
        assert out.numel() == rows
    call("nhv_sample", out.data_ptr(), logits.data_ptr(), logits.stride(0), temperatures.data_ptr(), seeds.data_ptr(),
         positions.data_ptr(), rows, logits.shape[1], st[0].data_ptr(), st[1].data_ptr(), words, ERROR_WORD_SLOTS, status,
         stream_ptr())


_sampler_scratch: dict = {}
_sampler_retired: list = []
