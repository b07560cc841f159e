"""Each kernel alone against a plain PyTorch fp32 reference of the same op, at sizes other than the
engine's tiny models: widths and vocabularies that are no power of two, odd group sizes, head sizes
in steps of 16, page sizes from 1 up, shuffled page tables."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


@pytest.fixture(scope="module")
def ops():
    from nanohybrid_vlm_b200.kernels import ops
    return ops


def dev(t):
    return t.cuda()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,vocab,n", [(96, 384, 7), (1000, 51, 33), (4096, 17, 3)])
def test_embed(ops, dtype, width, vocab, n):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(vocab, width, generator=g).to(dtype)
    ids = torch.randint(0, vocab, (n,), generator=g, dtype=torch.int32)
    out = torch.empty(n, width, dtype=dtype, device="cuda")
    ops.embed(out, dev(table), dev(ids))
    assert torch.equal(out.cpu(), table[ids.long()])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,rows,eps", [(96, 5, 1e-5), (1000, 3, 1e-6), (4096, 9, 1e-6), (12290, 2, 1e-3)])
def test_rmsnorm_and_fused_residual(ops, dtype, width, rows, eps):
    g = torch.Generator().manual_seed(1)
    x = (torch.randn(rows, width, generator=g) * 3).to(dtype)
    res = torch.randn(rows, width, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(width, generator=g)).to(dtype)
    out = torch.empty(rows, width, dtype=dtype, device="cuda")
    ops.rmsnorm(out, dev(x), dev(w), eps)
    torch.testing.assert_close(out.cpu().float(), plain.rms_norm(x, w, eps).float(), **tol(dtype))
    res_d = dev(res.clone())
    ops.rmsnorm(out, dev(x), dev(w), eps, residual=res_d)
    y, new_res = plain.add_rms_norm(x, res, w, eps)
    torch.testing.assert_close(out.cpu().float(), y.float(), **tol(dtype))
    torch.testing.assert_close(res_d.cpu().float(), new_res.float(), **tol(dtype))
    # gathered rows, nothing written back
    idx = torch.tensor([rows - 1, 0], dtype=torch.int32)
    out2 = torch.empty(2, width, dtype=dtype, device="cuda")
    res_d = dev(res.clone())
    ops.rmsnorm(out2, dev(x), dev(w), eps, residual=res_d, rows=dev(idx), write_residual=False)
    torch.testing.assert_close(out2.cpu().float(), y[idx.long()].float(), **tol(dtype))
    assert torch.equal(res_d.cpu(), res)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inter,rows", [(160, 5), (1001, 3), (12288, 4)])
def test_silu_mul(ops, dtype, inter, rows):
    g = torch.Generator().manual_seed(2)
    gu = (torch.randn(rows, 2 * inter, generator=g) * 2).to(dtype)
    out = torch.empty(rows, inter, dtype=dtype, device="cuda")
    ops.silu_mul(out, dev(gu))
    gf, uf = gu[:, :inter].float(), gu[:, inter:].float()
    ref = (gf * torch.sigmoid(gf) * uf).to(dtype)
    torch.testing.assert_close(out.cpu().float(), ref.float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (5, 384, 96), (67, 130, 70), (130, 65, 257)])
def test_gemm_simt(ops, dtype, M, N, K):
    g = torch.Generator().manual_seed(3)
    x = torch.randn(M, K, generator=g).to(dtype)
    w = torch.randn(N, K, generator=g).to(dtype)
    out = torch.empty(M, N, dtype=dtype, device="cuda")
    ops.linear_simt(out, dev(x), dev(w))
    ref = (x.double() @ w.double().t()).float()
    t = dict(rtol=1e-5, atol=1e-4) if dtype == torch.float32 else dict(rtol=2e-2, atol=1e-1)
    torch.testing.assert_close(out.cpu().float(), ref, **t)


def test_gemm_simt_rows_do_not_depend_on_the_batch(ops):
    """A row's result is the same bits whatever else is in the batch."""
    g = torch.Generator().manual_seed(4)
    x = dev(torch.randn(77, 300, generator=g))
    w = dev(torch.randn(190, 300, generator=g))
    full = torch.empty(77, 190, device="cuda")
    ops.linear_simt(full, x, w)
    for rows in ([3], [10, 11], list(range(60, 77))):
        sub = torch.empty(len(rows), 190, device="cuda")
        ops.linear_simt(sub, x[rows].contiguous(), w)
        assert torch.equal(sub, full[rows])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(3, 384, 96), (40, 1000, 256)])
def test_linear(ops, dtype, M, N, K):
    g = torch.Generator().manual_seed(5)
    x = torch.randn(M, K, generator=g).to(dtype)
    w = torch.randn(N, K, generator=g).to(dtype)
    ref = (x.double() @ w.double().t()).float()
    t = dict(rtol=1e-5, atol=1e-4) if dtype == torch.float32 else dict(rtol=2e-2, atol=1e-1)
    out = torch.empty(M, N, dtype=dtype, device="cuda")
    ops.linear(out, dev(x), dev(w))
    torch.testing.assert_close(out.cpu().float(), ref, **t)
    out32 = torch.empty(M, N, dtype=torch.float32, device="cuda")
    ops.linear(out32, dev(x), dev(w))
    torch.testing.assert_close(out32.cpu(), ref, **t)


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(384, 96), (1000, 264), (4096, 4096), (24577, 520), (50, 12288)])
def test_gemm_small_m(ops, M, N, K):
    """The decode step's weight-streaming product: plain, with float32 output, and the feed-forward's
    first half fused with its activation."""
    g = torch.Generator().manual_seed(30)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    ref = (x.double() @ w.double().t()).float()
    t = dict(rtol=2e-2, atol=2e-2 * ref.abs().max().item() / 4)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.linear_stream_k(out, dev(x), dev(w))
    torch.testing.assert_close(out.cpu().float(), ref, **t)
    out32 = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    ops.linear_stream_k(out32, dev(x), dev(w))
    assert torch.equal(out32.cpu(), out.cpu().float())           # the float32 form is the bfloat16 one, widened
    if N % 2 == 0:
        inter = N // 2
        act = torch.full((M, inter), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops.linear_stream_k(act, dev(x), dev(w), mode=2, up_row_offset=inter)
        gu = out.cpu().float()
        want = (gu[:, :inter] * torch.sigmoid(gu[:, :inter]) * gu[:, inter:]).to(torch.bfloat16)
        torch.testing.assert_close(act.cpu().float(), want.float(), rtol=1e-2, atol=1e-3)
    # a row's result does not depend on the other tokens of the batch
    if M > 1:
        one = torch.empty(1, N, dtype=torch.bfloat16, device="cuda")
        ops.linear_stream_k(one, dev(x[M - 1:M]), dev(w))
        assert torch.equal(one.cpu()[0], out.cpu()[M - 1])


@pytest.mark.parametrize("M", [1, 5, 8])
@pytest.mark.parametrize("N,K", [(384, 96), (1000, 264), (4096, 4096), (24578, 520), (50, 12288), (7, 40), (6144, 4096),
                                 (384, 192), (1000, 320)])
def test_gemm_from_slabs(ops, M, N, K):
    """The decode step's products from the copy of the weights that is cut into one share of rows per SM
    (csrc/gemm_slab.cu): plain, float32 output and the fused SwiGLU half, against fp64; shapes whose shares are 1,
    3, 7, 28, 42 and 167 rows, whose columns need padding to the stage (with K a multiple of 64, where a stage's
    columns of x come in one copy, and not), and whose last share is short; and what
    ``ops.linear`` takes by itself once ``prepare_streaming`` has registered the copy."""
    g = torch.Generator().manual_seed(31)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    ref = (x.double() @ w.double().t()).float()
    t = dict(rtol=2e-2, atol=2e-2 * ref.abs().max().item() / 4)
    xd, wd = dev(x), dev(w)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.linear_slab(out, xd, ops.slab_weight(wd, 0, sms), N, 0, sms)
    torch.testing.assert_close(out.cpu().float(), ref, **t)
    out32 = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    ops.linear_slab(out32, xd, ops.slab_weight(wd, 1, sms), N, 1, sms)
    assert torch.equal(out32.cpu(), out.cpu().float())           # the float32 form is the bfloat16 one, widened
    if N % 2 == 0:
        inter = N // 2
        act = torch.full((M, inter), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops.linear_slab(act, xd, ops.slab_weight(wd, 2, sms), inter, 2, sms)
        gu = out.cpu().float()
        want = (gu[:, :inter] * torch.sigmoid(gu[:, :inter]) * gu[:, inter:]).to(torch.bfloat16)
        torch.testing.assert_close(act.cpu().float(), want.float(), rtol=1e-2, atol=1e-3)
    if M > 1:                                                    # a row's result does not depend on the other tokens
        one = torch.empty(1, N, dtype=torch.bfloat16, device="cuda")
        ops.linear_slab(one, xd[M - 1:M], ops.slab_weight(wd, 0, sms), N, 0, sms)
        assert torch.equal(one.cpu()[0], out.cpu()[M - 1])
    assert ops.slab_error() == 0
    if K % 8 == 0:
        assert ops.prepare_streaming(wd, 0) == ops.slab_copy_bytes(wd, 0) and ops.prepare_streaming(wd, 0) == 0
        through_copy = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops.linear(through_copy, xd, wd)
        assert torch.equal(through_copy.cpu(), out.cpu())
        key = wd.data_ptr()
        assert key in ops._slabs
        del wd
        import gc
        gc.collect()
        assert key not in ops._slabs, "the copy outlived its matrix"


@pytest.mark.parametrize("M", [17, 33, 64, 100, 128])
@pytest.mark.parametrize("N,K", [(384, 96), (1000, 264), (4096, 4096), (4098, 520)])
def test_gemm_tcgen05(ops, M, N, K):
    """The tensor-memory product (tcgen05.mma, TMA operands, stream-K over the SMs): plain, with float32
    output, and fused with the feed-forward's activation; shapes that split tiles between blocks and
    shapes whose edges are padded by the copy engine."""
    g = torch.Generator().manual_seed(31)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    ref = (x.double() @ w.double().t()).float()
    t = dict(rtol=2e-2, atol=2e-2 * ref.abs().max().item() / 4)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.linear_tcgen05(out, dev(x), dev(w))
    torch.testing.assert_close(out.cpu().float(), ref, **t)
    out32 = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    ops.linear_tcgen05(out32, dev(x), dev(w), mode=1)
    assert torch.equal(out32.cpu(), out.cpu().float())
    if N % 2 == 0:
        inter = N // 2
        act = torch.full((M, inter), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops.linear_tcgen05(act, dev(x), dev(w), mode=2, up_row_offset=inter)
        gu = out.cpu().float()
        want = (gu[:, :inter] * torch.sigmoid(gu[:, :inter]) * gu[:, inter:]).to(torch.bfloat16)
        # the fused form cuts K between blocks at other places than the plain one, so gate and up may each
        # differ by one bfloat16 step before the activation
        torch.testing.assert_close(act.cpu().float(), want.float(), rtol=3e-2, atol=2e-2)
    assert ops.tcgen05_error() == 0


def make_pages(k, v, page_size, n_pages, rng, dtype):
    """Scatter one request's keys/values [T, nkv, d] over shuffled pages. Returns pages tensor and table."""
    T, nkv, d = k.shape
    need = -(-T // page_size)
    ids = rng.permutation(n_pages)[:need]
    pages = torch.full((n_pages, 2, nkv, page_size, d), float("nan")).to(dtype)
    for j in range(T):
        pages[ids[j // page_size], 0, :, j % page_size] = k[j]
        pages[ids[j // page_size], 1, :, j % page_size] = v[j]
    return pages, ids


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,rot,page", [(4, 2, 16, 16, 16), (6, 2, 32, 32, 8), (3, 3, 48, 24, 1), (14, 2, 80, 80, 5),
                                               (8, 1, 128, 128, 256), (2, 1, 256, 64, 32)])
def test_qk_norm_rope_store(ops, dtype, nq, nkv, d, rot, page):
    g = torch.Generator().manual_seed(6)
    T, max_pos, eps, theta = 23, 300, 1e-5, 5000.0
    qkv = torch.randn(T, (nq + 2 * nkv) * d, generator=g).to(dtype)
    qw = (1 + 0.1 * torch.randn(d, generator=g)).to(dtype)
    kw = (1 + 0.1 * torch.randn(d, generator=g)).to(dtype)
    positions = torch.randint(0, max_pos, (T,), generator=g, dtype=torch.int32)
    n_pages = -(-T // page) + 3
    perm = torch.randperm(n_pages * page, generator=g)[:T].to(torch.int32)
    perm[5] = -1                                      # a token that must not be stored
    cos, sin = plain.rope_table(rot, max_pos, theta)
    table = torch.cat((cos, sin), -1).contiguous()
    q_out = torch.empty(T, nq * d, dtype=dtype, device="cuda")
    pages = torch.zeros(n_pages, 2, nkv, page, d, dtype=dtype, device="cuda")
    ops.qk_norm_rope_store(dev(qkv), q_out, pages, dev(perm), dev(positions), dev(qw), dev(kw), dev(table), rot,
                           nq, nkv, d, eps)
    q, k, v = qkv.split([nq * d, nkv * d, nkv * d], -1)
    q, k, v = q.view(T, nq, d), k.view(T, nkv, d), v.view(T, nkv, d)

    def rope_partial(x):
        c, s = cos[positions.long()], sin[positions.long()]
        return torch.cat((plain.apply_rope(x[..., :rot], c, s), x[..., rot:]), -1)

    q_ref = rope_partial(plain.rms_norm(q, qw, eps))
    k_ref = rope_partial(plain.rms_norm(k, kw, eps))
    torch.testing.assert_close(q_out.cpu().float().view(T, nq, d), q_ref.float(), **tol(dtype))
    pc = pages.cpu()
    for t in range(T):
        s = int(perm[t])
        if s < 0:
            continue
        torch.testing.assert_close(pc[s // page, 0, :, s % page].float(), k_ref[t].float(), **tol(dtype))
        assert torch.equal(pc[s // page, 1, :, s % page], v[t])
    written = torch.zeros(n_pages * page, dtype=torch.bool)
    written[perm[perm >= 0].long()] = True
    flat = pc.permute(0, 3, 1, 2, 4).reshape(n_pages * page, -1)
    assert (flat[~written] == 0).all(), "a slot that no token maps to was written"


def reference_attention(q, k, v, scale, window):
    """q [n_new, nq, d] at the last n_new positions of k/v [T, nkv, d]; fp64 softmax."""
    T, nkv, d = k.shape
    n_new, nq, _ = q.shape
    G = nq // nkv
    out = torch.empty(n_new, nq, d, dtype=torch.float64)
    for i in range(n_new):
        pos = T - n_new + i
        lo = max(0, pos - window + 1) if window else 0
        for h in range(nq):
            s = (k[lo:pos + 1, h // G].double() @ q[i, h].double()) * scale
            p = torch.softmax(s, 0)
            out[i, h] = p @ v[lo:pos + 1, h // G].double()
    return out


ATTENTION_SHAPES = [(4, 2, 16, 16, 0), (6, 2, 32, 8, 0), (3, 3, 48, 1, 0), (14, 2, 80, 5, 0), (8, 1, 128, 64, 0), (6, 2, 192, 16, 0),
                    (18, 2, 64, 16, 0), (4, 2, 32, 8, 19), (2, 1, 256, 32, 40), (32, 8, 128, 256, 0),
                    (34, 1, 64, 16, 300)]


# shapes the tcgen05 prompt kernel takes: head sizes in steps of 64, pages in steps of 64 keys
TCGEN05_SHAPES = [(8, 1, 128, 64, 0), (32, 8, 128, 256, 0), (4, 2, 64, 64, 0), (6, 2, 64, 128, 37), (2, 1, 256, 64, 40),
                  (12, 4, 192, 64, 0), (3, 1, 128, 64, 0), (5, 5, 64, 192, 300)]


@pytest.mark.parametrize("kernel,dtype,nq,nkv,d,page,window",
                         [(k, t, *shape) for k, t in [("simt", torch.float32), ("simt", torch.bfloat16),
                                                      ("tensor_core", torch.bfloat16)] for shape in ATTENTION_SHAPES]
                         + [("tcgen05", torch.bfloat16, *shape) for shape in TCGEN05_SHAPES])
def test_attention_mixed_batch(ops, kernel, dtype, nq, nkv, d, page, window):
    """Five requests in one batch: a long prompt portion with earlier context, a single decoded token
    after hundreds of keys, a whole short prompt, a decoded token with few keys and a two-token portion;
    pages shuffled and the pool poisoned with NaN.  One far key is made to stand out: its score
    dominates, so losing it (a wrong page, an off-by-one at a page's edge or a split's edge) shows."""
    rng = np.random.default_rng(7)
    g = torch.Generator().manual_seed(7)
    lens, news = [173, 611, 9, 5, 258], [37, 1, 9, 1, 2]
    scale = d ** -0.5
    n_pages = sum(-(-L // page) for L in lens) + 4
    pages = torch.full((n_pages, 2, nkv, page, d), float("nan")).to(dtype)
    free = list(rng.permutation(n_pages))
    qs, refs, tables = [], [], []
    for L, n in zip(lens, news):
        k = torch.randn(L, nkv, d, generator=g).to(dtype)
        v = torch.randn(L, nkv, d, generator=g).to(dtype)
        q = torch.randn(n, nq, d, generator=g).to(dtype)
        far = 3 if not window else L - window               # the last query's farthest visible key
        if L > 100:
            q[-1, :] = 0
            q[-1, :, 0] = 6.0
            k[far, :, 0] = 8.0                              # score 48 * scale: stands out
            v[far] = 5.0
            if window:                                      # one key further is out of sight, however loud
                k[far - 1, :, 0] = 14.0
                v[far - 1] = -9.0
        ids = [free.pop() for _ in range(-(-L // page))]
        for j in range(L):
            pages[ids[j // page], 0, :, j % page] = k[j]
            pages[ids[j // page], 1, :, j % page] = v[j]
        tables.append(ids)
        qs.append(q)
        refs.append(reference_attention(q, k, v, scale, window))
    width = max(len(t) for t in tables)
    S = len(lens)
    bt = torch.full((S, width), -1, dtype=torch.int32)
    for i, t in enumerate(tables):
        bt[i, :len(t)] = torch.tensor(t, dtype=torch.int32)
    q_all = torch.cat(qs).reshape(-1, nq * d)
    cu = torch.tensor([0, *np.cumsum(news)], dtype=torch.int32)
    out = torch.full_like(q_all, float("nan"), device="cuda")
    kv = dev(torch.tensor(lens, dtype=torch.int32))
    if kernel == "simt":
        ops.attention_simt(out, dev(q_all), dev(pages), dev(bt), dev(cu), kv, S, sum(news), nq, nkv, d, scale, window)
    else:
        # "tensor_core": the mma.sync kernels alone; "tcgen05": prompt portions through the tcgen05 kernel and
        # single tokens through the decode kernel that streams the cache with TMA
        ops.USE_TCGEN05_ATTENTION = ops.USE_TMA_DECODE = kernel == "tcgen05"
        try:
            ops.attention_tensor_core(out, dev(q_all), dev(pages), dev(bt), dev(cu), kv, S,
                                      sum(n for n in news if n > 1), sum(1 for n in news if n > 1),
                                      sum(1 for n in news if n == 1), max(lens), nq, nkv, d, scale, window)
        finally:
            ops.USE_TCGEN05_ATTENTION = ops.USE_TMA_DECODE = True
        if kernel == "tcgen05":
            assert ops.take_wait_errors() == [], "a bounded wait of a kernel ran out"
    ref = torch.cat(refs).reshape(-1, nq * d).float()
    t = dict(rtol=1e-4, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(out.cpu().float(), ref, **t)


FUSED_SHAPES = [(32, 8, 128, 256, 0, 128, True), (6, 2, 64, 16, 0, 64, True), (4, 4, 32, 8, 19, 16, True),
                (9, 3, 96, 5, 0, 96, False), (2, 1, 256, 64, 40, 0, True), (34, 1, 64, 16, 300, 32, True),
                (6, 2, 192, 16, 0, 192, True), (5, 1, 160, 8, 0, 80, True), (4, 2, 224, 16, 0, 0, False)]
# shapes that the decode kernel with TMA takes (head sizes in steps of 64, pages in steps of 64 keys): groups of
# 1, 3, 5 and 34 heads (three head blocks), windows that end inside a tile, partial rotation, no norm
TMA_FUSED_SHAPES = [(32, 8, 128, 256, 0, 128, True), (2, 1, 256, 64, 40, 0, True), (6, 2, 64, 64, 0, 64, True),
                    (12, 4, 192, 64, 0, 96, True), (34, 1, 64, 128, 300, 32, True), (40, 8, 128, 64, 100, 128, False),
                    (3, 3, 128, 192, 0, 64, True)]


@pytest.mark.parametrize("tma,nq,nkv,d,page,window,rot,norm,many",
                         [(False, *s, False) for s in FUSED_SHAPES] + [(True, *s, False) for s in TMA_FUSED_SHAPES]
                         + [(True, *s, True) for s in TMA_FUSED_SHAPES[:4]])
def test_attention_decode_from_the_projection_output(ops, tma, nq, nkv, d, page, window, rot, norm, many):
    """A step of single tokens: the decode kernel given qkv as the projection wrote it (it norms, rotates and
    stores by itself) against ``reference_attention`` over keys and values gathered from the cache, with the new
    query and key heads normed and rotated apart in float64 (the plain implementation's formulas); the cache
    afterwards holds the new keys and values and nothing else has changed; and again without storing, as a
    layer that reads another layer's cache runs.  ``many``: 163 short requests instead of six, so that a block has
    several pieces."""
    from types import SimpleNamespace
    from nanohybrid_vlm_b200.kernels import attention_decode
    assert attention_decode.supports(d, nq, nkv, page) == tma or not tma
    ops.USE_TMA_DECODE = tma
    rng = np.random.default_rng(11)
    g = torch.Generator().manual_seed(11)
    lens = [611, 1, 64, 65, 200, 7]                          # keys of each request, the new token included
    if many:    # every block of the persistent kernel has several pieces: the rows of qkv of all but its first are copied ahead
        lens = rng.integers(1, 150, 160).tolist() + [611, 64, 65]
    S = len(lens)
    n_pages = sum(-(-L // page) for L in lens) + 3
    pages = (torch.randn(n_pages, 2, nkv, page, d, generator=g) * 0.5).to(torch.bfloat16)   # stale contents everywhere
    free = list(rng.permutation(n_pages))
    tables = [[int(free.pop()) for _ in range(-(-L // page))] for L in lens]
    for t, L in zip(tables, lens):                          # and NaN behind every request's last key, as in a fresh pool
        if L % page:
            pages[t[-1], :, :, L % page:] = float("nan")
    width = max(len(t) for t in tables)
    bt = torch.full((S, width), -1, dtype=torch.int32)
    for i, t in enumerate(tables):
        bt[i, :len(t)] = torch.tensor(t, dtype=torch.int32)
    slots = torch.tensor([t[(L - 1) // page] * page + (L - 1) % page for t, L in zip(tables, lens)], dtype=torch.int32)
    positions = torch.tensor([L - 1 for L in lens], dtype=torch.int32)
    qkv = torch.randn(S, (nq + 2 * nkv) * d, generator=g).to(torch.bfloat16)
    qw = (1 + 0.1 * torch.randn(d, generator=g)).to(torch.bfloat16) if norm else None
    kw = (1 + 0.1 * torch.randn(d, generator=g)).to(torch.bfloat16) if norm else None
    table = None
    if rot:
        cos, sin = plain.rope_table(rot, 1024, 10000.0)
        table = dev(torch.cat((cos, sin), -1).contiguous())
    batch = SimpleNamespace(n_seqs=S, n_prefill_seqs=0, n_prefill_tokens=0, n_decode_seqs=S, max_kv_len=max(lens),
                            cu_q=dev(torch.arange(S + 1, dtype=torch.int32)), kv_len=dev(torch.tensor(lens, dtype=torch.int32)),
                            positions=dev(positions), n_tokens=S)
    views = SimpleNamespace(block_tables=dev(bt), slot_mapping=dev(slots))
    scale = d ** -0.5

    # the reference: norm and rotation of the new heads in float64, rounded to bfloat16 where the cache and the
    # query are; then attention over the request's keys and values, the new ones in their slot
    def norm_rotate(x, w, pos):                              # x [heads, d]
        x = x.double()
        if w is not None:
            x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6)
            x = x.to(torch.bfloat16).double() * w.double()   # the norm rounds, then times the weight (layernorm.py:25,39)
            x = x.to(torch.bfloat16).double()
        if rot:
            c, s_ = cos[pos].double(), sin[pos].double()     # [rot / 2]
            x1, x2 = x[:, :rot // 2], x[:, rot // 2:rot]
            x = torch.cat((x1 * c - x2 * s_, x2 * c + x1 * s_, x[:, rot:]), -1)
        return x.to(torch.bfloat16)

    want = torch.empty(S, nq, d, dtype=torch.float64)
    new_k, new_v = [], []
    for i, L in enumerate(lens):
        row = qkv[i]
        qh = norm_rotate(row[:nq * d].view(nq, d), qw, L - 1)
        kh = norm_rotate(row[nq * d:(nq + nkv) * d].view(nkv, d), kw, L - 1)
        vh = row[(nq + nkv) * d:].view(nkv, d)
        new_k.append(kh); new_v.append(vh)
        ks = torch.cat([pages[t, 0] for t in tables[i]], 1)[:, :L].transpose(0, 1).clone()    # [L, nkv, d]
        vs = torch.cat([pages[t, 1] for t in tables[i]], 1)[:, :L].transpose(0, 1).clone()
        ks[L - 1], vs[L - 1] = kh, vh
        want[i] = reference_attention(qh[None], ks, vs, scale, window)[0]
    want = want.reshape(S, nq * d).float()
    pages_want = pages.clone()
    for i, L in enumerate(lens):
        pg, off = tables[i][(L - 1) // page], (L - 1) % page
        pages_want[pg, 0, :, off], pages_want[pg, 1, :, off] = new_k[i], new_v[i]

    # the two-kernel form gives the same (it has tests of its own above)
    pages_two = dev(pages.clone())
    q = torch.empty(S, nq * d, dtype=torch.bfloat16, device="cuda")
    ops.qk_norm_rope_store(dev(qkv), q, pages_two, views.slot_mapping, batch.positions, dev(qw) if norm else None,
                           dev(kw) if norm else None, table, rot, nq, nkv, d, 1e-6)

    # the fused form, storing
    pages_one = dev(pages.clone())
    got = torch.full((S, nq * d), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert ops.attention_decode_fused(got, dev(qkv), pages_one, views, batch, nq, nkv, d, scale, window,
                                      dev(qw) if norm else None, dev(kw) if norm else None, table, rot, 1e-6, 0.0, True)
    torch.testing.assert_close(got.cpu().float(), want, rtol=2e-2, atol=2e-2)
    # the cache: the new keys and values where they belong (one step of bfloat16 apart at most: the kernel's
    # float32 arithmetic against float64), every other slot untouched
    torch.testing.assert_close(pages_one.cpu().float(), pages_want.float(), rtol=1e-2, atol=1e-2, equal_nan=True)
    untouched = torch.ones(n_pages, 2, nkv, page, dtype=torch.bool)
    for i, L in enumerate(lens):
        untouched[tables[i][(L - 1) // page], :, :, (L - 1) % page] = False
    assert torch.equal(pages_one.cpu()[untouched].view(torch.int16), pages[untouched].view(torch.int16))

    # without storing: the new keys and values are in the cache already (the other run stored them)
    again = torch.full((S, nq * d), float("nan"), dtype=torch.bfloat16, device="cuda")
    before = pages_two.clone()
    assert ops.attention_decode_fused(again, dev(qkv), pages_two, views, batch, nq, nkv, d, scale, window,
                                      dev(qw) if norm else None, dev(kw) if norm else None, table, rot, 1e-6, 0.0, False)
    torch.testing.assert_close(again.cpu().float(), want, rtol=2e-2, atol=2e-2)
    assert torch.equal(pages_two.view(torch.int16), before.view(torch.int16))
    ops.USE_TMA_DECODE = True
    assert ops.take_wait_errors() == []


@pytest.mark.parametrize("vocab,rows", [(384, 5), (1000, 3), (151936, 4)])
def test_sampler(ops, vocab, rows):
    g = torch.Generator().manual_seed(8)
    logits = torch.randn(rows, vocab, generator=g) * 3
    temps = torch.tensor([0.0, 0.8, 1.5, 0.3, 1.0][:rows])
    seeds = torch.tensor([11, 2**40 + 5, 3, 99, 123456789][:rows], dtype=torch.int64)
    positions = torch.tensor([7, 0, 513, 40, 9][:rows], dtype=torch.int32)
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    ops.sample(out, dev(logits), dev(temps), dev(seeds), dev(positions))
    got = out.cpu().tolist()
    for r in range(rows):
        assert got[r] == plain.sample(logits[r], float(temps[r]), int(seeds[r]), int(positions[r]))
    # the same request draws the same token whatever else is in the batch
    out1 = torch.empty(1, dtype=torch.int32, device="cuda")
    ops.sample(out1, dev(logits[1:2]), dev(temps[1:2]), dev(seeds[1:2]), dev(positions[1:2]))
    assert out1.item() == got[1]


def test_sampler_follows_the_distribution(ops):
    """Over many seeds the exponential race picks token i with probability softmax(logits / T)_i."""
    logits = torch.tensor([2.0, 1.0, 0.0, -1.0, 0.5, -3.0, 1.5])
    T, n = 0.7, 20000
    rows = logits.repeat(n, 1)
    out = torch.empty(n, dtype=torch.int32, device="cuda")
    ops.sample(out, dev(rows), dev(torch.full((n,), T)), dev(torch.arange(n, dtype=torch.int64) * 7919 + 1),
               dev(torch.zeros(n, dtype=torch.int32)))
    freq = torch.bincount(out.cpu().long(), minlength=7).double() / n
    p = torch.softmax(logits.double() / T, 0)
    assert (freq - p).abs().max() < 4 * math.sqrt(0.25 / n)


@pytest.mark.parametrize("nq,nkv,d,page,window", [(32, 8, 128, 256, 0), (6, 2, 64, 64, 700), (16, 1, 128, 64, 0)])
def test_attention_decode_many_requests_through_the_tma_ring(ops, nq, nkv, d, page, window):
    """Forty single-token requests of 1 to 3,000 keys: every block of the persistent decode kernel walks many
    tiles, whole requests and the ends of requests that it shares with its neighbours, and the ring is reused
    many times over; against the float64 reference, with NaN wherever no key lies.  Among and behind them idle
    entries as a padded batch has them (one token, no page): their rows come back cleared."""
    from nanohybrid_vlm_b200.kernels import attention_decode
    assert attention_decode.supports(d, nq, nkv, page)
    rng = np.random.default_rng(5)
    g = torch.Generator().manual_seed(5)
    lens = [1, 2, 63, 64, 65, 3000, 2049] + rng.integers(1, 3000, 33).tolist()
    S = len(lens)
    n_pages = sum(-(-L // page) for L in lens) + 2
    pages = torch.full((n_pages, 2, nkv, page, d), float("nan")).to(torch.bfloat16)
    free = list(rng.permutation(n_pages))
    scale = d ** -0.5
    tables, qs, refs = [], [], []
    for L in lens:
        k = torch.randn(L, nkv, d, generator=g).to(torch.bfloat16)
        v = torch.randn(L, nkv, d, generator=g).to(torch.bfloat16)
        q = torch.randn(1, nq, d, generator=g).to(torch.bfloat16)
        if L > 300:                                          # one far key stands out: losing it shows
            far = L - window if window and L > window else 5
            q[0] = 0
            q[0, :, 1] = 6.0
            k[far, :, 1] = 8.0
            v[far] = 4.0
        ids = [int(free.pop()) for _ in range(-(-L // page))]
        kp = torch.full((len(ids) * page, nkv, d), float("nan")).to(torch.bfloat16)
        vp = kp.clone()
        kp[:L], vp[:L] = k, v
        pages[ids, 0] = kp.view(len(ids), page, nkv, d).transpose(1, 2)
        pages[ids, 1] = vp.view(len(ids), page, nkv, d).transpose(1, 2)
        tables.append(ids)
        qs.append(q)
        refs.append(reference_attention(q, k, v, scale, window))
    for at in (4, 21, S + 2, S + 3, S + 4, S + 5, S + 6):    # idle entries
        lens.insert(at, 1)
        tables.insert(at, [])
        qs.insert(at, torch.randn(1, nq, d, generator=g).to(torch.bfloat16))
        refs.insert(at, torch.zeros(1, nq, d))
    S = len(lens)
    width = max(len(t) for t in tables)
    bt = torch.full((S, width), -1, dtype=torch.int32)
    for i, t in enumerate(tables):
        bt[i, :len(t)] = torch.tensor(t, dtype=torch.int32)
    q_all = torch.cat(qs).reshape(S, nq * d)
    out = torch.full_like(q_all, float("nan"), device="cuda")
    cu = torch.arange(S + 1, dtype=torch.int32)
    for repeat in range(2):                                  # the scratch and the counters are left ready for the next launch
        out.fill_(float("nan"))
        ops.attention_tensor_core(out, dev(q_all), dev(pages), dev(bt), dev(cu), dev(torch.tensor(lens, dtype=torch.int32)), S,
                                  0, 0, S, max(lens), nq, nkv, d, scale, window)
        ref = torch.cat(refs).reshape(S, nq * d).float()
        torch.testing.assert_close(out.cpu().float(), ref, rtol=2e-2, atol=2e-2)
    assert ops.take_wait_errors() == []


def test_attention_of_more_requests_than_the_tensor_core_kernels_plan_for(ops):
    """600 single-token requests in one step: beyond the 512 that the tensor-core decode kernels plan for, so
    ``ops.attention`` runs the step on the CUDA-core kernel instead of refusing it in the middle of generation."""
    from types import SimpleNamespace
    from nanohybrid_vlm_b200.kernels import attention_mma
    nq, nkv, d, page, S = 4, 2, 16, 4, 600
    assert S > attention_mma.MAX_SEQS
    g = torch.Generator().manual_seed(2)
    rng = np.random.default_rng(2)
    lens = rng.integers(1, 20, S).tolist()
    per = [-(-L // page) for L in lens]
    n_pages = sum(per)
    pages = torch.full((n_pages, 2, nkv, page, d), float("nan")).to(torch.bfloat16)
    order = rng.permutation(n_pages).tolist()
    bt = torch.full((S, max(per)), -1, dtype=torch.int32)
    qs, refs = [], []
    for i, L in enumerate(lens):
        ids = [order.pop() for _ in range(per[i])]
        bt[i, :len(ids)] = torch.tensor(ids, dtype=torch.int32)
        k = torch.randn(L, nkv, d, generator=g).to(torch.bfloat16)
        v = torch.randn(L, nkv, d, generator=g).to(torch.bfloat16)
        q = torch.randn(1, nq, d, generator=g).to(torch.bfloat16)
        for j in range(L):
            pages[ids[j // page], 0, :, j % page], pages[ids[j // page], 1, :, j % page] = k[j], v[j]
        qs.append(q)
        refs.append(reference_attention(q, k, v, d ** -0.5, 0))
    q_all = torch.cat(qs).reshape(S, nq * d)
    out = torch.full_like(q_all, float("nan"), device="cuda")
    batch = SimpleNamespace(n_seqs=S, n_tokens=S, n_prefill_seqs=0, n_prefill_tokens=0, n_decode_seqs=S, max_kv_len=max(lens),
                            cu_q=dev(torch.arange(S + 1, dtype=torch.int32)), kv_len=dev(torch.tensor(lens, dtype=torch.int32)))
    ops.attention(out, dev(q_all), dev(pages), SimpleNamespace(block_tables=dev(bt)), batch, nq, nkv, d, d ** -0.5)
    torch.testing.assert_close(out.cpu().float(), torch.cat(refs).reshape(S, nq * d).float(), rtol=2e-2, atol=2e-2)


def test_attention_decode_one_long_request_split_over_many_blocks(ops):
    """One request of 20,000 keys beside a short one: every (request, KV head) is cut into about twenty pieces
    that as many blocks hand to the one that arrives last; against the float64 reference."""
    nq, nkv, d, page = 8, 2, 128, 256
    g = torch.Generator().manual_seed(9)
    lens = [20000, 5]
    S = len(lens)
    n_pages = sum(-(-L // page) for L in lens) + 1
    pages = torch.full((n_pages, 2, nkv, page, d), float("nan")).to(torch.bfloat16)
    rng = np.random.default_rng(9)
    free = list(rng.permutation(n_pages))
    tables, qs, refs = [], [], []
    for L in lens:
        k = torch.randn(L, nkv, d, generator=g).to(torch.bfloat16)
        v = torch.randn(L, nkv, d, generator=g).to(torch.bfloat16)
        q = torch.randn(1, nq, d, generator=g).to(torch.bfloat16)
        if L > 100:
            q[0] = 0
            q[0, :, 3] = 6.0
            k[7, :, 3] = 8.0                                  # a far key that stands out
            v[7] = 3.0
        ids = [int(free.pop()) for _ in range(-(-L // page))]
        kp = torch.full((len(ids) * page, nkv, d), float("nan")).to(torch.bfloat16)
        vp = kp.clone()
        kp[:L], vp[:L] = k, v
        pages[ids, 0] = kp.view(len(ids), page, nkv, d).transpose(1, 2)
        pages[ids, 1] = vp.view(len(ids), page, nkv, d).transpose(1, 2)
        tables.append(ids)
        qs.append(q)
        # the reference in slices of heads would be slow over 20,000 keys: one matrix product per KV head
        G = nq // nkv
        kk, vv = k.double(), v.double()
        sc = torch.einsum("hd,thd->ht", q[0].double(), kk.repeat_interleave(G, 1)) * d ** -0.5
        refs.append(torch.einsum("ht,thd->hd", torch.softmax(sc, -1), vv.repeat_interleave(G, 1)).reshape(1, nq * d))
    width = max(len(t) for t in tables)
    bt = torch.full((S, width), -1, dtype=torch.int32)
    for i, t in enumerate(tables):
        bt[i, :len(t)] = torch.tensor(t, dtype=torch.int32)
    q_all = torch.cat(qs).reshape(S, nq * d)
    out = torch.full_like(q_all, float("nan"), device="cuda")
    ops.attention_tensor_core(out, dev(q_all), dev(pages), dev(bt), dev(torch.arange(S + 1, dtype=torch.int32)),
                              dev(torch.tensor(lens, dtype=torch.int32)), S, 0, 0, S, max(lens), nq, nkv, d, d ** -0.5, 0)
    torch.testing.assert_close(out.cpu().float(), torch.cat(refs).float(), rtol=2e-2, atol=2e-2)
    assert ops.take_wait_errors() == []
