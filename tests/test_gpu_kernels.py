"""Each CUDA kernel alone against its plain PyTorch version, at sizes the engine's models do not use."""

from types import SimpleNamespace

import numpy as np
import pytest
import torch

from plain_ops import PlainOps

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def ops():
    from llmserve_b200.ops import get_ops

    return get_ops("cuda")


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def close(a, b, dtype, atol32=1e-5, rel16=0.01):
    a, b = a.float().cpu(), b.float().cpu()
    err = (a - b).abs().max().item()
    bound = atol32 * max(1.0, b.abs().max().item()) if dtype == "float32" else rel16 * b.abs().max().item()
    assert err <= bound, f"max error {err:.3e} > {bound:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,H,V", [(1, 24, 37), (7, 100, 50), (33, 2048, 300)])
def test_embedding(ops, dtype, T, H, V):
    table = rnd(V, H, dtype=DT[dtype])
    ids = torch.randint(0, V, (T,), dtype=torch.int32)
    got = ops.embedding(ids.cuda(), table.cuda())
    assert got.dtype == torch.float32
    assert torch.equal(got.cpu(), PlainOps().embedding(ids, table))


@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("res_dtype", [None, "float32", "bfloat16"])
@pytest.mark.parametrize("T,H", [(1, 40), (5, 1000), (19, 4100)])
def test_add_rmsnorm(ops, out_dtype, res_dtype, T, H):
    x = rnd(T, H, seed=1, scale=3.0)
    r = None if res_dtype is None else rnd(T, H, dtype=DT[res_dtype], seed=2)
    w = 1 + rnd(H, seed=3, scale=0.1)
    xg = x.clone().cuda()
    got = ops.add_rmsnorm(xg, None if r is None else r.cuda(), w.cuda(), 1e-5, DT[out_dtype])
    xr = x.clone()
    ref = PlainOps().add_rmsnorm(xr, r, w, 1e-5, DT[out_dtype])
    assert torch.allclose(xg.cpu(), xr, atol=1e-6), "residual stream"
    close(got, ref, out_dtype, atol32=2e-6, rel16=0.005)
    rows = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32)
    xg2 = x.clone().cuda()
    got = ops.add_rmsnorm(xg2, None if r is None else r.cuda(), w.cuda(), 1e-5, DT[out_dtype], rows=rows.cuda())
    ref = PlainOps().add_rmsnorm(x.clone(), r, w, 1e-5, DT[out_dtype], rows=rows)
    assert torch.equal(xg2.cpu(), x), "rows mode must not write x"
    close(got, ref, out_dtype, atol32=2e-6, rel16=0.005)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,I", [(1, 7), (3, 160), (40, 2744)])
def test_silu_mul(ops, dtype, T, I):
    gu = rnd(T, 2 * I, dtype=DT[dtype], scale=2.0)
    close(ops.silu_mul(gu.cuda()), PlainOps().silu_mul(gu), dtype, atol32=1e-6, rel16=0.005)


@pytest.mark.parametrize("T,N,K", [(1, 5, 3), (3, 130, 70), (65, 64, 257), (130, 1000, 96)])
@pytest.mark.parametrize("bias", [False, True])
def test_gemm_f32_is_true_float32_and_batch_invariant(ops, T, N, K, bias):
    a, w = rnd(T, K, seed=1), rnd(N, K, seed=2)
    b = rnd(N, seed=3) if bias else None
    got = ops.linear(a.cuda(), w.cuda(), None if b is None else b.cuda(), out_dtype=torch.float32).cpu()
    ref = a.double() @ w.double().T + (0 if b is None else b.double())
    assert (got.double() - ref).abs().max() < 2e-6 * K**0.5 * 4
    # the same row gives the same bits whatever else is in the batch
    alone = ops.linear(a[T // 2 : T // 2 + 1].cuda(), w.cuda(), None if b is None else b.cuda(),
                       out_dtype=torch.float32).cpu()
    assert torch.equal(alone[0], got[T // 2])


@pytest.mark.parametrize("T,N,K", [(1, 48, 64), (9, 520, 200), (16, 128, 64), (17, 2048, 2048),
                                   (8, 16384, 2048), (4, 49152, 2048), (8, 6144, 2048), (2, 2048, 8192),
                                   (64, 136, 1000), (100, 384, 8192), (256, 1000, 520), (300, 136, 1000)])
@pytest.mark.parametrize("bias", [False, True])
def test_linear_bf16(ops, T, N, K, bias):
    """Few rows run the tcgen05 kernel (with and without split K), many rows the library."""
    a, w = rnd(T, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, seed=2)
    b = rnd(N, dtype=torch.bfloat16, seed=3) if bias else None
    ref = a.double() @ w.double().T + (0 if b is None else b.double())
    for od in (torch.bfloat16, torch.float32):
        got = ops.linear(a.cuda(), w.cuda(), None if b is None else b.cuda(), out_dtype=od)
        assert got.dtype == od and got.shape == (T, N)
        err = (got.double().cpu() - ref).abs().max().item()
        # float32 accumulation: the error is the rounding of the output only (bf16) or ~1e-6 relative
        bound = (2.0**-8 if od == torch.bfloat16 else 3e-6 * K**0.5) * ref.abs().max().item()
        assert err <= bound, (od, err, bound)
    ops.check_kernel_errors()


@pytest.mark.parametrize("T,N,K", [(1, 2048, 2048), (8, 200, 8192), (33, 6144, 520), (64, 130, 64),
                                   (300, 256, 520), (2048, 192, 272)])
def test_linear_bf16_adds_into_the_residual_stream(ops, T, N, K):
    a, w = rnd(T, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, seed=2, scale=0.05)
    x = rnd(T, N, seed=5)
    xg = x.clone().cuda()
    got = ops.linear(a.cuda(), w.cuda(), None, out_dtype=torch.float32, accumulate_into=xg)
    if got is not None:  # the kernel set may decline to accumulate and hand the product back
        xg += got
    ref = x.double() + a.double() @ w.double().T
    assert (xg.double().cpu() - ref).abs().max() <= 3e-6 * K**0.5 * ref.abs().max()
    ops.check_kernel_errors()


def test_pointwise_kernels_read_float32_sums(ops):
    """Activations may reach rope and the SiLU gate as float32 sums and leave as bfloat16."""
    gu = rnd(5, 2 * 104, seed=1, scale=2.0)
    got = ops.silu_mul(gu.cuda(), out_dtype=torch.bfloat16)
    assert got.dtype == torch.bfloat16
    close(got, PlainOps().silu_mul(gu), "bfloat16", rel16=0.005)
    nq, nk, D, page = 6, 2, 48, 8
    case = paged_case(3, [1, 20, 2], [30, 20, 9], nq, nk, D, page, torch.bfloat16, seed=2)
    qkv, kp, vp, tables, positions, token_seq, step = case
    qkv32 = rnd(qkv.shape[0], qkv.shape[1], seed=3)
    ang = torch.outer(torch.arange(64, dtype=torch.float64), 1.0 / (1e4 ** (torch.arange(0, D, 2, dtype=torch.float64) / D)))
    cos, sin = ang.cos().float(), ang.sin().float()
    kw = dict(num_heads=nq, num_kv_heads=nk, head_dim=D, positions=positions, token_seq=token_seq,
              block_tables=tables, page_tokens=page, out_dtype=torch.bfloat16)
    kp_ref, vp_ref = kp.clone(), vp.clone()
    q_ref = PlainOps().rope_kv_write(qkv32.clone(), cos=cos, sin=sin, k_pages=kp_ref, v_pages=vp_ref, **kw)
    kp_g, vp_g = kp.cuda(), vp.cuda()
    gkw = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in kw.items()}
    q_g = ops.rope_kv_write(qkv32.cuda(), cos=cos.cuda(), sin=sin.cuda(), k_pages=kp_g, v_pages=vp_g, **gkw)
    assert q_g.dtype == torch.bfloat16 and q_g.shape == (qkv.shape[0], nq * D)
    close(q_g, q_ref, "bfloat16", rel16=0.005)
    close(kp_g, kp_ref, "bfloat16", rel16=0.005)
    close(vp_g, vp_ref, "bfloat16", rel16=0.005)


def test_skinny_gemm_sees_every_k_and_every_row(ops):
    """One-hot inputs: a wrong swizzle, k offset or row mapping shows up as a misplaced value."""
    T, N, K = 5, 300, 328
    w = (torch.arange(N * K, dtype=torch.float32).reshape(N, K) % 251 - 125).to(torch.bfloat16)
    for k in (0, 15, 16, 63, 64, 200, 327):
        a = torch.zeros(T, K, dtype=torch.bfloat16)
        a[:, k] = torch.arange(1, T + 1).to(torch.bfloat16)
        got = ops.linear(a.cuda(), w.cuda(), None, out_dtype=torch.float32).cpu()
        assert torch.equal(got, a.float() @ w.float().T), k


@pytest.mark.parametrize("T,N,K", [(1, 2048, 2048), (8, 6144, 2048), (13, 1000, 8192), (32, 49152, 960),
                                   (17, 136, 1000), (5, 128, 64)])
def test_few_rows_product_gives_the_same_bits_every_run_and_in_every_batch(ops, T, N, K):
    """A tile's sum over k is shared between blocks, which add their parts as fixed-point numbers:
    two runs agree bit for bit, and a row gives the same bits whatever other rows are in the batch."""
    a, w = rnd(T, K, dtype=torch.bfloat16, seed=1).cuda(), rnd(N, K, dtype=torch.bfloat16, seed=2).cuda()
    first = ops.linear(a, w, None, out_dtype=torch.float32)
    for _ in range(3):
        assert torch.equal(ops.linear(a, w, None, out_dtype=torch.float32), first)
    # a row among fewer rows: the same bits, as long as the kernel's tile is the same (16 columns
    # for up to 16 rows, 32 beyond: the two share K between blocks differently)
    few = 1 if T <= 16 else 17
    assert torch.equal(ops.linear(a[T - few :].contiguous(), w, None, out_dtype=torch.float32), first[T - few :])
    x = rnd(T, N, seed=3).cuda()
    x1, x2 = x.clone(), x.clone()
    ops.linear(a, w, None, accumulate_into=x1)
    ops.linear(a, w, None, accumulate_into=x2)
    assert torch.equal(x1, x2) and torch.equal(x1, x + first)
    ops.check_kernel_errors()


@pytest.mark.parametrize("T,I,K", [(1, 64, 64), (8, 2560, 960), (17, 160, 200), (32, 100, 520),
                                   (3, 8192, 2048), (16, 272, 192)])
@pytest.mark.parametrize("bias", [False, True])
def test_gated_silu_in_the_product_kernel(ops, T, I, K, bias):
    """Gate rows and their up rows meet in one tile (two boxes of 64 rows); the gate reaches its
    activation as a float32 sum. Intermediate sizes that are no multiple of 64 leave a ragged tile."""
    h = rnd(T, K, dtype=torch.bfloat16, seed=1)
    w = rnd(2 * I, K, dtype=torch.bfloat16, seed=2, scale=0.2)
    b = rnd(2 * I, dtype=torch.bfloat16, seed=3) if bias else None
    got = ops.gated_silu(h.cuda(), w.cuda(), None if b is None else b.cuda(), out_dtype=torch.bfloat16)
    assert got.dtype == torch.bfloat16 and got.shape == (T, I)
    gu = h.double() @ w.double().T + (0 if b is None else b.double())
    g, u = gu[:, :I], gu[:, I:]
    ref = g / (1 + torch.exp(-g)) * u
    assert (got.double().cpu() - ref).abs().max() <= 2.0**-7 * ref.abs().max()
    again = ops.gated_silu(h.cuda(), w.cuda(), None if b is None else b.cuda(), out_dtype=torch.bfloat16)
    assert torch.equal(got, again)
    ops.check_kernel_errors()


@pytest.mark.parametrize("nq,nk,D,page", [(4, 2, 16, 16), (4, 1, 32, 8), (6, 2, 64, 32), (15, 5, 64, 16),
                                          (32, 32, 64, 16), (8, 2, 128, 48), (3, 1, 48, 16)])
@pytest.mark.parametrize("bias,rope,writes", [(False, True, True), (True, True, True),
                                              (False, False, True), (False, True, False)])
def test_projection_rotation_and_cache_write_in_one_kernel(ops, nq, nk, D, page, bias, rope, writes):
    """q|k|v projection, rotation and the write of k and v into shuffled pages, against the plain
    product followed by the plain rotation; head size 48 (no whole heads per tile) takes the
    two-kernel path. Untouched cache slots must keep their stale contents."""
    K = 200
    q_lens, ctx_lens = [1, 1, 1, 1, 1], [30, 1, 17, 64, 9]
    _, kp, vp, tables, positions, token_seq, _ = paged_case(5, q_lens, ctx_lens, nq, nk, D, page,
                                                            torch.bfloat16, seed=4)
    T = sum(q_lens)
    h = rnd(T, K, dtype=torch.bfloat16, seed=5)
    w = rnd((nq + 2 * nk) * D, K, dtype=torch.bfloat16, seed=6, scale=0.1)
    b = rnd((nq + 2 * nk) * D, dtype=torch.bfloat16, seed=7) if bias else None
    ang = torch.outer(torch.arange(80, dtype=torch.float64), 1.0 / (1e4 ** (torch.arange(0, D, 2, dtype=torch.float64) / D)))
    cos, sin = (ang.cos().float(), ang.sin().float()) if rope else (None, None)
    kw = dict(num_heads=nq, num_kv_heads=nk, head_dim=D, positions=positions, token_seq=token_seq,
              block_tables=tables, page_tokens=page, out_dtype=torch.bfloat16)
    kp_ref, vp_ref = kp.clone(), vp.clone()
    q_ref = PlainOps().project_rope_kv_write(h, w, b, cos=cos, sin=sin, k_pages=kp_ref if writes else None,
                                             v_pages=vp_ref if writes else None, **kw)
    dev = lambda t: None if t is None else t.cuda()
    kp_g, vp_g = kp.cuda(), vp.cuda()
    gkw = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in kw.items()}
    q_g = ops.project_rope_kv_write(dev(h), dev(w), dev(b), cos=dev(cos), sin=dev(sin),
                                    k_pages=kp_g if writes else None, v_pages=vp_g if writes else None, **gkw)
    assert q_g.dtype == torch.bfloat16 and q_g.shape == (T, nq * D)
    close(q_g, q_ref, "bfloat16", rel16=0.005)
    close(kp_g, kp_ref, "bfloat16", rel16=0.005)
    close(vp_g, vp_ref, "bfloat16", rel16=0.005)
    if not writes:
        assert torch.equal(kp_g.cpu(), kp) and torch.equal(vp_g.cpu(), vp)
    ops.check_kernel_errors()


def paged_case(nseq, q_lens, ctx_lens, nq, nk, D, page, dtype, seed=0, shuffle=True):
    """Random q/k/v rows, a cache whose pages are handed out in shuffled order."""
    g = torch.Generator().manual_seed(seed)
    blocks = [-(-c // page) for c in ctx_lens]
    num_pages = sum(blocks) + 3
    order = torch.randperm(num_pages, generator=g).tolist() if shuffle else list(range(num_pages))
    width = max(blocks)
    tables = torch.zeros(nseq, width, dtype=torch.int32)
    it = iter(order)
    for s in range(nseq):
        for b in range(blocks[s]):
            tables[s, b] = next(it)
    T = sum(q_lens)
    qkv = (torch.randn(T, (nq + 2 * nk) * D, generator=g)).to(dtype)
    # stale contents everywhere: huge values that would wreck the result if ever read
    k_pages = torch.full((num_pages, nk, page, D), 300.0).to(dtype)
    v_pages = torch.full((num_pages, nk, page, D), -7e4 if dtype == torch.float32 else -3e4).to(dtype)
    cu = np.zeros(nseq + 1, dtype=np.int32)
    cu[1:] = np.cumsum(q_lens)
    # fill the cached part (positions before this step's tokens) with random rows
    for s in range(nseq):
        for p in range(ctx_lens[s] - q_lens[s]):
            pg, off = int(tables[s, p // page]), p % page
            k_pages[pg, :, off] = torch.randn(nk, D, generator=g).to(dtype)
            v_pages[pg, :, off] = torch.randn(nk, D, generator=g).to(dtype)
    positions = torch.cat([torch.arange(c - q, c) for q, c in zip(q_lens, ctx_lens)]).int()
    token_seq = torch.cat([torch.full((q,), s) for s, q in enumerate(q_lens)]).int()
    step = SimpleNamespace(cu_q=torch.from_numpy(cu), ctx_lens=torch.tensor(ctx_lens, dtype=torch.int32),
                           q_lens=np.asarray(q_lens, dtype=np.int32), decode_splits=0,
                           max_decode_ctx=max([c for q, c in zip(q_lens, ctx_lens) if q == 1] or [0]))
    return qkv, k_pages, v_pages, tables, positions, token_seq, step


def run_attention(ops, case, nq, nk, D, page, window, max_pos, theta=10000.0, splits=0, rope=True):
    qkv, kp, vp, tables, positions, token_seq, step = case
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.float64) / D))
    ang = torch.outer(torch.arange(max_pos, dtype=torch.float64), inv)
    cos, sin = (ang.cos().float(), ang.sin().float()) if rope else (None, None)
    scale = D**-0.5
    plain = PlainOps()
    q_ref, kp_ref, vp_ref = qkv.clone(), kp.clone(), vp.clone()
    kw = dict(num_heads=nq, num_kv_heads=nk, head_dim=D)
    q_ref = plain.rope_kv_write(q_ref, **kw, positions=positions, token_seq=token_seq, cos=cos, sin=sin,
                                k_pages=kp_ref, v_pages=vp_ref, block_tables=tables, page_tokens=page)
    ref = plain.paged_attention(q_ref, **kw, scale=scale, window=window, k_pages=kp_ref,
                                v_pages=vp_ref, block_tables=tables, page_tokens=page, step=step)
    dev = lambda t: None if t is None else t.cuda()
    ops.check_attention_shape(D, qkv.dtype)
    q_g, kp_g, vp_g = qkv.cuda(), kp.cuda(), vp.cuda()
    q_g = ops.rope_kv_write(q_g, **kw, positions=dev(positions), token_seq=dev(token_seq), cos=dev(cos),
                            sin=dev(sin), k_pages=kp_g, v_pages=vp_g, block_tables=dev(tables),
                            page_tokens=page, out_dtype=qkv.dtype)
    gstep = SimpleNamespace(cu_q=step.cu_q.cuda(), ctx_lens=step.ctx_lens.cuda(), decode_splits=splits,
                            max_decode_ctx=step.max_decode_ctx)
    plan = {k: torch.from_numpy(v).cuda() for k, v in ops.attention_plan(step, qkv.dtype, D).items()}
    got = ops.paged_attention(q_g, **kw, scale=scale, window=window, k_pages=kp_g, v_pages=vp_g,
                              block_tables=dev(tables), page_tokens=page, step=gstep, plan=plan)
    return got, ref, (q_g, q_ref, kp_g, kp_ref, vp_g, vp_ref)


@pytest.mark.parametrize("window,splits", [(0, 0), (0, 1), (0, 5), (40, 3)])
@pytest.mark.parametrize("nq,nk,D,page,bias,rope", [(4, 4, 64, 16, False, True), (8, 2, 64, 8, True, True),
                                                    (8, 1, 64, 64, False, False), (4, 2, 128, 16, True, True),
                                                    (32, 32, 64, 16, False, True)])
def test_projection_rotation_cache_write_and_attention_in_two_launches(ops, nq, nk, D, page, bias, rope,
                                                                       window, splits):
    """A step of single tokens: the product leaves fixed-point sums and the attention kernel makes
    its queries and the step's key and value from them. Contexts from the new token alone to
    several partitions; the pages must end up as after the separate rotation kernel, the output
    must match the plain product, rotation and attention, and the sums must be left zero."""
    K = 136
    ctx_lens = [1, 2, 16, 17, 33, 130, 700, 64]
    n = len(ctx_lens)
    _, kp, vp, tables, positions, token_seq, step = paged_case(n, [1] * n, ctx_lens, nq, nk, D, page,
                                                               torch.bfloat16, seed=nq + page)
    h = rnd(n, K, dtype=torch.bfloat16, seed=5)
    w = rnd((nq + 2 * nk) * D, K, dtype=torch.bfloat16, seed=6, scale=0.1)
    b = rnd((nq + 2 * nk) * D, dtype=torch.bfloat16, seed=7) if bias else None
    ang = torch.outer(torch.arange(720, dtype=torch.float64), 1.0 / (1e4 ** (torch.arange(0, D, 2, dtype=torch.float64) / D)))
    cos, sin = (ang.cos().float(), ang.sin().float()) if rope else (None, None)
    kw = dict(num_heads=nq, num_kv_heads=nk, head_dim=D, scale=D**-0.5, window=window, writes=True,
              page_tokens=page, out_dtype=torch.bfloat16)
    kp_ref, vp_ref = kp.clone(), vp.clone()
    ref = PlainOps().project_attend(h, w, b, positions=positions, token_seq=token_seq, cos=cos, sin=sin,
                                    k_pages=kp_ref, v_pages=vp_ref, block_tables=tables, step=step,
                                    plan=None, **kw)
    dev = lambda t: None if t is None else t.cuda()
    ops.check_attention_shape(D, torch.bfloat16)
    kp_g, vp_g = kp.cuda(), vp.cuda()
    gstep = SimpleNamespace(cu_q=step.cu_q.cuda(), ctx_lens=step.ctx_lens.cuda(), decode_splits=splits,
                            max_decode_ctx=step.max_decode_ctx)
    plan = {k: torch.from_numpy(v).cuda() for k, v in ops.attention_plan(step, torch.bfloat16, D).items()}
    before = ops.launches
    got = ops.project_attend(dev(h), dev(w), dev(b), positions=dev(positions), token_seq=dev(token_seq),
                             cos=dev(cos), sin=dev(sin), k_pages=kp_g, v_pages=vp_g, block_tables=dev(tables),
                             step=gstep, plan=plan, **kw)
    assert ops.launches - before == 2
    close(got, ref, "bfloat16", rel16=0.02)
    close(kp_g, kp_ref, "bfloat16", rel16=0.005)
    close(vp_g, vp_ref, "bfloat16", rel16=0.005)
    sums = ops._sums[(n, (nq + 2 * nk) * D)]
    assert int(sums.abs().max()) == 0, "the attention kernel must leave the product's sums zero"
    # the same again through the separate kernels: the pages, written from the same sums, agree bit for bit
    kp_2, vp_2 = kp.cuda(), vp.cuda()
    try:
        ops.fuse_rotation_into_attention = False
        got_2 = ops.project_attend(dev(h), dev(w), dev(b), positions=dev(positions), token_seq=dev(token_seq),
                                   cos=dev(cos), sin=dev(sin), k_pages=kp_2, v_pages=vp_2, block_tables=dev(tables),
                                   step=gstep, plan=plan, **kw)
    finally:
        ops.fuse_rotation_into_attention = True
    assert torch.equal(kp_2, kp_g) and torch.equal(vp_2, vp_g)
    assert (got.float() - got_2.float()).abs().max() <= 0.02 * got_2.float().abs().max()
    ops.check_kernel_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq,nk,D,page", [(4, 4, 64, 16), (6, 2, 48, 8), (8, 1, 128, 32), (5, 5, 16, 4), (3, 1, 80, 7)])
def test_rope_kv_write_and_attention_mixed_batch(ops, dtype, nq, nk, D, page):
    q_lens = [1, 70, 1, 2, 130, 1]
    ctx_lens = [1, 70, 513, 40, 300, 65]
    case = paged_case(6, q_lens, ctx_lens, nq, nk, D, page, DT[dtype], seed=4)
    got, ref, (q_g, q_ref, kp_g, kp_ref, vp_g, vp_ref) = run_attention(ops, case, nq, nk, D, page, 0, 600)
    close(q_g[:, : nq * D], q_ref[:, : nq * D], dtype, atol32=2e-6, rel16=0.005)
    close(kp_g, kp_ref, dtype, atol32=2e-6, rel16=0.005)
    assert torch.equal(vp_g.cpu(), vp_ref)
    close(got, ref, dtype, atol32=1e-5, rel16=0.02)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [1, 5, 64, 100])
def test_attention_window_edges(ops, dtype, window):
    q_lens, ctx_lens = [1, 97, 1, 3], [200, 150, 64, 66]
    case = paged_case(4, q_lens, ctx_lens, 4, 2, 32, 16, DT[dtype], seed=6)
    got, ref, _ = run_attention(ops, case, 4, 2, 32, 16, window, 256)
    close(got, ref, dtype, atol32=1e-5, rel16=0.02)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("splits", [1, 3, 16, 40, 64])
def test_decode_split_counts_agree(ops, dtype, splits):
    q_lens, ctx_lens = [1, 1, 1], [1000, 17, 255]
    case = paged_case(3, q_lens, ctx_lens, 6, 2, 64, 16, DT[dtype], seed=8)
    got, ref, _ = run_attention(ops, case, 6, 2, 64, 16, 0, 1024, splits=splits)
    close(got, ref, dtype, atol32=1e-5, rel16=0.02)


@pytest.mark.parametrize("window", [0, 37])
@pytest.mark.parametrize("page", [8, 16, 32, 48])  # 8: a tile of 16 keys straddles pages; 48: no power of two
@pytest.mark.parametrize("nq,nk,D", [(2, 2, 64), (2, 1, 64), (6, 2, 64), (4, 1, 64), (5, 1, 64), (8, 1, 64),
                                     (12, 1, 64), (16, 1, 64), (32, 2, 64),
                                     (3, 3, 128), (8, 2, 128), (8, 1, 128), (12, 1, 128)])
def test_decode_on_tensor_core_tiles(ops, nq, nk, D, page, window):
    """Single tokens in bfloat16: up to 8 query heads per key/value head (head sizes 64 and 128)
    and 9 to 16 heads (head size 64) take the two tensor-core kernels, 12 heads of size 128 the
    CUDA-core one. Contexts that end inside a tile of 16 keys, start inside one (window,
    partitions), and of one token."""
    ctx_lens = [1, 16, 17, 100, 333]
    case = paged_case(5, [1] * 5, ctx_lens, nq, nk, D, page, torch.bfloat16, seed=nq + page)
    for splits in (1, 4):
        got, ref, _ = run_attention(ops, case, nq, nk, D, page, window, 512, splits=splits)
        close(got, ref, "bfloat16", atol32=1e-5, rel16=0.02)


@pytest.mark.parametrize("batch,ctx,nq,nk", [(64, 2100, 8, 8), (64, 2100, 6, 2), (1, 2300, 32, 32), (40, 4100, 4, 2)])
def test_decode_over_long_contexts_at_large_batch(ops, batch, ctx, nq, nk):
    """The benchmark's decode shapes: 64 sequences of more than 2000 keys each (one partition per
    sequence), one sequence of 2300 keys (17 partitions, the variant that loads its first tile
    early), 40 sequences of 4100. All context lengths differ, pages are shuffled."""
    D, page = 64, 16
    ctx_lens = [ctx - 7 * i % 97 for i in range(batch)]
    case = paged_case(batch, [1] * batch, ctx_lens, nq, nk, D, page, torch.bfloat16, seed=batch)
    got, ref, _ = run_attention(ops, case, nq, nk, D, page, 0, 4200)
    close(got, ref, "bfloat16", atol32=1e-5, rel16=0.02)


@pytest.mark.parametrize("style", ["partial", "interleaved"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_rotations_are_a_permutation_and_a_table(ops, style, dtype):
    """The kernels rotate the pairs (i, i + D/2) of a head with cos/sin [positions, D/2]. A rotation
    of only the first R dims (pairs (i, i + R/2)) or of neighbouring dims (pairs (2i, 2i + 1)) is
    the same computation after a fixed reordering of the head's dims in q and k (rows of the
    projection, done once when weights are read: q . k does not change when both are reordered
    alike) with cos = 1, sin = 0 in the table for the pairs that stay as they are. Shown here on
    one sequence: prompt portion, then single tokens, against the rotation written out plainly."""
    nq, nk, D, page, R = 4, 2, 64, 16, 32
    n_prompt, n_new = 21, 3
    n = n_prompt + n_new
    g = torch.Generator().manual_seed(11)
    q = torch.randn(n, nq, D, generator=g, dtype=torch.float64)
    k = torch.randn(n, nk, D, generator=g, dtype=torch.float64)
    v = torch.randn(n, nk, D, generator=g, dtype=torch.float64)
    pos = torch.arange(n, dtype=torch.float64)
    if style == "partial":
        inv = 1.0 / (1e4 ** (torch.arange(0, R, 2, dtype=torch.float64) / R))
        pairs = [(i, i + R // 2) for i in range(R // 2)]                   # rotated pairs, their angles inv[i]
        rest = list(range(R, D))
    else:
        inv = 1.0 / (1e4 ** (torch.arange(0, D, 2, dtype=torch.float64) / D))
        pairs = [(2 * i, 2 * i + 1) for i in range(D // 2)]
        rest = []
    ang = pos[:, None] * inv[None, :]                                       # [n, len(pairs)]

    def rotate_plainly(x):
        y = x.clone()
        for j, (a, b) in enumerate(pairs):
            c, s_ = ang[:, j].cos()[:, None], ang[:, j].sin()[:, None]
            y[..., a] = x[..., a] * c - x[..., b] * s_
            y[..., b] = x[..., b] * c + x[..., a] * s_
        return y

    qr, kr = rotate_plainly(q), rotate_plainly(k)
    want = torch.zeros(n, nq, D, dtype=torch.float64)
    for h in range(nq):
        sc = (qr[:, h] @ kr[:, h // (nq // nk)].T) * D**-0.5
        sc = sc.masked_fill(torch.ones(n, n, dtype=torch.bool).triu(1), float("-inf"))
        want[:, h] = sc.softmax(-1) @ v[:, h // (nq // nk)]
    # the reordering: first halves of the pairs, then half of the untouched dims; then the second halves
    order = [a for a, _ in pairs] + rest[: len(rest) // 2] + [b for _, b in pairs] + rest[len(rest) // 2 :]
    assert sorted(order) == list(range(D))
    cos = torch.ones(n, D // 2, dtype=torch.float64)
    sin = torch.zeros(n, D // 2, dtype=torch.float64)
    cos[:, : len(pairs)], sin[:, : len(pairs)] = ang.cos(), ang.sin()
    dt = DT[dtype]
    qkv = torch.cat([q[:, :, order].reshape(n, -1), k[:, :, order].reshape(n, -1), v.reshape(n, -1)], 1).to(dt)
    ops.check_attention_shape(D, dt)
    pages = -(-n // page) + 1
    kp = torch.zeros(pages, nk, page, D, dtype=dt, device="cuda")
    vp = torch.zeros_like(kp)
    tables = torch.arange(pages, dtype=torch.int32).flip(0)[None].contiguous().cuda()
    got = []
    for a, b in [(0, n_prompt)] + [(i, i + 1) for i in range(n_prompt, n)]:
        T = b - a
        step = SimpleNamespace(cu_q=torch.tensor([0, T], dtype=torch.int32), ctx_lens=torch.tensor([b], dtype=torch.int32),
                               q_lens=np.asarray([T], dtype=np.int32), decode_splits=0, max_decode_ctx=b if T == 1 else 0)
        plan = {kk: torch.from_numpy(vv).cuda() for kk, vv in ops.attention_plan(step, dt, D).items()}
        gstep = SimpleNamespace(cu_q=step.cu_q.cuda(), ctx_lens=step.ctx_lens.cuda(), decode_splits=0,
                                max_decode_ctx=step.max_decode_ctx)
        qg = ops.rope_kv_write(qkv[a:b].contiguous().cuda(), num_heads=nq, num_kv_heads=nk, head_dim=D,
                               positions=torch.arange(a, b, dtype=torch.int32).cuda(),
                               token_seq=torch.zeros(T, dtype=torch.int32).cuda(), cos=cos.float().cuda(),
                               sin=sin.float().cuda(), k_pages=kp, v_pages=vp, block_tables=tables,
                               page_tokens=page, out_dtype=dt)
        got.append(ops.paged_attention(qg, num_heads=nq, num_kv_heads=nk, head_dim=D, scale=D**-0.5, window=0,
                                       k_pages=kp, v_pages=vp, block_tables=tables, page_tokens=page,
                                       step=gstep, plan=plan).double().cpu())
    got = torch.cat(got).view(n, nq, D)
    bound = 2e-5 if dtype == "float32" else 0.02 * float(want.abs().max())
    assert (got - want).abs().max() <= bound, float((got - want).abs().max())


@pytest.mark.parametrize("window", [0, 75])
@pytest.mark.parametrize("nq,nk,D,page", [(4, 4, 64, 16), (8, 1, 64, 64), (6, 2, 64, 32), (8, 2, 128, 16), (3, 3, 128, 128)])
def test_the_three_decode_kernels_agree(ops, nq, nk, D, page, window):
    """Single tokens on the CUDA cores, on mma.sync fed by plain loads, and on mma.sync fed by TMA
    (forced: alone it serves large grids only): ragged contexts from 1 key to several partitions,
    shuffled pages whose unused rows hold huge values, one and several partitions."""
    ctx_lens = [1, 15, 16, 17, 33, 130, 513, 700, 64, 129]
    n = len(ctx_lens)
    case = paged_case(n, [1] * n, ctx_lens, nq, nk, D, page, torch.bfloat16, seed=nq + D)
    outs = {}
    try:
        for kernel in (1, 2, 3):
            ops.attention_kernel = kernel
            for splits in (1, 3, 7):
                got, ref, _ = run_attention(ops, case, nq, nk, D, page, window, 1024, splits=splits)
                close(got, ref, "bfloat16", rel16=0.02)
                outs[kernel, splits] = got.float().cpu()
    finally:
        ops.attention_kernel = 0
    ops.check_kernel_errors()
    for splits in (1, 3, 7):
        assert (outs[3, splits] - outs[2, splits]).abs().max() <= 0.02 * outs[2, splits].abs().max()


def test_tma_fed_decode_ignores_rows_that_were_never_written(ops):
    """The TMA-fed kernel copies whole tiles of 16 rows; rows at or beyond the context length may
    hold any bits (here NaN and infinity) and must not reach the result."""
    nq, nk, D, page = 4, 2, 64, 32
    ctx_lens = [5, 40, 47, 200]
    case = list(paged_case(4, [1] * 4, ctx_lens, nq, nk, D, page, torch.bfloat16, seed=9))
    k_pages, v_pages, tables = case[1], case[2], case[3]
    for s, ctx in enumerate(ctx_lens):
        for pos in range(ctx, -(-ctx // page) * page):
            pg, off = int(tables[s, pos // page]), pos % page
            k_pages[pg, :, off] = float("nan")
            v_pages[pg, :, off] = float("inf") if pos % 2 else float("nan")
    try:
        ops.attention_kernel = 3
        for splits in (1, 2):
            got, ref, _ = run_attention(ops, tuple(case), nq, nk, D, page, 0, 512, splits=splits)
            assert torch.isfinite(got.float()).all()
            close(got, ref, "bfloat16", rel16=0.02)
    finally:
        ops.attention_kernel = 0
    ops.check_kernel_errors()


@pytest.mark.parametrize("kernel", [2, 3])
@pytest.mark.parametrize("group", [3, 8, 12])
def test_grouped_decode_finds_one_far_key(ops, group, kernel):
    """One key among 900 wins every head's softmax; the output must be its value row."""
    nk, D, page, ctx = 2, 64, 16, 900
    nq = nk * group
    for far in (0, 15, 16, 450, 899):
        case = list(paged_case(1, [1], [ctx], nq, nk, D, page, torch.bfloat16, seed=far))
        qkv, k_pages, v_pages, tables = case[0], case[1], case[2], case[3]
        q = torch.zeros(nq, D)
        q[:, 3] = 6.0
        qkv[0, : nq * D] = q.flatten().to(torch.bfloat16)
        pg, off = int(tables[0, far // page]), far % page
        if far == ctx - 1:  # the key of this step's token comes from the projection itself
            k = torch.zeros(nk, D); k[:, 3] = 30.0
            qkv[0, nq * D : (nq + nk) * D] = k.flatten().to(torch.bfloat16)
        else:
            k_pages[pg, :, off] = 0.0
            k_pages[pg, :, off, 3] = 30.0
        try:
            ops.attention_kernel = kernel  # 3 (TMA-fed) serves groups of up to 8; 12 falls to the other
            got, ref, _ = run_attention(ops, tuple(case), nq, nk, D, page, 0, 1024, splits=3, rope=False)
        finally:
            ops.attention_kernel = 0
        close(got, ref, "bfloat16", atol32=1e-5, rel16=0.02)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("far", [0, 15, 16, 700, 1023])
def test_one_far_key_stands_out(ops, dtype, far):
    """One key among a thousand is made to win the softmax; the output must be its value row."""
    nq = nk = 2
    D, page, ctx = 64, 16, 1024
    for q_lens in ([1], [24]):
        case = paged_case(1, q_lens, [ctx], nq, nk, D, page, DT[dtype], seed=far + 1)
        qkv, kp, vp, tables, positions, token_seq, step = case
        if far >= ctx - q_lens[0]:
            continue  # the far key must lie in the cached part
        qkv[-1, : nq * D] = 0
        qkv[-1, 3] = 8.0
        qkv[-1, D + 3] = 8.0  # both heads look along dimension 3
        pg, off = int(tables[0, far // page]), far % page
        kp[pg, :, off] = 0
        kp[pg, :, off, 3] = 20.0
        got, ref, _ = run_attention(ops, case, nq, nk, D, page, 0, ctx, rope=False)
        want = vp[pg, :, off].float().reshape(-1)
        assert (got[-1].float().cpu() - want).abs().max() < (1e-4 if dtype == "float32" else 0.02)
        close(got, ref, dtype, atol32=1e-5, rel16=0.02)


@pytest.mark.parametrize("page", [8, 16, 64, 128])
@pytest.mark.parametrize("nq,nk", [(4, 2), (3, 3)])
def test_the_three_prefill_kernels_agree(ops, page, nq, nk):
    """tcgen05 (head size 64), mma.sync and CUDA-core kernels on the same ragged batch."""
    q_lens, ctx_lens = [150, 64, 2, 300, 129], [150, 200, 70, 300, 1000]
    case = paged_case(5, q_lens, ctx_lens, nq, nk, 64, page, torch.bfloat16, seed=3)
    outs = []
    try:
        for kernel in (0, 1, 2):
            ops.attention_kernel = kernel
            got, ref, _ = run_attention(ops, case, nq, nk, 64, page, 0, 1024)
            close(got, ref, "bfloat16", rel16=0.02)
            outs.append(got.float().cpu())
    finally:
        ops.attention_kernel = 0
    ops.check_kernel_errors()
    assert (outs[0] - outs[1]).abs().max() <= 0.02 * outs[1].abs().max()


@pytest.mark.parametrize("far", [0, 63, 64, 700, 1900])
def test_tensor_core_prefill_finds_one_far_key(ops, far):
    """A long portion whose last query looks at one key among two thousand (tcgen05 path)."""
    nq = nk = 2
    D, page, ctx, q_len = 64, 16, 2048, 130
    case = paged_case(1, [q_len], [ctx], nq, nk, D, page, torch.bfloat16, seed=far + 7)
    qkv, kp, vp, tables, positions, token_seq, step = case
    qkv[-1, : nq * D] = 0
    qkv[-1, 5] = 8.0
    qkv[-1, D + 5] = 8.0
    pg, off = int(tables[0, far // page]), far % page
    kp[pg, :, off] = 0
    kp[pg, :, off, 5] = 20.0
    got, ref, _ = run_attention(ops, case, nq, nk, D, page, 0, ctx, rope=False)
    want = vp[pg, :, off].float().reshape(-1)
    assert (got[-1].float().cpu() - want).abs().max() < 0.02
    close(got, ref, "bfloat16", rel16=0.02)
    ops.check_kernel_errors()


def test_unsupported_head_size_is_refused(ops):
    with pytest.raises(ValueError, match="head size"):
        ops.check_attention_shape(40, torch.bfloat16)
    with pytest.raises(ValueError, match="head size"):
        ops.check_attention_shape(512, torch.float32)
