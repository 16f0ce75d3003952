"""Each kernel alone against a plain float32 reference of the same op, at other sizes than the
engine's tiny models use (widths and vocabularies that are no power of two, head sizes 48, 80 and
112, odd numbers of heads and groups)."""

import math

import numpy as np
import pytest
import torch

from tests.plain import llama_plain as P

pytestmark = pytest.mark.gpu

DT = [torch.float32, torch.bfloat16]


def dev(x):
    return x.to("cuda")


def tol(dtype, f32=1e-5, bf16=2e-2):
    return f32 if dtype == torch.float32 else bf16


@pytest.mark.parametrize("dtype", DT)
def test_embedding(dtype):
    from rust_llm_inference_server_b200 import ops
    table = torch.randn(301, 80).to(dtype)
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32)
    out = torch.empty(5, 80, device="cuda")
    ops.embedding(dev(ids), dev(table), out)
    assert torch.equal(out.cpu(), P.embedding(ids, table.float()))


@pytest.mark.parametrize("hidden,scale", [(80, None), (2048, None), (328, 5.5)])
def test_embedding_that_leaves_the_first_norm_to_the_product_after_it(hidden, scale):
    """The lookup of a decode step: the float32 rows as `embedding` writes them, bf16(row * norm
    weight), and the sums of squares of every 128 features; and the product that takes them gives
    what the norm followed by the product gives."""
    from rust_llm_inference_server_b200 import ops
    torch.manual_seed(hidden)
    table = torch.randn(301, hidden).bfloat16()
    ids = torch.tensor([0, 300, 17, 17, 5, 9, 250], dtype=torch.int32)
    w_norm = torch.randn(hidden)
    eps = 1e-5
    out = torch.empty(7, hidden, device="cuda")
    rows = ops.embedding_sink(dev(ids), dev(table), out, scale, ops.ResidualSink(out, dev(w_norm), eps))
    want = P.embedding(ids, table.float()) * (1.0 if scale is None else scale)
    assert torch.equal(out.cpu(), want)
    assert torch.equal(rows.x.cpu(), (want * w_norm).bfloat16())
    tiles = (hidden + 127) // 128
    assert rows.partials.shape == (tiles, 7)
    for j in range(tiles):
        ss = (want[:, j * 128:(j + 1) * 128].double() ** 2).sum(1)
        assert bool(((rows.partials[j].cpu().double() - ss).abs() <= 1e-5 * ss + 1e-12).all())
    w = (torch.randn(256, hidden) * 0.05).bfloat16()
    got = ops.linear(rows, dev(w)).float().cpu()
    ref = ops.linear(ops.rmsnorm(out.clone(), dev(w_norm), eps, torch.empty(7, hidden, dtype=torch.bfloat16, device="cuda")),
                     dev(w)).float().cpu()
    assert bool(((got - ref).abs() <= 2.0 ** -6 * ref.abs() + 2e-2).all())


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("hidden", [80, 1000, 4100])
def test_rmsnorm_with_residual_and_rows(dtype, hidden):
    from rust_llm_inference_server_b200 import ops
    torch.manual_seed(hidden)
    T = 7
    resid, delta = torch.randn(T, hidden) * 3, torch.randn(T, hidden).to(dtype)
    w = torch.randn(hidden)
    eps = 3e-6
    r = dev(resid.clone())
    out = torch.empty(T, hidden, dtype=dtype, device="cuda")
    ops.rmsnorm(r, dev(w), eps, out, dev(delta))
    want_resid = resid + delta.float()
    assert torch.allclose(r.cpu(), want_resid, atol=1e-6)
    want = P.rms_norm(want_resid, w, eps)
    assert (out.float().cpu() - want).abs().max() <= tol(dtype, 2e-5, 5e-2)
    out2 = torch.empty(T, hidden, dtype=dtype, device="cuda")
    ops.rmsnorm(r, dev(w), eps, out2)          # no delta: the residual stays
    assert torch.equal(out2, out) and torch.allclose(r.cpu(), want_resid, atol=1e-6)
    rows = torch.tensor([6, 0, 3], dtype=torch.int32)
    r3 = dev(resid.clone())
    out3 = torch.empty(3, hidden, dtype=dtype, device="cuda")
    ops.rmsnorm(r3, dev(w), eps, out3, dev(delta), dev(rows))
    assert torch.equal(out3, out[rows.long()]) and torch.equal(r3.cpu(), resid)


@pytest.mark.parametrize("dtype", DT)
def test_swiglu(dtype):
    from rust_llm_inference_server_b200 import ops
    gu = (torch.randn(5, 2 * 176) * 3).to(dtype)
    out = torch.empty(5, 176, dtype=dtype, device="cuda")
    ops.swiglu(dev(gu), out)
    g, u = gu.float()[:, :176], gu.float()[:, 176:]
    want = torch.nn.functional.silu(g) * u
    # one rounding of the result: half a unit in the last place, 2^-24 or 2^-9 relative
    rel = 2.0 ** -22 if dtype == torch.float32 else 2.0 ** -8
    assert bool(((out.float().cpu() - want).abs() <= rel * want.abs() + 1e-6).all())


@pytest.mark.parametrize("shape", [(1, 1, 1), (3, 301, 80), (70, 130, 257), (129, 64, 1000)])
def test_float32_matrix_product_is_true_float32_and_row_independent(shape):
    from rust_llm_inference_server_b200 import ops
    M, N, K = shape
    torch.manual_seed(M)
    a, w = torch.randn(M, K), torch.randn(N, K)
    out = ops.gemm_f32(dev(a), dev(w)).cpu()
    want = (a.double() @ w.double().t())
    assert (out.double() - want).abs().max() <= 1e-5 * max(1.0, math.sqrt(K))
    # TF32 would show an error near 1e-3 * |a||w|; and a row's result does not depend on the batch
    one = ops.gemm_f32(dev(a[M // 2:M // 2 + 1].contiguous()), dev(w)).cpu()
    assert torch.equal(one[0], out[M // 2])


@pytest.mark.parametrize("shape", [(1, 8, 8), (8, 3072, 2048), (3, 301, 80), (16, 520, 176), (13, 64, 8200), (5, 1000, 96),
                                   (8, 20000, 2048), (2, 2048, 8192), (4, 1500, 4104), (17, 520, 264), (40, 3072, 2048),
                                   (100, 1096, 1032), (128, 2048, 8192), (24, 3072, 2048), (32, 301, 80), (64, 2048, 8192),
                                   (48, 16384, 2048), (33, 1000, 4104), (64, 136, 64), (20, 128, 2048)])
def test_streaming_product_for_decode_rows(shape):
    """The tcgen05 weight-streaming kernel: few and many features (one CTA, clusters of 2 to 16
    splitting k), k that is no multiple of a stage, every row count up to 128."""
    from rust_llm_inference_server_b200 import ops
    M, N, K = shape
    torch.manual_seed(N)
    x, w = torch.randn(M, K).bfloat16(), (torch.randn(N, K) * 0.05).bfloat16()
    want = x.double() @ w.double().t()
    got32 = ops.stream_gemm(dev(x), dev(w), torch.float32).cpu()
    assert (got32.double() - want).abs().max() <= 2e-5 * max(1.0, math.sqrt(K))    # float32 sums of exact products
    got16 = ops.stream_gemm(dev(x), dev(w)).cpu()
    assert bool(((got16.double() - want).abs() <= 2.0 ** -8 * want.abs() + 1e-4).all())
    assert torch.equal(ops.stream_gemm(dev(x), dev(w)).cpu(), got16)                  # the same again: no race in the sums
    if M <= ops.STREAM_GEMM_ROWS:
        assert torch.equal(ops.linear(dev(x), dev(w)).cpu(), got16)               # `linear` takes this path
    one = ops.stream_gemm(dev(x[M // 2:M // 2 + 1].contiguous()), dev(w), torch.float32).cpu()
    assert torch.equal(one[0], got32[M // 2])                                     # a row ignores its neighbours
    ops.check_device_errors()


@pytest.mark.parametrize("M,N,K", [(1, 2048, 2048), (8, 2048, 8192), (16, 520, 264), (5, 1000, 4104), (3, 128, 64)])
def test_streaming_product_takes_a_norm_apart(M, N, K):
    """The norm between two decode products without a kernel of its own: the first product adds
    its result to the residual stream and leaves bf16(resid * weight) and sums of squares by 128
    features (one CTA, and clusters that split k; widths that are no multiple of 128), the second
    multiplies by the row's scale.  Against the plain formulas, and against itself run twice."""
    from rust_llm_inference_server_b200 import ops
    torch.manual_seed(N + K)
    x, w = torch.randn(M, K).bfloat16(), (torch.randn(N, K) * 0.05).bfloat16()
    resid0, nw, eps = torch.randn(M, N) * 2, torch.rand(N) + 0.5, 1e-5
    resid0[0, 3 % N] = 300.0                                  # one feature that carries most of a row's square
    resid = dev(resid0.clone())
    rows = ops.stream_gemm(dev(x), dev(w), sink=ops.ResidualSink(resid, dev(nw), eps))
    delta = x.double() @ w.double().t()
    new = resid.cpu()
    assert bool(((new.double() - resid0.double() - delta).abs() <= 2.0 ** -8 * delta.abs() + 1e-4).all())
    assert torch.equal(rows.x.cpu(), (new * nw).bfloat16())                   # from the sums it stored, exactly
    P_ = (N + 127) // 128
    assert rows.partials.shape == (P_, M) and rows.dim == N
    sq = torch.zeros(P_ * 128, M, dtype=torch.float64)
    sq[:N] = new.double().t() ** 2
    want_p = sq.view(P_, 128, M).sum(1)
    assert bool(((rows.partials.cpu().double() - want_p).abs() <= 1e-6 * want_p + 1e-12).all())
    resid2 = dev(resid0.clone())
    again = ops.stream_gemm(dev(x), dev(w), sink=ops.ResidualSink(resid2, dev(nw), eps))
    assert torch.equal(resid2, resid) and torch.equal(again.partials, rows.partials)      # no race in the sums
    one = dev(resid0[M // 2:M // 2 + 1].clone())
    r1 = ops.stream_gemm(dev(x[M // 2:M // 2 + 1].contiguous()), dev(w), sink=ops.ResidualSink(one, dev(nw), eps))
    assert torch.equal(one[0], resid[M // 2]) and torch.equal(r1.partials[:, 0], rows.partials[:, M // 2])   # a row ignores its neighbours

    # the second product: plain, float32 and gated epilogues apply the scale
    I = 264
    w2 = (torch.randn(2 * I, N) * 0.05).bfloat16()
    rstd = 1.0 / torch.sqrt((new.double() ** 2).mean(1) + eps)
    want = (rows.x.cpu().double() @ w2.double().t()) * rstd[:, None]
    got32 = ops.stream_gemm(rows, dev(w2), torch.float32).cpu()
    assert bool(((got32.double() - want).abs() <= 1e-5 * want.abs() + 2e-5 * math.sqrt(N)).all())
    got16 = ops.linear(rows, dev(w2)).cpu()
    assert bool(((got16.double() - want).abs() <= 2.0 ** -8 * want.abs() + 1e-4).all())
    gated = ops.stream_gemm(rows, dev(w2), swiglu4=True).cpu()
    g, u = want.view(M, -1, 2, 4)[:, :, 0].reshape(M, I), want.view(M, -1, 2, 4)[:, :, 1].reshape(M, I)
    wg = torch.nn.functional.silu(g) * u
    assert bool(((gated.double() - wg).abs() <= 2.0 ** -7 * wg.abs() + 1e-3).all())
    # and the whole against the norm as a kernel of its own followed by the product (two roundings apart)
    normed = P.rms_norm(new, nw, eps).bfloat16()
    ref = normed.double() @ w2.double().t()
    assert bool(((got32.double() - ref).abs() <= 2.0 ** -7 * ref.abs() + 2.0 ** -8 * ref.abs().max()).all())
    ops.check_device_errors()


def test_streaming_product_refuses_what_it_cannot_take():
    from rust_llm_inference_server_b200 import ops
    from rust_llm_inference_server_b200.ops.library import KernelError
    with pytest.raises(KernelError, match="rows"):
        ops.stream_gemm(dev(torch.randn(129, 64).bfloat16()), dev(torch.randn(8, 64).bfloat16()))
    with pytest.raises(KernelError, match="multiple of 8"):
        ops.stream_gemm(dev(torch.randn(2, 36).bfloat16()), dev(torch.randn(8, 36).bfloat16()))


@pytest.mark.parametrize("I,K,M", [(8, 16, 2), (176, 80, 7), (8192, 2048, 8), (500, 264, 33), (1024, 512, 128),
                                   (8192, 2048, 24), (448, 320, 64), (388, 2048, 32)])
def test_streaming_product_with_gating_and_interleaved_gating_kernel(I, K, M):
    from rust_llm_inference_server_b200 import ops
    torch.manual_seed(I)
    x = torch.randn(M, K).bfloat16()
    g, u = (torch.randn(I, K) * 0.1).bfloat16(), (torch.randn(I, K) * 0.1).bfloat16()
    w = torch.stack([g.view(-1, 4, K), u.view(-1, 4, K)], dim=1).reshape(2 * I, K).contiguous()
    gate, up = x.double() @ g.double().t(), x.double() @ u.double().t()
    want = torch.nn.functional.silu(gate) * up
    got = ops.stream_gemm(dev(x), dev(w), swiglu4=True).cpu()
    assert got.shape == (M, I)
    assert bool(((got.double() - want).abs() <= 2.0 ** -7 * want.abs() + 1e-3).all())
    # the two-kernel path of longer batches: product, then the gating kernel on the interleaved layout
    gu = (x.double() @ w.double().t()).float()
    for dtype in DT:
        out = torch.empty(M, I, dtype=dtype, device="cuda")
        ops.swiglu(dev(gu.to(dtype)), out, interleave=4)
        gq, uq = gu.to(dtype).double().view(M, -1, 2, 4)[:, :, 0].reshape(M, I), gu.to(dtype).double().view(M, -1, 2, 4)[:, :, 1].reshape(M, I)
        w2 = torch.nn.functional.silu(gq) * uq
        assert bool(((out.double().cpu() - w2).abs() <= 2.0 ** -7 * w2.abs() + 1e-5).all())


@pytest.mark.parametrize("pair", [True, False])
@pytest.mark.parametrize("shape,epilogue", [((128, 256, 64), "float32"), ((128, 256, 512), "float32"), ((300, 520, 200), "plain"),
                                            ((129, 264, 8), "float32"), ((333, 1008, 96), "swiglu4"),
                                            ((2048, 2048, 2048), "plain"), ((1024, 4096, 2048), "swiglu4"),
                                            ((700, 1536, 8192), "plain"), ((256, 256, 64), "plain"),
                                            ((2048 + 37, 19 * 256 + 24, 448), "plain"), ((40 * 256 + 1, 512, 72), "float32")])
def test_tcgen05_product_with_its_epilogues(shape, epilogue, pair):
    """The TMA-fed tensor-memory GEMM against a float32 product: whole tiles, ragged M, N and K,
    many tiles a CTA (both accumulator buffers in use, the ring of stages walked several times),
    and the SwiGLU epilogue; with two SMs to a tile of 256 x 256 (more than 128 rows) and with one
    CTA to a tile of 128 x 256, whose results are the same bits."""
    from rust_llm_inference_server_b200 import ops
    M, N, K = shape
    torch.manual_seed(M + N)
    x, w = torch.randn(M, K).bfloat16(), (torch.randn(N, K) * 0.05).bfloat16()
    ops.debug_set("gemm_pair", -1 if pair else 0)
    try:
        got = ops.gemm_tcgen05(dev(x), dev(w), epilogue).float().cpu()
        ops.check_device_errors()                      # no bounded wait ran out
        if pair:
            ops.debug_set("gemm_pair", 0)
            assert torch.equal(got, ops.gemm_tcgen05(dev(x), dev(w), epilogue).float().cpu())
    finally:
        ops.debug_set("gemm_pair", -1)
    want = (x.double() @ w.double().t())
    if epilogue == "swiglu4":
        r = want.view(M, -1, 2, 4)
        want = (torch.nn.functional.silu(r[:, :, 0]) * r[:, :, 1]).reshape(M, N // 2)
    rel = 2.0 ** -20 if epilogue == "float32" else 2.0 ** -7
    assert bool(((got.double() - want).abs() <= rel * want.abs() + 1e-5 * max(1.0, math.sqrt(K))).all())
    with pytest.raises(ops.KernelError):
        ops.gemm_tcgen05(dev(x[:64].contiguous()), dev(w), epilogue)        # fewer than 128 rows: refused


def cache_from(k, v, page_size, n_pages, seed=0):
    """Scatters contiguous k, v [(requests) x (len, nkv, d)] into a paged cache with shuffled,
    interleaved pages; returns caches [pages, nkv, page, d] and the block tables."""
    rng = np.random.default_rng(seed)
    nkv, d = k[0].shape[1:]
    kc = torch.full((n_pages, nkv, page_size, d), float("nan"))
    vc = torch.full((n_pages, nkv, page_size, d), float("nan"))
    perm = rng.permutation(n_pages).tolist()
    max_blocks = max((len(x) + page_size - 1) // page_size for x in k) + 1
    tables = torch.full((len(k), max_blocks), -1, dtype=torch.int32)
    for b, (kk, vv) in enumerate(zip(k, v)):
        for i in range(0, len(kk), page_size):
            page = perm.pop()
            tables[b, i // page_size] = page
            n = min(page_size, len(kk) - i)
            kc[page, :, :n] = kk[i:i + n].transpose(0, 1)
            vc[page, :, :n] = vv[i:i + n].transpose(0, 1)
    return kc, vc, tables


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("geom", [(6, 3, 48, 8), (5, 1, 80, 16), (8, 8, 16, 4), (4, 2, 112, 32)])
def test_rope_and_cache_write(dtype, geom):
    from rust_llm_inference_server_b200 import ops
    nh, nkv, d, ps = geom
    torch.manual_seed(nh)
    T = 9
    cfg = {"head_dim": d, "rope_theta": 25000.0, "hidden_size": nh * d, "num_attention_heads": nh,
           "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                            "high_freq_factor": 4.0, "original_max_position_embeddings": 32}}
    inv = P.inv_freqs(cfg)
    qkv = torch.randn(T, (nh + 2 * nkv) * d).to(dtype)
    positions = torch.tensor([0, 1, 2, 3, 100, 4095, 70000, 7, 8], dtype=torch.int32)
    n_pages = 12
    slots = torch.tensor([5 * ps + 1, 5 * ps + 2, 0, 11 * ps + ps - 1, 3 * ps, 3 * ps + 1, 7 * ps, 8 * ps + 2, 9 * ps],
                         dtype=torch.int32)
    kc = torch.zeros(n_pages, nkv, ps, d, dtype=dtype, device="cuda")
    vc = torch.zeros_like(kc)
    q_out = torch.empty(T, nh * d, dtype=dtype, device="cuda")
    ops.rope_cache(dev(qkv), q_out, kc, vc, dev(positions), dev(slots), dev(inv), nh, nkv, d, ps)
    x = qkv.float()
    q = x[:, :nh * d].view(T, nh, d)
    k = x[:, nh * d:(nh + nkv) * d].view(T, nkv, d)
    v = x[:, (nh + nkv) * d:].view(T, nkv, d)
    cos, sin = P.rope_tables(inv, positions)
    t = tol(dtype, 2e-5, 3e-2)   # position 70000: float32 angle, sin/cos of a large argument
    assert (q_out.float().cpu().view(T, nh, d) - P.apply_rope(q, cos, sin)).abs().max() <= t
    kr = P.apply_rope(k, cos, sin)
    for i in range(T):
        page, off = int(slots[i]) // ps, int(slots[i]) % ps
        assert (kc[page, :, off].float().cpu() - kr[i]).abs().max() <= t
        assert torch.equal(vc[page, :, off].float().cpu(), v[i])
    assert int((kc.float().abs().sum(dim=(1, 3)) > 0).sum()) == T      # nothing else was written
    # no rotation, nothing stored
    q2 = torch.empty_like(q_out)
    ops.rope_cache(dev(qkv), q2, None, None, dev(positions), None, None, nh, nkv, d, ps)
    assert torch.equal(q2.cpu(), qkv[:, :nh * d])


def attention_case(geom, lens, q_lens, page_size, dtype, window=None, seed=0, spike=None):
    """Requests with `lens` cached tokens each, the last q_lens[b] of them being this step's queries.
    Returns inputs for the kernels and the plain result [T, nh, d]."""
    nh, nkv, d = geom
    g = torch.Generator().manual_seed(seed)
    ks = [torch.randn(n, nkv, d, generator=g).to(dtype).float() for n in lens]
    vs = [torch.randn(n, nkv, d, generator=g).to(dtype).float() for n in lens]
    qs = [torch.randn(m, nh, d, generator=g).to(dtype).float() for m in q_lens]
    if spike is not None:
        # one far key carries the whole softmax: it is a scaled copy of the query, and its value
        # row is the only one that is not small
        b, qi, key = spike
        rep = nh // nkv
        for h in range(nkv):
            for r in range(1, rep):              # the heads of a group ask the same question
                qs[b][qi, h * rep + r] = qs[b][qi, h * rep]
            ks[b][key, h] = (qs[b][qi, h * rep] * 8.0).to(dtype).float()
        vs[b][key] = 7.0
    n_pages = sum((n + page_size - 1) // page_size for n in lens) + 3
    kc, vc, tables = cache_from(ks, vs, page_size, n_pages, seed)
    want = torch.cat([P.causal_attention(q, k, v, start_pos=len(k) - len(q), window=window)
                      for q, k, v in zip(qs, ks, vs)])
    q = torch.cat(qs).reshape(-1, nh * d)
    seq_of_token = torch.cat([torch.full((m,), b, dtype=torch.int32) for b, m in enumerate(q_lens)])
    positions = torch.cat([torch.arange(n - m, n, dtype=torch.int32) for n, m in zip(lens, q_lens)])
    return q.to(dtype), kc.to(dtype), vc.to(dtype), tables, seq_of_token, positions, want


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("geom,ps", [((6, 3, 48), 8), ((5, 1, 80), 16), ((8, 8, 16), 4), ((4, 2, 112), 32),
                                     ((32, 8, 64), 16), ((7, 7, 256), 16)])
def test_attention_for_any_query_lengths(dtype, geom, ps):
    from rust_llm_inference_server_b200 import ops
    nh, nkv, d = geom
    lens, q_lens = [1, 37, 130, 64, 33], [1, 1, 17, 64, 2]
    q, kc, vc, tables, sot, pos, want = attention_case(geom, lens, q_lens, ps, dtype, seed=nh)
    out = torch.empty(q.shape, dtype=dtype, device="cuda")
    ops.attention_generic(dev(q), dev(kc), dev(vc), out, dev(sot), dev(pos), dev(tables), nh, nkv, d, ps,
                          1 / math.sqrt(d))
    err = (out.float().cpu().view(-1, nh, d) - want).abs().max()
    assert err <= tol(dtype, 2e-5, 2e-2), err
    # a subset of the rows leaves the others untouched
    out2 = torch.zeros_like(out)
    rows = torch.tensor([0, 5, 80], dtype=torch.int32)
    ops.attention_generic(dev(q), dev(kc), dev(vc), out2, dev(sot), dev(pos), dev(tables), nh, nkv, d, ps,
                          1 / math.sqrt(d), token_rows=dev(rows))
    assert torch.equal(out2[rows.long()], out[rows.long()])
    others = torch.ones(out2.shape[0], dtype=torch.bool)
    others[rows.long()] = False
    assert float(out2[others.cuda()].float().abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DT)
def test_attention_finds_a_far_key_and_respects_page_edges(dtype):
    """The softmax sits on one key among hundreds: at a page's first and last slot, in the first
    page, and just behind the query.  A wrong page or offset would return a wrong value row."""
    from rust_llm_inference_server_b200 import ops
    geom, ps = (4, 2, 32), 16
    for key in (0, 15, 16, 31, 3, 303, 304, 598, 599):
        q, kc, vc, tables, sot, pos, want = attention_case(geom, [600, 40], [1, 1], ps, dtype, seed=key,
                                                           spike=(0, 0, key))
        out = torch.empty(q.shape, dtype=dtype, device="cuda")
        ops.attention_generic(dev(q), dev(kc), dev(vc), out, dev(sot), dev(pos), dev(tables), 4, 2, 32, ps,
                              1 / math.sqrt(32))
        got = out.float().cpu().view(-1, 4, 32)
        assert (got[0] - 7.0).abs().max() < 0.05, key         # the spiked value row, for every head
        assert (got - want).abs().max() <= tol(dtype, 1e-4, 3e-2)


@pytest.mark.parametrize("dtype", DT)
def test_attention_window_edge(dtype):
    """With a window of W keys the key at position - W + 1 is seen and the one before it is not."""
    from rust_llm_inference_server_b200 import ops
    geom, ps, W = (2, 1, 16), 8, 40
    n = 100
    for key, seen in ((n - W, True), (n - W - 1, False)):
        q, kc, vc, tables, sot, pos, want = attention_case(geom, [n], [1], ps, dtype, window=W, seed=3,
                                                           spike=(0, 0, key))
        out = torch.empty(q.shape, dtype=dtype, device="cuda")
        ops.attention_generic(dev(q), dev(kc), dev(vc), out, dev(sot), dev(pos), dev(tables), 2, 1, 16, ps,
                              0.25, window=W)
        got = out.float().cpu().view(-1, 2, 16)
        assert (got - want).abs().max() <= tol(dtype, 1e-4, 3e-2)
        assert ((got - 7.0).abs().max() < 0.05) == seen


@pytest.mark.parametrize("geom,ps", [((32, 8, 64), 16), ((24, 8, 128), 16), ((6, 3, 48), 8), ((5, 1, 80), 16),
                                     ((8, 8, 16), 4), ((12, 2, 128), 32), ((16, 2, 64), 16), ((7, 7, 256), 64)])
@pytest.mark.parametrize("splits", [1, 2, 5, 16])
def test_decode_attention_split_over_the_context(geom, ps, splits):
    """Context lengths of the reference's kernel test (1 + (i * 53) % 700, and a few long ones;
    crates/model/src/paged_attention.rs:423-527), every number of splits, rows in another order
    than the batch."""
    from rust_llm_inference_server_b200 import ops
    nh, nkv, d = geom
    lens = [1 + (i * 53) % 700 for i in range(9)] + [1, 32, 33, 2049]
    B = len(lens)
    q, kc, vc, tables, sot, pos, want = attention_case(geom, lens, [1] * B, ps, torch.bfloat16, seed=d + splits)
    order = torch.randperm(B, generator=torch.Generator().manual_seed(1)).to(torch.int32)   # row i holds request order[i]
    q_rows = q[order.long()].contiguous()
    out = torch.zeros(B, nh * d, dtype=torch.bfloat16, device="cuda")
    scratch = torch.empty(B * nh * splits * (d + 2), dtype=torch.float32, device="cuda")
    ctx = torch.tensor(lens, dtype=torch.int32)
    inv = torch.empty(B, dtype=torch.int32)
    inv[order.long()] = torch.arange(B, dtype=torch.int32)
    # request b's token sits in row inv[b]
    ops.attention_decode(dev(q_rows), dev(kc), dev(vc), out, dev(inv[torch.arange(B)].contiguous()),
                         dev(torch.arange(B, dtype=torch.int32)), dev(ctx), dev(tables), nh, nkv, d, ps,
                         1 / math.sqrt(d), 0, splits, scratch)
    got = out.float().cpu()[inv.long()].view(B, nh, d)
    err = (got - want).abs().max()
    assert err <= 2e-2, err


@pytest.mark.parametrize("geom,ps", [((32, 8, 64), 16), ((6, 3, 128), 16), ((4, 4, 64), 8), ((5, 1, 128), 32),
                                     ((8, 2, 64), 8), ((4, 1, 64), 32), ((12, 6, 64), 128), ((6, 1, 64), 64),
                                     ((8, 2, 128), 16), ((24, 8, 128), 8), ((4, 2, 128), 64), ((2, 1, 128), 32),
                                     ((4, 2, 128), 128), ((9, 3, 64), 16), ((5, 1, 64), 8), ((24, 8, 128), 16)])
@pytest.mark.parametrize("window", [None, 70])
def test_prefill_flash_attention_over_pages(geom, ps, window):
    """Portions of prompts of many lengths (one token short of a tile, exactly a tile, across
    tiles), starting at position 0 and deep in a context, against plain attention."""
    from rust_llm_inference_server_b200 import ops
    nh, nkv, d = geom
    lens = [300, 64, 65, 130, 700, 2, 191]
    q_lens = [300, 64, 2, 127, 129, 2, 63]
    q, kc, vc, tables, sot, pos, want = attention_case(geom, lens, q_lens, ps, torch.bfloat16, window=window, seed=d + ps)
    tiles = torch.tensor([(b, t0) for b, n in enumerate(q_lens) for t0 in range(0, n, 64)], dtype=torch.int32)
    cu = torch.tensor(np.cumsum([0] + q_lens), dtype=torch.int32)
    from rust_llm_inference_server_b200.ops.library import lib
    try:
        # the tcgen05 kernel lets 1, 2 or 4 CTAs of a cluster share a tile's blocks of keys (some then
        # have no block at all); 0: its own choice from the number of tiles and the longest context
        for splits in (1, 2, 4, 0):
            ops.debug_set("prefill_splits", splits)
            out = torch.zeros(q.shape, dtype=torch.bfloat16, device="cuda")
            ops.attention_prefill(dev(q), dev(kc), dev(vc), out, dev(tiles), dev(cu),
                                  dev(torch.tensor(lens, dtype=torch.int32)), dev(tables), nh, nkv, d, ps,
                                  1 / math.sqrt(d), window or 0, max(lens))
            err = (out.float().cpu().view(-1, nh, d) - want).abs().max()
            assert err <= 2.5e-2, (splits, err)
    finally:
        ops.debug_set("prefill_splits", 0)
    ops.check_device_errors()


@pytest.mark.parametrize("geom", [(8, 2, 64), (4, 1, 128)])
def test_prefill_flash_attention_finds_far_keys_and_the_causal_edge(geom):
    from rust_llm_inference_server_b200 import ops
    ps = 16
    nh, nkv, d = geom
    n, m = 1000, 200           # the last 200 tokens are queries
    cu = torch.tensor([0, m], dtype=torch.int32)
    tiles = torch.tensor([(0, t0) for t0 in range(0, m, 64)], dtype=torch.int32)
    for qi, key, seen in ((0, 3, True), (0, 800, True), (0, 801, False), (150, 950, True), (150, 951, False),
                          (199, 999, True), (64, 864, True), (63, 864, False), (100, 15, True), (100, 16, True)):
        q, kc, vc, tables, sot, pos, want = attention_case(geom, [n], [m], ps, torch.bfloat16, seed=key, spike=(0, qi, key))
        # few tiles and a long context: the kernel shares each tile's keys among the CTAs of a cluster
        out = torch.zeros(q.shape, dtype=torch.bfloat16, device="cuda")
        ops.attention_prefill(dev(q), dev(kc), dev(vc), out, dev(tiles), dev(cu), dev(torch.tensor([n], dtype=torch.int32)),
                              dev(tables), nh, nkv, d, ps, 1 / math.sqrt(d), 0, n)
        got = out.float().cpu().view(m, nh, d)
        assert (got - want).abs().max() <= 3e-2
        assert ((got[qi] - 7.0).abs().max() < 0.05) == seen, (qi, key)


@pytest.mark.parametrize("geom,tcgen05", [((8, 2, 64), True), ((8, 2, 64), False), ((6, 3, 128), False), ((4, 4, 64), False),
                                          ((4, 2, 128), True), ((4, 2, 128), False)])
@pytest.mark.parametrize("W", [70, 129])
def test_prefill_flash_attention_window_edge(geom, tcgen05, W):
    """With a window of W keys, the query at position p sees the key at p - W + 1 and not the one at
    p - W.  The softmax of one query row sits on exactly that key: rows at the start and at the end
    of a tile (the first visible key differs from row to row inside a tile), a portion deep in its
    context, pages behind every row's window gone from the block table, the tcgen05 and the
    mma.sync kernel, and 1, 2 and 4 CTAs sharing a tile's keys."""
    from rust_llm_inference_server_b200 import ops
    nh, nkv, d = geom
    ps, n, m = 16, 1000, 200
    cu = torch.tensor([0, m], dtype=torch.int32)
    tiles = torch.tensor([(0, t0) for t0 in range(0, m, 64)], dtype=torch.int32)
    first = n - m
    ops.debug_set("prefill_tcgen05", 1 if tcgen05 else 0)
    try:
        for qi in (0, 1, 63, 64, 127, 128, 199):
            p = first + qi
            for key, seen in ((p - W + 1, True), (p - W, False), (p, True)):
                q, kc, vc, tables, sot, pos, want = attention_case(geom, [n], [m], ps, torch.bfloat16, window=W,
                                                                   seed=qi + key, spike=(0, qi, key))
                tables = tables.clone()
                tables[0, :(first - W + 1) // ps] = -1          # no row of the portion looks that far back
                for splits in ((0, 1, 2, 4) if tcgen05 else (0,)):
                    ops.debug_set("prefill_splits", splits)
                    out = torch.zeros(q.shape, dtype=torch.bfloat16, device="cuda")
                    ops.attention_prefill(dev(q), dev(kc), dev(vc), out, dev(tiles), dev(cu),
                                          dev(torch.tensor([n], dtype=torch.int32)), dev(tables), nh, nkv, d, ps,
                                          1 / math.sqrt(d), W, n)
                    got = out.float().cpu().view(m, nh, d)
                    assert (got - want).abs().max() <= 3e-2, (qi, key, splits)
                    assert ((got[qi] - 7.0).abs().max() < 0.05) == seen, (qi, key, splits)
    finally:
        ops.debug_set("prefill_splits", 0)
        ops.debug_set("prefill_tcgen05", 1)
    ops.check_device_errors()


def test_decode_attention_far_key_and_window():
    from rust_llm_inference_server_b200 import ops
    geom, ps = (8, 2, 64), 16
    n = 3000
    for key, window, seen in ((5, 0, True), (1023, 0, True), (1024, 0, True), (2999, 0, True),
                              (n - 500, 500, True), (n - 501, 500, False)):
        q, kc, vc, tables, sot, pos, want = attention_case(geom, [n, 7], [1, 1], ps, torch.bfloat16, seed=key,
                                                           window=window or None, spike=(0, 0, key))
        for splits in (1, 7):
            out = torch.zeros(2, 8 * 64, dtype=torch.bfloat16, device="cuda")
            scratch = torch.empty(2 * 8 * splits * 66, dtype=torch.float32, device="cuda")
            ar = dev(torch.arange(2, dtype=torch.int32))
            ops.attention_decode(dev(q), dev(kc), dev(vc), out, ar, ar, dev(torch.tensor([n, 7], dtype=torch.int32)),
                                 dev(tables), 8, 2, 64, ps, 0.125, window, splits, scratch)
            got = out.float().cpu().view(2, 8, 64)
            assert (got - want).abs().max() <= 3e-2
            assert ((got[0] - 7.0).abs().max() < 0.05) == seen, (key, window, splits)


@pytest.mark.parametrize("geom,ps", [((32, 8, 64), 16), ((6, 3, 128), 16), ((8, 8, 64), 8), ((4, 1, 128), 32)])
@pytest.mark.parametrize("rotate,store,window", [(True, True, 0), (False, True, 0), (True, False, 0), (True, True, 70)])
def test_decode_attention_from_the_projection_equals_rotation_then_attention(geom, ps, rotate, store, window):
    """A step of single tokens: the kernel that rotates q and the newest key itself and stores that
    key gives the bits of the two-kernel path, in the output and in the cache.  Contexts that end
    at a page's and at a block's first and last slot, one token long, and long."""
    from types import SimpleNamespace
    from rust_llm_inference_server_b200 import ops
    nh, nkv, d = geom
    lens = [1, 2, 31, 32, 33, 64, 65, 700, 2049, ps, ps + 1, 3 * ps - 1]
    B = len(lens)
    g = torch.Generator().manual_seed(d + ps + window)
    n_pages = sum(-(-n // ps) for n in lens) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    max_blocks = max(-(-n // ps) for n in lens)
    tables = torch.zeros(B, max_blocks, dtype=torch.int32)
    slots = torch.zeros(B, dtype=torch.int32)
    for b, n in enumerate(lens):
        for i in range(-(-n // ps)):
            tables[b, i] = perm.pop()
        slots[b] = tables[b, (n - 1) // ps] * ps + (n - 1) % ps
    kc = (torch.randn(n_pages, nkv, ps, d, generator=g) * 0.7).bfloat16()
    vc = (torch.randn(n_pages, nkv, ps, d, generator=g) * 0.7).bfloat16()
    qkv = (torch.randn(B, (nh + 2 * nkv) * d, generator=g) * 0.7).bfloat16()
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32)
    inv_freq = dev((1.0 / 10000.0 ** (torch.arange(0, d, 2).float() / d)).contiguous()) if rotate else None
    ctx = dev(torch.tensor(lens, dtype=torch.int32))
    ar = dev(torch.arange(B, dtype=torch.int32))
    scale = 1 / math.sqrt(d)
    bufs = {}

    def buffer(name, shape, dtype):
        return bufs.setdefault((name, shape), torch.empty(shape, dtype=dtype, device="cuda"))

    for max_ctx in (max(lens), 4 * 128):          # many splits and few
        step = SimpleNamespace(n_decode=B, slots={0: dev(slots)}, block_tables={0: dev(tables)}, max_decode_ctx=max_ctx,
                               positions=dev(pos), dec_rows=ar, dec_seqs=ar, ctx_lens=ctx, buffer=buffer)
        # two kernels
        k1, v1 = dev(kc).clone(), dev(vc).clone()
        q1 = torch.empty(B, nh * d, dtype=torch.bfloat16, device="cuda")
        ops.rope_cache(dev(qkv), q1, k1 if store else None, v1 if store else None, step.positions,
                       step.slots[0] if store else None, inv_freq, nh, nkv, d, ps)
        out1 = torch.zeros(B, nh * d, dtype=torch.bfloat16, device="cuda")
        splits = ops.decode_splits(B, nkv, max_ctx)
        scratch = torch.empty(B * nh * splits * (d + 2), dtype=torch.float32, device="cuda")
        ops.attention_decode(q1, k1, v1, out1, ar, ar, ctx, step.block_tables[0], nh, nkv, d, ps, scale, window,
                             splits, scratch)
        # one kernel
        k2, v2 = dev(kc).clone(), dev(vc).clone()
        out2 = torch.zeros(B, nh * d, dtype=torch.bfloat16, device="cuda")
        ops.attention_decode_from_qkv(dev(qkv), k2, v2, out2, step, 0, inv_freq, store, nh, nkv, d, ps, scale, window)
        assert torch.equal(out1, out2)
        assert torch.equal(k1, k2) and torch.equal(v1, v2)
        if store:
            assert not torch.equal(k2, dev(kc))                  # the newest keys did arrive


@pytest.mark.parametrize("V", [1003, 4100, 50257, 128256, 200003])
def test_filtered_sampling_cluster_and_one_cta_kernels_agree(V):
    """The kernel that holds a row in the registers of a cluster picks the tokens of the kernel
    that reads the row pass after pass (which the test before compares with the plain rule), at
    vocabularies of every size class, with ties and with rows that a stride separates."""
    from rust_llm_inference_server_b200 import ops
    from rust_llm_inference_server_b200.ops.library import lib
    rng = np.random.default_rng(V)
    R = 12
    logits = (rng.normal(size=(R, V + 3)) * 2.5).astype(np.float32)
    logits[2, [7, V // 2, V - 1]] = logits[2, :V].max()
    logits[3, :V] = 0.25
    logits[4, 100:160] = np.sort(logits[4, :V])[-30]
    settings = [(0.8, 0, 0.9), (1.0, 40, 1.0), (0.5, 10, 0.5), (1.4, 0, 0.3), (0.9, 1, 1.0), (1.0, V + 5, 0.95)]
    params = np.zeros((R, 5), dtype=np.uint32)
    for r in range(R):
        T, k, p = settings[r % len(settings)]
        u = int(rng.integers(0, 1 << 53, dtype=np.uint64))
        params[r] = (np.float32(np.float32(1.0) / np.float32(T)).view(np.uint32), k, np.float32(p).view(np.uint32),
                     u & 0xFFFFFFFF, u >> 32)
    lt = torch.from_numpy(logits).cuda()[:, :V]                       # rows with a stride, not 16-byte aligned
    pt = torch.from_numpy(params.view(np.int32)).cuda()
    got = ops.sample_filtered(lt, pt).cpu().tolist()
    ops.debug_set("filtered_cluster", 0)
    try:
        want = ops.sample_filtered(lt, pt).cpu().tolist()
    finally:
        ops.debug_set("filtered_cluster", 1)
    assert got == want
    assert got[3] < V and all(0 <= t < V for t in got)


@pytest.mark.parametrize("V", [1003, 128256])
def test_repetition_penalty_on_the_device_equals_the_plain_rule(V):
    """Rows with a stride, histories with repeated tokens (penalised once), positive and negative
    logits, an exact zero, an empty history, and a row that is not in the list and must stay."""
    from rust_llm_inference_server_b200 import ops
    rng = np.random.default_rng(V)
    R = 5
    logits = rng.normal(size=(R, V)).astype(np.float32) * 4
    logits[1, 7] = 0.0
    hist = {0: rng.integers(0, V, size=900).tolist() + [3] * 40, 1: [7, 7, 7, V - 1, 0, V - 1], 3: [],
            4: rng.integers(0, 50, size=3000).tolist()}          # row 4: every token many times
    pens = {0: 1.3, 1: 2.0, 3: 1.7, 4: 0.8}
    order = [4, 0, 3, 1]                                          # the list names rows in any order
    flat, offs = [], [0]
    for r in order:
        flat += hist[r]
        offs.append(len(flat))
    big = np.concatenate([logits, np.full((R, 3), 9.0, np.float32)], axis=1)
    lt = torch.from_numpy(big).cuda()[:, :V]
    ops.repetition_penalty(lt, torch.tensor(order, dtype=torch.int32).cuda(),
                           torch.tensor(flat + [0], dtype=torch.int32).cuda()[:len(flat)],
                           torch.tensor(offs, dtype=torch.int32).cuda(),
                           torch.tensor([pens[r] for r in order], dtype=torch.float32).cuda())
    got = lt.cpu().numpy()
    for r in range(R):
        want = P.apply_repetition_penalty(logits[r], hist[r], pens[r]) if r in hist else logits[r]
        assert np.array_equal(got[r], want), r
    assert not np.array_equal(got[0], logits[0]) and np.array_equal(got[2], logits[2])


def test_sample_rows_equals_the_plain_sampler():
    from rust_llm_inference_server_b200 import ops
    rng = np.random.default_rng(0)
    R, V = 7, 1003
    logits = rng.normal(size=(R, V)).astype(np.float32) * 3
    logits[0, 5] = logits[0, 900] = logits[0].max() + 1     # a tie: the lowest id wins
    params = np.zeros((R, 2), dtype=np.uint32)
    temps = [0.0, 0.0, 0.7, 1.0, 1.5, 0.7, 0.3]
    keys = [0, 0, P.row_key(1, 10), P.row_key(1, 11), P.row_key(99, 5), P.row_key(2, 10), P.row_key(3, 3)]
    for r in range(R):
        if temps[r] > 0:
            params[r] = (keys[r], np.float32(np.float32(1.0) / np.float32(temps[r])).view(np.uint32))
    big = np.concatenate([logits, np.zeros((R, 5), np.float32)], axis=1)     # rows with a stride
    lt = torch.from_numpy(big).cuda()[:, :V]
    got = ops.sample_rows(lt, torch.from_numpy(params.view(np.int32)).cuda()).cpu().tolist()
    want = [P.sample_row(logits[r], temps[r], keys[r]) for r in range(R)]
    assert got == want and got[0] == 5
    # a row's choice does not depend on its neighbours
    alone = ops.sample_rows(lt[4:5], torch.from_numpy(params.view(np.int32)[4:5].copy()).cuda()).cpu().tolist()
    assert alone == [want[4]]
    # frequencies follow softmax(logits / T)
    small = torch.tensor([[0.0, 1.0, 2.0, -1.0]]).cuda().repeat(4000, 1)
    ps_ = np.zeros((4000, 2), dtype=np.uint32)
    for i in range(4000):
        ps_[i] = (P.row_key(7, i), np.float32(1 / 0.7).view(np.uint32))
    ids = ops.sample_rows(small, torch.from_numpy(ps_.view(np.int32)).cuda()).cpu().numpy()
    freq = np.bincount(ids, minlength=4) / 4000
    want_p = np.exp(np.array([0, 1, 2, -1]) / 0.7)
    assert np.abs(freq - want_p / want_p.sum()).max() < 0.03


def test_kernels_refuse_what_they_do_not_take():
    from rust_llm_inference_server_b200 import ops
    from rust_llm_inference_server_b200.ops import KernelError
    x = torch.randn(4, 8)
    with pytest.raises(KernelError, match="CUDA"):
        ops.gemm_f32(x, x)                                    # no CPU path
    with pytest.raises(KernelError, match="contiguous"):
        ops.gemm_f32(dev(torch.randn(8, 4)).t(), dev(x))
    with pytest.raises(KernelError, match="multiples of 16"):
        z = torch.zeros(1, 40, device="cuda")
        i = torch.zeros(1, dtype=torch.int32, device="cuda")
        ops.attention_generic(z, torch.zeros(1, 1, 4, 40, device="cuda"), torch.zeros(1, 1, 4, 40, device="cuda"),
                              z.clone(), i, i, torch.zeros(1, 1, dtype=torch.int32, device="cuda"), 1, 1, 40, 4, 1.0)
    with pytest.raises(KernelError, match="not supported"):
        ops.swiglu(dev(torch.randn(2, 8).half()), dev(torch.randn(2, 4).half()))


def test_filtered_sampling_on_the_device_equals_the_plain_rule():
    """Top-k / top-p rows: the kernel picks the token the plain rule picks, row by row, whatever
    its neighbours; frequencies follow the filtered softmax."""
    from rust_llm_inference_server_b200 import ops
    rng = np.random.default_rng(5)
    R, V = 24, 1003
    logits = (rng.normal(size=(R, V)) * 2.5).astype(np.float32)
    logits[3, [7, 500, 900]] = logits[3].max()                # exact ties at the top
    logits[[4, 8, 9]] = 0.25                                  # all equal: the lowest ids are the kept ones
    logits[13, 100:160] = np.sort(logits[13])[-30]            # sixty ties across the 40th place
    logits[14, 300:420] = np.sort(logits[14])[-4]             # ties across the top-10 and the nucleus edge
    settings = [(0.8, 0, 0.9), (1.0, 40, 1.0), (0.5, 10, 0.5), (1.4, 0, 0.3), (0.9, 1, 1.0), (1.0, 2000, 0.95)]
    params = np.zeros((R, 5), dtype=np.uint32)
    want = []
    for r in range(R):
        T, k, p = settings[r % len(settings)]
        u = (rng.integers(0, 1 << 53, dtype=np.uint64))
        params[r] = (np.float32(np.float32(1.0) / np.float32(T)).view(np.uint32), k, np.float32(p).view(np.uint32),
                     int(u) & 0xFFFFFFFF, int(u) >> 32)
        want.append(P.filtered_sample(logits[r], T, k, p, int(u)))
    lt = torch.from_numpy(logits).cuda()
    got = ops.sample_filtered(lt, torch.from_numpy(params.view(np.int32)).cuda()).cpu().tolist()
    assert got == want
    alone = ops.sample_filtered(lt[5:6], torch.from_numpy(params.view(np.int32)[5:6].copy()).cuda()).cpu().tolist()
    assert alone == [want[5]]
    small = torch.tensor([[0.0, 1.0, 2.0, -1.0, 0.5, 1.5]]).cuda().repeat(6000, 1)
    ps_ = np.zeros((6000, 5), dtype=np.uint32)
    us = rng.integers(0, 1 << 53, size=6000, dtype=np.uint64)
    for i in range(6000):
        ps_[i] = (np.float32(1 / 0.7).view(np.uint32), 4, np.float32(0.8).view(np.uint32), int(us[i]) & 0xFFFFFFFF, int(us[i]) >> 32)
    ids = ops.sample_filtered(small, torch.from_numpy(ps_.view(np.int32)).cuda()).cpu().numpy()
    freq = np.bincount(ids, minlength=6) / 6000
    assert np.abs(freq - P.filtered_distribution(np.array([0.0, 1.0, 2.0, -1.0, 0.5, 1.5], np.float32), 0.7, 4, 0.8)).max() < 0.03


def test_decode_attention_over_long_contexts():
    """Contexts of tens of thousands of keys: pieces whose slice of the block table no longer fits
    the kernel's shared-memory copy (it then reads the table from global memory), few and many
    pieces, against the float32 kernel for any query length."""
    from rust_llm_inference_server_b200 import ops
    torch.manual_seed(0)
    nh, nkv, d, ps = 8, 2, 64, 16
    B, ctx = 2, 20000
    n_pages = B * (ctx // ps + 1)
    kc = (torch.randn(n_pages, nkv, ps, d, device="cuda") * 0.5).bfloat16()
    vc = (torch.randn(n_pages, nkv, ps, d, device="cuda") * 0.5).bfloat16()
    vc[:, :, :, 0] = 1.0                                   # a column whose attention output must be 1
    q = torch.randn(B, nh * d, device="cuda").bfloat16()
    tables = torch.randperm(n_pages, device="cuda").to(torch.int32).view(B, -1)
    ar = torch.arange(B, dtype=torch.int32, device="cuda")
    ctxs = torch.tensor([ctx, ctx - 4097], dtype=torch.int32, device="cuda")
    ref = torch.zeros(B, nh * d, dtype=torch.float32, device="cuda")
    ops.attention_generic(q.float(), kc.float(), vc.float(), ref, ar, (ctxs - 1).contiguous(), tables, nh, nkv, d, ps, 0.125)
    for splits in (ops.decode_splits(B, nkv, ctx), 2, 32):
        out = torch.zeros_like(q)
        scratch = torch.empty(B * nh * splits * (d + 2), dtype=torch.float32, device="cuda")
        ops.attention_decode(q, kc, vc, out, ar, ar, ctxs, tables, nh, nkv, d, ps, 0.125, 0, splits, scratch)
        assert (out.float() - ref).abs().max() <= 4e-3, splits
        assert (out.float().view(B, nh, d)[:, :, 0] - 1.0).abs().max() <= 2 ** -7
    ops.check_device_errors()
