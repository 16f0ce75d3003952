"""Each part alone, built from its spec and a dictionary of tensors, against the plain function of
the same part: embedding, norm, position encoding, attention mixer (with and without a window,
with and without rotation), feed-forward, the pre-norm block, and the LM head."""

import math

import numpy as np
import pytest
import torch

from tests.plain import llama_plain as P

pytestmark = pytest.mark.gpu


class DictSource:
    def __init__(self, tensors, dtype):
        self.t, self.dtype, self.shared = tensors, dtype, {}

    def get(self, name, role="matrix", share=False):
        if share and (name, role) in self.shared:
            return self.shared[(name, role)]
        x = self.t[name].cuda()
        x = x.to(self.dtype) if role == "matrix" else x.float()
        if share:
            self.shared[(name, role)] = x
        return x


class FakeStep:
    """The fields of a step that parts read, made by hand: requests with `starts[b]` tokens in
    the cache and `lens[b]` new ones; pages handed out in a scrambled order."""

    def __init__(self, starts, lens, page_size, tables):
        self.n_seqs, self.n_tokens = len(lens), sum(lens)
        self.starts, self.q_lens = starts, lens
        self.q_starts = np.cumsum([0] + lens[:-1]).tolist()
        pos = np.concatenate([np.arange(s, s + n) for s, n in zip(starts, lens)])
        sot = np.concatenate([np.full(n, b) for b, n in enumerate(lens)])
        slots = np.array([tables[b][p // page_size] * page_size + p % page_size for b, p in zip(sot, pos)])
        i32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device="cuda")
        self.positions, self.seq_of_token, self.slots = i32(pos), i32(sot), [i32(slots)]
        width = max(len(t) for t in tables)
        self.block_tables = [i32([list(t) + [-1] * (width - len(t)) for t in tables])]
        self.ctx_lens = i32([s + n for s, n in zip(starts, lens)])
        dec = [b for b, n in enumerate(lens) if n == 1]
        self.n_decode = len(dec)
        self.dec_seqs = i32(dec) if dec else None
        self.dec_rows = i32([self.q_starts[b] for b in dec]) if dec else None
        self.max_decode_ctx = max([starts[b] + 1 for b in dec], default=0)
        self.all_decode = max(lens) == 1
        rows = [r for b, n in enumerate(lens) if n > 1 for r in range(self.q_starts[b], self.q_starts[b] + n)]
        self.n_prefill_tokens = len(rows)
        self.prefill_rows = i32(rows) if (dec and rows) else None
        tiles = [(b, t0) for b, n in enumerate(lens) if n > 1 for t0 in range(0, n, 64)]
        self.n_prefill_tiles = len(tiles)
        self.prefill_tiles = i32(tiles) if tiles else None
        self.cu_seqlens = i32(self.q_starts + [self.n_tokens])
        self._bufs = {}

    def buffer(self, name, shape, dtype):
        return torch.empty(tuple(shape), dtype=dtype, device="cuda")


def tol(dtype):
    return 2e-5 if dtype == torch.float32 else 3e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_and_feed_forward_parts(dtype):
    from rust_llm_inference_server_b200.parts import RMSNormSpec, SwiGLUSpec, build_feed_forward, build_norm
    torch.manual_seed(0)
    H, I, T = 80, 176, 6
    w = {"n": torch.randn(H) * 0.1 + 1, "g": torch.randn(I, H) * 0.1, "u": torch.randn(I, H) * 0.1,
         "d": torch.randn(H, I) * 0.1}
    if dtype == torch.bfloat16:
        w = {k: v.bfloat16().float() for k, v in w.items()}
    src = DictSource(w, dtype)
    step = FakeStep([0], [T], 8, [[0]])
    norm = build_norm(RMSNormSpec(H, 3e-6, "n"), dtype, "cuda")
    assert norm.tensors() == {"n": (H,)}
    norm.load(src)
    resid, delta = torch.randn(T, H), torch.randn(T, H).to(dtype)
    r = resid.cuda()
    out = norm.forward(r, delta.cuda(), step)
    want = P.rms_norm(resid + delta.float(), w["n"], 3e-6)
    assert (out.float().cpu() - want).abs().max() <= tol(dtype) and out.dtype == dtype
    ffn = build_feed_forward(SwiGLUSpec(H, I, "g", "u", "d"), dtype, "cuda")
    assert ffn.tensors() == {"g": (I, H), "u": (I, H), "d": (H, I)}
    ffn.load(src)
    x = torch.randn(T, H).to(dtype)
    got = ffn.forward(x.cuda(), step)
    want = P.swiglu_mlp(x.float(), {"p.gate_proj.weight": w["g"], "p.up_proj.weight": w["u"],
                                    "p.down_proj.weight": w["d"]}, "p.")
    assert (got.float().cpu() - want).abs().max() <= tol(dtype) * 3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,rotate", [(None, True), (5, True), (None, False)])
def test_attention_part_over_two_steps(dtype, window, rotate):
    """A portion of a prompt in one step, the rest beside a decoded token of another request in
    the next: the part's output equals plain attention over the whole sequences."""
    from rust_llm_inference_server_b200.parts import (GQAAttentionSpec, KVCacheSpec, LayerCache, NoPositionSpec,
                                                      RopeSpec, build_mixer)
    torch.manual_seed(1)
    H, nh, nkv, d, ps = 80, 6, 2, 16, 4
    cfg = {"head_dim": d, "rope_theta": 777.0, "hidden_size": H, "num_attention_heads": nh,
           "num_key_value_heads": nkv}
    w = {"q": torch.randn(nh * d, H) * 0.2, "k": torch.randn(nkv * d, H) * 0.2, "v": torch.randn(nkv * d, H) * 0.2,
         "o": torch.randn(H, nh * d) * 0.2}
    if dtype == torch.bfloat16:
        w = {k: v.bfloat16().float() for k, v in w.items()}
    spec = GQAAttentionSpec(H, nh, nkv, d, "q", "k", "v", "o",
                            position=RopeSpec(d, 777.0, None) if rotate else NoPositionSpec(), window=window)
    att = build_mixer(spec, dtype, "cuda")
    assert att.cache_spec() == KVCacheSpec(nkv, d, window) and att.state_spec() is None
    att.load(DictSource(w, dtype))
    n_a, n_b = 11, 7
    xa, xb = torch.randn(n_a, H).to(dtype), torch.randn(n_b, H).to(dtype)
    pool = torch.zeros(2, 9, nkv, ps, d, dtype=dtype, device="cuda")
    cache = LayerCache(pool[0], pool[1], 0, ps)
    tables = [[7, 2, 5], [0, 8]]
    # step 1: tokens 0..5 of A and 0..5 of B;  step 2: tokens 6..10 of A beside the last token of B
    s1 = FakeStep([0, 0], [6, 6], ps, tables)
    o1 = att.forward(torch.cat([xa[:6], xb[:6]]).cuda(), s1, cache, None)
    s2 = FakeStep([6, 6], [5, 1], ps, tables)
    o2 = att.forward(torch.cat([xa[6:], xb[6:]]).cuda(), s2, cache, None)
    got_a = torch.cat([o1[:6], o2[:5]]).float().cpu()
    got_b = torch.cat([o1[6:], o2[5:]]).float().cpu()

    def plain(x):
        n = x.shape[0]
        q = P.linear(x, w["q"]).view(n, nh, d)
        k = P.linear(x, w["k"]).view(n, nkv, d)
        v = P.linear(x, w["v"]).view(n, nkv, d)
        if dtype == torch.bfloat16:            # the product's output is stored in bfloat16
            q, k, v = (t.bfloat16().float() for t in (q, k, v))
        if rotate:
            cos, sin = P.rope_tables(P.inv_freqs(cfg), torch.arange(n))
            q, k = P.apply_rope(q, cos, sin), P.apply_rope(k, cos, sin)
        o = P.causal_attention(q, k, v, 0, window=window).reshape(n, nh * d)
        return P.linear(o, w["o"])

    for got, x in ((got_a, xa), (got_b, xb)):
        err = (got - plain(x.float())).abs().max()
        assert err <= tol(dtype) * 2, err


@pytest.mark.parametrize("window", [None, 9])
@pytest.mark.parametrize("rotate", [True, False])
def test_attention_part_in_steps_of_single_tokens(window, rotate):
    """Head size 64 in bfloat16: steps of single tokens take the kernel that rotates and stores
    the newest key itself.  A prompt in one step, then three steps of one token for each of two
    requests; the outputs equal plain attention over the whole sequences."""
    from rust_llm_inference_server_b200.parts import GQAAttentionSpec, LayerCache, NoPositionSpec, RopeSpec, build_mixer
    torch.manual_seed(2)
    dtype = torch.bfloat16
    H, nh, nkv, d, ps = 96, 4, 2, 64, 8
    cfg = {"head_dim": d, "rope_theta": 5000.0, "hidden_size": H, "num_attention_heads": nh, "num_key_value_heads": nkv}
    w = {"q": torch.randn(nh * d, H) * 0.2, "k": torch.randn(nkv * d, H) * 0.2, "v": torch.randn(nkv * d, H) * 0.2,
         "o": torch.randn(H, nh * d) * 0.1}     # 256 inputs: outputs of the size the other part tests have
    w = {k: v.bfloat16().float() for k, v in w.items()}
    spec = GQAAttentionSpec(H, nh, nkv, d, "q", "k", "v", "o",
                            position=RopeSpec(d, 5000.0, None) if rotate else NoPositionSpec(), window=window)
    att = build_mixer(spec, dtype, "cuda")
    att.load(DictSource(w, dtype))
    n_a, n_b, n_dec = 15, 6, 3
    xa, xb = torch.randn(n_a + n_dec, H).to(dtype), torch.randn(n_b + n_dec, H).to(dtype)
    pool = torch.zeros(2, 9, nkv, ps, d, dtype=dtype, device="cuda")
    cache = LayerCache(pool[0], pool[1], 0, ps)
    tables = [[7, 2, 5], [0, 8]]
    o = att.forward(torch.cat([xa[:n_a], xb[:n_b]]).cuda(), FakeStep([0, 0], [n_a, n_b], ps, tables), cache, None)
    got_a, got_b = [o[:n_a]], [o[n_a:]]
    for i in range(n_dec):
        step = FakeStep([n_a + i, n_b + i], [1, 1], ps, tables)
        assert step.all_decode
        o = att.forward(torch.stack([xa[n_a + i], xb[n_b + i]]).cuda(), step, cache, None)
        got_a.append(o[:1])
        got_b.append(o[1:])

    def plain(x):
        n = x.shape[0]
        q = P.linear(x, w["q"]).view(n, nh, d).bfloat16().float()
        k = P.linear(x, w["k"]).view(n, nkv, d).bfloat16().float()
        v = P.linear(x, w["v"]).view(n, nkv, d).bfloat16().float()
        if rotate:
            cos, sin = P.rope_tables(P.inv_freqs(cfg), torch.arange(n))
            q, k = P.apply_rope(q, cos, sin), P.apply_rope(k, cos, sin)
        return P.linear(P.causal_attention(q, k, v, 0, window=window).reshape(n, nh * d), w["o"])

    for got, x in ((got_a, xa), (got_b, xb)):
        err = (torch.cat(got).float().cpu() - plain(x.float())).abs().max()
        assert err <= tol(dtype) * 2, err


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prenorm_block(dtype):
    from rust_llm_inference_server_b200.config import LlamaConfig
    from rust_llm_inference_server_b200.models.llama import describe_llama
    from rust_llm_inference_server_b200.parts import LayerCache, build_block
    from rust_llm_inference_server_b200.weights import random_tensors
    from tests.tiny_configs import TINY_C
    cfg = LlamaConfig.from_dict(TINY_C)
    w = {k: v.float() for k, v in random_tensors(TINY_C, 5).items()}
    blk = build_block(describe_llama(cfg).layers[1], dtype, "cuda")
    for part in blk.parts():
        part.load(DictSource(w, dtype))
    T, ps = 13, 8
    x = torch.randn(T, cfg.hidden_size)
    pool = torch.zeros(2, 4, cfg.num_key_value_heads, ps, cfg.head_dim, dtype=dtype, device="cuda")
    step = FakeStep([0], [T], ps, [[3, 1]])
    resid = x.cuda()
    resid, delta = blk.forward(resid, None, step, LayerCache(pool[0], pool[1], 0, ps), None)
    got = resid.cpu() + delta.float().cpu()
    want = P.decoder_layer(x, w, 1, TINY_C, torch.arange(T))
    assert (got - want).abs().max() <= (1e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_and_lm_head_parts(dtype):
    """The two ends of the residual stream as parts: the table's rows widened to float32 (times a
    scale when the spec gives one), and float32 logits of chosen rows (scaled and capped smoothly
    when the spec says so); a tied pair shares one tensor on the device."""
    from rust_llm_inference_server_b200.parts import EmbeddingSpec, LMHeadSpec, build_embedding, build_lm_head
    V, H, T = 301, 80, 23
    g = torch.Generator().manual_seed(5)
    tensors = {"emb": (torch.randn(V, H, generator=g) * 0.5).bfloat16().float(),
               "head": (torch.randn(V, H, generator=g) * 0.5).bfloat16().float()}
    src = DictSource(tensors, dtype)
    ids = torch.randint(0, V, (T,), generator=g)
    step = FakeStep([0], [T], 8, [list(range(4))])
    for scale in (None, 3.5):
        emb = build_embedding(EmbeddingSpec(V, H, "emb", scale=scale), dtype, "cuda")
        assert emb.tensors() == {"emb": (V, H)}
        emb.load(src)
        out = torch.empty(T, H, dtype=torch.float32, device="cuda")
        emb.forward(ids.to(torch.int32).cuda(), out, step)
        want = P.embedding(ids, tensors["emb"]) * (1.0 if scale is None else np.float32(scale))
        assert torch.equal(out.cpu(), want)                   # a row select and one float32 product: exact
    h = (torch.randn(T, H, generator=g)).to(dtype)
    for name, ls, cap in (("emb", None, None), ("head", 2.0, None), ("head", None, 3.0), ("emb", 0.5, 1.25)):
        head = build_lm_head(LMHeadSpec(V, H, name, logit_scale=ls, soft_cap=cap), dtype, "cuda")
        head.load(src)
        if name == "emb":
            assert head.weight is emb.weight                  # tied: one copy
        got = head.forward(h.cuda(), step)
        assert got.dtype == torch.float32 and got.shape == (T, V)
        want = P.linear(h.float(), tensors[name]) * (1.0 if ls is None else ls)
        if cap is not None:
            want = cap * torch.tanh(want / cap)
        assert (got.cpu() - want).abs().max() <= (2e-5 if dtype == torch.float32 else 2e-2) * max(1.0, float(want.abs().max()))
