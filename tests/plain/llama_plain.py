"""Plain, slow implementation of the Llama decoder that the engine is checked against.

Whole sequences, no cache, float32 on the CPU, one function for each part.  It shares no code
with the package: it takes the raw `config.json` dictionary and a dictionary of tensors by
their checkpoint names.

It rests on the formulas of akshajnad/rust_llm_inference_server (each function cites the file
and lines it restates).  That project's model code is Rust on the candle library and cannot be
compiled in this environment (no Rust toolchain), so there is no run of it behind these
functions; the numeric anchors that need no compilation (the llama3-scaled inverse frequencies
printed in crates/model/src/rope.rs:147-156, the sampler's hash constants) are checked in
tests/test_plain.py.
"""

from __future__ import annotations

import math

import numpy as np
import torch


# --------------------------------------------------------------------------- configuration

def head_dim_of(cfg: dict) -> int:
    """crates/model/src/config.rs:44-47: `head_dim` if given, else hidden_size / heads."""
    hd = cfg.get("head_dim")
    return int(hd) if hd is not None else cfg["hidden_size"] // cfg["num_attention_heads"]


# --------------------------------------------------------------------------- position encoding

def inv_freqs(cfg: dict) -> torch.Tensor:
    """crates/model/src/rope.rs:19-49.  Everything in float32, as the reference does.

    base[j] = 1 / theta^(2j/d); with rope_type "llama3" each frequency is kept, divided by
    `factor`, or blended, depending on its wavelength against the original context length.
    """
    d = head_dim_of(cfg)
    f32 = np.float32
    theta = f32(cfg["rope_theta"])
    base = [f32(1.0) / np.power(theta, f32(i) / f32(d), dtype=f32) for i in range(0, d, 2)]
    s = cfg.get("rope_scaling")
    if s and s.get("rope_type", s.get("type")) == "llama3":
        factor = f32(s["factor"])
        low, high = f32(s["low_freq_factor"]), f32(s["high_freq_factor"])
        old = f32(s["original_max_position_embeddings"])
        low_wl, high_wl = old / low, old / high
        out = []
        for f in base:
            wl = f32(2.0) * f32(math.pi) / f
            if wl < high_wl:
                out.append(f)
            elif wl > low_wl:
                out.append(f / factor)
            else:
                smooth = (old / wl - low) / (high - low)
                out.append((f32(1.0) - smooth) * f / factor + smooth * f)
        base = out
    return torch.tensor(np.array(base, dtype=f32))


def rope_tables(inv: torch.Tensor, positions: torch.Tensor):
    """crates/model/src/rope.rs:61-78: angle[p, j] = p * inv_freq[j] in float32; cos and sin."""
    ang = positions.to(torch.float32)[:, None] * inv[None, :]
    return ang.cos(), ang.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """crates/model/src/rope.rs:111-117 (non-interleaved "rotate half").

    x is (tokens, heads, d).  out[j] = x[j] cos - x[j+d/2] sin; out[j+d/2] = x[j+d/2] cos + x[j] sin.
    """
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


# --------------------------------------------------------------------------- parts

def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """crates/model/src/layers.rs:199-204 and llama.rs:256-262: row lookup, no scaling."""
    return table[ids.long()]


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """crates/model/src/layers.rs:141-146: x / sqrt(mean(x^2) + eps) * w; eps used as float32
    (layers.rs:115); the weight multiplies directly."""
    eps32 = float(np.float32(eps))
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps32) * w


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """crates/model/src/layers.rs:75-82: weight stored (out, in); y = x W^T; no bias."""
    return x @ w.t()


def causal_attention(q, k, v, start_pos: int = 0, window: int | None = None):
    """crates/model/src/attention.rs:204-233.

    q (len, nh, d), k and v (total, nkv, d) with total = start_pos + len.  Query head h uses
    key/value head h // (nh // nkv).  scores = q k^T / sqrt(d) in float32, key c is hidden from
    query r = start_pos + i where c > r, softmax over keys in float32, out = p v.
    `window` (not in the reference's Llama; used by tests of the parts) also hides keys
    c <= r - window.
    """
    ln, nh, d = q.shape
    total, nkv, _ = k.shape
    n_rep = nh // nkv
    kk = k.repeat_interleave(n_rep, dim=1)
    vv = v.repeat_interleave(n_rep, dim=1)
    scores = torch.einsum("qhd,khd->hqk", q, kk) * (1.0 / math.sqrt(d))
    r = torch.arange(start_pos, start_pos + ln)[:, None]
    c = torch.arange(total)[None, :]
    hidden = c > r
    if window is not None:
        hidden = hidden | (c <= r - window)
    scores = scores.masked_fill(hidden[None], float("-inf"))
    p = torch.softmax(scores.float(), dim=-1)
    return torch.einsum("hqk,khd->qhd", p, vv)


def attention_block(x, w: dict, prefix: str, cfg: dict, positions: torch.Tensor):
    """crates/model/src/attention.rs:66-104: q/k/v projections, head split, rotation of q and k,
    attention, output projection.  x is (len, hidden) holding a whole sequence from position 0."""
    nh, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], head_dim_of(cfg)
    n = x.shape[0]
    q = linear(x, w[prefix + "q_proj.weight"]).view(n, nh, d)
    k = linear(x, w[prefix + "k_proj.weight"]).view(n, nkv, d)
    v = linear(x, w[prefix + "v_proj.weight"]).view(n, nkv, d)
    cos, sin = rope_tables(inv_freqs(cfg), positions)
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    o = causal_attention(q, k, v, 0).reshape(n, nh * d)
    return linear(o, w[prefix + "o_proj.weight"])


def swiglu_mlp(x, w: dict, prefix: str):
    """crates/model/src/layers.rs:178-186: down(silu(gate(x)) * up(x))."""
    g = linear(x, w[prefix + "gate_proj.weight"])
    u = linear(x, w[prefix + "up_proj.weight"])
    return linear(torch.nn.functional.silu(g) * u, w[prefix + "down_proj.weight"])


def decoder_layer(x, w: dict, i: int, cfg: dict, positions):
    """crates/model/src/llama.rs:264-271: x += attn(norm(x)); x += mlp(norm(x))."""
    p = f"model.layers.{i}."
    eps = cfg["rms_norm_eps"]
    h = rms_norm(x, w[p + "input_layernorm.weight"], eps)
    x = x + attention_block(h, w, p + "self_attn.", cfg, positions)
    h = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
    return x + swiglu_mlp(h, w, p + "mlp.")


def lm_head_weight(w: dict, cfg: dict):
    """crates/model/src/llama.rs:152-156: the embedding table when `tie_word_embeddings`
    (false when the key is absent, config.rs:19-20), else `lm_head.weight`."""
    if cfg.get("tie_word_embeddings", False):
        return w["model.embed_tokens.weight"]
    return w["lm_head.weight"]


def forward_logits(w: dict, cfg: dict, tokens, rows=None) -> torch.Tensor:
    """crates/model/src/llama.rs:218-311 for one whole sequence: float32 logits (len, vocab)
    at every position, or at the positions `rows` only (llama.rs:296-305 selects rows before the
    LM head in the same way)."""
    w = {k: v if v.dtype == torch.float32 else v.to(torch.float32) for k, v in w.items()}
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    positions = torch.arange(len(ids))
    x = embedding(ids, w["model.embed_tokens.weight"])
    for i in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, w, i, cfg, positions)
    x = rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    if rows is not None:
        x = x[torch.as_tensor(list(rows), dtype=torch.long)]
    return linear(x, lm_head_weight(w, cfg))


def greedy_generate(w: dict, cfg: dict, prompt, n_new: int):
    """Greedy continuation by recomputing the whole sequence each token (ties: lowest id,
    crates/engine/src/sampler.rs:238-246)."""
    toks = list(prompt)
    out = []
    for _ in range(n_new):
        t = argmax(forward_logits(w, cfg, toks)[-1].numpy())
        toks.append(t)
        out.append(t)
    return out


# --------------------------------------------------------------------------- sampling

M32 = 0xFFFFFFFF


def lowbias32(x: int) -> int:
    """crates/model/src/sampling.rs:11-18."""
    x &= M32
    x ^= x >> 16
    x = (x * 0x7FEB352D) & M32
    x ^= x >> 15
    x = (x * 0x846CA68B) & M32
    x ^= x >> 16
    return x


def row_key(seed: int, position: int) -> int:
    """crates/model/src/sampling.rs:21-23."""
    seed &= 0xFFFFFFFFFFFFFFFF
    return lowbias32(lowbias32(lowbias32(seed & M32) ^ (seed >> 32)) ^ (position & M32))


def uniform(h: int) -> np.float32:
    """crates/model/src/sampling.rs:61-63: top 23 bits plus a half, times 2^-23; in (0, 1)."""
    return np.float32((np.float32(h >> 9) + np.float32(0.5)) * np.float32(1.0 / 8388608.0))


def gumbel(key: int, v: int) -> np.float32:
    """crates/model/src/sampling.rs:54-57."""
    u = uniform(lowbias32(key ^ ((v * 0x9E3779B9) & M32)))
    return np.float32(-np.log(-np.log(u, dtype=np.float32), dtype=np.float32))


def argmax(logits) -> int:
    """crates/engine/src/sampler.rs:238-246: ties go to the lowest index."""
    return int(np.argmax(np.asarray(logits)))


def sample_row(logits, temperature: float, key: int) -> int:
    """crates/model/src/sampling.rs:86-100: greedy, or argmax(logit / T + gumbel noise), ties to
    the lowest id."""
    logits = np.asarray(logits, dtype=np.float32)
    if temperature < 1e-5:
        return argmax(logits)
    inv_t = np.float32(1.0) / np.float32(temperature)
    v = np.arange(len(logits), dtype=np.uint64)
    h = (key ^ ((v * 0x9E3779B9) & M32)).astype(np.uint64)
    # vectorised lowbias32
    h ^= h >> 16
    h = (h * 0x7FEB352D) & M32
    h ^= h >> 15
    h = (h * 0x846CA68B) & M32
    h ^= h >> 16
    u = ((h >> 9).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 8388608.0)
    g = -np.log(-np.log(u, dtype=np.float32), dtype=np.float32)
    s = logits * inv_t + g
    return int(np.argmax(s))


def apply_repetition_penalty(logits: np.ndarray, history, penalty: float) -> np.ndarray:
    """crates/engine/src/sampler.rs:225-235: every distinct seen token: divide a positive logit
    by the penalty, multiply a negative one."""
    out = np.array(logits, dtype=np.float32)
    for t in set(int(t) for t in history):
        if 0 <= t < len(out):
            out[t] = out[t] / np.float32(penalty) if out[t] > 0 else out[t] * np.float32(penalty)
    return out


def filtered_distribution(logits, temperature: float, top_k: int, top_p: float) -> np.ndarray:
    """crates/engine/src/sampler.rs:116-209: the distribution the host sampler draws from.

    weights exp((l - max)/T) in float64; top-k keeps the k highest (ties: lower id first);
    top-p keeps the shortest prefix of the descending order whose share of the mass (of the
    whole vocabulary, or of the top-k set) reaches top_p, the crossing token included.
    """
    logits = np.asarray(logits, dtype=np.float32)
    n = len(logits)
    w = np.exp((logits.astype(np.float64) - float(logits.max())) / float(temperature))
    order = sorted(range(n), key=lambda i: (-float(logits[i]), i))
    if top_k and top_k < n:
        order = order[:top_k]
    total = sum(w[i] for i in order) if (top_k and top_k < n) else float(w.sum())
    if top_p < 1.0:
        acc, keep = 0.0, len(order)
        for j, i in enumerate(order):
            acc += w[i] / total
            if acc >= top_p:
                keep = j + 1
                break
        order = order[:keep]
    p = np.zeros(n, dtype=np.float64)
    for i in order:
        p[i] = w[i]
    return p / p.sum()


def uniform_53(seed: int, position: int) -> int:
    """The engine's uniform for top-k / top-p rows as a 53-bit integer (u = this / 2^53): two
    rounds of the splitmix64 finaliser over (seed, position).  (The reference seeds a ChaCha8
    stream per request, crates/engine/src/sampler.rs:57-66; a hash of the position instead makes a
    draw independent of how many draws came before, so a preempted request repeats its tokens.)"""
    m = (1 << 64) - 1

    def mix(x):
        x = (x + 0x9E3779B97F4A7C15) & m
        x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & m
        x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & m
        return x ^ (x >> 31)

    return mix(mix(seed & m) ^ (position & m)) >> 11


def filtered_sample(logits, temperature: float, top_k: int, top_p: float, u53: int) -> int:
    """The engine's rule for top-k / top-p rows, restated slowly with Python integers.  Filtering
    as crates/engine/src/sampler.rs:116-209: the k highest logits (ties: lower id first), the
    shortest descending prefix whose share of the mass reaches top_p, the crossing token included.
    The reference then draws from the descending order with a ChaCha8 stream; here weights are
    fixed-point, w = floor(float32 exp((l - max) / T) * 2^40), and the draw is by inverse CDF in
    vocabulary order with the uniform u53 / 2^53: r = floor(u * kept mass), the first kept token
    whose running mass exceeds r."""
    l = np.asarray(logits, dtype=np.float32)
    inv_t = np.float32(1.0) / np.float32(temperature)
    w = [int(np.float32(np.exp(np.float32((x - l.max()) * inv_t), dtype=np.float32) * np.float32(2.0 ** 40))) for x in l]
    order = sorted(range(len(l)), key=lambda i: (-float(l[i]), i))
    if 0 < top_k < len(l):
        order = order[:top_k]
    mass = sum(w[i] for i in order)
    if np.float32(top_p) < 1:
        target = int(float(np.float32(top_p)) * float(mass))
        acc, keep = 0, len(order)
        for j, i in enumerate(order):
            acc += w[i]
            if acc >= target:
                keep = j + 1
                break
        order = order[:keep]
    kept = set(order)
    total = sum(w[i] for i in kept)
    r = ((u53 << 11) * total) >> 64
    acc = 0
    for v in range(len(l)):
        if v in kept:
            acc += w[v]
            if acc > r:
                return v
    return 0
