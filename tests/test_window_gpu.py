"""A toy architecture (it lives in this test only) whose layers alternate between attention over
all earlier tokens and attention over a window: two cache groups with block tables of their own.
Replayed in every way of cutting against plain attention, it also shows that the window group
gives pages back as decoding passes them, while the other group keeps everything."""

import os

import numpy as np
import pytest
import torch

from tests import replay_util as R
from tests.plain import llama_plain as P

pytestmark = pytest.mark.gpu

WINDOW = 24
CFG = {"architectures": ["ToyWindowForCausalLM"], "vocab_size": 199, "hidden_size": 128, "intermediate_size": 96,
       "num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 64, "rms_norm_eps": 1e-5, "rope_theta": 5000.0,
       "num_hidden_layers": 4, "max_position_embeddings": 1024}


def register():
    from rust_llm_inference_server_b200.config import register_architecture, registered_architectures
    from rust_llm_inference_server_b200.parts import (GQAAttentionSpec, LayerCall, LayerSpec, ModelSpec, RMSNormSpec,
                                                      RopeSpec, SwiGLUSpec)
    if "ToyWindowForCausalLM" in registered_architectures():
        return

    def describe(cfg):
        H, d = cfg["hidden_size"], cfg["head_dim"]
        layers = []
        for i in range(cfg["num_hidden_layers"]):
            p = f"l{i}."
            layers.append(LayerSpec(
                RMSNormSpec(H, cfg["rms_norm_eps"], p + "n1"),
                GQAAttentionSpec(H, cfg["num_attention_heads"], cfg["num_key_value_heads"], d, p + "q", p + "k",
                                 p + "v", p + "o", position=RopeSpec(d, cfg["rope_theta"], None),
                                 window=WINDOW if i % 2 else None),
                RMSNormSpec(H, cfg["rms_norm_eps"], p + "n2"),
                SwiGLUSpec(H, cfg["intermediate_size"], p + "gate", p + "up", p + "down")))
        return ModelSpec(cfg["vocab_size"], H, "embed", tuple(layers),
                         tuple(LayerCall(i, i) for i in range(len(layers))), RMSNormSpec(H, cfg["rms_norm_eps"], "final"),
                         "embed", cfg["max_position_embeddings"])

    def kinds(cfg):
        H, I, nh, nkv, d = (cfg[k] for k in ("hidden_size", "intermediate_size", "num_attention_heads",
                                             "num_key_value_heads", "head_dim"))
        out = {"embed": ((cfg["vocab_size"], H), "matrix"), "final": ((H,), "norm")}
        for i in range(cfg["num_hidden_layers"]):
            p = f"l{i}."
            out[p + "n1"] = out[p + "n2"] = ((H,), "norm")
            out[p + "q"] = ((nh * d, H), "matrix")
            out[p + "k"] = out[p + "v"] = ((nkv * d, H), "matrix")
            out[p + "o"] = ((H, nh * d), "matrix")
            out[p + "gate"] = out[p + "up"] = ((I, H), "matrix")
            out[p + "down"] = ((H, I), "matrix")
        return out

    register_architecture("ToyWindowForCausalLM", lambda d: d, describe, kinds)


def plain(w, toks):
    n = len(toks)
    nh, nkv, d, eps = CFG["num_attention_heads"], CFG["num_key_value_heads"], CFG["head_dim"], CFG["rms_norm_eps"]
    x = P.embedding(torch.tensor(toks), w["embed"])
    cos, sin = P.rope_tables(P.inv_freqs(CFG), torch.arange(n))
    for i in range(CFG["num_hidden_layers"]):
        p = f"l{i}."
        h = P.rms_norm(x, w[p + "n1"], eps)
        q = P.apply_rope(P.linear(h, w[p + "q"]).view(n, nh, d), cos, sin)
        k = P.apply_rope(P.linear(h, w[p + "k"]).view(n, nkv, d), cos, sin)
        v = P.linear(h, w[p + "v"]).view(n, nkv, d)
        o = P.causal_attention(q, k, v, 0, window=WINDOW if i % 2 else None).reshape(n, nh * d)
        x = x + P.linear(o, w[p + "o"])
        h = P.rms_norm(x, w[p + "n2"], eps)
        x = x + P.linear(torch.nn.functional.silu(P.linear(h, w[p + "gate"])) * P.linear(h, w[p + "up"]), w[p + "down"])
    return P.linear(P.rms_norm(x, w["final"], eps), w["embed"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_window_layers_have_a_cache_group_of_their_own(model_root, dtype):
    register()
    from rust_llm_inference_server_b200.engine.replay import ReplaySession
    from rust_llm_inference_server_b200.weights import write_random_model
    from safetensors.torch import load_file
    d = os.path.join(model_root, "toy_window")
    if not os.path.isdir(d):
        write_random_model(CFG, d, seed=21)
    w = {k: v.float() for k, v in load_file(os.path.join(d, "model.safetensors")).items()}
    rng = np.random.default_rng(4)
    reqs = {f"w{i}": rng.integers(0, CFG["vocab_size"], size=n).tolist() for i, n in enumerate([150, 40, 97, 23])}
    ref = {k: plain(w, v).numpy() for k, v in reqs.items()}
    tol = 1e-4 if dtype == "float32" else 4e-2
    for fam, steps in (("whole", R.whole_trace(reqs)), ("decode", R.decode_trace(reqs, tail=40)),
                       ("chunks", R.chunk_trace(reqs, seed=2)), ("mixed", R.mixed_trace(reqs, seed=3))):
        s = ReplaySession(d, dtype, R.live_token_peak(steps))
        assert [(g.window, g.slots) for g in s.storage.groups] == [(0, [0, 2]), (WINDOW, [1, 3])]
        got = R.collect(s.step, steps)
        worst = max(float(np.abs(v - ref[k[0]][k[1]]).max()) for k, v in got.items())
        assert worst <= tol, (fam, worst)
        assert s.cache.check_invariants() == ""
    # decoding token by token: the window group holds about WINDOW / page tokens' pages, the other grows
    s = ReplaySession(d, dtype, 256)
    toks = reqs["w0"]
    for i, t in enumerate(toks):
        s.step({"step": i, "entries": [{"id": "x", "tokens": [t], "want": []}], "end": []})
    full_pages = s.cache.group(0).num_pages - s.cache.num_free_pages(0)
    window_pages = s.cache.group(1).num_pages - s.cache.num_free_pages(1)
    assert full_pages == (len(toks) + 15) // 16
    assert window_pages <= WINDOW // 16 + 2 < full_pages
    assert s.cache.table(0, 1)[:3] == [-1, -1, -1]          # its first pages were given back
