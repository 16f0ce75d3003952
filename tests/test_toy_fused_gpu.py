"""A toy feed-forward, defined in this test only, that takes part in the norm fusion of short
steps: it says `fuses_norms`, hands `ops.ScaledRows` to its first product as they are and the
`sink` to its last.  Registered, built from a config and replayed against a plain restatement,
with the fusion on and off, without a change to the framework's files."""

import os
from dataclasses import dataclass

import numpy as np
import pytest
import torch

from tests import replay_util as R
from tests.plain import llama_plain as P

pytestmark = pytest.mark.gpu

CFG = {"architectures": ["ToyReluForCausalLM"], "vocab_size": 203, "hidden_size": 72, "intermediate_size": 104,
       "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32, "rms_norm_eps": 3e-6, "rope_theta": 9000.0,
       "num_hidden_layers": 3, "max_position_embeddings": 512}


@dataclass(frozen=True)
class ReluSpec:
    hidden: int
    intermediate: int
    prefix: str
    kind: str = "toy_relu_ff"


def register():
    from rust_llm_inference_server_b200 import ops
    from rust_llm_inference_server_b200.config import register_architecture, registered_architectures
    from rust_llm_inference_server_b200.parts import (FeedForward, GQAAttentionSpec, LayerCall, LayerSpec, ModelSpec,
                                                      RMSNormSpec, RopeSpec, register_feed_forward)
    if "ToyReluForCausalLM" in registered_architectures():
        return

    class ReluFF(FeedForward):
        """down(relu(up x)).  x may be ScaledRows and goes to the product as it is; the sink, if
        one is given, goes to the last product, whose return value is this part's."""

        graph_safe = True

        def __init__(self, spec, dtype, device):
            self.spec, self.dtype = spec, dtype

        def tensors(self):
            s = self.spec
            return {s.prefix + "up": (s.intermediate, s.hidden), s.prefix + "down": (s.hidden, s.intermediate)}

        def load(self, src):
            self.up = src.get(self.spec.prefix + "up").contiguous()
            self.down = src.get(self.spec.prefix + "down").contiguous()

        def fuses_norms(self, step):
            return ops.fuses_norms(step.n_tokens, self.dtype, self.spec.hidden, self.spec.intermediate)

        def forward(self, x, step, sink=None):
            h = torch.relu(ops.linear(x, self.up))
            return ops.linear(h, self.down, sink=sink) if sink is not None else ops.linear(h, self.down)

    def describe(cfg):
        H, d = cfg["hidden_size"], cfg["head_dim"]
        layers = []
        for i in range(cfg["num_hidden_layers"]):
            p = f"l{i}."
            layers.append(LayerSpec(
                RMSNormSpec(H, cfg["rms_norm_eps"], p + "n1"),
                GQAAttentionSpec(H, cfg["num_attention_heads"], cfg["num_key_value_heads"], d, p + "q", p + "k",
                                 p + "v", p + "o", position=RopeSpec(d, cfg["rope_theta"])),
                RMSNormSpec(H, cfg["rms_norm_eps"], p + "n2"),
                ReluSpec(H, cfg["intermediate_size"], p + "ff.")))
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
            out[p + "ff.up"] = ((I, H), "matrix")
            out[p + "ff.down"] = ((H, I), "matrix")
        return out

    register_feed_forward("toy_relu_ff", ReluFF, replace=True)
    register_architecture("ToyReluForCausalLM", lambda d: d, describe, kinds)


def plain(w, toks):
    n = len(toks)
    nh, nkv, d, eps = (CFG[k] for k in ("num_attention_heads", "num_key_value_heads", "head_dim", "rms_norm_eps"))
    inv = 1.0 / CFG["rope_theta"] ** (torch.arange(0, d, 2, dtype=torch.float32) / d)
    cos, sin = P.rope_tables(inv, torch.arange(n))
    x = P.embedding(torch.tensor(toks), w["embed"])
    for i in range(CFG["num_hidden_layers"]):
        p = f"l{i}."
        h = P.rms_norm(x, w[p + "n1"], eps)
        q = P.apply_rope(P.linear(h, w[p + "q"]).view(n, nh, d), cos, sin)
        k = P.apply_rope(P.linear(h, w[p + "k"]).view(n, nkv, d), cos, sin)
        v = P.linear(h, w[p + "v"]).view(n, nkv, d)
        x = x + P.linear(P.causal_attention(q, k, v, 0).reshape(n, nh * d), w[p + "o"])
        h = P.rms_norm(x, w[p + "n2"], eps)
        x = x + P.linear(torch.relu(P.linear(h, w[p + "ff.up"])), w[p + "ff.down"])
    return P.linear(P.rms_norm(x, w["final"], eps), w["embed"])


def test_a_toy_feed_forward_takes_part_in_the_norm_fusion(model_root, monkeypatch):
    register()
    from rust_llm_inference_server_b200 import ops
    from rust_llm_inference_server_b200.engine.replay import ReplaySession
    from rust_llm_inference_server_b200.weights import write_random_model
    from safetensors.torch import load_file
    d = os.path.join(model_root, "toy_relu")
    if not os.path.isdir(d):
        write_random_model(CFG, d, seed=21)
    w = {k: v.float() for k, v in load_file(os.path.join(d, "model.safetensors")).items()}
    rng = np.random.default_rng(4)
    reqs = {f"t{i}": rng.integers(0, CFG["vocab_size"], size=n).tolist() for i, n in enumerate([61, 20, 97])}
    ref = {k: plain(w, v).numpy() for k, v in reqs.items()}
    # float32: the parts as they are (no fusion in that path), every way of cutting
    for fam, steps in (("whole", R.whole_trace(reqs)), ("decode", R.decode_trace(reqs, tail=20)),
                       ("chunks", R.chunk_trace(reqs, seed=2)), ("mixed", R.mixed_trace(reqs, seed=3))):
        s = ReplaySession(d, "float32", R.live_token_peak(steps))
        got = R.collect(s.step, steps)
        worst = max(float(np.abs(v - ref[k[0]][k[1]]).max()) for k, v in got.items())
        assert worst <= 2e-4, (fam, worst)
    # bfloat16, single tokens and short portions: with the fusion on, the toy part's products do the
    # norms' work (fewer launches); on or off the logits are the plain ones to bfloat16 rounding
    steps = R.decode_trace(reqs, tail=20) + [dict(s, step=s["step"] + 1000) for s in R.chunk_trace(reqs, seed=5)]
    got, launches = {}, {}
    for fused in (True, False):
        monkeypatch.setattr(ops, "FUSE_NORMS", fused)
        s = ReplaySession(d, "bfloat16", R.live_token_peak(steps))
        s.model.graph_safe = False               # count launches, not graph replays
        before = ops.launch_count
        got[fused] = R.collect(s.step, steps)
        launches[fused] = ops.launch_count - before
        worst = max(float(np.abs(v - ref[k[0]][k[1]]).max()) for k, v in got[fused].items())
        assert worst <= 3e-2, (fused, worst)
    assert launches[True] < launches[False]
    assert max(float(np.abs(v - got[False][k]).max()) for k, v in got[True].items()) <= 2e-2
