"""A toy architecture whose two ends differ from Llama's: the embedding is multiplied by
sqrt(hidden), the logits are scaled and capped smoothly (cap * tanh(x / cap)), and a second variant
registers an LM head of its own kind.  Both are described, registered, built and replayed in every
way of cutting from this test alone; the framework's files name no embedding or head op."""

import math
import os
from dataclasses import dataclass

import numpy as np
import pytest
import torch

from tests import replay_util as R
from tests.plain import llama_plain as P

pytestmark = pytest.mark.gpu

CFG = {"architectures": ["ToyCappedForCausalLM"], "vocab_size": 333, "hidden_size": 72, "intermediate_size": 120,
       "num_attention_heads": 3, "num_key_value_heads": 3, "head_dim": 32, "rms_norm_eps": 1e-5, "rope_theta": 7000.0,
       "num_hidden_layers": 2, "max_position_embeddings": 512, "logit_scale": 4.0, "final_logit_cap": 1.0,
       "own_head": False}
CFG_OWN = {**CFG, "architectures": ["ToyBiasedHeadForCausalLM"], "own_head": True}


@dataclass(frozen=True)
class BiasedHeadSpec:
    vocab_size: int
    dim: int
    weight: str
    bias: str
    kind: str = "toy_biased_head"


def register():
    from rust_llm_inference_server_b200 import ops
    from rust_llm_inference_server_b200.config import register_architecture, registered_architectures
    from rust_llm_inference_server_b200.parts import (EmbeddingSpec, GQAAttentionSpec, LayerCall, LayerSpec, LMHeadSpec,
                                                      LogitsHead, ModelSpec, RMSNormSpec, RopeSpec, SwiGLUSpec,
                                                      register_lm_head)
    if "ToyCappedForCausalLM" in registered_architectures():
        return

    class BiasedHead(LogitsHead):
        """Logits with a bias per token, stored in 32-bit and kept so."""
        graph_safe = True

        def __init__(self, spec, dtype, device):
            self.spec = spec

        def tensors(self):
            return {self.spec.weight: (self.spec.vocab_size, self.spec.dim), self.spec.bias: (self.spec.vocab_size,)}

        def load(self, src):
            self.weight = src.get(self.spec.weight, share=True).contiguous()
            self.bias = src.get(self.spec.bias, "vector")

        def forward(self, h, step):
            return ops.linear(h, self.weight, out_dtype=torch.float32).add_(self.bias)

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
                SwiGLUSpec(H, cfg["intermediate_size"], p + "gate", p + "up", p + "down")))
        head = BiasedHeadSpec(cfg["vocab_size"], H, "embed", "head_bias") if cfg["own_head"] else \
            LMHeadSpec(cfg["vocab_size"], H, "embed", logit_scale=cfg["logit_scale"], soft_cap=cfg["final_logit_cap"])
        return ModelSpec(cfg["vocab_size"], H, EmbeddingSpec(cfg["vocab_size"], H, "embed", scale=math.sqrt(H)),
                         tuple(layers), tuple(LayerCall(i, i) for i in range(len(layers))),
                         RMSNormSpec(H, cfg["rms_norm_eps"], "final"), head, cfg["max_position_embeddings"])

    def kinds(cfg):
        H, I, nh, nkv, d = (cfg[k] for k in ("hidden_size", "intermediate_size", "num_attention_heads",
                                             "num_key_value_heads", "head_dim"))
        out = {"embed": ((cfg["vocab_size"], H), "matrix"), "final": ((H,), "norm")}
        if cfg["own_head"]:
            out["head_bias"] = ((cfg["vocab_size"],), "norm")
        for i in range(cfg["num_hidden_layers"]):
            p = f"l{i}."
            out[p + "n1"] = out[p + "n2"] = ((H,), "norm")
            out[p + "q"] = ((nh * d, H), "matrix")
            out[p + "k"] = out[p + "v"] = ((nkv * d, H), "matrix")
            out[p + "o"] = ((H, nh * d), "matrix")
            out[p + "gate"] = out[p + "up"] = ((I, H), "matrix")
            out[p + "down"] = ((H, I), "matrix")
        return out

    register_lm_head("toy_biased_head", BiasedHead, replace=True)
    register_architecture("ToyCappedForCausalLM", lambda d: d, describe, kinds)
    register_architecture("ToyBiasedHeadForCausalLM", lambda d: d, describe, kinds)


def plain(cfg, w, toks):
    n = len(toks)
    nh, nkv, d, eps = (cfg[k] for k in ("num_attention_heads", "num_key_value_heads", "head_dim", "rms_norm_eps"))
    x = P.embedding(torch.tensor(toks), w["embed"]) * np.float32(math.sqrt(cfg["hidden_size"]))
    inv = P.inv_freqs({"head_dim": d, "rope_theta": cfg["rope_theta"]})
    cos, sin = P.rope_tables(inv, torch.arange(n))
    for i in range(cfg["num_hidden_layers"]):
        p = f"l{i}."
        h = P.rms_norm(x, w[p + "n1"], eps)
        q = P.apply_rope(P.linear(h, w[p + "q"]).view(n, nh, d), cos, sin)
        k = P.apply_rope(P.linear(h, w[p + "k"]).view(n, nkv, d), cos, sin)
        v = P.linear(h, w[p + "v"]).view(n, nkv, d)
        x = x + P.linear(P.causal_attention(q, k, v, 0).reshape(n, nh * d), w[p + "o"])
        h = P.rms_norm(x, w[p + "n2"], eps)
        x = x + P.linear(torch.nn.functional.silu(P.linear(h, w[p + "gate"])) * P.linear(h, w[p + "up"]), w[p + "down"])
    logits = P.linear(P.rms_norm(x, w["final"], eps), w["embed"])
    if cfg["own_head"]:
        return logits + w["head_bias"]
    cap = cfg["final_logit_cap"]
    return cap * torch.tanh(logits * cfg["logit_scale"] / cap)


@pytest.mark.parametrize("cfg,name", [(CFG, "toy_capped"), (CFG_OWN, "toy_biased_head")])
def test_scaled_embedding_and_capped_logits_in_every_cutting(model_root, cfg, name):
    register()
    from rust_llm_inference_server_b200 import ops
    from rust_llm_inference_server_b200.engine.replay import ReplaySession
    from rust_llm_inference_server_b200.weights import write_random_model
    from safetensors.torch import load_file
    d = os.path.join(model_root, name)
    if not os.path.isdir(d):
        write_random_model(cfg, d, seed=44)
    w = {k: v.float() for k, v in load_file(os.path.join(d, "model.safetensors")).items()}
    rng = np.random.default_rng(12)
    reqs = {f"c{i}": rng.integers(0, cfg["vocab_size"], size=n).tolist() for i, n in enumerate([90, 41, 7, 130])}
    ref = {k: plain(cfg, w, v).numpy() for k, v in reqs.items()}
    if not cfg["own_head"]:
        flat = np.abs(np.concatenate([r.ravel() for r in ref.values()]))
        assert flat.max() < cfg["final_logit_cap"] and (flat > 0.8 * cfg["final_logit_cap"]).mean() > 0.01   # the cap bites
    for dtype, tol in (("float32", 2e-4), ("bfloat16", 6e-2)):
        ops.launches_by_kernel.clear()
        whole = None
        for fam, steps in (("whole", R.whole_trace(reqs)), ("decode", R.decode_trace(reqs, tail=32)),
                           ("chunks", R.chunk_trace(reqs, seed=5)), ("mixed", R.mixed_trace(reqs, seed=6))):
            s = ReplaySession(d, dtype, R.live_token_peak(steps))
            assert s.model.graph_safe
            got = R.collect(s.step, steps)
            worst = max(float(np.abs(v - ref[k[0]][k[1]]).max()) for k, v in got.items())
            assert worst <= tol, (dtype, fam, worst)
            if whole is None:
                whole = got
            elif dtype == "float32":
                assert max(float(np.abs(v - whole[k]).max()) for k, v in got.items()) <= 2e-5, fam
            assert s.cache.num_free_pages(0) == s.cache.group(0).num_pages
        assert bool(ops.launches_by_kernel.get("logit_transform")) == (not cfg["own_head"])
