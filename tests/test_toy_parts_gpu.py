"""The framework's generality, shown with toy parts that live in this test only: a mixer with
per-request state of its own, a run order that names a layer twice and lets a call read another
call's cache, all registered, built from a model folder and stepped without a change to the
framework's files.  The toy is no model of anyone's."""

import json
import os
from dataclasses import dataclass

import numpy as np
import pytest
import torch

from tests import replay_util as R
from tests.plain import llama_plain as P

pytestmark = pytest.mark.gpu

TOY_CONFIG = {
    "architectures": ["ToyStateForCausalLM"], "vocab_size": 211, "hidden_size": 48, "intermediate_size": 80,
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 16, "rms_norm_eps": 2e-5,
    "rope_theta": 1000.0, "max_position_embeddings": 512,
}


@dataclass(frozen=True)
class RunningMeanSpec:
    hidden: int
    weight: str
    kind: str = "toy_running_mean"


def register_toy():
    from rust_llm_inference_server_b200 import ops
    from rust_llm_inference_server_b200.config import register_architecture, registered_architectures
    from rust_llm_inference_server_b200.parts import (GQAAttentionSpec, LayerCall, LayerSpec, Mixer, ModelSpec,
                                                      RMSNormSpec, RopeSpec, StateSpec, SwiGLUSpec, register_mixer)

    class RunningMean(Mixer):
        """out[t] = W . mean(x[0..t]).  The running sum is the per-request state: it carries over
        the portions of a prompt and over decoded tokens, and starts again when a request starts."""

        def __init__(self, spec, dtype, device):
            self.spec, self.dtype = spec, dtype

        def tensors(self):
            return {self.spec.weight: (self.spec.hidden, self.spec.hidden)}

        def load(self, src):
            self.w = src.get(self.spec.weight).contiguous()

        def state_spec(self):
            return StateSpec((self.spec.hidden,), torch.float32)

        def forward(self, x, step, cache, state, writes_cache=True):
            assert cache is None and state is not None
            out = torch.empty_like(x)
            for b in range(step.n_seqs):
                lo, n, start, slot = step.q_starts[b], step.q_lens[b], step.starts[b], step.state_slot_ids[b]
                assert slot >= 0
                if start == 0:
                    state[slot].zero_()
                cs = state[slot] + torch.cumsum(x[lo:lo + n].float(), dim=0)
                state[slot].copy_(cs[-1])
                pos = torch.arange(start, start + n, device=x.device, dtype=torch.float32)
                out[lo:lo + n] = (cs / (pos + 1)[:, None]).to(self.dtype)
            return ops.linear(out.contiguous(), self.w)

    def describe(cfg: dict) -> ModelSpec:
        H = cfg["hidden_size"]
        att = lambda p: GQAAttentionSpec(H, cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                                         p + "q", p + "k", p + "v", p + "o",
                                         position=RopeSpec(cfg["head_dim"], cfg["rope_theta"], None))
        norm = lambda n: RMSNormSpec(H, cfg["rms_norm_eps"], n)
        ffn = lambda p: SwiGLUSpec(H, cfg["intermediate_size"], p + "gate", p + "up", p + "down")
        layers = (
            LayerSpec(norm("l0.n1"), att("l0.att."), norm("l0.n2"), ffn("l0.ffn.")),
            LayerSpec(norm("l1.n1"), RunningMeanSpec(H, "l1.mix.w"), norm("l1.n2"), ffn("l1.ffn.")),
            LayerSpec(norm("l2.n1"), att("l2.att."), norm("l2.n2"), ffn("l2.ffn.")),
        )
        # layer 0 runs twice (each call with a cache of its own), the state mixer runs twice (two
        # states), and layer 2 reads the keys and values that the first call of layer 0 stored
        order = (LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 2), LayerCall(1, 3), LayerCall(2, 0, writes_cache=False))
        return ModelSpec(cfg["vocab_size"], H, "embed", layers, order, norm("final"), "head",
                         cfg["max_position_embeddings"])

    def tensor_kinds(cfg: dict) -> dict:
        H, I, nh, nkv, d = (cfg[k] for k in ("hidden_size", "intermediate_size", "num_attention_heads",
                                             "num_key_value_heads", "head_dim"))
        out = {"embed": ((cfg["vocab_size"], H), "matrix"), "head": ((cfg["vocab_size"], H), "matrix"),
               "final": ((H,), "norm"), "l1.mix.w": ((H, H), "matrix")}
        for l in (0, 1, 2):
            out[f"l{l}.n1"] = out[f"l{l}.n2"] = ((H,), "norm")
            out[f"l{l}.ffn.gate"] = out[f"l{l}.ffn.up"] = ((I, H), "matrix")
            out[f"l{l}.ffn.down"] = ((H, I), "matrix")
        for l in (0, 2):
            out[f"l{l}.att.q"] = ((nh * d, H), "matrix")
            out[f"l{l}.att.k"] = out[f"l{l}.att.v"] = ((nkv * d, H), "matrix")
            out[f"l{l}.att.o"] = ((H, nh * d), "matrix")
        return out

    if "ToyStateForCausalLM" not in registered_architectures():
        register_mixer("toy_running_mean", RunningMean, replace=True)
        register_architecture("ToyStateForCausalLM", lambda d: d, describe, tensor_kinds)


def plain_toy(w, cfg, toks):
    """The toy model on a whole sequence with the plain functions."""
    H, nh, nkv, d, eps = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["rms_norm_eps"]
    n = len(toks)
    x = P.embedding(torch.tensor(toks), w["embed"])
    cos, sin = P.rope_tables(P.inv_freqs(cfg), torch.arange(n))

    def ffn(x, l):
        h = P.rms_norm(x, w[f"l{l}.n2"], eps)
        return x + P.linear(torch.nn.functional.silu(P.linear(h, w[f"l{l}.ffn.gate"])) * P.linear(h, w[f"l{l}.ffn.up"]),
                            w[f"l{l}.ffn.down"])

    def qkv(h, l):
        q = P.apply_rope(P.linear(h, w[f"l{l}.att.q"]).view(n, nh, d), cos, sin)
        k = P.apply_rope(P.linear(h, w[f"l{l}.att.k"]).view(n, nkv, d), cos, sin)
        return q, k, P.linear(h, w[f"l{l}.att.v"]).view(n, nkv, d)

    def att(x, l, kv=None):
        h = P.rms_norm(x, w[f"l{l}.n1"], eps)
        q, k, v = qkv(h, l)
        if kv is not None:
            k, v = kv
        o = P.causal_attention(q, k, v).reshape(n, nh * d)
        return ffn(x + P.linear(o, w[f"l{l}.att.o"]), l), (k, v)

    def mean(x, l):
        h = P.rms_norm(x, w[f"l{l}.n1"], eps)
        m = torch.cumsum(h, 0) / torch.arange(1, n + 1)[:, None]
        return ffn(x + P.linear(m, w[f"l{l}.mix.w"]), l)

    x, kv0 = att(x, 0)
    x = mean(x, 1)
    x, _ = att(x, 0)
    x = mean(x, 1)
    x, _ = att(x, 2, kv=kv0)
    return P.linear(P.rms_norm(x, w["final"], eps), w["head"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_toy_architecture_with_state_is_registered_built_and_stepped(model_root, dtype):
    register_toy()
    from rust_llm_inference_server_b200.engine.replay import ReplaySession
    from rust_llm_inference_server_b200.weights import write_random_model
    from safetensors.torch import load_file
    d = os.path.join(model_root, "toy_state")
    if not os.path.isdir(d):
        write_random_model(TOY_CONFIG, d, seed=11)
    w = {k: v.float() for k, v in load_file(os.path.join(d, "model.safetensors")).items()}
    rng = np.random.default_rng(2)
    reqs = {f"t{i}": rng.integers(0, 211, size=n).tolist() for i, n in enumerate([40, 9, 77, 130, 3])}
    ref = {k: plain_toy(w, TOY_CONFIG, v).numpy() for k, v in reqs.items()}
    tol = 1e-4 if dtype == "float32" else 3e-2
    for fam, steps in (("whole", R.whole_trace(reqs)), ("decode", R.decode_trace(reqs, tail=12)),
                       ("chunks", R.chunk_trace(reqs, seed=1)), ("mixed", R.mixed_trace(reqs, seed=2))):
        s = ReplaySession(d, dtype, R.live_token_peak(steps))
        assert len(s.storage.groups) == 1 and s.storage.groups[0].slots == [0, 2]      # two attention caches
        assert [x is not None for x in s.storage.states] == [False, True, False, True, False]  # two states
        got = R.collect(s.step, steps)
        worst = max(float(np.abs(v - ref[k[0]][k[1]]).max()) for k, v in got.items())
        assert worst <= tol, (fam, worst)
        assert s.cache.check_invariants() == "" and s.cache.num_free_state_slots() == s.cache.num_state_slots()


def test_generation_with_the_toy_goes_through_the_scheduler(model_root):
    """State slots are taken at admission and come back; preemption restarts the state."""
    register_toy()
    from rust_llm_inference_server_b200 import LLM, SamplingParams
    from rust_llm_inference_server_b200.weights import write_random_model
    from safetensors.torch import load_file
    d = os.path.join(model_root, "toy_state")
    if not os.path.isdir(d):
        write_random_model(TOY_CONFIG, d, seed=11)
    w = {k: v.float() for k, v in load_file(os.path.join(d, "model.safetensors")).items()}
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, 211, size=n).tolist() for n in (5, 30, 12, 21)]
    want = []
    for p in prompts:
        t = list(p)
        for _ in range(10):
            t.append(int(np.argmax(plain_toy(w, TOY_CONFIG, t)[-1].numpy())))
        want.append(t[len(p):])
    roomy = LLM(d, dtype="float32", max_seq_len=64, num_blocks=32, block_size=8, max_num_seqs=4, max_batched_tokens=16)
    assert not roomy.engine.sched.config().prefix_caching    # state cannot be skipped over
    assert [o.token_ids for o in roomy.generate(prompts, SamplingParams(max_tokens=10))] == want
    tight = LLM(d, dtype="float32", max_seq_len=48, num_blocks=9, block_size=8, max_num_seqs=4, max_batched_tokens=16)
    assert [o.token_ids for o in tight.generate(prompts, SamplingParams(max_tokens=10))] == want
    assert tight.engine.stats.preemptions > 0
    assert tight.engine.cache.num_free_state_slots() == 4 and tight.engine.sched.check() == ""
