"""The plain implementation itself: anchors that the reference states as numbers or as facts, and
consistency of its parts."""

import math

import numpy as np
import torch

from tests.plain import llama_plain as P

# crates/model/src/rope.rs:147-156: inverse frequencies of the Llama 3.2 1B configuration
# (theta 500000, head size 64, llama3 scaling 32 / 1 / 4 / 8192), as that file's test states them.
LLAMA32_INV_FREQ = [
    1.000000000e+00, 6.636012793e-01, 4.403666258e-01, 2.922278345e-01,
    1.939227581e-01, 1.286873817e-01, 8.539710194e-02, 5.666961893e-02,
    3.760603070e-02, 2.495540865e-02, 1.656044088e-02, 1.098952908e-02,
    7.292665076e-03, 4.839421250e-03, 3.211446106e-03, 1.290548011e-03,
    4.295567051e-04, 9.708286234e-05, 1.946163866e-05, 1.291476747e-05,
    8.570255886e-06, 5.687232260e-06, 3.774054449e-06, 2.504467147e-06,
    1.661967417e-06, 1.102883630e-06, 7.318749340e-07, 4.856731266e-07,
    3.222932889e-07, 2.138742303e-07, 1.419272024e-07, 9.418306490e-08,
]

CFG_1B = {
    "hidden_size": 2048, "intermediate_size": 8192, "num_hidden_layers": 16,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "vocab_size": 128256,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "max_position_embeddings": 131072,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
}


def test_llama3_inverse_frequencies_match_the_reference_constants():
    got = P.inv_freqs(CFG_1B).numpy()
    assert got.shape == (32,)
    rel = np.abs(got - np.array(LLAMA32_INV_FREQ)) / np.array(LLAMA32_INV_FREQ)
    assert rel.max() < 1e-6


def test_unscaled_frequencies_and_unknown_scaling_type():
    cfg = dict(CFG_1B, rope_scaling=None)
    base = P.inv_freqs(cfg).numpy()
    assert np.allclose(base, 500000.0 ** (-np.arange(0, 64, 2) / 64), rtol=1e-6)
    other = P.inv_freqs(dict(CFG_1B, rope_scaling={"rope_type": "linear", "factor": 4.0})).numpy()
    assert np.array_equal(base, other)   # only "llama3" is scaled (rope.rs:26)


def test_rope_rotates_pairs_of_halves_and_keeps_norms():
    x = torch.randn(5, 3, 16)
    cos, sin = P.rope_tables(P.inv_freqs({"head_dim": 16, "rope_theta": 10000.0,
                                          "hidden_size": 48, "num_attention_heads": 3}),
                             torch.arange(5))
    y = P.apply_rope(x, cos, sin)
    assert torch.allclose(y[0], x[0])            # position 0: no rotation
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    j = 3
    want = x[2, 1, j] * cos[2, j] - x[2, 1, j + 8] * sin[2, j]
    assert torch.allclose(y[2, 1, j], want)


def test_grouped_attention_equals_repeated_kv_textbook():
    torch.manual_seed(0)
    q, k, v = torch.randn(6, 4, 8), torch.randn(9, 2, 8), torch.randn(9, 2, 8)
    got = P.causal_attention(q, k, v, start_pos=3)
    for h in range(4):
        kv = h // 2
        for i in range(6):
            r = 3 + i
            s = (k[: r + 1, kv] @ q[i, h]) / math.sqrt(8)
            p = torch.softmax(s, 0)
            assert torch.allclose(got[i, h], p @ v[: r + 1, kv], atol=1e-5)


def test_window_hides_old_keys():
    torch.manual_seed(1)
    q, k, v = torch.randn(4, 1, 8), torch.randn(4, 1, 8), torch.randn(4, 1, 8)
    got = P.causal_attention(q, k, v, 0, window=2)
    s = (k[2:4, 0] @ q[3, 0]) / math.sqrt(8)
    assert torch.allclose(got[3, 0], torch.softmax(s, 0) @ v[2:4, 0], atol=1e-5)


def test_rms_norm_uses_eps_as_float32_and_weight_directly():
    x = torch.tensor([[3.0, 4.0]])
    w = torch.tensor([2.0, 0.5])
    got = P.rms_norm(x, w, 1e-5)
    rms = math.sqrt((9 + 16) / 2 + float(np.float32(1e-5)))
    assert torch.allclose(got, torch.tensor([[3 / rms * 2, 4 / rms * 0.5]]), atol=1e-6)


def test_tied_default_is_false():
    w = {"model.embed_tokens.weight": torch.zeros(2, 2), "lm_head.weight": torch.ones(2, 2)}
    assert P.lm_head_weight(w, {}) is w["lm_head.weight"]
    assert P.lm_head_weight(w, {"tie_word_embeddings": True}) is w["model.embed_tokens.weight"]


# ---- sampler facts stated by the reference ----

def test_hash_constants_and_uniform_range():
    assert P.lowbias32(0) == 0
    # the 23-bit rule: the largest and smallest hashes stay strictly inside (0, 1)
    # (crates/model/src/sampling.rs:58-63,198-205)
    for h in (0, 1, 0xFFFFFFFF, 0xFFFFFE00, 0x1FF):
        u = float(P.uniform(h))
        assert 0.0 < u < 1.0
    hs = np.arange(0, 1 << 23, 4099, dtype=np.uint64) << 9
    us = ((hs >> 9).astype(np.float32) + np.float32(0.5)) * np.float32(1 / 8388608.0)
    assert us.min() > 0 and us.max() < 1


def test_greedy_ties_go_to_the_lowest_id():
    # crates/model/src/sampling.rs:185-195 and crates/engine/src/sampler.rs:279-282
    assert P.sample_row([1.0, 3.0, 3.0, 2.0], 0.0, 0) == 1
    assert P.sample_row([5.0, 5.0], 0.0, 0) == 0
    assert P.argmax([2.0, 7.0, 7.0]) == 1


def test_repetition_penalty_values():
    # crates/engine/src/sampler.rs:402-406: [2, -2, 1] with tokens 0 and 1 seen, penalty 2
    out = P.apply_repetition_penalty(np.array([2.0, -2.0, 1.0]), [0, 1, 1], 2.0)
    assert out.tolist() == [1.0, -4.0, 1.0]


def test_gumbel_max_frequencies_follow_the_softmax():
    logits = np.array([0.0, 1.0, 2.0, -1.0], dtype=np.float32)
    T = 0.7
    counts = np.zeros(4)
    for i in range(4000):
        counts[P.sample_row(logits, T, P.row_key(1234, i))] += 1
    want = np.exp(logits / T) / np.exp(logits / T).sum()
    assert np.abs(counts / counts.sum() - want).max() < 0.03


def test_filtered_distribution_top_k_and_top_p():
    logits = np.log(np.array([0.5, 0.25, 0.15, 0.1], dtype=np.float32))
    p = P.filtered_distribution(logits, 1.0, 0, 0.7)      # 0.5 + 0.25 crosses 0.7
    assert np.allclose(p, [2 / 3, 1 / 3, 0, 0], atol=1e-6)
    p = P.filtered_distribution(logits, 1.0, 3, 1.0)
    assert p[3] == 0 and np.isclose(p.sum(), 1)
    p = P.filtered_distribution(logits, 1.0, 1, 1.0)
    assert p.tolist() == [1, 0, 0, 0]


def test_whole_model_is_causal(model_root):
    from tests.tiny_configs import TINY_A, load_plain_weights, make_model_dir
    w = load_plain_weights(make_model_dir(model_root, "A"))
    toks = list(range(3, 23))
    full = P.forward_logits(w, TINY_A, toks)
    part = P.forward_logits(w, TINY_A, toks[:11])
    assert torch.allclose(full[:11], part, atol=1e-5)
