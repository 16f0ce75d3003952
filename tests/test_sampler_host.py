"""The host sampler and the device sampler's key (no GPU): facts the reference states
(crates/engine/src/sampler.rs:264-407) checked against the plain implementation."""

import numpy as np

from rust_llm_inference_server_b200.sampling import Sampler, SamplingParams, lowbias32, row_key, unit_uniform
from tests.plain import llama_plain as P


def test_hashes_equal_the_plain_implementation():
    for x in (0, 1, 12345, 0xFFFFFFFF, 0x9E3779B9):
        assert lowbias32(x) == P.lowbias32(x)
    for seed, pos in ((0, 0), (5, 17), (2 ** 40 + 3, 9), (2 ** 64 - 1, 2 ** 31)):
        assert row_key(seed, pos) == P.row_key(seed, pos)
    us = [unit_uniform(7, i) for i in range(2000)]
    assert 0 <= min(us) and max(us) < 1 and abs(np.mean(us) - 0.5) < 0.03
    assert unit_uniform(7, 3) == unit_uniform(7, 3) != unit_uniform(8, 3)


def test_modes():
    assert Sampler(SamplingParams()).device_mode(5) == (0, 0)
    k, bits = Sampler(SamplingParams(temperature=0.5, seed=9)).device_mode(5)
    assert k == P.row_key(9, 5) and bits == int(np.float32(2.0).view(np.uint32))
    assert Sampler(SamplingParams(temperature=0.5, top_p=0.9)).device_mode(0) is None
    assert Sampler(SamplingParams(temperature=0.5, top_k=3)).device_mode(0) is None
    # a repetition penalty changes the logits on the device first, not the way of drawing
    assert Sampler(SamplingParams(repetition_penalty=1.1)).device_mode(0) == (0, 0)
    assert Sampler(SamplingParams(temperature=0.5, top_k=3, repetition_penalty=1.1)).filtered_mode(0) is not None
    assert Sampler(SamplingParams(top_p=0.5)).device_mode(0) == (0, 0)   # greedy ignores filters


def test_greedy_ties_penalty_and_top_k_one():
    s = Sampler(SamplingParams(top_k=4, top_p=0.3))
    assert s.sample_host(np.array([1, 3, 3, 2], np.float32), [], 0) == 1
    s = Sampler(SamplingParams(repetition_penalty=2.0))
    assert s.sample_host(np.array([2.0, 1.5, -1.0], np.float32), [0, 0, 2], 0) == 1
    s = Sampler(SamplingParams(temperature=1.0, top_k=1, seed=3))
    assert all(s.sample_host(np.array([0.1, 0.9, 0.5], np.float32), [], i) == 1 for i in range(50))


def check_distribution(params, logits, n=30000, tol=0.015):
    s = Sampler(params)
    counts = np.zeros(len(logits))
    for i in range(n):
        counts[s.sample_host(logits, [], i)] += 1
    want = P.filtered_distribution(logits, params.temperature, params.top_k, params.top_p)
    assert np.abs(counts / n - want).max() < tol
    assert set(np.nonzero(counts)[0]) <= set(np.nonzero(want)[0])


def test_every_mode_draws_from_the_filtered_softmax():
    rng = np.random.default_rng(0)
    logits = rng.normal(size=40).astype(np.float32) * 2
    check_distribution(SamplingParams(temperature=0.8, seed=1), logits)
    check_distribution(SamplingParams(temperature=1.3, top_k=5, seed=2), logits)
    check_distribution(SamplingParams(temperature=0.8, top_p=0.9, seed=3), logits)
    check_distribution(SamplingParams(temperature=1.0, top_k=12, top_p=0.6, seed=4), logits)
    # a nucleus wider than 64 candidates (the reference grows its candidate set, sampler.rs:167-170)
    flat = np.zeros(500, np.float32)
    check_distribution(SamplingParams(temperature=1.0, top_p=0.5, seed=5), flat, n=20000, tol=0.01)


def test_same_seed_same_tokens_other_seed_other_tokens():
    logits = np.linspace(-1, 1, 50).astype(np.float32)
    a = [Sampler(SamplingParams(temperature=1.0, top_p=0.95, seed=11)).sample_host(logits, [], i) for i in range(40)]
    b = [Sampler(SamplingParams(temperature=1.0, top_p=0.95, seed=11)).sample_host(logits, [], i) for i in range(40)]
    c = [Sampler(SamplingParams(temperature=1.0, top_p=0.95, seed=12)).sample_host(logits, [], i) for i in range(40)]
    assert a == b and a != c


def test_filtered_draw_equals_the_plain_rule_and_follows_the_filtered_softmax():
    from rust_llm_inference_server_b200.sampling import filtered_draw, unit_uniform_53
    rng = np.random.default_rng(1)
    for trial in range(30):
        n = int(rng.integers(5, 300))
        logits = (rng.normal(size=n) * rng.uniform(0.5, 4)).astype(np.float32)
        if trial % 5 == 0:
            logits[rng.integers(0, n, size=3)] = logits.max()          # exact ties at the top
        T, k, p = float(rng.uniform(0.3, 1.5)), int(rng.integers(0, n + 3)), float(rng.choice([1.0, 0.9, 0.5, 0.1]))
        if k == 0 and p >= 1.0:
            p = 0.9
        for pos in range(4):
            u = unit_uniform_53(trial, pos)
            assert u == P.uniform_53(trial, pos)
            want = P.filtered_sample(logits, T, k, p, u)
            got = filtered_draw(logits, np.float32(1.0) / np.float32(T), k, p, u)
            assert got == want, (trial, pos, n, T, k, p)
    logits = (rng.normal(size=40) * 2).astype(np.float32)
    for T, k, p in ((0.8, 0, 0.9), (1.3, 5, 1.0), (1.0, 12, 0.6)):
        counts = np.zeros(40)
        for i in range(20000):
            counts[filtered_draw(logits, np.float32(1.0) / np.float32(T), k, p, unit_uniform_53(99, i))] += 1
        want = P.filtered_distribution(logits, T, k, p)
        assert np.abs(counts / 20000 - want).max() < 0.015
