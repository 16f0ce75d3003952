"""A short soak of the engine loop (role of the reference's soak run, scripts/bench/soak.sh:
concurrency with hang-ups, every block returned): a few hundred random requests of every sampling
kind through a pool so small that requests are preempted, with a shared prefix, cancellations and
requests that arrive while others decode.  Nothing leaks, nothing fails, and in float32 a sample
of the requests gives the same tokens when run alone."""

import random

import pytest

from tests.tiny_configs import CONFIGS, make_model_dir

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("which,dtype,n", [("D", "bfloat16", 240), ("B", "float32", 160)])
def test_random_requests_through_a_tight_pool(model_root, which, dtype, n):
    from rust_llm_inference_server_b200 import LLM, SamplingParams, ops
    d = make_model_dir(model_root, which)
    V = CONFIGS[which]["vocab_size"]
    rng = random.Random(7)
    opts = dict(dtype=dtype, max_seq_len=240, num_blocks=32, block_size=16, max_batched_tokens=96)
    llm = LLM(d, max_num_seqs=8, prefix_caching=True, **opts)
    eng = llm.engine
    shared = [rng.randrange(V) for _ in range(48)]

    def make():
        p = [rng.randrange(V) for _ in range(rng.choice([1, 2, 5, 17, 33, 64, 100]))]
        if rng.random() < 0.3:
            p = shared + p[:40]
        kind, mt = rng.random(), rng.randint(1, 50)
        if kind < 0.4:
            return p, SamplingParams(max_tokens=mt)
        if kind < 0.6:
            return p, SamplingParams(max_tokens=mt, temperature=0.8, seed=rng.randrange(1000))
        if kind < 0.8:
            return p, SamplingParams(max_tokens=mt, temperature=1.0, top_k=rng.choice([0, 5, 40]),
                                     top_p=rng.choice([1.0, 0.9]), seed=rng.randrange(1000))
        return p, SamplingParams(max_tokens=min(mt, 30), temperature=0.7, repetition_penalty=1.3, seed=rng.randrange(1000))

    pending = [make() for _ in range(n)]
    live, done, asked, steps = {}, {}, {}, 0
    while pending or eng.has_work():
        while pending and len(live) < 20 and rng.random() < 0.7:
            p, sp = pending.pop()
            rid = eng.add_request(p, sp)
            live[rid] = asked[rid] = (p, sp)
        if not eng.has_work():
            continue
        for o in eng.step():
            done[o.request_id] = o
            live.pop(o.request_id, None)
        steps += 1
        if live and rng.random() < 0.01:                  # a client hangs up
            rid = rng.choice(sorted(live))
            eng.cancel(rid)
            live.pop(rid)
            asked.pop(rid)
        if steps % 100 == 0:
            assert eng.sched.check() == ""
    st = eng.stats
    assert eng.sched.check() == "" and eng.cache.num_free_pages(0) == 32 and eng.cache.num_free_state_slots() == 8
    assert st.failed_requests == 0 and st.preemptions > 0 and st.prefix_hit_tokens > 0
    assert set(done) == set(asked)
    assert all(o.finish_reason == "length" and len(o.token_ids) == asked[r][1].max_tokens for r, o in done.items())
    ops.check_device_errors()
    if dtype == "float32":
        solo = LLM(d, max_num_seqs=1, **opts)
        for rid in rng.sample(sorted(done), 25):
            p, sp = asked[rid]
            assert solo.generate([p], sp)[0].token_ids == done[rid].token_ids, rid
