"""Generation through the Python entry point on the GPU: greedy tokens equal the plain
implementation's; batching, portions, preemption and prefix reuse change nothing; sampling is
reproducible and does not depend on the batch."""

import numpy as np
import pytest

from tests.plain import llama_plain as P
from tests.tiny_configs import CONFIGS, load_plain_weights, make_model_dir

pytestmark = pytest.mark.gpu


def prompts_for(which, lens, seed=1):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, CONFIGS[which]["vocab_size"], size=n).tolist() for n in lens]


def same_or_near_tie(which, w, prompt, got, want, dtype):
    """float32: the same tokens.  bfloat16: the reference's rule (crates/model/tests/parity.rs:30-35):
    sequences may part only where the float32 logits of the two candidates are within 0.02."""
    if got == want:
        return True
    if dtype == "float32":
        return False
    i = next(k for k, (a, b) in enumerate(zip(got, want)) if a != b)
    lg = P.forward_logits(w, CONFIGS[which], prompt + want[:i])[-1].numpy()
    return abs(float(lg[got[i]]) - float(lg[want[i]])) < 0.02 and lg[want[i]] >= np.sort(lg)[-2] - 1e-6


def make_llm(model_root, which, dtype, **kw):
    from rust_llm_inference_server_b200 import LLM
    opts = dict(max_seq_len=128, num_blocks=64, block_size=8, max_num_seqs=4, max_batched_tokens=2048)
    opts.update(kw)
    return LLM(make_model_dir(model_root, which), dtype=dtype, **opts)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_equals_the_plain_implementation(model_root, dtype):
    """Tiny configuration A of the workload: prompts of 1, 7, 13 and 32 tokens, 16 greedy tokens."""
    from rust_llm_inference_server_b200 import SamplingParams
    w = load_plain_weights(make_model_dir(model_root, "A"))
    prompts = prompts_for("A", [1, 7, 13, 32])
    llm = make_llm(model_root, "A", dtype)
    outs = llm.generate(prompts, SamplingParams(max_tokens=16))
    for p, o in zip(prompts, outs):
        want = P.greedy_generate(w, CONFIGS["A"], p, 16)
        if dtype == "float32":
            assert o.token_ids == want
        else:
            # a flip is tolerated only at a near tie of the float32 logits
            # (the reference's rule, crates/model/tests/parity.rs:30-35)
            for i, (a, b) in enumerate(zip(o.token_ids, want)):
                if a != b:
                    lg = np.sort(P.forward_logits(w, CONFIGS["A"], p + want[:i])[-1].numpy())
                    assert lg[-1] - lg[-2] < 0.02
                    break
        assert o.finish_reason == "length" and len(o.token_ids) == 16 and o.prompt_token_ids == p


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batching_portions_preemption_and_prefix_reuse_change_nothing(model_root, dtype):
    from rust_llm_inference_server_b200 import SamplingParams
    which = "B"
    shared = prompts_for(which, [48], seed=5)[0]
    prompts = prompts_for(which, [3, 60, 21, 90]) + [shared + [7, 8, 9], shared + [11] * 20]
    sp = SamplingParams(max_tokens=24)
    base = make_llm(model_root, which, dtype, max_seq_len=256, num_blocks=64, block_size=16, max_num_seqs=1,
                    prefix_caching=False)
    solo = [base.generate([p], sp)[0].token_ids for p in prompts]
    w = load_plain_weights(make_model_dir(model_root, which))

    solo_tokens = solo

    class Same:
        """`outputs == solo` under the rule of `same_or_near_tie`."""
        def __eq__(self, outs):
            return all(same_or_near_tie(which, w, p, o, s, dtype) for p, o, s in zip(prompts, outs, solo_tokens))
    solo = Same()

    batched = make_llm(model_root, which, dtype, max_seq_len=256, num_blocks=64, block_size=16, max_num_seqs=6,
                       prefix_caching=False)
    assert solo == [o.token_ids for o in batched.generate(prompts, sp)]

    cut = make_llm(model_root, which, dtype, max_seq_len=256, num_blocks=64, block_size=16, max_num_seqs=4,
                   max_batched_tokens=16, prefix_caching=False)
    assert solo == [o.token_ids for o in cut.generate(prompts, sp)]

    tight = make_llm(model_root, which, dtype, max_seq_len=256, num_blocks=12, block_size=16, max_num_seqs=6,
                     prefix_caching=True)
    assert solo == [o.token_ids for o in tight.generate(prompts, sp)]
    assert tight.engine.stats.preemptions > 0
    assert tight.engine.sched.check() == "" and tight.engine.cache.num_free_pages(0) == 12

    for seats in (1, 2):
        pc = make_llm(model_root, which, dtype, max_seq_len=256, num_blocks=64, block_size=16,
                      max_num_seqs=seats, prefix_caching=True)
        assert solo == [o.token_ids for o in pc.generate(prompts, sp)]
        if seats == 1:   # one after the other: the second holder of the prefix finds its three full pages
            assert pc.engine.stats.prefix_hit_tokens >= 48
        assert solo == [o.token_ids for o in pc.generate(prompts, sp)]      # now everything is cached
        full_pages = sum((len(p) - 1) // 16 * 16 for p in prompts)   # never the page of the last token
        assert pc.engine.stats.prefix_hit_tokens >= full_pages + (48 if seats == 1 else 0)

    static = make_llm(model_root, which, dtype, max_seq_len=256, num_blocks=64, block_size=16, max_num_seqs=3,
                      scheduler="static")
    assert solo == [o.token_ids for o in static.generate(prompts, sp)]


def test_seeded_sampling_is_reproducible_and_ignores_neighbours(model_root):
    from rust_llm_inference_server_b200 import SamplingParams
    which = "B"
    prompts = prompts_for(which, [5, 40, 17, 9])
    llm = make_llm(model_root, which, "float32", max_seq_len=256, block_size=16)
    w = load_plain_weights(make_model_dir(model_root, which))
    for sp in (SamplingParams(max_tokens=12, temperature=0.8, seed=3),
               SamplingParams(max_tokens=12, temperature=0.8, top_p=0.9, seed=3),
               SamplingParams(max_tokens=12, temperature=1.1, top_k=20, repetition_penalty=1.2, seed=3)):
        a = [o.token_ids for o in llm.generate(prompts, sp)]
        b = [llm.generate([p], sp)[0].token_ids for p in prompts]
        assert a == b
        sp2 = SamplingParams(**{**sp.__dict__, "seed": 4})
        assert [o.token_ids for o in llm.generate(prompts, sp2)] != a
    # temperature-only rows are drawn on the device with the reference's noise: replay with the plain sampler
    sp = SamplingParams(max_tokens=6, temperature=0.8, seed=3)
    got = llm.generate([prompts[0]], sp)[0].token_ids
    toks = list(prompts[0])
    for t in got:
        lg = P.forward_logits(w, CONFIGS[which], toks)[-1].numpy()
        assert P.sample_row(lg, 0.8, P.row_key(3, len(toks))) == t
        toks.append(t)
    # top-k / top-p rows are filtered and drawn on the device: replay with the plain rule
    sp = SamplingParams(max_tokens=6, temperature=0.9, top_k=12, top_p=0.85, seed=11)
    got = llm.generate([prompts[1]], sp)[0].token_ids
    toks = list(prompts[1])
    for t in got:
        lg = P.forward_logits(w, CONFIGS[which], toks)[-1].numpy()
        assert P.filtered_sample(lg, 0.9, 12, 0.85, P.uniform_53(11, len(toks))) == t
        toks.append(t)
    # a repetition penalty changes the logits on the device before either sampler: greedy and filtered
    # rows with a penalty, in one batch with a row that has none, replayed with the plain rules
    sps = [SamplingParams(max_tokens=10, repetition_penalty=1.8),
           SamplingParams(max_tokens=10, temperature=0.9, top_k=12, top_p=0.85, repetition_penalty=1.5, seed=11),
           SamplingParams(max_tokens=10)]
    outs = llm.generate(prompts[:3], sps)
    assert outs[2].token_ids == llm.generate([prompts[2]], sps[2])[0].token_ids
    assert outs[0].token_ids != llm.generate([prompts[0]], sps[2])[0].token_ids      # the penalty shows
    for p, sp, o in zip(prompts[:2], sps[:2], outs[:2]):
        toks = list(p)
        for t in o.token_ids:
            lg = P.forward_logits(w, CONFIGS[which], toks)[-1].numpy()
            lg = P.apply_repetition_penalty(lg, toks, sp.repetition_penalty)
            want = int(np.argmax(lg)) if sp.temperature == 0 else \
                P.filtered_sample(lg, sp.temperature, sp.top_k, sp.top_p, P.uniform_53(sp.seed, len(toks)))
            assert want == t
            toks.append(t)


def test_end_of_sequence_and_limits(model_root, tmp_path):
    import json, os, shutil
    from rust_llm_inference_server_b200 import LLM, SamplingParams
    from rust_llm_inference_server_b200.engine.engine import RequestError
    src = make_model_dir(model_root, "A")
    w = load_plain_weights(src)
    p = prompts_for("A", [9])[0]
    want = P.greedy_generate(w, CONFIGS["A"], p, 10)
    eos = want[4]
    d = str(tmp_path / "with_eos")
    shutil.copytree(src, d)
    cfg = json.load(open(os.path.join(d, "config.json")))
    cfg["eos_token_id"] = eos
    json.dump(cfg, open(os.path.join(d, "config.json"), "w"))
    llm = LLM(d, dtype="float32", max_seq_len=64, num_blocks=16, block_size=8, max_num_seqs=2)
    o = llm.generate([p], SamplingParams(max_tokens=10))[0]
    first = want.index(eos)
    assert o.finish_reason == "stop" and o.token_ids == want[:first]     # the end token is not appended
    o = llm.generate([p], SamplingParams(max_tokens=10, ignore_eos=True))[0]
    assert o.finish_reason == "length" and o.token_ids == want
    with pytest.raises(RequestError, match="exceeds max_seq_len"):
        llm.generate([p], SamplingParams(max_tokens=60))
    with pytest.raises(RequestError):
        llm.generate([[]], SamplingParams())
    with pytest.raises(RequestError, match="vocabulary"):
        llm.generate([[1, 999]], SamplingParams())
    assert llm.engine.cache.num_free_pages(0) == 16


def test_decode_ahead_changes_no_token(model_root, tmp_path):
    """The loop that launches a step before the one before it has been read gives the tokens,
    finish reasons and order of events of the step-by-step loop: greedy and seeded sampling,
    requests of different lengths (so that the batch shrinks), an end-of-sequence token that
    arrives while the next step is already in flight, a cancelled request, and requests that
    arrive while others decode."""
    import json, os, shutil
    from rust_llm_inference_server_b200 import LLM, SamplingParams
    src = make_model_dir(model_root, "B")
    w = load_plain_weights(src)
    prompts = prompts_for("B", [5, 19, 9, 33], seed=4)
    # an end-of-sequence token that the first request meets after a few tokens
    greedy = P.greedy_generate(w, CONFIGS["B"], prompts[0], 12)
    eos = next(t for i, t in enumerate(greedy) if i >= 3 and t not in greedy[:i])     # first met after a few tokens
    d = str(tmp_path / "with_eos")
    shutil.copytree(src, d)
    cfg = json.load(open(os.path.join(d, "config.json")))
    cfg["eos_token_id"] = int(eos)
    json.dump(cfg, open(os.path.join(d, "config.json"), "w"))
    opts = dict(dtype="float32", max_seq_len=128, num_blocks=64, block_size=8, max_num_seqs=4)
    runs = {}
    for ahead in (False, True):
        llm = LLM(d, decode_ahead=ahead, **opts)
        sps = [SamplingParams(max_tokens=20), SamplingParams(max_tokens=7, ignore_eos=True),
               SamplingParams(max_tokens=25, temperature=0.8, seed=5, ignore_eos=True),
               SamplingParams(max_tokens=16, temperature=1.0, top_k=9, top_p=0.9, seed=6, ignore_eos=True)]
        outs = llm.generate(prompts, sps)
        runs[ahead] = [(o.token_ids, o.finish_reason) for o in outs]
        # the stream of events: a request joins while the others decode, another is cancelled
        eng = llm.engine
        a = eng.add_request(prompts[1], SamplingParams(max_tokens=12, ignore_eos=True))
        b = eng.add_request(prompts[2], SamplingParams(max_tokens=30, ignore_eos=True))
        seen, done, step = {a: [], b: []}, {}, 0
        c = None
        while eng.has_work():
            for o in eng.step():
                done[o.request_id] = (o.token_ids, o.finish_reason)
            for rid, t in eng.last_step.new_tokens.items():
                seen.setdefault(rid, []).append(t)
            step += 1
            if step == 4:
                c = eng.add_request(prompts[3], SamplingParams(max_tokens=6, ignore_eos=True))
            if step == 9:
                eng.cancel(b)
        assert b not in done and done[a][0] == seen[a] and done[c][0] == seen[c] and len(seen[c]) == 6
        runs[ahead].append((done[a], done[c], seen[b][:8]))
        assert eng.sched.check() == "" and eng.sched.num_running() == 0
        if ahead:
            assert llm.engine._decode_ahead
    assert runs[True] == runs[False]
    assert runs[True][0] == (greedy[:greedy.index(eos)], "stop")           # ended by the end-of-sequence token
