"""The engine loop on the GPU where it is easiest to get wrong: pages that run out while every
request decodes (with and without decode-ahead), a step that fails, the kernels' error word, and
the timing records."""

import numpy as np
import pytest

from tests.plain import llama_plain as P
from tests.test_generate_gpu import make_llm, prompts_for, same_or_near_tie
from tests.tiny_configs import CONFIGS, load_plain_weights, make_model_dir

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("pool", [dict(num_blocks=5, block_size=8, lens=[8, 8], max_tokens=24),
                                  dict(num_blocks=4, block_size=16, lens=[16, 16], max_tokens=32)])
def test_pages_run_out_while_everybody_decodes(model_root, dtype, pool):
    """Admission reserves a request's known length only, so decoding requests take new pages, and
    with too few of them the newest request is preempted and recomputes later
    (crates/engine/src/scheduler.rs:227-246); greedy output is unchanged by it
    (crates/engine/tests/engine.rs, "preemption+recompute leaves greedy output unchanged").  Nobody
    is waiting when it happens, so the loop is in the middle of launching steps ahead."""
    from rust_llm_inference_server_b200 import SamplingParams
    which = "A"
    w = load_plain_weights(make_model_dir(model_root, which))
    prompts = prompts_for(which, pool["lens"], seed=7)
    sp = SamplingParams(max_tokens=pool["max_tokens"])
    opts = dict(max_seq_len=128, num_blocks=pool["num_blocks"], block_size=pool["block_size"], max_num_seqs=4)
    solo_llm = make_llm(model_root, which, dtype, **{**opts, "max_num_seqs": 1})
    solo = [solo_llm.generate([p], sp)[0].token_ids for p in prompts]
    for ahead, check_pages in ((False, True), (True, True), (True, False)):
        llm = make_llm(model_root, which, dtype, decode_ahead=ahead, **opts)
        llm.engine._ahead_checks_pages = check_pages
        outs = llm.generate(prompts, sp)
        for p, o, s in zip(prompts, outs, solo):
            assert o.finish_reason == "length" and len(o.token_ids) == pool["max_tokens"]
            assert same_or_near_tie(which, w, p, o.token_ids, s, dtype), (ahead, check_pages)
        st = llm.engine.stats
        assert st.preemptions > 0 and st.failed_requests == 0
        assert (st.ahead_fallbacks > 0) == (ahead and not check_pages)
        assert llm.engine.sched.check() == "" and llm.engine.cache.num_free_pages(0) == pool["num_blocks"]


def test_a_failed_step_fails_only_its_requests(model_root):
    """A step that raises ends the requests of that step with reason "error" and gives their pages
    back; requests that were not part of it are served as if nothing had happened
    (crates/engine/src/engine.rs:516-528).  The failure is made on the host: the launch of one
    chosen step raises before anything reaches the GPU."""
    from rust_llm_inference_server_b200 import SamplingParams, ops
    which = "A"
    prompts = prompts_for(which, [9, 14, 6, 11], seed=3)
    sp = SamplingParams(max_tokens=12)
    for ahead in (False, True):
        llm = make_llm(model_root, which, "float32", max_num_seqs=2, decode_ahead=ahead)
        want = [o.token_ids for o in llm.generate(prompts, sp)]
        eng = llm.engine
        real, calls = eng.runner.forward, {"n": 0}

        def failing(st, real=real, calls=calls):
            calls["n"] += 1
            if calls["n"] == 4:                     # a decode step of the first two requests
                raise ops.KernelError("injected")
            return real(st)
        eng.runner.forward = failing
        outs = llm.generate(prompts, sp)
        eng.runner.forward = real
        failed = [o for o in outs if o.finish_reason == "error"]
        assert len(failed) == 2 and all("injected" in o.error for o in failed)
        assert {o.request_id for o in failed} == {outs[0].request_id, outs[1].request_id}
        assert all(o.token_ids == w[:len(o.token_ids)] and len(o.token_ids) < 12 for o, w in zip(outs[:2], want[:2]))
        assert [o.token_ids for o in outs[2:]] == want[2:] and all(o.finish_reason == "length" for o in outs[2:])
        assert eng.stats.failed_requests == 2 and eng.sched.check() == "" and not eng.has_work()
        assert eng.cache.num_free_pages(0) == 64
        if ahead:
            continue
        # a batch that the step function refuses (a token id outside the vocabulary got into a
        # request's history) is a StepError of that step: the same path
        a = eng.add_request(prompts[0], sp)
        b = eng.add_request(prompts[1], sp)
        c = eng.add_request(prompts[2], sp)              # waits for a seat
        eng.step()
        eng.step()
        eng.seqs[a].tokens[-1] = 10 ** 6
        by_id = {o.request_id: o for o in eng.run_to_completion()}
        assert by_id[a].finish_reason == by_id[b].finish_reason == "error" and "vocabulary" in by_id[a].error
        assert by_id[c].finish_reason == "length" and by_id[c].token_ids == want[2]
        assert eng.sched.check() == "" and eng.cache.num_free_pages(0) == 64


def test_an_error_word_from_the_device_fails_the_step(model_root):
    """A bounded wait that runs out inside a kernel leaves an error word; it travels to the host
    with the step's ids, and the step's requests fail instead of going on with what the kernel left.
    No wait is made to run out here: the word is set where the host reads it."""
    from rust_llm_inference_server_b200 import SamplingParams
    llm = make_llm(model_root, "A", "bfloat16", max_num_seqs=2)
    eng = llm.engine
    prompts = prompts_for("A", [5, 9, 7], seed=2)
    sp = SamplingParams(max_tokens=8)
    want = [o.token_ids for o in llm.generate(prompts, sp)]
    assert eng._device_error(0) == 0 and eng._device_error(1) == 0      # the word really arrives, and is zero
    real, calls = eng._device_error, {"n": 0}

    def once(slot):
        calls["n"] += 1
        return 1 if calls["n"] == 3 else real(slot)
    eng._device_error = once
    outs = llm.generate(prompts, sp)
    assert [o.finish_reason for o in outs] == ["error", "error", "length"]
    assert "bounded wait" in outs[0].error and outs[2].token_ids == want[2]
    assert eng.sched.check() == "" and eng.cache.num_free_pages(0) == 64


def test_timing_records_and_named_spans(model_root):
    """Per-step host times (crates/engine/src/engine.rs:717-724) and, when switched on, CUDA-event
    spans around the stages of the forward pass (crates/model/src/profile.rs:22-49)."""
    from rust_llm_inference_server_b200 import SamplingParams
    from rust_llm_inference_server_b200.ops import profile
    llm = make_llm(model_root, "B", "bfloat16", max_seq_len=256, block_size=16)
    prompts = prompts_for("B", [40, 3], seed=9)
    base = [o.token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=6))]
    st = llm.engine.stats
    assert st.total_prep_us > 0 and st.total_forward_us > 0 and st.total_sample_us > 0 and st.total_wait_us >= 0
    assert st.prep_us > 0 and st.forward_us > 0
    assert profile.take_report() == {}                    # off: nothing is recorded
    profile.enable(True)
    try:
        got = [o.token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=6))]
        rep = profile.take_report()
    finally:
        profile.enable(False)
    assert got == base
    layers, steps = CONFIGS["B"]["num_hidden_layers"], 6
    for name in ("embedding", "qkv proj", "o proj", "mlp gate+up, silu*up", "mlp down proj", "lm head", "sampler"):
        assert name in rep and rep[name][0] > 0, name
    assert rep["qkv proj"][1] == layers * steps and rep["embedding"][1] == steps and rep["sampler"][1] == steps
    none = (0.0, 0)
    assert rep.get("attention", none)[1] + rep.get("rope + kv write + attention", none)[1] == layers * steps
    assert "stage" in profile.format_report(rep)
