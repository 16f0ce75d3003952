"""What the small replay matrix cannot show: the layer sizes of Llama 3.2 1B (two layers of them)
against the plain implementation under the reference's own bound, and decode steps of many
requests at once, which go through other kernels than steps of a few."""

import numpy as np
import pytest
import torch

from tests import replay_util as R
from tests.plain import llama_plain as P
from tests.tiny_configs import CONFIGS, load_plain_weights, make_model_dir

pytestmark = pytest.mark.gpu

# crates/model/tests/parity.rs:19-24: top-64 logits and the logsumexp of every position within
# 5e-4 in float32 and 0.15 in reduced precision; :30-35: a greedy choice may differ in reduced
# precision only where the float32 margin between the two candidates is below 0.02.
TOPK = 64
BOUND = {"float32": 5e-4, "bfloat16": 0.15}
NEAR_TIE = 0.02
# With random weights the rounding errors at two candidates are independent, and top-2 margins of a
# few hundredths are common, so the margin rule above needs the size of the noise beside it.  The
# noise is measured on every row (the rms error over the whole vocabulary: 0.0094 of the logits'
# spread at the 1B sizes and 0.0112 at the 3B sizes in bfloat16, 3e-6 and 4e-6 in float32, the same
# for whole prompts, single tokens and mixed steps) and bounded; a choice may then differ where
# the margin is below four times that row's own noise.  A fault at a row raises its noise past the bound long before it reaches 0.15.
ROW_NOISE = {"float32": 1e-5, "bfloat16": 0.015}      # rms error of a row / spread of its logits


def check_rows(got: np.ndarray, ref: np.ndarray, dtype: str, what: str, noise_rule: bool = False):
    assert got.shape == ref.shape and np.isfinite(got).all(), what
    worst = 0.0
    for r in range(ref.shape[0]):
        top = np.argsort(-ref[r])[:TOPK]
        d = float(np.abs(got[r, top] - ref[r, top]).max())
        lse_g = float(torch.logsumexp(torch.from_numpy(got[r]), 0))
        lse_r = float(torch.logsumexp(torch.from_numpy(ref[r]), 0))
        worst = max(worst, d, abs(lse_g - lse_r))
        near = NEAR_TIE
        if noise_rule:
            noise = float(np.sqrt(np.mean((got[r].astype(np.float64) - ref[r]) ** 2)))
            assert noise <= ROW_NOISE[dtype] * float(ref[r].std()), \
                f"{what}: row {r} has rms error {noise} over logits of spread {ref[r].std()}"
            near = max(near, 4 * noise)
        a, b = int(np.argmax(got[r])), int(top[0])
        if a != b:
            assert dtype != "float32" and ref[r, b] - ref[r, a] < near, \
                f"{what}: row {r} picks {a}, the plain implementation {b} by {ref[r, b] - ref[r, a]}"
    assert worst <= BOUND[dtype], f"{what}: top-{TOPK} logits / logsumexp differ by {worst}"
    return worst


def session(model_root, which, dtype, max_tokens, page_size=16):
    from rust_llm_inference_server_b200.engine.replay import ReplaySession
    return ReplaySession(make_model_dir(model_root, which), dtype, max_tokens, page_size)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["1B2L", "3B2L"])
def test_llama_layer_sizes_against_the_plain_implementation(model_root, which, dtype):
    """Two layers at the sizes of Llama 3.2 1B (H 2048, 32 query : 8 key/value heads of 64, I 8192,
    seed 4) and 3B (H 3072, 24 : 8 heads of 128, seed 5); V 128256, llama3 scaling, tied.
    A prompt whole; most of it in one step and the last 32 tokens one by one; and steps that mix a
    portion of one request with single tokens of another."""
    from rust_llm_inference_server_b200 import ops
    cfg = CONFIGS[which]
    rng = np.random.default_rng(21)
    a = rng.integers(0, cfg["vocab_size"], size=301).tolist()
    b = rng.integers(0, cfg["vocab_size"], size=140).tolist()
    w = load_plain_weights(make_model_dir(model_root, which))
    rows_a = sorted(set([0, 1, 63, 64, 127, 128, 255] + list(range(301 - 33, 301))))
    rows_b = list(range(100, 140))
    ref_a = P.forward_logits(w, cfg, a, rows=rows_a).numpy()
    ref_b = P.forward_logits(w, cfg, b, rows=rows_b).numpy()
    del w
    ops.launches_by_kernel.clear()
    s = session(model_root, which, dtype, 512)

    # whole
    out = s.step({"step": 0, "entries": [{"id": "a", "tokens": a, "want": rows_a}], "end": ["a"]})
    check_rows(out.numpy(), ref_a, dtype, f"{which} {dtype} whole", noise_rule=True)
    # most of it in one step, the last 32 one by one
    head = 301 - 32
    got = [s.step({"step": 1, "entries": [{"id": "a", "tokens": a[:head], "want": [head - 1]}], "end": []}).numpy()]
    for i in range(head, 301):
        got.append(s.step({"step": 2 + i, "entries": [{"id": "a", "tokens": [a[i]], "want": [0]}],
                           "end": ["a"] if i == 300 else []}).numpy())
    check_rows(np.concatenate(got), ref_a[-33:], dtype, f"{which} {dtype} last 32 one by one", noise_rule=True)
    # mixed: b's first 100 tokens, then b token by token beside portions of a
    s.step({"step": 400, "entries": [{"id": "b", "tokens": b[:100], "want": []}], "end": []})
    got_b, pos_a, k = [], 0, 0
    portions = [33, 2, 64, 17, 40, 5, 9, 31, 3, 1, 20, 12, 7, 2, 10, 45]
    got_a = {}
    for i in range(100, 140):
        entries = [{"id": "b", "tokens": [b[i]], "want": [0]}]
        if pos_a < 301:
            n = min(portions[k % len(portions)], 301 - pos_a)
            want = [r - pos_a for r in rows_a if pos_a <= r < pos_a + n]
            entries.insert(k % 2, {"id": "a", "tokens": a[pos_a:pos_a + n], "want": want})
            k += 1
        out = s.step({"step": 401 + i, "entries": entries, "end": []}).numpy()
        r = 0
        for e in entries:
            for wv in e["want"]:
                if e["id"] == "b":
                    got_b.append(out[r])
                else:
                    got_a[pos_a + wv] = out[r]
                r += 1
        if len(entries) == 2:
            pos_a += n
    assert pos_a == 301
    check_rows(np.stack(got_b), ref_b, dtype, f"{which} {dtype} single tokens beside portions", noise_rule=True)
    check_rows(np.stack([got_a[r] for r in rows_a]), ref_a, dtype, f"{which} {dtype} portions beside single tokens", noise_rule=True)
    s.step({"step": 999, "entries": [], "end": ["a", "b"]})
    assert s.cache.check_invariants() == "" and s.cache.num_free_pages(0) == s.cache.group(0).num_pages
    if dtype == "bfloat16":
        for k in ("attention_prefill.tcgen05", "attention_decode.mma.tma", "attention_decode_qkv.mma.tma",
                  "gemm_tcgen05.swiglu4", "stream_gemm.sink", "stream_gemm.scaled.swiglu"):
            assert ops.launches_by_kernel.get(k), (k, sorted(ops.launches_by_kernel))
        assert not ops.launches_by_kernel.get("attention_prefill.mma") and not ops.launches_by_kernel.get("attention_generic")
        assert s.runner._graph_launches > 0
    ops.check_device_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which,n_req,lo,hi", [("D", 32, 5, 60), ("D", 20, 500, 700), ("E", 40, 3, 90), ("A", 24, 1, 40)])
def test_many_requests_prefilled_in_one_step_and_decoded_together(model_root, which, n_req, lo, hi, dtype):
    """The reference's paged batch (crates/model/tests/parity.rs:254-324): all prompts in one
    step, then 32 steps in which every request decodes one token, over block tables whose pages
    are interleaved among the requests.  In bfloat16 a step of more than 16 rows takes the library
    product, the norm kernels and decode attention with few pieces: the batch-64 point of the
    benchmark runs this path and no other test does."""
    from rust_llm_inference_server_b200 import ops
    cfg = CONFIGS[which]
    rng = np.random.default_rng(100 + n_req)
    lens = rng.integers(lo, hi + 1, size=n_req).tolist()
    steps_dec = 32
    toks = {f"q{i}": rng.integers(0, cfg["vocab_size"], size=n + steps_dec).tolist() for i, n in enumerate(lens)}
    w = load_plain_weights(make_model_dir(model_root, which))
    ref = {name: P.forward_logits(w, cfg, t, rows=range(lens[i] - 1, lens[i] + steps_dec)).numpy()
           for i, (name, t) in enumerate(toks.items())}
    page = 16
    total = sum((n + steps_dec + 63) // 64 * 64 for n in lens)
    s = session(model_root, which, dtype, total, page)
    # pages handed out in rounds, one page a request, so that every table is interleaved with the others
    ids = {name: s._seq(name) for name in toks}
    for upto in range(page, max(lens) + page, page):
        for i, name in enumerate(toks):
            assert s.cache.reserve(ids[name], min(upto, lens[i]))
    tables = [list(s.cache.table(ids[name], 0)) for name in toks]
    assert any(np.any(np.diff(t) != 1) for t in tables if len(t) > 1) or max(lens) <= page
    ops.launches_by_kernel.clear()
    out = s.step({"step": 0, "entries": [{"id": name, "tokens": t[:lens[i]], "want": [lens[i] - 1]}
                                         for i, (name, t) in enumerate(toks.items())], "end": []}).numpy()
    got = {name: [out[i]] for i, name in enumerate(toks)}
    for k in range(steps_dec):
        out = s.step({"step": 1 + k, "entries": [{"id": name, "tokens": [t[lens[i] + k]], "want": [0]}
                                                 for i, (name, t) in enumerate(toks.items())],
                      "end": list(toks) if k == steps_dec - 1 else []}).numpy()
        for i, name in enumerate(toks):
            got[name].append(out[i])
    tol = {"float32": 1e-4, "bfloat16": 3e-2}[dtype]
    worst, where = 0.0, None
    for name in toks:
        d = np.abs(np.stack(got[name]) - ref[name]).max(axis=1)
        if float(d.max()) > worst:
            worst, where = float(d.max()), (name, int(d.argmax()))
    assert worst <= tol, f"{which} {dtype}: {n_req} requests differ from the plain logits by {worst} at {where}"
    assert s.cache.check_invariants() == "" and s.cache.num_free_pages(0) == s.cache.group(0).num_pages
    if dtype == "bfloat16" and which != "A":
        assert s.runner._graph_launches > 0
        dec = [k for k in ops.launches_by_kernel if k.startswith("attention_decode_qkv.mma")]
        assert dec and ops.launches_by_kernel.get("rmsnorm") and not ops.launches_by_kernel.get("stream_gemm.sink"), \
            sorted(ops.launches_by_kernel)
    ops.check_device_errors()
