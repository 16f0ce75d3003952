"""Trace replay on the GPU against the plain implementation, in float32 and bfloat16: each request
alone and whole; most of it in one step and the last 32 tokens one by one; in portions of
changing size; and mixed, up to four live requests in a pool so small that pages are used again."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import replay_util as R
from tests.plain import llama_plain as P
from tests.tiny_configs import CONFIGS, load_plain_weights, make_model_dir

pytestmark = pytest.mark.gpu

# |logit| is about 1 for these models.  float32: the reference's own bound for its tiny model
# (crates/model/src/llama.rs:354) is 1e-4.  bfloat16: inputs and weights of every product are
# rounded to 8 bits of mantissa.
TOL = {"float32": 1e-4, "bfloat16": 3e-2}
TOL_BETWEEN_MODES = {"float32": 1e-5, "bfloat16": 2e-2}


def requests_for(which: str, seed: int = 1) -> dict:
    cfg = CONFIGS[which]
    rng = np.random.default_rng(seed)
    lens = {"A": [1, 7, 13, 32, 100], "B": [3, 50, 97, 200, 64, 17], "C": [130, 33, 2, 71, 40],
            "D": [300, 150, 40, 2, 200, 129], "E": [260, 31, 140, 5, 90]}[which]
    return {f"r{i}": rng.integers(0, cfg["vocab_size"], size=n).tolist() for i, n in enumerate(lens)}


_plain_cache: dict = {}


def plain_logits(model_root, which):
    if which not in _plain_cache:
        w = load_plain_weights(make_model_dir(model_root, which))
        _plain_cache[which] = {name: P.forward_logits(w, CONFIGS[which], toks).numpy()
                               for name, toks in requests_for(which).items()}
    return _plain_cache[which]


def session(model_root, which, dtype, max_tokens, page_size=16):
    from rust_llm_inference_server_b200.engine.replay import ReplaySession
    return ReplaySession(make_model_dir(model_root, which), dtype, max_tokens, page_size)


# Which kernels a configuration's bfloat16 replay has to go through (names of
# `ops.launches_by_kernel`): a configuration that silently took a slower path would still give the
# right logits.
KERNELS_BF16 = {
    "D": ["attention_prefill.tcgen05", "attention_decode.mma.tma", "attention_decode_qkv.mma.tma",
          "gemm_tcgen05.swiglu4", "stream_gemm.sink", "stream_gemm.scaled", "stream_gemm.scaled.swiglu",
          "rope_cache", "rmsnorm", "rmsnorm.rows", "embedding", "embedding.sink"],
    "E": ["attention_prefill.tcgen05", "attention_decode.mma.tma", "attention_decode_qkv.mma.tma", "stream_gemm.sink",
          "stream_gemm.scaled"],
    "A": ["attention_generic", "attention_decode.cuda_core"],
}


def compare(got: dict, ref: dict, tol: float, what: str):
    worst, where = 0.0, None
    for (name, pos), row in got.items():
        d = float(np.abs(row - ref[name][pos]).max())
        if not np.isfinite(d):
            d = float("inf")
        if d > worst:
            worst, where = d, (name, pos)
    assert worst <= tol, f"{what}: max |logit difference| {worst} at request/position {where}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which,page", [("A", 16), ("A", 8), ("B", 16), ("C", 16), ("D", 16), ("D", 32), ("E", 16), ("E", 64),
                                        ("E", 128)])
def test_all_ways_of_cutting_give_the_plain_logits(model_root, which, page, dtype):
    from rust_llm_inference_server_b200 import ops
    ops.launches_by_kernel.clear()
    reqs = requests_for(which)
    ref = plain_logits(model_root, which)
    families = {
        "whole": R.whole_trace(reqs),
        "decode": R.decode_trace(reqs),
        "chunks": R.chunk_trace(reqs, seed=3),
        "mixed": R.mixed_trace(reqs, seed=4),
        "mixed2": R.mixed_trace(dict(reversed(list(reqs.items()))), seed=5, max_live=3),
    }
    results = {}
    for fam, steps in families.items():
        s = session(model_root, which, dtype, R.live_token_peak(steps, max(64, page)), page)   # the smallest pool allowed
        results[fam] = R.collect(s.step, steps)
        if dtype == "bfloat16" and fam == "decode" and which in ("D", "E"):
            assert s.runner._graph_launches > 0            # single tokens ran from captured graphs
        assert s.cache.check_invariants() == ""
        assert s.cache.num_free_pages(0) == s.cache.group(0).num_pages, fam   # everything given back
        compare(results[fam], ref, TOL[dtype], f"{which} {dtype} {fam} vs plain")
    whole = {k: v for k, v in results["whole"].items()}
    for fam in ("decode", "chunks", "mixed", "mixed2"):
        sub = {k: v for k, v in results[fam].items()}
        worst = max(float(np.abs(v - whole[k]).max()) for k, v in sub.items())
        assert worst <= TOL_BETWEEN_MODES[dtype], f"{which} {dtype}: {fam} differs from whole by {worst}"
    if dtype == "bfloat16":
        expected = list(KERNELS_BF16.get(which, []))
        if (which, page) == ("E", 128):      # a page larger than the tcgen05 kernel's block of 64 keys: the mma.sync kernel
            expected[expected.index("attention_prefill.tcgen05")] = "attention_prefill.mma"
        missing = [k for k in expected if not ops.launches_by_kernel.get(k)]
        assert not missing, f"{which}: never launched {missing}; launched {sorted(ops.launches_by_kernel)}"
    else:
        fast = [k for k in ops.launches_by_kernel if "tcgen05" in k or "mma" in k or "stream_gemm" in k]
        assert not fast, f"the float32 path went through {fast}"
    ops.check_device_errors()

@pytest.mark.parametrize("which", ["A", "B", "C"])
def test_norms_inside_the_products_and_norms_as_kernels_agree(model_root, which, monkeypatch):
    """Steps of up to 16 rows take the norms apart into the epilogues of the products around them
    (`ops.ScaledRows`, `ops.ResidualSink`); with that switched off every norm is a kernel of its
    own.  Both ways: the plain logits, each other to rounding, and fewer launches with it on."""
    from rust_llm_inference_server_b200 import ops
    reqs = requests_for(which)
    ref = plain_logits(model_root, which)
    steps = R.decode_trace(reqs)
    got, launches = {}, {}
    for fused in (True, False):
        monkeypatch.setattr(ops, "FUSE_NORMS", fused)
        s = session(model_root, which, "bfloat16", R.live_token_peak(steps))
        s.model.graph_safe = False           # count launches, not graph replays
        before = ops.launch_count
        got[fused] = R.collect(s.step, steps)
        launches[fused] = ops.launch_count - before
        compare(got[fused], ref, TOL["bfloat16"], f"{which} norms {'inside' if fused else 'as kernels'} vs plain")
    worst = max(float(np.abs(v - got[False][k]).max()) for k, v in got[True].items())
    assert worst <= TOL_BETWEEN_MODES["bfloat16"], worst
    if CONFIGS[which]["hidden_size"] % 8 == 0 and CONFIGS[which]["intermediate_size"] % 8 == 0:
        assert launches[True] < launches[False]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(model_root, dtype):
    """One token at a time from the very first token, over many pages."""
    which = "B"
    cfg = CONFIGS[which]
    toks = np.random.default_rng(9).integers(0, cfg["vocab_size"], size=230).tolist()
    w = load_plain_weights(make_model_dir(model_root, which))
    ref = P.forward_logits(w, cfg, toks).numpy()
    s = session(model_root, which, dtype, 256)
    for i, t in enumerate(toks):
        out = s.step({"step": i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": []})
        d = float(np.abs(out[0].numpy() - ref[i]).max())
        assert d <= TOL[dtype], f"{dtype}: token {i} differs by {d}"


def test_trace_run_program(model_root, tmp_path):
    """bin/trace_run as a user runs it: steps on standard input, `done <step>` lines, .f32 files."""
    which = "A"
    reqs = requests_for(which)
    ref = plain_logits(model_root, which)
    steps = R.mixed_trace(reqs, seed=7)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for dtype in ("float32", "bfloat16"):
        out_dir = tmp_path / dtype
        proc = subprocess.run(
            [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", make_model_dir(model_root, which),
             "--dtype", dtype, "--out", str(out_dir), "--max-tokens", str(R.live_token_peak(steps))]
            + (["--page-size", "8"] if dtype == "float32" else []),
            input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert proc.stdout.split("\n")[:len(steps)] == [f"done {s['step']}" for s in steps]
        V = CONFIGS[which]["vocab_size"]

        def read(st):
            n = sum(len(e["want"]) for e in st["entries"])
            arr = np.fromfile(out_dir / f"{st['step']}.f32", dtype="<f4")
            assert arr.size == n * V
            return torch.from_numpy(arr.reshape(n, V))

        compare(R.collect(read, steps), ref, TOL[dtype], f"trace_run {dtype}")


def test_step_function_refuses_bad_batches(model_root):
    from rust_llm_inference_server_b200.engine import StepEntry, StepError
    s = session(model_root, "A", "float32", 64)
    r = s.runner
    with pytest.raises(StepError):
        r.step([])
    with pytest.raises(StepError, match="empty sequence"):
        r.step([StepEntry(0, [], 0)])
    with pytest.raises(StepError, match="no page reserved"):
        r.step([StepEntry(0, [1, 2, 3], 0, [2])])
    s.cache.reserve(0, 8)
    with pytest.raises(StepError, match="vocabulary"):
        r.step([StepEntry(0, [1, 256], 0)])
    with pytest.raises(StepError, match="exceeds max_seq_len"):
        r.step([StepEntry(0, [1] * 65, 0)])
    with pytest.raises(StepError, match="twice"):
        r.step([StepEntry(0, [1], 0), StepEntry(0, [2], 1)])
    with pytest.raises(StepError, match="outside"):
        r.step([StepEntry(0, [1, 2], 0, [2])])
    assert r.step([StepEntry(0, [1, 2], 0)]) is None       # nothing wanted: no logits
    assert r.step([StepEntry(0, [3], 2, [0])]).shape == (1, 256)
