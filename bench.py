#!/usr/bin/env python3
"""Benchmark of the decode step (and a 2,048-token prefill) at the Llama-3.2-1B layer sizes with
random bfloat16 weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  `value` is decoded tokens a second over K device-timed decode steps of a
batch of 8 requests whose context ends at 4,096 tokens (teacher-forced random tokens, sampler
kernel included, CUDA events around the K steps).  `e2e` is the same quantity through the Python
entry point (`LLM.stream`): every step uploads its inputs from pinned host memory and reads its
sampled token ids back.  Method after the reference's own micro-benchmarks (warm-up, then a timed
loop with a device synchronisation on both sides, crates/model/examples/decode_profile.rs:47-62).
"""

from __future__ import annotations

import argparse
import json
import os
import shutil
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# configs[2] of the baseline description: Llama-3.2-1B sizes
CONFIG_1B = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 2048, "intermediate_size": 8192, "num_hidden_layers": 16,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "vocab_size": 128256,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "max_position_embeddings": 131072,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "tie_word_embeddings": True,
}
CONTEXT = 4096
PREFILL_TOKENS = 2048
SEED = 4

# configs[3] and configs[4] of the baseline description: Llama-3.2-3B and Llama-3.1-8B sizes
CONFIG_3B = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 3072, "intermediate_size": 8192, "num_hidden_layers": 28,
    "num_attention_heads": 24, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 128256,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "max_position_embeddings": 131072,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "tie_word_embeddings": True,
}
CONFIG_8B = {
    "architectures": ["LlamaForCausalLM"],
    "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 32,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 128256,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "max_position_embeddings": 131072,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "tie_word_embeddings": False,
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks() -> tuple:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(d.get(k), (int, float)):
                    out[k] = float(d[k])
            return out, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.lines: list = []

    def start(self):
        exe = shutil.which("nvidia-smi")
        if not exe:
            return
        idx = os.environ.get("CUDA_VISIBLE_DEVICES", "0").split(",")[0] or "0"
        try:
            self.proc = subprocess.Popen(
                [exe, "-i", idx, f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


def weight_bytes(cfg: dict, n_layers: int, elem: int = 2) -> int:
    """What a decode step reads of the weights: every layer's matrices and the LM head's table once
    (the embedding rows of a few tokens do not count)."""
    H, I, d = cfg["hidden_size"], cfg["intermediate_size"], cfg["head_dim"]
    nh, nkv, V = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["vocab_size"]
    per_layer = ((nh + 2 * nkv) * d * H + H * nh * d + 3 * I * H) * elem + 2 * H * 4
    return n_layers * per_layer + V * H * elem + H * 4


def kv_bytes_per_token(cfg: dict, n_layers: int, elem: int = 2) -> int:
    return 2 * n_layers * cfg["num_key_value_heads"] * cfg["head_dim"] * elem


def prefill_flops(cfg: dict, n_layers: int, T: int) -> float:
    H, I, d = cfg["hidden_size"], cfg["intermediate_size"], cfg["head_dim"]
    nh, nkv, V = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["vocab_size"]
    proj = 2.0 * T * ((nh + 2 * nkv) * d * H + H * nh * d + 3 * I * H)
    attn = 2.0 * T * T * nh * d          # causal: QK^T and PV over half the square
    return n_layers * (proj + attn) + 2.0 * V * H


def run_reference(args) -> int:
    print(json.dumps({
        "impl": "reference",
        "unavailable": "the reference is a Rust workspace on the candle library (Metal kernels); pip finds "
                       "neither setup.py nor pyproject.toml and there is no cargo/rustc here, so it cannot be installed",
    }))
    return 0


def decode_run(llm, B: int, steps: int, warmup: int, ctx_end: int, torch, fill: bool = True, clocks=None):
    """Device-timed decode: B requests, each step one teacher-forced token per request and the
    sampler kernel; the last step's context is `ctx_end`.  Returns (ms per step, launches per step)."""
    import numpy as np
    from rust_llm_inference_server_b200.engine import StepEntry
    from rust_llm_inference_server_b200.ops import profile

    eng = llm.engine
    runner, cache = eng.runner, eng.cache
    V = llm.model.spec.vocab_size
    rng = np.random.default_rng(B)
    total = warmup + steps
    ctx0 = ctx_end - total
    ids = list(range(10_000, 10_000 + B))
    for sid in ids:
        assert cache.acquire_state_slot(sid) >= 0
        assert cache.reserve(sid, ctx_end), "cache pool too small for the benchmark"
    # fill the cache up to ctx0 with a prompt cut into portions of at most 2,048 tokens
    for sid in ids:
        pos = 0 if fill else ctx0      # (profiler captures skip the fill: the pages then hold zeros)
        while pos < ctx0:
            n = min(2048, ctx0 - pos)
            runner.step([StepEntry(sid, rng.integers(0, V, size=n).tolist(), pos, [])])
            pos += n
    params = torch.zeros((B, 2), dtype=torch.int32, device=llm.model.device)     # greedy rows
    out_ids = torch.empty((B,), dtype=torch.int32, device=llm.model.device)
    toks = rng.integers(0, V, size=(total, B))
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    launches = 0
    if clocks is not None:          # sample clocks over the warm-up and the timed steps only
        clocks.start()
        time.sleep(0.5)             # let nvidia-smi come up before anything is timed
    for i in range(total):
        if i == warmup:
            torch.cuda.synchronize()
            if profile.enabled:
                profile.take_report()       # the table covers the timed steps only
            l0 = runner.launches
            start.record()
        logits = runner.step([StepEntry(sid, [int(toks[i, b])], ctx0 + i, [0]) for b, sid in enumerate(ids)])
        runner.sample(logits, params, out_ids)
    end.record()
    torch.cuda.synchronize()
    launches = runner.launches - l0
    ms = start.elapsed_time(end) / steps
    for sid in ids:
        cache.free(sid)
    return ms, launches / steps


def percentile(xs, q):
    if not xs:
        return None
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(round(q / 100.0 * (len(xs) - 1))))]


def serve_poisson(llm, prompts, outputs, arrivals, torch):
    """Feeds requests to the engine loop as their arrival times come (wall clock) and steps it
    until all have finished.  Returns per-request time to first token (from the intended arrival),
    the gaps between a request's tokens, and the wall time from the first arrival to the last token."""
    from rust_llm_inference_server_b200 import SamplingParams
    eng = llm.engine
    n = len(prompts)
    first, last, gaps, done = {}, {}, [], {}
    nxt = 0
    rid_of = {}
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    while len(done) < n:
        now = time.perf_counter() - t0
        while nxt < n and arrivals[nxt] <= now:
            rid = eng.add_request(prompts[nxt], SamplingParams(max_tokens=outputs[nxt], ignore_eos=True))
            rid_of[rid] = nxt
            nxt += 1
        if not eng.has_work():
            time.sleep(max(0.0, min(0.001, arrivals[nxt] - now)))
            continue
        finished = eng.step()
        t = time.perf_counter() - t0
        for rid in eng.last_step.new_tokens:
            i = rid_of[rid]
            if i not in first:
                first[i] = t - arrivals[i]
            else:
                gaps.append(t - last[i])
            last[i] = t
        for o in finished:
            done[rid_of[o.request_id]] = o
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    return first, gaps, wall, done


def workload_3b(args, torch, np) -> dict:
    """configs[3]: 64 requests, prompts U[128, 2048], outputs U[64, 512], seeded Poisson arrivals,
    prompts cut into portions of 512 tokens, through `LLMEngine.add_request` / `step` (the numbers
    the reference publishes for its server sweep, README.md:187-191,208-214: throughput, time to the
    first token, time between tokens, preemptions, prefix hits)."""
    from rust_llm_inference_server_b200 import LLM
    cfg = dict(CONFIG_3B)
    n_full = cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = args.layers or n_full
    rng = np.random.default_rng(5)
    n = 64
    p_lens = rng.integers(128, 2049, size=n).tolist()
    o_lens = rng.integers(64, 513, size=n).tolist()
    prompts = [rng.integers(0, cfg["vocab_size"], size=k).tolist() for k in p_lens]
    arrivals = np.cumsum(rng.exponential(1.0 / args.rate, size=n)).tolist()
    page = 16
    kv_tok = kv_bytes_per_token(cfg, cfg["num_hidden_layers"])
    runs = {}
    llm = None
    for name, pool_tokens in (("roomy", sum(p + o for p, o in zip(p_lens, o_lens)) + 64 * page),
                              ("tight", 40960)):
        del llm
        torch.cuda.empty_cache()
        llm = LLM.from_random(cfg, 5, dtype="bfloat16", on_device=True, max_seq_len=2048 + 512 + page,
                              num_blocks=pool_tokens // page, block_size=page, max_num_seqs=64,
                              max_batched_tokens=512, prefix_caching=True)
        # warm-up outside the timed region: a stream of the same shape (other tokens), so that the
        # decode shapes the run meets have their graphs; a serving process does this once at start-up
        w_prompts = [rng.integers(0, cfg["vocab_size"], size=k).tolist() for k in p_lens]
        serve_poisson(llm, w_prompts, o_lens, arrivals, torch)
        st = llm.engine.stats
        pre0, hit0, steps0 = st.preemptions, st.prefix_hit_tokens, st.steps
        clocks = ClockSampler()
        clocks.start()
        time.sleep(0.3)
        first, gaps, wall, done = serve_poisson(llm, prompts, o_lens, arrivals, torch)
        clk = clocks.stop()
        assert all(len(done[i].token_ids) == o_lens[i] for i in range(n))
        out_tokens = sum(o_lens)
        ms = lambda x: None if x is None else round(x * 1e3, 2)
        runs[name] = {
            "pool_tokens": pool_tokens, "pool_gb": round(pool_tokens * kv_tok / 2 ** 30, 2),
            "wall_s": round(wall, 3), "output_tokens_per_s": round(out_tokens / wall, 1),
            "total_tokens_per_s": round((out_tokens + sum(p_lens)) / wall, 1),
            "ttft_ms_p50": ms(percentile(list(first.values()), 50)), "ttft_ms_p99": ms(percentile(list(first.values()), 99)),
            "itl_ms_p50": ms(percentile(gaps, 50)), "itl_ms_p99": ms(percentile(gaps, 99)),
            "preemptions": st.preemptions - pre0, "prefix_hit_tokens": st.prefix_hit_tokens - hit0,
            "steps": st.steps - steps0, "failed": st.failed_requests, "clocks": clk,
        }
    return {
        "workload": "3b", "metric": "continuous batching, 64 requests in a Poisson stream (Llama-3.2-3B sizes, random bf16 weights)",
        "impl": "ours", "dtype": "bf16", "n_gpus": 1,
        "data": "synthetic: uniform-random token ids, random-init weights N(0,0.02) seed 5 (device generator)",
        "config": {"model": "llama-3.2-3b-sizes", "layers": cfg["num_hidden_layers"], "layers_in_config": n_full,
                   "hidden": 3072, "heads": 24, "kv_heads": 8, "head_dim": 128, "intermediate": 8192, "vocab": 128256,
                   "requests": n, "prompt_tokens": sum(p_lens), "output_tokens": sum(o_lens), "rate_per_s": args.rate,
                   "max_batched_tokens": 512, "max_num_seqs": 64, "page_size": page, "prefix_caching": True},
        "runs": runs,
    }


def workload_8b(args, torch, np) -> dict:
    """configs[4]: 32 requests with 2,048-token prompts, a quarter of which share their first
    1,024 tokens, through the engine (prefill in portions, prefix reuse), then device-timed decode
    steps of the 32 whose context ends at 8,192 tokens, against the HBM roofline."""
    from rust_llm_inference_server_b200 import LLM, SamplingParams
    cfg = dict(CONFIG_8B)
    n_full = cfg["num_hidden_layers"]
    n_layers = args.layers or n_full
    cfg["num_hidden_layers"] = n_layers
    pk, pk_src = peaks()
    rng = np.random.default_rng(6)
    B, ctx, page = 32, 8192, 16
    llm = LLM.from_random(cfg, 6, dtype="bfloat16", on_device=True, max_seq_len=ctx + page,
                          num_blocks=B * (ctx + page) // page + 64, block_size=page, max_num_seqs=B,
                          max_batched_tokens=2048, prefix_caching=True)
    V = cfg["vocab_size"]
    shared = rng.integers(0, V, size=1024).tolist()
    prompts = [(shared + rng.integers(0, V, size=1024).tolist()) if i % 4 == 0 else rng.integers(0, V, size=2048).tolist()
               for i in range(B)]
    sp = SamplingParams(max_tokens=16, ignore_eos=True)
    llm.generate([rng.integers(0, V, size=300).tolist()], SamplingParams(max_tokens=4, ignore_eos=True))   # warm-up
    st = llm.engine.stats
    hit0 = st.prefix_hit_tokens
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = llm.generate(prompts, sp)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    assert all(len(o.token_ids) == 16 for o in outs)
    engine_part = {"prompt_tokens": 2048 * B, "prefix_hit_tokens": st.prefix_hit_tokens - hit0, "wall_s": round(wall, 3),
                   "prompt_tokens_per_s": round(2048 * B / wall, 1), "preemptions": st.preemptions}
    steps = min(args.steps, 64)
    clocks = ClockSampler()
    ms, launches = decode_run(llm, B, steps, args.warmup, ctx, torch, clocks=clocks)
    clk = clocks.stop()
    mean_ctx = ctx - steps / 2
    step_bytes = weight_bytes(cfg, n_layers) + B * mean_ctx * kv_bytes_per_token(cfg, n_layers)
    achieved = step_bytes / (ms / 1e3) / 1e9
    return {
        "workload": "8b", "metric": "decode tokens/s, batch 32, context 8192 (Llama-3.1-8B sizes, random bf16 weights)",
        "value": round(B / (ms / 1e3), 1), "unit": "tokens/s", "ms_per_step": round(ms, 4), "steps": steps, "warmup": args.warmup,
        "impl": "ours", "dtype": "bf16", "n_gpus": 1,
        "data": "synthetic: uniform-random token ids, random-init weights N(0,0.02) seed 6 (device generator)",
        "config": {"model": "llama-3.1-8b-sizes", "layers": n_layers, "layers_in_config": n_full, "hidden": 4096,
                   "heads": 32, "kv_heads": 8, "head_dim": 128, "intermediate": 14336, "vocab": V, "tied": False,
                   "global_batch": B, "seq_len": ctx, "page_size": page, "kv_dtype": "bf16"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk_src,
                     "bytes_per_step": int(step_bytes)},
        "prompts_through_the_engine": engine_part, "gpu_launches": int(round(launches * steps)), "clocks": clk,
    }


def workload_1b_fp32(args, torch, np) -> dict:
    """The true 32-bit path at the 1B sizes: a 2,048-token prefill and decode steps of a batch of 8
    at a context of 4,096 (FFMA products, float32 cache and attention; no tensor cores)."""
    from rust_llm_inference_server_b200 import LLM
    from rust_llm_inference_server_b200.engine import StepEntry
    cfg = dict(CONFIG_1B)
    n_full = cfg["num_hidden_layers"]
    n_layers = args.layers or n_full
    cfg["num_hidden_layers"] = n_layers
    B, ctx, page = 8, CONTEXT, 16
    llm = LLM.from_random(cfg, SEED, dtype="float32", on_device=True, max_seq_len=ctx + page,
                          num_blocks=B * (ctx + page) // page + 64, block_size=page, max_num_seqs=B,
                          max_batched_tokens=2048, prefix_caching=False)
    runner, cache = llm.engine.runner, llm.engine.cache
    rng = np.random.default_rng(0)
    pre = []
    for it in range(4):
        sid = 500 + it
        cache.acquire_state_slot(sid)
        assert cache.reserve(sid, PREFILL_TOKENS)
        toks = rng.integers(0, cfg["vocab_size"], size=PREFILL_TOKENS).tolist()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        runner.step([StepEntry(sid, toks, 0, [PREFILL_TOKENS - 1])])
        e.record()
        torch.cuda.synchronize()
        pre.append(s.elapsed_time(e))
        cache.free(sid)
    prefill_ms = statistics.median(pre[1:])
    steps = min(args.steps, 32)
    clocks = ClockSampler()
    ms, launches = decode_run(llm, B, steps, args.warmup, ctx, torch, clocks=clocks)
    clk = clocks.stop()
    pk, pk_src = peaks()
    step_bytes = weight_bytes(cfg, n_layers, 4) + B * (ctx - steps / 2) * kv_bytes_per_token(cfg, n_layers, 4)
    achieved = step_bytes / (ms / 1e3) / 1e9
    return {
        "workload": "1b-fp32", "metric": "decode tokens/s, batch 8, context 4096, true float32 path (Llama-3.2-1B sizes)",
        "value": round(B / (ms / 1e3), 1), "unit": "tokens/s", "ms_per_step": round(ms, 4), "steps": steps, "warmup": args.warmup,
        "impl": "ours", "dtype": "fp32", "n_gpus": 1,
        "config": {"model": "llama-3.2-1b-sizes", "layers": n_layers, "layers_in_config": n_full, "global_batch": B,
                   "seq_len": ctx, "page_size": page, "kv_dtype": "fp32"},
        "prefill": {"value": round(PREFILL_TOKENS / (prefill_ms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(prefill_ms, 3),
                    "tflops": round(prefill_flops(cfg, n_layers, PREFILL_TOKENS) / (prefill_ms / 1e3) / 1e12, 2)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk_src},
        "gpu_launches": int(round(launches * steps)), "clocks": clk,
    }


def print_timeline(records: list) -> None:
    """One decode step product by product (microseconds since the first product of the step started):
    when the launch's first CTA started, when its wait for the kernel before it passed, when its
    products were done, and when it ended; the gap is from the end of the product before to this
    one's wait passing, which for QKV -> O holds the attention kernel."""
    if not records:
        return
    t0 = records[0]["start"]
    us = lambda v: "      -" if v is None else f"{(v - t0) / 1e3:7.2f}"
    print(f"{'N x K':>15} | {'start':>7} {'waited':>7} {'done':>7} {'barrier':>7} {'sent':>7} {'arrived':>7} {'end':>7} | after the wait | gap before | grid before done",
          file=sys.stderr)
    prev = None
    for r in records:
        gap = "" if prev is None else f"{(r['wait_passed'] - prev) / 1e3:6.2f}"
        print(f"{r['N']:>7} x {r['K']:>5} | {us(r['start'])} {us(r['wait_passed'])} {us(r['products_done'])} {us(r['cluster_barrier'])} "
              f"{us(r['sent'])} {us(r['sums_arrived'])} {us(r['end'])} | {(r['end'] - r['wait_passed']) / 1e3:14.2f} | {gap:>10} | {us(r['grid_before_done'])}",
              file=sys.stderr)
        prev = r["end"]


WORKLOADS = {"3b": workload_3b, "8b": workload_8b, "1b-fp32": workload_1b_fp32}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (both numbers are reported)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=CONTEXT, help="context length at the last timed decode step")
    ap.add_argument("--no-fill", action="store_true",
                    help="with --only decode: do not compute the cached context first (keeps profiler captures short)")
    ap.add_argument("--only", default=None, choices=["decode", "prefill"],
                    help="run one part only and print a short line (for profiler captures of a small case)")
    ap.add_argument("--sizes", default="1b", choices=["1b", "3b", "8b"],
                    help="with --only: the layer sizes to run it at (the default line is always the 1B's)")
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS),
                    help="one of the other measured configurations instead of the default line: 3b (continuous "
                         "batching under a Poisson stream), 8b (batch 32 at 8,192 of context), 1b-fp32")
    ap.add_argument("--rate", type=float, default=48.0, help="--workload 3b: mean arrivals a second")
    ap.add_argument("--timeline", action="store_true",
                    help="with --only decode and RLIS_TIMELINE=1 in the environment (a build of the kernels with "
                         "the stamps compiled in): lay the last step out product by product from the stamps the "
                         "streaming products' first CTAs take of the device's timer (printed to stderr)")
    ap.add_argument("--spans", action="store_true",
                    help="with --only: time the stages of the step with CUDA-event spans (RLIS_PROFILE) and "
                         "print the table to stderr; steps then run eagerly, not from graphs")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)

    import numpy as np
    import torch

    from rust_llm_inference_server_b200 import LLM, SamplingParams, ops
    from rust_llm_inference_server_b200.ops import profile

    if args.workload:
        print(json.dumps(WORKLOADS[args.workload](args, torch, np)))
        return 0
    pk, pk_src = peaks()
    cfg = dict({"1b": CONFIG_1B, "3b": CONFIG_3B, "8b": CONFIG_8B}[args.sizes if args.only else "1b"])
    n_layers_full = cfg["num_hidden_layers"]
    n_layers = args.layers or n_layers_full
    cfg["num_hidden_layers"] = n_layers
    B = args.batch
    total = args.warmup + args.steps
    page = 16
    max_b = max(B, 64)
    context = args.context
    if args.only:
        max_b = B
    pool_tokens = max_b * (context + page)
    llm = LLM.from_random(cfg, SEED, dtype="bfloat16", on_device=True, max_seq_len=max(context, PREFILL_TOKENS) + page,
                          num_blocks=pool_tokens // page + 64, block_size=page, max_num_seqs=max_b,
                          max_batched_tokens=max(2048, max_b), prefix_caching=False)
    runner = llm.engine.runner

    # ---- prefill of one 2,048-token prompt ----
    from rust_llm_inference_server_b200.engine import StepEntry
    rng = np.random.default_rng(0)
    V = cfg["vocab_size"]
    cache = llm.engine.cache
    if args.only and args.spans:
        profile.enable(True)
    if args.only == "decode":
        if args.timeline:
            ops.stream_timeline(True)
        ms, launches = decode_run(llm, B, args.steps, args.warmup, context, torch, fill=not args.no_fill)
        print(json.dumps({"only": "decode", "batch": B, "context": context, "ms_per_step": round(ms, 4),
                          "launches_per_step": launches}))
        if args.timeline:
            print_timeline(ops.read_stream_timeline(4 * n_layers + 1))
        if args.spans:
            print(profile.format_report(profile.take_report()), file=sys.stderr)
        return 0
    pre_ms = []
    for it in range(5 if not args.only else args.warmup + args.steps):
        sid = 500 + it
        cache.acquire_state_slot(sid)
        assert cache.reserve(sid, PREFILL_TOKENS)
        toks = rng.integers(0, V, size=PREFILL_TOKENS).tolist()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        if args.only and args.spans and it == args.warmup:
            profile.take_report()           # the table covers the timed steps only
        s.record()
        runner.step([StepEntry(sid, toks, 0, [PREFILL_TOKENS - 1])])
        e.record()
        torch.cuda.synchronize()
        pre_ms.append(s.elapsed_time(e))
        cache.free(sid)
    prefill_ms = statistics.median(pre_ms[2:] if not args.only else pre_ms[args.warmup:])
    if args.only == "prefill":
        print(json.dumps({"only": "prefill", "tokens": PREFILL_TOKENS, "ms": round(prefill_ms, 3)}))
        if args.spans:
            print(profile.format_report(profile.take_report()), file=sys.stderr)
        return 0
    pf = prefill_flops(cfg, n_layers, PREFILL_TOKENS)
    prefill = {"value": round(PREFILL_TOKENS / (prefill_ms / 1e3), 1), "tokens": PREFILL_TOKENS,
               "ms": round(prefill_ms, 3),
               "frac": round(pf / (prefill_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}

    # ---- decode points at batch 1 and 64, then the headline batch under the clock sampler ----
    points = {}
    for b in (1, 64):
        ms, _ = decode_run(llm, b, max(16, min(args.steps, 64)), args.warmup, context, torch)
        points[f"decode_b{b}"] = round(b / (ms / 1e3), 1)
    clocks = ClockSampler()
    ms, launches = decode_run(llm, B, args.steps, args.warmup, context, torch, clocks=clocks)
    clk = clocks.stop()
    value = B / (ms / 1e3)
    mean_ctx = context - args.steps / 2
    step_bytes = weight_bytes(cfg, n_layers) + B * mean_ctx * kv_bytes_per_token(cfg, n_layers)
    achieved = step_bytes / (ms / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk_src}

    # ---- end to end through the Python entry point ----
    # The prompts finish their prefill in different steps (the token budget cuts them), so the
    # requests do not decode in lockstep; each gets enough output that all B decode together for
    # warmup + steps steps, the last of which sees a context of about `context` tokens.
    stagger = B * (context // 2048 + 1)
    e2e_out = total + stagger + 8
    prompts = [rng.integers(0, V, size=context - e2e_out - 1).tolist() for _ in range(B)]
    sp = SamplingParams(max_tokens=e2e_out, ignore_eos=True)
    eng = llm.engine
    h2d0 = d2h0 = h2d1 = d2h1 = 0
    t0 = t1 = None
    n_decode = 0
    for ev in llm.stream(prompts, sp):
        if not (ev.all_decoding and ev.n_seqs == B) or t1 is not None:
            continue
        n_decode += 1
        if n_decode == args.warmup:
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            h2d0, d2h0 = eng.stats.h2d_bytes, eng.stats.d2h_bytes
        elif n_decode == args.warmup + args.steps:
            torch.cuda.synchronize()
            t1 = time.perf_counter()
            h2d1, d2h1 = eng.stats.h2d_bytes, eng.stats.d2h_bytes
    e2e_ms = (t1 - t0) * 1e3 / args.steps
    e2e = {"value": round(B / (e2e_ms / 1e3), 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
           "h2d_bytes_per_step": (h2d1 - h2d0) // args.steps, "d2h_bytes_per_step": (d2h1 - d2h0) // args.steps}

    line = {
        "metric": "decode tokens/s, batch 8, context 4096 (Llama-3.2-1B sizes, random bf16 weights)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: uniform-random token ids, random-init weights N(0,0.02) seed 4",
        "impl": "ours",
        "config": {
            "model": "llama-3.2-1b-sizes", "layers": n_layers, "layers_in_config": n_layers_full,
            "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": V,
            "tied": True, "rope": "theta 5e5 llama3 32/1/4/8192", "eps": 1e-5,
            "global_batch": B, "seq_len": context, "page_size": page, "parallelism": "single GPU",
            "l2": "inputs larger than L2 (weights 2.47 GB per step)", "kv_dtype": "bf16",
        },
        "prefill": prefill, "roofline": roofline, "points": points, "e2e": e2e,
        "gpu_launches": int(round(launches * args.steps)), "clocks": clk,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
