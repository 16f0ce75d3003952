"""Command line in the reference's manner (crates/server/src/main.rs:22-127): subcommands
`generate` and `perplexity` with its option names, meanings and defaults where it has them, plus
`replay` (trace replay) and `random-weights`.  Prompts are token ids (`--prompt-ids`); `--prompt`
takes text when a `tokenizer.json` is given and the `tokenizers` package is present."""

from __future__ import annotations

import argparse
import json
import os
import sys


def _model_args(p):
    p.add_argument("--model", required=True, help="a folder with config.json and *.safetensors")
    p.add_argument("--tokenizer", default=None, help="folder with tokenizer.json (only for --prompt / --file text)")
    p.add_argument("--dtype", default="bf16", choices=["f32", "bf16", "float32", "bfloat16"],
                   help="weight and activation type (the reference's f16 is not offered)")
    p.add_argument("--device", default="cuda", help="cuda or cuda:N; there is no CPU path")
    p.add_argument("--max-seq-len", type=int, default=2048, help="longest prompt plus completion, in tokens")


def _engine_args(p):
    p.add_argument("--kv-cache-gb", type=float, default=1.0, help="size of the page pool, allocated at startup")
    p.add_argument("--block-size", type=int, default=16, help="tokens per page")
    p.add_argument("--max-num-seqs", type=int, default=64, help="most sequences in one step")
    p.add_argument("--max-batched-tokens", type=int, default=2048,
                   help="most tokens in one step; longer prompts are prefilled in portions")
    p.add_argument("--scheduler", default="continuous", choices=["continuous", "static"])
    p.add_argument("--attention", default="v2", choices=["v2"],
                   help="v2 = paged-attention kernels (the reference's v1 gather path is not built)")
    p.add_argument("--no-prefix-caching", action="store_true", help="disable automatic prefix caching")


def _tokenizer(path):
    try:
        from tokenizers import Tokenizer
    except ImportError:
        raise SystemExit("--prompt needs the `tokenizers` package; pass token ids with --prompt-ids instead")
    f = os.path.join(path, "tokenizer.json") if os.path.isdir(path) else path
    return Tokenizer.from_file(f)


def run_generate(a) -> int:
    from . import LLM, SamplingParams
    tok = None
    if a.prompt_ids is not None:
        prompt = [int(t) for t in a.prompt_ids.replace(",", " ").split()]
    elif a.prompt is not None:
        if not a.tokenizer:
            raise SystemExit("--prompt needs --tokenizer; or pass --prompt-ids")
        tok = _tokenizer(a.tokenizer)
        prompt = tok.encode(a.prompt).ids
    else:
        raise SystemExit("one of --prompt-ids or --prompt is required")
    llm = LLM(a.model, dtype=a.dtype, max_seq_len=a.max_seq_len, kv_cache_gb=a.kv_cache_gb,
              block_size=a.block_size, max_num_seqs=max(1, a.max_num_seqs), max_batched_tokens=a.max_batched_tokens,
              scheduler=a.scheduler, prefix_caching=not a.no_prefix_caching, device=a.device)
    sp = SamplingParams(temperature=a.temperature, top_p=a.top_p, top_k=a.top_k,
                        repetition_penalty=a.repetition_penalty, seed=a.seed, max_tokens=a.max_tokens)
    out = None
    for ev in llm.stream([prompt], sp):
        for t in ev.new_tokens.values():
            sys.stdout.write(tok.decode([t]) if tok else f"{t} ")
            sys.stdout.flush()
        if ev.finished:
            out = ev.finished[0]
    reason = {"stop": "Stop", "length": "Length"}[out.finish_reason]
    # the reference's closing line (crates/server/src/main.rs:249-256)
    print(f"\n\nprompt {len(prompt)} tok | output {len(out.token_ids)} tok ({reason}) | "
          f"ttft {out.ttft * 1e3:.1f}ms | decode {out.decode_tokens_per_sec:.1f} tok/s", file=sys.stderr)
    return 0


def run_perplexity(a) -> int:
    from .engine.perplexity import perplexity
    from .models import load_model
    if a.token_file:
        with open(a.token_file) as f:
            tokens = [int(t) for t in f.read().replace(",", " ").split()]
    else:
        if not a.tokenizer:
            raise SystemExit("--file is text and needs --tokenizer; or pass --token-file with token ids")
        with open(a.file, encoding="utf-8") as f:
            tokens = _tokenizer(a.tokenizer).encode(f.read()).ids
    model = load_model(a.model, a.dtype, a.device)
    bos = tokens[0] if a.token_file is None else (model.config.bos_token_id if getattr(model.config, "bos_token_id", None) is not None else tokens[0])
    print(f"{len(tokens)} tokens", file=sys.stderr)

    def progress(done, total, ppl):
        if done % 50 == 0 or done == total:
            print(f"[{done}/{total}] ppl {ppl:.4f}", file=sys.stderr)

    r = perplexity(model, tokens, bos, a.ctx, a.max_windows, progress=progress)
    print(f"PPL = {r.ppl:.4f} +/- {r.ppl_stderr:.4f} over {r.tokens_scored} tokens "
          f"({r.windows} windows of {r.ctx}) in {r.seconds:.1f}s", file=sys.stderr)
    print(json.dumps(r.to_dict()))
    return 0


def run_replay(a) -> int:
    from .engine.replay import run_replay as go
    return go(a.model, {"f32": "float32", "bf16": "bfloat16"}.get(a.dtype, a.dtype), a.out, a.max_tokens)


def run_random_weights(a) -> int:
    from .weights import write_random_model
    with open(a.config) as f:
        cfg = json.load(f)
    print(write_random_model(cfg, a.out, a.seed, a.store_dtype))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="rlis")
    sub = ap.add_subparsers(dest="command", required=True)
    g = sub.add_parser("generate", help="generate a completion for one prompt and stream it to stdout")
    _model_args(g)
    _engine_args(g)
    g.add_argument("--prompt", default=None)
    g.add_argument("--prompt-ids", default=None, help="token ids, separated by commas or spaces")
    g.add_argument("--max-tokens", type=int, default=128)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--repetition-penalty", type=float, default=1.0)
    g.add_argument("--seed", type=int, default=None)
    g.set_defaults(fn=run_generate)
    p = sub.add_parser("perplexity", help="perplexity of a text or token file (llama.cpp-compatible method)")
    _model_args(p)
    p.add_argument("--file", default="models/wikitext-2-raw/wiki.test.raw")
    p.add_argument("--token-file", default=None, help="token ids instead of text")
    p.add_argument("--ctx", type=int, default=512, help="window length; the second half of each window is scored")
    p.add_argument("--max-windows", type=int, default=0, help="score only the first N windows (0 = all)")
    p.set_defaults(fn=run_perplexity)
    r = sub.add_parser("replay", help="trace replay (see bin/trace_run)")
    r.add_argument("--model", required=True)
    r.add_argument("--dtype", required=True)
    r.add_argument("--out", required=True)
    r.add_argument("--max-tokens", type=int, required=True)
    r.set_defaults(fn=run_replay)
    w = sub.add_parser("random-weights", help="write a model folder with random weights from a config.json and a seed")
    w.add_argument("--config", required=True)
    w.add_argument("--seed", type=int, required=True)
    w.add_argument("--out", required=True)
    w.add_argument("--store-dtype", default="bfloat16", choices=["bfloat16", "float32"])
    w.set_defaults(fn=run_random_weights)
    a = ap.parse_args(argv)
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
