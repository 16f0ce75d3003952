"""The command line and perplexity on the GPU, against the plain implementation."""

import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests.plain import llama_plain as P
from tests.tiny_configs import CONFIGS, load_plain_weights, make_model_dir

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def rlis(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bin", "rlis"), *args], capture_output=True,
                          text=True, timeout=600)


def test_generate_subcommand_prints_tokens_and_the_closing_line(model_root):
    d = make_model_dir(model_root, "A")
    w = load_plain_weights(d)
    prompt = [5, 9, 200, 31]
    r = rlis("generate", "--model", d, "--dtype", "f32", "--prompt-ids", ",".join(map(str, prompt)),
             "--max-tokens", "8", "--max-seq-len", "64", "--kv-cache-gb", "0.001", "--block-size", "8",
             "--max-num-seqs", "2")
    assert r.returncode == 0, r.stderr[-2000:]
    assert [int(t) for t in r.stdout.split()] == P.greedy_generate(w, CONFIGS["A"], prompt, 8)
    assert "prompt 4 tok | output 8 tok (Length) | ttft" in r.stderr and "tok/s" in r.stderr


def test_perplexity_equals_the_plain_computation(model_root, tmp_path):
    which = "B"
    d = make_model_dir(model_root, which)
    w = load_plain_weights(d)
    rng = np.random.default_rng(0)
    toks = rng.integers(0, CONFIGS[which]["vocab_size"], size=3 * 32 + 5).tolist()
    f = tmp_path / "toks.txt"
    f.write_text(" ".join(map(str, toks)))
    r = rlis("perplexity", "--model", d, "--dtype", "f32", "--token-file", str(f), "--ctx", "32")
    assert r.returncode == 0, r.stderr[-2000:]
    rep = json.loads(r.stdout.strip().splitlines()[-1])
    nll = []
    for wdw in range(3):                       # crates/engine/src/perplexity.rs:46-66
        chunk = toks[wdw * 32:(wdw + 1) * 32]
        chunk[0] = toks[0]
        lp = torch.log_softmax(P.forward_logits(w, CONFIGS[which], chunk), -1)
        nll += [-float(lp[i, chunk[i + 1]]) for i in range(16, 31)]
    assert rep["windows"] == 3 and rep["tokens_scored"] == 45 and rep["ctx"] == 32
    assert abs(rep["mean_nll"] - np.mean(nll)) < 1e-4
    assert abs(rep["ppl"] - math.exp(np.mean(nll))) < 1e-2


def test_random_weights_subcommand(tmp_path):
    cfg = tmp_path / "c.json"
    cfg.write_text(json.dumps(CONFIGS["A"]))
    r = rlis("random-weights", "--config", str(cfg), "--seed", "0", "--out", str(tmp_path / "m"))
    assert r.returncode == 0, r.stderr[-2000:]
    assert sorted(os.listdir(tmp_path / "m")) == ["config.json", "model.safetensors"]
