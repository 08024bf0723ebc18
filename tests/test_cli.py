"""The command line: flag names and defaults of the reference (no GPU), and a run end to end (GPU)."""
import json
import os
import subprocess
import sys

import pytest

from helpers import ROOT, random_tokens
from rocmforge_b200.cli import build_parser


def test_flags_and_defaults_follow_the_reference():
    a = build_parser().parse_args(["-m", "x", "-p", "hi"])
    # src/main.rs:82-96: max_tokens 256, temperature 1.0, top_p 0.9
    assert (a.model, a.prompt, a.max_tokens, a.temperature, a.top_p) == ("x", ["hi"], 256, 1.0, 0.9)
    assert not (a.no_template or a.list_tensors or a.debug or a.gpu)
    for alias in ("-t", "--temp", "--temperature"):                       # src/main.rs:106
        assert build_parser().parse_args(["-m", "x", "-p", "y", alias, "0.7"]).temperature == 0.7
    b = build_parser().parse_args(["--model", "x", "--prompt", "a", "--prompt", "b", "--max-tokens", "5", "--top-p",
                                   "0.5", "--gpu", "--no-template", "--debug", "--top-k", "3", "--seed", "0x10"])
    assert b.prompt == ["a", "b"] and b.max_tokens == 5 and b.top_p == 0.5 and b.gpu and b.no_template and b.debug
    assert b.top_k == 3 and b.seed == 16


def test_list_tensors_needs_no_gpu(folders):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "rocmforge"), "--model", folders("A"),
                          "--list-tensors"], capture_output=True, text=True)
    assert out.returncode == 0
    lines = out.stdout.strip().splitlines()
    assert any(l.startswith("model.embed_tokens.weight\tfloat32\t[256, 64]") for l in lines) and len(lines) == 26      # tied head: not stored


def test_errors_exit_with_1(folders):
    run = lambda *a: subprocess.run([sys.executable, os.path.join(ROOT, "bin", "rocmforge"), *a],
                                    capture_output=True, text=True)
    assert run("--prompt", "x").returncode == 1                             # no model
    assert run("--model", folders("A")).returncode == 1                     # no prompt
    assert run("--list-tensors").returncode == 1


@pytest.mark.gpu
def test_cli_generates_and_reports(folders):
    from plain import sampling_plain as S
    from plain.qwen2_plain import PlainModel
    prompt = random_tokens(256, 6, 3)
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "rocmforge"), "--model", folders("A"), "--dtype",
                          "float32", "--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "5", "--temperature",
                          "0", "--stop-ids", "", "--debug"], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    got = [int(l.split("token_id=")[1]) for l in out.stderr.splitlines() if l.startswith("[Generated]")]
    p = PlainModel(folders("A"))
    want, _ = S.generate(lambda t: p.logits(t)[-1], prompt, max_tokens=5)
    assert got == want
    assert "Prefill:" in out.stderr and "tokens in" in out.stderr and "ended by max_tokens" in out.stderr
    # --debug as the reference means it: ten candidates after the prompt, five for each of the first steps, the
    # first candidate being the token that greedy decoding took
    assert "[Prompt logits]" in out.stderr and "Top-10 tokens" in out.stderr and "[Token 3 logits]" in out.stderr
    assert "[Token 4 logits]" not in out.stderr
    firsts = [int(l.split("id=")[1]) for l in out.stderr.splitlines() if l.strip().startswith("1.")]
    assert firsts == want[:4]
    # random prompts by length, graphs off, statistics as JSON
    js = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "rocmforge"), "--model", folders("A"), "--dtype",
                         "float32", "--prompt-len", "9", "--prompt-len", "20", "--max-tokens", "4", "--temperature", "0",
                         "--stop-ids", "", "--no-graph", "--stats-json", "-"], capture_output=True, text=True)
    assert js.returncode == 0, js.stderr
    stats = json.loads(js.stdout.strip().splitlines()[-1])
    assert stats["prompt_tokens"] == 29 and stats["generated_tokens"] == 8 and stats["graphs"] is False
    assert [r["reason"] for r in stats["results"]] == ["max_tokens", "max_tokens"]
    bad = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "rocmforge"), "--model", folders("A"),
                          "--prompt-ids", "999"], capture_output=True, text=True)
    assert bad.returncode == 1 and "Error:" in bad.stderr
