"""Tiny configurations, folders with random weights, and comparison helpers for the tests."""
from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Three tiny configurations that differ in every size and option.
TINY_A = dict(   # grouped queries (4 heads on 2 kv heads), tied head, no window
    seed=0, architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
    num_key_value_heads=2, head_dim=16, intermediate_size=176, vocab_size=256, rope_theta=10000.0,
    rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=128, use_sliding_window=False,
    sliding_window=None, max_window_layers=2, eos_token_id=7)
TINY_B = dict(   # one kv head for 3 heads, untied head, other eps/theta, longer context
    seed=1, architectures=["Qwen2ForCausalLM"], num_hidden_layers=3, hidden_size=96, num_attention_heads=3,
    num_key_value_heads=1, head_dim=32, intermediate_size=240, vocab_size=384, rope_theta=1e6,
    rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=256, use_sliding_window=False,
    sliding_window=4096, max_window_layers=3)
TINY_C = dict(   # as many kv heads as heads, head_dim given and != hidden/heads, a window from layer 2 on
    seed=2, architectures=["Qwen2ForCausalLM"], num_hidden_layers=4, hidden_size=80, num_attention_heads=5,
    num_key_value_heads=5, head_dim=48, intermediate_size=112, vocab_size=300, rope_theta=50000.0,
    rms_norm_eps=3e-6, tie_word_embeddings=True, max_position_embeddings=512, use_sliding_window=True,
    sliding_window=24, max_window_layers=2, eos_token_id=[3, 5])
# Two more whose head sizes (64, 128) and widths let the bfloat16 engine take its tuned kernels (tcgen05 products
# of every orientation, tiled prefill attention, chunked decode attention) instead of the generic ones.
TINY_D = dict(   # head_dim 64, 2 query heads per kv head
    seed=3, architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=256, num_attention_heads=4,
    num_key_value_heads=2, head_dim=64, intermediate_size=328, vocab_size=520, rope_theta=1e6,
    rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=1024, use_sliding_window=False)
TINY_E = dict(   # head_dim 128, 8 query heads on one kv head, a window of 200 from layer 1 on
    seed=4, architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=320, num_attention_heads=8,
    num_key_value_heads=1, head_dim=128, intermediate_size=264, vocab_size=300, rope_theta=1e4,
    rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=1024, use_sliding_window=True,
    sliding_window=200, max_window_layers=1)
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E}

F32_ATOL, F32_RTOL = 2e-5, 1e-4          # maeddesg/ROCmForge compares at 1e-4 (tests/gpu_test_utils.rs:12)
BF16_REL_TO_MAX = 2e-2                   # bfloat16 path against the plain model on the same weights


def config_dict(cfg: dict) -> dict:
    return {k: v for k, v in cfg.items() if k != "seed"}


def write_tiny(cfg: dict, folder: str, dtype: str = "float32", device: str = "cpu") -> None:
    import rocmforge_b200 as rf
    from rocmforge_b200.config import Qwen2Config, architecture_for
    c = Qwen2Config.from_dict(config_dict(cfg))
    spec = architecture_for(c.architecture).build(c)
    dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    rf.write_model_folder(folder, c.to_dict(), spec.param_specs(), cfg["seed"], dt, device=device)


def random_tokens(vocab: int, n: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def assert_logits_close(got, ref, dtype: str, what: str = ""):
    got = torch.as_tensor(np.asarray(got), dtype=torch.float64)
    ref = torch.as_tensor(np.asarray(ref), dtype=torch.float64)
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    diff = (got - ref).abs()
    if dtype == "float32":
        bound = F32_ATOL + F32_RTOL * ref.abs()
    else:
        bound = torch.full_like(ref, BF16_REL_TO_MAX * float(ref.abs().max()))
    bad = diff > bound
    if bad.any():
        idx = torch.nonzero(bad)[0].tolist()
        raise AssertionError(f"{what}: {int(bad.sum())} of {bad.numel()} logits differ; first at {idx}: "
                             f"got {got[tuple(idx)].item():.6g}, plain {ref[tuple(idx)].item():.6g}, "
                             f"max diff {diff.max().item():.3g}")


class TraceRun:
    """Drives bin/trace_run as a child process, one step at a time."""

    def __init__(self, folder: str, dtype: str, out_dir: str, max_tokens: int, env=None):
        self.out_dir = out_dir
        self.vocab = json.load(open(os.path.join(folder, "config.json")))["vocab_size"]
        self.proc = subprocess.Popen(
            [os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out_dir,
             "--max-tokens", str(max_tokens)], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
        self.n = 0

    def step(self, entries, end=()):
        """entries: [(id, tokens, want)] -> float32 array [wanted, vocab] or None."""
        msg = {"step": self.n, "entries": [{"id": i, "tokens": list(t), "want": list(w)} for i, t, w in entries],
               "end": list(end)}
        self.proc.stdin.write(json.dumps(msg) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline().strip()
        assert line == f"done {self.n}", f"trace_run answered {line!r} (exit code {self.proc.poll()})"
        path = os.path.join(self.out_dir, f"{self.n}.f32")
        self.n += 1
        if any(len(w) for _, _, w in entries):
            return np.fromfile(path, dtype="<f4").reshape(-1, self.vocab)
        assert not os.path.exists(path)
        return None

    def close(self) -> int:
        self.proc.stdin.close()
        return self.proc.wait(timeout=120)
