#!/usr/bin/env python3
"""Decode and prefill throughput of the Qwen2.5-7B shape with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl ours|reference]

Prints ONE JSON line.  ``value`` is decoded tokens per second at the given batch, timed on
the device with CUDA events around K replayed decode steps whose sampled ids feed the next
step; ``e2e`` is the same rate through ``rocmforge_b200.LLM.generate`` with token ids going
in from the host and coming back to it every step (W warm-up steps, then K timed steps of one call); ``prefill`` is one step of 2,048 prompt
tokens; ``roofline`` relates the decode step to the HBM bandwidth; ``points`` holds batch 1
and batch 64.  maeddesg/ROCmForge publishes no number for this metric (its figures are for
4-bit weights on an RX 9070 XT), so ``vs_baseline`` is null.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "Qwen2.5-7B bf16 decode tok/s at batch 1/8/64; prefill tok/s at 2,048 tokens"

# BASELINE.json configs[2] (the headline), configs[3] and configs[4]
SHAPE_7B = dict(architectures=["Qwen2ForCausalLM"], num_hidden_layers=28, hidden_size=3584,
                num_attention_heads=28, num_key_value_heads=4, head_dim=128, intermediate_size=18944,
                vocab_size=152064, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False,
                use_sliding_window=False, max_position_embeddings=4096)
SHAPE_05B = dict(architectures=["Qwen2ForCausalLM"], num_hidden_layers=24, hidden_size=896,
                 num_attention_heads=14, num_key_value_heads=2, head_dim=64, intermediate_size=4864,
                 vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=True,
                 use_sliding_window=False, max_position_embeddings=32768)
SHAPE_14B = dict(architectures=["Qwen2ForCausalLM"], num_hidden_layers=48, hidden_size=5120,
                 num_attention_heads=40, num_key_value_heads=8, head_dim=128, intermediate_size=13824,
                 vocab_size=152064, rope_theta=1e6, rms_norm_eps=1e-5, tie_word_embeddings=False,
                 use_sliding_window=False, max_position_embeddings=32768)
CONTEXT = 4096
PROMPT_LEN = 512
PREFILL_TOKENS = 2048
SETTLE_STEPS = 48                    # untimed decode steps before any decode timing of the default run (see main)
PREFILL_CHUNK = 16384          # most prompt tokens run in one step when a batch of prompts is brought into the cache


def peaks():
    """Measured peaks if the driver wrote them, else the pool's earlier measurement."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    if os.path.exists(path):
        try:
            raw = json.load(open(path))
            out["hbm_gbs"] = float(raw.get("hbm_gbs", out["hbm_gbs"]))
            out["bf16_tflops"] = float(raw.get("bf16_tflops", out["bf16_tflops"]))
            if "bf16_tflops_sustained" in raw:
                out["bf16_tflops_sustained"] = float(raw["bf16_tflops_sustained"])
            if "sm_max_mhz" in raw:
                out["sm_max_mhz"] = float(raw["sm_max_mhz"])
            out["source"] = "measured"
        except Exception:
            pass
    return out


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass

    def summary(self, t0, t1):
        rows = [r for t, r in self.rows if t0 <= t <= t1] or [r for _, r in self.rows[-3:]]
        sm, mx, reasons = [], 0, set()
        for r in rows:
            try:
                sm.append(float(r[0]))
                mx = max(mx, float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def step_bytes(cfg, batch, mean_ctx, elem=2):
    """Bytes a decode step has to read: every weight it uses once, and the cache of the live requests
    (``mean_ctx`` positions per request on average); ``elem`` bytes per weight and cache element."""
    L, H, V = cfg.num_hidden_layers, cfg.hidden_size, cfg.vocab_size
    Q, KV, I = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim, cfg.intermediate_size
    per_layer = (H * (Q + 2 * KV) + Q * H + 3 * H * I) * elem + (Q + 2 * KV + 2 * H) * elem
    weights = L * per_layer + V * H * elem + H * elem          # a tied output matrix is read once, as the head
    kv = batch * mean_ctx * 2 * KV * elem * L
    return weights + kv


def prefill_flops(cfg, lengths):
    """Products and causal attention of whole prompts of the given lengths, logits for the last row of each."""
    L, H, V = cfg.num_hidden_layers, cfg.hidden_size, cfg.vocab_size
    Q, KV, I = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim, cfg.intermediate_size
    if isinstance(lengths, int):
        lengths = [lengths]
    T = float(sum(lengths))
    linear = 2.0 * T * (H * (Q + 2 * KV) + Q * H + 3 * H * I)
    attn = sum(2.0 * 2.0 * (t * (t + 1) / 2.0) * cfg.head_dim * cfg.num_attention_heads for t in lengths)
    return L * (linear + attn) + 2.0 * V * H * len(lengths)


def random_prompts(n, length, vocab, seed):
    """``length``: one length for all, or (low, high) for lengths drawn uniformly from that range (seeded)."""
    import torch
    g = torch.Generator().manual_seed(seed)
    if isinstance(length, tuple):
        lens = torch.randint(length[0], length[1] + 1, (n,), generator=g).tolist()
    else:
        lens = [length] * n
    return [torch.randint(0, vocab, (m,), generator=g).tolist() for m in lens]


def no_kernel_gave_up(model):
    """Raise if a bounded wait of a kernel ran out since the last look: a number timed over such a step means nothing."""
    from rocmforge_b200.kernels import tensor_core
    tensor_core.check_status(model.device)


def prefill_prompts(model, cache, slots, prompts):
    """Bring the prompts into the cache, at most PREFILL_CHUNK tokens a step; the argmax of each last row."""
    from rocmforge_b200 import StepRequest, kernels
    first, i = [], 0
    while i < len(prompts):
        j, t = i, 0
        while j < len(prompts) and (j == i or t + len(prompts[j]) <= PREFILL_CHUNK):
            t += len(prompts[j])
            j += 1
        logits = model.step(cache, [StepRequest(s, p, [len(p) - 1]) for s, p in zip(slots[i:j], prompts[i:j])])
        first += kernels.argmax(logits).cpu().tolist()
        i = j
    return first


class LoopMismatch(RuntimeError):
    pass


def check_loop(model, prompts, first, ids, n_check):
    """The ids that the device loop produced, compared with a second, untimed run of the same requests in which
    the host feeds every step (``DecodeRunner.logits`` + argmax): each of the first ``n_check`` steps gets the loop's
    own ids as input and must pick the loop's next ids, or differ only where the two best logits are a rounding
    error apart.  A position that did not advance or a page that was not reserved shows here."""
    import torch
    from rocmforge_b200 import kernels
    from rocmforge_b200.engine.graph import DecodeRunner
    B = len(prompts)
    n_check = min(n_check, ids.shape[0])
    cache = model.new_cache(max_tokens=sum((len(p) + n_check + 64) // 64 * 64 for p in prompts), max_slots=B)
    runner = DecodeRunner(model, cache)
    slots = [cache.alloc_slot() for _ in range(B)]
    again = prefill_prompts(model, cache, slots, prompts)
    if again != first:
        raise LoopMismatch("the prompts gave other first tokens on a second run")
    host_ids = ids[:n_check].cpu()
    feed = first
    for k in range(n_check):
        logits = runner.logits(slots, feed)
        got = kernels.argmax(logits).cpu()
        bad = torch.nonzero(got != host_ids[k]).flatten().tolist()
        for b in bad:
            row = logits[b]
            margin = abs(float(row[int(got[b])]) - float(row[int(host_ids[k][b])]))
            if margin > 2e-2 * float(row.abs().max()):
                raise LoopMismatch(f"step {k}, sequence {b}: the device loop picked {int(host_ids[k][b])}, "
                                   f"the checked step {int(got[b])} (logits {margin:.4g} apart)")
        feed = host_ids[k].tolist()
    return n_check


def decode_rate(model, prompts, steps, warmup, check=16):
    """Device-timed decode: the prompts in steps of at most PREFILL_CHUNK tokens, then ``steps`` replayed steps
    whose sampled ids feed the next step on the device.  The loop's ids are checked afterwards (``check`` steps)."""
    import torch
    from rocmforge_b200.engine.graph import DecodeRunner
    batch = len(prompts)
    cache = model.new_cache(max_tokens=sum((len(p) + warmup + steps + 64) // 64 * 64 for p in prompts), max_slots=batch)
    runner = DecodeRunner(model, cache)
    slots = [cache.alloc_slot() for _ in range(batch)]
    first = prefill_prompts(model, cache, slots, prompts)
    ids, _, _, _ = runner.greedy_loop(slots, first, warmup)
    torch.cuda.synchronize()
    t0 = time.time()
    ids2, start, end, launches = runner.greedy_loop(slots, ids[-1].cpu().tolist(), steps)
    torch.cuda.synchronize()
    t1 = time.time()
    ms = start.elapsed_time(end)
    mean_ctx = sum(len(p) for p in prompts) / batch + warmup + steps / 2.0
    all_ids = torch.cat([ids, ids2])
    del runner, cache
    torch.cuda.empty_cache()
    checked = check_loop(model, prompts, first, all_ids, check) if check else 0
    torch.cuda.empty_cache()
    no_kernel_gave_up(model)
    return {"tok_s": batch * steps / (ms / 1e3), "ms_per_step": ms / steps, "launches": launches * steps,
            "mean_ctx": mean_ctx, "t0": t0, "t1": t1, "checked_steps": checked}


def ablation(model, batch, steps=32, prompt_len=PROMPT_LEN):
    """Where a replayed decode step's time goes: every kind of kernel in turn is replaced by a stand-in that launches
    nothing and returns a buffer of the right shape, the step's graph is captured anew and timed.  The difference to
    the whole step is what that kernel costs inside the chain (with its overlaps), which a profiler's serialised,
    cold-cache replay does not show.  Results are garbage while a stand-in is in place; only the time is read."""
    import torch
    from rocmforge_b200 import kernels
    from rocmforge_b200.kernels import tensor_core as tc
    from rocmforge_b200.engine.graph import DecodeRunner
    cfg = model.config
    L = cfg.num_hidden_layers
    buffers = {}

    def buffer(key, shape, dtype):
        if key not in buffers:
            buffers[key] = torch.zeros(shape, dtype=dtype, device=model.device)
        return buffers[key]

    def run():
        cache = model.new_cache(max_tokens=batch * (prompt_len + 256), max_slots=batch)
        runner = DecodeRunner(model, cache)
        slots = [cache.alloc_slot() for _ in range(batch)]
        for s in slots:                                  # prompt_len cached positions (their content does not matter)
            cache.prepare([s], [prompt_len])
            cache.commit([s], [prompt_len])
        runner.greedy_loop(slots, [1] * batch, 4)
        torch.cuda.synchronize()
        _, start, end, _ = runner.greedy_loop(slots, [1] * batch, steps)
        torch.cuda.synchronize()
        return start.elapsed_time(end) / steps * 1e3     # us a step

    def no_norm(h, weight, eps, dt, pending=None, rows=None, out=None):
        return buffer(("norm", rows is None), (h.shape[0] if rows is None else rows.shape[0], h.shape[1]), dt)

    def no_rope(qkv, nh, nkv, hd, inv, *a, **kw):
        return buffer("q", (qkv.shape[1] if qkv.dim() == 3 else qkv.shape[0], nh * hd), torch.bfloat16)

    def no_attention(q, nh, nkv, hd, *a, **kw):
        return buffer("o", (q.shape[0], nh * hd), torch.bfloat16)

    real_skinny, real_resnorm = tc.gemm_tc_skinny, tc.gemm_tc_skinny_resnorm

    def without(pred):
        def f(x, w, bias=None, *, mode=tc.STORE, splits=1, out=None, row_ss=None):
            if not pred(w, mode):
                return real_skinny(x, w, bias, mode=mode, splits=splits, out=out, row_ss=row_ss)
            if out is not None:
                return out
            M, N = x.shape[0], w.shape[0]
            shape = (splits, M, N) if mode == tc.PARTIAL else (M, N // 2 if mode == tc.SWIGLU else N)
            return buffer(("gemm", shape, mode), shape, torch.bfloat16 if mode in (tc.STORE, tc.SWIGLU) else torch.float32)

        def g(x, w, bias, h, norm_weight, splits=1, row_ss=None):
            if not pred(w, tc.RESNORM):
                return real_resnorm(x, w, bias, h, norm_weight, splits=splits, row_ss=row_ss)
            M, N = x.shape[0], w.shape[0]
            return (buffer(("normed", M, N), (M, N), torch.bfloat16),
                    buffer(("ss", M, N), ((N + 127) // 128, M), torch.float32))
        return [(tc, "gemm_tc_skinny", f), (tc, "gemm_tc_skinny_resnorm", g)]

    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    QKV = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim
    cases = [("norm kernels (first layer and final norm when the others are fused)", [(kernels, "add_rmsnorm", no_norm)]),
             ("rotation + cache write", [(kernels, "rope_kv_write", no_rope)]),
             ("attention", [(kernels, "attention_decode_warps", no_attention)]),
             ("q|k|v product", without(lambda w, m: w.shape[0] == QKV and m == tc.PARTIAL)),
             ("o product", without(lambda w, m: tuple(w.shape) == (H, cfg.num_attention_heads * cfg.head_dim))),
             ("gate/up product", without(lambda w, m: m == tc.SWIGLU)),
             ("down product", without(lambda w, m: tuple(w.shape) == (H, I))),
             ("output matrix (per step)", without(lambda w, m: w.shape[0] == V)),
             ("all products", without(lambda w, m: True))]
    whole = run()
    rows = [{"kernel": "whole step", "us_per_step": round(whole, 1)}]
    for name, patches in cases:
        saved = [(module, attr, getattr(module, attr)) for module, attr, _ in patches]
        for module, attr, stand_in in patches:
            setattr(module, attr, stand_in)
        try:
            t = run()
        finally:
            for module, attr, real in saved:
                setattr(module, attr, real)
        per_step = "per step" in name or name == "all products"
        rows.append({"kernel": name, "us_per_step": round(whole - t, 1),
                     "us_per_layer": None if per_step else round((whole - t) / L, 2)})
    if model.options.fused_norm:
        # what fusing the norms into the products before them is worth: the same step with the norms as kernels
        model.options.fused_norm = False
        try:
            rows.append({"kernel": "whole step with the norms as kernels of their own", "us_per_step": round(run(), 1)})
        finally:
            model.options.fused_norm = True
    return rows


def e2e_rate(llm, prompts, steps, temperature=0.0, top_p=1.0, warmup=0):
    """The same through LLM.generate: token ids from the host in, sampled ids back to the host, every step.  One call
    generates warmup + steps + 1 tokens per request; the time of the last ``steps`` decode steps counts (the steps right
    after a batch of prompts run at lower clocks for some tens of milliseconds: the power cap after the prompts' burst)."""
    import torch
    batch = len(prompts)
    stamps = []

    def on_token(i, tok):
        if i == 0:
            stamps.append(time.perf_counter())
    llm.generate(prompts, max_tokens=min(steps, 8) + 1, temperature=temperature, top_p=top_p, stop_token_ids=[])     # warm-up, graphs
    stamps.clear()
    out = llm.generate(prompts, max_tokens=warmup + steps + 1, temperature=temperature, top_p=top_p, stop_token_ids=[],
                       on_token=on_token)
    torch.cuda.synchronize()
    no_kernel_gave_up(llm.model)
    stamps = stamps[warmup:]
    n = len(stamps) - 1
    dt = stamps[-1] - stamps[0]
    from rocmforge_b200.engine.batch import StepBatch
    h2d = StepBatch.layout(batch, batch, batch, decode_extras=True)[1] * 4 + batch * 4 / 64.0     # descriptor + a block-table entry per 64 steps
    return {"value": batch * n / dt, "unit": "tok/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": batch * 4,
            "steps": n, "generated": sum(len(r.tokens) for r in out)}


def prefill_rate(model, tokens, repeats, seed):
    """Median time in ms of one step that runs a prompt of ``tokens`` tokens and gives the last row's logits."""
    import torch
    from rocmforge_b200 import StepRequest
    cache = model.new_cache(max_tokens=tokens + 64, max_slots=2)
    prompt = random_prompts(1, tokens, model.spec.vocab_size, seed)[0]
    times = []
    for r in range(repeats + 1):
        s = cache.alloc_slot()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        model.step(cache, [StepRequest(s, prompt, [tokens - 1])])
        end.record()
        torch.cuda.synchronize()
        if r > 0:                                       # the first run warms up
            times.append(start.elapsed_time(end))
        cache.free_slot(s)
    times.sort()
    del cache
    torch.cuda.empty_cache()
    no_kernel_gave_up(model)
    return times[len(times) // 2]


def other_shapes(pk, seed, only=None):
    """BASELINE.json's two further configurations, as flat numbers for ``points``: the 0.5B shape in bfloat16 and in
    true 32-bit (a batch of 64 with prompt lengths uniform in 16..1,024, 256 decode steps; device-timed, its share of
    the HBM bandwidth, and end to end), and the 14B shape (a prompt of 8,192 tokens; decoding at batch 1 and 16 at
    that context)."""
    import torch
    import rocmforge_b200 as rf
    from rocmforge_b200.config import Qwen2Config
    out = {}
    hbm, tf = pk["hbm_gbs"], pk["bf16_tflops"]
    if only in (None, "0.5b"):
        cfg = Qwen2Config.from_dict(SHAPE_05B)
        prompts = random_prompts(64, (16, 1024), cfg.vocab_size, seed + 10)
        for dtype, tag, elem in ((torch.bfloat16, "bf16", 2), (torch.float32, "fp32", 4)):
            model = rf.Model.random(cfg, seed=seed, dtype=dtype)
            r = decode_rate(model, prompts, 256, 8)
            key = f"qwen0.5b_{tag}_b64_ragged"
            out[key + "_tok_s"] = round(r["tok_s"], 1)
            out[key + "_ms_per_step"] = round(r["ms_per_step"], 4)
            out[key + "_hbm_frac"] = round(step_bytes(cfg, 64, r["mean_ctx"], elem) / (r["ms_per_step"] / 1e3) / 1e9 / hbm, 4)
            llm = rf.LLM(model, cache_tokens=sum((len(p) + 256 + 80) // 64 * 64 for p in prompts), max_batch=64)
            out[key + "_e2e_tok_s"] = round(e2e_rate(llm, prompts, 128 if elem == 2 else 32, warmup=8)["value"], 1)
            del llm
            if elem == 4:
                # the 32-bit products run on the CUDA cores: 148 SMs x 128 lanes x 2 flops at the highest SM clock
                ffma = 148 * 128 * 2 * pk.get("sm_max_mhz", 1965.0) * 1e6
                ms = prefill_rate(model, PREFILL_TOKENS, 2, seed + 13)
                out["qwen0.5b_fp32_prefill2048_tok_s"] = round(PREFILL_TOKENS / (ms / 1e3), 1)
                out["qwen0.5b_fp32_prefill2048_ffma_frac"] = round(prefill_flops(cfg, PREFILL_TOKENS) / (ms / 1e3) / ffma, 4)
            del model
            torch.cuda.empty_cache()
    if only in (None, "14b"):
        cfg = Qwen2Config.from_dict(SHAPE_14B)
        model = rf.Model.random(cfg, seed=seed, dtype=torch.bfloat16)
        ms = prefill_rate(model, 8192, 2, seed + 11)
        out["qwen14b_prefill8192_tok_s"] = round(8192 / (ms / 1e3), 1)
        out["qwen14b_prefill8192_ms"] = round(ms, 2)
        out["qwen14b_prefill8192_frac"] = round(prefill_flops(cfg, 8192) / (ms / 1e3) / (tf * 1e12), 4)
        for batch in (1, 16):
            prompts = random_prompts(batch, 8192 - 48, cfg.vocab_size, seed + 12 + batch)
            r = decode_rate(model, prompts, 32, 8, check=4)
            key = f"qwen14b_decode_b{batch}_ctx8192"
            out[key + "_tok_s"] = round(r["tok_s"], 1)
            out[key + "_hbm_frac"] = round(step_bytes(cfg, batch, r["mean_ctx"]) / (r["ms_per_step"] / 1e3) / 1e9 / hbm, 4)
        del model
        torch.cuda.empty_cache()
    return out


def reference_arm():
    # maeddesg/ROCmForge is a Rust crate with HIP kernels for AMD GPUs: it has no Python package to
    # install with pip, no Rust toolchain is present, and it has no CUDA path or bf16/safetensors support.
    print(json.dumps({"impl": "reference",
                      "unavailable": "maeddesg/ROCmForge is a Rust+HIP (AMD ROCm) crate: not pip-installable, "
                                     "no cargo/rustc/hipcc here, no CUDA or bf16 path to run on a B200"}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="only the headline batch (quick check)")
    ap.add_argument("--only", choices=["decode", "prefill", "ablate", "0.5b", "14b"], default=None,
                    help="run one phase only and print a short line (small cases for profilers)")
    ap.add_argument("--shape", choices=["7b", "0.5b", "14b"], default="7b",
                    help="layer sizes for --only decode / prefill / ablate (the full run always measures all three)")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN, help="prompt length of --only decode / ablate")
    ap.add_argument("--fused-norm", action="store_true", help="--only runs: products of few tokens prepare the norm that follows")
    ap.add_argument("--fused-norm-max", type=int, default=None,
                    help="--only runs: most tokens of a step for which products prepare the norm that follows them")
    ap.add_argument("--dtype", choices=["bf16", "fp32"], default="bf16", help="--only decode / prefill: the bfloat16 or the true 32-bit path")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS, help="--only prefill: tokens of the prompt")
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not measured")
        return 2
    warmup = max(args.warmup, 3)

    import torch
    import rocmforge_b200 as rf
    from rocmforge_b200.config import Qwen2Config

    pk = peaks()
    if args.only in ("0.5b", "14b"):
        print(json.dumps({"only": args.only, **other_shapes(pk, args.seed, args.only)}))
        return 0
    raw = dict({"7b": SHAPE_7B, "0.5b": SHAPE_05B, "14b": SHAPE_14B}[args.shape if args.only else "7b"])
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    cfg = Qwen2Config.from_dict(raw)
    V = cfg.vocab_size
    model = rf.Model.random(cfg, seed=args.seed, dtype=torch.float32 if (args.only and args.dtype == "fp32") else torch.bfloat16)
    if args.only and args.fused_norm:
        model.options.fused_norm = True
    if args.only and args.fused_norm_max is not None:
        model.options.fused_norm_max_tokens = args.fused_norm_max

    if args.only == "decode":
        r = decode_rate(model, random_prompts(args.batch, args.prompt_len, V, args.seed), args.steps, warmup)
        print(json.dumps({"only": "decode", "shape": args.shape, "layers": cfg.num_hidden_layers, "batch": args.batch,
                          "ms_per_step": round(r["ms_per_step"], 4), "tok_s": round(r["tok_s"], 1),
                          "checked_steps": r["checked_steps"]}))
        return 0
    if args.only == "ablate":
        for row in ablation(model, args.batch, prompt_len=args.prompt_len):
            print(json.dumps(row))
        return 0
    if args.only == "prefill":
        ms = prefill_rate(model, args.prefill_tokens, 4, args.seed + 2)
        print(json.dumps({"only": "prefill", "shape": args.shape, "layers": cfg.num_hidden_layers, "tokens": args.prefill_tokens,
                          "ms": round(ms, 3),
                          "frac": round(prefill_flops(cfg, args.prefill_tokens) / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}))
        return 0
    # the prompt step first, and few of them: a few steps of 25 ms are a burst, like the product the peak was measured
    # with (nine in a row run into the power cap and come out 5 % slower: that is the sustained figure's case)
    pre_ms = prefill_rate(model, PREFILL_TOKENS, 3, args.seed + 2)
    sampler = ClockSampler()
    sampler.start()
    # Steady decoding is what every decode number of this run means.  The steps right after a batch of prompts run at
    # lower clocks (the power cap after the prompts' burst: 8 prompts of 512 tokens are 45 ms at full power, and the
    # next 17 or so decode steps take 2.9 ms instead of 2.6), so each timing runs max(W, SETTLE_STEPS) untimed steps
    # first and then times exactly K; what the first steps after the prompts give end to end stands in `points`.
    settle = max(warmup, SETTLE_STEPS)
    main_run = decode_rate(model, random_prompts(args.batch, PROMPT_LEN, V, args.seed), args.steps, settle)
    clocks = sampler.summary(main_run["t0"], main_run["t1"])
    llm = rf.LLM(model, cache_tokens=args.batch * (PROMPT_LEN + settle + args.steps + 80), max_batch=args.batch)
    e2e = e2e_rate(llm, random_prompts(args.batch, PROMPT_LEN, V, args.seed + 1), args.steps, warmup=settle)
    e2e["untimed_steps"] = settle
    e2e_first = e2e_rate(llm, random_prompts(args.batch, PROMPT_LEN, V, args.seed + 1), args.steps, warmup=warmup)
    # the reference's own default is sampled decoding (temperature 1.0, top-p 0.9): the same loop with the device sampler
    sampled = e2e_rate(llm, random_prompts(args.batch, PROMPT_LEN, V, args.seed + 5), max(args.steps // 2, 16),
                       temperature=1.0, top_p=0.9, warmup=settle)
    llm.cache = llm.engine = None
    del llm
    torch.cuda.empty_cache()
    points = {}
    if not args.skip_points:
        for b, st in ((1, args.steps), (64, max(args.steps // 2, 16))):
            r = decode_rate(model, random_prompts(b, PROMPT_LEN, V, args.seed + 3 + b), st, settle)
            points[f"decode_b{b}"] = round(r["tok_s"], 1)
            points[f"decode_b{b}_hbm_frac"] = round(step_bytes(cfg, b, r["mean_ctx"]) / (r["ms_per_step"] / 1e3) / 1e9
                                                   / pk["hbm_gbs"], 4)
    points["e2e_sampled_t1.0_p0.9"] = round(sampled["value"], 1)
    points[f"e2e_steps_{warmup + 1}_to_{warmup + args.steps}_after_the_prompts"] = round(e2e_first["value"], 1)
    nbytes = step_bytes(cfg, args.batch, main_run["mean_ctx"])
    achieved = nbytes / (main_run["ms_per_step"] / 1e3) / 1e9
    flops = prefill_flops(cfg, PREFILL_TOKENS)
    del model
    torch.cuda.empty_cache()
    if not args.skip_points:
        points.update(other_shapes(pk, args.seed))
    sampler.stop()

    line = {
        "metric": METRIC, "value": round(main_run["tok_s"], 1), "unit": "tok/s", "n_gpus": 1,
        "steps": args.steps, "warmup": warmup, "untimed_steps": settle, "ms_per_step": round(main_run["ms_per_step"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random token ids, random-init weights N(0, 0.02)", "impl": "ours",
        "config": {"model": "Qwen2.5-7B shape", "layers": cfg.num_hidden_layers, "layers_of_config": 28,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN,
                   "context_at_timing": int(main_run["mean_ctx"]), "parallelism": "none (1 GPU)",
                   "cache_page": 64, "l2": "inputs larger than L2 (15 GB of weights per step)",
                   "peaks": pk["source"],
                   "decode_timing": f"value, e2e, decode_b1, decode_b64: prompts of {PROMPT_LEN} tokens, {settle} untimed decode "
                                    "steps (the clocks settle after the prompts' burst), then exactly `steps` timed",
                   "points_qwen0.5b": "Qwen2.5-0.5B shape, 24 layers, hidden 896, 14/2 heads of 64, intermediate 4864, "
                                      "vocab 151936 tied; batch 64, prompts uniform 16..1024 (seeded), 256 steps; bf16 and fp32",
                   "points_qwen14b": "Qwen2.5-14B shape, 48 layers, hidden 5120, 40/8 heads of 128, intermediate 13824, "
                                     "vocab 152064; prefill 8192 at batch 1, decode batch 1 and 16 at context 8192, 32 steps"},
        "e2e": e2e,
        "gpu_launches": main_run["launches"],
        "loop_ids_checked_steps": main_run["checked_steps"],
        "clocks": clocks,
        "prefill": {"value": round(PREFILL_TOKENS / (pre_ms / 1e3), 1), "tokens": PREFILL_TOKENS,
                    "ms": round(pre_ms, 3), "frac": round(flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
