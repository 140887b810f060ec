#!/usr/bin/env python3
"""Throughput of the engine at Qwen3-8B layer sizes with random weights, on one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--batch 8] [--layers L] [--prompt-len 2048] [--context 4096]

A "step" is one decode step of a batch of sequences that were prefilled to --prompt-len tokens.
`value` is decoded tokens per second of K steps timed on the device (CUDA events, after W warm-up
steps); every step reads all weights (about 15 GB, far larger than the 126 MB L2), so no flush is
needed between steps.  `e2e` is the same through the Python entry point with host tokens in and
out of every step, over at least 64 steps that follow an untimed round (which holds the capture of
the step's CUDA graph).  `prefill` times one 2,048-token prompt through `Engine.step` (host packing
and upload included); `points` holds decode at batch 1 and 64 and, unless --no-workloads, the two
other workloads the baseline names, run through `generate` and timed by its own statistics on the
host: 16 unequal prompts of 32 to 1,024 tokens with 256 decode steps at Qwen3-0.6B sizes, and 8
prompts of 1,024 tokens with 128 decode steps at Qwen3-32B sizes.  `fp32_check` compares the
bfloat16 engine with the true 32-bit engine on the same full-size model (a 64-token prompt).
One JSON line goes to standard output.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=4096,
                num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                intermediate_size=12288, rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=40960,
                tie_word_embeddings=False, eos_token_id=151645)
# The other two sizes the reference architecture is usually quoted at (same layer formulas).
SIZES = {
    "8b": {},
    "0.6b": dict(hidden_size=1024, num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8,
                 intermediate_size=3072, tie_word_embeddings=True),
    "32b": dict(hidden_size=5120, num_hidden_layers=64, num_attention_heads=64, num_key_value_heads=8,
                intermediate_size=25600),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "source": "measured"}
    except (OSError, KeyError, ValueError):
        return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        def pump():
            for line in self.proc.stdout:
                self.rows.append((time.time(), line.strip()))
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, windows) -> dict:
        sm, mx, reasons = [], [], set()
        for ts, line in self.rows:
            if not any(a <= ts <= b for a, b in windows):
                continue
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm() -> int:
    # The reference is a Rust workspace (Cargo.toml, no setup.py / pyproject.toml): pip cannot
    # install it, there is no Rust toolchain in this image, and its GPU backends need Vulkan or Metal.
    print(json.dumps({"impl": "reference", "unavailable":
                      "xigh/herbert-rs is a Rust workspace with Vulkan/Metal GPU backends: no Python package to install offline, no cargo/rustc in the image, no graphics stack on the box"}))
    return 0


WORKLOADS = {
    # the baseline's fourth and fifth configurations (Qwen3-0.6B and Qwen3-32B layer sizes), as written there
    "0.6b": dict(size="0.6b", prompts=16, min_len=32, max_len=1024, steps=256),
    "32b": dict(size="32b", prompts=8, min_len=1024, max_len=1024, steps=128),
}


def run_workload(name: str, windows: list) -> dict:
    """One of the baseline's other workloads through the public `generate`: decode tokens per second
    by the loop's own statistics (host clock around the decode steps, tokens read back every step)."""
    import numpy as np
    import torch

    import herbert_rs_b200 as hb

    w = WORKLOADS[name]
    cfg = dict(QWEN3_8B)
    cfg.update(SIZES[w["size"]])
    rng = np.random.default_rng(1)
    lens = [int(n) for n in rng.integers(w["min_len"], w["max_len"] + 1, w["prompts"])]
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in lens]
    rt = hb.Runtime("cuda", torch.bfloat16)
    model = hb.random_model(cfg, 0, rt)
    per_seq = max(lens) + w["steps"] + 1
    engine = hb.Engine(model, max_tokens=hb.Engine.pages_for(per_seq, w["prompts"]) * rt.page_size, max_slots=w["prompts"])
    opt = hb.GenerationOptions(max_tokens=w["steps"] + 1, ignore_eos=True)      # the first token comes from the prompts' step
    greedy = hb.SamplingParams(temperature=0.0)
    hb.generate(engine, prompts, hb.GenerationOptions(max_tokens=12, ignore_eos=True), greedy)    # untimed: graph capture, workspace growth
    torch.cuda.synchronize()
    t0 = time.time()
    res = hb.generate(engine, prompts, opt, greedy)
    windows.append((t0, time.time()))
    st = res.stats
    out = {"decode_tok_s": round(st.decode_tokens_per_second, 1), "prefill_tok_s": round(st.prefill_tokens_per_second, 1),
           "decode_steps": st.decode_steps, "prompt_tokens": st.prompt_tokens, "ms_per_step": round(st.decode_seconds / max(1, st.decode_steps) * 1e3, 4),
           "layers": cfg["num_hidden_layers"], "prompts": w["prompts"]}
    del engine, model
    torch.cuda.empty_cache()
    return out


def fp32_check(cfg: dict, bf16_engine, n_tokens: int = 64) -> dict:
    """The bfloat16 engine against the true 32-bit engine on the same model (same seed, same
    weights: bfloat16 values widened exactly) at full size: logits at every position of a prompt."""
    import numpy as np
    import torch

    import herbert_rs_b200 as hb

    ids = np.random.default_rng(7).integers(0, cfg["vocab_size"], n_tokens).tolist()
    s = bf16_engine.alloc_slot()
    low = bf16_engine.step([(s, ids)], "all").double().cpu()
    bf16_engine.free_slot(s)
    rt = hb.Runtime("cuda", torch.float32)
    eng = hb.Engine(hb.random_model(cfg, 0, rt), max_tokens=hb.Engine.pages_for(n_tokens) * rt.page_size, max_slots=1)
    s = eng.alloc_slot()
    ref = eng.step([(s, ids)], "all").double().cpu()
    eng.free_slot(s)
    eng.check_kernels()
    del eng
    torch.cuda.empty_cache()
    top2 = ref.topk(2, dim=-1).values
    gap = top2[:, 0] - top2[:, 1]
    differ = low.argmax(-1) != ref.argmax(-1)
    # where the two engines choose another token, how far apart the 32-bit engine's two best logits were there,
    # and how much lower it rates the bfloat16 engine's choice: both small against max_abs_err if the choice was a near-tie
    lost = (ref.max(-1).values - ref.gather(1, low.argmax(-1, keepdim=True))[:, 0])
    return {"tokens": n_tokens, "layers": cfg["num_hidden_layers"], "max_abs_err": round(float((low - ref).abs().max()), 5),
            "logit_std": round(float(ref.std()), 4), "argmax_agree": round(float((~differ).double().mean()), 4),
            "median_top2_gap": round(float(gap.median()), 5),
            "largest_gap_where_they_differ": round(float(gap[differ].max()) if bool(differ.any()) else 0.0, 5),
            "largest_logit_given_up": round(float(lost.max()), 5)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--size", default="8b", choices=sorted(SIZES), help="layer sizes: Qwen3-8B (the headline), 0.6B or 32B")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the size has (both numbers are reported)")
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 decode points")
    ap.add_argument("--no-prefill", action="store_true", help="skip the 2,048-token prefill measurement")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end measurement")
    ap.add_argument("--no-workloads", action="store_true", help="skip the 0.6B and 32B workloads of the baseline")
    ap.add_argument("--no-fp32-check", action="store_true", help="skip the comparison with the 32-bit engine")
    ap.add_argument("--no-pdl", action="store_true", help="prompts without programmatic dependent launch")
    ap.add_argument("--pdl-graph", type=int, default=None, help="programmatic dependent launch inside recorded decode steps (0, 1, 2)")
    ap.add_argument("--workload", default=None, choices=["0.6b", "32b"],
                    help="run only this workload of the baseline and print its line")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py measures one GPU only (asked for {args.gpus}): this library has no multi-GPU path")
        return 2
    args.warmup = max(args.warmup, 3)
    if args.workload is not None:
        sampler, windows = ClockSampler(), []
        sampler.start()
        out = run_workload(args.workload, windows)
        sampler.stop()
        w = WORKLOADS[args.workload]
        print(json.dumps({"metric": f"Qwen3-{w['size'].upper()} decode tok/s through generate ({w['prompts']} prompts of {w['min_len']}..{w['max_len']} tokens, {w['steps']} steps)",
                          "value": out["decode_tok_s"], "unit": "tokens/s", "n_gpus": 1, "impl": "ours", "dtype": "bf16",
                          "data": "synthetic", "workload": out, "clocks": sampler.summary(windows)}))
        return 0

    import numpy as np
    import torch

    import herbert_rs_b200 as hb
    from herbert_rs_b200 import ops
    from herbert_rs_b200.sampling import device_choose

    if args.no_pdl:
        ops.options.pdl_eager = False
    if args.pdl_graph is not None:
        ops.options.pdl_graph = args.pdl_graph
    pk = peaks()
    cfg = dict(QWEN3_8B)
    cfg.update(SIZES[args.size])
    layers_full = cfg["num_hidden_layers"]
    if args.layers is None:
        args.layers = layers_full
    cfg["num_hidden_layers"] = args.layers
    rt = hb.Runtime("cuda", torch.bfloat16)
    model = hb.random_model(cfg, 0, rt)
    max_b = args.batch if args.no_points else max(args.batch, 64)
    engine = hb.Engine(model, max_tokens=max_b * args.context, max_slots=max_b, max_seq_len=args.context)
    rng = np.random.default_rng(0)
    V = cfg["vocab_size"]
    greedy = hb.SamplingParams(temperature=0.0)
    sampler = ClockSampler()
    sampler.start()
    windows = []

    def events():
        return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def prefill_batch(B):
        slots = [engine.alloc_slot() for _ in range(B)]
        for s in slots:                      # one prompt per step keeps the workspace at prefill size
            engine.step([(s, rng.integers(0, V, args.prompt_len).tolist())], None)
        return slots

    def decode_device(B, steps, warmup):
        """K decode steps timed on the device: step buffer upload, graph replay, argmax."""
        slots = prefill_batch(B)
        toks = rng.integers(0, V, (steps + warmup, B)).tolist()
        out = torch.empty(B, dtype=torch.int32, device="cuda")
        def one(i):
            batch = engine._prepare([(s, [toks[i][j]]) for j, s in enumerate(slots)], "last")
            logits = engine._forward(batch)
            engine._finish(batch)
            device_choose(logits, greedy, batch.uniforms, out)
        for i in range(warmup):
            one(i)
        torch.cuda.synchronize()
        lens = [engine.length(s) for s in slots]
        e0, e1 = events()
        t0 = time.time()
        e0.record()
        for i in range(warmup, warmup + steps):
            one(i)
        e1.record()
        torch.cuda.synchronize()
        windows.append((t0, time.time()))
        ms = e0.elapsed_time(e1)
        ops.check_kernel_errors()
        for s in slots:
            engine.free_slot(s)
        mean_len = sum(lens) / B + (steps + 1) / 2.0
        return ms / steps, mean_len

    def decode_e2e(B, steps, warmup):
        """The same through the public call: host token ids in, host token ids out, every step."""
        slots = prefill_batch(B)
        last = rng.integers(0, V, B).tolist()
        for _ in range(warmup):
            last = engine.step_and_choose([(s, [t]) for s, t in zip(slots, last)], greedy)
        torch.cuda.synchronize()
        t0 = time.time()
        for _ in range(steps):
            last = engine.step_and_choose([(s, [t]) for s, t in zip(slots, last)], greedy)
        dt = time.time() - t0
        windows.append((t0, t0 + dt))
        h2d, d2h = engine.h2d_bytes_last, engine.d2h_bytes_last
        for s in slots:
            engine.free_slot(s)
        return dt / steps, h2d, d2h

    result = {}
    # ---- prefill of one prompt -------------------------------------------------------------------
    if not args.no_prefill:
        T = args.prompt_len
        times = []
        for i in range(3 + 3):
            s = engine.alloc_slot()
            ids = rng.integers(0, V, T).tolist()
            e0, e1 = events()
            t0 = time.time()
            e0.record()
            engine.step([(s, ids)], "last")          # host packing, upload, every kernel, logits of the last token
            e1.record()
            torch.cuda.synchronize()
            engine.free_slot(s)
            if i >= 3:
                times.append(e0.elapsed_time(e1))
                windows.append((t0, time.time()))
        ms = statistics.median(times)
        c = model.config
        per_layer = 2 * T * (c.hidden_size * (c.q_dim + 2 * c.kv_dim) + c.q_dim * c.hidden_size + 3 * c.hidden_size * c.intermediate_size)
        attn = 4 * c.num_attention_heads * c.head_dim * T * (T + 1) // 2
        flops = args.layers * (per_layer + attn) + 2 * c.hidden_size * c.vocab_size
        result["prefill"] = {"value": round(T / (ms / 1e3), 1), "tokens": T, "ms": round(ms, 3),
                             "frac": round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}

    # ---- the headline: decode at --batch -----------------------------------------------------------
    B = args.batch
    launches0 = ops.launch_count()
    ms_step, mean_len = decode_device(B, args.steps, args.warmup)
    kernels_per_step = engine.kernels_per_graph.get(B, 0) + 1       # + the argmax launch
    value = B / (ms_step / 1e3)
    step_bytes = model.weight_bytes(rows=B) + int(B * mean_len * engine.cache.bytes_per_token())
    achieved = step_bytes / (ms_step / 1e3) / 1e9
    result["roofline"] = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                          "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"]}
    if not args.no_e2e:
        s_step, h2d, d2h = decode_e2e(B, max(64, args.steps), max(8, args.warmup))
        result["e2e"] = {"value": round(B / s_step, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}
    if not args.no_points:
        pts = {}
        for b in (1, 64):
            ms_b, _ = decode_device(b, max(8, args.steps // 2), args.warmup)
            pts[f"decode_b{b}"] = round(b / (ms_b / 1e3), 1)
        result["points"] = pts
    if not args.no_fp32_check:
        result["fp32_check"] = fp32_check(cfg, engine)
    if not args.no_workloads and args.size == "8b" and args.layers == layers_full:
        del engine, model
        torch.cuda.empty_cache()
        for name in ("0.6b", "32b"):
            out = run_workload(name, windows)
            result.setdefault("points", {})[f"qwen3_{name}_workload_decode"] = out["decode_tok_s"]
            result.setdefault("workloads", {})[name] = out
    sampler.stop()
    clocks = sampler.summary(windows)

    line = {
        "metric": "Qwen3-8B decode tok/s at batch 1, 8, 64; prefill tok/s at 2,048 tokens",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded uniform-random token ids, random-init weights N(0, 0.02)",
        "impl": "ours", "gpu_launches": kernels_per_step * args.steps,
        "config": {"model": f"Qwen3-{args.size.upper()} layer sizes", "layers": args.layers, "layers_full": layers_full,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "global_batch": B, "seq_len": args.prompt_len, "context": args.context, "parallelism": "single-gpu",
                   "page_size": rt.page_size, "l2": "inputs larger than L2 (all weights read every step)",
                   "cache_fill": "prefill of random prompts", "kernels_per_step": kernels_per_step,
                   "timing": "value: CUDA events around upload + graph replay + argmax; e2e: host clock, tokens in and out"},
        "clocks": clocks,
    }
    line.update(result)
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
