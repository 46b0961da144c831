#!/usr/bin/env python3
"""Decode and prefill throughput of rust-inference_b200 at Qwen3-8B shapes on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step of the whole batch.  The default run has the layer
sizes of Qwen3-8B with random bfloat16 weights, a batch of 8 and a context of
4,096 tokens: every sequence's cache is filled so that the W warm-up and K timed
steps end at exactly 4,096 tokens.  One JSON line is printed:

  value      decoded tokens a second at batch 8, timed on the device with CUDA
             events around the K steps (step function plus greedy selection)
  e2e        the same through the Python entry point (LLM.generate): token ids
             from host memory in, token ids back to the host every step
  prefill    a 2,048-token prompt in one step; frac = flops / time / bf16 peak
  roofline   decode step: bytes it has to read (every weight once, the cache of
             the live requests) / time, against the copy bandwidth
  points     decode tokens a second at batch 1 and 64 (device-timed), and the same through
             the Python entry point (e2e_b1, e2e_b64)

    python bench.py --workload 14b | 32b

runs the workloads that the reference's figures are quoted on for the larger sizes, whole
and through the Python entry point (LLM.generate, host token ids in and out): Qwen3-14B
shapes with 16 unequal prompts of 256 to 2,048 tokens and 256 greedy steps, Qwen3-32B shapes
with 8 prompts of 1,024 tokens and 512 steps at temperature 0.7.  One JSON line each: decode
tokens a second (value), ms per step, the prompts' tokens a second with their fraction of the
bf16 peak, and the decode step's fraction of the copy bandwidth for its own bytes.

Peaks come from MEASURED_PEAKS.json beside this file when it exists, else from
the fallback figures (6.65 TB/s, 1.59 PFLOP/s).  A decode step reads more than
15 GB of weights, far more than the 126 MB of L2, so no L2 flush is needed
between timed steps.
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

QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 36, "hidden_size": 4096,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
    "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 40960,
}
# the other sizes the reference's measurements name (the same family, other widths and depths): --model
SHAPES = {
    "8b": {},
    "14b": {"num_hidden_layers": 40, "hidden_size": 5120, "num_attention_heads": 40, "intermediate_size": 17408},
    "32b": {"num_hidden_layers": 64, "hidden_size": 5120, "num_attention_heads": 64, "intermediate_size": 25600},
}
CONTEXT = 4096
PREFILL_TOKENS = 2048
METRIC = "decode tok/s at batch 8, context 4096 (Qwen3-8B shapes, bf16)"


def peaks():
    hbm, tf, src = 6650.0, 1590.0, "fallback"
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            with open(p) as f:
                d = json.load(f)
            hbm = float(d.get("hbm_gbs", hbm))
            tf = float(d.get("bf16_tflops", tf))
            src = "measured"
        except (OSError, ValueError):
            pass
    return hbm, tf, src


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs (read-only)."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [x.strip() for x in line.split(",")]))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, windows):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, r in self.rows:
            if len(r) < 6 or not any(a <= t <= b for a, b in windows):
                continue
            try:
                sm.append(int(float(r[0])))
                mx = max(mx, int(float(r[1])))
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm() -> dict:
    """The reference is a Rust crate whose engine is the `runner` binary (src/bin/runner.rs): look for a Rust
    toolchain, build the crate with its CUDA backend from the copy under baseline/_ref, and say which step
    failed.  Where it can be built it still cannot run this metric: its runner takes one text prompt (batch 1,
    a tokenizer folder) and its checkpoint script has no Qwen3-8B preset (scripts/synthetic_checkpoint.py:18-35)."""
    import shutil
    why = None
    cargo = shutil.which("cargo")
    ref = os.path.join(ROOT, "baseline", "_ref")
    if cargo is None or shutil.which("rustc") is None:
        why = ("thanhauco/rust-inference is a Rust crate (Cargo.toml, no Python package); cargo and rustc "
               "are not installed here and pip finds nothing to install")
    elif not os.path.exists(os.path.join(ref, "Cargo.toml")):
        why = "cargo was found, but there is no copy of the reference under baseline/_ref to build"
    else:
        try:
            r = subprocess.run([cargo, "build", "--release", "--offline", "--features", "cuda", "--bin", "runner"],
                               cwd=ref, capture_output=True, text=True, timeout=3000)
            if r.returncode != 0:
                tail = r.stderr.strip().splitlines()[-1] if r.stderr.strip() else "no message"
                why = f"cargo build --offline --features cuda failed: {tail}"
            else:
                why = ("the reference's runner was built, but it generates for one text prompt at batch 1 with a "
                       "tokenizer folder: it has no batch-8 decode at Qwen3-8B shapes to time")
        except (OSError, subprocess.TimeoutExpired) as e:
            why = f"cargo build did not finish: {e}"
    return {"impl": "reference", "unavailable": why}


def prefill_flops(cfg, lens) -> float:
    """Matrix products of the layers for every token, the head for one row per sequence, causal attention."""
    L, D, H, KV, Dh, I, V = (cfg[k] for k in ("num_hidden_layers", "hidden_size", "num_attention_heads",
                                               "num_key_value_heads", "head_dim", "intermediate_size", "vocab_size"))
    layer_params = D * (H + 2 * KV) * Dh + H * Dh * D + 3 * D * I
    total = 0.0
    for T in lens:
        total += 2.0 * T * layer_params * L + 2.0 * D * V + 4.0 * Dh * H * T * (T + 1) / 2 * L
    return total


WORKLOADS = {
    # BASELINE.json configs[3] and [4]: what the reference names beside its figures for these sizes
    "14b": dict(model="14b", batch=16, prompt=(256, 2048), steps=256, temperature=0.0,
                what="16 unequal prompts uniform in [256, 2048] tokens, then 256 greedy decode steps each"),
    "32b": dict(model="32b", batch=8, prompt=(1024, 1024), steps=512, temperature=0.7,
                what="8 prompts of 1,024 tokens, then 512 decode steps each at temperature 0.7, seed fixed"),
}


def run_workload(a) -> int:
    import numpy as np
    import torch

    import rust_inference_b200 as ri
    from rust_inference_b200 import ops
    from rust_inference_b200.engine import Engine, Model

    w = WORKLOADS[a.workload]
    cfg = dict(QWEN3_8B, **SHAPES[w["model"]])
    full_layers = cfg["num_hidden_layers"]
    if a.layers:
        cfg["num_hidden_layers"] = a.layers
    name = f"Qwen3-{w['model'].upper()}"
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    hbm_gbs, bf16_tflops, peak_src = peaks()
    rng = np.random.default_rng(20)
    B, steps = w["batch"], (a.steps if a.steps_given else w["steps"])
    lens = [int(n) for n in rng.integers(w["prompt"][0], w["prompt"][1] + 1, size=B)]
    prompts = [[int(t) for t in rng.integers(0, cfg["vocab_size"], size=n)] for n in lens]
    model = Model.from_random(cfg, seed=1, dtype="bfloat16", device=dev)
    page = 32
    longest = -(-(max(lens) + steps) // page) * page
    engine = Engine(model, max_tokens=sum(-(-(n + steps) // page) * page for n in lens), max_seqs=B, max_seq_len=longest)
    llm = ri.LLM(engine=engine)
    clocks = ClockSampler()
    clocks.start()
    windows, runs = [], []
    for _ in range(2):           # the first run loads the kernels and records the CUDA graphs; the second is reported
        n0 = ops.launch_count()
        t_a = time.time()
        res = llm.generate(prompts, max_new_tokens=steps, temperature=w["temperature"], seed=20, ignore_eos=True,
                           return_result=True)
        windows = [(t_a, time.time())]
        runs.append((res.stats, ops.launch_count() - n0))
    clocks.stop()
    st, launches = runs[-1]
    ms_step = st.decode_s / st.decode_steps * 1e3
    kv = engine.cache.bytes_per_token()
    step_bytes = model.weight_bytes() + kv * sum(n + (st.decode_steps + 1) / 2.0 for n in lens)
    achieved = step_bytes / (ms_step / 1e3) / 1e9
    L, D, H, KV, Dh, I, V = (cfg[k] for k in ("num_hidden_layers", "hidden_size", "num_attention_heads",
                                               "num_key_value_heads", "head_dim", "intermediate_size", "vocab_size"))
    line = {
        "metric": f"decode tok/s through LLM.generate, {name} shapes, bf16: {w['what']}",
        "value": round(st.decode_tokens / st.decode_s, 1), "unit": "tok/s", "n_gpus": 1, "steps": st.decode_steps,
        "warmup": "one whole run of the workload before the reported one", "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random-init weights N(0,0.02), uniform random token ids, seeded prompt lengths",
        "config": {"model": name + " shapes", "layers": L, "layers_full": full_layers, "hidden": D, "heads": H,
                   "kv_heads": KV, "head_dim": Dh, "intermediate": I, "vocab": V, "global_batch": B,
                   "prompt_tokens_min": min(lens), "prompt_tokens_max": max(lens), "prompt_tokens_total": sum(lens),
                   "decode_steps": st.decode_steps, "temperature": w["temperature"], "parallelism": "1 GPU",
                   "timing": "host clock of LLM.generate (ids on the host every step)", "peaks": peak_src},
        "prefill": {"value": round(st.prefill_tokens / st.prefill_s, 1), "tokens": st.prefill_tokens,
                    "ms": round(st.prefill_s * 1e3, 3),
                    "frac": round(prefill_flops(cfg, lens) / st.prefill_s / (bf16_tflops * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_gbs, "unit": "GB/s",
                     "frac": round(achieved / hbm_gbs, 4)},
        "e2e": {"value": round(st.decode_tokens / st.decode_s, 1), "unit": "tok/s",
                "h2d_bytes_per_step": (7 * B + 1) * 4, "d2h_bytes_per_step": B * 4},
        "clocks": clocks.summary(windows), "gpu_launches": launches, "graph_replays": engine.graph_replays,
        "impl": "ours", "workload": a.workload,
    }
    print(json.dumps(line))
    return 0


def main() -> int:
    global CONTEXT, PREFILL_TOKENS, METRIC
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=32,
                    help="untimed decode steps before the timed ones (right behind the prompt step the clock sits lower under the power cap)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the 36 of the configuration (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--model", default="8b", choices=sorted(SHAPES), help="layer sizes: Qwen3-8B (the default), 14B or 32B")
    ap.add_argument("--context", type=int, default=CONTEXT,
                    help="context length that the timed decode steps end at (the default is the configuration's; named in config)")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                    help="tokens of the timed prompt step (the default is what the line's contract names; named in config)")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--workload", choices=sorted(WORKLOADS),
                    help="run a whole workload of the larger sizes through LLM.generate instead of the default line")
    a = ap.parse_args()
    a.steps_given = a.steps is not None
    if a.steps is None:
        a.steps = 64
    if a.impl == "reference":
        print(json.dumps(reference_arm()))
        return 0
    if a.gpus != 1:
        print(f"bench.py measures one GPU: this library runs on a single device, --gpus {a.gpus} is not supported")
        return 2
    if a.context != CONTEXT:
        METRIC = METRIC.replace(f"context {CONTEXT}", f"context {a.context}")
    CONTEXT, PREFILL_TOKENS = a.context, a.prefill_tokens
    if a.workload:
        return run_workload(a)
    if a.warmup < 3:
        a.warmup = 3

    import torch

    import rust_inference_b200 as ri
    from rust_inference_b200 import ops
    from rust_inference_b200.engine import Engine, Entry, Model

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    cfg = dict(QWEN3_8B, **SHAPES[a.model])
    name = f"Qwen3-{a.model.upper()}"
    full_layers = cfg["num_hidden_layers"]
    if a.layers:
        cfg["num_hidden_layers"] = a.layers
    K, Wm, B = a.steps, a.warmup, a.batch
    ctx0 = CONTEXT - (K + Wm)
    hbm_gbs, bf16_tflops, peak_src = peaks()

    model = Model.from_random(cfg, seed=1, dtype="bfloat16", device=dev)
    max_b = B if a.skip_points else max(B, 64)
    engine = Engine(model, max_tokens=max_b * CONTEXT, max_seqs=max_b, max_seq_len=CONTEXT)
    for g in engine.cache.groups:                 # the cache holds random keys and values
        g.k.normal_(0.0, 0.5)
        g.v.normal_(0.0, 0.5)
    V = cfg["vocab_size"]
    gen = torch.Generator().manual_seed(0)
    kv_bytes_per_token = engine.cache.bytes_per_token()
    weight_bytes = model.weight_bytes()
    clocks = ClockSampler()
    clocks.start()
    windows = []

    def decode_run(batch, steps, warm):
        slots = [engine.new_sequence() for _ in range(batch)]
        engine.cache.extend([(s, CONTEXT - (steps + warm)) for s in slots])      # as if a prompt had been run
        engine.cache.upload()
        toks = torch.randint(0, V, (steps + warm, batch), generator=gen).tolist()
        launches0 = ops.launch_count()
        for i in range(warm):
            ops.argmax(engine.step([Entry(s, [t]) for s, t in zip(slots, toks[i])]))
        torch.cuda.synchronize()
        launches1 = ops.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t_a = time.time()
        e0.record()
        for i in range(warm, warm + steps):
            ops.argmax(engine.step([Entry(s, [t]) for s, t in zip(slots, toks[i])]))
        e1.record()
        torch.cuda.synchronize()
        windows.append((t_a, time.time()))
        ms = e0.elapsed_time(e1)
        launches = ops.launch_count() - launches1
        mean_len = CONTEXT - steps / 2.0
        for s in slots:
            engine.release(s)
        engine.check_device_errors()
        return ms / steps, batch * steps / (ms / 1e3), launches, mean_len

    ms_step, value, launches, mean_len = decode_run(B, K, Wm)
    step_bytes = weight_bytes + B * mean_len * kv_bytes_per_token
    achieved = step_bytes / (ms_step / 1e3) / 1e9

    # ---- prefill of 2,048 tokens ---------------------------------------------------------------
    prompt = torch.randint(0, V, (PREFILL_TOKENS,), generator=gen).tolist()
    times = []
    for i in range(3 + 3):
        s = engine.new_sequence()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t_a = time.time()
        e0.record()
        engine.step([Entry(s, prompt)])
        e1.record()
        torch.cuda.synchronize()
        if i >= 3:
            times.append(e0.elapsed_time(e1))
            windows.append((t_a, time.time()))
        engine.release(s)
    pre_ms = statistics.median(times)
    L, D, H, KV, Dh, I = (cfg[k] for k in ("num_hidden_layers", "hidden_size", "num_attention_heads",
                                            "num_key_value_heads", "head_dim", "intermediate_size"))
    T = PREFILL_TOKENS
    flops = prefill_flops(cfg, [T])
    prefill = {"value": round(T / (pre_ms / 1e3), 1), "tokens": T, "ms": round(pre_ms, 3),
               "frac": round(flops / (pre_ms / 1e3) / (bf16_tflops * 1e12), 4)}

    points = {}
    if not a.skip_points:
        for b in (1, 64):
            _, v, _, _ = decode_run(b, min(K, 32), Wm)
            points[f"decode_b{b}"] = round(v, 1)

    # ---- end to end through the Python entry point ----------------------------------------------
    e2e = None
    if not a.skip_e2e:
        llm = ri.LLM(engine=engine)                 # the loaded model and its cache, through the public entry point
        # one call: the prompts, then Wm decode steps that are not counted and K that are (their times are the
        # host's, from one step's ids on the host to the next step's), the last at the full context length
        prompts = torch.randint(0, V, (B, ctx0), generator=gen).tolist()
        t_a = time.time()
        res = llm.generate(prompts, max_new_tokens=K + Wm, ignore_eos=True, return_result=True)
        windows.append((t_a, time.time()))
        st = res.stats
        timed = st.decode_step_s[-K:]
        e2e = {"value": round(sum(n for _, n in timed) / sum(t for t, _ in timed), 1), "unit": "tok/s",
               "h2d_bytes_per_step": (7 * B + 1) * 4, "d2h_bytes_per_step": B * 4,
               "prefill_tok_s": round(st.prefill_tokens / st.prefill_s, 1), "steps": len(timed),
               "warmup_steps": st.decode_steps - len(timed)}
        if not a.skip_points:
            # the same at batch 1 and 64
            for b in (1, 64):
                kb = min(K, 32)
                pb = torch.randint(0, V, (b, CONTEXT - (kb + Wm)), generator=gen).tolist()
                t_a = time.time()
                rb = llm.generate(pb, max_new_tokens=kb + Wm, ignore_eos=True, return_result=True)
                windows.append((t_a, time.time()))
                tb = rb.stats.decode_step_s[-kb:]
                points[f"e2e_b{b}"] = round(sum(n for _, n in tb) / sum(t for t, _ in tb), 1)
    clocks.stop()

    line = {
        "metric": METRIC.replace("batch 8", f"batch {B}").replace("Qwen3-8B", name), "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": Wm,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random-init weights N(0,0.02), uniform random token ids",
        "config": {"model": name + " shapes", "layers": L, "layers_full": full_layers, "hidden": D, "heads": H,
                   "kv_heads": KV, "head_dim": Dh, "intermediate": I, "vocab": V, "global_batch": B,
                   "seq_len": CONTEXT, "ctx_start": ctx0, "prefill_tokens": T, "parallelism": "1 GPU",
                   "l2": "inputs larger than L2 (weights read per step >> 126 MB)", "page_size": engine.cache.page_size,
                   "rope_theta": cfg["rope_theta"], "rms_norm_eps": cfg["rms_norm_eps"], "peaks": peak_src},
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_gbs, "unit": "GB/s",
                     "frac": round(achieved / hbm_gbs, 4)},
        "points": points, "clocks": clocks.summary(windows), "gpu_launches": launches,
        "graph_replays": engine.graph_replays, "impl": "ours",
    }
    if e2e is not None:
        line["e2e"] = e2e
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
