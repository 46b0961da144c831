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
  points     decode tokens a second at batch 1 and 64

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


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=32,
                    help="untimed decode steps before the timed ones (right behind the prompt step the clock sits lower under the power cap)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the 36 of the configuration (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--model", default="8b", choices=sorted(SHAPES), help="layer sizes: Qwen3-8B (the default), 14B or 32B")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-points", action="store_true")
    a = ap.parse_args()
    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "thanhauco/rust-inference is a Rust crate (Cargo.toml, no Python package); cargo and rustc "
                          "are not installed here and pip finds nothing to install"}))
        return 0
    if a.gpus != 1:
        print(f"bench.py measures one GPU: this library runs on a single device, --gpus {a.gpus} is not supported")
        return 2
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
    layer_params = D * (H + 2 * KV) * Dh + H * Dh * D + 3 * D * I
    flops = 2.0 * T * layer_params * L + 2.0 * 1 * D * V + 4.0 * Dh * H * T * (T + 1) / 2 * L
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
