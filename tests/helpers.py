"""Shared test machinery: model folders from seeds, traces in the three ways of
cutting the work, running them through trace replay, comparing with the plain model."""
from __future__ import annotations

import io
import json
import os
import subprocess
import sys

import numpy as np

import plain_qwen3 as plain

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Tolerances: max|got - want| <= rel * max|want| + abs per row of logits.
#  float32: the reference's own bound for its f32 engine against the float64 model is 2e-4 * max|want| + 1e-5
#           (tests/model_parity.rs:23-28 there).  The worst row of any replay test here (tiny models, the large
#           models' layer shapes, Qwen3-8B's width with the head of 151,936 rows) comes to 0.044 of that bound, so
#           the tests hold the engine to an eighth of it: 2.5e-5, a little under three times the worst seen.
#  bfloat16: activations are rounded to 8 significant bits between parts; with the residual stream in float32
#           the worst row seen is 1.84 % of the largest logit (8B layer shapes, 64 sequences decoding together),
#           and the bound is twice that.  The reference accepts far more for its bf16 path (cosine > 0.995,
#           tests/cuda_parity.rs:154-166).
TOL = {"float32": (2.5e-5, 1e-5), "bfloat16": (3.7e-2, 1e-3)}


def make_model_dir(tmp_path, config, seed, stored="float32", name="model"):
    from rust_inference_b200.weights import write_random_model
    d = os.path.join(str(tmp_path), name)
    write_random_model(dict(config), seed, d, dtype=stored)
    return d


def random_requests(rng, vocab, lengths):
    return {f"r{i}": [int(t) for t in rng.integers(0, vocab, size=n)] for i, n in enumerate(lengths)}


# ---- three ways of cutting the same requests into steps ---------------------------------------

def trace_whole(requests):
    """Each request alone and whole, all positions wanted."""
    return [{"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]}
            for i, (rid, toks) in enumerate(requests.items())]


def trace_tail(requests, tail=32):
    """Each request alone: all but the last ``tail`` tokens in one step, the rest one by one."""
    steps, n = [], 0
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        n += 1
        for j in range(head, len(toks)):
            steps.append({"step": n, "entries": [{"id": rid, "tokens": [toks[j]], "want": [0]}],
                          "end": [rid] if j == len(toks) - 1 else []})
            n += 1
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def trace_batches(requests, batch_size, decode_tokens):
    """Batches of ``batch_size`` requests that start together: request i brings all
    but its last ``decode_tokens[i]`` tokens in the first step, then everyone goes on
    by one token a step; shorter requests end earlier.  Batches follow one another, so
    slots and pages of ended requests are used again."""
    steps, n = [], 0
    items = list(requests.items())
    for b0 in range(0, len(items), batch_size):
        batch = items[b0:b0 + batch_size]
        heads = {}
        for k, (rid, toks) in enumerate(batch):
            d = min(decode_tokens[(b0 + k) % len(decode_tokens)], len(toks) - 1)
            heads[rid] = len(toks) - d
        ends = [rid for rid, toks in batch if heads[rid] == len(toks)]
        steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[:heads[rid]],
                                              "want": list(range(heads[rid]))} for rid, toks in batch], "end": ends})
        n += 1
        live = [(rid, toks) for rid, toks in batch if heads[rid] < len(toks)]
        j = 0
        while live:
            entries = [{"id": rid, "tokens": [toks[heads[rid] + j]], "want": [0]} for rid, toks in live]
            ends = [rid for rid, toks in live if heads[rid] + j == len(toks) - 1]
            steps.append({"step": n, "entries": entries, "end": ends})
            n += 1
            live = [(rid, toks) for rid, toks in live if rid not in ends]
            j += 1
    return steps


def max_live_tokens(steps):
    """The --max-tokens a trace needs: live requests' token counts, each rounded up to 64."""
    held, worst = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum(-(-v // 64) * 64 for v in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return worst


# ---- running a trace ----------------------------------------------------------------------------

def collect(steps, out_dir, vocab):
    """{(request id, position): logits row} from the files a replay wrote."""
    pos, rows = {}, {}
    for s in steps:
        wanted = [(e["id"], pos.get(e["id"], 0) + w) for e in s["entries"] for w in e["want"]]
        for e in s["entries"]:
            pos[e["id"]] = pos.get(e["id"], 0) + len(e["tokens"])
        path = os.path.join(out_dir, f"{s['step']}.f32")
        if wanted:
            arr = np.fromfile(path, dtype="<f4").reshape(len(wanted), vocab)
            for key, row in zip(wanted, arr):
                rows[key] = row
        else:
            assert not os.path.exists(path), "a step without wanted places wrote a file"
    return rows


def replay_subprocess(model_dir, dtype, steps, out_dir, max_tokens=None, env=None, timeout=900):
    """Run bin/trace_run as a user would: a process, steps on stdin, `done` lines back."""
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens or max_live_tokens(steps))]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    try:
        for s in steps:
            proc.stdin.write(json.dumps(s) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline()
            assert line.strip() == f"done {s['step']}", f"expected 'done {s['step']}', got {line!r}"
        proc.stdin.close()
        assert proc.wait(timeout=timeout) == 0
    finally:
        if proc.poll() is None:
            proc.kill()


def replay_inprocess(model_dir, dtype, steps, out_dir, max_tokens=None, device="cpu", model=None):
    """The replay program's function in this process; ``model``: a model built already (no folder is read)."""
    from rust_inference_b200 import trace
    lines = [json.dumps(s) for s in steps]
    buf = io.StringIO()
    rc = trace.run(model_dir, dtype, out_dir, max_tokens or max_live_tokens(steps), lines=lines, out=buf, device=device,
                   model=model)
    assert rc == 0
    assert buf.getvalue().split("\n")[:-1] == [f"done {s['step']}" for s in steps]


# ---- comparing ------------------------------------------------------------------------------------

def plain_logits(model_dir, requests, dtype="float32"):
    cfg, W = plain.load_model_dir(model_dir, round_to_bf16=(dtype == "bfloat16"))
    return {rid: plain.forward_logits(cfg, W, toks) for rid, toks in requests.items()}


def assert_rows_close(rows, want_by_request, dtype, what=""):
    rel, ab = TOL[dtype]
    worst = 0.0
    for (rid, p), got in sorted(rows.items()):
        want = want_by_request[rid][p]
        bound = rel * np.abs(want).max() + ab
        err = np.abs(got.astype(np.float64) - want).max()
        worst = max(worst, err / bound)
        assert err <= bound, (f"{what}: request {rid} position {p}: max error {err:.3e} exceeds {bound:.3e} "
                              f"(first wrong place of this request: "
                              f"{first_wrong(rows, want_by_request, rid, rel, ab)})")
    return worst


def first_wrong(rows, want_by_request, rid, rel, ab):
    for (r, p) in sorted(k for k in rows if k[0] == rid):
        want = want_by_request[rid][p]
        if np.abs(rows[(r, p)] - want).max() > rel * np.abs(want).max() + ab:
            return p
    return None


def assert_rows_identical(rows_by_cutting, what=""):
    """float32: the logits of a (request, position) are the same bits however the work was cut
    (the reference holds `Last` bit-equal to the row of `All`, tests/model_parity.rs:86-98)."""
    labels = list(rows_by_cutting)
    base = rows_by_cutting[labels[0]]
    for label in labels[1:]:
        other = rows_by_cutting[label]
        assert set(other) == set(base), f"{what}: {label} and {labels[0]} hold different places"
        for key in sorted(base):
            if not np.array_equal(base[key], other[key]):
                diff = np.abs(base[key].astype(np.float64) - other[key]).max()
                raise AssertionError(f"{what}: request {key[0]} position {key[1]}: {labels[0]} and {label} differ "
                                     f"(max {diff:.3e}); float32 logits must not depend on the cutting")
