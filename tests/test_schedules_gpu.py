"""Schedules that the other replay tests do not reach, each against the plain model:

* many sequences decoding together (14, 15, 24 and 64: the tcgen05 weight-streaming linear of 13 to
  32 tokens, the library products above that, the same linear when it is asked for there, the decode
  attention whose runs of pages pass through several sequences), on the tiny configuration with
  heads of 128 and on two layers of Qwen3-8B's shapes;
* steps that are neither whole prompts nor one token each: a prompt brought in pieces, and a step
  in which one sequence brings a prompt while others go on by one token;
* a window group whose sequence brings several tokens after pages behind the window went back.
"""
import os

import numpy as np
import pytest
import torch

import helpers as H
import plain_qwen3 as plain
from tiny_configs import ALL

pytestmark = pytest.mark.gpu


def _together(reqs, decode):
    """One batch of all requests: the prompts in one step, then one token each; request i decodes
    decode[i % len(decode)] tokens, so the batch shrinks on the way."""
    return H.trace_batches(reqs, len(reqs), decode)


def _decoded_rows(rows, reqs, decode):
    """The rows of decode steps only (the prompt step is the other tests' business)."""
    keep = {}
    for i, (rid, toks) in enumerate(reqs.items()):
        d = min(decode[i % len(decode)], len(toks) - 1)
        for p in range(len(toks) - d, len(toks)):
            keep[(rid, p)] = rows[(rid, p)]
    return keep


# ---- many sequences decoding together ----------------------------------------------------------------------

@pytest.fixture(scope="module")
def tiny_d(tmp_path_factory):
    cfg, stored = ALL["D"]
    return cfg, H.make_model_dir(tmp_path_factory.mktemp("sched"), cfg, seed=61, stored=stored, name="D")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seqs,stream_tc", [(14, False), (24, False), (64, False), (64, True)])
def test_many_sequences_decode_together_tiny(tmp_path, tiny_d, dtype, seqs, stream_tc):
    if stream_tc and dtype == "float32":
        pytest.skip("the tcgen05 weight-streaming linear is a bfloat16 kernel")
    cfg, d = tiny_d
    rng = np.random.default_rng(seqs)
    decode = [40, 44, 47, 52]
    lens = [int(rng.integers(1, 70)) + decode[i % 4] for i in range(seqs)]
    reqs = H.random_requests(rng, cfg["vocab_size"], lens)
    want = H.plain_logits(d, reqs, dtype)
    steps = _together(reqs, decode)
    env = dict(os.environ)
    if stream_tc:
        env["RUST_INFERENCE_B200_STREAM_TC_WIDE"] = "256"      # every linear of 13 to 128 tokens with 256 outputs or more
    out = str(tmp_path / "out")
    H.replay_subprocess(d, dtype, steps, out, env=env)
    rows = H.collect(steps, out, cfg["vocab_size"])
    assert len(rows) == sum(lens)
    worst = H.assert_rows_close(rows, want, dtype, f"{seqs} sequences together, {dtype}")
    print(f"tiny D, {seqs} sequences, {dtype}, stream_tc={stream_tc}: worst error / bound = {worst:.3f}")


LARGE_8B = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 2,
            "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
            "intermediate_size": 12288, "vocab_size": 2003, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
            "tie_word_embeddings": False, "max_position_embeddings": 4096}


@pytest.fixture(scope="module")
def large_8b(tmp_path_factory):
    import shutil
    d = H.make_model_dir(tmp_path_factory.mktemp("sched8b"), LARGE_8B, seed=89, stored="bfloat16", name="large")
    rng = np.random.default_rng(12)
    decode = [40, 43]
    lens = [int(rng.integers(1, 9)) + decode[i % 2] for i in range(64)]
    reqs = H.random_requests(rng, LARGE_8B["vocab_size"], lens)
    # stored in bfloat16: one plain model for both dtypes of the engine
    yield d, reqs, decode, H.plain_logits(d, reqs, "float32")
    shutil.rmtree(d, ignore_errors=True)


@pytest.mark.parametrize("dtype,seqs,wide", [("float32", 24, None), ("bfloat16", 24, None), ("bfloat16", 15, None), ("bfloat16", 8, None), ("bfloat16", 64, None),
                                             ("bfloat16", 64, 2000), ("float32", 64, None)])
def test_many_sequences_decode_together_at_8b_layer_shapes(tmp_path, monkeypatch, large_8b, dtype, seqs, wide):
    """Two layers of Qwen3-8B's shapes (width 4096, 32 heads over 8 kv heads of 128, feed-forward 12288) and a
    vocabulary of 2,003; `wide` lowers the number of outputs from which the tcgen05 weight-streaming linear is
    taken, so that the output head of 2,003 rows runs on it inside the engine."""
    from rust_inference_b200 import ops
    d, all_reqs, decode, want = large_8b
    reqs = dict(list(all_reqs.items())[:seqs])
    if wide is not None:
        monkeypatch.setattr(ops, "STREAM_TC_WIDE", wide)
    steps = _together(reqs, decode)
    out = str(tmp_path / "out")
    H.replay_inprocess(d, dtype, steps, out, device="cuda")
    rows = H.collect(steps, out, LARGE_8B["vocab_size"])
    worst = H.assert_rows_close(_decoded_rows(rows, reqs, decode), want, dtype, f"8B shapes, {seqs} together, {dtype}")
    print(f"8B layer shapes, {seqs} sequences, {dtype}, wide={wide}: worst error / bound = {worst:.3f}")


# ---- steps that are neither whole prompts nor one token each ------------------------------------------------

def _run_plan(model_dir, dtype, plan, max_tokens=4096, max_seqs=8):
    """plan: a list of steps, each a list of (request id, tokens); the logits of every token are wanted.
    Returns {(request id, position): row} and the engine."""
    from rust_inference_b200.engine import Engine, Entry, Model
    model = Model.from_dir(model_dir, dtype, "cuda:0")
    eng = Engine(model, max_tokens=max_tokens, max_seqs=max_seqs)
    slots, pos, rows = {}, {}, {}
    for step in plan:
        entries = []
        for rid, toks in step:
            if rid not in slots:
                slots[rid] = eng.new_sequence()
                pos[rid] = 0
            entries.append(Entry(slots[rid], toks, "all"))
        logits = eng.step(entries).float().cpu().numpy()
        i = 0
        for rid, toks in step:
            for _ in toks:
                rows[(rid, pos[rid])] = logits[i]
                pos[rid] += 1
                i += 1
        assert i == logits.shape[0]
    eng.check_device_errors()
    eng.cache.check()
    return rows, eng


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C", "D"])
def test_prompts_in_pieces_and_steps_of_prompts_and_single_tokens(tmp_path, name, dtype):
    cfg, stored = ALL[name]
    d = H.make_model_dir(tmp_path, cfg, seed=71, stored=stored, name=name)
    rng = np.random.default_rng(9)
    top = min(cfg["max_position_embeddings"], 200)
    n = {"a": min(75, top), "b": min(60, top), "c": min(120, top), "e": min(66, top)}
    reqs = {rid: [int(t) for t in rng.integers(0, cfg["vocab_size"], size=k)] for rid, k in n.items()}
    a, b, c, e = (reqs[r] for r in "abce")
    plan = [
        [("a", a[:40])],                                         # a prompt in two pieces ...
        [("a", a[40:70])],
        [("a", a[70:71]), ("b", b[:20])],                        # ... then one token while b brings its prompt
        [("a", a[71:72]), ("b", b[20:21]), ("c", c[:45])],       # two go on by one token, c joins with a prompt
        [("a", a[72:73]), ("b", b[21:22]), ("c", c[45:46])],     # a decode step of three
        [("a", a[73:75]), ("b", b[22:55]), ("c", c[46:47])],     # pieces of 2 and 33 tokens beside a single token
        [("b", b[55:]), ("c", c[47:]), ("e", e[:1])],            # the rests, and a prompt of one token
        [("e", e[1:])],
    ]
    rows, eng = _run_plan(d, dtype, plan)
    assert len(rows) == sum(n.values())
    want = H.plain_logits(d, reqs, dtype)
    worst = H.assert_rows_close(rows, want, dtype, f"{name} {dtype} pieces and mixed steps")
    print(f"{name} {dtype}: pieces and mixed steps, worst error / bound = {worst:.3f}")
    if dtype == "float32":
        # the same requests whole, on a fresh engine: bit for bit the same rows
        whole, _ = _run_plan(d, dtype, [[(rid, toks)] for rid, toks in reqs.items()])
        for key, row in rows.items():
            assert np.array_equal(row, whole[key]), f"{name}: row {key} differs between the cuttings"


# ---- several tokens after pages behind a window went back -----------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("Dh", [32, 64])
def test_window_attention_in_portions_after_pages_went_back(dtype, Dh):
    """The attention part with a window of 40 keys, its sequence brought in portions of many and of two
    tokens.  After a portion the pages wholly behind the window go back to the pool; the next portion's first
    block of 64 keys then starts with an unmapped page (first visible key at 36, 38 and 101 of its block of 64):
    that is no error, and what lies in shared memory for it must not reach the result.  The freed pages are
    filled with NaN to show it.  Head size 32: the mma.sync prefill kernel; 64: the tcgen05 one."""
    from rust_inference_b200 import ops
    from rust_inference_b200.cache import Cache
    from rust_inference_b200.config import AttentionSpec, RMSNormSpec, RopeSpec
    from rust_inference_b200.parts import BuildEnv, build_part
    from rust_inference_b200.parts.base import StepContext
    DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    rng = np.random.default_rng(6)
    D, Hh, KV, window, n = 48, 4, 2, 40, 260
    spec = AttentionSpec(hidden_size=D, num_heads=Hh, num_kv_heads=KV, head_dim=Dh,
                         position=RopeSpec(head_dim=Dh, theta=10000.0), qk_norm=RMSNormSpec(size=Dh, eps=1e-6), window=window)
    part = build_part("mixer", spec, BuildEnv(DT, torch.device("cuda")))
    W = {"q_proj.weight": (Hh * Dh, D), "k_proj.weight": (KV * Dh, D), "v_proj.weight": (KV * Dh, D), "o_proj.weight": (D, Hh * Dh)}
    W = {k: (rng.standard_normal(s) * 0.2).astype(np.float32) for k, s in W.items()}
    if dtype == "bfloat16":
        W = {k: plain.bf16_round(w) for k, w in W.items()}
    G = {"q_norm.weight": (1 + 0.1 * rng.standard_normal(Dh)).astype(np.float32),
         "k_norm.weight": (1 + 0.1 * rng.standard_normal(Dh)).astype(np.float32)}
    dev = lambda a, t=torch.float32: torch.as_tensor(np.ascontiguousarray(a)).to("cuda", dtype=t).contiguous()
    part.load({**{k: dev(w, DT) for k, w in W.items()}, **{k: dev(g) for k, g in G.items()}})
    part.prepare(512)
    cache = Cache([part.cache_request()], num_slots=2, num_pages=12, max_pages_per_seq=12, dtype=DT, device="cuda")
    cache.alloc_slot()
    slot = cache.alloc_slot()
    x = rng.standard_normal((n, D)).astype(np.float32)
    x = plain.bf16_round(x) if dtype == "bfloat16" else x
    outs = []
    i32 = lambda a: dev(np.asarray(a), torch.int32)
    group = cache.groups[0]
    ops.error_flag("cuda").zero_()
    for lo, hi in [(0, 75), (75, 77), (77, 140), (140, 142), (142, 143), (143, 260)]:
        cache.extend([(slot, hi - lo)])
        cache.upload()
        mapped = set(int(p) for p in group.pages.table[slot] if p >= 0)
        for p in range(group.k.shape[1]):                 # pages that are nobody's: anything may lie there
            if p not in mapped:
                group.k[:, p] = float("nan")
                group.v[:, p] = float("nan")
        ctx = StepContext(tok_seq=i32(np.zeros(hi - lo)), tok_pos=i32(np.arange(lo, hi)), seq_slot=i32([slot]),
                          seq_start=i32([0, hi - lo]), seq_len=i32([hi]), num_tokens=hi - lo, num_seqs=1,
                          max_new=hi - lo, max_len=hi)
        outs.append(part(dev(x[lo:hi], DT), ctx, cache.layer(0)).float().cpu().numpy())
        cache.after_step([slot])
    assert int(ops.error_flag("cuda").item()) == 0, "a page behind the window was reported as an error"
    got = np.concatenate(outs)
    assert np.isfinite(got).all()
    q = plain.rms_norm(plain.linear(x, W["q_proj.weight"]).reshape(n, Hh, Dh), G["q_norm.weight"], 1e-6)
    k = plain.rms_norm(plain.linear(x, W["k_proj.weight"]).reshape(n, KV, Dh), G["k_norm.weight"], 1e-6)
    v = plain.linear(x, W["v_proj.weight"]).reshape(n, KV, Dh)
    cos, sin = plain.rope_cos_sin(np.arange(n), Dh, 10000.0)
    o = plain.causal_attention(plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin), v, window=window)
    want = plain.linear(o.reshape(n, Hh * Dh), W["o_proj.weight"])
    assert np.abs(got - want).max() <= (2e-5 if dtype == "float32" else 4e-2) * np.abs(want).max()
    assert (group.pages.table[slot] >= 0).sum() <= 3
    cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_window_architecture_in_portions(tmp_path, dtype):
    """The toy architecture with a full and a windowed cache group (defined in test_parts_gpu.py), its prompts
    brought in portions through Engine.step, against its plain model."""
    from test_parts_gpu import MixedConfig, mixed_plain
    cfg = MixedConfig()
    d = H.make_model_dir(tmp_path, cfg.to_dict(), seed=8, stored="float32" if dtype == "float32" else "bfloat16", name="mixed")
    W = {k: v.astype(np.float64) for k, v in plain.read_safetensors(d + "/model.safetensors").items()}
    rng = np.random.default_rng(3)
    reqs = {rid: [int(t) for t in rng.integers(0, cfg.vocab_size, size=k)] for rid, k in (("a", 150), ("b", 90))}
    a, b = reqs["a"], reqs["b"]
    plan = [[("a", a[:75])], [("a", a[75:77]), ("b", b[:50])], [("a", a[77:140]), ("b", b[50:51])],
            [("a", a[140:142]), ("b", b[51:53])], [("a", a[142:]), ("b", b[53:])]]
    rows, eng = _run_plan(d, dtype, plan)
    want, close_call = {}, set()
    for rid, toks in reqs.items():
        margins = []
        want[rid] = mixed_plain(cfg, W, toks, margins)
        close_call |= {(rid, t) for t, m in enumerate(margins) if dtype == "bfloat16" and m < 0.05}
    H.assert_rows_close({k: r for k, r in rows.items() if k not in close_call}, want, dtype, f"mixed in portions {dtype}")
