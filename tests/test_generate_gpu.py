"""Generation on the GPU through the entry points: greedy against the plain model,
long decoding across pages, chunks and graph buckets, the first tokens of a sequence,
slots that are used again, temperature sampling with streams per request, the command line."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers as H
import plain_qwen3 as plain
from tiny_configs import ALL

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    base = tmp_path_factory.mktemp("gen")
    return {n: H.make_model_dir(base, cfg, seed=31 + i, stored=stored, name=n) for i, (n, (cfg, stored)) in enumerate(ALL.items())}


def _margin_ok(cfg, W, prompt, tokens, min_margin):
    """True while the plain model's top-2 gap along `tokens` stays above min_margin."""
    seq = list(prompt)
    for t in tokens:
        row = np.sort(plain.forward_logits(cfg, W, seq)[-1])
        if row[-1] - row[-2] < min_margin:
            return False
        seq.append(t)
    return True


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("A", "bfloat16"), ("B", "bfloat16")])
def test_greedy_generation_matches_plain(dirs, name, dtype):
    import rust_inference_b200 as ri
    cfg, _ = ALL[name]
    rng = np.random.default_rng(3)
    lens = [5, 9, 13, 1, 17, 2, 30] if name == "A" else [1, 17, 40, 3]
    prompts = [[int(t) for t in rng.integers(0, cfg["vocab_size"], size=n)] for n in lens]
    # three slots for seven requests: batches follow one another on the same slots
    llm = ri.LLM(dirs[name], dtype=dtype, max_seqs=3, max_pages=12, pages_per_seq=4)
    got = llm.generate(prompts, max_new_tokens=8, ignore_eos=True)
    pcfg, W = plain.load_model_dir(dirs[name], round_to_bf16=(dtype == "bfloat16"))
    for p, g in zip(prompts, got):
        want = plain.generate_plain(pcfg, W, p, 8, ignore_eos=True)
        if dtype == "float32":
            assert g == want
        else:
            # bfloat16 can flip a choice whose two best logits nearly tie; up to there it must agree
            k = next((i for i, (a, b) in enumerate(zip(g, want)) if a != b), len(g))
            assert k == len(g) or not _margin_ok(pcfg, W, p, want[:k + 1], 0.02), (g, want)
    llm.engine.cache.check()
    assert llm.engine.cache.slots.live_count == 0
    assert llm.engine.cache.free_pages() == 12


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(dirs, tmp_path, dtype):
    """One token, then 299 single-token steps (graphs, page and chunk edges, the bucket
    edge at 1,024 with config C's prompt): every position's logits against the plain model."""
    for name, prompt_len, total in (("B", 1, 250), ("C", 1000, 1060), ("D", 1000, 1050)):
        cfg, _ = ALL[name]
        rng = np.random.default_rng(11)
        reqs = H.random_requests(rng, cfg["vocab_size"], [total])
        steps = H.trace_tail(reqs, tail=total - prompt_len)
        out = str(tmp_path / f"long_{name}_{dtype}")
        H.replay_subprocess(dirs[name], dtype, steps, out)
        rows = H.collect(steps, out, cfg["vocab_size"])
        want = H.plain_logits(dirs[name], reqs, dtype)
        H.assert_rows_close(rows, want, dtype, f"long decoding {name}")


def test_stale_cache_of_a_reused_slot_is_not_read(dirs):
    """A long request fills a slot and ends; a short one takes the same slot and pages.
    Keys of the first must not leak: its logits equal those on a fresh engine, bit for bit."""
    from rust_inference_b200.engine import Engine, Entry, Model
    cfg, _ = ALL["C"]
    model = Model.from_dir(dirs["C"], "float32", "cuda:0")
    rng = np.random.default_rng(5)
    long_req = [int(t) for t in rng.integers(0, cfg["vocab_size"], size=200)]
    short = [int(t) for t in rng.integers(0, cfg["vocab_size"], size=37)]
    eng = Engine(model, max_tokens=512, max_seqs=1)
    s = eng.new_sequence()
    eng.step([Entry(s, long_req)])
    eng.release(s)
    s2 = eng.new_sequence()
    assert s2 == s
    a = eng.step([Entry(s2, short, "all")]).clone()
    b = eng.step([Entry(s2, [3], "all")]).clone()
    fresh = Engine(model, max_tokens=512, max_seqs=1)
    f = fresh.new_sequence()
    assert torch.equal(a, fresh.step([Entry(f, short, "all")]))
    assert torch.equal(b, fresh.step([Entry(f, [3], "all")]))


def test_temperature_sampling_streams(dirs):
    """Request i draws from its own stream: alone or in a batch it gets the same tokens,
    and in float32 they are the plain sampler's."""
    import rust_inference_b200 as ri
    from rust_inference_b200.sampling import request_seed
    cfg, _ = ALL["B"]
    rng = np.random.default_rng(8)
    prompts = [[int(t) for t in rng.integers(0, cfg["vocab_size"], size=n)] for n in (1, 17, 6)]
    llm = ri.LLM(dirs["B"], dtype="float32", max_seqs=4, max_pages=16, pages_per_seq=4)
    kw = dict(max_new_tokens=12, temperature=0.8, seed=1234, ignore_eos=True)
    together = llm.generate(prompts, **kw)
    pcfg, W = plain.load_model_dir(dirs["B"])
    for i, p in enumerate(prompts):
        want = plain.generate_plain(pcfg, W, p, 12, ignore_eos=True, temperature=0.8, rng=plain.PlainRng(request_seed(1234, i)))
        assert together[i] == want
    assert llm.generate(prompts[:1], **kw)[0] == together[0]
    assert llm.generate(prompts, **{**kw, "seed": 99}) != together
    # top-k 1 is greedy whatever the temperature; the penalty changes the choice somewhere
    greedy = llm.generate(prompts, max_new_tokens=12, ignore_eos=True)
    assert llm.generate(prompts, max_new_tokens=12, ignore_eos=True, temperature=1.5, top_k=1) == greedy
    pen = llm.generate(prompts, max_new_tokens=12, ignore_eos=True, repetition_penalty=1.8)
    for p, g in zip(prompts, pen):
        want = plain.generate_plain(pcfg, W, p, 12, ignore_eos=True, repetition_penalty=1.8)
        assert g == want


def test_stop_tokens_and_command_line(dirs):
    cfg, _ = ALL["B"]
    pcfg, W = plain.load_model_dir(dirs["B"], round_to_bf16=False)
    prompt = [5, 17, 3, 200]
    free = plain.generate_plain(pcfg, W, prompt, 10, ignore_eos=True)
    stop = free[4]
    want = plain.generate_plain(pcfg, W, prompt, 10, stop_ids=[stop])
    assert len(want) < 10
    root = H.ROOT
    cmd = [sys.executable, os.path.join(root, "bin", "runner"), dirs["B"], "--prompt", " ".join(map(str, prompt)),
           "-p", "1,2,3", "-n", "10", "--dtype", "float32", "--stop-ids", str(stop), "--max-pages", "8",
           "--pages-per-seq", "4", "--profile"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    assert r.stdout.endswith("\n")
    lines = r.stdout[:-1].split("\n")             # one line per prompt; a request that stops at once gives an empty one
    assert len(lines) == 2
    assert [int(t) for t in lines[0].split()] == want
    assert [int(t) for t in lines[1].split()] == plain.generate_plain(pcfg, W, [1, 2, 3], 10, stop_ids=[stop])
    assert "prefill: 7 tokens" in r.stderr and "decode:" in r.stderr and "kernel launches" in r.stderr
    # --profile: a line per section, largest first, with its share and its calls
    table = r.stderr[r.stderr.index("section "):].split("\n")
    rows = {line[:22].strip(): line[22:].split() for line in table[1:] if "%" in line}
    for name in ("embedding", "rmsnorm", "attn q/k/v proj", "attn norm/rope/append", "attention", "attn o proj",
                 "mlp gate/up", "mlp down", "lm head", "sampling"):
        assert name in rows, (name, r.stderr)
    secs = [float(v[0]) for v in rows.values()]
    assert secs == sorted(secs, reverse=True) and abs(sum(float(v[1].rstrip("%")) for v in rows.values()) - 100) < 1
    assert int(rows["attention"][2]) == int(rows["mlp down"][2]) == 3 * int(rows["lm head"][2])      # three layers
    bad = subprocess.run(cmd[:3] + ["--prompt", "99999"], capture_output=True, text=True, timeout=600)
    assert bad.returncode == 1 and "vocabulary" in bad.stderr


@pytest.mark.parametrize("temperature", [0.0, 0.8])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sequences_of_a_batch_end_at_different_steps(dirs, dtype, temperature):
    """Batches whose members end in different steps: by a stop token, by the token limit, by the longest
    sequence the cache holds.  In the loop that a GPU takes (the next step is launched from the device's ids
    before the host has read them) a stopped sequence runs one step too many on a slot that is given back
    right after; the others go on in a smaller batch.  Every request's tokens and reason: in float32 the plain
    model's, and in both dtypes those of the loop that reads every step's ids first."""
    import rust_inference_b200 as ri
    from rust_inference_b200.engine.generate import generate
    from rust_inference_b200.sampling import SamplingParams, request_seed
    cfg, _ = ALL["B"]
    rng = np.random.default_rng(17)
    lens = [1, 17, 6, 40, 3, 9, 22]
    prompts = [[int(t) for t in rng.integers(0, cfg["vocab_size"], size=n)] for n in lens]
    pcfg, W = plain.load_model_dir(dirs["B"], round_to_bf16=(dtype == "bfloat16"))
    max_new, seed, max_len = 30, 77, 64
    sampling = dict(temperature=temperature) if temperature else {}

    def plain_run(i, limit, stops):
        return plain.generate_plain(pcfg, W, prompts[i], limit, stop_ids=stops, ignore_eos=not stops,
                                    rng=plain.PlainRng(request_seed(seed, i)), **sampling)
    # stop tokens taken from what the requests generate when nothing stops them, at different depths
    free = [plain_run(i, 12, ()) for i in range(len(prompts))]
    stops = {free[0][5], free[2][9], free[4][2], free[5][7]}
    llm = ri.LLM(dirs["B"], dtype=dtype, max_seqs=3, max_pages=6, pages_per_seq=max_len // 32)
    params = SamplingParams(temperature, 0, 1.0, 1.0, seed)
    results = {}
    for pipelined in (True, False):
        res = generate(llm.engine, prompts, max_new, params, stop_ids=stops, pipelined=pipelined)
        results[pipelined] = res
        llm.engine.cache.check()
        assert llm.engine.cache.slots.live_count == 0 and llm.engine.cache.free_pages() == 6
        assert res.stats.batches == 3
    assert results[True].tokens == results[False].tokens
    assert results[True].finish_reasons == results[False].finish_reasons
    reasons = results[True].finish_reasons
    assert len(set(reasons)) > 1
    if dtype == "float32":
        # (what the plain model does with these prompts and seeds; bfloat16 may choose otherwise somewhere)
        assert reasons[3] == "cache" and len(results[True].tokens[3]) == max_len - lens[3] + 1
        assert {"stop", "length", "cache"} <= set(reasons)
        for batch in ([0, 1, 2], [3, 4, 5]):
            assert len({len(results[True].tokens[i]) for i in batch}) > 1, "the batch's members ended together"
        for i in range(len(prompts)):
            limit = min(max_new, max_len - lens[i] + 1)
            want = plain_run(i, limit, stops)
            assert results[True].tokens[i] == want, f"request {i}"
            assert reasons[i] == ("stop" if len(want) < limit else "cache" if limit < max_new else "length")
