"""The generation loop's decisions: batches, stop tokens, sequences that end earlier,
slots given back and used again.  A scripted engine stands in for the model, then the
real engine runs on the CPU stand-ins of the kernels against the plain model."""
import numpy as np
import pytest
import torch

import helpers as H
import plain_qwen3 as plain
from rust_inference_b200.engine import generate, plan_batches
from rust_inference_b200.sampling import SamplingParams
from tiny_configs import ALL


class ScriptedEngine:
    """Logits that make request-independent greedy tokens: after a sequence of n tokens the
    next token is (sum of the sequence) % vocab."""

    class _Spec:
        vocab_size = 50
        stop_ids = (49,)

    class _Model:
        pass

    class _Slots:
        num_slots = 3

    class _Cache:
        page_size, num_pages = 32, 12

    def __init__(self):
        self.model = self._Model()
        self.model.spec = self._Spec()
        self.cache = self._Cache()
        self.cache.slots = self._Slots()
        self.device = torch.device("cpu")
        self.max_seq_len = 64
        self.free, self.live, self.log = [2, 1, 0], {}, []

    def new_sequence(self):
        s = self.free.pop()
        self.live[s] = []
        return s

    def release(self, slot):
        assert slot in self.live, "slot released twice"
        del self.live[slot]
        self.free.append(slot)

    def step(self, entries):
        self.log.append([(e.slot, len(e.tokens)) for e in entries])
        out = torch.zeros(len(entries), 50)
        for i, e in enumerate(entries):
            self.live[e.slot].extend(e.tokens)
            out[i, sum(self.live[e.slot]) % 50] = 1.0
        return out

    def check_device_errors(self):
        pass


def _expected(prompt, n, stops=(49,)):
    seq, out = list(prompt), []
    while len(out) < n:
        t = sum(seq) % 50
        if t in stops:
            break
        out.append(t)
        seq.append(t)
    return out


def test_loop_decisions(emulated_ops):
    eng = ScriptedEngine()
    prompts = [[1, 2, 3], [10], [4, 4], [48], [7, 7, 7, 7], [20, 29], [5]]
    res = generate(eng, prompts, max_new_tokens=6)
    assert res.tokens == [_expected(p, 6) for p in prompts]
    assert res.finish_reasons[5] == "stop" and res.tokens[5] == []      # 20+29 = 49: a stop token at once
    assert res.finish_reasons[0] == "length"
    assert not eng.live and sorted(eng.free) == [0, 1, 2]               # every slot came back, once
    assert res.stats.batches == 3                                       # three slots: 3 + 3 + 1 requests
    first = eng.log[0]
    assert [n for _, n in first] == [3, 1, 2]                           # unequal prompts in one step
    assert all(n == 1 for step in eng.log[1:3] for _, n in step)        # then one token each
    assert res.stats.prefill_tokens == sum(len(p) for p in prompts)
    # every token after a request's first was sampled from a one-token step
    assert res.stats.decode_tokens == sum(n for step in eng.log for _, n in step) - res.stats.prefill_tokens
    # ignore_eos keeps going through stop tokens
    res2 = generate(ScriptedEngine(), prompts, max_new_tokens=4, ignore_eos=True)
    assert res2.tokens == [_expected(p, 4, stops=()) for p in prompts]
    # the cache's longest sequence ends a request
    eng3 = ScriptedEngine()
    eng3.max_seq_len = 5
    res3 = generate(eng3, [[1, 1, 1]], max_new_tokens=10, ignore_eos=True)
    assert len(res3.tokens[0]) == 3 and res3.finish_reasons[0] == "cache"


def test_plan_batches():
    assert plan_batches([5, 9, 13, 2], 8, max_seqs=3, page_size=32, num_pages=100, max_seq_len=128) == [[0, 1, 2], [3]]
    # pages: each request needs ceil((n + new) / 32) pages
    assert plan_batches([30, 30, 30], 10, max_seqs=8, page_size=32, num_pages=4, max_seq_len=128) == [[0, 1], [2]]
    assert plan_batches([1, 1, 1], 1, 8, 32, 100, 128, batch_size=2) == [[0, 1], [2]]
    with pytest.raises(ValueError):
        plan_batches([200], 1, 8, 32, 100, 128)
    with pytest.raises(ValueError):
        plan_batches([0], 1, 8, 32, 100, 128)


@pytest.mark.parametrize("name", ["A", "B"])
def test_generate_matches_plain_on_cpu(tmp_path, emulated_ops, name):
    from rust_inference_b200 import LLM
    from rust_inference_b200.engine import Model
    cfg, stored = ALL[name]
    d = H.make_model_dir(tmp_path, cfg, 9, stored=stored)
    rng = np.random.default_rng(1)
    lens = [5, 9, 13, 1, 17] if name == "A" else [1, 17, 3]
    prompts = [[int(t) for t in rng.integers(0, cfg["vocab_size"], size=n)] for n in lens]
    llm = LLM(model=Model.from_dir(d, "float32", "cpu"), max_seqs=2, max_pages=8, pages_per_seq=2)
    pcfg, W = plain.load_model_dir(d)
    got = llm.generate(prompts, max_new_tokens=8, ignore_eos=True)
    assert got == [plain.generate_plain(pcfg, W, p, 8, ignore_eos=True) for p in prompts]
    # temperature sampling: request i draws from its own stream
    from rust_inference_b200.sampling import request_seed
    got = llm.generate(prompts, max_new_tokens=6, temperature=0.8, seed=11, stop_ids=[3])
    want = [plain.generate_plain(pcfg, W, p, 6, stop_ids=[3], temperature=0.8, rng=plain.PlainRng(request_seed(11, i)))
            for i, p in enumerate(prompts)]
    assert got == want
    llm.engine.cache.check()
    assert llm.engine.cache.slots.live_count == 0


def test_section_timers_are_off_by_default_and_cost_nothing():
    from rust_inference_b200 import profiler
    assert not profiler.enabled()
    with profiler.section("anything") as s:
        assert s is profiler.section("other")           # one shared object that does nothing
    assert profiler.snapshot() == [] and profiler.report().count("\n") == 1
    profiler.enable(True)                               # without a GPU there is nothing to time with
    import torch
    assert profiler.enabled() == torch.cuda.is_available()
    profiler.enable(False)
