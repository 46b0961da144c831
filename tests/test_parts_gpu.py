"""Each kind of part alone against its plain formula, and toy architectures defined in
this file and registered without touching the package: one whose mixer keeps state of
its own (one layer with the toy mixer, one with attention, the first layer scheduled
twice, once more at the end, reading its own state on); a position encoding with a rule
of its own; and one with two kinds of cache (all keys, a window), a layer that reads the
cache another layer wrote, and a feed-forward that routes tokens to experts."""
import math
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import helpers as H
import plain_qwen3 as plain
from rust_inference_b200.config import (AttentionSpec, LayerSpec, ModelSpec, RMSNormSpec, RopeSpec, ScheduleEntry,
                                        SwiGLUSpec, register_architecture)
from rust_inference_b200.parts import BuildEnv, CacheRequest, Mixer, ParamInfo, build_part, register_mixer

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.ascontiguousarray(a)).to("cuda", dtype=dtype).contiguous()


def env(dtype):
    return BuildEnv(DT[dtype], torch.device("cuda"))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_part(dtype):
    rng = np.random.default_rng(0)
    part = build_part("norm", RMSNormSpec(size=88, eps=2e-5), env(dtype))
    gain = (1 + 0.1 * rng.standard_normal(88)).astype(np.float32)
    part.load({"weight": dev(gain)})
    x = rng.standard_normal((5, 88)).astype(np.float32)
    got = part(dev(x)).float().cpu().numpy()
    want = plain.rms_norm(x, gain, 2e-5)
    assert np.abs(got - want).max() <= (2e-6 if dtype == "float32" else 8e-3) * np.abs(want).max()


def test_rope_part_table():
    part = build_part("position", RopeSpec(head_dim=64, theta=1e6, rotary_dim=48, scaling=1.0), env("float32"))
    part.prepare(300)
    table = part.fused_table().cpu().numpy()
    cos, sin = plain.rope_cos_sin(np.arange(300), 48, 1e6)
    assert table.shape == (300, 24, 2)
    assert np.abs(table[..., 0] - cos).max() < 1e-7 and np.abs(table[..., 1] - sin).max() < 1e-7


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("inter,tokens", [(104, 9), (100, 9), (104, 40), (2048, 3)])
def test_swiglu_part(dtype, inter, tokens):
    """Widths that are and are not multiples of 8 (gate/up interleaved or not), few tokens (the
    fused kernel in bfloat16) and many (library product, then the gate kernel)."""
    rng = np.random.default_rng(1)
    part = build_part("ffn", SwiGLUSpec(hidden_size=72, intermediate_size=inter), env(dtype))
    W = {n: (rng.standard_normal(s) * 0.1).astype(np.float32) for n, s in
         (("gate_proj.weight", (inter, 72)), ("up_proj.weight", (inter, 72)), ("down_proj.weight", (72, inter)))}
    if dtype == "bfloat16":
        W = {n: plain.bf16_round(w) for n, w in W.items()}
    part.load({n: dev(w, DT[dtype]) for n, w in W.items()})
    x = rng.standard_normal((tokens, 72)).astype(np.float32)
    x = plain.bf16_round(x) if dtype == "bfloat16" else x
    got = part(dev(x, DT[dtype]), None).float().cpu().numpy()
    want = plain.swiglu_mlp(x, {"m." + n: w for n, w in W.items()}, "m.")
    assert np.abs(got - want).max() <= (1e-5 if dtype == "float32" else 3e-2) * np.abs(want).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [0, 20])
def test_attention_part_over_two_steps(dtype, window):
    """The attention part with a cache of its own: a prompt step, then single tokens, against
    the plain attention block on the whole sequence; with a window, pages behind it are freed."""
    from rust_inference_b200.cache import Cache
    from rust_inference_b200.parts.base import StepContext
    rng = np.random.default_rng(2)
    D, Hh, KV, Dh = 40, 4, 2, 16
    spec = AttentionSpec(hidden_size=D, num_heads=Hh, num_kv_heads=KV, head_dim=Dh,
                         position=RopeSpec(head_dim=Dh, theta=10000.0), qk_norm=RMSNormSpec(size=Dh, eps=1e-6), window=window)
    part = build_part("mixer", spec, env(dtype))
    W = {"q_proj.weight": (Hh * Dh, D), "k_proj.weight": (KV * Dh, D), "v_proj.weight": (KV * Dh, D), "o_proj.weight": (D, Hh * Dh)}
    W = {n: (rng.standard_normal(s) * 0.2).astype(np.float32) for n, s in W.items()}
    if dtype == "bfloat16":
        W = {n: plain.bf16_round(w) for n, w in W.items()}
    G = {"q_norm.weight": (1 + 0.1 * rng.standard_normal(Dh)).astype(np.float32),
         "k_norm.weight": (1 + 0.1 * rng.standard_normal(Dh)).astype(np.float32)}
    part.load({**{n: dev(w, DT[dtype]) for n, w in W.items()}, **{n: dev(g) for n, g in G.items()}})
    part.prepare(256)
    cache = Cache([part.cache_request()], num_slots=3, num_pages=8, max_pages_per_seq=8, dtype=DT[dtype], device="cuda")
    cache.alloc_slot()
    slot = cache.alloc_slot()
    n, first = 90, 50
    x = rng.standard_normal((n, D)).astype(np.float32)
    x = plain.bf16_round(x) if dtype == "bfloat16" else x
    outs = []
    for lo, hi in [(0, first)] + [(i, i + 1) for i in range(first, n)]:
        before = cache.extend([(slot, hi - lo)])[0]
        cache.upload()
        i32 = lambda a: dev(np.asarray(a), torch.int32)
        ctx = StepContext(tok_seq=i32(np.zeros(hi - lo)), tok_pos=i32(np.arange(lo, hi)), seq_slot=i32([slot]),
                          seq_start=i32([0, hi - lo]), seq_len=i32([hi]), num_tokens=hi - lo, num_seqs=1,
                          max_new=hi - lo, max_len=hi)
        assert before == lo
        outs.append(part(dev(x[lo:hi], DT[dtype]), ctx, cache.layer(0)).float().cpu().numpy())
        cache.after_step([slot])
    got = np.concatenate(outs)
    # plain: the block of plain_qwen3 with this window
    cfg = {"num_attention_heads": Hh, "num_key_value_heads": KV, "head_dim": Dh, "hidden_size": D,
           "rms_norm_eps": 1e-6, "rope_theta": 10000.0}
    Wp = {"a." + k: v for k, v in {**W, **G}.items()}
    q = plain.rms_norm(plain.linear(x, W["q_proj.weight"]).reshape(n, Hh, Dh), G["q_norm.weight"], 1e-6)
    k = plain.rms_norm(plain.linear(x, W["k_proj.weight"]).reshape(n, KV, Dh), G["k_norm.weight"], 1e-6)
    v = plain.linear(x, W["v_proj.weight"]).reshape(n, KV, Dh)
    cos, sin = plain.rope_cos_sin(np.arange(n), Dh, 10000.0)
    o = plain.causal_attention(plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin), v, window=window)
    want = plain.linear(o.reshape(n, Hh * Dh), W["o_proj.weight"])
    if window == 0:
        assert np.allclose(want, plain.attention_block(x, Wp, "a.", cfg, np.arange(n)))
    assert np.abs(got - want).max() <= (2e-5 if dtype == "float32" else 4e-2) * np.abs(want).max()
    if window:
        assert (cache.groups[0].pages.table[slot] >= 0).sum() <= 2        # pages behind the window went back
    cache.check()


# ---- a toy architecture with a stateful mixer, all of it defined here --------------------------------------

@dataclass(frozen=True)
class DecaySpec:
    hidden_size: int
    state_size: int
    decay: float
    kind: str = "toy_decay"


@register_mixer("toy_decay")
class DecayMixer(Mixer):
    """s <- decay * s + x W_in ;  y = s W_out, token after token, s kept per sequence."""

    @classmethod
    def param_infos(cls, spec):
        return {"in_proj.weight": ParamInfo((spec.state_size, spec.hidden_size)),
                "out_proj.weight": ParamInfo((spec.hidden_size, spec.state_size))}

    def load(self, tensors):
        self.w_in, self.w_out = tensors["in_proj.weight"].float(), tensors["out_proj.weight"].float()

    def cache_request(self):
        return CacheRequest(state_shape=(self.spec.state_size,), state_dtype=torch.float32)

    def __call__(self, x, ctx, cache):
        u = x.float() @ self.w_in.t()
        y = torch.empty_like(u)
        t0 = 0
        for slot, n in zip(ctx.host_seq_slot, ctx.host_new):
            s = cache.state[slot]
            for t in range(t0, t0 + n):
                s = self.spec.decay * s + u[t]
                y[t] = s
            cache.state[slot] = s
            t0 += n
        return (y @ self.w_out.t()).to(x.dtype)


@register_architecture("ToyStateLM")
@dataclass(frozen=True)
class ToyConfig:
    vocab_size: int = 97
    hidden_size: int = 48
    state_size: int = 24
    decay: float = 0.9

    @classmethod
    def from_dict(cls, d):
        return cls(**{k: d[k] for k in ("vocab_size", "hidden_size", "state_size", "decay") if k in d})

    def validate(self):
        pass

    def to_dict(self):
        return {"architectures": ["ToyStateLM"], "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                "state_size": self.state_size, "decay": self.decay}

    def to_spec(self):
        D = self.hidden_size
        norm = RMSNormSpec(size=D, eps=1e-5)
        ffn = SwiGLUSpec(hidden_size=D, intermediate_size=2 * D)
        attn = AttentionSpec(hidden_size=D, num_heads=3, num_kv_heads=1, head_dim=16,
                             position=RopeSpec(head_dim=16, theta=1e4), qk_norm=None)

        def layer(i, mixer):
            return LayerSpec(mixer=mixer, ffn=ffn, mixer_norm=norm, ffn_norm=norm, names=(
                ("mixer", f"layers.{i}.mixer."), ("ffn", f"layers.{i}.ffn."), ("mixer_norm", f"layers.{i}.norm1."),
                ("ffn_norm", f"layers.{i}.norm2.")))
        layers = (layer(0, DecaySpec(D, self.state_size, self.decay)), layer(1, attn))
        # layer 0 runs twice; its second run has a state of its own (cache entry 2)
        schedule = (ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2))
        return ModelSpec(architecture="ToyStateLM", vocab_size=self.vocab_size, hidden_size=D, layers=layers,
                         schedule=schedule, final_norm=norm, tie_embeddings=True, max_positions=512,
                         embedding_name="embed.weight", head_name="head.weight", final_norm_prefix="norm.")


def toy_plain(cfg, W, ids):
    D = cfg.hidden_size
    h = W["embed.weight"][np.asarray(ids)]
    n = len(ids)

    def ffn(x, p):
        return plain.swiglu_mlp(x, W, p)

    def decay(x):
        u = x @ W["layers.0.mixer.in_proj.weight"].T
        s, out = np.zeros(cfg.state_size), []
        for t in range(n):
            s = cfg.decay * s + u[t]
            out.append(s)
        return np.array(out) @ W["layers.0.mixer.out_proj.weight"].T

    def attn(x):
        q = plain.linear(x, W["layers.1.mixer.q_proj.weight"]).reshape(n, 3, 16)
        k = plain.linear(x, W["layers.1.mixer.k_proj.weight"]).reshape(n, 1, 16)
        v = plain.linear(x, W["layers.1.mixer.v_proj.weight"]).reshape(n, 1, 16)
        cos, sin = plain.rope_cos_sin(np.arange(n), 16, 1e4)
        o = plain.causal_attention(plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin), v)
        return plain.linear(o.reshape(n, 48), W["layers.1.mixer.o_proj.weight"])
    for i, mix in ((0, decay), (1, attn), (0, decay)):
        p = f"layers.{i}."
        h = h + mix(plain.rms_norm(h, W[p + "norm1.weight"], 1e-5))
        h = h + ffn(plain.rms_norm(h, W[p + "norm2.weight"], 1e-5), p + "ffn.")
    return plain.rms_norm(h, W["norm.weight"], 1e-5) @ W["embed.weight"].T


def test_toy_architecture_registers_builds_and_steps(tmp_path):
    cfg = ToyConfig()
    d = H.make_model_dir(tmp_path, cfg.to_dict(), seed=3, stored="float32", name="toy")
    W = plain.read_safetensors(d + "/model.safetensors")
    rng = np.random.default_rng(0)
    reqs = H.random_requests(rng, cfg.vocab_size, [7, 40, 3, 66, 21])
    want = {rid: toy_plain(cfg, W, toks) for rid, toks in reqs.items()}
    import os
    env = dict(os.environ, PYTHONPATH=os.path.dirname(os.path.abspath(__file__)))
    for label, steps in (("whole", H.trace_whole(reqs)), ("tail", H.trace_tail(reqs, tail=32)),
                         ("batches", H.trace_batches(reqs, 2, [5, 0, 9]))):
        out = str(tmp_path / f"toy_{label}")
        # in this process: the toy parts are registered here, not in a fresh interpreter
        H.replay_inprocess(d, "float32", steps, out, device="cuda")
        rows = H.collect(steps, out, cfg.vocab_size)
        H.assert_rows_close(rows, want, "float32", f"toy {label}")


# ---- a toy position encoding with a rule of its own (no cos/sin table), defined here -----------------------

@dataclass(frozen=True)
class GrowSpec:
    rate: float
    kind: str = "toy_grow"


from rust_inference_b200.parts import PositionEncoding, register_position  # noqa: E402


@register_position("toy_grow")
class GrowPosition(PositionEncoding):
    """q <- q * (1 + rate*pos), k <- k / (1 + rate*pos): scores then depend on both positions."""
    graph_safe = True            # everything it uses reaches it through device tensors

    def apply(self, q, k, ctx):
        f = (1.0 + self.spec.rate * ctx.tok_pos.float())[:, None, None]
        return (q.float() * f).to(q.dtype), (k.float() / f).to(k.dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_part_with_a_position_encoding_of_its_own(dtype):
    from rust_inference_b200.cache import Cache
    from rust_inference_b200.parts.base import StepContext
    rng = np.random.default_rng(4)
    D, Hh, KV, Dh, n, first = 48, 4, 2, 16, 70, 40
    spec = AttentionSpec(hidden_size=D, num_heads=Hh, num_kv_heads=KV, head_dim=Dh, position=GrowSpec(rate=0.01),
                         qk_norm=RMSNormSpec(size=Dh, eps=1e-6))
    part = build_part("mixer", spec, env(dtype))
    W = {"q_proj.weight": (Hh * Dh, D), "k_proj.weight": (KV * Dh, D), "v_proj.weight": (KV * Dh, D), "o_proj.weight": (D, Hh * Dh)}
    W = {k: (rng.standard_normal(s) * 0.2).astype(np.float32) for k, s in W.items()}
    if dtype == "bfloat16":
        W = {k: plain.bf16_round(w) for k, w in W.items()}
    G = {"q_norm.weight": (1 + 0.1 * rng.standard_normal(Dh)).astype(np.float32),
         "k_norm.weight": (1 + 0.1 * rng.standard_normal(Dh)).astype(np.float32)}
    part.load({**{k: dev(w, DT[dtype]) for k, w in W.items()}, **{k: dev(g) for k, g in G.items()}})
    part.prepare(128)
    cache = Cache([part.cache_request()], num_slots=2, num_pages=4, max_pages_per_seq=4, dtype=DT[dtype], device="cuda")
    slot = cache.alloc_slot()
    x = rng.standard_normal((n, D)).astype(np.float32)
    x = plain.bf16_round(x) if dtype == "bfloat16" else x
    outs = []
    i32 = lambda a: dev(np.asarray(a), torch.int32)
    for lo, hi in [(0, first)] + [(i, i + 1) for i in range(first, n)]:
        cache.extend([(slot, hi - lo)])
        cache.upload()
        ctx = StepContext(tok_seq=i32(np.zeros(hi - lo)), tok_pos=i32(np.arange(lo, hi)), seq_slot=i32([slot]),
                          seq_start=i32([0, hi - lo]), seq_len=i32([hi]), num_tokens=hi - lo, num_seqs=1,
                          max_new=hi - lo, max_len=hi)
        outs.append(part(dev(x[lo:hi], DT[dtype]), ctx, cache.layer(0)).float().cpu().numpy())
    got = np.concatenate(outs)
    f = (1.0 + 0.01 * np.arange(n))[:, None, None]
    q = plain.rms_norm(plain.linear(x, W["q_proj.weight"]).reshape(n, Hh, Dh), G["q_norm.weight"], 1e-6) * f
    k = plain.rms_norm(plain.linear(x, W["k_proj.weight"]).reshape(n, KV, Dh), G["k_norm.weight"], 1e-6) / f
    v = plain.linear(x, W["v_proj.weight"]).reshape(n, KV, Dh)
    want = plain.linear(plain.causal_attention(q, k, v).reshape(n, Hh * Dh), W["o_proj.weight"])
    assert np.abs(got - want).max() <= (2e-5 if dtype == "float32" else 4e-2) * np.abs(want).max()


# ---- a toy architecture with two kinds of cache and a routed feed-forward, all of it defined here -------------
#
# layer 0: attention over all keys (head size 64: in bfloat16 the tcgen05 and the streaming kernels) + SwiGLU
# layer 1: attention over a window of 40 keys, other head counts and size (a cache group of its own, pages behind
#          the window go back) + a feed-forward that routes every token to one of three small experts
# layer 2: attention that appends nothing: its queries read the keys and values that layer 0 wrote + SwiGLU

from rust_inference_b200.parts import FeedForward, register_ffn  # noqa: E402


@dataclass(frozen=True)
class RoutedSpec:
    hidden_size: int
    expert_size: int
    experts: int
    kind: str = "toy_routed"


@register_ffn("toy_routed")
class RoutedFfn(FeedForward):
    """Router logits in float32, the best expert takes the token: y = W2[e] relu(W1[e] x) * softmax(logits)[e]."""
    graph_safe = True            # device tensors only, no host decisions

    @classmethod
    def param_infos(cls, spec):
        E, I, D = spec.experts, spec.expert_size, spec.hidden_size
        infos = {"router.weight": ParamInfo((E, D))}
        for e in range(E):
            infos[f"experts.{e}.w1.weight"] = ParamInfo((I, D))
            infos[f"experts.{e}.w2.weight"] = ParamInfo((D, I))
        return infos

    def load(self, tensors):
        E = self.spec.experts
        self.router = tensors["router.weight"].float()
        self.w1 = torch.stack([tensors[f"experts.{e}.w1.weight"] for e in range(E)]).float()
        self.w2 = torch.stack([tensors[f"experts.{e}.w2.weight"] for e in range(E)]).float()

    def __call__(self, x, ctx):
        xf = x.float()
        probs = torch.softmax(xf @ self.router.t(), dim=-1)
        best = probs.argmax(dim=-1)
        hid = torch.relu(torch.einsum("td,tid->ti", xf, self.w1[best]))
        y = torch.einsum("ti,tdi->td", hid, self.w2[best]) * probs.gather(1, best[:, None])
        return y.to(x.dtype)


@register_architecture("ToyMixedLM")
@dataclass(frozen=True)
class MixedConfig:
    vocab_size: int = 131
    hidden_size: int = 72
    window: int = 40

    @classmethod
    def from_dict(cls, d):
        return cls(**{k: d[k] for k in ("vocab_size", "hidden_size", "window") if k in d})

    def validate(self):
        pass

    def to_dict(self):
        return {"architectures": ["ToyMixedLM"], "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                "window": self.window}

    def to_spec(self):
        D = self.hidden_size
        norm = RMSNormSpec(size=D, eps=1e-6)
        wide = AttentionSpec(hidden_size=D, num_heads=4, num_kv_heads=2, head_dim=64,
                             position=RopeSpec(head_dim=64, theta=1e4), qk_norm=RMSNormSpec(size=64, eps=1e-6))
        near = AttentionSpec(hidden_size=D, num_heads=2, num_kv_heads=1, head_dim=32,
                             position=RopeSpec(head_dim=32, theta=1e5), qk_norm=None, window=self.window)
        dense = SwiGLUSpec(hidden_size=D, intermediate_size=104)
        routed = RoutedSpec(hidden_size=D, expert_size=40, experts=3)

        def layer(i, mixer, ffn):
            return LayerSpec(mixer=mixer, ffn=ffn, mixer_norm=norm, ffn_norm=norm, names=(
                ("mixer", f"layers.{i}.attn."), ("ffn", f"layers.{i}.ffn."), ("mixer_norm", f"layers.{i}.norm1."),
                ("ffn_norm", f"layers.{i}.norm2.")))
        layers = (layer(0, wide, dense), layer(1, near, routed), layer(2, wide, dense))
        schedule = (ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(2, 0, writes=False))
        return ModelSpec(architecture="ToyMixedLM", vocab_size=self.vocab_size, hidden_size=D, layers=layers,
                         schedule=schedule, final_norm=norm, tie_embeddings=False, max_positions=1024,
                         embedding_name="embed.weight", head_name="head.weight", final_norm_prefix="norm.")


def mixed_plain(cfg, W, ids, margins=None):
    """Logits; `margins` (a list) receives, per position, how far the router's best logit is ahead of the second,
    as a fraction of the largest."""
    n = len(ids)
    h = W["embed.weight"][np.asarray(ids)]

    def qkv(x, p, H_, KV, Dh, theta, normed):
        q = plain.linear(x, W[p + "q_proj.weight"]).reshape(n, H_, Dh)
        k = plain.linear(x, W[p + "k_proj.weight"]).reshape(n, KV, Dh)
        v = plain.linear(x, W[p + "v_proj.weight"]).reshape(n, KV, Dh)
        if normed:
            q, k = plain.rms_norm(q, W[p + "q_norm.weight"], 1e-6), plain.rms_norm(k, W[p + "k_norm.weight"], 1e-6)
        cos, sin = plain.rope_cos_sin(np.arange(n), Dh, theta)
        return plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin), v

    def routed(x, p):
        logits = x @ W[p + "router.weight"].T
        probs = np.exp(logits - logits.max(-1, keepdims=True))
        probs /= probs.sum(-1, keepdims=True)
        out = np.zeros_like(x)
        if margins is not None:
            top = np.sort(logits, axis=-1)
            margins.extend(((top[:, -1] - top[:, -2]) / np.abs(logits).max(-1)).tolist())
        for t in range(n):
            e = int(np.argmax(probs[t]))
            hid = np.maximum(W[p + f"experts.{e}.w1.weight"] @ x[t], 0.0)
            out[t] = (W[p + f"experts.{e}.w2.weight"] @ hid) * probs[t, e]
        return out

    # layer 0
    x = plain.rms_norm(h, W["layers.0.norm1.weight"], 1e-6)
    q0, k0, v0 = qkv(x, "layers.0.attn.", 4, 2, 64, 1e4, True)
    h = h + plain.linear(plain.causal_attention(q0, k0, v0).reshape(n, 256), W["layers.0.attn.o_proj.weight"])
    h = h + plain.swiglu_mlp(plain.rms_norm(h, W["layers.0.norm2.weight"], 1e-6), W, "layers.0.ffn.")
    # layer 1: a window
    x = plain.rms_norm(h, W["layers.1.norm1.weight"], 1e-6)
    q1, k1, v1 = qkv(x, "layers.1.attn.", 2, 1, 32, 1e5, False)
    h = h + plain.linear(plain.causal_attention(q1, k1, v1, window=cfg.window).reshape(n, 64), W["layers.1.attn.o_proj.weight"])
    h = h + routed(plain.rms_norm(h, W["layers.1.norm2.weight"], 1e-6), "layers.1.ffn.")
    # layer 2: its own queries over layer 0's keys and values
    x = plain.rms_norm(h, W["layers.2.norm1.weight"], 1e-6)
    q2, _, _ = qkv(x, "layers.2.attn.", 4, 2, 64, 1e4, True)
    h = h + plain.linear(plain.causal_attention(q2, k0, v0).reshape(n, 256), W["layers.2.attn.o_proj.weight"])
    h = h + plain.swiglu_mlp(plain.rms_norm(h, W["layers.2.norm2.weight"], 1e-6), W, "layers.2.ffn.")
    return plain.rms_norm(h, W["norm.weight"], 1e-6) @ W["head.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_with_two_cache_groups_a_shared_cache_and_routing(tmp_path, dtype):
    from rust_inference_b200.engine import Engine, Model
    cfg = MixedConfig()
    d = H.make_model_dir(tmp_path, cfg.to_dict(), seed=8, stored="float32" if dtype == "float32" else "bfloat16", name="mixed")
    W = plain.read_safetensors(d + "/model.safetensors")
    model = Model.from_dir(d, dtype, "cuda:0")
    groups = Engine(model, max_tokens=2048, max_seqs=3).cache.groups
    assert len(groups) == 2 and sorted(g.req.window for g in groups) == [0, cfg.window]
    rng = np.random.default_rng(2)
    reqs = H.random_requests(rng, cfg.vocab_size, [7, 90, 33, 150, 64, 41])
    W64 = {k: v.astype(np.float64) for k, v in W.items()}
    want, close_call = {}, set()
    for rid, toks in reqs.items():
        margins = []
        want[rid] = mixed_plain(cfg, W64, toks, margins)
        # in bfloat16 a token whose two best experts nearly tie may go to the other one: a choice, not an error
        close_call |= {(rid, t) for t, m in enumerate(margins) if dtype == "bfloat16" and m < 0.05}
    assert len(close_call) < 0.3 * sum(len(t) for t in reqs.values())
    for label, steps in (("whole", H.trace_whole(reqs)), ("tail", H.trace_tail(reqs, tail=32)),
                         ("batches", H.trace_batches(reqs, 3, [12, 0, 35]))):
        out = str(tmp_path / f"mixed_{label}")
        H.replay_inprocess(d, dtype, steps, out, device="cuda")      # in this process: the toy parts live here
        rows = H.collect(steps, out, cfg.vocab_size)
        assert len(rows) == sum(len(t) for t in reqs.values())
        H.assert_rows_close({k: r for k, r in rows.items() if k not in close_call}, want, dtype, f"mixed {dtype} {label}")


# ---- a toy architecture with an arrangement, an embedding and an output head of its own, all defined here ------
#
# One norm per layer whose output feeds the mixer and the feed-forward side by side (their outputs are added
# to the stream together); an embedding scaled by sqrt(width) plus learned positions; a head with a bias and a soft-cap.

from rust_inference_b200.parts import (BlockBase, Part, norm_before, register_block, register_embedding,  # noqa: E402
                                       register_head)


@dataclass(frozen=True)
class ParallelLayerSpec:
    norm: object
    mixer: object
    ffn: object
    names: tuple = ()
    arrangement: str = "toy_parallel"

    def prefix(self, part):
        return dict(self.names)[part]


@register_block("toy_parallel")
class ParallelBlock(BlockBase):
    @classmethod
    def slots(cls, spec):
        return (("norm", "norm", spec.norm), ("mixer", "mixer", spec.mixer), ("ffn", "ffn", spec.ffn))

    def __call__(self, resid, delta, ctx, cache):
        x = norm_before(self.norm, resid, delta, self.mixer)
        a, f = self.mixer(x, ctx, cache), self.ffn(x, ctx)
        return resid, (a.float() + f.float()).to(a.dtype)


@dataclass(frozen=True)
class ScaledEmbeddingSpec:
    vocab_size: int
    hidden_size: int
    scale: float
    positions: int
    kind: str = "toy_scaled"


@register_embedding("toy_scaled")
class ScaledEmbedding(Part):
    """table[id] * scale + learned[position]: the positions come from the step's context."""
    @classmethod
    def param_infos(cls, spec):
        return {"weight": ParamInfo((spec.vocab_size, spec.hidden_size)),
                "positions": ParamInfo((spec.positions, spec.hidden_size))}

    def load(self, tensors):
        self.table, self.learned = tensors["weight"], tensors["positions"].float()

    def __call__(self, ids, ctx):
        from rust_inference_b200 import ops
        return ops.embed(ids, self.table) * self.spec.scale + self.learned[ctx.tok_pos.long()]


@dataclass(frozen=True)
class CappedHeadSpec:
    vocab_size: int
    hidden_size: int
    cap: float
    kind: str = "toy_capped"


@register_head("toy_capped")
class CappedHead(Part):
    @classmethod
    def param_infos(cls, spec):
        return {"weight": ParamInfo((spec.vocab_size, spec.hidden_size)), "bias": ParamInfo((spec.vocab_size,), "gain")}

    def load(self, tensors):
        self.weight, self.bias = tensors["weight"], tensors["bias"]

    def __call__(self, x):
        from rust_inference_b200 import ops
        z = ops.linear(x, self.weight, out_dtype=torch.float32) + self.bias
        return self.spec.cap * torch.tanh(z / self.spec.cap)


@register_architecture("ToyParallelLM")
@dataclass(frozen=True)
class ParallelConfig:
    vocab_size: int = 83
    hidden_size: int = 40
    cap: float = 2.5

    @classmethod
    def from_dict(cls, d):
        return cls(**{k: d[k] for k in ("vocab_size", "hidden_size", "cap") if k in d})

    def validate(self):
        pass

    def to_dict(self):
        return {"architectures": ["ToyParallelLM"], "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                "cap": self.cap}

    def to_spec(self):
        D = self.hidden_size
        norm = RMSNormSpec(size=D, eps=1e-5)
        attn = AttentionSpec(hidden_size=D, num_heads=2, num_kv_heads=2, head_dim=24,
                             position=RopeSpec(head_dim=24, theta=1e4), qk_norm=None)
        layers = tuple(ParallelLayerSpec(norm=norm, mixer=attn, ffn=SwiGLUSpec(hidden_size=D, intermediate_size=56), names=(
            ("norm", f"blocks.{i}.norm."), ("mixer", f"blocks.{i}.attn."), ("ffn", f"blocks.{i}.ffn."))) for i in range(2))
        return ModelSpec(architecture="ToyParallelLM", vocab_size=self.vocab_size, hidden_size=D, layers=layers,
                         schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 1)), final_norm=norm, tie_embeddings=False,
                         max_positions=256, embedding_name="tok.weight", head_name="out.weight", final_norm_prefix="norm.",
                         head_optional=False,
                         embedding=ScaledEmbeddingSpec(self.vocab_size, D, math.sqrt(D), 256),
                         head=CappedHeadSpec(self.vocab_size, D, self.cap))


def parallel_plain(cfg, W, ids):
    n, D = len(ids), cfg.hidden_size
    h = W["tok.weight"][np.asarray(ids)] * math.sqrt(D) + W["tok.positions"][:n]
    for i in range(2):
        p = f"blocks.{i}."
        x = plain.rms_norm(h, W[p + "norm.weight"], 1e-5)
        q = plain.linear(x, W[p + "attn.q_proj.weight"]).reshape(n, 2, 24)
        k = plain.linear(x, W[p + "attn.k_proj.weight"]).reshape(n, 2, 24)
        v = plain.linear(x, W[p + "attn.v_proj.weight"]).reshape(n, 2, 24)
        cos, sin = plain.rope_cos_sin(np.arange(n), 24, 1e4)
        a = plain.causal_attention(plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin), v)
        h = h + plain.linear(a.reshape(n, 48), W[p + "attn.o_proj.weight"]) + plain.swiglu_mlp(x, W, p + "ffn.")
    z = plain.rms_norm(h, W["norm.weight"], 1e-5) @ W["out.weight"].T + W["out.bias"]
    return cfg.cap * np.tanh(z / cfg.cap)


def test_toy_architecture_with_its_own_arrangement_embedding_and_head(tmp_path):
    from rust_inference_b200.engine import expected_tensors
    cfg = ParallelConfig()
    names = set(expected_tensors(cfg.to_spec()))
    assert {"tok.weight", "tok.positions", "out.weight", "out.bias", "blocks.1.norm.weight", "blocks.0.attn.q_proj.weight",
            "blocks.1.ffn.down_proj.weight"} <= names and not any("norm1" in n or "mixer_norm" in n for n in names)
    d = H.make_model_dir(tmp_path, cfg.to_dict(), seed=12, stored="float32", name="parallel")
    W = {k: v.astype(np.float64) for k, v in plain.read_safetensors(d + "/model.safetensors").items()}
    reqs = H.random_requests(np.random.default_rng(1), cfg.vocab_size, [9, 50, 33, 70])
    want = {rid: parallel_plain(cfg, W, toks) for rid, toks in reqs.items()}
    by_cutting = {}
    for label, steps in (("whole", H.trace_whole(reqs)), ("tail", H.trace_tail(reqs, tail=32)),
                         ("batches", H.trace_batches(reqs, 3, [7, 0, 20]))):
        out = str(tmp_path / f"parallel_{label}")
        H.replay_inprocess(d, "float32", steps, out, device="cuda")
        by_cutting[label] = H.collect(steps, out, cfg.vocab_size)
        H.assert_rows_close(by_cutting[label], want, "float32", f"toy parallel {label}")
    H.assert_rows_identical(by_cutting, "toy parallel")


def test_attention_refuses_a_per_head_norm_it_does_not_have():
    @dataclass(frozen=True)
    class OtherNormSpec:
        size: int
        eps: float
        kind: str = "layernorm"
    spec = AttentionSpec(hidden_size=32, num_heads=2, num_kv_heads=1, head_dim=16, qk_norm=OtherNormSpec(16, 1e-5))
    with pytest.raises(ValueError, match="per-head norm"):
        build_part("mixer", spec, env("float32"))


# ---- the remaining parts alone: embedding, output head, the arrangement of a layer -----------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_and_head_parts(dtype):
    from rust_inference_b200.config import EmbeddingSpec, HeadSpec
    rng = np.random.default_rng(5)
    V, D = 333, 56
    table = rng.standard_normal((V, D)).astype(np.float32)
    table = plain.bf16_round(table) if dtype == "bfloat16" else table
    emb = build_part("embedding", EmbeddingSpec(V, D), env(dtype))
    emb.load({"weight": dev(table, DT[dtype])})
    ids = np.array([0, 332, 7, 7, 100], dtype=np.int32)
    rows = emb(dev(ids, torch.int32))
    assert rows.dtype == torch.float32 and np.array_equal(rows.cpu().numpy(), plain.embedding(ids, table).astype(np.float32))
    head = build_part("head", HeadSpec(V, D), env(dtype))
    head.load({"weight": emb.table})                  # tied: the embedding's own storage
    assert head.weight.data_ptr() == emb.table.data_ptr()
    x = rng.standard_normal((4, D)).astype(np.float32)
    x = plain.bf16_round(x) if dtype == "bfloat16" else x
    logits = head(dev(x, DT[dtype]))
    want = plain.linear(x, table)
    assert logits.dtype == torch.float32 and logits.shape == (4, V)
    assert np.abs(logits.cpu().numpy() - want).max() <= (1e-5 if dtype == "float32" else 2e-2) * np.abs(want).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prenorm_block_alone(dtype):
    """One layer's arrangement by itself: the pending output of the part before is added by the first norm, the
    block's own outputs by the norms after them; against the plain decoder layer on a whole sequence."""
    from rust_inference_b200.cache import Cache
    from rust_inference_b200.parts import build_block
    from rust_inference_b200.parts.base import StepContext
    rng = np.random.default_rng(8)
    D, Hh, KV, Dh, I, n = 48, 3, 1, 16, 72, 37
    norm = RMSNormSpec(size=D, eps=1e-5)
    attn = AttentionSpec(hidden_size=D, num_heads=Hh, num_kv_heads=KV, head_dim=Dh, position=RopeSpec(head_dim=Dh, theta=1e4),
                         qk_norm=RMSNormSpec(size=Dh, eps=1e-5))
    spec = LayerSpec(mixer=attn, ffn=SwiGLUSpec(hidden_size=D, intermediate_size=I), mixer_norm=norm, ffn_norm=norm)
    block = build_block(spec, env(dtype))
    assert [name for name, _, _, _ in block.parts()] == ["mixer_norm", "mixer", "ffn_norm", "ffn"]
    p = "model.layers.0."
    W = {p + "self_attn.q_proj.weight": (Hh * Dh, D), p + "self_attn.k_proj.weight": (KV * Dh, D),
         p + "self_attn.v_proj.weight": (KV * Dh, D), p + "self_attn.o_proj.weight": (D, Hh * Dh),
         p + "mlp.gate_proj.weight": (I, D), p + "mlp.up_proj.weight": (I, D), p + "mlp.down_proj.weight": (D, I)}
    W = {k: (rng.standard_normal(s) * 0.2).astype(np.float32) for k, s in W.items()}
    if dtype == "bfloat16":
        W = {k: plain.bf16_round(w) for k, w in W.items()}
    for k in ("input_layernorm.weight", "post_attention_layernorm.weight"):
        W[p + k] = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    for k in ("self_attn.q_norm.weight", "self_attn.k_norm.weight"):
        W[p + k] = (1 + 0.1 * rng.standard_normal(Dh)).astype(np.float32)
    role = lambda k: torch.float32 if "norm" in k else DT[dtype]
    take = lambda prefix: {k[len(prefix):]: dev(w, role(k)) for k, w in W.items() if k.startswith(prefix)}
    block.mixer_norm.load(take(p + "input_layernorm."))
    block.ffn_norm.load(take(p + "post_attention_layernorm."))
    block.mixer.load(take(p + "self_attn."))
    block.ffn.load(take(p + "mlp."))
    block.mixer.prepare(64)
    cache = Cache([block.mixer.cache_request()], num_slots=1, num_pages=2, max_pages_per_seq=2, dtype=DT[dtype], device="cuda")
    slot = cache.alloc_slot()
    cache.extend([(slot, n)])
    cache.upload()
    i32 = lambda a: dev(np.asarray(a), torch.int32)
    ctx = StepContext(tok_seq=i32(np.zeros(n)), tok_pos=i32(np.arange(n)), seq_slot=i32([slot]), seq_start=i32([0, n]),
                      seq_len=i32([n]), num_tokens=n, num_seqs=1, max_new=n, max_len=n)
    h0 = rng.standard_normal((n, D)).astype(np.float32)
    pending = rng.standard_normal((n, D)).astype(np.float32) * 0.1
    pending = plain.bf16_round(pending) if dtype == "bfloat16" else pending
    resid = dev(h0)
    resid_out, delta = block(resid, dev(pending, DT[dtype]), ctx, cache.layer(0))
    got = resid_out.float().cpu().numpy() + delta.float().cpu().numpy()
    cfg = {"num_attention_heads": Hh, "num_key_value_heads": KV, "head_dim": Dh, "hidden_size": D, "rms_norm_eps": 1e-5,
           "rope_theta": 1e4}
    want = plain.decoder_layer(h0.astype(np.float64) + pending, {k: w.astype(np.float64) for k, w in W.items()}, 0, cfg, np.arange(n))
    assert np.abs(got - want).max() <= (2e-5 if dtype == "float32" else 3e-2) * np.abs(want).max()
