"""Each CUDA kernel alone against a plain float64 restatement, at sizes other than
the engine's configurations (odd widths, head sizes in steps of 16, vocabularies
that are no power of two)."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# elementwise kernels: one rounding of the output in bfloat16 (2^-8 relative)
ETOL = {"float32": 2e-6, "bfloat16": 5e-3}


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.ascontiguousarray(a)).to("cuda", dtype=dtype).contiguous()


def rnd(rng, *shape, scale=1.0, dtype="float32"):
    x = (rng.standard_normal(shape) * scale).astype(np.float32)
    return plain.bf16_round(x) if dtype == "bfloat16" else x


def close(got, want, tol, what):
    got = got.detach().float().cpu().numpy().astype(np.float64)
    err = np.abs(got - want).max()
    bound = tol * max(1e-6, np.abs(want).max())
    assert err <= bound, f"{what}: max error {err:.3e} > {bound:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embed(dtype):
    from rust_inference_b200 import ops
    rng = np.random.default_rng(0)
    table = rnd(rng, 1000, 72, dtype=dtype)
    ids = rng.integers(0, 1000, size=37)
    got = ops.embed(dev(ids, torch.int32), dev(table, DT[dtype]))
    assert got.dtype == torch.float32
    close(got, plain.embedding(ids, table), 0, "embed")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim", [24, 72, 1000, 5120])
def test_rmsnorm(dtype, dim):
    from rust_inference_b200 import ops
    rng = np.random.default_rng(dim)
    resid = rnd(rng, 19, dim)
    delta = rnd(rng, 19, dim, dtype=dtype)
    gain = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    eps = 1e-5
    r = dev(resid)
    got = ops.rmsnorm(r, dev(gain), eps, DT[dtype])
    close(got, plain.rms_norm(resid, gain, eps), ETOL[dtype], "rmsnorm")
    close(r, resid.astype(np.float64), 0, "rmsnorm must not touch the stream without a delta")
    got = ops.rmsnorm(r, dev(gain), eps, DT[dtype], delta=dev(delta, DT[dtype]))
    total = resid.astype(np.float64) + delta
    close(got, plain.rms_norm(total, gain, eps), ETOL[dtype], "add+rmsnorm")
    close(r, total, 2e-7, "add+rmsnorm writes the sum back in float32")
    rows = np.array([3, 3, 0, 18], dtype=np.int32)
    r2 = dev(resid)
    got = ops.rmsnorm(r2, dev(gain), eps, DT[dtype], delta=dev(delta, DT[dtype]), rows=dev(rows, torch.int32))
    close(got, plain.rms_norm(total[rows], gain, eps), ETOL[dtype], "gathered add+rmsnorm")
    close(r2, resid.astype(np.float64), 0, "gathered norm leaves the stream alone")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim,n_rows", [(72, 513), (4096, 1026), (5120, 700), (12288, 600)])
def test_rmsnorm_of_many_rows_equals_rows_taken_a_few_at_a_time(dtype, dim, n_rows):
    """A prompt step's norm runs several rows per block; each row's bits are those of the same
    row normed in a small call, at a row count that is no multiple of the rows per block."""
    from rust_inference_b200 import ops
    rng = np.random.default_rng(dim + n_rows)
    resid = rnd(rng, n_rows, dim)
    delta = rnd(rng, n_rows, dim, dtype=dtype)
    gain = dev((1 + 0.1 * rng.standard_normal(dim)).astype(np.float32))
    r = dev(resid)
    got = ops.rmsnorm(r, gain, 1e-6, DT[dtype], delta=dev(delta, DT[dtype]))
    total = resid.astype(np.float64) + delta
    close(got, plain.rms_norm(total, gain.cpu().numpy(), 1e-6), ETOL[dtype], "many-row add+rmsnorm")
    for lo in (0, n_rows - 5):
        r_few = dev(resid[lo:lo + 5])
        few = ops.rmsnorm(r_few, gain, 1e-6, DT[dtype], delta=dev(delta[lo:lo + 5], DT[dtype]))
        assert torch.equal(few, got[lo:lo + 5]) and torch.equal(r_few, r[lo:lo + 5])
    no_delta = ops.rmsnorm(r, gain, 1e-6, DT[dtype])
    assert torch.equal(no_delta, got)


@pytest.mark.parametrize("n,k", [(40, 1024), (7200, 2048), (24, 256), (9, 24)])
def test_rmsnorm_with_a_weight_hint(n, k):
    """Naming the matrix that the next linear reads changes no result (the kernel only asks for a
    part of it to be brought into L2), whether the matrix has fewer rows than the hint covers, more,
    rows of a single stage or rows that the hint does not take."""
    from rust_inference_b200 import ops
    rng = np.random.default_rng(n)
    dim = 72
    resid, delta = rnd(rng, 5, dim), rnd(rng, 5, dim, dtype="bfloat16")
    gain = dev((1 + 0.1 * rng.standard_normal(dim)).astype(np.float32))
    w = torch.zeros((n, k), dtype=torch.bfloat16, device="cuda")
    r1, r2 = dev(resid), dev(resid)
    want = ops.rmsnorm(r1, gain, 1e-6, torch.bfloat16, delta=dev(delta, torch.bfloat16))
    got = ops.rmsnorm(r2, gain, 1e-6, torch.bfloat16, delta=dev(delta, torch.bfloat16), then=w)
    torch.cuda.synchronize()
    assert torch.equal(got, want) and torch.equal(r1, r2)
    assert not w.any()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_silu_mul(dtype):
    from rust_inference_b200 import ops
    rng = np.random.default_rng(1)
    gu = rnd(rng, 7, 2 * 88, scale=3.0, dtype=dtype)
    got = ops.silu_mul(dev(gu, DT[dtype]))
    g, u = gu[:, :88].astype(np.float64), gu[:, 88:].astype(np.float64)
    close(got, plain.silu(g) * u, ETOL[dtype], "silu_mul")
    for block in (8, 11, 44):          # gate and up alternating in blocks
        v = gu.reshape(7, 88 // block, 2, block).astype(np.float64)
        want = plain.silu(v[:, :, 0]) * v[:, :, 1]
        close(ops.silu_mul(dev(gu, DT[dtype]), block), want.reshape(7, 88), ETOL[dtype], f"silu_mul block {block}")


@pytest.mark.parametrize("shape", [(1, 64, 64), (5, 37, 70), (64, 192, 96), (130, 257, 1000), (3, 1000, 24)])
def test_linear_f32(shape):
    from rust_inference_b200 import ops
    M, N, K = shape
    rng = np.random.default_rng(M + N)
    x, w = rnd(rng, M, K), rnd(rng, N, K)
    got = ops.linear(dev(x), dev(w))
    close(got, plain.linear(x, w), 3e-6, f"linear_f32 {shape}")
    # a row's result does not depend on the rows around it
    alone = ops.linear(dev(x[M - 1:M]), dev(w))
    assert torch.equal(alone[0], got[M - 1])


@pytest.mark.parametrize("shape", [(1, 64, 64), (5, 48, 80), (300, 264, 1000), (8, 100, 4096), (3, 257, 1544),
                                   (9, 40, 72), (16, 4096, 264), (2, 151936, 96), (17, 64, 64)])
def test_linear_bf16(shape, monkeypatch):
    from rust_inference_b200 import ops
    M, N, K = shape
    if M <= 16:
        monkeypatch.setattr(ops, "SKINNY_MAX_TOKENS", 16)      # the mma.sync kernel over its whole range of tokens
    rng = np.random.default_rng(M)
    x, w = rnd(rng, M, K, dtype="bfloat16"), rnd(rng, N, K, dtype="bfloat16")
    want = plain.linear(x, w)
    close(ops.linear(dev(x, torch.bfloat16), dev(w, torch.bfloat16)), want, 5e-3, "linear bf16")
    full = ops.linear(dev(x, torch.bfloat16), dev(w, torch.bfloat16), out_dtype=torch.float32)
    close(full, want, 2e-5, "linear bf16 -> f32")
    if M <= 16:      # the weight-streaming kernel: a token alone gives the same bits as in the batch
        alone = ops.linear(dev(x[M - 1:M], torch.bfloat16), dev(w, torch.bfloat16), out_dtype=torch.float32)
        assert torch.equal(alone[0], full[M - 1])


@pytest.mark.parametrize("shape", [(1, 32, 64), (5, 208, 520), (16, 4096, 1024), (9, 48, 72)])
def test_linear_swiglu_fused(shape, monkeypatch):
    """The weight-streaming linear with the SiLU gate in its epilogue: gate and up rows interleaved
    in blocks of 8, widths and depths that end inside a tile or a stage."""
    from rust_inference_b200 import ops
    monkeypatch.setattr(ops, "SKINNY_MAX_TOKENS", 16)          # the kernel's whole range of tokens
    M, N, K = shape                      # N rows of gate and up together
    rng = np.random.default_rng(N)
    x = rnd(rng, M, K, dtype="bfloat16")
    gate, up = rnd(rng, N // 2, K, scale=0.2, dtype="bfloat16"), rnd(rng, N // 2, K, scale=0.2, dtype="bfloat16")
    w = np.stack([gate.reshape(-1, 8, K), up.reshape(-1, 8, K)], axis=1).reshape(N, K)
    got = ops.linear_swiglu(dev(x, torch.bfloat16), dev(w, torch.bfloat16), 8)
    assert got.shape == (M, N // 2)
    g, u = plain.linear(x, gate), plain.linear(x, up)
    close(got, g / (1.0 + np.exp(-g)) * u, 5e-3, f"fused swiglu {shape}")
    alone = ops.linear_swiglu(dev(x[M - 1:M], torch.bfloat16), dev(w, torch.bfloat16), 8)
    assert torch.equal(alone[0], got[M - 1])


@pytest.mark.parametrize("shape", [(17, 100, 72), (40, 257, 1544), (64, 4096, 4096), (128, 1000, 12288), (65, 24576, 512),
                                   (33, 130, 8), (13, 4096, 1544), (16, 264, 4096)])
def test_linear_stream_tc(shape):
    """The tcgen05 weight-streaming linear (up to 128 tokens): widths and depths that end inside a tile or a
    stage, splits of K over a cluster with the partial tiles added in a fixed order, twice in a row."""
    from rust_inference_b200 import ops
    M, N, K = shape
    rng = np.random.default_rng(N)
    x, w = rnd(rng, M, K, dtype="bfloat16"), rnd(rng, N, K, dtype="bfloat16")
    want = plain.linear(x, w)
    xd, wd = dev(x, torch.bfloat16), dev(w, torch.bfloat16)
    full = ops.linear_stream_tc(xd, wd, out_dtype=torch.float32)
    close(full, want, 2e-5, f"linear_stream_tc {shape} -> f32")
    close(ops.linear_stream_tc(xd, wd), want, 5e-3, f"linear_stream_tc {shape}")
    again = ops.linear_stream_tc(xd, wd, out_dtype=torch.float32)
    assert torch.equal(again, full)
    assert int(ops.error_flag("cuda").item()) == 0
    # a token's result does not depend on the tokens around it (as long as the kernel is the same)
    if M > 13:
        fewer = ops.linear_stream_tc(dev(x[:13], torch.bfloat16), wd, out_dtype=torch.float32)
        assert torch.equal(fewer, full[:13])


@pytest.mark.parametrize("M,taken", [(1, False), (2, False), (3, True), (8, True), (12, True), (40, True), (128, True)])
def test_gate_up_product_of_a_few_tokens_on_the_tcgen05_kernel(M, taken, monkeypatch):
    """At Qwen3-8B's feed-forward shape (24,576 gate and up rows of 4,096) the product of 3 to 128 tokens with the SiLU
    gate runs on the tcgen05 weight-streaming kernel, fewer tokens on the mma.sync one; both ways (above 12 tokens
    the other way is the product and the gate apart) give the product and the gate of the plain formulas, and a
    smaller matrix stays where it was."""
    from rust_inference_b200 import ops
    N, K = 24576, 4096
    rng = np.random.default_rng(M)
    x = rnd(rng, M, K, dtype="bfloat16")
    w = rnd(rng, N, K, scale=0.05, dtype="bfloat16")
    xd, wd = dev(x, torch.bfloat16), dev(w, torch.bfloat16)
    assert ops._gated_on_stream_tc(M, N, K, xd.device) == taken
    assert not ops._gated_on_stream_tc(8, 6144, 4096, xd.device)
    got = ops.linear_swiglu(xd, wd, 8)
    v = plain.linear(x, w).reshape(M, N // 16, 2, 8)
    want = (plain.silu(v[:, :, 0]) * v[:, :, 1]).reshape(M, N // 2)
    close(got, want, 1e-2, f"gate/up product of {M} tokens")
    monkeypatch.setattr(ops, "_GATED_STREAM_TC", not taken)          # the other kernel
    if taken:
        other = ops.linear_swiglu(xd, wd, 8)
        close(other, got.float().cpu().numpy().astype(np.float64), 1e-2, "mma.sync against tcgen05")
    assert int(ops.error_flag("cuda").item()) == 0


@pytest.mark.parametrize("shape", [(13, 208, 520), (17, 4096, 1024), (32, 24576, 4096), (24, 48, 72), (64, 1040, 2048)])
def test_linear_stream_tc_gated(shape):
    """The tcgen05 weight-streaming linear with the SiLU gate in its epilogue (gate and up rows alternating in blocks
    of 8): alone in its cluster and with K split, widths that end inside a tile of 128 rows."""
    from rust_inference_b200 import ops
    M, N, K = shape                      # N rows of gate and up together
    rng = np.random.default_rng(N + M)
    x = rnd(rng, M, K, dtype="bfloat16")
    gate, up = rnd(rng, N // 2, K, scale=0.2, dtype="bfloat16"), rnd(rng, N // 2, K, scale=0.2, dtype="bfloat16")
    nb = N // 16
    w = np.stack([gate.reshape(nb, 8, K), up.reshape(nb, 8, K)], axis=1).reshape(N, K)
    g, u = plain.linear(x, gate), plain.linear(x, up)
    want = plain.silu(g) * u
    xd, wd = dev(x, torch.bfloat16), dev(w, torch.bfloat16)
    got = ops.linear_stream_tc(xd, wd, gated=True)
    assert got.shape == (M, N // 2)
    close(got, want, 5e-3, f"gated linear_stream_tc {shape}")
    assert torch.equal(ops.linear_stream_tc(xd, wd, gated=True), got)
    # the same through the feed-forward's entry point, against the product followed by the separate gate
    fused = ops.linear_swiglu(xd, wd, 8)
    apart = ops.silu_mul(ops.linear_stream_tc(xd, wd), 8)
    close(fused, apart.float().cpu().numpy().astype(np.float64), 1e-2, "fused against product and gate apart")
    assert int(ops.error_flag("cuda").item()) == 0


def test_linear_takes_the_streaming_kernel_for_wide_outputs(monkeypatch):
    """`ops.linear` for 33 to 128 tokens hands matrices with many outputs (an output head) to the tcgen05
    streaming kernel and the others to the library; the threshold lowered, both ways give the same product."""
    from rust_inference_b200 import ops
    rng = np.random.default_rng(5)
    x, w = rnd(rng, 40, 200, dtype="bfloat16"), rnd(rng, 333, 200, dtype="bfloat16")
    xd, wd = dev(x, torch.bfloat16), dev(w, torch.bfloat16)
    want = plain.linear(x, w)
    library = ops.linear(xd, wd, out_dtype=torch.float32)
    n0 = ops.launch_count()
    monkeypatch.setattr(ops, "STREAM_TC_WIDE", 300)
    own = ops.linear(xd, wd, out_dtype=torch.float32)
    assert ops.launch_count() == n0 + 1, "the streaming kernel counts as a launch of this package, the library does not"
    close(own, want, 2e-5, "linear (streaming kernel)")
    close(library, want, 2e-5, "linear (library)")
    assert torch.equal(own, ops.linear_stream_tc(xd, wd, out_dtype=torch.float32))
    # up to 32 tokens the streaming kernel is taken whatever the width (it is the faster one inside a decode step)
    n0 = ops.launch_count()
    few = ops.linear(xd[:24], wd, out_dtype=torch.float32)
    assert ops.launch_count() == n0 + 1
    close(few, want[:24], 2e-5, "linear (streaming kernel, 24 tokens)")


def _paged(rng, lens, KV, Dh, P, dtype, extra_pages=3):
    """Random pools with a shuffled page table for sequences of the given lengths."""
    pages_per = [-(-n // P) for n in lens]
    total = sum(pages_per) + extra_pages
    order = rng.permutation(total)
    mpps = max(pages_per) + 1
    table = np.full((len(lens) + 2, mpps), -1, dtype=np.int32)
    slots = rng.permutation(len(lens) + 2)[:len(lens)]
    k = 0
    for b, n in enumerate(pages_per):
        table[slots[b], :n] = order[k:k + n]
        k += n
    return table, slots.astype(np.int32), total


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,KV,Dh,window,full", [(4, 2, 16, 0, True), (6, 1, 32, 0, True), (3, 3, 48, 0, False),
                                                 (8, 2, 128, 0, False), (5, 5, 80, 37, False), (4, 1, 256, 0, False),
                                                 (2, 1, 64, 5, False), (6, 2, 64, 0, True), (8, 2, 128, 0, True),
                                                 (3, 1, 256, 0, True)])
def test_norm_rope_append_then_attention(dtype, H, KV, Dh, window, full):
    """New tokens of several sequences against an existing cache: the appended keys and
    values land in the right page rows and every query sees exactly its keys."""
    from rust_inference_b200 import ops
    rng = np.random.default_rng(H * 1000 + Dh)
    P = 32
    old = [0, 31, 64, 70]                     # cache lengths before the step
    new = [40, 1, 3, 27]                      # tokens each sequence brings
    lens = [a + b for a, b in zip(old, new)]
    table, slots, total = _paged(rng, lens, KV, Dh, P, dtype)
    tdt = DT[dtype]
    eps, theta, rot = 1e-5, 10000.0, Dh if full else Dh - 16     # whole head rotated, or all but the last 16
    # full k/v history in plain form (already normed and rotated), then the new raw tokens
    k_hist = [rnd(rng, n, KV, Dh, dtype=dtype) for n in old]
    v_hist = [rnd(rng, n, KV, Dh, dtype=dtype) for n in old]
    k_pool = np.zeros((total, KV, P, Dh), dtype=np.float32)
    v_pool = np.zeros_like(k_pool)
    for b, n in enumerate(old):
        for j in range(n):
            pg = table[slots[b], j // P]
            k_pool[pg, :, j % P] = k_hist[b][j]
            v_pool[pg, :, j % P] = v_hist[b][j]
    T = sum(new)
    qkv = rnd(rng, T, (H + 2 * KV) * Dh, dtype=dtype)
    qg = (1 + 0.1 * rng.standard_normal(Dh)).astype(np.float32)
    kg = (1 + 0.1 * rng.standard_normal(Dh)).astype(np.float32)
    tok_seq = np.concatenate([np.full(n, b) for b, n in enumerate(new)]).astype(np.int32)
    tok_pos = np.concatenate([np.arange(o, o + n) for o, n in zip(old, new)]).astype(np.int32)
    # rope table as the position part builds it
    from rust_inference_b200.config import RopeSpec
    from rust_inference_b200.parts import BuildEnv, build_part
    rope = build_part("position", RopeSpec(head_dim=Dh, theta=theta, rotary_dim=rot),
                      BuildEnv(tdt, torch.device("cuda")))
    rope.prepare(max(lens) + 1)
    kp, vp = dev(k_pool, tdt), dev(v_pool, tdt)
    args = (dev(table, torch.int32), dev(tok_seq, torch.int32), dev(tok_pos, torch.int32), dev(slots, torch.int32))
    q = ops.qk_norm_rope_append(dev(qkv, tdt), H, KV, Dh, dev(qg), dev(kg), eps, rope.fused_table(), rot, kp, vp, *args)
    starts = np.concatenate([[0], np.cumsum(new)]).astype(np.int32)
    out = ops.attention(q, kp, vp, args[0], args[3], dev(starts, torch.int32), dev(np.array(lens), torch.int32), max(new),
                        1.0 / math.sqrt(Dh), window)
    torch.cuda.synchronize()
    assert int(ops.error_flag("cuda").item()) == 0

    # plain: per sequence, norm + partial rope of the new q/k, then attention over history + new
    x = qkv.reshape(T, H + 2 * KV, Dh).astype(np.float64)
    t0 = 0
    tol = {"float32": 1e-5, "bfloat16": 2e-2}[dtype]
    for b, (o, n) in enumerate(zip(old, new)):
        xs = x[t0:t0 + n]
        cos, sin = plain.rope_cos_sin(np.arange(o, o + n), rot, theta)

        def enc(t, gain):
            t = plain.rms_norm(t, gain, eps)
            return np.concatenate([plain.apply_rope(t[..., :rot], cos, sin), t[..., rot:]], axis=-1)
        qn, kn, vn = enc(xs[:, :H], qg), enc(xs[:, H:H + KV], kg), xs[:, H + KV:]
        if dtype == "bfloat16":      # what the cache holds is rounded
            qn, kn = plain.bf16_round(qn.astype(np.float32)).astype(np.float64), plain.bf16_round(kn.astype(np.float32)).astype(np.float64)
        kall = np.concatenate([k_hist[b].astype(np.float64), kn])
        vall = np.concatenate([v_hist[b].astype(np.float64), vn])
        qall = np.concatenate([np.zeros((o, H, Dh)), qn])
        want = plain.causal_attention(qall, kall, vall, window=window)[o:]
        close(q[t0:t0 + n], qn, {"float32": 2e-6, "bfloat16": 5e-3}[dtype], f"q of sequence {b}")
        close(out[t0:t0 + n], want, tol, f"attention of sequence {b}")
        # appended rows
        for j in (o, o + n - 1):
            pg = table[slots[b], j // P]
            close(kp[pg, :, j % P], kn[j - o], {"float32": 2e-6, "bfloat16": 5e-3}[dtype], f"appended key {j} of sequence {b}")
            close(vp[pg, :, j % P], vn[j - o], 0, f"appended value {j} of sequence {b}")
        t0 += n


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,KV,Dh,P,window", [(4, 2, 20, 32, 0), (6, 2, 64, 16, 0), (3, 1, 36, 48, 0), (8, 2, 128, 32, 45),
                                             (40, 1, 512, 32, 0), (2, 2, 8, 5, 7)])
def test_attention_rows_any_page_size_and_cutting(dtype, H, KV, Dh, P, window):
    """The attention of the float32 path alone: head sizes that are no multiple of 4 or of 16, page sizes other
    than 32 (strips shorter than a warp), a group larger than a block holds at head size 512; against the plain
    attention, and bit for bit the same whether a sequence's queries come in one step, in pieces or one by one
    beside other sequences."""
    from rust_inference_b200 import ops
    rng = np.random.default_rng(Dh * 7 + P)
    tdt = DT[dtype]
    lens = [70, 33, 101]
    table, slots, total = _paged(rng, lens, KV, Dh, P, dtype)
    ks = [rnd(rng, n, KV, Dh, scale=0.5, dtype=dtype) for n in lens]
    vs = [rnd(rng, n, KV, Dh, dtype=dtype) for n in lens]
    qs = [rnd(rng, n, H, Dh, dtype=dtype) for n in lens]
    k_pool = np.full((total, KV, P, Dh), np.nan, dtype=np.float32)        # rows nobody wrote must not matter
    v_pool = np.full_like(k_pool, np.nan)
    for b, n in enumerate(lens):
        for j in range(n):
            pg = table[slots[b], j // P]
            k_pool[pg, :, j % P], v_pool[pg, :, j % P] = ks[b][j], vs[b][j]
    kp, vp, tb = dev(k_pool, tdt), dev(v_pool, tdt), dev(table, torch.int32)
    scale = 1.0 / math.sqrt(Dh)

    def run(pieces):
        """pieces: per sequence (first query, one past the last); the cache is taken to hold the keys up to there"""
        live = [(b, lo, hi) for b, (lo, hi) in enumerate(pieces) if hi > lo]
        q = np.concatenate([qs[b][lo:hi] for b, lo, hi in live])
        starts = np.concatenate([[0], np.cumsum([hi - lo for _, lo, hi in live])])
        out = ops.attention(dev(q, tdt), kp, vp, tb, dev(slots[[b for b, _, _ in live]], torch.int32),
                            dev(starts, torch.int32), dev(np.array([hi for _, _, hi in live]), torch.int32),
                            max(hi - lo for _, lo, hi in live), scale, window).float().cpu().numpy()
        return {(b, lo + i): out[starts[k] + i] for k, (b, lo, hi) in enumerate(live) for i in range(hi - lo)}

    whole = run([(0, n) for n in lens])
    assert _take_error(ops) == 0
    for b, n in enumerate(lens):
        want = plain.causal_attention(qs[b].astype(np.float64), ks[b].astype(np.float64), vs[b].astype(np.float64), window=window)
        got = torch.from_numpy(np.stack([whole[(b, i)] for i in range(n)]))
        close(got, want, {"float32": 1e-5, "bfloat16": 2e-2}[dtype], f"sequence {b}")
    cut = {}
    cut.update(run([(0, 40), (0, 1), (0, 17)]))
    cut.update(run([(40, 41), (1, 33), (17, 18)]))
    cut.update(run([(41, 70), (0, 0), (18, 101)]))
    assert set(cut) == set(whole)
    for key in whole:
        assert np.array_equal(cut[key], whole[key]), f"row {key} depends on the cutting"


def test_attention_far_key_stands_out():
    """One key far back among hundreds gets nearly all the weight: a kernel that
    skipped or misplaced it would return another value row."""
    from rust_inference_b200 import ops
    rng = np.random.default_rng(3)
    for dtype in ("float32", "bfloat16"):
        H, KV, Dh, P, n = 4, 2, 64, 32, 700
        tdt = DT[dtype]
        table, slots, total = _paged(rng, [n], KV, Dh, P, dtype)
        k = rnd(rng, n, KV, Dh, scale=0.1, dtype=dtype)
        v = rnd(rng, n, KV, Dh, dtype=dtype)
        q = rnd(rng, 1, H, Dh, scale=0.1, dtype=dtype)
        far = 37
        k[far, 1] = q[0, 2] * 400.0           # head 2 reads kv head 1
        k = plain.bf16_round(k) if dtype == "bfloat16" else k
        k_pool = np.zeros((total, KV, P, Dh), dtype=np.float32)
        v_pool = np.zeros_like(k_pool)
        for j in range(n):
            pg = table[slots[0], j // P]
            k_pool[pg, :, j % P], v_pool[pg, :, j % P] = k[j], v[j]
        out = ops.attention(dev(q, tdt), dev(k_pool, tdt), dev(v_pool, tdt), dev(table, torch.int32),
                            dev(slots, torch.int32), dev(np.array([0, 1]), torch.int32), dev(np.array([n]), torch.int32),
                            1, 1.0 / math.sqrt(Dh), 0)
        qall = np.concatenate([np.zeros((n - 1, H, Dh)), q.astype(np.float64)])
        want = plain.causal_attention(qall, k.astype(np.float64), v.astype(np.float64))[n - 1:]
        assert np.abs(want[0, 2] - v[far, 1]).max() < 1e-2     # the far key really dominates
        close(out, want, {"float32": 1e-5, "bfloat16": 2e-2}[dtype], "far key")


def test_argmax_first_maximum():
    from rust_inference_b200 import ops
    rng = np.random.default_rng(4)
    x = rng.standard_normal((5, 151937)).astype(np.float32)
    x[0, 777] = x[0, 150000] = 9.0            # a tie: the lower index wins
    x[1, 151936] = 8.0                        # the very last element
    x[2, 0] = 8.0
    got = ops.argmax(dev(x)).cpu().numpy()
    assert got.tolist() == [int(np.argmax(r)) for r in x]
    assert got[0] == 777 and got[1] == 151936 and got[2] == 0


@pytest.mark.parametrize("vocab", [50, 1000, 151936])
def test_sample_matches_plain(vocab):
    """The device sampler picks the plain sampler's token for the same uniform number."""
    from rust_inference_b200 import ops
    rng = np.random.default_rng(vocab)
    rows = 12
    logits = (rng.standard_normal((rows, vocab)) * 3).astype(np.float32)
    logits[3, 10] = logits[3, 20] = logits[3].max() + 1.0      # equal logits at the top
    cases = [dict(temperature=0.0), dict(temperature=0.8), dict(temperature=1.3, top_k=5),
             dict(temperature=1.0, top_p=0.6), dict(temperature=0.7, top_k=40, top_p=0.9),
             dict(temperature=0.9, repetition_penalty=1.5), dict(temperature=0.0, repetition_penalty=3.0),
             dict(temperature=1.0, top_k=1)]
    seen = np.zeros((rows, vocab), dtype=np.uint8)
    hist = [list(rng.integers(0, vocab, size=20)) + [int(np.argmax(logits[r]))] for r in range(rows)]
    for r in range(rows):
        seen[r, hist[r]] = 1
    for c in cases:
        u = rng.random(rows).astype(np.float32)
        got = ops.sample(dev(logits), dev(np.full(rows, c.get("temperature", 0.0), dtype=np.float32)), dev(u),
                         top_k=dev(np.full(rows, c.get("top_k", 0)), torch.int32),
                         top_p=dev(np.full(rows, c.get("top_p", 1.0), dtype=np.float32)),
                         penalty=dev(np.full(rows, c.get("repetition_penalty", 1.0), dtype=np.float32)),
                         seen=dev(seen, torch.uint8)).cpu().numpy()

        # the plain sampler sums 150 000 probabilities one by one in float32, which moves the
        # boundaries far out in the tail by about 1e-5; the device sums exactly.  So the device
        # token is held against the same rule evaluated in float64, with u and top_p moved by
        # what float32 exp can account for
        for r in range(rows):
            ok = {_ideal_sample(logits[r], hist[r], float(u[r]) + du, dp=dp, **c)
                  for du in (0.0, -2e-6, 2e-6) for dp in (0.0, -2e-6, 2e-6)}
            assert got[r] in ok, f"{c} row {r}: device {got[r]}, float64 rule {sorted(ok)}"
        if vocab <= 1000:      # short sums: the plain sampler itself agrees

            class Fixed:
                def __init__(self, v):
                    self.v = v

                def next_f32(self):
                    return np.float32(self.v)
            want = [plain.plain_sample(logits[r], hist[r], Fixed(u[r]), **c) for r in range(rows)]
            assert sum(int(g != w) for g, w in zip(got, want)) <= 1, f"{c}: device {got}, plain {want}"


@pytest.mark.parametrize("vocab", [16384, 40001, 151936])
def test_sample_with_several_blocks_per_row_picks_the_same_token(vocab, monkeypatch):
    """Large vocabularies are sampled by several blocks per row, as one kernel whose blocks meet at a barrier per
    row after every pass, or (batches too large for that) as a kernel per pass; the token is the one the one-block
    kernel picks, for every mix of options within a batch (rows with and without top-k, top-p, a penalty, greedy rows)."""
    from rust_inference_b200 import ops
    rng = np.random.default_rng(vocab)
    rows = 37
    logits = (rng.standard_normal((rows, vocab)) * 3).astype(np.float32)
    logits[5, 100] = logits[5, 9000] = logits[5].max() + 0.5             # equal logits at the top
    logits[6, :] = 0.25                                                   # a flat row
    temperature = rng.choice([0.0, 0.5, 0.8, 1.0, 1.7], size=rows).astype(np.float32)
    top_k = rng.choice([0, 0, 1, 7, 50, 3000], size=rows).astype(np.int32)
    top_p = rng.choice([1.0, 1.0, 0.95, 0.6, 0.1], size=rows).astype(np.float32)
    penalty = rng.choice([1.0, 1.0, 1.3, 2.5], size=rows).astype(np.float32)
    seen = (rng.random((rows, vocab)) < 0.01).astype(np.uint8)
    seen_rows = rng.permutation(rows).astype(np.int32)
    args = dict(top_k=dev(top_k, torch.int32), top_p=dev(top_p), penalty=dev(penalty), seen=dev(seen, torch.uint8),
                seen_rows=dev(seen_rows, torch.int32))
    for trial in range(6):
        u = rng.random(rows).astype(np.float32)
        if trial == 0:
            u[:4] = [0.0, 0.99999994, 0.5, 1e-7]
        monkeypatch.setattr(ops, "_SAMPLE_WIDE", True)
        monkeypatch.setattr(ops, "SAMPLE_ONE_KERNEL", True)
        fused = ops.sample(dev(logits), dev(temperature), dev(u), **args).cpu().numpy()
        monkeypatch.setattr(ops, "SAMPLE_ONE_KERNEL", False)
        wide = ops.sample(dev(logits), dev(temperature), dev(u), **args).cpu().numpy()
        monkeypatch.setattr(ops, "_SAMPLE_WIDE", False)
        one = ops.sample(dev(logits), dev(temperature), dev(u), **args).cpu().numpy()
        assert wide.tolist() == one.tolist(), trial
        assert fused.tolist() == one.tolist(), trial
    # without the searches that a caller rules out: plain temperature rows
    monkeypatch.setattr(ops, "_SAMPLE_WIDE", True)
    u = rng.random(rows).astype(np.float32)
    t = dev(np.full(rows, 0.7, dtype=np.float32))
    wide = ops.sample(dev(logits), t, dev(u), uses_top_k=False, uses_top_p=False).cpu().numpy()
    monkeypatch.setattr(ops, "SAMPLE_ONE_KERNEL", True)
    fused = ops.sample(dev(logits), t, dev(u), uses_top_k=False, uses_top_p=False).cpu().numpy()
    # a batch of 300 rows: more blocks than the device holds at once with many slices, so fewer slices per row
    big = np.tile(logits, (9, 1))[:300]
    ub = rng.random(300).astype(np.float32)
    tb = dev(np.full(300, 0.7, dtype=np.float32))
    fused_big = ops.sample(dev(big), tb, dev(ub), uses_top_k=False, uses_top_p=False).cpu().numpy()
    monkeypatch.setattr(ops, "_SAMPLE_WIDE", False)
    one = ops.sample(dev(logits), t, dev(u)).cpu().numpy()
    assert wide.tolist() == one.tolist() and fused.tolist() == one.tolist()
    assert fused_big.tolist() == ops.sample(dev(big), tb, dev(ub)).cpu().numpy().tolist()
    assert int(ops.error_flag("cuda").item()) == 0


def _ideal_sample(logits, history, u, dp=0.0, temperature=0.0, top_k=0, top_p=1.0, repetition_penalty=1.0):
    """The reference's rule (src/sampling.rs:73-128 there) with exact sums."""
    x = np.array(logits, dtype=np.float32)
    if repetition_penalty != 1.0:
        pen = np.float32(repetition_penalty)
        for t in set(int(t) for t in history):
            x[t] = x[t] / pen if x[t] > 0 else x[t] * pen
    if temperature <= 0:
        return int(np.argmax(x))
    z = (x / np.float32(temperature)).astype(np.float32)
    order = np.lexsort((np.arange(len(z)), -z.astype(np.float64)))
    if 0 < top_k < len(z):
        order = order[:top_k]
    p = np.exp(z[order].astype(np.float64) - float(z[order[0]]))
    p /= p.sum()
    if top_p < 1.0:
        cum = np.cumsum(p)
        keep = int(np.searchsorted(cum, top_p + dp, side="left")) + 1
        p = p[:keep] / p[:keep].sum()
    cum = np.cumsum(p)
    j = int(np.searchsorted(cum, u, side="right"))
    return int(order[min(j, len(p) - 1)])


def test_sample_frequencies_and_top_p():
    """p = [0.25, 0.75]: the share of token 1 over many draws (src/sampling.rs:166-177 there)."""
    from rust_inference_b200 import ops
    from rust_inference_b200.sampling import XorShiftRng
    n = 4000
    logits = np.tile(np.array([[0.0, math.log(3.0)]], dtype=np.float32), (n, 1))
    rng = XorShiftRng(7)
    u = np.array([rng.next_f32() for _ in range(n)], dtype=np.float32)
    got = ops.sample(dev(logits), dev(np.ones(n, dtype=np.float32)), dev(u)).cpu().numpy()
    assert abs(got.mean() - 0.75) < 0.03
    # top_p 0.5: the first token alone has 0.84 of the mass
    logits = np.tile(np.array([[3.0, 1.0, 0.5, 0.0]], dtype=np.float32), (50, 1))
    got = ops.sample(dev(logits), dev(np.ones(50, dtype=np.float32)), dev(u[:50]),
                     top_p=dev(np.full(50, 0.5, dtype=np.float32))).cpu().numpy()
    assert (got == 0).all()


def _fill_pools(rng, lens, KV, Dh, dtype, scale=1.0, junk_nan=False):
    P = 32
    table, slots, total = _paged(rng, lens, KV, Dh, P, dtype)
    k = [rnd(rng, n, KV, Dh, scale=scale, dtype=dtype) for n in lens]
    v = [rnd(rng, n, KV, Dh, dtype=dtype) for n in lens]
    k_pool = (rng.standard_normal((total, KV, P, Dh)) * 50).astype(np.float32)     # junk where nothing is stored:
    v_pool = (rng.standard_normal((total, KV, P, Dh)) * 50).astype(np.float32)     # a kernel that reads it is caught
    if junk_nan:
        k_pool[:], v_pool[:] = np.nan, np.nan
    for b, n in enumerate(lens):
        for j in range(n):
            pg = table[slots[b], j // P]
            k_pool[pg, :, j % P], v_pool[pg, :, j % P] = k[b][j], v[b][j]
    return table, slots, k, v, k_pool, v_pool


@pytest.mark.parametrize("H,KV,Dh,window", [(4, 2, 16, 0), (6, 1, 32, 0), (3, 3, 48, 0), (32, 8, 128, 0), (5, 5, 80, 37),
                                            (4, 1, 256, 0), (2, 1, 64, 200), (20, 1, 64, 0), (34, 2, 32, 129)])
def test_attention_decode_kernel(H, KV, Dh, window):
    """Split-KV decode attention: lengths around page and chunk edges, groups of 1 to 20
    heads (more than the 16 rows of one pass), windows, a shuffled page table."""
    from rust_inference_b200 import ops
    rng = np.random.default_rng(H * 131 + Dh)
    lens = [1, 31, 32, 33, 127, 128, 129, 300, 700, 1025]
    table, slots, k, v, k_pool, v_pool = _fill_pools(rng, lens, KV, Dh, "bfloat16", scale=0.5)
    q = rnd(rng, len(lens), H, Dh, dtype="bfloat16")
    bt = torch.bfloat16
    out = ops.attention_decode(dev(q, bt), dev(k_pool, bt), dev(v_pool, bt), dev(table, torch.int32),
                               dev(slots, torch.int32), dev(np.array(lens), torch.int32), 1.0 / math.sqrt(Dh), window,
                               max(lens))
    torch.cuda.synchronize()
    assert int(ops.error_flag("cuda").item()) == 0
    for b, n in enumerate(lens):
        qall = np.concatenate([np.zeros((n - 1, H, Dh)), q[b:b + 1].astype(np.float64)])
        want = plain.causal_attention(qall, k[b].astype(np.float64), v[b].astype(np.float64), window=window)[n - 1:]
        close(out[b:b + 1], want, 2e-2, f"decode attention, length {n}")
    # the same sequence alone: the kernel that works in chunks of 128 keys gives the same bits, nothing depends on
    # the batch; the streaming kernel (head sizes 64 and 128, up to 16 heads per kv head) cuts the batch's pages
    # into equal runs, so the pieces that are added up are other pieces: the same up to the output's rounding
    one = ops.attention_decode(dev(q[8:9], bt), dev(k_pool, bt), dev(v_pool, bt), dev(table, torch.int32),
                               dev(slots[8:9], torch.int32), dev(np.array(lens[8:9]), torch.int32),
                               1.0 / math.sqrt(Dh), window, 2048)
    if Dh in (64, 128) and H // KV <= 16:
        close(one[0], out[8].float().cpu().numpy().astype(np.float64), 2 ** -7, "alone and in the batch")
    else:
        assert torch.equal(one[0], out[8])
    # and the same call again gives the same bits
    again = ops.attention_decode(dev(q, bt), dev(k_pool, bt), dev(v_pool, bt), dev(table, torch.int32),
                                 dev(slots, torch.int32), dev(np.array(lens), torch.int32), 1.0 / math.sqrt(Dh), window,
                                 max(lens))
    assert torch.equal(again, out)


@pytest.mark.parametrize("H,KV,Dh", [(8, 2, 128), (4, 4, 64), (6, 2, 32), (20, 1, 64)])
def test_attention_decode_unwritten_rows_are_nan(H, KV, Dh):
    """The rows of a sequence's last page past its end may hold anything, not-a-number included
    (a weight of zero times that would still be not-a-number)."""
    from rust_inference_b200 import ops
    rng = np.random.default_rng(Dh)
    lens = [1, 5, 31, 33, 64, 100, 129, 257]
    table, slots, k, v, k_pool, v_pool = _fill_pools(rng, lens, KV, Dh, "bfloat16", scale=0.5, junk_nan=True)
    q = rnd(rng, len(lens), H, Dh, dtype="bfloat16")
    bt = torch.bfloat16
    out = ops.attention_decode(dev(q, bt), dev(k_pool, bt), dev(v_pool, bt), dev(table, torch.int32),
                               dev(slots, torch.int32), dev(np.array(lens), torch.int32), 1.0 / math.sqrt(Dh), 0,
                               max(lens))
    assert int(ops.error_flag("cuda").item()) == 0
    assert bool(torch.isfinite(out.float()).all())
    for b, n in enumerate(lens):
        qall = np.concatenate([np.zeros((n - 1, H, Dh)), q[b:b + 1].astype(np.float64)])
        want = plain.causal_attention(qall, k[b].astype(np.float64), v[b].astype(np.float64))[n - 1:]
        close(out[b:b + 1], want, 2e-2, f"decode attention, length {n}")


def test_attention_decode_far_key():
    from rust_inference_b200 import ops
    rng = np.random.default_rng(9)
    H, KV, Dh, n = 8, 2, 128, 3000
    table, slots, k, v, k_pool, v_pool = _fill_pools(rng, [n], KV, Dh, "bfloat16", scale=0.1)
    q = rnd(rng, 1, H, Dh, scale=0.1, dtype="bfloat16")
    bt = torch.bfloat16
    for far in (0, 31, 32, 1500, 2999):
        kk = k[0].copy()
        kk[far, 1] = plain.bf16_round(q[0, 5] * 300.0)          # head 5 reads kv head 1
        kp = k_pool.copy()
        kp[table[slots[0], far // 32], 1, far % 32] = kk[far, 1]
        out = ops.attention_decode(dev(q, bt), dev(kp, bt), dev(v_pool, bt), dev(table, torch.int32),
                                   dev(slots, torch.int32), dev(np.array([n]), torch.int32), 1.0 / math.sqrt(Dh), 0, n)
        got = out[0, 5].float().cpu().numpy()
        assert np.abs(got - v[0][far, 1]).max() < 2e-2, f"key {far} should take all the weight"


@pytest.mark.parametrize("H,KV,Dh,window", [(4, 2, 16, 0), (6, 1, 32, 0), (3, 3, 48, 0), (8, 2, 128, 0), (5, 5, 80, 37),
                                            (4, 1, 256, 0), (2, 1, 64, 100), (4, 4, 96, 64)])
def test_attention_prefill_kernel(H, KV, Dh, window):
    """New tokens of several sequences against what their caches already hold: tiles that
    start in the middle of a page, sequences shorter than a tile, several tiles, windows."""
    from rust_inference_b200 import ops
    rng = np.random.default_rng(H * 77 + Dh)
    old = [0, 31, 64, 70, 0, 500, 0]
    new = [40, 1, 3, 27, 200, 130, 64]
    lens = [a + b for a, b in zip(old, new)]
    table, slots, k, v, k_pool, v_pool = _fill_pools(rng, lens, KV, Dh, "bfloat16", scale=0.5)
    T = sum(new)
    q = rnd(rng, T, H, Dh, dtype="bfloat16")
    starts = np.concatenate([[0], np.cumsum(new)]).astype(np.int32)
    bt = torch.bfloat16
    out = ops.attention_prefill(dev(q, bt), dev(k_pool, bt), dev(v_pool, bt), dev(table, torch.int32),
                                dev(slots, torch.int32), dev(starts, torch.int32), dev(np.array(lens), torch.int32),
                                max(new), 1.0 / math.sqrt(Dh), window)
    torch.cuda.synchronize()
    assert int(ops.error_flag("cuda").item()) == 0
    for b, (o, n) in enumerate(zip(old, new)):
        qall = np.concatenate([np.zeros((o, H, Dh)), q[starts[b]:starts[b + 1]].astype(np.float64)])
        want = plain.causal_attention(qall, k[b].astype(np.float64), v[b].astype(np.float64), window=window)[o:]
        close(out[starts[b]:starts[b + 1]], want, 2e-2, f"prefill attention, sequence {b}")
    # sequence 4 alone: the same bits
    one = ops.attention_prefill(dev(q[starts[4]:starts[5]], bt), dev(k_pool, bt), dev(v_pool, bt),
                                dev(table, torch.int32), dev(slots[4:5], torch.int32),
                                dev(np.array([0, new[4]]), torch.int32), dev(np.array(lens[4:5]), torch.int32), new[4],
                                1.0 / math.sqrt(Dh), window)
    assert torch.equal(one, out[starts[4]:starts[5]])


@pytest.mark.parametrize("Dh,window", [(128, 0), (64, 0), (128, 300)])
def test_attention_prefill_more_work_items_than_sms(Dh, window, monkeypatch):
    """The tcgen05 prefill kernel keeps one block per SM that takes its work items (256 rows of a sequence and a
    head) one after the other: 288 items here, of which those past a sequence's rows are empty, so every block
    passes from one item to the next (its buffers and barriers keep their turns across items), with sequences of
    unequal lengths, old keys in the cache and a window.  Against the plain attention for two heads and against
    the mma.sync kernel for all."""
    from rust_inference_b200 import ops
    H, KV = 16, 4
    rng = np.random.default_rng(Dh + window)
    old = [100, 0, 33]
    new = [700, 1300, 257]
    lens = [a + b for a, b in zip(old, new)]
    table, slots, k, v, k_pool, v_pool = _fill_pools(rng, lens, KV, Dh, "bfloat16", scale=0.5)
    T = sum(new)
    q = rnd(rng, T, H, Dh, dtype="bfloat16")
    starts = np.concatenate([[0], np.cumsum(new)]).astype(np.int32)
    bt = torch.bfloat16
    args = (dev(q, bt), dev(k_pool, bt), dev(v_pool, bt), dev(table, torch.int32), dev(slots, torch.int32),
            dev(starts, torch.int32), dev(np.array(lens), torch.int32), max(new), 1.0 / math.sqrt(Dh), window)
    out = ops.attention_prefill(*args)
    torch.cuda.synchronize()
    assert int(ops.error_flag("cuda").item()) == 0
    heads, kv_heads = [0, 13], [0, 3]
    for b, (o, n) in enumerate(zip(old, new)):
        qall = np.concatenate([np.zeros((o, 2, Dh)), q[starts[b]:starts[b + 1]][:, heads].astype(np.float64)])
        want = plain.causal_attention(qall, k[b][:, kv_heads].astype(np.float64), v[b][:, kv_heads].astype(np.float64),
                                      window=window)[o:]
        close(out[starts[b]:starts[b + 1]][:, heads], want, 2e-2, f"prefill attention, sequence {b}")
    again = ops.attention_prefill(*args)
    assert torch.equal(again, out)
    monkeypatch.setattr(ops, "_NO_TCGEN05", True)
    other = ops.attention_prefill(*args)
    close(out, other.float().cpu().numpy().astype(np.float64), 2e-2, "tcgen05 against mma.sync")
    assert int(ops.error_flag("cuda").item()) == 0


@pytest.mark.parametrize("H,KV,Dh", [(8, 2, 128), (4, 4, 64), (6, 2, 32)])
def test_attention_prefill_unwritten_rows_are_nan(H, KV, Dh):
    """As for decoding: what the pool holds past a sequence's end, not-a-number included, changes nothing."""
    from rust_inference_b200 import ops
    rng = np.random.default_rng(Dh + 1)
    old = [0, 10, 64, 0, 200]
    new = [40, 23, 1, 129, 100]
    lens = [a + b for a, b in zip(old, new)]
    table, slots, k, v, k_pool, v_pool = _fill_pools(rng, lens, KV, Dh, "bfloat16", scale=0.5, junk_nan=True)
    q = rnd(rng, sum(new), H, Dh, dtype="bfloat16")
    starts = np.concatenate([[0], np.cumsum(new)]).astype(np.int32)
    bt = torch.bfloat16
    out = ops.attention_prefill(dev(q, bt), dev(k_pool, bt), dev(v_pool, bt), dev(table, torch.int32),
                                dev(slots, torch.int32), dev(starts, torch.int32), dev(np.array(lens), torch.int32),
                                max(new), 1.0 / math.sqrt(Dh), 0)
    assert int(ops.error_flag("cuda").item()) == 0
    assert bool(torch.isfinite(out.float()).all())
    for b, (o, n) in enumerate(zip(old, new)):
        qall = np.concatenate([np.zeros((o, H, Dh)), q[starts[b]:starts[b + 1]].astype(np.float64)])
        want = plain.causal_attention(qall, k[b].astype(np.float64), v[b].astype(np.float64))[o:]
        close(out[starts[b]:starts[b + 1]], want, 2e-2, f"prefill attention, sequence {b}")


@pytest.mark.parametrize("H,KV,Dh,window,seqs,longest", [(8, 8, 64, 0, 44, 1100), (16, 4, 128, 0, 44, 1100),
                                                         (6, 2, 32, 300, 44, 1100), (12, 1, 128, 500, 44, 1100),
                                                         (16, 8, 128, 0, 196, 200)])
def test_attention_decode_many_sequences(H, KV, Dh, window, seqs, longest):
    """Many sequences: the streaming kernel's runs of pages that pass from one (sequence, kv head) to the
    next several times, that end inside one, sequences of a single page, windows that leave some
    sequences fewer pages than others; more sequences than a warp has lanes."""
    from rust_inference_b200 import ops
    rng = np.random.default_rng(H + Dh)
    lens = [int(n) for n in rng.integers(1, longest, size=seqs)] + [longest - 76, longest - 75, 33, 1]
    table, slots, k, v, k_pool, v_pool = _fill_pools(rng, lens, KV, Dh, "bfloat16", scale=0.5)
    q = rnd(rng, len(lens), H, Dh, dtype="bfloat16")
    bt = torch.bfloat16
    args = (dev(k_pool, bt), dev(v_pool, bt), dev(table, torch.int32), dev(slots, torch.int32),
            dev(np.array(lens), torch.int32), 1.0 / math.sqrt(Dh), window)
    out = ops.attention_decode(dev(q, bt), *args, max(lens))
    torch.cuda.synchronize()
    assert int(ops.error_flag("cuda").item()) == 0
    for b in range(0, len(lens), 3 if seqs < 100 else 11):
        n = lens[b]
        qall = np.concatenate([np.zeros((n - 1, H, Dh)), q[b:b + 1].astype(np.float64)])
        want = plain.causal_attention(qall, k[b].astype(np.float64), v[b].astype(np.float64), window=window)[n - 1:]
        close(out[b:b + 1], want, 2e-2, f"decode attention, sequence {b} of length {n}")
    again = ops.attention_decode(dev(q, bt), *args, max(lens))     # the same call, the same bits
    assert torch.equal(again, out)
    other = ops.attention_decode(dev(q, bt), *args, 2048)           # more scratch memory: possibly another cut of the pages
    close(other, out.float().cpu().numpy().astype(np.float64), 2 ** -7, "another cut of the pages")


def _take_error(ops):
    flag = ops.error_flag("cuda")
    torch.cuda.synchronize()
    code = int(flag.item())
    flag.zero_()
    return code


def test_kernels_report_indices_they_must_not_follow():
    """An id outside the vocabulary, a position beyond the rotary table, an unmapped or impossible page: the
    kernel leaves the access out, sets the error word (1, 3, 2, 4, 7) and goes on; nothing faults."""
    from rust_inference_b200 import ops
    from rust_inference_b200.config import RopeSpec
    from rust_inference_b200.parts import BuildEnv, build_part
    rng = np.random.default_rng(3)
    bt = torch.bfloat16
    assert _take_error(ops) == 0
    # 1: token id == vocabulary size
    table = dev(rnd(rng, 50, 64, dtype="bfloat16"), bt)
    ops.embed(dev(np.array([3, 50, 7]), torch.int32), table)
    assert _take_error(ops) == 1
    for Dh, H, KV in ((128, 8, 2), (32, 4, 2)):
        lens = [70, 33]
        pt, slots, k, v, k_pool, v_pool = _fill_pools(rng, lens, KV, Dh, "bfloat16", scale=0.5)
        kp, vp = dev(k_pool, bt), dev(v_pool, bt)
        i32 = lambda a: dev(np.asarray(a), torch.int32)
        rope = build_part("position", RopeSpec(head_dim=Dh, theta=1e4), BuildEnv(bt, torch.device("cuda")))
        rope.prepare(80)
        qkv = dev(rnd(rng, 2, (H + 2 * KV) * Dh, dtype="bfloat16"), bt)
        meta = (i32(pt), i32([0, 1]), i32([69, 32]), i32(slots))
        # 3: a position beyond the rotary table (80 rows, or more if a part with the same sizes made a longer one)
        ops.qk_norm_rope_append(qkv, H, KV, Dh, None, None, 0.0, rope.fused_table(), Dh, kp, vp, i32(pt), i32([0, 1]),
                                i32([69, rope.fused_table().shape[0] + 15]), i32(slots))
        assert _take_error(ops) == 3
        # 2: append to a page that is not mapped, and to one that cannot exist
        for bad in (-1, k_pool.shape[0] + 5):
            broken = pt.copy()
            broken[slots[0], 69 // 32] = bad
            ops.qk_norm_rope_append(qkv, H, KV, Dh, None, None, 0.0, rope.fused_table(), Dh, kp, vp, i32(broken), *meta[1:])
            assert _take_error(ops) == 2
        # 4: attention that meets such a page: decode (one token each), prefill (several), the kernel of the float32 path
        q1 = dev(rnd(rng, 2, H, Dh, dtype="bfloat16"), bt)
        qn = dev(rnd(rng, 10, H, Dh, dtype="bfloat16"), bt)
        for bad in (-1, k_pool.shape[0] + 5):
            broken = pt.copy()
            broken[slots[0], 1] = bad
            out = ops.attention_decode(q1, kp, vp, i32(broken), i32(slots), i32(lens), 0.1, 0, max(lens))
            assert _take_error(ops) == 4 and out.shape == q1.shape
            out = ops.attention_prefill(qn, kp, vp, i32(broken), i32(slots), i32([0, 5, 10]), i32(lens), 5, 0.1, 0)
            assert _take_error(ops) == 4 and out.shape == qn.shape
            out = ops.attention(q1, kp, vp, i32(broken), i32(slots), i32([0, 1, 2]), i32([70, 33]), 1, 0.1, 0)
            assert _take_error(ops) == 4 and out.shape == q1.shape
        # 7: a sequence longer than the decode attention's scratch memory covers (`max_len` sizes it): the keys
        # beyond are left out, nothing is read or written past the partial results
        lens = [300, 33]
        pt, slots, k, v, k_pool, v_pool = _fill_pools(rng, lens, KV, Dh, "bfloat16", scale=0.5)
        out = ops.attention_decode(q1, dev(k_pool, bt), dev(v_pool, bt), i32(pt), i32(slots), i32(lens), 0.1, 0, 128)
        assert _take_error(ops) == 7 and bool(torch.isfinite(out.float()).all())
    assert _take_error(ops) == 0


def test_a_wait_that_runs_out_ends_in_error_5_and_the_context_lives(tmp_path):
    """Every wait on an mbarrier inside the kernels is bounded (about 4 ms).  The weight-streaming linear is built
    here with a test-only define that makes block 0 leave out one copy of its first stage when K is 1024, so that
    stage's barrier never completes: the waiting warp must give up, report error 5 and start no further copies, the
    kernel must return, the other blocks' outputs must be right, and the next launch (another K: nothing is left out)
    must be right with the error word untouched.  Nothing hangs or faults: the wait is the bounded one."""
    import os
    import subprocess
    import sys
    code = r'''
import time, torch
import rust_inference_b200
from rust_inference_b200 import ops
torch.manual_seed(0)
flag = ops.error_flag("cuda")
x = torch.randn(3, 1024, device="cuda").to(torch.bfloat16)
w = torch.randn(40, 1024, device="cuda").to(torch.bfloat16)
ops.linear(x[:, :512].contiguous(), w[:, :512].contiguous())      # builds and loads the library (another K: nothing is left out)
torch.cuda.synchronize()
assert int(flag.item()) == 0
t0 = time.perf_counter()
y = ops.linear(x, w)
torch.cuda.synchronize()
ms = (time.perf_counter() - t0) * 1e3
assert int(flag.item()) == 5, int(flag.item())
flag.zero_()
want = x.float() @ w.float().t()
assert torch.allclose(y.float()[:, 16:], want[:, 16:], rtol=2e-2, atol=0.3), "outputs of the other blocks"
x2 = torch.randn(5, 2048, device="cuda").to(torch.bfloat16)
w2 = torch.randn(40, 2048, device="cuda").to(torch.bfloat16)
y2 = ops.linear(x2, w2)
torch.cuda.synchronize()
assert int(flag.item()) == 0
assert torch.allclose(y2.float(), x2.float() @ w2.float().t(), rtol=2e-2, atol=0.3)
print("gave up after %.1f ms" % ms)
'''
    env = dict(os.environ, RUST_INFERENCE_B200_DEFINES="SK_TEST_DROP_COPY_K=1024", PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout + r.stderr
    ms = float(r.stdout.split("after")[1].split()[0])
    assert 3.0 <= ms <= 2000.0, r.stdout


def test_a_wait_that_runs_out_in_the_tcgen05_linear(tmp_path):
    """The same for the tcgen05 weight-streaming linear, whose way out of a wait that has run out passes the
    cluster's barriers and the release of its tensor memory: built with a test-only define, the first block of a
    launch with K = 1536 leaves out the copy of W of its first stage.  The issuing lane and then the copying lane
    give up (about 4 ms each), error 5 is reported, the kernel returns, the other tiles' outputs are right and
    the next launch is right.  Nothing hangs or faults: the waits are the bounded ones."""
    import os
    import subprocess
    import sys
    code = r'''
import time, torch
import rust_inference_b200
from rust_inference_b200 import ops
torch.manual_seed(0)
flag = ops.error_flag("cuda")
x = torch.randn(20, 1536, device="cuda").to(torch.bfloat16)
w = torch.randn(300, 1536, device="cuda").to(torch.bfloat16)
ops.linear_stream_tc(x[:, :512].contiguous(), w[:, :512].contiguous())      # builds and loads the library (another K: nothing is left out)
torch.cuda.synchronize()
assert int(flag.item()) == 0
t0 = time.perf_counter()
y = ops.linear_stream_tc(x, w)
torch.cuda.synchronize()
ms = (time.perf_counter() - t0) * 1e3
assert int(flag.item()) == 5, int(flag.item())
flag.zero_()
want = x.float() @ w.float().t()
assert torch.allclose(y.float()[:, 128:], want[:, 128:], rtol=2e-2, atol=0.5), "outputs of the other tiles"
x2 = torch.randn(20, 2048, device="cuda").to(torch.bfloat16)
w2 = torch.randn(300, 2048, device="cuda").to(torch.bfloat16)
y2 = ops.linear_stream_tc(x2, w2)
torch.cuda.synchronize()
assert int(flag.item()) == 0
assert torch.allclose(y2.float(), x2.float() @ w2.float().t(), rtol=2e-2, atol=0.5)
print("gave up after %.1f ms" % ms)
'''
    env = dict(os.environ, RUST_INFERENCE_B200_DEFINES="LT_TEST_DROP_COPY_K=1536", PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout + r.stderr
    ms = float(r.stdout.split("after")[1].split()[0])
    assert 3.0 <= ms <= 2000.0, r.stdout


def test_a_wait_that_runs_out_in_the_streaming_decode_attention(tmp_path):
    """The same for the streaming decode attention (a ring of copies per warp): built with a test-only define, a copy
    of the first page of keys is left out in sequences of exactly 700 keys.  The warp gives up, reports error 5, starts
    no further copy and waits (bounded) for those it had started; the kernel returns, the other sequence of the
    launch is right, and so is the next launch."""
    import os
    import subprocess
    import sys
    code = r'''
import math, time, torch
import rust_inference_b200
from rust_inference_b200 import ops
torch.manual_seed(0)
flag = ops.error_flag("cuda")
H, KV, Dh = 8, 2, 128
bt = torch.bfloat16
i32 = lambda a: torch.tensor(a, dtype=torch.int32, device="cuda")
def run(lens):
    q = torch.randn(len(lens), H, Dh, device="cuda").to(bt)
    per = [-(-n // 32) for n in lens]
    k_pool = (torch.randn(sum(per), KV, 32, Dh, device="cuda") * 0.5).to(bt)
    v_pool = torch.randn(sum(per), KV, 32, Dh, device="cuda").to(bt)
    table = torch.full((len(lens), max(per)), -1, dtype=torch.int32)
    p = 0
    for b, n in enumerate(per):
        table[b, :n] = torch.arange(p, p + n, dtype=torch.int32)
        p += n
    out = ops.attention_decode(q, k_pool, v_pool, table.cuda(), i32(list(range(len(lens)))), i32(lens), 1.0 / math.sqrt(Dh), 0, max(lens))
    torch.cuda.synchronize()
    want = []
    for b, n in enumerate(lens):
        ids = table[b, :per[b]].long().cuda()
        rows = []
        for h in range(H):
            kk = k_pool[ids][:, h // (H // KV)].reshape(-1, Dh)[:n].float()
            vv = v_pool[ids][:, h // (H // KV)].reshape(-1, Dh)[:n].float()
            w = torch.softmax(kk @ q[b, h].float() / math.sqrt(Dh), 0)
            rows.append(w @ vv)
        want.append(torch.stack(rows))
    return out.float(), want
run([701, 300])                                                    # builds and loads the library (other lengths: nothing is left out)
assert int(flag.item()) == 0
t0 = time.perf_counter()
out, want = run([700, 300])
ms = (time.perf_counter() - t0) * 1e3
assert int(flag.item()) == 5, int(flag.item())
flag.zero_()
assert torch.allclose(out[1], want[1], rtol=2e-2, atol=2e-2), "the sequence of 300 keys"
assert torch.allclose(out[0, 4:], want[0][4:], rtol=2e-2, atol=2e-2), "the other kv head of the sequence of 700 keys"
out, want = run([701, 300])
assert int(flag.item()) == 0
for b in range(2):
    assert torch.allclose(out[b], want[b], rtol=2e-2, atol=2e-2)
print("gave up after %.1f ms" % ms)
'''
    env = dict(os.environ, RUST_INFERENCE_B200_DEFINES="ADS_TEST_DROP_COPY_LEN=700", PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout + r.stderr
    ms = float(r.stdout.split("after")[1].split()[0])
    assert 3.0 <= ms <= 2000.0, r.stdout


def test_a_wait_that_runs_out_in_the_tcgen05_attention(tmp_path):
    """The same for the tcgen05 prefill attention (barriers between a copying lane, two issuing lanes and eight warps
    of row threads; tensor memory to give back): built with a test-only define, a copy of the first block of keys is
    left out in sequences of exactly 100 keys.  Error 5 is reported, the kernel returns, a sequence of another length
    in the same launch is right, and so is the next launch."""
    import os
    import subprocess
    import sys
    code = r'''
import math, time, torch
import rust_inference_b200
from rust_inference_b200 import ops
torch.manual_seed(0)
flag = ops.error_flag("cuda")
H, KV, Dh = 2, 1, 128
bt = torch.bfloat16
i32 = lambda a: torch.tensor(a, dtype=torch.int32, device="cuda")
def run(new):
    T = sum(new)
    q = torch.randn(T, H, Dh, device="cuda").to(bt)
    pages = sum(-(-n // 32) for n in new)
    k_pool = (torch.randn(pages, KV, 32, Dh, device="cuda") * 0.5).to(bt)
    v_pool = torch.randn(pages, KV, 32, Dh, device="cuda").to(bt)
    table = torch.full((len(new), 8), -1, dtype=torch.int32)
    p = 0
    for b, n in enumerate(new):
        for j in range(-(-n // 32)):
            table[b, j] = p
            p += 1
    starts = [0]
    for n in new:
        starts.append(starts[-1] + n)
    out = ops.attention_prefill(q, k_pool, v_pool, table.cuda(), i32(list(range(len(new)))), i32(starts), i32(new), max(new),
                                1.0 / math.sqrt(Dh), 0)
    torch.cuda.synchronize()
    want = []
    for b, n in enumerate(new):
        ids = table[b, :-(-n // 32)].long().cuda()
        kk = k_pool[ids][:, 0].reshape(-1, Dh)[:n].float()
        vv = v_pool[ids][:, 0].reshape(-1, Dh)[:n].float()
        qq = q[starts[b]:starts[b + 1]].float()
        s = torch.einsum("thd,kd->htk", qq, kk) / math.sqrt(Dh)
        s = s.masked_fill(torch.triu(torch.ones(n, n, dtype=torch.bool, device="cuda"), 1), float("-inf"))
        want.append(torch.einsum("htk,kd->thd", torch.softmax(s, -1), vv))
    return out.float(), want, starts
run([101, 70])                                                     # builds and loads the library (other lengths: nothing is left out)
assert int(flag.item()) == 0
t0 = time.perf_counter()
out, want, starts = run([100, 70])
ms = (time.perf_counter() - t0) * 1e3
assert int(flag.item()) == 5, int(flag.item())
flag.zero_()
assert torch.allclose(out[starts[1]:starts[2]], want[1], rtol=2e-2, atol=2e-2), "the sequence of 70 keys"
out, want, starts = run([101, 70])
assert int(flag.item()) == 0
for b in range(2):
    assert torch.allclose(out[starts[b]:starts[b + 1]], want[b], rtol=2e-2, atol=2e-2)
print("gave up after %.1f ms" % ms)
'''
    env = dict(os.environ, RUST_INFERENCE_B200_DEFINES="TC_TEST_DROP_COPY_LEN=100", PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout + r.stderr
    ms = float(r.stdout.split("after")[1].split()[0])
    assert 3.0 <= ms <= 2000.0, r.stdout


@pytest.mark.parametrize("Dh,window,n", [(128, 100, 450), (64, 33, 300), (32, 64, 257), (48, 1, 90)])
def test_window_edges_stand_out(Dh, window, n):
    """The two keys at a window's edge get a score far above all others in two heads: in head 0 the last key
    outside the window (position pos - window), in head 1 the first one inside (pos - window + 1).  A kernel that
    is off by one at the edge returns the outside key's value row in head 0, or misses the inside key's in head 1.
    Checked for the newest token through the decode kernels, the float32-order kernel in both dtypes, and for
    several query positions at once through the prefill kernels (head sizes 64 and 128: tcgen05; others: mma.sync)."""
    from rust_inference_b200 import ops
    rng = np.random.default_rng(Dh + window)
    H, KV = 2, 1
    bt = torch.bfloat16
    scale = 1.0 / math.sqrt(Dh)
    new = 70                                         # the last `new` positions are this step's queries
    table, slots, k, v, k_pool, v_pool = _fill_pools(rng, [n], KV, Dh, "bfloat16", scale=0.1)
    q = rnd(rng, new, H, Dh, scale=0.1, dtype="bfloat16")
    # per checked query one direction that only it and the two keys at its window's edge carry
    kk = k[0].copy()
    q = q.astype(np.float32)
    dims = rng.permutation(Dh)
    checks = []
    for c, t in enumerate((0, new // 2, new - 1)):
        pos = n - new + t
        outside, inside = pos - window, pos - window + 1
        if outside < 0:
            continue
        q[t, :, dims[c]] += 40.0
        kk[outside, 0, dims[c]] += 60.0
        kk[inside, 0, dims[c]] += 30.0
        checks.append((t, pos, outside, inside))
    q = plain.bf16_round(q)
    assert checks
    kk = plain.bf16_round(kk)
    kp = k_pool.copy()
    for j in range(n):
        kp[table[slots[0], j // 32], :, j % 32] = kk[j]
    want = plain.causal_attention(np.concatenate([np.zeros((n - new, H, Dh)), q.astype(np.float64)]),
                                  kk.astype(np.float64), v[0].astype(np.float64), window=window)[n - new:]
    i32 = lambda a: dev(np.asarray(a), torch.int32)
    args = (i32(table), i32(slots), i32([0, new]), i32([n]), new, scale, window)
    outs = {"prefill": ops.attention_prefill(dev(q, bt), dev(kp, bt), dev(v_pool, bt), *args),
            "rows bfloat16": ops.attention(dev(q, bt), dev(kp, bt), dev(v_pool, bt), *args),
            "rows float32": ops.attention(dev(q), dev(kp), dev(v_pool), *args)}
    last = dev(q[new - 1:new], bt)
    outs_last = {"decode": ops.attention_decode(last, dev(kp, bt), dev(v_pool, bt), i32(table), i32(slots), i32([n]),
                                                scale, window, n)}
    assert _take_error(ops) == 0
    for t, pos, outside, inside in checks:
        # (the plain attention agrees that the edge decides: the inside key takes nearly all the weight)
        assert np.abs(want[t, 0] - v[0][inside, 0]).max() < 0.05 * np.abs(v[0]).max()
        for name, out in outs.items():
            got = out[t].float().cpu().numpy()
            assert np.abs(got - want[t]).max() <= 2e-2 * np.abs(want).max(), (name, t, pos, "window edge")
            assert np.abs(got[0] - v[0][outside, 0]).max() > 0.2, (name, t, "took the key outside the window")
    got = outs_last["decode"][0].float().cpu().numpy()
    assert np.abs(got - want[new - 1]).max() <= 2e-2 * np.abs(want).max(), "decode, window edge"
