"""The allocation-free decode attention entry point, called the way its users call it:
through the exported C symbol of the shared library, with nothing but inputs and outputs.

Some hosts of this code cannot allocate device memory around a call (a fixed memory
budget handed out at start-up, a loop that must not block in the driver's allocator,
a program without torch).  For them `ri_attention_decode_noalloc` keeps its scratch
memory in a fixed array inside the library.  This test checks that it gives what the
ordinary entry point gives (within the tolerance of the attention tests: the ordinary one
takes another kernel for these sizes) and what the plain attention gives, on calls in a row
that share that array; that it refuses, before anything is launched, a call that would not
fit, a null pointer and a misaligned pointer; and that a sequence longer than `max_chunks`
covers is reported through the error word instead of being followed past the array.  It sits in a file of its own that is collected
last, and passes alone in a fresh process as well as after the other tests.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, seqs, H, KV, Dh, max_len):
    g = torch.Generator(device="cuda").manual_seed(seed)
    P = 32
    lens = torch.randint(1, max_len + 1, (seqs,), generator=g, device="cuda", dtype=torch.int32)
    lens[0] = max_len
    pages_per = (max_len + P - 1) // P
    num_pages = seqs * pages_per + 5
    perm = torch.randperm(num_pages, generator=g, device="cuda").to(torch.int32)
    table = perm[:seqs * pages_per].view(seqs, pages_per).contiguous()
    slot = torch.randperm(seqs, generator=g, device="cuda").to(torch.int32)
    q = torch.randn((seqs, H, Dh), generator=g, device="cuda").to(torch.bfloat16)
    k = (torch.randn((num_pages, KV, P, Dh), generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    v = torch.randn((num_pages, KV, P, Dh), generator=g, device="cuda").to(torch.bfloat16)
    return q, k, v, table, slot, lens


def _plain_decode(q, k, v, table, slot, lens, scale, window):
    """The newest token's attention over each sequence's pages, by the plain model's function."""
    import helpers  # noqa: F401  (puts tests/ on the path)
    import plain_qwen3 as plain
    qn, kn, vn = q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy()
    tn, sn, ln = table.cpu().numpy(), slot.cpu().numpy(), lens.cpu().numpy()
    Dh = qn.shape[-1]
    out = np.zeros(qn.shape)
    for b in range(qn.shape[0]):
        n = int(ln[b])
        pages = tn[sn[b], :-(-n // 32)]
        keys = kn[pages].transpose(0, 2, 1, 3).reshape(-1, kn.shape[1], Dh)[:n]
        vals = vn[pages].transpose(0, 2, 1, 3).reshape(-1, vn.shape[1], Dh)[:n]
        # the newest query alone: a row of zeros for the earlier positions, whose results are not looked at
        qs = np.zeros((n,) + qn.shape[1:])
        qs[-1] = qn[b] * scale * np.sqrt(Dh)              # causal_attention scales by 1/sqrt(Dh) itself
        out[b] = plain.causal_attention(qs, keys, vals, window=window)[-1]
    return out


def test_no_alloc_entry_point_matches_the_ordinary_one():
    from rust_inference_b200 import ops
    from rust_inference_b200.csrc import build
    H, KV, Dh = 8, 2, 64
    lib = ctypes.CDLL(build.compile_library("attention_decode_noalloc", {"RI_HEAD_DIM": Dh}))
    fn = lib.ri_attention_decode_noalloc
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [P] * 7 + [I] * 8 + [F, I, P, P]
    fn.restype = I
    lib.ri_last_error.restype = ctypes.c_char_p
    lib.ri_attention_decode_noalloc_bytes.restype = ctypes.c_longlong
    lib.ri_attention_decode_noalloc_bytes.argtypes = [I] * 4
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    scale = 1.0 / math.sqrt(Dh)
    # two calls in a row with different sizes and lengths: the second finds the first one's leftovers
    for seed, seqs, max_len, window in ((1, 5, 700, 0), (2, 3, 300, 0), (3, 4, 1000, 150)):
        q, k, v, table, slot, lens = _case(seed, seqs, H, KV, Dh, max_len)
        want = ops.attention_decode(q, k, v, table, slot, lens, scale, window, max_len)
        out = torch.full_like(q, float("nan"))
        chunks = -(-max_len // 128)
        before = torch.cuda.memory_allocated()
        rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), table.data_ptr(), slot.data_ptr(),
                lens.data_ptr(), seqs, H, KV, Dh, table.shape[1], 32, k.shape[0], chunks, scale, window,
                err.data_ptr(), torch.cuda.current_stream().cuda_stream)
        assert rc == 0, lib.ri_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert int(err.item()) == 0
        got, ref = out.float(), want.float()
        assert torch.isfinite(got).all()
        # the tolerance of the attention tests (2 % of the largest value): against the ordinary entry point
        # (which takes its streaming kernel for these sizes) and against the plain attention
        assert float((got - ref).abs().max()) <= 2e-2 * float(ref.abs().max())
        plain_out = torch.from_numpy(_plain_decode(q, k, v, table, slot, lens, scale, window)).float().cuda()
        assert float((got - plain_out).abs().max()) <= 2e-2 * float(plain_out.abs().max())
    # a call that does not fit the fixed array is refused, with the numbers in the message
    big_seqs, big_chunks = 64, 64
    assert lib.ri_attention_decode_noalloc_bytes(big_seqs, H, Dh, big_chunks) > (8 << 20)
    rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), table.data_ptr(), slot.data_ptr(),
            lens.data_ptr(), big_seqs, H, KV, Dh, table.shape[1], 32, k.shape[0], big_chunks, scale, 0,
            err.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc != 0 and b"fixed array" in lib.ri_last_error()
    # refused on the host, before any launch: a null pointer, a misaligned q, a page table without columns
    args = [q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), table.data_ptr(), slot.data_ptr(),
            lens.data_ptr(), seqs, H, KV, Dh, table.shape[1], 32, k.shape[0], chunks, scale, 0, err.data_ptr(),
            torch.cuda.current_stream().cuda_stream]
    for at, value, word in ((0, None, b"null"), (2, None, b"null"), (0, q.data_ptr() + 2, b"aligned"),
                            (1, k.data_ptr() + 8, b"aligned"), (11, 0, b"page table")):
        bad = list(args)
        bad[at] = value
        rc = fn(*bad)
        assert rc != 0 and word in lib.ri_last_error(), lib.ri_last_error()
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    # a sequence longer than max_chunks * 128: not followed past the array, reported as error 7
    rc = fn(*(args[:14] + [1] + args[15:]))
    assert rc == 0, lib.ri_last_error().decode()
    torch.cuda.synchronize()
    assert int(err.item()) == 7 and bool(torch.isfinite(out.float()).all())
