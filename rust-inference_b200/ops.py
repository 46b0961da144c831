"""The kernels of ``csrc/`` as Python functions on torch CUDA tensors.

Each function checks shapes, dtypes and devices, allocates its output with
torch and launches on torch's current stream.  There is no other
implementation behind these names: on a machine without the compiled
libraries (or without nvcc to make them) they raise.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
_P = ctypes.c_void_p
_I = ctypes.c_int
_L = ctypes.c_longlong
_F = ctypes.c_float

_SIGNATURES = {
    ("elementwise", "ri_embed_rows"): [_P, _P, _P, _I, _I, _I, _I, _P, _P],
    ("elementwise", "ri_rmsnorm"): [_P, _P, _P, _P, _P, _I, _I, _F, _I, _I, _P, _I, _I, _P],
    ("elementwise", "ri_add_rows"): [_P, _P, _L, _I, _P],
    ("elementwise", "ri_silu_mul"): [_P, _P, _I, _I, _I, _I, _P],
    ("rope_kv", "ri_qk_norm_rope_append"): [_P] * 10 + [_F, _P, _I, _I] + [_I] * 9 + [_P, _P],
    ("attention_rows", "ri_attention_rows"): [_P] * 8 + [_I] * 8 + [_F, _I, _I, _P, _P],
    ("linear_f32", "ri_linear_f32"): [_P, _P, _P, _I, _I, _I, _P],
    ("sampling", "ri_sample"): [_P, _L, _I, _I, _P, _P, _L, _P, _P, _P, _P, _P, _P, _P, _L, _I, _I, _P, _I, _P],
    ("sampling", "ri_sample_work_bytes"): [_I, _I],
    ("sampling", "ri_argmax"): [_P, _L, _I, _I, _P, _P, _P, _P],
    ("sampling", "ri_mark_seen"): [_P, _L, _P, _P, _I, _I, _P],
    ("attention_decode", "ri_attention_decode"): [_P] * 9 + [_I] * 8 + [_F, _I, _P, _P],
    ("linear_skinny", "ri_linear_skinny"): [_P, _P, _P, _I, _I, _I, _I, _I, _P, _P],
    ("linear_stream_tc", "ri_linear_stream_tc"): [_P, _P, _P, _I, _I, _I, _I, _I, _P, _P],
    ("attention_prefill_tc", "ri_attention_prefill_tc"): [_P] * 8 + [_I] * 9 + [_F, _I, _P, _P],
    ("attention_prefill", "ri_attention_prefill"): [_P] * 8 + [_I] * 8 + [_F, _I, _P, _P],
}
DECODE_CHUNK = 128          # keys per partial result of the decode attention kernel
MAX_FAST_HEAD_DIM = 256
TCGEN05_HEAD_DIMS = (64, 128)   # head sizes the tcgen05 prefill attention kernel is built for
_NO_TCGEN05 = os.environ.get("RUST_INFERENCE_B200_NO_TCGEN05") == "1"   # for comparisons
# the skinny linear applies the SiLU gate in its epilogue (one kernel less per layer: 2 % faster at batch 1 of
# Qwen3-8B shapes, 0.3 % at batch 8); RUST_INFERENCE_B200_FUSED_SWIGLU=0 takes the separate kernel, for comparisons
_FUSED_SWIGLU = os.environ.get("RUST_INFERENCE_B200_FUSED_SWIGLU", "1") != "0"
_WEIGHT_HINTS = os.environ.get("RUST_INFERENCE_B200_WEIGHT_HINTS", "1") != "0"
# Up to here the bfloat16 linear is this package's mma.sync weight-streaming kernel whatever the matrix; the kernel takes
# up to 16 tokens, and from 13 to 16 it is taken for the matrices whose grid of 16-row blocks sits well on the SMs: all
# blocks there at once, and either at most two per SM (they then have the ring of three stages) or nearly three
# (with two or three blocks of the two-stage ring an SM has enough bytes on their way; a grid that leaves most SMs
# two of them does not).  The others go to the tcgen05 kernel below.  Measured inside the decode step (ms a step;
# everything on the mma.sync kernel / everything on the tcgen05 one / by this rule, with the gate/up product on the
# tcgen05 kernel): Qwen3-8B shapes (grids of 384, 256 and 256 blocks for 148 SMs) 13 tokens 4.73 / 4.59 / 4.34,
# 16 tokens 5.48 / 4.91 / 4.71; Qwen3-14B shapes (448, 320 and 320 blocks: none sits well) 16 tokens 7.87 / 7.20 / 7.20,
# and 7.51 with the matrices of 320 blocks on the mma.sync kernel.
# RUST_INFERENCE_B200_SKINNY_MAX=8..16 moves the first limit, for comparisons.
SKINNY_MAX_TOKENS = min(16, max(1, int(os.environ.get("RUST_INFERENCE_B200_SKINNY_MAX", "12"))))
SKINNY_KERNEL_TOKENS = 16          # what the kernel takes
SKINNY_BLOCKS_PER_SM = 3           # its blocks of 16 rows that share an SM (two with the ring of three stages)
_sm_count = {}


def _takes_skinny(M: int, N: int, K: int, device) -> bool:
    """Whether a bfloat16 linear of M tokens with a matrix [N, K] runs on the mma.sync weight-streaming kernel."""
    if K % 8 or M > SKINNY_KERNEL_TOKENS:
        return False
    if M <= SKINNY_MAX_TOKENS:
        return True
    key = str(device)
    if key not in _sm_count:
        _sm_count[key] = torch.cuda.get_device_properties(device).multi_processor_count
    fill = -(-N // 16) / _sm_count[key]                  # blocks per SM
    return fill <= 2.0 or 2.5 <= fill <= SKINNY_BLOCKS_PER_SM
# For 13 to 128 tokens there is a tcgen05 weight-streaming kernel of this package (linear_stream_tc).  Measured inside
# the decode step at Qwen3-8B shapes against the library product (cuBLAS): the step is 2.8 % faster with it at 24
# tokens and 1.9 % at 32, the same at 40, and 1.5 to 2 % slower from 48 on (at 64 tokens a layer's products are
# half tensor-core-bound, and the library's tiles do better there); the output head (65,536 outputs and more) is
# faster on it at every token count.  So it is taken up to STREAM_TC_SMALL tokens and for wide matrices;
# RUST_INFERENCE_B200_STREAM_TC=1 takes it for all linears of 13 to 128 tokens, =0 for none but the wide ones.
STREAM_TC_MAX_TOKENS = 128
STREAM_TC_SMALL = 32
STREAM_TC_WIDE = int(os.environ.get("RUST_INFERENCE_B200_STREAM_TC_WIDE", "65536"))   # from this many outputs on it is taken anyway
_STREAM_TC = os.environ.get("RUST_INFERENCE_B200_STREAM_TC", "")
# the selection of a token other than the greedy one: from this many logits a row on, several blocks per row
SAMPLE_WIDE_VOCAB = 16384
_SAMPLE_WIDE = os.environ.get("RUST_INFERENCE_B200_SAMPLE_WIDE", "1") != "0"
# ... and those passes as one kernel whose blocks meet at barriers per row (0: a kernel per pass, for comparisons)
SAMPLE_ONE_KERNEL = os.environ.get("RUST_INFERENCE_B200_SAMPLE_ONE_KERNEL", "1") != "0"
_fn_cache = {}


class KernelError(RuntimeError):
    pass


def _fn(lib_name: str, fn_name: str, defines=None):
    key = (lib_name, fn_name, tuple(sorted((defines or {}).items())))
    f = _fn_cache.get(key)
    if f is None:
        lib = _build.library(lib_name, defines)
        f = getattr(lib, fn_name)
        f.argtypes = _SIGNATURES[(lib_name, fn_name)]
        f.restype = _L if fn_name.endswith("_bytes") else _I
        _fn_cache[key] = f = (f, lib)
    return f


_launches = [0]


def launch_count() -> int:
    """Kernels of this package launched so far (graph replays count what they replay)."""
    return _launches[0]


def add_launches(n: int) -> None:
    _launches[0] += n


def _call(lib_name: str, fn_name: str, *args, defines=None):
    f, lib = _fn(lib_name, fn_name, defines)
    rc = f(*args)
    _launches[0] += 1
    if rc != 0:
        raise KernelError(f"{fn_name}: {lib.ri_last_error().decode(errors='replace')} (code {rc})")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"the kernels work in float32 or bfloat16, not {dtype}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, name: str, dtype=None, shape=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise KernelError(f"{name} must have shape {tuple(shape)}, got {tuple(t.shape)}")


_err_flags = {}


def error_flag(device) -> torch.Tensor:
    """One int32 per device that kernels set when they meet an index they must
    not follow (an unmapped page, a token id or position out of range).  The
    engine reads it whenever it synchronises anyway."""
    dev = torch.device(device)
    key = (dev.type, dev.index if dev.index is not None else torch.cuda.current_device())
    f = _err_flags.get(key)
    if f is None:
        f = torch.zeros(1, dtype=torch.int32, device=dev)
        _err_flags[key] = f
    return f


ERROR_TEXT = {1: "token id outside the vocabulary", 2: "cache write to an unmapped page",
              3: "position beyond the rotary table", 4: "attention read from an unmapped page",
              5: "a bounded wait inside a kernel ran out (copy or tensor-core completion never arrived)",
              6: "the tcgen05 attention kernel's shared memory does not start on a multiple of 1024 bytes "
                 "(set RUST_INFERENCE_B200_NO_TCGEN05=1 to use the mma.sync kernel)",
              7: "a sequence is longer than the scratch memory given to the decode attention covers "
                 "(max_chunks x 128 keys): the keys beyond were left out"}


# ---------------------------------------------------------------------------------------
def embed(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """float32 rows ``table[ids]``: [tokens, dim]."""
    _need(ids, "ids", torch.int32)
    _need(table, "table")
    tokens, (vocab, dim) = ids.numel(), table.shape
    out = torch.empty((tokens, dim), dtype=torch.float32, device=table.device)
    _call("elementwise", "ri_embed_rows", ids.data_ptr(), table.data_ptr(), out.data_ptr(), tokens, dim, vocab,
          _code(table.dtype), error_flag(table.device).data_ptr(), _stream())
    return out


def _weight_hint(then: Optional[torch.Tensor], tokens: int) -> Optional[torch.Tensor]:
    """``then`` if the linear over it will be the weight-streaming kernel for ``tokens`` rows."""
    if (_WEIGHT_HINTS and then is not None and tokens <= SKINNY_MAX_TOKENS and then.dtype == torch.bfloat16
            and then.dim() == 2 and then.is_contiguous()):
        return then
    return None


def rmsnorm(resid: torch.Tensor, gain: torch.Tensor, eps: float, out_dtype: torch.dtype,
            delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
            then: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMSNorm of the float32 residual stream ``resid`` [n, dim].

    With ``delta`` (compute dtype, same shape) the sum resid + delta is normed,
    and written back into ``resid`` unless ``rows`` is given.  With ``rows``
    (int32 indices) only those rows are normed, in that order.  ``then`` names the
    weight matrix [N, K] of the linear that reads the result next: for a handful of
    rows in bfloat16 the kernel asks for the start of it to be brought into L2 (a
    hint; it changes no result)."""
    _need(resid, "resid", torch.float32)
    n, dim = resid.shape
    _need(gain, "gain", torch.float32, (dim,))
    if delta is not None:
        _need(delta, "delta", out_dtype, (n, dim))
    if rows is not None:
        _need(rows, "rows", torch.int32)
    n_out = n if rows is None else rows.numel()
    out = torch.empty((n_out, dim), dtype=out_dtype, device=resid.device)
    hint = _weight_hint(then, n_out)
    _call("elementwise", "ri_rmsnorm", resid.data_ptr(), _ptr(delta), _ptr(rows), gain.data_ptr(), out.data_ptr(),
          n_out, dim, float(eps), 1, _code(out_dtype), _ptr(hint), hint.shape[0] if hint is not None else 0,
          hint.shape[1] if hint is not None else 0, _stream())
    return out


def add_rows(resid: torch.Tensor, delta: torch.Tensor) -> None:
    """resid += delta (float32 += compute dtype)."""
    _need(resid, "resid", torch.float32)
    _need(delta, "delta", None, resid.shape)
    _call("elementwise", "ri_add_rows", resid.data_ptr(), delta.data_ptr(), resid.numel(), _code(delta.dtype), _stream())


def silu_mul(gate_up: torch.Tensor, block: Optional[int] = None) -> torch.Tensor:
    """silu(gate) * up for ``gate_up`` [rows, 2*inter], in which gate and up columns alternate
    in blocks of ``block`` channels (default: all gates, then all ups)."""
    _need(gate_up, "gate_up")
    rows, two = gate_up.shape
    if two % 2:
        raise KernelError("silu_mul: the last dimension must be even")
    inter = two // 2
    block = inter if block is None else int(block)
    out = torch.empty((rows, inter), dtype=gate_up.dtype, device=gate_up.device)
    _call("elementwise", "ri_silu_mul", gate_up.data_ptr(), out.data_ptr(), rows, inter, block,
          _code(gate_up.dtype), _stream())
    return out


def linear_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, block: int) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T) for ``w_gate_up`` [2*inter, K] with gate and up rows alternating in
    blocks of ``block``.  A handful of bfloat16 tokens with block 8 run as one kernel (the product's
    epilogue applies the gate); otherwise the product and ``silu_mul`` run one after the other."""
    M, K = x.shape
    N = w_gate_up.shape[0]
    if (x.dtype == torch.bfloat16 and block == 8 and N % 16 == 0 and K % 8 == 0 and _FUSED_SWIGLU
            and _gated_on_stream_tc(M, N, K, x.device)):
        return linear_stream_tc(x, w_gate_up, gated=True)
    if (x.dtype == torch.bfloat16 and _takes_skinny(M, N, K, x.device) and block == 8 and N % 16 == 0
            and _FUSED_SWIGLU):
        _need(x, "x")
        _need(w_gate_up, "w_gate_up", x.dtype)
        y = torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
        _call("linear_skinny", "ri_linear_skinny", x.data_ptr(), w_gate_up.data_ptr(), y.data_ptr(), M, N, K, 0, 1,
              error_flag(x.device).data_ptr(), _stream())
        return y
    if (x.dtype == torch.bfloat16 and block == 8 and N % 16 == 0 and _FUSED_SWIGLU
            and _takes_stream_tc(M, N, K)):
        return linear_stream_tc(x, w_gate_up, gated=True)
    return silu_mul(linear(x, w_gate_up), block)


# The gate/up product of a handful of tokens is the one layer linear that the tcgen05 kernel does better than the
# mma.sync one, where its grid fills the device: a large matrix (many waves of 16-row blocks for the mma.sync kernel,
# whose successor can only come in with the last wave) that the tcgen05 kernel covers in one wave with at least two
# shares of K per tile.  Measured inside the decode step at Qwen3-8B shapes (24,576 x 4,096; ms a step, tcgen05 /
# mma.sync): 12 tokens 4.24 / 4.46, 8 tokens 3.75 / 3.90, 4 tokens 3.35 / 3.43, 3 tokens 3.30 / 3.33; 2 tokens
# 3.16 / 3.13 and 1 token 3.02 / 3.01 the other way round; at 14B and 32B shapes (one share of K: 272 and 400 blocks
# for 148 SMs) 6.01 / 5.93 and 12.52 / 12.44, so those stay where they are.  The other layer linears at 8B shapes lose
# 1 to 3 % on it each.  Against the library product above 32 tokens: 40 tokens 7.47 / 7.58, 64 tokens 10.03 / 10.11.
GATED_STREAM_TC_MIN_TOKENS = 3
GATED_STREAM_TC_MIN_ELEMENTS = 90_000_000
_GATED_STREAM_TC = os.environ.get("RUST_INFERENCE_B200_GATED_STREAM_TC", "1") != "0"
_splits_cache = {}


def _gated_on_stream_tc(M: int, N: int, K: int, device) -> bool:
    if not _GATED_STREAM_TC or M < GATED_STREAM_TC_MIN_TOKENS or M > STREAM_TC_MAX_TOKENS or N * K < GATED_STREAM_TC_MIN_ELEMENTS:
        return False
    key = (N, K, str(device))
    if key not in _splits_cache:
        _, lib = _fn("linear_stream_tc", "ri_linear_stream_tc")
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        _splits_cache[key] = int(lib.ri_linear_stream_tc_splits(int(N), int(K), int(sms)))
    return _splits_cache[key] >= 2


def _takes_stream_tc(M: int, N: int, K: int) -> bool:
    """Whether a bfloat16 linear of M tokens (more than the mma.sync kernel takes) runs on the tcgen05 streaming kernel."""
    return M <= STREAM_TC_MAX_TOKENS and K % 8 == 0 and (
        _STREAM_TC == "1" or N >= STREAM_TC_WIDE or (M <= STREAM_TC_SMALL and _STREAM_TC != "0"))


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """y = x w^T for x [M, K], w [N, K].

    float32: this package's own FMA kernel (no tensor cores, no TF32).
    bfloat16, up to 12 tokens (up to 16 for matrices of one wave of blocks): this package's weight-streaming
    tensor-core kernel (mma.sync).
    bfloat16, from there to 32 tokens (and up to 128 for wide matrices such as the output head): this package's
    tcgen05 weight-streaming kernel.
    bfloat16, more tokens: the library GEMM (cuBLAS through torch), as the
    reference engine uses cuBLAS for its linears (src/cuda/mod.rs:186-232 there).
    ``out_dtype`` float32 keeps the float32 accumulator (used for the logits)."""
    _need(x, "x")
    _need(w, "w", x.dtype)
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"linear: x has {K} columns, w has {K2}")
    if x.dtype == torch.float32:
        y = torch.empty((M, N), dtype=torch.float32, device=x.device)
        _call("linear_f32", "ri_linear_f32", x.data_ptr(), w.data_ptr(), y.data_ptr(), M, N, K, _stream())
        return y
    if x.dtype != torch.bfloat16:
        raise KernelError(f"linear: dtype {x.dtype}")
    if _takes_skinny(M, N, K, x.device):
        # a handful of tokens: the weight-streaming kernel of this package
        y = torch.empty((M, N), dtype=torch.float32 if out_dtype == torch.float32 else torch.bfloat16, device=x.device)
        _call("linear_skinny", "ri_linear_skinny", x.data_ptr(), w.data_ptr(), y.data_ptr(), M, N, K,
              1 if out_dtype == torch.float32 else 0, 0, error_flag(x.device).data_ptr(), _stream())
        return y
    if _takes_stream_tc(M, N, K):
        return linear_stream_tc(x, w, out_dtype)
    if out_dtype == torch.float32:
        return torch.mm(x, w.t(), out_dtype=torch.float32)
    return torch.mm(x, w.t())


def linear_stream_tc(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                     gated: bool = False) -> torch.Tensor:
    """y = x w^T in bfloat16 for up to 128 tokens on tcgen05: weight rows as the M side of the product, tokens as N,
    K split over a thread-block cluster whose partial tiles are added through distributed shared memory.
    ``gated``: w holds gate and up rows alternating in blocks of 8, and y [M, N/2] = silu(gate) * up."""
    _need(x, "x", torch.bfloat16)
    _need(w, "w", torch.bfloat16)
    M, K = x.shape
    if M > STREAM_TC_MAX_TOKENS or K % 8 or w.shape[1] != K:
        raise KernelError(f"linear_stream_tc: x {tuple(x.shape)}, w {tuple(w.shape)}: at most {STREAM_TC_MAX_TOKENS} tokens, K a multiple of 8")
    N = w.shape[0]
    if gated and N % 16:
        raise KernelError(f"linear_stream_tc: {N} gate and up rows are not whole blocks of 8 and 8")
    y = torch.empty((M, N // 2 if gated else N), dtype=torch.float32 if out_dtype == torch.float32 else torch.bfloat16,
                    device=x.device)
    _call("linear_stream_tc", "ri_linear_stream_tc", x.data_ptr(), w.data_ptr(), y.data_ptr(), M, N, K,
          1 if out_dtype == torch.float32 else 0, 1 if gated else 0, error_flag(x.device).data_ptr(), _stream())
    return y


def qk_norm_rope_append(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                        q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor], eps: float,
                        rope_table: Optional[torch.Tensor], rotary_dim: int,
                        k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
                        tok_seq: torch.Tensor, tok_pos: torch.Tensor, seq_slot: torch.Tensor,
                        write_kv: bool = True) -> torch.Tensor:
    """Norm and rotate the q and k heads of ``qkv`` [tokens, (H+2KV)*Dh], append k
    and v to the pools [pages, KV, page_size, Dh]; returns q [tokens, H, Dh]."""
    _need(qkv, "qkv")
    tokens = qkv.shape[0]
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise KernelError(f"qkv has {qkv.shape[1]} columns, expected {(num_heads + 2 * num_kv_heads) * head_dim}")
    if k_pool is None:                 # nothing is appended (write_kv False): any valid pointers will do
        if write_kv:
            raise KernelError("qk_norm_rope_append: appending needs the cache pools")
        pages, page_size = 1, 1
        k_pool = v_pool = qkv
        page_table = tok_seq.view(1, -1) if page_table is None else page_table
    else:
        pages, kvh, page_size, dh = k_pool.shape
        if (kvh, dh) != (num_kv_heads, head_dim) or v_pool.shape != k_pool.shape:
            raise KernelError(f"cache pools {tuple(k_pool.shape)} / {tuple(v_pool.shape)} do not fit {num_kv_heads} kv heads of {head_dim}")
        _need(k_pool, "k_pool", qkv.dtype)
        _need(v_pool, "v_pool", qkv.dtype)
    _need(page_table, "page_table", torch.int32)
    for t, n in ((tok_seq, "tok_seq"), (tok_pos, "tok_pos"), (seq_slot, "seq_slot")):
        _need(t, n, torch.int32)
    for g, n in ((q_gain, "q_gain"), (k_gain, "k_gain")):
        if g is not None:
            _need(g, n, torch.float32, (head_dim,))
    rope_rows = 0
    if rope_table is not None:
        _need(rope_table, "rope_table", torch.float32)
        if rope_table.dim() != 3 or rope_table.shape[1] != rotary_dim // 2 or rope_table.shape[2] != 2:
            raise KernelError(f"rope table must be [positions, {rotary_dim // 2}, 2], got {tuple(rope_table.shape)}")
        rope_rows = rope_table.shape[0]
    q = torch.empty((tokens, num_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
    _call("rope_kv", "ri_qk_norm_rope_append", qkv.data_ptr(), q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
          page_table.data_ptr(), tok_seq.data_ptr(), tok_pos.data_ptr(), seq_slot.data_ptr(), _ptr(q_gain),
          _ptr(k_gain), float(eps), _ptr(rope_table), rope_rows, rotary_dim, tokens, num_heads, num_kv_heads,
          head_dim, page_table.shape[1], page_size, pages, 1 if write_kv else 0, _code(qkv.dtype),
          error_flag(qkv.device).data_ptr(), _stream())
    return q


def attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
              seq_slot: torch.Tensor, seq_start: torch.Tensor, seq_len: torch.Tensor, max_new: int, scale: float,
              window: int = 0) -> torch.Tensor:
    """Causal attention of the step's new tokens (q [tokens, H, Dh], sequences back to back as
    ``seq_start`` says) over the paged cache, which already holds their keys and values: float32 or
    bfloat16, any head size up to 512, any page size.  Every (token, head) is computed in one fixed
    order that depends on its own position only, so the result does not depend on the step's cutting."""
    _need(q, "q")
    tokens, H, Dh = q.shape
    pages, KV, page_size, dh = k_pool.shape
    if dh != Dh or v_pool.shape != k_pool.shape:
        raise KernelError(f"attention: pools {tuple(k_pool.shape)} do not fit head_dim {Dh}")
    _need(k_pool, "k_pool", q.dtype)
    _need(v_pool, "v_pool", q.dtype)
    _need(page_table, "page_table", torch.int32)
    seqs = seq_slot.numel()
    _need(seq_slot, "seq_slot", torch.int32, (seqs,))
    _need(seq_start, "seq_start", torch.int32, (seqs + 1,))
    _need(seq_len, "seq_len", torch.int32, (seqs,))
    out = torch.empty_like(q)
    _call("attention_rows", "ri_attention_rows", q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(),
          page_table.data_ptr(), seq_slot.data_ptr(), seq_start.data_ptr(), seq_len.data_ptr(), seqs, int(max_new),
          H, KV, Dh, page_table.shape[1], page_size, pages, float(scale), int(window), _code(q.dtype),
          error_flag(q.device).data_ptr(), _stream())
    return out


def fast_attention_supported(dtype: torch.dtype, head_dim: int, page_size: int) -> bool:
    """Whether the tensor-core attention kernels take this case (else the float32-order kernel of ``attention`` does)."""
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= MAX_FAST_HEAD_DIM and page_size == 32


def _decode_parts(head_dim: int, chunks: int) -> int:
    """Partial results per (sequence, head) that the decode attention's scratch memory must have room for."""
    _, lib = _fn("attention_decode", "ri_attention_decode", {"RI_HEAD_DIM": head_dim})
    return int(lib.ri_attention_decode_parts(int(chunks)))


def attention_decode(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
                     seq_slot: torch.Tensor, seq_len: torch.Tensor, scale: float, window: int,
                     max_len: int) -> torch.Tensor:
    """Attention of one new token per sequence (q [seqs, H, Dh], bfloat16) over the
    paged cache, keys split into chunks of ``DECODE_CHUNK``; ``max_len`` bounds the
    sequences' lengths after this step and sizes the scratch memory."""
    _need(q, "q", torch.bfloat16)
    seqs, H, Dh = q.shape
    pages, KV, page_size, dh = k_pool.shape
    if dh != Dh or v_pool.shape != k_pool.shape:
        raise KernelError(f"attention_decode: pools {tuple(k_pool.shape)} do not fit head_dim {Dh}")
    if not fast_attention_supported(q.dtype, Dh, page_size):
        raise KernelError(f"attention_decode: head_dim {Dh} with pages of {page_size} is not supported")
    _need(k_pool, "k_pool", torch.bfloat16)
    _need(v_pool, "v_pool", torch.bfloat16)
    _need(page_table, "page_table", torch.int32)
    _need(seq_slot, "seq_slot", torch.int32, (seqs,))
    _need(seq_len, "seq_len", torch.int32, (seqs,))
    chunks = max(1, -(-int(max_len) // DECODE_CHUNK))
    parts = _decode_parts(Dh, chunks)
    o_part = torch.empty((seqs, H, parts, Dh), dtype=torch.float32, device=q.device)
    ml_part = torch.empty((seqs, H, parts, 2), dtype=torch.float32, device=q.device)
    out = torch.empty_like(q)
    _call("attention_decode", "ri_attention_decode", q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
          out.data_ptr(), o_part.data_ptr(), ml_part.data_ptr(), page_table.data_ptr(), seq_slot.data_ptr(),
          seq_len.data_ptr(), seqs, H, KV, Dh, page_table.shape[1], page_size, pages, chunks, float(scale),
          int(window), error_flag(q.device).data_ptr(), _stream(), defines={"RI_HEAD_DIM": Dh})
    return out


def attention_prefill(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
                      seq_slot: torch.Tensor, seq_start: torch.Tensor, seq_len: torch.Tensor, max_new: int,
                      scale: float, window: int) -> torch.Tensor:
    """Attention of the step's new tokens (q [tokens, H, Dh], bfloat16, sequences back
    to back as ``seq_start`` says) over the paged cache, which already holds their keys
    and values; ``max_new`` is the most tokens one sequence brings."""
    _need(q, "q", torch.bfloat16)
    tokens, H, Dh = q.shape
    pages, KV, page_size, dh = k_pool.shape
    if dh != Dh or v_pool.shape != k_pool.shape:
        raise KernelError(f"attention_prefill: pools {tuple(k_pool.shape)} do not fit head_dim {Dh}")
    if not fast_attention_supported(q.dtype, Dh, page_size):
        raise KernelError(f"attention_prefill: head_dim {Dh} with pages of {page_size} is not supported")
    _need(k_pool, "k_pool", torch.bfloat16)
    _need(v_pool, "v_pool", torch.bfloat16)
    _need(page_table, "page_table", torch.int32)
    seqs = seq_slot.numel()
    _need(seq_slot, "seq_slot", torch.int32, (seqs,))
    _need(seq_start, "seq_start", torch.int32, (seqs + 1,))
    _need(seq_len, "seq_len", torch.int32, (seqs,))
    out = torch.empty_like(q)
    if Dh in TCGEN05_HEAD_DIMS and not _NO_TCGEN05:
        # head sizes of 64 and 128: the tcgen05 / tensor-memory kernel
        _call("attention_prefill_tc", "ri_attention_prefill_tc", q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
              out.data_ptr(), page_table.data_ptr(), seq_slot.data_ptr(), seq_start.data_ptr(), seq_len.data_ptr(),
              q.shape[0], seqs, int(max_new), H, KV, Dh, page_table.shape[1], page_size, pages, float(scale), int(window),
              error_flag(q.device).data_ptr(), _stream(), defines={"RI_HEAD_DIM": Dh})
        return out
    _call("attention_prefill", "ri_attention_prefill", q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
          out.data_ptr(), page_table.data_ptr(), seq_slot.data_ptr(), seq_start.data_ptr(), seq_len.data_ptr(),
          seqs, int(max_new), H, KV, Dh, page_table.shape[1], page_size, pages, float(scale), int(window),
          error_flag(q.device).data_ptr(), _stream(), defines={"RI_HEAD_DIM": Dh})
    return out


def argmax(logits: torch.Tensor) -> torch.Tensor:
    """First index of each row's maximum: int32 [rows]."""
    _need(logits, "logits", torch.float32)
    rows, vocab = logits.shape
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    slices = min(128, max(1, -(-vocab // 2048)))           # ri_argmax_slices of the library
    part_val = part_idx = None
    if slices > 1:
        part_val = torch.empty((rows, slices), dtype=torch.float32, device=logits.device)
        part_idx = torch.empty((rows, slices), dtype=torch.int32, device=logits.device)
    _call("sampling", "ri_argmax", logits.data_ptr(), logits.stride(0), rows, vocab, out.data_ptr(), _ptr(part_val),
          _ptr(part_idx), _stream())
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor,
           top_k: Optional[torch.Tensor] = None, top_p: Optional[torch.Tensor] = None,
           penalty: Optional[torch.Tensor] = None, seen: Optional[torch.Tensor] = None,
           seen_rows: Optional[torch.Tensor] = None, uses_top_k: bool = True, uses_top_p: bool = True) -> torch.Tensor:
    """One token per row of float32 ``logits`` [rows, vocab]; the options are
    per-row device tensors (temperature float32, top_k int32, top_p float32,
    penalty float32), ``uniform`` the per-row number in [0, 1).

    From ``SAMPLE_WIDE_VOCAB`` logits a row on, several blocks work on each row (the same
    token, bit for bit); a caller that knows that no row has a top-k or a top-p says so
    with ``uses_top_k`` / ``uses_top_p`` and saves those searches."""
    _need(logits, "logits", torch.float32)
    rows, vocab = logits.shape
    _need(temperature, "temperature", torch.float32, (rows,))
    _need(uniform, "uniform", torch.float32, (rows,))
    if top_k is not None:
        _need(top_k, "top_k", torch.int32, (rows,))
    if top_p is not None:
        _need(top_p, "top_p", torch.float32, (rows,))
    if penalty is not None:
        _need(penalty, "penalty", torch.float32, (rows,))
    seen_stride = 0
    if seen is not None:
        _need(seen, "seen", torch.uint8)
        if seen.shape[1] != vocab:
            raise KernelError("seen must be [rows, vocab]")
        seen_stride = seen.stride(0)
        if seen_rows is not None:
            _need(seen_rows, "seen_rows", torch.int32, (rows,))
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    work, work_bytes = None, 0
    if _SAMPLE_WIDE and vocab >= SAMPLE_WIDE_VOCAB:
        f, _ = _fn("sampling", "ri_sample_work_bytes")
        work_bytes = int(f(rows, vocab))
        work = torch.empty(work_bytes, dtype=torch.uint8, device=logits.device)
    k_on, p_on = bool(uses_top_k and top_k is not None), bool(uses_top_p and top_p is not None)
    _call("sampling", "ri_sample", logits.data_ptr(), logits.stride(0), rows, vocab, _ptr(seen), _ptr(seen_rows),
          seen_stride, temperature.data_ptr(), _ptr(top_k), _ptr(top_p), _ptr(penalty), uniform.data_ptr(),
          out.data_ptr(), _ptr(work), work_bytes, int(k_on), int(p_on), error_flag(logits.device).data_ptr(),
          int(SAMPLE_ONE_KERNEL), _stream())
    if work is not None and not SAMPLE_ONE_KERNEL:
        add_launches(2 + 12 * (1 + k_on + p_on) + p_on)          # one was counted by the call
    return out


def mark_seen(seen: torch.Tensor, rows: torch.Tensor, tokens: torch.Tensor) -> None:
    """seen[rows[i], tokens[i]] = 1."""
    _need(seen, "seen", torch.uint8)
    _need(rows, "rows", torch.int32)
    _need(tokens, "tokens", torch.int32, rows.shape)
    _call("sampling", "ri_mark_seen", seen.data_ptr(), seen.stride(0), rows.data_ptr(), tokens.data_ptr(),
          rows.numel(), seen.shape[1], _stream())
