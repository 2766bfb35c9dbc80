"""Python entry to the CUDA kernels: argument checks, then a ctypes call on the current stream.

Every function works on CUDA tensors only and raises if given anything else;
there is no host implementation behind them.  ``GemmOut`` is how a matrix
product hands its result to the next kernel: either the finished matrix or
split-K partial sums that the consumer adds up in float.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass

import torch

from . import _build

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

_c_int, _c_ll, _c_float, _c_ptr = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p

_SIGNATURES = {
    "elementwise": {
        "qt_embedding": [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_ptr],
        "qt_add_bias": [_c_ptr, _c_ptr, _c_int, _c_int, _c_ptr],
        "qt_add_rmsnorm": [_c_ptr, _c_ptr, _c_int, _c_int, _c_ll, _c_ptr, _c_float, _c_ptr, _c_int, _c_ptr, _c_int,
                           _c_int, _c_ptr],
        "qt_qk_norm_rope_write": [_c_ptr, _c_int, _c_int, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr,
                                  _c_int, _c_ptr, _c_ptr, _c_float, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int,
                                  _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr],
        "qt_swiglu": [_c_ptr, _c_int, _c_int, _c_ll, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr],
    },
    "attention": {
        "qt_attention_prefill": [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int,
                                 _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_ptr],
        "qt_attention_decode": [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_int,
                                _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_ptr, _c_ptr, _c_ptr],
    },
    "attention_mma": {
        "qt_attention_decode_mma": [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int,
                                    _c_int, _c_int, _c_int, _c_float, _c_int, _c_ptr, _c_ptr, _c_ptr],
        "qt_attention_decode_ws": [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int,
                                   _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr],
        "qt_attention_prefill_mma": [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int,
                                     _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_ptr],
    },
    "attention_tc": {
        "qt_attention_prefill_tc": [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int,
                                    _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_ptr, _c_ptr],
    },
    "gemm_simt": {
        "qt_gemm_simt": [_c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_ptr],
    },
    "gemm_tc": {
        "qt_gemm_tc": [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ll, _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
        "qt_gemm_tc_pair": [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ll, _c_int, _c_ptr,
                            _c_ptr, _c_int, _c_ptr, _c_ptr],
        "qt_gemm_tc_pair_slots": [],
    },
    "gemm_fused": {
        "qt_gemm_fused": [_c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                          _c_ptr, _c_int, _c_int, _c_float,
                          _c_ptr, _c_int, _c_int,
                          _c_ptr, _c_ptr, _c_ptr, _c_ptr,
                          _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_float,
                          _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
    },
    "sampling": {
        "qt_argmax": [_c_ptr, _c_ptr, _c_int, _c_int, _c_ptr],
        "qt_sample": [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr],
        "qt_sample_keyed": [_c_ptr, _c_float, _c_ll, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_float, _c_ptr],
        "qt_feed_tokens": [_c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_ptr],
    },
}
_BOUND: dict[str, ctypes._CFuncPtr] = {}


class KernelError(RuntimeError):
    pass


def _fn(library: str, name: str):
    fn = _BOUND.get(name)
    if fn is None:
        lib = _build.load_library(library)
        fn = getattr(lib, name)
        fn.argtypes = _SIGNATURES[library][name]
        fn.restype = _c_int
        _BOUND[name] = fn
    return fn


_LAUNCHES = 0


def launch_count() -> int:
    """Kernel launches made through this module since the process started."""
    return _LAUNCHES


def count_launches(n: int) -> None:
    """Account for kernels launched outside this module's calls (a replayed CUDA graph of them)."""
    global _LAUNCHES
    _LAUNCHES += n


def _call(library: str, name: str, *args, launches: int = 1) -> None:
    global _LAUNCHES
    _LAUNCHES += launches
    code = _fn(library, name)(*args)
    if code != 0:
        raise KernelError(f"{name} failed ({code}): {_build.last_error(library)}")


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_RAW_DEVICE = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """The current stream's handle.  Asked for at every launch, so by torch's two direct calls where it has them:
    building a Stream object costs as much host time as the rest of a launch."""
    if _RAW_STREAM is not None and _RAW_DEVICE is not None:
        return _RAW_STREAM(_RAW_DEVICE())
    return torch.cuda.current_stream().cuda_stream


def _ptr(tensor: torch.Tensor | None) -> int | None:
    return None if tensor is None else tensor.data_ptr()


def _need(tensor: torch.Tensor, name: str, dtype=None, shape=None) -> None:
    if not isinstance(tensor, torch.Tensor) or not tensor.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no host path)")
    if dtype is not None and tensor.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {tensor.dtype}")
    if not tensor.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if shape is not None and tuple(tensor.shape) != tuple(shape):
        raise KernelError(f"{name} must have shape {tuple(shape)}, got {tuple(tensor.shape)}")


def _code(tensor: torch.Tensor, name: str) -> int:
    if tensor.dtype not in _CODES:
        raise KernelError(f"{name}: element type {tensor.dtype} is neither float32 nor bfloat16")
    return _CODES[tensor.dtype]


@dataclass
class GemmOut:
    """Result of a matrix product: ``tensor`` is [splits, M, N]; the value is the sum over splits.

    Rows and columns are dense (stride N, 1); the stride between splits may be larger than M * N
    when the tensor is a view of a larger buffer.
    """

    tensor: torch.Tensor

    def __post_init__(self) -> None:
        t = self.tensor
        if t.dim() != 3 or t.stride(2) != 1 or t.stride(1) != t.shape[2]:
            raise KernelError(f"GemmOut needs a [splits, M, N] tensor with dense rows, got {tuple(t.shape)} / {t.stride()}")

    @property
    def n_splits(self) -> int:
        return self.tensor.shape[0]

    @property
    def split_stride(self) -> int:
        return self.tensor.stride(0) if self.tensor.shape[0] > 1 else 0

    @property
    def rows(self) -> int:
        return self.tensor.shape[1]

    @property
    def cols(self) -> int:
        return self.tensor.shape[2]

    def value(self) -> torch.Tensor:
        """The finished matrix in float (for tests and host-side use)."""
        return self.tensor.float().sum(dim=0)


# ----------------------------------------------------------------------------- elementwise
def embedding(residual: torch.Tensor, table: torch.Tensor, ids: torch.Tensor) -> None:
    """residual[t] = table[ids[t]] in float.  ids: int32 [T]."""
    tokens, hidden = residual.shape
    _need(residual, "residual", torch.float32)
    _need(table, "table")
    _need(ids, "ids", torch.int32, (tokens,))
    if table.shape[1] != hidden:
        raise KernelError(f"embedding: table width {table.shape[1]} != stream width {hidden}")
    _call("elementwise", "qt_embedding", _ptr(residual), _ptr(table), _ptr(ids), tokens, hidden, table.shape[0],
          _code(table, "table"), _stream())


def add_bias(out: torch.Tensor, bias: torch.Tensor) -> None:
    """out [T, N] float32 += bias [N] float32, in place: the bias of a projection on its float sums."""
    _need(out, "out", torch.float32)
    _need(bias, "bias", torch.float32, (out.shape[-1],))
    if out.dim() != 2:
        raise KernelError(f"add_bias: out must be [rows, cols], got {tuple(out.shape)}")
    _call("elementwise", "qt_add_bias", _ptr(out), _ptr(bias), out.shape[0], out.shape[1], _stream())


def add_rmsnorm(residual: torch.Tensor, delta: GemmOut | None, weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: torch.Tensor | None = None) -> None:
    """stream += delta; out = rmsnorm(stream) * weight.

    Without ``rows`` every row of ``residual`` [T, H] is updated in place and normed into ``out`` [T, H].
    With ``rows`` (int32 [K]) only those rows are normed into ``out`` [K, H] and the stream is left as it is.
    """
    hidden = residual.shape[1]
    _need(residual, "residual", torch.float32)
    _need(weight, "weight", torch.float32, (hidden,))
    n_rows = residual.shape[0] if rows is None else rows.shape[0]
    _need(out, "out", shape=(n_rows, hidden))
    if rows is not None:
        _need(rows, "rows", torch.int32)
    if delta is not None:
        if not delta.tensor.is_cuda or (delta.rows, delta.cols) != tuple(residual.shape):
            raise KernelError(f"add_rmsnorm: delta {tuple(delta.tensor.shape)} does not match the stream {tuple(residual.shape)}")
    _call("elementwise", "qt_add_rmsnorm", _ptr(residual), _ptr(delta.tensor) if delta else None,
          _code(delta.tensor, "delta") if delta else F32, delta.n_splits if delta else 1,
          delta.split_stride if delta else 0, _ptr(weight), float(eps), _ptr(out), _code(out, "out"), _ptr(rows),
          n_rows, hidden, _stream())


def qk_norm_rope_write(qkv: GemmOut, q_out: torch.Tensor, k_cache: torch.Tensor | None, v_cache: torch.Tensor | None,
                       token_seq: torch.Tensor, token_pos: torch.Tensor, block_table: torch.Tensor | None,
                       q_weight: torch.Tensor | None, k_weight: torch.Tensor | None, eps: float,
                       cos_sin: torch.Tensor | None, num_heads: int, num_kv_heads: int, head_dim: int,
                       page_tokens: int, ring_tokens: int, write_kv: bool = True, kv_in_proj: bool = True,
                       interleaved: bool = False) -> None:
    """Per-head q/k RMSNorm, rotation and the cache write, from the fused projection output.

    qkv [*, T, (nq + 2 nkv) d]; q_out [T, nq, d]; caches [pages, nkv, page_tokens, d]; cos_sin float [P, rd]
    (cos | sin of the rd/2 pair angles); pairs are (i, i + rd/2), or (2i, 2i + 1) with ``interleaved``.
    """
    tokens = qkv.rows
    width = (num_heads + (2 * num_kv_heads if kv_in_proj else 0)) * head_dim
    if qkv.cols != width:
        raise KernelError(f"qk_norm_rope_write: projection width {qkv.cols} != (nq + 2 nkv) d = {width}")
    _need(q_out, "q_out", shape=(tokens, num_heads, head_dim))
    _need(token_seq, "token_seq", torch.int32, (tokens,))
    _need(token_pos, "token_pos", torch.int32, (tokens,))
    for name, w in (("q_weight", q_weight), ("k_weight", k_weight)):
        if w is not None:
            _need(w, name, torch.float32, (head_dim,))
    rotary_dim, max_pos = 0, 0
    if cos_sin is not None:
        _need(cos_sin, "cos_sin", torch.float32)
        max_pos, rotary_dim = cos_sin.shape
    max_blocks = 0
    if write_kv:
        _need(block_table, "block_table", torch.int32)
        max_blocks = block_table.shape[1]
        for name, cache in (("k_cache", k_cache), ("v_cache", v_cache)):
            _need(cache, name, q_out.dtype)
            if tuple(cache.shape[1:]) != (num_kv_heads, page_tokens, head_dim):
                raise KernelError(f"{name}: shape {tuple(cache.shape)} is not [pages, {num_kv_heads}, {page_tokens}, {head_dim}]")
    _call("elementwise", "qt_qk_norm_rope_write", _ptr(qkv.tensor), _code(qkv.tensor, "qkv"), qkv.n_splits,
          qkv.split_stride, _ptr(q_out), _ptr(k_cache), _ptr(v_cache), _code(q_out, "q_out"), _ptr(token_seq),
          _ptr(token_pos), _ptr(block_table), max_blocks, _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(cos_sin),
          rotary_dim, max_pos, tokens, num_heads, num_kv_heads, head_dim, page_tokens, ring_tokens,
          1 if write_kv else 0, 1 if kv_in_proj else 0, 1 if interleaved else 0, _stream())


SWIGLU_GROUP = 16      # rows of gate and of up that alternate in a weight laid out for the GEMM's gated epilogue
# gate activations of a gated feed-forward, act(gate) * up: names a configuration may use -> the kernels' codes
ACTIVATIONS = {"silu": 0, "swish": 0, "gelu_pytorch_tanh": 1, "gelu_tanh": 1, "gelu": 2, "relu": 3}


def activation_code(name: str) -> int:
    try:
        return ACTIVATIONS[name]
    except KeyError:
        raise KernelError(f"unknown gate activation {name!r}; the kernels compute {sorted(ACTIVATIONS)}") from None



def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, group: int) -> torch.Tensor:
    """[gate; up] with the rows alternating ``group`` of gate and ``group`` of up (``group`` 0: gate, then up)."""
    if group == 0:
        return torch.cat((gate, up), dim=0)
    inter, hidden = gate.shape
    if inter % group:
        raise KernelError(f"rows in groups of {group} do not divide {inter}")
    return torch.stack((gate.view(inter // group, group, hidden), up.view(inter // group, group, hidden)), dim=1).reshape(2 * inter, hidden)


def swiglu(gate_up: GemmOut, out: torch.Tensor, group: int = 0, activation: str = "silu") -> None:
    """out[t, i] = act(gate[t, i]) * up[t, i] where gate_up[t] holds gate then up (``group`` 0) or alternates
    ``group`` elements of gate and ``group`` of up; ``activation`` is one of ``ACTIVATIONS``."""
    tokens, inter = out.shape
    _need(out, "out")
    if (gate_up.rows, gate_up.cols) != (tokens, 2 * inter):
        raise KernelError(f"swiglu: input {tuple(gate_up.tensor.shape)} does not match output {tuple(out.shape)}")
    _call("elementwise", "qt_swiglu", _ptr(gate_up.tensor), _code(gate_up.tensor, "gate_up"), gate_up.n_splits,
          gate_up.split_stride, _ptr(out), _code(out, "out"), tokens, inter, int(group), activation_code(activation), _stream())


# ----------------------------------------------------------------------------- attention
def _check_attention(q, k_cache, v_cache, out, block_table, num_kv_heads, page_tokens):
    _need(q, "q")
    tokens, num_heads, head_dim = q.shape
    _need(out, "out", q.dtype, q.shape)
    _need(k_cache, "k_cache", q.dtype)
    _need(v_cache, "v_cache", q.dtype, k_cache.shape)
    if tuple(k_cache.shape[1:]) != (num_kv_heads, page_tokens, head_dim):
        raise KernelError(f"cache shape {tuple(k_cache.shape)} is not [pages, {num_kv_heads}, {page_tokens}, {head_dim}]")
    _need(block_table, "block_table", torch.int32)
    return tokens, num_heads, head_dim


def attention_mma_supported(q: torch.Tensor, page_tokens: int) -> bool:
    """The tensor-core attention kernels take bfloat16, head sizes in steps of 16 up to 128, pages of 64 tokens."""
    return q.dtype == torch.bfloat16 and q.shape[2] % 16 == 0 and q.shape[2] <= 128 and page_tokens == 64


def attention_tc_supported(q: torch.Tensor, page_tokens: int) -> bool:
    """The tcgen05 prefill attention takes bfloat16, head size 64 or 128, pages of 64 tokens."""
    return q.dtype == torch.bfloat16 and q.shape[2] in (64, 128) and page_tokens == 64


def _pick_attention(q: torch.Tensor, page_tokens: int, impl: str | None, prefill: bool = False) -> str:
    if impl is None:
        if prefill and attention_tc_supported(q, page_tokens):
            return "tc"
        return "mma" if attention_mma_supported(q, page_tokens) else "generic"
    if impl == "tc" and not (prefill and attention_tc_supported(q, page_tokens)):
        raise KernelError(f"the tcgen05 attention kernel does not take {q.dtype}, head_dim={q.shape[2]}, pages of {page_tokens}")
    if impl == "mma" and not attention_mma_supported(q, page_tokens):
        raise KernelError(f"the tensor-core attention kernels do not take {q.dtype}, head_dim={q.shape[2]}, pages of {page_tokens}")
    if impl not in ("tc", "mma", "generic"):
        raise KernelError(f"unknown attention implementation {impl!r}")
    return impl


def attention_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                      block_table: torch.Tensor, seq_start: torch.Tensor, seq_past: torch.Tensor, max_q_len: int,
                      num_kv_heads: int, page_tokens: int, ring_tokens: int, window: int | None, scale: float,
                      impl: str | None = None) -> None:
    """Causal attention of packed sequences over the cache (which already holds this step's keys).
    ``impl`` forces a kernel ("tc": tcgen05, "mma": mma.sync, "generic"); by default the shape decides."""
    _, num_heads, head_dim = _check_attention(q, k_cache, v_cache, out, block_table, num_kv_heads, page_tokens)
    n_seqs = seq_past.shape[0]
    _need(seq_start, "seq_start", torch.int32, (n_seqs + 1,))
    _need(seq_past, "seq_past", torch.int32)
    if block_table.shape[0] < n_seqs:
        raise KernelError("attention_prefill: block table has fewer rows than sequences")
    choice = _pick_attention(q, page_tokens, impl, prefill=True)
    if choice == "tc":
        _call("attention_tc", "qt_attention_prefill_tc", _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), q.shape[0],
              k_cache.shape[0], _ptr(block_table), block_table.shape[1], _ptr(seq_start), _ptr(seq_past), n_seqs,
              int(max_q_len), num_heads, num_kv_heads, head_dim, page_tokens, ring_tokens, int(window or 0), float(scale),
              _ptr(_status_word(q.device)), _stream())
        return
    if choice == "mma":
        _call("attention_mma", "qt_attention_prefill_mma", _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out),
              _ptr(block_table), block_table.shape[1], _ptr(seq_start), _ptr(seq_past), n_seqs, int(max_q_len), num_heads,
              num_kv_heads, head_dim, page_tokens, ring_tokens, int(window or 0), float(scale), _stream())
        return
    _call("attention", "qt_attention_prefill", _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _code(q, "q"),
          _ptr(block_table), block_table.shape[1], _ptr(seq_start), _ptr(seq_past), n_seqs, int(max_q_len), num_heads,
          num_kv_heads, head_dim, page_tokens, ring_tokens, int(window or 0), float(scale), _stream())


def _ws_merges_in_cluster(n_splits: int, warps: int, group: int, head_dim: int) -> bool:
    """Whether qt_attention_decode_ws merges its blocks in one launch (the rule of attention_mma.cu)."""
    if os.environ.get("QT_B200_DECODE_CLUSTER", "1").startswith("0") or not 2 <= n_splits <= 8:
        return False
    rows = min(group, 16)
    rings = 16 * (head_dim + 8) * 2 + warps * 4 * 32 * (head_dim + 8) * 2
    return rings + n_splits * (rows * head_dim + 2 * rows) * 4 <= 227 * 1024


DECODE_WARPS_MAX = 6     # warps per block of the one-range-per-warp decode kernel


def attention_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                     block_table: torch.Tensor, seq_len: torch.Tensor, num_kv_heads: int, page_tokens: int,
                     ring_tokens: int, window: int | None, scale: float, n_splits: int,
                     part_acc: torch.Tensor | None, part_ml: torch.Tensor | None, impl: str | None = None,
                     warps: int = 1) -> None:
    """One query token per sequence; ``seq_len`` counts the keys it sees (its own included).

    With ``n_splits`` > 1 the keys of each sequence are cut into that many ranges whose partial
    results pass through ``part_acc`` (float, >= B nq splits d) and ``part_ml`` (float, >= B nq splits 2).
    The tensor-core kernels are "ws" (every warp of a block walks a range of its own: n_splits * warps
    ranges, n_splits partial results; the default where it applies) and "mma" (the four warps of a block
    share each tile); "generic" takes every element type and head size.
    """
    n_seqs, num_heads, head_dim = _check_attention(q, k_cache, v_cache, out, block_table, num_kv_heads, page_tokens)
    _need(seq_len, "seq_len", torch.int32, (n_seqs,))
    if n_splits > 1:
        _need(part_acc, "part_acc", torch.float32)
        _need(part_ml, "part_ml", torch.float32)
        if part_acc.numel() < n_seqs * num_heads * n_splits * head_dim or part_ml.numel() < n_seqs * num_heads * n_splits * 2:
            raise KernelError("attention_decode: scratch is too small for this batch and split count")
    if impl == "ws" and not attention_mma_supported(q, page_tokens):
        raise KernelError(f"the tensor-core attention kernels do not take {q.dtype}, head_dim={q.shape[2]}, pages of {page_tokens}")
    picked = "ws" if impl == "ws" else _pick_attention(q, page_tokens, impl)
    if picked == "mma" and impl is None:
        picked = "ws"
    common = (_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), block_table.shape[1], _ptr(seq_len),
              n_seqs, num_heads, num_kv_heads, head_dim, page_tokens, ring_tokens, int(window or 0), float(scale), int(n_splits))
    launches = 2 if n_splits > 1 else 1
    if picked == "ws" and _ws_merges_in_cluster(n_splits, warps, num_heads // num_kv_heads, head_dim):
        launches = 1
    if picked == "ws":
        _call("attention_mma", "qt_attention_decode_ws", *common, int(warps), _ptr(part_acc), _ptr(part_ml), _stream(), launches=launches)
    elif picked == "mma":
        _call("attention_mma", "qt_attention_decode_mma", *common, _ptr(part_acc), _ptr(part_ml), _stream(), launches=launches)
    else:
        _call("attention", "qt_attention_decode", *common[:4], _code(q, "q"), *common[4:], _ptr(part_acc), _ptr(part_ml),
              _stream(), launches=launches)


# ----------------------------------------------------------------------------- matrix product
def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: GemmOut) -> None:
    """out = a [M, K] @ w [N, K]^T on the FMA pipe (float accumulation, any sizes)."""
    _need(a, "a")
    _need(w, "w", a.dtype)
    if a.shape[1] != w.shape[1] or out.n_splits != 1 or (out.rows, out.cols) != (a.shape[0], w.shape[0]):
        raise KernelError(f"gemm: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.tensor.shape)} do not fit")
    _call("gemm_simt", "qt_gemm_simt", _ptr(a), _ptr(w), _code(a, "a"), _ptr(out.tensor), _code(out.tensor, "out"),
          a.shape[0], w.shape[0], a.shape[1], _stream())


# ----------------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    _need(logits, "logits", torch.float32)
    _need(out, "out", torch.int32, (logits.shape[0],))
    _call("sampling", "qt_argmax", _ptr(logits), _ptr(out), logits.shape[0], logits.shape[1], _stream())


def feed_tokens(ids: torch.Tensor, chosen: torch.Tensor, vocab: int) -> None:
    """ids[i] (a row number of ``chosen``, or negative) becomes the token chosen for that row (0 if negative)."""
    _need(ids, "ids", torch.int32)
    _need(chosen, "chosen", torch.int32)
    _call("sampling", "qt_feed_tokens", _ptr(ids), _ptr(chosen), ids.numel(), chosen.numel(), int(vocab), _stream())


def sample(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor, out: torch.Tensor) -> None:
    rows = logits.shape[0]
    _need(logits, "logits", torch.float32)
    _need(temperature, "temperature", torch.float32, (rows,))
    _need(uniform, "uniform", torch.float32, (rows,))
    _need(out, "out", torch.int32, (rows,))
    _call("sampling", "qt_sample", _ptr(logits), _ptr(temperature), _ptr(uniform), _ptr(out), rows, logits.shape[1],
          _stream())


def sample_keyed(logits: torch.Tensor, temperature: float, seed: int, keys: torch.Tensor, out: torch.Tensor,
                 top_k: int = 0, top_p: float = 1.0) -> None:
    """Temperature sampling with the uniform number of each row made on the device from (seed, request, step);
    ``keys`` int32 [rows, 2] holds each row's request and step number.  ``top_k`` > 0 keeps the k largest logits (and
    what ties with the k-th), ``top_p`` < 1 of those the most likely tokens whose renormalised probabilities first sum
    to it (and what ties with the last)."""
    rows = logits.shape[0]
    if not 0.0 < top_p <= 1.0 or top_k < 0:
        raise KernelError(f"sample: top_k={top_k} must not be negative and top_p={top_p} must lie in (0, 1]")
    _need(logits, "logits", torch.float32)
    _need(keys, "keys", torch.int32, (rows, 2))
    _need(out, "out", torch.int32, (rows,))
    seed &= (1 << 64) - 1
    _call("sampling", "qt_sample_keyed", _ptr(logits), float(temperature), seed - (1 << 64) if seed >> 63 else seed, _ptr(keys),
          _ptr(out), rows, logits.shape[1], int(top_k), float(top_p), _stream())


_STATUS: dict[int, torch.Tensor] = {}
_TC_TILES = (16, 32, 64, 128, 256)
_SM_COUNTS: dict[int, int] = {}


def sm_count(device: torch.device | str | None = None) -> int:
    """Streaming multiprocessors of ``device`` (asked once per device)."""
    device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _SM_COUNTS:
        _SM_COUNTS[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return _SM_COUNTS[index]

TC_MAX_BLOCK_TOKENS = 128      # tokens per block that ``gemm`` gives the one-block kernel (256 measured slower at every split count)


def _status_word(device: torch.device) -> torch.Tensor:
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _STATUS:
        _STATUS[index] = torch.zeros(4, dtype=torch.int32, device=device)
    return _STATUS[index]


def status_word(device: torch.device | str = "cuda") -> torch.Tensor:
    """The device words the tensor-core kernels report into (word 0: the code of a wait that ran out, else 0)."""
    return _status_word(torch.device(device))


def check_status(device: torch.device | str = "cuda") -> None:
    """Raise if a bounded wait inside a tensor-core kernel ran out since the last check (synchronises)."""
    word = _status_word(torch.device(device))
    code = int(word[0].item())
    if code != 0:
        word.zero_()
        tail = _PAIR_TAIL.get(word.device.index)
        if tail is not None:
            tail[1].zero_()                    # flags of the pair kernel's last wave that the failed launch left up
        role = {1: "the TMA producer", 2: "the MMA issuer", 3: "the epilogue", 4: "the MMA issuer (for a free accumulator)",
                5: "a kernel whose shared memory was less aligned than its launch allowed for",
                6: "a pair that finishes a tile (for another pair's sums)"}.get(code, f"role {code}")
        raise KernelError(f"gemm_tc: a wait of {role} ran out; the result of that launch is invalid")


def tc_token_tile(rows: int) -> int:
    for tile in _TC_TILES:
        if rows <= tile:
            return min(tile, TC_MAX_BLOCK_TOKENS)
    return TC_MAX_BLOCK_TOKENS


def tc_normalise_splits(k: int, wanted: int) -> int:
    """The largest split count <= ``wanted`` that leaves no split without a 64-wide K block."""
    blocks = -(-k // 64)
    wanted = max(1, min(wanted, blocks))
    per = -(-blocks // wanted)
    return -(-blocks // per)


def gemm_tc_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: GemmOut, token_tile: int | None = None, stages: int = 0,
            swiglu: bool = False, activation: str = "silu") -> None:
    """out = a [M, K] @ w [N, K]^T on the tcgen05 tensor cores; bfloat16 inputs, K a multiple of 8.

    ``out`` is [1, M, N] bfloat16 or float, or [splits, M, N] float for split-K partial sums.  With ``swiglu`` the
    rows of ``w`` alternate SWIGLU_GROUP of a gate and of an up projection and ``out`` [1, M, N / 2] (bfloat16)
    receives act(gate) * up from the epilogue.
    """
    _need(a, "a", torch.bfloat16)
    _need(w, "w", torch.bfloat16)
    rows, k = a.shape
    cols = w.shape[0] // 2 if swiglu else w.shape[0]
    if k != w.shape[1] or (out.rows, out.cols) != (rows, cols) or (swiglu and (out.n_splits != 1 or w.shape[0] % (2 * SWIGLU_GROUP)
                                                                                   or out.tensor.dtype != torch.bfloat16)):
        raise KernelError(f"gemm: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.tensor.shape)} do not fit")
    if rows == 0:
        return
    if not out.tensor.is_cuda or out.tensor.dtype not in _CODES:
        raise KernelError("gemm_tc: the output must be a bfloat16 or float32 CUDA tensor")
    tile = token_tile or tc_token_tile(rows)
    _call("gemm_tc", "qt_gemm_tc", _ptr(a), _ptr(w), _ptr(out.tensor), _code(out.tensor, "out"), rows, w.shape[0], k, tile,
          out.n_splits, out.split_stride, int(stages), 1 if swiglu else 0, activation_code(activation) if swiglu else 0,
          _ptr(_status_word(a.device)), _stream())


_PAIR_TAIL: dict[int, tuple[torch.Tensor, torch.Tensor, int]] = {}


def _pair_tail(device: torch.device) -> tuple[torch.Tensor, torch.Tensor, int]:
    """Scratch of the pair kernel's last wave (one accumulator tile per resident pair, and the flags that guard the
    slots), made once per device: (slots, flags, pairs)."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _PAIR_TAIL:
        pairs = max(1, sm_count(device) // 2)  # one resident pair per TPC at most
        floats = _fn("gemm_tc", "qt_gemm_tc_pair_slots")()
        _PAIR_TAIL[index] = (torch.empty(pairs * floats, dtype=torch.float32, device=device),
                             torch.zeros(pairs * 8, dtype=torch.int32, device=device), pairs)
    return _PAIR_TAIL[index]


def pair_tail_mode() -> int:
    """``QT_B200_PAIR_TAIL``: 0 or unset = every tile of the pair kernel by one pair; -1 = the last wave by K ranges
    where the kernel's model of the time saved says it pays; 1 = wherever the tiles do not divide by the pairs.
    Off by default: launched alone at full clocks the cut saves up to a quarter of a product with a long K and a
    half-empty last wave, but a whole prefill runs at the power limit, where idle pairs in a last wave leave their
    power to the others, and measured the same or slower with it."""
    return int(os.environ.get("QT_B200_PAIR_TAIL", "0"))


def gemm_tc_pair(a: torch.Tensor, w: torch.Tensor, out: GemmOut, swiglu: bool = False, activation: str = "silu",
                 tail: int | None = None) -> None:
    """The same product by pairs of blocks on the two SMs of a TPC (tcgen05 cta_group::2): 256 weight rows x
    256 tokens per tile, each block staging half of both operands; one persistent pair per TPC with two
    accumulators in tensor memory.  Meant for many tokens; ``out`` may be [splits, M, N] float partial sums, which
    pays for a few hundred tokens whose tiles alone do not fill the TPCs.

    With ``swiglu`` the rows of ``w`` alternate SWIGLU_GROUP of a gate and of an up projection
    (``interleave_gate_up``) and ``out`` [1, M, N / 2] receives act(gate) * up from the epilogue."""
    _need(a, "a", torch.bfloat16)
    _need(w, "w", torch.bfloat16)
    rows, k = a.shape
    cols = w.shape[0] // 2 if swiglu else w.shape[0]
    if k != w.shape[1] or (out.rows, out.cols) != (rows, cols) or (swiglu and (out.n_splits != 1 or w.shape[0] % (2 * SWIGLU_GROUP))):
        raise KernelError(f"gemm: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.tensor.shape)} do not fit")
    if rows == 0:
        return
    if not out.tensor.is_cuda or out.tensor.dtype not in _CODES:
        raise KernelError("gemm_tc_pair: the output must be a bfloat16 or float32 CUDA tensor")
    tail = pair_tail_mode() if tail is None else int(tail)
    slots, flags, pairs = _pair_tail(a.device) if tail != 0 and out.n_splits == 1 else (None, None, 0)
    _call("gemm_tc", "qt_gemm_tc_pair", _ptr(a), _ptr(w), _ptr(out.tensor), _code(out.tensor, "out"), rows, w.shape[0], k,
          1 if swiglu else 0, activation_code(activation) if swiglu else 0, out.n_splits, out.split_stride,
          tail, _ptr(slots) if slots is not None else None, _ptr(flags) if flags is not None else None, pairs,
          _ptr(_status_word(a.device)), _stream())


def gemm_uses_pairs(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether ``gemm`` gives this product to the pair kernel (a static choice by element type and shape)."""
    if not gemm_tc_supported(a, w):
        return False
    # more than 256 tokens; or more than one block's 128 with a weight whose tiles fill the machine unsplit (the fused
    # gate/up projection, the head), which single blocks would read once per token tile
    return a.shape[0] > _TC_TILES[-1] or (a.shape[0] > TC_MAX_BLOCK_TOKENS and w.shape[0] >= 128 * sm_count(a.device))


def gemm(a: torch.Tensor, w: torch.Tensor, out: GemmOut) -> None:
    """out = a @ w^T with the kernel that fits the element type and shape (a static choice):
    tensor cores for bfloat16 with 16-byte aligned rows, the FMA kernel for float32 and the rest."""
    if gemm_tc_supported(a, w):
        if gemm_uses_pairs(a, w):
            gemm_tc_pair(a, w, out)         # more tokens than one block's tile: pairs of blocks, a third less operand traffic
        else:
            gemm_tc(a, w, out)
    elif out.n_splits == 1:
        gemm_simt(a, w, out)
    else:
        raise KernelError("gemm: split-K output is only produced by the tensor-core kernel")


# ----------------------------------------------------------------------------- products of a decode step, fused
FUSED_MAX_ROWS = 128        # most tokens the fused product takes (one token tile per block)
FUSED_MAX_SPLITS = 8        # blocks of a cluster that share a weight tile
_EPI_STORE, _EPI_RESIDUAL, _EPI_SWIGLU, _EPI_QKV = 0, 1, 2, 3


def fused_enabled(role: str) -> bool:
    """``QT_B200_FUSED`` in the environment: "0" turns the fused products off, a comma-separated list keeps only the
    named ones ("qkv", "gate", "attn_out", "mlp_out"); unset or "1": all of them."""
    setting = os.environ.get("QT_B200_FUSED", "1")
    if setting in ("1", ""):
        return True
    return setting != "0" and role in setting.split(",")


@dataclass
class ScaledRows:
    """Rows handed from an RMSNorm to the product behind it with the norm half done: ``tensor`` [M, K] holds
    bf16(r * g) for the stream rows r and the norm's weight g, and the rows' factor rsqrt(mean(r^2) + eps) is
    still to be applied, by the product's epilogue (the product is linear in its input).  ``sq`` [tiles, M]
    holds the sums of squares of r over ``tiles`` column ranges; mean(r^2) = sum over tiles / ``width``."""

    tensor: torch.Tensor
    sq: torch.Tensor
    width: int
    eps: float

    @property
    def shape(self):
        return self.tensor.shape


def fused_supported(w: torch.Tensor) -> bool:
    """The fused products take bfloat16 weights [N, K] with K a multiple of 8, 16-byte aligned."""
    return w.dtype == torch.bfloat16 and w.dim() == 2 and w.shape[1] % 8 == 0 and w.data_ptr() % 16 == 0 and w.is_contiguous()


def fused_qkv_supported(head_dim: int, rotary_dim: int) -> bool:
    """The fused q/k-norm + rotation + cache write needs whole heads inside a 128-row weight tile and rotation
    pairs that four-element pieces can exchange."""
    return head_dim >= 16 and 128 % head_dim == 0 and rotary_dim % 8 == 0 and rotary_dim <= head_dim


def _fused(x, w: torch.Tensor, splits: int, epilogue: int, *, out=None, residual=None, norm_w=None, xw=None, sq_out=None,
           q_out=None, k_cache=None, v_cache=None, token_seq=None, token_pos=None, block_table=None, q_w=None, k_w=None,
           qk_eps=0.0, cos_sin=None, nq=0, nkv=0, d=0, page_tokens=0, ring_tokens=0, write_kv=False, stages: int = 0,
           act: int = 0, interleaved: bool = False) -> None:
    scaled = x if isinstance(x, ScaledRows) else None
    a = scaled.tensor if scaled is not None else x
    _need(a, "x", torch.bfloat16)
    _need(w, "w", torch.bfloat16)
    rows, k = a.shape
    if k != w.shape[1]:
        raise KernelError(f"gemm_fused: x {tuple(a.shape)} and w {tuple(w.shape)} do not fit")
    if not 0 < rows <= FUSED_MAX_ROWS:
        raise KernelError(f"gemm_fused: {rows} tokens (1..{FUSED_MAX_ROWS})")
    if scaled is not None:
        _need(scaled.sq, "sq", torch.float32)
        if scaled.sq.dim() != 2 or scaled.sq.shape[1] != rows:
            raise KernelError(f"gemm_fused: sums of squares {tuple(scaled.sq.shape)} for {rows} rows")
    rotary_dim, max_pos = (0, 0) if cos_sin is None else (cos_sin.shape[1], cos_sin.shape[0])
    _call("gemm_fused", "qt_gemm_fused", _ptr(a), _ptr(w), rows, w.shape[0], k, tc_token_tile(rows), int(splits), int(stages), epilogue,
          _ptr(scaled.sq) if scaled is not None else None, scaled.sq.shape[0] if scaled is not None else 0,
          scaled.width if scaled is not None else 0, float(scaled.eps) if scaled is not None else 0.0,
          _ptr(out), _CODES.get(out.dtype, -1) if out is not None else 0, int(act),
          _ptr(residual), _ptr(norm_w), _ptr(xw), _ptr(sq_out),
          _ptr(q_out), _ptr(k_cache), _ptr(v_cache), _ptr(token_seq), _ptr(token_pos), _ptr(block_table),
          block_table.shape[1] if block_table is not None else 0, _ptr(q_w), _ptr(k_w), float(qk_eps),
          _ptr(cos_sin), rotary_dim, max_pos, nq, nkv, d, page_tokens, ring_tokens, 1 if write_kv else 0,
          1 if interleaved else 0, _ptr(_status_word(a.device)), _stream())


def gemm_fused_store(x, w: torch.Tensor, out: torch.Tensor, splits: int = 1, stages: int = 0) -> None:
    """out [M, N] (float or bfloat16) = x w^T, times the rows' deferred norm factor if ``x`` is ``ScaledRows``."""
    _need(out, "out", shape=(x.shape[0], w.shape[0]))
    _fused(x, w, splits, _EPI_STORE, out=out, stages=stages)


def gemm_fused_residual(x, w: torch.Tensor, residual: torch.Tensor, norm_weight: torch.Tensor | None = None,
                        eps: float = 0.0, xw: torch.Tensor | None = None, sq: torch.Tensor | None = None, splits: int = 1,
                        stages: int = 0) -> "ScaledRows | None":
    """residual [M, N] (float, in place) += x w^T.  With ``norm_weight`` [N] the RMSNorm that follows is prepared in
    the same launch: ``xw`` [M, N] = bf16(residual * norm_weight) and ``sq`` [ceil(N / 128), M] = the rows' sums of
    squares per 128 columns; returns them as ``ScaledRows`` for the product behind the norm."""
    rows, n = x.shape[0], w.shape[0]
    _need(residual, "residual", torch.float32, (rows, n))
    if norm_weight is None:
        _fused(x, w, splits, _EPI_RESIDUAL, residual=residual, stages=stages)
        return None
    _need(norm_weight, "norm_weight", torch.float32, (n,))
    _need(xw, "xw", torch.bfloat16, (rows, n))
    _need(sq, "sq", torch.float32, (-(-n // 128), rows))
    _fused(x, w, splits, _EPI_RESIDUAL, residual=residual, norm_w=norm_weight, xw=xw, sq_out=sq, stages=stages)
    return ScaledRows(xw, sq, n, float(eps))


def gemm_fused_swiglu(x, w: torch.Tensor, out: torch.Tensor, splits: int = 1, stages: int = 0, activation: str = "silu") -> None:
    """out [M, N / 2] (bfloat16) = act(gate) * up for a weight whose rows alternate SWIGLU_GROUP of gate and of up."""
    if w.shape[0] % (2 * SWIGLU_GROUP):
        raise KernelError(f"gemm_fused_swiglu: {w.shape[0]} rows are not gate and up rows in groups of {SWIGLU_GROUP}")
    _need(out, "out", torch.bfloat16, (x.shape[0], w.shape[0] // 2))
    _fused(x, w, splits, _EPI_SWIGLU, out=out, stages=stages, act=activation_code(activation))


def gemm_fused_qkv(x, w: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor | None, v_cache: torch.Tensor | None,
                   token_seq: torch.Tensor, token_pos: torch.Tensor, block_table: torch.Tensor | None,
                   q_weight: torch.Tensor | None, k_weight: torch.Tensor | None, eps: float, cos_sin: torch.Tensor | None,
                   num_heads: int, num_kv_heads: int, head_dim: int, page_tokens: int, ring_tokens: int,
                   write_kv: bool = True, splits: int = 1, stages: int = 0, interleaved: bool = False) -> None:
    """The fused projection [q; k; v] (or q alone) with per-head q/k RMSNorm, rotation and the cache write done in
    its epilogue: what ``gemm`` followed by ``qk_norm_rope_write`` does, in one launch."""
    rows = x.shape[0]
    rotary_dim = 0 if cos_sin is None else cos_sin.shape[1]
    if not fused_qkv_supported(head_dim, rotary_dim):
        raise KernelError(f"gemm_fused_qkv: head_dim={head_dim} with rotary_dim={rotary_dim} is not taken")
    _need(q_out, "q_out", torch.bfloat16, (rows, num_heads, head_dim))
    _need(token_seq, "token_seq", torch.int32, (rows,))
    _need(token_pos, "token_pos", torch.int32, (rows,))
    for name, weight in (("q_weight", q_weight), ("k_weight", k_weight)):
        if weight is not None:
            _need(weight, name, torch.float32, (head_dim,))
    if cos_sin is not None:
        _need(cos_sin, "cos_sin", torch.float32)
    if write_kv:
        _need(block_table, "block_table", torch.int32)
        for name, cache in (("k_cache", k_cache), ("v_cache", v_cache)):
            _need(cache, name, torch.bfloat16)
            if tuple(cache.shape[1:]) != (num_kv_heads, page_tokens, head_dim):
                raise KernelError(f"{name}: shape {tuple(cache.shape)} is not [pages, {num_kv_heads}, {page_tokens}, {head_dim}]")
    _fused(x, w, splits, _EPI_QKV, q_out=q_out, k_cache=k_cache if write_kv else None, v_cache=v_cache if write_kv else None,
           token_seq=token_seq, token_pos=token_pos, block_table=block_table if write_kv else None, q_w=q_weight, k_w=k_weight,
           qk_eps=eps, cos_sin=cos_sin, nq=num_heads, nkv=num_kv_heads, d=head_dim, page_tokens=page_tokens,
           ring_tokens=ring_tokens, write_kv=write_kv, stages=stages, interleaved=interleaved)
