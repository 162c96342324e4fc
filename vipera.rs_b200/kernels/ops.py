"""Python face of the CUDA kernels: one function per launcher, called through ctypes.

Every function takes torch tensors that already live on the GPU, checks what the kernel
cannot check for itself (device, dtype, contiguity, extents), and launches on torch's
current stream.  There is no fallback: a tensor that is not on a CUDA device, a missing
compiler or a kernel that reports an error raises.
"""
from __future__ import annotations

import ctypes
import functools
import os
from typing import Optional

import torch

from ..build import load_kernel_library
from ..errors import InternalError, InvalidArgumentError, UnsupportedError

F32, BF16 = 0, 1
EPI_STORE, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2
EPI_GATED = EPI_SWIGLU   # the gated unit over interleaved gate and up rows; its activation is an argument
ACT_SILU, ACT_GELU_TANH, ACT_RELU2 = 0, 1, 2
ACTIVATIONS = {"silu": ACT_SILU, "gelu_tanh": ACT_GELU_TANH}   # of a gated unit's gate
UNIT_ACTIVATIONS = {**ACTIVATIONS, "relu2": ACT_RELU2}          # of a unit without a gate (relu2: the square of relu)
ROPE_NONE, ROPE_NEOX, ROPE_INTERLEAVED = 0, 1, 2
SAMPLE_OK, SAMPLE_NO_FINITE, SAMPLE_NO_MASS, SAMPLE_NEEDS_HOST = 0, 1, 2, 3

_c_int, _c_float, _c_void = ctypes.c_int, ctypes.c_float, ctypes.c_void_p
_functions = {}

_STATUS_TEXT = {
    -1: "unsupported element type",
    -2: "a size this kernel does not take",
    -3: "bad argument",
    -4: "the CUDA driver gave no entry point for tensor maps",
    -5: "a bounded wait inside the kernel ran out",
}


def _function(library: str, name: str, argtypes):
    key = (library, name)
    fn = _functions.get(key)
    if fn is None:
        fn = getattr(load_kernel_library(library), name)
        fn.argtypes = argtypes
        fn.restype = _c_int
        _functions[key] = fn
    return fn


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise UnsupportedError(f"kernels take float32 and bfloat16, not {dtype}")


def _stream() -> int:
    """The raw handle of torch's current stream on the current device."""
    try:
        return torch._C._cuda_getCurrentRawStream(torch.cuda.current_device())
    except AttributeError:  # a torch without that shortcut
        return torch.cuda.current_stream().cuda_stream


def feed_tokens(src: torch.Tensor, dst: torch.Tensor, own: int) -> None:
    """dst[i] = src[i] for i < own, src[0] for the rest of dst: a step's drawn tokens as the next
    step's input, on the device."""
    fn = _function("sampling", "vipera_feed_tokens", [_c_void, _c_void, _c_int, _c_int, _c_void])
    _check(fn(_gpu(src, "src", torch.int32), _gpu(dst, "dst", torch.int32), int(own), int(dst.numel()), _stream()),
           "feed_tokens", kernels=1)


def stream_synchronize() -> None:
    """Wait for the current stream (a direct call; torch's own builds a stream object first)."""
    fn = _function("sampling", "vipera_stream_synchronize", [_c_void])
    _check(fn(_stream()), "stream_synchronize", kernels=0)


launches = 0  # kernels launched through this module (replayed graphs add what they captured)


class KernelProfile:
    """Device time of a step by class of kernel, as the reference splits a pass into its kinds
    of work (crates/vipera-backend-cpu/src/profile.rs:226-275).  While one is installed
    (``ops.profile = KernelProfile()``) every launcher records a CUDA event behind its launch;
    the time between two events goes to the class of the later one.  Steps must then be
    launched kernel by kernel (a replayed graph launches nothing through this module)."""

    CLASSES = {
        "embed": "embed", "rmsnorm": "norm", "rope_cache": "rope_kv",
        "gemm_tc": "proj", "gemm_tc_rope": "proj", "gemv_small": "proj", "gemm_simt": "proj",
        "attention": "attention", "attention_prefill": "attention", "attention_prefill_tc": "attention",
        "attention_decode": "attention", "mlstm": "recurrence", "mamba_scan": "recurrence", "gla": "recurrence",
        "lightning": "recurrence", "moe": "experts",
        "layernorm": "norm", "causal_conv": "conv",
        "argmax": "sample", "sample": "sample", "apply_penalties": "sample", "feed_tokens": "sample",
        "logprobs": "sample",
    }
    ORDER = ("proj", "experts", "attention", "recurrence", "norm", "conv", "rope_kv", "embed", "sample", "other")

    def __init__(self):
        self._events = []
        self._marks = []
        self._start = None
        self.totals = {}   # kind of step -> {"steps": n, "ms": total, class: ms}

    def _event(self):
        return self._events.pop() if self._events else torch.cuda.Event(enable_timing=True)

    def begin(self) -> None:
        self._marks = []
        self._start = self._event()
        self._start.record()

    def mark(self, what: str) -> None:
        if self._start is None:
            return
        event = self._event()
        event.record()
        self._marks.append((self.CLASSES.get(what, "other"), event))

    def end(self, kind: str) -> dict:
        """Wait for the step and add it to the totals of its kind; returns the running averages."""
        if self._start is None:
            return {}
        torch.cuda.current_stream().synchronize()
        split = {}
        before = self._start
        for name, event in self._marks:
            split[name] = split.get(name, 0.0) + before.elapsed_time(event)
            before = event
        total = self._start.elapsed_time(before) if self._marks else 0.0
        self._events.extend(event for _, event in self._marks)
        self._events.append(self._start)
        self._start, self._marks = None, []
        totals = self.totals.setdefault(kind, {"steps": 0, "ms": 0.0})
        totals["steps"] += 1
        totals["ms"] += total
        for name, ms in split.items():
            totals[name] = totals.get(name, 0.0) + ms
        return totals

    def line(self, kind: str) -> str:
        totals = self.totals.get(kind)
        if not totals or not totals["steps"]:
            return f"PROFILE {kind} 0"
        steps, average = totals["steps"], totals["ms"] / totals["steps"]
        parts = [f"PROFILE {kind} {steps} {average:.3f} ms:"]
        for name in self.ORDER:
            if name in totals:
                ms = totals[name] / steps
                parts.append(f"{name} {ms:.3f}ms ({100.0 * ms / average if average else 0.0:.0f}%)")
        return " ".join(parts)


profile: Optional[KernelProfile] = None


def _check(status: int, what: str, kernels: int = 1) -> None:
    global launches
    if status == 0:
        launches += kernels
        if profile is not None:
            profile.mark(what)
        return
    if status > 0:
        text = f"CUDA error {status}"
        try:
            text = f"CUDA error {status}: " + torch.cuda.cudart().cudaGetErrorString(status)  # type: ignore[attr-defined]
        except Exception:
            pass
    else:
        text = _STATUS_TEXT.get(status, f"status {status}")
    raise InternalError(f"{what}: {text}")


def _gpu(tensor: torch.Tensor, name: str, dtype=None) -> int:
    if not tensor.is_cuda:
        raise InternalError(f"{name} is not on a CUDA device; this engine has no CPU path")
    if not tensor.is_contiguous():
        raise InvalidArgumentError(f"{name} must be contiguous")
    if dtype is not None and tensor.dtype != dtype:
        raise InvalidArgumentError(f"{name} must be {dtype}, got {tensor.dtype}")
    return tensor.data_ptr()


def _opt(tensor: Optional[torch.Tensor], name: str, dtype=None):
    return None if tensor is None else _gpu(tensor, name, dtype)


# ----------------------------------------------------------------------------------------
def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[t, :] = scale * table[tokens[t], :] as float32."""
    fn = _function("rowwise", "vipera_embed",
                   [_c_void, _c_int, _c_void, _c_void, _c_int, _c_int, _c_int, _c_float, _c_void])
    count, hidden = out.shape
    if table.shape[1] != hidden or tokens.numel() != count:
        raise InvalidArgumentError("embed: shapes of table, tokens and out do not agree")
    _check(fn(_gpu(table, "table"), dtype_code(table.dtype), _gpu(tokens, "tokens", torch.int32),
              _gpu(out, "out", torch.float32), count, hidden, table.shape[0], float(scale), _stream()), "embed")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r, :] = rmsnorm(x[rows[r], :]) * weight (rows defaults to all rows in order)."""
    fn = _function("rowwise", "vipera_rmsnorm",
                   [_c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_float, _c_void])
    hidden = x.shape[1]
    count = out.shape[0]
    if out.shape[1] != hidden or weight.numel() != hidden:
        raise InvalidArgumentError("rmsnorm: widths of x, weight and out do not agree")
    if rows is None and x.shape[0] != count:
        raise InvalidArgumentError("rmsnorm: x and out have different row counts")
    if rows is not None and rows.numel() != count:
        raise InvalidArgumentError("rmsnorm: one row index is needed for each output row")
    _check(fn(_gpu(x, "x", torch.float32), _gpu(weight, "weight", torch.float32),
              _opt(rows, "rows", torch.int32), _gpu(out, "out"), dtype_code(out.dtype), count, hidden,
              float(eps), _stream()), "rmsnorm")


_sm_counts = {}


def sm_count(device) -> int:
    """The number of multiprocessors of `device`, asked once."""
    key = str(device)
    count = _sm_counts.get(key)
    if count is None:
        count = _sm_counts[key] = int(torch.cuda.get_device_properties(device).multi_processor_count)
    return count


def rope_cache(qkv: torch.Tensor, q_out: torch.Tensor, *, num_heads: int, num_kv_heads: int, head_dim: int,
               positions: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], style: int,
               k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
               token_seq: Optional[torch.Tensor], block_table: Optional[torch.Tensor], page_size: int,
               write_cache: bool, value_dim: Optional[int] = None, rot_dims: Optional[int] = None) -> None:
    """Rotate q and k of a float32 [tokens, (heads + 2 kv_heads) * d] product; write q to
    q_out [tokens, heads * d] and k, v into their cache pages.  ``rot_dims`` (default d): only
    the first that many values of a head turn, with tables of width rot_dims/2; ``value_dim``
    (default d): a value row's size, the product then being [tokens, (heads + kv_heads) * d +
    kv_heads * value_dim]."""
    value_dim = head_dim if value_dim is None else int(value_dim)
    rot_dims = head_dim if rot_dims is None else int(rot_dims)
    if style == ROPE_NONE:
        rot_dims = head_dim if head_dim % 2 == 0 else 0    # nothing turns; an odd head size takes the general form
    if value_dim != head_dim or rot_dims != head_dim:
        return _rope_cache_partial(qkv, q_out, num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim,
                                   value_dim=value_dim, rot_dims=rot_dims, positions=positions, cos=cos, sin=sin,
                                   style=style, k_pool=k_pool, v_pool=v_pool, token_seq=token_seq,
                                   block_table=block_table, page_size=page_size, write_cache=write_cache)
    fn = _function("rope_cache", "vipera_rope_cache",
                   [_c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void, _c_void, _c_void, _c_int,
                    _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_void])
    count = qkv.shape[0]
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise InvalidArgumentError("rope_cache: qkv width does not match the head counts")
    if q_out.shape[0] != count or q_out.shape[1] != num_heads * head_dim:
        raise InvalidArgumentError("rope_cache: q_out has the wrong shape")
    if style != ROPE_NONE:
        if cos is None or sin is None or cos.shape[1] != head_dim // 2:
            raise InvalidArgumentError("rope_cache: a cos/sin table of width d/2 is needed")
    if write_cache:
        if k_pool is None or v_pool is None or k_pool.dtype != q_out.dtype:
            raise InvalidArgumentError("rope_cache: cache pools must have the activation dtype")
        if k_pool.shape[1:] != (page_size, num_kv_heads, head_dim) or v_pool.shape != k_pool.shape:
            raise InvalidArgumentError("rope_cache: cache pools must be [pages, page_size, kv_heads, d]")
    width = 0 if block_table is None else block_table.shape[1]
    _check(fn(_gpu(qkv, "qkv", torch.float32), _gpu(q_out, "q_out"), dtype_code(q_out.dtype), count,
              num_heads, num_kv_heads, head_dim, _gpu(positions, "positions", torch.int32),
              _opt(cos, "cos", torch.float32), _opt(sin, "sin", torch.float32), style,
              _opt(k_pool, "k_pool"), _opt(v_pool, "v_pool"), _opt(token_seq, "token_seq", torch.int32),
              _opt(block_table, "block_table", torch.int32), width, page_size, 1 if write_cache else 0,
              _stream()), "rope_cache")


def _rope_cache_partial(qkv, q_out, *, num_heads, num_kv_heads, head_dim, value_dim, rot_dims, positions, cos, sin,
                        style, k_pool, v_pool, token_seq, block_table, page_size, write_cache) -> None:
    fn = _function("rope_cache", "vipera_rope_cache_partial",
                   [_c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void, _c_void, _c_void,
                    _c_int, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_void])
    count = qkv.shape[0]
    if qkv.shape[1] != (num_heads + num_kv_heads) * head_dim + num_kv_heads * value_dim:
        raise InvalidArgumentError("rope_cache: qkv width does not match the head counts and sizes")
    if q_out.shape[0] != count or q_out.shape[1] != num_heads * head_dim:
        raise InvalidArgumentError("rope_cache: q_out has the wrong shape")
    if rot_dims % 2 or not 0 <= rot_dims <= head_dim:
        raise InvalidArgumentError("rope_cache: the rotated values must be an even count within the head")
    if style != ROPE_NONE and rot_dims:
        if cos is None or sin is None or cos.shape[1] != rot_dims // 2 or sin.shape != cos.shape:
            raise InvalidArgumentError("rope_cache: cos/sin tables of width rot_dims/2 are needed")
    if write_cache:
        if k_pool is None or v_pool is None or k_pool.dtype != q_out.dtype or v_pool.dtype != q_out.dtype:
            raise InvalidArgumentError("rope_cache: cache pools must have the activation dtype")
        if k_pool.shape[1:] != (page_size, num_kv_heads, head_dim) or \
                v_pool.shape[1:] != (page_size, num_kv_heads, value_dim):
            raise InvalidArgumentError("rope_cache: cache pools must be [pages, page_size, kv_heads, d] and "
                                       "[pages, page_size, kv_heads, value size]")
    width = 0 if block_table is None else block_table.shape[1]
    _check(fn(_gpu(qkv, "qkv", torch.float32), _gpu(q_out, "q_out"), dtype_code(q_out.dtype), count,
              num_heads, num_kv_heads, head_dim, value_dim, rot_dims, _gpu(positions, "positions", torch.int32),
              _opt(cos, "cos", torch.float32), _opt(sin, "sin", torch.float32), style,
              _opt(k_pool, "k_pool"), _opt(v_pool, "v_pool"), _opt(token_seq, "token_seq", torch.int32),
              _opt(block_table, "block_table", torch.int32), width, page_size, 1 if write_cache else 0,
              _stream()), "rope_cache")


def rope_cache_blend(qkv: torch.Tensor, q_out: torch.Tensor, *, num_heads: int, num_kv_heads: int, head_dim: int,
                     value_dim: int, rot_dims: int, positions: torch.Tensor, cos: Optional[torch.Tensor],
                     sin: Optional[torch.Tensor], style: int, k_pool: torch.Tensor, v_pool: torch.Tensor,
                     token_seq: torch.Tensor, block_table: torch.Tensor, page_size: int, write_cache: bool,
                     publish: Optional[torch.Tensor] = None, blend_with: Optional[torch.Tensor] = None,
                     blend: Optional[torch.Tensor] = None) -> None:
    """The general rotation and cache write over a float32 product whose rows may hold more than
    q, k and v (the rest is not read), with values that are published or blended: ``publish``
    float32 [tokens, kv_heads * value_dim] receives the values as projected; with ``blend_with`` (the
    same shape) the cached values are ``(1 - b) v + b blend_with``, b the 32-bit number ``blend``."""
    fn = _function("rope_cache", "vipera_rope_cache_blend",
                   [_c_void, ctypes.c_longlong, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void,
                    _c_void, _c_void, _c_int, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_void, _c_void,
                    _c_void, _c_void])
    count = qkv.shape[0]
    v_width = num_kv_heads * value_dim
    if qkv.dim() != 2 or qkv.stride(1) != 1 or qkv.shape[1] < (num_heads + num_kv_heads) * head_dim + v_width:
        raise InvalidArgumentError("rope_cache: qkv rows are too short for the head counts and sizes")
    if q_out.shape[0] != count or q_out.shape[1] != num_heads * head_dim:
        raise InvalidArgumentError("rope_cache: q_out has the wrong shape")
    if rot_dims % 2 or not 0 <= rot_dims <= head_dim:
        raise InvalidArgumentError("rope_cache: the rotated values must be an even count within the head")
    if style != ROPE_NONE and rot_dims:
        if cos is None or sin is None or cos.shape[1] != rot_dims // 2 or sin.shape != cos.shape:
            raise InvalidArgumentError("rope_cache: cos/sin tables of width rot_dims/2 are needed")
    if write_cache and (k_pool.dtype != q_out.dtype or v_pool.dtype != q_out.dtype or
                        k_pool.shape[1:] != (page_size, num_kv_heads, head_dim) or
                        v_pool.shape[1:] != (page_size, num_kv_heads, value_dim)):
        raise InvalidArgumentError("rope_cache: cache pools must be [pages, page_size, kv_heads, d] and "
                                   "[pages, page_size, kv_heads, value size] of the activation dtype")
    for other in (publish, blend_with):
        if other is not None and (tuple(other.shape) != (count, v_width) or not other.is_contiguous()):
            raise InvalidArgumentError("rope_cache: published and blended values are [tokens, kv_heads * value size]")
    if blend_with is not None and (blend is None or blend.numel() != 1):
        raise InvalidArgumentError("rope_cache: blending needs one 32-bit number")
    _check(fn(_gpu(qkv, "qkv", torch.float32), int(qkv.stride(0)), _gpu(q_out, "q_out"), dtype_code(q_out.dtype), count,
              num_heads, num_kv_heads, head_dim, value_dim, rot_dims, _gpu(positions, "positions", torch.int32),
              _opt(cos, "cos", torch.float32), _opt(sin, "sin", torch.float32), style, _gpu(k_pool, "k_pool"),
              _gpu(v_pool, "v_pool"), _gpu(token_seq, "token_seq", torch.int32),
              _gpu(block_table, "block_table", torch.int32), block_table.shape[1], page_size, 1 if write_cache else 0,
              _opt(publish, "publish", torch.float32), _opt(blend_with, "blend_with", torch.float32),
              _opt(blend, "blend", torch.float32), _stream()), "rope_cache")


def gemm_simt(a: torch.Tensor, w: torch.Tensor, *, epilogue: int = EPI_STORE,
              bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
              resid: Optional[torch.Tensor] = None, activation: int = ACT_SILU) -> None:
    """a[M, K] times w[N, K] transposed, on the CUDA cores with float32 accumulation.  ``bias``
    counts in every ending (for the gated unit it is interleaved like the rows);
    ``activation`` is the gated unit's."""
    fn = _function("gemm_simt", "vipera_gemm_simt_act",
                   [_c_void, _c_int, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void, _c_void, _c_int,
                    _c_void, _c_int, _c_void])
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise InvalidArgumentError(f"gemm: inner sizes differ ({k} and {w.shape[1]})")
    _check_gemm_outputs(m, n, epilogue, bias, out, resid)
    _check(fn(_gpu(a, "a"), dtype_code(a.dtype), _gpu(w, "w"), dtype_code(w.dtype), m, n, k, epilogue,
              _opt(bias, "bias", torch.float32), _opt(out, "out"),
              dtype_code(out.dtype) if out is not None else F32, _opt(resid, "resid", torch.float32),
              int(activation), _stream()), "gemm_simt")


def _check_gemm_outputs(m, n, epilogue, bias, out, resid) -> None:
    if bias is not None and bias.numel() != n:
        raise InvalidArgumentError("gemm: bias must have one value per row of the matrix")
    if epilogue == EPI_STORE:
        if out is None or tuple(out.shape) != (m, n):
            raise InvalidArgumentError(f"gemm: out must be [{m}, {n}]")
    elif epilogue == EPI_RESIDUAL:
        if resid is None or tuple(resid.shape) != (m, n):
            raise InvalidArgumentError(f"gemm: resid must be [{m}, {n}]")
    elif epilogue == EPI_SWIGLU:
        if n % 32:
            raise UnsupportedError("gemm: SwiGLU needs an intermediate size that is a multiple of 16")
        if out is None or tuple(out.shape) != (m, n // 2):
            raise InvalidArgumentError(f"gemm: out must be [{m}, {n // 2}]")
    else:
        raise InvalidArgumentError(f"gemm: unknown epilogue {epilogue}")


def attention(q: torch.Tensor, out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, *,
              token_seq: torch.Tensor, positions: torch.Tensor, block_table: torch.Tensor,
              num_heads: int, num_kv_heads: int, head_dim: int, scale: float, window: int = 0,
              value_dim: Optional[int] = None, keep_first: int = 0, sink: bool = False, chunk: int = 0,
              out_scale: float = 1.0, sink_values: Optional[torch.Tensor] = None,
              gate: Optional[torch.Tensor] = None, gate_offset: int = 0) -> None:
    """Causal grouped-query attention of every token of the step over its request's pages.
    ``value_dim``: a value row's size (default d); ``keep_first``: with a window, that many
    first keys stay visible; ``sink``: one is added to the softmax's denominator; ``chunk``:
    instead of a window, a query sees the earlier keys of its own chunk of that many positions
    (chunks counted from position 0); ``out_scale`` multiplies the output.  ``sink_values``
    float32 [heads]: exp(sink_h) joins head h's denominator instead of one.  ``gate`` float32
    [tokens, width]: the output is multiplied by the sigmoid of the heads * value_dim values that
    start at column ``gate_offset`` of the token's row."""
    fn = _function("attention", "vipera_attention_gated",
                   [_c_void, _c_void, _c_int, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int,
                    _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int, _c_int, _c_float, _c_void,
                    _c_void, ctypes.c_longlong, _c_void])
    if chunk and window:
        raise InvalidArgumentError("attention: a mask is a window or chunks, not both")
    count = q.shape[0]
    value_dim = head_dim if value_dim is None else int(value_dim)
    for size in (head_dim, value_dim):
        if not 0 < size <= 256:
            raise UnsupportedError(f"attention: head size {size} is not within 1 to 256")
    if q.shape[1] != num_heads * head_dim or tuple(out.shape) != (count, num_heads * value_dim) or out.dtype != q.dtype:
        raise InvalidArgumentError("attention: q must be [tokens, heads * d] and out [tokens, heads * value size], of one dtype")
    if k_pool.dtype != q.dtype or v_pool.dtype != q.dtype or v_pool.shape[:3] != k_pool.shape[:3]:
        raise InvalidArgumentError("attention: cache pools must match q's dtype and each other")
    page_size = k_pool.shape[1]
    if k_pool.shape[2:] != (num_kv_heads, head_dim) or v_pool.shape[3] != value_dim:
        raise InvalidArgumentError("attention: cache pools must be [pages, page_size, kv_heads, d] and "
                                   "[pages, page_size, kv_heads, value size]")
    if sink_values is not None and sink_values.numel() != num_heads:
        raise InvalidArgumentError("attention: one sink score per query head")
    gate_pointer, gate_stride = None, 0
    if gate is not None:
        if gate.dim() != 2 or gate.shape[0] != count or gate.stride(1) != 1 or \
                not 0 <= gate_offset <= gate.shape[1] - num_heads * value_dim:
            raise InvalidArgumentError("attention: the gate must hold heads * value size values per token")
        gate_pointer = _gpu(gate, "gate", torch.float32) + 4 * int(gate_offset)
        gate_stride = int(gate.stride(0))
    _check(fn(_gpu(q, "q"), _gpu(out, "out"), dtype_code(q.dtype), _gpu(k_pool, "k_pool"), _gpu(v_pool, "v_pool"),
              _gpu(token_seq, "token_seq", torch.int32), _gpu(positions, "positions", torch.int32),
              _gpu(block_table, "block_table", torch.int32), block_table.shape[1], page_size, count,
              num_heads, num_kv_heads, head_dim, value_dim, float(scale), int(window or 0),
              int(keep_first or 0) if window else 0, 1 if sink else 0, int(chunk or 0), float(out_scale),
              _opt(sink_values, "sink_values", torch.float32), gate_pointer, gate_stride, _stream()), "attention")


# ----------------------------------------------------------------------------------------
_argmax_scratch = {}


def argmax(logits: torch.Tensor, tokens: torch.Tensor, status: Optional[torch.Tensor] = None) -> None:
    """tokens[r] = index of the best finite logit of row r, ties to the lowest index."""
    fn = _function("sampling", "vipera_argmax", [_c_void, _c_int, _c_int, _c_void, _c_void, _c_void, _c_void])
    rows, vocab = logits.shape
    scratch = _argmax_scratch.get(str(logits.device))
    if scratch is None or scratch.numel() < 64 * rows:
        scratch = torch.empty(64 * max(rows, 256), dtype=torch.int32, device=logits.device)
        _argmax_scratch[str(logits.device)] = scratch
    _check(fn(_gpu(logits, "logits", torch.float32), rows, vocab, _gpu(tokens, "tokens", torch.int32),
              _opt(status, "status", torch.int32), scratch.data_ptr(), _stream()), "argmax", kernels=2)


def sample(logits: torch.Tensor, *, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           min_p: torch.Tensor, uniform: torch.Tensor, tokens: torch.Tensor, status: torch.Tensor) -> None:
    fn = _function("sampling", "vipera_sample",
                   [_c_void, _c_int, _c_int, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void])
    rows, vocab = logits.shape
    _check(fn(_gpu(logits, "logits", torch.float32), rows, vocab,
              _gpu(temperature, "temperature", torch.float32), _gpu(top_k, "top_k", torch.int32),
              _gpu(top_p, "top_p", torch.float32), _gpu(min_p, "min_p", torch.float32),
              _gpu(uniform, "uniform", torch.float64), _gpu(tokens, "tokens", torch.int32),
              _gpu(status, "status", torch.int32), _stream()), "sample")


def logprobs(logits: torch.Tensor, rows: torch.Tensor, tokens: torch.Tensor, temperature: torch.Tensor, top_n: int):
    """Log-probabilities of ``tokens[i]`` in row ``rows[i]`` of ``logits`` at ``temperature[i]``
    (0: as 1), and the ``top_n`` most likely ids of each row with theirs.  Returns device tensors
    (chosen [n], top ids [n, top_n], top values [n, top_n])."""
    fn = _function("sampling", "vipera_logprobs",
                   [_c_void, _c_int, _c_int, _c_void, _c_void, _c_void, _c_int, _c_void, _c_void, _c_void, _c_void])
    count = rows.numel()
    chosen = torch.empty(count, dtype=torch.float32, device=logits.device)
    top_ids = torch.empty((count, max(top_n, 1)), dtype=torch.int32, device=logits.device)
    top_values = torch.empty((count, max(top_n, 1)), dtype=torch.float32, device=logits.device)
    _check(fn(_gpu(logits, "logits", torch.float32), logits.shape[1], count, _gpu(rows, "rows", torch.int32),
              _gpu(tokens, "tokens", torch.int32), _gpu(temperature, "temperature", torch.float32), int(top_n),
              chosen.data_ptr(), top_ids.data_ptr(), top_values.data_ptr(), _stream()), "logprobs")
    return chosen, top_ids[:, :top_n], top_values[:, :top_n]


def apply_penalties(logits: torch.Tensor, *, entry_row, entry_id, entry_count, entry_bias,
                    repetition, presence, frequency) -> None:
    fn = _function("sampling", "vipera_apply_penalties",
                   [_c_void, _c_int, _c_int, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void])
    _check(fn(_gpu(logits, "logits", torch.float32), logits.shape[1], entry_row.numel(),
              _gpu(entry_row, "entry_row", torch.int32), _gpu(entry_id, "entry_id", torch.int32),
              _gpu(entry_count, "entry_count", torch.int32), _gpu(entry_bias, "entry_bias", torch.float32),
              _gpu(repetition, "repetition", torch.float32), _gpu(presence, "presence", torch.float32),
              _gpu(frequency, "frequency", torch.float32), _stream()), "apply_penalties")


# ----------------------------------------------------------------------------------------
# tensor-core products
# ----------------------------------------------------------------------------------------
_tc_state = {}
buffer_generation = 0  # goes up whenever a shared kernel buffer moves; captured graphs are then stale


SAMPLER_MAX_ROWS = 4096
SAMPLER_MAX_TOP_K = 4096  # the largest top-k the device sampler draws without the host (kMaxCandidates in sampling.cu)
_WORDS_HEAD = 8  # int32 words in front of the sampler's outputs; the first is the kernel status word


def _tc_buffers(device, scratch_bytes: int):
    """Scratch for the partial sums of split products and the status word of the kernels with
    bounded waits, per device.  The scratch grows on demand and is shared by all products,
    which run one after another on one stream.  The status word is the first word of a small
    buffer that also receives the sampler's token ids and row states, so that one copy to the
    host brings all three."""
    global buffer_generation
    state = _tc_state.setdefault(str(device), {"scratch": None, "status": None, "words": None})
    if state["status"] is None:
        state["words"] = torch.zeros(_WORDS_HEAD + 2 * SAMPLER_MAX_ROWS, dtype=torch.int32, device=device)
        state["status"] = state["words"][:1]
    if scratch_bytes and (state["scratch"] is None or state["scratch"].numel() * 4 < scratch_bytes):
        state["scratch"] = torch.empty(max(scratch_bytes // 4, 8 << 20), dtype=torch.float32, device=device)
        buffer_generation += 1
    return state


def sampler_words(device, rows: int):
    """(whole, tokens, states): int32 device views for `rows` sampled rows, laid out so that
    ``whole`` (the status word's neighbourhood, then tokens, then row states) is one
    contiguous copy."""
    words = _tc_buffers(device, 0)["words"]
    return (words[:_WORDS_HEAD + 2 * rows], words[_WORDS_HEAD:_WORDS_HEAD + rows],
            words[_WORDS_HEAD + rows:_WORDS_HEAD + 2 * rows])


def raise_on_kernel_status(device, code: int) -> None:
    """`code` is the status word as just read: non-zero means a bounded wait ran out."""
    if code:
        _tc_buffers(device, 0)["status"].zero_()
        _function("gemm_tc", "vipera_gemm_tc_reset", [_c_void])(_stream())
        raise InternalError(f"a tensor-core kernel gave up waiting (code {code}); the step's results are invalid")


_workspace_sizes = {}


def gemm_tc_workspace(m: int, n: int, k: int):
    size = _workspace_sizes.get((m, n, k))
    if size is None:
        fn = _function("gemm_tc", "vipera_gemm_tc_workspace",
                       [_c_int, _c_int, _c_int, ctypes.POINTER(ctypes.c_size_t)])
        scratch = ctypes.c_size_t(0)
        _check(fn(m, n, k, ctypes.byref(scratch)), "gemm_tc_workspace", kernels=0)
        if len(_workspace_sizes) > 65536:
            _workspace_sizes.clear()
        size = _workspace_sizes[(m, n, k)] = scratch.value
    return size


def _even_ok(n: int, epilogue: int, out) -> bool:
    return n % 4 == 0 and (epilogue == EPI_RESIDUAL or
                           (epilogue == EPI_STORE and out is not None and out.dtype == torch.float32))


_plans = {}


def gemm_tc_plan(m: int, n: int, k: int, epilogue: int = EPI_STORE, even_ok: bool = False):
    """The form the tensor-core product takes for these sizes: a dict with `swapped`, `tile`,
    `splits`, `even_shares` (equal shares of all k-blocks per block instead of whole tiles) and
    `blocks`.  `even_ok`: the ending is one that can take other blocks' partial sums (float32
    output or the residual stream, rows a multiple of 16 bytes)."""
    key = (int(m), int(n), int(k), int(epilogue), bool(even_ok), _even_shares_mode[0])
    plan = _plans.get(key)
    if plan is None:
        fn = _function("gemm_tc", "vipera_gemm_tc_plan", [_c_int] * 5 + [ctypes.POINTER(_c_int)])
        form = (_c_int * 6)()
        _check(fn(key[0], key[1], key[2], key[3], int(key[4]), form), "gemm_tc_plan", kernels=0)
        if len(_plans) > 65536:
            _plans.clear()
        plan = _plans[key] = {"swapped": bool(form[0]), "tile": form[1], "splits": form[2],
                              "even_shares": bool(form[3]), "blocks": form[4], "pairs": bool(form[5])}
    return plan


_even_shares_mode = [None]


def gemm_tc_even_shares(mode: int) -> int:
    """Sets when the product takes even shares (0 never, 1 where its estimate favours them, 2
    wherever the ending allows) and returns the mode before; -1 only asks."""
    before = _function("gemm_tc", "vipera_gemm_tc_even_shares", [_c_int])(int(mode))
    if mode >= 0:
        _even_shares_mode[0] = (_even_shares_mode[0], "even", int(mode))
        _workspace_sizes.clear()
    return before


def gemm_tc_pairs(mode: int) -> int:
    """Sets when the product runs on pairs of blocks that share tiles of 256 tokens (0 never, 1
    where its estimate favours them, 2 wherever the form allows) and returns the mode before; -1
    only asks."""
    before = _function("gemm_tc", "vipera_gemm_tc_pairs", [_c_int])(int(mode))
    if mode >= 0:
        _even_shares_mode[0] = (_even_shares_mode[0], "pairs", int(mode))   # a new key for the kept plans
        _workspace_sizes.clear()
    return before


def gemm_tc(a: torch.Tensor, w: torch.Tensor, *, epilogue: int = EPI_STORE,
            bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
            resid: Optional[torch.Tensor] = None, activation: int = ACT_SILU) -> None:
    """a[M, K] times w[N, K] transposed in bfloat16 on the tensor cores (tcgen05, TMA).  ``bias``
    counts in every ending (for the gated unit it is interleaved like the rows); ``activation``
    is the gated unit's."""
    fn = _function("gemm_tc", "vipera_gemm_tc_act",
                   [_c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_void, _c_void, _c_int, _c_void, _c_int, _c_void,
                    ctypes.c_size_t, _c_void, _c_void])
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise InvalidArgumentError(f"gemm: inner sizes differ ({k} and {w.shape[1]})")
    if k % 8:
        raise UnsupportedError(f"gemm_tc: inner size {k} is not a multiple of 8")
    _check_gemm_outputs(m, n, epilogue, bias, out, resid)
    scratch_bytes = gemm_tc_workspace(m, n, k)
    state = _tc_buffers(a.device, scratch_bytes)
    scratch = state["scratch"]
    _check(fn(_gpu(a, "a", torch.bfloat16), _gpu(w, "w", torch.bfloat16), m, n, k, epilogue,
              _opt(bias, "bias", torch.float32), _opt(out, "out"),
              dtype_code(out.dtype) if out is not None else F32, _opt(resid, "resid", torch.float32),
              int(activation), None if scratch is None else scratch.data_ptr(),
              0 if scratch is None else scratch.numel() * 4,
              state["status"].data_ptr(), _stream()), "gemm_tc",
           kernels=2 if scratch_bytes and gemm_tc_plan(m, n, k, epilogue, _even_ok(n, epilogue, out))["splits"] > 1 else 1)


class _GemmRope(ctypes.Structure):
    _fields_ = [
        ("positions", _c_void), ("token_entry", _c_void), ("block_table", _c_void), ("cos_table", _c_void),
        ("sin_table", _c_void), ("q_out", _c_void), ("k_pool", _c_void), ("v_pool", _c_void),
        ("table_width", _c_int), ("page_size", _c_int), ("num_heads", _c_int), ("num_kv_heads", _c_int),
        ("head_dim", _c_int), ("rope_style", _c_int), ("write_cache", _c_int),
    ]


_rope_takes = {}


def gemm_tc_rope_takes(tokens: int, n: int, k: int, head_dim: int) -> bool:
    """Whether the tensor-core product can end with rotation and cache write for these sizes."""
    key = (int(tokens), int(n), int(k), int(head_dim))
    known = _rope_takes.get(key)
    if known is None:
        fn = _function("gemm_tc", "vipera_gemm_tc_rope_takes", [_c_int] * 4)
        if len(_rope_takes) > 65536:
            _rope_takes.clear()
        known = _rope_takes[key] = bool(fn(*key))
    return known


def gemm_tc_rope(a: torch.Tensor, w: torch.Tensor, *, bias: Optional[torch.Tensor], q_out: torch.Tensor,
                 num_heads: int, num_kv_heads: int, head_dim: int, positions: torch.Tensor,
                 cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], style: int, k_pool: torch.Tensor,
                 v_pool: torch.Tensor, token_entry: torch.Tensor, block_table: torch.Tensor, page_size: int,
                 write_cache: bool) -> None:
    """The q/k/v product of a step on the tensor cores with bias, rotation of q and k and the
    write of keys and values into their pages as its ending (bfloat16; from 192 tokens on in the
    product kernel itself, below that in the kernel that adds the partial sums of the cut K)."""
    size = _function("gemm_tc", "vipera_gemm_tc_rope_size", [])()
    if size != ctypes.sizeof(_GemmRope):
        raise InternalError("the q/k/v ending's structure differs from its Python mirror")
    fn = _function("gemm_tc", "vipera_gemm_tc_rope",
                   [_c_void, _c_void, _c_int, _c_int, _c_int, _c_void, ctypes.POINTER(_GemmRope), _c_void,
                    ctypes.c_size_t, _c_void, _c_void])
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or n != (num_heads + 2 * num_kv_heads) * head_dim:
        raise InvalidArgumentError("gemm_tc_rope: the matrix must be [(heads + 2 kv_heads) * d, K]")
    if tuple(q_out.shape) != (m, num_heads * head_dim):
        raise InvalidArgumentError("gemm_tc_rope: q_out must be [tokens, heads * d]")
    if style not in (ROPE_NONE, ROPE_NEOX):
        raise UnsupportedError("gemm_tc_rope: rotary styles none and neox")
    r = _GemmRope()
    r.positions = _gpu(positions, "positions", torch.int32)
    r.token_entry = _gpu(token_entry, "token_entry", torch.int32)
    r.block_table = _gpu(block_table, "block_table", torch.int32)
    r.cos_table = _opt(cos, "cos", torch.float32)
    r.sin_table = _opt(sin, "sin", torch.float32)
    r.q_out = _gpu(q_out, "q_out", torch.bfloat16)
    r.k_pool = _gpu(k_pool, "k_pool", torch.bfloat16)
    r.v_pool = _gpu(v_pool, "v_pool", torch.bfloat16)
    r.table_width, r.page_size = int(block_table.shape[1]), int(page_size)
    r.num_heads, r.num_kv_heads, r.head_dim = int(num_heads), int(num_kv_heads), int(head_dim)
    r.rope_style, r.write_cache = int(style), 1 if write_cache else 0
    # (fewer than 192 tokens: K is cut, and the kernel that adds the partial sums has the ending)
    scratch_bytes = gemm_tc_workspace(m, n, k)
    state = _tc_buffers(a.device, scratch_bytes)
    scratch = state["scratch"]
    _check(fn(_gpu(a, "a", torch.bfloat16), _gpu(w, "w", torch.bfloat16), m, n, k, _opt(bias, "bias", torch.float32),
              ctypes.byref(r), None if scratch is None else scratch.data_ptr(),
              0 if scratch is None else scratch.numel() * 4, state["status"].data_ptr(), _stream()), "gemm_tc_rope",
           kernels=2 if m < 192 else 1)


def wait_probe(device, limit: int = 4096) -> None:
    """Launch a block whose bounded wait runs out after `limit` polls (on a barrier nothing
    arrives at, with no copy in flight): the status word then holds what a product kernel
    writes when one of its waits gives up.  For testing how that is reported."""
    fn = _function("gemm_tc", "vipera_gemm_tc_wait_probe", [_c_void, _c_int, _c_void])
    _check(fn(kernel_status_word(device).data_ptr(), int(limit), _stream()), "wait_probe")


def check_kernel_status(device) -> None:
    """After a synchronisation: raise if a tensor-core kernel's bounded wait ran out."""
    state = _tc_state.get(str(device))
    if state is None or state["status"] is None:
        return
    raise_on_kernel_status(device, int(state["status"].item()))


# ----------------------------------------------------------------------------------------
# bfloat16 attention on the tensor cores
# ----------------------------------------------------------------------------------------
MMA_HEAD_DIMS = (64, 128)
TC_ATTENTION_HEAD_DIMS = (64, 128)


def _gate_pointer(gate: Optional[torch.Tensor], gate_offset: int, rows: int, width: int, what: str):
    """(address of the first gate value, floats between rows) of a float32 [rows, >= offset + width] tensor."""
    if gate is None:
        return None, 0
    if gate.dim() != 2 or gate.shape[0] != rows or gate.stride(1) != 1 or not 0 <= gate_offset <= gate.shape[1] - width:
        raise InvalidArgumentError(f"{what}: the gate must hold heads * value size values per token")
    return _gpu(gate, "gate", torch.float32) + 4 * int(gate_offset), int(gate.stride(0))


def attention_tc_takes_gate(gate: Optional[torch.Tensor], gate_offset: int) -> bool:
    """The tensor-core ending reads the gate four values at a time."""
    return gate is None or (gate_offset % 4 == 0 and gate.stride(0) % 4 == 0 and gate.data_ptr() % 16 == 0)


def attention_prefill(q: torch.Tensor, out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, *,
                      entry_starts: torch.Tensor, entry_pos0: torch.Tensor, block_table: torch.Tensor,
                      num_entries: int, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                      window: int = 0, skip_single: bool = False, keep_first: int = 0, sink: bool = False,
                      mask_chunk: int = 0, sink_values: Optional[torch.Tensor] = None,
                      gate: Optional[torch.Tensor] = None, gate_offset: int = 0) -> None:
    """Flash-style attention of a step whose entries bring any number of tokens (bfloat16,
    head sizes 64 and 128), on tcgen05 with accumulators in tensor memory
    (VIPERA_ATTENTION_TC=0 keeps it on the mma.sync kernel).
    ``skip_single`` leaves entries of one token out: attention_decode with ``entry_starts`` runs them.
    ``keep_first`` (with a window: that many first keys stay visible) and ``sink`` (one added to the
    softmax's denominator) are served by the mma.sync kernel, and so is ``mask_chunk`` (instead of
    a window: a query sees the earlier keys of its own chunk of that many positions; the kernels
    take it as a negative window).  ``sink_values`` float32 [heads] (a learned sink: exp(sink_h) joins
    head h's denominator) and ``gate`` (float32 [tokens, width]: the output is multiplied by the sigmoid
    of the heads * d values from column ``gate_offset`` on) are served by the tcgen05 kernel's ending,
    with a plain window only."""
    if mask_chunk:
        if window:
            raise InvalidArgumentError("attention_prefill: a mask is a window or chunks, not both")
        window = -int(mask_chunk)
    if head_dim not in MMA_HEAD_DIMS:
        raise UnsupportedError(f"attention_prefill: head size {head_dim} (built: 64, 128)")
    count = q.shape[0]
    if q.shape[1] != num_heads * head_dim or out.shape != q.shape:
        raise InvalidArgumentError("attention_prefill: q and out must be [tokens, heads * d]")
    if k_pool.shape[2:] != (num_kv_heads, head_dim) or v_pool.shape != k_pool.shape:
        raise InvalidArgumentError("attention_prefill: cache pools must be [pages, page_size, kv_heads, d]")
    pointers = (_gpu(q, "q", torch.bfloat16), _gpu(out, "out", torch.bfloat16), _gpu(k_pool, "k_pool", torch.bfloat16),
                _gpu(v_pool, "v_pool", torch.bfloat16), _gpu(entry_starts, "entry_starts", torch.int32),
                _gpu(entry_pos0, "entry_pos0", torch.int32), _gpu(block_table, "block_table", torch.int32))
    sizes = (block_table.shape[1], k_pool.shape[1], num_entries, count, num_heads, num_kv_heads, head_dim,
             float(scale), int(window or 0))
    kinds = [_c_void] * 7 + [_c_int] * 7 + [_c_float, _c_int]
    skip = 1 if skip_single else 0
    keep_first = int(keep_first or 0) if window > 0 else 0
    if sink_values is not None or gate is not None:
        if keep_first or window < 0 or (sink and sink_values is None) or not attention_tc_takes_gate(gate, gate_offset):
            raise UnsupportedError("attention_prefill: a learned sink and an output gate come with a plain window only")
        if sink_values is not None and sink_values.numel() != num_heads:
            raise InvalidArgumentError("attention_prefill: one sink score per query head")
        gate_pointer, gate_stride = _gate_pointer(gate, gate_offset, count, num_heads * head_dim, "attention_prefill")
        fn = _function("attention_tc", "vipera_attention_prefill_tc_gated",
                       kinds + [_c_int, _c_int, _c_void, _c_void, ctypes.c_longlong, _c_void, _c_void])
        _check(fn(*pointers, *sizes, k_pool.shape[0], skip, _opt(sink_values, "sink_values", torch.float32), gate_pointer,
                  gate_stride, kernel_status_word(q.device).data_ptr(), _stream()), "attention_prefill_tc")
        return
    if keep_first or sink:
        fn = _function("attention_mma", "vipera_attention_prefill_kept", kinds + [_c_int, _c_int, _c_int, _c_void])
        _check(fn(*pointers, *sizes, skip, keep_first, 1 if sink else 0, _stream()), "attention_prefill")
        return
    if head_dim in TC_ATTENTION_HEAD_DIMS and window >= 0 and os.environ.get("VIPERA_ATTENTION_TC", "1") != "0":
        fn = _function("attention_tc", "vipera_attention_prefill_tc", kinds + [_c_int, _c_int, _c_void, _c_void])
        _check(fn(*pointers, *sizes, k_pool.shape[0], skip, kernel_status_word(q.device).data_ptr(), _stream()),
               "attention_prefill_tc")
        return
    fn = _function("attention_mma", "vipera_attention_prefill", kinds + [_c_int, _c_void])
    _check(fn(*pointers, *sizes, skip, _stream()), "attention_prefill")


# The split-key kernel's blocks that an SM holds at once (its launch bounds and shared memory).
DECODE_BLOCKS_PER_SM = 3
# The cut by whole waves serves steps whose longest history is above DECODE_SHORT_HISTORY keys and
# whose histories hold at least DECODE_LONG_WORK rows of keys per layer (entries x KV heads x keys):
# launches of some 30 microseconds and more.
DECODE_SHORT_HISTORY = 4096
DECODE_LONG_WORK = 1 << 18


@functools.lru_cache(maxsize=4096)
def decode_splits(num_entries: int, num_kv_heads: int, max_keys: int, sm_count: int):
    """How a decode step's keys are cut: (keys per split, splits).  A block is an (entry, KV
    head, split) and folds its split 128 keys at a time, 32 for each of its four warps.

    Short launches: a split is 128 keys, so that every block asks for all its keys at once,
    before it waits for the kernel ahead, and the whole cache of the step is in flight together;
    only when that would make more than 64 splits, or more than sixteen blocks per SM, do splits
    grow.  Long histories of many entries: the kernel runs for tens of microseconds and what
    counts is that its blocks fill whole waves (the GPU holds three blocks an SM at once; 512 blocks take as long
    as 888, measured), so the cut is the one a small model of the launch's time likes best: per
    wave a fixed cost and a cost per 128 keys, which is the memory's when the wave is full and a
    block's own latency when it is not; the constants are fitted to launches timed at batch 1 to
    64 and 8,192 to 32,768 keys."""
    base = max(1, num_entries * num_kv_heads)
    if max_keys <= DECODE_SHORT_HISTORY or base * max_keys < DECODE_LONG_WORK:
        # For the next power of two of keys, the splits past the longest history included (their
        # blocks leave at once): measured, the step at batch 8 and 8,192 keys is 0.1 ms faster
        # with these 64 splits than with the 36 of the same size that hold keys.
        bound = 128
        while bound < max_keys:
            bound *= 2
        most = max(1, min(64, (16 * sm_count) // base))
        chunk = max(128, -(-bound // most))
        chunk = -(-chunk // 128) * 128
        return chunk, max(1, -(-bound // chunk))
    slots = DECODE_BLOCKS_PER_SM * max(1, sm_count)
    fixed, per_tile_full, per_tile_alone, combine, per_split = 2.7, 3.7, 2.75, 3.0, 0.02   # microseconds
    best = None
    seen = set()
    for wanted in range(1, 65):
        chunk = -(-(-(-max_keys // wanted)) // 128) * 128
        if chunk in seen:
            continue
        seen.add(chunk)
        splits = max(1, -(-max_keys // chunk))
        tiles = chunk / 128
        full, rest = divmod(base * splits, slots)
        time = full * (fixed + tiles * per_tile_full)
        if rest:
            time += fixed + tiles * max(per_tile_full * rest / slots, per_tile_alone)
        time += combine + per_split * splits
        if best is None or time < best[0] - 1e-9:
            best = (time, chunk, splits)
    return best[1], best[2]


def attention_decode(q: torch.Tensor, out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, *,
                     positions: torch.Tensor, block_table: torch.Tensor, num_heads: int, num_kv_heads: int,
                     head_dim: int, scale: float, window: int, chunk: int, num_splits: int,
                     scratch: torch.Tensor, entry_starts: Optional[torch.Tensor] = None, keep_first: int = 0,
                     sink: bool = False, mask_chunk: int = 0, sink_values: Optional[torch.Tensor] = None,
                     gate: Optional[torch.Tensor] = None, gate_offset: int = 0) -> None:
    """Split-key attention of the entries that bring one token (bfloat16, head sizes 64 and
    128); the partial results of the splits are combined by a second kernel.  Without
    ``entry_starts`` every entry brings one token (q and out are [entries, heads * d], positions
    one per entry).  With ``entry_starts`` [entries + 1] the step has portions too: q and out
    are [tokens, heads * d], ``positions`` holds each entry's first position, and entries of
    more than one token are skipped (attention_prefill with ``skip_single`` runs them).
    ``keep_first`` (with a window: that many first keys stay visible; they are one more split, so
    the scratch is sized for ``num_splits + 1``) and ``sink`` (one added to the softmax's denominator).
    ``mask_chunk``: instead of a window, chunks of that many positions (passed on as a negative window).
    ``sink_values`` float32 [heads]: a learned sink per query head; ``gate`` float32 [rows of q, width]: the
    output is multiplied by the sigmoid of the heads * d values from column ``gate_offset`` on."""
    if mask_chunk:
        if window:
            raise InvalidArgumentError("attention_decode: a mask is a window or chunks, not both")
        window = -int(mask_chunk)
    fn = _function("attention_mma", "vipera_attention_decode_gated",
                   [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int,
                    _c_int, _c_float, _c_int, _c_int, _c_int, _c_void, ctypes.c_size_t, _c_void, _c_int, _c_int,
                    _c_void, _c_void, ctypes.c_longlong, _c_void])
    if sink_values is not None and sink_values.numel() != num_heads:
        raise InvalidArgumentError("attention_decode: one sink score per query head")
    gate_pointer, gate_stride = _gate_pointer(gate, gate_offset, q.shape[0], num_heads * head_dim, "attention_decode")
    if head_dim not in MMA_HEAD_DIMS:
        raise UnsupportedError(f"attention_decode: head size {head_dim} (built: 64, 128)")
    count = block_table.shape[0]
    if q.shape[1] != num_heads * head_dim or out.shape != q.shape:
        raise InvalidArgumentError("attention_decode: q and out must be [rows, heads * d]")
    if k_pool.shape[2:] != (num_kv_heads, head_dim) or v_pool.shape != k_pool.shape:
        raise InvalidArgumentError("attention_decode: cache pools must be [pages, page_size, kv_heads, d]")
    if positions.numel() != count or (entry_starts is None and q.shape[0] != count):
        raise InvalidArgumentError("attention_decode: one position and one block table row per entry")
    if entry_starts is not None and entry_starts.numel() != count + 1:
        raise InvalidArgumentError("attention_decode: entry_starts must hold one more item than there are entries")
    _check(fn(_gpu(q, "q", torch.bfloat16), _gpu(out, "out", torch.bfloat16), _gpu(k_pool, "k_pool", torch.bfloat16),
              _gpu(v_pool, "v_pool", torch.bfloat16), _gpu(positions, "positions", torch.int32),
              _gpu(block_table, "block_table", torch.int32), block_table.shape[1], k_pool.shape[1], count,
              num_heads, num_kv_heads, head_dim, float(scale), int(window or 0), int(chunk), int(num_splits),
              _gpu(scratch, "scratch", torch.float32), scratch.numel(), _opt(entry_starts, "entry_starts", torch.int32),
              int(keep_first or 0) if window > 0 else 0, 1 if sink else 0, _opt(sink_values, "sink_values", torch.float32),
              gate_pointer, gate_stride, _stream()), "attention_decode", kernels=2)


def attention_decode_scratch_floats(num_entries: int, num_heads: int, head_dim: int, num_splits: int) -> int:
    rows = num_entries * num_heads * num_splits
    return (2 * rows + 3) // 4 * 4 + rows * head_dim


# ----------------------------------------------------------------------------------------
# products for at most 8 tokens, with the norm in front and the ending behind fused in
# ----------------------------------------------------------------------------------------
GEMV_MAX_TOKENS = 32
GEMV_STORE, GEMV_RESIDUAL, GEMV_SWIGLU, GEMV_ROPE_CACHE = 0, 1, 2, 3


def gemv_small_takes(tokens: int, k: int, n: int) -> bool:
    """Whether the small-token kernel takes `tokens` tokens against a matrix of `n` rows and
    inner size `k` (the activations a block stages must fit in its shared memory)."""
    fn = getattr(load_kernel_library("gemv_small"), "vipera_gemv_small_takes")
    fn.argtypes, fn.restype = [_c_int, _c_int, _c_int], _c_int
    return bool(fn(int(tokens), int(k), int(n)))


class _GemvParams(ctypes.Structure):
    _fields_ = [
        ("weight", _c_void), ("N", _c_int), ("K", _c_int), ("T", _c_int),
        ("x32", _c_void), ("norm_weight", _c_void), ("eps", _c_float), ("rows", _c_void), ("a16", _c_void),
        ("epilogue", _c_int), ("bias", _c_void), ("out", _c_void), ("out_dtype", _c_int), ("resid", _c_void),
        ("num_heads", _c_int), ("num_kv_heads", _c_int), ("head_dim", _c_int), ("rope_style", _c_int),
        ("positions", _c_void), ("cos_table", _c_void), ("sin_table", _c_void), ("q_out", _c_void),
        ("k_pool", _c_void), ("v_pool", _c_void), ("token_entry", _c_void), ("block_table", _c_void),
        ("table_width", _c_int), ("page_size", _c_int), ("write_cache", _c_int), ("activation", _c_int),
    ]


_gemv_checked = False


def gemv_small(w: torch.Tensor, *, a: Optional[torch.Tensor] = None, x: Optional[torch.Tensor] = None,
               norm_weight: Optional[torch.Tensor] = None, eps: float = 0.0, rows: Optional[torch.Tensor] = None,
               tokens: Optional[int] = None, epilogue: int = GEMV_STORE, bias: Optional[torch.Tensor] = None,
               out: Optional[torch.Tensor] = None, resid: Optional[torch.Tensor] = None, rope: Optional[dict] = None,
               activation: int = ACT_SILU) -> None:
    """w[N, K] (bfloat16) times at most 32 tokens.  The input is either ``a`` (bfloat16 [T, K])
    or the float32 residual stream ``x`` with an RMSNorm (``norm_weight``, ``eps``, optional
    ``rows`` choosing which rows of x are the tokens) computed on the way.  ``rope`` holds
    the arguments of the rotary/cache ending (see GQAttention)."""
    global _gemv_checked
    fn = _function("gemv_small", "vipera_gemv_small", [ctypes.POINTER(_GemvParams), _c_void])
    if not _gemv_checked:
        size = _function("gemv_small", "vipera_gemv_params_size", [])()
        if size != ctypes.sizeof(_GemvParams):
            raise InternalError(f"gemv_small: parameter block is {ctypes.sizeof(_GemvParams)} bytes here, {size} in the kernel")
        _gemv_checked = True
    n, k = w.shape
    p = _GemvParams()
    p.weight, p.N, p.K = _gpu(w, "w", torch.bfloat16), n, k
    if (a is None) == (x is None):
        raise InvalidArgumentError("gemv_small: give either a or x")
    if a is not None:
        if a.shape[1] != k:
            raise InvalidArgumentError("gemv_small: inner sizes differ")
        p.a16, p.T = _gpu(a, "a", torch.bfloat16), a.shape[0]
    else:
        if x.shape[1] != k or norm_weight is None or norm_weight.numel() != k:
            raise InvalidArgumentError("gemv_small: x and norm_weight must have the weight's inner size")
        p.x32, p.norm_weight, p.eps = _gpu(x, "x", torch.float32), _gpu(norm_weight, "norm_weight", torch.float32), float(eps)
        p.rows = _opt(rows, "rows", torch.int32)
        p.T = int(tokens if tokens is not None else (rows.numel() if rows is not None else x.shape[0]))
    t = p.T
    if not gemv_small_takes(t, k, n):
        raise UnsupportedError(f"gemv_small does not take {t} tokens against an inner size of {k}")
    p.epilogue = epilogue
    if epilogue == GEMV_ROPE_CACHE:
        r = rope
        p.bias = _opt(bias, "bias", torch.float32)
        p.num_heads, p.num_kv_heads, p.head_dim, p.rope_style = r["num_heads"], r["num_kv_heads"], r["head_dim"], r["style"]
        p.positions = _gpu(r["positions"], "positions", torch.int32)
        p.cos_table, p.sin_table = _opt(r["cos"], "cos", torch.float32), _opt(r["sin"], "sin", torch.float32)
        q_out = r["q_out"]
        if tuple(q_out.shape) != (t, r["num_heads"] * r["head_dim"]):
            raise InvalidArgumentError("gemv_small: q_out has the wrong shape")
        p.q_out = _gpu(q_out, "q_out", torch.bfloat16)
        p.write_cache = 1 if r["write_cache"] else 0
        if r["write_cache"]:
            p.k_pool, p.v_pool = _gpu(r["k_pool"], "k_pool", torch.bfloat16), _gpu(r["v_pool"], "v_pool", torch.bfloat16)
            p.token_entry = _gpu(r["token_entry"], "token_entry", torch.int32)
            p.block_table = _gpu(r["block_table"], "block_table", torch.int32)
            p.table_width, p.page_size = r["block_table"].shape[1], r["page_size"]
    else:
        _check_gemm_outputs(t, n, epilogue, bias, out, resid)
        p.bias = _opt(bias, "bias", torch.float32)
        p.activation = int(activation)
        p.out = _opt(out, "out")
        p.out_dtype = dtype_code(out.dtype) if out is not None else F32
        p.resid = _opt(resid, "resid", torch.float32)
    _check(fn(ctypes.byref(p), _stream()), "gemv_small")


# ----------------------------------------------------------------------------------------
# the matrix-memory cell (mLSTM)
# ----------------------------------------------------------------------------------------
class _MlstmParams(ctypes.Structure):
    _fields_ = [
        ("proj", _c_void), ("proj_width", _c_int),
        ("q_off", _c_int), ("k_off", _c_int), ("v_off", _c_int), ("g_off", _c_int), ("i_off", _c_int), ("f_off", _c_int),
        ("heads", _c_int), ("dim", _c_int), ("vdim", _c_int), ("tile", _c_int), ("num_entries", _c_int),
        ("q_scale", _c_float), ("gate_cap", _c_float), ("denom_eps", _c_float),
        ("entry_starts", _c_void), ("state_slots", _c_void), ("fresh", _c_void), ("state", _c_void),
        ("state_stride", ctypes.c_longlong), ("o_raw", _c_void), ("nm_scratch", _c_void),
        ("chunk_state", _c_void), ("chunk_n", _c_void), ("chunk_aux", _c_void), ("max_jobs", _c_int),
    ]


_mlstm_checked = False


def mlstm_state_floats(heads: int, dim: int, vdim: int) -> int:
    """Floats of one request's state row: S [heads, d, dv], n [heads, d], m [heads], rounded up
    to a multiple of four (the same rule as the kernel file's)."""
    return (heads * (dim * vdim + dim + 1) + 3) // 4 * 4


MLSTM_CHUNK = 64   # tokens of a chunk in the tensor-core form (kTcChunk in mlstm.cu)


def mlstm_tc_takes(dim: int, vdim: int) -> bool:
    """Whether the tensor-core form of the cell's portions takes these sizes."""
    return dim in (64, 128, 256)


def mlstm_takes(dim: int, vdim: int) -> bool:
    fn = getattr(load_kernel_library("mlstm"), "vipera_mlstm_tile")
    fn.argtypes, fn.restype = [_c_int, _c_int], _c_int
    return fn(int(dim), int(vdim)) > 0


def mlstm(proj: torch.Tensor, *, offsets, heads: int, dim: int, vdim: int, q_scale: float, gate_cap: float,
          denom_eps: float, entry_starts: torch.Tensor, state_slots: torch.Tensor, fresh: torch.Tensor,
          token_entry: torch.Tensor, num_entries: int, single: bool, state: torch.Tensor, o_raw: torch.Tensor,
          nm_scratch: torch.Tensor, norm_weight: torch.Tensor, norm_eps: float, out: torch.Tensor,
          chunk_scratch=None) -> None:
    """The mLSTM cell over a step.  ``proj`` is the float32 product [tokens, width] that holds q, k,
    v, the output gate and the two gates' pre-activations at ``offsets`` (q, k, v, g, i, f);
    ``state`` is [slots, mlstm_state_floats]; ``out`` [tokens, heads * vdim] receives the cell's
    output after the head norm (times ``norm_weight``) and the output gate.  ``single`` promises
    that every entry brings one token.  ``chunk_scratch`` (float32 tensors: states [jobs, heads * d
    * dv], n [jobs, heads * d], aux [jobs, heads * 4], with jobs >= tokens // MLSTM_CHUNK + entries)
    lets a bfloat16 run compute all chunks of the step at once instead of walking each entry's."""
    global _mlstm_checked
    fn = _function("mlstm", "vipera_mlstm",
                   [ctypes.POINTER(_MlstmParams), _c_int, _c_int, _c_int, _c_void, _c_float, _c_void, _c_int, _c_void,
                    _c_void])
    if not _mlstm_checked:
        size = _function("mlstm", "vipera_mlstm_params_size", [])()
        if size != ctypes.sizeof(_MlstmParams):
            raise InternalError(f"mlstm: parameter block is {ctypes.sizeof(_MlstmParams)} bytes here, {size} in the kernel")
        _mlstm_checked = True
    tokens, width = proj.shape
    if tuple(out.shape) != (tokens, heads * vdim):
        raise InvalidArgumentError("mlstm: out must be [tokens, heads * value size]")
    if state.dim() != 2 or state.shape[1] != mlstm_state_floats(heads, dim, vdim):
        raise InvalidArgumentError("mlstm: state rows have the wrong size")
    if o_raw.numel() < tokens * heads * vdim or nm_scratch.numel() < num_entries * heads * (dim + 1):
        raise InvalidArgumentError("mlstm: scratch buffers are too small")
    if norm_weight.numel() != heads * vdim:
        raise InvalidArgumentError("mlstm: the head norm's weight must have heads * value size values")
    p = _MlstmParams()
    p.proj, p.proj_width = _gpu(proj, "proj", torch.float32), width
    p.q_off, p.k_off, p.v_off, p.g_off, p.i_off, p.f_off = (int(x) for x in offsets)
    p.heads, p.dim, p.vdim, p.tile, p.num_entries = heads, dim, vdim, 0, int(num_entries)
    p.q_scale, p.gate_cap, p.denom_eps = float(q_scale), float(gate_cap), float(denom_eps)
    p.entry_starts = _gpu(entry_starts, "entry_starts", torch.int32)
    p.state_slots = _gpu(state_slots, "state_slots", torch.int32)
    p.fresh = _gpu(fresh, "fresh", torch.int32)
    p.state, p.state_stride = _gpu(state, "state", torch.float32), state.shape[1]
    p.o_raw = _gpu(o_raw, "o_raw", torch.float32)
    p.nm_scratch = _gpu(nm_scratch, "nm_scratch", torch.float32)
    if chunk_scratch is not None:
        states, ns, aux = chunk_scratch
        jobs = states.shape[0]
        if jobs < tokens // MLSTM_CHUNK + num_entries or ns.shape[0] < jobs or aux.shape[0] < jobs:
            raise InvalidArgumentError("mlstm: the chunk scratch holds too few chunks for this step")
        if states.shape[1] != heads * dim * vdim or ns.shape[1] != heads * dim or aux.shape[1] != heads * 4:
            raise InvalidArgumentError("mlstm: the chunk scratch has the wrong row sizes")
        p.chunk_state, p.chunk_n = _gpu(states, "chunk states", torch.float32), _gpu(ns, "chunk n", torch.float32)
        p.chunk_aux, p.max_jobs = _gpu(aux, "chunk aux", torch.float32), tokens // MLSTM_CHUNK + num_entries
    # a bfloat16 run's portions go through the tensor-core form where it takes the sizes
    # (VIPERA_MLSTM_TC=0 keeps them on the CUDA cores)
    tensor_cores = out.dtype == torch.bfloat16 and os.environ.get("VIPERA_MLSTM_TC", "1") != "0"
    _check(fn(ctypes.byref(p), tokens, 1 if single else 0, 1 if tensor_cores else 0,
              _gpu(norm_weight, "norm_weight", torch.float32),
              float(norm_eps), _gpu(out, "out"), dtype_code(out.dtype), _gpu(token_entry, "token_entry", torch.int32),
              _stream()), "mlstm", kernels=4 if (chunk_scratch is not None and tensor_cores and not single) else 2)


def kernel_status_word(device) -> torch.Tensor:
    """The device word in which kernels with bounded waits report that one ran out."""
    return _tc_buffers(device, 0)["status"]


# ----------------------------------------------------------------------------------------
# layer norm, short causal convolutions, norm over whole q/k rows
# ----------------------------------------------------------------------------------------
def layernorm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, out: torch.Tensor, eps: float,
              rows: Optional[torch.Tensor] = None, accumulate: bool = False) -> None:
    """out[r, :] = layernorm(x[rows[r], :]) * weight + bias; with ``accumulate`` the float32 ``out``
    receives out + that instead (a normalised sublayer output joining the residual stream)."""
    fn = _function("rowwise", "vipera_layernorm",
                   [_c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_float, _c_int, _c_void])
    hidden = x.shape[1]
    count = out.shape[0]
    if out.shape[1] != hidden or weight.numel() != hidden or bias.numel() != hidden:
        raise InvalidArgumentError("layernorm: widths of x, weight, bias and out do not agree")
    if rows is None and x.shape[0] != count:
        raise InvalidArgumentError("layernorm: x and out have different row counts")
    if rows is not None and rows.numel() != count:
        raise InvalidArgumentError("layernorm: one row index is needed for each output row")
    if accumulate and (out.dtype != torch.float32 or out.data_ptr() == x.data_ptr()):
        raise InvalidArgumentError("layernorm: accumulation needs a float32 target other than the input")
    _check(fn(_gpu(x, "x", torch.float32), _gpu(weight, "weight", torch.float32), _gpu(bias, "bias", torch.float32),
              _opt(rows, "rows", torch.int32), _gpu(out, "out"), dtype_code(out.dtype), count, hidden,
              float(eps), 1 if accumulate else 0, _stream()), "layernorm")


CONV_ACT_NONE, CONV_ACT_SILU = 0, 1
CONV_ACTIVATIONS = {"none": CONV_ACT_NONE, "silu": CONV_ACT_SILU}
CONV_MAX_TAPS = 16


class _ConvParams(ctypes.Structure):
    _fields_ = [
        ("x", _c_void), ("x_stride", ctypes.c_longlong), ("weight", _c_void), ("bias", _c_void),
        ("state", _c_void), ("state_stride", ctypes.c_longlong), ("entry_starts", _c_void), ("token_entry", _c_void),
        ("state_slots", _c_void), ("fresh", _c_void), ("out", _c_void), ("out_f32", _c_void), ("clear", _c_void),
        ("channels", _c_int), ("taps", _c_int), ("num_tokens", _c_int), ("num_entries", _c_int),
        ("add_input", _c_int), ("activation", _c_int), ("segments", _c_int),
    ]


_struct_checked = set()


def _check_struct(library: str, name: str, struct) -> None:
    """The parameter block's size here and in the kernel file must agree."""
    if (library, name) in _struct_checked:
        return
    size = _function(library, name, [])()
    if size != ctypes.sizeof(struct):
        raise InternalError(f"{library}: parameter block is {ctypes.sizeof(struct)} bytes here, {size} in the kernel")
    _struct_checked.add((library, name))


def causal_conv(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], *, channels: int,
                state: Optional[torch.Tensor], entry_starts: torch.Tensor, token_entry: torch.Tensor,
                state_slots: torch.Tensor, fresh: torch.Tensor, num_entries: int, single: bool,
                add_input: bool, activation: int = CONV_ACT_NONE, out: Optional[torch.Tensor] = None,
                out_f32: Optional[torch.Tensor] = None, clear: Optional[torch.Tensor] = None) -> None:
    """A causal convolution over time per channel: ``y_t = act(sum_j w[:, j] x_(t - taps + 1 + j) + b)
    (+ x_t)`` over the first ``channels`` columns of the float32 ``x`` [tokens, >= channels] (rows
    may be strided).  ``state`` [slots, taps - 1, channels] float32 (slots may be strided) holds each
    request's last inputs: read where an entry is not fresh, written at the entry's end.  ``out``
    (any run type) and ``out_f32`` receive y; ``clear`` [tokens, channels] float32 is zeroed."""
    fn = _function("seqconv", "vipera_causal_conv", [ctypes.POINTER(_ConvParams), _c_int, _c_int, _c_void])
    _check_struct("seqconv", "vipera_causal_conv_params_size", _ConvParams)
    tokens = x.shape[0]
    taps = weight.shape[1]
    if weight.shape[0] != channels or x.shape[1] < channels or x.stride(1) != 1 or x.dtype != torch.float32 or not x.is_cuda:
        raise InvalidArgumentError("causal_conv: x must be float32 [tokens, >= channels] with unit inner stride")
    if taps > CONV_MAX_TAPS:
        raise UnsupportedError(f"causal_conv: {taps} taps; the kernel takes up to {CONV_MAX_TAPS}")
    if out is None and out_f32 is None:
        raise InvalidArgumentError("causal_conv: no output")
    for name, tensor in (("out", out), ("out_f32", out_f32), ("clear", clear)):
        if tensor is not None and tuple(tensor.shape) != (tokens, channels):
            raise InvalidArgumentError(f"causal_conv: {name} must be [tokens, channels]")
    p = _ConvParams()
    p.x, p.x_stride = x.data_ptr(), x.stride(0)
    p.weight, p.bias = _gpu(weight, "weight", torch.float32), _opt(bias, "bias", torch.float32)
    if state is not None and taps > 1:
        if tuple(state.shape[1:]) != (taps - 1, channels) or state.dtype != torch.float32 or \
                state.stride(2) != 1 or state.stride(1) != channels:
            raise InvalidArgumentError("causal_conv: state must be float32 [slots, taps - 1, channels]")
        p.state, p.state_stride = state.data_ptr(), state.stride(0)
    elif taps > 1:
        raise InvalidArgumentError("causal_conv: a convolution of several taps needs its state")
    p.entry_starts = _gpu(entry_starts, "entry_starts", torch.int32)
    p.token_entry = _gpu(token_entry, "token_entry", torch.int32)
    p.state_slots = _gpu(state_slots, "state_slots", torch.int32)
    p.fresh = _gpu(fresh, "fresh", torch.int32)
    p.out = _opt(out, "out")
    p.out_f32 = _opt(out_f32, "out_f32", torch.float32)
    p.clear = _opt(clear, "clear", torch.float32)
    p.channels, p.taps, p.num_tokens, p.num_entries = int(channels), int(taps), int(tokens), int(num_entries)
    p.add_input, p.activation = 1 if add_input else 0, int(activation)
    _check(fn(ctypes.byref(p), dtype_code(out.dtype) if out is not None else F32, 1 if single else 0, _stream()),
           "causal_conv")


def qk_prepare(qkv: torch.Tensor, q_out: torch.Tensor, *, num_heads: int, num_kv_heads: int, head_dim: int,
               value_dim: int, rot_dims: int, q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor],
               eps: float, values_from_keys: bool, positions: torch.Tensor, cos: Optional[torch.Tensor],
               sin: Optional[torch.Tensor], style: int, k_pool: torch.Tensor, v_pool: torch.Tensor,
               token_seq: torch.Tensor, block_table: torch.Tensor, page_size: int, write_cache: bool) -> None:
    """As ``rope_cache`` in its general form, with an RMS norm over the whole q row and the whole k
    row (weights ``q_norm`` [heads * d], ``k_norm`` [kv_heads * d]) in front of the rotation, and,
    with ``values_from_keys``, the keys as projected (before norm and rotation) stored as the values:
    the float32 product is then [tokens, (heads + kv_heads) * d]."""
    fn = _function("rope_cache", "vipera_qk_prepare",
                   [_c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void, _c_void, _c_float,
                    _c_int, _c_void, _c_void, _c_void, _c_int, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int,
                    _c_void])
    count = qkv.shape[0]
    width = (num_heads + num_kv_heads) * head_dim + (0 if values_from_keys else num_kv_heads * value_dim)
    if qkv.shape[1] != width:
        raise InvalidArgumentError("qk_prepare: the product's width does not match the head counts and sizes")
    if tuple(q_out.shape) != (count, num_heads * head_dim):
        raise InvalidArgumentError("qk_prepare: q_out has the wrong shape")
    if style == ROPE_NONE:
        rot_dims = 0
    elif cos is None or sin is None or cos.shape[1] != rot_dims // 2 or sin.shape != cos.shape:
        raise InvalidArgumentError("qk_prepare: cos/sin tables of width rot_dims/2 are needed")
    if q_norm is not None and q_norm.numel() != num_heads * head_dim or \
            k_norm is not None and k_norm.numel() != num_kv_heads * head_dim:
        raise InvalidArgumentError("qk_prepare: a norm weight must have one value per value of its row")
    if k_pool.dtype != q_out.dtype or v_pool.dtype != q_out.dtype or \
            k_pool.shape[1:] != (page_size, num_kv_heads, head_dim) or \
            v_pool.shape[1:] != (page_size, num_kv_heads, value_dim):
        raise InvalidArgumentError("qk_prepare: cache pools must be [pages, page_size, kv_heads, d] and "
                                   "[pages, page_size, kv_heads, value size] of the activation dtype")
    _check(fn(_gpu(qkv, "qkv", torch.float32), _gpu(q_out, "q_out"), dtype_code(q_out.dtype), count, num_heads,
              num_kv_heads, head_dim, value_dim, int(rot_dims), _opt(q_norm, "q_norm", torch.float32),
              _opt(k_norm, "k_norm", torch.float32), float(eps), 1 if values_from_keys else 0,
              _gpu(positions, "positions", torch.int32), _opt(cos, "cos", torch.float32), _opt(sin, "sin", torch.float32),
              int(style), _gpu(k_pool, "k_pool"), _gpu(v_pool, "v_pool"), _gpu(token_seq, "token_seq", torch.int32),
              _gpu(block_table, "block_table", torch.int32), block_table.shape[1], int(page_size),
              1 if write_cache else 0, _stream()), "rope_cache")


TALK_MAX_HEADS = 64


@functools.lru_cache(maxsize=4096)
def talk_splits(tokens: int, max_keys: int, sm_count: int):
    """How the keys of attention_talk are cut: (keys per split, splits).  A block is a (token,
    split); steps of many tokens need no cut, steps of few tokens get enough splits for two
    blocks an SM, of at least 64 keys each."""
    wanted = max(1, -(-2 * sm_count // max(tokens, 1)))
    splits = max(1, min(wanted, -(-max(max_keys, 1) // 64)))
    keys = -(-(-(-max(max_keys, 1) // splits)) // 32) * 32
    return keys, max(1, -(-max(max_keys, 1) // keys))


def attention_talk(q: torch.Tensor, out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, mix: torch.Tensor, *,
                   token_seq: torch.Tensor, positions: torch.Tensor, block_table: torch.Tensor, num_heads: int,
                   num_kv_heads: int, head_dim: int, value_dim: int, scale: float, out_scale: float = 1.0,
                   split_keys: int, num_splits: int, stats: torch.Tensor, partial: Optional[torch.Tensor]) -> None:
    """Causal softmax attention whose normalised head weights are mixed by ``mix`` [heads, heads]
    (``w_h = sum_g mix[h, g] p_g``) before head h applies them to the values of its own KV head.
    The keys are cut into ``num_splits`` splits of ``split_keys`` keys (see ``talk_splits``; every
    position of the step must lie below their product); ``stats`` is a float32 scratch of
    2 * tokens * splits * heads values and ``partial`` one of splits * tokens * heads * value_dim
    (needed with more than one split)."""
    fn = _function("attention_talk", "vipera_attention_talk",
                   [_c_void, _c_void, _c_int, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int,
                    _c_int, _c_int, _c_int, _c_int, _c_float, _c_float, _c_int, _c_int, _c_void, _c_void, _c_void])
    count = q.shape[0]
    if num_heads > TALK_MAX_HEADS:
        raise UnsupportedError(f"attention_talk: {num_heads} heads; the kernel takes up to {TALK_MAX_HEADS}")
    if q.shape[1] != num_heads * head_dim or tuple(out.shape) != (count, num_heads * value_dim) or out.dtype != q.dtype:
        raise InvalidArgumentError("attention_talk: q must be [tokens, heads * d] and out [tokens, heads * value size]")
    page_size = k_pool.shape[1]
    if k_pool.dtype != q.dtype or v_pool.dtype != q.dtype or k_pool.shape[2:] != (num_kv_heads, head_dim) or \
            v_pool.shape[1:] != (page_size, num_kv_heads, value_dim):
        raise InvalidArgumentError("attention_talk: cache pools do not match q and the head sizes")
    if tuple(mix.shape) != (num_heads, num_heads):
        raise InvalidArgumentError("attention_talk: the mixing matrix must be [heads, heads]")
    if stats.numel() < 2 * count * num_splits * num_heads or \
            (num_splits > 1 and (partial is None or partial.numel() < num_splits * count * num_heads * value_dim)):
        raise InvalidArgumentError("attention_talk: a scratch buffer is too small")
    _check(fn(_gpu(q, "q"), _gpu(out, "out"), dtype_code(q.dtype), _gpu(k_pool, "k_pool"), _gpu(v_pool, "v_pool"),
              _gpu(mix, "mix", torch.float32), _gpu(token_seq, "token_seq", torch.int32),
              _gpu(positions, "positions", torch.int32), _gpu(block_table, "block_table", torch.int32),
              block_table.shape[1], page_size, count, num_heads, num_kv_heads, head_dim, value_dim, float(scale),
              float(out_scale), int(split_keys), int(num_splits), _gpu(stats, "stats", torch.float32),
              _opt(partial, "partial", torch.float32), _stream()), "attention", kernels=2 if num_splits == 1 else 3)


def attention_talk_prefill(q: torch.Tensor, out: torch.Tensor, pairs: torch.Tensor, k_pool: torch.Tensor,
                           v_pool: torch.Tensor, mix: torch.Tensor, *, entry_starts: torch.Tensor, entry_pos0: torch.Tensor,
                           block_table: torch.Tensor, num_entries: int, num_heads: int, num_kv_heads: int, head_dim: int,
                           scale: float, out_scale: float = 1.0) -> None:
    """The same result as ``attention_talk`` for steps with portions, on the tensor cores (bfloat16,
    head sizes 64 and 128, values as long as keys): the flash kernel computes softmax(q_g k^T) v_c
    for every pair of a query head g and a KV head c into the float32 ``pairs`` [tokens, heads * kv_heads * d],
    and a second kernel forms ``out[t, h] = out_scale * sum_g mix[h, g] pairs[t, g, kv(h)]`` in 32-bit
    (mixing the heads' weights is linear in them, and the values are shared)."""
    if head_dim not in MMA_HEAD_DIMS:
        raise UnsupportedError(f"attention_talk_prefill: head size {head_dim} (built: 64, 128)")
    count = q.shape[0]
    if q.shape[1] != num_heads * head_dim or out.shape != q.shape or \
            tuple(pairs.shape) != (count, num_heads * num_kv_heads * head_dim):
        raise InvalidArgumentError("attention_talk_prefill: q and out must be [tokens, heads * d], pairs [tokens, heads * kv_heads * d]")
    if k_pool.shape[2:] != (num_kv_heads, head_dim) or v_pool.shape != k_pool.shape:
        raise InvalidArgumentError("attention_talk_prefill: cache pools must be [pages, page_size, kv_heads, d]")
    if tuple(mix.shape) != (num_heads, num_heads):
        raise InvalidArgumentError("attention_talk_prefill: the mixing matrix must be [heads, heads]")
    fn = _function("attention_mma", "vipera_attention_prefill_pairs", [_c_void] * 7 + [_c_int] * 7 + [_c_float, _c_void])
    _check(fn(_gpu(q, "q", torch.bfloat16), _gpu(pairs, "pairs", torch.float32), _gpu(k_pool, "k_pool", torch.bfloat16),
              _gpu(v_pool, "v_pool", torch.bfloat16), _gpu(entry_starts, "entry_starts", torch.int32),
              _gpu(entry_pos0, "entry_pos0", torch.int32), _gpu(block_table, "block_table", torch.int32),
              block_table.shape[1], k_pool.shape[1], int(num_entries), count, num_heads, num_kv_heads, head_dim,
              float(scale), _stream()), "attention_prefill")
    fn = _function("attention_talk", "vipera_talk_combine",
                   [_c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_void])
    _check(fn(pairs.data_ptr(), _gpu(mix, "mix", torch.float32), _gpu(out, "out", torch.bfloat16), BF16, count, num_heads,
              num_kv_heads, head_dim, float(out_scale), _stream()), "attention")


def attention_talk_decode(q: torch.Tensor, out: torch.Tensor, pairs: torch.Tensor, k_pool: torch.Tensor,
                          v_pool: torch.Tensor, mix: torch.Tensor, *, positions: torch.Tensor, block_table: torch.Tensor,
                          num_heads: int, num_kv_heads: int, head_dim: int, scale: float, chunk: int, num_splits: int,
                          scratch: torch.Tensor, out_scale: float = 1.0) -> None:
    """``attention_talk_prefill`` for a step of single tokens: the split-key kernel computes every
    (query head, KV head) pair into the float32 ``pairs`` [entries, heads * kv_heads * d] (``chunk``, ``num_splits``
    and ``scratch`` as for ``attention_decode``, the scratch sized for heads * kv_heads heads), then
    the mix of the pairs' outputs."""
    if head_dim not in MMA_HEAD_DIMS:
        raise UnsupportedError(f"attention_talk_decode: head size {head_dim} (built: 64, 128)")
    count = q.shape[0]
    if q.shape[1] != num_heads * head_dim or out.shape != q.shape or \
            tuple(pairs.shape) != (count, num_heads * num_kv_heads * head_dim) or positions.numel() != count:
        raise InvalidArgumentError("attention_talk_decode: q and out must be [entries, heads * d], pairs [entries, heads * kv_heads * d]")
    if k_pool.shape[2:] != (num_kv_heads, head_dim) or v_pool.shape != k_pool.shape:
        raise InvalidArgumentError("attention_talk_decode: cache pools must be [pages, page_size, kv_heads, d]")
    fn = _function("attention_mma", "vipera_attention_decode_pairs",
                   [_c_void] * 6 + [_c_int] * 6 + [_c_float, _c_int, _c_int, _c_void, ctypes.c_size_t, _c_void])
    _check(fn(_gpu(q, "q", torch.bfloat16), _gpu(pairs, "pairs", torch.float32), _gpu(k_pool, "k_pool", torch.bfloat16),
              _gpu(v_pool, "v_pool", torch.bfloat16), _gpu(positions, "positions", torch.int32),
              _gpu(block_table, "block_table", torch.int32), block_table.shape[1], k_pool.shape[1], count, num_heads,
              num_kv_heads, head_dim, float(scale), int(chunk), int(num_splits), _gpu(scratch, "scratch", torch.float32),
              scratch.numel(), _stream()), "attention_decode", kernels=2)
    fn = _function("attention_talk", "vipera_talk_combine",
                   [_c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_void])
    _check(fn(pairs.data_ptr(), _gpu(mix, "mix", torch.float32), _gpu(out, "out", torch.bfloat16), BF16, count, num_heads,
              num_kv_heads, head_dim, float(out_scale), _stream()), "attention")


# ----------------------------------------------------------------------------------------
# recurrences with a state of fixed size: Mamba's selective scan, gated linear attention
# ----------------------------------------------------------------------------------------
class _ScanParams(ctypes.Structure):
    _fields_ = [
        ("x", _c_void), ("dt_pre", _c_void), ("bc", _c_void), ("z", _c_void), ("z_stride", ctypes.c_longlong),
        ("z_offset", _c_int), ("a", _c_void), ("d", _c_void), ("state", _c_void), ("entry_starts", _c_void),
        ("state_slots", _c_void), ("fresh", _c_void), ("out", _c_void),
        ("channels", _c_int), ("states", _c_int), ("num_entries", _c_int), ("lanes", _c_int),
        ("mode", _c_int), ("num_jobs", _c_int), ("chunk_state", _c_void), ("chunk_dt", _c_void),
    ]


SCAN_CHUNK = 64   # tokens of a chunk in the recurrences' chunked forms (kScanChunk in mamba.cu, kGlaChunk in gla.cu)


def scan_jobs(tokens: int, num_entries: int) -> int:
    """The most chunks a step of `tokens` tokens in `num_entries` entries has."""
    return tokens // SCAN_CHUNK + num_entries


def mamba_scan(x: torch.Tensor, dt_pre: torch.Tensor, bc: torch.Tensor, z: torch.Tensor, z_offset: int, *,
               a: torch.Tensor, d: torch.Tensor, state: torch.Tensor, entry_starts: torch.Tensor,
               state_slots: torch.Tensor, fresh: torch.Tensor, num_entries: int, out: torch.Tensor,
               chunk_scratch=None) -> None:
    """Mamba's selective scan.  ``x`` (after convolution and silu) and ``dt_pre`` (the step-size
    product with its bias, before softplus) are float32 [tokens, channels]; ``bc`` float32 [tokens,
    2 * states] holds B then C; the gate's pre-activation is column ``z_offset + c`` of the float32
    ``z``; ``a`` [channels, states] is -exp(A_log), ``d`` [channels]; ``state`` float32 [slots,
    channels * states]; ``out`` [tokens, channels] receives y * silu(z).  ``chunk_scratch`` (float32
    tensors [jobs, channels * states] and [jobs, channels] with jobs >= scan_jobs(tokens, entries))
    lets the step's chunks of SCAN_CHUNK tokens run side by side instead of each entry's tokens in a row."""
    fn = _function("mamba", "vipera_mamba_scan", [ctypes.POINTER(_ScanParams), _c_int, _c_void])
    _check_struct("mamba", "vipera_mamba_scan_params_size", _ScanParams)
    tokens, channels = x.shape
    states = a.shape[1]
    if tuple(dt_pre.shape) != (tokens, channels) or tuple(bc.shape) != (tokens, 2 * states) or \
            tuple(out.shape) != (tokens, channels) or tuple(a.shape) != (channels, states) or d.numel() != channels:
        raise InvalidArgumentError("mamba_scan: shapes do not agree")
    if z.shape[0] != tokens or z.shape[1] < z_offset + channels or z.dtype != torch.float32 or not z.is_contiguous():
        raise InvalidArgumentError("mamba_scan: the gate's rows are too short")
    if state.dim() != 2 or state.shape[1] != channels * states:
        raise InvalidArgumentError("mamba_scan: state rows must hold channels * states floats")
    p = _ScanParams()
    p.x, p.dt_pre, p.bc = _gpu(x, "x", torch.float32), _gpu(dt_pre, "dt_pre", torch.float32), _gpu(bc, "bc", torch.float32)
    p.z, p.z_stride, p.z_offset = z.data_ptr(), z.shape[1], int(z_offset)
    p.a, p.d = _gpu(a, "a", torch.float32), _gpu(d, "d", torch.float32)
    p.state = _gpu(state, "state", torch.float32)
    p.entry_starts = _gpu(entry_starts, "entry_starts", torch.int32)
    p.state_slots = _gpu(state_slots, "state_slots", torch.int32)
    p.fresh = _gpu(fresh, "fresh", torch.int32)
    p.out = _gpu(out, "out")
    p.channels, p.states, p.num_entries = int(channels), int(states), int(num_entries)
    if chunk_scratch is not None:
        chunk_state, chunk_dt = chunk_scratch
        jobs = scan_jobs(tokens, num_entries)
        if chunk_state.shape[0] < jobs or chunk_dt.shape[0] < jobs or chunk_state.shape[1] != channels * states or \
                chunk_dt.shape[1] != channels:
            raise InvalidArgumentError("mamba_scan: the chunk scratch has the wrong shape")
        p.num_jobs = jobs
        p.chunk_state, p.chunk_dt = _gpu(chunk_state, "chunk states", torch.float32), _gpu(chunk_dt, "chunk dt", torch.float32)
    _check(fn(ctypes.byref(p), dtype_code(out.dtype), _stream()), "mamba_scan", kernels=3 if chunk_scratch is not None else 1)


class _GlaParams(ctypes.Structure):
    _fields_ = [
        ("proj", _c_void), ("proj_width", ctypes.c_longlong),
        ("q_off", _c_int), ("k_off", _c_int), ("v_off", _c_int), ("g_off", _c_int),
        ("z", _c_void), ("log_alpha", _c_void), ("state", _c_void), ("entry_starts", _c_void), ("state_slots", _c_void),
        ("fresh", _c_void), ("partial", _c_void), ("norm_weight", _c_void), ("out", _c_void),
        ("heads", _c_int), ("dim", _c_int), ("vdim", _c_int), ("num_entries", _c_int), ("num_tokens", _c_int),
        ("shares", _c_int), ("q_scale", _c_float), ("inv_tau", _c_float), ("eps", _c_float), ("out_scale", _c_float),
        ("mode", _c_int), ("num_jobs", _c_int), ("chunk_state", _c_void), ("chunk_decay", _c_void),
    ]


def gla_shares(dim: int) -> int:
    """How many row shares of a head's state the scan kernel writes partial outputs for."""
    fn = getattr(load_kernel_library("gla"), "vipera_gla_shares")
    fn.argtypes, fn.restype = [_c_int], _c_int
    return int(fn(int(dim)))


def gla(proj: torch.Tensor, z: torch.Tensor, *, offsets, heads: int, dim: int, vdim: int, q_scale: float, tau: float,
        norm_weight: torch.Tensor, norm_eps: float, out_scale: float, state: torch.Tensor, entry_starts: torch.Tensor,
        state_slots: torch.Tensor, fresh: torch.Tensor, num_entries: int, partial: torch.Tensor, out: torch.Tensor,
        log_decay: torch.Tensor, chunk_scratch=None) -> None:
    """Gated linear attention over a step.  ``proj`` float32 [tokens, width] holds q, k, v and the
    output gate's pre-activation at ``offsets``; ``z`` float32 [tokens, heads * dim] the decays'
    pre-activations (the decays take their place; ``log_decay``, of the same shape, receives their logarithms); ``state`` float32 [slots, heads * dim * vdim]; ``partial`` float32 scratch of
    gla_shares(dim) * tokens * heads * vdim values; ``out`` [tokens, heads * vdim] receives the
    normalised, gated and scaled output.  ``chunk_scratch`` (float32 tensors [jobs, heads * dim * vdim]
    and [jobs, heads * dim] with jobs >= scan_jobs(tokens, entries)) lets the step's chunks of SCAN_CHUNK
    tokens run side by side instead of each entry's tokens in a row."""
    fn = _function("gla", "vipera_gla", [ctypes.POINTER(_GlaParams), _c_int, _c_void])
    _check_struct("gla", "vipera_gla_params_size", _GlaParams)
    tokens = proj.shape[0]
    if tuple(z.shape) != (tokens, heads * dim) or tuple(log_decay.shape) != tuple(z.shape) or \
            tuple(out.shape) != (tokens, heads * vdim):
        raise InvalidArgumentError("gla: z must be [tokens, heads * d] and out [tokens, heads * value size]")
    if state.dim() != 2 or state.shape[1] != heads * dim * vdim:
        raise InvalidArgumentError("gla: state rows must hold heads * d * value size floats")
    if partial.numel() < gla_shares(dim) * tokens * heads * vdim or norm_weight.numel() != vdim:
        raise InvalidArgumentError("gla: the scratch is too small or the norm weight has the wrong size")
    p = _GlaParams()
    p.proj, p.proj_width = _gpu(proj, "proj", torch.float32), proj.shape[1]
    p.q_off, p.k_off, p.v_off, p.g_off = (int(o) for o in offsets)
    p.z, p.state = _gpu(z, "z", torch.float32), _gpu(state, "state", torch.float32)
    p.log_alpha = _gpu(log_decay, "log_decay", torch.float32)
    p.entry_starts = _gpu(entry_starts, "entry_starts", torch.int32)
    p.state_slots = _gpu(state_slots, "state_slots", torch.int32)
    p.fresh = _gpu(fresh, "fresh", torch.int32)
    p.partial = _gpu(partial, "partial", torch.float32)
    p.norm_weight = _gpu(norm_weight, "norm_weight", torch.float32)
    p.out = _gpu(out, "out")
    p.heads, p.dim, p.vdim, p.num_entries, p.num_tokens = int(heads), int(dim), int(vdim), int(num_entries), int(tokens)
    p.q_scale, p.inv_tau, p.eps, p.out_scale = float(q_scale), 1.0 / float(tau), float(norm_eps), float(out_scale)
    if chunk_scratch is not None:
        chunk_state, chunk_decay = chunk_scratch
        jobs = scan_jobs(tokens, num_entries)
        if chunk_state.shape[0] < jobs or chunk_decay.shape[0] < jobs or chunk_state.shape[1] != heads * dim * vdim or \
                chunk_decay.shape[1] != heads * dim:
            raise InvalidArgumentError("gla: the chunk scratch has the wrong shape")
        p.num_jobs = jobs
        p.chunk_state = _gpu(chunk_state, "chunk states", torch.float32)
        p.chunk_decay = _gpu(chunk_decay, "chunk decays", torch.float32)
    _check(fn(ctypes.byref(p), dtype_code(out.dtype), _stream()), "gla", kernels=5 if chunk_scratch is not None else 3)


# ----------------------------------------------------------------------------------------
# norms over groups of a row, and a sublayer's gated, normed and scaled way into the stream
# ----------------------------------------------------------------------------------------
def group_rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float, groups: int,
                  rows: Optional[torch.Tensor] = None) -> None:
    """out[r, g, :] = x[rows[r], g, :] / sqrt(mean(x[rows[r], g, :]^2) + eps) * weight[g, :]: the row
    is cut into ``groups`` equal consecutive parts, each divided by its own root mean square.  The
    float32 ``out`` may be ``x`` itself (without ``rows``)."""
    fn = _function("groupnorm", "vipera_group_rmsnorm",
                   [_c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_float, _c_void])
    hidden = x.shape[1]
    count = out.shape[0]
    if out.shape[1] != hidden or weight.numel() != hidden or hidden % int(groups):
        raise InvalidArgumentError("group_rmsnorm: widths of x, weight and out do not agree, or the groups do not divide them")
    if rows is None and x.shape[0] != count:
        raise InvalidArgumentError("group_rmsnorm: x and out have different row counts")
    if rows is not None and (rows.numel() != count or out.data_ptr() == x.data_ptr()):
        raise InvalidArgumentError("group_rmsnorm: one row index per output row, and no norm in place with row indices")
    _check(fn(_gpu(x, "x", torch.float32), _gpu(weight, "weight", torch.float32), _opt(rows, "rows", torch.int32),
              _gpu(out, "out"), dtype_code(out.dtype), count, hidden, int(groups), float(eps), _stream()), "rmsnorm")


def gated_norm_add(branch: torch.Tensor, parts: int, gate: Optional[torch.Tensor], coefficient: torch.Tensor,
                   residual: torch.Tensor, eps: float, groups: int) -> None:
    """``y = (sum_p branch[r, p, :]) * sigmoid(gate[r, :])`` (no gate: the sum itself), then
    ``residual[r, g, :] += coefficient[g, :] * y[g, :] / sqrt(mean(y[g, :]^2) + eps)`` over ``groups``
    equal parts of the row.  ``branch`` is float32 [rows, parts * hidden] (its first part is used
    as scratch), ``gate`` float32 [rows, hidden] holds pre-activations."""
    fn = _function("groupnorm", "vipera_gated_norm_add",
                   [_c_void, _c_int, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_float, _c_void])
    count, hidden = residual.shape
    if branch.numel() != count * int(parts) * hidden or coefficient.numel() != hidden or hidden % int(groups):
        raise InvalidArgumentError("gated_norm_add: shapes of the branch, the coefficients and the stream do not agree")
    if gate is not None and tuple(gate.shape) != (count, hidden):
        raise InvalidArgumentError("gated_norm_add: the gate must be [rows, hidden]")
    _check(fn(_gpu(branch, "branch", torch.float32), int(parts), _opt(gate, "gate", torch.float32),
              _gpu(coefficient, "coefficient", torch.float32), _gpu(residual, "residual", torch.float32), count, hidden,
              int(groups), float(eps), _stream()), "rmsnorm")


# ----------------------------------------------------------------------------------------
# attention over a cached low-rank latent
# ----------------------------------------------------------------------------------------
class _LatentParams(ctypes.Structure):
    _fields_ = [
        ("proj", _c_void), ("proj_width", ctypes.c_longlong), ("q_off", _c_int), ("g_off", _c_int), ("kv_off", _c_int),
        ("up_k", _c_void), ("up_v", _c_void), ("norm_weight", _c_void), ("positions", _c_void), ("token_entry", _c_void),
        ("block_table", _c_void), ("cos_table", _c_void), ("sin_table", _c_void), ("k_pool", _c_void), ("v_pool", _c_void),
        ("qa", _c_void), ("latent_out", _c_void), ("out", _c_void),
        ("num_tokens", _c_int), ("heads", _c_int), ("d", _c_int), ("rot", _c_int), ("dv", _c_int), ("rank", _c_int),
        ("table_width", _c_int), ("page_size", _c_int), ("scale", _c_float), ("eps", _c_float),
        ("part", _c_void), ("split_keys", _c_int), ("num_splits", _c_int),
        ("stage", _c_int), ("padded_tokens", _c_int), ("a_heads", _c_void), ("qa_heads", _c_void), ("q_rot", _c_void),
        ("l_heads", _c_void), ("o_heads", _c_void), ("tile_group", _c_void),
        ("window", _c_int), ("pairing", _c_int),
    ]


@functools.lru_cache(maxsize=4096)
def latent_plan(tokens: int, heads: int, max_keys: int, sm_count: int):
    """How the tensor-core fold over the latents cuts a step: (tokens per tile, heads per tile,
    keys per split, splits)."""
    fn = _function("latent", "vipera_latent_plan", [_c_int] * 4 + [ctypes.POINTER(_c_int)])
    plan = (_c_int * 4)()
    _check(fn(int(tokens), int(heads), int(max_keys), int(sm_count), plan), "latent_plan", kernels=0)
    return tuple(plan)


def latent_part_floats(tokens: int, heads: int, rank: int, max_keys: int, sm_count: int) -> int:
    """Floats of scratch the fold's splits need for a step (0 when it runs without splits)."""
    splits = latent_plan(tokens, heads, max_keys, sm_count)[3]
    return splits * tokens * heads * (rank + 2) if splits > 1 else 0


def latent_attention(proj: torch.Tensor, *, q_off: int, g_off: int, kv_off: int, up_k: torch.Tensor, up_v: torch.Tensor,
                     norm_weight: Optional[torch.Tensor], eps: float, positions: torch.Tensor, token_entry: torch.Tensor,
                     block_table: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, k_pool: torch.Tensor,
                     v_pool: torch.Tensor, qa: torch.Tensor, latent_out: torch.Tensor, out: torch.Tensor, heads: int,
                     head_dim: int, rot_dim: int, value_dim: int, scale: float, max_keys: int = 0,
                     part: Optional[torch.Tensor] = None, head_major: Optional[dict] = None, window: int = 0,
                     pairing: int = ROPE_INTERLEAVED) -> None:
    """Causal softmax attention whose keys and values are products of a cached latent.  ``proj``
    float32 [tokens, width] holds q (head by head [head_dim | rot_dim]) at column ``q_off``, the
    output gate's pre-activation at ``g_off`` (negative: no gate) and the down projection
    [rank | rot_dim] at ``kv_off`` (negative: the step's tokens are in the cache already, written
    by another layer).  ``k_pool`` [pages, page_size, 1, rank] receives the normed latents,
    ``v_pool`` [pages, page_size, 1, rot_dim] the rotated key part the heads share.  ``up_k``
    [heads * head_dim, rank] and ``up_v`` [heads, rank, value_dim] (each head's value matrix
    transposed) are in the pools' type, as is ``out`` [tokens, heads * value_dim]; ``qa`` float32
    [tokens, heads, rank + rot_dim] and ``latent_out`` float32 [tokens, heads, rank] are scratch.
    ``max_keys`` (at least the longest history of the step) and ``part`` (float32,
    latent_part_floats(...)) let a step of few tokens cut its keys between blocks.  ``head_major``
    (bfloat16): the products with the up matrices run as grouped tensor-core products, a head a
    group, over rows padded to ``padded`` tokens per head: ``up_k_t`` [heads, rank, head_dim],
    ``up_v_rows`` [heads, value_dim, rank] and the scratch ``a_heads`` (bfloat16 [heads * padded,
    head_dim]), ``qa_heads`` (float32 [heads * padded, rank]), ``q_rot`` (float32 [tokens, heads *
    rot_dim]), ``l_heads`` (bfloat16 [heads * padded, rank]), ``o_heads`` (float32 [heads * padded,
    value_dim]) and ``tile_group`` (int32 [heads * padded / 128]).  ``window`` > 0: a query at position
    p sees keys p - window + 1 .. p.  ``pairing``: which values of the rotated part turn together,
    ROPE_INTERLEAVED (2i, 2i + 1) or ROPE_NEOX (i, i + rot_dim / 2)."""
    fn = _function("latent", "vipera_latent_attention", [ctypes.POINTER(_LatentParams), _c_int, _c_void])
    _check_struct("latent", "vipera_latent_params_size", _LatentParams)
    tokens = proj.shape[0]
    rank = k_pool.shape[3]
    page_size = k_pool.shape[1]
    if tuple(k_pool.shape[1:]) != (page_size, 1, rank) or tuple(v_pool.shape[1:]) != (page_size, 1, rot_dim) or \
            k_pool.dtype != v_pool.dtype:
        raise InvalidArgumentError("latent_attention: the pools must be [pages, page_size, 1, rank] and [pages, page_size, 1, rot_dim]")
    if tuple(up_k.shape) != (heads * head_dim, rank) or tuple(up_v.shape) != (heads, rank, value_dim) or \
            up_k.dtype != k_pool.dtype or up_v.dtype != k_pool.dtype or out.dtype != k_pool.dtype:
        raise InvalidArgumentError("latent_attention: the up matrices and the output must match the pools' type and sizes")
    if tuple(out.shape) != (tokens, heads * value_dim) or qa.numel() < tokens * heads * (rank + rot_dim) or \
            latent_out.numel() < tokens * heads * rank:
        raise InvalidArgumentError("latent_attention: the output or a scratch buffer is too small")
    if tuple(cos.shape[1:]) != (rot_dim // 2,) or cos.shape != sin.shape:
        raise InvalidArgumentError("latent_attention: cos/sin tables of width rot_dim/2 are needed")
    if kv_off >= 0 and (norm_weight is None or norm_weight.numel() != rank):
        raise InvalidArgumentError("latent_attention: a layer that writes the cache needs the latent's norm weight")
    p = _LatentParams()
    p.proj, p.proj_width = _gpu(proj, "proj", torch.float32), proj.shape[1]
    p.q_off, p.g_off, p.kv_off = int(q_off), int(g_off), int(kv_off)
    p.up_k, p.up_v = _gpu(up_k, "up_k"), _gpu(up_v, "up_v")
    p.norm_weight = _opt(norm_weight, "norm_weight", torch.float32)
    p.positions = _gpu(positions, "positions", torch.int32)
    p.token_entry = _gpu(token_entry, "token_entry", torch.int32)
    p.block_table = _gpu(block_table, "block_table", torch.int32)
    p.cos_table, p.sin_table = _gpu(cos, "cos", torch.float32), _gpu(sin, "sin", torch.float32)
    p.k_pool, p.v_pool = _gpu(k_pool, "k_pool"), _gpu(v_pool, "v_pool")
    p.qa, p.latent_out = _gpu(qa, "qa", torch.float32), _gpu(latent_out, "latent_out", torch.float32)
    p.out = _gpu(out, "out")
    p.num_tokens, p.heads, p.d, p.rot, p.dv, p.rank = int(tokens), int(heads), int(head_dim), int(rot_dim), int(value_dim), int(rank)
    p.table_width, p.page_size = int(block_table.shape[1]), int(page_size)
    p.scale, p.eps = float(scale), float(eps)
    if pairing not in (ROPE_INTERLEAVED, ROPE_NEOX):
        raise InvalidArgumentError("latent_attention: the rotated part turns as interleaved pairs or as halves")
    p.window, p.pairing = int(window or 0), 1 if pairing == ROPE_NEOX else 0
    p.part, p.split_keys, p.num_splits = None, 0, 1
    if part is not None and max_keys > 0:
        _, _, split_keys, splits = latent_plan(tokens, heads, int(max_keys), sm_count(proj.device))
        if splits > 1:
            if part.numel() < splits * tokens * heads * (rank + 2):
                raise InvalidArgumentError("latent_attention: the scratch of the splits is too small")
            p.part, p.split_keys, p.num_splits = _gpu(part, "part", torch.float32), int(split_keys), int(splits)
    if head_major is not None:
        m = head_major
        padded = int(m["padded"])
        if padded % 128 or padded < tokens or tuple(m["up_k_t"].shape) != (heads, rank, head_dim) or \
                tuple(m["up_v_rows"].shape) != (heads, value_dim, rank) or \
                tuple(m["a_heads"].shape) != (heads * padded, head_dim) or tuple(m["qa_heads"].shape) != (heads * padded, rank) or \
                tuple(m["l_heads"].shape) != (heads * padded, rank) or tuple(m["o_heads"].shape) != (heads * padded, value_dim) or \
                m["q_rot"].numel() < tokens * heads * rot_dim or m["tile_group"].numel() < heads * padded // 128:
            raise InvalidArgumentError("latent_attention: the head-major buffers do not match the step")
        p.padded_tokens = padded
        p.a_heads, p.l_heads = _gpu(m["a_heads"], "a_heads", torch.bfloat16), _gpu(m["l_heads"], "l_heads", torch.bfloat16)
        p.qa_heads, p.q_rot = _gpu(m["qa_heads"], "qa_heads", torch.float32), _gpu(m["q_rot"], "q_rot", torch.float32)
        p.o_heads, p.tile_group = _gpu(m["o_heads"], "o_heads", torch.float32), _gpu(m["tile_group"], "tile_group", torch.int32)
        code = dtype_code(k_pool.dtype)
        p.stage = 1
        _check(fn(ctypes.byref(p), code, _stream()), "attention", kernels=2 if kv_off >= 0 else 1)
        gemm_tc_grouped(m["a_heads"], m["up_k_t"], m["tile_group"], epilogue=EPI_STORE, out=m["qa_heads"], what="attention")
        p.stage = 2
        _check(fn(ctypes.byref(p), code, _stream()), "attention", kernels=2 if p.num_splits > 1 else 1)
        gemm_tc_grouped(m["l_heads"], m["up_v_rows"], m["tile_group"], epilogue=EPI_STORE, out=m["o_heads"], what="attention")
        p.stage = 3
        _check(fn(ctypes.byref(p), code, _stream()), "attention")
        return
    _check(fn(ctypes.byref(p), dtype_code(k_pool.dtype), _stream()), "attention", kernels=4 if kv_off >= 0 else 3)


# ----------------------------------------------------------------------------------------
# linear attention with one constant decay per head
# ----------------------------------------------------------------------------------------
class _LightningParams(ctypes.Structure):
    _fields_ = [
        ("proj", _c_void), ("proj_width", ctypes.c_longlong),
        ("q_off", _c_int), ("k_off", _c_int), ("v_off", _c_int), ("g_off", _c_int),
        ("decay", _c_void), ("state", _c_void), ("entry_starts", _c_void), ("state_slots", _c_void), ("fresh", _c_void),
        ("raw", _c_void), ("norm_weight", _c_void), ("out", _c_void), ("chunk_state", _c_void),
        ("heads", _c_int), ("d", _c_int), ("dv", _c_int), ("num_entries", _c_int), ("num_tokens", _c_int),
        ("num_jobs", _c_int), ("eps", _c_float), ("activated", _c_int),
    ]


def lightning(proj: torch.Tensor, *, offsets, heads: int, dim: int, vdim: int, decay: torch.Tensor,
              norm_weight: torch.Tensor, norm_eps: float, state: torch.Tensor, entry_starts: torch.Tensor,
              state_slots: torch.Tensor, fresh: torch.Tensor, num_entries: int, raw: torch.Tensor, out: torch.Tensor,
              chunk_state: Optional[torch.Tensor] = None) -> None:
    """Linear attention with a constant decay per head over a step: ``S = decay_h S + k v^T``,
    ``o = S^T q`` with q, k, v the silu of their projections.  ``proj`` float32 [tokens, width]
    holds the pre-activations of q, k, v and the output gate at ``offsets``; ``state`` float32
    [slots, heads * dim * vdim]; ``raw`` float32 [tokens, heads * vdim] is scratch; ``out`` [tokens,
    heads * vdim] receives the heads' outputs divided by their root mean square over the whole row,
    times ``norm_weight`` and the sigmoid of the gate.  ``chunk_state`` (float32 [jobs, heads * dim *
    vdim], jobs >= scan_jobs(tokens, entries)) lets the step's chunks of SCAN_CHUNK tokens run side
    by side instead of each entry's tokens in a row."""
    fn = _function("lightning", "vipera_lightning", [ctypes.POINTER(_LightningParams), _c_int, _c_void])
    _check_struct("lightning", "vipera_lightning_params_size", _LightningParams)
    tokens = proj.shape[0]
    if tuple(out.shape) != (tokens, heads * vdim) or raw.numel() < tokens * heads * vdim or decay.numel() != heads or \
            norm_weight.numel() != heads * vdim:
        raise InvalidArgumentError("lightning: out must be [tokens, heads * value size], with one decay per head and one "
                                   "norm weight per value of the row")
    if state.dim() != 2 or state.shape[1] != heads * dim * vdim:
        raise InvalidArgumentError("lightning: state rows must hold heads * d * value size floats")
    p = _LightningParams()
    p.proj, p.proj_width = _gpu(proj, "proj", torch.float32), proj.shape[1]
    p.q_off, p.k_off, p.v_off, p.g_off = (int(o) for o in offsets)
    p.decay, p.state = _gpu(decay, "decay", torch.float32), _gpu(state, "state", torch.float32)
    p.entry_starts = _gpu(entry_starts, "entry_starts", torch.int32)
    p.state_slots = _gpu(state_slots, "state_slots", torch.int32)
    p.fresh = _gpu(fresh, "fresh", torch.int32)
    p.raw, p.norm_weight = _gpu(raw, "raw", torch.float32), _gpu(norm_weight, "norm_weight", torch.float32)
    p.out = _gpu(out, "out")
    p.heads, p.d, p.dv, p.num_entries, p.num_tokens = int(heads), int(dim), int(vdim), int(num_entries), int(tokens)
    p.eps = float(norm_eps)
    if chunk_state is not None:
        jobs = scan_jobs(tokens, num_entries)
        if chunk_state.shape[0] < jobs or chunk_state.shape[1] != heads * dim * vdim:
            raise InvalidArgumentError("lightning: the chunk scratch has the wrong shape")
        p.num_jobs = jobs
        p.chunk_state = _gpu(chunk_state, "chunk states", torch.float32)
    _check(fn(ctypes.byref(p), dtype_code(out.dtype), _stream()), "lightning", kernels=5 if chunk_state is not None else 2)


# ----------------------------------------------------------------------------------------
# mixture of gated units
# ----------------------------------------------------------------------------------------
class _MoeParams(ctypes.Structure):
    _fields_ = [
        ("h", _c_void), ("router", _c_void), ("gate_up", _c_void), ("down", _c_void),
        ("chosen", _c_void), ("weight", _c_void), ("order", _c_void), ("rank", _c_void), ("tiles", _c_void),
        ("tile_expert", _c_void), ("act", _c_void), ("rows", _c_void), ("xs", _c_void), ("ys", _c_void),
        ("num_tokens", _c_int), ("hidden", _c_int), ("ff", _c_int), ("experts", _c_int), ("top", _c_int),
        ("groups", _c_int), ("keep", _c_int), ("group_top", _c_int), ("max_tiles", _c_int),
        ("softmax_scores", _c_int), ("renormalize", _c_int), ("activation", _c_int),
        ("gate_group", _c_int), ("tile_rows", _c_int), ("padded", _c_int),
        ("correction", _c_void), ("identity", _c_int), ("always", _c_int), ("slots", _c_int), ("gated", _c_int),
        ("route_scale", _c_float), ("renorm_eps", _c_float),
    ]


MOE_SKINNY_ROWS, MOE_PLAIN_ROWS, MOE_GROUPED_ROWS = 8, 32, 128   # kSkinnyRows, kTileRows in moe.cu; kTileX in gemm_tc.cu
MOE_SKINNY_MOST = int(os.environ.get("VIPERA_MOE_SKINNY_MOST", 64))   # assignments up to which a step takes the 8-row tiles
MOE_GATE_GROUP = 16   # gate and up rows alternate in groups of this many where the tensor-core ending is to read them


def moe_form(tokens: int, top: int, hidden: int, ff: int, gate_group: int, dtype: torch.dtype):
    """(rows of a tile, padded) for a step: 8-row tiles on the CUDA cores for few assignments;
    grouped tensor-core products over runs padded to 128 rows in bfloat16 where the sizes allow
    (rows that are whole 16-byte vectors, gate and up rows interleaved in sixteens); else 32-row tiles."""
    if tokens * top <= MOE_SKINNY_MOST and 8 * max(hidden, ff) * 4 <= 200 * 1024:
        return MOE_SKINNY_ROWS, False
    if dtype == torch.bfloat16 and hidden % 8 == 0 and ff % 16 == 0 and gate_group == MOE_GATE_GROUP:
        return MOE_GROUPED_ROWS, True
    return MOE_PLAIN_ROWS, False


def moe_max_tiles(tokens: int, top: int, experts: int, tile_rows: int = MOE_SKINNY_ROWS) -> int:
    """The most tiles of `tile_rows` assignments a step of `tokens` tokens has."""
    return tokens * top // tile_rows + min(experts, tokens * top)


def moe_capacity(tokens: int, top: int, experts: int) -> int:
    """Sorted places a step can need in any form (runs padded to whole tiles of 128 at most)."""
    return max(tokens * top, moe_max_tiles(tokens, top, experts, MOE_GROUPED_ROWS) * MOE_GROUPED_ROWS)


def moe_scratch_words(tokens: int, top: int, experts: int) -> int:
    return moe_capacity(tokens, top, experts) + tokens * top + 1 + 4 * moe_max_tiles(tokens, top, experts)


def gemm_tc_grouped(a: torch.Tensor, w: torch.Tensor, tile_group: torch.Tensor, *, epilogue: int, out: torch.Tensor,
                    activation: int = ACT_SILU, what: str = "gemm_tc") -> None:
    """a[M, K] (M a multiple of 128) times one of the matrices w[G, N, K], transposed: rows 128 i ..
    128 i + 127 use matrix tile_group[i] (int32, written on the device ahead of this call).
    Endings: plain store, or the gated unit over interleaved gate and up rows."""
    fn = _function("gemm_tc", "vipera_gemm_tc_grouped",
                   [_c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_void, _c_int, _c_void, _c_int, _c_int, _c_void, _c_void])
    m, k = a.shape
    groups, n = w.shape[0], w.shape[1]
    if w.shape[2] != k or m % 128 or tile_group.numel() < m // 128 or k % 8:
        raise InvalidArgumentError("gemm_tc_grouped: sizes do not match")
    width = n // 2 if epilogue == EPI_SWIGLU else n
    if tuple(out.shape) != (m, width):
        raise InvalidArgumentError(f"gemm_tc_grouped: out must be [{m}, {width}]")
    state = _tc_buffers(a.device, 0)
    _check(fn(_gpu(a, "a", torch.bfloat16), _gpu(w, "w", torch.bfloat16), m, n, k, groups,
              _gpu(tile_group, "tile_group", torch.int32), epilogue, _gpu(out, "out"), dtype_code(out.dtype), int(activation),
              state["status"].data_ptr(), _stream()), what)


def moe(h: torch.Tensor, *, router: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, gate_group: int, top: int,
        groups: int, keep: int, group_top: int, softmax_scores: bool, renormalize: bool, activation: int,
        chosen: torch.Tensor, weight: torch.Tensor, scratch: torch.Tensor, act: torch.Tensor, rows: torch.Tensor,
        xs: Optional[torch.Tensor] = None, ys: Optional[torch.Tensor] = None, gated: bool = True,
        correction: Optional[torch.Tensor] = None, identity: int = 0, always: int = 0, route_scale: float = 1.0,
        renorm_eps: float = 0.0) -> None:
    """A mixture of gated units over a step.  ``h`` [tokens, hidden]; ``router`` float32 [experts,
    hidden]; ``gate_up`` [experts, 2 ff, hidden] (``gate_group`` gate rows, then the up rows of the
    same features, and so on) and ``down`` [experts, hidden, ff] in h's type.  ``chosen`` int32 and
    ``weight`` float32 [tokens, top] receive each token's experts and their weights; ``rows``
    float32 [tokens, top, hidden] receives each chosen expert's weighted output (their sum over
    ``top`` is the mixture's output).  ``scratch`` int32 of moe_scratch_words(...) words; ``act``
    [moe_capacity(...), ff] in h's type; ``xs`` (h's type) and ``ys`` (float32) [moe_capacity(...),
    hidden] for the form that runs on the tensor cores.

    ``gated`` false: units without a gate, ``D act(U h)``; ``gate_up`` is then [matrices, ff, hidden].
    ``correction`` float32 [router outputs]: added to the scores for the choice only.  ``identity``:
    the last that many router outputs have no matrices and return the token's row times their weight.
    ``always``: that many further units, behind the router's own in ``gate_up`` and ``down``, which every
    token uses with weight 1; ``top`` stays the router's count, and ``chosen``, ``weight`` and ``rows``
    hold ``top + always`` places per token, sized by the caller with moe_capacity(tokens, top + always,
    matrices) and so on.  ``renormalize`` divides the weights by their sum + ``renorm_eps``;
    ``route_scale`` multiplies them."""
    fn = _function("moe", "vipera_moe", [ctypes.POINTER(_MoeParams), _c_int, _c_void])
    _check_struct("moe", "vipera_moe_params_size", _MoeParams)
    tokens, hidden = h.shape
    matrices, ff = gate_up.shape[0], gate_up.shape[1] // (2 if gated else 1)
    outputs, identity, always = router.shape[0], int(identity), int(always)
    if outputs - identity + always != matrices or identity < 0 or always < 0 or router.shape[1] != hidden or \
            tuple(gate_up.shape) != (matrices, (2 if gated else 1) * ff, hidden) or \
            tuple(down.shape) != (matrices, hidden, ff) or gate_up.dtype != h.dtype or down.dtype != h.dtype:
        raise InvalidArgumentError("moe: the experts' matrices do not match h, the router and each other")
    if correction is not None and correction.numel() != outputs:
        raise InvalidArgumentError("moe: one correction per router output")
    router_top = int(top)
    top = router_top + always      # a token's assignments
    experts = matrices             # what the tiles are counted over
    assignments = tokens * top
    tile_rows, padded = moe_form(tokens, top, hidden, ff, int(gate_group) if gated else MOE_GATE_GROUP, h.dtype)
    if padded and (xs is None or ys is None):
        tile_rows, padded = MOE_PLAIN_ROWS, False
    tiles = moe_max_tiles(tokens, top, experts, tile_rows)
    capacity = tiles * tile_rows if padded else assignments
    if chosen.numel() < assignments or weight.numel() < assignments or scratch.numel() < moe_scratch_words(tokens, top, experts) or \
            act.numel() < capacity * ff or act.dtype != h.dtype or rows.numel() < assignments * hidden:
        raise InvalidArgumentError("moe: a scratch buffer is too small")
    p = _MoeParams()
    p.h, p.router = _gpu(h, "h"), _gpu(router, "router", torch.float32)
    p.gate_up, p.down = _gpu(gate_up, "gate_up"), _gpu(down, "down")
    p.chosen, p.weight = _gpu(chosen, "chosen", torch.int32), _gpu(weight, "weight", torch.float32)
    base = _gpu(scratch, "scratch", torch.int32)
    places = moe_capacity(tokens, top, experts)
    most = moe_max_tiles(tokens, top, experts)
    p.order, p.rank, p.tiles = base, base + 4 * places, base + 4 * (places + assignments)
    p.tile_expert = base + 4 * (places + assignments + 1 + 3 * most)
    p.act, p.rows = _gpu(act, "act"), _gpu(rows, "rows", torch.float32)
    p.num_tokens, p.hidden, p.ff, p.experts, p.top = int(tokens), int(hidden), int(ff), int(outputs), router_top
    p.correction = _opt(correction, "correction", torch.float32)
    p.identity, p.always, p.slots, p.gated = identity, always, top, int(bool(gated))
    p.route_scale, p.renorm_eps = float(route_scale), float(renorm_eps)
    p.groups, p.keep, p.group_top, p.max_tiles = int(groups), int(keep), int(group_top), int(tiles)
    p.softmax_scores, p.renormalize, p.activation = int(bool(softmax_scores)), int(bool(renormalize)), int(activation)
    p.gate_group, p.tile_rows, p.padded = int(gate_group), int(tile_rows), int(padded)
    if not padded:
        _check(fn(ctypes.byref(p), dtype_code(h.dtype), _stream()), "moe", kernels=4)
        return
    if xs.numel() < capacity * hidden or ys.numel() < capacity * hidden or xs.dtype != h.dtype:
        raise InvalidArgumentError("moe: a scratch buffer is too small")
    p.xs, p.ys = _gpu(xs, "xs"), _gpu(ys, "ys", torch.float32)
    _check(fn(ctypes.byref(p), dtype_code(h.dtype), _stream()), "moe", kernels=3)
    tile_expert = scratch[places + assignments + 1 + 3 * most:places + assignments + 1 + 3 * most + tiles]
    xs_rows = xs.view(-1)[:capacity * hidden].view(capacity, hidden)
    act_rows = act.view(-1)[:capacity * ff].view(capacity, ff)
    ys_rows = ys.view(-1)[:capacity * hidden].view(capacity, hidden)
    gemm_tc_grouped(xs_rows, gate_up, tile_expert, epilogue=EPI_GATED if gated else EPI_STORE, out=act_rows,
                    activation=activation, what="moe")
    gemm_tc_grouped(act_rows, down, tile_expert, epilogue=EPI_STORE, out=ys_rows, what="moe")
    scatter = _function("moe", "vipera_moe_scatter", [ctypes.POINTER(_MoeParams), _c_void])
    _check(scatter(ctypes.byref(p), _stream()), "moe")


def add_rows(rows: torch.Tensor, parts: int, target: torch.Tensor) -> None:
    """target[t, :] += sum_p rows[t, p, :] (float32), the places added in their order."""
    fn = _function("moe", "vipera_moe_add_rows", [_c_void, _c_int, _c_void, _c_int, _c_int, _c_void])
    count, hidden = target.shape
    if rows.numel() != count * int(parts) * hidden:
        raise InvalidArgumentError("add_rows: rows must hold parts rows of the target's width per token")
    _check(fn(_gpu(rows, "rows", torch.float32), int(parts), _gpu(target, "target", torch.float32), count, hidden, _stream()),
           "moe")


LATENT_MAX_RANK, LATENT_MAX_ROT = 512, 128   # kMaxRank, kMaxRot in latent.cu
MOE_MAX_EXPERTS = 1024                       # kMaxExperts in moe.cu
