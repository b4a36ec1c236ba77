"""Python wrappers of the CUDA entry points.

Every wrapper checks devices, dtypes, contiguity and shapes on the host and
then launches on torch's current stream; memory comes from torch's allocator.
Nothing here computes on the CPU or calls a library model/attention routine.
A kernel that cannot take a size raises UnsupportedError with the reason.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from ..errors import InvalidError, KernelUnavailableError, UnsupportedError
from . import library

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}


def _code(dtype: torch.dtype) -> int:
    try:
        return _CODES[dtype]
    except KeyError:
        raise UnsupportedError(f"kernels take float32 or bfloat16, not {dtype}") from None


def _lib():
    return library.load()


def _stream() -> ctypes.c_void_p:
    # the raw handle of torch's current stream; the Stream object torch.cuda.current_stream()
    # builds costs several microseconds per launch, which a short prompt's ~150 launches feel
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _check(t: torch.Tensor, name: str, dtype=None, dims: Optional[int] = None) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelUnavailableError(f"{name} must be a CUDA tensor: there is no CPU path")
    if not t.is_contiguous():
        raise InvalidError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise InvalidError(f"{name} must be {dtype}, got {t.dtype}")
    if dims is not None and t.dim() != dims:
        raise InvalidError(f"{name} must have {dims} dimensions, got {tuple(t.shape)}")


_launches = 0


def launch_count() -> int:
    """How many kernels of this library have been launched (or captured) by this process."""
    return _launches


def _done(code: int, what: str, launches: int = 1) -> None:
    global _launches
    if code == 0:
        _launches += launches
        return
    if code == -1:
        raise InvalidError(f"{what}: bad argument")
    if code == -2:
        raise UnsupportedError(f"{what}: size not supported by this kernel")
    raise RuntimeError(f"{what}: CUDA error {code}")



ROW_RESERVE = 32  # rows an activation buffer holds at least (see _activation)


def _activation(rows: int, width: int, dtype: torch.dtype, device) -> torch.Tensor:
    """An uninitialised [rows, width] activation whose storage holds at least ROW_RESERVE rows: the
    tensor-core product may then name 32 rows in its tensor map of this operand, which TMA handles
    faster than fewer (the rows beyond `rows` only feed accumulator rows that are never stored)."""
    return torch.empty((max(rows, ROW_RESERVE), width), dtype=dtype, device=device)[:rows]


# --------------------------------------------------------------------------- embedding
def embed_rows(table: torch.Tensor, ids: torch.Tensor, scale: Optional[float] = None) -> torch.Tensor:
    """float32 [T, h] rows of `table` ([vocab, h], float32 or bfloat16) at int32 ids [T],
    multiplied by `scale` when one is given."""
    _check(table, "table", dims=2)
    _check(ids, "ids", torch.int32, 1)
    out = torch.empty((ids.numel(), table.shape[1]), dtype=torch.float32, device=table.device)
    _done(_lib().lrm_embed_rows(_ptr(table), _code(table.dtype), _ptr(ids), _ptr(out),
                                ids.numel(), table.shape[1], table.shape[0],
                                ctypes.c_float(1.0 if scale is None else scale), _stream()), "embed_rows")
    return out


# --------------------------------------------------------------------------- norm
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
             rows: Optional[torch.Tensor] = None, partials: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMSNorm of float32 rows; see csrc/norm.cu for `rows` and `partials`."""
    _check(x, "x", torch.float32, 2)
    _check(weight, "weight", dims=1)
    hidden = x.shape[1]
    if weight.shape[0] != hidden:
        raise InvalidError(f"norm weight has {weight.shape[0]} elements, rows have {hidden}")
    n_rows = x.shape[0]
    if rows is not None:
        _check(rows, "rows", torch.int32, 1)
        n_rows = rows.numel()
    n_partials, stride = 0, 0
    if partials is not None:
        _check(partials, "partials", torch.float32, 3)
        if tuple(partials.shape[1:]) != tuple(x.shape):
            raise InvalidError("partials must be [n, T, h]")
        n_partials, stride = partials.shape[0], x.numel()
    out = _activation(n_rows, hidden, out_dtype, x.device)
    _done(_lib().lrm_rms_norm(_ptr(x), _ptr(weight), _code(weight.dtype), _ptr(out), _code(out_dtype),
                              _ptr(rows), _ptr(partials), n_partials, ctypes.c_longlong(stride),
                              n_rows, hidden, ctypes.c_float(eps), _stream()), "rms_norm")
    return out


def rms_norm_add_(stream: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float, mult: float = 1.0,
                  next_weight: Optional[torch.Tensor] = None, next_eps: Optional[float] = None,
                  out_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """stream += mult * RMSnorm(y) * weight, in place (stream and y float32 [T, h]: a norm behind a
    sublayer). With `next_weight` (same dtype as `weight`) the updated rows are normalized again in the
    same launch and returned as [T, h] in `out_dtype`: the norm in front of the next sublayer."""
    _check(stream, "stream", torch.float32, 2)
    _check(y, "y", torch.float32, 2)
    _check(weight, "weight", dims=1)
    T, hidden = stream.shape
    if tuple(y.shape) != (T, hidden) or weight.numel() != hidden:
        raise InvalidError("rms_norm_add_: y must match the stream, and the weight its rows")
    out = None
    if next_weight is not None:
        _check(next_weight, "next_weight", weight.dtype, 1)
        if next_weight.numel() != hidden or out_dtype is None:
            raise InvalidError("rms_norm_add_: the second norm needs a weight per column and an output type")
        out = _activation(T, hidden, out_dtype, stream.device)
    _done(_lib().lrm_rms_norm_add(_ptr(stream), _ptr(y), _ptr(weight), _code(weight.dtype), ctypes.c_float(mult),
                                  ctypes.c_float(eps), _ptr(next_weight), _ptr(out),
                                  _code(out_dtype) if out is not None else F32,
                                  ctypes.c_float(next_eps if next_eps is not None else eps), T, hidden, _stream()),
          "rms_norm_add_")
    return out


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float, out_dtype: torch.dtype,
               rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """(x - mean) / sqrt(variance + eps) * weight + bias over float32 rows [T, h] (all, or those `rows`
    names); weight and bias float32 [h]. -> [T or len(rows), h] in `out_dtype`."""
    _check(x, "x", torch.float32, 2)
    _check(weight, "weight", torch.float32, 1)
    _check(bias, "bias", torch.float32, 1)
    hidden = x.shape[1]
    if weight.numel() != hidden or bias.numel() != hidden:
        raise InvalidError("layer_norm: weight and bias must have one entry per column")
    n_rows = x.shape[0]
    if rows is not None:
        _check(rows, "rows", torch.int32, 1)
        n_rows = rows.numel()
    out = _activation(n_rows, hidden, out_dtype, x.device)
    _done(_lib().lrm_layer_norm(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), _code(out_dtype), _ptr(rows), n_rows,
                                hidden, ctypes.c_float(eps), _stream()), "layer_norm")
    return out


def layer_norm_add_(stream: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float,
                    mult: float = 1.0, cast_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """stream += mult * layer_norm(y), in place (both float32 [T, h]: a norm behind a sublayer). With
    `cast_dtype` the updated rows are also returned in that type, for a sublayer that reads the
    stream itself."""
    _check(stream, "stream", torch.float32, 2)
    _check(y, "y", torch.float32, 2)
    _check(weight, "weight", torch.float32, 1)
    _check(bias, "bias", torch.float32, 1)
    T, hidden = stream.shape
    if tuple(y.shape) != (T, hidden) or weight.numel() != hidden or bias.numel() != hidden:
        raise InvalidError("layer_norm_add_: y must match the stream, weight and bias its rows")
    out = _activation(T, hidden, cast_dtype, stream.device) if cast_dtype is not None else None
    _done(_lib().lrm_layer_norm_add(_ptr(stream), _ptr(y), _ptr(weight), _ptr(bias), ctypes.c_float(mult), _ptr(out),
                                    _code(cast_dtype or torch.float32), T, hidden, ctypes.c_float(eps), _stream()),
          "layer_norm_add_")
    return out


# --------------------------------------------------------------------------- matrix products
STORE, ADD, SILU_GATE = "store", "add", "silu_gate"


def linear(x: torch.Tensor, weight: torch.Tensor, epilogue: str = STORE,
           out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """y = x . weight^T with weight [out, in] as stored.

    epilogue "store": returns [M, N] in `out_dtype` (default: x's dtype).
    epilogue "add":   adds into `out`, a float32 [M, N] tensor (the residual stream), in place.
    epilogue "silu_gate": weight rows alternate in blocks of 8 gate / 8 up rows;
                      returns silu(gate) * up as [M, N/2] (bfloat16 inputs only).
    float32 inputs run the true 32-bit kernel; bfloat16 inputs the tensor-core kernels.
    """
    _check(x, "x", dims=2)
    _check(weight, "weight", dims=2)
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K:
        raise InvalidError(f"linear: x has {K} columns, weight has {weight.shape[1]}")
    if x.dtype != weight.dtype:
        raise InvalidError(f"linear: x is {x.dtype}, weight is {weight.dtype}")
    lib = _lib()
    if epilogue == ADD:
        if out is None:
            raise InvalidError("linear: epilogue 'add' needs the tensor to add into")
        _check(out, "out", torch.float32, 2)
        if tuple(out.shape) != (M, N):
            raise InvalidError(f"linear: out must be [{M}, {N}]")
    if x.dtype == torch.float32:
        if epilogue == SILU_GATE:
            raise UnsupportedError("linear: the float32 kernel has no fused gate epilogue")
        if epilogue == STORE:
            if out_dtype not in (None, torch.float32):
                raise InvalidError("linear: float32 inputs give float32 outputs")
            out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        _done(lib.lrm_gemm_f32(_ptr(x), _ptr(weight), _ptr(out), M, N, K,
                               1 if epilogue == ADD else 0, _stream()), "gemm_f32")
        return out
    if x.dtype != torch.bfloat16:
        raise UnsupportedError(f"linear: dtype {x.dtype}")
    if epilogue == STORE:
        out_dtype = out_dtype or torch.bfloat16
        out = _activation(M, N, out_dtype, x.device)
        mode = 0 if out_dtype == torch.bfloat16 else 1
        if out_dtype not in (torch.bfloat16, torch.float32):
            raise UnsupportedError(f"linear: out dtype {out_dtype}")
    elif epilogue == ADD:
        mode = 2
    elif epilogue == SILU_GATE:
        if N % 16 != 0:
            raise UnsupportedError("linear: the fused gate epilogue needs a multiple of 16 rows")
        out = _activation(M, N // 2, torch.bfloat16, x.device)
        mode = 3
    else:
        raise InvalidError(f"linear: unknown epilogue {epilogue!r}")
    from . import gemm_dispatch
    gemm_dispatch.gemm_bf16(x, weight, out, mode)
    return out


def linear_slices(x: torch.Tensor, weight: torch.Tensor) -> Optional[torch.Tensor]:
    """x . weight^T as float32 partial products over K slices [slices, M, N] (their sum in plane
    order is the product), or None when this product is not cut. Only narrow bfloat16 products
    are cut; rms_norm(partials=...) or add_planes_ adds the planes to the residual stream."""
    _check(x, "x", dims=2)
    _check(weight, "weight", dims=2)
    if weight.shape[1] != x.shape[1]:
        raise InvalidError(f"linear: x has {x.shape[1]} columns, weight has {weight.shape[1]}")
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        return None
    from . import gemm_dispatch
    return gemm_dispatch.gemm_bf16_slices(x, weight)


def add_planes_(x: torch.Tensor, planes: torch.Tensor) -> torch.Tensor:
    """x += planes[0] + planes[1] + ... (in that order); x float32, planes [n, *x.shape] float32."""
    _check(x, "x", torch.float32)
    _check(planes, "planes", torch.float32)
    if tuple(planes.shape[1:]) != tuple(x.shape):
        raise InvalidError(f"add_planes_: planes {tuple(planes.shape)} do not match {tuple(x.shape)}")
    _done(_lib().lrm_add_planes(_ptr(x), _ptr(planes), planes.shape[0], ctypes.c_longlong(x.numel()),
                                _stream()), "add_planes_")
    return x


def scale_(x: torch.Tensor, factor: float) -> torch.Tensor:
    """x *= factor in place (float32)."""
    _check(x, "x", torch.float32)
    _done(_lib().lrm_scale_inplace(_ptr(x), ctypes.c_float(factor), ctypes.c_longlong(x.numel()), _stream()),
          "scale_")
    return x


def silu_mul(gate_up: torch.Tensor, block: int) -> torch.Tensor:
    """silu(gate) * up from [T, 2I] whose columns alternate in blocks of `block` gate / up."""
    _check(gate_up, "gate_up", dims=2)
    inter = gate_up.shape[1] // 2
    if gate_up.shape[1] % 2 or inter % block:
        raise InvalidError("silu_mul: width must be 2*I with I a multiple of the block")
    out = _activation(gate_up.shape[0], inter, gate_up.dtype, gate_up.device)
    _done(_lib().lrm_silu_mul(_ptr(gate_up), _ptr(out), _code(gate_up.dtype),
                              ctypes.c_longlong(gate_up.shape[0]), inter, block, _stream()), "silu_mul")
    return out


def clamped_gate_mul(gate_up: torch.Tensor, block: int, limit: float, alpha: float,
                     out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """g sigmoid(alpha g) (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit), from [T, 2I]
    whose columns alternate in blocks of `block` gate / up (float32, or the output's type)."""
    _check(gate_up, "gate_up", dims=2)
    inter = gate_up.shape[1] // 2
    if gate_up.shape[1] % 2 or inter % block:
        raise InvalidError("clamped_gate_mul: width must be 2*I with I a multiple of the block")
    out_dtype = out_dtype or gate_up.dtype
    out = _activation(gate_up.shape[0], inter, out_dtype, gate_up.device)
    _done(_lib().lrm_clamped_gate_mul(_ptr(gate_up), _code(gate_up.dtype), _ptr(out), _code(out_dtype),
                                      ctypes.c_longlong(gate_up.shape[0]), inter, block, ctypes.c_float(limit),
                                      ctypes.c_float(alpha), _stream()), "clamped_gate_mul")
    return out


def relu_squared(x: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """max(x, 0)^2 elementwise; x [T, I] float32 or the output's type."""
    _check(x, "x", dims=2)
    out_dtype = out_dtype or x.dtype
    out = _activation(x.shape[0], x.shape[1], out_dtype, x.device)
    _done(_lib().lrm_relu_squared(_ptr(x), _code(x.dtype), _ptr(out), _code(out_dtype), ctypes.c_longlong(x.numel()),
                                  _stream()), "relu_squared")
    return out


def gelu_tanh_mul(gate_up: torch.Tensor, block: int, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """gelu(gate) * up with the tanh form of GELU, 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))), from
    [T, 2I] whose columns alternate in blocks of `block` gate / up (float32, or the output's type)."""
    _check(gate_up, "gate_up", dims=2)
    inter = gate_up.shape[1] // 2
    if gate_up.shape[1] % 2 or inter % block:
        raise InvalidError("gelu_tanh_mul: width must be 2*I with I a multiple of the block")
    out_dtype = out_dtype or gate_up.dtype
    out = _activation(gate_up.shape[0], inter, out_dtype, gate_up.device)
    _done(_lib().lrm_gelu_tanh_mul(_ptr(gate_up), _code(gate_up.dtype), _ptr(out), _code(out_dtype),
                                   ctypes.c_longlong(gate_up.shape[0]), inter, block, _stream()), "gelu_tanh_mul")
    return out


def tanh_columns(src: torch.Tensor, column: int, width: int, out_dtype: torch.dtype) -> torch.Tensor:
    """tanh of the columns column .. column + width of src [T, W] -> [T, width] in `out_dtype`."""
    _check(src, "src", dims=2)
    if width <= 0 or column < 0 or column + width > src.shape[1]:
        raise InvalidError("tanh_columns: columns outside the activation")
    out = _activation(src.shape[0], width, out_dtype, src.device)
    _done(_lib().lrm_tanh_columns(_column_ptr(src, column), _code(src.dtype), ctypes.c_longlong(src.shape[1]), _ptr(out),
                                  _code(out_dtype), ctypes.c_longlong(src.shape[0]), width, _stream()), "tanh_columns")
    return out


def token_shift(h: torch.Tensor, mix: torch.Tensor, last: torch.Tensor, cu_seqlens: torch.Tensor,
                seq_of_token: torch.Tensor, slots: torch.Tensor) -> torch.Tensor:
    """h[t] + (h[t-1] - h[t]) * mix per channel, h [T, W] packed sequences; the row before a sequence's
    first token of the step is last[slot] (float32 [slots, 1, W]: the sequence's previous h, zeros at
    its start). The kernel also rewrites `last` with every sequence's newest row of h."""
    _check(h, "h", dims=2)
    _check(mix, "mix", torch.float32, 1)
    _check(last, "last", torch.float32, 3)
    T, W = h.shape
    if mix.numel() != W or tuple(last.shape[1:]) != (1, W):
        raise InvalidError("token_shift: shapes do not agree")
    for name, t in (("cu_seqlens", cu_seqlens), ("seq_of_token", seq_of_token), ("slots", slots)):
        _check(t, name, torch.int32, 1)
    out = _activation(T, W, h.dtype, h.device)
    _done(_lib().lrm_token_shift(_ptr(h), _code(h.dtype), _ptr(mix), _ptr(last), _ptr(out), _ptr(cu_seqlens),
                                 _ptr(seq_of_token), _ptr(slots), T, W, _stream()), "token_shift")
    return out


def scaled_add_(x: torch.Tensor, y: torch.Tensor, factor: torch.Tensor) -> torch.Tensor:
    """x[t, :] += factor * y[t, :] with one factor per column; all float32."""
    _check(x, "x", torch.float32, 2)
    _check(y, "y", torch.float32, 2)
    _check(factor, "factor", torch.float32, 1)
    if x.shape != y.shape or factor.numel() != x.shape[1]:
        raise InvalidError("scaled_add_: shapes do not agree")
    _done(_lib().lrm_scaled_add(_ptr(x), _ptr(y), _ptr(factor), ctypes.c_longlong(x.shape[0]), x.shape[1], _stream()),
          "scaled_add_")
    return x


def scaled_add_norm_(x: torch.Tensor, y: torch.Tensor, factor: torch.Tensor, weight: torch.Tensor, eps: float,
                     out_dtype: torch.dtype) -> torch.Tensor:
    """x[t, :] += factor * y[t, :] (all float32), and in the same pass the updated rows' RMS norm,
    x / sqrt(mean(x^2) + eps) * weight -> [T, W] in `out_dtype`."""
    _check(x, "x", torch.float32, 2)
    _check(y, "y", torch.float32, 2)
    _check(factor, "factor", torch.float32, 1)
    _check(weight, "weight", dims=1)
    if x.shape != y.shape or factor.numel() != x.shape[1] or weight.numel() != x.shape[1]:
        raise InvalidError("scaled_add_norm_: shapes do not agree")
    out = _activation(x.shape[0], x.shape[1], out_dtype, x.device)
    _done(_lib().lrm_scaled_add_norm(_ptr(x), _ptr(y), _ptr(factor), _ptr(weight), _code(weight.dtype),
                                     ctypes.c_float(eps), _ptr(out), _code(out_dtype), ctypes.c_longlong(x.shape[0]),
                                     x.shape[1], _stream()), "scaled_add_norm_")
    return out


def row_gate_(y: torch.Tensor, x: torch.Tensor, weight: torch.Tensor,
              planes: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[t, :] = sigmoid(x[t, :] . weight) * y[t, :] (+ planes[0][t, :] + planes[1][t, :] + ..., in that
    order): y float32 [T, N], x [T, W], weight float32 [W], planes float32 [n, T, N]."""
    _check(y, "y", torch.float32, 2)
    _check(x, "x", dims=2)
    _check(weight, "weight", torch.float32, 1)
    if x.shape[0] != y.shape[0] or weight.numel() != x.shape[1]:
        raise InvalidError("row_gate_: shapes do not agree")
    count = 0
    if planes is not None and planes.shape[0]:
        _check(planes, "planes", torch.float32, 3)
        if tuple(planes.shape[1:]) != tuple(y.shape):
            raise InvalidError("row_gate_: planes must be [n, T, N]")
        count = planes.shape[0]
    _done(_lib().lrm_row_gate(_ptr(y), _ptr(x), _code(x.dtype), _ptr(weight), y.shape[0], x.shape[1], y.shape[1],
                              _ptr(planes if count else None), count, _stream()), "row_gate_")
    return y


def add_(x: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """x += delta, x float32 (the residual sum is always 32-bit)."""
    _check(x, "x", torch.float32)
    _check(delta, "delta")
    if x.shape != delta.shape:
        raise InvalidError(f"add_: shapes {tuple(x.shape)} and {tuple(delta.shape)}")
    _done(_lib().lrm_add_inplace(_ptr(x), _ptr(delta), _code(delta.dtype),
                                 ctypes.c_longlong(x.numel()), _stream()), "add_")
    return x


def cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    _check(x, "x")
    if x.dtype == dtype:
        return x
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    _done(_lib().lrm_cast(_ptr(x), _code(x.dtype), _ptr(out), _code(dtype),
                          ctypes.c_longlong(x.numel()), _stream()), "cast")
    return out


# --------------------------------------------------------------------------- rope + cache store
def rope_store(qkv: torch.Tensor, q_heads: int, kv_heads: int, head_dim: int,
               inv_freq: Optional[torch.Tensor], rotary: int, positions: torch.Tensor,
               kv=None, dest_rows: Optional[torch.Tensor] = None,
               keep_packed: bool = True) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
    """Rotate q and k of a fused [T, (Hq+2Hk)*d] projection and store k, v.

    Returns (q [T,Hq,d], k [T,Hk,d] or None, v [T,Hk,d] or None); k and v are
    returned when `keep_packed`, and written to the paged cache view `kv` at
    `dest_rows` (int32 [T]: page * page_size + row, < 0 = not stored) when given.
    """
    _check(qkv, "qkv", dims=2)
    T = qkv.shape[0]
    if qkv.shape[1] != (q_heads + 2 * kv_heads) * head_dim:
        raise InvalidError("rope_store: qkv width does not match the head geometry")
    if head_dim % 2:
        raise UnsupportedError("rope_store: head size must be even")
    _check(positions, "positions", torch.int32, 1)
    if inv_freq is not None:
        _check(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.numel() != rotary // 2:
            raise InvalidError("rope_store: inv_freq must have rotary/2 entries")
    dev = qkv.device
    q = torch.empty((T, q_heads, head_dim), dtype=qkv.dtype, device=dev)
    k = torch.empty((T, kv_heads, head_dim), dtype=qkv.dtype, device=dev) if keep_packed else None
    v = torch.empty((T, kv_heads, head_dim), dtype=qkv.dtype, device=dev) if keep_packed else None
    k_pages = v_pages = None
    page_size = 1
    if kv is not None:
        k_pages, v_pages, page_size = kv.k, kv.v, kv.page_size
        _check(k_pages, "k pages", qkv.dtype, 4)
        _check(v_pages, "v pages", qkv.dtype, 4)
        _check(dest_rows, "dest_rows", torch.int32, 1)
        if dest_rows.numel() != T:
            raise InvalidError("rope_store: one destination row per token")
        if tuple(k_pages.shape[1:]) != (kv_heads, page_size, head_dim):
            raise InvalidError("rope_store: cache pages do not match the head geometry")
    _done(_lib().lrm_rope_store(_ptr(qkv), _code(qkv.dtype), _ptr(q), _ptr(k), _ptr(v),
                                _ptr(k_pages), _ptr(v_pages), _ptr(dest_rows if kv is not None else None),
                                _ptr(positions), _ptr(inv_freq), rotary, T, q_heads,
                                kv_heads, head_dim, page_size, _stream()), "rope_store")
    return q, k, v


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """float32 [T, R/2, 2]: (cos, sin) of float32(position) * inv_freq, the angles rope_store forms."""
    _check(positions, "positions", torch.int32, 1)
    _check(inv_freq, "inv_freq", torch.float32, 1)
    T, half = positions.numel(), inv_freq.numel()
    table = torch.empty((T, half, 2), dtype=torch.float32, device=positions.device)
    _done(_lib().lrm_rope_table(_ptr(positions), _ptr(inv_freq), _ptr(table), T, half, _stream()), "rope_table")
    return table


def linear_rope_store(x: torch.Tensor, weight: torch.Tensor, q_heads: int, kv_heads: int, head_dim: int,
                      table: Optional[torch.Tensor], kv=None, dest_rows: Optional[torch.Tensor] = None):
    """rope_store(linear(x, weight)) for a prompt in one launch where the tensor-core product takes
    the shape: (q [T,Hq,d], k [T,Hk,d], v [T,Hk,d]), with k and v also written to the cache view
    `kv` at `dest_rows`; None where it does not (nothing was launched). `table` from rope_table
    (rotation of the whole head) or None (no rotation). Bit-equal to the two separate kernels."""
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or x.dim() != 2:
        return None
    T = x.shape[0]
    if table is not None and tuple(table.shape) != (T, head_dim // 2, 2):
        return None
    if kv is not None and (kv.k.dtype != torch.bfloat16 or tuple(kv.k.shape[1:]) != (kv_heads, kv.page_size, head_dim)):
        return None
    q = torch.empty((T, q_heads, head_dim), dtype=x.dtype, device=x.device)
    k = torch.empty((T, kv_heads, head_dim), dtype=x.dtype, device=x.device)
    v = torch.empty((T, kv_heads, head_dim), dtype=x.dtype, device=x.device)
    from . import gemm_dispatch
    if not gemm_dispatch.gemm_bf16_qkv(x, weight, q, k, v, kv, dest_rows, table):
        return None
    return q, k, v


def qkv_bias_store(qkv: torch.Tensor, bias: Optional[torch.Tensor], q_heads: int, kv_heads: int, head_dim: int,
                   value_dim: int, kv=None, dest_rows: Optional[torch.Tensor] = None, keep_packed: bool = True):
    """Split a fused [T, Hq*d + Hk*d + Hk*dv] projection without rotation (value_dim 0: a projection
    without values; v is then None and nothing is stored as values): add `bias` (float32, the
    row's width, or None), and return (q [T,Hq,d], k [T,Hk,d] or None, v [T,Hk,dv] or None); k and
    v are returned when `keep_packed`, and written to the paged cache view `kv` at `dest_rows`
    when given (see rope_store)."""
    _check(qkv, "qkv", dims=2)
    T = qkv.shape[0]
    width = q_heads * head_dim + kv_heads * (head_dim + value_dim)
    if qkv.shape[1] != width:
        raise InvalidError("qkv_bias_store: qkv width does not match the head geometry")
    if bias is not None:
        _check(bias, "bias", torch.float32, 1)
        if bias.numel() != width:
            raise InvalidError("qkv_bias_store: one bias per projected column")
    dev = qkv.device
    q = torch.empty((T, q_heads, head_dim), dtype=qkv.dtype, device=dev)
    k = torch.empty((T, kv_heads, head_dim), dtype=qkv.dtype, device=dev) if keep_packed else None
    v = torch.empty((T, kv_heads, value_dim), dtype=qkv.dtype, device=dev) if keep_packed and value_dim else None
    k_pages = v_pages = None
    page_size = 1
    if kv is not None and kv_heads > 0:
        k_pages, v_pages, page_size = kv.k, kv.v if value_dim else None, kv.page_size
        _check(k_pages, "k pages", qkv.dtype, 4)
        if value_dim:
            _check(v_pages, "v pages", qkv.dtype, 4)
        _check(dest_rows, "dest_rows", torch.int32, 1)
        if dest_rows.numel() != T:
            raise InvalidError("qkv_bias_store: one destination row per token")
        if (tuple(k_pages.shape[1:]) != (kv_heads, page_size, head_dim)
                or (value_dim and tuple(v_pages.shape[1:]) != (kv_heads, page_size, value_dim))):
            raise InvalidError("qkv_bias_store: cache pages do not match the head geometry")
    _done(_lib().lrm_qkv_bias_store(_ptr(qkv), _code(qkv.dtype), _ptr(bias), _ptr(q), _ptr(k), _ptr(v),
                                    _ptr(k_pages), _ptr(v_pages), _ptr(dest_rows if k_pages is not None else None),
                                    T, q_heads, kv_heads, head_dim, value_dim, page_size, _stream()),
          "qkv_bias_store")
    return q, k, v


def shaped_qkv_store(qkv: torch.Tensor, q_heads: int, kv_heads: int, head_dim: int, value_dim: int,
                     positions: torch.Tensor, out_dtype: torch.dtype, bias: Optional[torch.Tensor] = None,
                     taps: Optional[torch.Tensor] = None, tails: Optional[torch.Tensor] = None,
                     cu_seqlens: Optional[torch.Tensor] = None, seq_of_token: Optional[torch.Tensor] = None,
                     slots: Optional[torch.Tensor] = None, row_norm=None, row_eps: float = 0.0,
                     inv_freq: Optional[torch.Tensor] = None, rotary: int = 0, adjacent_pairs: bool = False,
                     head_norm_eps: Optional[float] = None, kv=None, dest_rows: Optional[torch.Tensor] = None,
                     keep_packed: bool = True):
    """Split a fused [T, Hq*d + Hk*d + Hk*dv] projection (float32, or `out_dtype`) whose queries and
    keys are shaped on the way, each step only if asked for and in this order: `bias` (float32
    [row]); a causal convolution per channel (`taps` float32 [n, row], the last row the current
    token's, with the sequences' `tails`
    float32 [slots, n - 1, row] of unbiased projections, rewritten afterwards); an RMS norm over all
    query columns and one over all key columns (`row_norm` = (q weight, k weight), `row_eps`); the
    rotation of each head's first `rotary` dimensions by `inv_freq` (float64 [rotary/2]; split halves,
    or neighbours with `adjacent_pairs`); each head divided by its root mean square
    (`head_norm_eps`). Returns (q [T,Hq,d], k, v) like qkv_bias_store, and writes the cache view."""
    _check(qkv, "qkv", dims=2)
    T = qkv.shape[0]
    width = q_heads * head_dim + kv_heads * (head_dim + value_dim)
    if qkv.shape[1] != width:
        raise InvalidError("shaped_qkv_store: qkv width does not match the head geometry")
    _check(positions, "positions", torch.int32, 1)
    if bias is not None:
        _check(bias, "bias", torch.float32, 1)
        if bias.numel() != width:
            raise InvalidError("shaped_qkv_store: one bias per projected column")
    n = 0
    if taps is not None:
        _check(taps, "taps", torch.float32, 2)
        n = taps.shape[0]
        if taps.shape[1] != width:
            raise InvalidError("shaped_qkv_store: one tap per projected column in every row of taps")
        if n > 1:
            _check(tails, "tails", torch.float32, 3)
            if tuple(tails.shape[1:]) != (n - 1, width):
                raise InvalidError("shaped_qkv_store: tails must be [slots, taps - 1, row]")
            for name, t in (("cu_seqlens", cu_seqlens), ("seq_of_token", seq_of_token), ("slots", slots)):
                _check(t, name, torch.int32, 1)
    q_norm = k_norm = None
    if row_norm is not None:
        q_norm, k_norm = row_norm
        _check(q_norm, "q norm", torch.float32, 1)
        if q_norm.numel() != q_heads * head_dim:
            raise InvalidError("shaped_qkv_store: the query norm's weight covers all query columns")
        if kv_heads:
            _check(k_norm, "k norm", torch.float32, 1)
            if k_norm.numel() != kv_heads * head_dim:
                raise InvalidError("shaped_qkv_store: the key norm's weight covers all key columns")
        else:
            k_norm = None
    if rotary:
        _check(inv_freq, "inv_freq", torch.float64, 1)
        if inv_freq.numel() != rotary // 2 or rotary % 2 or rotary > head_dim:
            raise InvalidError("shaped_qkv_store: one frequency per rotated pair")
    dev = qkv.device
    q = torch.empty((T, q_heads, head_dim), dtype=out_dtype, device=dev)
    k = torch.empty((T, kv_heads, head_dim), dtype=out_dtype, device=dev) if keep_packed and kv_heads else None
    v = torch.empty((T, kv_heads, value_dim), dtype=out_dtype, device=dev) if keep_packed and kv_heads and value_dim else None
    k_pages = v_pages = None
    page_size = 1
    if kv is not None and kv_heads > 0:
        k_pages, v_pages, page_size = kv.k, kv.v if value_dim else None, kv.page_size
        _check(k_pages, "k pages", out_dtype, 4)
        if value_dim:
            _check(v_pages, "v pages", out_dtype, 4)
        _check(dest_rows, "dest_rows", torch.int32, 1)
        if dest_rows.numel() != T:
            raise InvalidError("shaped_qkv_store: one destination row per token")
        if (tuple(k_pages.shape[1:]) != (kv_heads, page_size, head_dim)
                or (value_dim and tuple(v_pages.shape[1:]) != (kv_heads, page_size, value_dim))):
            raise InvalidError("shaped_qkv_store: cache pages do not match the head geometry")
    _done(_lib().lrm_shaped_qkv_store(
        _ptr(qkv), _code(qkv.dtype), _ptr(bias), _ptr(taps), n, _ptr(tails if n > 1 else None),
        _ptr(cu_seqlens if n > 1 else None), _ptr(seq_of_token if n > 1 else None), _ptr(slots if n > 1 else None),
        _ptr(positions), _ptr(q_norm), _ptr(k_norm), ctypes.c_float(row_eps), _ptr(inv_freq if rotary else None),
        rotary, int(bool(adjacent_pairs)), int(head_norm_eps is not None),
        ctypes.c_float(head_norm_eps if head_norm_eps is not None else 0.0), _ptr(q), _ptr(k), _ptr(v),
        _ptr(k_pages), _ptr(v_pages), _ptr(dest_rows if k_pages is not None else None), _code(out_dtype), T, q_heads,
        kv_heads, head_dim, value_dim, page_size, _stream()), "shaped_qkv_store")
    if n > 1:
        conv_tail_update_(qkv, 0, width, n, tails, cu_seqlens, slots)
    return q, k, v


# --------------------------------------------------------------------------- fixed-size state mixers
def _f32(shape, device) -> torch.Tensor:
    return torch.empty(shape, dtype=torch.float32, device=device)


def _column_ptr(t: torch.Tensor, column: int) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr() + column * t.element_size())


def retention_prepare(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, heads: int, head_dim: int,
                      value_dim: int, positions: torch.Tensor, inv_freq: Optional[torch.Tensor], rotary: int,
                      k_scale: float):
    """From a fused projection [T, W] (q at column q_off, k at k_off, both [heads*d]; v at v_off
    [heads*dv]): float32 q and k rotated on their first `rotary` dimensions (split-half, angle =
    position * inv_freq), k times k_scale, and v widened. -> q, k [T,H,d], v [T,H,dv]."""
    _check(proj, "proj", dims=2)
    _check(positions, "positions", torch.int32, 1)
    T = proj.shape[0]
    if rotary:
        _check(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.numel() != rotary // 2:
            raise InvalidError("retention_prepare: inv_freq must have rotary/2 entries")
    if max(q_off, k_off) + heads * head_dim > proj.shape[1] or v_off + heads * value_dim > proj.shape[1]:
        raise InvalidError("retention_prepare: columns outside the projection")
    q, k = _f32((T, heads, head_dim), proj.device), _f32((T, heads, head_dim), proj.device)
    v = _f32((T, heads, value_dim), proj.device)
    _done(_lib().lrm_retention_prepare(_ptr(proj), _code(proj.dtype), ctypes.c_longlong(proj.shape[1]), q_off, k_off,
                                       v_off, _ptr(positions), _ptr(inv_freq if rotary else None), rotary,
                                       ctypes.c_float(k_scale), _ptr(q), _ptr(k), _ptr(v), T, heads, head_dim,
                                       value_dim, _stream()), "retention_prepare")
    return q, k, v


def delta_prepare(proj: torch.Tensor, conv_off: int, b_off: int, a: torch.Tensor, dt_bias: torch.Tensor,
                  rate: torch.Tensor, taps: torch.Tensor, tails: torch.Tensor, cu_seqlens: torch.Tensor,
                  seq_of_token: torch.Tensor, slots: torch.Tensor, heads: int, kv_heads: int, head_dim: int,
                  value_dim: int, unit_eps: float, q_scale: float):
    """Inputs of the gated delta rule from a fused projection [T, W]: the columns conv_off .. (q | k
    | v channels) pass a short causal convolution (taps float32 [C, n]; inputs before the step come
    from, and afterwards go to, `tails` float32 [slots, n-1, C]) and SiLU; q and k become unit
    vectors per head (q also times q_scale); g = exp(-rate_h softplus(a + dt_bias)) per head and key
    channel (a: the first H*d columns of a float32 [T, >= H*d] activation); b = sigmoid of the H
    columns at b_off.
    -> q, k [T,G,d], v [T,H,dv], g [T,H,d], b [T,H], all float32."""
    _check(proj, "proj", dims=2)
    T = proj.shape[0]
    C = 2 * kv_heads * head_dim + heads * value_dim
    _check(a, "a", torch.float32, 2)
    _check(dt_bias, "dt_bias", torch.float32, 1)
    _check(rate, "rate", torch.float32, 1)
    _check(taps, "taps", torch.float32, 2)
    _check(tails, "tails", torch.float32, 3)
    n = taps.shape[1]
    for name, t in (("cu_seqlens", cu_seqlens), ("seq_of_token", seq_of_token), ("slots", slots)):
        _check(t, name, torch.int32, 1)
    if (a.shape[0] != T or a.shape[1] < heads * head_dim or dt_bias.numel() != heads * head_dim or rate.numel() != heads
            or taps.shape[0] != C or tuple(tails.shape[1:]) != (max(n - 1, 0), C)
            or conv_off + C > proj.shape[1] or b_off + heads > proj.shape[1]):
        raise InvalidError("delta_prepare: shapes do not agree")
    dev = proj.device
    q, k = _f32((T, kv_heads, head_dim), dev), _f32((T, kv_heads, head_dim), dev)
    v, g, b = _f32((T, heads, value_dim), dev), _f32((T, heads, head_dim), dev), _f32((T, heads), dev)
    _done(_lib().lrm_delta_prepare(_ptr(proj), _code(proj.dtype), ctypes.c_longlong(proj.shape[1]), conv_off, b_off,
                                   _ptr(a), ctypes.c_longlong(a.shape[1]), _ptr(dt_bias), _ptr(rate), _ptr(taps), n, _ptr(tails), _ptr(cu_seqlens),
                                   _ptr(seq_of_token), _ptr(slots), _ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(b), T,
                                   slots.numel(), heads, kv_heads, head_dim, value_dim, ctypes.c_float(unit_eps),
                                   ctypes.c_float(q_scale), _stream()), "delta_prepare", launches=2 if n > 1 else 1)
    return q, k, v, g, b


def linear_state_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, state: torch.Tensor,
                      cu_seqlens: torch.Tensor, slots: torch.Tensor, head_decay: Optional[torch.Tensor] = None,
                      g: Optional[torch.Tensor] = None, beta: Optional[torch.Tensor] = None,
                      token_decay: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Token-by-token update and read-out of a per-sequence, per-head matrix state (float32
    [slots, H, d, dv], updated in place). With `head_decay` [H]: S <- a S + k v^T. With `token_decay`
    [T,H]: S <- a_t S + k v^T, one decay per head and token. With `g` [T,H,d]
    and `beta` [T,H]: S <- diag(g) S, then S <- S + k (beta (v - S^T k))^T. o = S^T q after the
    update. q, k float32 [T,KH,d] (query head h reads q/k head h // (H/KH)), v float32 [T,H,dv].
    -> o float32 [T,H,dv]."""
    for name, t, dims in (("q", q, 3), ("k", k, 3), ("v", v, 3), ("state", state, 4)):
        _check(t, name, torch.float32, dims)
    _check(cu_seqlens, "cu_seqlens", torch.int32, 1)
    _check(slots, "slots", torch.int32, 1)
    T, KH, d = q.shape
    H, dv = v.shape[1], v.shape[2]
    if k.shape != q.shape or v.shape[0] != T or tuple(state.shape[1:]) != (H, d, dv) or H % KH:
        raise InvalidError("linear_state_scan: shapes do not agree")
    if (g is not None) + (head_decay is not None) + (token_decay is not None) != 1:
        raise InvalidError("linear_state_scan: give head_decay, token_decay, or g and beta")
    if token_decay is not None:
        _check(token_decay, "token_decay", torch.float32, 2)
        if tuple(token_decay.shape) != (T, H):
            raise InvalidError("linear_state_scan: token_decay must be [T,H]")
        beta = token_decay  # the kernel reads the decays where the delta rule's step sizes would be
    elif g is not None:
        _check(g, "g", torch.float32, 3)
        _check(beta, "beta", torch.float32, 2)
        if tuple(g.shape) != (T, H, d) or tuple(beta.shape) != (T, H):
            raise InvalidError("linear_state_scan: g must be [T,H,d] and beta [T,H]")
    else:
        _check(head_decay, "head_decay", torch.float32, 1)
        if head_decay.numel() != H:
            raise InvalidError("linear_state_scan: one decay per head")
    out = _f32((T, H, dv), q.device)
    _done(_lib().lrm_linear_state_scan(_ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(head_decay), _ptr(beta), _ptr(state),
                                       _ptr(out), _ptr(cu_seqlens), _ptr(slots), slots.numel(), H, KH, d, dv,
                                       _stream()), "linear_state_scan")
    return out


def general_delta_prepare(proj: torch.Tensor, r_off: int, k_off: int, v_off: int, a_off: int, z: torch.Tensor,
                          z_bias: torch.Tensor, a_bias: torch.Tensor, decay_scale: float, unit_eps: float,
                          heads: int, head_dim: int, value_dim: int):
    """Inputs of the generalized delta rule from a fused projection [T, W] (r, k, a at their columns,
    each [heads*d]; v [heads*dv]) and the decay's float32 pre-activation z [T, heads*d]:
    g = exp(-decay_scale sigmoid(z + z_bias)), look = k / sqrt(sum k^2 + unit_eps) per head,
    put = -sigmoid(a + a_bias) look. -> r, k, v, g, look, put, all float32 [T, heads, d or dv]."""
    _check(proj, "proj", dims=2)
    _check(z, "z", torch.float32, 2)
    T, W = proj.shape
    n = heads * head_dim
    for name, t in (("z_bias", z_bias), ("a_bias", a_bias)):
        _check(t, name, torch.float32, 1)
        if t.numel() != n:
            raise InvalidError(f"general_delta_prepare: {name} has one entry per head and key channel")
    if tuple(z.shape) != (T, n) or max(r_off, k_off, a_off) + n > W or v_off + heads * value_dim > W:
        raise InvalidError("general_delta_prepare: columns outside the projection")
    dev = proj.device
    r, k, g, look, put = (_f32((T, heads, head_dim), dev) for _ in range(5))
    v = _f32((T, heads, value_dim), dev)
    _done(_lib().lrm_general_delta_prepare(_ptr(proj), _code(proj.dtype), ctypes.c_longlong(W), r_off, k_off, v_off,
                                           a_off, _ptr(z), _ptr(z_bias), _ptr(a_bias), ctypes.c_float(decay_scale),
                                           ctypes.c_float(unit_eps), _ptr(r), _ptr(k), _ptr(v), _ptr(g), _ptr(look),
                                           _ptr(put), T, heads, head_dim, value_dim, _stream()),
          "general_delta_prepare")
    return r, k, v, g, look, put


def general_delta_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, look: torch.Tensor,
                       put: torch.Tensor, state: torch.Tensor, cu_seqlens: torch.Tensor,
                       slots: torch.Tensor) -> torch.Tensor:
    """The generalized delta rule on the per-sequence, per-head matrix state (float32 [slots, H, d, dv],
    updated in place): S <- diag(g) S + put (look^T S) + k v^T, both terms reading the old S; o = S^T q
    after the update. q, k, g, look, put float32 [T,H,d], v float32 [T,H,dv]. -> o float32 [T,H,dv]."""
    for name, t, dims in (("q", q, 3), ("k", k, 3), ("v", v, 3), ("g", g, 3), ("look", look, 3), ("put", put, 3),
                          ("state", state, 4)):
        _check(t, name, torch.float32, dims)
    _check(cu_seqlens, "cu_seqlens", torch.int32, 1)
    _check(slots, "slots", torch.int32, 1)
    T, H, d = q.shape
    dv = v.shape[2]
    if any(t.shape != q.shape for t in (k, g, look, put)) or tuple(v.shape[:2]) != (T, H) \
            or tuple(state.shape[1:]) != (H, d, dv):
        raise InvalidError("general_delta_scan: shapes do not agree")
    out = _f32((T, H, dv), q.device)
    _done(_lib().lrm_general_delta_scan(_ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(look), _ptr(put), _ptr(state),
                                        _ptr(out), _ptr(cu_seqlens), _ptr(slots), slots.numel(), H, d, dv, _stream()),
          "general_delta_scan")
    return out


def conv_tail_update_(proj: torch.Tensor, column: int, channels: int, taps: int, tails: torch.Tensor,
                      cu_seqlens: torch.Tensor, slots: torch.Tensor) -> None:
    """Every sequence's tail [slots, taps - 1, channels] becomes the last taps - 1 inputs (columns
    column .. column + channels of proj [T, W]) its sequence has seen, after a kernel of the caller
    made the convolution itself."""
    if taps <= 1:
        return
    _check(proj, "proj", dims=2)
    _check(tails, "tails", torch.float32, 3)
    if column + channels > proj.shape[1] or tuple(tails.shape[1:]) != (taps - 1, channels):
        raise InvalidError("conv_tail_update_: shapes do not agree")
    _done(_lib().lrm_conv_tail_update(_ptr(proj), _code(proj.dtype), ctypes.c_longlong(proj.shape[1]), column,
                                      channels, taps, _ptr(tails), _ptr(cu_seqlens), _ptr(slots), slots.numel(),
                                      _stream()), "conv_tail_update_")


def ssd_prepare(proj: torch.Tensor, conv_off: int, dt_off: int, dt_bias: torch.Tensor, rate: torch.Tensor,
                taps: torch.Tensor, conv_bias: Optional[torch.Tensor], tails: Optional[torch.Tensor],
                cu_seqlens: torch.Tensor, seq_of_token: torch.Tensor, slots: torch.Tensor, heads: int, groups: int,
                state: int, value_dim: int):
    """Inputs of a state-space mixer from its projection [T, W]: the heads * value_dim + 2 groups *
    state channels at conv_off (x | B | C) pass a causal convolution (taps float32 [C, n], bias,
    inputs before the step from `tails` [slots, n - 1, C], which is only read) and SiLU; dt =
    softplus(dt + dt_bias) from the `heads` columns at dt_off; decay = exp(-rate dt).
    -> q (= C), k (= B) [T,G,N], v (= dt x), x [T,H,dv], decay [T,H], all float32."""
    _check(proj, "proj", dims=2)
    T = proj.shape[0]
    C = heads * value_dim + 2 * groups * state
    for name, t in (("dt_bias", dt_bias), ("rate", rate)):
        _check(t, name, torch.float32, 1)
        if t.numel() != heads:
            raise InvalidError(f"ssd_prepare: one entry of {name} per head")
    _check(taps, "taps", torch.float32, 2)
    n = taps.shape[1]
    if conv_bias is not None:
        _check(conv_bias, "conv_bias", torch.float32, 1)
    if n > 1:
        _check(tails, "tails", torch.float32, 3)
    for name, t in (("cu_seqlens", cu_seqlens), ("seq_of_token", seq_of_token), ("slots", slots)):
        _check(t, name, torch.int32, 1)
    if (taps.shape[0] != C or conv_off + C > proj.shape[1] or dt_off + heads > proj.shape[1] or heads % groups
            or (conv_bias is not None and conv_bias.numel() != C)
            or (n > 1 and tuple(tails.shape[1:]) != (n - 1, C))):
        raise InvalidError("ssd_prepare: shapes do not agree")
    dev = proj.device
    q, k = _f32((T, groups, state), dev), _f32((T, groups, state), dev)
    v, x, decay = _f32((T, heads, value_dim), dev), _f32((T, heads, value_dim), dev), _f32((T, heads), dev)
    _done(_lib().lrm_ssd_prepare(_ptr(proj), _code(proj.dtype), ctypes.c_longlong(proj.shape[1]), conv_off, dt_off,
                                 _ptr(dt_bias), _ptr(rate), _ptr(taps), _ptr(conv_bias), n,
                                 _ptr(tails) if n > 1 else ctypes.c_void_p(0), _ptr(cu_seqlens), _ptr(seq_of_token),
                                 _ptr(slots), _ptr(q), _ptr(k), _ptr(v), _ptr(x), _ptr(decay), T, heads, groups, state,
                                 value_dim, _stream()), "ssd_prepare")
    return q, k, v, x, decay


def skip_gate_part_norm(o: torch.Tensor, x: torch.Tensor, skip: torch.Tensor, z: torch.Tensor, z_column: int,
                        weight: torch.Tensor, parts: int, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """y = (o + skip_h x) * silu(z), each of `parts` equal parts of a row divided by its own root mean
    square (eps inside the root), times weight. o, x float32 [T,H,dv]; skip float32 [H]; z: the H*dv
    columns at z_column of an activation [T, W]; weight float32 [H*dv]. -> [T, H*dv] in out_dtype."""
    _check(o, "o", torch.float32, 3)
    _check(x, "x", torch.float32, 3)
    _check(skip, "skip", torch.float32, 1)
    _check(weight, "weight", torch.float32, 1)
    _check(z, "z", dims=2)
    T, H, dv = o.shape
    inner = H * dv
    if (x.shape != o.shape or skip.numel() != H or weight.numel() != inner or z.shape[0] != T
            or z_column + inner > z.shape[1] or parts <= 0 or inner % parts):
        raise InvalidError("skip_gate_part_norm: shapes do not agree")
    out = _activation(T, inner, out_dtype, o.device)
    _done(_lib().lrm_skip_gate_part_norm(_ptr(o), _ptr(x), _ptr(skip), _column_ptr(z, z_column), _code(z.dtype),
                                         ctypes.c_longlong(z.shape[1]), _ptr(weight), _ptr(out), _code(out_dtype), T,
                                         inner, dv, parts, ctypes.c_float(eps), _stream()), "skip_gate_part_norm")
    return out


def capped_gates(gates: torch.Tensor, i_column: int, f_column: int, i_bias: torch.Tensor, f_bias: torch.Tensor,
                 cap: float, top: torch.Tensor, cu_seqlens: torch.Tensor, slots: torch.Tensor):
    """Stabilized exponential gates of a matrix memory. From pre-activations (columns i_column + h and
    f_column + h of gates [T, W]): i = cap tanh((. + i_bias) / cap), f = logsigmoid(cap tanh((. +
    f_bias) / cap)); the running maximum m <- max(f + m, i) is carried in `top` float32 [slots, H].
    -> decay = exp(f + m_before - m), take = exp(i - m), floor = exp(-m), float32 [T,H] each."""
    _check(gates, "gates", dims=2)
    _check(i_bias, "i_bias", torch.float32, 1)
    _check(f_bias, "f_bias", torch.float32, 1)
    _check(top, "top", torch.float32, 2)
    _check(cu_seqlens, "cu_seqlens", torch.int32, 1)
    _check(slots, "slots", torch.int32, 1)
    T, H = gates.shape[0], i_bias.numel()
    if f_bias.numel() != H or top.shape[1] != H or max(i_column, f_column) + H > gates.shape[1]:
        raise InvalidError("capped_gates: shapes do not agree")
    decay, take, floor = (_f32((T, H), gates.device) for _ in range(3))
    _done(_lib().lrm_mlstm_gates(_ptr(gates), _code(gates.dtype), ctypes.c_longlong(gates.shape[1]), i_column,
                                 f_column, _ptr(i_bias), _ptr(f_bias), ctypes.c_float(cap), _ptr(top),
                                 _ptr(cu_seqlens), _ptr(slots), _ptr(decay), _ptr(take), _ptr(floor), slots.numel(), H,
                                 T, _stream()), "capped_gates")
    return decay, take, floor


def memory_prepare(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, take: torch.Tensor, q_scale: float,
                   heads: int, head_dim: int, value_dim: int, padded: int):
    """Float32 inputs of a matrix memory's scan from its projection [T, W]: q (heads * head_dim columns
    at q_off) times q_scale, k, and v' = take [v | 1 | 0 ..] of `padded` > value_dim columns per head:
    the 1 carries the normalizer through the scan as one more value column.
    -> q, k [T,H,d], v' [T,H,padded]."""
    _check(proj, "proj", dims=2)
    _check(take, "take", torch.float32, 2)
    T = proj.shape[0]
    if (tuple(take.shape) != (T, heads) or padded <= value_dim
            or max(q_off, k_off) + heads * head_dim > proj.shape[1] or v_off + heads * value_dim > proj.shape[1]):
        raise InvalidError("memory_prepare: shapes do not agree")
    dev = proj.device
    q, k = _f32((T, heads, head_dim), dev), _f32((T, heads, head_dim), dev)
    v = _f32((T, heads, padded), dev)
    _done(_lib().lrm_mlstm_prepare(_ptr(proj), _code(proj.dtype), ctypes.c_longlong(proj.shape[1]), q_off, k_off,
                                   v_off, _ptr(take), ctypes.c_float(q_scale), _ptr(q), _ptr(k), _ptr(v), T, heads,
                                   head_dim, value_dim, padded, _stream()), "memory_prepare")
    return q, k, v


def short_conv(src: torch.Tensor, column: int, channels: int, in_bias: Optional[torch.Tensor], taps: torch.Tensor,
               conv_bias: Optional[torch.Tensor], tails: torch.Tensor, cu_seqlens: torch.Tensor,
               seq_of_token: torch.Tensor, slots: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """A causal convolution per channel over the columns column .. column + channels of src [T, W]
    (+ in_bias, float32 [channels]): taps float32 [channels, n], the last tap on the current token,
    zeros before a sequence's start; + conv_bias. Inputs before the step come from, and the step's
    last n - 1 inputs go to, `tails` float32 [slots, n - 1, channels]. -> [T, channels] in out_dtype."""
    _check(src, "src", dims=2)
    _check(taps, "taps", torch.float32, 2)
    T = src.shape[0]
    n = taps.shape[1]
    for name, t in (("cu_seqlens", cu_seqlens), ("seq_of_token", seq_of_token), ("slots", slots)):
        _check(t, name, torch.int32, 1)
    for name, t in (("in_bias", in_bias), ("conv_bias", conv_bias)):
        if t is not None:
            _check(t, name, torch.float32, 1)
            if t.numel() != channels:
                raise InvalidError(f"short_conv: {name} must have one entry per channel")
    if n > 1:
        _check(tails, "tails", torch.float32, 3)
    if taps.shape[0] != channels or column + channels > src.shape[1] or \
            (n > 1 and tuple(tails.shape[1:]) != (n - 1, channels)):
        raise InvalidError("short_conv: shapes do not agree")
    out = _activation(T, channels, out_dtype, src.device)
    _done(_lib().lrm_short_conv(_ptr(src), _code(src.dtype), ctypes.c_longlong(src.shape[1]), column, _ptr(in_bias),
                                _ptr(taps), _ptr(conv_bias), n, _ptr(tails) if n > 1 else ctypes.c_void_p(0),
                                _ptr(cu_seqlens), _ptr(seq_of_token), _ptr(slots), _ptr(out), _code(out_dtype), T,
                                slots.numel(), channels, _stream()), "short_conv", launches=2 if n > 1 else 1)
    return out


def gated_linear_scan(u: torch.Tensor, gates: torch.Tensor, y: torch.Tensor, y_column: int,
                      y_bias: Optional[torch.Tensor], rate: torch.Tensor, state: torch.Tensor,
                      cu_seqlens: torch.Tensor, slots: torch.Tensor, longest: int, blocks: int) -> torch.Tensor:
    """S <- a S + sqrt(1 - a^2) (i u) per channel with a = exp(-rate sigmoid(gr)), i = sigmoid(gi); the
    result is S gelu_tanh(y + y_bias). u [T, C] (activation type); gates float32 [T, 2C], per block of
    C / blocks channels its gr then its gi; y: columns y_column .. of a float32 [T, W] activation;
    rate float32 [C]; state float32 [slots, C], updated in place. `longest`: most tokens of one
    sequence in the step (launch geometry only). -> [T, C] in u's type."""
    _check(u, "u", dims=2)
    T, C = u.shape
    _check(gates, "gates", torch.float32, 2)
    _check(y, "y", torch.float32, 2)
    _check(rate, "rate", torch.float32, 1)
    _check(state, "state", torch.float32, 2)
    _check(cu_seqlens, "cu_seqlens", torch.int32, 1)
    _check(slots, "slots", torch.int32, 1)
    if y_bias is not None:
        _check(y_bias, "y_bias", torch.float32, 1)
    if (tuple(gates.shape) != (T, 2 * C) or y.shape[0] != T or y_column + C > y.shape[1] or rate.numel() != C
            or state.shape[1] != C or C % blocks or (y_bias is not None and y_bias.numel() != C)):
        raise InvalidError("gated_linear_scan: shapes do not agree")
    out = _activation(T, C, u.dtype, u.device)
    _done(_lib().lrm_gated_linear_scan(_ptr(u), _code(u.dtype), _ptr(gates), _ptr(y), ctypes.c_longlong(y.shape[1]),
                                       y_column, _ptr(y_bias), _ptr(rate), _ptr(state), _ptr(out), _ptr(cu_seqlens),
                                       _ptr(slots), slots.numel(), longest, C, blocks, _stream()),
          "gated_linear_scan")
    return out


def blockwise_linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                     row_scale: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
                     x_column: int = 0, x_block: Optional[int] = None, out: Optional[torch.Tensor] = None,
                     out_column: int = 0, out_block: Optional[int] = None) -> torch.Tensor:
    """out[t, b, :] = (weight[b] . x[t, b, :] + bias[b]) * row_scale[t, b] with weight [B, n, m] ([out,
    in] per block), bias float32 [B, n], row_scale float32 [T, B] (or [T, B * n]: one factor per output). Block b of row t of x [T, W] starts
    at column x_column + b * x_block (default: m, blocks side by side); the result goes to a new
    [T, B * n] tensor in out_dtype, or into `out` [T, W'] at column out_column + b * out_block."""
    _check(x, "x", dims=2)
    _check(weight, "weight", dims=3)
    T = x.shape[0]
    B, n, m = weight.shape
    x_block = m if x_block is None else x_block
    if x_column + (B - 1) * x_block + m > x.shape[1]:
        raise InvalidError("blockwise_linear: blocks outside the input row")
    if bias is not None:
        _check(bias, "bias", torch.float32, 2)
        if tuple(bias.shape) != (B, n):
            raise InvalidError("blockwise_linear: bias must be [blocks, out]")
    if row_scale is not None:
        _check(row_scale, "row_scale", torch.float32, 2)
        if tuple(row_scale.shape) not in ((T, B), (T, B * n)):
            raise InvalidError("blockwise_linear: row_scale must be [T, blocks] or [T, blocks * out]")
    if out is None:
        out = _activation(T, B * n, out_dtype or x.dtype, x.device)
        out_column, out_block = 0, n
    else:
        _check(out, "out", dims=2)
        out_block = n if out_block is None else out_block
        if out.shape[0] != T or out_column + (B - 1) * out_block + n > out.shape[1]:
            raise InvalidError("blockwise_linear: blocks outside the output row")
    _done(_lib().lrm_blockwise_linear(_column_ptr(x, x_column), _code(x.dtype), ctypes.c_longlong(x.shape[1]),
                                      ctypes.c_longlong(x_block), _ptr(weight), _code(weight.dtype), _ptr(bias),
                                      _ptr(row_scale), n if row_scale is not None and row_scale.shape[1] == B * n
                                      and n > 1 else 1, _column_ptr(out, out_column), _code(out.dtype),
                                      ctypes.c_longlong(out.shape[1]), ctypes.c_longlong(out_block), T, B, n, m,
                                      _stream()), "blockwise_linear")
    return out


def rope_heads(src: torch.Tensor, src_column: int, src_head: int, dst: torch.Tensor, dst_column: int, dst_head: int,
               positions: torch.Tensor, inv_freq: torch.Tensor, heads: int) -> torch.Tensor:
    """For every token and head: the 2 * len(inv_freq) columns of src [T, W] at src_column + h * src_head,
    rotated by position (pairs i, i + half, angle = float(position) * inv_freq[i]), written to dst
    [T, W'] at dst_column + h * dst_head."""
    _check(src, "src", dims=2)
    _check(dst, "dst", src.dtype, 2)
    _check(positions, "positions", torch.int32, 1)
    _check(inv_freq, "inv_freq", torch.float32, 1)
    T, rot = src.shape[0], 2 * inv_freq.numel()
    if (dst.shape[0] != T or positions.numel() != T or src_column + (heads - 1) * src_head + rot > src.shape[1]
            or dst_column + (heads - 1) * dst_head + rot > dst.shape[1]):
        raise InvalidError("rope_heads: columns outside a row")
    _done(_lib().lrm_rope_heads(_column_ptr(src, src_column), _code(src.dtype), ctypes.c_longlong(src.shape[1]),
                                ctypes.c_longlong(src_head), _column_ptr(dst, dst_column),
                                ctypes.c_longlong(dst.shape[1]), ctypes.c_longlong(dst_head), _ptr(positions),
                                _ptr(inv_freq), rot, T, heads, _stream()), "rope_heads")
    return dst


def latent_prepare(proj: torch.Tensor, q_column: int, q_weight: Optional[torch.Tensor], c_column: int,
                   c_weight: Optional[torch.Tensor], rot: int, positions: torch.Tensor,
                   inv_freq: Optional[torch.Tensor], eps: float, gate_column: int, heads: int,
                   out_dtype: torch.dtype, kv=None, dest_rows: Optional[torch.Tensor] = None,
                   keep_packed: bool = True, q_width: int = 0):
    """From a fused down-projection [T, W]: the normed query latent [T, q_rank] (out_dtype; without
    `q_weight` the `q_width` query columns as they are, for queries that have no latent), the gates
    sigmoid(.) float32 [T, heads] (`heads`: how many gate columns there are), and, when the row has key/value columns (c_column >= 0), the rows
    [RMSnorm(latent) * c_weight | rotated shared key part] [T, kv_rank + rot], returned when
    `keep_packed` and written into the paged cache view `kv` (one key head of that width) at
    `dest_rows`. Norm weights float32. -> (cq, rows or None, gate)."""
    _check(proj, "proj", dims=2)
    if q_weight is not None:
        _check(q_weight, "q_weight", torch.float32, 1)
    _check(positions, "positions", torch.int32, 1)
    T, q_rank = proj.shape[0], q_weight.numel() if q_weight is not None else q_width
    kv_rank = 0
    if c_column >= 0:
        _check(c_weight, "c_weight", torch.float32, 1)
        kv_rank = c_weight.numel()
        if rot:
            _check(inv_freq, "inv_freq", torch.float32, 1)
            if inv_freq.numel() * 2 != rot:
                raise InvalidError("latent_prepare: inv_freq must have rot/2 entries")
        if c_column + kv_rank + rot > proj.shape[1]:
            raise InvalidError("latent_prepare: key/value columns outside the projection")
    if q_column + q_rank > proj.shape[1] or gate_column + heads > proj.shape[1]:
        raise InvalidError("latent_prepare: columns outside the projection")
    cq = _activation(T, q_rank, out_dtype, proj.device)
    gate = _f32((T, heads), proj.device)
    rows, pages, dest = None, None, None
    if c_column >= 0:
        if keep_packed:
            rows = torch.empty((T, kv_rank + rot), dtype=out_dtype, device=proj.device)
        if kv is not None:
            pages, dest = kv.k, dest_rows
            _check(pages, "k pages", out_dtype, 4)
            _check(dest, "dest_rows", torch.int32, 1)
            if pages.shape[1] != 1 or pages.shape[3] != kv_rank + rot or dest.numel() != T:
                raise InvalidError("latent_prepare: the cache keeps one key head of width kv_rank + rot")
    _done(_lib().lrm_latent_prepare(_ptr(proj), _code(proj.dtype), ctypes.c_longlong(proj.shape[1]), q_column, q_rank,
                                    _ptr(q_weight), c_column, kv_rank, _ptr(c_weight), rot, _ptr(positions),
                                    _ptr(inv_freq), ctypes.c_float(eps), _ptr(cq), _ptr(rows), _ptr(pages), _ptr(dest),
                                    gate_column, heads, _ptr(gate), _code(out_dtype), T, _stream()), "latent_prepare")
    return cq, rows, gate


GATE_SILU, GATE_SIGMOID = 1, 2


def head_norm_gate(o: torch.Tensor, eps: float, out_dtype: torch.dtype, weight: Optional[torch.Tensor] = None,
                   gate: Optional[torch.Tensor] = None, gate_column: int = 0, gate_act: int = GATE_SILU,
                   out_scale: float = 1.0, value_dim: Optional[int] = None, floor: Optional[torch.Tensor] = None,
                   floor_eps: float = 0.0) -> torch.Tensor:
    """Per token and head: o / sqrt(mean(o^2) + eps) [* weight] [* act(gate)] * out_scale, o float32
    [T,H,dv] -> [T, H*dv] in `out_dtype`. `gate` is a [T, W] activation whose columns gate_column ..
    gate_column + H*dv hold the gate's pre-activation; act: GATE_SILU or GATE_SIGMOID. `weight`
    float32 [dv] (shared by the heads) or [H*dv]. `value_dim` < o.shape[2]: only the first value_dim
    columns of a head are values. With `floor` float32 [T,H] a head is first divided by
    max(|o[value_dim]|, floor) + floor_eps: column value_dim is then a normalizer's read-out."""
    _check(o, "o", torch.float32, 3)
    T, H, o_stride = o.shape
    dv = o_stride if value_dim is None else value_dim
    if not 0 < dv <= o_stride or (floor is not None and dv == o_stride):
        raise InvalidError("head_norm_gate: value_dim outside the head's row")
    w_stride = 0
    if weight is not None:
        _check(weight, "weight", torch.float32, 1)
        if weight.numel() not in (dv, H * dv):
            raise InvalidError("head_norm_gate: weight must have one entry per value dimension, or per head and dimension")
        w_stride = dv if weight.numel() == H * dv and H > 1 else 0
    if floor is not None:
        _check(floor, "floor", torch.float32, 2)
        if tuple(floor.shape) != (T, H):
            raise InvalidError("head_norm_gate: floor must be [T,H]")
    gate_ptr, stride = ctypes.c_void_p(0), 0
    gate_code = _code(out_dtype)
    if gate is not None:
        _check(gate, "gate", dims=2)
        gate_code = _code(gate.dtype)
        if gate.shape[0] != T or gate_column + H * dv > gate.shape[1]:
            raise InvalidError("head_norm_gate: gate columns outside the activation")
        gate_ptr, stride = _column_ptr(gate, gate_column), gate.shape[1]
    out = _activation(T, H * dv, out_dtype, o.device)
    _done(_lib().lrm_head_norm_gate(_ptr(o), o_stride, _ptr(weight), w_stride, _ptr(floor), ctypes.c_float(floor_eps),
                                    gate_ptr, gate_code, ctypes.c_longlong(stride), gate_act, _ptr(out),
                                    _code(out_dtype), T, H, dv, ctypes.c_float(eps), ctypes.c_float(out_scale),
                                    _stream()), "head_norm_gate")
    return out


# --------------------------------------------------------------------------- mixture of experts
def moe_route(logits: torch.Tensor, bias: Optional[torch.Tensor], top: int):
    """The `top` largest of each row of float32 logits [T, E] (+ bias [E]), lower index first on a
    tie, and the softmax over the chosen ones. -> ids int32 [T, top], weights float32 [T, top]."""
    _check(logits, "logits", torch.float32, 2)
    T, E = logits.shape
    if bias is not None:
        _check(bias, "bias", torch.float32, 1)
        if bias.numel() != E:
            raise InvalidError("moe_route: one bias per expert")
    if not 0 < top <= E:
        raise InvalidError("moe_route: top must be between 1 and the number of experts")
    ids = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    weights = _f32((T, top), logits.device)
    _done(_lib().lrm_moe_route(_ptr(logits), _ptr(bias), _ptr(ids), _ptr(weights), T, E, top, _stream()), "moe_route")
    return ids, weights


@dataclass(frozen=True)
class Scoring:
    """A router that scores with the softmax over all its outputs: the choice is made on the scores
    plus `correction` (float32 [E] or None), among the outputs of the `keep` best of `groups` equal
    groups of neighbours (a group counts by its largest corrected score); the weights are the
    chosen scores, divided by (their sum + `mass_eps`) with `renormalize`, then times `weight_scale`."""

    correction: Optional[torch.Tensor] = None
    groups: int = 1
    keep: int = 1
    renormalize: bool = False
    mass_eps: float = 0.0
    weight_scale: float = 1.0

    def arguments(self):
        return (_ptr(self.correction), self.groups, self.keep, int(self.renormalize), ctypes.c_float(self.mass_eps),
                ctypes.c_float(self.weight_scale))


def moe_route_scored(logits: torch.Tensor, top: int, scoring: Scoring):
    """The scored router's choice from float32 logits [T, E]. -> ids int32 [T, top], weights float32
    [T, top]."""
    _check(logits, "logits", torch.float32, 2)
    T, E = logits.shape
    _check_scoring(scoring, E, top)
    ids = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    weights = _f32((T, top), logits.device)
    _done(_lib().lrm_moe_route_scored(_ptr(logits), _ptr(scoring.correction), _ptr(ids), _ptr(weights), T, E, top,
                                      *scoring.arguments()[1:], _stream()),
          "moe_route_scored")
    return ids, weights


def _check_scoring(scoring: Scoring, E: int, top: int) -> None:
    if scoring.correction is not None:
        _check(scoring.correction, "correction", torch.float32, 1)
        if scoring.correction.numel() != E:
            raise InvalidError("router: one correction per output")
    g, k = scoring.groups, scoring.keep
    if g <= 0 or E % g or not 0 < k <= g or not 0 < top <= k * (E // g):
        raise InvalidError("router: groups must divide the outputs, and the kept groups hold at least `top` of them")


def moe_identity_add_(out: torch.Tensor, x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
                      experts: int) -> torch.Tensor:
    """out[t] += (sum of weights[t, c] over the choices with ids[t, c] >= experts) * x[t]: the share of
    identity experts, which return their input. out float32 [T, width]; x [T, width]."""
    _check(out, "out", torch.float32, 2)
    _check(x, "x", dims=2)
    _check(ids, "ids", torch.int32, 2)
    _check(weights, "weights", torch.float32, 2)
    if x.shape != out.shape or ids.shape[0] != out.shape[0] or weights.shape != ids.shape:
        raise InvalidError("moe_identity_add_: shapes do not agree")
    _done(_lib().lrm_moe_identity_add(_ptr(out), _ptr(x), _code(x.dtype), _ptr(ids), _ptr(weights), out.shape[0],
                                      out.shape[1], experts, ids.shape[1], _stream()), "moe_identity_add_")
    return out


def moe_router(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], top: int,
               scoring: Optional[Scoring] = None):
    """moe_route(x . weight^T, bias, top) in one launch: float32 logits from x [T, width] (float32, or
    bfloat16 widened exactly) and float32 weight [E, width], a CTA per token. For steps of few
    tokens; None where the kernel does not take the sizes (the caller makes the product and routes).
    With `scoring` the choice is the scored router's (moe_route_scored) and `bias` is not used."""
    _check(x, "x", dims=2)
    _check(weight, "weight", torch.float32, 2)
    T, width = x.shape
    E = weight.shape[0]
    if weight.shape[1] != width or not 0 < top <= E:
        raise InvalidError("moe_router: shapes do not agree")
    if bias is not None:
        _check(bias, "bias", torch.float32, 1)
    if scoring is not None:
        _check_scoring(scoring, E, top)
    if 4 * (width + (3 * E + scoring.groups // 4 + 1 if scoring is not None else E)) > 48 * 1024:
        return None
    ids = torch.empty((T, top), dtype=torch.int32, device=x.device)
    weights = _f32((T, top), x.device)
    extra = (1, *scoring.arguments()) if scoring is not None else (0, None, 1, 1, 0, ctypes.c_float(0.0), ctypes.c_float(1.0))
    _done(_lib().lrm_moe_router(_ptr(x), _code(x.dtype), _ptr(weight), _ptr(bias), _ptr(ids), _ptr(weights), None,
                                T, width, E, top, *extra, _stream()), "moe_router")
    return ids, weights


ACT_CLAMPED_GATE, ACT_SILU = 0, 1


def moe_experts_rows(x: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, ids: torch.Tensor,
                     weights: torch.Tensor, limit: float, alpha: float, act: int = ACT_CLAMPED_GATE,
                     x32: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Every token's chosen experts, token by token: planes float32 [n, T, width] whose sum in plane
    order is sum_c weights[t,c] * expert_ids[t,c](x[t]). gate_up [E, 2 ff, width] (an expert's gate
    rows, then its up rows), down [width, E, ff]. An id of E or more is an identity expert: its
    output is its input (x32, float32 [T, width], where the caller has the input unrounded)."""
    _check(x, "x", dims=2)
    T, width = x.shape
    _check(gate_up, "gate_up", dims=3)
    _check(down, "down", gate_up.dtype, 3)
    E, ff = gate_up.shape[0], gate_up.shape[1] // 2
    if tuple(gate_up.shape) != (E, 2 * ff, width) or tuple(down.shape) != (width, E, ff):
        raise InvalidError("moe_experts_rows: gate_up must be [E, 2 ff, width] and down [width, E, ff]")
    _check(ids, "ids", torch.int32, 2)
    _check(weights, "weights", torch.float32, 2)
    top = ids.shape[1]
    if ids.shape[0] != T or tuple(weights.shape) != (T, top):
        raise InvalidError("moe_experts_rows: one row of choices per token")
    if T > 65535:
        raise UnsupportedError("moe_experts_rows: more than 65535 tokens in one step")
    if x32 is not None:
        _check(x32, "x32", torch.float32, 2)
        if x32.shape != x.shape:
            raise InvalidError("moe_experts_rows: x32 must match x")
    lib = _lib()
    slices = int(lib.lrm_moe_rows_slices(T, top, ff))
    planes = _f32((top * slices, T, width), x.device)
    _done(lib.lrm_moe_experts_rows(_ptr(x), _code(x.dtype), _ptr(gate_up), _ptr(down), _code(gate_up.dtype),
                                   _ptr(ids), _ptr(weights), _ptr(planes), T, width, ff, E, top, slices,
                                   ctypes.c_float(limit), ctypes.c_float(alpha), act, _ptr(x32), _stream()),
          "moe_experts_rows")
    return planes


def moe_dense_gate(gate_up: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, experts: int, limit: float,
                   alpha: float, out_dtype: Optional[torch.dtype] = None, act: int = ACT_CLAMPED_GATE) -> torch.Tensor:
    """From every expert's gate and up for every token, [T, E * 2 ff] (an expert's ff gate columns,
    then its ff up columns; float32, or the output's type): y [T, E * ff] = weight(t, e) * act(gate,
    up) in `out_dtype` (default: the input's), zero where token t did not choose expert e."""
    _check(gate_up, "gate_up", dims=2)
    _check(ids, "ids", torch.int32, 2)
    _check(weights, "weights", torch.float32, 2)
    T, top = ids.shape
    if gate_up.shape[0] != T or gate_up.shape[1] % (2 * experts) or tuple(weights.shape) != (T, top):
        raise InvalidError("moe_dense_gate: shapes do not agree")
    ff = gate_up.shape[1] // (2 * experts)
    out_dtype = out_dtype or gate_up.dtype
    y = _activation(T, experts * ff, out_dtype, gate_up.device)
    _done(_lib().lrm_moe_dense_gate(_ptr(gate_up), _code(gate_up.dtype), _code(out_dtype), _ptr(ids), _ptr(weights), _ptr(y), T, ff,
                                    experts, top, ctypes.c_float(limit), ctypes.c_float(alpha), act, _stream()),
          "moe_dense_gate")
    return y


def add_row_(x: torch.Tensor, row: torch.Tensor) -> torch.Tensor:
    """x[t, :] += row for every row t; both float32."""
    _check(x, "x", torch.float32, 2)
    _check(row, "row", torch.float32, 1)
    if row.numel() != x.shape[1]:
        raise InvalidError("add_row_: the row must be as wide as x")
    _done(_lib().lrm_add_row(_ptr(x), _ptr(row), ctypes.c_longlong(x.shape[0]), x.shape[1], _stream()), "add_row_")
    return x


# --------------------------------------------------------------------------- attention
def _check_slopes(slopes: Optional[torch.Tensor], heads: int) -> None:
    if slopes is not None:
        _check(slopes, "slopes", torch.float32, 1)
        if slopes.numel() != heads:
            raise InvalidError("one distance slope per query head")


def _check_extras(extras, heads: int) -> None:
    if extras is not None and extras.sinks is not None:
        _check(extras.sinks, "sinks", torch.float32, 1)
        if extras.sinks.numel() != heads:
            raise InvalidError("one sink per query head")


def attention_prefill(q: torch.Tensor, k: torch.Tensor, v: Optional[torch.Tensor], cu_seqlens: torch.Tensor,
                      seq_of_token: torch.Tensor, max_seq_len: int, scale: float,
                      window: Optional[int] = None, slopes: Optional[torch.Tensor] = None,
                      out_scale: float = 1.0, extras=None, value_dim: Optional[int] = None) -> torch.Tensor:
    """Causal GQA over the step's own packed k, v (sequences start at position 0). -> [T, Hq*dv]
    (v may have another head width dv than q and k). `slopes` (float32 [Hq]): a key n positions
    behind the query loses slopes[h] * n from its score. `out_scale` multiplies the result.
    v None: the values are the first `value_dim` columns (default: all) of the key rows.
    `extras` (attention_dispatch.Extras): per-head sinks, a query temperature."""
    _check(q, "q", dims=3)
    _check(k, "k", q.dtype, 3)
    _check_extras(extras, q.shape[1])
    if v is None:
        dv = k.shape[2] if value_dim is None else value_dim
        if not 0 < dv <= k.shape[2] or q.shape[1] % k.shape[1] or k.shape[0] != q.shape[0] or k.shape[2] != q.shape[2]:
            raise InvalidError("attention_prefill: q and k shapes do not agree")
        _check(cu_seqlens, "cu_seqlens", torch.int32, 1)
        _check(seq_of_token, "seq_of_token", torch.int32, 1)
        _check_slopes(slopes, q.shape[1])
        out = _activation(q.shape[0], q.shape[1] * dv, q.dtype, q.device)
        from . import attention_dispatch
        attention_dispatch.prefill(q, k, None, out, cu_seqlens, seq_of_token, max_seq_len, scale, window or 0,
                                   slopes, out_scale, extras, dv)
        return out
    _check(v, "v", q.dtype, 3)
    _check(cu_seqlens, "cu_seqlens", torch.int32, 1)
    _check(seq_of_token, "seq_of_token", torch.int32, 1)
    T, Hq, d = q.shape
    Hk = k.shape[1]
    if k.shape[:2] != v.shape[:2] or k.shape[0] != T or k.shape[2] != d or Hq % Hk:
        raise InvalidError("attention_prefill: q, k, v shapes do not agree")
    _check_slopes(slopes, Hq)
    out = _activation(T, Hq * v.shape[2], q.dtype, q.device)
    from . import attention_dispatch
    attention_dispatch.prefill(q, k, v, out, cu_seqlens, seq_of_token, max_seq_len, scale, window or 0,
                               slopes, out_scale, extras)
    return out


def _value_dim(kv) -> int:
    """Head width of a cache view's values (which may be the first columns of its key rows)."""
    return kv.value_dim if getattr(kv, "value_dim", None) else kv.v.shape[3]


def attention_decode(q: torch.Tensor, kv, slots: torch.Tensor, kv_lens: torch.Tensor,
                     max_kv_len: int, scale: float, window: Optional[int] = None,
                     slopes: Optional[torch.Tensor] = None, out_scale: float = 1.0, extras=None) -> torch.Tensor:
    """One query per sequence over its cached keys (the newest already stored). -> [B, Hq*dv]"""
    _check_extras(extras, q.shape[1])
    _check(q, "q", dims=3)
    _check(kv.k, "k pages", q.dtype, 4)
    _check(kv.v, "v pages", q.dtype, 4)
    _check(kv.page_table, "page table", torch.int32, 2)
    _check(slots, "slots", torch.int32, 1)
    _check(kv_lens, "kv_lens", torch.int32, 1)
    B, Hq, d = q.shape
    if tuple(kv.k.shape[1:]) != (kv.kv_heads, kv.page_size, d) or Hq % kv.kv_heads:
        raise InvalidError("attention_decode: cache pages do not match the query geometry")
    _check_slopes(slopes, Hq)
    out = _activation(B, Hq * _value_dim(kv), q.dtype, q.device)
    from . import attention_dispatch
    attention_dispatch.decode(q, kv, out, slots, kv_lens, max_kv_len, scale, window or 0, slopes, out_scale, extras)
    return out


def attention_extend(q: torch.Tensor, kv, cu_seqlens: torch.Tensor, seq_of_token: torch.Tensor,
                     positions: torch.Tensor, slots: torch.Tensor, kv_lens: torch.Tensor, max_seq_len: int,
                     scale: float, window: Optional[int] = None, slopes: Optional[torch.Tensor] = None,
                     out_scale: float = 1.0, extras=None) -> torch.Tensor:
    """Several queries per sequence over the cache, which already holds the step's own keys:
    query t (packed, of sequence seq_of_token[t]) sees the keys up to positions[t]. -> [T, Hq*d]"""
    _check(q, "q", dims=3)
    _check(kv.k, "k pages", q.dtype, 4)
    _check(kv.v, "v pages", q.dtype, 4)
    _check(kv.page_table, "page table", torch.int32, 2)
    T, Hq, d = q.shape
    for name, t, n in (("cu_seqlens", cu_seqlens, None), ("seq_of_token", seq_of_token, T),
                       ("positions", positions, T), ("slots", slots, cu_seqlens.numel() - 1),
                       ("kv_lens", kv_lens, cu_seqlens.numel() - 1)):
        _check(t, name, torch.int32, 1)
        if n is not None and t.numel() != n:
            raise InvalidError(f"attention_extend: {name} must have {n} entries")
    if tuple(kv.k.shape[1:]) != (kv.kv_heads, kv.page_size, d) or Hq % kv.kv_heads:
        raise InvalidError("attention_extend: cache pages do not match the query geometry")
    _check_slopes(slopes, Hq)
    out = _activation(T, Hq * _value_dim(kv), q.dtype, q.device)
    from . import attention_dispatch
    _check_extras(extras, Hq)
    attention_dispatch.extend(q, kv, out, cu_seqlens, seq_of_token, positions, slots, kv_lens, max_seq_len,
                              scale, window or 0, slopes, out_scale, extras)
    return out


def attention_decode_fused_supported(dtype, head_dim: int, page_size: int, rotary: int, window) -> bool:
    from . import attention_dispatch
    return attention_dispatch.decode_fused_supported(dtype, head_dim, page_size, rotary, window)


def attention_decode_prefers_fused(seqs: int, kv_heads: int, group: int, head_dim: int, max_kv_len: int) -> bool:
    """Whether the one-launch kernel is expected to beat the separate kernels for this step's geometry."""
    from . import attention_dispatch
    return attention_dispatch.decode_prefers_fused(seqs, kv_heads, group, head_dim, max_kv_len)


def attention_decode_fused(qkv: torch.Tensor, q_heads: int, inv_freq: Optional[torch.Tensor], rotary: int,
                           positions: torch.Tensor, kv, dest_rows: torch.Tensor, slots: torch.Tensor,
                           kv_lens: torch.Tensor, max_kv_len: int, scale: float,
                           order: Optional[torch.Tensor] = None, fill: int = 4) -> torch.Tensor:
    """A decode step's attention from its fused, unrotated [B, (Hq+2Hk)*d] projection: rotates q and
    the new k, stores the new k and v at `dest_rows`, attends over the cache (kv_lens counts the new
    token) and merges the splits, in one launch. -> [B, Hq*d]. `order` (int32 [B], made on the host and
    copied before the step, because the kernel reads it before it waits for the kernels ahead of
    it): the sequences' work is handed out in this order, longest first when lengths are unequal;
    `fill`: their mean length in quarters of the longest (launch geometry only)."""
    _check(qkv, "qkv", torch.bfloat16, 2)
    d, Hk = kv.head_dim, kv.kv_heads
    if qkv.shape[1] != (q_heads + 2 * Hk) * d or q_heads % Hk:
        raise InvalidError("attention_decode_fused: qkv width does not match the head geometry")
    _check(kv.k, "k pages", qkv.dtype, 4)
    _check(kv.v, "v pages", qkv.dtype, 4)
    if tuple(kv.k.shape[1:]) != (Hk, kv.page_size, d):
        raise InvalidError("attention_decode_fused: cache pages do not match the head geometry")
    _check(kv.page_table, "page table", torch.int32, 2)
    B = qkv.shape[0]
    for name, t in (("positions", positions), ("dest_rows", dest_rows), ("slots", slots), ("kv_lens", kv_lens)):
        _check(t, name, torch.int32, 1)
        if t.numel() != B:
            raise InvalidError(f"attention_decode_fused: one entry of {name} per sequence")
    if inv_freq is not None:
        _check(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.numel() != rotary // 2:
            raise InvalidError("attention_decode_fused: inv_freq must have rotary/2 entries")
    else:
        rotary = 0
    if not attention_decode_fused_supported(qkv.dtype, d, kv.page_size, rotary, kv.window):
        raise UnsupportedError("attention_decode_fused: geometry not supported; use rope_store and attention_decode")
    out = _activation(B, q_heads * d, qkv.dtype, qkv.device)
    from . import attention_dispatch
    if order is not None:
        _check(order, "order", torch.int32, 1)
        if order.numel() != B:
            raise InvalidError("attention_decode_fused: one entry of order per sequence")
    attention_dispatch.decode_fused(qkv, positions, inv_freq, rotary, kv, dest_rows, out, slots, kv_lens,
                                    max_kv_len, q_heads, scale, order, fill)
    return out


def attend(projected: torch.Tensor, **geometry) -> torch.Tensor:
    """A layer's attention for one step from its projection (see attention_dispatch.attend)."""
    from . import attention_dispatch
    return attention_dispatch.attend(projected, **geometry)


# --------------------------------------------------------------------------- sampling
def _pick_scratch(logits: torch.Tensor):
    pieces = _lib().lrm_pick_pieces(logits.shape[1])
    values = torch.empty((logits.shape[0], pieces), dtype=torch.float32, device=logits.device)
    ids = torch.empty((logits.shape[0], pieces), dtype=torch.int32, device=logits.device)
    return values, ids


PICK_ROWS = 12  # up to this many rows the streaming product is the head's fastest kernel, and it can choose

_pick_words_by_device = {}


def _pick_words(device: torch.device) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per device: 64 running-best words and 64 flags for the head product that chooses in its
    epilogue. Zero between calls (the kernel that reads the winners clears them), so every call
    on a stream can share them; reset_pick_scratch() zeroes them after a failed step."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _pick_words_by_device:
        _pick_words_by_device[index] = (torch.zeros(64, dtype=torch.int64, device=device),
                                        torch.zeros(64, dtype=torch.int32, device=device))
    return _pick_words_by_device[index]


def reset_pick_scratch() -> None:
    for best, bad in _pick_words_by_device.values():
        best.zero_()
        bad.zero_()


def linear_pick(x: torch.Tensor, weight: torch.Tensor, temperature: Optional[float] = None, seed: int = 0,
                keys: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """int32 [M]: the token chosen from the logits x . weight^T of each row, without writing the
    logits: every CTA of the head product offers its best (score, id) per row to the row's
    running best with an atomic maximum, and a second small kernel reads the winners.
    temperature None: greedy, as argmax_rows; else a draw from softmax(logits / temperature) with
    the noise of sample_gumbel_rows for the same seed and keys (int64 [M]). -1 marks a row with a
    non-finite logit. None when no kernel takes this product that way (float32, more rows than
    the streaming product is the fastest for, unaligned): the caller then writes the logits and
    picks from them."""
    _check(x, "x", dims=2)
    _check(weight, "weight", dims=2)
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K:
        raise InvalidError(f"linear_pick: x has {K} columns, weight has {weight.shape[1]}")
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or M > PICK_ROWS:
        return None
    lib = _lib()
    if not lib.lrm_gemm_bf16_stream_supports(M, N, K) or x.data_ptr() % 16 or weight.data_ptr() % 16:
        return None
    if temperature is not None:
        if keys is None or not temperature > 0:
            raise InvalidError("linear_pick: temperature sampling needs a positive temperature and one key per row")
        _check(keys, "keys", torch.int64, 1)
        if keys.numel() != M:
            raise InvalidError("linear_pick: one key per row")
    best, bad = _pick_words(x.device)
    out = torch.empty((M,), dtype=torch.int32, device=x.device)
    _done(lib.lrm_gemm_bf16_stream_pick(_ptr(x), _ptr(weight), M, N, K, _ptr(best), _ptr(bad), _ptr(out),
                                        ctypes.c_float(temperature if temperature is not None else 1.0),
                                        ctypes.c_ulonglong(seed & ((1 << 64) - 1)),
                                        _ptr(keys if temperature is not None else None), _stream()),
          "gemm_bf16_stream_pick", launches=2)
    return out


def argmax_rows(logits: torch.Tensor) -> torch.Tensor:
    """int32 [n]: largest logit per row, lowest id on ties, -1 for a row with a non-finite logit."""
    _check(logits, "logits", torch.float32, 2)
    out = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
    values, ids = _pick_scratch(logits)
    _done(_lib().lrm_argmax_rows(_ptr(logits), _ptr(out), _ptr(values), _ptr(ids), logits.shape[0],
                                 logits.shape[1], _stream()), "argmax_rows", launches=2)
    return out


def sample_gumbel_rows(logits: torch.Tensor, temperature: float, seed: int, keys: torch.Tensor) -> torch.Tensor:
    """int32 [n]: a draw from softmax(logits / temperature) per row; `keys` int64 [n] names each row's stream."""
    _check(logits, "logits", torch.float32, 2)
    _check(keys, "keys", torch.int64, 1)
    if keys.numel() != logits.shape[0]:
        raise InvalidError("sample_gumbel_rows: one key per row")
    if not temperature > 0:
        raise InvalidError("sample_gumbel_rows: temperature must be positive")
    out = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
    values, ids = _pick_scratch(logits)
    _done(_lib().lrm_sample_gumbel_rows(_ptr(logits), _ptr(out), _ptr(values), _ptr(ids), logits.shape[0],
                                        logits.shape[1], ctypes.c_float(temperature),
                                        ctypes.c_ulonglong(seed & ((1 << 64) - 1)), _ptr(keys),
                                        _stream()), "sample_gumbel_rows", launches=2)
    return out
