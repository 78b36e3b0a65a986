"""The operations a decoder step is made of, each a call into a hand-written CUDA kernel.

Tensors are torch tensors on a CUDA device (torch is used for memory and for the library matrix
product only); every function launches on torch's current stream.  There is no CPU implementation and
no fallback: a tensor on another device, a missing compiler or a failed build raises.

Matrix products: float32 runs ``gemm_f32`` (FFMA, no tensor-core mode).  bfloat16 runs the weight-streaming
``mma.sync`` kernel up to 8 rows (decode of few sequences) and otherwise the library product (cuBLAS through
``torch.nn.functional.linear``), as the reference does for every linear layer (fms/modules/linear.py:119-156) —
except the gated feed-forward product, which from ``TENSOR_CORE_ROWS_GLU`` (512) rows on, where its tiles of 256
rows fit the number of rows to 6%, takes the tcgen05 kernel
with the tokens on the instruction's rows (prefill; pairs of thread blocks on one tile, the activation in its
epilogue), and the fused projection of queries, keys and values, which from ``TENSOR_CORE_ROWS_QKV`` (2,048) rows
on takes the same kernel with the rotation and the cache write in its epilogue.  The same kernel takes the plain
products from ``FMS_B200_TC_ROWS`` rows on where that is set; measured through whole prefills the library's plain
products are ahead, so by default it is not.
The gated feed-forward product of 9 to 128 rows takes a tcgen05 kernel of this library with the weights on the
instruction's rows and the activation in its epilogue (``gemm_bf16_mid.cu``); the same kernel can take the plain
products and the fused projection up to 256 rows (clusters of blocks share a tile along K; projection + rotation
+ cache write in its epilogue; ``FMS_B200_MID_OPS``), where the library's product is still ahead of it.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .build import load_library

F32, BF16 = 0, 1
_P, _I, _F, _U64, _L = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_ulonglong, ctypes.c_long

_SIGNATURES = {
    "fms_embed_rows": [_P, _I, _P, _P, _I, _I, _I, _F, _P, _P],
    "fms_add_rmsnorm": [_P, _P, _P, _I, _F, _P, _I, _P, _I, _I, _I, _P],
    "fms_gated_activation": [_P, _P, _I, _I, _I, _I, _P],
    "fms_rope_store": [_P, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _I, _I, _I, _P],
    "fms_decode_advance": [_P, _P, _P, _P, _P, _I, _I, _P],
    "fms_rotary_table": [_P, _P, _P, _P, _I, _I, _P],
    "fms_gemm_f32": [_P, _P, _P, _P, _I, _I, _I, _P],
    "fms_linear_bf16_skinny": [_P, _P, _P, _P, _I, _I, _I, _I, _P],
    "fms_glu_bf16_skinny": [_P, _P, _P, _P, _I, _I, _I, _I, _P],
    "fms_qkv_rope_store_bf16_skinny": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P,
                                       _I, _I, _I, _P],
    "fms_linear_bf16_mid": [_P, _P, _P, _P, _I, _I, _I, _I, _P, _P],
    "fms_glu_bf16_mid": [_P, _P, _P, _P, _I, _I, _I, _I, _P, _P],
    "fms_qkv_rope_store_bf16_mid": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P,
                                    _I, _I, _I, _P],
    "fms_gemm_bf16_tc": [_P, _P, _P, _P, _I, _I, _I, _I, _P, _P],
    "fms_glu_bf16_tc": [_P, _P, _P, _P, _I, _I, _I, _I, _P, _P],
    "fms_qkv_rope_store_bf16_tc": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P,
                                   _I, _I, _I, _P],
    "fms_argmax": [_P, _P, _I, _I, _P],
    "fms_sample": [_P, _P, _I, _I, _F, _I, _U64, _P, _I, _P],
    "fms_attention_prefill": [_P, _P, _I, _P, _P, _P, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _I, _I, _P, _P],
    "fms_attention_decode": [_P, _P, _I, _P, _P, _P, _I, _I, _P, _P, _P, _I, _I, _P, _P, _I, _I, _I, _F, _I, _I, _I, _L, _P, _P,
                             _P],
}
_functions = {}
# kernels launched through this module since import (a decode-attention call over several splits launches two)
launches = 0


class KernelError(RuntimeError):
    pass


def _fn(library: str, name: str):
    key = (library, name)
    f = _functions.get(key)
    if f is None:
        lib = load_library(library)
        f = getattr(lib, name)
        f.argtypes = _SIGNATURES[name]
        f.restype = ctypes.c_int
        _functions[key] = f = (f, lib)
    return f


def _call(library: str, name: str, *args):
    global launches
    f, lib = _fn(library, name)
    launches += 1
    rc = f(*args)
    if rc != 0:
        raise KernelError(f"{name}: {lib.fms_last_error().decode(errors='replace')}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle (the direct getter where torch has it: a step makes some hundred launches)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"dtype {dtype} has no kernel: float32 and bfloat16 have")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("a tensor on the CPU reached a CUDA kernel; this library has no CPU path")
    if not t.is_contiguous():
        raise KernelError("a non-contiguous tensor reached a CUDA kernel")
    return t.data_ptr()


_error_flags = {}


def error_flag(device) -> torch.Tensor:
    """An int32 on the device that kernels set when they meet what the host should have prevented (a token
    id outside the vocabulary, a position without a cache block).  ``check_error_flag`` reads it."""
    device = torch.device(device)
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    if key not in _error_flags:
        _error_flags[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_flags[key]


_work_counters = {}
WORK_COUNTERS = 4096


def _work_counter(device) -> torch.Tensor:
    """An int32 on the device that is 0 between launches: the persistent decode-attention kernel's warps draw
    their units from it, and the kernel that merges the splits puts it back.  Every call hands out the next of
    4,096, so that launches in flight at the same time (other streams, the launches inside captured graphs) do
    not share one."""
    device = torch.device(device)
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    if key not in _work_counters:
        _work_counters[key] = [torch.zeros(WORK_COUNTERS, dtype=torch.int32, device=device), 0]
    entry = _work_counters[key]
    entry[1] = (entry[1] + 1) % WORK_COUNTERS
    return entry[0][entry[1]:entry[1] + 1]


def check_error_flag(device) -> None:
    """Raises if a kernel met something the host should have prevented; in a bounds-checked build
    (FMS_B200_DEBUG_BOUNDS=1) also if any kernel computed an index outside its array.  Synchronises."""
    flag = error_flag(device)
    v = int(flag.item())
    from .build import bounds_violations

    outside = bounds_violations()
    if outside:
        raise KernelError("bounds-checked build: " + "; ".join(outside))
    if v:
        flag.zero_()
        raise KernelError({1: "a token id outside the vocabulary reached the embedding",
                           2: "a token's position has no cache block",
                           4: "a kernel gave up waiting for a copy or for the tensor cores",
                           8: "decode attention was launched with fewer key splits than a sequence's length needs",
                           16: "a kernel's bounds check met an index outside its array"}.get(v, f"device error flag {v}"))


# ---- embedding ---------------------------------------------------------------------------------------
def embed(table: torch.Tensor, tokens: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """Float32 rows of ``table`` at ``tokens``, times ``scale``: the start of the residual stream."""
    n, dim = tokens.shape[0], table.shape[1]
    out = torch.empty((n, dim), dtype=torch.float32, device=table.device)
    _call("elementwise", "fms_embed_rows", _ptr(table), _code(table.dtype), _ptr(tokens), _ptr(out), n, dim,
          table.shape[0], float(scale), _ptr(error_flag(table.device)), _stream())
    return out


# ---- norm --------------------------------------------------------------------------------------------
def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], gain: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """residual (float32, in place) += delta; returns gain * rmsnorm(residual) in ``out_dtype``.  With
    ``rows`` only those rows are computed and the residual is not written."""
    dim = residual.shape[1]
    n = rows.shape[0] if rows is not None else residual.shape[0]
    if residual.dtype != torch.float32:
        raise KernelError("the residual stream is float32")
    if delta is not None and delta.dtype != out_dtype:
        raise KernelError(f"sublayer output is {delta.dtype}, compute dtype is {out_dtype}")
    out = torch.empty((n, dim), dtype=out_dtype, device=residual.device)
    _call("elementwise", "fms_add_rmsnorm", _ptr(residual), _ptr(delta), _ptr(gain), _code(gain.dtype), float(eps),
          _ptr(out), _code(out_dtype), _ptr(rows), n, dim, residual.shape[0], _stream())
    return out


# ---- linear ------------------------------------------------------------------------------------------
def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """x [rows, in] times weight [out, in] transposed (+ bias).  ``out_dtype`` defaults to x's dtype."""
    out_dtype = out_dtype or x.dtype
    _ptr(x), _ptr(weight)
    if weight.dtype == torch.float32:
        # true float32: also taken by a float32-stored matrix inside a bfloat16 model
        x32 = x if x.dtype == torch.float32 else x.float()
        b32 = None if bias is None else (bias if bias.dtype == torch.float32 else bias.float())
        y = torch.empty((x.shape[0], weight.shape[0]), dtype=torch.float32, device=x.device)
        _call("gemm_f32", "fms_gemm_f32", _ptr(x32), _ptr(weight), _ptr(b32), _ptr(y), x.shape[0], weight.shape[0],
              weight.shape[1], _stream())
        return y if out_dtype == torch.float32 else y.to(out_dtype)
    if weight.dtype != torch.bfloat16 or x.dtype != torch.bfloat16:
        raise KernelError(f"linear: x {x.dtype}, weight {weight.dtype}")
    if x.shape[0] <= SKINNY_ROWS and weight.shape[1] % 8 == 0 and (bias is None or bias.dtype == torch.bfloat16):
        # few rows (decode): the weight-streaming tensor-core kernel
        y = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype, device=x.device)
        _call("gemm_bf16_skinny", "fms_linear_bf16_skinny", _ptr(x), _ptr(weight), _ptr(bias), _ptr(y), _code(out_dtype),
              x.shape[0], weight.shape[0], weight.shape[1], _stream())
        return y
    if _mid_fits(x, weight, bias):
        y = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype, device=x.device)
        _call("gemm_bf16_mid", "fms_linear_bf16_mid", _ptr(x), _ptr(weight), _ptr(bias), _ptr(y), _code(out_dtype),
              x.shape[0], weight.shape[0], weight.shape[1], _ptr(error_flag(x.device)), _stream())
        return y
    if _tensor_core_fits(x, weight, bias):
        return linear_tensor_core(x, weight, bias, out_dtype)
    if out_dtype == torch.float32:
        y = torch.mm(x, weight.t(), out_dtype=torch.float32)
        return y if bias is None else y + bias.float()
    b = None if bias is None else bias.to(torch.bfloat16)
    return torch.nn.functional.linear(x, weight, b)


# Rows from which the tcgen05 kernel with the tokens on the instruction's rows (gemm_bf16_tc.cu) is used instead of the
# library's product.  Measured through whole prefills at the 8B sizes (ms; library for everything / own gated product
# only / own for everything).  The policies taking turns in one warmed-up process: 1,100 tokens 15.4 / 16.4 / 19.6;
# 2,048 tokens 27.5 / 27.5 / 27.5; 4,096 tokens 56.0 / 54.8 / 54.9.  Each in a process of its own: 512 tokens 8.0 /
# 7.8 / 7.8; 1,024 tokens 14.8 / 12.8 / -; 1,280 tokens 17.7 / 17.6 / 19.1; 8,192 tokens 117.0 / 118.7 / 123.2.  The
# own kernel works on tiles of 256 rows, so it loses where the last tile is mostly padding (1,100 rows: a sixth is).
# So the gated product, whose activation the own kernel has in its epilogue, takes the own kernel from 512 rows on
# where at most 6% of the computed rows are padding, and everything else stays with the library unless
# FMS_B200_TC_ROWS / FMS_B200_TC_ROWS_GLU / FMS_B200_TC_MAX_PADDING say otherwise (both row limits were 1,024 once, which
# cost prompts of 1,025 to 1,800 tokens up to a quarter of their time).
TENSOR_CORE_ROWS = int(os.environ.get("FMS_B200_TC_ROWS", str(1 << 30)))
TENSOR_CORE_ROWS_GLU = int(os.environ.get("FMS_B200_TC_ROWS_GLU", "512"))
# The projection with the rotation and the cache write in the own kernel's epilogue, against the library's product and
# the rotation kernel after it, whole prefills in processes of their own (ms, fused / two kernels): 1,024 tokens 14.5 /
# 14.1; 2,048 tokens 26.5 / 26.6; 3,000 tokens 40.0 / 41.0; 4,096 tokens 53.3 / 54.3; 8,192 tokens 121.2 / 120.1.
TENSOR_CORE_ROWS_QKV = int(os.environ.get("FMS_B200_TC_ROWS_QKV", "2048"))
TENSOR_CORE_MAX_PADDING = float(os.environ.get("FMS_B200_TC_MAX_PADDING", "1.06"))  # rows computed over rows asked for
USE_TENSOR_CORE_GEMM = os.environ.get("FMS_B200_TC_GEMM", "1") != "0"


# The tcgen05 kernel with the weights on the instruction's rows (gemm_bf16_mid.cu), for SKINNY_ROWS + 1 to MID_ROWS
# rows.  By default it takes the gated feed-forward product up to 128 rows, where it is ahead of the library's
# product followed by the activation kernel (a decode step of batch 16 at the 8B sizes: 3.75 against 3.86 ms; batch 32:
# 4.59 against 4.66; batch 64: at par; batch 96: 6.80 against 6.90; batch 128: 7.89 against 7.93; batch 256: 13.70
# against 12.99, hence no further).  The plain products and the fused projection, whose matrices have too few
# rows for one block a tile and so run as clusters that add their sums, are 3 to 9 us a product behind the library
# (batch 16: 4.02 ms with them, batch 64: 6.47) and stay with it unless FMS_B200_MID_OPS names them
# ("linear,glu,qkv"; FMS_B200_MID_ROWS up to 256; FMS_B200_MID_GEMM=0 turns the kernel off).
MID_ROWS = min(256, int(os.environ.get("FMS_B200_MID_ROWS", "128")))
USE_MID_GEMM = os.environ.get("FMS_B200_MID_GEMM", "1") != "0"
MID_OPS = os.environ.get("FMS_B200_MID_OPS", "glu").split(",")


def _mid_fits(x, weight, bias, op: str = "linear") -> bool:
    return (USE_MID_GEMM and op in MID_OPS and SKINNY_ROWS < x.shape[0] <= MID_ROWS and weight.shape[1] % 8 == 0
            and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and (bias is None or bias.dtype == torch.bfloat16))


def _tensor_core_fits(x, weight, bias, rows_from: Optional[int] = None) -> bool:
    rows_from = TENSOR_CORE_ROWS if rows_from is None else rows_from
    return (USE_TENSOR_CORE_GEMM and x.shape[0] >= rows_from and weight.shape[1] % 8 == 0
            and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and (bias is None or bias.dtype == torch.bfloat16))


def linear_tensor_core(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                       out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """The product on the tcgen05 tensor cores (TMA-fed, accumulator in tensor memory): bfloat16 in, bfloat16 or
    float32 out.  K must be a multiple of 8."""
    out_dtype = out_dtype or x.dtype
    y = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype, device=x.device)
    _call("gemm_bf16_tc", "fms_gemm_bf16_tc", _ptr(x), _ptr(weight), _ptr(bias), _ptr(y), _code(out_dtype), x.shape[0],
          weight.shape[0], weight.shape[1], _ptr(error_flag(x.device)), _stream())
    return y


def gated_linear_tensor_core(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                             activation: int) -> torch.Tensor:
    """act(x Wg^T) * (x Wu^T) in one tcgen05 kernel: gate and up rows share a tile, the epilogue multiplies."""
    hidden = weight.shape[0] // 2
    y = torch.empty((x.shape[0], hidden), dtype=torch.bfloat16, device=x.device)
    _call("gemm_bf16_tc", "fms_glu_bf16_tc", _ptr(x), _ptr(weight), _ptr(bias), _ptr(y), x.shape[0], hidden,
          weight.shape[1], int(activation), _ptr(error_flag(x.device)), _stream())
    return y


SKINNY_ROWS = 8  # rows up to which the weight-streaming kernels are used (more rows re-read x too often)


# ---- feed-forward ------------------------------------------------------------------------------------
def gated_linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], activation: int) -> torch.Tensor:
    """act(x Wg^T) * (x Wu^T) for weight = [Wg; Wu]: one kernel for few bfloat16 rows, else the product
    followed by ``gated_activation``."""
    hidden = weight.shape[0] // 2
    if (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[0] <= SKINNY_ROWS
            and weight.shape[1] % 8 == 0 and (bias is None or bias.dtype == torch.bfloat16)):
        _ptr(x), _ptr(weight)
        y = torch.empty((x.shape[0], hidden), dtype=torch.bfloat16, device=x.device)
        _call("gemm_bf16_skinny", "fms_glu_bf16_skinny", _ptr(x), _ptr(weight), _ptr(bias), _ptr(y), x.shape[0], hidden,
              weight.shape[1], int(activation), _stream())
        return y
    if _mid_fits(x, weight, bias, "glu"):
        _ptr(x), _ptr(weight)
        y = torch.empty((x.shape[0], hidden), dtype=torch.bfloat16, device=x.device)
        _call("gemm_bf16_mid", "fms_glu_bf16_mid", _ptr(x), _ptr(weight), _ptr(bias), _ptr(y), x.shape[0], hidden,
              weight.shape[1], int(activation), _ptr(error_flag(x.device)), _stream())
        return y
    # the own kernel works on tiles of 256 rows: where the last one would be mostly padding, the library is ahead
    if (_tensor_core_fits(x, weight, bias, TENSOR_CORE_ROWS_GLU)
            and (x.shape[0] + 255) // 256 * 256 <= TENSOR_CORE_MAX_PADDING * x.shape[0]):
        return gated_linear_tensor_core(x, weight, bias, activation)
    return gated_activation(linear(x, weight, bias), activation)


def gated_activation(gate_up: torch.Tensor, activation: int) -> torch.Tensor:
    """act(gate) * up for rows [gate | up]."""
    n, two_f = gate_up.shape
    hidden = two_f // 2
    out = torch.empty((n, hidden), dtype=gate_up.dtype, device=gate_up.device)
    _call("elementwise", "fms_gated_activation", _ptr(gate_up), _ptr(out), _code(gate_up.dtype), n, hidden,
          int(activation), _stream())
    return out


# ---- attention ---------------------------------------------------------------------------------------
def rope_store(qkv: torch.Tensor, inv_freq: Optional[torch.Tensor], batch, view, nheads: int, kvheads: int,
               head_dim: int, writes_cache: bool = True) -> torch.Tensor:
    """Rotates q and k of ``qkv`` [tokens, (nheads + 2 kvheads) head_dim] by each token's position, writes k
    and v into the cache at the token's slot and place, returns the rotated q [tokens, nheads head_dim].  The
    rotation sees ``batch.position_ids`` where the batch has them (sequences that did not start at position 0),
    else the token's place in the cache, ``batch.positions``; ``inv_freq`` None rotates nothing."""
    n = qkv.shape[0]
    if view.keys.dtype != qkv.dtype:
        raise KernelError(f"cache is {view.keys.dtype}, activations are {qkv.dtype}")
    q = torch.empty((n, nheads * head_dim), dtype=qkv.dtype, device=qkv.device)
    _call("elementwise", "fms_rope_store", _ptr(qkv), _code(qkv.dtype), _ptr(q), _ptr(inv_freq), _ptr(batch.positions),
          _ptr(getattr(batch, "position_ids", None)), _ptr(batch.token_seq), _ptr(batch.slots), _ptr(view.keys),
          _ptr(view.values), _ptr(view.table),
          view.table.shape[1], view.block_tokens, n, nheads, kvheads, head_dim, 1 if writes_cache else 0,
          _ptr(error_flag(qkv.device)), batch.slots.shape[0], view.table.shape[0], view.keys.shape[0], _stream())
    return q


FUSE_QKV_ROPE = os.environ.get("FMS_B200_FUSE_QKV_ROPE", "1") != "0"


def rotary_table(inv_freq: torch.Tensor, batch) -> torch.Tensor:
    """[tokens, head_dim / 2, 2] float32: (sin, cos) of every token's rotation angles, made once a step and kept
    with the batch (``batch.scratch``, which the decoder empties when a step starts) for every layer that rotates by
    the same frequencies."""
    scratch = getattr(batch, "scratch", None)
    key = ("rotary_table", inv_freq.data_ptr())
    if scratch is not None and key in scratch:
        return scratch[key]
    n, half = batch.positions.shape[0], inv_freq.shape[0]
    out = torch.empty((n, half, 2), dtype=torch.float32, device=inv_freq.device)
    _call("elementwise", "fms_rotary_table", _ptr(inv_freq), _ptr(batch.positions), _ptr(getattr(batch, "position_ids", None)),
          _ptr(out), n, half, _stream())
    if scratch is not None:
        scratch[key] = out
    return out


def qkv_rope_store(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor],
                   batch, view, nheads: int, kvheads: int, head_dim: int, writes_cache: bool = True) -> torch.Tensor:
    """An attention layer's fused projection and what follows it: qkv = x weight^T (+ bias), q and k rotated by each
    token's position, k and v written into the cache, the rotated q returned.  For a few bfloat16 rows (a decode
    step) this is one kernel, the weight-streaming product with the rotation and the cache write in its epilogue;
    else the product and ``rope_store`` one after the other."""
    if (FUSE_QKV_ROPE and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[0] <= SKINNY_ROWS
            and weight.shape[1] % 8 == 0 and head_dim % 2 == 0 and (bias is None or bias.dtype == torch.bfloat16)
            and view.keys.dtype == torch.bfloat16 and weight.shape[0] == (nheads + 2 * kvheads) * head_dim):
        n = x.shape[0]
        q = torch.empty((n, nheads * head_dim), dtype=x.dtype, device=x.device)
        _call("gemm_bf16_skinny", "fms_qkv_rope_store_bf16_skinny", _ptr(x), _ptr(weight), _ptr(bias), _ptr(q),
              _ptr(inv_freq), _ptr(batch.positions), _ptr(getattr(batch, "position_ids", None)), _ptr(batch.token_seq),
              _ptr(batch.slots), _ptr(view.keys), _ptr(view.values), _ptr(view.table), view.table.shape[1],
              view.block_tokens, n, weight.shape[1], nheads,
              kvheads, head_dim, 1 if writes_cache else 0, _ptr(error_flag(x.device)), batch.slots.shape[0],
              view.table.shape[0], view.keys.shape[0], _stream())
        return q
    if (FUSE_QKV_ROPE and _mid_fits(x, weight, bias, "qkv") and head_dim % 2 == 0 and view.keys.dtype == torch.bfloat16
            and weight.shape[0] == (nheads + 2 * kvheads) * head_dim):
        n = x.shape[0]
        q = torch.empty((n, nheads * head_dim), dtype=x.dtype, device=x.device)
        _call("gemm_bf16_mid", "fms_qkv_rope_store_bf16_mid", _ptr(x), _ptr(weight), _ptr(bias), _ptr(q), _ptr(inv_freq),
              _ptr(batch.positions), _ptr(getattr(batch, "position_ids", None)), _ptr(batch.token_seq), _ptr(batch.slots),
              _ptr(view.keys), _ptr(view.values), _ptr(view.table), view.table.shape[1], view.block_tokens, n,
              weight.shape[1], nheads, kvheads, head_dim, 1 if writes_cache else 0, _ptr(error_flag(x.device)),
              batch.slots.shape[0], view.table.shape[0], view.keys.shape[0], _stream())
        return q
    if (FUSE_QKV_ROPE and _tensor_core_fits(x, weight, bias, TENSOR_CORE_ROWS_QKV) and head_dim % 16 == 0
            and (x.shape[0] + 255) // 256 * 256 <= TENSOR_CORE_MAX_PADDING * x.shape[0]
            and view.keys.dtype == torch.bfloat16 and weight.shape[0] == (nheads + 2 * kvheads) * head_dim):
        # many tokens: the tcgen05 product with the rotation and the cache write in its epilogue; the angles' sines and
        # cosines come from a table that the step's first such layer makes for all layers with the same frequencies
        n = x.shape[0]
        q = torch.empty((n, nheads * head_dim), dtype=x.dtype, device=x.device)
        table = None if inv_freq is None else rotary_table(inv_freq, batch)
        _call("gemm_bf16_tc", "fms_qkv_rope_store_bf16_tc", _ptr(x), _ptr(weight), _ptr(bias), _ptr(q), _ptr(table),
              _ptr(batch.positions), _ptr(batch.token_seq), _ptr(batch.slots),
              _ptr(view.keys), _ptr(view.values), _ptr(view.table), view.table.shape[1], view.block_tokens, n,
              weight.shape[1], nheads, kvheads, head_dim, 1 if writes_cache else 0, _ptr(error_flag(x.device)),
              batch.slots.shape[0], view.table.shape[0], view.keys.shape[0], _stream())
        return q
    return rope_store(linear(x, weight, bias), inv_freq, batch, view, nheads, kvheads, head_dim, writes_cache)


def _attention_library(head_dim: int) -> str:
    return f"attention_hd{head_dim}"


_attn_constants = {}


def attention_constants(head_dim: int, dtype: torch.dtype, nheads: int, kvheads: int):
    """(keys per decode split, positions per prefill tile) of the library built for this head size."""
    key = (head_dim, dtype, nheads, kvheads)
    if key not in _attn_constants:
        lib = load_library(_attention_library(head_dim))
        _attn_constants[key] = (int(lib.fms_attn_split_tokens()),
                                int(lib.fms_attn_prefill_tile_positions(_code(dtype), nheads, kvheads)))
    return _attn_constants[key]


def attention(q: torch.Tensor, batch, view, nheads: int, kvheads: int, head_dim: int, scale: float,
              window: int) -> torch.Tensor:
    """Causal softmax attention of the step's queries over the cache (which already holds the step's own
    keys and values).  One query per sequence takes the split-key decode kernels, else the prefill kernel."""
    out = torch.empty_like(q)
    lib = _attention_library(head_dim)
    split, tile_rows = attention_constants(head_dim, q.dtype, nheads, kvheads)
    common = (_ptr(q), _ptr(out), _code(q.dtype), _ptr(view.keys), _ptr(view.values), _ptr(view.table),
              view.table.shape[1], view.block_tokens, _ptr(batch.slots), _ptr(batch.first_row), _ptr(batch.len_after))
    if batch.decode:
        n_splits = (batch.max_len_after + split - 1) // split
        part_o = torch.empty((batch.n_seqs, nheads, n_splits, head_dim), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((batch.n_seqs, nheads, n_splits, 2), dtype=torch.float32, device=q.device)
        # total_len (what the host knows of the sequences' lengths) chooses between the two bfloat16 decode kernels
        _call(lib, "fms_attention_decode", *common, batch.n_seqs, n_splits, _ptr(part_o), _ptr(part_ml), nheads,
              kvheads, head_dim, float(scale), int(window), view.keys.shape[0], view.table.shape[0],
              int(getattr(batch, "total_len", 0)),
              _ptr(_work_counter(q.device)), _ptr(error_flag(q.device)), _stream())
        if n_splits > 1 or q.dtype == torch.float32:
            global launches
            launches += 1  # the kernel that merges the splits
    else:
        tiles = batch.query_tiles(tile_rows)
        _call(lib, "fms_attention_prefill", *common, _ptr(tiles), tiles.shape[0], nheads, kvheads, head_dim,
              float(scale), int(window), view.keys.shape[0], view.table.shape[0], _ptr(error_flag(q.device)), _stream())
    return out


def attention_stream_launches(head_dim: int) -> int:
    """How often this process has launched (or captured) the streaming decode-attention kernel of a head size."""
    lib = load_library(f"attention_hd{head_dim}")
    lib.fms_attn_stream_launches.restype = ctypes.c_long
    return int(lib.fms_attn_stream_launches())


def decode_advance(positions: torch.Tensor, lengths: torch.Tensor, offsets: Optional[torch.Tensor] = None,
                   position_ids: Optional[torch.Tensor] = None, slots: Optional[torch.Tensor] = None,
                   spare_slot: int = -1) -> None:
    """positions[i] = lengths[i]; lengths[i] += 1 — the bookkeeping of a decode step, on the device.  With
    ``offsets`` (sequences that did not start at position 0) also position_ids[i] = positions[i] + offsets[i].
    With ``slots``: a row in ``spare_slot`` (one that only fills the step up to a captured size) restarts at
    position 0 every step."""
    _call("elementwise", "fms_decode_advance", _ptr(positions), _ptr(lengths), _ptr(offsets), _ptr(position_ids),
          _ptr(slots), int(spare_slot), positions.shape[0], _stream())


# ---- sampling ----------------------------------------------------------------------------------------
def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    rows, vocab = logits.shape
    if logits.dtype != torch.float32:
        raise KernelError("logits are float32")
    out = out if out is not None else torch.empty((rows,), dtype=torch.int32, device=logits.device)
    _call("sampling", "fms_argmax", _ptr(logits), _ptr(out), rows, vocab, _stream())
    return out


def sample(logits: torch.Tensor, temperature: float, top_k: int, seed: int, requests: torch.Tensor, step: int,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    rows, vocab = logits.shape
    if logits.dtype != torch.float32:
        raise KernelError("logits are float32")
    out = out if out is not None else torch.empty((rows,), dtype=torch.int32, device=logits.device)
    _call("sampling", "fms_sample", _ptr(logits), _ptr(out), rows, vocab, float(temperature), int(top_k),
          int(seed) & 0xFFFFFFFFFFFFFFFF, _ptr(requests), int(step), _stream())
    return out
