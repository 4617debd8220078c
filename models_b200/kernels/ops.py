"""Python faces of the CUDA launchers: shape and dtype checks, then one C call on the current stream.

There is no CPU path and no library stand-in: a tensor that is not on a CUDA device, or a kernel
library that cannot be built, raises.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .build import load_library

_F32, _BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return _F32
    if dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"kernels take float32 or bfloat16 storage, got {dtype}")


def _cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError(
                "models_b200 kernels run on a CUDA device only (got a tensor on "
                f"{t.device}); there is no CPU path")


def _p(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _stream():
    """The current stream of the current device, as the raw handle the launchers take (the two
    calls below are what torch.cuda.current_stream() ends in, without its Python layers: this runs
    once per kernel launch)."""
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice()))


_launches = [0]


def launch_count() -> int:
    """Launches of this package's own kernels so far (graph replays count the kernels they hold)."""
    return _launches[0]


def add_launches(n: int) -> None:
    _launches[0] += n


_recorded = [None]  # a list while launches are being recorded (see `recording`), else None


class recording:
    """`with ops.recording() as names:` collects, in order, which launcher of this module ran each of this
    package's kernels (the function's name says which form of a product it is).  For reports, not for hot loops."""

    def __enter__(self):
        self.before, _recorded[0] = _recorded[0], []
        return _recorded[0]

    def __exit__(self, *exc):
        _recorded[0] = self.before
        return False


def _run(lib, status: int):
    if status != 0:
        raise KernelError(lib.mb_last_error().decode("utf-8", "replace"))
    _launches[0] += 1
    if _recorded[0] is not None:
        import sys
        _recorded[0].append(sys._getframe(1).f_code.co_name)


def _int32(t: Optional[torch.Tensor], name: str):
    if t is not None and (t.dtype != torch.int32 or not t.is_contiguous()):
        raise KernelError(f"{name} must be a contiguous int32 tensor, got {t.dtype}")


# ------------------------------------------------------------------------------------ libraries

def elementwise():
    return load_library("mb_elementwise", ["elementwise.cu"])


def attention_rows():
    return load_library("mb_attention_rows", ["attention_rows.cu"])


def attention_tc(head_dim: int):
    """The tensor-core attention kernels, compiled for this head size at first use."""
    return load_library("mb_attention_tc", ["attention_tc.cu"], {"MB_HEAD_DIM": int(head_dim)})


def attention_tc_takes(dtype: torch.dtype, head_dim: int, page_size: int) -> bool:
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256 and page_size == 64


def prefill_attention_tc(head_dim: int):
    """The tcgen05 prefill attention, compiled for this head size (64 or 128) at first use."""
    return load_library("mb_prefill_attention_tcgen05", ["prefill_attention_tcgen05.cu"], {"MB_HEAD_DIM": int(head_dim)})


TCGEN05_ATTENTION_MIN_ROWS = 33  # shorter steps go to the mma.sync kernel, whose blocks take 64 query rows


def prefill_attention_tcgen05_takes(q: torch.Tensor, out: torch.Tensor, head_dim: int, max_q_len: int) -> bool:
    """Head sizes 64 and 128, steps of more than a few tokens, rows that TMA and 16-byte stores can address."""
    return (head_dim in (64, 128) and max_q_len >= TCGEN05_ATTENTION_MIN_ROWS and q.stride(0) % 8 == 0
            and out.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0)


def gemm32():
    return load_library("mb_gemm_f32", ["gemm_f32.cu"])


def sampling():
    return load_library("mb_sampling", ["sampling.cu"])


def random_init():
    return load_library("mb_random_init", ["random_init.cu"])


def random_normal(out: torch.Tensor, key, mean: float, std: float) -> torch.Tensor:
    """Fills `out` (contiguous float32 or bfloat16) with mean + std * z, z standard normal from the
    counter-based generator keyed by `key` (two 32-bit words): the values of weights/philox_normal.py."""
    _cuda(out)
    if not out.is_contiguous():
        raise KernelError("random_normal fills a contiguous tensor")
    lib = random_init()
    _run(lib, lib.mb_random_normal(_p(out), _code(out.dtype), ctypes.c_size_t(out.numel()), ctypes.c_uint32(key[0]),
                                   ctypes.c_uint32(key[1]), ctypes.c_float(mean), ctypes.c_float(std), _stream()))
    return out


# ------------------------------------------------------------------------------------ element-wise

def embed_gather(table: torch.Tensor, tokens: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """Rows of `table` ([vocab, width]) picked by `tokens` (int32), as the float residual stream."""
    _cuda(table, tokens)
    _int32(tokens, "tokens")
    if table.dim() != 2 or not table.is_contiguous():
        raise KernelError("embedding table must be a contiguous [vocab, width] matrix")
    rows, (vocab, width) = tokens.numel(), table.shape
    out = torch.empty((rows, width), dtype=torch.float32, device=table.device)
    lib = elementwise()
    _run(lib, lib.mb_embed_gather(_p(table), _code(table.dtype), _p(tokens), _p(out), rows, width, vocab,
                                  ctypes.c_float(scale), _stream()))
    return out


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None, write_x: bool = True) -> torch.Tensor:
    """x (float residual, [T, width]) += delta, then RMSNorm with `weight` (float).  With `rows`
    only those rows are normalised (and x is left alone).  Returns the normalised rows."""
    _cuda(x, delta, weight, rows)
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous():
        raise KernelError("the residual stream must be a contiguous float32 [rows, width] tensor")
    width = x.shape[1]
    if weight.dtype != torch.float32 or weight.numel() != width:
        raise KernelError(f"norm weight must be float32 of {width} elements, got {weight.dtype} of {weight.numel()}")
    if delta is not None and (delta.shape != x.shape or not delta.is_contiguous()):
        raise KernelError(f"delta {tuple(delta.shape)} must match the residual stream {tuple(x.shape)}")
    _int32(rows, "rows")
    out_rows = rows.numel() if rows is not None else x.shape[0]
    out = torch.empty((out_rows, width), dtype=out_dtype, device=x.device)
    lib = elementwise()
    _run(lib, lib.mb_add_rmsnorm(_p(x), _p(delta), _code(delta.dtype) if delta is not None else 0, _p(weight), _p(out),
                                 _code(out_dtype), _p(rows), out_rows, width, ctypes.c_float(eps),
                                 1 if (write_x and rows is None) else 0, _stream()))
    return out


def rope_cache_write(qkv: torch.Tensor, positions: Optional[torch.Tensor], cos: Optional[torch.Tensor],
                     sin: Optional[torch.Tensor], k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                     slot_mapping: Optional[torch.Tensor], heads: int, kv_heads: int, head_dim: int, rotary_dim: int,
                     interleaved: bool, page_size: int, write_cache: bool) -> None:
    """Rotates the query heads of `qkv` ([T, (heads + 2*kv_heads) * head_dim]) in place; rotates the
    key heads and copies the value heads into the pools at `slot_mapping`."""
    _cuda(qkv, positions, cos, sin, k_pool, v_pool, slot_mapping)
    if qkv.dim() != 2 or qkv.stride(1) != 1:
        raise KernelError("qkv must be a [tokens, columns] tensor with unit column stride")
    need = (heads + (2 * kv_heads if write_cache else 0)) * head_dim
    if qkv.shape[1] < need:
        raise KernelError(f"qkv rows have {qkv.shape[1]} columns, {need} are needed")
    _int32(positions, "positions")
    _int32(slot_mapping, "slot_mapping")
    if rotary_dim > 0:
        if cos is None or sin is None or cos.dtype != torch.float32 or sin.dtype != torch.float32:
            raise KernelError("rotation needs float32 cos/sin tables")
        if cos.shape[-1] != rotary_dim // 2 or cos.shape != sin.shape or not cos.is_contiguous() or not sin.is_contiguous():
            raise KernelError(f"cos/sin tables must be contiguous [positions, {rotary_dim // 2}]")
    if write_cache and (k_pool.dtype != qkv.dtype or v_pool.dtype != qkv.dtype):
        raise KernelError(f"cache pools ({k_pool.dtype}) must have the dtype of qkv ({qkv.dtype})")
    lib = elementwise()
    _run(lib, lib.mb_rope_cache_write(_p(qkv), _code(qkv.dtype), qkv.stride(0), _p(positions), _p(cos), _p(sin),
                                      _p(k_pool), _p(v_pool), _p(slot_mapping), qkv.shape[0], heads, kv_heads,
                                      head_dim, rotary_dim, 1 if interleaved else 0, page_size,
                                      1 if write_cache else 0, _stream()))


ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "relu2": 2}  # the codes of csrc/common.cuh (MB_ACT_*)


def activation_code(activation: str) -> int:
    if activation not in ACTIVATIONS:
        raise KernelError(f"gate activation {activation!r} is not built (known: {', '.join(sorted(ACTIVATIONS))})")
    return ACTIVATIONS[activation]


def gated_epilogue(activation: str = "silu") -> int:
    """The epilogue code of a gate/up product that stores act(gate) * up: EPI_SWIGLU with the
    activation in the bits above it (silu gives EPI_SWIGLU itself)."""
    return EPI_SWIGLU | (activation_code(activation) << 8)


def swiglu(gate_up: torch.Tensor, activation: str = "silu") -> torch.Tensor:
    """act(gate) * up for a [rows, 2*width] tensor whose first half of columns is the gate."""
    _cuda(gate_up)
    if gate_up.dim() != 2 or not gate_up.is_contiguous() or gate_up.shape[1] % 2:
        raise KernelError("gate_up must be a contiguous [rows, 2*width] tensor")
    rows, width = gate_up.shape[0], gate_up.shape[1] // 2
    out = torch.empty((rows, width), dtype=gate_up.dtype, device=gate_up.device)
    lib = elementwise()
    _run(lib, lib.mb_swiglu(_p(gate_up), _p(out), _code(gate_up.dtype), rows, width, activation_code(activation), _stream()))
    return out


def logit_epilogue(logits: torch.Tensor, scale: float, softcap: float) -> torch.Tensor:
    """In place on float32 logits [rows, vocab]: times `scale`, then softcap * tanh(logits / softcap)
    unless softcap is 0."""
    _cuda(logits)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("logit_epilogue takes float32 [rows, vocab] logits")
    lib = elementwise()
    _run(lib, lib.mb_logit_epilogue(_p(logits), logits.stride(0), logits.shape[0], logits.shape[1], ctypes.c_float(scale),
                                    ctypes.c_float(softcap), _stream()))
    return logits


def bias_add(x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    _cuda(x, bias)
    if not x.is_contiguous() or bias.dtype != torch.float32 or bias.numel() != x.shape[-1]:
        raise KernelError("bias_add needs a contiguous x and a float32 bias of x's width")
    lib = elementwise()
    _run(lib, lib.mb_bias_add(_p(x), _code(x.dtype), _p(bias), x.numel() // x.shape[-1], x.shape[-1], _stream()))
    return x


def residual_add(x: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    _cuda(x, delta)
    if x.dtype != torch.float32 or not x.is_contiguous() or not delta.is_contiguous() or delta.shape != x.shape:
        raise KernelError("residual_add needs a contiguous float32 x and a delta of the same shape")
    lib = elementwise()
    _run(lib, lib.mb_residual_add(_p(x), _p(delta), _code(delta.dtype), ctypes.c_size_t(x.numel()), _stream()))
    return x


def layernorm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float, out_dtype: torch.dtype,
              rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Layer norm with gain and bias (None: no bias) of the float residual rows x [T, width] (of the rows picked by `rows`,
    if given): mean, variance and the result in float, stored as `out_dtype`."""
    _cuda(x, weight, bias, rows)
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous():
        raise KernelError("the residual stream must be a contiguous float32 [rows, width] tensor")
    width = x.shape[1]
    for name, t in (("weight", weight), ("bias", bias)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != width or not t.is_contiguous()):
            raise KernelError(f"layer norm {name} must be contiguous float32 of {width} elements")
    _int32(rows, "rows")
    out_rows = rows.numel() if rows is not None else x.shape[0]
    out = torch.empty((out_rows, width), dtype=out_dtype, device=x.device)
    lib = elementwise()
    _run(lib, lib.mb_layernorm(_p(x), _p(weight), _p(bias), _p(out), _code(out_dtype), _p(rows), out_rows, width,
                               ctypes.c_float(eps), _stream()))
    return out


def outnorm_add(x: torch.Tensor, a: torch.Tensor, weight: torch.Tensor, scale: torch.Tensor, eps: float,
                b: Optional[torch.Tensor] = None, gain_a: Optional[torch.Tensor] = None, gain_b: Optional[torch.Tensor] = None,
                copy_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """x += scale * LN(y) in place on the float32 stream x [T, width], where LN(y) = (y - mean) / sqrt(var + eps) * weight
    (no bias) and y is the sublayer's float32 result `a`, or -- given a second result `b` -- the mean of the two after an RMS
    norm each, y = 1/2 (a / rms(a) * gain_a + b / rms(b) * gain_b).  With `copy_dtype` the new rows of x are also returned
    in that type (what the next sublayer's products read)."""
    _cuda(x, a, b, gain_a, gain_b, weight, scale)
    width = x.shape[1]
    for name, t in (("x", x), ("a", a), ("b", b)):
        if t is not None and (t.dtype != torch.float32 or tuple(t.shape) != tuple(x.shape) or not t.is_contiguous()):
            raise KernelError(f"outnorm_add: {name} must be contiguous float32 {tuple(x.shape)}")
    for name, t in (("weight", weight), ("scale", scale), ("gain_a", gain_a), ("gain_b", gain_b)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != width or not t.is_contiguous()):
            raise KernelError(f"outnorm_add: {name} must be contiguous float32 of {width} elements")
    if b is not None and (gain_a is None or gain_b is None):
        raise KernelError("outnorm_add: two results need two gains")
    copy = torch.empty_like(x, dtype=copy_dtype) if copy_dtype is not None else None
    lib = elementwise()
    _run(lib, lib.mb_outnorm_add(_p(x), _p(a), _p(b), _p(gain_a), _p(gain_b), _p(weight), _p(scale), _p(copy),
                                 _code(copy_dtype) if copy_dtype is not None else _F32, x.shape[0], width, ctypes.c_float(eps), _stream()))
    return copy


def pair_norm_mean(a: torch.Tensor, b: torch.Tensor, gain_a: torch.Tensor, gain_b: torch.Tensor, eps: float) -> torch.Tensor:
    """1/2 (a / rms(a) * gain_a + b / rms(b) * gain_b) row by row, rms(v) = sqrt(mean(v^2) + eps); float32 [T, width]."""
    _cuda(a, b, gain_a, gain_b)
    width = a.shape[1]
    for name, t in (("a", a), ("b", b)):
        if t.dtype != torch.float32 or tuple(t.shape) != tuple(a.shape) or not t.is_contiguous():
            raise KernelError(f"pair_norm_mean: {name} must be contiguous float32 {tuple(a.shape)}")
    for name, t in (("gain_a", gain_a), ("gain_b", gain_b)):
        if t.dtype != torch.float32 or t.numel() != width or not t.is_contiguous():
            raise KernelError(f"pair_norm_mean: {name} must be contiguous float32 of {width} elements")
    out = torch.empty_like(a)
    lib = elementwise()
    _run(lib, lib.mb_outnorm_add(_p(out), _p(a), _p(b), _p(gain_a), _p(gain_b), None, None, None, _F32, a.shape[0], width,
                                 ctypes.c_float(eps), _stream()))
    return out


def store_rows(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """The float32 rows x stored as `dtype` (what a matrix product of that type reads)."""
    _cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("store_rows: the rows must be contiguous float32")
    out = torch.empty_like(x, dtype=dtype)
    lib = elementwise()
    _run(lib, lib.mb_store_rows(_p(x), _p(out), _code(dtype), ctypes.c_size_t(x.numel()), _stream()))
    return out


def _columns(t: torch.Tensor, name: str):
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{name} must be a [rows, columns] tensor (or column slice) with unit column stride")


def activate(src: torch.Tensor, dst: torch.Tensor, activation: str, scale: float = 1.0) -> torch.Tensor:
    """dst = scale * act(src), element by element; both may be column slices of wider tensors."""
    _cuda(src, dst)
    _columns(src, "src")
    _columns(dst, "dst")
    if src.shape != dst.shape or src.dtype != dst.dtype:
        raise KernelError(f"activate: {tuple(src.shape)} {src.dtype} does not fit {tuple(dst.shape)} {dst.dtype}")
    lib = elementwise()
    _run(lib, lib.mb_activate(_p(src), src.stride(0), _p(dst), dst.stride(0), _code(src.dtype), src.shape[0], src.shape[1],
                              activation_code(activation), ctypes.c_float(scale), _stream()))
    return dst


def xielu(src: torch.Tensor, dst: torch.Tensor, a_pos: float, a_neg: float, scale: float = 1.0) -> torch.Tensor:
    """dst = scale * (a_pos z^2 + z/2 where z > 0, a_neg (exp(z) - 1 - z) + z/2 elsewhere), element by element; both may
    be column slices of wider tensors."""
    _cuda(src, dst)
    _columns(src, "src")
    _columns(dst, "dst")
    if src.shape != dst.shape or src.dtype != dst.dtype:
        raise KernelError(f"xielu: {tuple(src.shape)} {src.dtype} does not fit {tuple(dst.shape)} {dst.dtype}")
    lib = elementwise()
    _run(lib, lib.mb_xielu(_p(src), src.stride(0), _p(dst), dst.stride(0), _code(src.dtype), src.shape[0], src.shape[1],
                           ctypes.c_float(a_pos), ctypes.c_float(a_neg), ctypes.c_float(scale), _stream()))
    return dst


def gated_residual_add(x: torch.Tensor, gate: torch.Tensor, bias: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """x += sigmoid(gate + bias) * delta for the float32 residual stream x [rows, width]; gate [rows, width] may be a
    column slice, bias is float32 [width], delta contiguous [rows, width]; float arithmetic."""
    _cuda(x, gate, bias, delta)
    _columns(gate, "gate")
    if x.dtype != torch.float32 or not x.is_contiguous() or x.dim() != 2:
        raise KernelError("gated_residual_add: x must be a contiguous float32 [rows, width] tensor")
    if gate.shape != x.shape or delta.shape != x.shape or not delta.is_contiguous():
        raise KernelError(f"gated_residual_add: gate {tuple(gate.shape)} and delta {tuple(delta.shape)} must match x {tuple(x.shape)}")
    if bias.dtype != torch.float32 or bias.numel() != x.shape[1] or not bias.is_contiguous():
        raise KernelError(f"gated_residual_add: bias must be contiguous float32 of {x.shape[1]} elements")
    lib = elementwise()
    _run(lib, lib.mb_gated_residual_add(_p(x), _p(gate), gate.stride(0), _code(gate.dtype), _p(bias), _p(delta), _code(delta.dtype),
                                        x.shape[0], x.shape[1], _stream()))
    return x


# ------------------------------------------------------------------------------------ attention

def paged_attention_rows(q: torch.Tensor, out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                         block_table: torch.Tensor, cu_q: torch.Tensor, kv_lens: torch.Tensor, max_q_len: int,
                         heads: int, kv_heads: int, head_dim: int, window: Optional[int], scale: float) -> None:
    """q: [T, >= heads*head_dim] (may be a column slice of a wider tensor); out: [T, heads*head_dim].
    Pools: [pages, kv_heads, page_size, head_dim]."""
    _cuda(q, out, k_pool, v_pool, block_table, cu_q, kv_lens)
    _int32(block_table, "block_table")
    _int32(cu_q, "cu_q")
    _int32(kv_lens, "kv_lens")
    if q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("q and out need unit column stride")
    if k_pool.dim() != 4 or k_pool.shape[1] != kv_heads or k_pool.shape[3] != head_dim or not k_pool.is_contiguous():
        raise KernelError(f"k_pool must be contiguous [pages, {kv_heads}, page_size, {head_dim}], got {tuple(k_pool.shape)}")
    if v_pool.shape != k_pool.shape or not v_pool.is_contiguous():
        raise KernelError("v_pool must match k_pool")
    if not (q.dtype == out.dtype == k_pool.dtype == v_pool.dtype):
        raise KernelError("q, out and the pools must share one dtype")
    sequences = kv_lens.numel()
    lib = attention_rows()
    _run(lib, lib.mb_paged_attention_rows(_p(q), q.stride(0), _p(out), out.stride(0), _code(q.dtype), _p(k_pool),
                                          _p(v_pool), _p(block_table), block_table.shape[1], _p(cu_q), _p(kv_lens),
                                          sequences, max_q_len, heads, kv_heads, head_dim, k_pool.shape[2],
                                          window or 0, ctypes.c_float(scale), _stream()))


def talking_attention_library():
    return load_library("mb_talking_attention", ["talking_attention.cu"])


def rotate_store(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, positions: torch.Tensor, cos: Optional[torch.Tensor],
                 sin: Optional[torch.Tensor], k_pool: torch.Tensor, v_pool: torch.Tensor, slot_mapping: torch.Tensor,
                 heads: int, kv_heads: int, head_dim: int, value_dim: int, rotary_dim: int) -> None:
    """Rotates the query heads of q ([T, heads*head_dim], in place) and the key heads of k by the tables
    (split-half pairs over the first `rotary_dim` coordinates; 0: none), and stores keys and values (value
    heads of `value_dim`) in the pools at `slot_mapping`.  q, k and v may be column slices of one tensor."""
    _cuda(q, k, v, positions, cos, sin, k_pool, v_pool, slot_mapping)
    for name, t, width in (("q", q, heads * head_dim), ("k", k, kv_heads * head_dim), ("v", v, kv_heads * value_dim)):
        _columns(t, name)
        if t.shape[1] != width or t.shape[0] != q.shape[0]:
            raise KernelError(f"rotate_store: {name} is {tuple(t.shape)}, {width} columns are needed")
    _int32(positions, "positions")
    _int32(slot_mapping, "slot_mapping")
    if rotary_dim > 0:
        if cos is None or sin is None or cos.dtype != torch.float32 or sin.dtype != torch.float32:
            raise KernelError("rotation needs float32 cos/sin tables")
        if cos.shape[-1] != rotary_dim // 2 or cos.shape != sin.shape or not cos.is_contiguous() or not sin.is_contiguous():
            raise KernelError(f"cos/sin tables must be contiguous [positions, {rotary_dim // 2}]")
    if not (q.dtype == k.dtype == v.dtype == k_pool.dtype == v_pool.dtype):
        raise KernelError("q, k, v and the cache pools must share one dtype")
    page_size = k_pool.shape[2]
    if (tuple(k_pool.shape[1:]) != (kv_heads, page_size, head_dim) or tuple(v_pool.shape[1:]) != (kv_heads, page_size, value_dim)
            or not k_pool.is_contiguous() or not v_pool.is_contiguous()):
        raise KernelError(f"pools must be contiguous [pages, {kv_heads}, page_size, {head_dim}] and [.., {value_dim}]")
    lib = talking_attention_library()
    _run(lib, lib.mb_rotate_store(_p(q), q.stride(0), _p(k), k.stride(0), _p(v), v.stride(0), _code(q.dtype), _p(positions),
                                  _p(cos), _p(sin), _p(k_pool), _p(v_pool), _p(slot_mapping), q.shape[0], heads, kv_heads,
                                  head_dim, value_dim, rotary_dim, page_size, _stream()))


_tickets = {}  # device -> every ticket array handed out so far (captured steps keep using theirs), the last one current


def _zero_tickets(device, count: int) -> torch.Tensor:
    """`count` int32 zeros that the kernels that take tickets leave zero again, so that one array serves every call
    on the device's streams in turn."""
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    arrays = _tickets.setdefault(key, [])
    if not arrays or arrays[-1].numel() < count:
        arrays.append(torch.zeros(max(count, 256), dtype=torch.int32, device=device))
    return arrays[-1]


def talking_attention_tc_library(heads: int, head_dim: int, value_dim: int):
    """The tensor-core form, compiled for this head count and these key and value sizes at first use."""
    return load_library("mb_talking_attention_tc", ["talking_attention_tc.cu"],
                        {"MB_HEADS": int(heads), "MB_KEY_DIM": int(head_dim), "MB_VALUE_DIM": int(value_dim)})


TALKING_TC_MIN_ROWS = 8  # steps that bring fewer tokens to every sequence go to the kernel with a block per token


def talking_attention_tc_takes(q: torch.Tensor, out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, heads: int,
                               kv_heads: int, head_dim: int, value_dim: int, max_q_len: int) -> bool:
    """bfloat16; one warp per head, so at most 16 heads; key and value sizes multiples of 16, with values no wider
    than the registers of a block of that many warps hold as an accumulator; 16-byte query rows; and a block's
    shared memory (queries of 16 tokens, two chunks of keys and values of every key/value head, the heads' weights)."""
    if q.dtype != torch.bfloat16 or max_q_len < TALKING_TC_MIN_ROWS or not 1 <= heads <= 16:
        return False
    if head_dim % 16 or value_dim % 16 or not 16 <= head_dim <= 256 or not 16 <= value_dim <= (256 if heads <= 8 else 128):
        return False
    if q.stride(0) % 8 or out.stride(0) % 2 or q.data_ptr() % 16 or out.data_ptr() % 4 or k_pool.data_ptr() % 16 or v_pool.data_ptr() % 16:
        return False
    block = (heads * 16 * (2 * head_dim + 16) + 2 * kv_heads * 32 * (2 * head_dim + 2 * value_dim + 32) + 4 * (2 * 16 * 516 + heads * heads))
    return block <= 227 * 1024


def talking_attention(q: torch.Tensor, out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                      block_table: torch.Tensor, cu_q: torch.Tensor, kv_lens: torch.Tensor, max_q_len: int, heads: int,
                      kv_heads: int, head_dim: int, value_dim: int, window: Optional[int], keep_first: int, scale: float,
                      talk: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None, out_scale: float = 1.0,
                      kernel: Optional[str] = None, most_positions: Optional[int] = None) -> None:
    """Causal attention over the paged cache with softmax weights mixed across heads by `talk` (float32
    [heads, heads]; None: not mixed), a window that also keeps the first `keep_first` positions, value heads
    of `value_dim`, and an output gate: out_h = out_scale * sigmoid(gate[:, h]) * sum_j w'_h(j) v(j).
    q [T, heads*head_dim], out [T, heads*value_dim], gate [T, heads] (or None) may be column slices.
    `kernel`: None picks the decode form for steps of one token per sequence (the visible keys cut into chunks
    with a block each; `most_positions`, a bound of every sequence's cache length that does not change from
    step to step, sizes its grid: by default what the page table can address), the tensor-core form where it
    applies (bfloat16 steps of many tokens), else the form with a block per token; "decode", "tc" or "rows" asks
    for one of them."""
    if kernel not in (None, "tc", "rows", "decode"):
        raise KernelError(f"talking_attention: unknown kernel {kernel!r}")
    _cuda(q, out, k_pool, v_pool, block_table, cu_q, kv_lens, talk, gate)
    _int32(block_table, "block_table")
    _int32(cu_q, "cu_q")
    _int32(kv_lens, "kv_lens")
    _columns(q, "q")
    _columns(out, "out")
    if q.shape[1] != heads * head_dim or out.shape[1] != heads * value_dim or q.shape[0] != out.shape[0]:
        raise KernelError(f"talking_attention: q {tuple(q.shape)} and out {tuple(out.shape)} do not fit {heads} heads of "
                          f"{head_dim} and {value_dim}")
    page_size = k_pool.shape[2]
    if (tuple(k_pool.shape[1:]) != (kv_heads, page_size, head_dim) or tuple(v_pool.shape[1:]) != (kv_heads, page_size, value_dim)
            or not k_pool.is_contiguous() or not v_pool.is_contiguous()):
        raise KernelError(f"pools must be contiguous [pages, {kv_heads}, page_size, {head_dim}] and [.., {value_dim}]")
    if not (q.dtype == out.dtype == k_pool.dtype == v_pool.dtype):
        raise KernelError("q, out and the pools must share one dtype")
    if talk is not None and (talk.dtype != torch.float32 or tuple(talk.shape) != (heads, heads) or not talk.is_contiguous()):
        raise KernelError(f"talk must be a contiguous float32 [{heads}, {heads}] matrix")
    if gate is not None:
        _columns(gate, "gate")
        if gate.dtype != q.dtype or tuple(gate.shape) != (q.shape[0], heads):
            raise KernelError(f"gate must be [{q.shape[0]}, {heads}] of q's dtype")
    if kernel == "decode" or (kernel is None and max_q_len == 1):
        if max_q_len != 1:
            raise KernelError("the decode form takes one token per sequence")
        sequences = kv_lens.numel()
        bound = most_positions or block_table.shape[1] * page_size
        lib = talking_attention_library()
        lib.mb_talking_decode_scratch_floats.restype = ctypes.c_size_t
        scratch = torch.empty((lib.mb_talking_decode_scratch_floats(sequences, heads, value_dim, bound, window or 0, keep_first),),
                              dtype=torch.float32, device=q.device)
        _run(lib, lib.mb_talking_attention_decode(
            _p(q), q.stride(0), _p(out), out.stride(0), _code(q.dtype), _p(k_pool), _p(v_pool), _p(block_table),
            block_table.shape[1], _p(cu_q), _p(kv_lens), sequences, bound, _p(talk), _p(gate),
            gate.stride(0) if gate is not None else 0, heads, kv_heads, head_dim, value_dim, page_size, window or 0, keep_first,
            ctypes.c_float(scale), ctypes.c_float(out_scale), _p(scratch), _p(_zero_tickets(q.device, sequences)), _stream()))
        _launches[0] += 1  # two kernels
        return
    if kernel == "tc" or (kernel is None and talking_attention_tc_takes(q, out, k_pool, v_pool, heads, kv_heads, head_dim, value_dim,
                                                                      max_q_len)):
        if q.dtype != torch.bfloat16:
            raise KernelError("the tensor-core form takes bfloat16")
        lib = talking_attention_tc_library(heads, head_dim, value_dim)
        _run(lib, lib.mb_talking_attention_tc(
            _p(q), q.stride(0), _p(out), out.stride(0), _p(k_pool), _p(v_pool), _p(block_table), block_table.shape[1], _p(cu_q),
            _p(kv_lens), kv_lens.numel(), max_q_len, _p(talk), _p(gate), gate.stride(0) if gate is not None else 0, kv_heads,
            page_size, window or 0, keep_first, ctypes.c_float(scale), ctypes.c_float(out_scale), _stream()))
        return
    lib = talking_attention_library()
    _run(lib, lib.mb_talking_attention_rows(
        _p(q), q.stride(0), _p(out), out.stride(0), _code(q.dtype), _p(k_pool), _p(v_pool), _p(block_table),
        block_table.shape[1], _p(cu_q), _p(kv_lens), kv_lens.numel(), max_q_len, _p(talk), _p(gate),
        gate.stride(0) if gate is not None else 0, heads, kv_heads, head_dim, value_dim, page_size, window or 0, keep_first,
        ctypes.c_float(scale), ctypes.c_float(out_scale), _stream()))


def gated_attention_library():
    return load_library("mb_gated_attention", ["gated_attention.cu"])


def norm_store(q: Optional[torch.Tensor], k: torch.Tensor, v: Optional[torch.Tensor], positions: torch.Tensor,
               q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor], eps: float, temperature_coef: float,
               temperature_every: int, k_pool: torch.Tensor, v_pool: Optional[torch.Tensor], slot_mapping: torch.Tensor,
               heads: int, kv_heads: int, head_dim: int, value_dim: int) -> None:
    """Per head: q (in place) = q / rms(q) * q_gain * (1 + coef * ln(floor((p + 1) / every) + 1)); keys
    k / rms(k) * k_gain and values (as they are) go into the pools at `slot_mapping`.  rms(x) = sqrt(mean(x^2) + eps)
    over the head; a gain of None leaves that side as it is; `heads` 0: there are no queries (q None); `value_dim` 0:
    there are no values (v, v_pool None).  q, k, v may be column slices of one tensor."""
    _cuda(q, k, v, positions, q_gain, k_gain, k_pool, v_pool, slot_mapping)
    _int32(positions, "positions")
    _int32(slot_mapping, "slot_mapping")
    tokens = k.shape[0]
    for name, t, width in (("q", q, heads * head_dim), ("k", k, kv_heads * head_dim), ("v", v, kv_heads * value_dim)):
        if t is None:
            if width:
                raise KernelError(f"norm_store: {name} is missing")
            continue
        _columns(t, name)
        if t.shape[1] != width or t.shape[0] != tokens or t.dtype != k.dtype:
            raise KernelError(f"norm_store: {name} is {tuple(t.shape)} {t.dtype}; [{tokens}, {width}] {k.dtype} is needed")
    for name, gain in (("q_gain", q_gain), ("k_gain", k_gain)):
        if gain is not None and (gain.dtype != torch.float32 or gain.numel() != head_dim or not gain.is_contiguous()):
            raise KernelError(f"norm_store: {name} must be contiguous float32 of {head_dim} elements")
    page_size = k_pool.shape[2]
    if tuple(k_pool.shape[1:]) != (kv_heads, page_size, head_dim) or not k_pool.is_contiguous() or k_pool.dtype != k.dtype:
        raise KernelError(f"norm_store: the key pool must be contiguous [pages, {kv_heads}, page_size, {head_dim}] of {k.dtype}")
    if value_dim and (tuple(v_pool.shape[1:]) != (kv_heads, page_size, value_dim) or not v_pool.is_contiguous()
                      or v_pool.dtype != k.dtype):
        raise KernelError(f"norm_store: the value pool must be contiguous [pages, {kv_heads}, page_size, {value_dim}] of {k.dtype}")
    lib = gated_attention_library()
    _run(lib, lib.mb_norm_store(_p(q), q.stride(0) if q is not None else 0, _p(k), k.stride(0), _p(v),
                                v.stride(0) if v is not None else 0, _code(k.dtype), _p(positions), _p(q_gain), _p(k_gain),
                                ctypes.c_float(eps), ctypes.c_float(temperature_coef), int(temperature_every), _p(k_pool),
                                _p(v_pool) if value_dim else None, _p(slot_mapping), tokens, heads, kv_heads, head_dim, value_dim,
                                page_size, _stream()))


def rotate_norm_store(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, positions: torch.Tensor, cos: Optional[torch.Tensor],
                      sin: Optional[torch.Tensor], rotary_dim: int, interleaved: bool, unit_norm: bool, eps: float,
                      value_cos: Optional[torch.Tensor], value_sin: Optional[torch.Tensor], value_rotary_dim: int,
                      k_pool: torch.Tensor, v_pool: torch.Tensor, slot_mapping: torch.Tensor, heads: int, kv_heads: int,
                      head_dim: int, value_dim: int) -> None:
    """Per head: q (in place) and k (into the key pool at `slot_mapping`) are rotated by the token's position over their
    first `rotary_dim` coordinates (float32 tables [positions, rotary_dim / 2]; pairs (i, i + rotary_dim / 2), or
    (2i, 2i + 1) when `interleaved`) and then, with `unit_norm`, divided by sqrt(mean(x^2) + eps) over the head; v is rotated
    over its first `value_rotary_dim` coordinates by tables of its own and stored in the value pool.  q, k, v may be column
    slices of one tensor.  Heads of up to 256 coordinates."""
    _cuda(q, k, v, positions, cos, sin, value_cos, value_sin, k_pool, v_pool, slot_mapping)
    _int32(positions, "positions")
    _int32(slot_mapping, "slot_mapping")
    tokens = k.shape[0]
    for name, t, width in (("q", q, heads * head_dim), ("k", k, kv_heads * head_dim), ("v", v, kv_heads * value_dim)):
        _columns(t, name)
        if t.shape[1] != width or t.shape[0] != tokens or t.dtype != k.dtype:
            raise KernelError(f"rotate_norm_store: {name} is {tuple(t.shape)} {t.dtype}; [{tokens}, {width}] {k.dtype} is needed")
    for name, dim, tables in (("rotary_dim", rotary_dim, (cos, sin)), ("value_rotary_dim", value_rotary_dim, (value_cos, value_sin))):
        if dim:
            for table in tables:
                if table is None or table.dtype != torch.float32 or table.dim() != 2 or table.shape[1] * 2 != dim or not table.is_contiguous():
                    raise KernelError(f"rotate_norm_store: {name} {dim} needs contiguous float32 tables [positions, {dim // 2}]")
    page_size = k_pool.shape[2]
    if tuple(k_pool.shape[1:]) != (kv_heads, page_size, head_dim) or not k_pool.is_contiguous() or k_pool.dtype != k.dtype:
        raise KernelError(f"rotate_norm_store: the key pool must be contiguous [pages, {kv_heads}, page_size, {head_dim}] of {k.dtype}")
    if tuple(v_pool.shape[1:]) != (kv_heads, page_size, value_dim) or not v_pool.is_contiguous() or v_pool.dtype != k.dtype:
        raise KernelError(f"rotate_norm_store: the value pool must be contiguous [pages, {kv_heads}, page_size, {value_dim}] of {k.dtype}")
    lib = gated_attention_library()
    _run(lib, lib.mb_rotate_norm_store(_p(q), q.stride(0), _p(k), k.stride(0), _p(v), v.stride(0), _code(k.dtype), _p(positions),
                                       _p(cos) if rotary_dim else None, _p(sin) if rotary_dim else None, int(rotary_dim),
                                       1 if interleaved else 0, 1 if unit_norm else 0, ctypes.c_float(eps),
                                       _p(value_cos) if value_rotary_dim else None, _p(value_sin) if value_rotary_dim else None,
                                       int(value_rotary_dim), _p(k_pool), _p(v_pool), _p(slot_mapping), tokens, heads, kv_heads,
                                       head_dim, value_dim, page_size, _stream()))


def project_norm_rotate_store(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_bias: Optional[torch.Tensor],
                              k_bias: Optional[torch.Tensor], v_bias: Optional[torch.Tensor], q_gain: Optional[torch.Tensor],
                              k_gain: Optional[torch.Tensor], eps: float, positions: torch.Tensor, cos: Optional[torch.Tensor],
                              sin: Optional[torch.Tensor], rotary_dim: int, interleaved: bool, k_pool: torch.Tensor,
                              v_pool: torch.Tensor, slot_mapping: torch.Tensor, heads: int, kv_heads: int, head_dim: int,
                              value_dim: int) -> None:
    """Projections normalised as a whole: q <- (q + q_bias) / rms(q + q_bias) * q_gain over ALL heads of the row at once
    (rms(x) = sqrt(mean(x^2) + eps); a gain of None: no norm), the same for k; then every head's first `rotary_dim` coordinates
    are rotated by the token's position (float32 tables [positions, rotary_dim / 2]; pairs (i, i + rotary_dim / 2), or
    (2i, 2i + 1) when `interleaved`); q is rewritten in place, k goes into the key pool at `slot_mapping`, v + v_bias into the
    value pool.  q, k, v may be column slices of one tensor; biases and gains are float32."""
    _cuda(q, k, v, q_bias, k_bias, v_bias, q_gain, k_gain, positions, cos, sin, k_pool, v_pool, slot_mapping)
    _int32(positions, "positions")
    _int32(slot_mapping, "slot_mapping")
    tokens = k.shape[0]
    for name, t, width, extra in (("q", q, heads * head_dim, (q_bias, q_gain)), ("k", k, kv_heads * head_dim, (k_bias, k_gain)),
                                  ("v", v, kv_heads * value_dim, (v_bias,))):
        _columns(t, name)
        if t.shape[1] != width or t.shape[0] != tokens or t.dtype != k.dtype:
            raise KernelError(f"project_norm_rotate_store: {name} is {tuple(t.shape)} {t.dtype}; [{tokens}, {width}] {k.dtype} is needed")
        for vector in extra:
            if vector is not None and (vector.dtype != torch.float32 or vector.numel() != width or not vector.is_contiguous()):
                raise KernelError(f"project_norm_rotate_store: the bias and gain of {name} must be contiguous float32 of {width} elements")
    if rotary_dim:
        for table in (cos, sin):
            if table is None or table.dtype != torch.float32 or table.dim() != 2 or table.shape[1] * 2 != rotary_dim or not table.is_contiguous():
                raise KernelError(f"project_norm_rotate_store: rotary_dim {rotary_dim} needs contiguous float32 tables [positions, {rotary_dim // 2}]")
    page_size = k_pool.shape[2]
    if tuple(k_pool.shape[1:]) != (kv_heads, page_size, head_dim) or not k_pool.is_contiguous() or k_pool.dtype != k.dtype:
        raise KernelError(f"project_norm_rotate_store: the key pool must be contiguous [pages, {kv_heads}, page_size, {head_dim}] of {k.dtype}")
    if tuple(v_pool.shape[1:]) != (kv_heads, page_size, value_dim) or not v_pool.is_contiguous() or v_pool.dtype != k.dtype:
        raise KernelError(f"project_norm_rotate_store: the value pool must be contiguous [pages, {kv_heads}, page_size, {value_dim}] of {k.dtype}")
    lib = gated_attention_library()
    _run(lib, lib.mb_project_norm_rotate_store(
        _p(q), q.stride(0), _p(k), k.stride(0), _p(v), v.stride(0), _code(k.dtype), _p(q_bias), _p(k_bias), _p(v_bias), _p(q_gain),
        _p(k_gain), ctypes.c_float(eps), _p(positions), _p(cos) if rotary_dim else None, _p(sin) if rotary_dim else None,
        int(rotary_dim), 1 if interleaved else 0, _p(k_pool), _p(v_pool), _p(slot_mapping), tokens, heads, kv_heads, head_dim,
        value_dim, page_size, _stream()))


GATE_KINDS = {None: 0, "head": 1, "element": 2}


def gated_attention_tc_library(key_dim: int, value_dim: int, shared_rows: bool):
    """The tensor-core form, compiled for these key and value sizes at first use."""
    return load_library("mb_gated_attention_tc", ["gated_attention_tc.cu"],
                        {"MB_KEY_DIM": int(key_dim), "MB_VALUE_DIM": int(value_dim), "MB_SHARED_ROWS": 1 if shared_rows else 0})


GATED_TC_MIN_ROWS = 8  # steps that bring fewer tokens to every sequence go to the kernel with a warp per (token, head)


def gated_attention_tc_takes(q: torch.Tensor, out: torch.Tensor, k_pool: torch.Tensor, head_dim: int, value_dim: int,
                             max_q_len: int, gate: Optional[torch.Tensor], gate_kind: Optional[str] = "element") -> bool:
    """bfloat16, cache pages of 64, key and value sizes multiples of 16 up to 256, 16-byte query rows."""
    if q.dtype != torch.bfloat16 or max_q_len < GATED_TC_MIN_ROWS or k_pool.shape[2] != 64:
        return False
    if head_dim % 16 or value_dim % 16 or not 16 <= head_dim <= 256 or not 16 <= value_dim <= 256:
        return False
    if q.stride(0) % 8 or q.data_ptr() % 16 or out.stride(0) % 2 or out.data_ptr() % 4 or k_pool.data_ptr() % 16:
        return False
    return gate is None or gate_kind != "element" or (gate.stride(0) % 2 == 0 and gate.data_ptr() % 4 == 0)


def gated_decode_runs(sequences: int, heads: int, kv_heads: int, pages: int, multiprocessors: int = 148):
    """(runs, pages per run) for a decode step whose page tables are `pages` wide.  A block's four warps take a run's
    chunks of 32 keys in turn, and a warp's chunks cost it one wait for memory after another: runs of two pages (a chunk
    per warp) as long as that makes at most 64 runs and no more than eight blocks per multiprocessor, longer ones beyond."""
    group = heads // kv_heads
    blocks = sequences * kv_heads * (-(-group // (4 if group <= 4 else 8)))
    span = max(2 if pages > 1 else 1, -(-pages // 64))
    while span < pages and blocks * (-(-pages // span)) > 8 * multiprocessors:
        span *= 2
    span = min(span, pages)
    return -(-pages // span), span


def gated_attention(q: torch.Tensor, out: torch.Tensor, k_pool: torch.Tensor, v_pool: Optional[torch.Tensor],
                    block_table: torch.Tensor, cu_q: torch.Tensor, kv_lens: torch.Tensor, max_q_len: int, heads: int,
                    kv_heads: int, head_dim: int, value_dim: int, weights: str, scale: float, slope_exponent: float = 0.0,
                    head_bias: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                    gate_kind: Optional[str] = None, kernel: Optional[str] = None, head_scale: Optional[torch.Tensor] = None,
                    softcap: float = 0.0, sink: bool = False, turn_cos: Optional[torch.Tensor] = None,
                    turn_sin: Optional[torch.Tensor] = None, block: int = 0) -> None:
    """Causal attention over the paged cache with `weights` "softmax" or "sigmoid" (independent sigmoids of the scores,
    not normalised over keys); score = scale * q.k - 2^(-slope_exponent (h + 1) / heads) * (i - j) + head_bias[h]
    (slope_exponent 0: no distance term; head_bias None: 0).  `v_pool` None: the values are the first `value_dim`
    coordinates of the key rows.  gate_kind "head": out_h *= sigmoid(gate[:, h]); "element": out *= sigmoid(gate),
    gate [T, heads * value_dim].  q [T, heads * head_dim], out [T, heads * value_dim] and gate may be column slices.
    `head_scale` [heads] float32: score = scale * head_scale[h] * q.k ...; `softcap` c > 0: the score, after everything
    else, becomes c * tanh(score / c); `sink`: the softmax's denominator has one more term of score 0 without a value;
    `turn_cos`, `turn_sin` (float32 [positions, value_dim / 2]): the values were stored rotated by their own positions
    (pairs 2m, 2m + 1), and every head's sum is turned back by the query's position before any gate.
    `block` n > 0: query i sees key j <= i only if floor(i / n) = floor(j / n), blocks of n positions counted from the
    sequence's position 0.
    `kernel`: None picks the decode form for steps of one token per sequence (the keys cut into runs with a block each;
    the grid follows the page table's width, not the lengths, so that a captured step stays valid), the tensor-core form
    where it applies (bfloat16 steps of many tokens), else the form with a warp per (token, head); "decode", "tc" or
    "rows" asks for one of them."""
    if weights not in ("softmax", "sigmoid"):
        raise KernelError(f"gated_attention: weights must be 'softmax' or 'sigmoid', got {weights!r}")
    if kernel not in (None, "tc", "rows", "decode"):
        raise KernelError(f"gated_attention: unknown kernel {kernel!r}")
    if gate_kind not in GATE_KINDS or (gate_kind is None) != (gate is None):
        raise KernelError(f"gated_attention: gate kind {gate_kind!r} does not fit the gate given")
    _cuda(q, out, k_pool, v_pool, block_table, cu_q, kv_lens, head_bias, gate)
    _int32(block_table, "block_table")
    _int32(cu_q, "cu_q")
    _int32(kv_lens, "kv_lens")
    _columns(q, "q")
    _columns(out, "out")
    if q.shape[1] != heads * head_dim or out.shape[1] != heads * value_dim or q.shape[0] != out.shape[0]:
        raise KernelError(f"gated_attention: q {tuple(q.shape)} and out {tuple(out.shape)} do not fit {heads} heads of "
                          f"{head_dim} and {value_dim}")
    page_size = k_pool.shape[2]
    if tuple(k_pool.shape[1:]) != (kv_heads, page_size, head_dim) or not k_pool.is_contiguous():
        raise KernelError(f"gated_attention: the key pool must be contiguous [pages, {kv_heads}, page_size, {head_dim}]")
    values = k_pool if v_pool is None else v_pool
    if v_pool is not None and (tuple(v_pool.shape[1:]) != (kv_heads, page_size, value_dim) or not v_pool.is_contiguous()):
        raise KernelError(f"gated_attention: the value pool must be contiguous [pages, {kv_heads}, page_size, {value_dim}]")
    if v_pool is None and value_dim > head_dim:
        raise KernelError(f"gated_attention: values of {value_dim} cannot be read from key rows of {head_dim}")
    if not (q.dtype == out.dtype == k_pool.dtype == values.dtype):
        raise KernelError("gated_attention: q, out and the pools must share one dtype")
    if head_bias is not None and (head_bias.dtype != torch.float32 or head_bias.numel() != heads or not head_bias.is_contiguous()):
        raise KernelError(f"gated_attention: head_bias must be contiguous float32 of {heads} elements")
    if gate is not None:
        _columns(gate, "gate")
        if gate.dtype != q.dtype or tuple(gate.shape) != (q.shape[0], heads if gate_kind == "head" else heads * value_dim):
            raise KernelError(f"gated_attention: a gate of kind {gate_kind!r} cannot be {tuple(gate.shape)} {gate.dtype}")
    if head_scale is not None and (head_scale.dtype != torch.float32 or head_scale.numel() != heads or not head_scale.is_contiguous()):
        raise KernelError(f"gated_attention: head_scale must be contiguous float32 of {heads} elements")
    if (turn_cos is None) != (turn_sin is None):
        raise KernelError("gated_attention: turning the result back needs both tables")
    if turn_cos is not None:
        _cuda(turn_cos, turn_sin)
        for table in (turn_cos, turn_sin):
            if table.dtype != torch.float32 or table.dim() != 2 or table.shape[1] * 2 != value_dim or not table.is_contiguous():
                raise KernelError(f"gated_attention: the tables that turn the result back must be contiguous float32 [positions, {value_dim // 2}]")
    if sink and weights != "softmax":
        raise KernelError("gated_attention: a sink belongs to softmax weights")
    if block < 0:
        raise KernelError(f"gated_attention: a block of {block} positions")
    extras = (_p(head_scale), ctypes.c_float(softcap), 1 if sink else 0, _p(turn_cos), _p(turn_sin), int(block))
    softmax = 1 if weights == "softmax" else 0
    sequences = kv_lens.numel()
    gate_stride = gate.stride(0) if gate is not None else 0
    if kernel == "decode" or (kernel is None and max_q_len == 1):
        if max_q_len != 1:
            raise KernelError("the decode form takes one token per sequence")
        runs, span = gated_decode_runs(sequences, heads, kv_heads, block_table.shape[1], _sm_count(q.device))
        lib = gated_attention_library()
        lib.mb_gated_attention_decode_scratch_floats.restype = ctypes.c_size_t
        scratch = torch.empty((lib.mb_gated_attention_decode_scratch_floats(sequences, heads, value_dim, runs),), dtype=torch.float32,
                              device=q.device)
        _run(lib, lib.mb_gated_attention_decode(
            _p(q), q.stride(0), _p(out), out.stride(0), _code(q.dtype), _p(k_pool), _p(values), values.shape[3], _p(block_table),
            block_table.shape[1], _p(cu_q), _p(kv_lens), _p(head_bias), _p(gate), gate_stride, GATE_KINDS[gate_kind], sequences,
            heads, kv_heads, head_dim, value_dim, page_size, softmax, ctypes.c_float(scale), ctypes.c_float(slope_exponent), runs,
            span, _p(scratch), *extras, _stream()))
        _launches[0] += 1  # two kernels
        return
    if kernel == "tc" or (kernel is None and gated_attention_tc_takes(q, out, k_pool, head_dim, value_dim, max_q_len, gate, gate_kind)):
        if not gated_attention_tc_takes(q, out, k_pool, head_dim, value_dim, max(max_q_len, GATED_TC_MIN_ROWS), gate, gate_kind):
            raise KernelError("the tensor-core form takes bfloat16, pages of 64 and key and value sizes that are multiples of 16 up to 256")
        lib = gated_attention_tc_library(head_dim, value_dim, v_pool is None)
        _run(lib, lib.mb_gated_attention_tc(
            _p(q), q.stride(0), _p(out), out.stride(0), _p(k_pool), _p(values), _p(block_table), block_table.shape[1], _p(cu_q),
            _p(kv_lens), _p(head_bias), _p(gate), gate_stride, GATE_KINDS[gate_kind], sequences, max_q_len, heads, kv_heads,
            page_size, softmax, ctypes.c_float(scale), ctypes.c_float(slope_exponent), *extras, _stream()))
        return
    lib = gated_attention_library()
    _run(lib, lib.mb_gated_attention_rows(
        _p(q), q.stride(0), _p(out), out.stride(0), _code(q.dtype), _p(k_pool), _p(values), values.shape[3], _p(block_table),
        block_table.shape[1], _p(cu_q), _p(kv_lens), _p(head_bias), _p(gate), gate_stride, GATE_KINDS[gate_kind], sequences,
        max_q_len, heads, kv_heads, head_dim, value_dim, page_size, softmax, ctypes.c_float(scale), ctypes.c_float(slope_exponent),
        *extras, _stream()))


def head_linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, heads: int, gate: Optional[torch.Tensor] = None,
                tensor_cores: bool = True) -> None:
    """One small matrix per head: out[t, h, :] = weight[h] . x[t, h, :] for weight [heads, n_out, n_in], x [T, heads * n_in],
    out [T, heads * n_out] (column slices allowed); with `gate` [T, heads], out[t, h, :] *= sigmoid(gate[t, h]).
    bfloat16 steps of 16 tokens and more with sizes that are multiples of 16 run on the tensor cores unless
    `tensor_cores` is False."""
    _cuda(x, weight, out, gate)
    _columns(x, "x")
    _columns(out, "out")
    if weight.dim() != 3 or weight.shape[0] != heads or not weight.is_contiguous():
        raise KernelError(f"head_linear: weight must be contiguous [{heads}, n_out, n_in], got {tuple(weight.shape)}")
    n_out, n_in = weight.shape[1], weight.shape[2]
    if tuple(x.shape) != (out.shape[0], heads * n_in) or out.shape[1] != heads * n_out or not (x.dtype == weight.dtype == out.dtype):
        raise KernelError(f"head_linear: x {tuple(x.shape)} {x.dtype} and out {tuple(out.shape)} {out.dtype} do not fit "
                          f"{heads} matrices of {n_out} x {n_in} {weight.dtype}")
    if gate is not None:
        _columns(gate, "gate")
        if tuple(gate.shape) != (x.shape[0], heads) or gate.dtype != x.dtype:
            raise KernelError(f"head_linear: gate must be [{x.shape[0]}, {heads}] of x's dtype")
    lib = gated_attention_library()
    _run(lib, lib.mb_head_linear(_p(x), x.stride(0), _p(weight), _p(out), out.stride(0), _code(x.dtype), _p(gate),
                                 gate.stride(0) if gate is not None else 0, x.shape[0], heads, n_in, n_out,
                                 1 if tensor_cores else 0, _stream()))


RETENTION_RUN = 64  # tokens of a run when a long step's recurrence is walked in runs


def retention_library():
    return load_library("mb_retention", ["retention.cu"])


def retention_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, positions: torch.Tensor,
                   cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary_dim: int, decay: torch.Tensor,
                   key_scale: float, eps: float, state: torch.Tensor, slots: torch.Tensor, cu_q: torch.Tensor, heads: int,
                   head_dim: int, value_dim: int, out: Optional[torch.Tensor], out_scale: float = 1.0, max_q_len: int = 1,
                   run_length: Optional[int] = None, input_activation: Optional[str] = None,
                   raw_out: Optional[torch.Tensor] = None) -> None:
    """Retention over the new tokens of every sequence: q and k rotated over their first `rotary_dim` coordinates
    (split-half pairs, float32 tables by position), k times key_scale; S = decay_h S + k v^T from the sequence's row of
    `state` (float32 [slots, heads, head_dim, value_dim], updated in place); o = S^T q; out = out_scale * o / rms(o) *
    silu(g) per head, rms(o) = sqrt(mean(o^2) + eps).  q, k, v, g are column slices with one row stride.
    Of `positions` only each sequence's first entry is read: its new tokens stand at consecutive positions.
    `input_activation` (a name of the activation table): q, k and v pass it as they are read.  `raw_out` (float32
    [tokens, heads * value_dim], may be a column slice): out_scale * o is written there and nothing else (no norm, no gate;
    `g` and `out` may then be None) -- what follows is the caller's, for instance `group_norm_gate`.
    `max_q_len`: the most new tokens of any sequence.  Beyond `run_length` tokens (None: RETENTION_RUN once a step brings
    more than twice as many) the sequences are walked in runs of that many tokens at once, through scratch memory."""
    _cuda(q, k, v, g, positions, cos, sin, decay, state, slots, cu_q, out, raw_out)
    _int32(positions, "positions")
    _int32(slots, "slots")
    _int32(cu_q, "cu_q")
    tokens = q.shape[0]
    if raw_out is not None:
        _columns(raw_out, "raw_out")
        if raw_out.dtype != torch.float32 or tuple(raw_out.shape) != (tokens, heads * value_dim):
            raise KernelError(f"retention_scan: raw_out must be float32 [{tokens}, {heads * value_dim}]")
        g = v if g is None else g  # (not read)
    elif g is None or out is None:
        raise KernelError("retention_scan: without raw_out the gate rows and `out` are needed")
    for name, t, width in (("q", q, heads * head_dim), ("k", k, heads * head_dim), ("v", v, heads * value_dim),
                           ("g", g, heads * value_dim), ("out", out, heads * value_dim)):
        if t is None:
            continue
        _columns(t, name)
        if tuple(t.shape) != (tokens, width) or t.dtype != q.dtype:
            raise KernelError(f"retention_scan: {name} is {tuple(t.shape)} {t.dtype}; [{tokens}, {width}] {q.dtype} is needed")
    if not (q.stride(0) == k.stride(0) == v.stride(0) == g.stride(0)):
        raise KernelError("retention_scan: q, k, v and g must share one row stride")
    if state.dtype != torch.float32 or tuple(state.shape[1:]) != (heads, head_dim, value_dim) or not state.is_contiguous():
        raise KernelError(f"retention_scan: the state must be contiguous float32 [slots, {heads}, {head_dim}, {value_dim}]")
    if decay.dtype != torch.float32 or decay.numel() != heads or not decay.is_contiguous():
        raise KernelError(f"retention_scan: decay must be contiguous float32 of {heads} elements")
    if rotary_dim:
        if cos is None or sin is None or cos.dtype != torch.float32 or sin.dtype != torch.float32:
            raise KernelError("retention_scan: rotation needs float32 cos/sin tables")
        if cos.shape[-1] != rotary_dim // 2 or cos.shape != sin.shape or not cos.is_contiguous() or not sin.is_contiguous():
            raise KernelError(f"retention_scan: cos/sin tables must be contiguous [positions, {rotary_dim // 2}]")
    lib = retention_library()
    if run_length is None:
        run_length = RETENTION_RUN if max_q_len > 2 * RETENTION_RUN else 0
    sequences = cu_q.numel() - 1
    lib.mb_retention_scratch_floats.restype = ctypes.c_size_t
    floats = lib.mb_retention_scratch_floats(sequences, heads, head_dim, value_dim, max_q_len, run_length)
    scratch = torch.empty((floats,), dtype=torch.float32, device=q.device) if floats else None
    _run(lib, lib.mb_retention_scan(_p(q), _p(k), _p(v), _p(g), q.stride(0), _code(q.dtype), _p(positions), _p(cos), _p(sin),
                                    rotary_dim, _p(decay), ctypes.c_float(key_scale), ctypes.c_float(eps), _p(state), _p(slots),
                                    _p(cu_q), sequences, heads, head_dim, value_dim, _p(out), out.stride(0) if out is not None else 0,
                                    ctypes.c_float(out_scale), max_q_len, run_length, _p(scratch),
                                    activation_code(input_activation) if input_activation is not None else -1, _p(raw_out),
                                    raw_out.stride(0) if raw_out is not None else 0, _stream()))
    if floats:
        _launches[0] += 2  # three kernels


def group_norm_gate(raw: torch.Tensor, gain: torch.Tensor, gate: torch.Tensor, out: torch.Tensor, eps: float,
                    gate_activation: str = "sigmoid") -> None:
    """out = raw / sqrt(mean(raw^2) + eps) * gain * act(gate) over whole rows (all heads together): raw float32, gain
    float32 [width], gate and out of one storage type; all three may be column slices.  act: "sigmoid" or "silu"."""
    if gate_activation not in ("sigmoid", "silu"):
        raise KernelError(f"group_norm_gate: the gate's activation must be 'sigmoid' or 'silu', got {gate_activation!r}")
    _cuda(raw, gain, gate, out)
    for name, t in (("raw", raw), ("gate", gate), ("out", out)):
        _columns(t, name)
    rows, width = raw.shape
    if raw.dtype != torch.float32 or gate.shape != raw.shape or out.shape != raw.shape or gate.dtype != out.dtype:
        raise KernelError(f"group_norm_gate: raw {tuple(raw.shape)} {raw.dtype}, gate {tuple(gate.shape)} {gate.dtype}, out "
                          f"{tuple(out.shape)} {out.dtype} do not fit")
    if gain.dtype != torch.float32 or gain.numel() != width or not gain.is_contiguous():
        raise KernelError(f"group_norm_gate: gain must be contiguous float32 of {width} elements")
    lib = retention_library()
    _run(lib, lib.mb_group_norm_gate(_p(raw), raw.stride(0), _p(gain), _p(gate), gate.stride(0), _p(out), out.stride(0),
                                     _code(out.dtype), rows, width, ctypes.c_float(eps), 1 if gate_activation == "sigmoid" else 0,
                                     _stream()))


def gated_recurrence_library():
    return load_library("mb_gated_recurrence", ["gated_recurrence.cu"])


def mingru_scan(zin: torch.Tensor, xin: torch.Tensor, gin: torch.Tensor, z_bias: torch.Tensor, x_bias: torch.Tensor,
                state: torch.Tensor, slots: torch.Tensor, cu_q: torch.Tensor, max_q_len: int, out: torch.Tensor,
                out_scale: float = 1.0) -> None:
    """minGRU over the new tokens of every sequence: z = sigmoid(zin + z_bias), u = xin + x_bias, candidate
    u + 1/2 (u >= 0) or sigmoid(u); S = (1 - z) S + z candidate from the sequence's row of `state` (float32
    [slots, width], updated in place); out = out_scale * S * silu(gin).  zin, xin, gin are column slices
    with one row stride; arithmetic in float."""
    _cuda(zin, xin, gin, z_bias, x_bias, state, slots, cu_q, out)
    _int32(slots, "slots")
    _int32(cu_q, "cu_q")
    width = state.shape[1]
    for name, t in (("zin", zin), ("xin", xin), ("gin", gin), ("out", out)):
        _columns(t, name)
        if t.shape != zin.shape or t.shape[1] != width or t.dtype != zin.dtype:
            raise KernelError(f"mingru_scan: {name} is {tuple(t.shape)} {t.dtype}; [{zin.shape[0]}, {width}] {zin.dtype} is needed")
    if not (zin.stride(0) == xin.stride(0) == gin.stride(0)):
        raise KernelError("mingru_scan: zin, xin and gin must share one row stride")
    if state.dtype != torch.float32 or not state.is_contiguous():
        raise KernelError("mingru_scan: the state must be contiguous float32 [slots, width]")
    for name, t in (("z_bias", z_bias), ("x_bias", x_bias)):
        if t.dtype != torch.float32 or t.numel() != width or not t.is_contiguous():
            raise KernelError(f"mingru_scan: {name} must be contiguous float32 of {width} elements")
    lib = gated_recurrence_library()
    _run(lib, lib.mb_mingru_scan(_p(zin), _p(xin), _p(gin), zin.stride(0), _code(zin.dtype), _p(z_bias), _p(x_bias), _p(state),
                                 _p(slots), _p(cu_q), cu_q.numel() - 1, max_q_len, width, _p(out), out.stride(0),
                                 ctypes.c_float(out_scale), _stream()))


def gated_delta_library():
    return load_library("mb_gated_delta", ["gated_delta.cu"])


CONV_ACTIVATIONS = {None: 0, "silu": 1}


def _state_rows(state: torch.Tensor, offset: int, floats: int, name: str):
    """The address and the row stride of the part of a per-sequence state [slots, n] float32 that starts `offset` floats in."""
    if state.dtype != torch.float32 or state.dim() != 2 or not state.is_contiguous() or offset < 0 or offset + floats > state.shape[1]:
        raise KernelError(f"{name}: the state must be contiguous float32 [slots, n] with {floats} floats from {offset} on in every row")
    return ctypes.c_void_p(state.data_ptr() + 4 * offset), ctypes.c_size_t(state.shape[1])


def short_conv(x: torch.Tensor, weights: torch.Tensor, state: torch.Tensor, state_offset: int, slots: torch.Tensor, cu_q: torch.Tensor,
               max_q_len: int, in_bias: Optional[torch.Tensor] = None, out_bias: Optional[torch.Tensor] = None,
               activation: Optional[str] = None, store_tail: bool = False, split_per: int = 0):
    """A short causal convolution over time per channel: with x_t = x[t] (+ in_bias) and `weights` [channels, taps] whose last
    column meets the current token, out[t] = act(sum_i weights[:, taps - 1 - i] * x_(t - i) (+ out_bias)) as float32
    [tokens, channels].  The inputs before a step's first token come from the sequence's tail, [taps - 1, channels] float32 at
    `state_offset` floats into its row of `state` (zeros for a new sequence); with `store_tail` the new tail is stored by the
    same kernel (else the state is left as it is).  `split_per` n > 0: also returns the results as two bfloat16 numbers
    each (the rounding and the rest), block by block of n channels, [tokens, channels / n * 2 n] with a block's roundings before
    its rests: (out, split)."""
    _cuda(x, weights, state, slots, cu_q, in_bias, out_bias)
    _int32(slots, "slots")
    _int32(cu_q, "cu_q")
    _columns(x, "x")
    channels, taps = weights.shape
    if x.shape[1] != channels or weights.dtype != torch.float32 or not weights.is_contiguous():
        raise KernelError(f"short_conv: float32 weights [channels, taps] must fit rows of {x.shape[1]} channels, got {tuple(weights.shape)} {weights.dtype}")
    for name, t in (("in_bias", in_bias), ("out_bias", out_bias)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != channels or not t.is_contiguous()):
            raise KernelError(f"short_conv: {name} must be contiguous float32 of {channels} elements")
    if activation not in CONV_ACTIVATIONS:
        raise KernelError(f"short_conv: activation {activation!r} is not built (known: silu or none)")
    tail, stride = _state_rows(state, state_offset, (taps - 1) * channels, "short_conv")
    out = torch.empty((x.shape[0], channels), dtype=torch.float32, device=x.device)
    if split_per and (split_per < 0 or channels % split_per):
        raise KernelError(f"short_conv: {channels} channels are no whole blocks of {split_per}")
    split = torch.empty((x.shape[0], 2 * channels), dtype=torch.bfloat16, device=x.device) if split_per else None
    lib = gated_delta_library()
    _run(lib, lib.mb_short_conv(_p(x), x.stride(0), _code(x.dtype), _p(in_bias), _p(weights), _p(out_bias), CONV_ACTIVATIONS[activation],
                                _p(out), out.stride(0), tail, stride, _p(slots), _p(cu_q), cu_q.numel() - 1, max_q_len, channels, taps,
                                1 if store_tail else 0, _p(split), int(split_per), _stream()))
    return (out, split) if split_per else out


def gated_delta_scan(conv: torch.Tensor, q_at: int, k_at: int, v_at: int, a_in: torch.Tensor, b_in: torch.Tensor, gate_in: torch.Tensor,
                     decay: torch.Tensor, dt_bias: torch.Tensor, gain: torch.Tensor, unit_eps: float, eps: float, state: torch.Tensor,
                     state_offset: int, slots: torch.Tensor, cu_q: torch.Tensor, heads: int, kv_heads: int, dim: int, vdim: int,
                     out: torch.Tensor, out_scale: float = 1.0) -> None:
    """The gated delta rule over the new tokens of every sequence.  `conv` float32 [tokens, n] holds the convolved q (kv_heads
    heads of `dim` from column q_at), k (from k_at) and v (heads heads of `vdim` from v_at); q and k become unit vectors
    x / sqrt(sum x^2 + unit_eps), q times dim^-1/2 (in place: `conv` is changed); beta = sigmoid(b_in), g = exp(decay * softplus(a_in + dt_bias)) per head
    (decay = -exp(A_log)); per head, from the sequence's float32 state S [heads, dim, vdim] at `state_offset` floats into its
    row of `state` (updated in place): S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q; out = out_scale * o / rms(o)
    * gain * silu(gate_in), rms over the head (eps `eps`).  a_in, b_in [tokens, heads], gate_in and out [tokens, heads * vdim]
    are column slices; a_in, b_in and gate_in share one row stride."""
    _cuda(conv, a_in, b_in, gate_in, decay, dt_bias, gain, state, slots, cu_q, out)
    _int32(slots, "slots")
    _int32(cu_q, "cu_q")
    tokens = conv.shape[0]
    if conv.dtype != torch.float32 or conv.stride(1) != 1 or max(q_at, k_at) + kv_heads * dim > conv.shape[1] or v_at + heads * vdim > conv.shape[1]:
        raise KernelError(f"gated_delta_scan: the convolved rows {tuple(conv.shape)} {conv.dtype} do not hold the q, k and v parts")
    for name, t, width in (("a_in", a_in, heads), ("b_in", b_in, heads), ("gate_in", gate_in, heads * vdim), ("out", out, heads * vdim)):
        _columns(t, name)
        if tuple(t.shape) != (tokens, width) or t.dtype != out.dtype:
            raise KernelError(f"gated_delta_scan: {name} is {tuple(t.shape)} {t.dtype}; [{tokens}, {width}] {out.dtype} is needed")
    if not (a_in.stride(0) == b_in.stride(0) == gate_in.stride(0)):
        raise KernelError("gated_delta_scan: a_in, b_in and gate_in must share one row stride")
    for name, t, n in (("decay", decay, heads), ("dt_bias", dt_bias, heads), ("gain", gain, vdim)):
        if t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous():
            raise KernelError(f"gated_delta_scan: {name} must be contiguous float32 of {n} elements")
    rows, stride = _state_rows(state, state_offset, heads * dim * vdim, "gated_delta_scan")
    raw = torch.empty((tokens, heads * vdim), dtype=torch.float32, device=conv.device)  # the read-outs, between the walk and the norm
    lib = gated_delta_library()
    _run(lib, lib.mb_gated_delta_scan(_p(conv), conv.stride(0), _p(a_in), _p(b_in), _p(gate_in), a_in.stride(0), _code(out.dtype), _p(decay),
                                      _p(dt_bias), _p(gain), ctypes.c_float(unit_eps), ctypes.c_float(eps), rows, stride, _p(slots),
                                      _p(cu_q), cu_q.numel() - 1, tokens, _p(raw), _p(out), out.stride(0), ctypes.c_float(out_scale), heads,
                                      kv_heads, dim, vdim, q_at, k_at, v_at, _stream()))
    _launches[0] += 2  # three kernels: unit vectors, the walk, norm and gate


def rglru_scan(gates: torch.Tensor, per: int, u: torch.Tensor, y_in: torch.Tensor, r_bias: torch.Tensor, i_bias: torch.Tensor,
               y_bias: torch.Tensor, rate: torch.Tensor, state: torch.Tensor, state_offset: int, slots: torch.Tensor, cu_q: torch.Tensor,
               max_q_len: int, out: torch.Tensor, out_scale: float = 1.0) -> None:
    """The real-gated linear recurrent unit over the new tokens of every sequence: with r = sigmoid(r_sum + r_bias),
    i = sigmoid(i_sum + i_bias), a = exp(rate * r) (rate <= 0 per channel): S = a S + sqrt(1 - a^2) * i * u from the sequence's
    float32 state [width] at `state_offset` floats into its row of `state` (updated in place); out = out_scale * S *
    gelu_tanh(y_in + y_bias).  `gates` float32 [tokens, 2 * width] holds the sums block by block of `per` channels: the r sums
    of block 0, its i sums, the r sums of block 1, ...; u float32 [tokens, width]; y_in and out column slices."""
    _cuda(gates, u, y_in, r_bias, i_bias, y_bias, rate, state, slots, cu_q, out)
    _int32(slots, "slots")
    _int32(cu_q, "cu_q")
    tokens, width = u.shape
    if gates.dtype != torch.float32 or u.dtype != torch.float32 or gates.stride(1) != 1 or u.stride(1) != 1 or tuple(gates.shape) != (tokens, 2 * width):
        raise KernelError(f"rglru_scan: gates {tuple(gates.shape)} and u {tuple(u.shape)} must be float32 [tokens, 2 * width] and [tokens, width]")
    for name, t in (("y_in", y_in), ("out", out)):
        _columns(t, name)
        if tuple(t.shape) != (tokens, width) or t.dtype != out.dtype:
            raise KernelError(f"rglru_scan: {name} is {tuple(t.shape)} {t.dtype}; [{tokens}, {width}] {out.dtype} is needed")
    for name, t in (("r_bias", r_bias), ("i_bias", i_bias), ("y_bias", y_bias), ("rate", rate)):
        if t.dtype != torch.float32 or t.numel() != width or not t.is_contiguous():
            raise KernelError(f"rglru_scan: {name} must be contiguous float32 of {width} elements")
    rows, stride = _state_rows(state, state_offset, width, "rglru_scan")
    lib = gated_recurrence_library()
    _run(lib, lib.mb_rglru_scan(_p(gates), gates.stride(0), int(per), _p(u), u.stride(0), _p(y_in), y_in.stride(0), _code(out.dtype),
                                _p(r_bias), _p(i_bias), _p(y_bias), _p(rate), rows, stride, _p(slots), _p(cu_q), cu_q.numel() - 1,
                                max_q_len, width, _p(out), out.stride(0), ctypes.c_float(out_scale), _stream()))


def _check_paged(q, out, k_pool, v_pool, block_table, cu_q, kv_lens, kv_heads, head_dim):
    _cuda(q, out, k_pool, v_pool, block_table, cu_q, kv_lens)
    _int32(block_table, "block_table")
    _int32(cu_q, "cu_q")
    _int32(kv_lens, "kv_lens")
    if q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("q and out need unit column stride")
    if k_pool.dim() != 4 or k_pool.shape[1] != kv_heads or k_pool.shape[3] != head_dim or not k_pool.is_contiguous():
        raise KernelError(f"k_pool must be contiguous [pages, {kv_heads}, page_size, {head_dim}], got {tuple(k_pool.shape)}")
    if v_pool.shape != k_pool.shape or not v_pool.is_contiguous():
        raise KernelError("v_pool must match k_pool")
    if not (q.dtype == out.dtype == k_pool.dtype == v_pool.dtype == torch.bfloat16):
        raise KernelError("the tensor-core attention kernels take bfloat16 q, out and pools")


_decode_block_bytes = {}


LONG_KEYS = 1024  # up to so many cached positions the split depends on the batch size alone


def decode_span(max_kv_len: int) -> int:
    """The class of context lengths that share one split of the keys: 0 up to LONG_KEYS positions, else
    the next power of two.  A captured decode step is valid for one class."""
    if max_kv_len <= LONG_KEYS:
        return 0
    span = LONG_KEYS
    while span < max_kv_len:
        span *= 2
    return span


SHARED_MEMORY_PER_SM = 227 * 1024  # what a block of sm_100a can be given


def decode_splits(sequences: int, heads: int, kv_heads: int, head_dim: int = 64, keys: int = 0,
                  window: Optional[int] = None, multiprocessors: Optional[int] = None, page_size: int = 64) -> int:
    """How many blocks share one sequence's keys.

    Up to LONG_KEYS cached positions (`keys`; 0: unknown, taken as short): a power of two, at most 8
    (they form one thread-block cluster), with which all blocks of the call are resident at once -- a
    second, partly filled round of blocks costs more than longer blocks do (measured: 16 sequences of
    1,100 positions at head size 128 take 22 us with 2 splits, 29 with 4, 38 with 8).  The kernel runs
    with three page stages when there are four or more splits (or heads of 96 and more, or blocks so
    few that all of them fit the multiprocessors with three) and with two otherwise, and a block's shared
    memory follows from that; so does the count.  It depends on the
    batch size rounded up to a power of two only, so a batch padded to such a size is split like the
    unpadded one.

    Longer contexts: what counts is that enough blocks are in flight to keep memory busy, and a
    cluster's eight are too few for one or two sequences (one sequence of 32,768 positions, head size
    64: 58 us with 8 splits, 26 us with 32).  Up to four sequences the count is what makes one round of
    blocks (at most 400: they then run with the deep page ring, and a second, partly filled round costs
    more than it gives: 2 sequences of 32,768 positions take 29 us with 16 splits, 39 with 32; 4
    sequences 57 us with 8, 65 with 16).  Larger batches have blocks enough anyway; there the count is
    one block per 16 pages (64 pages for heads wider than 64, whose pages are twice as large) within
    2,048 blocks in all (8 sequences of 65,536 positions: 175 us with 32 splits, 184 with 16; 16
    sequences of 16,384: 94 us with 16, 100 with 8).  Always at most 64 and at least 4 pages each; above
    8 the partial results meet in scratch memory and a second kernel.  `keys` is rounded up to its class
    (decode_span), so the count is the same for every length of a class.  `multiprocessors`: those of
    the device the call runs on (None: the current device's)."""
    if multiprocessors is None:
        multiprocessors = _sm_count(torch.device("cuda", torch.cuda.current_device()))
    rounded = 1
    while rounded < sequences:
        rounded *= 2
    base = rounded * kv_heads * (-(-(heads // kv_heads) // 16))
    if head_dim not in _decode_block_bytes:
        lib = attention_tc(head_dim)
        lib.mb_decode_block_bytes.restype = ctypes.c_size_t
        _decode_block_bytes[head_dim] = {stages: int(lib.mb_decode_block_bytes(stages)) + 1024 for stages in (2, 3)}
        _decode_block_bytes[head_dim]["wide"] = int(lib.mb_decode_stages(1)) == 3  # three stages whatever the split

    def power_of_two_up_to(limit: int) -> int:
        splits = 1
        while splits * 2 <= limit:
            splits *= 2
        return splits

    def fitting(stages: int) -> int:
        resident = max(1, SHARED_MEMORY_PER_SM // _decode_block_bytes[head_dim][stages])
        return power_of_two_up_to(max(1, min(8, (resident * multiprocessors) // max(1, base))))

    with_three = fitting(3)
    short = with_three if _decode_block_bytes[head_dim]["wide"] or with_three >= 4 else min(2, fitting(2))
    # (eight blocks to a sequence only for a handful of sequences: with more, a block is left with a page or two, and the
    # cluster's meeting costs more than the shorter walk saves -- batch 8: 0.772 ms per step with four, 0.810 with eight)
    short = min(short, max(4, 256 // max(1, base)))
    span = decode_span(keys)
    if span == 0:
        return short
    visible = min(span, window) if window else span
    pages = -(-visible // page_size)
    by_length = pages // (16 if head_dim <= 64 else 64)
    one_round = power_of_two_up_to(max(1, 400 // base))
    want = one_round if one_round >= 8 else max(one_round, by_length)
    want = power_of_two_up_to(max(1, min(want, 64, 2048 // base, pages // 4)))
    return want if want > 8 else short


def decode_attention(q: torch.Tensor, out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                     block_table: torch.Tensor, cu_q: torch.Tensor, kv_lens: torch.Tensor, heads: int, kv_heads: int,
                     head_dim: int, window: Optional[int], scale: float, splits: int, use_scratch: bool = False) -> None:
    """One query token per sequence (row cu_q[s] of q) against its cached keys and values.  The keys
    of a sequence are split over `splits` blocks; 2, 4 or 8 of them combine inside a thread-block
    cluster, other counts (or use_scratch) through scratch memory and a second kernel."""
    _check_paged(q, out, k_pool, v_pool, block_table, cu_q, kv_lens, kv_heads, head_dim)
    sequences = kv_lens.numel()
    lib = attention_tc(head_dim)
    scratch = None
    if splits > 1 and (use_scratch or splits not in (2, 4, 8)):
        lib.mb_decode_scratch_floats.restype = ctypes.c_size_t
        scratch = torch.empty((lib.mb_decode_scratch_floats(sequences, heads, splits),), dtype=torch.float32, device=q.device)
    _run(lib, lib.mb_decode_attention(_p(q), q.stride(0), _p(out), out.stride(0), _p(k_pool), _p(v_pool),
                                      _p(block_table), block_table.shape[1], _p(cu_q), _p(kv_lens), sequences, heads,
                                      kv_heads, k_pool.shape[2], window or 0, ctypes.c_float(scale), splits,
                                      _p(scratch), _stream()))
    if scratch is not None:
        _launches[0] += 1  # the combine kernel


def prefill_attention(q: torch.Tensor, out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                      block_table: torch.Tensor, cu_q: torch.Tensor, kv_lens: torch.Tensor, max_q_len: int, heads: int,
                      kv_heads: int, head_dim: int, window: Optional[int], scale: float, kernel: Optional[str] = None) -> None:
    """Any number of new tokens per sequence; their keys and values are already in the cache.
    `kernel`: None picks the tcgen05 kernel where it applies, else the mma.sync one; "tcgen05" or
    "mma" asks for one of them."""
    _check_paged(q, out, k_pool, v_pool, block_table, cu_q, kv_lens, kv_heads, head_dim)
    if kernel not in (None, "tcgen05", "mma"):
        raise KernelError(f"prefill_attention: unknown kernel {kernel!r}")
    if kernel == "tcgen05" or (kernel is None and prefill_attention_tcgen05_takes(q, out, head_dim, max_q_len)):
        if head_dim not in (64, 128):
            raise KernelError(f"the tcgen05 prefill attention is built for head sizes 64 and 128, got {head_dim}")
        lib = prefill_attention_tc(head_dim)
        _run(lib, lib.mb_prefill_attention_tcgen05(
            _p(q), q.stride(0), q.shape[0], _p(out), out.stride(0), _p(k_pool), _p(v_pool), k_pool.shape[0],
            _p(block_table), block_table.shape[1], _p(cu_q), _p(kv_lens), kv_lens.numel(), max_q_len, heads, kv_heads,
            k_pool.shape[2], window or 0, ctypes.c_float(scale), _stream()))
        return
    lib = attention_tc(head_dim)
    _run(lib, lib.mb_prefill_attention(_p(q), q.stride(0), _p(out), out.stride(0), _p(k_pool), _p(v_pool),
                                       _p(block_table), block_table.shape[1], _p(cu_q), _p(kv_lens), kv_lens.numel(),
                                       max_q_len, heads, kv_heads, k_pool.shape[2], window or 0, ctypes.c_float(scale),
                                       _stream()))


# ------------------------------------------------------------------------------------ matrix products

def gemm_f32(a: torch.Tensor, w: torch.Tensor, row_invariant: bool = True) -> torch.Tensor:
    """a [m, k] . w[n, k]^T in true 32-bit arithmetic."""
    _cuda(a, w)
    if a.dtype != torch.float32 or w.dtype != torch.float32:
        raise KernelError(f"gemm_f32 takes float32 operands, got {a.dtype} and {w.dtype}")
    if a.dim() != 2 or w.dim() != 2 or a.shape[1] != w.shape[1] or a.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError(f"gemm_f32: shapes {tuple(a.shape)} x {tuple(w.shape)}^T do not fit")
    m, k = a.shape
    n = w.shape[0]
    c = torch.empty((m, n), dtype=torch.float32, device=a.device)
    lib = gemm32()
    _run(lib, lib.mb_gemm_f32(_p(a), a.stride(0), _p(w), w.stride(0), _p(c), n, m, n, k, 1 if row_invariant else 0,
                              _stream()))
    return c


SKINNY_ROWS, SKINNY_NORM_ROWS = 32, 16
EPI_BF16, EPI_F32, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2, 3


def skinny():
    return load_library("mb_skinny_gemm", ["skinny_gemm.cu"])


def skinny_takes(weight: torch.Tensor, rows: int, with_norm: bool = False) -> bool:
    """Whether the decode matrix product takes this weight with this many activation rows."""
    return (weight.dtype == torch.bfloat16 and weight.dim() == 2 and weight.stride(1) == 1 and weight.shape[1] % 8 == 0
            and weight.stride(0) % 8 == 0 and weight.data_ptr() % 16 == 0
            and 0 < rows <= (SKINNY_NORM_ROWS if with_norm else SKINNY_ROWS))


SKINNY_PAYS_ROWS = 8  # one 8-column MMA tile of activations: beyond it a block's activations crowd out its weight rings


def skinny_pays(weight: torch.Tensor, rows: int, with_norm: bool = False) -> bool:
    """Whether the decode matrix product is the one to use: it takes up to 32 rows, but with more than 8
    its blocks hold twice the activations in shared memory, half as many of them fit a multiprocessor,
    and a library product streams the weights faster (measured at 16 and 32 rows on every layer shape
    of the 1B, 3B and 8B models)."""
    return rows <= SKINNY_PAYS_ROWS and skinny_takes(weight, rows, with_norm)


_multiprocessors = {}


def _sm_count(device) -> int:
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _multiprocessors:
        _multiprocessors[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _multiprocessors[index]


def multiprocessors(device) -> int:
    """Multiprocessors of a CUDA device (asked of the driver once)."""
    return _sm_count(torch.device(device))


def skinny_gemm(weight: torch.Tensor, epilogue: int, x: Optional[torch.Tensor] = None, xf: Optional[torch.Tensor] = None,
                gain: Optional[torch.Tensor] = None, eps: float = 0.0, rows: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None, norm_parts=None, emit_gain: Optional[torch.Tensor] = None):
    """Few activation rows times weight^T ([n, k] bfloat16).  Activations: `x` (bfloat16 [rows, k]), or
    `xf` (the float32 residual rows, optionally gathered by `rows`) normalised on the fly with `gain`
    and `eps`.  Epilogues: EPI_BF16 / EPI_F32 store [rows, n]; EPI_RESIDUAL adds into `out` (float32
    [rows, n]); EPI_SWIGLU takes weight = [gate rows; up rows] and stores act(gate) * up [rows, n/2].
    `norm_parts` and `emit_gain` as for wide_gemm: `x` is then the rows times a norm's gain, divided by their
    root mean square in the epilogue; a residual product can prepare the next norm's rows the same way."""
    _cuda(weight, x, xf, gain, rows, out, emit_gain)
    n, k = weight.shape
    norm = gain is not None
    if norm:
        if xf is None or xf.dtype != torch.float32 or xf.stride(1) != 1 or xf.shape[1] != k:
            raise KernelError("the norm prologue needs float32 rows of the weight's width")
        if gain.dtype != torch.float32 or gain.numel() != k:
            raise KernelError("the norm gain must be float32 of the weight's width")
        _int32(rows, "rows")
        batch = rows.numel() if rows is not None else xf.shape[0]
    else:
        if x is None or x.dtype != torch.bfloat16 or x.stride(1) != 1 or x.shape[1] != k:
            raise KernelError("activations must be bfloat16 rows of the weight's width")
        batch = x.shape[0]
    if not skinny_takes(weight, batch, norm):
        raise KernelError(f"skinny_gemm does not take a {tuple(weight.shape)} {weight.dtype} weight with {batch} rows")
    kind = epilogue & 0xFF  # a gated epilogue carries its activation above
    out_cols = n // 2 if kind == EPI_SWIGLU else n
    if kind == EPI_RESIDUAL:
        if out is None or out.dtype != torch.float32 or out.shape != (batch, n) or out.stride(1) != 1:
            raise KernelError("the residual epilogue adds into a float32 [rows, n] tensor")
    elif out is None:
        out = torch.empty((batch, out_cols), dtype=torch.float32 if kind == EPI_F32 else torch.bfloat16,
                          device=weight.device)
    if norm and norm_parts is not None:
        raise KernelError("a product normalises float32 rows itself or takes rows with parts of their sums of squares, not both")
    ssq, count, _, _, part_eps = _norm_args(norm_parts, batch, SSQ_COLUMNS)
    if norm_parts is not None and norm_parts[2] != k:
        raise KernelError("the norm's width is the product's k")
    emit_rows = emit_ssq = None
    written = ctypes.c_int(0)
    if emit_gain is not None:
        if kind != EPI_RESIDUAL or emit_gain.dtype != torch.float32 or emit_gain.numel() != n:
            raise KernelError("the next norm's rows come from the residual epilogue, with a float32 gain of the output's width")
        emit_rows = torch.empty((batch, n), dtype=torch.bfloat16, device=weight.device)
        emit_ssq = torch.empty((-(-n // 16), SSQ_COLUMNS), dtype=torch.float32, device=weight.device)
    lib = skinny()
    _run(lib, lib.mb_skinny_gemm(_p(weight), weight.stride(0), n, k, batch, _p(x), x.stride(0) if x is not None else 0,
                                 _p(xf), xf.stride(0) if xf is not None else 0, _p(gain),
                                 part_eps if norm_parts is not None else ctypes.c_float(eps), _p(rows),
                                 _p(out), out.stride(0), epilogue, _sm_count(weight.device), 1, ssq, count, _p(emit_gain),
                                 _p(emit_rows), emit_rows.stride(0) if emit_rows is not None else 0, _p(emit_ssq),
                                 ctypes.byref(written), _stream()))
    if emit_gain is not None:
        return out, emit_rows, emit_ssq, written.value
    return out


def skinny_gemm_gated_residual(weight: torch.Tensor, x: torch.Tensor, out: torch.Tensor, gate: torch.Tensor, bias: torch.Tensor) -> None:
    """out += sigmoid(gate + bias) * (x . weight^T) for few rows: the residual epilogue of the decode product with a
    gate on what it adds.  x bfloat16 [rows, k], weight bfloat16 [n, k], out the float32 stream [rows, n], gate bfloat16
    [rows, n] (a column slice is fine), bias float32 [n]."""
    _cuda(weight, x, out, gate, bias)
    n, k = weight.shape
    batch = x.shape[0]
    if x.dtype != torch.bfloat16 or x.stride(1) != 1 or x.shape[1] != k or not skinny_takes(weight, batch):
        raise KernelError(f"skinny_gemm_gated_residual does not take a {tuple(weight.shape)} weight with {tuple(x.shape)} {x.dtype} rows")
    if out.dtype != torch.float32 or tuple(out.shape) != (batch, n) or out.stride(1) != 1:
        raise KernelError("the residual epilogue adds into a float32 [rows, n] tensor")
    _columns(gate, "gate")
    if gate.dtype != torch.bfloat16 or tuple(gate.shape) != (batch, n) or bias.dtype != torch.float32 or bias.numel() != n \
            or not bias.is_contiguous():
        raise KernelError("the gate must be bfloat16 [rows, n] and its bias float32 [n]")
    lib = skinny()
    _run(lib, lib.mb_skinny_gemm_gated_residual(_p(weight), weight.stride(0), n, k, batch, _p(x), x.stride(0), _p(out), out.stride(0),
                                                _p(gate), gate.stride(0), _p(bias), _sm_count(weight.device), 1, _stream()))


def skinny_qkv_rope(weight: torch.Tensor, xf: Optional[torch.Tensor], gain: Optional[torch.Tensor], eps: float, heads: int,
                    kv_heads: int, head_dim: int, positions: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                    k_pool: torch.Tensor, v_pool: torch.Tensor, slot_mapping: torch.Tensor, x: Optional[torch.Tensor] = None,
                    norm_parts=None) -> torch.Tensor:
    """The q/k/v product of an attention layer on few rows with everything around it folded in: RMSNorm
    of the float32 residual rows `xf` before it, rotation of queries and keys (split-half pairs over
    the whole head) and the paged cache write of keys and values after it.  Returns the rotated
    queries, bfloat16 [rows, heads * head_dim].  In place of `xf` and `gain`: `x`, the rows times the gain as
    bfloat16, with `norm_parts` (as for wide_gemm); the division by the root mean square then happens in the epilogue."""
    _cuda(weight, xf, x, gain, positions, cos, sin, k_pool, v_pool, slot_mapping)
    if (xf is None) == (x is None) or (x is not None and norm_parts is None):
        raise KernelError("skinny_qkv_rope takes float32 rows with a gain, or gained bfloat16 rows with parts of their sums of squares")
    batch, k = (xf if xf is not None else x).shape
    if weight.shape != ((heads + 2 * kv_heads) * head_dim, k) or not skinny_takes(weight, batch, True):
        raise KernelError(f"skinny_qkv_rope does not take a {tuple(weight.shape)} {weight.dtype} weight with {batch} rows")
    if xf is not None and (xf.dtype != torch.float32 or xf.stride(1) != 1 or gain.dtype != torch.float32 or gain.numel() != k):
        raise KernelError("skinny_qkv_rope needs float32 residual rows and gain")
    if x is not None and (x.dtype != torch.bfloat16 or x.stride(1) != 1 or x.stride(0) % 8 or x.data_ptr() % 16 or norm_parts[2] != k):
        raise KernelError("skinny_qkv_rope needs aligned bfloat16 rows of the weight's width")
    _int32(positions, "positions")
    _int32(slot_mapping, "slot_mapping")
    if cos.dtype != torch.float32 or cos.shape[-1] != head_dim // 2 or cos.shape != sin.shape or not cos.is_contiguous():
        raise KernelError(f"cos/sin tables must be contiguous float32 [positions, {head_dim // 2}]")
    if k_pool.dtype != torch.bfloat16 or k_pool.shape != v_pool.shape or k_pool.shape[1] != kv_heads or k_pool.shape[3] != head_dim:
        raise KernelError("cache pools must be bfloat16 [pages, kv_heads, page_size, head_dim]")
    q = torch.empty((batch, heads * head_dim), dtype=torch.bfloat16, device=weight.device)
    ssq, count, _, _, part_eps = _norm_args(norm_parts, batch, SSQ_COLUMNS)
    lib = skinny()
    _run(lib, lib.mb_skinny_qkv_rope(_p(weight), weight.stride(0), k, batch, _p(x), x.stride(0) if x is not None else 0, _p(xf),
                                     xf.stride(0) if xf is not None else 0, _p(gain),
                                     part_eps if norm_parts is not None else ctypes.c_float(eps), _p(q), q.stride(0), heads,
                                     kv_heads, head_dim, _p(positions), _p(cos), _p(sin), _p(k_pool), _p(v_pool),
                                     _p(slot_mapping), k_pool.shape[2], _sm_count(weight.device), 1, ssq, count, _stream()))
    return q


def gemm_tc():
    return load_library("mb_gemm_tcgen05", ["gemm_tcgen05.cu"])


TCGEN05_MIN_ROWS = 9  # fewer rows take the narrow decode product
WIDE_ROWS = 128  # most activation rows of the wide decode product


def gemm_tcgen05_takes(weight: torch.Tensor, epilogue: int = EPI_BF16, rows: Optional[int] = None) -> bool:
    """Whether a tcgen05 matrix product takes this weight and, if `rows` is given, is the one to use for
    so many rows: above 128 the prefill form; from 9 to 128 the wide decode form (fewer rows take the
    narrow decode product)."""
    epilogue &= 0xFF
    n = weight.shape[0] // 2 if epilogue == EPI_SWIGLU else weight.shape[0]
    if rows is not None and rows < TCGEN05_MIN_ROWS:
        return False
    return (weight.dtype == torch.bfloat16 and weight.dim() == 2 and weight.stride(1) == 1 and weight.shape[1] % 8 == 0
            and weight.stride(0) % 8 == 0 and weight.data_ptr() % 16 == 0 and n % 8 == 0
            and (epilogue != EPI_SWIGLU or weight.shape[0] % 2 == 0))


_split_tickets = {}


def gemm_tcgen05(a: torch.Tensor, weight: torch.Tensor, epilogue: int = EPI_BF16, out: Optional[torch.Tensor] = None,
                 tile_width: int = 0, pair: int = 0, arrival_order: bool = False) -> torch.Tensor:
    """a [m, k] . weight[n, k]^T on the tcgen05 tensor cores (bfloat16 in, float accumulation).
    Epilogues as for skinny_gemm: EPI_BF16 / EPI_F32 store, EPI_RESIDUAL adds into `out` (float32
    [m, n]), EPI_SWIGLU stores act(gate) * up for weight = [gate rows; up rows].  tile_width 0 lets
    the launcher choose between tiles of 128 and 256 output columns.  pair 2: tiles of 256 rows by
    256 columns on pairs of blocks (tcgen05 cta_group::2).  Where the residual epilogue splits K over
    blocks (few tiles, a long K) the parts are summed in their order through scratch memory, so a
    result is the same bits in every run; `arrival_order` lets each part add into `out` as it finishes
    instead (a little quicker, the last bit of an element then depends on timing)."""
    _cuda(a, weight, out)
    if a.dtype != torch.bfloat16 or a.dim() != 2 or a.stride(1) != 1 or a.shape[1] != weight.shape[1]:
        raise KernelError(f"gemm_tcgen05: activations {tuple(a.shape)} {a.dtype} do not fit the weight {tuple(weight.shape)}")
    if not gemm_tcgen05_takes(weight, epilogue) or a.stride(0) % 8 or a.data_ptr() % 16:
        raise KernelError(f"gemm_tcgen05 does not take a {tuple(weight.shape)} {weight.dtype} weight")
    m, k = a.shape
    n_w = weight.shape[0]
    kind = epilogue & 0xFF
    n = n_w // 2 if kind == EPI_SWIGLU else n_w
    if kind == EPI_RESIDUAL:
        if out is None or out.dtype != torch.float32 or out.shape != (m, n) or out.stride(1) != 1:
            raise KernelError("the residual epilogue adds into a float32 [m, n] tensor")
    elif out is None:
        out = torch.empty((m, n), dtype=torch.float32 if kind == EPI_F32 else torch.bfloat16, device=a.device)
    lib = gemm_tc()
    sms = _sm_count(a.device)
    partial = tickets = None
    if kind == EPI_RESIDUAL and not arrival_order:
        need_partial, need_tickets = ctypes.c_size_t(0), ctypes.c_size_t(0)
        lib.mb_gemm_tcgen05_scratch(sms, ctypes.byref(need_partial), ctypes.byref(need_tickets))
        partial = torch.empty((need_partial.value,), dtype=torch.float32, device=a.device)  # touched only where K is split
        key = a.device.index if a.device.index is not None else torch.cuda.current_device()
        tickets = _split_tickets.get(key)
        if tickets is None:
            # zero once; every launch leaves the tickets at zero
            tickets = _split_tickets[key] = torch.zeros((need_tickets.value,), dtype=torch.int32, device=a.device)
    _run(lib, lib.mb_gemm_tcgen05(_p(a), a.stride(0), _p(weight), weight.stride(0), _p(out), out.stride(0), m, n_w, k,
                                  epilogue, sms, tile_width, pair, _p(partial), _p(tickets), _stream()))
    return out


def gemm_tcgen05_qkv_rope_takes(weight: torch.Tensor, rows: int, heads: int, kv_heads: int, head_dim: int) -> bool:
    """Whether the prefill q/k/v product with folded rotation and cache write applies: a weight the
    tcgen05 product takes for so many rows, heads of 64 or 128."""
    return (head_dim in (64, 128) and weight.shape[0] == (heads + 2 * kv_heads) * head_dim and rows > WIDE_ROWS
            and gemm_tcgen05_takes(weight, EPI_BF16, rows))


def gemm_tcgen05_qkv_rope(a: torch.Tensor, weight: torch.Tensor, heads: int, kv_heads: int, head_dim: int,
                          positions: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, k_pool: torch.Tensor,
                          v_pool: torch.Tensor, slot_mapping: torch.Tensor) -> torch.Tensor:
    """The q/k/v product of an attention layer over a whole prompt with what follows it folded into
    its epilogue: rotation of queries and keys (split-half pairs over the whole head) and the paged
    cache write of keys and values.  Returns the rotated queries, bfloat16 [rows, heads * head_dim]."""
    _cuda(a, weight, positions, cos, sin, k_pool, v_pool, slot_mapping)
    m, k = a.shape
    if a.dtype != torch.bfloat16 or a.stride(1) != 1 or a.stride(0) % 8 or a.data_ptr() % 16 or weight.shape[1] != k:
        raise KernelError(f"gemm_tcgen05_qkv_rope: activations {tuple(a.shape)} {a.dtype} do not fit the weight {tuple(weight.shape)}")
    if not gemm_tcgen05_qkv_rope_takes(weight, m, heads, kv_heads, head_dim):
        raise KernelError(f"gemm_tcgen05_qkv_rope does not take a {tuple(weight.shape)} {weight.dtype} weight with {m} rows "
                          f"and heads of {head_dim}")
    _int32(positions, "positions")
    _int32(slot_mapping, "slot_mapping")
    if positions.numel() < m or slot_mapping.numel() < m:
        raise KernelError("positions and slot_mapping must hold one entry per row")
    if cos.dtype != torch.float32 or cos.shape[-1] != head_dim // 2 or cos.shape != sin.shape or not cos.is_contiguous():
        raise KernelError(f"cos/sin tables must be contiguous float32 [positions, {head_dim // 2}]")
    if (k_pool.dtype != torch.bfloat16 or k_pool.shape != v_pool.shape or k_pool.dim() != 4 or k_pool.shape[1] != kv_heads
            or k_pool.shape[3] != head_dim or not k_pool.is_contiguous() or not v_pool.is_contiguous()):
        raise KernelError("cache pools must be contiguous bfloat16 [pages, kv_heads, page_size, head_dim]")
    q = torch.empty((m, heads * head_dim), dtype=torch.bfloat16, device=a.device)
    lib = gemm_tc()
    _run(lib, lib.mb_gemm_tcgen05_qkv_rope(_p(a), a.stride(0), _p(weight), weight.stride(0), _p(q), q.stride(0), m, k, heads,
                                           kv_heads, head_dim, _p(positions), _p(cos), _p(sin), _p(k_pool), _p(v_pool),
                                           _p(slot_mapping), k_pool.shape[2], _sm_count(a.device), _stream()))
    return q


def wide_gemm_lib():
    return load_library("mb_wide_gemm_tcgen05", ["wide_gemm_tcgen05.cu"])


SSQ_COLUMNS = 128  # columns of a table of parts of sums of squares: one per activation row


def _norm_args(norm_parts, rows: int, columns: Optional[int] = None):
    """(ssq_parts, count, row stride, width, eps) of a product whose activations still lack the division by the
    root mean square, as the C launchers take them.  The table is [parts, columns] float32 with a column per
    activation row (`columns` given: exactly so many)."""
    if norm_parts is None:
        return None, 0, 0, 0, ctypes.c_float(0.0)
    ssq, count, width, eps = norm_parts
    if (ssq.dtype != torch.float32 or ssq.dim() != 2 or ssq.stride(1) != 1 or ssq.shape[1] < rows or ssq.shape[0] < count or count <= 0
            or (columns is not None and (ssq.shape[1] != columns or ssq.stride(0) != columns))):
        raise KernelError(f"parts of sums of squares must be a float32 [parts, {columns or 'rows'}] table with a column per row")
    return _p(ssq), int(count), ssq.stride(0), int(width), ctypes.c_float(eps)


def wide_gemm(x: torch.Tensor, weight: torch.Tensor, epilogue: int = EPI_BF16, out: Optional[torch.Tensor] = None,
              norm_parts=None, emit_gain: Optional[torch.Tensor] = None):
    """Up to 128 activation rows times weight^T on the tcgen05 tensor cores with the weights as the
    128-row operand (decode at wide batches); K is split over the blocks of a cluster where a matrix has
    few row tiles, their sums meeting in distributed shared memory in a fixed order.  Epilogues as for
    skinny_gemm.

    The RMSNorm before a product can ride in it: `x` is then the rows times the norm's gain, and
    `norm_parts` = (parts of the rows' sums of squares [parts, 128], how many parts, the rows' width, eps);
    the results are scaled by 1 / rms.  The residual epilogue can prepare the NEXT norm the same way: with
    `emit_gain` (that norm's gain) it returns (out, rows of the new `out` times the gain as bfloat16, parts of
    their sums of squares, how many parts)."""
    _cuda(x, weight, out, emit_gain)
    if x.dtype != torch.bfloat16 or x.dim() != 2 or x.stride(1) != 1 or x.shape[1] != weight.shape[1] or x.shape[0] > WIDE_ROWS:
        raise KernelError(f"wide_gemm: activations {tuple(x.shape)} {x.dtype} do not fit the weight {tuple(weight.shape)}")
    if not gemm_tcgen05_takes(weight, epilogue) or x.stride(0) % 8 or x.data_ptr() % 16:
        raise KernelError(f"wide_gemm does not take a {tuple(weight.shape)} {weight.dtype} weight")
    batch, k = x.shape
    n_w = weight.shape[0]
    kind = epilogue & 0xFF
    n = n_w // 2 if kind == EPI_SWIGLU else n_w
    if kind == EPI_RESIDUAL:
        if out is None or out.dtype != torch.float32 or out.shape != (batch, n) or out.stride(1) != 1:
            raise KernelError("the residual epilogue adds into a float32 [rows, n] tensor")
    elif out is None:
        out = torch.empty((batch, n), dtype=torch.float32 if kind == EPI_F32 else torch.bfloat16, device=x.device)
    emit_rows = emit_ssq = None
    written = ctypes.c_int(0)
    if emit_gain is not None:
        if kind != EPI_RESIDUAL or emit_gain.dtype != torch.float32 or emit_gain.numel() != n:
            raise KernelError("the next norm's rows come from the residual epilogue, with a float32 gain of the output's width")
        emit_rows = torch.empty((batch, n), dtype=torch.bfloat16, device=x.device)
        emit_ssq = torch.empty((8 * -(-n // 128), SSQ_COLUMNS), dtype=torch.float32, device=x.device)
    ssq, count, _, width, eps = _norm_args(norm_parts, batch, SSQ_COLUMNS)
    lib = wide_gemm_lib()
    _run(lib, lib.mb_wide_gemm(_p(x), x.stride(0), _p(weight), weight.stride(0), _p(out), out.stride(0), batch, n_w, k,
                               epilogue, _sm_count(x.device), ssq, count, width, eps, _p(emit_gain), _p(emit_rows),
                               emit_rows.stride(0) if emit_rows is not None else 0, _p(emit_ssq), ctypes.byref(written), _stream()))
    if emit_gain is not None:
        return out, emit_rows, emit_ssq, written.value
    return out


def wide_qkv_rope_takes(weight: torch.Tensor, rows: int, heads: int, kv_heads: int, head_dim: int) -> bool:
    """Whether the wide q/k/v product with folded rotation and cache write applies: a bfloat16 weight the
    tcgen05 products take, 9 to 128 rows, a head size that divides 128."""
    return (head_dim >= 16 and 128 % head_dim == 0 and weight.shape[0] == (heads + 2 * kv_heads) * head_dim
            and SKINNY_PAYS_ROWS < rows <= WIDE_ROWS and gemm_tcgen05_takes(weight, EPI_BF16))


def wide_qkv_rope(x: torch.Tensor, weight: torch.Tensor, heads: int, kv_heads: int, head_dim: int, positions: torch.Tensor,
                  cos: torch.Tensor, sin: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                  slot_mapping: torch.Tensor, norm_parts=None) -> torch.Tensor:
    """The q/k/v product of an attention layer on 9 to 128 rows with what follows it folded in: rotation of
    queries and keys (split-half pairs over the whole head) and the paged cache write of keys and values.
    Returns the rotated queries, bfloat16 [rows, heads * head_dim].  `norm_parts` as for wide_gemm."""
    _cuda(x, weight, positions, cos, sin, k_pool, v_pool, slot_mapping)
    batch, k = x.shape
    if x.dtype != torch.bfloat16 or x.stride(1) != 1 or x.stride(0) % 8 or x.data_ptr() % 16 or weight.shape[1] != k:
        raise KernelError(f"wide_qkv_rope: activations {tuple(x.shape)} {x.dtype} do not fit the weight {tuple(weight.shape)}")
    if not wide_qkv_rope_takes(weight, batch, heads, kv_heads, head_dim):
        raise KernelError(f"wide_qkv_rope does not take a {tuple(weight.shape)} {weight.dtype} weight with {batch} rows and heads of {head_dim}")
    _int32(positions, "positions")
    _int32(slot_mapping, "slot_mapping")
    if positions.numel() < batch or slot_mapping.numel() < batch:
        raise KernelError("positions and slot_mapping must hold one entry per row")
    if cos.dtype != torch.float32 or cos.shape[-1] != head_dim // 2 or cos.shape != sin.shape or not cos.is_contiguous():
        raise KernelError(f"cos/sin tables must be contiguous float32 [positions, {head_dim // 2}]")
    if (k_pool.dtype != torch.bfloat16 or k_pool.shape != v_pool.shape or k_pool.dim() != 4 or k_pool.shape[1] != kv_heads
            or k_pool.shape[3] != head_dim or not k_pool.is_contiguous() or not v_pool.is_contiguous()):
        raise KernelError("cache pools must be contiguous bfloat16 [pages, kv_heads, page_size, head_dim]")
    q = torch.empty((batch, heads * head_dim), dtype=torch.bfloat16, device=x.device)
    ssq, count, _, width, eps = _norm_args(norm_parts, batch, SSQ_COLUMNS)
    lib = wide_gemm_lib()
    _run(lib, lib.mb_wide_qkv_rope(_p(x), x.stride(0), _p(weight), weight.stride(0), _p(q), q.stride(0), batch, k, heads, kv_heads,
                                   head_dim, _p(positions), _p(cos), _p(sin), _p(k_pool), _p(v_pool), _p(slot_mapping),
                                   k_pool.shape[2], _sm_count(x.device), ssq, count, width, eps, _stream()))
    return q


def tensor_core_gemm(a: torch.Tensor, weight: torch.Tensor, epilogue: int = EPI_BF16, out: Optional[torch.Tensor] = None,
                     norm_parts=None, emit_gain: Optional[torch.Tensor] = None):
    """The tcgen05 product for this many rows: up to 128 the wide decode form, above the prefill form.  The norms
    around a product ride in the wide form only (`norm_parts`, `emit_gain`, see wide_gemm): over a whole prompt a
    norm kernel runs at the speed of memory, and a residual epilogue that does its work, one tile per block with
    nothing to hide behind, was measured to cost as much (4 us each at 2,048 rows of 2,048)."""
    if a.shape[0] <= WIDE_ROWS:
        return wide_gemm(a, weight, epilogue, out, norm_parts=norm_parts, emit_gain=emit_gain)
    if norm_parts is not None or emit_gain is not None:
        raise KernelError("the norms ride in the products of up to 128 rows only")
    return gemm_tcgen05(a, weight, epilogue, out)


def prefill_attention_tcgen05_status(head_dim: int) -> int:
    """0 unless a bounded wait inside the tcgen05 prefill attention ever gave up (1 + (role << 8))."""
    return int(prefill_attention_tc(head_dim).mb_prefill_attention_tc_status())


def gemm_tcgen05_status() -> int:
    """0 unless a bounded wait inside a tcgen05 kernel ever gave up (then it names the role)."""
    return int(gemm_tc().mb_gemm_tc_status()) or int(wide_gemm_lib().mb_wide_gemm_status())


# ------------------------------------------------------------------------------------ the fused decode step

def decode_step_lib(head_dim: int):
    """The whole-step decode kernel, compiled for this head size at first use."""
    return load_library("mb_decode_step", ["decode_step.cu"], {"MB_HEAD_DIM": int(head_dim)})


def decode_step(lib, step, sms: int) -> None:
    """Launches csrc/decode_step.cu with the ctypes record `step` (engine/fused_decode.py builds it)."""
    _run(lib, lib.mb_decode_step(ctypes.byref(step), sms, _stream()))


# ------------------------------------------------------------------------------------ sampling

def argmax_rows(logits: torch.Tensor) -> torch.Tensor:
    _cuda(logits)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("argmax_rows takes float32 [rows, vocab] logits")
    out = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
    lib = sampling()
    _run(lib, lib.mb_argmax_rows(_p(logits), logits.stride(0), logits.shape[0], logits.shape[1], _p(out), _stream()))
    return out


def sample_max_sorted() -> int:
    return int(sampling().mb_sample_max_sorted())


def sample_rows(logits: torch.Tensor, work: torch.Tensor, counts: Optional[torch.Tensor], temperature: torch.Tensor,
                top_k: torch.Tensor, top_p: torch.Tensor, penalty: torch.Tensor, history: Optional[torch.Tensor],
                history_len: Optional[torch.Tensor], seeds: Optional[torch.Tensor], counters: Optional[torch.Tensor],
                uniforms: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                max_candidates: int = 0, history_rows: Optional[torch.Tensor] = None, append: bool = False) -> torch.Tensor:
    """One token per row of `logits` by the sampling pipeline.  `max_candidates`: the caller's bound on
    min(top_k, vocabulary) over the rows, 0 if it has none; when every row keeps at most
    sample_max_sorted() candidates a row is spread over a cluster of blocks instead of one block.
    The earlier tokens of the rows (for the repetition penalty) are the rows of `history`, or the int32
    arrays whose device addresses `history_rows` (int64 per row, 0: none) holds; `history_len` counts
    them either way.  With `append` the kernel stores each row's new id behind its history (the arrays
    of `history_rows` need room for it)."""
    _cuda(logits, work, counts, temperature, top_k, top_p, penalty, history, history_len, seeds, counters, uniforms, history_rows)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("sample_rows takes float32 [rows, vocab] logits")
    rows, vocab = logits.shape
    if work.dtype != torch.float32 or work.numel() < rows * vocab:
        raise KernelError("sample_rows needs rows*vocab floats of scratch")
    if counts is not None and (counts.dtype != torch.int32 or counts.numel() < rows * vocab):
        raise KernelError("sample_rows needs rows*vocab int32 counters for the repetition penalty")
    for name, t, dt in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
                        ("top_p", top_p, torch.float32), ("penalty", penalty, torch.float32)):
        if t.dtype != dt or t.numel() < rows:
            raise KernelError(f"{name} must hold {rows} values of {dt}")
    _int32(history, "history")
    _int32(history_len, "history_len")
    if (history is not None or history_rows is not None) and (counts is None or history_len is None):
        raise KernelError("a token history needs its lengths and the counters scratch")
    if history_rows is not None and (history is not None or history_rows.dtype != torch.int64 or history_rows.numel() < rows):
        raise KernelError(f"history_rows must hold {rows} int64 addresses and comes instead of a history matrix")
    if append and history_rows is None:
        raise KernelError("appending needs history_rows: a row of a history matrix has no room of its own")
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    lib = sampling()
    _run(lib, lib.mb_sample_rows(_p(logits), logits.stride(0), rows, vocab, _p(work), _p(counts), _p(temperature),
                                 _p(top_k), _p(top_p), _p(penalty), _p(history),
                                 history.stride(0) if history is not None else 0, _p(history_rows), 1 if append else 0,
                                 _p(history_len), _p(seeds),
                                 _p(counters), _p(uniforms), _p(out), int(max_candidates), _stream()))
    return out


# ------------------------------------------------------------------------------------ several residual streams

def hyper_streams_library():
    return load_library("mb_hyper_streams", ["hyper_streams.cu"])


def _streams_of(x: torch.Tensor, width: int, name: str) -> int:
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous() or x.shape[1] % width:
        raise KernelError(f"{name}: the streams must be contiguous float32 [tokens, streams * {width}], got {tuple(x.shape)} {x.dtype}")
    return x.shape[1] // width


def stream_copies(x: torch.Tensor, streams: int) -> torch.Tensor:
    """[tokens, streams * width] float32 whose every copy is x [tokens, width]."""
    _cuda(x)
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous():
        raise KernelError("stream_copies: x must be contiguous float32 [tokens, width]")
    out = torch.empty((x.shape[0], streams * x.shape[1]), dtype=torch.float32, device=x.device)
    lib = hyper_streams_library()
    _run(lib, lib.mb_stream_copies(_p(x), _p(out), x.shape[0], x.shape[1], streams, _stream()))
    return out


def stream_sum(x: torch.Tensor, width: int) -> torch.Tensor:
    """The copies of x [tokens, streams * width] added up: [tokens, width] float32."""
    _cuda(x)
    streams = _streams_of(x, width, "stream_sum")
    out = torch.empty((x.shape[0], width), dtype=torch.float32, device=x.device)
    lib = hyper_streams_library()
    _run(lib, lib.mb_stream_sum(_p(x), _p(out), x.shape[0], width, streams, _stream()))
    return out


def hyper_read_norm(x: torch.Tensor, coefficients: torch.Tensor, gain: torch.Tensor, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """u = sum_s coefficients[s] x_s over the copies of x [tokens, streams * width]; returns u / sqrt(mean(u^2) + eps) * gain
    as [tokens, width] of `out_dtype`.  All arithmetic float32."""
    _cuda(x, coefficients, gain)
    width = gain.numel()
    streams = _streams_of(x, width, "hyper_read_norm")
    if coefficients.dtype != torch.float32 or coefficients.numel() != streams or not coefficients.is_contiguous() \
            or gain.dtype != torch.float32 or not gain.is_contiguous():
        raise KernelError(f"hyper_read_norm: {streams} float32 coefficients and a float32 gain are needed")
    out = torch.empty((x.shape[0], width), dtype=out_dtype, device=x.device)
    lib = hyper_streams_library()
    _run(lib, lib.mb_hyper_read_norm(_p(x), _p(coefficients), _p(gain), _p(out), _code(out_dtype), x.shape[0], width, streams,
                                     ctypes.c_float(eps), _stream()))
    return out


def hyper_write(x: torch.Tensor, y: torch.Tensor, out_coefficients: torch.Tensor, mix: torch.Tensor) -> None:
    """All copies of x [tokens, streams * width] at once from the old ones: x_t <- sum_s mix[s, t] x_s + out_coefficients[t] * y
    for y [tokens, width] (float32 or bfloat16, may be a column slice)."""
    _cuda(x, y, out_coefficients, mix)
    _columns(y, "y")
    width = y.shape[1]
    streams = _streams_of(x, width, "hyper_write")
    if y.shape[0] != x.shape[0]:
        raise KernelError(f"hyper_write: y {tuple(y.shape)} does not fit the streams {tuple(x.shape)}")
    for name, t, count in (("out_coefficients", out_coefficients, streams), ("mix", mix, streams * streams)):
        if t.dtype != torch.float32 or t.numel() != count or not t.is_contiguous():
            raise KernelError(f"hyper_write: {name} must be contiguous float32 of {count} elements")
    lib = hyper_streams_library()
    _run(lib, lib.mb_hyper_write(_p(x), _p(y), y.stride(0), _code(y.dtype), _p(out_coefficients), _p(mix), x.shape[0], width, streams,
                                 _stream()))


def hyper_write_read_norm(x: torch.Tensor, y: torch.Tensor, out_coefficients: torch.Tensor, mix: torch.Tensor, coefficients: torch.Tensor,
                          gain: torch.Tensor, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """`hyper_write(x, y, out_coefficients, mix)` and then `hyper_read_norm(x, coefficients, gain, eps, out_dtype)` in one pass
    over the copies (the same bits as the two calls); y float32 [tokens, width]."""
    _cuda(x, y, out_coefficients, mix, coefficients, gain)
    _columns(y, "y")
    width = y.shape[1]
    streams = _streams_of(x, width, "hyper_write_read_norm")
    if y.shape[0] != x.shape[0] or y.dtype != torch.float32 or gain.numel() != width:
        raise KernelError(f"hyper_write_read_norm: y {tuple(y.shape)} {y.dtype} does not fit the streams {tuple(x.shape)}")
    for name, t, count in (("out_coefficients", out_coefficients, streams), ("mix", mix, streams * streams), ("coefficients", coefficients, streams),
                           ("gain", gain, width)):
        if t.dtype != torch.float32 or t.numel() != count or not t.is_contiguous():
            raise KernelError(f"hyper_write_read_norm: {name} must be contiguous float32 of {count} elements")
    out = torch.empty((x.shape[0], width), dtype=out_dtype, device=x.device)
    lib = hyper_streams_library()
    _run(lib, lib.mb_hyper_write_read_norm(_p(x), _p(y), y.stride(0), _p(out_coefficients), _p(mix), _p(coefficients), _p(gain), _p(out),
                                           _code(out_dtype), x.shape[0], width, streams, ctypes.c_float(eps), _stream()))
    return out


def hyper_max_streams() -> int:
    return hyper_streams_library().mb_hyper_max_streams()


# ------------------------------------------------------------------------------------ routed experts

def routed_experts_library():
    return load_library("mb_routed_experts", ["routed_experts.cu"])


def router_topk(x: torch.Tensor, router: torch.Tensor, top: int, scored: bool = False, correction: Optional[torch.Tensor] = None,
                groups: int = 1, keep: int = 1, weight_scale: float = 1.0):
    """Router logits z = router . x in float32 sums; per token the `top` experts with the largest logits (ties to the lower
    index) as int32 [tokens, top], largest first, and the softmax over the chosen logits as float32 [tokens, top].
    `scored`: the scores s = softmax(z) over all experts are taken first; the choice runs on s + correction (float32
    [experts], or None); the experts form `groups` equal groups of neighbours, a group counts by its largest choice score and
    only the `keep` best groups' experts can be chosen; the weights are weight_scale * s of the chosen, not renormalised."""
    _cuda(x, router, correction)
    if correction is not None and (correction.dtype != torch.float32 or correction.numel() != router.shape[0] or not correction.is_contiguous()):
        raise KernelError(f"router_topk: the correction must be contiguous float32 of {router.shape[0]} elements")
    _columns(x, "x")
    if router.dim() != 2 or not router.is_contiguous() or router.dtype != x.dtype or router.shape[1] != x.shape[1]:
        raise KernelError(f"router_topk: the router {tuple(router.shape)} {router.dtype} does not fit rows {tuple(x.shape)} {x.dtype}")
    tokens, experts = x.shape[0], router.shape[0]
    chosen = torch.empty((tokens, top), dtype=torch.int32, device=x.device)
    weights = torch.empty((tokens, top), dtype=torch.float32, device=x.device)
    lib = routed_experts_library()
    _run(lib, lib.mb_router_topk(_p(x), x.stride(0), _p(router), _code(x.dtype), _p(chosen), _p(weights), tokens, x.shape[1], experts,
                                 top, 1 if scored else 0, _p(correction), int(groups), int(keep), ctypes.c_float(weight_scale), _stream()))
    return chosen, weights


class RoutePlan:
    """The (token, choice) entries of a step grouped by expert: `sorted` [entries] entry ids (token * top + choice) by expert
    and in ascending order within one, `offsets` [experts + 1], and the tiles of rows a grouped product's blocks own."""

    def __init__(self, chosen: torch.Tensor, experts: int):
        lib = routed_experts_library()
        self.entries = chosen.numel()
        self.top = chosen.shape[1]
        self.experts = experts
        self.max_tiles = lib.mb_route_max_tiles(self.entries, experts)
        ints = torch.empty((experts + 1 + self.entries + 2 * self.max_tiles,), dtype=torch.int32, device=chosen.device)
        self.offsets = ints[:experts + 1]
        self.sorted = ints[experts + 1:experts + 1 + self.entries]
        self.tile_expert = ints[experts + 1 + self.entries:experts + 1 + self.entries + self.max_tiles]
        self.tile_row = ints[experts + 1 + self.entries + self.max_tiles:]
        _run(lib, lib.mb_route_sort(_p(chosen), self.entries, experts, _p(self.offsets), _p(self.sorted), _p(self.tile_expert),
                                    _p(self.tile_row), self.max_tiles, _stream()))


def route_sort(chosen: torch.Tensor, experts: int) -> RoutePlan:
    _cuda(chosen)
    _int32(chosen, "chosen")
    if chosen.dim() != 2:
        raise KernelError("route_sort: chosen must be [tokens, top]")
    return RoutePlan(chosen, experts)


def _expert_weights(w: torch.Tensor, experts: int, name: str):
    if w.dim() != 3 or w.shape[0] != experts or not w.is_contiguous():
        raise KernelError(f"{name}: expert matrices must be contiguous [{experts}, n, k], got {tuple(w.shape)}")


def expert_first_product(x: torch.Tensor, gate_w: torch.Tensor, up_w: torch.Tensor, plan: RoutePlan, limit: float, slope: float,
                         tensor_cores: bool = True, up_offset: float = 1.0) -> torch.Tensor:
    """mid [entries, n] (rows in the plan's sorted order, x's dtype): for every entry of expert e and its token's row x,
    g = min(gate_w[e] . x, limit), u = clamp(up_w[e] . x, -limit, limit), mid = g * sigmoid(slope * g) * (u + 1)."""
    _cuda(x, gate_w, up_w)
    _columns(x, "x")
    _expert_weights(gate_w, plan.experts, "expert_first_product")
    _expert_weights(up_w, plan.experts, "expert_first_product")
    if gate_w.shape != up_w.shape or gate_w.shape[2] != x.shape[1] or not (gate_w.dtype == up_w.dtype == x.dtype):
        raise KernelError(f"expert_first_product: matrices {tuple(gate_w.shape)} / {tuple(up_w.shape)} do not fit rows {tuple(x.shape)}")
    n, k = gate_w.shape[1], gate_w.shape[2]
    mid = torch.empty((plan.entries, n), dtype=x.dtype, device=x.device)
    lib = routed_experts_library()
    _run(lib, lib.mb_expert_product(_p(x), x.stride(0), _p(gate_w), _p(up_w), _p(mid), None, n, _code(x.dtype), _p(plan.sorted),
                                    _p(plan.offsets), _p(plan.tile_expert), _p(plan.tile_row), plan.max_tiles, plan.top, n, k,
                                    ctypes.c_float(limit), ctypes.c_float(slope), ctypes.c_float(up_offset), 1, 1 if tensor_cores else 0, _stream()))
    return mid


def expert_second_product(mid: torch.Tensor, down_w: torch.Tensor, plan: RoutePlan, tensor_cores: bool = True) -> torch.Tensor:
    """slot_out float32 [entries, n], row token * top + choice: down_w[e] . mid row of that entry (float32 sums)."""
    _cuda(mid, down_w)
    _expert_weights(down_w, plan.experts, "expert_second_product")
    if mid.dim() != 2 or not mid.is_contiguous() or mid.shape[0] != plan.entries or down_w.shape[2] != mid.shape[1] or down_w.dtype != mid.dtype:
        raise KernelError(f"expert_second_product: matrices {tuple(down_w.shape)} do not fit rows {tuple(mid.shape)}")
    n, k = down_w.shape[1], down_w.shape[2]
    slot_out = torch.empty((plan.entries, n), dtype=torch.float32, device=mid.device)
    lib = routed_experts_library()
    _run(lib, lib.mb_expert_product(_p(mid), mid.stride(0), _p(down_w), None, None, _p(slot_out), n, _code(mid.dtype), _p(plan.sorted),
                                    _p(plan.offsets), _p(plan.tile_expert), _p(plan.tile_row), plan.max_tiles, plan.top, n, k,
                                    ctypes.c_float(0.0), ctypes.c_float(0.0), ctypes.c_float(0.0), 0, 1 if tensor_cores else 0, _stream()))
    return slot_out


class PaddedRoutePlan:
    """The entries of a step grouped by expert with every expert's rows starting on a multiple of `tile` rows, for grouped
    products on the tensor cores whose tiles of rows each belong to one expert.  `sorted` [rows]: the entry at every row (-1
    at rows that fill a tile up), `position` [entries]: the row of every entry, `tile_group` [tiles]: the expert of every
    tile (-1 past the last one)."""

    def __init__(self, chosen: torch.Tensor, experts: int):
        lib = routed_experts_library()
        self.entries = chosen.numel()
        self.top = chosen.shape[1]
        self.experts = experts
        self.tile = lib.mb_route_group_tile()
        self.max_tiles = lib.mb_route_pad_max_tiles(self.entries, experts)
        self.rows = self.max_tiles * self.tile
        ints = torch.empty((self.rows + self.entries + self.max_tiles,), dtype=torch.int32, device=chosen.device)
        self.sorted = ints[:self.rows]
        self.position = ints[self.rows:self.rows + self.entries]
        self.tile_group = ints[self.rows + self.entries:]
        _run(lib, lib.mb_route_pad(_p(chosen), self.entries, experts, _p(self.sorted), _p(self.position), _p(self.tile_group),
                                   self.max_tiles, _stream()))


def route_pad_takes(experts: int) -> bool:
    return experts <= routed_experts_library().mb_route_pad_max_experts()


def route_pad(chosen: torch.Tensor, experts: int) -> PaddedRoutePlan:
    _cuda(chosen)
    _int32(chosen, "chosen")
    if chosen.dim() != 2 or not chosen.is_contiguous():
        raise KernelError("route_pad: chosen must be contiguous [tokens, top]")
    return PaddedRoutePlan(chosen, experts)


def gather_rows(x: torch.Tensor, plan: PaddedRoutePlan) -> torch.Tensor:
    """bfloat16 [plan.rows, k]: row r is x[plan.sorted[r] // top], zeros at rows that fill a tile up; the rows of tiles past
    the last one are not written."""
    _cuda(x)
    _columns(x, "x")
    if x.dtype != torch.bfloat16:
        raise KernelError("gather_rows: bfloat16 rows are needed")
    out = torch.empty((plan.rows, x.shape[1]), dtype=torch.bfloat16, device=x.device)
    lib = routed_experts_library()
    _run(lib, lib.mb_gather_rows(_p(x), x.stride(0), _p(plan.sorted), _p(plan.tile_group), _p(out), plan.rows, plan.top, x.shape[1],
                                 _stream()))
    return out


def grouped_product_takes(gate_up: torch.Tensor, down: torch.Tensor) -> bool:
    """Whether the grouped tcgen05 products take these expert matrices: gate_up [2, experts, ff, width] (gate rows of all
    experts, then up rows), down [experts, width, ff], bfloat16, rows on 16-byte boundaries."""
    if gate_up.dtype != torch.bfloat16 or down.dtype != torch.bfloat16 or gate_up.dim() != 4 or down.dim() != 3:
        return False
    _, experts, ff, width = gate_up.shape
    return (gate_up.is_contiguous() and down.is_contiguous() and width % 8 == 0 and ff % 8 == 0 and gate_up.data_ptr() % 16 == 0
            and down.data_ptr() % 16 == 0 and 2 * experts * ff < 2 ** 31 and route_pad_takes(experts))


def grouped_first_product(a: torch.Tensor, gate_up: torch.Tensor, plan: PaddedRoutePlan, limit: float, slope: float,
                          up_offset: float = 1.0) -> torch.Tensor:
    """mid bfloat16 [plan.rows, ff]: for the rows of a tile of expert e, g = min(gate[e] . a, limit),
    u = clamp(up[e] . a, -limit, limit), mid = g * sigmoid(slope * g) * (u + 1), on the tcgen05 tensor cores."""
    _cuda(a, gate_up)
    _, experts, ff, width = gate_up.shape
    if a.dtype != torch.bfloat16 or not a.is_contiguous() or tuple(a.shape) != (plan.rows, width) or experts != plan.experts:
        raise KernelError(f"grouped_first_product: rows {tuple(a.shape)} do not fit matrices {tuple(gate_up.shape)}")
    mid = torch.empty((plan.rows, ff), dtype=torch.bfloat16, device=a.device)
    lib = gemm_tc()
    _run(lib, lib.mb_gemm_tcgen05_grouped(_p(a), a.stride(0), _p(gate_up), width, 2 * experts * ff, _p(mid), ff, plan.rows, ff, width,
                                          1, experts * ff, _p(plan.tile_group), ctypes.c_float(limit), ctypes.c_float(slope), ctypes.c_float(up_offset),
                                          _sm_count(a.device), _stream()))
    return mid


def grouped_second_product(mid: torch.Tensor, down: torch.Tensor, plan: PaddedRoutePlan) -> torch.Tensor:
    """float32 [plan.rows, width]: row r of a tile of expert e is down[e] . mid[r] (float32 sums)."""
    _cuda(mid, down)
    experts, width, ff = down.shape
    if mid.dtype != torch.bfloat16 or not mid.is_contiguous() or tuple(mid.shape) != (plan.rows, ff) or experts != plan.experts:
        raise KernelError(f"grouped_second_product: rows {tuple(mid.shape)} do not fit matrices {tuple(down.shape)}")
    out = torch.empty((plan.rows, width), dtype=torch.float32, device=mid.device)
    lib = gemm_tc()
    _run(lib, lib.mb_gemm_tcgen05_grouped(_p(mid), ff, _p(down), ff, experts * width, _p(out), width, plan.rows, width, ff, 0, 0,
                                          _p(plan.tile_group), ctypes.c_float(0.0), ctypes.c_float(0.0), ctypes.c_float(0.0), _sm_count(mid.device),
                                          _stream()))
    return out


GROUPED_ROWS_PER_EXPERT = 32  # from so many entries per expert on average a step pads the experts' rows to tiles of 128

EXPERT_ROWS_ENTRIES = 64  # up to so many (token, choice) entries a step's experts run entry by entry, without sorting


def expert_rows_first(x: torch.Tensor, gate_w: torch.Tensor, up_w: torch.Tensor, chosen: torch.Tensor, limit: float,
                      slope: float, up_offset: float = 1.0) -> torch.Tensor:
    """The first product for a step of few tokens: mid [tokens * top, n] (row token * top + choice, x's dtype), each row
    clamped_swish(gate_w[e] . x, up_w[e] . x) for its token's row x and its chosen expert e.  Every entry streams its
    expert's matrices once; nothing is sorted."""
    _cuda(x, gate_w, up_w, chosen)
    _columns(x, "x")
    _int32(chosen, "chosen")
    experts = gate_w.shape[0]
    _expert_weights(gate_w, experts, "expert_rows_first")
    _expert_weights(up_w, experts, "expert_rows_first")
    if gate_w.shape != up_w.shape or gate_w.shape[2] != x.shape[1] or not (gate_w.dtype == up_w.dtype == x.dtype) \
            or chosen.dim() != 2 or chosen.shape[0] != x.shape[0] or not chosen.is_contiguous():
        raise KernelError(f"expert_rows_first: matrices {tuple(gate_w.shape)} / {tuple(up_w.shape)} and choices {tuple(chosen.shape)} "
                          f"do not fit rows {tuple(x.shape)}")
    n, k, top = gate_w.shape[1], gate_w.shape[2], chosen.shape[1]
    mid = torch.empty((chosen.numel(), n), dtype=x.dtype, device=x.device)
    lib = routed_experts_library()
    _run(lib, lib.mb_expert_rows(_p(x), x.stride(0), _p(gate_w), _p(up_w), _p(mid), None, n, _code(x.dtype), _p(chosen), chosen.numel(),
                                 top, experts, n, k, ctypes.c_float(limit), ctypes.c_float(slope), ctypes.c_float(up_offset), 1, _stream()))
    return mid


def expert_rows_second(mid: torch.Tensor, down_w: torch.Tensor, chosen: torch.Tensor) -> torch.Tensor:
    """slot_out float32 [tokens * top, n]: row i is down_w[e_i] . mid[i] for entry i's chosen expert (float32 sums)."""
    _cuda(mid, down_w, chosen)
    _int32(chosen, "chosen")
    experts = down_w.shape[0]
    _expert_weights(down_w, experts, "expert_rows_second")
    if mid.dim() != 2 or not mid.is_contiguous() or mid.shape[0] != chosen.numel() or down_w.shape[2] != mid.shape[1] \
            or down_w.dtype != mid.dtype or not chosen.is_contiguous():
        raise KernelError(f"expert_rows_second: matrices {tuple(down_w.shape)} do not fit rows {tuple(mid.shape)}")
    n, k = down_w.shape[1], down_w.shape[2]
    slot_out = torch.empty((mid.shape[0], n), dtype=torch.float32, device=mid.device)
    lib = routed_experts_library()
    _run(lib, lib.mb_expert_rows(_p(mid), mid.stride(0), _p(down_w), None, None, _p(slot_out), n, _code(mid.dtype), _p(chosen),
                                 chosen.numel(), chosen.shape[1], experts, n, k, ctypes.c_float(0.0), ctypes.c_float(0.0), ctypes.c_float(0.0), 0, _stream()))
    return slot_out


def clamped_swish(gate: torch.Tensor, up: torch.Tensor, out: torch.Tensor, limit: float, slope: float, up_offset: float = 1.0) -> None:
    """out = g * sigmoid(slope * g) * (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit); gate and up column
    slices of one tensor."""
    _cuda(gate, up, out)
    for name, t in (("gate", gate), ("up", up), ("out", out)):
        _columns(t, name)
    if gate.shape != up.shape or out.shape != gate.shape or gate.stride(0) != up.stride(0) or not (gate.dtype == up.dtype == out.dtype):
        raise KernelError("clamped_swish: gate, up and out must share shape and dtype, gate and up one row stride")
    lib = routed_experts_library()
    _run(lib, lib.mb_clamped_swish(_p(gate), _p(up), gate.stride(0), _p(out), out.stride(0), _code(gate.dtype), gate.shape[0],
                                   gate.shape[1], ctypes.c_float(limit), ctypes.c_float(slope), ctypes.c_float(up_offset), _stream()))


def expert_combine(slot_out: torch.Tensor, weights: torch.Tensor, shared: Optional[torch.Tensor] = None,
                   score: Optional[torch.Tensor] = None, position: Optional[torch.Tensor] = None,
                   chosen: Optional[torch.Tensor] = None, experts: int = 0, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = sum_s weights[t, s] * slot_out[t * top + s] (+ sigmoid(score[t]) * shared[t]) as float32 [tokens, width];
    shared float32 [tokens, width], score one number per token ([tokens, 1], may be a column slice; None: the shared expert
    is added as it is).  With `position` (int32 [tokens * top]) entry t * top + s has its row of slot_out at
    position[t * top + s].  With `chosen` (int32 [tokens, top]), `experts` and `rows` ([tokens, width], the rows the experts
    read): an entry whose expert is >= `experts` is an identity expert, its result is rows[t] and slot_out is not read for it."""
    _cuda(slot_out, weights, shared, score, position, chosen, rows)
    tokens, top = weights.shape
    width = slot_out.shape[1]
    if position is not None and (position.dtype != torch.int32 or position.numel() != tokens * top or not position.is_contiguous()):
        raise KernelError("expert_combine: position must be contiguous int32 [tokens * top]")
    if slot_out.dtype != torch.float32 or not slot_out.is_contiguous() or (position is None and slot_out.shape[0] != tokens * top) \
            or weights.dtype != torch.float32 or not weights.is_contiguous():
        raise KernelError("expert_combine: slot_out float32 [tokens * top, width] and weights float32 [tokens, top] are needed")
    if score is not None and shared is None:
        raise KernelError("expert_combine: gate scores without a shared expert")
    dtype = _F32
    if shared is not None:
        if shared.dtype != torch.float32 or not shared.is_contiguous() or tuple(shared.shape) != (tokens, width):
            raise KernelError("expert_combine: shared must be contiguous float32 [tokens, width]")
        if score is not None:
            _columns(score, "score")
            if score.shape[0] != tokens:
                raise KernelError("expert_combine: one gate score per token is needed")
            dtype = _code(score.dtype)
    if (chosen is None) != (rows is None):
        raise KernelError("expert_combine: identity experts need both the choices and the tokens' rows")
    if chosen is not None:
        _int32(chosen, "chosen")
        _columns(rows, "rows")
        if tuple(chosen.shape) != (tokens, top) or not chosen.is_contiguous() or tuple(rows.shape) != (tokens, width):
            raise KernelError("expert_combine: choices [tokens, top] and rows [tokens, width] are needed")
        if score is not None and score.dtype != rows.dtype:
            raise KernelError("expert_combine: gate scores and rows must share one dtype")
        dtype = _code(rows.dtype)
    out = torch.empty((tokens, width), dtype=torch.float32, device=slot_out.device)
    lib = routed_experts_library()
    _run(lib, lib.mb_expert_combine(_p(slot_out), _p(weights), _p(shared), _p(score), score.stride(0) if score is not None else 0,
                                    dtype, _p(out), tokens, width, top, _p(position), _p(chosen), int(experts), _p(rows),
                                    rows.stride(0) if rows is not None else 0, _stream()))
    return out
