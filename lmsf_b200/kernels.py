"""Python faces of the CUDA kernels in `csrc/`.

Each function checks what the kernel cannot check (device, dtype, contiguity), takes the
launching stream from torch and raises `KernelError` with the library's own message when
the kernel refuses a size.  There is no CPU path: tensors that are not on a CUDA device
are an error.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional, Sequence, Tuple

import torch

from .csrc.build import load_library

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dt}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The handle of the current stream of the current device (asked at every launch: graphs are captured on
    another stream).  The raw getter saves building a Stream object, about 2 us a launch."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("lmsf_b200 kernels run on CUDA tensors only; got a tensor on " + str(t.device))
    return t.data_ptr()


def _i32(t: Optional[torch.Tensor], name: str) -> Optional[int]:
    if t is None:
        return None
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous int32 tensor")
    return _ptr(t)


_FUNCS = {}


def _func(source: str, name: str, argtypes, defines: Tuple[str, ...] = ()):
    key = (source, name, defines)
    f = _FUNCS.get(key)
    if f is None:
        lib = load_library(source, defines)
        f = getattr(lib, name)
        f.argtypes = argtypes
        f.restype = c_int
        _FUNCS[key] = f
    return f


_LAUNCHES = 0


def launch_count() -> int:
    """Kernels of this package launched so far (launches replayed from a CUDA graph are added by the runner)."""
    return _LAUNCHES


def add_launches(n: int) -> None:
    global _LAUNCHES
    _LAUNCHES += n


def _check(rc: int, source: str, prefix: str, defines: Tuple[str, ...] = ()):
    global _LAUNCHES
    if rc == 0:
        _LAUNCHES += 1
        return
    if rc < 0:
        lib = load_library(source, defines)
        getter = getattr(lib, prefix + "_last_error")
        getter.restype = ctypes.c_char_p
        raise KernelError(getter().decode())
    raise KernelError(f"CUDA error {rc} at the launch of a kernel of {source}")


# ----------------------------------------------------------------------------- embedding

def embedding(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, error_flag: Optional[torch.Tensor] = None,
              scale: float = 1.0):
    """out[t, :] = table[ids[t], :] (times `scale`, if it is not 1); out and table share one dtype."""
    n, hidden = out.shape
    if table.dtype != out.dtype or table.shape[1] != hidden or not (out.is_contiguous() and table.is_contiguous()):
        raise KernelError("embedding: out and table must be contiguous, of one dtype and one width")
    if scale != 1.0:
        f = _func("embedding.cu", "lmsf_embedding_scaled",
                  [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p])
        rc = f(_ptr(out), _ptr(table), _i32(ids, "ids"), n, hidden, table.shape[0], float(scale), dtype_code(out.dtype),
               _i32(error_flag, "error_flag"), _stream())
        _check(rc, "embedding.cu", "lmsf_embedding")
        return
    f = _func("embedding.cu", "lmsf_embedding",
              [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    rc = f(_ptr(out), _ptr(table), _i32(ids, "ids"), n, hidden, table.shape[0], dtype_code(out.dtype),
           _i32(error_flag, "error_flag"), _stream())
    _check(rc, "embedding.cu", "lmsf_embedding")


def embedding_pairs(out: torch.Tensor, table: torch.Tensor, pairs: torch.Tensor, ids: torch.Tensor, positions: torch.Tensor,
                    token_seq: torch.Tensor, cu_q: torch.Tensor, state_slot: torch.Tensor, last: torch.Tensor, buckets: int,
                    mul_prev: int, mul_cur: int, scale: float = 1.0, error_flag: Optional[torch.Tensor] = None):
    """out[t] = table[id_t] * scale + pairs[(id_{t-1} * mul_prev + id_t * mul_cur) mod buckets] in float32; a request's first
    token takes pairs[buckets].  `last` (int32, one per state slot) holds the token before a portion and receives the
    portion's last token.  out: float32 [n, hidden]; table [vocab, hidden] and pairs [buckets + 1, hidden] of one dtype."""
    n, hidden = out.shape
    if out.dtype != torch.float32 or not out.is_contiguous() or table.shape[1] != hidden or not table.is_contiguous() or \
            pairs.shape != (buckets + 1, hidden) or pairs.dtype != table.dtype or not pairs.is_contiguous():
        raise KernelError("embedding_pairs: out float32 [n, hidden], table [vocab, hidden], pairs [buckets + 1, hidden]")
    if last.dtype != torch.int32 or not last.is_contiguous():
        raise KernelError("embedding_pairs: the slots' last tokens must be contiguous int32")
    f = _func("embedding.cu", "lmsf_embedding_pairs",
              [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
               c_int, c_longlong, c_longlong, c_float, c_int, c_void_p, c_void_p])
    rc = f(_ptr(out), _ptr(table), _ptr(pairs), _i32(ids, "ids"), _i32(positions, "positions"), _i32(token_seq, "token_seq"),
           _i32(cu_q, "cu_q"), _i32(state_slot, "state_slot"), _ptr(last), n, hidden, table.shape[0], int(buckets),
           int(mul_prev), int(mul_cur), float(scale), dtype_code(table.dtype), _i32(error_flag, "error_flag"), _stream())
    _check(rc, "embedding.cu", "lmsf_embedding")


def patch_tokens(token_ids: torch.Tensor, dst: torch.Tensor, src: torch.Tensor, source: torch.Tensor):
    """token_ids[dst[i]] = source[src[i]] wherever dst[i] >= 0 (all int32, on the device)."""
    f = _func("embedding.cu", "lmsf_patch_tokens", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    rc = f(_i32(token_ids, "token_ids"), _i32(dst, "dst"), _i32(src, "src"), _i32(source, "source"), dst.numel(), _stream())
    _check(rc, "embedding.cu", "lmsf_embedding")


# ----------------------------------------------------------------------------- rmsnorm

def add_rmsnorm(h: torch.Tensor, x: torch.Tensor, res: Optional[torch.Tensor], w: torch.Tensor, eps: float, mode: int):
    """mode 0: h = norm(x) w.  mode 1: res = float(x); h = norm(res) w.  mode 2: res += float(x); h = norm(res) w.
    x, h: [n, hidden] float32 or bfloat16; res: float32; w: [hidden] of x's dtype or float32."""
    n, hidden = x.shape
    if h.shape != x.shape or h.dtype != x.dtype or not (x.is_contiguous() and h.is_contiguous()):
        raise KernelError("rmsnorm: h and x must be contiguous and alike")
    if res is not None and (res.dtype != torch.float32 or res.shape != x.shape or not res.is_contiguous()):
        raise KernelError("rmsnorm: the residual must be contiguous float32 of x's shape")
    if w.shape != (hidden,) or not w.is_contiguous():
        raise KernelError(f"rmsnorm: weight of shape {tuple(w.shape)} for width {hidden}")
    f = _func("rmsnorm.cu", "lmsf_add_rmsnorm",
              [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p])
    rc = f(_ptr(h), _ptr(x), _ptr(res), _ptr(w), n, hidden, float(eps), mode, dtype_code(x.dtype),
           dtype_code(w.dtype), _stream())
    _check(rc, "rmsnorm.cu", "lmsf_rmsnorm")


def finish_rmsnorm(h: torch.Tensor, res: torch.Tensor, sumsq: torch.Tensor, w: torch.Tensor, eps: float):
    """h = (res / rms) w, where sumsq[m] adds up to the sum of squares of row m of res: the second half of a norm whose
    first half `gemm_skinny_residual` did, for a product that cannot take a prenormed input."""
    n, hidden = res.shape
    if h.shape != res.shape or h.dtype != torch.bfloat16 or not (h.is_contiguous() and res.is_contiguous()) or res.dtype != torch.float32:
        raise KernelError("finish_rmsnorm: h must be bfloat16 and res float32, contiguous and of one shape")
    if sumsq.dtype != torch.float32 or sumsq.dim() != 2 or sumsq.shape[0] < n or sumsq.stride(1) != 1:
        raise KernelError("finish_rmsnorm: the sums of squares must be float32 [rows, parts]")
    if w.shape != (hidden,) or not w.is_contiguous():
        raise KernelError(f"finish_rmsnorm: weight of shape {tuple(w.shape)} for width {hidden}")
    f = _func("rmsnorm.cu", "lmsf_finish_rmsnorm",
              [c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_int, c_int, c_float, c_int, c_int, c_void_p])
    rc = f(_ptr(h), _ptr(res), _ptr(sumsq), sumsq.shape[1], sumsq.stride(0), _ptr(w), n, hidden, float(eps),
           dtype_code(h.dtype), dtype_code(w.dtype), _stream())
    _check(rc, "rmsnorm.cu", "lmsf_rmsnorm")


# ----------------------------------------------------------------------------- rope + cache write

def rope_cache_write(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor], positions: torch.Tensor,
                     token_seq: Optional[torch.Tensor], block_table: Optional[torch.Tensor], block_size: int,
                     cache: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor], rot_dim: int, is_neox: bool,
                     n_q_heads: int, n_kv_heads: int, head_dim: int, error_flag: Optional[torch.Tensor] = None):
    """Rotates q in place; writes rotated k and v into `cache` [pages, 2, n_kv_heads, block_size, head_dim]
    at the page that `block_table[token_seq[t], positions[t] // block_size]` names.  q, k, v: [n, heads*head_dim]
    views whose last dimension is contiguous (row strides are free).  cache None: q only."""
    n = q.shape[0]
    for name, t, heads in (("q", q, n_q_heads), ("k", k, n_kv_heads), ("v", v, n_kv_heads)):
        if t is None:
            continue
        if t.dim() != 2 or t.shape[1] != heads * head_dim or t.stride(1) != 1 or t.shape[0] != n:
            raise KernelError(f"rope_cache: {name} must be [n, {heads * head_dim}] with a contiguous last dimension")
        if t.dtype != q.dtype:
            raise KernelError("rope_cache: q, k, v must share one dtype")
    page_stride = 0
    max_blocks = 0
    if cache is not None:
        if cache.dtype != q.dtype or not cache.is_contiguous() or tuple(cache.shape[1:]) != (2, n_kv_heads, block_size, head_dim):
            raise KernelError(f"rope_cache: cache of shape {tuple(cache.shape)} does not match "
                              f"[pages, 2, {n_kv_heads}, {block_size}, {head_dim}] of {q.dtype}")
        page_stride = cache.stride(0)
        max_blocks = block_table.shape[1]
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_dim // 2):
        raise KernelError("rope_cache: inv_freq must hold rot_dim / 2 float32 values")
    f = _func("rope_cache.cu", "lmsf_rope_cache_write",
              [c_void_p, c_void_p, c_void_p, c_longlong, c_longlong, c_longlong, c_void_p, c_void_p, c_void_p, c_int,
               c_int, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
               c_void_p])
    rc = f(_ptr(q), _ptr(k), _ptr(v), q.stride(0), k.stride(0) if k is not None else 0,
           v.stride(0) if v is not None else 0, _i32(positions, "positions"), _i32(token_seq, "token_seq"),
           _i32(block_table, "block_table"), max_blocks, block_size, _ptr(cache), page_stride, _ptr(inv_freq),
           rot_dim, int(is_neox), n, n_q_heads, n_kv_heads, head_dim, dtype_code(q.dtype),
           _i32(error_flag, "error_flag"), _stream())
    _check(rc, "rope_cache.cu", "lmsf_rope_cache")


def qk_norm_rope_cache_write(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor], positions: torch.Tensor,
                             token_seq: Optional[torch.Tensor], block_table: Optional[torch.Tensor], block_size: int,
                             cache: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor], rot_dim: int, is_neox: bool,
                             n_q_heads: int, n_kv_heads: int, head_dim: int, norm_dim: int, wq: Optional[torch.Tensor],
                             wk: Optional[torch.Tensor], eps: float, error_flag: Optional[torch.Tensor] = None,
                             weightless: bool = False, v_norm_dim: int = 0):
    """Per head: RMS norm of q and k over their first `norm_dim` values (float32 weights wq, wk [norm_dim]; None: no
    norm, or with `weightless` a division by the root mean square alone), then the rotation of the first `rot_dim`
    values, then k and v into `cache` as `rope_cache_write` does; one kernel, rounded once.  v_norm_dim > 0: every value
    head is divided by the root mean square of its first v_norm_dim values on the way.  q is changed in place.  cache
    None: q only."""
    n = q.shape[0]
    for name, t, heads in (("q", q, n_q_heads), ("k", k, n_kv_heads), ("v", v, n_kv_heads)):
        if t is None:
            continue
        if t.dim() != 2 or t.shape[1] != heads * head_dim or t.stride(1) != 1 or t.shape[0] != n or t.dtype != q.dtype:
            raise KernelError(f"qk_norm_rope: {name} must be [n, {heads * head_dim}] with a contiguous last dimension, of one dtype")
    page_stride = max_blocks = 0
    if cache is not None:
        if cache.dtype != q.dtype or not cache.is_contiguous() or tuple(cache.shape[1:]) != (2, n_kv_heads, block_size, head_dim):
            raise KernelError(f"qk_norm_rope: cache of shape {tuple(cache.shape)} does not match "
                              f"[pages, 2, {n_kv_heads}, {block_size}, {head_dim}] of {q.dtype}")
        page_stride, max_blocks = cache.stride(0), block_table.shape[1]
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_dim // 2):
        raise KernelError("qk_norm_rope: inv_freq must hold rot_dim / 2 float32 values")
    f = _func("qk_norm_rope.cu", "lmsf_qk_norm_rope_cache_write_unit",
              [c_void_p, c_void_p, c_void_p, c_longlong, c_longlong, c_longlong, c_void_p, c_void_p, c_void_p, c_int,
               c_int, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
               c_float, c_int, c_void_p, c_int, c_int, c_void_p])
    rc = f(_ptr(q), _ptr(k), _ptr(v), q.stride(0), k.stride(0) if k is not None else 0,
           v.stride(0) if v is not None else 0, _i32(positions, "positions"), _i32(token_seq, "token_seq"),
           _i32(block_table, "block_table"), max_blocks, block_size, _ptr(cache), page_stride, _ptr(inv_freq),
           rot_dim, int(is_neox), n, n_q_heads, n_kv_heads, head_dim, norm_dim, _f32vec(wq, norm_dim, "wq"),
           _f32vec(wk, norm_dim, "wk"), float(eps), dtype_code(q.dtype), _i32(error_flag, "error_flag"), int(bool(weightless)),
           int(v_norm_dim or 0), _stream())
    _check(rc, "qk_norm_rope.cu", "lmsf_qk_norm_rope")


# ----------------------------------------------------------------------------- attention (generic)

GENERIC_MAX_HEAD_DIM = 512     # the plain attention kernel holds a head's accumulator in registers up to this size


def _per_head(t: Optional[torch.Tensor], heads: int, what: str) -> None:
    if t is not None and (t.dtype != torch.float32 or t.shape != (heads,) or not t.is_contiguous()):
        raise KernelError(f"attention: {what} must be float32 [n_q_heads]")


_GENERIC_MASKED_ARGS = [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_int, c_int, c_void_p,
                        c_void_p, c_float, c_float, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                        c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_void_p]
_GENERIC_WEIGHTS_ARGS = [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_int, c_int, c_void_p,
                         c_void_p, c_float, c_float, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                         c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]


def attention_generic(out: torch.Tensor, q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                      block_size: int, token_seq: torch.Tensor, positions: torch.Tensor, scale: float, window: int,
                      n_q_heads: int, n_kv_heads: int, head_dim: int, softcap: float = 0.0,
                      slopes: Optional[torch.Tensor] = None, chunk: int = 0,
                      log_bias: Optional[Tuple[torch.Tensor, torch.Tensor]] = None, sinks: Optional[torch.Tensor] = None,
                      gate: Optional[torch.Tensor] = None, keep_first: int = 0, sigmoid: bool = False,
                      head_bias: Optional[torch.Tensor] = None):
    """out[t] = softmax(scale q[t] K^T) V over the keys lo..positions[t] of token t's request, read from pages.
    q, out: [n, n_q_heads * head_dim] (last dimension contiguous); window <= 0 means all keys; softcap > 0 caps the
    scaled scores smoothly, softcap * tanh(score / softcap); slopes (float32 [n_q_heads]) adds
    slopes[head] * (key position - query position) to the scaled scores.  chunk > 0: a query at position p sees the keys
    p - p % chunk .. p only.  log_bias (r1, r2), float32 [n_q_heads] each: r1 * log(1 + r2 * distance) is taken off the
    scaled scores.  sinks (float32 [n_q_heads]): exp(sink) is one more term of the softmax's denominator.  gate ([n,
    n_q_heads] view of q's dtype): head h's output is multiplied by sigmoid(gate[t, h]).  keep_first (with a window): the
    request's first keep_first keys stay visible behind the window.  sigmoid: a visible key's weight is sigmoid(score), not
    normalised over the keys.  head_bias (float32 [n_q_heads]): added to every scaled score of its head."""
    n = q.shape[0]
    if q.stride(1) != 1 or out.stride(1) != 1 or q.shape[1] != n_q_heads * head_dim or out.shape != q.shape:
        raise KernelError("attention: q and out must be [n, heads * head_dim] with a contiguous last dimension")
    if cache.dtype != q.dtype or out.dtype != q.dtype or not cache.is_contiguous() or \
            tuple(cache.shape[1:]) != (2, n_kv_heads, block_size, head_dim):
        raise KernelError(f"attention: cache of shape {tuple(cache.shape)} / {cache.dtype} does not match the heads")
    _per_head(slopes, n_q_heads, "slopes")
    _per_head(sinks, n_q_heads, "sinks")
    _per_head(head_bias, n_q_heads, "the bias per head")
    r1, r2 = log_bias if log_bias is not None else (None, None)
    _per_head(r1, n_q_heads, "the logarithmic bias")
    _per_head(r2, n_q_heads, "the logarithmic bias")
    if gate is not None and (gate.shape != (n, n_q_heads) or gate.stride(1) != 1 or gate.dtype != q.dtype):
        raise KernelError("attention: the gate must be [n, heads] of q's dtype")
    f = _func("attention_generic.cu", "lmsf_attention_generic_weights", _GENERIC_WEIGHTS_ARGS)
    rc = f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(cache), cache.stride(0),
           _i32(block_table, "block_table"), block_table.shape[1], block_size, _i32(token_seq, "token_seq"),
           _i32(positions, "positions"), float(scale), float(softcap or 0.0), _ptr(slopes), int(window or 0), n, n_q_heads,
           n_kv_heads, head_dim, dtype_code(q.dtype), 0, _ptr(gate), gate.stride(0) if gate is not None else 0,
           int(chunk or 0), _ptr(r1), _ptr(r2), _ptr(sinks), int(keep_first or 0), 1 if sigmoid else 0, _ptr(head_bias), _stream())
    _check(rc, "attention_generic.cu", "lmsf_attention_generic")


# ----------------------------------------------------------------------------- gated activation

ACT_CODES = {"silu": 0, "swish": 0, "gelu_tanh": 1, "gelu_pytorch_tanh": 1}


def gated_act(out: torch.Tensor, x: torch.Tensor, act: str = "silu"):
    """out[t, i] = act(x[t, i]) * x[t, d + i]; x: [n, 2 d], out: [n, d] contiguous."""
    n, d = out.shape
    if x.shape != (n, 2 * d) or x.stride(1) != 1 or not out.is_contiguous() or x.dtype != out.dtype:
        raise KernelError("gated_act: x must be [n, 2d] and out [n, d] of one dtype")
    if act not in ACT_CODES:
        raise KernelError(f"gated_act: unknown activation {act!r} (known: {', '.join(sorted(ACT_CODES))})")
    f = _func("activation.cu", "lmsf_gated_act", [c_void_p, c_void_p, c_int, c_int, c_longlong, c_int, c_int, c_void_p])
    rc = f(_ptr(out), _ptr(x), n, d, x.stride(0), ACT_CODES[act], dtype_code(out.dtype), _stream())
    _check(rc, "activation.cu", "lmsf_activation")


def poly_norm(out: torch.Tensor, x: torch.Tensor, coef: torch.Tensor, eps: float):
    """out[t] = a N(x[t]) + b N(x[t]^2) + c N(x[t]^3) + e with (a, b, c, e) = coef (float32 [4] on the device), powers element
    by element and N the division of a row by its root mean square (eps inside the root); float32 inside.  x: [n, d] view,
    out: [n, d] contiguous, one dtype."""
    n, d = out.shape
    if x.shape != (n, d) or x.stride(1) != 1 or not out.is_contiguous() or x.dtype != out.dtype:
        raise KernelError("poly_norm: x and out must be [n, d] of one dtype")
    f = _func("activation.cu", "lmsf_poly_norm", [c_void_p, c_void_p, c_int, c_int, c_longlong, c_void_p, c_float, c_int, c_void_p])
    rc = f(_ptr(out), _ptr(x), n, d, x.stride(0), _f32vec(coef, 4, "coef"), float(eps), dtype_code(out.dtype), _stream())
    _check(rc, "activation.cu", "lmsf_activation")


def clamped_glu(out: torch.Tensor, x: torch.Tensor, limit: float, alpha: float = 1.702):
    """out[t, i] = g * sigmoid(alpha * g) * (u + 1) with g = min(x[t, i], limit), u = clamp(x[t, d + i], -limit, limit);
    x: [n, 2 d], out: [n, d] contiguous."""
    n, d = out.shape
    if x.shape != (n, 2 * d) or x.stride(1) != 1 or not out.is_contiguous() or x.dtype != out.dtype:
        raise KernelError("clamped_glu: x must be [n, 2d] and out [n, d] of one dtype")
    f = _func("activation.cu", "lmsf_clamped_glu", [c_void_p, c_void_p, c_int, c_int, c_longlong, c_float, c_float, c_int, c_void_p])
    rc = f(_ptr(out), _ptr(x), n, d, x.stride(0), float(limit), float(alpha), dtype_code(out.dtype), _stream())
    _check(rc, "activation.cu", "lmsf_activation")


def gelu_mul_gather(out: torch.Tensor, a: torch.Tensor, table: torch.Tensor, offset: int, ids: torch.Tensor,
                    error_flag: Optional[torch.Tensor] = None):
    """out[t, i] = gelu_tanh(a[t, i]) * table[ids[t], offset + i]; a: [n, d] view, table: [vocab, width] contiguous."""
    n, d = out.shape
    if a.shape != (n, d) or a.stride(1) != 1 or not out.is_contiguous() or a.dtype != out.dtype or table.dtype != out.dtype \
            or table.dim() != 2 or not table.is_contiguous():
        raise KernelError("gelu_mul_gather: a and out [n, d] and a contiguous table [vocab, width] of one dtype")
    f = _func("activation.cu", "lmsf_gelu_mul_gather",
              [c_void_p, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    rc = f(_ptr(out), _ptr(a), a.stride(0), _ptr(table), table.shape[1], int(offset), _i32(ids, "ids"), table.shape[0], n, d,
           dtype_code(out.dtype), _i32(error_flag, "error_flag"), _stream())
    _check(rc, "activation.cu", "lmsf_activation")


def scale_softcap_(x: torch.Tensor, scale: float = 1.0, cap: float = 0.0):
    """x <- cap * tanh(x * scale / cap) in place (cap 0: x * scale); x: contiguous float32."""
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("scale_softcap: x must be contiguous float32")
    f = _func("activation.cu", "lmsf_scale_softcap", [c_void_p, c_longlong, c_float, c_float, c_void_p])
    rc = f(_ptr(x), x.numel(), float(scale), float(cap or 0.0), _stream())
    _check(rc, "activation.cu", "lmsf_activation")


def bias_add(x: torch.Tensor, bias: torch.Tensor):
    """x[t, :] += bias in place (sum in float32); x: [n, d] with a contiguous last dimension, bias: [d] of x's dtype."""
    n, d = x.shape
    if bias.shape != (d,) or bias.dtype != x.dtype or x.stride(1) != 1 or not bias.is_contiguous():
        raise KernelError(f"bias_add: x {tuple(x.shape)} / {x.dtype} and bias {tuple(bias.shape)} / {bias.dtype} do not match")
    f = _func("activation.cu", "lmsf_bias_add", [c_void_p, c_void_p, c_int, c_int, c_longlong, c_int, c_void_p])
    rc = f(_ptr(x), _ptr(bias), n, d, x.stride(0), dtype_code(x.dtype), _stream())
    _check(rc, "activation.cu", "lmsf_activation")


# ----------------------------------------------------------------------------- SIMT matrix product

def gemm_tn_simt(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor):
    """out[M, N] = a[M, K] w[N, K]^T, float32 FMA accumulation in ascending k (true 32-bit when a, w are float32)."""
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N) or a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError(f"gemm: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    if a.dtype != w.dtype:
        raise KernelError("gemm: a and w must share one dtype")
    f = _func("gemm_simt.cu", "lmsf_gemm_tn_simt",
              [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int, c_int,
               c_void_p])
    rc = f(_ptr(out), _ptr(a), _ptr(w), M, N, K, a.stride(0), w.stride(0), out.stride(0), dtype_code(a.dtype),
           dtype_code(out.dtype), _stream())
    _check(rc, "gemm_simt.cu", "lmsf_gemm_simt")


# ----------------------------------------------------------------------------- weight-streaming product (M <= 16)

SKINNY_MAX_M = 16
# build-time constants of gemm_skinny.cu; experiments override them, e.g. LMSF_SKINNY_DEFINES=LMSF_SKINNY_STAGES=5
SKINNY_DEFINES: Tuple[str, ...] = tuple(d for d in os.environ.get("LMSF_SKINNY_DEFINES", "").split(",") if d)


def gemm_skinny_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and 0 < x.shape[0] <= SKINNY_MAX_M
            and x.shape[1] % 8 == 0 and x.stride(1) == 1 and w.stride(1) == 1 and w.stride(0) % 8 == 0
            and x.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0 and x.data_ptr() % 16 == 0)


def _prenorm_args(prenorm, M: int, what: str):
    """(sums of squares [>= M, parts] float32, eps, width) of a prenormed input -> the kernel's five arguments."""
    if prenorm is None:
        return None, 0, 0, 0.0, 0
    sumsq, eps, width = prenorm
    if sumsq.dtype != torch.float32 or sumsq.dim() != 2 or sumsq.shape[0] < M or sumsq.stride(1) != 1:
        raise KernelError(f"{what}: the sums of squares must be float32 [rows, parts]")
    return _ptr(sumsq), sumsq.shape[1], sumsq.stride(0), float(eps), int(width)


def gemm_skinny(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, fuse_act: Optional[str] = None, prenorm=None):
    """out[M, N] = x[M, K] w[N, K]^T for M <= 16 (bfloat16 in, bfloat16 or float32 out).  With fuse_act
    ("silu", "gelu_tanh") w is [2 N_out, K] (gate rows, then up rows) and out[M, N_out] = act(x gate^T) * (x up^T).
    prenorm = (sumsq, eps, width): x is a residual stream times a norm weight and the sums of row m are multiplied by
    1 / sqrt(sum(sumsq[m]) / width + eps) first (what `gemm_skinny_residual` leaves)."""
    M, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if fuse_act else N
    if not gemm_skinny_supported(x, w) or w.shape[1] != K or out.shape != (M, n_out) or out.stride(1) != 1:
        raise KernelError(f"gemm_skinny: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} are not taken")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("gemm_skinny: out must be bfloat16 or float32")
    if fuse_act is not None and fuse_act not in ACT_CODES:
        raise KernelError(f"gemm_skinny: unknown activation {fuse_act!r}")
    f = _func("gemm_skinny.cu", "lmsf_gemm_skinny",
              [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int, c_int,
               c_void_p, c_int, c_longlong, c_float, c_int, c_void_p], SKINNY_DEFINES)
    rc = f(_ptr(out), _ptr(x), _ptr(w), M, N, K, x.stride(0), w.stride(0), out.stride(0),
           ACT_CODES[fuse_act] if fuse_act else -1, int(out.dtype == torch.float32),
           *_prenorm_args(prenorm, M, "gemm_skinny"), _stream())
    _check(rc, "gemm_skinny.cu", "lmsf_gemm_skinny", SKINNY_DEFINES)


def gemm_skinny_residual_parts(n: int) -> int:
    """Partial sums of squares per row that `gemm_skinny_residual` leaves for n output features."""
    return (n + 15) // 16


def gemm_skinny_residual(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, res: torch.Tensor, norm_w: torch.Tensor,
                         sumsq: torch.Tensor):
    """A product, the residual add after it and the first half of the RMSNorm after that, for M <= 16 rows:
    res[M, N] (float32) += bfloat16(x w^T); out[M, N] (bfloat16) = res * norm_w; sumsq[m, b] = the sum of squares of
    row m's new residual values 16 b .. 16 b + 15.  `gemm_skinny(..., prenorm=(sumsq, eps, N))` is the other half."""
    M, K = x.shape
    N = w.shape[0]
    if not gemm_skinny_supported(x, w) or w.shape[1] != K or out.shape != (M, N) or out.stride(1) != 1 or out.dtype != torch.bfloat16:
        raise KernelError(f"gemm_skinny_residual: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} are not taken")
    if res.dtype != torch.float32 or res.shape != (M, N) or res.stride(1) != 1:
        raise KernelError("gemm_skinny_residual: the residual must be float32 of the output's shape")
    if norm_w.shape != (N,) or not norm_w.is_contiguous() or norm_w.dtype not in (torch.float32, torch.bfloat16):
        raise KernelError("gemm_skinny_residual: the norm weight must be [N], float32 or bfloat16")
    if (sumsq.dtype != torch.float32 or sumsq.dim() != 2 or sumsq.shape[0] < M or sumsq.stride(1) != 1
            or sumsq.shape[1] != gemm_skinny_residual_parts(N)):
        raise KernelError("gemm_skinny_residual: the sums of squares must be float32 [rows, gemm_skinny_residual_parts(N)]")
    f = _func("gemm_skinny.cu", "lmsf_gemm_skinny_residual",
              [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int, c_void_p, c_longlong,
               c_void_p, c_int, c_void_p, c_longlong, c_void_p], SKINNY_DEFINES)
    rc = f(_ptr(out), out.stride(0), _ptr(x), x.stride(0), _ptr(w), w.stride(0), M, N, K, _ptr(res), res.stride(0),
           _ptr(norm_w), int(norm_w.dtype == torch.float32), _ptr(sumsq), sumsq.stride(0), _stream())
    _check(rc, "gemm_skinny.cu", "lmsf_gemm_skinny", SKINNY_DEFINES)


def gemm_skinny_qkv_rope_supported(x: torch.Tensor, w: torch.Tensor, head_dim: int, rot_dim: int, is_neox: bool) -> bool:
    return (gemm_skinny_supported(x, w) and head_dim % 16 == 0
            and (rot_dim == 0 or (rot_dim % 16 == 0 if is_neox else rot_dim % 2 == 0)))


def gemm_skinny_qkv_rope(q_out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, positions: torch.Tensor, token_seq: torch.Tensor,
                         block_table: torch.Tensor, block_size: int, cache: torch.Tensor, inv_freq: Optional[torch.Tensor],
                         rot_dim: int, is_neox: bool, n_q_heads: int, n_kv_heads: int, head_dim: int,
                         error_flag: Optional[torch.Tensor] = None, prenorm=None):
    """The merged q, k, v projection of up to 16 single tokens (x [M, K] bfloat16, w [(heads + 2 kv heads) * head_dim, K])
    with the rotary encoding and the cache write in its epilogue: q_out [M, heads * head_dim] gets the rotated q, the
    pages of `cache` the rotated k and v.  The same values as gemm_skinny followed by rope_cache_write.  prenorm: as in
    `gemm_skinny`."""
    M, K = x.shape
    if (not gemm_skinny_qkv_rope_supported(x, w, head_dim, rot_dim if inv_freq is not None else 0, is_neox)
            or w.shape != ((n_q_heads + 2 * n_kv_heads) * head_dim, K) or q_out.shape != (M, n_q_heads * head_dim)
            or q_out.dtype != torch.bfloat16 or q_out.stride(1) != 1):
        raise KernelError(f"gemm_skinny_qkv_rope: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(q_out.shape)} are not taken")
    if not cache.is_contiguous() or tuple(cache.shape[1:]) != (2, n_kv_heads, block_size, head_dim) or cache.dtype != torch.bfloat16:
        raise KernelError(f"gemm_skinny_qkv_rope: cache of shape {tuple(cache.shape)} does not match the heads")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_dim // 2):
        raise KernelError("gemm_skinny_qkv_rope: inv_freq must be float32 [rot_dim / 2]")
    f = _func("gemm_skinny.cu", "lmsf_gemm_skinny_qkv_rope",
              [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p,
               c_int, c_int, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
               c_void_p, c_int, c_longlong, c_float, c_int, c_void_p], SKINNY_DEFINES)
    rc = f(_ptr(q_out), q_out.stride(0), _ptr(x), x.stride(0), _ptr(w), w.stride(0), M, K, _i32(positions, "positions"),
           _i32(token_seq, "token_seq"), _i32(block_table, "block_table"), block_table.shape[1], block_size, _ptr(cache),
           cache.stride(0), _ptr(inv_freq) if inv_freq is not None else None, int(rot_dim), int(bool(is_neox)), n_q_heads,
           n_kv_heads, head_dim, _i32(error_flag, "error_flag"), *_prenorm_args(prenorm, M, "gemm_skinny_qkv_rope"), _stream())
    _check(rc, "gemm_skinny.cu", "lmsf_gemm_skinny", SKINNY_DEFINES)


# ----------------------------------------------------------------------------- the device's error word

_ERROR_WORDS = {}


def error_word(device) -> torch.Tensor:
    """The int32 word of a device in which kernels report errors that they cannot return (a wait that ran out,
    an id outside a table); the model runner reads and clears it after a step."""
    key = torch.device(device).index or 0
    w = _ERROR_WORDS.get(key)
    if w is None:
        w = _ERROR_WORDS[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return w


# ----------------------------------------------------------------------------- sampling

def sample(out: torch.Tensor, logits: torch.Tensor, temperature: Optional[torch.Tensor] = None,
           seed: Optional[torch.Tensor] = None, step: Optional[torch.Tensor] = None):
    """out[r] = greedy or temperature sample of logits[r] (float32).  temperature [rows] float32,
    seed [rows] int64 (bit pattern of an unsigned 64-bit seed), step [rows] int32; all None: greedy."""
    rows, vocab = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 with a contiguous last dimension")
    if out.dtype != torch.int32 or out.shape != (rows,) or not out.is_contiguous():
        raise KernelError("sample: out must be int32 [rows]")
    if temperature is not None and (temperature.dtype != torch.float32 or temperature.shape != (rows,)):
        raise KernelError("sample: temperature must be float32 [rows]")
    if seed is not None and (seed.dtype != torch.int64 or seed.shape != (rows,)):
        raise KernelError("sample: seed must be int64 [rows]")
    parts = 1 if vocab < 16384 else min(32, max(1, vocab // 8192))
    scratch = torch.empty(rows * parts * 2, dtype=torch.float64, device=logits.device) if parts > 1 else None
    f = _func("sampling.cu", "lmsf_sample",
              [c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p])
    rc = f(_ptr(out), _ptr(logits), logits.stride(0), rows, vocab, _ptr(temperature), _ptr(seed), _i32(step, "step"),
           parts, _ptr(scratch), _stream())
    _check(rc, "sampling.cu", "lmsf_sampling")
    if parts > 1:
        add_launches(1)


def apply_penalties(logits: torch.Tensor, rows: torch.Tensor, tokens: torch.Tensor, out_counts: torch.Tensor,
                    presence: torch.Tensor, frequency: torch.Tensor, repetition: torch.Tensor):
    """In place on float32 logits [n_rows, vocab]: for every listed (row, token) pair the repetition, frequency
    and presence penalties of that row; out_counts is how often the token occurs in the row's output so far
    (0: it occurs in the prompt only).  presence / frequency / repetition: float32 [n_rows]."""
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("apply_penalties: logits must be float32 with a contiguous last dimension")
    n = rows.numel()
    for t in (presence, frequency, repetition):
        if t.dtype != torch.float32 or t.shape != (logits.shape[0],):
            raise KernelError("apply_penalties: per-row penalties must be float32 [n_rows]")
    f = _func("sampling.cu", "lmsf_apply_penalties",
              [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    rc = f(_ptr(logits), logits.stride(0), _i32(rows, "rows"), _i32(tokens, "tokens"), _i32(out_counts, "out_counts"),
           n, _ptr(presence), _ptr(frequency), _ptr(repetition), _stream())
    _check(rc, "sampling.cu", "lmsf_sampling")


def sample_filtered(out: torch.Tensor, logits: torch.Tensor, temperature: torch.Tensor, seed: torch.Tensor,
                    step: torch.Tensor, top_k: Optional[torch.Tensor], top_p: Optional[torch.Tensor],
                    min_p: Optional[torch.Tensor], row_ids: Optional[torch.Tensor] = None):
    """Temperature sampling of the rows in row_ids (None: all) among the tokens kept by top_k (int32, <= 0 off),
    top_p (float32, 1 off) and min_p (float32, 0 off); per-row arrays are indexed by row."""
    rows, vocab = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or out.dtype != torch.int32 or out.shape != (rows,):
        raise KernelError("sample_filtered: logits float32 [rows, vocab], out int32 [rows]")
    n = rows if row_ids is None else row_ids.numel()
    f = _func("sampling.cu", "lmsf_sample_filtered",
              [c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
               c_void_p, c_void_p])
    rc = f(_ptr(out), _ptr(logits), logits.stride(0), n, vocab, _ptr(temperature), _ptr(seed), _i32(step, "step"),
           _i32(top_k, "top_k"), _ptr(top_p), _ptr(min_p), _i32(row_ids, "row_ids"), _stream())
    _check(rc, "sampling.cu", "lmsf_sampling")


# ----------------------------------------------------------------------------- tensor-core attention (bfloat16)

MMA_MAX_HEAD_DIM = 256


def mma_attention_supported(dtype: torch.dtype, head_dim: int) -> bool:
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= MMA_MAX_HEAD_DIM


MMA_KV_STAGES = None   # pipeline depth of the attention kernels, a build-time constant of attention_mma.cu (None: its own choice)


def _mma_defines(head_dim: int) -> Tuple[str, ...]:
    if MMA_KV_STAGES is None:
        return (f"LMSF_HEAD_DIM={head_dim}",)
    return (f"LMSF_HEAD_DIM={head_dim}", f"LMSF_KV_STAGES={MMA_KV_STAGES}")


def _check_paged(q, out, cache, n_q_heads, n_kv_heads, head_dim, block_size, what, kv_planes=2):
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError(f"{what}: bfloat16 only")
    if q.stride(1) != 1 or out.stride(1) != 1 or q.shape[1] != n_q_heads * head_dim or out.shape != q.shape:
        raise KernelError(f"{what}: q and out must be [n, heads * head_dim] with a contiguous last dimension")
    if kv_planes not in (1, 2) or not cache.is_contiguous() or \
            tuple(cache.shape[1:]) != (kv_planes, n_kv_heads, block_size, head_dim):
        raise KernelError(f"{what}: cache of shape {tuple(cache.shape)} does not match the heads")
    if (q.data_ptr() | out.data_ptr()) % 4 or (q.stride(0) | out.stride(0)) % 2 or cache.data_ptr() % 16:
        raise KernelError(f"{what}: q/out rows must be 4-byte aligned and the cache 16-byte aligned")




def _score_extras(n_q_heads: int, chunk, log_bias, sinks, keep_first=0, sigmoid=False, head_bias=None):
    """(chunk, r1, r2, sinks, keep_first, sigmoid, head_bias) as the tensor-core attention kernels take them: what a design
    adds to the causal softmax.  chunk > 0: a query at position p sees the keys p - p % chunk .. p only.  log_bias (r1, r2),
    float32 [n_q_heads] each: r1 * log(1 + r2 * distance) is taken off the scaled scores.  sinks, float32 [n_q_heads]:
    exp(sink) is one more term of the softmax's denominator.  keep_first (with a window): the request's first keys stay
    visible behind it.  sigmoid: a visible key's weight is sigmoid(score), not normalised.  head_bias, float32 [n_q_heads]:
    added to the scaled scores."""
    _per_head(head_bias, n_q_heads, "the bias per head")
    r1, r2 = log_bias if log_bias is not None else (None, None)
    _per_head(r1, n_q_heads, "the logarithmic bias")
    _per_head(r2, n_q_heads, "the logarithmic bias")
    _per_head(sinks, n_q_heads, "sinks")
    if chunk is not None and int(chunk) < 0:
        raise KernelError(f"attention: a chunk of {chunk} positions")
    return int(chunk or 0), _ptr(r1), _ptr(r2), _ptr(sinks), int(keep_first or 0), 1 if sigmoid else 0, _ptr(head_bias)


_DECODE_WIDTHS = {}


def decode_widths(head_dim: int, group: int = 1) -> Tuple[Tuple[int, float, Tuple[int, ...]], ...]:
    """The widths a decode block comes in, widest first; for each: its warps, the rate at which one block streams
    keys (its bytes in flight, in units of 64 KB) and, for cluster sizes 1..8, how many clusters of that many blocks
    the device holds at a time (it depends on the group of query heads per kv head, which sizes a block's shared
    memory).  Head sizes up to 64 have one width: four of its blocks fit an SM anyway."""
    key = (head_dim, min(16, max(1, group)))
    t = _DECODE_WIDTHS.get(key)
    if t is None:
        lib = load_library("attention_mma.cu", _mma_defines(head_dim))
        lib.lmsf_attention_decode_max_clusters.restype = c_int
        lib.lmsf_attention_decode_max_clusters.argtypes = [c_int, c_int, c_int]
        lib.lmsf_attention_decode_stream_bytes.restype = c_int
        lib.lmsf_attention_decode_stream_bytes.argtypes = [c_int]
        widths = []
        for warps in ((4,) if head_dim <= 64 else (4, 2)):
            clusters = tuple(max(1, lib.lmsf_attention_decode_max_clusters(s, key[1], warps)) for s in range(1, 9))
            widths.append((warps, lib.lmsf_attention_decode_stream_bytes(warps) / 65536.0, clusters))
        t = _DECODE_WIDTHS[key] = tuple(widths)
    return t


# The cost model of decode_plan, in units of the time in which a block with 64 KB in flight streams 32 KB (about
# 1.5 us on B200); fitted to B200 measurements of 8 and 40 kv heads, 2,048 to 8,000 keys, 16 to 128 requests, both
# widths, 1 to 8 splits, alone and inside decode steps.
DECODE_WAVE_COST = 6.0          # what a wave of blocks costs before and after its keys
DECODE_SPLIT_COST = 4.0         # adding the splits of a request up
DECODE_GLOBAL_MERGE_COST = 6.0  # more when more than 8 splits add up through global memory
DECODE_SATURATION = 240.0       # blocks with 64 KB in flight that saturate the memory
DECODE_BLOCK_COST = 1.3         # what a block costs the slot it runs in, beside its keys (tables, first loads, its part of the sum)
DECODE_MUST_GAIN = 0.95         # a narrower block or a further split is taken when the model gives it 5 % less


def decode_plan(n_served: int, n_kv_heads: int, group: int, max_ctx: int, head_dim: int,
                widths: Sequence[Tuple[int, float, Sequence[int]]], mean_ctx: Optional[float] = None) -> Tuple[int, int]:
    """(splits, warps): into how many blocks the keys of a request are split, and how wide the blocks are.  Up to 8
    splits form a thread-block cluster (they add up through its shared memory) and clusters[s - 1] such clusters
    run at a time; more splits add up through global memory.  The choice minimises the sum over the waves of
    (fixed cost + keys per split / rate), where a block streams at the rate of its own bytes in flight or, when more
    blocks are resident than saturate the memory, at its share of the device: few long requests want wide blocks
    and many splits, many requests narrow blocks, of which twice as many are resident, and no second, partly filled
    wave.  Every split keeps at least 128 keys.  mean_ctx: the requests' mean number of keys, when it is far below
    max_ctx (one long request among short ones): every request gets the same number of splits, so the longest one
    sets the time of a wave unless it is split as if it were nearly alone; the short requests' extra blocks find
    no keys and cost only their slots (64 requests of the 8B shape, one with 30,000 keys among 63 with 500, took
    0.8 ms a layer planned for 64 requests of 30,000 keys, the long request's 8 blocks streaming alone).  Measured on B200 (head size 128, 8 kv heads, 2,048 keys):
    5 requests take 20.5 us with 6 splits (45 clusters fit) and 30.7 us with 7 (37 fit); 48 requests 100 us at best
    with wide blocks (2 splits) and 95 us with narrow ones (1 split); a decode step of 20 requests 4.72 ms with wide
    blocks and one split, 4.42 ms with narrow ones and 3."""
    per_request = n_kv_heads * ((group + 15) // 16)
    n_blocks1 = n_served * per_request                            # blocks of the launch per split
    # the requests that matter for the time of a wave: all of them, or as many as would hold the keys at max_ctx each
    work_served = n_served if not mean_ctx else max(1, min(n_served, -(-int(n_served * mean_ctx) // max(1, max_ctx))))
    base = work_served * per_request
    tiles = -(-max_ctx // 64)
    cap = max(1, -(-max_ctx // 128))
    tile_work = head_dim / 128.0                  # a 64-key tile of k and v in units of 32 KB
    best = None
    for warps, rate, clusters in widths:
        slots = clusters[0]
        for s in list(range(1, 9)) + [12, 16, 24, 32, 48, 64]:
            if s > cap:
                break
            per_wave = clusters[s - 1] if s <= 8 else max(1, slots // s)      # (request, head group) pairs per wave
            work = -(-tiles // s) * tile_work
            cost = (DECODE_SPLIT_COST if s > 1 else 0.0) + (DECODE_GLOBAL_MERGE_COST if s > 8 else 0.0)
            cost += DECODE_BLOCK_COST * n_blocks1 * s / (per_wave * s)
            left = base
            while left > 0:
                n = min(left, per_wave) * s
                cost += DECODE_WAVE_COST + work / min(rate, DECODE_SATURATION / n)
                left -= per_wave
            # candidates come widest first and with few splits first; a later one must be better by 5 %: measured,
            # near-ties of the model go to either side by a per cent, and wide blocks with few splits never lose more
            if best is None or cost < best[0] * DECODE_MUST_GAIN:
                best = (cost, s, warps)
    return best[1], best[2]


DECODE_COUNTER_SLOTS = 65536     # counters of delivered splits at the start of the scratch (attention_mma.cu)


def attention_decode_scratch_floats(n_seqs_total: int, n_q_heads: int, n_splits: int, head_dim: int) -> int:
    return 0 if n_splits <= 1 else DECODE_COUNTER_SLOTS + n_seqs_total * n_q_heads * n_splits * (head_dim + 1)


def attention_decode(out: torch.Tensor, q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                     block_size: int, seq_ids: Optional[torch.Tensor], n_served: int, cu_q: torch.Tensor,
                     ctx_len: torch.Tensor, scale: float, window: int, n_q_heads: int, n_kv_heads: int,
                     head_dim: int, n_splits: int, scratch: Optional[torch.Tensor], warps: int = 0, kv_planes: int = 2,
                     chunk: int = 0, log_bias=None, sinks: Optional[torch.Tensor] = None, keep_first: int = 0,
                     sigmoid: bool = False, head_bias: Optional[torch.Tensor] = None):
    """Attention of requests that bring ONE query token each (row cu_q[s] of q), over their ctx_len[s] keys
    in pages.  seq_ids: int32 [n_served] rows of the block table that are served (None: all, in order).
    scratch: float32, at least attention_decode_scratch_floats(...) values when n_splits > 1, all zero when it is
    first used (torch.zeros); the kernel leaves its counters zero, so one buffer serves every later call.
    warps: the width of the blocks, 4 or 2 (decode_plan chooses it with n_splits); 0 leaves it to the kernel.
    kv_planes 1: the cache holds one vector per token and kv head that is key and value at once.
    chunk, log_bias, sinks: see _score_extras."""
    _check_paged(q, out, cache, n_q_heads, n_kv_heads, head_dim, block_size, "attention_decode", kv_planes)
    extras = _score_extras(n_q_heads, chunk, log_bias, sinks, keep_first, sigmoid, head_bias)
    n_total = block_table.shape[0]
    need = attention_decode_scratch_floats(n_total, n_q_heads, n_splits, head_dim)
    if need and (scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need):
        raise KernelError(f"attention_decode: {n_splits} splits need {need} float32 values of scratch")
    d = _mma_defines(head_dim)
    if warps not in (0, 2, 4):
        raise KernelError(f"attention_decode: blocks have 2 or 4 warps, not {warps}")
    f = _func("attention_mma.cu", "lmsf_attention_decode_width",
              [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_void_p, c_int,
               c_void_p, c_int, c_int, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_void_p,
               c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p], d)
    rc = f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(cache), cache.stride(0), block_size, n_kv_heads,
           _i32(block_table, "block_table"), block_table.shape[1], _i32(seq_ids, "seq_ids"), n_served, n_total,
           _i32(cu_q, "cu_q"), _i32(ctx_len, "ctx_len"), float(scale), int(window or 0), n_q_heads, head_dim,
           n_splits, warps, _ptr(scratch) if need else None, int(kv_planes), *extras, _stream())
    _check(rc, "attention_mma.cu", "lmsf_attention_mma", d)


def decode_items_capacity(n_served: int, n_kv_heads: int, group: int, slots: int) -> int:
    """Entries of the list of work items of a launch with splits per request: one per request and as many more as
    the device holds blocks for."""
    return n_served + slots // (n_kv_heads * ((group + 15) // 16)) + 1


def attention_decode_items_scratch_floats(capacity: int, n_q_heads: int, head_dim: int) -> int:
    return DECODE_COUNTER_SLOTS + capacity * n_q_heads * (head_dim + 1)


def decode_build_items(items: torch.Tensor, ctx_len: torch.Tensor, seq_ids: Optional[torch.Tensor], n_served: int,
                       window: int, n_q_heads: int, n_kv_heads: int, head_dim: int, slots: int, chunk: int = 0):
    """Fills `items` (int32 [capacity, 4]) on the device: request s gets ceil(keys_s / T) splits, with T the smallest
    number of keys for which all blocks fit the `slots` blocks that the device holds at a time; entries that are
    left over are padding.  The attention of requests that differ much in length runs over this list
    (attention_decode_items): each block then has about the same number of keys."""
    if items.dtype != torch.int32 or items.dim() != 2 or items.shape[1] != 4 or not items.is_contiguous():
        raise KernelError("decode_build_items: items must be a contiguous int32 tensor [capacity, 4]")
    d = _mma_defines(head_dim)
    f = _func("attention_mma.cu", "lmsf_attention_decode_build_items",
              [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p], d)
    rc = f(_i32(ctx_len, "ctx_len"), _i32(seq_ids, "seq_ids"), n_served, int(window or 0), n_q_heads, n_kv_heads,
           int(slots), items.shape[0], _ptr(items), int(chunk or 0), _stream())
    _check(rc, "attention_mma.cu", "lmsf_attention_mma", d)


def attention_decode_items(out: torch.Tensor, q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                           block_size: int, items: torch.Tensor, cu_q: torch.Tensor, ctx_len: torch.Tensor,
                           scale: float, window: int, n_q_heads: int, n_kv_heads: int, head_dim: int, warps: int,
                           scratch: torch.Tensor, kv_planes: int = 2, chunk: int = 0, log_bias=None,
                           sinks: Optional[torch.Tensor] = None, keep_first: int = 0,
                           sigmoid: bool = False, head_bias: Optional[torch.Tensor] = None):
    """attention_decode with splits per request, over a list made by decode_build_items.  scratch: float32, at
    least attention_decode_items_scratch_floats(capacity, ...) values, zero when first used."""
    _check_paged(q, out, cache, n_q_heads, n_kv_heads, head_dim, block_size, "attention_decode_items", kv_planes)
    extras = _score_extras(n_q_heads, chunk, log_bias, sinks, keep_first, sigmoid, head_bias)
    need = attention_decode_items_scratch_floats(items.shape[0], n_q_heads, head_dim)
    if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
        raise KernelError(f"attention_decode_items: a list of {items.shape[0]} entries needs {need} float32 values of scratch")
    d = _mma_defines(head_dim)
    f = _func("attention_mma.cu", "lmsf_attention_decode_items",
              [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_void_p, c_int,
               c_void_p, c_int, c_int, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_void_p, c_int,
               c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p], d)
    rc = f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(cache), cache.stride(0), block_size, n_kv_heads,
           _i32(block_table, "block_table"), block_table.shape[1], _ptr(items), items.shape[0], block_table.shape[0],
           _i32(cu_q, "cu_q"), _i32(ctx_len, "ctx_len"), float(scale), int(window or 0), n_q_heads, head_dim, int(warps),
           _ptr(scratch), int(kv_planes), *extras, _stream())
    _check(rc, "attention_mma.cu", "lmsf_attention_mma", d)


def attention_prefill(out: torch.Tensor, q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                      block_size: int, tile_seq: torch.Tensor, tile_q0: torch.Tensor, n_tiles: int, cu_q: torch.Tensor,
                      ctx_len: torch.Tensor, scale: float, window: int, n_q_heads: int, n_kv_heads: int, head_dim: int,
                      kv_planes: int = 2, chunk: int = 0, log_bias=None, sinks: Optional[torch.Tensor] = None, keep_first: int = 0,
                      sigmoid: bool = False, head_bias: Optional[torch.Tensor] = None):
    """Attention of prompt portions.  Tile i covers the query tokens tile_q0[i] .. tile_q0[i] + 63 (counted
    inside the portion) of request tile_seq[i]."""
    _check_paged(q, out, cache, n_q_heads, n_kv_heads, head_dim, block_size, "attention_prefill", kv_planes)
    extras = _score_extras(n_q_heads, chunk, log_bias, sinks, keep_first, sigmoid, head_bias)
    d = _mma_defines(head_dim)
    f = _func("attention_mma.cu", "lmsf_attention_prefill",
              [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_void_p, c_int,
               c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int,
               c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p], d)
    rc = f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(cache), cache.stride(0), block_size, n_kv_heads,
           _i32(block_table, "block_table"), block_table.shape[1], _i32(tile_seq, "tile_seq"),
           _i32(tile_q0, "tile_q0"), n_tiles, _i32(cu_q, "cu_q"), _i32(ctx_len, "ctx_len"), float(scale),
           int(window or 0), n_q_heads, head_dim, int(kv_planes), *extras, _stream())
    _check(rc, "attention_mma.cu", "lmsf_attention_mma", d)


# ----------------------------------------------------------------------------- tcgen05 prefill attention

TC_HEAD_DIMS = (64, 128)
TC_Q_TILE = 128


def tc_attention_supported(dtype: torch.dtype, head_dim: int) -> bool:
    return dtype == torch.bfloat16 and head_dim in TC_HEAD_DIMS


def attention_prefill_tc(out: torch.Tensor, q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                         block_size: int, tile_seq: torch.Tensor, tile_q0: torch.Tensor, n_tiles: int, cu_q: torch.Tensor,
                         ctx_len: torch.Tensor, scale: float, window: int, n_q_heads: int, n_kv_heads: int, head_dim: int,
                         error_flag: Optional[torch.Tensor] = None, kv_planes: int = 2, chunk: int = 0, log_bias=None,
                         sinks: Optional[torch.Tensor] = None, keep_first: int = 0,
                         sigmoid: bool = False, head_bias: Optional[torch.Tensor] = None):
    """Attention of prompt portions on tcgen05 tensor cores (head size 64 or 128).  Tile i covers the query
    tokens tile_q0[i] .. tile_q0[i] + 127 (counted inside the portion) of request tile_seq[i]."""
    _check_paged(q, out, cache, n_q_heads, n_kv_heads, head_dim, block_size, "attention_prefill_tc", kv_planes)
    extras = _score_extras(n_q_heads, chunk, log_bias, sinks, keep_first, sigmoid, head_bias)
    d = _mma_defines(head_dim)[:1]
    f = _func("attention_tc.cu", "lmsf_attention_prefill_tc",
              [c_void_p, c_longlong, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_longlong, c_int, c_int,
               c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_void_p,
               c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p], d)
    rc = f(_ptr(q), q.stride(0), q.shape[0], _ptr(out), out.stride(0), _ptr(cache), cache.stride(0), cache.shape[0], block_size,
           n_kv_heads, _i32(block_table, "block_table"), block_table.shape[1], _i32(tile_seq, "tile_seq"),
           _i32(tile_q0, "tile_q0"), n_tiles, _i32(cu_q, "cu_q"), _i32(ctx_len, "ctx_len"), float(scale),
           int(window or 0), n_q_heads, head_dim, _i32(error_flag, "error_flag"), int(kv_planes), *extras, _stream())
    _check(rc, "attention_tc.cu", "lmsf_attention_tc", d)


# ----------------------------------------------------------------------------- norms around a float32 residual stream

def _f32vec(t: Optional[torch.Tensor], n: int, name: str) -> Optional[int]:
    if t is None:
        return None
    if t.dtype != torch.float32 or t.shape != (n,) or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous float32 vector of {n} values")
    return _ptr(t)


def stream_norm(res: torch.Tensor, y: Optional[torch.Tensor] = None, w_post: Optional[torch.Tensor] = None,
                layer_scale: Optional[torch.Tensor] = None, eps_post: float = 0.0, first: Optional[torch.Tensor] = None,
                vec: Optional[torch.Tensor] = None, h: Optional[torch.Tensor] = None, w_next: Optional[torch.Tensor] = None,
                eps_next: float = 0.0, branch_scale: float = 1.0):
    """What lies between two branches of a block that norms a branch before and after it, in one kernel, float32 inside:
    res += branch_scale * norm(y) * w_post * layer_scale (if y); res += first + vec (whichever is given);
    h = norm(res) * w_next (if h; without w_next h is the stream itself in the activation type).
    res, first: float32 [n, hidden]; y, h: [n, hidden] of the activation type; the vectors are float32 [hidden]."""
    n, hidden = res.shape
    if res.dtype != torch.float32 or not res.is_contiguous():
        raise KernelError("stream_norm: the residual stream must be contiguous float32")
    act = y if y is not None else h
    for name, t in (("y", y), ("h", h)):
        if t is not None and (t.shape != res.shape or not t.is_contiguous() or t.dtype != act.dtype):
            raise KernelError(f"stream_norm: {name} must be contiguous, of the stream's shape and of one activation type")
    if first is not None and (first.dtype != torch.float32 or first.shape != res.shape or not first.is_contiguous()):
        raise KernelError("stream_norm: `first` must be contiguous float32 of the stream's shape")
    if act is None and first is None and vec is None:
        return
    f = _func("stream_norm.cu", "lmsf_stream_norm",
              [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float,
               c_float, c_float, c_int, c_void_p])
    rc = f(_ptr(res), _ptr(y), _f32vec(w_post, hidden, "w_post"), _f32vec(layer_scale, hidden, "layer_scale"), _ptr(first),
           _f32vec(vec, hidden, "vec"), _ptr(h), _f32vec(w_next, hidden, "w_next"), n, hidden, float(eps_post),
           float(eps_next), float(branch_scale), dtype_code(act.dtype) if act is not None else F32, _stream())
    _check(rc, "stream_norm.cu", "lmsf_stream_norm")


def gated_branches(res: torch.Tensor, z: torch.Tensor, bias: Optional[torch.Tensor], y1: torch.Tensor,
                   y2: Optional[torch.Tensor] = None, h: Optional[torch.Tensor] = None, w_next: Optional[torch.Tensor] = None,
                   eps_next: float = 0.0):
    """res += sigmoid(z[:, :D] + bias[:D]) * y1 + sigmoid(z[:, D:] + bias[D:]) * y2 (y2 may be None), then h = norm(res) *
    w_next if h is given; one kernel, float32 inside.  res: float32 [n, D]; z: float32 [n, D or 2 D] (last dimension
    contiguous); bias: float32 of z's width; y1, y2, h: contiguous [n, D] of the activation type."""
    n, hidden = res.shape
    width = (2 if y2 is not None else 1) * hidden
    if res.dtype != torch.float32 or not res.is_contiguous():
        raise KernelError("gated_branches: the residual stream must be contiguous float32")
    if z.dtype != torch.float32 or z.shape != (n, width) or z.stride(1) != 1:
        raise KernelError(f"gated_branches: the gate logits must be float32 [n, {width}]")
    for name, t in (("y1", y1), ("y2", y2), ("h", h)):
        if t is not None and (t.shape != res.shape or not t.is_contiguous() or t.dtype != y1.dtype):
            raise KernelError(f"gated_branches: {name} must be contiguous, of the stream's shape and of one activation type")
    f = _func("stream_norm.cu", "lmsf_gated_branches",
              [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int,
               c_void_p])
    rc = f(_ptr(res), _ptr(z), z.stride(0), _f32vec(bias, width, "bias"), _ptr(y1), _ptr(y2), _ptr(h),
           _f32vec(w_next, hidden, "w_next"), n, hidden, float(eps_next), dtype_code(y1.dtype), _stream())
    _check(rc, "stream_norm.cu", "lmsf_stream_norm")


def token_shift(out: torch.Tensor, h: torch.Tensor, mix: torch.Tensor, state: torch.Tensor, positions: torch.Tensor,
                token_seq: torch.Tensor, cu_q: torch.Tensor, state_slot: torch.Tensor):
    """out[t] = h[t] + (h[t - 1] - h[t]) * mix; h[t - 1] is zero for a request's first token and comes from `state`
    (float32 [slots, hidden], which then receives the portion's last row) for a portion's first token."""
    n, hidden = h.shape
    if out.shape != h.shape or out.dtype != h.dtype or not (out.is_contiguous() and h.is_contiguous()) or out.data_ptr() == h.data_ptr():
        raise KernelError("token_shift: out and h must be different contiguous tensors of one shape and dtype")
    if state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] != hidden or not state.is_contiguous():
        raise KernelError("token_shift: the state must be contiguous float32 [slots, hidden]")
    f = _func("stream_norm.cu", "lmsf_token_shift",
              [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    rc = f(_ptr(out), _ptr(h), _f32vec(mix, hidden, "mix"), _ptr(state), _i32(positions, "positions"),
           _i32(token_seq, "token_seq"), _i32(cu_q, "cu_q"), _i32(state_slot, "state_slot"), n, hidden, dtype_code(h.dtype), _stream())
    _check(rc, "stream_norm.cu", "lmsf_stream_norm")


def stream_concat(out: torch.Tensor, a: torch.Tensor, b: torch.Tensor):
    """out = [a | b] in out's type: two float32 streams [n, D] side by side, [n, 2 D]."""
    n, hidden = a.shape
    if a.dtype != torch.float32 or b.dtype != torch.float32 or b.shape != a.shape or out.shape != (n, 2 * hidden) or \
            not (a.is_contiguous() and b.is_contiguous() and out.is_contiguous()):
        raise KernelError("stream_concat: two contiguous float32 streams [n, D] and out [n, 2 D]")
    f = _func("stream_norm.cu", "lmsf_stream_concat", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    rc = f(_ptr(out), _ptr(a), _ptr(b), n, hidden, dtype_code(out.dtype), _stream())
    _check(rc, "stream_norm.cu", "lmsf_stream_norm")


def stream_begin(res: torch.Tensor, x: torch.Tensor):
    """res = float(x): an embedding's output becomes the float32 residual stream."""
    if res.dtype != torch.float32 or res.shape != x.shape or not (res.is_contiguous() and x.is_contiguous()):
        raise KernelError("stream_begin: res must be contiguous float32 of x's shape")
    f = _func("stream_norm.cu", "lmsf_stream_begin", [c_void_p, c_void_p, c_longlong, c_int, c_void_p])
    rc = f(_ptr(res), _ptr(x), x.numel(), dtype_code(x.dtype), _stream())
    _check(rc, "stream_norm.cu", "lmsf_stream_norm")


def embed_norm(res: torch.Tensor, keep: Optional[torch.Tensor], table: torch.Tensor, ids: torch.Tensor, w: torch.Tensor,
               eps: float, scale: float = 1.0, error_flag: Optional[torch.Tensor] = None):
    """res[t] = norm(table[ids[t]] * scale) * w in float32 (and the same again in `keep`, if given)."""
    n, hidden = res.shape
    if res.dtype != torch.float32 or not res.is_contiguous() or table.shape[1] != hidden or not table.is_contiguous():
        raise KernelError("embed_norm: res must be contiguous float32 [n, hidden] and the table [vocab, hidden]")
    if keep is not None and (keep.dtype != torch.float32 or keep.shape != res.shape or not keep.is_contiguous()):
        raise KernelError("embed_norm: `keep` must be like res")
    f = _func("stream_norm.cu", "lmsf_embed_norm",
              [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p, c_void_p])
    rc = f(_ptr(res), _ptr(keep), _ptr(table), _i32(ids, "ids"), _f32vec(w, hidden, "w"), n, hidden, table.shape[0],
           float(eps), float(scale), dtype_code(table.dtype), _i32(error_flag, "error_flag"), _stream())
    _check(rc, "stream_norm.cu", "lmsf_stream_norm")


# ----------------------------------------------------------------------------- linear attention with a decay per head

LIGHTNING_ACTS = {None: 0, "none": 0, "silu": 1}
LIGHTNING_MAX_DK = 256


def lightning_scan(out: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, state: torch.Tensor,
                   decay: torch.Tensor, cu_q: torch.Tensor, state_slot: torch.Tensor, n_seqs: int, heads: int, dk: int,
                   dv: int, act: Optional[str] = "silu", items: Optional[torch.Tensor] = None,
                   scratch: Optional[torch.Tensor] = None, mode: int = 0):
    """Per request (tokens cu_q[s]..cu_q[s+1]) and head: S = decay S + act(k_t) act(v_t)^T, out_t = S^T act(q_t), with
    S = state[state_slot[s], head] (float32 [dk, dv]) read before and written after.  q, k: [n, heads * dk] and
    v: [n, heads * dv] views with a contiguous last dimension; out: float32 [n, heads * dv].
    items (int32 [n_items, 4]: request, first token, end token, index in scratch): the launch serves these instead of
    every request whole.  mode 1: every item from a zero state, its final state to scratch[index] (no outputs);
    mode 2: every item from the state in scratch[index], outputs only (see lightning_prefix)."""
    n = q.shape[0]
    for name, t, width in (("q", q, heads * dk), ("k", k, heads * dk), ("v", v, heads * dv)):
        if t.dim() != 2 or t.shape != (n, width) or t.stride(1) != 1 or t.dtype != q.dtype:
            raise KernelError(f"lightning: {name} must be [n, {width}] with a contiguous last dimension, of one dtype")
    if out.dtype != torch.float32 or out.shape != (n, heads * dv) or out.stride(1) != 1:
        raise KernelError("lightning: out must be float32 [n, heads * dv]")
    if state.dtype != torch.float32 or tuple(state.shape[1:]) != (heads, dk, dv) or not state.is_contiguous():
        raise KernelError(f"lightning: the state must be contiguous float32 [slots, {heads}, {dk}, {dv}]")
    if decay.dtype != torch.float32 or decay.shape != (heads,) or not decay.is_contiguous():
        raise KernelError("lightning: one float32 decay per head")
    n_items = n_seqs
    if items is not None:
        if items.dtype != torch.int32 or items.dim() != 2 or items.shape[1] != 4 or not items.is_contiguous():
            raise KernelError("lightning: items must be a contiguous int32 tensor [n_items, 4]")
        n_items = items.shape[0]
    if mode != 0 and (items is None or scratch is None or scratch.dtype != torch.float32 or not scratch.is_contiguous()
                      or tuple(scratch.shape[1:]) != (heads, dk, dv)):
        raise KernelError(f"lightning: modes 1 and 2 need items and a float32 scratch [chunks, {heads}, {dk}, {dv}]")
    f = _func("lightning.cu", "lmsf_lightning_scan",
              [c_void_p, c_void_p, c_void_p, c_longlong, c_longlong, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p,
               c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p])
    rc = f(_ptr(q), _ptr(k), _ptr(v), q.stride(0), k.stride(0), v.stride(0), _ptr(out), out.stride(0), _ptr(state),
           _ptr(decay), _i32(cu_q, "cu_q"), _i32(state_slot, "state_slot"), n_items, heads, dk, dv, LIGHTNING_ACTS[act],
           dtype_code(q.dtype), _ptr(items), _ptr(scratch), int(mode), _stream())
    _check(rc, "lightning.cu", "lmsf_lightning")


def lightning_prefix(scratch: torch.Tensor, state: torch.Tensor, decay: torch.Tensor, state_slot: torch.Tensor,
                     items: torch.Tensor, spans: torch.Tensor):
    """Between the two passes over chunks: scratch[c] (what chunk c adds from a zero state) becomes the state before chunk
    c, in the order of each request's chunks; the state after the last chunk goes to the request's slot.
    spans: int32 [n, 4] = (request, first chunk item, end chunk item, 0)."""
    heads, dk, dv = state.shape[1:]
    if spans.dtype != torch.int32 or spans.dim() != 2 or spans.shape[1] != 4 or not spans.is_contiguous():
        raise KernelError("lightning: spans must be a contiguous int32 tensor [n, 4]")
    f = _func("lightning.cu", "lmsf_lightning_prefix",
              [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    rc = f(_ptr(scratch), _ptr(state), _ptr(decay), _i32(state_slot, "state_slot"), _ptr(items), _ptr(spans), spans.shape[0],
           heads, dk, dv, _stream())
    _check(rc, "lightning.cu", "lmsf_lightning")


def gated_norm(out: torch.Tensor, x: torch.Tensor, gate: torch.Tensor, w: torch.Tensor, eps: float):
    """out = norm(x) * w * sigmoid(gate), the norm over a whole row, float32 inside.  x: float32 [n, width];
    gate: [n, width] view of the activation type; out: contiguous, of the activation type."""
    n, width = x.shape
    if x.dtype != torch.float32 or x.stride(1) != 1 or gate.shape != x.shape or gate.stride(1) != 1 or \
            out.shape != x.shape or not out.is_contiguous() or out.dtype != gate.dtype:
        raise KernelError("gated_norm: x float32 [n, width], gate and out [n, width] of the activation type")
    f = _func("lightning.cu", "lmsf_gated_norm",
              [c_void_p, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_int, c_int, c_float, c_int, c_void_p])
    rc = f(_ptr(out), _ptr(x), x.stride(0), _ptr(gate), gate.stride(0), _f32vec(w, width, "w"), n, width, float(eps),
           dtype_code(out.dtype), _stream())
    _check(rc, "lightning.cu", "lmsf_lightning")


# ----------------------------------------------------------------------------- recurrent mixers with a state matrix per head

CONV_MAX_TAPS = 8
SCAN_MAX_DK = 256


def _rows(t: torch.Tensor, width: int, name: str, dtype: Optional[torch.dtype] = None):
    if t.dim() != 2 or t.shape[1] != width or t.stride(1) != 1 or (dtype is not None and t.dtype != dtype):
        raise KernelError(f"{name} must be [n, {width}] with a contiguous last dimension" + (f" of {dtype}" if dtype else ""))


def causal_conv(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
                state_offset: int, cu_q: torch.Tensor, state_slot: torch.Tensor, n_seqs: int, max_q: int, act: str = "silu"):
    """out[t, c] = act(bias[c] + sum_j w[c, j] x[t - (taps - 1) + j, c]) per request (tokens cu_q[s]..cu_q[s + 1]); the
    inputs before a portion come from state[slot, state_offset : state_offset + (taps - 1) * C] ([taps - 1, C], float32),
    which then takes the portion's last inputs.  x, out: [n, C] views; w: float32 [C, taps]; state: float32 [slots, size]."""
    n, C = x.shape
    taps = w.shape[1]
    _rows(x, C, "causal_conv: x")
    _rows(out, C, "causal_conv: out", x.dtype)
    if out.shape[0] != n or w.dtype != torch.float32 or w.shape != (C, taps) or not w.is_contiguous():
        raise KernelError("causal_conv: w must be contiguous float32 [channels, taps]")
    if state.dtype != torch.float32 or state.dim() != 2 or not state.is_contiguous() or \
            state_offset < 0 or state_offset + (taps - 1) * C > state.shape[1]:
        raise KernelError("causal_conv: the state must be contiguous float32 [slots, size] with room for [taps - 1, channels]")
    f = _func("recurrent.cu", "lmsf_causal_conv",
              [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_int,
               c_int, c_int, c_int, c_int, c_int, c_void_p])
    rc = f(_ptr(out), out.stride(0), _ptr(x), x.stride(0), _ptr(w), _f32vec(bias, C, "bias"),
           state.data_ptr() + 4 * state_offset, state.stride(0), _i32(cu_q, "cu_q"), _i32(state_slot, "state_slot"), n_seqs,
           int(max_q), C, taps, {"none": 0, None: 0, "silu": 1}[act], dtype_code(x.dtype), _stream())
    _check(rc, "recurrent.cu", "lmsf_recurrent")


def gated_scan(out: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, dt: torch.Tensor,
               beta: Optional[torch.Tensor], dt_bias: torch.Tensor, a_log: torch.Tensor, skip: Optional[torch.Tensor],
               state: torch.Tensor, cu_q: torch.Tensor, state_slot: torch.Tensor, n_seqs: int, heads: int, qk_heads: int,
               dk: int, dv: int, delta: bool, k_times_dt: bool = False, unit_qk: bool = False, unit_eps: float = 1e-6,
               q_scale: float = 1.0):
    """Per request, head h and token: step = softplus(dt[t, h] + dt_bias[h]), a = exp(-exp(a_log[h]) * step);
    plain rule: S = a S + (step k) v^T (k v^T without k_times_dt); delta rule: S = a S, u = sigmoid(beta[t, h]) (v - S^T k),
    S += k u^T; out[t, h] = S^T q + skip[h] v.  Head h reads q/k head h // (heads / qk_heads); unit_qk makes q and k unit
    vectors first (x / sqrt(sum x^2 + unit_eps)) and multiplies q by q_scale.  S = the first heads * dv * dk values of
    state[slot] (float32 [slots, size], stored [head][dv][dk]), read before and written after.
    q, k: [n, qk_heads * dk]; v: [n, heads * dv]; dt, beta: [n, heads] (views of one dtype); out: float32 [n, heads * dv].
    Two launches: one prepares q, k and the tokens' decays in a scratch that this function allocates, one scans."""
    n = q.shape[0]
    _rows(q, qk_heads * dk, "gated_scan: q")
    _rows(k, qk_heads * dk, "gated_scan: k", q.dtype)
    _rows(v, heads * dv, "gated_scan: v", q.dtype)
    _rows(dt, heads, "gated_scan: dt", q.dtype)
    if beta is not None:
        _rows(beta, heads, "gated_scan: beta", q.dtype)
    _rows(out, heads * dv, "gated_scan: out", torch.float32)
    if state.dtype != torch.float32 or state.dim() != 2 or not state.is_contiguous() or state.shape[1] < heads * dv * dk:
        raise KernelError("gated_scan: the state must be contiguous float32 [slots, >= heads * dv * dk]")
    f = _func("recurrent.cu", "lmsf_gated_scan",
              [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_longlong, c_longlong, c_longlong, c_void_p, c_longlong,
               c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int,
               c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p, c_int, c_void_p])
    need = _func("recurrent.cu", "lmsf_gated_scan_scratch_floats", [c_int, c_int, c_int, c_int])
    need.restype = c_longlong
    scratch = torch.empty(int(need(n, heads, qk_heads, dk)), dtype=torch.float32, device=q.device)
    rc = f(_ptr(out), out.stride(0), _ptr(q), _ptr(k), _ptr(v), q.stride(0), k.stride(0), v.stride(0), _ptr(dt), dt.stride(0),
           _ptr(beta), beta.stride(0) if beta is not None else 0, _f32vec(dt_bias, heads, "dt_bias"),
           _f32vec(a_log, heads, "a_log"), _f32vec(skip, heads, "skip"), _ptr(state), state.stride(0), _i32(cu_q, "cu_q"),
           _i32(state_slot, "state_slot"), n_seqs, n, heads, qk_heads, dk, dv, int(delta), int(k_times_dt), int(unit_qk),
           float(unit_eps), float(q_scale), _ptr(scratch), dtype_code(q.dtype), _stream())
    _check(rc, "recurrent.cu", "lmsf_recurrent")
    add_launches(1)                                            # two launches: prepare and scan


def grouped_gated_norm(out: torch.Tensor, x: torch.Tensor, gate: Optional[torch.Tensor], w: torch.Tensor, group_size: int,
                       eps: float, gate_act: str = "silu", gate_first: bool = False):
    """Per group of `group_size` columns: out = x / rms(x) * w * act(gate), or with gate_first out = y / rms(y) * w for
    y = x * act(gate).  x: float32 [n, width]; gate, out: [n, width] views of the activation type; w: float32, its length
    divides into a row (a weight shorter than the row is shared by the groups)."""
    n, width = x.shape
    _rows(x, width, "grouped_gated_norm: x", torch.float32)
    _rows(out, width, "grouped_gated_norm: out")
    if gate is not None:
        _rows(gate, width, "grouped_gated_norm: gate", out.dtype)
    if width % group_size or w.dtype != torch.float32 or w.dim() != 1 or not w.is_contiguous() or width % w.numel() \
            or (w.numel() % group_size and group_size % w.numel()):
        raise KernelError("grouped_gated_norm: the groups and the weight must divide a row")
    f = _func("recurrent.cu", "lmsf_grouped_gated_norm",
              [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_float,
               c_int, c_int, c_int, c_void_p])
    rc = f(_ptr(out), out.stride(0), _ptr(x), x.stride(0), _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(w),
           w.numel(), n, width // group_size, group_size, float(eps), int(gate_act == "silu"), int(gate_first),
           dtype_code(out.dtype), _stream())
    _check(rc, "recurrent.cu", "lmsf_recurrent")


# ----------------------------------------------------------------------------- attention over a cached low-rank vector

def latent_norm_cache_write(x: torch.Tensor, w: torch.Tensor, eps: float, cache: torch.Tensor, positions: torch.Tensor,
                            token_seq: torch.Tensor, block_table: torch.Tensor, block_size: int, rank: int,
                            error_flag: Optional[torch.Tensor] = None):
    """cache[page of token t][slot] = norm(x[t]) * w, zero-padded to the cache's width.
    x: [n, rank] view (last dimension contiguous); cache: [pages, 1, 1, block_size, padded rank]."""
    n = x.shape[0]
    padded = cache.shape[-1]
    if x.shape != (n, rank) or x.stride(1) != 1 or cache.dtype != x.dtype or not cache.is_contiguous() or \
            tuple(cache.shape[1:]) != (1, 1, block_size, padded) or padded < rank:
        raise KernelError(f"latent cache: x [n, {rank}] and a cache [pages, 1, 1, {block_size}, >= {rank}] of one dtype")
    f = _func("latent_cache.cu", "lmsf_latent_norm_cache_write",
              [c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
               c_int, c_float, c_int, c_void_p, c_void_p])
    rc = f(_ptr(x), x.stride(0), _f32vec(w, rank, "w"), _ptr(cache), cache.stride(0), _i32(positions, "positions"),
           _i32(token_seq, "token_seq"), _i32(block_table, "block_table"), block_table.shape[1], block_size, n, rank, padded,
           float(eps), dtype_code(x.dtype), _i32(error_flag, "error_flag"), _stream())
    _check(rc, "latent_cache.cu", "lmsf_latent_cache")


def latent_norm_rope_cache_write(x: torch.Tensor, w: torch.Tensor, eps: float, cache: torch.Tensor, positions: torch.Tensor,
                                 token_seq: torch.Tensor, block_table: torch.Tensor, block_size: int, rank: int, rot_dim: int,
                                 rot_n: int, inv_freq: Optional[torch.Tensor], error_flag: Optional[torch.Tensor] = None):
    """cache[page of token t][slot] = [norm(x[t, :rank]) * w | key part | zeros]: the key part x[t, rank:rank + rot_dim] has
    its first rot_n values rotated by the token's position (value i pairs with value i + rot_n / 2; inv_freq float32
    [rot_n / 2]).  x: [n, rank + rot_dim] view; cache: [pages, 1, 1, block_size, padded]."""
    n = x.shape[0]
    padded = cache.shape[-1]
    if x.shape != (n, rank + rot_dim) or x.stride(1) != 1 or cache.dtype != x.dtype or not cache.is_contiguous() or \
            tuple(cache.shape[1:]) != (1, 1, block_size, padded) or padded < rank + rot_dim:
        raise KernelError(f"latent cache: x [n, {rank + rot_dim}] and a cache [pages, 1, 1, {block_size}, >= {rank + rot_dim}] of one dtype")
    if rot_n and (inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_n // 2 or not inv_freq.is_contiguous()):
        raise KernelError("latent cache: inv_freq must hold rot_n / 2 float32 values")
    f = _func("latent_cache.cu", "lmsf_latent_norm_rope_cache_write",
              [c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
               c_int, c_float, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p])
    rc = f(_ptr(x), x.stride(0), _f32vec(w, rank, "w"), _ptr(cache), cache.stride(0), _i32(positions, "positions"),
           _i32(token_seq, "token_seq"), _i32(block_table, "block_table"), block_table.shape[1], block_size, n, rank, padded,
           float(eps), int(rot_dim), int(rot_n), _ptr(inv_freq), dtype_code(x.dtype), _i32(error_flag, "error_flag"), _stream())
    _check(rc, "latent_cache.cu", "lmsf_latent_cache")


def latent_query_rope(qa: torch.Tensor, q: torch.Tensor, positions: torch.Tensor, heads: int, plain: int, rot_dim: int,
                      rot_n: int, inv_freq: Optional[torch.Tensor], rank: int, padded: int):
    """qa[t, h, rank:rank + rot_dim] = the rotated part q[t, h, plain:plain + rot_dim] of every head, its first rot_n values
    rotated by the token's position; qa[t, h, rank + rot_dim:padded] = 0.  q: [n, heads * (plain + rot_dim)] view,
    qa: [n, heads * padded]."""
    n = q.shape[0]
    if q.shape != (n, heads * (plain + rot_dim)) or q.stride(1) != 1 or qa.shape != (n, heads * padded) or qa.stride(1) != 1 \
            or qa.dtype != q.dtype:
        raise KernelError("latent query: q [n, heads * (plain + rot_dim)] and qa [n, heads * padded] of one dtype")
    if rot_n and (inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_n // 2 or not inv_freq.is_contiguous()):
        raise KernelError("latent query: inv_freq must hold rot_n / 2 float32 values")
    f = _func("latent_cache.cu", "lmsf_latent_query_rope",
              [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int,
               c_int, c_void_p])
    rc = f(_ptr(q), q.stride(0), _ptr(qa), qa.stride(0), _i32(positions, "positions"), n, heads, plain, rot_dim, int(rot_n),
           _ptr(inv_freq), rank, padded, dtype_code(q.dtype), _stream())
    _check(rc, "latent_cache.cu", "lmsf_latent_cache")


def head_gate_(x: torch.Tensor, gate: torch.Tensor, heads: int, head_dim: int):
    """x[t, h, :] *= sigmoid(gate[t, h]) in place.  x: [n, heads * head_dim], gate: [n, heads] (views, last dimension contiguous)."""
    n = x.shape[0]
    if x.shape != (n, heads * head_dim) or gate.shape != (n, heads) or x.stride(1) != 1 or gate.stride(1) != 1 or x.dtype != gate.dtype:
        raise KernelError("head_gate: x [n, heads * head_dim] and gate [n, heads] of one dtype")
    f = _func("latent_cache.cu", "lmsf_head_gate", [c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_void_p])
    rc = f(_ptr(x), x.stride(0), _ptr(gate), gate.stride(0), n, heads, head_dim, dtype_code(x.dtype), _stream())
    _check(rc, "latent_cache.cu", "lmsf_latent_cache")


def value_gate_(x: torch.Tensor, gate: torch.Tensor, heads: int, head_dim: int, value_dim: int):
    """x[t, h, d] *= sigmoid(gate[t, h, d]) for d < value_dim, in place.  x: [n, heads * head_dim], gate: [n, heads * value_dim]
    (views, last dimension contiguous)."""
    n = x.shape[0]
    if x.shape != (n, heads * head_dim) or gate.shape != (n, heads * value_dim) or x.stride(1) != 1 or gate.stride(1) != 1 or \
            x.dtype != gate.dtype:
        raise KernelError("value_gate: x [n, heads * head_dim] and gate [n, heads * value_dim] of one dtype")
    f = _func("latent_cache.cu", "lmsf_value_gate", [c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_void_p])
    rc = f(_ptr(x), x.stride(0), _ptr(gate), gate.stride(0), n, heads, head_dim, value_dim, dtype_code(x.dtype), _stream())
    _check(rc, "latent_cache.cu", "lmsf_latent_cache")


def attention_shared_kv(out: torch.Tensor, q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, block_size: int,
                        token_seq: torch.Tensor, positions: torch.Tensor, scale: float, window: int, n_q_heads: int,
                        head_dim: int, gate: Optional[torch.Tensor] = None, sinks: Optional[torch.Tensor] = None):
    """Attention of n_q_heads query heads over ONE cached vector per token that is key and value at once
    (cache [pages, 1, 1, block_size, head_dim]); out[t, h] = sigmoid(gate[t, h]) * softmax(scale q K^T) K when a gate
    ([n, n_q_heads] view) is given; sinks (float32 [n_q_heads]): exp(sink) is one more term of the softmax's denominator.
    The plain kernel: any mix of tokens, fixed summation order."""
    n = q.shape[0]
    if q.stride(1) != 1 or out.stride(1) != 1 or q.shape[1] != n_q_heads * head_dim or out.shape != q.shape:
        raise KernelError("attention: q and out must be [n, heads * head_dim] with a contiguous last dimension")
    if cache.dtype != q.dtype or out.dtype != q.dtype or not cache.is_contiguous() or \
            tuple(cache.shape[1:]) != (1, 1, block_size, head_dim):
        raise KernelError(f"attention: cache of shape {tuple(cache.shape)} / {cache.dtype} is not [pages, 1, 1, {block_size}, {head_dim}]")
    if gate is not None and (gate.shape != (n, n_q_heads) or gate.stride(1) != 1 or gate.dtype != q.dtype):
        raise KernelError("attention: the gate must be [n, heads] of q's dtype")
    _per_head(sinks, n_q_heads, "sinks")
    f = _func("attention_generic.cu", "lmsf_attention_generic_masked", _GENERIC_MASKED_ARGS)
    rc = f(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(cache), cache.stride(0),
           _i32(block_table, "block_table"), block_table.shape[1], block_size, _i32(token_seq, "token_seq"),
           _i32(positions, "positions"), float(scale), 0.0, None, int(window or 0), n, n_q_heads, 1, head_dim,
           dtype_code(q.dtype), 1, _ptr(gate), gate.stride(0) if gate is not None else 0, 0, None, None, _ptr(sinks),
           _stream())
    _check(rc, "attention_generic.cu", "lmsf_attention_generic")


def gemm_tn_simt_batched(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor):
    """out[:, b, :] = a[:, b, :] w[b]^T for every b.  a: [M, B, K], out: [M, B, N] (views: the last dimension
    contiguous, any row and batch strides); w: [B, N, K].  float32 FMA accumulation in ascending k."""
    M, B, K = a.shape
    N = w.shape[1]
    if w.shape != (B, N, K) or out.shape != (M, B, N) or a.stride(2) != 1 or w.stride(2) != 1 or out.stride(2) != 1 \
            or a.dtype != w.dtype:
        raise KernelError(f"gemm: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    f = _func("gemm_simt.cu", "lmsf_gemm_tn_simt_batched",
              [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int, c_longlong,
               c_longlong, c_longlong, c_int, c_int, c_void_p])
    rc = f(_ptr(out), _ptr(a), _ptr(w), M, N, K, a.stride(0), w.stride(1), out.stride(0), B, a.stride(1), w.stride(0),
           out.stride(1), dtype_code(a.dtype), dtype_code(out.dtype), _stream())
    _check(rc, "gemm_simt.cu", "lmsf_gemm_simt")


# ----------------------------------------------------------------------------- routed experts

MOE_ACTS = {None: 0, "none": 0, "relu2": 1}
_MOE_TILE_ROWS: Optional[int] = None


def moe_tile_rows() -> int:
    global _MOE_TILE_ROWS
    if _MOE_TILE_ROWS is None:
        lib = load_library("moe.cu")
        lib.lmsf_moe_tile_rows.restype = c_int
        _MOE_TILE_ROWS = int(lib.lmsf_moe_tile_rows())
    return _MOE_TILE_ROWS


MOE_TC_TILE_ROWS = 128      # rows per tile of the tensor-core product (csrc/moe_tc.cu)


def moe_max_tiles(pairs: int, experts: int, tile_rows: int) -> int:
    """An upper bound of the row tiles of `pairs` (token, choice) pairs over `experts` experts, whatever the routing."""
    return pairs // tile_rows + min(experts, pairs)


def moe_grouped_tc_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0
            and a.stride(1) == 1 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and w.is_contiguous())


def moe_grouped_tc(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, gather: Optional[torch.Tensor], tiles: torch.Tensor,
                   meta: torch.Tensor, act: Optional[str] = None, error_flag: Optional[torch.Tensor] = None):
    """`moe_grouped` on the tensor cores (bfloat16 operands, a tile list of MOE_TC_TILE_ROWS rows a tile; out bfloat16 or float32)."""
    E, N, K = w.shape
    if not moe_grouped_tc_supported(a, w) or a.shape[1] != K or out.shape[1] != N or out.stride(1) != 1:
        raise KernelError(f"moe_tc: shapes {tuple(a.shape)} x {tuple(w.shape)} -> {tuple(out.shape)} are not taken")
    f = _func("moe_tc.cu", "lmsf_moe_grouped_tc",
              [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong,
               c_int, c_int, c_void_p, c_void_p])
    rc = f(_ptr(out), _ptr(a), _ptr(w), _i32(gather, "gather"), _i32(tiles, "tiles"), _i32(meta, "meta"), tiles.shape[0], E, N, K,
           a.stride(0), out.stride(0), MOE_ACTS[act], dtype_code(out.dtype), _i32(error_flag, "error_flag"), _stream())
    _check(rc, "moe_tc.cu", "lmsf_moe_tc")


def moe_topk(ids: torch.Tensor, wts: torch.Tensor, logits: torch.Tensor, bias: Optional[torch.Tensor], experts: int):
    """ids, wts [n, top]: the `top` largest of logits[t, :experts] + bias and the softmax over those alone."""
    n, top = ids.shape
    if logits.dtype != torch.float32 or logits.shape[0] != n or logits.shape[1] < experts or logits.stride(1) != 1:
        raise KernelError("moe: the router's logits must be float32 [n, >= experts]")
    if wts.dtype != torch.float32 or wts.shape != ids.shape or not wts.is_contiguous():
        raise KernelError("moe: one float32 weight per choice")
    f = _func("moe.cu", "lmsf_moe_topk", [c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p])
    rc = f(_ptr(logits), logits.stride(0), _f32vec(bias, experts, "bias"), n, experts, top, _i32(ids, "ids"), _ptr(wts), _stream())
    _check(rc, "moe.cu", "lmsf_moe")


def moe_topk_sigmoid(ids: torch.Tensor, wts: torch.Tensor, logits: torch.Tensor, correction: Optional[torch.Tensor],
                     experts: int, n_groups: int = 1, keep: int = 1, weight_scale: float = 1.0):
    """ids, wts [n, top]: scores s = sigmoid(logits[t, :experts]); the `top` largest s + correction among the experts
    of the `keep` best of `n_groups` groups of neighbours (a group's score: the sum of its two largest s + correction);
    the weights are the chosen s times weight_scale, not renormalised."""
    n, top = ids.shape
    if logits.dtype != torch.float32 or logits.shape[0] != n or logits.shape[1] < experts or logits.stride(1) != 1:
        raise KernelError("moe: the router's logits must be float32 [n, >= experts]")
    if wts.dtype != torch.float32 or wts.shape != ids.shape or not wts.is_contiguous():
        raise KernelError("moe: one float32 weight per choice")
    f = _func("moe.cu", "lmsf_moe_topk_sigmoid",
              [c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p])
    rc = f(_ptr(logits), logits.stride(0), _f32vec(correction, experts, "correction"), n, experts, top, int(n_groups), int(keep),
           float(weight_scale), _i32(ids, "ids"), _ptr(wts), _stream())
    _check(rc, "moe.cu", "lmsf_moe")


def moe_topk_softmax_all(ids: torch.Tensor, wts: torch.Tensor, logits: torch.Tensor, correction: Optional[torch.Tensor],
                         outputs: int, weight_scale: float = 1.0):
    """ids, wts [n, top]: scores s = softmax(logits[t, :outputs]) over all router outputs; the `top` largest s + correction;
    the weights are the chosen s times weight_scale, not renormalised."""
    n, top = ids.shape
    if logits.dtype != torch.float32 or logits.shape[0] != n or logits.shape[1] < outputs or logits.stride(1) != 1:
        raise KernelError("moe: the router's logits must be float32 [n, >= outputs]")
    if wts.dtype != torch.float32 or wts.shape != ids.shape or not wts.is_contiguous():
        raise KernelError("moe: one float32 weight per choice")
    f = _func("moe.cu", "lmsf_moe_topk_softmax_all",
              [c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p])
    rc = f(_ptr(logits), logits.stride(0), _f32vec(correction, outputs, "correction"), n, outputs, top, float(weight_scale),
           _i32(ids, "ids"), _ptr(wts), _stream())
    _check(rc, "moe.cu", "lmsf_moe")


def moe_align(ids: torch.Tensor, experts: int, tile_rows: int, offsets: torch.Tensor, pair_row: torch.Tensor,
              row_token: torch.Tensor, tiles: torch.Tensor, meta: torch.Tensor):
    """Sorts the (token, choice) pairs by expert on the device: offsets [experts + 1], pair_row [n, top] (row of each
    pair in expert order), row_token [pairs], tiles [max_tiles, 4] and meta[0] = number of tiles."""
    n, top = ids.shape
    f = _func("moe.cu", "lmsf_moe_align",
              [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p])
    rc = f(_i32(ids, "ids"), n * top, top, experts, int(tile_rows), _i32(offsets, "offsets"), _i32(pair_row, "pair_row"),
           _i32(row_token, "row_token"), _i32(tiles, "tiles"), tiles.shape[0], _i32(meta, "meta"), _stream())
    _check(rc, "moe.cu", "lmsf_moe")


def moe_grouped(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, gather: Optional[torch.Tensor], tiles: torch.Tensor,
                meta: torch.Tensor, act: Optional[str] = None):
    """out[row] = act(a[gather[row] or row] w[expert of row]^T) for every row of the tile list.  w: [experts, N, K]."""
    E, N, K = w.shape
    if a.shape[1] != K or a.stride(1) != 1 or out.shape[1] != N or out.stride(1) != 1 or a.dtype != w.dtype or not w.is_contiguous():
        raise KernelError(f"moe: shapes {tuple(a.shape)} x {tuple(w.shape)} -> {tuple(out.shape)}")
    f = _func("moe.cu", "lmsf_moe_grouped",
              [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_int,
               c_int, c_int, c_void_p])
    rc = f(_ptr(out), _ptr(a), _ptr(w), _i32(gather, "gather"), _i32(tiles, "tiles"), _i32(meta, "meta"), tiles.shape[0], N, K,
           a.stride(0), out.stride(0), MOE_ACTS[act], dtype_code(a.dtype), dtype_code(out.dtype), _stream())
    _check(rc, "moe.cu", "lmsf_moe")


def moe_combine(out: torch.Tensor, down: torch.Tensor, pair_row: torch.Tensor, wts: Optional[torch.Tensor],
                shared: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                identity: Optional[Tuple[torch.Tensor, int, torch.Tensor]] = None):
    """out[t] = sum_j wts[t, j] * down[pair_row[t, j]] + sigmoid(gate[t]) * shared[t].  down: float32 [pairs, width];
    gate: float32 [n] view (any stride); shared: [n, width] of out's dtype.  wts None: every weight is 1.  identity (ids [n,
    top], experts, x [n, width] of out's dtype): a choice numbered `experts` or more adds wts[t, j] * x[t] instead."""
    n, width = out.shape
    top = pair_row.shape[1]
    if wts is not None and (wts.dtype != torch.float32 or tuple(wts.shape) != (n, top) or not wts.is_contiguous()):
        raise KernelError("moe: one contiguous float32 weight per (token, choice)")
    if down.dtype != torch.float32 or down.shape[1] != width or not down.is_contiguous() or not out.is_contiguous():
        raise KernelError("moe: down must be contiguous float32 [pairs, width] and out contiguous [n, width]")
    if shared is not None and (shared.shape != out.shape or shared.dtype != out.dtype or not shared.is_contiguous()):
        raise KernelError("moe: the shared expert's output must be like out")
    if gate is not None and (gate.dtype != torch.float32 or gate.dim() != 1 or gate.shape[0] != n):
        raise KernelError("moe: one float32 gate value per token")
    ids, experts, x = identity if identity is not None else (None, 0, None)
    if identity is not None and (tuple(ids.shape) != (n, top) or x.shape != out.shape or x.dtype != out.dtype or not x.is_contiguous()):
        raise KernelError("moe: experts that return their input need the choices [n, top] and the input, like out")
    f = _func("moe.cu", "lmsf_moe_combine_identity",
              [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_void_p,
               c_int, c_void_p, c_void_p])
    rc = f(_ptr(out), _ptr(down), _i32(pair_row, "pair_row"), _ptr(wts), top, _ptr(shared), _ptr(gate),
           gate.stride(0) if gate is not None else 0, n, width, dtype_code(out.dtype), _i32(ids, "ids"), int(experts), _ptr(x),
           _stream())
    _check(rc, "moe.cu", "lmsf_moe")


GLU_ACTS = {"silu": 0, "swish": 0, "gelu_tanh": 1}


def moe_weighted_glu(out: torch.Tensor, y: torch.Tensor, pair_row: torch.Tensor, wts: Optional[torch.Tensor], act: str = "silu"):
    """out[r] = act(w y[r, :F]) * (w y[r, F:]) for the row r = pair_row[pair] of every (token, choice) pair and its routing
    weight w = wts[pair] (None: 1): gated experts whose weight multiplies what the expert reads.  y: [pairs, 2 F]."""
    pairs, F = out.shape
    if y.shape != (pairs, 2 * F) or not (y.is_contiguous() and out.is_contiguous()) or y.dtype != out.dtype:
        raise KernelError("moe: y must be contiguous [pairs, 2 F] and out [pairs, F] of one dtype")
    if pair_row.numel() != pairs or (wts is not None and (wts.dtype != torch.float32 or wts.numel() != pairs or not wts.is_contiguous())):
        raise KernelError("moe: one row and one float32 weight per pair")
    if act not in GLU_ACTS:
        raise KernelError(f"moe: unknown gated activation {act!r} (known: {', '.join(sorted(GLU_ACTS))})")
    f = _func("moe.cu", "lmsf_moe_weighted_glu", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    rc = f(_ptr(out), _ptr(y), _i32(pair_row, "pair_row"), _ptr(wts), pairs, F, GLU_ACTS[act], dtype_code(out.dtype), _stream())
    _check(rc, "moe.cu", "lmsf_moe")


def relu2_(x: torch.Tensor):
    """x <- max(x, 0)^2 in place."""
    if not x.is_contiguous():
        raise KernelError("relu2: x must be contiguous")
    f = _func("moe.cu", "lmsf_relu2", [c_void_p, c_longlong, c_int, c_void_p])
    rc = f(_ptr(x), x.numel(), dtype_code(x.dtype), _stream())
    _check(rc, "moe.cu", "lmsf_moe")
