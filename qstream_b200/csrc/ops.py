"""Python face of the kernel library: one function per `extern "C"` entry point.

Tensors are torch CUDA tensors used as typed device buffers; every launch goes on
torch's current stream, so the calls can be captured in a CUDA graph.  There is no
other implementation behind these functions: if the library cannot be built or
loaded, or a tensor is not on a CUDA device, the call raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_double, c_float, c_int, c_longlong, c_uint, c_ulonglong, c_void_p

import torch

from ..errors import QsError, QStreamError
from . import build as _build

F32, BF16 = 0, 1
ACT_NONE, ACT_GELU_TANH, ACT_GELU_ERF, ACT_SILU, ACT_SIGMOID, ACT_TANH, ACT_RELU2 = 0, 1, 2, 3, 4, 5, 6
ACTIVATIONS = {None: ACT_NONE, "none": ACT_NONE, "gelu_new": ACT_GELU_TANH, "gelu": ACT_GELU_ERF,
               "silu": ACT_SILU, "sigmoid": ACT_SIGMOID, "tanh": ACT_TANH, "relu2": ACT_RELU2}

_lib = None

_SIGNATURES = {
    "qs_abi_version": ([], c_int),
    "qs_embedding": ([c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p], c_int),
    "qs_layernorm": ([c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float,
                      c_longlong, c_longlong, c_int, c_void_p], c_int),
    "qs_gather_rows": ([c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_longlong, c_void_p], c_int),
    "qs_add": ([c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_void_p], c_int),
    "qs_linear_simt": ([c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p,
                        c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_void_p], c_int),
    "qs_rope_store": ([c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_longlong, c_longlong,
                       c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                       c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_longlong, c_float, c_int, c_void_p], c_int),
    "qs_norm_rope_store": ([c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_longlong, c_longlong, c_void_p, c_int, c_void_p, c_int,
                            c_float, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                            c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p], c_int),
    "qs_attention": ([c_void_p, c_void_p, c_int, c_longlong, c_longlong, c_void_p, c_void_p, c_void_p, c_int,
                      c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p,
                      c_int, c_float, c_int, c_int, c_void_p, c_int, c_int, c_void_p], c_int),
    "qs_pair_diff_norm": ([c_void_p, c_int, c_longlong, c_void_p, c_int, c_longlong, c_int, c_int, c_int, c_float, c_float,
                           c_float, c_void_p], c_int),
    "qs_delta_prepare": ([c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int,
                          c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p,
                          c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
                          c_void_p], c_int),
    "qs_conv_state_update": ([c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int,
                              c_void_p, c_void_p, c_int, c_void_p], c_int),
    "qs_hyper_spread": ([c_void_p, c_longlong, c_int, c_int, c_int, c_void_p, c_longlong, c_void_p], c_int),
    "qs_hyper_mix_norm": ([c_void_p, c_longlong, c_int, c_int, c_int, c_void_p, c_longlong, c_float, c_void_p, c_longlong,
                           c_float, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_float,
                           c_void_p, c_int, c_longlong, c_int, c_void_p], c_int),
    "qs_residual_rmsnorm": ([c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_int,
                             c_longlong, c_float, c_void_p, c_int, c_float, c_int, c_int, c_float, c_void_p], c_int),
    "qs_gated_group_norm": ([c_void_p, c_int, c_longlong, c_void_p, c_int, c_longlong, c_void_p, c_int, c_void_p, c_int,
                             c_longlong, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p], c_int),
    "qs_clamped_glu": ([c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int, c_float, c_float, c_float, c_void_p], c_int),
    "qs_activate": ([c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_void_p], c_int),
    "qs_gated_act": ([c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_void_p], c_int),
    "qs_embedding_hashed": ([c_void_p, c_int, c_void_p, c_void_p, c_int, c_float, c_longlong, c_longlong, c_longlong,
                             c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_void_p], c_int),
    "qs_keep_last_rows": ([c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_int, c_void_p], c_int),
    "qs_state_scan": ([c_int, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_int,
                       c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_int,
                       c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                       c_void_p, c_void_p, c_longlong, c_float, c_int, c_float, c_void_p], c_int),
    "qs_delta_chunk_prefix": ([c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                               c_void_p], c_int),
    "qs_mlstm_gates": ([c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_longlong, c_float, c_void_p, c_longlong,
                        c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p], c_int),
    "qs_mlstm_output": ([c_void_p, c_int, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_int,
                         c_void_p, c_int, c_longlong, c_int, c_int, c_int, c_float, c_void_p], c_int),
    "qs_branch_norm": ([c_void_p, c_int, c_longlong, c_void_p, c_int, c_longlong, c_void_p, c_int, c_longlong, c_void_p,
                        c_int, c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p], c_int),
    "qs_latent_prepare": ([c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_int, c_int, c_void_p, c_longlong,
                           c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_float, c_float, c_int, c_void_p, c_void_p,
                           c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p], c_int),
    "qs_latent_q_rotate": ([c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_int,
                            c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_void_p], c_int),
    "qs_head_linear": ([c_void_p, c_longlong, c_longlong, c_void_p, c_longlong, c_longlong, c_void_p, c_int, c_int, c_int,
                        c_int, c_int, c_void_p], c_int),
    "qs_moe_route": ([c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int,
                      c_int, c_float, c_int, c_int, c_int, c_void_p], c_int),
    "qs_moe_expert_up": ([c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                          c_int, c_int, c_int, c_void_p], c_int),
    "qs_moe_expert_down": ([c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                            c_void_p, c_int, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_void_p], c_int),
    "qs_moe_sort": ([c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p], c_int),
    "qs_moe_combine": ([c_void_p, c_longlong, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                        c_longlong, c_void_p, c_int, c_int, c_int, c_void_p], c_int),
    "qs_token_shift": ([c_void_p, c_longlong, c_longlong, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_longlong,
                        c_void_p, c_void_p, c_int, c_int, c_int, c_void_p], c_int),
    "qs_argmax": ([c_void_p, c_void_p, c_int, c_int, c_longlong, c_void_p], c_int),
    "qs_repeat_penalty": ([c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_void_p, c_float, c_void_p], c_int),
    "qs_sample": ([c_void_p, c_void_p, c_int, c_int, c_longlong, c_float, c_int, c_float, c_void_p, c_void_p], c_int),
    "qs_random_fill": ([c_void_p, c_int, c_longlong, c_ulonglong, c_int, c_double, c_longlong, c_void_p], c_int),
    "qs_convert": ([c_void_p, c_int, c_void_p, c_int, c_longlong, c_void_p], c_int),
    "qs_check_finite": ([c_void_p, c_int, c_int, c_int, c_longlong, c_int, c_void_p, c_void_p, c_void_p], c_int),
    "qs_canary_fill": ([c_void_p, c_longlong, c_uint, c_void_p], c_int),
    "qs_canary_check": ([c_void_p, c_longlong, c_uint, c_void_p, c_void_p], c_int),
    "qs_selftest_bounded_wait": ([c_void_p, c_int, c_void_p], c_int),
    "qs_take_tokens": ([c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p], c_int),
    "qs_zero_pages": ([c_void_p, c_longlong, c_longlong, c_int, c_void_p, c_int, c_int, c_void_p], c_int),
}


def library():
    """The loaded kernel library; built on first use."""
    global _lib
    if _lib is None:
        path = _build.build()
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as e:
            raise QStreamError(QsError.INTERNAL, f"cannot load {path}: {e}") from None
        lib.qs_last_error.restype = ctypes.c_char_p
        lib.qs_last_error.argtypes = []
        for name, (argtypes, restype) in _SIGNATURES.items():
            if not hasattr(lib, name):
                continue                    # optional entry points are bound by their own modules
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = restype
        _lib = lib
    return _lib


def bind(name: str, argtypes, restype=c_int):
    """Bind one more entry point (used by modules that own further kernels)."""
    lib = library()
    try:
        fn = getattr(lib, name)
    except AttributeError:
        raise QStreamError(QsError.INTERNAL, f"the kernel library has no entry point '{name}'") from None
    fn.argtypes = argtypes
    fn.restype = restype
    return fn


_launches = 0


def launch_count() -> int:
    """How many kernels of the library have been launched (replayed graph nodes included)."""
    return _launches


def count_launches(n: int) -> None:
    global _launches
    _launches += n


def check(rc: int) -> None:
    global _launches
    _launches += 1
    if rc != 0:
        detail = library().qs_last_error().decode(errors="replace")
        try:
            code = QsError(rc)
        except ValueError:
            code = QsError.INTERNAL
        raise QStreamError(code, detail)


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise QStreamError(QsError.INVALID_INPUT, f"kernels take float32 or bfloat16, got {t.dtype}")


def ptr(t) -> int | None:
    if t is None:
        return None
    if not t.is_cuda:
        raise QStreamError(QsError.INVALID_INPUT, "kernels run on CUDA tensors only; there is no CPU path")
    return t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream() -> int:
    """The current CUDA stream's handle (the capturing stream while a graph is captured)."""
    if _raw_stream is not None:                       # a plain C call: the Stream object costs ten times as much
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _rows(t: torch.Tensor):
    """(rows, width, row stride) of a 2-D tensor whose rows are contiguous."""
    if t.dim() != 2 or t.stride(1) != 1:
        raise QStreamError(QsError.INVALID_INPUT, f"need a 2-D tensor with contiguous rows, got "
                           f"shape {tuple(t.shape)} strides {t.stride()}")
    return t.shape[0], t.shape[1], t.stride(0)


def _int32(t: torch.Tensor, what: str):
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise QStreamError(QsError.INVALID_INPUT, f"{what} must be a contiguous int32 tensor")
    return ptr(t)


# ------------------------------------------------------------------------------- wrappers

def embedding(table: torch.Tensor, tokens: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    V, D = table.shape
    T = tokens.numel()
    out = torch.empty((T, D), dtype=out_dtype, device=table.device)
    check(library().qs_embedding(ptr(out), dtype_code(out), ptr(table), dtype_code(table),
                                 _int32(tokens, "tokens"), T, D, V, stream()))
    return out


def layernorm(x: torch.Tensor, weight: torch.Tensor, bias, eps: float, out=None, settled=False) -> torch.Tensor:
    """`settled`: weight and bias were complete before the previous kernel of the stream began (a model's
    are); the kernel then fetches them while that kernel still runs."""
    rows, D, ldx = _rows(x)
    if out is None:
        out = torch.empty((rows, D), dtype=x.dtype, device=x.device)
    _, _, ldo = _rows(out)
    if weight.numel() != D or (bias is not None and bias.numel() != D):
        raise QStreamError(QsError.INVALID_INPUT, f"layernorm: width {D} but weight {tuple(weight.shape)}")
    check(library().qs_layernorm(ptr(out), ptr(x), dtype_code(x), ptr(weight), dtype_code(weight),
                                 ptr(bias), dtype_code(bias) if bias is not None else 0, rows, D,
                                 float(eps), ldx, ldo, int(bool(settled)), stream()))
    return out


def gather_rows(x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    _, D, ldx = _rows(x)
    n = rows.numel()
    out = torch.empty((n, D), dtype=x.dtype, device=x.device)
    check(library().qs_gather_rows(ptr(out), ptr(x), dtype_code(x), _int32(rows, "rows"), n, D, ldx, stream()))
    return out


def add(a: torch.Tensor, b: torch.Tensor, c=None) -> torch.Tensor:
    for t in (b, c):
        if t is not None and (t.shape != a.shape or t.dtype != a.dtype or not t.is_contiguous()):
            raise QStreamError(QsError.INVALID_INPUT, "add: operands differ in shape, type or layout")
    if not a.is_contiguous():
        raise QStreamError(QsError.INVALID_INPUT, "add: operands must be contiguous")
    out = torch.empty_like(a)
    check(library().qs_add(ptr(out), ptr(a), ptr(b), ptr(c), dtype_code(a), a.numel(), stream()))
    return out


def linear_simt(x, weight, bias=None, activation=None, residuals=(), out_dtype=None, out=None) -> torch.Tensor:
    """act(x W^T + bias) + residuals, accumulated in true 32-bit on the CUDA cores."""
    M, K, lda = _rows(x)
    N, K2 = weight.shape
    if K2 != K or not weight.is_contiguous():
        raise QStreamError(QsError.INVALID_INPUT, f"linear: x is [{M}, {K}] but weight is {tuple(weight.shape)}")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype or x.dtype, device=x.device)
    elif out.shape != (M, N) or out.stride(1) != 1:
        raise QStreamError(QsError.INVALID_INPUT, "linear: the output view does not fit")
    res = list(residuals) + [None, None]
    ldr = N
    for r in res[:2]:
        if r is not None:
            if r.shape != (M, N) or r.dtype != x.dtype or r.stride(1) != 1:
                raise QStreamError(QsError.INVALID_INPUT, "linear: residual differs in shape or type")
            ldr = r.stride(0)
    if len(residuals) > 2 or (len(residuals) == 2 and res[0].stride(0) != res[1].stride(0)):
        raise QStreamError(QsError.INVALID_INPUT, "linear: at most two residuals of one layout")
    check(library().qs_linear_simt(ptr(out), dtype_code(out), ptr(x), dtype_code(x), ptr(weight),
                                   dtype_code(weight), ptr(bias), dtype_code(bias) if bias is not None else 0,
                                   ACTIVATIONS[activation], ptr(res[0]), ptr(res[1]), M, N, K, lda, out.stride(0), ldr,
                                   stream()))
    return out


def rope_store(q, k, v, n_heads, n_kv_heads, head_dim, rotary_dim, cos_sin, tok_slot, tok_pos,
               page_table, page_tokens, k_cache, v_cache, status, settled=False, v_head_dim=None,
               v_first=None, v_mix=0.0, half_layout=False) -> None:
    """Rotate q (in place) and k, and write k and v into the paged cache entry.
    `half_layout`: the rotated pairs are (i, i + rotary_dim / 2) instead of (2i, 2i + 1), with the same angles.
    k = v = None (n_kv_heads = 0): rotate q only (no page table is needed then).
    `v_head_dim`: the values' head size where it differs from the keys'.  `v_first` (same shape as v):
    the cache keeps (1 - v_mix) v + v_mix v_first instead of v.
    `settled`: slots, positions, page table and the table of angles were complete before the previous kernel
    of the stream began (a step's own are); the kernel then reads them early."""
    ref = k if k is not None else q
    T = ref.shape[0]
    max_pos = cos_sin.shape[0] if cos_sin is not None else 0
    check(library().qs_rope_store(
        ptr(q), ptr(k), ptr(v), dtype_code(ref), q.stride(0) if q is not None else 0,
        k.stride(0) if k is not None else 0, v.stride(0) if v is not None else 0,
        n_heads if q is not None else 0, n_kv_heads, head_dim, rotary_dim if cos_sin is not None else 0,
        ptr(cos_sin), max_pos, _int32(tok_slot, "tok_slot"), _int32(tok_pos, "tok_pos"),
        _int32(page_table, "page_table") if page_table is not None else None,
        page_table.shape[1] if page_table is not None else 0, page_tokens, ptr(k_cache), ptr(v_cache), T,
        ptr(status), int(bool(settled)), int(v_head_dim or head_dim), ptr(v_first),
        v_first.stride(0) if v_first is not None else 0, float(v_mix), int(bool(half_layout)), stream()))


def norm_rope_store(q, k, v, q_weight, k_weight, eps, n_heads, n_kv_heads, head_dim, rotary_dim, cos_sin, tok_slot, tok_pos,
                    page_table, page_tokens, k_cache, v_cache, status, v_head_dim=None, half_layout=False) -> None:
    """One RMS norm over the whole row of q [T, n_heads * head_dim] (weight `q_weight` of that size, `eps` inside the root)
    and one over the whole row of k, then the rotation of every head's first `rotary_dim` dims and the cache write, in
    one kernel: q is changed in place, the cache keeps the normed and rotated k and the values v as they are (v may be
    k: the keys as projected).  k = v = None (n_kv_heads = 0): a layer with queries only."""
    T = q.shape[0]
    max_pos = cos_sin.shape[0] if cos_sin is not None else 0
    check(library().qs_norm_rope_store(
        ptr(q), ptr(k), ptr(v), dtype_code(q), q.stride(0), k.stride(0) if k is not None else 0,
        v.stride(0) if v is not None else 0, ptr(q_weight), _code(q_weight), ptr(k_weight), _code(k_weight), float(eps),
        int(n_heads), int(n_kv_heads) if k is not None else 0, int(head_dim), int(v_head_dim or head_dim),
        int(rotary_dim) if cos_sin is not None else 0, ptr(cos_sin), max_pos, _int32(tok_slot, "tok_slot"), _int32(tok_pos, "tok_pos"),
        _int32(page_table, "page_table") if page_table is not None else None,
        page_table.shape[1] if page_table is not None else 0, int(page_tokens), ptr(k_cache), ptr(v_cache), T, ptr(status),
        int(bool(half_layout)), stream()))


def attention(q, n_heads, n_kv_heads, head_dim, scale, window, tok_slot, tok_pos, page_table,
              page_tokens, k_cache, v_cache, status, out=None, v_head_dim=None, softcap=0.0, chunk=0, keep_first=0,
              sink=None, maps=1, out_dtype=None) -> torch.Tensor:
    """Causal attention of every token over its sequence's cache (generic kernel).  `v_head_dim`: the values'
    head size where it differs from the keys'; `softcap` c > 0: scores become c tanh(s / c) before the softmax.
    A query at position p sees the last `window` keys (window > 0), or the keys of its own chunk of `chunk`
    positions counted from 0 (chunk > 0), else all up to p; with `keep_first` also the sequence's first keep_first
    keys.  `sink` (float32 [n_heads]): exp(sink_h) joins each softmax's denominator without key or value.
    `maps` m > 1: a cached key row holds m keys of head_dim side by side and `n_heads` counts m query heads per
    head, query head j reading key j % m of its key head; all of them read the same values.  `out_dtype`
    torch.float32: the result in 32-bit whatever the queries' type."""
    T = q.shape[0]
    if sink is not None and (sink.dtype != torch.float32 or sink.numel() != n_heads or not sink.is_contiguous()):
        raise QStreamError(QsError.INVALID_INPUT, "attention: the sinks must be float32, one per query head")
    dv = int(v_head_dim or head_dim)
    if out is None:
        out = torch.empty((T, n_heads * dv), dtype=out_dtype or q.dtype, device=q.device)
    check(library().qs_attention(
        ptr(out), ptr(q), dtype_code(q), out.stride(0), q.stride(0), ptr(k_cache), ptr(v_cache),
        _int32(page_table, "page_table"), page_table.shape[1], page_tokens, _int32(tok_slot, "tok_slot"),
        _int32(tok_pos, "tok_pos"), T, n_heads, n_kv_heads, head_dim, float(scale), int(window),
        ptr(status), dv, float(softcap or 0.0), int(chunk), int(keep_first), ptr(sink), int(maps),
        dtype_code(out), stream()))
    return out


def pair_diff_norm(a, n_heads: int, value_dim: int, lam: float, mult: float, eps: float, out_dtype) -> torch.Tensor:
    """a [T, n_heads * 2 * value_dim], per head the outputs of two attention maps side by side; returns
    [T, n_heads * value_dim]: o = a1 - lam a2, divided by its root mean square over the head (eps inside the
    root), times `mult`; 32-bit arithmetic, rounded once."""
    rows, n, lda = _rows(a)
    if n != n_heads * 2 * value_dim:
        raise QStreamError(QsError.INVALID_INPUT, f"pair_diff_norm: width {n} is not {n_heads} x 2 x {value_dim}")
    out = torch.empty((rows, n_heads * value_dim), dtype=out_dtype, device=a.device)
    check(library().qs_pair_diff_norm(ptr(out), dtype_code(out), out.stride(0), ptr(a), dtype_code(a), lda, rows, n_heads,
                                      value_dim, float(lam), float(mult), float(eps), stream()))
    return out


# ------------------------------------------------------------------------------- a residual stream in several copies

def _f32_vector(t, n, what):
    if t is not None and (t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous()):
        raise QStreamError(QsError.INVALID_INPUT, f"{what} must be {n} contiguous float32 values")
    return ptr(t)


def hyper_spread(src: torch.Tensor, streams: int) -> torch.Tensor:
    """x [T, streams * D] float32 whose `streams` copies all equal src [T, D] (float32)."""
    rows, D, lds = _rows(src)
    if src.dtype != torch.float32:
        raise QStreamError(QsError.INVALID_INPUT, "hyper_spread: the source must be float32")
    x = torch.empty((rows, streams * D), dtype=torch.float32, device=src.device)
    check(library().qs_hyper_spread(ptr(x), x.stride(0), rows, int(streams), D, ptr(src), lds, stream()))
    return x


def hyper_mix_norm(x, streams: int, width: int, y=None, y_scale: float = 1.0, y2=None, y2_scale: float = 1.0,
                   layer_scale=None, mix=None, out_weights=None, in_weights=None, norm_weight=None, offset: float = 0.0,
                   eps: float = 0.0, out_dtype=None, plain_sum: bool = False):
    """The residual stream x [T, streams * width] (float32, `streams` copies side by side) written and read in one pass.
    Write (y given, changed in place): x_t <- sum_s mix[s][t] x_s + out_weights[t] * layer_scale . (y_scale y + y2_scale y2).
    Read (out_dtype given): u = sum_s in_weights[s] x_s of the new x, returned as u / sqrt(mean(u^2) + eps) * (offset +
    norm_weight) in out_dtype, or as it is if `plain_sum`.  mix [streams, streams] ([from, to]), out_weights and
    in_weights [streams] are float32; None stands for the identity, ones and ones.  Returns the read (None without one)."""
    rows, n, ldx = _rows(x)
    S, D = int(streams), int(width)
    if x.dtype != torch.float32 or n != S * D:
        raise QStreamError(QsError.INVALID_INPUT, f"hyper_mix_norm: the stream must be float32 [T, {S} x {D}], not {tuple(x.shape)}")
    ldy = ldy2 = 0
    if y is not None:
        r1, n1, ldy = _rows(y)
        if (r1, n1) != (rows, D):
            raise QStreamError(QsError.INVALID_INPUT, "hyper_mix_norm: the branch differs from a copy of the stream in shape")
    if y2 is not None:
        r2, n2, ldy2 = _rows(y2)
        if y is None or (r2, n2) != (rows, D) or y2.dtype != y.dtype:
            raise QStreamError(QsError.INVALID_INPUT, "hyper_mix_norm: the second branch differs from the first")
    h = torch.empty((rows, D), dtype=out_dtype, device=x.device) if out_dtype is not None else None
    check(library().qs_hyper_mix_norm(
        ptr(x), ldx, rows, S, D, ptr(y), ldy, float(y_scale), ptr(y2), ldy2, float(y2_scale), _code(y), ptr(layer_scale),
        _code(layer_scale), _f32_vector(mix, S * S, "hyper_mix_norm: mix"), _f32_vector(out_weights, S, "hyper_mix_norm: out"),
        _f32_vector(in_weights, S, "hyper_mix_norm: in"), ptr(norm_weight), _code(norm_weight), float(offset), float(eps),
        ptr(h), _code(h), h.stride(0) if h is not None else 0, int(bool(plain_sum)), stream()))
    return h


# ------------------------------------------------------------------------------- a 32-bit residual stream, RMS norms

def _code(t) -> int:
    return dtype_code(t) if t is not None else 0


def rmsnorm(x, weight, eps: float, offset: float = 0.0, out_dtype=None, update=None, mult: float = 1.0,
            want_norm: bool = True):
    """h = x / sqrt(mean(x^2) + eps) * (offset + weight), statistics in 32-bit; h in `out_dtype` (default: x's).
    With `update` (a tensor of x's shape): x <- x + mult * update first, in place and in x's type, in the same
    pass; `want_norm=False` then only updates.  Returns h (None without a norm)."""
    rows, D, ldx = _rows(x)
    h = None
    if want_norm:
        if weight is None or weight.numel() != D:
            raise QStreamError(QsError.INVALID_INPUT, f"rmsnorm: width {D} but weight {None if weight is None else tuple(weight.shape)}")
        h = torch.empty((rows, D), dtype=out_dtype or x.dtype, device=x.device)
    ldy = 0
    if update is not None:
        r2, D2, ldy = _rows(update)
        if (r2, D2) != (rows, D):
            raise QStreamError(QsError.INVALID_INPUT, "rmsnorm: the update differs from x in shape")
    check(library().qs_residual_rmsnorm(ptr(h), _code(h), D, ptr(x) if update is not None else None, ptr(x),
                                        dtype_code(x), ldx, ptr(update), _code(update), ldy, float(mult),
                                        ptr(weight) if want_norm else None, _code(weight) if want_norm else 0,
                                        float(offset), rows, D, float(eps), stream()))
    return h


def gated_group_norm(o, group: int, weight, gate, gate_activation, eps: float, out_dtype, gate_span: int = 1) -> torch.Tensor:
    """out = o / sqrt(mean over each group of `group` consecutive elements of o^2 + eps) * weight * act(gate);
    group 0: no norm; weight and gate may be None.  `gate_span` n > 1: the gate has one column for every n
    neighbouring columns of o (a value per head, say).  Sums in 32-bit."""
    rows, n, ldi = _rows(o)
    out = torch.empty((rows, n), dtype=out_dtype, device=o.device)
    ldg = 0
    if gate is not None:
        r2, n2, ldg = _rows(gate)
        if (r2, n2 * int(gate_span)) != (rows, n):
            raise QStreamError(QsError.INVALID_INPUT, "gated_group_norm: the gate differs from o in shape")
    if weight is not None and weight.numel() != n:
        raise QStreamError(QsError.INVALID_INPUT, f"gated_group_norm: width {n} but weight {tuple(weight.shape)}")
    check(library().qs_gated_group_norm(ptr(out), dtype_code(out), n, ptr(o), dtype_code(o), ldi, ptr(weight),
                                        _code(weight), ptr(gate), _code(gate), ldg, ACTIVATIONS[gate_activation],
                                        rows, n, int(group), float(eps), int(gate_span), stream()))
    return out


def activate(x: torch.Tensor, activation) -> torch.Tensor:
    """x <- act(x) in place (32-bit arithmetic, rounded once)."""
    rows, n, ld = _rows(x)
    check(library().qs_activate(ptr(x), ld, dtype_code(x), rows, n, ACTIVATIONS[activation], stream()))
    return x


def gated_act(ab: torch.Tensor, activation) -> torch.Tensor:
    """out = act(a) * b for ab = [a | b] ([rows, 2 F]), in 32-bit, rounded once."""
    rows, two_f, ldi = _rows(ab)
    F = two_f // 2
    out = torch.empty((rows, F), dtype=ab.dtype, device=ab.device)
    check(library().qs_gated_act(ptr(out), F, ptr(ab), ldi, dtype_code(ab), rows, F, ACTIVATIONS[activation], stream()))
    return out


def clamped_glu(ab: torch.Tensor, limit: float, alpha: float = 1.702, shift: float = 1.0) -> torch.Tensor:
    """For ab = [a | b] ([rows, 2 F]): g = min(a, limit), u = clamp(b, -limit, limit), out = g sigmoid(alpha g) (u + shift),
    in 32-bit, rounded once; limit <= 0: no clamp."""
    rows, two_f, ldi = _rows(ab)
    F = two_f // 2
    out = torch.empty((rows, F), dtype=ab.dtype, device=ab.device)
    check(library().qs_clamped_glu(ptr(out), F, ptr(ab), ldi, dtype_code(ab), rows, F, float(limit), float(alpha),
                                   float(shift), stream()))
    return out


def embedding_hashed(table, pair, scale: float, buckets: int, mul_prev: int, mul_cur: int, tokens, tok_slot, tok_pos,
                     last_token, out_dtype) -> torch.Tensor:
    """x = table[token] * scale + pair[(previous * mul_prev + token * mul_cur) mod buckets] (row `buckets` for a
    sequence's first token); `pair` may be None.  `last_token`: int32 [slots, 1], each sequence's last token of
    earlier steps.  Rows with a negative slot are zero."""
    V, D = table.shape
    T = tokens.numel()
    out = torch.empty((T, D), dtype=out_dtype, device=table.device)
    if pair is not None and (pair.dtype != table.dtype or pair.shape != (buckets + 1, D)):
        raise QStreamError(QsError.INVALID_INPUT, "embedding: the pair table does not fit")
    check(library().qs_embedding_hashed(ptr(out), dtype_code(out), ptr(table), ptr(pair), dtype_code(table), float(scale),
                                        int(buckets), int(mul_prev), int(mul_cur), _int32(tokens, "tokens"),
                                        _int32(tok_slot, "tok_slot"), _int32(tok_pos, "tok_pos"),
                                        ptr(last_token), last_token.stride(0) if last_token is not None else 0,
                                        T, D, V, stream()))
    return out


def keep_last_rows(dst: torch.Tensor, src: torch.Tensor, seq_start, seq_slot, n_seq: int) -> None:
    """dst[slot] = the last row of `src` that each sequence of the step brought (rows of whole 4-byte words)."""
    row_bytes = (src.shape[1] if src.dim() == 2 else 1) * src.element_size()
    check(library().qs_keep_last_rows(ptr(dst), dst.stride(0) * dst.element_size(), ptr(src),
                                      src.stride(0) * src.element_size(), row_bytes, _int32(seq_start, "seq_start"),
                                      _int32(seq_slot, "seq_slot"), int(n_seq), stream()))


def state_scan(mode: str, q, k, v, state, seq_start, seq_slot, n_seq, n_heads, key_dim, value_dim, head_decay=None,
               decay_logits=None, bonus=None, in_activation=None, chunks=None, token_decay=None, token_weight=None,
               q_scale: float = 1.0, key_decay=None, qk_group: int = 1, want_output: bool = True,
               decay_power: float = 0.0) -> torch.Tensor:
    """Walk each sequence's tokens of this step through a per-head matrix state (float32 [slots, heads, value_dim,
    key_dim], updated in place); returns o [T, heads * value_dim] in float32.
    mode "decay": S <- decay_h S + k v^T, o = S^T q.  mode "wkv": o = (S + diag(bonus) k v^T)^T q, then
    S <- diag(exp(-exp(decay_logits))) S + k v^T.  mode "gated": S <- a_t S + b_t k v^T, o = S^T (q q_scale) with
    a = `token_decay`, b = `token_weight` (float32 [T, heads]); here `value_dim` counts one column more than v holds:
    a column of ones, whose state is the normaliser n <- a_t n + b_t k and whose output n.q is each head's last element.
    mode "delta": S' = diag(g_t) S, u = beta_t (v - S'^T k), S <- S' + k u^T, o = S^T q, with g = `key_decay` (float32
    [T, heads * key_dim]) and beta = `token_weight` (float32 [T, heads]); q and k hold heads / `qk_group` heads, head h
    reading number h // qk_group.  With `chunks` the delta rule runs the same walk three times over the chunks side by
    side (what a chunk does to an identity, what it writes from an empty state, and, once a prefix over the chunks has
    given each its starting state, the chunk's outputs).  In mode "decay" `q_scale` multiplies q as well.
    mode "gla": S <- diag(w_t) S + k v^T, o = S^T (q q_scale), w_t = sigmoid(decay_logits)^`decay_power` per token and key
    channel (float32 [T, heads * key_dim]), taken in 32-bit inside the walk.
    `chunks` = (chunk_start, chunk_ids, seq_chunk, n_chunks), int32 device tensors: every sequence of the step cut
    into consecutive chunks (rows chunk_start[c] .. chunk_start[c + 1] of the packed batch; sequence s owns chunks
    seq_chunk[s] .. seq_chunk[s + 1]; chunk_ids = 0 .. n_chunks - 1).  The chunks then run side by side and a
    prefix over each sequence's chunks joins them; the result equals the walk in order up to 32-bit rounding."""
    T = q.shape[0]
    if state.dtype != torch.float32 or state.stride(-1) != 1:
        raise QStreamError(QsError.INVALID_INPUT, "state_scan: the state must be float32")
    if mode == "delta" and chunks is not None:
        return _delta_in_chunks(q, k, v, state, seq_slot, n_seq, n_heads, key_dim, value_dim, key_decay, token_weight, qk_group, chunks)
    o = torch.empty((T, n_heads * value_dim), dtype=torch.float32, device=q.device) if want_output else None
    if v is None and mode != "delta":
        raise QStreamError(QsError.INVALID_INPUT, "state_scan: only the delta rule walks without values")
    chunk_start = chunk_ids = seq_chunk = chunk_state = chunk_decay = None
    n_chunks = 0
    if chunks is not None:
        chunk_start, chunk_ids, seq_chunk, n_chunks = chunks
        chunk_state = torch.empty((n_chunks, n_heads * value_dim * key_dim), dtype=torch.float32, device=q.device)
        chunk_decay = torch.empty((n_chunks, n_heads * key_dim), dtype=torch.float32, device=q.device)
    per_token = token_decay if token_decay is not None else token_weight
    if mode == "gla" and (decay_logits is None or decay_logits.dtype != torch.float32 or not decay_power > 0):
        raise QStreamError(QsError.INVALID_INPUT, "state_scan: gated linear attention takes float32 decay logits and a positive power")
    if mode == "delta":
        decay_logits = key_decay
        if key_decay.dtype != torch.float32 or token_weight.dtype != torch.float32:
            raise QStreamError(QsError.INVALID_INPUT, "state_scan: the delta rule takes float32 decays and step sizes")
    if mode == "gated" and (token_decay.dtype != torch.float32 or token_decay.stride() != token_weight.stride()):
        raise QStreamError(QsError.INVALID_INPUT, "state_scan: the tokens' decays and weights must be float32 of one layout")
    check(library().qs_state_scan(
        {"decay": 0, "wkv": 1, "gated": 2, "delta": 3, "gla": 4}[mode], ptr(o), o.stride(0) if o is not None else 0, ptr(q), q.stride(0),
        ptr(k), k.stride(0), ptr(v), v.stride(0) if v is not None else 0,
        dtype_code(q), ptr(decay_logits), decay_logits.stride(0) if decay_logits is not None else 0, ptr(head_decay),
        ptr(bonus), _code(bonus), ptr(state), state.stride(0), _int32(seq_start, "seq_start"),
        _int32(seq_slot, "seq_slot"), int(n_seq), T, n_heads, key_dim, value_dim, ACTIVATIONS[in_activation],
        ptr(chunk_start), ptr(chunk_ids), int(n_chunks), ptr(seq_chunk), ptr(chunk_state), ptr(chunk_decay),
        ptr(token_decay), ptr(token_weight), per_token.stride(0) if per_token is not None else 0, float(q_scale),
        int(qk_group), float(decay_power), stream()))
    return o


def _delta_in_chunks(q, k, v, state, seq_slot, n_seq, n_heads, key_dim, value_dim, key_decay, token_weight, qk_group, chunks):
    """The delta rule of a long prompt, its chunks side by side.  A chunk acts on the state it starts from as
    S <- P S + Q: P is what the chunk's walk (values of zero) makes of an identity, Q what it writes from an empty state;
    `qs_delta_chunk_prefix` then gives every chunk its starting state and the slot its last one, and the walk runs once
    more for the outputs.  The same arithmetic as the walk in order, regrouped; nothing is divided by a decay."""
    chunk_start, chunk_ids, seq_chunk, n_chunks = chunks
    dev = q.device
    P = torch.eye(key_dim, dtype=torch.float32, device=dev).repeat(n_chunks, n_heads, 1, 1)
    Q = torch.zeros((n_chunks, n_heads, value_dim, key_dim), dtype=torch.float32, device=dev)
    walk = dict(key_decay=key_decay, token_weight=token_weight, qk_group=qk_group)
    state_scan("delta", q, k, None, P, chunk_start, chunk_ids, n_chunks, n_heads, key_dim, key_dim, want_output=False, **walk)
    state_scan("delta", q, k, v, Q, chunk_start, chunk_ids, n_chunks, n_heads, key_dim, value_dim, want_output=False, **walk)
    start = torch.empty_like(Q)
    check(library().qs_delta_chunk_prefix(ptr(P), ptr(Q), ptr(start), ptr(state), state.stride(0), _int32(seq_chunk, "seq_chunk"),
                                          _int32(seq_slot, "seq_slot"), int(n_seq), n_heads, key_dim, value_dim, stream()))
    return state_scan("delta", q, k, v, start, chunk_start, chunk_ids, n_chunks, n_heads, key_dim, value_dim, **walk)


def delta_prepare(q, k, v, conv_q, conv_k, conv_v, conv_state, a, b, a_log, tok_slot, tok_pos, n_qk_heads, n_heads,
                  key_dim, value_dim, q_scale: float, unit_eps: float):
    """What a gated delta rule needs between its projections and its scan.  q, k [T, n_qk_heads * key_dim] and v
    [T, n_heads * value_dim] (views of one product's result) pass a causal convolution over time per channel (taps
    [channels, n], tap n - 1 weighing the token itself; the n - 1 inputs before a step's first token come from
    `conv_state` [slots, n - 1, channels of q | k | v]) and silu; q and k become unit vectors per head
    (x / sqrt(sum x^2 + unit_eps)), q times q_scale.  a float32 [T, n_heads * key_dim] gives the decays
    exp(-exp(a_log_h) softplus(a)), b float32 [T, n_heads] the step sizes sigmoid(b).  Returns float32 q, k, v, decays,
    step sizes.  Call `conv_state_update` afterwards."""
    T = q.shape[0]
    nq, nv = n_qk_heads * key_dim, n_heads * value_dim
    taps = conv_q.shape[1]
    if q.stride(0) != k.stride(0) or q.stride(0) != v.stride(0) or not (conv_q.dtype == conv_k.dtype == conv_v.dtype):
        raise QStreamError(QsError.INVALID_INPUT, "delta_prepare: q, k, v must be views of one product")
    if a.dtype != torch.float32 or b.dtype != torch.float32:
        raise QStreamError(QsError.INVALID_INPUT, "delta_prepare: the decays' and step sizes' inputs must be float32")
    f32 = dict(dtype=torch.float32, device=q.device)
    qo, ko, vo = torch.empty((T, nq), **f32), torch.empty((T, nq), **f32), torch.empty((T, nv), **f32)
    go, bo = torch.empty((T, n_heads * key_dim), **f32), torch.empty((T, n_heads), **f32)
    check(library().qs_delta_prepare(
        ptr(qo), ptr(ko), ptr(vo), ptr(go), ptr(bo), ptr(q), ptr(k), ptr(v), q.stride(0), dtype_code(q), ptr(conv_q),
        ptr(conv_k), ptr(conv_v), dtype_code(conv_q), taps, ptr(conv_state), conv_state.stride(0) if conv_state is not None else 0,
        ptr(a), a.stride(0), ptr(b), b.stride(0), ptr(a_log), dtype_code(a_log), _int32(tok_slot, "tok_slot"),
        _int32(tok_pos, "tok_pos"), T, n_qk_heads, n_heads, key_dim, value_dim, float(q_scale), float(unit_eps), stream()))
    return qo, ko, vo, go, bo


def conv_state_update(conv_state, q, k, v, n_qk: int, n_v: int, taps: int, seq_start, seq_slot, n_seq: int) -> None:
    """Leave in `conv_state` [slots, taps - 1, 2 n_qk + n_v] the last taps - 1 inputs (q | k | v, before the
    convolution) of what each of the step's sequences held and the step brought."""
    if taps <= 1:
        return
    check(library().qs_conv_state_update(ptr(conv_state), conv_state.stride(0), ptr(q), ptr(k), ptr(v), q.stride(0),
                                         dtype_code(q), int(n_qk), int(n_v), int(taps), _int32(seq_start, "seq_start"),
                                         _int32(seq_slot, "seq_slot"), int(n_seq), stream()))


def mlstm_gates(raw, cap: float, m_state, seq_start, seq_slot, n_seq: int, n_heads: int):
    """The mLSTM's exponential gates as factors of its recurrence.  raw float32 [T, 2 heads] = (input | forget gate
    projections, bias included); log gates i = cap tanh(. / cap), f = logsigmoid(cap tanh(. / cap)); with the running
    maximum m (float32 [slots, heads], 0 for an empty sequence, updated in place): m_t = max(f + m_{t-1}, i),
    a_t = exp(f + m_{t-1} - m_t), b_t = exp(i - m_t).  Returns (a, b, m), each float32 [T, heads]."""
    T = raw.shape[0]
    if raw.dtype != torch.float32 or raw.shape[1] != 2 * n_heads or raw.stride(1) != 1 or m_state.dtype != torch.float32:
        raise QStreamError(QsError.INVALID_INPUT, "mlstm_gates: float32 [T, 2 heads] gates and a float32 state")
    abm = torch.empty((3, T, n_heads), dtype=torch.float32, device=raw.device)
    # scratch for the three-kernel form that steps with long sequences take
    before = torch.empty((n_seq, n_heads), dtype=torch.float32, device=raw.device) if T >= 128 * max(n_seq, 1) else None
    check(library().qs_mlstm_gates(ptr(abm[0]), ptr(abm[1]), ptr(abm[2]), n_heads, ptr(raw), raw.stride(0), float(cap),
                                   ptr(m_state), m_state.stride(0), _int32(seq_start, "seq_start"),
                                   _int32(seq_slot, "seq_slot"), int(n_seq), T, n_heads, ptr(before), stream()))
    return abm[0], abm[1], abm[2]


def mlstm_output(o, m, weight, gate, n_heads: int, value_dim: int, eps: float, out_dtype) -> torch.Tensor:
    """From the gated scan's o [T, heads * (value_dim + 1)] (each head's last element the normaliser's product n.q) and
    the running maxima m [T, heads]: y = o / (max(|n.q|, exp(-m)) + 1e-6), each head divided by its root mean square,
    times weight, times sigmoid(gate) -> [T, heads * value_dim]."""
    rows, _, ldi = _rows(o)
    _, n, ldgate = _rows(gate)
    out = torch.empty((rows, n_heads * value_dim), dtype=out_dtype, device=o.device)
    check(library().qs_mlstm_output(ptr(out), dtype_code(out), out.stride(0), ptr(o), ldi, ptr(m), m.stride(0), ptr(weight),
                                    dtype_code(weight), ptr(gate), dtype_code(gate), ldgate, rows, n_heads, value_dim,
                                    float(eps), stream()))
    return out


def branch_norm(x, weight, eps: float, center: bool, out_dtype=None, branch=None, branch_weight=None, want_norm=True,
                in_place=False):
    """With `branch`: x <- x + norm(branch) * branch_weight (in place; without a weight the plain sum).  With
    `want_norm`: returns h = norm(x) * weight in `out_dtype` (`in_place`: written over x); without a weight h is the
    new x itself in `out_dtype`.  norm is the layer norm without bias (`center`) or the RMS norm, statistics in 32-bit,
    eps inside the root."""
    rows, D, ldx = _rows(x)
    h = None
    if want_norm:
        if weight is not None and weight.numel() != D:
            raise QStreamError(QsError.INVALID_INPUT, f"norm: width {D} but weight {None if weight is None else tuple(weight.shape)}")
        h = x if in_place else torch.empty((rows, D), dtype=out_dtype or x.dtype, device=x.device)
    ldy = 0
    if branch is not None:
        r2, D2, ldy = _rows(branch)
        if (r2, D2) != (rows, D) or (branch_weight is not None and branch_weight.numel() != D):
            raise QStreamError(QsError.INVALID_INPUT, "norm: the branch differs from x in shape")
    check(library().qs_branch_norm(ptr(h), _code(h), h.stride(0) if h is not None else 0, ptr(x), dtype_code(x), ldx,
                                   ptr(branch), _code(branch), ldy, ptr(branch_weight) if branch is not None else None,
                                   _code(branch_weight), ptr(weight) if want_norm else None,
                                   _code(weight) if want_norm else 0, rows, D, float(eps), int(bool(center)), stream()))
    return h


def latent_prepare(dq, q_norm, q_rank, dkv, kv_norm, kv_rank, rot_dim, rot_dims, freq, mag, eps, tok_slot, tok_pos,
                   page_table, page_tokens, k_cache, v_cache, status, interleaved=False):
    """RMS norm of the query latent dq [T, q_rank] -> returned; RMS norm of the key latent dkv[:, :kv_rank] and the
    rotation (pairs (i, i + rot_dims / 2), or (2i, 2i + 1) if `interleaved`; `freq` float64 [rot_dims / 2], cos and sin
    times `mag`) of dkv[:, kv_rank:], written
    into the cache entry as keys [c | rotated part] and values c.  dkv None: a layer that reads another's cache."""
    ref = dq if dq is not None else dkv
    T = ref.shape[0]
    cq = torch.empty((T, q_rank), dtype=dq.dtype, device=dq.device) if dq is not None else None
    check(library().qs_latent_prepare(
        ptr(cq), cq.stride(0) if cq is not None else 0, ptr(dq), dq.stride(0) if dq is not None else 0, ptr(q_norm),
        _code(q_norm), int(q_rank), ptr(dkv), dkv.stride(0) if dkv is not None else 0, ptr(kv_norm), _code(kv_norm),
        int(kv_rank), int(rot_dim), int(rot_dims), ptr(freq), float(mag), float(eps), dtype_code(ref),
        _int32(tok_slot, "tok_slot"), _int32(tok_pos, "tok_pos"),
        _int32(page_table, "page_table") if dkv is not None else None, page_table.shape[1] if dkv is not None else 0,
        int(page_tokens), ptr(k_cache) if dkv is not None else None, ptr(v_cache) if dkv is not None else None, T,
        ptr(status), int(bool(interleaved)), stream()))
    return cq


def latent_q_rotate(q_abs, q, n_heads, dim, rot_dim, kv_rank, rot_dims, freq, mag, tok_slot, tok_pos, interleaved=False) -> None:
    """q [T, heads * (dim + rot_dim)]: every head's last rot_dim elements, rotated, go to q_abs
    [T, heads * (kv_rank + rot_dim)] behind the head's first kv_rank elements."""
    check(library().qs_latent_q_rotate(ptr(q_abs), q_abs.stride(0), ptr(q), q.stride(0), dtype_code(q), int(n_heads),
                                       int(dim), int(rot_dim), int(kv_rank), int(rot_dims), ptr(freq), float(mag),
                                       _int32(tok_slot, "tok_slot"), _int32(tok_pos, "tok_pos"), q.shape[0],
                                       int(bool(interleaved)), stream()))


def head_linear(out, x, w, n_heads: int) -> None:
    """out[:, h * N : (h + 1) * N] = x[:, h * Kx : h * Kx + K] @ w[h].T for every head h, where w is [heads, N, K], out
    is [T, heads * N'] with N' >= N (head h's results at the start of its N' columns) and x is [T, heads * Kx] with
    Kx >= K: one launch for all heads, for steps of few tokens; 32-bit sums."""
    H, N, K = w.shape
    T = x.shape[0]
    if H != n_heads or x.shape[1] % H or out.shape[1] % H or w.dtype != x.dtype or out.dtype != x.dtype or not w.is_contiguous():
        raise QStreamError(QsError.INVALID_INPUT, "head_linear: operands do not fit")
    check(library().qs_head_linear(ptr(out), out.stride(0), out.shape[1] // H, ptr(x), x.stride(0), x.shape[1] // H, ptr(w),
                                   dtype_code(x), T, H, N, K, stream()))


def head_products(out, x, w, n_heads: int) -> None:
    """The same as `head_linear` for steps of many tokens: one matrix product per head (tensor cores where the
    operands allow), all launched by one call and dealt to several streams."""
    from . import gemm_tc
    H, N, K = w.shape
    T = x.shape[0]
    if H != n_heads or x.shape[1] % H or out.shape[1] % H or w.dtype != x.dtype or out.dtype != x.dtype or not w.is_contiguous():
        raise QStreamError(QsError.INVALID_INPUT, "head_products: operands do not fit")
    head_x, head_o = x.shape[1] // H, out.shape[1] // H
    use_tc = gemm_tc.takes(x[:, :K], w[0]) and head_x % 8 == 0
    ws, counters = gemm_tc.scratch(x.device) if use_tc else (None, None)
    rc = bind("qs_head_products", [c_void_p, c_int, c_longlong, c_longlong, c_void_p, c_int, c_longlong, c_longlong, c_void_p, c_int,
                                    c_int, c_int, c_int, c_int, c_int, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p])(
        ptr(out), dtype_code(out), out.stride(0), head_o, ptr(x), dtype_code(x), x.stride(0), head_x, ptr(w), dtype_code(w),
        T, H, N, K, int(use_tc), ptr(ws), ws.numel() if use_tc else 0, ptr(counters), counters.numel() if use_tc else 0,
        ptr(gemm_tc.status_word(x.device)) if use_tc else None, stream())
    count_launches(H - 1)
    check(rc)


# ------------------------------------------------------------------------------- routed experts

def moe_route(z, correction, n_experts, top, groups, keep, scale, gate_col=-1, scores="sigmoid", group_score="top2"):
    """z float32 [T, >= n_experts] router logits.  Returns (idx int32 [T, top], weights float32 [T, top], shared gate
    float32 [T] = sigmoid(z[:, gate_col]) or None): see csrc/moe.cu for the rule.  `scores`: "sigmoid" or "softmax" (over
    all experts); `group_score`: "top2" (the sum of a group's two largest) or "max"; `correction` may be None."""
    T = z.shape[0]
    if z.dtype != torch.float32 or z.stride(1) != 1:
        raise QStreamError(QsError.INVALID_INPUT, "moe_route: router logits must be float32 rows")
    idx = torch.empty((T, top), dtype=torch.int32, device=z.device)
    wts = torch.empty((T, top), dtype=torch.float32, device=z.device)
    gate = torch.empty((T,), dtype=torch.float32, device=z.device) if gate_col >= 0 else None
    check(library().qs_moe_route(ptr(idx), ptr(wts), ptr(gate), ptr(z), z.stride(0), ptr(correction), _code(correction), T,
                                 int(n_experts), int(top), int(groups), int(keep), float(scale), int(gate_col),
                                 {"sigmoid": 0, "softmax": 1}[scores], {"top2": 0, "max": 1}[group_score], stream()))
    return idx, wts, gate


def moe_experts_indirect(x, w_up, w_down, idx, wts, tok_slot, activation, add=None, add_scale=None, glu=None) -> torch.Tensor:
    """sum_j wts[t, j] W_down[idx[t, j]] act(W_up[idx[t, j]] x[t]) (+ add[t] * add_scale[t]) in float32 [T, D]; every
    pair finds its expert's matrices (w_up [E, F, D], w_down [E, D, F]) on the device: for steps of few tokens.
    `glu` = (limit, alpha, shift): gated experts, w_up [E, 2 F, D] holding an expert's gate rows above its up rows; the
    hidden vector is `clamped_glu` of the two halves."""
    T, D, ldx = _rows(x)
    E, F, _ = w_up.shape
    top = idx.shape[1]
    if w_up.dtype != x.dtype or w_down.dtype != x.dtype or not w_up.is_contiguous() or not w_down.is_contiguous():
        raise QStreamError(QsError.INVALID_INPUT, "experts: matrices and activations must share a type")
    hidden = torch.empty((T * top, F), dtype=x.dtype, device=x.device)
    out = torch.empty((T, D), dtype=torch.float32, device=x.device)
    check(library().qs_moe_expert_up(ptr(hidden), F, ptr(x), ldx, ptr(w_up), dtype_code(x), _int32(idx, "idx"),
                                     _int32(tok_slot, "tok_slot"), T, top, D, F, ACTIVATIONS[None if glu else activation], stream()))
    if glu:
        hidden = clamped_glu(hidden, *glu)
        F = F // 2
    check(library().qs_moe_expert_down(ptr(out), D, ptr(hidden), F, ptr(w_down), dtype_code(x), _int32(idx, "idx"), ptr(wts),
                                       _int32(tok_slot, "tok_slot"), ptr(add), _code(add),
                                       add.stride(0) if add is not None else 0, ptr(add_scale), T, top, D, F, stream()))
    return out


def moe_sort(idx, n_experts: int):
    """The (token, choice) pairs ordered by expert: (offsets int32 [E + 1], place_token int32 [pairs], pair_place int32
    [pairs])."""
    T, top = idx.shape
    meta = torch.empty((n_experts + 1 + 2 * T * top,), dtype=torch.int32, device=idx.device)
    offsets, place_token, pair_place = meta[:n_experts + 1], meta[n_experts + 1:n_experts + 1 + T * top], meta[n_experts + 1 + T * top:]
    check(library().qs_moe_sort(ptr(offsets), ptr(place_token), ptr(pair_place), _int32(idx, "idx"), T * top, top,
                                int(n_experts), stream()))
    return offsets, place_token, pair_place


def expert_products(out, x, w_all, offsets) -> None:
    """out[rows of e] = x[rows of e] @ w_all[e].T for every expert e, rows offsets[e] .. offsets[e + 1] (a list on the
    host); w_all is [experts, N, K].  One call launches all the products."""
    import numpy as np
    from . import gemm_tc
    E, N, K = w_all.shape
    rows, K2, lda = _rows(x)
    if K2 != K or out.shape != (rows, N) or out.stride(1) != 1 or not w_all.is_contiguous() or len(offsets) != E + 1:
        raise QStreamError(QsError.INVALID_INPUT, "expert_products: operands do not fit")
    bounds = np.ascontiguousarray(offsets, dtype=np.int32)
    use_tc = gemm_tc.takes(x, w_all[0])
    ws, counters = gemm_tc.scratch(x.device) if use_tc else (None, None)
    rc = bind("qs_expert_products", [c_void_p, c_int, c_longlong, c_void_p, c_int, c_longlong, c_void_p, c_int, c_void_p, c_int,
                                      c_int, c_int, c_int, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p])(
        ptr(out), dtype_code(out), out.stride(0), ptr(x), dtype_code(x), lda, ptr(w_all), dtype_code(w_all),
        bounds.ctypes.data, E, N, K, int(use_tc), ptr(ws), ws.numel() if use_tc else 0, ptr(counters),
        counters.numel() if use_tc else 0, ptr(gemm_tc.status_word(x.device)) if use_tc else None, stream())
    count_launches(sum(1 for e in range(E) if offsets[e + 1] > offsets[e]) - 1)
    check(rc)


def moe_combine(y, pair_place, wts, tok_slot, add=None, add_scale=None) -> torch.Tensor:
    """out[t] = sum_j wts[t, j] y[pair_place[t, j]] (+ add[t] * add_scale[t]) in float32."""
    _, D, ldy = _rows(y)
    T, top = wts.shape
    out = torch.empty((T, D), dtype=torch.float32, device=y.device)
    check(library().qs_moe_combine(ptr(out), D, ptr(y), dtype_code(y), ldy, ptr(pair_place), ptr(wts),
                                   _int32(tok_slot, "tok_slot"), ptr(add), _code(add), add.stride(0) if add is not None else 0,
                                   ptr(add_scale), T, top, D, stream()))
    return out


def token_shift(h, mu, last_row, tok_slot, tok_pos) -> torch.Tensor:
    """out[m] = h + (h shifted down by one token - h) * mu[m]: [n_mix, T, D] in h's type; mu float32 [n_mix, D];
    `last_row` [slots, D] holds each sequence's last row of earlier steps."""
    T, D, ldh = _rows(h)
    n_mix = mu.shape[0]
    out = torch.empty((n_mix, T, D), dtype=h.dtype, device=h.device)
    check(library().qs_token_shift(ptr(out), D, T * D, ptr(h), ldh, dtype_code(h), ptr(mu), ptr(last_row),
                                   last_row.stride(0), _int32(tok_slot, "tok_slot"), _int32(tok_pos, "tok_pos"),
                                   T, D, n_mix, stream()))
    return out


def argmax(logits: torch.Tensor, out=None) -> torch.Tensor:
    rows, V, ld = _rows(logits)
    if logits.dtype != torch.float32:
        raise QStreamError(QsError.INVALID_INPUT, "argmax: logits must be float32")
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    check(library().qs_argmax(ptr(out), ptr(logits), rows, V, ld, stream()))
    return out


def repeat_penalty(logits, recent, n_recent, penalty: float) -> None:
    rows, V, ld = _rows(logits)
    check(library().qs_repeat_penalty(ptr(logits), rows, V, ld, _int32(recent, "recent"), recent.shape[1],
                                      _int32(n_recent, "n_recent"), float(penalty), stream()))


def sample(logits, temperature: float, top_k: int, top_p: float, draws, out=None) -> torch.Tensor:
    rows, V, ld = _rows(logits)
    if logits.dtype != torch.float32 or draws.dtype != torch.float32 or draws.numel() != rows:
        raise QStreamError(QsError.INVALID_INPUT, "sample: logits and draws must be float32, one draw per row")
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    check(library().qs_sample(ptr(out), ptr(logits), rows, V, ld, float(temperature), int(top_k),
                              float(top_p), ptr(draws), stream()))
    return out


# ------------------------------------------------------------------------------- utility kernels

_FILL_TYPES = {torch.float32: 0, torch.bfloat16: 1, torch.int32: 2}
_CONVERT_IN = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def random_fill(out: torch.Tensor, key: int, kind: int, a: float, first: int = 0) -> torch.Tensor:
    """Fill `out` (contiguous; float32, bfloat16 or int32) with elements first.. of the stream `key`:
    kind 0 N(0, a), kind 1 1 + U(-a, a), kind 2 integers below a."""
    if not out.is_contiguous() or out.dtype not in _FILL_TYPES:
        raise QStreamError(QsError.INVALID_INPUT, "random fill: need a contiguous float32, bfloat16 or int32 tensor")
    check(library().qs_random_fill(ptr(out), _FILL_TYPES[out.dtype], out.numel(), int(key) & (2**64 - 1), int(kind),
                                   float(a), int(first), stream()))
    return out


def convert(src: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """A copy of `src` (float32, bfloat16 or float16, contiguous) in float32 or bfloat16, rounded to
    nearest even."""
    if not src.is_contiguous() or src.dtype not in _CONVERT_IN or dtype not in (torch.float32, torch.bfloat16):
        raise QStreamError(QsError.INVALID_INPUT, f"convert: {src.dtype} -> {dtype} is not offered")
    out = torch.empty(src.shape, dtype=dtype, device=src.device)
    check(library().qs_convert(ptr(out), _FILL_TYPES[dtype], ptr(src), _CONVERT_IN[src.dtype], src.numel(), stream()))
    return out


def check_finite(x: torch.Tensor, tag: int, record: torch.Tensor, row_slot=None) -> None:
    """Scan x [rows, width]; the first value that is not finite sets record = (1, tag, row, column).
    Rows with a negative `row_slot` entry are skipped."""
    rows, width, ld = _rows(x)
    check(library().qs_check_finite(ptr(x), dtype_code(x), rows, width, ld, int(tag),
                                    _int32(row_slot, "row_slot") if row_slot is not None else None,
                                    _int32(record, "record"), stream()))


def canary_fill(words: torch.Tensor, pattern: int) -> None:
    check(library().qs_canary_fill(ptr(words), words.numel() * words.element_size() // 4, pattern & 0xFFFFFFFF, stream()))


def canary_check(words: torch.Tensor, pattern: int, damaged: torch.Tensor) -> None:
    """Adds the number of damaged guard words to damaged[0] (int32 [2] on the device)."""
    check(library().qs_canary_check(ptr(words), words.numel() * words.element_size() // 4, pattern & 0xFFFFFFFF,
                                    _int32(damaged, "damaged"), stream()))


def take_tokens(dst: torch.Tensor, src: torch.Tensor, idx: torch.Tensor, n: int) -> None:
    """dst[j] = src[idx[j]] for j < n where idx[j] >= 0 (all int32, on the device)."""
    check(library().qs_take_tokens(_int32(dst, "dst"), _int32(src, "src"), _int32(idx, "idx"), int(n),
                                   src.numel(), stream()))


def zero_pages(storage: torch.Tensor, pages: torch.Tensor) -> None:
    """Zero the listed pages (int32, device) of every entry of a cache tensor [entries, pages, ...]."""
    if not storage.is_contiguous():
        raise QStreamError(QsError.INVALID_INPUT, "zero pages: the cache tensor must be contiguous")
    page_bytes = storage.stride(1) * storage.element_size()
    check(library().qs_zero_pages(ptr(storage), storage.stride(0) * storage.element_size(), page_bytes,
                                  storage.shape[0], _int32(pages, "pages"), pages.numel(), storage.shape[1], stream()))


def selftest_bounded_wait(status: torch.Tensor, polls: int = 2000) -> None:
    """Launch a kernel that waits, with the library's polling loop, on a barrier nothing completes: after
    `polls` polls it records code 199 in `status` (int32 on the device) and returns."""
    check(library().qs_selftest_bounded_wait(_int32(status, "status"), int(polls), stream()))
