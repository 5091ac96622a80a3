"""Python faces of the CUDA launchers: tensors in, one kernel launch out.

Every function checks devices, dtypes and layout, passes raw pointers and the current
stream to the C launcher, and raises on a refused size.  There is no CPU path: a tensor
that is not on a CUDA device is an error, and so is a missing compiler or library.
Shapes in the docstrings use N = rows (tokens) of the step, R = entries (requests) of the
step, H = model width.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import build

_c_int, _c_float, _c_void_p, _c_ll = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong

_ERR = {1: "a size the kernel does not take", 2: "the launch failed", 3: "a dtype the kernel does not take"}


class KernelError(RuntimeError):
    pass


def _check(rc: int, what: str) -> None:
    if rc != 0:
        detail = ""
        if rc == 2:
            detail = f" ({torch.cuda.get_device_name()}: the kernels are built for sm_100a only)"
        raise KernelError(f"{what}: {_ERR.get(rc, rc)}{detail}")


def _ptr(t: Optional[torch.Tensor], what: str = "tensor") -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError(f"{what} is on {t.device}: neurogrid_b200 kernels run on a CUDA device only "
                          "(there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")
    return t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_current_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """The current stream's handle (the capture stream while a graph is being captured).  Asked
    from the C layer directly: a step launches a hundred kernels and more, and building a
    stream object for each costs as much as the launch."""
    if _raw_stream is not None and _current_device is not None:
        return _raw_stream(_current_device())
    return torch.cuda.current_stream().cuda_stream


def _act_flag(t: torch.Tensor, what: str) -> int:
    if t.dtype == torch.bfloat16:
        return 1
    if t.dtype == torch.float32:
        return 0
    raise KernelError(f"{what} has dtype {t.dtype}; the kernels take float32 or bfloat16")


def _f32(t: Optional[torch.Tensor], what: str):
    if t is not None and t.dtype != torch.float32:
        raise KernelError(f"{what} must be float32, got {t.dtype}")
    return t


def _i32(t: Optional[torch.Tensor], what: str):
    if t is not None and t.dtype != torch.int32:
        raise KernelError(f"{what} must be int32, got {t.dtype}")
    return t


_fn_cache = {}


def _fn(lib_name: str, symbol: str, argtypes, defines=None):
    key = (lib_name, symbol, tuple(sorted((defines or {}).items())))
    f = _fn_cache.get(key)
    if f is None:
        f = getattr(build.load(lib_name, defines), symbol)
        f.argtypes = argtypes
        f.restype = _c_int
        _fn_cache[key] = f
    return f


# ----------------------------------------------------------------------------- elementwise
def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, status: torch.Tensor,
          accumulate: bool = False, scale: float = 1.0) -> None:
    """out[N,H] (float32) = table[tokens] * scale; a token outside the table gives zeros and a status bit.
    ``accumulate``: out += table[tokens] instead (``tokens`` are then positions into a table of
    learned positions; one outside the table sets the bad-position bit)."""
    n, H = out.shape
    V = table.shape[0]
    f = _fn("elementwise", "ng_embed", [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int,
                                       _c_void_p, _c_int, _c_int, _c_float, _c_void_p])
    _f32(out, "embed out"), _i32(tokens, "tokens"), _i32(status, "status")
    _check(f(_ptr(table, "embedding table"), _act_flag(table, "embedding table"), _ptr(tokens), _ptr(out),
             n, H, V, _ptr(status), int(accumulate), 4 if accumulate else 1, float(scale), _stream()), "embed")


def _partials(delta: Optional[torch.Tensor], h: torch.Tensor, act: int):
    """(delta_f32, n_partials, stride): ``delta`` is [N,H] of the activation dtype, or a stack
    [S,N,H] of float32 partial sums (split-K products) that are added in ascending order."""
    if delta is None:
        return 0, 1, 0
    if delta.dim() == 3:
        if delta.dtype != torch.float32 or delta.shape[1:] != h.shape:
            raise KernelError("a stack of partial sums must be float32 [S, N, H]")
        return 1, delta.shape[0], delta.shape[1] * delta.shape[2]
    if delta.shape != h.shape or _act_flag(delta, "delta") != act:
        raise KernelError("delta must have the residual stream's shape and the activation dtype")
    return (1 if delta.dtype == torch.float32 else 0), 1, 0


def gather_tokens(dst: torch.Tensor, src: torch.Tensor, idx: torch.Tensor) -> None:
    """dst[i] = src[idx[i]] where idx[i] >= 0 (int32 all): device-sampled tokens into a step's tokens."""
    _i32(dst, "dst"), _i32(src, "src"), _i32(idx, "idx")
    f = _fn("elementwise", "ng_gather_i32", [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p])
    _check(f(_ptr(dst), _ptr(src), _ptr(idx), dst.numel(), _stream()), "gather_tokens")


def add_rmsnorm(h: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, out: torch.Tensor,
                eps: float, rows: Optional[torch.Tensor] = None) -> None:
    """h[N,H] float32 (+= delta if given); out[i] = rmsnorm(h[rows[i] if rows else i]) * weight.
    ``delta`` may be a float32 stack [S,N,H] of partial sums."""
    n_out, H = out.shape
    act = _act_flag(out, "norm out")
    _f32(h, "residual stream"), _f32(weight, "norm weight"), _i32(rows, "rows")
    d32, n_part, stride = _partials(delta, h, act)
    f = _fn("elementwise", "ng_add_rmsnorm", [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int,
                                             _c_int, _c_float, _c_int, _c_int, _c_int, _c_ll, _c_void_p])
    _check(f(_ptr(h), _ptr(delta), _ptr(weight), _ptr(out), _ptr(rows), n_out, H, float(eps), act, d32, n_part,
             stride, _stream()), "add_rmsnorm")


def add_layernorm(h: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, out: torch.Tensor,
                  eps: float, rows: Optional[torch.Tensor] = None, post: Optional[torch.Tensor] = None) -> None:
    """h[N,H] float32 (+= delta if given, as for ``add_rmsnorm``); out[i] = (x - mean(x)) * rsqrt(var(x) + eps) * weight
    for x = h[rows[i] if rows else i], var the mean of the squared deviations, no bias.  ``post`` (float32 [H]) is
    added to h after the norm has read it: a vector that belongs to what the layer adds to the stream later."""
    n_out, H = out.shape
    act = _act_flag(out, "norm out")
    _f32(h, "residual stream"), _f32(weight, "norm weight"), _i32(rows, "rows"), _f32(post, "post")
    d32, n_part, stride = _partials(delta, h, act)
    f = _fn("elementwise", "ng_add_layernorm", [_c_void_p] * 6 + [_c_int, _c_int, _c_float, _c_int, _c_int, _c_int, _c_ll,
                                               _c_void_p])
    _check(f(_ptr(h), _ptr(delta), _ptr(weight), _ptr(out), _ptr(rows), _ptr(post), n_out, H, float(eps), act, d32, n_part,
             stride, _stream()), "add_layernorm")


def residual_add(h: torch.Tensor, delta: torch.Tensor) -> None:
    """h (float32) += delta (or the sum of a float32 stack [S,N,H])."""
    _f32(h, "residual stream")
    n_part = delta.shape[0] if delta.dim() == 3 else 1
    f = _fn("elementwise", "ng_residual_add", [_c_void_p, _c_void_p, _c_ll, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(h), _ptr(delta), h.numel(), int(delta.dtype == torch.bfloat16), n_part, _stream()), "residual_add")


GATE_ACTIVATIONS = ("silu", "gelu_tanh")


def _column_block(out: torch.Tensor, what: str) -> int:
    """Row pitch of ``out`` [N, I], which may be a block of columns of a wider row-major buffer."""
    if out.dim() != 2 or out.stride(1) != 1 or not out.is_cuda:
        raise KernelError(f"{what} must be a CUDA matrix, or a block of columns of one")
    return out.stride(0) if out.shape[0] > 1 else max(out.stride(0), out.shape[1])


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu") -> None:
    """out[N,I] = act(gate_up[:, :I]) * gate_up[:, I:], act = silu or the tanh form of gelu.  ``out`` may be a block
    of columns of a wider buffer."""
    n, I = out.shape
    if gate_up.shape != (n, 2 * I) or gate_up.dtype != out.dtype or activation not in GATE_ACTIVATIONS:
        raise KernelError(f"swiglu: gate_up {tuple(gate_up.shape)} does not match out {tuple(out.shape)}")
    ldo = _column_block(out, "swiglu out")
    f = _fn("elementwise", "ng_swiglu", [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(gate_up), out.data_ptr(), n, I, ldo, int(activation == "gelu_tanh"), _act_flag(out, "swiglu out"),
             _stream()), "swiglu")


# ----------------------------------------------------------------------------- float32 product
def gemm_f32(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out[M,N] = a[M,K] @ w[N,K]^T (+ bias), float32 throughout, FFMA only."""
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm_f32: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit")
    _f32(a, "a"), _f32(w, "w"), _f32(bias, "bias"), _f32(out, "out")
    f = _fn("gemm_f32", "ng_gemm_f32", [_c_void_p] * 4 + [_c_int] * 6 + [_c_void_p])
    _check(f(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), M, N, K, K, K, N, _stream()), "gemm_f32")


# ----------------------------------------------------------------------------- short convolution
def shortconv(p: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
              out: torch.Tensor, cu_q: torch.Tensor, ctx_before: torch.Tensor, slots: torch.Tensor,
              n_entries: int, max_q: int) -> None:
    """p[N,3H] = B|C|x (or a float32 stack [S,N,3H] of partial sums); out[N,H] = C * conv(B*x);
    state[slots, L-1, H] float32 carries B*x."""
    n, H = out.shape
    L = weight.shape[1]
    n_part, stride = _stack(p, (n, 3 * H), out.dtype, "shortconv input")
    if weight.shape[0] != H or state.shape[1:] != (L - 1, H):
        raise KernelError("shortconv: shapes do not fit")
    _f32(weight, "conv weight"), _f32(bias, "conv bias"), _f32(state, "conv state")
    _i32(cu_q, "cu_q"), _i32(ctx_before, "ctx_before"), _i32(slots, "slots")
    if not 2 <= L <= 8:
        raise KernelError(f"shortconv: width {L} is outside [2, 8]")
    f = _fn("shortconv", "ng_shortconv", [_c_void_p] * 8 + [_c_int] * 6 + [_c_ll, _c_void_p], {"NG_CONV_L": L})
    _check(f(_ptr(p), _ptr(weight), _ptr(bias), _ptr(state), _ptr(out), _ptr(cu_q), _ptr(ctx_before),
             _ptr(slots), n_entries, max_q, H, L, _act_flag(out, "conv out"), n_part, stride, _stream()), "shortconv")


def _stack(t: torch.Tensor, shape, act_dtype, what: str):
    """(n_partials, stride) of an input that is [*shape] in the activation dtype or a float32
    stack [S, *shape] of partial sums."""
    if t.dim() == len(shape) + 1:
        if t.dtype != torch.float32 or tuple(t.shape[1:]) != tuple(shape):
            raise KernelError(f"{what}: a stack of partial sums must be float32 [S, {', '.join(map(str, shape))}]")
        n = 1
        for d in shape:
            n *= d
        return t.shape[0], n
    if tuple(t.shape) != tuple(shape) or t.dtype != act_dtype:
        raise KernelError(f"{what}: expected {tuple(shape)} {act_dtype}, got {tuple(t.shape)} {t.dtype}")
    return 1, 0


# ----------------------------------------------------------------------------- attention
def rope_pairs(head_dim: int) -> int:
    """The rope kernel's specialisation for a head size: pairs of a head that one lane handles."""
    if head_dim <= 0 or head_dim % 2 or head_dim > 256:
        raise KernelError(f"rope_cache: head size {head_dim} is not an even number up to 256")
    return 1 if head_dim <= 64 else 2 if head_dim <= 128 else 4


def rope_cache(qkv: torch.Tensor, q_out: torch.Tensor, q_weight: Optional[torch.Tensor],
               k_weight: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor], half_pairing: bool,
               pos_scale: float, k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
               table: torch.Tensor, positions: torch.Tensor, row_entry: torch.Tensor, n_heads: int,
               n_kv_heads: int, head_dim: int, eps: float, status: torch.Tensor) -> None:
    """Per-head norm of q and k, rotation, q -> q_out[N, nH*hd], k and v -> pages[P, nKV, page, hd].

    ``n_kv_heads`` 0 (with no pages) handles a layer that only reads another layer's cache.
    """
    n = q_out.shape[0]
    if q_out.shape != (n, n_heads * head_dim):
        raise KernelError("rope_cache: shapes do not fit")
    n_part, stride = _stack(qkv, (n, (n_heads + 2 * n_kv_heads) * head_dim), q_out.dtype, "rope_cache input")
    act = _act_flag(q_out, "q_out")
    page_size = num_pages = 1
    if n_kv_heads:
        if k_pages.dtype != q_out.dtype or k_pages.shape != v_pages.shape or k_pages.shape[1] != n_kv_heads \
                or k_pages.shape[3] != head_dim:
            raise KernelError("rope_cache: pages do not fit the projection")
        num_pages, page_size = k_pages.shape[0], k_pages.shape[2]
    _f32(q_weight, "q norm weight"), _f32(k_weight, "k norm weight"), _f32(inv_freq, "inv_freq")
    _i32(table, "table"), _i32(positions, "positions"), _i32(row_entry, "row_entry"), _i32(status, "status")
    f = _fn("rope_cache", "ng_rope_cache",
            [_c_void_p] * 5 + [_c_int, _c_float] + [_c_void_p] * 3 + [_c_int] + [_c_void_p] * 2 + [_c_int] * 6
            + [_c_float, _c_void_p, _c_int, _c_int, _c_ll, _c_void_p], {"NG_ROPE_PAIRS": rope_pairs(head_dim)})
    _check(f(_ptr(qkv), _ptr(q_out), _ptr(q_weight), _ptr(k_weight), _ptr(inv_freq), int(half_pairing),
             float(pos_scale), _ptr(k_pages), _ptr(v_pages), _ptr(table), table.shape[1], _ptr(positions),
             _ptr(row_entry), n, n_heads, n_kv_heads, head_dim, page_size, num_pages, float(eps), _ptr(status),
             act, n_part, stride, _stream()), "rope_cache")


def attention_generic(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, table: torch.Tensor,
                      positions: torch.Tensor, row_entry: torch.Tensor, out: torch.Tensor, n_heads: int,
                      window: Optional[int], scale: float, slopes: Optional[torch.Tensor] = None) -> None:
    """out[N, nH*hd] = softmax(q k^T * scale - bias, keys max(0,pos-window+1)..pos) v over the pages;
    bias = slopes[head] * (query position - key position) when ``slopes`` (float32 [nH]) is given."""
    n = q.shape[0]
    num_pages, n_kv, page_size, hd = k_pages.shape
    if q.shape != (n, n_heads * hd) or out.shape != q.shape or q.dtype != k_pages.dtype or out.dtype != q.dtype:
        raise KernelError("attention: shapes or dtypes do not fit")
    _i32(table, "table"), _i32(positions, "positions"), _i32(row_entry, "row_entry")
    f = _fn("attention_generic", "ng_attention_generic",
            [_c_void_p] * 4 + [_c_int] + [_c_void_p] * 3 + [_c_int] * 7 + [_c_float, _c_void_p, _c_int, _c_void_p])
    _check(f(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(table), table.shape[1], _ptr(positions),
             _ptr(row_entry), _ptr(out), n, n_heads, n_kv, hd, page_size, num_pages, int(window or 0),
             float(scale), _slopes(slopes, n_heads), _act_flag(q, "q"), _stream()), "attention_generic")


def _slopes(slopes: Optional[torch.Tensor], n_heads: int) -> Optional[int]:
    if slopes is None:
        return None
    if slopes.dtype != torch.float32 or slopes.numel() != n_heads:
        raise KernelError(f"score slopes must be float32 [{n_heads}]")
    return _ptr(slopes, "score slopes")


def attn_prefill_bf16(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, table: torch.Tensor,
                      cu_q: torch.Tensor, ctx_before: torch.Tensor, out: torch.Tensor, n_entries: int, max_q: int,
                      n_heads: int, window: Optional[int], scale: float, skip_single: bool,
                      slopes: Optional[torch.Tensor] = None) -> None:
    """Tensor-core flash attention of the step's portions (bfloat16); entries of one token are
    left to the decode kernel when ``skip_single``."""
    num_pages, n_kv, page_size, hd = k_pages.shape
    if q.dtype != torch.bfloat16 or k_pages.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attn_prefill_bf16 takes bfloat16 tensors")
    if q.shape[1] != n_heads * hd or out.shape != q.shape or v_pages.shape != k_pages.shape:
        raise KernelError("attn_prefill_bf16: shapes do not fit")
    _i32(table, "table"), _i32(cu_q, "cu_q"), _i32(ctx_before, "ctx_before")
    f = _fn("attention_bf16", "ng_attn_prefill_bf16",
            [_c_void_p] * 4 + [_c_int] + [_c_void_p] * 3 + [_c_int] * 8 + [_c_float, _c_int, _c_void_p, _c_void_p],
            {"NG_HEAD_DIM": hd})
    _check(f(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(table), table.shape[1], _ptr(cu_q), _ptr(ctx_before),
             _ptr(out), n_entries, max_q, n_heads, n_kv, hd, page_size, num_pages, int(window or 0), float(scale),
             int(skip_single), _slopes(slopes, n_heads), _stream()), "attn_prefill_bf16")


ATTN_BACKEND = os.environ.get("NEUROGRID_B200_ATTN", "sm100")     # "sm100": tcgen05 prefill kernel; "mma": mma.sync


def attn_prefill_sm100_takes(head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 prefill kernel takes this shape (else the mma.sync kernel runs)."""
    return ATTN_BACKEND == "sm100" and head_dim == 64 and page_size in (8, 16, 32, 64)


def attn_prefill_scratch_floats(n_rows: int, n_heads: int, head_dim: int, n_splits: int) -> int:
    """float32 values the tcgen05 prefill kernel needs when it cuts the keys into ``n_splits`` runs."""
    return n_rows * n_heads * n_splits * (head_dim + 2) if n_splits > 1 else 0


def attn_prefill_sm100(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, table: torch.Tensor,
                       cu_q: torch.Tensor, ctx_before: torch.Tensor, out: torch.Tensor, n_entries: int, max_q: int,
                       n_heads: int, window: Optional[int], scale: float, skip_single: bool,
                       slopes: Optional[torch.Tensor] = None, scratch: Optional[torch.Tensor] = None,
                       n_splits: int = 1) -> None:
    """Flash attention of the step's portions on tcgen05/TMA/TMEM (bfloat16, head size 64).
    ``n_splits`` > 1: the keys of every block of rows are cut into that many runs, each a block of
    its own, merged by a second kernel through ``scratch`` (``attn_prefill_scratch_floats`` float32
    values); for long contexts whose blocks would fill the GPU unevenly."""
    num_pages, n_kv, page_size, hd = k_pages.shape
    if q.dtype != torch.bfloat16 or k_pages.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attn_prefill_sm100 takes bfloat16 tensors")
    if q.shape[1] != n_heads * hd or out.shape != q.shape or v_pages.shape != k_pages.shape:
        raise KernelError("attn_prefill_sm100: shapes do not fit")
    need = attn_prefill_scratch_floats(q.shape[0], n_heads, hd, n_splits)
    if need and (scratch is None or scratch.numel() < need or scratch.dtype != torch.float32):
        raise KernelError(f"attn_prefill_sm100 needs {need} float32 values of scratch")
    _i32(table, "table"), _i32(cu_q, "cu_q"), _i32(ctx_before, "ctx_before")
    f = _fn("attention_sm100", "ng_attn_prefill_sm100",
            [_c_void_p] * 4 + [_c_int] + [_c_void_p] * 3 + [_c_int] * 9 + [_c_float, _c_int, _c_void_p, _c_void_p, _c_int,
                                                                             _c_void_p, _c_void_p])
    _check(f(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(table), table.shape[1], _ptr(cu_q), _ptr(ctx_before),
             _ptr(out), q.shape[0], n_entries, max_q, n_heads, n_kv, hd, page_size, num_pages, int(window or 0),
             float(scale), int(skip_single), _slopes(slopes, n_heads), _ptr(scratch) if need else None, int(n_splits),
             _ptr(_gemm_status(q.device)), _stream()),
           "attn_prefill_sm100")


def attn_decode_scratch_floats(n_rows: int, n_heads: int, head_dim: int, n_splits: int) -> int:
    return n_rows * n_heads * n_splits * (head_dim + 2) if n_splits > 1 else 0


def attn_decode_bf16(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, table: torch.Tensor,
                     cu_q: torch.Tensor, ctx_before: torch.Tensor, out: torch.Tensor,
                     scratch: Optional[torch.Tensor], n_entries: int, n_heads: int, window: Optional[int],
                     scale: float, n_splits: int, max_ctx: int, slopes: Optional[torch.Tensor] = None) -> None:
    """Split-context attention of the entries that bring one token (bfloat16).  ``max_ctx`` bounds
    the keys any entry sees (its tokens after the step); ``scratch`` holds
    ``attn_decode_scratch_floats`` float32 values when ``n_splits`` > 1."""
    num_pages, n_kv, page_size, hd = k_pages.shape
    if q.dtype != torch.bfloat16 or k_pages.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attn_decode_bf16 takes bfloat16 tensors")
    if q.shape[1] != n_heads * hd or out.shape != q.shape or v_pages.shape != k_pages.shape:
        raise KernelError("attn_decode_bf16: shapes do not fit")
    need = attn_decode_scratch_floats(q.shape[0], n_heads, hd, n_splits)
    if need and (scratch is None or scratch.numel() < need or scratch.dtype != torch.float32):
        raise KernelError(f"attn_decode_bf16 needs {need} float32 values of scratch")
    _i32(table, "table"), _i32(cu_q, "cu_q"), _i32(ctx_before, "ctx_before")
    f = _fn("attention_bf16", "ng_attn_decode_bf16",
            [_c_void_p] * 4 + [_c_int] + [_c_void_p] * 4 + [_c_int] * 7 + [_c_float, _c_int, _c_int, _c_void_p, _c_void_p],
            {"NG_HEAD_DIM": hd})
    _check(f(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(table), table.shape[1], _ptr(cu_q), _ptr(ctx_before),
             _ptr(out), _ptr(scratch), n_entries, n_heads, n_kv, hd, page_size, num_pages, int(window or 0),
             float(scale), int(n_splits), int(max_ctx), _slopes(slopes, n_heads), _stream()), "attn_decode_bf16")


# ----------------------------------------------------------------------------- attention with float32 weights
def qkv_prep(qkv: torch.Tensor, q_out: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
             inv_freq: Optional[torch.Tensor], k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
             table: torch.Tensor, positions: torch.Tensor, row_entry: torch.Tensor, n_q: int, n_k: int, n_v: int,
             dim: int, vdim: int, eps: float, status: torch.Tensor, *, whole: bool = False, q_temp_coef: float = 0.0,
             q_temp_every: int = 1, half_pairing: bool = False, unit_norm: bool = False) -> None:
    """qkv[N, (n_q + n_k) * dim + n_v * vdim]: every q and k head (a map of a head counts as one) gets its RMS norm
    over ``dim`` (if its weight is given; float32, shared by all heads) and the rotation of its first
    2 * len(inv_freq) coordinates in pairs (2i, 2i+1) by position * inv_freq[i]; q -> q_out[N, n_q * dim],
    k -> k_pages[P, n_k, page, dim], v -> v_pages[P, n_v, page, vdim].  n_k = n_v = 0 (no pages): a layer that
    reads another layer's keys and values.  ``whole``: ONE norm over all of a row's q (n_q * dim values) and one over
    all of its k, the weights then float32 [n_q * dim] and [n_k * dim].  ``q_temp_coef`` c, ``q_temp_every`` m: q is
    multiplied by 1 + c * ln(floor((position + 1) / m) + 1) after its norm.  ``half_pairing``: the rotated coordinates
    pair as (i, i + rot_dims/2).  ``unit_norm`` (without norm weights): every q and k head is divided by its root mean
    square all the same.  ``qkv`` may have further columns behind v; they are not read."""
    n = q_out.shape[0]
    if q_out.shape != (n, n_q * dim) or qkv.dim() != 2 or qkv.shape[0] != n \
            or qkv.shape[1] < (n_q + n_k) * dim + n_v * vdim or qkv.dtype != q_out.dtype:
        raise KernelError("qkv_prep: shapes or dtypes do not fit")
    page_size = num_pages = 1
    if n_k or n_v:
        if k_pages.dtype != q_out.dtype or v_pages.dtype != q_out.dtype or k_pages.shape[1:] != (n_k, k_pages.shape[2], dim) \
                or v_pages.shape != (k_pages.shape[0], n_v, k_pages.shape[2], vdim):
            raise KernelError("qkv_prep: pages do not fit the projection")
        num_pages, page_size = k_pages.shape[0], k_pages.shape[2]
    _f32(q_weight, "q norm weight"), _f32(k_weight, "k norm weight"), _f32(inv_freq, "inv_freq")
    _i32(table, "table"), _i32(positions, "positions"), _i32(row_entry, "row_entry"), _i32(status, "status")
    rot_dims = 2 * inv_freq.numel() if inv_freq is not None else 0
    if whole and (q_weight is None or q_weight.numel() != n_q * dim or (n_k and (k_weight is None or k_weight.numel() != n_k * dim))):
        raise KernelError("qkv_prep: a norm over the whole projection needs weights of the projection's length")
    f = _fn("mapped_attention", "ng_qkv_prep", [_c_void_p] * 5 + [_c_int] + [_c_void_p] * 3 + [_c_int] + [_c_void_p] * 2
            + [_c_int] * 8 + [_c_float, _c_void_p, _c_int, _c_float, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(qkv), _ptr(q_out), _ptr(q_weight), _ptr(k_weight), _ptr(inv_freq), rot_dims,
             _ptr(k_pages) if n_k else None, _ptr(v_pages) if n_v else None, _ptr(table), table.shape[1], _ptr(positions),
             _ptr(row_entry), n, n_q, n_k, n_v, dim, vdim, page_size, num_pages, float(eps), _ptr(status),
             int(bool(whole)), float(q_temp_coef), int(q_temp_every), qkv.shape[1], int(bool(half_pairing)),
             int(bool(unit_norm)), _act_flag(q_out, "q_out"), _stream()), "qkv_prep")


def mapped_attention_partial_floats(n_rows: int, n_heads: int, n_maps: int, vdim: int, n_splits: int) -> int:
    return n_rows * n_heads * n_splits * n_maps * (vdim + 2) if n_splits > 1 else 0


def mapped_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, table: torch.Tensor,
                     positions: torch.Tensor, row_entry: torch.Tensor, out: torch.Tensor, n_heads: int, n_maps: int,
                     window: Optional[int], keep_first: int, scale: float, softcap: float, lam: float, head_norm: bool,
                     post_scale: float, eps: float, n_splits: int = 1, partial: Optional[torch.Tensor] = None,
                     slopes: Optional[torch.Tensor] = None, sinks: Optional[torch.Tensor] = None, chunk: int = 0) -> None:
    """Attention with float32 scores and weights over keys [P, G * n_maps, page, dim] and values [P, G, page, vdim]:
    per head and map m, a_m = softmax(cap(scale * q_m . k_m)) v over the keys j <= pos with pos - j < window or
    j < keep_first (window None: all), cap(s) = softcap * tanh(s / softcap) (softcap 0: none); the head's output is
    a_0 (one map) or a_0 - lam * a_1 (two), then, with ``head_norm``, over its root mean square (eps) times
    ``post_scale``.  ``out`` [N, n_heads * vdim] may be a block of columns of a wider buffer.  ``n_splits`` > 1 cuts
    every row's keys into runs, a block each, merged through ``partial`` (float32,
    ``mapped_attention_partial_floats`` values): for steps of few rows.  ``slopes`` (float32 [n_heads]): slope[head] *
    (position - key position) is taken off every score; ``sinks`` (float32 [n_heads]): every softmax's denominator
    also holds exp(sink[head]), a term that has no key and no value.  ``chunk`` > 0: a row also sees only the keys of
    its own chunk, floor(j / chunk) = floor(pos / chunk)."""
    n = q.shape[0]
    num_pages, n_k, page_size, dim = k_pages.shape
    n_g, vdim = v_pages.shape[1], v_pages.shape[3]
    if n_k != n_g * n_maps or q.shape != (n, n_heads * n_maps * dim) or out.shape != (n, n_heads * vdim) \
            or q.dtype != k_pages.dtype or out.dtype != q.dtype or v_pages.dtype != q.dtype \
            or v_pages.shape[0] != num_pages or v_pages.shape[2] != page_size:
        raise KernelError("mapped_attention: shapes or dtypes do not fit")
    _i32(table, "table"), _i32(positions, "positions"), _i32(row_entry, "row_entry"), _f32(partial, "partial")
    need = mapped_attention_partial_floats(n, n_heads, n_maps, vdim, n_splits)
    if need and (partial is None or partial.numel() < need):
        raise KernelError(f"mapped_attention: the runs need {need} float32 values")
    f = _fn("mapped_attention", "ng_mapped_attention", [_c_void_p] * 4 + [_c_int] + [_c_void_p] * 3 + [_c_int, _c_void_p]
            + [_c_int] * 11 + [_c_float] * 5 + [_c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(table), table.shape[1], _ptr(positions), _ptr(row_entry),
             out.data_ptr(), _column_block(out, "attention out"), _ptr(partial) if need else None, n, n_heads, n_g, n_maps,
             dim, vdim, page_size, num_pages, int(window or 0), int(keep_first), int(n_splits), float(scale),
             float(softcap or 0.0), float(lam), float(post_scale), float(eps), int(bool(head_norm)),
             _slopes(slopes, n_heads), _slopes(sinks, n_heads), int(chunk or 0), _act_flag(q, "q"), _stream()), "mapped_attention")


MAPPED_BACKEND = os.environ.get("NEUROGRID_B200_MAPPED", "mma")     # "mma": tensor-core kernel for long bfloat16 steps; "ffma"


def mapped_attention_mma_takes(dim: int, vdim: int, dtype) -> bool:
    """Whether the tensor-core kernel takes these sizes (bfloat16; key and value sizes multiples of 16 up to 128)."""
    return MAPPED_BACKEND == "mma" and dtype == torch.bfloat16 and dim % 16 == 0 and vdim % 16 == 0 \
        and 16 <= dim <= 128 and 16 <= vdim <= 128


def mapped_attention_mma(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, table: torch.Tensor,
                         cu_q: torch.Tensor, ctx_before: torch.Tensor, out: torch.Tensor, n_entries: int, max_q: int,
                         n_heads: int, n_maps: int, window: Optional[int], keep_first: int, scale: float, softcap: float,
                         lam: float, head_norm: bool, post_scale: float, eps: float,
                         slopes: Optional[torch.Tensor] = None, sinks: Optional[torch.Tensor] = None, chunk: int = 0) -> None:
    """``mapped_attention`` for long bfloat16 steps on the tensor cores: scores are float32 sums of exact bfloat16
    products, the float32 softmax weights enter the weighted sum as three bfloat16 terms each.  Rows are named by
    ``cu_q`` [R+1] and ``ctx_before`` [R]; ``max_q`` bounds the longest entry."""
    n = q.shape[0]
    num_pages, n_k, page_size, dim = k_pages.shape
    n_g, vdim = v_pages.shape[1], v_pages.shape[3]
    if n_k != n_g * n_maps or q.shape != (n, n_heads * n_maps * dim) or out.shape != (n, n_heads * vdim) \
            or q.dtype != torch.bfloat16 or k_pages.dtype != torch.bfloat16 or v_pages.dtype != torch.bfloat16 \
            or out.dtype != torch.bfloat16 or v_pages.shape[0] != num_pages or v_pages.shape[2] != page_size:
        raise KernelError("mapped_attention_mma: shapes or dtypes do not fit")
    _i32(table, "table"), _i32(cu_q, "cu_q"), _i32(ctx_before, "ctx_before")
    f = _fn("mapped_attention_mma", "ng_mapped_attention_mma", [_c_void_p] * 4 + [_c_int] + [_c_void_p] * 3 + [_c_int] * 12
            + [_c_float] * 5 + [_c_int, _c_void_p, _c_void_p, _c_int, _c_void_p], {"NG_MA_D": dim, "NG_MA_DV": vdim})
    _check(f(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(table), table.shape[1], _ptr(cu_q), _ptr(ctx_before),
             out.data_ptr(), _column_block(out, "attention out"), n_entries, max_q, n_heads, n_g, n_maps, dim, vdim,
             page_size, num_pages, int(window or 0), int(keep_first), float(scale), float(softcap or 0.0), float(lam),
             float(post_scale), float(eps), int(bool(head_norm)), _slopes(slopes, n_heads), _slopes(sinks, n_heads),
             int(chunk or 0), _stream()), "mapped_attention_mma")


def mapped_attention_group_takes(dim: int, vdim: int, n_heads: int, n_kv_heads: int, dtype) -> bool:
    """Whether single-token entries can run with the heads of a KV group as the rows of a tensor-core tile."""
    return mapped_attention_mma_takes(dim, vdim, dtype) and n_heads // n_kv_heads <= 16


def mapped_attention_group(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, table: torch.Tensor,
                           cu_q: torch.Tensor, ctx_before: torch.Tensor, row_entry: torch.Tensor, out: torch.Tensor,
                           partial: torch.Tensor, n_entries: int, n_heads: int, n_maps: int, window: Optional[int],
                           keep_first: int, scale: float, softcap: float, lam: float, head_norm: bool, post_scale: float,
                           eps: float, n_splits: int, slopes: Optional[torch.Tensor] = None,
                           sinks: Optional[torch.Tensor] = None, chunk: int = 0) -> None:
    """``mapped_attention`` for a step whose entries bring one token each (bfloat16), on the tensor cores: the query
    heads of a KV group are the rows of a tile, every row's keys are cut into ``n_splits`` runs (a block each), and the
    runs' states pass through ``partial`` (float32, ``mapped_attention_partial_floats`` values, also for one run) to
    the kernel that merges them, combines the maps and norms the heads."""
    n = q.shape[0]
    num_pages, n_k, page_size, dim = k_pages.shape
    n_g, vdim = v_pages.shape[1], v_pages.shape[3]
    if n_k != n_g * n_maps or q.shape != (n, n_heads * n_maps * dim) or out.shape != (n, n_heads * vdim) \
            or q.dtype != torch.bfloat16 or k_pages.dtype != torch.bfloat16 or v_pages.dtype != torch.bfloat16 \
            or out.dtype != torch.bfloat16 or v_pages.shape[0] != num_pages or v_pages.shape[2] != page_size:
        raise KernelError("mapped_attention_group: shapes or dtypes do not fit")
    need = n * n_heads * n_splits * n_maps * (vdim + 2)
    if partial is None or partial.dtype != torch.float32 or partial.numel() < need:
        raise KernelError(f"mapped_attention_group: the runs need {need} float32 values")
    _i32(table, "table"), _i32(cu_q, "cu_q"), _i32(ctx_before, "ctx_before"), _i32(row_entry, "row_entry")
    defines = {"NG_MA_D": dim, "NG_MA_DV": vdim}
    f = _fn("mapped_attention_mma", "ng_mapped_attention_group", [_c_void_p] * 4 + [_c_int] + [_c_void_p] * 3 + [_c_int] * 11
            + [_c_float] * 2 + [_c_void_p, _c_int, _c_void_p], defines)
    _check(f(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(table), table.shape[1], _ptr(cu_q), _ptr(ctx_before), _ptr(partial),
             n_entries, int(n_splits), n_heads, n_g, n_maps, dim, vdim, page_size, num_pages, int(window or 0), int(keep_first),
             float(scale), float(softcap or 0.0), _slopes(slopes, n_heads), int(chunk or 0), _stream()), "mapped_attention_group")
    g = _fn("mapped_attention", "ng_mapped_attention_merge", [_c_void_p] * 3 + [_c_int] * 6 + [_c_float] * 3
            + [_c_int, _c_void_p, _c_int, _c_void_p])
    _check(g(_ptr(partial), _ptr(row_entry), out.data_ptr(), _column_block(out, "attention out"), n, n_heads, n_maps, vdim,
             int(n_splits), float(lam), float(post_scale), float(eps), int(bool(head_norm)), _slopes(sinks, n_heads), 1, _stream()),
           "mapped_attention_merge")


# ----------------------------------------------------------------------------- input convolution
def input_conv(u: torch.Tensor, weight: torch.Tensor, state: torch.Tensor, out: torch.Tensor, cu_q: torch.Tensor,
               ctx_before: torch.Tensor, slots: torch.Tensor, n_entries: int, max_q: int) -> None:
    """out[N,H] = u + causal conv of u over time per channel (weight [H, L] float32; tap L-1 is the current
    token); state[slots, L-1, H] float32 carries each request's last L-1 inputs."""
    n, H = u.shape
    L = weight.shape[1]
    if out.shape != u.shape or out.dtype != u.dtype or weight.shape[0] != H or state.shape[1:] != (L - 1, H):
        raise KernelError("input_conv: shapes do not fit")
    _f32(weight, "conv weight"), _f32(state, "conv state")
    _i32(cu_q, "cu_q"), _i32(ctx_before, "ctx_before"), _i32(slots, "slots")
    f = _fn("input_conv", "ng_input_conv", [_c_void_p] * 7 + [_c_int] * 5 + [_c_void_p])
    _check(f(_ptr(u), _ptr(weight), _ptr(state), _ptr(out), _ptr(cu_q), _ptr(ctx_before), _ptr(slots), n_entries,
             max_q, H, L, _act_flag(u, "conv input"), _stream()), "input_conv")


# ----------------------------------------------------------------------------- retention
def retention(x: torch.Tensor, inv_freq: Optional[torch.Tensor], rot_dims: int, decay: torch.Tensor,
              state: torch.Tensor, out: torch.Tensor, cu_q: torch.Tensor, ctx_before: torch.Tensor,
              slots: torch.Tensor, n_entries: int, n_heads: int, key_dim: int, value_dim: int, eps: float,
              scratch: Optional[torch.Tensor] = None, state_scratch: Optional[torch.Tensor] = None,
              max_q: int = 0) -> None:
    """x[N, 2*nH*(dk+dv)] = q|k|v|g;  per head S = decay*S + k v^T, o = S^T q, out[N, nH*dv] = o/rms(o) * silu(g);
    state[slots, nH, dk, dv] float32.  q, k rotated on their first ``rot_dims`` coordinates (pairs i, i+rot_dims/2).
    With ``scratch`` (float32 [N, nH*dv]), ``state_scratch`` (``retention_chunked_scratch`` float32 values) and
    ``max_q`` (the longest portion) the kernels for long portions run, which regroup the sums chunk by chunk and run
    the chunks side by side (``retention_chunked_takes`` tells whether they take the head sizes); else the
    token-by-token kernel."""
    n = x.shape[0]
    if x.shape[1] != 2 * n_heads * (key_dim + value_dim) or out.shape != (n, n_heads * value_dim) \
            or out.dtype != x.dtype or state.shape[1:] != (n_heads, key_dim, value_dim) or decay.numel() != n_heads:
        raise KernelError("retention: shapes do not fit")
    if rot_dims and (inv_freq is None or inv_freq.numel() != rot_dims // 2):
        raise KernelError("retention: inv_freq must hold rot_dims/2 frequencies")
    _f32(inv_freq, "inv_freq"), _f32(decay, "decay"), _f32(state, "retention state"), _f32(scratch, "retention scratch")
    _i32(cu_q, "cu_q"), _i32(ctx_before, "ctx_before"), _i32(slots, "slots")
    act = _act_flag(x, "retention input")
    if scratch is not None:
        need = retention_chunked_scratch(n, n_entries, n_heads, key_dim, value_dim)
        if scratch.shape != out.shape or state_scratch is None or state_scratch.dtype != torch.float32 \
                or state_scratch.numel() < need or max_q <= 0:
            raise KernelError(f"retention: the chunked kernels need a scratch of the output's shape, {need} float32 "
                              "values for the chunks' states and the longest portion's length")
        f = _fn("retention", "ng_retention_chunked", [_c_void_p, _c_void_p, _c_int] + [_c_void_p] * 8 + [_c_int] * 6
                + [_c_float, _c_int, _c_void_p])
        _check(f(_ptr(x), _ptr(inv_freq), int(rot_dims), _ptr(decay), _ptr(state), _ptr(out), _ptr(scratch),
                 _ptr(state_scratch), _ptr(cu_q), _ptr(ctx_before), _ptr(slots), n_entries, n, int(max_q), n_heads,
                 key_dim, value_dim, float(eps), act, _stream()), "retention (chunked)")
        return
    f = _fn("retention", "ng_retention", [_c_void_p, _c_void_p, _c_int] + [_c_void_p] * 6 + [_c_int] * 4
            + [_c_float, _c_int, _c_void_p])
    _check(f(_ptr(x), _ptr(inv_freq), int(rot_dims), _ptr(decay), _ptr(state), _ptr(out), _ptr(cu_q),
             _ptr(ctx_before), _ptr(slots), n_entries, n_heads, key_dim, value_dim, float(eps), act, _stream()), "retention")


def retention_chunked_scratch(n_rows: int, n_entries: int, n_heads: int, key_dim: int, value_dim: int) -> int:
    """float32 values the chunked retention kernels need for the chunks' states."""
    return (n_rows // 32 + n_entries + 1) * n_heads * key_dim * value_dim


def retention_chunked_takes(key_dim: int, value_dim: int) -> bool:
    f = _fn("retention", "ng_retention_chunked_takes", [_c_int, _c_int])
    return bool(f(int(key_dim), int(value_dim)))


# ----------------------------------------------------------------------------- latent attention
def latent_prep(x: torch.Tensor, wq: torch.Tensor, wkv: torch.Tensor, cq_out: torch.Tensor, pages: torch.Tensor,
                gate_out: torch.Tensor, table: torch.Tensor, positions: torch.Tensor, row_entry: torch.Tensor,
                n_heads: int, eps: float, status: torch.Tensor, *, rot: int = 0, inv_freq: Optional[torch.Tensor] = None,
                half_pairing: bool = False) -> None:
    """x[N, rq+rkv+rot+nH] = c_q raw | c raw | key part raw | gate logits;  cq_out[N, rq] = rmsnorm(c_q raw) * wq;
    rmsnorm(c raw) * wkv goes to the row's place in pages[P, 1, page, rp] and behind it the key part (``rot`` columns,
    not normed), rotated by the row's position in pairs (2i, 2i+1) or (i, i+rot/2) with ``inv_freq`` [rot/2]; the
    columns behind are zero.  gate_out[N, nH] float32 = sigmoid(gate logits), nH the gate's columns.  ``wkv`` and
    ``pages`` None: a layer that reads another layer's latents (the row has no c and no key part)."""
    n, rq = cq_out.shape
    rkv = wkv.numel() if wkv is not None else 0
    num_pages, one, page_size, rp = pages.shape if pages is not None else (0, 1, 1, 0)
    if x.shape != (n, rq + rkv + rot + n_heads) or wq.numel() != rq or one != 1 or rp < rkv + rot \
            or gate_out.shape != (n, n_heads) or cq_out.dtype != x.dtype or (pages is not None and pages.dtype != x.dtype) \
            or (rkv == 0) != (pages is None) or (rot and (inv_freq is None or inv_freq.numel() != rot // 2 or not rkv)):
        raise KernelError("latent_prep: shapes or dtypes do not fit")
    _f32(wq, "dq norm"), _f32(wkv, "dkv norm"), _f32(gate_out, "gate"), _f32(inv_freq, "inv_freq")
    _i32(table, "table"), _i32(positions, "positions"), _i32(row_entry, "row_entry"), _i32(status, "status")
    f = _fn("latent", "ng_latent_prep", [_c_void_p] * 7 + [_c_int] + [_c_void_p] * 2 + [_c_int] * 7
            + [_c_float, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(x), _ptr(wq), _ptr(wkv), _ptr(cq_out), _ptr(pages), _ptr(gate_out), _ptr(table), table.shape[1],
             _ptr(positions), _ptr(row_entry), n, rq, rkv, rp, n_heads, page_size, num_pages, float(eps),
             _ptr(status), int(rot), _ptr(inv_freq) if rot else None, int(bool(half_pairing)),
             _act_flag(x, "latent input"), _stream()), "latent_prep")


def latent_rope_q(q: torch.Tensor, positions: torch.Tensor, row_entry: torch.Tensor, inv_freq: torch.Tensor,
                  n_heads: int, offset: int, half_pairing: bool = False) -> None:
    """q[N, nH * rp]: columns offset..offset + 2 len(inv_freq) of every head are rotated in place by the row's position,
    in pairs (2i, 2i+1) or (i, i + rot/2); angles float32."""
    n = q.shape[0]
    rp, rot = q.shape[1] // n_heads, 2 * inv_freq.numel()
    if q.shape[1] != n_heads * rp or offset + rot > rp:
        raise KernelError("latent_rope_q: shapes do not fit")
    _f32(inv_freq, "inv_freq"), _i32(positions, "positions"), _i32(row_entry, "row_entry")
    f = _fn("latent", "ng_latent_rope_q", [_c_void_p] * 4 + [_c_int] * 7 + [_c_void_p])
    _check(f(_ptr(q), _ptr(positions), _ptr(row_entry), _ptr(inv_freq), n, n_heads, rp, int(offset), rot,
             int(bool(half_pairing)), _act_flag(q, "q"), _stream()), "latent_rope_q")


def head_up_gate(o: torch.Tensor, w: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out[N, nH * dv] = (W[h] o[N, h, :rank]) * gate for o [N, nH * rp] and W [nH, dv, rank] of the activation type,
    gate float32 [N, nH * dv] or None; float32 sums, one rounding.  ``out`` may be a block of columns of a wider buffer."""
    n = o.shape[0]
    n_heads, dv, rank = w.shape
    rp = o.shape[1] // n_heads
    if o.shape[1] != n_heads * rp or rank > rp or out.shape != (n, n_heads * dv) or w.dtype != o.dtype or out.dtype != o.dtype \
            or (gate is not None and gate.shape != (n, n_heads * dv)):
        raise KernelError("head_up_gate: shapes or dtypes do not fit")
    _f32(gate, "gate")
    f = _fn("latent", "ng_head_up_gate", [_c_void_p] * 4 + [_c_int] * 7 + [_c_void_p])
    _check(f(_ptr(o), _ptr(w), _ptr(gate), out.data_ptr(), n, n_heads, rp, rank, dv, _column_block(out, "head_up_gate out"),
             _act_flag(o, "weighted latents"), _stream()), "head_up_gate")


def latent_core_takes(n_heads: int, rank: int) -> bool:
    """Whether the latent attention core takes this many heads of this many (padded) latent columns."""
    return n_heads <= 64 and rank <= 256 and (32 * (rank + 1) + n_heads * rank) * 4 <= 200 * 1024


def latent_core(q: torch.Tensor, pages: torch.Tensor, table: torch.Tensor, positions: torch.Tensor,
                row_entry: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor, n_heads: int,
                window: Optional[int], scale: float, n_splits: int = 1, partial: Optional[torch.Tensor] = None) -> None:
    """out[N, nH*r] = gate[N, nH] * softmax(q_h . c_j * scale over the visible j) c_j, every head reading the same
    latent pages[P, 1, page, r] as keys and as values; float32 scores, weights and sums.  ``n_splits`` > 1 cuts every
    row's keys into that many runs, each a block of its own, merged through ``partial`` (float32,
    ``latent_core_partial_floats`` values): for steps of few rows."""
    n = q.shape[0]
    num_pages, one, page_size, rp = pages.shape
    if q.shape != (n, n_heads * rp) or out.shape != q.shape or one != 1 or q.dtype != pages.dtype or out.dtype != q.dtype \
            or (gate is not None and gate.shape != (n, n_heads)):
        raise KernelError("latent_core: shapes or dtypes do not fit")
    _f32(gate, "gate"), _i32(table, "table"), _i32(positions, "positions"), _i32(row_entry, "row_entry")
    _f32(partial, "partial")
    if n_splits > 1 and (partial is None or partial.numel() < latent_core_partial_floats(n, n_heads, rp, n_splits)):
        raise KernelError("latent_core: the runs need latent_core_partial_floats float32 values")
    f = _fn("latent", "ng_latent_core", [_c_void_p] * 3 + [_c_int] + [_c_void_p] * 4 + [_c_int] * 6
            + [_c_float, _c_int, _c_void_p, _c_int, _c_void_p])
    _check(f(_ptr(q), _ptr(pages), _ptr(table), table.shape[1], _ptr(positions), _ptr(row_entry), _ptr(gate), _ptr(out),
             n, n_heads, rp, page_size, num_pages, int(window or 0), float(scale), int(n_splits),
             _ptr(partial) if n_splits > 1 else None, _act_flag(q, "q"), _stream()), "latent_core")


LATENT_BACKEND = os.environ.get("NEUROGRID_B200_LATENT", "mma")     # "mma": tensor-core core for long bfloat16 steps; "ffma"


def latent_core_mma_takes(n_heads: int, rank: int, dtype) -> bool:
    """Whether the tensor-core latent core takes this shape (bfloat16, up to 16 heads, a rank in 32s up to 256)."""
    return LATENT_BACKEND == "mma" and dtype == torch.bfloat16 and n_heads <= 16 and rank % 32 == 0 and 32 <= rank <= 256


def latent_core_mma(q: torch.Tensor, pages: torch.Tensor, table: torch.Tensor, positions: torch.Tensor,
                    row_entry: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor, n_heads: int,
                    window: Optional[int], scale: float) -> None:
    """``latent_core`` for long bfloat16 steps on the tensor cores: the heads of a row are the rows of an MMA tile;
    scores are float32 sums of exact bfloat16 products, the float32 softmax weights enter the weighted sum as three
    bfloat16 terms each, so the sum is a float32 sum."""
    n = q.shape[0]
    num_pages, one, page_size, rp = pages.shape
    if q.shape != (n, n_heads * rp) or out.shape != q.shape or one != 1 or q.dtype != torch.bfloat16 \
            or pages.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or (gate is not None and gate.shape != (n, n_heads)):
        raise KernelError("latent_core_mma: shapes or dtypes do not fit")
    _f32(gate, "gate"), _i32(table, "table"), _i32(positions, "positions"), _i32(row_entry, "row_entry")
    f = _fn("latent_mma", "ng_latent_core_mma", [_c_void_p] * 3 + [_c_int] + [_c_void_p] * 4 + [_c_int] * 6 + [_c_float, _c_void_p],
            {"NG_LAT_RANK": rp})
    _check(f(_ptr(q), _ptr(pages), _ptr(table), table.shape[1], _ptr(positions), _ptr(row_entry), _ptr(gate), _ptr(out),
             n, n_heads, rp, page_size, num_pages, int(window or 0), float(scale), _stream()), "latent_core_mma")


def latent_core_partial_floats(n_rows: int, n_heads: int, rank: int, n_splits: int) -> int:
    return n_rows * n_heads * n_splits * (rank + 2) if n_splits > 1 else 0


def head_gate(y: torch.Tensor, gate: torch.Tensor, n_heads: int) -> None:
    """y[N, nH*w] *= gate[N, nH] (float32) head by head, in place."""
    n = y.shape[0]
    if y.shape[1] % n_heads or gate.shape != (n, n_heads):
        raise KernelError("head_gate: shapes do not fit")
    _f32(gate, "gate")
    f = _fn("latent", "ng_head_gate", [_c_void_p, _c_void_p] + [_c_int] * 4 + [_c_void_p])
    _check(f(_ptr(y), _ptr(gate), n, n_heads, y.shape[1] // n_heads, _act_flag(y, "head_gate"), _stream()), "head_gate")


# ----------------------------------------------------------------------------- gated delta rule
def gated_delta(p: torch.Tensor, conv_weight: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor,
                norm_weight: torch.Tensor, conv_state: torch.Tensor, state: torch.Tensor, conv_out: torch.Tensor,
                o_raw: torch.Tensor, out: torch.Tensor, cu_q: torch.Tensor, ctx_before: torch.Tensor, slots: torch.Tensor,
                row_entry: torch.Tensor, n_entries: int, max_q: int, n_heads: int, n_qk_heads: int, key_dim: int,
                value_dim: int, eps: float, chunk_scratch: torch.Tensor | None = None) -> None:
    """p[N, C + nH*dv + 2*nH] = q (nG*dk) | k (nG*dk) | v (nH*dv) | gate (nH*dv) | a (nH) | b (nH), C the first three.
    The q, k, v channels pass a causal convolution per channel (conv_weight float32 [C, L], tap L-1 on the current
    token; conv_state [slots, L-1, C] float32 carries a request's last inputs) and silu; q and k become unit vectors
    per head, q times dk^(-1/2); beta = sigmoid(b), g = exp(-exp(a_log) * softplus(a + dt_bias)); per value head
    (query/key head h // (nH / nG)):  S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q, with
    state[slots, nH, dk, dv] float32; out[N, nH*dv] = o / rms(o) * norm_weight * silu(gate).  ``conv_out``
    (float32 [N, C]) and ``o_raw`` (float32 [N, nH*dv]) are scratch.  Everything after the projections is float32.
    With ``chunk_scratch`` (``gated_delta_chunked_scratch`` float32 values) the recurrence runs chunk by chunk, most of
    a portion's work side by side (``gated_delta_chunked_takes`` tells whether the kernels take the head sizes); else
    token by token.  The two differ by rounding only."""
    n = p.shape[0]
    C = (2 * n_qk_heads * key_dim) + n_heads * value_dim
    ldp = C + n_heads * value_dim + 2 * n_heads
    L = conv_weight.shape[1]
    if p.shape != (n, ldp) or conv_weight.shape != (C, L) or conv_state.shape[1:] != (L - 1, C) \
            or state.shape[1:] != (n_heads, key_dim, value_dim) or conv_out.shape != (n, C) \
            or o_raw.shape != (n, n_heads * value_dim) or out.shape != o_raw.shape or out.dtype != p.dtype \
            or a_log.numel() != n_heads or dt_bias.numel() != n_heads or norm_weight.numel() != value_dim:
        raise KernelError("gated_delta: shapes do not fit")
    for t, what in ((conv_weight, "conv weight"), (a_log, "A_log"), (dt_bias, "dt_bias"), (norm_weight, "norm weight"),
                    (conv_state, "conv state"), (state, "state"), (conv_out, "conv scratch"), (o_raw, "output scratch")):
        _f32(t, what)
    _i32(cu_q, "cu_q"), _i32(ctx_before, "ctx_before"), _i32(slots, "slots"), _i32(row_entry, "row_entry")
    act = _act_flag(p, "gated_delta input")
    f = _fn("gated_delta", "ng_gd_conv_silu", [_c_void_p, _c_int] + [_c_void_p] * 6 + [_c_int] * 5 + [_c_void_p])
    _check(f(_ptr(p), ldp, _ptr(conv_weight), _ptr(conv_state), _ptr(conv_out), _ptr(cu_q), _ptr(ctx_before), _ptr(slots),
             n_entries, int(max_q), C, L, act, _stream()), "gated_delta (convolution)")
    if chunk_scratch is not None:
        need = gated_delta_chunked_scratch(n, n_entries, n_heads, key_dim, value_dim)
        _f32(chunk_scratch, "chunk scratch")
        if chunk_scratch.numel() < need or not gated_delta_chunked_takes(key_dim, value_dim):
            raise KernelError(f"gated_delta: the chunked kernels need {need} float32 values of scratch and head sizes they take")
        f = _fn("gated_delta", "ng_gated_delta_chunked", [_c_void_p, _c_void_p] + [_c_int] * 3 + [_c_void_p] * 8 + [_c_int] * 8
                + [_c_void_p])
        _check(f(_ptr(conv_out), _ptr(p), ldp, C + n_heads * value_dim, C + n_heads * value_dim + n_heads, _ptr(a_log),
                 _ptr(dt_bias), _ptr(state), _ptr(o_raw), _ptr(chunk_scratch), _ptr(cu_q), _ptr(ctx_before), _ptr(slots),
                 n_entries, n, int(max_q), n_heads, n_qk_heads, key_dim, value_dim, act, _stream()), "gated_delta (chunked)")
    else:
        f = _fn("gated_delta", "ng_gated_delta", [_c_void_p, _c_void_p] + [_c_int] * 3 + [_c_void_p] * 7 + [_c_int] * 6
                + [_c_void_p])
        _check(f(_ptr(conv_out), _ptr(p), ldp, C + n_heads * value_dim, C + n_heads * value_dim + n_heads, _ptr(a_log),
                 _ptr(dt_bias), _ptr(state), _ptr(o_raw), _ptr(cu_q), _ptr(ctx_before), _ptr(slots), n_entries, n_heads,
                 n_qk_heads, key_dim, value_dim, act, _stream()), "gated_delta")
    f = _fn("gated_delta", "ng_gd_finish", [_c_void_p, _c_void_p, _c_int, _c_int] + [_c_void_p] * 3 + [_c_int] * 3
            + [_c_float, _c_int, _c_void_p])
    _check(f(_ptr(o_raw), _ptr(p), ldp, C, _ptr(norm_weight), _ptr(row_entry), _ptr(out), n, n_heads, value_dim, float(eps),
             act, _stream()), "gated_delta (head norm)")


def gated_delta_chunked_scratch(n_rows: int, n_entries: int, n_heads: int, key_dim: int, value_dim: int) -> int:
    """float32 values the chunked gated delta kernels need for the chunks' tiles and states."""
    return (n_rows // 32 + n_entries + 1) * n_heads * (64 * key_dim + 32 + key_dim * value_dim)


def gated_delta_chunked_takes(key_dim: int, value_dim: int) -> bool:
    f = _fn("gated_delta", "ng_gd_chunked_takes", [_c_int, _c_int])
    return bool(f(int(key_dim), int(value_dim)))


# ----------------------------------------------------------------------------- small parts of a layer or a model
def pair_embed(table: torch.Tensor, tokens: torch.Tensor, state: torch.Tensor, cu_q: torch.Tensor, ctx_before: torch.Tensor,
               slots: torch.Tensor, row_entry: torch.Tensor, h: torch.Tensor, n_entries: int, vocab: int, buckets: int,
               mul_prev: int, mul_cur: int, status: torch.Tensor) -> None:
    """h[N,H] (float32) += table[(previous token * mul_prev + token * mul_cur) mod buckets], row ``buckets`` of the
    table for a request's first token.  ``state`` int32 [slots] carries each request's last token between steps."""
    n, H = h.shape
    if table.shape != (buckets + 1, H) or state.dim() != 1:
        raise KernelError("pair_embed: shapes do not fit")
    _f32(h, "residual stream"), _i32(tokens, "tokens"), _i32(state, "previous tokens"), _i32(status, "status")
    _i32(cu_q, "cu_q"), _i32(ctx_before, "ctx_before"), _i32(slots, "slots"), _i32(row_entry, "row_entry")
    f = _fn("elementwise", "ng_pair_embed", [_c_void_p, _c_int] + [_c_void_p] * 7 + [_c_int] * 5 + [_c_ll, _c_ll, _c_void_p, _c_void_p])
    _check(f(_ptr(table, "pair table"), _act_flag(table, "pair table"), _ptr(tokens), _ptr(state), _ptr(cu_q), _ptr(ctx_before),
             _ptr(slots), _ptr(row_entry), _ptr(h), n, n_entries, H, int(vocab), int(buckets), int(mul_prev), int(mul_cur),
             _ptr(status), _stream()), "pair_embed")


def _maybe_stack(t: torch.Tensor, n: int, H: int, act_dtype, what: str):
    """(is float32, parts, stride) of [N,H] in the activation dtype or float32, or a float32 stack [S,N,H]."""
    if t.dim() == 3:
        if t.dtype != torch.float32 or tuple(t.shape[1:]) != (n, H):
            raise KernelError(f"{what}: a stack of partial sums must be float32 [S, {n}, {H}]")
        return 1, t.shape[0], n * H
    if tuple(t.shape) != (n, H) or t.dtype not in (act_dtype, torch.float32):
        raise KernelError(f"{what}: expected [{n}, {H}] of {act_dtype}")
    return int(t.dtype == torch.float32), 1, 0


def pair_norm_mean(a: torch.Tensor, b: torch.Tensor, wa: torch.Tensor, wb: torch.Tensor, out: torch.Tensor, eps: float,
                   act_dtype, accumulate: bool = False) -> None:
    """out[N,H] float32 (+)= 0.5 * (a / rms(a) * wa + b / rms(b) * wb), rms over a row with eps inside the root.
    a and b: [N,H] of the activation dtype, or float32 stacks [S,N,H] of partial sums."""
    n, H = out.shape
    a32, ap, as_ = _maybe_stack(a, n, H, act_dtype, "pair_norm_mean a")
    b32, bp, bs_ = _maybe_stack(b, n, H, act_dtype, "pair_norm_mean b")
    _f32(out, "out"), _f32(wa, "weight"), _f32(wb, "weight")
    f = _fn("elementwise", "ng_pair_norm_mean", [_c_void_p, _c_int, _c_int, _c_ll, _c_void_p, _c_int, _c_int, _c_ll]
            + [_c_void_p] * 3 + [_c_int, _c_int, _c_float, _c_int, _c_int, _c_void_p])
    _check(f(_ptr(a), a32, ap, as_, _ptr(b), b32, bp, bs_, _ptr(wa), _ptr(wb), _ptr(out), n, H, float(eps),
             int(bool(accumulate)), int(act_dtype == torch.bfloat16), _stream()), "pair_norm_mean")


def linear_relu_squared(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out = relu(x @ weight^T + bias)^2: in the product's epilogue where the tcgen05 kernel runs the product (steps of
    few rows), else the product and one pass over it; both square the same rounded value."""
    if x.dtype == torch.bfloat16 and x.is_cuda and out.dtype == torch.bfloat16 and gemm_sm100_ok(x, weight):
        gemm_sm100(x, weight, bias, out, relu_squared=True)
        return
    linear(x, weight, bias, out)
    relu_squared_(out)


def relu_squared_(x: torch.Tensor) -> None:
    """x <- relu(x)^2 in place."""
    f = _fn("elementwise", "ng_unary", [_c_void_p, _c_ll, _c_int, _c_float, _c_int, _c_void_p])
    _check(f(_ptr(x), x.numel(), 0, 0.0, _act_flag(x, "activation"), _stream()), "relu_squared")


def softcap_(x: torch.Tensor, cap: float) -> None:
    """x <- cap * tanh(x / cap) in place (float32 logits)."""
    _f32(x, "logits")
    f = _fn("elementwise", "ng_unary", [_c_void_p, _c_ll, _c_int, _c_float, _c_int, _c_void_p])
    _check(f(_ptr(x), x.numel(), 1, float(cap), 0, _stream()), "softcap")


def gate_mul(y: torch.Tensor, gate: Optional[torch.Tensor], activation: str = "sigmoid", scale: float = 1.0) -> None:
    """y[N, I] <- y * act(gate) * scale in place, act sigmoid, silu or (``gate`` None) nothing; float32 math.  Both may
    be blocks of columns of wider buffers."""
    n, I = y.shape
    act = 0 if gate is None else {"sigmoid": 1, "silu": 2}[activation]
    if gate is not None and (gate.shape != y.shape or gate.dtype != y.dtype):
        raise KernelError("gate_mul: the gate must have the shape and dtype of what it multiplies")
    f = _fn("elementwise", "ng_gate_mul", [_c_void_p, _c_void_p] + [_c_int] * 5 + [_c_float, _c_int, _c_void_p])
    _check(f(y.data_ptr(), gate.data_ptr() if gate is not None else None, n, I, _column_block(y, "gate_mul y"),
             _column_block(gate, "gate_mul gate") if gate is not None else 0, act, float(scale), _act_flag(y, "gate_mul y"),
             _stream()), "gate_mul")


def hc_step(streams: torch.Tensor, n_streams: int, *, x0: Optional[torch.Tensor] = None, delta: Optional[torch.Tensor] = None,
            mix: Optional[torch.Tensor] = None, out_w: Optional[torch.Tensor] = None, in_w: Optional[torch.Tensor] = None,
            norm_w: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
            sum_out: Optional[torch.Tensor] = None, eps: float = 0.0, act_dtype=None) -> None:
    """What lies between two sublayers of a model whose residual stream is ``n_streams`` copies, streams[N, S * H]
    float32.  ``x0`` [N,H] float32: every copy is x0 (a sequence's start).  ``delta`` (the output y of the sublayer
    before: [N,H] of the activation dtype or a float32 stack of partial sums) with ``mix`` [S,S] ([from, to]) and
    ``out_w`` [S]: x_t <- sum_s mix[s,t] x_s + out_w[t] y for all t at once.  ``in_w`` [S] with ``norm_w`` [H] and
    ``out`` [N,H]: out = rmsnorm(sum_t in_w[t] x_t) * norm_w.  ``sum_out`` [N,H] float32: the sum of the copies."""
    n = streams.shape[0]
    H = streams.shape[1] // n_streams
    if streams.shape[1] != n_streams * H:
        raise KernelError("hc_step: the streams do not divide into copies")
    _f32(streams, "streams"), _f32(x0, "x0"), _f32(mix, "mix"), _f32(out_w, "out_w"), _f32(in_w, "in_w"), _f32(norm_w, "norm weight")
    _f32(sum_out, "sum_out")
    act_dtype = out.dtype if out is not None else (act_dtype or torch.float32)
    act = int(act_dtype == torch.bfloat16)
    d32, n_part, stride = 0, 1, 0
    if delta is not None:
        d32, n_part, stride = _maybe_stack(delta, n, H, act_dtype, "hc_step delta")
        if mix is None or mix.numel() != n_streams * n_streams or out_w is None or out_w.numel() != n_streams:
            raise KernelError("hc_step: an update needs the mixing matrix and the output weights")
    if in_w is not None and (in_w.numel() != n_streams or norm_w is None or norm_w.numel() != H or out is None or out.shape != (n, H)):
        raise KernelError("hc_step: the read-out needs its weights, the norm's weight and an output [N, H]")
    for t in (x0, sum_out):
        if t is not None and t.shape != (n, H):
            raise KernelError("hc_step: x0 and sum_out are [N, H]")
    f = _fn("hyper", "ng_hc_step", [_c_void_p] * 3 + [_c_int, _c_int, _c_ll] + [_c_void_p] * 6 + [_c_int] * 3
            + [_c_float, _c_int, _c_void_p])
    _check(f(_ptr(streams), _ptr(x0), _ptr(delta), d32, n_part, stride, _ptr(mix), _ptr(out_w), _ptr(in_w), _ptr(norm_w),
             _ptr(out), _ptr(sum_out), n, int(n_streams), H, float(eps), act, _stream()), "hc_step")


# ----------------------------------------------------------------------------- gated linear attention
GATED_LINEAR_CHUNK = 32      # tokens of a chunk in the chunk-by-chunk kernels


def gated_linear(x: torch.Tensor, z: torch.Tensor, norm_w: torch.Tensor, state: torch.Tensor, out: torch.Tensor,
                 cu_q: torch.Tensor, ctx_before: torch.Tensor, slots: torch.Tensor, n_entries: int, n_heads: int,
                 key_dim: int, value_dim: int, tau: float, eps: float, out_scale: float = 1.0,
                 scratch: Optional[torch.Tensor] = None, state_scratch: Optional[torch.Tensor] = None, max_q: int = 0) -> None:
    """x[N, 2*nH*(dk+dv)] = q|k|v|g and z[N, nH*dk] (decay logits);  per head S = diag(alpha) S + k v^T with
    alpha = sigmoid(z)^(1/tau) per key channel, o = S^T (q dk^(-1/2)), out = o/rms(o) * norm_w * silu(g) * out_scale;
    state[slots, nH, dk, dv] float32.  ``out`` [N, nH*dv] of the activation dtype may be a block of columns of a wider
    buffer.  With ``scratch`` (float32 [N, nH*dv]), ``state_scratch`` (``gated_linear_chunked_scratch`` float32 values)
    and ``max_q`` (the longest portion) the kernels for long portions run, which regroup the sums chunk by chunk
    (``gated_linear_chunked_takes`` tells whether they take the head sizes); else the token-by-token kernel."""
    n = x.shape[0]
    if x.shape[1] != 2 * n_heads * (key_dim + value_dim) or z.shape != (n, n_heads * key_dim) or z.dtype != x.dtype \
            or out.shape != (n, n_heads * value_dim) or out.dtype != x.dtype or norm_w.numel() != value_dim \
            or state.shape[1:] != (n_heads, key_dim, value_dim):
        raise KernelError("gated_linear: shapes or dtypes do not fit")
    _f32(norm_w, "head norm weight"), _f32(state, "state"), _i32(cu_q, "cu_q"), _i32(ctx_before, "ctx_before"), _i32(slots, "slots")
    _f32(scratch, "scratch"), _f32(state_scratch, "state scratch")
    ldo = _column_block(out, "gated_linear out")
    act = _act_flag(x, "gated_linear input")
    if scratch is not None:
        need = gated_linear_chunked_scratch(n, n_entries, n_heads, key_dim, value_dim)
        if scratch.shape != (n, n_heads * value_dim) or state_scratch is None or state_scratch.numel() < need or max_q <= 0:
            raise KernelError(f"gated_linear: the chunked kernels need a scratch of the output's shape, {need} float32 "
                              "values for the chunks' states and the longest portion's length")
        f = _fn("gated_linear", "ng_gated_linear_chunked", [_c_void_p] * 10 + [_c_int] * 6 + [_c_float] * 3 + [_c_int, _c_int, _c_void_p])
        _check(f(_ptr(x), _ptr(z), _ptr(norm_w), _ptr(state), out.data_ptr(), _ptr(scratch), _ptr(state_scratch), _ptr(cu_q),
                 _ptr(ctx_before), _ptr(slots), n_entries, n, int(max_q), n_heads, key_dim, value_dim, float(tau), float(eps),
                 float(out_scale), ldo, act, _stream()), "gated_linear (chunked)")
        return
    f = _fn("gated_linear", "ng_gated_linear", [_c_void_p] * 8 + [_c_int] * 4 + [_c_float] * 3 + [_c_int, _c_int, _c_void_p])
    _check(f(_ptr(x), _ptr(z), _ptr(norm_w), _ptr(state), out.data_ptr(), _ptr(cu_q), _ptr(ctx_before), _ptr(slots), n_entries,
             n_heads, key_dim, value_dim, float(tau), float(eps), float(out_scale), ldo, act, _stream()), "gated_linear")


def gated_linear_chunked_scratch(n_rows: int, n_entries: int, n_heads: int, key_dim: int, value_dim: int) -> int:
    """float32 values the chunked kernels need: per chunk and head the state before it and the chunk's whole decay."""
    return (n_rows // GATED_LINEAR_CHUNK + n_entries + 1) * n_heads * (key_dim * value_dim + key_dim)


def gated_linear_chunked_takes(key_dim: int, value_dim: int) -> bool:
    """Whether the chunk-by-chunk kernels take the head sizes."""
    f = _fn("gated_linear", "ng_gated_linear_chunked_takes", [_c_int, _c_int])
    return bool(f(int(key_dim), int(value_dim)))


def scale_(x: torch.Tensor, factor: float) -> None:
    """x <- x * factor in place (float32 logits)."""
    _f32(x, "logits")
    f = _fn("elementwise", "ng_unary", [_c_void_p, _c_ll, _c_int, _c_float, _c_int, _c_void_p])
    _check(f(_ptr(x), x.numel(), 2, float(factor), 0, _stream()), "scale")


# ----------------------------------------------------------------------------- routed experts
def moe_router_sigmoid(x: torch.Tensor, w_router: torch.Tensor, correction: Optional[torch.Tensor],
                       w_shared_gate: Optional[torch.Tensor], weights: torch.Tensor, top_k: int, n_groups: int = 1,
                       keep_groups: int = 1, *, softmax_scores: bool = False, group_max: bool = False,
                       route_scale: float = 1.0) -> None:
    """weights[N, E (+1)] float32: scores s = sigmoid(W_r x); the top_k experts by s + correction among the experts
    of the keep_groups best of n_groups groups of neighbours (a group's score: its two largest choice scores) get
    s / (sum of the chosen s + 1e-20), the others zero.  With ``w_shared_gate`` (float32 [H]) the last column
    receives sigmoid(w . x).  ``softmax_scores``: s = softmax(W_r x) over all experts instead; ``group_max``: a group's
    score is its largest choice score; ``route_scale`` multiplies the weights."""
    n, H = x.shape
    E = w_router.shape[0]
    ldw = weights.shape[1]
    if w_router.shape != (E, H) or weights.shape[0] != n or ldw != E + (w_shared_gate is not None) \
            or (correction is not None and correction.numel() != E) or (w_shared_gate is not None and w_shared_gate.numel() != H):
        raise KernelError("moe_router_sigmoid: shapes do not fit")
    _f32(w_router, "router weight"), _f32(correction, "correction"), _f32(w_shared_gate, "shared gate"), _f32(weights, "weights")
    f = _fn("moe", "ng_moe_router_sigmoid", [_c_void_p] * 5 + [_c_int] * 9 + [_c_float, _c_int, _c_void_p])
    _check(f(_ptr(x), _ptr(w_router), _ptr(correction), _ptr(w_shared_gate), _ptr(weights), n, H, E, ldw, int(top_k),
             int(n_groups), int(keep_groups), int(bool(softmax_scores)), int(bool(group_max)), float(route_scale),
             _act_flag(x, "router input"), _stream()), "moe_router_sigmoid")


def moe_clamped_glu_scaled(gate_up: torch.Tensor, weights: torch.Tensor, out: torch.Tensor, n_experts: int, expert_ff: int,
                           limit: float, shared_limit: float, alpha: float, shared_gated: bool) -> None:
    """out[N, I] = g' sigmoid(alpha g') (u' + 1) * w with g' = min(gate, limit), u' = clamp(up, -limit, limit); columns of
    expert e use ``limit`` and w = weights[N, e], the shared expert's columns behind them ``shared_limit`` and
    w = weights[N, E] (``shared_gated``) or 1."""
    n, I = out.shape
    if gate_up.shape != (n, 2 * I) or gate_up.dtype != out.dtype or weights.shape[0] != n or I < n_experts * expert_ff:
        raise KernelError("moe_clamped_glu_scaled: shapes do not fit")
    _f32(weights, "routing weights")
    f = _fn("moe", "ng_moe_clamped_glu_scaled", [_c_void_p, _c_void_p, _c_int, _c_void_p] + [_c_int] * 4 + [_c_float] * 3
            + [_c_int, _c_int, _c_void_p])
    _check(f(_ptr(gate_up), _ptr(weights), weights.shape[1], _ptr(out), n, I, int(n_experts), int(expert_ff), float(limit),
             float(shared_limit), float(alpha), int(bool(shared_gated)), _act_flag(out, "moe act"), _stream()),
           "moe_clamped_glu_scaled")


def moe_router(x: torch.Tensor, w_router: torch.Tensor, b_router: Optional[torch.Tensor], weights: torch.Tensor,
               top_k: int) -> None:
    """weights[N, E] float32: softmax over the top_k largest of W_r x + b at the chosen experts, zero elsewhere."""
    n, H = x.shape
    E = w_router.shape[0]
    if w_router.shape != (E, H) or weights.shape != (n, E) or (b_router is not None and b_router.numel() != E):
        raise KernelError("moe_router: shapes do not fit")
    _f32(w_router, "router weight"), _f32(b_router, "router bias"), _f32(weights, "routing weights")
    f = _fn("moe", "ng_moe_router", [_c_void_p] * 4 + [_c_int] * 5 + [_c_void_p])
    _check(f(_ptr(x), _ptr(w_router), _ptr(b_router), _ptr(weights), n, H, E, int(top_k), _act_flag(x, "router input"),
             _stream()), "moe_router")


def moe_scale(act: torch.Tensor, weights: torch.Tensor, expert_ff: int, shared_gated: bool = False) -> None:
    """act[N, ld]: columns e*ff..(e+1)*ff are multiplied by weights[N, e], in place; columns behind E*ff stay, or, with
    ``shared_gated`` (weights then has a column E), are multiplied by weights[N, E]."""
    n, ld = act.shape
    E = weights.shape[1] - int(bool(shared_gated))
    if weights.shape[0] != n or ld < E * expert_ff:
        raise KernelError("moe_scale: shapes do not fit")
    _f32(weights, "routing weights")
    f = _fn("moe", "ng_moe_scale", [_c_void_p, _c_void_p] + [_c_int] * 7 + [_c_void_p])
    _check(f(_ptr(act), _ptr(weights), n, E, int(expert_ff), ld, weights.shape[1], int(bool(shared_gated)),
             _act_flag(act, "moe act"), _stream()), "moe_scale")


def moe_swiglu_scaled(gate_up: torch.Tensor, weights: torch.Tensor, out: torch.Tensor, expert_ff: int,
                      shared_gated: bool = False) -> None:
    """out[N, I] = silu(gate_up[:, :I]) * gate_up[:, I:], columns e*ff..(e+1)*ff times weights[N, e] (float32); with
    ``shared_gated`` the columns behind E*ff times weights[N, E]."""
    n, I = out.shape
    E = weights.shape[1] - int(bool(shared_gated))
    if gate_up.shape != (n, 2 * I) or gate_up.dtype != out.dtype or weights.shape[0] != n or I < E * expert_ff:
        raise KernelError("moe_swiglu_scaled: shapes do not fit")
    _f32(weights, "routing weights")
    f = _fn("moe", "ng_moe_swiglu_scaled", [_c_void_p] * 3 + [_c_int] * 7 + [_c_void_p])
    _check(f(_ptr(gate_up), _ptr(weights), _ptr(out), n, I, E, int(expert_ff), weights.shape[1], int(bool(shared_gated)),
             _act_flag(out, "moe act"), _stream()), "moe_swiglu_scaled")


# ----------------------------------------------------------------------------- per-layer token input
def token_side(h: torch.Tensor, tokens: torch.Tensor, table: torch.Tensor, w_gate: torch.Tensor,
               w_proj: torch.Tensor, w_norm: torch.Tensor, row_entry: torch.Tensor, eps: float,
               status: torch.Tensor, scratch: Optional[torch.Tensor] = None) -> None:
    """h[N,H] float32 += rmsnorm(W_proj (gelu_tanh(W_gate h) * table[tokens])) * w_norm; all float32.
    ``w_proj`` is given transposed, [dim, H].  ``scratch`` (float32, ``token_side_scratch`` values): steps of few
    rows deal the same sums to many blocks through it; without it a block takes whole rows."""
    n, H = h.shape
    V, dim = table.shape
    if w_gate.shape != (dim, H) or w_proj.shape != (dim, H) or w_norm.numel() != H:
        raise KernelError("token_side: shapes do not fit")
    for t, what in ((h, "residual stream"), (table, "token table"), (w_gate, "gate"), (w_proj, "proj"), (w_norm, "norm")):
        _f32(t, what)
    _i32(tokens, "tokens"), _i32(row_entry, "row_entry"), _i32(status, "status"), _f32(scratch, "scratch")
    if scratch is not None and scratch.numel() < token_side_scratch(n, H, dim):
        raise KernelError("token_side: the scratch is too small")
    f = _fn("token_side", "ng_token_side", [_c_void_p] * 7 + [_c_int] * 4 + [_c_float, _c_void_p, _c_void_p, _c_void_p])
    _check(f(_ptr(h), _ptr(tokens), _ptr(table), _ptr(w_gate), _ptr(w_proj), _ptr(w_norm), _ptr(row_entry), n, H, dim, V,
             float(eps), _ptr(status), _ptr(scratch), _stream()), "token_side")


def token_side_scratch(n_rows: int, H: int, dim: int) -> int:
    """float32 values of scratch with which a step of ``n_rows`` rows runs the few-rows kernels (0: none needed)."""
    return n_rows * (dim + H + (H + 127) // 128) if n_rows < 128 else 0


# ----------------------------------------------------------------------------- sampling
def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor], top_p: Optional[torch.Tensor],
           uniform: Optional[torch.Tensor], out: torch.Tensor, scratch: Optional[torch.Tensor]) -> None:
    """out[W] int32: argmax where temperature <= 0 (or None), else a draw; scratch[W,V] float32."""
    W, V = logits.shape
    _f32(logits, "logits"), _f32(temperature, "temperature"), _f32(top_p, "top_p"), _f32(uniform, "uniform")
    _i32(out, "sample out"), _f32(scratch, "sample scratch")
    if temperature is not None and (uniform is None or scratch is None or scratch.numel() < W * V):
        raise KernelError("sample: a draw needs uniform numbers and W*V floats of scratch")
    f = _fn("sampling", "ng_sample", [_c_void_p, _c_int, _c_int] + [_c_void_p] * 6)
    _check(f(_ptr(logits), W, V, _ptr(temperature), _ptr(top_p), _ptr(uniform), _ptr(out), _ptr(scratch),
             _stream()), "sample")


# ----------------------------------------------------------------------------- tensor-core products
_GEMM_ARGS = [_c_void_p] * 4 + [_c_int] * 9 + [_c_void_p, _c_void_p]
# Steps of at most FUSE_MAX_ROWS rows (bfloat16, tcgen05 backend) add the products that end a
# mixer or a feed-forward straight into the float32 residual stream (red.global.add in the
# epilogue): the norm kernel that follows has no partial sums to read.  Measured on the decode
# graph of the 1.2B shape: batch 8 0.887 -> 0.852 ms, batch 64 1.329 -> 1.233 ms.
FUSE_MAX_ROWS = int(os.environ.get("NEUROGRID_B200_FUSE_ROWS", "64"))
FUSE_RED = os.environ.get("NEUROGRID_B200_FUSE_RED", "1") == "1"
GEMM_BACKEND = os.environ.get("NEUROGRID_B200_GEMM", "sm100")     # "sm100": tcgen05 kernel; "cublas": vendor library
# Rows up to which the tcgen05 kernel is used.  It streams weights at memory speed, which is the
# whole job when a step has few rows; for long portions the vendor library's product is still
# faster than this one-tile-per-block kernel, so it stands there.
SM100_MAX_ROWS = int(os.environ.get("NEUROGRID_B200_GEMM_MAX_ROWS", "64"))
_status_word = {}


def _gemm_status(device) -> torch.Tensor:
    t = _status_word.get(device)
    if t is None:
        t = _status_word[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return t


def gemm_status(device) -> int:
    """Error bits the tcgen05 kernels recorded on ``device`` (8 = a bounded wait ran out); clears them."""
    t = _status_word.get(torch.device(device))
    if t is None:
        return 0
    own = int(t.item())
    if own:
        t.zero_()
    return own


def gemm_sm100_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tcgen05 kernel is used for these operands (else the library's product)."""
    return (GEMM_BACKEND == "sm100" and x.shape[0] <= SM100_MAX_ROWS and gemm_sm100_takes(x, w))


def gemm_sm100_takes(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tcgen05 kernel can take these operands at all."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_cuda and x.dim() == 2
            and x.shape[1] % 8 == 0 and x.is_contiguous() and w.is_contiguous()
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_sm100(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, *,
               splits: int = 1, token_tile: int = 0, relu_squared: bool = False) -> None:
    """out = x @ w^T on tcgen05/TMA.  out bf16 [M,N] (+ bias), or float32 [M,N], or float32
    [S,M,N] partial sums over S = splits of K (``gemm_splits`` tells S for a K).  ``relu_squared`` (bf16 out): the
    epilogue squares what is positive of the rounded result and zeroes the rest, as ``relu_squared_`` over it would."""
    M, K = x.shape
    N = w.shape[0]
    if relu_squared and out.dtype != torch.bfloat16:
        raise KernelError("gemm_sm100: the squared relu rides in the bf16 epilogue only")
    if out.dtype == torch.bfloat16:
        epi, s_eff = (5 if relu_squared else 0), 1
        if out.shape != (M, N) or splits != 1:
            raise KernelError("gemm_sm100: bf16 output is [M, N] without splits")
    else:
        epi = 1
        s_eff = gemm_splits(K, splits)
        if bias is not None or tuple(out.shape) not in (((M, N),) if s_eff == 1 else ()) + ((s_eff, M, N),):
            raise KernelError(f"gemm_sm100: float32 output must be [{s_eff}, {M}, {N}] (no bias)")
    f = _fn("gemm_sm100", "ng_gemm_sm100", _GEMM_ARGS)
    _check(f(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), M, N, K, N, N, epi, s_eff, 0, token_tile,
             _ptr(_gemm_status(x.device)), _stream()), "gemm_sm100")


def gemm_splits(K: int, splits: int) -> int:
    total = -(-K // 64)
    splits = max(1, min(splits, total))
    per = -(-total // splits)
    return -(-total // per)


def gemm_swiglu_sm100(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, *, token_tile: int = 0,
                      activation: str = "silu") -> None:
    """out[M,I] = act(x wg^T) * (x wu^T) with w_gate_up = [wg (I rows); wu (I rows)]: the gate is
    applied in the product's epilogue (act = silu or the tanh form of gelu).  ``out`` may be a block of columns
    of a wider buffer."""
    M, K = x.shape
    I = out.shape[1]
    if w_gate_up.shape != (2 * I, K) or out.shape[0] != M or out.dtype != torch.bfloat16 or activation not in GATE_ACTIVATIONS:
        raise KernelError("gemm_swiglu_sm100: shapes do not fit")
    ldc = _column_block(out, "gemm_swiglu_sm100 out")
    status = _ptr(_gemm_status(w_gate_up.device))
    f = _fn("gemm_sm100", "ng_gemm_sm100", _GEMM_ARGS)
    _check(f(_ptr(x), _ptr(w_gate_up), None, out.data_ptr(), M, I, K, 2 * I, ldc, 4 if activation == "gelu_tanh" else 2, 1, I,
             token_tile, status, _stream()), "gemm_swiglu_sm100")


# ----------------------------------------------------------------------------- matrix products
_SMS = {}


def sm_count(device) -> int:
    key = str(device)
    if key not in _SMS:
        _SMS[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _SMS[key]


MAX_RESIDUAL_SPLITS = 16


def linear_to_residual(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], ws, name: str,
                       residual: Optional[torch.Tensor] = None):
    """A product whose consumer can add partial sums (``add_rmsnorm``, ``residual_add``,
    ``shortconv``, ``rope_cache``).  Returns [M,N] in the activation dtype, or, for few rows on
    the tcgen05 path, a float32 stack [S,M,N] of split-K partial sums: with few rows the product
    is a stream of the weights, and splitting K puts every SM on it.

    ``residual`` (float32 [M,N]): the product is added straight into it when the kernel can
    do that, and None is returned: nothing is left for the caller to add."""
    M, K = x.shape
    N = weight.shape[0]
    if bias is None and M <= 64 and gemm_sm100_ok(x, weight):
        tiles = -(-N // 128)
        want = min(MAX_RESIDUAL_SPLITS, max(1, sm_count(weight.device) // tiles), max(1, -(-K // 64) // 4))
        s = gemm_splits(K, want)
        if FUSE_RED and residual is not None and M <= FUSE_MAX_ROWS:
            _f32(residual, "residual")
            f = _fn("gemm_sm100", "ng_gemm_sm100", _GEMM_ARGS)
            _check(f(_ptr(x), _ptr(weight), None, _ptr(residual), M, N, K, N, N, 3, s, 0, 0,
                     _ptr(_gemm_status(weight.device)), _stream()), "gemm_sm100 (residual add)")
            return None
        if s > 1:
            # partial sums exist for steps of at most 64 rows only
            buf = ws.flat(name + "_partials", s * M * N, torch.float32,
                          reserve=MAX_RESIDUAL_SPLITS * min(ws.max_rows, 64) * N)
            buf = buf[: s * M * N].view(s, M, N)
            gemm_sm100(x, weight, None, buf, splits=s)
            return buf
    out = ws.buf(name, M, N, x.dtype)
    linear(x, weight, bias, out)
    return out


def residual_add_fusable(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether ``linear_to_residual(x, weight, None, ..., residual=h)`` adds the product into ``h`` itself."""
    return FUSE_RED and x.shape[0] <= min(64, FUSE_MAX_ROWS) and gemm_sm100_ok(x, weight)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out = x @ weight^T (+ bias).  float32: the FFMA kernel above.  bfloat16: the tcgen05
    kernel of this package, or the vendor library's product (``NEUROGRID_B200_GEMM=cublas``,
    and for operands the kernel does not take; the reference uses cuBLAS for every
    contraction, gpu/cuda/matmul.cu:316-355); float32 accumulation either way; ``out`` may be
    float32 (logits)."""
    if x.dtype == torch.float32:
        gemm_f32(x, weight, bias, out)
        return
    if not x.is_cuda:
        raise KernelError("linear: tensors must be on a CUDA device (there is no CPU path)")
    if gemm_sm100_ok(x, weight) and (bias is None or out.dtype == torch.bfloat16):
        gemm_sm100(x, weight, bias, out)
        return
    if out.dtype == torch.float32:
        torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
        if bias is not None:
            out += bias
    elif bias is not None:
        torch.addmm(bias, x, weight.t(), out=out)
    else:
        torch.mm(x, weight.t(), out=out)
