"""Python faces of the CUDA kernels: argument checks, output allocation, launch.

Every function takes CUDA tensors and launches on torch's current stream, so a
step can be captured into a CUDA graph.  A CPU tensor, a non-contiguous tensor,
a wrong element type or a size the kernel does not take raises; nothing here
falls back to a library implementation.

Matrix products without a fused epilogue go to cuBLAS through ``torch`` in the
bfloat16 mode, where the reference engine also calls a library
(src/backends/cuda/ops/gemm_cublaslt.cc:391-396); the 32-bit mode runs the
library's own fp32 FFMA kernel so that no reduced-precision matrix mode can
enter.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import library

# The library GEMM behind ``torch.mm`` may add its split-K partial sums in bf16; sums are
# to be fp32 here (a small result of large terms otherwise carries the rounding of the
# terms).  A process-wide torch setting: this package turns it off where it is imported.
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False

F32, BF16 = 0, 1

_ERRORS = {
    -1: "element type not supported by this kernel",
    -2: "a size this kernel does not take",
    -3: "pointer or stride not aligned as the kernel requires",
    -4: "shared memory need exceeds the device limit for these sizes",
    -5: "this combination of options is not built",
}


class KernelError(RuntimeError):
    pass


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"element type {t.dtype} is not float32 or bfloat16")


def _chk(name: str, t: Optional[torch.Tensor], dtype=None, optional: bool = False):
    if t is None:
        if optional:
            return
        raise KernelError(f"{name}: tensor required")
    if not isinstance(t, torch.Tensor):
        raise KernelError(f"{name}: expected a tensor, got {type(t).__name__}")
    if not t.is_cuda:
        raise KernelError(
            f"{name}: tensor is on {t.device}; the kernels run on a CUDA device only "
            "(there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name}: tensor must be contiguous, strides {t.stride()}")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """The current CUDA stream's handle.  ``torch.cuda.current_stream()`` costs several
    microseconds of Python per call (device lookups, a Stream object); with a few hundred
    launches in an eager step that adds up, so the raw getter is used where torch has it."""
    if _raw_stream is not None and _raw_device is not None:
        return ctypes.c_void_p(_raw_stream(_raw_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(code: int, what: str):
    if code == 0:
        return
    if code < 0:
        raise KernelError(f"{what}: {_ERRORS.get(code, f'error {code}')}")
    raise KernelError(f"{what}: CUDA error {code} at launch")


def _lib():
    return library.load()


LAUNCHES = [0]        # launches of this library's own kernels issued through this module
LIBRARY_CALLS = [0]   # matrix products handed to cuBLAS


def _count(n: int = 1):
    LAUNCHES[0] += n


# Steps of at most this many tokens launch their kernels with programmatic stream
# serialisation, and their dense projections stream the weights with this library's own
# kernel (SMALL_M_DENSE_ROWS below is the same number on purpose).  Beyond it the dense
# projections go to the library GEMM and dependent launch is off: a step that mixes
# dependent launches with the library's plain launches measured far slower than either
# (batch 32: 11.7 ms mixed, 9.8 ms own kernels + dependent launch, 9.2 ms library GEMMs
# without it; batch 16: 7.3 / 5.9 / 6.0 ms).
DEPENDENT_LAUNCH_MAX_TOKENS = 16


def set_dependent_launch(on: bool) -> None:
    """Let the kernels of the coming launches start while their predecessor drains
    (programmatic dependent launch).  Worth it for steps of a few tokens."""
    _lib().ix_dependent_launch_flag(1 if on else 0)


# ---------------------------------------------------------------------------
# Sizes the kernels refuse.  Parts call these when a model is built, so that a model the
# kernels cannot run is refused with the offending size named, before weights are read;
# the kernels' own checks remain (they return "a size this kernel does not take").
def check_attention_limits(heads: int, kv_heads: int, head_dim: int, dtype, where: str = "",
                           allow_odd: bool = False):
    lib = _lib()
    most = lib.ix_attention_max_head_dim()
    if head_dim > most:
        raise KernelError(f"{where}: head size {head_dim} exceeds the largest the attention "
                          f"kernels take ({most})")
    if head_dim % 2 and not allow_odd:
        raise KernelError(f"{where}: head size {head_dim} is odd")
    if heads > 65535 or heads % max(1, kv_heads):
        raise KernelError(f"{where}: {heads} heads over {kv_heads} key/value heads is not a "
                          "grouping the attention kernels take (a multiple, at most 65535)")


def check_router_limits(hidden: int, num_experts: int, top_k: int, where: str = ""):
    lib = _lib()
    if top_k > lib.ix_router_max_topk():
        raise KernelError(f"{where}: {top_k} experts per token exceed the router kernel's "
                          f"limit of {lib.ix_router_max_topk()}")
    if num_experts > lib.ix_router_max_experts():
        raise KernelError(f"{where}: {num_experts} experts exceed the dispatch kernels' limit "
                          f"of {lib.ix_router_max_experts()}")
    if top_k > num_experts:
        raise KernelError(f"{where}: {top_k} experts per token of {num_experts}")


def check_router_group_limits(group_count: int, where: str = ""):
    most = _lib().ix_router_max_groups()
    if group_count > most:
        raise KernelError(f"{where}: {group_count} router groups exceed the selection "
                          f"kernel's limit of {most}")


def embed(table: torch.Tensor, ids: torch.Tensor, out: Optional[torch.Tensor] = None,
          scale: float = 1.0):
    """out[t] = table[ids[t]] * scale, widened to fp32 (the residual stream)."""
    _chk("table", table)
    _chk("ids", ids, torch.int32)
    V, H = table.shape
    T = ids.numel()
    if out is None:
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    _chk("out", out, torch.float32)
    _check(_lib().ix_embed(_ptr(table), _dtype_code(table), _ptr(ids), T, H, V, _ptr(out),
                           ctypes.c_float(scale), _stream()), "embed")
    _count()
    return out


class CombinePending:
    """The output of a mixture-of-experts block that has not been written yet: the
    expert rows, where each token's rows are, their weights and the shared expert's
    part.  ``add_rmsnorm`` consumes it in the same pass that adds it to the residual;
    ``materialize`` writes it out like ``moe_combine``."""

    def __init__(self, y, dest, topk_w, shared, shared_logit):
        self.y, self.dest, self.topk_w = y, dest, topk_w
        self.shared, self.shared_logit = shared, shared_logit
        self.shape = (topk_w.shape[0], y.shape[1])
        self.dtype = y.dtype

    def materialize(self):
        return moe_combine(self.y, self.dest, self.topk_w, self.shared, self.shared_logit)


def moe_combine_pending(y, dest, topk_w, shared, shared_logit):
    """``moe_combine`` deferred into the next residual add + norm where that kernel
    exists (bfloat16, width a multiple of 8); the combined tensor otherwise."""
    if y.dtype == torch.bfloat16 and y.shape[1] % 8 == 0 and y.shape[1] <= 8192:
        return CombinePending(y, dest, topk_w, shared, shared_logit)
    return moe_combine(y, dest, topk_w, shared, shared_logit)


def add_rmsnorm(resid: torch.Tensor, delta, gain: torch.Tensor,
                eps: float, out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None):
    """resid += delta (kept when ``rows`` is None); returns RMSNorm(resid) * gain.

    With ``rows`` the listed rows are gathered, normalised and returned without
    writing the residual back.  ``delta`` may be a ``CombinePending``."""
    if isinstance(delta, CombinePending):
        if rows is None and out_dtype == torch.bfloat16 and delta.shape == tuple(resid.shape):
            _chk("resid", resid, torch.float32)
            _chk("gain", gain, torch.float32)
            T, H = resid.shape
            out = torch.empty((T, H), dtype=out_dtype, device=resid.device)
            code = _lib().ix_combine_add_rmsnorm(
                _ptr(resid), _ptr(delta.y), _ptr(delta.dest), _ptr(delta.topk_w),
                _ptr(delta.shared), _ptr(delta.shared_logit), _ptr(gain), _ptr(out), T, H,
                delta.topk_w.shape[1], ctypes.c_float(eps), _stream())
            _check(code, "combine_add_rmsnorm")
            _count()
            return out
        delta = delta.materialize()
    _chk("resid", resid, torch.float32)
    _chk("gain", gain, torch.float32)
    _chk("delta", delta, optional=True)
    _chk("rows", rows, torch.int32, optional=True)
    T, H = resid.shape
    if gain.numel() != H:
        raise KernelError(f"add_rmsnorm: gain has {gain.numel()} entries, rows have {H}")
    if delta is not None and (delta.shape != resid.shape or delta.dtype != out_dtype):
        raise KernelError("add_rmsnorm: delta must match the residual's shape and the "
                          f"activation type ({tuple(delta.shape)}, {delta.dtype})")
    R = T if rows is None else rows.numel()
    out = torch.empty((R, H), dtype=out_dtype, device=resid.device)
    _check(_lib().ix_add_rmsnorm(_ptr(resid), _ptr(delta), _ptr(gain), _ptr(rows), _ptr(out),
                                 _dtype_code(out), R, H, ctypes.c_float(eps),
                                 1 if rows is None else 0, _stream()), "add_rmsnorm")
    _count()
    return out


def silu_mul(gu: torch.Tensor):
    _chk("gu", gu)
    T, two_i = gu.shape
    if two_i % 2:
        raise KernelError("silu_mul: width must be even (gate | up)")
    out = torch.empty((T, two_i // 2), dtype=gu.dtype, device=gu.device)
    _check(_lib().ix_silu_mul(_ptr(gu), _ptr(out), _dtype_code(gu), T, two_i // 2, _stream()),
           "silu_mul")
    _count()
    return out


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None):
    """x[M,K] . w[N,K]^T.  bfloat16: cuBLAS, fp32 accumulation.  float32: own FFMA kernel."""
    _chk("x", x)
    _chk("w", w)
    if x.dtype != w.dtype:
        raise KernelError(f"linear: activations are {x.dtype} but weights are {w.dtype}")
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"linear: inner sizes differ ({K} vs {K2})")
    out_dtype = out_dtype or x.dtype
    if M <= SMALL_M_DENSE_ROWS and _streams_weights(x, w):
        return gemm_small_m(x, w.unsqueeze(0), None, None, False, M, out_dtype=out_dtype,
                            rows_per_pass=M)
    if x.dtype == torch.bfloat16:
        LIBRARY_CALLS[0] += 1
        if out_dtype == torch.bfloat16:
            return torch.mm(x, w.t())
        return torch.mm(x, w.t(), out_dtype=out_dtype)
    return gemm_generic(x, w.unsqueeze(0), None, None, dual=False, out_dtype=out_dtype)


def gemm_generic(x: torch.Tensor, w: torch.Tensor, rows: Optional[torch.Tensor],
                 offsets: Optional[torch.Tensor], dual: bool,
                 out_dtype: Optional[torch.dtype] = None, num_out_rows: Optional[int] = None):
    """CUDA-core product, single (offsets None) or grouped by expert."""
    _chk("x", x)
    _chk("w", w)
    _chk("rows", rows, torch.int32, optional=True)
    _chk("offsets", offsets, torch.int32, optional=True)
    E, w_rows, K = w.shape
    N = w_rows // 2 if dual else w_rows
    if x.shape[1] != K:
        raise KernelError(f"gemm: inner sizes differ ({x.shape[1]} vs {K})")
    out_dtype = out_dtype or x.dtype
    if offsets is None:
        M = x.shape[0]
        A = M
    else:
        M = 0
        A = num_out_rows if num_out_rows is not None else (
            rows.numel() if rows is not None else x.shape[0])
    out = torch.empty((A, N), dtype=out_dtype, device=x.device)
    code = _lib().ix_gemm_generic(
        _ptr(x), _ptr(rows), _ptr(offsets), _ptr(w), _ptr(out), _dtype_code(x),
        F32 if out_dtype == torch.float32 else BF16, 1 if dual else 0, M, N, K, E, A, _stream())
    _check(code, "gemm_generic")
    _count()
    return out


def qkv_rope_append(qkv: torch.Tensor, bias: Optional[torch.Tensor], positions: torch.Tensor,
                    inv_freq: Optional[torch.Tensor], rotary_dim: int, heads: int, kv_heads: int,
                    head_dim: int, k_cache: Optional[torch.Tensor],
                    v_cache: Optional[torch.Tensor], slots: Optional[torch.Tensor],
                    want_dense_kv: bool = False, value_dim: int = 0):
    """Split + bias + rotate; returns q [T,heads,hd] (and dense k, v when asked);
    writes k, v into the paged cache at ``slots`` when a cache is given.  ``value_dim``:
    the size of a value head when it differs from ``head_dim`` (the row is then
    q | k | v with v of kv_heads * value_dim, and the value pages are that wide)."""
    _chk("qkv", qkv)
    _chk("bias", bias, torch.float32, optional=True)
    _chk("positions", positions, torch.int32)
    _chk("inv_freq", inv_freq, torch.float32, optional=True)
    _chk("slots", slots, torch.int32, optional=True)
    T, width = qkv.shape
    vd = value_dim or head_dim
    if width != (heads + kv_heads) * head_dim + kv_heads * vd:
        raise KernelError(f"qkv_rope_append: row width {width} is not (heads+kv_heads)*head_dim "
                          "+ kv_heads*value_dim")
    if bias is not None and bias.numel() != width:
        raise KernelError("qkv_rope_append: bias length does not match the fused row")
    if rotary_dim and (inv_freq is None or inv_freq.numel() != rotary_dim // 2):
        raise KernelError("qkv_rope_append: inv_freq must have rotary_dim/2 entries")
    page_size = 1
    if k_cache is not None:
        _chk("k_cache", k_cache, qkv.dtype)
        _chk("v_cache", v_cache, qkv.dtype)
        if slots is None:
            raise KernelError("qkv_rope_append: a cache needs slots")
        P, ckv, page_size, chd = k_cache.shape
        if ckv != kv_heads or chd != head_dim or \
                tuple(v_cache.shape) != (P, ckv, page_size, vd):
            raise KernelError("qkv_rope_append: cache geometry does not match the heads")
    q = torch.empty((T, heads, head_dim), dtype=qkv.dtype, device=qkv.device)
    k = v = None
    if want_dense_kv:
        k = torch.empty((T, kv_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
        v = torch.empty((T, kv_heads, vd), dtype=qkv.dtype, device=qkv.device)
    code = _lib().ix_qkv_rope_append(
        _ptr(qkv), _ptr(bias), _ptr(positions), _ptr(inv_freq), rotary_dim, _ptr(slots), _ptr(q),
        _ptr(k_cache), _ptr(v_cache), page_size, _ptr(k), _ptr(v), _dtype_code(qkv), T, heads,
        kv_heads, head_dim, vd, _stream())
    _check(code, "qkv_rope_append")
    _count()
    return (q, k, v) if want_dense_kv else q


USE_FUSED_QKV = True


def qkv_project_applies(x: torch.Tensor, w: torch.Tensor, heads: int, kv_heads: int,
                        head_dim: int, rotary_dim: int) -> bool:
    """Whether ``qkv_project_rope_append`` takes this step: bfloat16, a few tokens, a full
    rotation or none."""
    return bool(USE_FUSED_QKV and x.is_cuda and x.dtype == torch.bfloat16
                and w.dtype == torch.bfloat16 and x.is_contiguous()
                and _lib().ix_qkv_project_rope_applies(x.shape[0], x.shape[1], heads, kv_heads,
                                                       head_dim, rotary_dim))


def qkv_project_rope_append(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor],
                            positions: torch.Tensor, inv_freq: Optional[torch.Tensor],
                            rotary_dim: int, heads: int, kv_heads: int, head_dim: int,
                            k_cache: torch.Tensor, v_cache: torch.Tensor, slots: torch.Tensor):
    """For a step of a few tokens: q = rotate(x . Wq^T + bq) returned as [T, heads, hd],
    rotate(x . Wk^T + bk) and x . Wv^T + bv written into the cache pages at ``slots``, in one
    launch (``linear`` followed by ``qkv_rope_append`` otherwise)."""
    _chk("x", x, torch.bfloat16)
    _chk("w", w, torch.bfloat16)
    _chk("bias", bias, torch.float32, optional=True)
    _chk("positions", positions, torch.int32)
    _chk("inv_freq", inv_freq, torch.float32, optional=True)
    _chk("slots", slots, torch.int32)
    _chk("k_cache", k_cache, torch.bfloat16)
    _chk("v_cache", v_cache, torch.bfloat16)
    T, K = x.shape
    width = (heads + 2 * kv_heads) * head_dim
    if w.shape != (width, K) or (bias is not None and bias.numel() != width):
        raise KernelError("qkv_project_rope_append: weight or bias does not match the heads")
    P, ckv, page_size, chd = k_cache.shape
    if ckv != kv_heads or chd != head_dim or v_cache.shape != k_cache.shape:
        raise KernelError("qkv_project_rope_append: cache geometry does not match the heads")
    if rotary_dim and (inv_freq is None or inv_freq.numel() != rotary_dim // 2):
        raise KernelError("qkv_project_rope_append: inv_freq must have rotary_dim/2 entries")
    if positions.numel() != T or slots.numel() != T:
        raise KernelError("qkv_project_rope_append: one position and one slot per token")
    q = torch.empty((T, heads, head_dim), dtype=torch.bfloat16, device=x.device)
    code = _lib().ix_qkv_project_rope_append(
        _ptr(x), _ptr(w), _ptr(bias), _ptr(positions), _ptr(inv_freq), rotary_dim, _ptr(slots),
        _ptr(q), _ptr(k_cache), _ptr(v_cache), page_size, T, K, heads, kv_heads, head_dim,
        _stream())
    _check(code, "qkv_project_rope_append")
    _count()
    return q


def paged_attention_generic(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                            block_table: torch.Tensor, seq_of_token: torch.Tensor,
                            positions: torch.Tensor, window: int, scale: float,
                            softcap: float = 0.0, keep_first: int = 0, sink: bool = False):
    _chk("q", q)
    _chk("k_cache", k_cache, q.dtype)
    _chk("v_cache", v_cache, q.dtype)
    _chk("block_table", block_table, torch.int32)
    _chk("seq_of_token", seq_of_token, torch.int32)
    _chk("positions", positions, torch.int32)
    T, heads, hd = q.shape
    P, kvh, page, chd = k_cache.shape
    vd = v_cache.shape[3]
    if chd != hd or tuple(v_cache.shape[:3]) != (P, kvh, page):
        raise KernelError("paged_attention: cache head size differs from the query's")
    out = torch.empty((T, heads, vd), dtype=q.dtype, device=q.device)
    code = _lib().ix_paged_attention_generic(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), _ptr(seq_of_token),
        _ptr(positions), _ptr(out), _dtype_code(q), T, heads, kvh, hd, vd, page,
        block_table.shape[1], window, ctypes.c_float(scale), ctypes.c_float(softcap),
        int(keep_first), 1 if sink else 0, _stream())
    _check(code, "paged_attention_generic")
    _count()
    return out


def paged_attention_tiled(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                          block_table: torch.Tensor, cu_q: torch.Tensor, q_pos0: torch.Tensor,
                          window: int, scale: float, softcap: float = 0.0, keep_first: int = 0,
                          sink: bool = False):
    """CUDA-core attention for a ragged batch, tiled (32 queries of a sequence against 64
    keys at a time in shared memory, fp32 math): sequence s brings the queries
    q[cu_q[s]:cu_q[s+1]] at positions q_pos0[s], q_pos0[s]+1, ...  Any element type, head
    sizes that are a multiple of 4 up to 256; the value pages may have a head size of
    their own (the output then has it)."""
    _chk("q", q)
    _chk("k_cache", k_cache, q.dtype)
    _chk("v_cache", v_cache, q.dtype)
    _chk("block_table", block_table, torch.int32)
    _chk("cu_q", cu_q, torch.int32)
    _chk("q_pos0", q_pos0, torch.int32)
    T, heads, hd = q.shape
    P, kvh, page, chd = k_cache.shape
    S = q_pos0.numel()
    vd = v_cache.shape[3]
    if chd != hd or tuple(v_cache.shape[:3]) != (P, kvh, page):
        raise KernelError("paged_attention_tiled: cache geometry differs from the query's")
    if cu_q.numel() != S + 1 or block_table.shape[0] != S:
        raise KernelError("paged_attention_tiled: cu_q, q_pos0 and block_table disagree")
    out = torch.empty((T, heads, vd), dtype=q.dtype, device=q.device)
    code = _lib().ix_paged_attention_tiled(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), _ptr(cu_q), _ptr(q_pos0),
        _ptr(out), _dtype_code(q), T, S, heads, kvh, hd, vd, page, block_table.shape[1], window,
        ctypes.c_float(scale), ctypes.c_float(softcap), int(keep_first), 1 if sink else 0,
        _stream())
    _check(code, "paged_attention_tiled")
    _count()
    return out


# A batch with at least this many queries a sequence on average goes to the tiled
# CUDA-core kernel where the tensor-core kernels do not apply; fewer (single decoded
# tokens, mostly) to the kernel that gives every (token, head) a block of its own.
TILED_ATTENTION_MIN_QUERIES = 4


# below this many tokens the router runs as two kernels (logits by one warp per (token,
# expert), then selection); from it on as one fused kernel (equal at 128 tokens, 13 us
# against 19-21 us at 200-256)
ROUTER_FEW_TOKENS = 128


def router_topk(x: torch.Tensor, w: torch.Tensor, top_k: int, renormalize: bool, scale: float,
                extra_w: Optional[torch.Tensor] = None,
                correction: Optional[torch.Tensor] = None, group_count: int = 0,
                group_keep: int = 0, renorm_eps: Optional[float] = None
                ) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """fp32 router logits, softmax over all experts, top-k (ties to the lower index).

    ``correction`` (fp32 [E]) is added to the scores for the choice alone; with
    ``group_count`` > 0 the outputs form that many equal groups of neighbours and only
    outputs of the ``group_keep`` groups with the largest corrected score can be chosen;
    ``renorm_eps`` >= 0 divides the chosen scores by (their sum + renorm_eps).

    Returns (weights [T,k] fp32, experts [T,k] int32, x.extra_w [T] fp32 or None).
    Few tokens: one warp per (token, expert) computes the logits and one warp per
    token selects; many tokens: one fused kernel over 4 to 16 tokens per block.  Both form
    a dot product in the same order, so a token's routing is the same in either."""
    _chk("x", x)
    _chk("w", w, torch.float32)
    _chk("extra_w", extra_w, torch.float32, optional=True)
    T, H = x.shape
    E = w.shape[0]
    if w.shape[1] != H or (extra_w is not None and extra_w.numel() != H):
        raise KernelError("router_topk: weight width differs from the activations'")
    tw = torch.empty((T, top_k), dtype=torch.float32, device=x.device)
    ti = torch.empty((T, top_k), dtype=torch.int32, device=x.device)
    ex = torch.empty((T,), dtype=torch.float32, device=x.device) if extra_w is not None else None
    few = T < ROUTER_FEW_TOKENS   # few tokens: logits by many blocks, then a selection kernel
    scratch = torch.empty((T, E), dtype=torch.float32, device=x.device) if few else None
    ruled = (correction is not None or group_count > 0
             or (renorm_eps is not None and renorm_eps >= 0))
    if ruled:
        _chk("correction", correction, torch.float32, optional=True)
        if correction is not None and correction.numel() != E:
            raise KernelError("router_topk: one correction per router output")
        code = _lib().ix_router_topk_ruled(
            _ptr(x), _ptr(w), _ptr(extra_w), _dtype_code(x), T, H, E, top_k,
            1 if renormalize else 0, ctypes.c_float(scale), _ptr(correction), int(group_count),
            int(group_keep), ctypes.c_float(-1.0 if renorm_eps is None else renorm_eps),
            _ptr(tw), _ptr(ti), _ptr(ex), _ptr(scratch), _stream())
    else:
        code = _lib().ix_router_topk(
            _ptr(x), _ptr(w), _ptr(extra_w), _dtype_code(x), T, H, E, top_k,
            1 if renormalize else 0, ctypes.c_float(scale), _ptr(tw), _ptr(ti), _ptr(ex),
            _ptr(scratch), _stream())
    _check(code, "router_topk")
    _count(2 if few else 1)
    return tw, ti, ex


def moe_dispatch(topk_idx: torch.Tensor, num_experts: int):
    """offsets[E+1], rows[A] (token of each grouped row), dest[A] (grouped row of t*k+slot)."""
    _chk("topk_idx", topk_idx, torch.int32)
    T, k = topk_idx.shape
    dev = topk_idx.device
    offsets = torch.empty((num_experts + 1,), dtype=torch.int32, device=dev)
    rows = torch.empty((T * k,), dtype=torch.int32, device=dev)
    dest = torch.empty((T * k,), dtype=torch.int32, device=dev)
    n_scratch = _lib().ix_moe_dispatch_scratch_ints(T, num_experts, k)
    scratch = torch.empty((n_scratch,), dtype=torch.int32, device=dev) if n_scratch else None
    _check(_lib().ix_moe_dispatch(_ptr(topk_idx), T, num_experts, k, _ptr(offsets), _ptr(rows),
                                  _ptr(dest), _ptr(scratch), _stream()), "moe_dispatch")
    _count(3 if n_scratch else 1)
    return offsets, rows, dest


def moe_combine(y: torch.Tensor, dest: torch.Tensor, topk_w: torch.Tensor,
                shared: Optional[torch.Tensor], shared_logit: Optional[torch.Tensor]):
    _chk("y", y)
    _chk("dest", dest, torch.int32)
    _chk("topk_w", topk_w, torch.float32)
    _chk("shared", shared, y.dtype, optional=True)
    _chk("shared_logit", shared_logit, torch.float32, optional=True)
    T, k = topk_w.shape
    H = y.shape[1]
    out = torch.empty((T, H), dtype=y.dtype, device=y.device)
    _check(_lib().ix_moe_combine(_ptr(y), _ptr(dest), _ptr(topk_w), _ptr(shared),
                                 _ptr(shared_logit), _ptr(out), _dtype_code(y), T, H, k,
                                 _stream()), "moe_combine")
    _count()
    return out


def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor] = None,
           seeds: Optional[torch.Tensor] = None, top_p: Optional[torch.Tensor] = None,
           top_k: Optional[torch.Tensor] = None, min_p: Optional[torch.Tensor] = None,
           out: Optional[torch.Tensor] = None):
    """Token ids [R] int32 from fp32 logits [R,V]; greedy where temperature <= 0 or absent."""
    _chk("logits", logits, torch.float32)
    _chk("temperature", temperature, torch.float32, optional=True)
    _chk("seeds", seeds, torch.int64, optional=True)
    _chk("top_p", top_p, torch.float32, optional=True)
    _chk("top_k", top_k, torch.int32, optional=True)
    _chk("min_p", min_p, torch.float32, optional=True)
    R, V = logits.shape
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    _chk("out", out, torch.int32)
    _check(_lib().ix_sample(_ptr(logits), R, V, _ptr(temperature), _ptr(top_p), _ptr(top_k),
                            _ptr(min_p), _ptr(seeds), _ptr(out), _stream()), "sample")
    _count()
    return out


def apply_penalties(logits: torch.Tensor, hist_ids: Optional[torch.Tensor],
                    hist_counts: Optional[torch.Tensor], penalties: Optional[torch.Tensor],
                    mask_ids: Optional[torch.Tensor]) -> None:
    """Penalties and masks on fp32 logits [R,V], in place, before a token is chosen:
    ``hist_ids`` / ``hist_counts`` [R,H] int32 (distinct generated ids and how often, -1
    padded) with ``penalties`` [R,3] (presence, frequency, repetition), and ``mask_ids``
    [R,M] int32 (tokens set to -inf, -1 padded); either group may be absent."""
    _chk("logits", logits, torch.float32)
    _chk("hist_ids", hist_ids, torch.int32, optional=True)
    _chk("hist_counts", hist_counts, torch.int32, optional=True)
    _chk("penalties", penalties, torch.float32, optional=True)
    _chk("mask_ids", mask_ids, torch.int32, optional=True)
    R, V = logits.shape
    if (hist_ids is None) != (hist_counts is None) or (hist_ids is None) != (penalties is None):
        raise KernelError("apply_penalties: history ids, counts and penalties come together")
    if hist_ids is not None and (hist_ids.shape != hist_counts.shape or hist_ids.shape[0] != R
                                 or tuple(penalties.shape) != (R, 3)):
        raise KernelError("apply_penalties: history or penalties do not match the rows")
    if mask_ids is not None and mask_ids.shape[0] != R:
        raise KernelError("apply_penalties: mask does not match the rows")
    if hist_ids is None and mask_ids is None:
        return
    _check(_lib().ix_apply_penalties(
        _ptr(logits), R, V, _ptr(hist_ids), _ptr(hist_counts),
        0 if hist_ids is None else hist_ids.shape[1], _ptr(penalties), _ptr(mask_ids),
        0 if mask_ids is None else mask_ids.shape[1], _stream()), "apply_penalties")
    _count()


def max_top_logprobs() -> int:
    return int(_lib().ix_logprobs_max_top())


def token_logprobs(logits: torch.Tensor, chosen: torch.Tensor,
                   want_k: Optional[torch.Tensor] = None, top: int = 0):
    """Log-probabilities under softmax(logits) of the chosen tokens [R] and of each row's
    ``want_k[r]`` most probable tokens (ties to the lower id; a negative entry skips the
    row): (chosen_lp [R] fp32, top_ids [R,top] int32 with -1 where unused, top_lps)."""
    _chk("logits", logits, torch.float32)
    _chk("chosen", chosen, torch.int32)
    _chk("want_k", want_k, torch.int32, optional=True)
    R, V = logits.shape
    if chosen.numel() != R or (want_k is not None and want_k.numel() != R):
        raise KernelError("token_logprobs: one chosen token and one count per row")
    if not 0 <= top <= max_top_logprobs():
        raise KernelError(f"token_logprobs: at most {max_top_logprobs()} alternatives")
    dev = logits.device
    chosen_lp = torch.empty((R,), dtype=torch.float32, device=dev)
    top_ids = torch.empty((R, top), dtype=torch.int32, device=dev) if top else None
    top_lps = torch.empty((R, top), dtype=torch.float32, device=dev) if top else None
    _check(_lib().ix_token_logprobs(_ptr(logits), R, V, _ptr(chosen), _ptr(want_k), top,
                                    _ptr(chosen_lp), _ptr(top_ids), _ptr(top_lps), _stream()),
           "token_logprobs")
    _count()
    return chosen_lp, top_ids, top_lps


def append_kv(k: torch.Tensor, v: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
              slots: torch.Tensor):
    """Write dense k, v rows [T,kv_heads,hd] into the paged cache at ``slots``."""
    _chk("k", k)
    _chk("v", v, k.dtype)
    _chk("k_cache", k_cache, k.dtype)
    _chk("v_cache", v_cache, k.dtype)
    _chk("slots", slots, torch.int32)
    T, kvh, hd = k.shape
    P, ckv, page, chd = k_cache.shape
    if (ckv, chd) != (kvh, hd) or v.shape != k.shape or v_cache.shape != k_cache.shape:
        raise KernelError("append_kv: cache geometry does not match the rows")
    _check(_lib().ix_append_kv(_ptr(k), _ptr(v), _ptr(slots), _ptr(k_cache), _ptr(v_cache), page,
                               _dtype_code(k), T, kvh, hd, _stream()), "append_kv")
    _count()


_DECODE_HEAD_SIZES = {torch.bfloat16: (64, 128, 256), torch.float32: (64, 128)}


# Decode attention forms: "tma" (keys and values brought in by TMA), "mma" (the same
# arithmetic fed by cp.async), "scalar" (CUDA cores; fp32 and sizes the others refuse).
USE_TMA_DECODE = True


def _tma_decode_applies(q, page: int) -> bool:
    return (q.dtype == torch.bfloat16 and q.shape[2] in (64, 128)
            and page in (8, 16, 32, 64))


def paged_attention_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                           block_table: torch.Tensor, kv_len: torch.Tensor, max_kv_len: int,
                           window: int, scale: float, splits: Optional[int] = None,
                           kernel: Optional[str] = None, out: Optional[torch.Tensor] = None,
                           softcap: float = 0.0):
    """Split-KV attention for a batch in which sequence s brings the one query q[s]
    at position kv_len[s] - 1.  ``kernel`` picks a form ("tma", "mma", "scalar");
    None takes the fastest that applies."""
    _chk("q", q)
    _chk("k_cache", k_cache, q.dtype)
    _chk("v_cache", v_cache, q.dtype)
    _chk("block_table", block_table, torch.int32)
    _chk("kv_len", kv_len, torch.int32)
    S, heads, hd = q.shape
    P, kvh, page, chd = k_cache.shape
    if chd != hd or v_cache.shape != k_cache.shape:
        raise KernelError("paged_attention_decode: cache geometry differs from the query's")
    if hd not in _DECODE_HEAD_SIZES.get(q.dtype, ()):
        raise KernelError(f"paged_attention_decode: head size {hd} with {q.dtype} is not built; "
                          "use the general kernel")
    if kv_len.numel() != S or block_table.shape[0] != S:
        raise KernelError("paged_attention_decode: one query per sequence is required")
    if kernel is None:
        if USE_TMA_DECODE and _tma_decode_applies(q, page):
            kernel = "tma"
        else:
            kernel = "mma"
    if kernel not in ("tma", "mma", "scalar"):
        raise KernelError(f"paged_attention_decode: no kernel form {kernel!r}")
    if softcap > 0 and kernel != "tma":
        raise KernelError("paged_attention_decode: only the TMA form squashes scores")
    if kernel == "tma" and not _tma_decode_applies(q, page):
        raise KernelError(f"paged_attention_decode: the TMA form takes bf16, head size 64 or 128 "
                          f"and a page of 8, 16, 32 or 64 keys (got {q.dtype}, {hd}, {page})")
    lib = _lib()
    if splits is None:
        pick = lib.ix_attn_decode_tma_splits if kernel == "tma" else lib.ix_attn_decode_splits
        splits = pick(S, heads, kvh, int(max_kv_len))
    if out is None:
        out = torch.empty_like(q)
    else:
        _chk("out", out, q.dtype)
        if out.shape != q.shape:
            raise KernelError("paged_attention_decode: out must have the query's shape")
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.empty((S, heads, splits, hd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((S, heads, splits, 2), dtype=torch.float32, device=q.device)
    if kernel == "tma":
        code = lib.ix_paged_attention_decode_tma_capped(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), P, _ptr(block_table), _ptr(kv_len),
            _ptr(part_o), _ptr(part_ml), _ptr(out), S, heads, kvh, hd, page,
            block_table.shape[1], window, ctypes.c_float(scale), ctypes.c_float(softcap), splits,
            _ptr(_tc_status(q.device)), _stream())
    else:
        entry = (lib.ix_paged_attention_decode_scalar if kernel == "scalar"
                 else lib.ix_paged_attention_decode)
        code = entry(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), _ptr(kv_len), _ptr(part_o),
            _ptr(part_ml), _ptr(out), _dtype_code(q), S, heads, kvh, hd, page,
            block_table.shape[1], window, ctypes.c_float(scale), splits, _stream())
    _check(code, "paged_attention_decode")
    _count(2 if splits > 1 else 1)
    return out


_PREFILL_HEAD_SIZES = {torch.bfloat16: (64, 128)}


# Prompt attention forms: "tc" (tcgen05, S and O in tensor memory, K/V by TMA) and
# "mma" (mma.sync tiles fed by cp.async; any page size).
USE_TCGEN05_ATTENTION = True


def _tc_prefill_applies(q, page: int) -> bool:
    return (q.dtype == torch.bfloat16 and q.shape[2] in (64, 128)
            and page in (8, 16, 32, 64))


def paged_attention_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                            block_table: torch.Tensor, cu_q: torch.Tensor, q_pos0: torch.Tensor,
                            window: int, scale: float, kernel: Optional[str] = None,
                            out: Optional[torch.Tensor] = None, splits: Optional[int] = None,
                            max_kv_len: Optional[int] = None, softcap: float = 0.0):
    """Tensor-core attention for a ragged batch: sequence s brings the queries
    q[cu_q[s]:cu_q[s+1]] at positions q_pos0[s], q_pos0[s]+1, ...  ``kernel`` picks a
    form ("tc", "mma"); None takes the fastest that applies.  ``splits`` (tcgen05 form):
    runs the keys of a query tile are cut into, merged afterwards; None lets the kernel
    module choose (more than one only for few queries over a long context, which it
    judges from ``max_kv_len``, the longest context of the step, or else from the width
    of the block table)."""
    _chk("q", q, torch.bfloat16)
    _chk("k_cache", k_cache, q.dtype)
    _chk("v_cache", v_cache, q.dtype)
    _chk("block_table", block_table, torch.int32)
    _chk("cu_q", cu_q, torch.int32)
    _chk("q_pos0", q_pos0, torch.int32)
    T, heads, hd = q.shape
    P, kvh, page, chd = k_cache.shape
    S = q_pos0.numel()
    if chd != hd or v_cache.shape != k_cache.shape:
        raise KernelError("paged_attention_prefill: cache geometry differs from the query's")
    if hd not in _PREFILL_HEAD_SIZES.get(q.dtype, ()):
        raise KernelError(f"paged_attention_prefill: head size {hd} is not built; use the "
                          "general kernel")
    if cu_q.numel() != S + 1 or block_table.shape[0] != S:
        raise KernelError("paged_attention_prefill: cu_q, q_pos0 and block_table disagree")
    if kernel is None:
        kernel = "tc" if USE_TCGEN05_ATTENTION and _tc_prefill_applies(q, page) else "mma"
    if kernel not in ("tc", "mma"):
        raise KernelError(f"paged_attention_prefill: no kernel form {kernel!r}")
    if softcap > 0 and kernel != "tc":
        raise KernelError("paged_attention_prefill: only the tcgen05 form squashes scores")
    if kernel == "tc" and not _tc_prefill_applies(q, page):
        raise KernelError(f"paged_attention_prefill: the tcgen05 form takes bf16, head size 64 "
                          f"or 128 and a page of 8, 16, 32 or 64 keys (got {q.dtype}, {hd}, "
                          f"{page})")
    if out is None:
        out = torch.empty_like(q)
    else:
        _chk("out", out, q.dtype)
        if out.shape != q.shape:
            raise KernelError("paged_attention_prefill: out must have the query's shape")
    launches = 1
    if kernel == "tc":
        if splits is None:
            keys = int(max_kv_len) if max_kv_len else block_table.shape[1] * page
            splits = _lib().ix_attn_prefill_tc_splits(T, S, heads, keys, window)
        if not 1 <= splits <= 64:
            raise KernelError(f"paged_attention_prefill: splits must be 1..64, got {splits}")
        part_o = part_ml = None
        if splits > 1:
            part_o = torch.empty((T, heads, splits, hd), dtype=torch.float32, device=q.device)
            part_ml = torch.empty((T, heads, splits, 2), dtype=torch.float32, device=q.device)
            launches = 2
        if softcap > 0:
            code = _lib().ix_paged_attention_prefill_tc_capped(
                _ptr(q), _ptr(k_cache), _ptr(v_cache), P, _ptr(block_table), _ptr(cu_q),
                _ptr(q_pos0), _ptr(out), T, S, heads, kvh, hd, page, block_table.shape[1],
                window, ctypes.c_float(scale), ctypes.c_float(softcap), splits, _ptr(part_o),
                _ptr(part_ml), _ptr(_tc_status(q.device)), _stream())
        else:
            code = _lib().ix_paged_attention_prefill_tc(
                _ptr(q), _ptr(k_cache), _ptr(v_cache), P, _ptr(block_table), _ptr(cu_q),
                _ptr(q_pos0), _ptr(out), T, S, heads, kvh, hd, page, block_table.shape[1],
                window, ctypes.c_float(scale), splits, _ptr(part_o), _ptr(part_ml),
                _ptr(_tc_status(q.device)), _stream())
    else:
        code = _lib().ix_paged_attention_prefill(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), _ptr(cu_q), _ptr(q_pos0),
            _ptr(out), _dtype_code(q), T, S, heads, kvh, hd, page, block_table.shape[1], window,
            ctypes.c_float(scale), _stream())
    _check(code, "paged_attention_prefill")
    _count(launches)
    return out


def paged_attention_prefill_exact(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                                  block_table: torch.Tensor, cu_q: torch.Tensor,
                                  q_pos0: torch.Tensor, window: int, scale: float,
                                  keep_first: int = 0, sink: bool = False,
                                  kernel: Optional[str] = None):
    """Tensor-core attention for a ragged batch of bfloat16 queries whose softmax weights
    keep 16 bits in their product with the values (each weight enters as two bfloat16 terms
    into the same fp32 accumulator): for decoders that want scores and weights in 32-bit
    arithmetic.  Key and value heads of 64 or 128 entries each; ``keep_first`` and ``sink``
    as in ``paged_attention``.  ``kernel``: "tc" (tcgen05; keys and values of the same size,
    pages of 8 to 64 keys), "mma" (mma.sync; the sizes may differ, any page size); None
    takes the first that applies."""
    _chk("q", q, torch.bfloat16)
    _chk("k_cache", k_cache, q.dtype)
    _chk("v_cache", v_cache, q.dtype)
    _chk("block_table", block_table, torch.int32)
    _chk("cu_q", cu_q, torch.int32)
    _chk("q_pos0", q_pos0, torch.int32)
    T, heads, hd = q.shape
    P, kvh, page, chd = k_cache.shape
    vd = v_cache.shape[3]
    S = q_pos0.numel()
    if chd != hd or tuple(v_cache.shape[:3]) != (P, kvh, page):
        raise KernelError("paged_attention_prefill_exact: cache geometry differs from the "
                          "query's")
    if cu_q.numel() != S + 1 or block_table.shape[0] != S:
        raise KernelError("paged_attention_prefill_exact: cu_q, q_pos0 and block_table disagree")
    out = torch.empty((T, heads, vd), dtype=q.dtype, device=q.device)
    tc_ok = bool(_lib().ix_paged_attention_prefill_tc_exact_applies(hd, vd, page))
    if kernel is None:
        kernel = "tc" if USE_TCGEN05_ATTENTION and tc_ok else "mma"
    if kernel not in ("tc", "mma") or (kernel == "tc" and not tc_ok):
        raise KernelError(f"paged_attention_prefill_exact: no kernel form {kernel!r} for heads of "
                          f"{hd} / {vd} and pages of {page}")
    if kernel == "tc":
        _check(_lib().ix_paged_attention_prefill_tc_exact(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), P, _ptr(block_table), _ptr(cu_q),
            _ptr(q_pos0), _ptr(out), T, S, heads, kvh, hd, page, block_table.shape[1], window,
            ctypes.c_float(scale), int(keep_first), 1 if sink else 0,
            _ptr(_tc_status(q.device)), _stream()), "paged_attention_prefill_tc_exact")
        _count()
        return out
    _check(_lib().ix_paged_attention_prefill_exact(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), _ptr(cu_q), _ptr(q_pos0),
        _ptr(out), T, S, heads, kvh, hd, vd, page, block_table.shape[1], window,
        ctypes.c_float(scale), int(keep_first), 1 if sink else 0, _stream()),
        "paged_attention_prefill_exact")
    _count()
    return out


def paged_attention_decode_exact(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                                 block_table: torch.Tensor, kv_len: torch.Tensor, max_kv_len: int,
                                 window: int, scale: float, splits: Optional[int] = None,
                                 keep_first: int = 0, sink: bool = False):
    """Split-KV tensor-core attention (mma.sync) for a batch in which sequence s brings the
    one bfloat16 query q[s] at position kv_len[s] - 1, with softmax weights that keep 16 bits
    in their product with the values; key and value heads of 64 or 128 entries each."""
    _chk("q", q, torch.bfloat16)
    _chk("k_cache", k_cache, q.dtype)
    _chk("v_cache", v_cache, q.dtype)
    _chk("block_table", block_table, torch.int32)
    _chk("kv_len", kv_len, torch.int32)
    S, heads, hd = q.shape
    P, kvh, page, chd = k_cache.shape
    vd = v_cache.shape[3]
    if chd != hd or tuple(v_cache.shape[:3]) != (P, kvh, page):
        raise KernelError("paged_attention_decode_exact: cache geometry differs from the query's")
    if kv_len.numel() != S or block_table.shape[0] != S:
        raise KernelError("paged_attention_decode_exact: one query per sequence is required")
    lib = _lib()
    if splits is None:
        span = min(int(max_kv_len), window + keep_first) if window > 0 else int(max_kv_len)
        splits = lib.ix_attn_decode_splits(S, heads, kvh, span)
    out = torch.empty((S, heads, vd), dtype=q.dtype, device=q.device)
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.empty((S, heads, splits, vd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((S, heads, splits, 2), dtype=torch.float32, device=q.device)
    _check(lib.ix_paged_attention_decode_exact(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), _ptr(kv_len), _ptr(part_o),
        _ptr(part_ml), _ptr(out), S, heads, kvh, hd, vd, page, block_table.shape[1], window,
        ctypes.c_float(scale), splits, int(keep_first), 1 if sink else 0, _stream()),
        "paged_attention_decode_exact")
    _count(2 if splits > 1 else 1)
    return out


# The fp32-weights path takes the tensor-core kernels with 16-bit weights where they apply.
USE_EXACT_TC_ATTENTION = True


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    block_table: torch.Tensor, step, window: int, scale: float,
                    softcap: float = 0.0, fp32_weights: bool = False, keep_first: int = 0,
                    sink: bool = False):
    """Causal attention of this step's queries over the paged cache.  ``keep_first``: with
    a window, the sequence's first tokens stay visible beside it; ``sink``: one is added
    to the softmax's denominator (both run on the fp32-arithmetic kernels).  With ``softcap``
    > 0 a score s becomes softcap * tanh(s / softcap) before the softmax.  With
    ``fp32_weights``, or value pages whose head size differs from the keys', the
    fp32-arithmetic kernels run whatever the element type.

    ``step`` carries the batch description (``seq_of_token``, ``positions``, ``cu_q``,
    ``q_pos0``, ``kv_len``, ``max_q_len``, ``max_kv_len``, ``all_decode``).  Steps of
    single tokens go to the split-KV kernel; everything else, and head sizes the
    tuned kernels do not take, to the general kernel."""
    hd = q.shape[2]
    page = k_cache.shape[2]
    if fp32_weights or v_cache.shape[3] != hd or sink or (keep_first and window > 0):
        return _paged_attention_softcap(q, k_cache, v_cache, block_table, step, window, scale,
                                        softcap, keep_first if window > 0 else 0, sink)
    if softcap > 0 and not (scale > 0 and USE_TMA_DECODE and _tma_decode_applies(q, page)
                            and USE_TCGEN05_ATTENTION and _tc_prefill_applies(q, page)):
        # of the tuned kernels only the TMA decode form and the tcgen05 prompt form squash
        return _paged_attention_softcap(q, k_cache, v_cache, block_table, step, window, scale,
                                        softcap)
    if step.all_decode and hd in _DECODE_HEAD_SIZES.get(q.dtype, ()):
        return paged_attention_decode(q, k_cache, v_cache, block_table, step.kv_len,
                                      step.max_kv_len, window, scale, softcap=softcap)
    if hd in _PREFILL_HEAD_SIZES.get(q.dtype, ()):
        nd = getattr(step, "num_decode_seqs", 0)
        if 0 < nd < step.num_seqs and getattr(step, "cu_q_prompt", None) is not None:
            # a mixed batch: its single tokens (they come first) go to the split-KV kernel,
            # which streams their keys at full rate, the prompt portions to the tiled one
            out = torch.empty_like(q)
            paged_attention_decode(q[:nd], k_cache, v_cache, block_table[:nd], step.kv_len[:nd],
                                   step.max_kv_len, window, scale, out=out[:nd], softcap=softcap)
            paged_attention_prefill(q[nd:], k_cache, v_cache, block_table[nd:],
                                    step.cu_q_prompt, step.q_pos0[nd:], window, scale,
                                    out=out[nd:], max_kv_len=step.max_kv_len, softcap=softcap)
            return out
        return paged_attention_prefill(q, k_cache, v_cache, block_table, step.cu_q, step.q_pos0,
                                       window, scale, max_kv_len=step.max_kv_len,
                                       softcap=softcap)
    return _paged_attention_softcap(q, k_cache, v_cache, block_table, step, window, scale, 0.0)


def paged_attention_decode_any(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                               block_table: torch.Tensor, kv_len: torch.Tensor, max_kv_len: int,
                               window: int, scale: float, softcap: float = 0.0,
                               splits: Optional[int] = None, keep_first: int = 0,
                               sink: bool = False):
    """Split-KV attention in fp32 arithmetic for a batch in which sequence s brings the one
    query q[s] at position kv_len[s] - 1: any head size up to 512, value heads of a size
    of their own, any element type.  Returns [S, heads, value size]."""
    _chk("q", q)
    _chk("k_cache", k_cache, q.dtype)
    _chk("v_cache", v_cache, q.dtype)
    _chk("block_table", block_table, torch.int32)
    _chk("kv_len", kv_len, torch.int32)
    S, heads, hd = q.shape
    P, kvh, page, chd = k_cache.shape
    vd = v_cache.shape[3]
    if chd != hd or v_cache.shape[:3] != k_cache.shape[:3]:
        raise KernelError("paged_attention_decode_any: cache geometry differs from the query's")
    if kv_len.numel() != S or block_table.shape[0] != S:
        raise KernelError("paged_attention_decode_any: one query per sequence is required")
    lib = _lib()
    if splits is None:
        splits = lib.ix_attn_decode_any_splits(S, heads, kvh, hd, vd, int(max_kv_len))
    out = torch.empty((S, heads, vd), dtype=q.dtype, device=q.device)
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.empty((S, heads, splits, vd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((S, heads, splits, 2), dtype=torch.float32, device=q.device)
    _check(lib.ix_paged_attention_decode_any(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), _ptr(kv_len), _ptr(part_o),
        _ptr(part_ml), _ptr(out), _dtype_code(q), S, heads, kvh, hd, vd, page,
        block_table.shape[1], window, ctypes.c_float(scale), ctypes.c_float(softcap), splits,
        int(keep_first), 1 if sink else 0, _stream()), "paged_attention_decode_any")
    _count(2 if splits > 1 else 1)
    return out


# From this many keys on a step of single tokens goes to the split-KV form of the
# fp32-arithmetic kernels; below it a block per (token, head) walks them as fast.
DECODE_ANY_MIN_KEYS = 128


def _paged_attention_softcap(q, k_cache, v_cache, block_table, step, window, scale, softcap,
                             keep_first=0, sink=False):
    """The fp32-arithmetic kernels (squashed scores or not)."""
    hd = q.shape[2]
    if (USE_EXACT_TC_ATTENTION and softcap == 0.0 and scale > 0 and q.dtype == torch.bfloat16
            and getattr(step, "all_decode", False) and getattr(step, "kv_len", None) is not None
            and step.num_tokens == step.num_seqs
            and _lib().ix_paged_attention_decode_exact_applies(hd, v_cache.shape[3])):
        return paged_attention_decode_exact(q, k_cache, v_cache, block_table, step.kv_len,
                                            step.max_kv_len, window, scale,
                                            keep_first=keep_first, sink=sink)
    if (getattr(step, "all_decode", False) and getattr(step, "kv_len", None) is not None
            and step.num_tokens == step.num_seqs and step.max_kv_len >= DECODE_ANY_MIN_KEYS
            and max(hd, v_cache.shape[3]) <= 512):
        return paged_attention_decode_any(q, k_cache, v_cache, block_table, step.kv_len,
                                          step.max_kv_len, window, scale, softcap,
                                          keep_first=keep_first, sink=sink)
    if (USE_EXACT_TC_ATTENTION and softcap == 0.0 and scale > 0 and q.dtype == torch.bfloat16
            and _lib().ix_paged_attention_prefill_exact_applies(hd, v_cache.shape[3])
            and getattr(step, "cu_q", None) is not None):
        nd = getattr(step, "num_decode_seqs", 0)
        if (0 < nd < step.num_seqs and getattr(step, "cu_q_prompt", None) is not None
                and getattr(step, "kv_len", None) is not None):
            # a mixed batch: its single tokens (they come first) go to the split-KV kernel,
            # the prompt portions to the tiled one
            single = paged_attention_decode_exact(
                q[:nd], k_cache, v_cache, block_table[:nd], step.kv_len[:nd], step.max_kv_len,
                window, scale, keep_first=keep_first, sink=sink)
            rest = paged_attention_prefill_exact(
                q[nd:], k_cache, v_cache, block_table[nd:], step.cu_q_prompt, step.q_pos0[nd:],
                window, scale, keep_first, sink)
            return torch.cat([single, rest], dim=0)
        return paged_attention_prefill_exact(q, k_cache, v_cache, block_table, step.cu_q,
                                             step.q_pos0, window, scale, keep_first, sink)
    if (step.num_tokens >= TILED_ATTENTION_MIN_QUERIES * step.num_seqs
            and _lib().ix_paged_attention_tiled_applies(hd)
            and _lib().ix_paged_attention_tiled_applies(v_cache.shape[3])
            and getattr(step, "cu_q", None) is not None):
        return paged_attention_tiled(q, k_cache, v_cache, block_table, step.cu_q, step.q_pos0,
                                     window, scale, softcap, keep_first, sink)
    return paged_attention_generic(q, k_cache, v_cache, block_table, step.seq_of_token,
                                   step.positions, window, scale, softcap, keep_first, sink)


USE_TCGEN05 = True           # prompt-sized grouped products go to the tcgen05 kernel
TCGEN05_MAX_EXPERTS = 1024   # its per-expert tile prefix lives in shared memory
# grouped: up to this many rows per expert on average stream the weights with the
# mma.sync kernel; beyond, the persistent tcgen05 kernel is faster (measured crossover at
# 60 experts: between 24 and 32 tokens of top-4 routing)
SMALL_M_ROWS_PER_GROUP = 2
SMALL_M_DENSE_ROWS = 16      # dense: up to this many rows stream the weights once


def gemm_small_m(x: torch.Tensor, w: torch.Tensor, rows: Optional[torch.Tensor],
                 offsets: Optional[torch.Tensor], dual: bool, num_out_rows: int,
                 out_dtype: Optional[torch.dtype] = None, rows_per_pass: int = 8,
                 active_groups: int = 0, offsets_settled: bool = False,
                 glu_clamp: Optional[Tuple[float, float, float]] = None):
    """Weight-streaming product for few rows per weight matrix (bf16 inputs).
    ``offsets_settled``: the kernel that wrote ``offsets`` is at least two launches back
    in this stream (so the launch may read it, and start on its weights, before waiting
    for its predecessor).  ``glu_clamp`` (dual only): (limit, slope, shift) of the clamped
    gated unit instead of silu(gate) * up."""
    _chk("x", x, torch.bfloat16)
    _chk("w", w, torch.bfloat16)
    _chk("rows", rows, torch.int32, optional=True)
    _chk("offsets", offsets, torch.int32, optional=True)
    E, w_rows, K = w.shape
    N = w_rows // 2 if dual else w_rows
    if x.shape[1] != K:
        raise KernelError(f"gemm_small_m: inner sizes differ ({x.shape[1]} vs {K})")
    if glu_clamp is not None and (not dual or glu_clamp[0] <= 0):
        raise KernelError("gemm_small_m: the clamped unit needs the dual form and a limit > 0")
    limit, alpha, shift = glu_clamp if glu_clamp is not None else (0.0, 1.0, 0.0)
    out_dtype = out_dtype or x.dtype
    out = torch.empty((num_out_rows, N), dtype=out_dtype, device=x.device)
    code = _lib().ix_gemm_small_m_act(
        _ptr(x), _ptr(rows), _ptr(offsets), _ptr(w), _ptr(out),
        F32 if out_dtype == torch.float32 else BF16, 1 if dual else 0,
        0 if offsets is not None else x.shape[0], N, K, E, rows_per_pass,
        active_groups or min(E, num_out_rows), 1 if offsets_settled else 0,
        ctypes.c_float(limit), ctypes.c_float(alpha), ctypes.c_float(shift), _stream())
    _check(code, "gemm_small_m")
    _count()
    return out


def gather_rows(x: torch.Tensor, rows: torch.Tensor):
    """out[i] = x[rows[i]] with 16-byte copies (row size must be a multiple of 16 bytes)."""
    _chk("x", x)
    _chk("rows", rows, torch.int32)
    n = rows.numel()
    out = torch.empty((n, x.shape[1]), dtype=x.dtype, device=x.device)
    _check(_lib().ix_gather_rows(_ptr(x), _ptr(rows), _ptr(out), n,
                                 x.shape[1] * x.element_size(), _stream()), "gather_rows")
    _count()
    return out


_TC_STATUS = {}


def _tc_status(device) -> torch.Tensor:
    key = torch.device(device).index or 0
    if key not in _TC_STATUS:
        _TC_STATUS[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _TC_STATUS[key]


_STATUS_ROLES = {
    1: "grouped_gemm_tc: the TMA producer", 2: "grouped_gemm_tc: the MMA issuer",
    3: "grouped_gemm_tc: the epilogue",
    11: "paged_attention_decode (TMA form): the copying warp",
    12: "paged_attention_decode (TMA form): a computing warp",
    21: "paged_attention_prefill (tcgen05 form): the copying warp",
    22: "paged_attention_prefill (tcgen05 form): the MMA issuer",
    23: "paged_attention_prefill (tcgen05 form): a softmax warp",
    24: "paged_attention_prefill (tcgen05 form): shared memory not on a 1024-byte mark;",
}


def check_async_errors():
    """Raise if a kernel gave up on one of its bounded mbarrier waits.  Reads a status
    word from the device, so it synchronises; call it where the host waits for
    results anyway."""
    for key, st in _TC_STATUS.items():
        code = int(st.item())
        if code:
            st.zero_()
            role = _STATUS_ROLES.get(code, "a kernel")
            raise KernelError(f"cuda:{key}: {role} waited past its limit (status {code}); "
                              "the output of that call is not valid")


def grouped_gemm_tc(a: torch.Tensor, offsets: torch.Tensor, w: torch.Tensor, dual: bool):
    """Grouped product on tcgen05 tensor cores: ``a`` [rows, K] already grouped by
    expert, ``w`` [E, N or 2N, K]; returns [rows, N] bf16."""
    _chk("a", a, torch.bfloat16)
    _chk("w", w, torch.bfloat16)
    _chk("offsets", offsets, torch.int32)
    E, w_rows, K = w.shape
    N = w_rows // 2 if dual else w_rows
    if a.shape[1] != K:
        raise KernelError(f"grouped_gemm_tc: inner sizes differ ({a.shape[1]} vs {K})")
    out = torch.empty((a.shape[0], N), dtype=torch.bfloat16, device=a.device)
    code = _lib().ix_grouped_gemm_tc(_ptr(a), _ptr(offsets), _ptr(w), _ptr(out),
                                     1 if dual else 0, a.shape[0], N, K, E,
                                     _ptr(_tc_status(a.device)), _stream())
    _check(code, "grouped_gemm_tc")
    _count()
    return out


# The persistent streaming kernel measured faster than the one-block-per-tile kernel only
# while a handful of experts have rows (one sequence decoding: 15 + 8 us against 17 + 12 us a
# layer at 60 experts of 1408 x 2048), equal at 8 assignments and slower beyond.
USE_STREAM_GROUPED = True
STREAM_GROUPED_MAX_ROWS = 4


def gemm_stream_grouped(x: torch.Tensor, w: torch.Tensor, rows: Optional[torch.Tensor],
                        offsets: torch.Tensor, dual: bool, num_out_rows: int,
                        rows_per_pass: int = 8):
    """Grouped weight-streaming product, persistent form (few rows per expert, bf16)."""
    _chk("x", x, torch.bfloat16)
    _chk("w", w, torch.bfloat16)
    _chk("rows", rows, torch.int32, optional=True)
    _chk("offsets", offsets, torch.int32)
    E, w_rows, K = w.shape
    N = w_rows // 2 if dual else w_rows
    if x.shape[1] != K:
        raise KernelError(f"gemm_stream_grouped: inner sizes differ ({x.shape[1]} vs {K})")
    if offsets.numel() != E + 1:
        raise KernelError("gemm_stream_grouped: offsets must have one entry per expert plus one")
    out = torch.empty((num_out_rows, N), dtype=torch.bfloat16, device=x.device)
    code = _lib().ix_gemm_stream_grouped(_ptr(x), _ptr(rows), _ptr(offsets), _ptr(w), _ptr(out),
                                         1 if dual else 0, N, K, E, rows_per_pass, _stream())
    _check(code, "gemm_stream_grouped")
    _count()
    return out


def _stream_grouped_applies(x: torch.Tensor, w: torch.Tensor, num_rows: int) -> bool:
    return (USE_STREAM_GROUPED and num_rows <= STREAM_GROUPED_MAX_ROWS
            and _streams_weights(x, w) and w.shape[-1] >= 256 and w.shape[0] <= 1024)


def _streams_weights(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the weight-streaming kernel takes these operands: bf16, K in 16-byte chunks."""
    return x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[-1] % 8 == 0


def grouped_gate_up_swiglu(x: torch.Tensor, rows: torch.Tensor, offsets: torch.Tensor,
                           w_gate_up: torch.Tensor):
    """act[r] = silu(x[rows[r]] . Wg[e]^T) * (x[rows[r]] . Wu[e]^T), e from offsets.

    ``w_gate_up``: [E, 2I, H], per expert the gate rows then the up rows."""
    A = rows.numel()
    per = A / w_gate_up.shape[0]
    if _stream_grouped_applies(x, w_gate_up, A):
        return gemm_stream_grouped(x, w_gate_up, rows, offsets, True, A,
                                   rows_per_pass=8 if per <= 2 else 16)
    if per <= SMALL_M_ROWS_PER_GROUP and _streams_weights(x, w_gate_up):
        return gemm_small_m(x, w_gate_up, rows, offsets, True, A,
                            rows_per_pass=8 if per <= 2 else 16)
    if USE_TCGEN05 and _streams_weights(x, w_gate_up) and w_gate_up.shape[0] <= TCGEN05_MAX_EXPERTS:
        return grouped_gemm_tc(gather_rows(x, rows), offsets, w_gate_up, True)
    return gemm_generic(x, w_gate_up, rows, offsets, dual=True, num_out_rows=A)


def grouped_down(act: torch.Tensor, offsets: torch.Tensor, w_down: torch.Tensor,
                 offsets_settled: bool = False):
    """y[r] = act[r] . Wd[e]^T with ``w_down`` [E, H, I].  ``offsets_settled``: see
    ``gemm_small_m`` (true when this follows ``grouped_gate_up_swiglu`` on the same
    offsets, as in a mixture layer)."""
    A = act.shape[0]
    per = A / w_down.shape[0]
    if _stream_grouped_applies(act, w_down, A):
        return gemm_stream_grouped(act, w_down, None, offsets, False, A,
                                   rows_per_pass=8 if per <= 2 else 16)
    if per <= SMALL_M_ROWS_PER_GROUP and _streams_weights(act, w_down):
        return gemm_small_m(act, w_down, None, offsets, False, A,
                            rows_per_pass=8 if per <= 2 else 16, offsets_settled=offsets_settled)
    if USE_TCGEN05 and _streams_weights(act, w_down) and w_down.shape[0] <= TCGEN05_MAX_EXPERTS:
        return grouped_gemm_tc(act, offsets, w_down, False)
    return gemm_generic(act, w_down, None, offsets, dual=False, num_out_rows=A)


def gate_up_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor):
    """Dense SwiGLU front half: silu(x . Wg^T) * (x . Wu^T) with ``w_gate_up`` [2I, H]."""
    _chk("x", x)
    _chk("w_gate_up", w_gate_up, x.dtype)
    M = x.shape[0]
    if M <= SMALL_M_DENSE_ROWS and _streams_weights(x, w_gate_up):
        return gemm_small_m(x, w_gate_up.unsqueeze(0), None, None, True, M, rows_per_pass=M)
    return silu_mul(linear(x, w_gate_up))


# ---------------------------------------------------------------------------
# Parts of decoders that normalise a sublayer's output, shift tokens, gate or clamp
# ---------------------------------------------------------------------------
def token_shift(resid: torch.Tensor, mix: torch.Tensor, state: torch.Tensor, step,
                out_dtype: torch.dtype):
    """out[t] = x[t] + (x[t-1] - x[t]) * mix in fp32, returned in ``out_dtype``.  The row
    before a sequence's first token of this step comes from ``state[state_slot[s]]``
    ([slots, width] fp32), which then receives the sequence's last row of this step."""
    _chk("resid", resid, torch.float32)
    _chk("mix", mix, torch.float32)
    _chk("state", state, torch.float32)
    T, W = resid.shape
    if mix.numel() != W or state.shape[1] != W:
        raise KernelError("token_shift: mix and state must have the residual's width")
    out = torch.empty((T, W), dtype=out_dtype, device=resid.device)
    _check(_lib().ix_token_shift(_ptr(resid), _ptr(mix), _ptr(state), _ptr(step.cu_q),
                                 _ptr(step.seq_of_token), _ptr(step.state_slot), _ptr(out),
                                 _dtype_code(out), T, W, _stream()), "token_shift")
    _count()
    return out


def group_norm_add(resid: torch.Tensor, delta: torch.Tensor, gain: torch.Tensor, groups: int,
                   eps: float, cast_dtype: Optional[torch.dtype] = None):
    """resid += grouped_rms_norm(delta) * gain, in place and in fp32: each row of ``delta``
    in ``groups`` equal consecutive parts, each part over its own root mean square.
    With ``cast_dtype`` the new residual is also returned in that element type."""
    _chk("resid", resid, torch.float32)
    _chk("delta", delta)
    _chk("gain", gain, torch.float32)
    T, W = resid.shape
    if delta.shape != resid.shape or gain.numel() != W:
        raise KernelError("group_norm_add: delta and gain must match the residual")
    if groups <= 0 or W % groups:
        raise KernelError(f"group_norm_add: width {W} does not split into {groups} equal parts")
    cast = (torch.empty((T, W), dtype=cast_dtype, device=resid.device)
            if cast_dtype is not None else None)
    _check(_lib().ix_group_norm_add(
        _ptr(resid), _ptr(delta), _dtype_code(delta), _ptr(gain), _ptr(cast),
        _dtype_code(cast) if cast is not None else _dtype_code(delta), T, W, groups,
        ctypes.c_float(eps), _stream()), "group_norm_add")
    _count()
    return cast


def group_norm_rows(resid: torch.Tensor, rows: Optional[torch.Tensor], gain: torch.Tensor,
                    groups: int, eps: float, out_dtype: torch.dtype):
    """grouped_rms_norm(resid[rows]) * gain in ``out_dtype`` (every row when ``rows`` is None)."""
    _chk("resid", resid, torch.float32)
    _chk("rows", rows, torch.int32, optional=True)
    _chk("gain", gain, torch.float32)
    T, W = resid.shape
    if gain.numel() != W or groups <= 0 or W % groups:
        raise KernelError(f"group_norm_rows: width {W}, gain {gain.numel()}, groups {groups}")
    R = T if rows is None else rows.numel()
    out = torch.empty((R, W), dtype=out_dtype, device=resid.device)
    _check(_lib().ix_group_norm_rows(_ptr(resid), _ptr(rows), _ptr(gain), _ptr(out),
                                     _dtype_code(out), R, W, groups, ctypes.c_float(eps),
                                     _stream()), "group_norm_rows")
    _count()
    return out


def glu_clamped(gu: torch.Tensor, limit: float, alpha: float, up_shift: float):
    """[T, 2I] (gate | up) -> min(g, L) * sigmoid(alpha * min(g, L)) * (clamp(u, -L, L) + up_shift)."""
    _chk("gu", gu)
    T, two_i = gu.shape
    if two_i % 2:
        raise KernelError("glu_clamped: width must be even (gate | up)")
    out = torch.empty((T, two_i // 2), dtype=gu.dtype, device=gu.device)
    _check(_lib().ix_glu_clamped(_ptr(gu), _ptr(out), _dtype_code(gu), T, two_i // 2,
                                 ctypes.c_float(limit), ctypes.c_float(alpha),
                                 ctypes.c_float(up_shift), _stream()), "glu_clamped")
    _count()
    return out


def gate_up_glu_clamped(x: torch.Tensor, w_gate_up: torch.Tensor, limit: float, alpha: float,
                        up_shift: float):
    """Front half of a clamped-GLU feed-forward: the fused gate|up product and the
    activation; one weight-streaming kernel for a few rows."""
    _chk("x", x)
    _chk("w_gate_up", w_gate_up, x.dtype)
    M = x.shape[0]
    if M <= SMALL_M_DENSE_ROWS and _streams_weights(x, w_gate_up) and limit > 0:
        return gemm_small_m(x, w_gate_up.unsqueeze(0), None, None, True, M, rows_per_pass=M,
                            glu_clamp=(limit, alpha, up_shift))
    return glu_clamped(linear(x, w_gate_up), limit, alpha, up_shift)


# From this many weights a matrix, a batched product of at most 16 rows a matrix streams the
# weights with this library's kernel (per-head products of a few ten thousand weights stay
# with the library, where they measured equal or faster).
BATCHED_STREAM_MIN_WEIGHTS = 1 << 20


def batched_linear(x: torch.Tensor, w: torch.Tensor):
    """out[b] = x[b] . w[b]^T for x [B, M, K] (any strides with unit inner stride) and
    w [B, N, K]: one library call batched over the leading dimension (per-head
    products).  float32 operands are multiplied in true 32-bit.  (For a few rows per
    matrix the grouped weight-streaming kernel, one group per matrix, was measured too:
    equal at 16 heads, slower at 8 and at 32 - a decode step of 0.85 against 0.74 ms at
    width 4096 -, so the library keeps these products at every size.)"""
    if not (x.is_cuda and w.is_cuda):
        raise KernelError("batched_linear: tensors must be on a CUDA device")
    if x.dtype != w.dtype or x.dim() != 3 or w.dim() != 3 or x.shape[0] != w.shape[0] \
            or x.shape[2] != w.shape[2]:
        raise KernelError(f"batched_linear: {tuple(x.shape)} {x.dtype} against "
                          f"{tuple(w.shape)} {w.dtype}")
    if x.dtype == torch.float32 and torch.backends.cuda.matmul.allow_tf32:
        raise KernelError("batched_linear: TF32 is switched on; 32-bit products must be exact")
    B, M, K = x.shape
    if (M <= SMALL_M_DENSE_ROWS and w.shape[1] * K >= BATCHED_STREAM_MIN_WEIGHTS
            and x.is_contiguous() and w.is_contiguous() and _streams_weights(x, w)):
        # a few rows against large matrices: each matrix is a group of the weight-streaming
        # kernel, its rows one pass (the library's batched product reads such weights at a
        # fraction of the memory rate)
        offsets = torch.arange(0, (B + 1) * M, M, dtype=torch.int32, device=x.device)
        out = gemm_small_m(x.view(B * M, K), w, None, offsets, False, B * M,
                           rows_per_pass=8 if M <= 8 else 16, active_groups=B)
        return out.view(B, M, w.shape[1])
    LIBRARY_CALLS[0] += 1
    return torch.bmm(x, w.transpose(1, 2))


def latent_prepare(proj: torch.Tensor, q_off: int, kv_off: int, positions: torch.Tensor,
                   freq: torch.Tensor, mag: float, gain: torch.Tensor, eps: float, heads: int,
                   dim: int, rot_dim: int, rot_dims: int, rank: int,
                   cache: Optional[torch.Tensor], slots: Optional[torch.Tensor]):
    """From the fused projection ``proj`` [T, *]: RMS-norm the latent (columns ``kv_off`` ..
    + rank), rotate the shared key part behind it and each head's rotated query part
    (head h's query is ``dim`` plain then ``rot_dim`` rotated columns from ``q_off`` on;
    interleaved pairs, the first ``rot_dims`` entries turn), write the record
    [latent | rotated key] into ``cache`` ([pages, 1, page, rank + rot_dim]) at ``slots``.
    Returns the rotated query parts [T, heads, rot_dim] and the plain ones, heads
    outermost, [heads, T, dim]."""
    _chk("proj", proj)
    _chk("positions", positions, torch.int32)
    _chk("freq", freq, torch.float32)
    _chk("gain", gain, torch.float32)
    _chk("cache", cache, proj.dtype, optional=True)
    _chk("slots", slots, torch.int32, optional=True)
    T, ld = proj.shape
    if q_off + heads * (dim + rot_dim) > ld or kv_off + rank + rot_dim > ld:
        raise KernelError("latent_prepare: the projection is narrower than its parts")
    if freq.numel() * 2 != rot_dims or gain.numel() != rank:
        raise KernelError("latent_prepare: one frequency per rotated pair, one gain per latent")
    if cache is not None and (cache.shape[1] != 1 or cache.shape[3] != rank + rot_dim):
        raise KernelError("latent_prepare: cache records must be [1, page, rank + rot_dim]")
    q_rot = torch.empty((T, heads, rot_dim), dtype=proj.dtype, device=proj.device)
    q_plain = torch.empty((heads, T, dim), dtype=proj.dtype, device=proj.device)
    _check(_lib().ix_latent_prepare(
        _ptr(proj), ctypes.c_longlong(ld), q_off, kv_off, _ptr(positions), _ptr(freq),
        ctypes.c_float(mag), _ptr(gain), ctypes.c_float(eps), _ptr(slots), _ptr(cache),
        _ptr(q_rot), _ptr(q_plain), _dtype_code(proj), T, heads, dim, rot_dim, rot_dims, rank,
        _stream()), "latent_prepare")
    _count()
    return q_rot, q_plain


# Latent attention forms: "mma" (mma.sync tensor cores; bf16, latent sizes 64 / 128 / 256 /
# 512, rotated part a multiple of 16) and "general" (CUDA cores in fp32; any sizes, either
# element type).  Which one runs depends on the model's sizes and element type only,
# never on the batch, so a position's result does not change with its neighbours.
USE_MMA_LATENT_ATTENTION = True


def check_latent_attention_limits(rank: int, rot_dim: int, where: str = ""):
    most = _lib().ix_latent_attention_max_rank()
    if rank > most:
        raise KernelError(f"{where}: latent size {rank} exceeds the largest the attention "
                          f"kernels take ({most})")
    if (rank + rot_dim) * 41 * 4 > 200 * 1024 and not _lib().ix_latent_attention_mma_applies(
            rank, rot_dim):
        raise KernelError(f"{where}: records of {rank} + {rot_dim} entries do not fit the "
                          "general attention kernel's shared memory")


def _mma_latent_applies(q_lat, q_rot) -> bool:
    return bool(q_lat.dtype == torch.bfloat16 and q_lat.is_cuda
                and _lib().ix_latent_attention_mma_applies(q_lat.shape[2], q_rot.shape[2]))


def latent_attention(q_lat: torch.Tensor, q_rot: torch.Tensor, cache: torch.Tensor,
                     block_table: torch.Tensor, step, window: int, scale: float,
                     kernel: Optional[str] = None):
    """Attention of this step's queries over cached latent records.

    ``q_lat`` [heads, T, rank] (the query with the key matrix folded in), ``q_rot``
    [T, heads, rot_dim], ``cache`` [pages, 1, page, rank + rot_dim].  Scores are
    (q_lat . latent + q_rot . key_rot) * scale over the keys a position sees (itself and
    the ``window`` - 1 before it; all earlier ones when ``window`` is 0); returns
    sum_j p_j latent_j as [heads, T, rank].  ``step`` carries ``seq_of_token``,
    ``positions``, ``cu_q``, ``q_pos0`` and the host list ``q_lens``.  ``kernel`` picks a
    form ("mma", "general"); None takes the tensor-core form where it applies."""
    _chk("q_lat", q_lat)
    _chk("q_rot", q_rot, q_lat.dtype)
    _chk("cache", cache, q_lat.dtype)
    _chk("block_table", block_table, torch.int32)
    H, T, rank = q_lat.shape
    dr = q_rot.shape[2]
    P, one, page, dk = cache.shape
    if one != 1 or dk != rank + dr or q_rot.shape[:2] != (T, H):
        raise KernelError("latent_attention: queries and cache records disagree")
    if kernel is None:
        kernel = "mma" if USE_MMA_LATENT_ATTENTION and _mma_latent_applies(q_lat, q_rot) \
            else "general"
    if kernel not in ("mma", "general"):
        raise KernelError(f"latent_attention: no kernel form {kernel!r}")
    out = torch.empty((H, T, rank), dtype=q_lat.dtype, device=q_lat.device)
    if kernel == "mma":
        if not _mma_latent_applies(q_lat, q_rot):
            raise KernelError("latent_attention: the tensor-core form takes bf16, a latent of "
                              f"64, 128, 256 or 512 and a rotated part in sixteens (got "
                              f"{q_lat.dtype}, {rank}, {dr})")
        lib = _lib()
        # blocks of 64 (token, head) rows; of 16 where every sequence brings one token and
        # the heads would leave most of 64 rows empty
        rows = 16 if (max(step.q_lens) == 1 and H % 64 and H % 64 <= 32) else 64
        tpt = lib.ix_latent_attention_mma_tokens_per_tile(H, rows)
        tiles = sum(-(-int(n) // tpt) for n in step.q_lens)
        S = len(step.q_lens)
        # few blocks over long runs of keys: the keys are cut into chunks, merged afterwards
        max_kv = int(getattr(step, "max_kv_len", 0) or block_table.shape[1] * page)
        span = min(window + tpt - 1, max_kv) if window > 0 else max_kv
        ct = ctypes.c_int(0)
        nchunks = lib.ix_latent_attention_mma_chunks(tiles * -(-H // rows), span, ctypes.byref(ct))
        part_o = part_ml = None
        if ct.value > 0:
            part_o = torch.empty((T, H, nchunks, rank), dtype=torch.float32, device=q_lat.device)
            part_ml = torch.empty((T, H, nchunks, 2), dtype=torch.float32, device=q_lat.device)
        _check(lib.ix_latent_attention_mma(
            _ptr(q_lat), ctypes.c_longlong(T * rank), ctypes.c_longlong(rank), _ptr(q_rot),
            _ptr(cache), _ptr(block_table), block_table.shape[1], _ptr(step.cu_q),
            _ptr(step.q_pos0), S, _ptr(out), ctypes.c_longlong(T * rank),
            ctypes.c_longlong(rank), T, H, rank, dr, page, window, ctypes.c_float(scale), tiles,
            rows, ct.value, nchunks, _ptr(part_o), _ptr(part_ml), _stream()), "latent_attention (mma)")
        if ct.value > 0:
            _count()
        _count()
        return out
    _check(_lib().ix_latent_attention(
        _ptr(q_lat), ctypes.c_longlong(T * rank), ctypes.c_longlong(rank), _ptr(q_rot),
        _ptr(cache), _ptr(block_table), block_table.shape[1], _ptr(step.seq_of_token),
        _ptr(step.positions), _ptr(out), ctypes.c_longlong(T * rank), ctypes.c_longlong(rank),
        _dtype_code(q_lat), T, H, rank, dr, page, window, ctypes.c_float(scale), _stream()),
        "latent_attention")
    _count()
    return out


def gate_heads(o: torch.Tensor, proj: torch.Tensor, gate_off: int):
    """out[t, h * D + j] = o[h, t, j] * sigmoid(proj[t, gate_off + h * D + j]) for
    o [heads, T, D]: the output gate, with the heads laid beside each other again."""
    _chk("o", o)
    _chk("proj", proj, o.dtype)
    H, T, D = o.shape
    if proj.shape[0] != T or gate_off + H * D > proj.shape[1]:
        raise KernelError("gate_heads: the gate columns do not fit the projection")
    out = torch.empty((T, H * D), dtype=o.dtype, device=o.device)
    gate = proj.view(-1)[gate_off:]
    _check(_lib().ix_gate_heads(_ptr(o), ctypes.c_void_p(gate.data_ptr()),
                                ctypes.c_longlong(proj.shape[1]), _ptr(out), _dtype_code(o), T, H,
                                D, _stream()), "gate_heads")
    _count()
    return out


# ---------------------------------------------------------------------------
# Parts of decoders with a parallel arrangement, recurrent mixers and tied keys/values
# ---------------------------------------------------------------------------
def embed_sinusoid(table: torch.Tensor, ids: torch.Tensor, positions: torch.Tensor,
                   freq: torch.Tensor, scale: float = 1.0):
    """out[t] = table[ids[t]] * scale + pos(positions[t]) in fp32; entry 2i of pos(p) is
    sin(p * freq[i]), entry 2i+1 cos(p * freq[i])."""
    _chk("table", table)
    _chk("ids", ids, torch.int32)
    _chk("positions", positions, torch.int32)
    _chk("freq", freq, torch.float32)
    V, W = table.shape
    T = ids.numel()
    if positions.numel() != T or freq.numel() != (W + 1) // 2:
        raise KernelError("embed_sinusoid: one position per token and one frequency per pair")
    out = torch.empty((T, W), dtype=torch.float32, device=table.device)
    _check(_lib().ix_embed_sinusoid(_ptr(table), _dtype_code(table), _ptr(ids), _ptr(positions),
                                    _ptr(freq), T, W, V, _ptr(out), ctypes.c_float(scale),
                                    _stream()), "embed_sinusoid")
    _count()
    return out


def add_rmsnorm_sum(resid: torch.Tensor, terms, vector: Optional[torch.Tensor], gains,
                    eps: float, out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None):
    """resid += sum(terms) + vector (kept when ``rows`` is None), then one normed view of the
    rows per gain: RMSNorm(resid) * gain.  ``terms``: up to three tensors shaped like
    ``resid``, each fp32 or bfloat16 (a mixture's output that is still unwritten is combined
    in the same pass when it has the output's element type, written out first otherwise);
    ``vector``: fp32 [width] added to every row, or None; ``gains``: one or two fp32 [width].
    With ``rows`` the listed rows are gathered and the residual is left as it was."""
    _chk("resid", resid, torch.float32)
    _chk("vector", vector, torch.float32, optional=True)
    _chk("rows", rows, torch.int32, optional=True)
    T, W = resid.shape
    # one term may be a mixture's output that was never written; the kernel combines it
    combine = None
    for t in terms:
        if isinstance(t, CombinePending) and combine is None and t.dtype == out_dtype \
                and t.shape == tuple(resid.shape):
            combine = t
    terms = [t.materialize() if hasattr(t, "materialize") else t for t in terms
             if t is not combine]
    while len(terms) > 3:                      # more than the kernel adds at once
        terms = [terms[0].to(torch.float32) + terms[1].to(torch.float32)] + terms[2:]
    for i, t in enumerate(terms):
        _chk(f"terms[{i}]", t)
        if t.shape != resid.shape:
            raise KernelError(f"add_rmsnorm_sum: term {i} is {tuple(t.shape)}, the residual "
                              f"{tuple(resid.shape)}")
    if not 1 <= len(gains) <= 2:
        raise KernelError("add_rmsnorm_sum: one or two gains")
    for g in gains:
        _chk("gain", g, torch.float32)
        if g.numel() != W:
            raise KernelError(f"add_rmsnorm_sum: gain has {g.numel()} entries, rows have {W}")
    if vector is not None and vector.numel() != W:
        raise KernelError("add_rmsnorm_sum: the vector must have the residual's width")
    R = T if rows is None else rows.numel()
    outs = [torch.empty((R, W), dtype=out_dtype, device=resid.device) for _ in gains]
    d = terms + [None] * (3 - len(terms))
    codes = [_dtype_code(t) if t is not None else 0 for t in d]
    _check(_lib().ix_add_rmsnorm_sum(
        _ptr(resid), _ptr(d[0]), codes[0], _ptr(d[1]), codes[1], _ptr(d[2]), codes[2],
        _ptr(vector), _ptr(rows), _ptr(gains[0]), _ptr(gains[1] if len(gains) > 1 else None),
        _ptr(outs[0]), _ptr(outs[1] if len(outs) > 1 else None), _dtype_code(outs[0]), R, W,
        ctypes.c_float(eps), 1 if rows is None else 0,
        _ptr(combine.y if combine else None), _ptr(combine.dest if combine else None),
        _ptr(combine.topk_w if combine else None), _ptr(combine.shared if combine else None),
        _ptr(combine.shared_logit if combine else None),
        combine.topk_w.shape[1] if combine else 0, _stream()), "add_rmsnorm_sum")
    _count()
    return tuple(outs)


def qk_norm_append(qk: torch.Tensor, q_gain: torch.Tensor, k_gain: torch.Tensor,
                   positions: torch.Tensor, heads: int, kv_heads: int, head_dim: int, eps: float,
                   temp_coef: float, temp_every: int, k_cache: Optional[torch.Tensor],
                   v_cache: Optional[torch.Tensor], slots: Optional[torch.Tensor]):
    """``qk`` [T, (heads + kv_heads) * head_dim] holds q then k.  Returns q [T, heads, hd],
    RMS-normed per head with ``q_gain`` and multiplied by 1 + temp_coef * ln(floor((p + 1)
    / temp_every) + 1) (``temp_every`` 0: by 1); writes k RMS-normed with ``k_gain`` into
    ``k_cache`` and k as it is into ``v_cache`` at ``slots`` when caches are given."""
    _chk("qk", qk)
    _chk("q_gain", q_gain, torch.float32)
    _chk("k_gain", k_gain, torch.float32)
    _chk("positions", positions, torch.int32)
    _chk("k_cache", k_cache, qk.dtype, optional=True)
    _chk("v_cache", v_cache, qk.dtype, optional=True)
    _chk("slots", slots, torch.int32, optional=True)
    T = qk.shape[0]
    if qk.shape[1] != (heads + kv_heads) * head_dim or q_gain.numel() != head_dim \
            or k_gain.numel() != head_dim:
        raise KernelError("qk_norm_append: sizes of the projection or the gains do not fit")
    page = 1
    if k_cache is not None:
        if v_cache is None or v_cache.shape != k_cache.shape or k_cache.shape[1] != kv_heads \
                or k_cache.shape[3] != head_dim or slots is None or slots.numel() != T:
            raise KernelError("qk_norm_append: cache geometry differs from the projection's")
        page = k_cache.shape[2]
    q = torch.empty((T, heads, head_dim), dtype=qk.dtype, device=qk.device)
    _check(_lib().ix_qk_norm_append(
        _ptr(qk), _dtype_code(qk), _ptr(q_gain), _ptr(k_gain), _ptr(positions), _ptr(q),
        _ptr(k_cache), _ptr(v_cache), _ptr(slots), T, heads, kv_heads, head_dim, page,
        ctypes.c_float(eps), ctypes.c_float(temp_coef), int(temp_every), _stream()),
        "qk_norm_append")
    _count()
    return q


def _row_view(name: str, t: torch.Tensor, width: int) -> int:
    """The row stride of a 2-d view with unit inner stride (a slice of columns of a
    projection's output, for instance)."""
    if not isinstance(t, torch.Tensor) or not t.is_cuda or t.dim() != 2 or t.shape[1] != width \
            or (width > 1 and t.stride(1) != 1):
        raise KernelError(f"{name}: expected a CUDA view [rows, {width}] with unit inner stride")
    return max(int(t.stride(0)), width)


def shift_mix(x: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, step):
    """out[m, t] = x[t] + (x[t-1] - x[t]) * mu[m], computed in fp32, in x's element type.
    The row before a sequence's first token of this step comes from
    ``state[state_slot[s]]`` ([slots, width] fp32), which then takes the sequence's last
    row of this step."""
    _chk("x", x)
    _chk("mu", mu, torch.float32)
    _chk("state", state, torch.float32)
    T, W = x.shape
    if mu.dim() != 2 or mu.shape[1] != W or state.shape[1] != W:
        raise KernelError("shift_mix: mu and state must have the input's width")
    out = torch.empty((mu.shape[0], T, W), dtype=x.dtype, device=x.device)
    _check(_lib().ix_shift_mix(_ptr(x), _dtype_code(x), _ptr(mu), _ptr(state), _ptr(step.cu_q),
                               _ptr(step.seq_of_token), _ptr(step.state_slot), _ptr(out), T, W,
                               mu.shape[0], _stream()), "shift_mix")
    _count()
    return out


_DECAY_FORMS = {"exp_exp_tanh": 0, "sigmoid_root": 1, "exp_rate_softplus": 2}


def lowrank_decay(x: torch.Tensor, w2t: torch.Tensor, b: Optional[torch.Tensor], mode: str,
                  tau: float = 1.0, head_log_rate: Optional[torch.Tensor] = None):
    """fp32 [T, C] decays from the inner activations ``x`` [T, R] of a low-rank product
    (a view with unit inner stride): z = act(x) . w2t + b with the outer matrix transposed,
    ``w2t`` fp32 [R, C], then "exp_exp_tanh": exp(-exp(z)) with act = tanh; "sigmoid_root":
    sigmoid(z)^(1/tau) with act the identity; "exp_rate_softplus": exp(-exp(A_h) *
    softplus(z)) with act the identity, where ``head_log_rate`` fp32 [heads] holds A and
    the C channels are split evenly over the heads."""
    _chk("w2t", w2t, torch.float32)
    _chk("head_log_rate", head_log_rate, torch.float32, optional=True)
    _chk("b", b, torch.float32, optional=True)
    if mode not in _DECAY_FORMS:
        raise KernelError(f"lowrank_decay: unknown form {mode!r}; known: {sorted(_DECAY_FORMS)}")
    R, C = w2t.shape
    ldx = _row_view("lowrank_decay: x", x, R)
    T = x.shape[0]
    per_head = 0
    if mode == "exp_rate_softplus":
        if head_log_rate is None or C % head_log_rate.numel():
            raise KernelError("lowrank_decay: this form needs a rate per head that splits "
                              "the channels evenly")
        per_head = C // head_log_rate.numel()
    out = torch.empty((T, C), dtype=torch.float32, device=x.device)
    _check(_lib().ix_lowrank_decay(_ptr(x), _dtype_code(x), ctypes.c_longlong(ldx), _ptr(w2t),
                                   _ptr(b), _ptr(out), T, C, R, _DECAY_FORMS[mode],
                                   ctypes.c_float(tau), _ptr(head_log_rate), per_head,
                                   _stream()), "lowrank_decay")
    _count()
    return out


def linear_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor,
                      bonus: Optional[torch.Tensor], state: torch.Tensor, step, heads: int,
                      dim: int, vdim: int, q_scale: float = 1.0, bonus_form: bool = False):
    """Walks every sequence's tokens of this step in order, per head with a state
    S [dim, vdim] in ``state[state_slot[s]]`` ([slots, heads, dim, vdim] fp32, updated):
    plain form S = diag(w_t) S + k_t v_t^T, o_t = S^T q_t; bonus form o_t = (S + diag(u)
    k_t v_t^T)^T q_t, then S = diag(w_t) S + k_t v_t^T.  q, k [T, heads * dim] and
    v [T, heads * vdim] are views with unit inner stride, ``decay`` fp32 [T, heads * dim],
    ``bonus`` fp32 [heads, dim].  Returns fp32 [T, heads, vdim]."""
    ldq = _row_view("linear_recurrence: q", q, heads * dim)
    ldk = _row_view("linear_recurrence: k", k, heads * dim)
    ldv = _row_view("linear_recurrence: v", v, heads * vdim)
    _chk("decay", decay, torch.float32)
    _chk("bonus", bonus, torch.float32, optional=True)
    _chk("state", state, torch.float32)
    T = q.shape[0]
    if not (q.dtype == k.dtype == v.dtype) or k.shape[0] != T or v.shape[0] != T \
            or decay.shape != (T, heads * dim) or tuple(state.shape[1:]) != (heads, dim, vdim):
        raise KernelError("linear_recurrence: q, k, v, decay and state do not fit together")
    if bonus_form and (bonus is None or bonus.numel() != heads * dim):
        raise KernelError("linear_recurrence: the bonus form needs u [heads, dim]")
    out = torch.empty((T, heads, vdim), dtype=torch.float32, device=q.device)
    seg_len, nseg = recurrence_segments(int(getattr(step, "max_q_len", 0) or T), step.num_seqs,
                                        heads, vdim)
    scratch = None
    if nseg > 1:
        scratch = torch.empty((_lib().ix_linear_recurrence_scratch_floats(
            step.num_seqs, heads, dim, vdim, nseg),), dtype=torch.float32, device=q.device)
    _check(_lib().ix_linear_recurrence(
        _ptr(q), ctypes.c_longlong(ldq), _ptr(k), ctypes.c_longlong(ldk), _ptr(v),
        ctypes.c_longlong(ldv), _dtype_code(q), _ptr(decay), _ptr(bonus), _ptr(state),
        _ptr(step.cu_q), _ptr(step.state_slot), _ptr(out), step.num_seqs, heads, dim, vdim,
        ctypes.c_float(q_scale), 1 if bonus_form else 0, seg_len, nseg, _ptr(scratch),
        _stream()), "linear_recurrence")
    _count(2 if nseg > 1 else 1)
    return out


# A sequence's tokens are walked in order by one block per (head, 32 value columns): a long
# prompt alone leaves most of the GPU idle.  From RECURRENCE_SEGMENT_MIN tokens on, the
# longest sequence of a step is cut into segments that are walked side by side (one pass
# for the segments' own states, one that joins them and writes the outputs), as many as
# fill the multiprocessors about once (RECURRENCE_BLOCKS), none shorter than 64 tokens.
RECURRENCE_SEGMENT_MIN = 128
RECURRENCE_BLOCKS = 1024
RECURRENCE_MAX_SEGMENTS = 64


def recurrence_segments(max_q_len: int, num_seqs: int, heads: int, vdim: int):
    """(tokens per segment, segments) for a step whose longest sequence brings
    ``max_q_len`` tokens; (0, 1): every sequence is walked from end to end."""
    if max_q_len < RECURRENCE_SEGMENT_MIN:
        return 0, 1
    base = max(1, num_seqs * heads * (-(-vdim // 32)))
    want = max(1, min(RECURRENCE_MAX_SEGMENTS, RECURRENCE_BLOCKS // base))
    seg_len = max(64, -(-(-(-max_q_len // want)) // 16) * 16)
    nseg = -(-max_q_len // seg_len)
    return (0, 1) if nseg <= 1 else (seg_len, nseg)


def check_recurrence_limits(dim: int, where: str = ""):
    most = _lib().ix_linear_recurrence_max_dim()
    if dim > most:
        raise KernelError(f"{where}: {dim} key entries per head exceed the recurrence "
                          f"kernel's {most}")


_GATE_FORMS = {"silu": 0, "sigmoid": 1}


def head_norm_gate(o: torch.Tensor, gain: torch.Tensor, gate: torch.Tensor, eps: float,
                   out_dtype: torch.dtype, gate_form: str = "silu"):
    """out[t, h] = o[t, h] / sqrt(mean(o[t, h]^2) + eps) * gain * act(gate[t, h]) (act:
    silu, or sigmoid with ``gate_form`` "sigmoid") for
    o fp32 [T, heads, vdim]; ``gain`` fp32 [vdim] (shared by the heads) or [heads * vdim];
    ``gate`` a view [T, heads * vdim] with unit inner stride in ``out_dtype``."""
    _chk("o", o, torch.float32)
    _chk("gain", gain, torch.float32)
    T, H, V = o.shape
    ldg = _row_view("head_norm_gate: gate", gate, H * V)
    if gain.numel() not in (V, H * V) or gate.dtype != out_dtype or gate.shape[0] != T:
        raise KernelError("head_norm_gate: gain or gate do not fit the heads")
    out = torch.empty((T, H * V), dtype=out_dtype, device=o.device)
    _check(_lib().ix_head_norm_gate(
        _ptr(o), _ptr(gain), 1 if (gain.numel() == H * V and H > 1) else 0, _ptr(gate),
        _dtype_code(gate), ctypes.c_longlong(ldg), _ptr(out), _dtype_code(out), T, H, V,
        ctypes.c_float(eps), _GATE_FORMS[gate_form], _stream()), "head_norm_gate")
    _count()
    return out


# ---------------------------------------------------------------------------
# Faces of csrc/delta_parts.cu
def add_scaled_norm(resid: torch.Tensor, delta, delta_scale: float,
                    vector: Optional[torch.Tensor], gain: torch.Tensor, eps: float,
                    out_dtype: torch.dtype, center: bool = True,
                    rows: Optional[torch.Tensor] = None):
    """resid += delta_scale * delta + vector (kept when ``rows`` is None), then the norm of
    the rows times ``gain``: with ``center`` (x - mean) / sqrt(mean((x - mean)^2) + eps),
    else x / sqrt(mean(x^2) + eps).  ``delta`` [T, H] fp32 or bfloat16 (or not yet written:
    anything with ``materialize``), ``vector`` fp32 [H]; either may be None.  With ``rows``
    the listed rows are gathered, normalised and returned without writing the residual."""
    if hasattr(delta, "materialize"):
        delta = delta.materialize()
    _chk("resid", resid, torch.float32)
    _chk("gain", gain, torch.float32)
    _chk("delta", delta, optional=True)
    _chk("vector", vector, torch.float32, optional=True)
    _chk("rows", rows, torch.int32, optional=True)
    T, H = resid.shape
    if gain.numel() != H or (vector is not None and vector.numel() != H):
        raise KernelError("add_scaled_norm: gain or vector do not fit the rows")
    if delta is not None and delta.shape != resid.shape:
        raise KernelError("add_scaled_norm: delta must have the residual's shape")
    R = T if rows is None else rows.numel()
    out = torch.empty((R, H), dtype=out_dtype, device=resid.device)
    _check(_lib().ix_add_scaled_norm(
        _ptr(resid), _ptr(delta), _dtype_code(delta) if delta is not None else F32,
        ctypes.c_float(delta_scale), _ptr(vector), _ptr(gain), _ptr(rows), _ptr(out),
        _dtype_code(out), R, H, ctypes.c_float(eps), 1 if center else 0,
        1 if rows is None and (delta is not None or vector is not None) else 0, _stream()),
        "add_scaled_norm")
    _count()
    return out


def stream_concat(resid: torch.Tensor, delta, delta_scale: float,
                  vector: Optional[torch.Tensor], first: torch.Tensor, out_dtype: torch.dtype):
    """[T, 2 H] in ``out_dtype``: row t is [resid[t] + delta_scale * delta[t] + vector ;
    first[t]] (``resid`` and ``first`` fp32 [T, H]; ``resid`` is not written)."""
    if hasattr(delta, "materialize"):
        delta = delta.materialize()
    _chk("resid", resid, torch.float32)
    _chk("first", first, torch.float32)
    _chk("delta", delta, optional=True)
    _chk("vector", vector, torch.float32, optional=True)
    T, H = resid.shape
    if first.shape != resid.shape or (delta is not None and delta.shape != resid.shape):
        raise KernelError("stream_concat: the tensors must have the residual's shape")
    out = torch.empty((T, 2 * H), dtype=out_dtype, device=resid.device)
    _check(_lib().ix_stream_concat(
        _ptr(resid), _ptr(delta), _dtype_code(delta) if delta is not None else F32,
        ctypes.c_float(delta_scale), _ptr(vector), _ptr(first), _ptr(out), _dtype_code(out), T, H,
        _stream()), "stream_concat")
    _count()
    return out


def causal_conv(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor],
                state: torch.Tensor, step, silu: bool = True):
    """Causal convolution over time per channel with the activation: x [T, C] (a view with
    unit inner stride), ``w`` fp32 [C, taps] whose last column multiplies the current
    token, ``bias`` fp32 [C] or None, ``state`` fp32 [slots, taps - 1, C]: a request's last
    taps - 1 inputs, read for the tokens before this step's first and moved on (None with
    one tap, which keeps nothing).  Returns
    [T, C] in x's element type."""
    _chk("w", w, torch.float32)
    _chk("bias", bias, torch.float32, optional=True)
    C, taps = w.shape
    _chk("state", state, torch.float32, optional=taps == 1)
    ldx = _row_view("causal_conv: x", x, C)
    T = x.shape[0]
    if (state is not None and tuple(state.shape[1:]) != (taps - 1, C)) or \
            (bias is not None and bias.numel() != C):
        raise KernelError("causal_conv: state or bias do not fit the channels and taps")
    out = torch.empty((T, C), dtype=x.dtype, device=x.device)
    _check(_lib().ix_causal_conv(
        _ptr(x), _dtype_code(x), ctypes.c_longlong(ldx), _ptr(w), _ptr(bias), _ptr(state),
        _ptr(step.cu_q), _ptr(step.seq_of_token), _ptr(step.state_slot), _ptr(out), T,
        step.num_seqs, C, taps, 1 if silu else 0, _stream()), "causal_conv")
    _count(2 if taps > 1 else 1)
    return out


def ssd_recurrence(xbc: torch.Tensor, dt_raw: torch.Tensor, dt_bias: torch.Tensor,
                   a_log: torch.Tensor, d_skip: torch.Tensor, state: torch.Tensor, step,
                   heads: int, vdim: int, nstate: int, groups: int):
    """State-space recurrence with a scalar decay per head.  ``xbc`` [T, heads * vdim +
    2 groups * nstate] holds x | B | C; ``dt_raw`` [T, heads] (a view) the step sizes
    before their bias and softplus; ``state`` fp32 [slots, heads, nstate, vdim], updated.
    Per head: dt = softplus(dt_raw + dt_bias), S = exp(-exp(a_log) dt) S + dt B x^T,
    y = S^T C + d_skip x.  Returns fp32 [T, heads * vdim]."""
    for name, t in (("dt_bias", dt_bias), ("a_log", a_log), ("d_skip", d_skip),
                    ("state", state)):
        _chk(name, t, torch.float32)
    width = heads * vdim + 2 * groups * nstate
    ld = _row_view("ssd_recurrence: xbc", xbc, width)
    ld_dt = _row_view("ssd_recurrence: dt", dt_raw, heads)
    T = xbc.shape[0]
    if dt_raw.dtype != xbc.dtype or dt_raw.shape[0] != T or \
            tuple(state.shape[1:]) != (heads, nstate, vdim) or \
            not (dt_bias.numel() == a_log.numel() == d_skip.numel() == heads):
        raise KernelError("ssd_recurrence: inputs and state do not fit together")
    out = torch.empty((T, heads * vdim), dtype=torch.float32, device=xbc.device)
    seg_len, nseg = recurrence_segments(int(getattr(step, "max_q_len", 0) or T), step.num_seqs,
                                        heads, vdim)
    scratch = None
    if nseg > 1:
        scratch = torch.empty((_lib().ix_ssd_recurrence_scratch_floats(
            step.num_seqs, heads, nstate, vdim, nseg),), dtype=torch.float32, device=xbc.device)
    _check(_lib().ix_ssd_recurrence(
        _ptr(xbc), ctypes.c_longlong(ld), _ptr(dt_raw), ctypes.c_longlong(ld_dt),
        _dtype_code(xbc), _ptr(dt_bias), _ptr(a_log), _ptr(d_skip), _ptr(state), _ptr(step.cu_q),
        _ptr(step.state_slot), _ptr(out), step.num_seqs, heads, vdim, nstate, groups, seg_len,
        nseg, _ptr(scratch), _stream()), "ssd_recurrence")
    _count(2 if nseg > 1 else 1)
    return out


def delta_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, beta_raw: torch.Tensor,
                     decay: torch.Tensor, state: torch.Tensor, step, heads: int, kv_heads: int,
                     dim: int, vdim: int, unit_eps: float, q_scale: float):
    """Gated delta rule.  q, k [T, kv_heads * dim], v [T, heads * vdim], ``beta_raw``
    [T, heads] are views with unit inner stride; ``decay`` fp32 [T, heads * dim]; ``state``
    fp32 [slots, heads, dim, vdim], updated.  q and k become unit vectors per head
    (x / sqrt(sum x^2 + unit_eps)), q also times ``q_scale``; beta = sigmoid(beta_raw).
    Per head: S = diag(g) S; u = beta (v - S^T k); S += k u^T; o = S^T q.  Returns fp32
    [T, heads, vdim]."""
    ldq = _row_view("delta_recurrence: q", q, kv_heads * dim)
    ldk = _row_view("delta_recurrence: k", k, kv_heads * dim)
    ldv = _row_view("delta_recurrence: v", v, heads * vdim)
    ldb = _row_view("delta_recurrence: beta", beta_raw, heads)
    _chk("decay", decay, torch.float32)
    _chk("state", state, torch.float32)
    T = q.shape[0]
    if not (q.dtype == k.dtype == v.dtype == beta_raw.dtype) or \
            decay.shape != (T, heads * dim) or tuple(state.shape[1:]) != (heads, dim, vdim):
        raise KernelError("delta_recurrence: inputs and state do not fit together")
    out = torch.empty((T, heads, vdim), dtype=torch.float32, device=q.device)
    # the kernel's side knows how many of its blocks the device holds at once
    seg = ctypes.c_int(0)
    nseg = _lib().ix_delta_recurrence_segments(
        _dtype_code(q), step.num_seqs, heads, dim, vdim,
        int(getattr(step, "max_q_len", 0) or T), RECURRENCE_SEGMENT_MIN, RECURRENCE_MAX_SEGMENTS,
        ctypes.byref(seg))
    if nseg < 1:
        _check(nseg, "delta_recurrence_segments")
    seg_len = seg.value
    scratch = None
    if nseg > 1:
        scratch = torch.empty((_lib().ix_delta_recurrence_scratch_floats(
            step.num_seqs, heads, dim, vdim, nseg),), dtype=torch.float32, device=q.device)
    _check(_lib().ix_delta_recurrence(
        _ptr(q), ctypes.c_longlong(ldq), _ptr(k), ctypes.c_longlong(ldk), _ptr(v),
        ctypes.c_longlong(ldv), _ptr(beta_raw), ctypes.c_longlong(ldb), _dtype_code(q),
        _ptr(decay), _ptr(state), _ptr(step.cu_q), _ptr(step.state_slot), _ptr(out),
        step.num_seqs, heads, kv_heads, dim, vdim, ctypes.c_float(unit_eps),
        ctypes.c_float(q_scale), seg_len, nseg, _ptr(scratch), _stream()), "delta_recurrence")
    _count(2 if nseg > 1 else 1)
    return out


def gated_group_norm(y: torch.Tensor, z: torch.Tensor, gain: torch.Tensor, groups: int,
                     eps: float):
    """groupnorm(y * silu(z)) * gain: y fp32 [T, W], z [T, W] a view in the run's element
    type; the row is RMS-normed in ``groups`` equal parts.  Returns [T, W] in z's type."""
    _chk("y", y, torch.float32)
    _chk("gain", gain, torch.float32)
    T, W = y.shape
    ldz = _row_view("gated_group_norm: z", z, W)
    if gain.numel() != W or z.shape[0] != T or groups <= 0 or W % groups:
        raise KernelError("gated_group_norm: gain, gate or groups do not fit the rows")
    out = torch.empty((T, W), dtype=z.dtype, device=y.device)
    _check(_lib().ix_gated_group_norm(_ptr(y), _ptr(z), _dtype_code(z), ctypes.c_longlong(ldz),
                                      _ptr(gain), _ptr(out), T, W, groups, ctypes.c_float(eps),
                                      _stream()), "gated_group_norm")
    _count()
    return out


def normed_pair_mean(left: torch.Tensor, right: torch.Tensor, gain_left: torch.Tensor,
                     gain_right: torch.Tensor, eps: float):
    """fp32 [T, W]: (left / rms(left) * gain_left + right / rms(right) * gain_right) / 2."""
    _chk("left", left)
    _chk("right", right, left.dtype)
    _chk("gain_left", gain_left, torch.float32)
    _chk("gain_right", gain_right, torch.float32)
    T, W = left.shape
    if right.shape != left.shape or gain_left.numel() != W or gain_right.numel() != W:
        raise KernelError("normed_pair_mean: shapes differ")
    out = torch.empty((T, W), dtype=torch.float32, device=left.device)
    _check(_lib().ix_normed_pair_mean(_ptr(left), _ptr(right), _dtype_code(left), _ptr(gain_left),
                                      _ptr(gain_right), _ptr(out), T, W, ctypes.c_float(eps),
                                      _stream()), "normed_pair_mean")
    _count()
    return out


def relu_squared(x: torch.Tensor):
    """max(x, 0)^2 in x's element type."""
    _chk("x", x)
    out = torch.empty_like(x)
    _check(_lib().ix_relu_squared(_ptr(x), _ptr(out), _dtype_code(x),
                                  ctypes.c_longlong(x.numel()), _stream()), "relu_squared")
    _count()
    return out


def table_route(token_ids: torch.Tensor, table: torch.Tensor, num_experts: int):
    """(weights fp32 [T, top], experts int32 [T, top]): row ``token id`` of ``table``
    int32 [vocab, top]; every weight is 1 / top."""
    _chk("token_ids", token_ids, torch.int32)
    _chk("table", table, torch.int32)
    T = token_ids.numel()
    vocab, top = table.shape
    idx = torch.empty((T, top), dtype=torch.int32, device=table.device)
    wts = torch.empty((T, top), dtype=torch.float32, device=table.device)
    _check(_lib().ix_table_route(_ptr(token_ids), _ptr(table), _ptr(idx), _ptr(wts), T, top,
                                 vocab, num_experts, _stream()), "table_route")
    _count()
    return wts, idx


def scale_rows(x: torch.Tensor, scale: float):
    """x *= scale in place (fp32)."""
    _chk("x", x, torch.float32)
    _check(_lib().ix_scale_rows(_ptr(x), ctypes.c_float(scale), ctypes.c_longlong(x.numel()),
                                _stream()), "scale_rows")
    _count()
    return x


def check_delta_limits(dim: int, taps: int, where: str = ""):
    most = _lib().ix_delta_recurrence_max_dim()
    if dim > most:
        raise KernelError(f"{where}: {dim} state entries per column exceed the recurrence "
                          f"kernels' {most}")
    if not 1 <= taps <= 16:
        raise KernelError(f"{where}: a convolution of {taps} taps is not one the kernel takes "
                          "(1 to 16)")


def embed_pair_norm(table: torch.Tensor, pair_table: torch.Tensor, gain: torch.Tensor, step,
                    prev_state: torch.Tensor, buckets: int, mul_prev: int, mul_cur: int,
                    eps: float):
    """fp32 [T, H]: rmsnorm(table[token] + pair_table[row]) * gain with row = (previous *
    mul_prev + token * mul_cur) mod buckets, row ``buckets`` at position 0.  The previous
    token of a sequence's first token in this step comes from ``prev_state`` (int32
    [slots, 1]), which then takes the sequence's last token of the step."""
    _chk("table", table)
    _chk("pair_table", pair_table, table.dtype)
    _chk("gain", gain, torch.float32)
    _chk("prev_state", prev_state, torch.int32)
    V, H = table.shape
    if pair_table.shape != (buckets + 1, H) or gain.numel() != H:
        raise KernelError("embed_pair_norm: the pair table must be [buckets + 1, width] and "
                          "the gain [width]")
    T = step.token_ids.numel()
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    _check(_lib().ix_embed_pair_norm(
        _ptr(table), _ptr(pair_table), _dtype_code(table), _ptr(gain), _ptr(step.token_ids),
        _ptr(step.positions), _ptr(step.seq_of_token), _ptr(step.cu_q), _ptr(step.state_slot),
        _ptr(prev_state), _ptr(out), T, H, ctypes.c_longlong(buckets),
        ctypes.c_longlong(mul_prev), ctypes.c_longlong(mul_cur), ctypes.c_float(eps),
        _stream()), "embed_pair_norm")
    _count()
    return out


def attention_prepare(qkv: torch.Tensor, positions: torch.Tensor, freq: Optional[torch.Tensor],
                      magnitude: float, rotary_dim: int, interleaved: bool, heads: int,
                      kv_heads: int, head_dim: int, value_dim: int,
                      q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor], eps: float,
                      head_unit: bool, earlier: Optional[torch.Tensor],
                      lam: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                      v_cache: Optional[torch.Tensor], slots: Optional[torch.Tensor],
                      want_dense_kv: bool = False):
    """Prepares a step's q, k and v rows (``qkv`` [T, q | k | v], a view with unit inner
    stride) for attention, per token and in fp32: with gains, the RMS norm of the whole q
    row and of the whole k row; the rotation of the first ``rotary_dim`` entries of every
    q and k head by position * ``freq`` (pairs are neighbours when ``interleaved``, else
    half a rotation apart; cos and sin times ``magnitude``); with ``head_unit`` every q
    and k head divided by its root mean square; with ``earlier`` ([T, kv_heads *
    value_dim], a view) the values become (1 - lam) v + lam earlier.  Returns q [T, heads,
    head_dim]; writes k and v into the pages at ``slots`` (and returns them densely when
    asked)."""
    _chk("positions", positions, torch.int32)
    _chk("freq", freq, torch.float32, optional=True)
    _chk("q_gain", q_gain, torch.float32, optional=True)
    _chk("k_gain", k_gain, torch.float32, optional=True)
    _chk("lam", lam, torch.float32, optional=True)
    _chk("slots", slots, torch.int32, optional=True)
    dq, dk, dv = heads * head_dim, kv_heads * head_dim, kv_heads * value_dim
    ld = _row_view("attention_prepare: qkv", qkv, dq + dk + dv)
    T = qkv.shape[0]
    ld_e = 0
    if earlier is not None:
        if earlier.dtype != qkv.dtype or earlier.shape[0] != T or lam is None:
            raise KernelError("attention_prepare: the earlier values must match the rows, and "
                              "need their weight")
        ld_e = _row_view("attention_prepare: earlier", earlier, dv)
    if rotary_dim and (freq is None or freq.numel() != rotary_dim // 2):
        raise KernelError("attention_prepare: freq must have rotary_dim / 2 entries")
    if (q_gain is None) != (k_gain is None) or (
            q_gain is not None and (q_gain.numel() != dq or k_gain.numel() != dk)):
        raise KernelError("attention_prepare: one gain per q entry and per k entry")
    page_size = 1
    if k_cache is not None:
        _chk("k_cache", k_cache, qkv.dtype)
        _chk("v_cache", v_cache, qkv.dtype)
        if slots is None or slots.numel() != T:
            raise KernelError("attention_prepare: a cache needs one slot per token")
        P, ckv, page_size, chd = k_cache.shape
        if ckv != kv_heads or chd != head_dim or \
                tuple(v_cache.shape) != (P, ckv, page_size, value_dim):
            raise KernelError("attention_prepare: cache geometry does not match the heads")
    q = torch.empty((T, heads, head_dim), dtype=qkv.dtype, device=qkv.device)
    k = v = None
    if want_dense_kv:
        k = torch.empty((T, kv_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
        v = torch.empty((T, kv_heads, value_dim), dtype=qkv.dtype, device=qkv.device)
    _check(_lib().ix_attention_prepare(
        _ptr(qkv), ctypes.c_longlong(ld), _dtype_code(qkv), _ptr(positions), _ptr(freq),
        ctypes.c_float(magnitude), int(rotary_dim), 1 if interleaved else 0, heads, kv_heads,
        head_dim, value_dim, _ptr(q_gain), _ptr(k_gain), ctypes.c_float(eps),
        1 if head_unit else 0, _ptr(earlier), ctypes.c_longlong(ld_e), _ptr(lam), _ptr(slots),
        _ptr(q), _ptr(k_cache), _ptr(v_cache), page_size, _ptr(k), _ptr(v), T, _stream()),
        "attention_prepare")
    _count()
    return (q, k, v) if want_dense_kv else q


def glu_bias_act(gu: torch.Tensor, bias: Optional[torch.Tensor], activation: str = "gelu_tanh"):
    """act(g + b_g) * (u + b_u) for rows laid out g | u (``bias`` fp32 [2 I] laid out the
    same way, or None); ``activation`` "gelu_tanh" or "silu"."""
    _chk("gu", gu)
    _chk("bias", bias, torch.float32, optional=True)
    if activation not in ("gelu_tanh", "silu"):
        raise KernelError(f"glu_bias_act: no activation {activation!r}")
    T, two_i = gu.shape
    if two_i % 2 or (bias is not None and bias.numel() != two_i):
        raise KernelError("glu_bias_act: rows are gate | up, with one bias entry each")
    out = torch.empty((T, two_i // 2), dtype=gu.dtype, device=gu.device)
    _check(_lib().ix_glu_bias_act(_ptr(gu), _ptr(bias), _ptr(out), _dtype_code(gu), T,
                                  two_i // 2, 1 if activation == "silu" else 0, _stream()),
           "glu_bias_act")
    _count()
    return out


def identity_rows(x: torch.Tensor, rows: torch.Tensor, offsets: torch.Tensor,
                  first_identity: int, y: torch.Tensor):
    """y[r] = x[rows[r]] for the grouped rows of the router's outputs from
    ``first_identity`` on (experts that return their input); ``offsets`` has one entry per
    router output plus one."""
    _chk("x", x)
    _chk("y", y, x.dtype)
    _chk("rows", rows, torch.int32)
    _chk("offsets", offsets, torch.int32)
    if y.shape[1] != x.shape[1] or y.shape[0] != rows.numel():
        raise KernelError("identity_rows: y must hold one row of x's width per grouped row")
    _check(_lib().ix_identity_rows(_ptr(x), _ptr(rows), _ptr(offsets), int(first_identity),
                                   offsets.numel() - 1, _ptr(y), _dtype_code(x), rows.numel(),
                                   x.shape[1], _stream()), "identity_rows")
    _count()
    return y
