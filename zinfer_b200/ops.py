"""Python face of the kernel library: one function per kernel entry point.

The library is built on first use (see ``csrc/build.py``) and loaded with ctypes.
Every function takes CUDA tensors, checks what the kernel assumes, launches on the
current torch stream and raises :class:`KernelError` with the kernel's own message
if it refuses.  There is no fallback of any kind: without the library, or with
tensors that are not on a CUDA device, these functions fail.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import profiling as _prof
from .csrc import build as _build


class KernelError(RuntimeError):
    pass


_LIB = None
F32, BF16 = 0, 1


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        path = _build.library_path()
        try:
            _LIB = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load the kernel library {path}: {e}") from None
        _LIB.zi_last_error.restype = ctypes.c_char_p
        _LIB.zi_gemm_tcgen05_plan.restype = ctypes.c_longlong
        _LIB.zi_attention_decode_workspace_floats.restype = ctypes.c_longlong
    return _LIB


def kernel_status() -> int:
    """Reads and clears the status words of the tcgen05 kernels (synchronises).
    0: every bounded wait inside them completed; else the code of the wait that ran out."""
    return int(lib().zi_gemm_tcgen05_status())   # one word for the products and the tcgen05 attention


def require_kernel_status_ok(where: str) -> None:
    """Raises if a bounded wait inside a tensor-core kernel ran out since the last check (its
    results are then not to be trusted).  Synchronises; the engine calls it where it waits for
    the device anyway, and every so many steps."""
    code = kernel_status()
    if code != 0:
        raise KernelError(f"{where}: a wait inside a tensor-core kernel ran out (code {code}); its results are invalid")


def selftest_wait_runs_out(code: int = 77, tries: int = 4096) -> None:
    """Launches one CTA that waits ``tries`` times on a barrier nobody arrives at, so that the wait
    runs out and the kernel records ``code`` in the status word, the way a stuck product would.
    Returns normally (nothing faults or hangs); :func:`require_kernel_status_ok` then raises."""
    _check(lib().zi_selftest_wait_runs_out(code, tries, _stream()), "selftest_wait_runs_out")


def gemm_pair_kernel(on: bool) -> bool:
    """Switches the matrix product's kernel for CTA pairs (tcgen05 ``cta_group::2``: two SMs on one
    tile of 256 tokens x 256 weight rows, each loading half of the weight rows) on or off for
    products of 256 tokens and more; returns the setting before.  Off unless
    ``ZINFER_B200_GEMM_PAIR=1``: measured equal to the single-CTA kernel inside a prefill step,
    where both run at the pace the power limit allows."""
    return bool(lib().zi_gemm_tcgen05_pair_enable(1 if on else 0))


def library_file() -> str:
    return _build.library_path()


def _tag(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _ptr(t: Optional[torch.Tensor]):
    if t is None:
        return ctypes.c_void_p(0)
    if not t.is_cuda:
        raise KernelError("kernels take CUDA tensors; there is no CPU path")
    return ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


LAUNCHES = 0   # kernel launches issued through this module (graph replays are counted by their owner)


def _check(code: int, what: str) -> None:
    global LAUNCHES
    LAUNCHES += 1
    if code != 0:
        msg = lib().zi_last_error().decode("utf-8", "replace")
        raise KernelError(f"{what}: {msg} (code {code})")


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _nb(*tensors) -> int:
    """Bytes of the given tensors (None counts nothing)."""
    return sum(t.numel() * t.element_size() for t in tensors if t is not None)


def _i32(t: torch.Tensor, name: str) -> torch.Tensor:
    _need(t.dtype == torch.int32 and t.is_contiguous(), f"{name} must be a contiguous int32 tensor")
    return t


class Partials:
    """A split-K matrix product whose partial sums have not been added yet:
    ``data`` [splits, M, N] float32.  The consumers below (residual add + norm, SwiGLU,
    q/k norm + rotary) add the splits themselves, in order, which saves a kernel and a
    round trip through memory; ``sum(dtype)`` adds them for any other consumer."""

    def __init__(self, data: torch.Tensor):
        self.data = data

    @property
    def shape(self):
        return self.data.shape[1:]

    @property
    def splits(self) -> int:
        return self.data.shape[0]

    def sum(self, dtype: torch.dtype) -> torch.Tensor:
        out = torch.empty(tuple(self.shape), dtype=dtype, device=self.data.device)
        S, M, N = self.data.shape
        h = torch.zeros((M, N), dtype=torch.float32, device=self.data.device)
        _check(lib().zi_residual_add_partials(_ptr(h), _ptr(self.data), S, ctypes.c_longlong(M * N),
                                              ctypes.c_longlong(M * N), _stream()), "partials.sum")
        return h if dtype == torch.float32 else h.to(dtype)


# ------------------------------------------------------------------ elementwise
def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rows ``ids`` of ``table`` [V, H] as the 32-bit residual stream [T, H]."""
    V, H = table.shape
    T = ids.shape[0]
    _need(table.is_contiguous(), "embedding table must be contiguous")
    _i32(ids, "ids")
    if out is None:
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    with _prof.region("embed_gather", lambda: T * H * table.element_size() + _nb(out, ids)):
        _check(lib().zi_embed_gather(_ptr(out), _ptr(table), _tag(table), _ptr(ids), T, H, V, _stream()), "embed_gather")
    return out


def patch_tokens(ids: torch.Tensor, prev: torch.Tensor, dst: torch.Tensor, src: torch.Tensor) -> None:
    """``ids[dst[i]] = prev[src[i]]`` where ``dst[i] >= 0``: feeds tokens sampled by the
    step before without a round trip through the host."""
    for t, name in ((ids, "ids"), (prev, "prev"), (dst, "dst"), (src, "src")):
        _i32(t, name)
    _check(lib().zi_patch_tokens(_ptr(ids), _ptr(prev), _ptr(dst), _ptr(src), dst.numel(), _stream()), "patch_tokens")


def add_rmsnorm(h: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``h += delta`` in place (32-bit), then RMSNorm of every row.

    ``rows`` (int32, repeats allowed) picks rows instead: the result has one row per entry,
    the norm of ``h[row] + delta[row]``, and ``h`` is left unchanged."""
    T, H = h.shape
    _need(h.dtype == torch.float32 and h.is_contiguous(), "the residual stream is contiguous float32")
    _need(weight.dtype == torch.float32 and weight.numel() == H, "norm weight must be float32 of the row's width")
    part, splits, zstride = None, 0, 0
    if isinstance(delta, Partials):
        _need(tuple(delta.shape) == tuple(h.shape), "delta must match the residual stream")
        part, splits, zstride, delta = delta.data, delta.splits, T * H, None
    elif delta is not None:
        _need(delta.shape == h.shape and delta.is_contiguous(), "delta must match the residual stream")
    n = T if rows is None else _i32(rows, "rows").shape[0]
    if out is None:
        out = torch.empty((n, H), dtype=out_dtype, device=h.device)
    with _prof.region("add_rmsnorm", lambda: (2 if rows is None else 1) * n * H * 4 + _nb(out, weight)
                      + (n * H * delta.element_size() if delta is not None else 0) + splits * n * H * 4):
        _check(lib().zi_add_rmsnorm(_ptr(h), _ptr(delta), _tag(delta) if delta is not None else F32, _ptr(part), splits,
                                    ctypes.c_longlong(zstride), _ptr(weight), ctypes.c_float(eps), _ptr(out), _tag(out),
                                    _ptr(rows), n, H, _stream()), "add_rmsnorm")
    return out


def residual_add(h: torch.Tensor, delta) -> None:
    if isinstance(delta, Partials):
        delta = delta.sum(torch.float32)
    _need(h.dtype == torch.float32 and h.is_contiguous() and delta.is_contiguous() and delta.shape == h.shape,
          "residual_add: shapes must match and be contiguous")
    with _prof.region("residual_add", lambda: 2 * _nb(h) + _nb(delta)):
        _check(lib().zi_residual_add(_ptr(h), _ptr(delta), _tag(delta), ctypes.c_longlong(h.numel()), _stream()),
               "residual_add")


def swiglu(gate_up, out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
           interleave: int = 0) -> torch.Tensor:
    """``silu(gate) * up`` for ``gate_up`` [T, 2I]: gate then up (``interleave`` 0), or blocks
    of 2 * ``interleave`` columns holding ``interleave`` gate values and then the up values of
    the same features."""
    if isinstance(gate_up, Partials):
        T, two_i = gate_up.shape
        I = two_i // 2
        if I % 4 == 0:
            res = torch.empty((T, I), dtype=out_dtype or torch.bfloat16, device=gate_up.data.device)
            with _prof.region("swiglu (partial sums)", lambda: _nb(res, gate_up.data)):
                _check(lib().zi_swiglu_partials(_ptr(res), _tag(res), _ptr(gate_up.data), gate_up.splits,
                                                ctypes.c_longlong(T * two_i), T, I, interleave, _stream()), "swiglu")
            return res
        gate_up = gate_up.sum(out_dtype or torch.bfloat16)
    T, two_i = gate_up.shape
    _need(two_i % 2 == 0 and gate_up.is_contiguous(), "swiglu input is contiguous [T, 2I]")
    I = two_i // 2
    if out is None:
        out = torch.empty((T, I), dtype=gate_up.dtype, device=gate_up.device)
    with _prof.region("swiglu", lambda: _nb(out, gate_up)):
        _check(lib().zi_swiglu(_ptr(out), _ptr(gate_up), _tag(gate_up), T, I, interleave, _stream()), "swiglu")
    return out


SWIGLU_INTERLEAVE = 64   # block of gate rows followed by the up rows of the same features


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, block: int = SWIGLU_INTERLEAVE) -> torch.Tensor:
    """[2I, K] with rows in blocks of 2 * block: ``block`` gate rows, then the up rows of the
    same features (what the fused SwiGLU epilogue of the tensor-core product reads)."""
    I, K = gate.shape
    _need(I % block == 0, f"interleaving needs the width {I} to be a multiple of {block}")
    return torch.stack([gate.view(I // block, block, K), up.view(I // block, block, K)], dim=1).reshape(2 * I, K).contiguous()


def linear_swiglu(x: torch.Tensor, w_interleaved: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``silu(x Wg^T) * (x Wu^T)`` for a gate/up weight interleaved by :func:`interleave_gate_up`.
    On the tensor-core path without a K split the SwiGLU runs in the product's epilogue;
    otherwise the product is followed by the SwiGLU kernel."""
    M, K = x.shape
    N2 = w_interleaved.shape[0]
    if (GEMM_BACKEND != "simt" and x.dtype == torch.bfloat16 and w_interleaved.dtype == torch.bfloat16 and M > 0
            and x.stride(1) == 1 and w_interleaved.is_contiguous()
            and lib().zi_gemm_tcgen05_supported(_ptr(x), _ptr(w_interleaved), K, x.stride(0), w_interleaved.stride(0))):
        out = torch.empty((M, N2 // 2), dtype=out_dtype or x.dtype, device=x.device)
        with _prof.region(f"linear+swiglu N={N2} K={K}", lambda: _nb(w_interleaved, out) + M * K * 2, 2 * M * N2 * K) as rec:
            code = lib().zi_gemm_tcgen05_swiglu(_ptr(out), _tag(out), _ptr(x), _ptr(w_interleaved), M, N2, K, x.stride(0),
                                                w_interleaved.stride(0), out.stride(0), _sm_count(x.device), _stream())
            rec["keep"] = code != -2      # -2: this shape is better served by the product followed by the SwiGLU kernel
        if code != -2:
            _check(code, "linear_swiglu")
            return out
    gu = linear(x, w_interleaved, out_dtype=out_dtype or x.dtype, allow_partials=True)
    return swiglu(gu, out_dtype=out_dtype or x.dtype, interleave=SWIGLU_INTERLEAVE)


def rope_table(n_pos: int, head_dim: int, theta: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    cos = torch.empty((n_pos, head_dim // 2), dtype=torch.float32, device=device)
    sin = torch.empty_like(cos)
    _check(lib().zi_rope_table(_ptr(cos), _ptr(sin), n_pos, head_dim, ctypes.c_float(theta), _stream()), "rope_table")
    return cos, sin


def qk_norm_rope_store(qkv, num_heads: int, num_kv_heads: int, head_dim: int,
                       q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                       cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], positions: torch.Tensor,
                       k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                       slots: Optional[torch.Tensor], page_size: int, write_kv: bool = True,
                       out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """On the fused projection rows [q heads | k heads | v heads]: per-head RMSNorm of q
    and k (when weights are given), rotary positions (when tables are given); k and v go
    into their page slots.  Returns q [T, >= heads * d]: ``qkv`` itself, rewritten in
    place, or a new tensor when ``qkv`` came as split-K partial sums."""
    width = (num_heads + 2 * num_kv_heads) * head_dim if write_kv else num_heads * head_dim
    part, splits, zstride = None, 0, 0
    if isinstance(qkv, Partials):
        T = qkv.shape[0]
        _need(qkv.shape[1] == width, "partial sums must have exactly the heads' width")
        part, splits, zstride = qkv.data, qkv.splits, T * width
        q_out = torch.empty((T, num_heads * head_dim), dtype=out_dtype or torch.bfloat16, device=part.device)
        src, src_stride, dtype_tag = None, 0, _tag(q_out)
    else:
        T = qkv.shape[0]
        _need(qkv.stride(1) == 1, "qkv rows must be dense")
        _need(qkv.shape[1] >= width, "qkv is narrower than its heads")
        q_out, src, src_stride, dtype_tag = qkv, qkv, qkv.stride(0), _tag(qkv)
    for wt in (q_weight, k_weight):
        if wt is not None:
            _need(wt.dtype == torch.float32 and wt.numel() == head_dim, "q/k norm weights are float32 [head_dim]")
    n_table = 0
    if cos is not None:
        _need(cos.shape == sin.shape and cos.shape[1] == head_dim // 2 and cos.dtype == torch.float32,
              "rotary tables are float32 [positions, head_dim/2]")
        n_table = cos.shape[0]
    _i32(positions, "positions")
    if write_kv:
        _need(k_cache is not None and v_cache is not None and slots is not None, "writing needs pages and slots")
        _need(k_cache.dtype == q_out.dtype and v_cache.dtype == q_out.dtype, "cache pages have the activations' dtype")
        _i32(slots, "slots")
    with _prof.region("qk_norm_rope_store", lambda: (2 * T * width * q_out.element_size() if part is None else
                                                      _nb(part) + T * width * q_out.element_size())):
        _check(lib().zi_qk_norm_rope_store(
            _ptr(src), dtype_tag, T, src_stride, _ptr(part), splits, ctypes.c_longlong(zstride), _ptr(q_out),
            q_out.stride(0), num_heads, num_kv_heads, head_dim, _ptr(q_weight), _ptr(k_weight), ctypes.c_float(eps),
            _ptr(cos), _ptr(sin), n_table, _ptr(positions), _ptr(k_cache), _ptr(v_cache), _ptr(slots), page_size,
            1 if write_kv else 0, _stream()), "qk_norm_rope_store")
    return q_out


# ------------------------------------------------------------------------ matrices
_SM_COUNT: dict[int, int] = {}
GEMM_BACKEND = os.environ.get("ZINFER_B200_GEMM", "auto")   # auto | simt  (simt: CUDA cores only, for comparisons)


def _sm_count(device: torch.device) -> int:
    idx = device.index or 0
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _SM_COUNT[idx]


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           out: Optional[torch.Tensor] = None, allow_partials: bool = False):
    """``x [M, K] @ weight [N, K]^T`` with 32-bit accumulation.

    With ``allow_partials`` a product that was split along K may come back as
    :class:`Partials` (its consumer adds the splits) instead of a tensor.

    bfloat16 operands that meet TMA's alignment rules go to the tcgen05 kernel; float32
    operands (the true 32-bit path), mixed types and unaligned shapes go to the
    CUDA-core kernel."""
    M, K = x.shape
    N, K2 = weight.shape
    _need(K == K2, f"linear: x has {K} columns, weight has {K2}")
    _need(x.stride(1) == 1 and weight.is_contiguous(), "linear: operands must be dense along K")
    if (GEMM_BACKEND != "simt" and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and M > 0
            and lib().zi_gemm_tcgen05_supported(_ptr(x), _ptr(weight), K, x.stride(0), weight.stride(0))):
        plan = (ctypes.c_int * 3)()
        sms = _sm_count(x.device)
        need = lib().zi_gemm_tcgen05_plan(M, N, K, sms, plan)
        ws = torch.empty((need // 4,), dtype=torch.float32, device=x.device) if need else None
        defer = allow_partials and need > 0 and out is None
        if out is None and not defer:
            out = torch.empty((M, N), dtype=out_dtype or x.dtype, device=x.device)
        with _prof.region(f"linear N={N} K={K}", lambda: _nb(weight) + M * K * 2 + (_nb(ws) if defer else _nb(out)),
                          2 * M * N * K):
            _check(lib().zi_gemm_tcgen05(_ptr(out), _tag(out) if out is not None else BF16, _ptr(x), _ptr(weight), M, N, K,
                                         x.stride(0), weight.stride(0), out.stride(0) if out is not None else N, _ptr(ws),
                                         ctypes.c_longlong(need), sms, 1 if defer else 0, _stream()), "linear (tcgen05)")
        return Partials(ws.view(plan[2], M, N)) if defer else out
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype or x.dtype, device=x.device)
    _need(out.stride(1) == 1, "linear: output rows must be dense")
    with _prof.region(f"linear (CUDA cores) N={N} K={K}", lambda: _nb(weight, out) + M * K * x.element_size(), 2 * M * N * K):
        _check(lib().zi_gemm_simt(_ptr(out), _tag(out), _ptr(x), _tag(x), _ptr(weight), _tag(weight), M, N, K,
                                  x.stride(0), weight.stride(0), out.stride(0), _stream()), "linear")
    return out


def linear_argmax(x: torch.Tensor, weight: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """The 32-bit product ``x [M, K] @ weight [N, K]^T`` and each row's argmax (first maximum, NaN
    counted as -inf, as :func:`argmax` has it).  For up to 128 rows on the tensor-core path the
    product's epilogue leaves one candidate per 32 weight rows and a small kernel picks among them,
    so the [M, N] result is not read again; otherwise the product is followed by the argmax kernel."""
    M, K = x.shape
    N = weight.shape[0]
    if (GEMM_BACKEND != "simt" and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and M > 0
            and x.stride(1) == 1 and weight.is_contiguous()
            and lib().zi_gemm_tcgen05_supported(_ptr(x), _ptr(weight), K, x.stride(0), weight.stride(0))):
        units = lib().zi_gemm_argmax_units(N)
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        cand_val = torch.empty((M, units), dtype=torch.float32, device=x.device)
        cand_idx = torch.empty((M, units), dtype=torch.int32, device=x.device)
        with _prof.region(f"linear+argmax N={N} K={K}", lambda: _nb(weight, out) + M * K * 2, 2 * M * N * K) as rec:
            code = lib().zi_gemm_tcgen05_argmax(_ptr(out), _ptr(x), _ptr(weight), M, N, K, x.stride(0), weight.stride(0),
                                                out.stride(0), _ptr(cand_val), _ptr(cand_idx), _sm_count(x.device), _stream())
            rec["keep"] = code != -2      # -2: more than 128 rows, or K would be split
        if code != -2:
            _check(code, "linear_argmax")
            ids = torch.empty((M,), dtype=torch.int32, device=x.device)
            with _prof.region("argmax (candidates)", lambda: _nb(cand_val, cand_idx)):
                _check(lib().zi_argmax_candidates(_ptr(ids), _ptr(cand_val), _ptr(cand_idx), M, units, _stream()),
                       "argmax (candidates)")
            return out, ids
    out = linear(x, weight, out_dtype=torch.float32)
    return out, argmax(out)


# ----------------------------------------------------------------------- attention
def attention_tile_rows() -> int:
    return int(lib().zi_paged_attention_tile_rows())


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor,
                    cu_q: torch.Tensor, kv_lens: torch.Tensor, tile_seq: torch.Tensor, tile_q0: torch.Tensor,
                    num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, window: Optional[int],
                    scale: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of the step's query tokens over their requests' pages.

    ``q`` [T, >= num_heads*head_dim] (row stride free), caches [pages, kv heads,
    page_size, head_dim], ``block_tables`` [n, W], ``cu_q`` [n+1] token offsets,
    ``kv_lens`` [n] keys per request including this step's tokens, ``tile_seq`` and
    ``tile_q0`` the request and first token of each query tile."""
    T = q.shape[0]
    _need(q.stride(1) == 1, "q rows must be dense")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous(), "cache pages must be contiguous")
    _need(tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim), "cache pages are [pages, kv heads, page, d]")
    _need(k_cache.dtype == q.dtype, "cache pages have the activations' dtype")
    for name, t in (("block_tables", block_tables), ("cu_q", cu_q), ("kv_lens", kv_lens), ("tile_seq", tile_seq),
                    ("tile_q0", tile_q0)):
        _i32(t, name)
    if out is None:
        out = torch.empty((T, num_heads * head_dim), dtype=q.dtype, device=q.device)
    with _prof.region("attention (exact, CUDA cores)"):
        _check(lib().zi_paged_attention(
            _ptr(out), out.stride(0), _ptr(q), q.stride(0), _tag(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables),
            block_tables.stride(0), _ptr(cu_q), _ptr(kv_lens), _ptr(tile_seq), _ptr(tile_q0), tile_seq.shape[0],
            num_heads, num_kv_heads, head_dim, page_size, int(window or 0), ctypes.c_float(scale), _stream()),
            "paged_attention")
    return out


ATTENTION_BACKEND = os.environ.get("ZINFER_B200_ATTENTION", "auto")   # auto | generic
# Which tensor-core prefill kernel: "tcgen05" (S, P and O in tensor memory, TMA-fed, two query
# tiles per CTA so that one tile's softmax runs under the other's products: 61 us for a prompt of
# 2,048 tokens of 32 heads of 128, head size 128 only) with "mma" (mma.sync flash attention, 160 us)
# for the shapes the first does not take; or "mma" always.
PREFILL_ATTENTION = os.environ.get("ZINFER_B200_PREFILL_ATTENTION", "tcgen05")


def _attention_work(step, decode: bool, num_heads: int, num_kv_heads: int, head_dim: int, elt: int) -> tuple[int, int]:
    """(bytes, flops) of the attention of a step's decode requests (one token) or of its others:
    every key and value of those requests once, their queries and outputs; 4 d per (query, key) pair."""
    nbytes = flops = 0
    for q, c in zip(step.q_lens, step.ctx_lens):
        if (q == 1) != decode:
            continue
        nbytes += 2 * (c + q) * num_kv_heads * head_dim * elt + 2 * q * num_heads * head_dim * elt
        flops += 4 * num_heads * head_dim * (q * c + q * (q + 1) // 2)
    return nbytes, flops


def attention_prefill_tile_rows() -> int:
    return int(lib().zi_attention_prefill_tile_rows())


def attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor, step,
              num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, window: Optional[int],
              scale: float) -> torch.Tensor:
    """Attention of a step's query tokens over their pages, by the fastest kernel that
    takes the shape: in bfloat16 with head sizes 64/128 (decode also 256) the
    tensor-core kernels (requests that bring one token go to the split-key decode
    kernel, the others to the prefill kernel); otherwise, and always in float32, the
    exact CUDA-core kernel.  ``step`` is the StepContext (its request arrays)."""
    T = q.shape[0]
    L = lib()
    fast = ATTENTION_BACKEND != "generic" and q.dtype == torch.bfloat16
    dec_ok = fast and step.n_dec > 0 and L.zi_attention_mma_supported(num_heads, num_kv_heads, head_dim, 1)
    pf_ok = fast and step.n_pf_tiles > 0 and L.zi_attention_mma_supported(num_heads, num_kv_heads, head_dim, 0) \
        and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0
    if (step.n_dec > 0 and not dec_ok) or (step.n_pf_tiles > 0 and not pf_ok):
        return paged_attention(q, k_cache, v_cache, block_tables, step.cu_q, step.kv_lens, step.tile_seq, step.tile_q0,
                               num_heads, num_kv_heads, head_dim, page_size, window, scale)
    _need(q.stride(1) == 1 and k_cache.is_contiguous() and v_cache.is_contiguous(), "attention: dense operands")
    _need(tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim) and k_cache.dtype == q.dtype,
          "cache pages are [pages, kv heads, page, d] in the activations' dtype")
    out = torch.empty((T, num_heads * head_dim), dtype=q.dtype, device=q.device)
    win = int(window or 0)
    work = lambda decode: _attention_work(step, decode, num_heads, num_kv_heads, head_dim, q.element_size()) \
        if _prof.ACTIVE is not None else (0, 0)
    if step.n_pf_tiles > 0 and PREFILL_ATTENTION == "tcgen05" and L.zi_attention_prefill_tcgen05_supported(
            num_heads, num_kv_heads, head_dim, page_size, _ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache)):
        with _prof.region("attention (prefill, tcgen05)", *work(False)):
            _check(L.zi_attention_prefill_tcgen05(
                _ptr(out), out.stride(0), _ptr(q), q.stride(0), T, _ptr(k_cache), _ptr(v_cache),
                ctypes.c_longlong(k_cache.shape[0]), _ptr(block_tables), block_tables.stride(0), _ptr(step.cu_q),
                _ptr(step.kv_lens), _ptr(step.pf_tile_seq), _ptr(step.pf_tile_q0), step.n_pf_tiles, num_heads, num_kv_heads,
                head_dim, page_size, win, ctypes.c_float(scale), _stream()), "attention (prefill, tcgen05)")
    elif step.n_pf_tiles > 0:
        with _prof.region("attention (prefill, mma.sync)", *work(False)):
            _check(L.zi_attention_prefill_mma(
                _ptr(out), out.stride(0), _ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables),
                block_tables.stride(0), _ptr(step.cu_q), _ptr(step.kv_lens), _ptr(step.pf_tile_seq), _ptr(step.pf_tile_q0),
                step.n_pf_tiles, num_heads, num_kv_heads, head_dim, page_size, win, ctypes.c_float(scale), _stream()),
                "attention (prefill)")
    if step.n_dec > 0:
        splits = decode_splits(step.n_dec, num_kv_heads, _sm_count(q.device), step.max_kv_len)
        need = L.zi_attention_decode_workspace_floats(step.n_dec, num_heads, num_kv_heads, head_dim, splits)
        ws = torch.empty((need,), dtype=torch.float32, device=q.device) if need else None
        with _prof.region("attention (decode)", *work(True)):
            _check(L.zi_attention_decode_mma(
                _ptr(out), out.stride(0), _ptr(ws), _ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache),
                ctypes.c_longlong(k_cache.shape[0]), _ptr(block_tables),
                block_tables.stride(0), _ptr(step.cu_q), _ptr(step.kv_lens), _ptr(step.dec_seq), step.n_dec, num_heads,
                num_kv_heads, head_dim, page_size, win, ctypes.c_float(scale), splits, _stream()), "attention (decode)")
    return out


def decode_splits(n_dec: int, num_kv_heads: int, sm_count: int, max_kv_len: Optional[int] = None,
                  fixed_us: float = 3.0) -> int:
    """Key splits of the decode attention.  Its blocks are (request, kv head, split), two fit on an SM
    at once, and a block costs a fixed time (``fixed_us``: launch, prologue, merge; more in the fused
    kernel, which also makes q, k and v) plus its share of the walk over the keys (about 0.02 us a key
    for a block's four warps).  Any split costs the kernel that merges the splits: about 5 us in the
    chain of a decode step, and 0.25 us more per split.  The split count (at most 32, never more than
    tiles of 64 keys) that makes the sum smallest; one, when the blocks already fill more than half of
    the GPU and the keys are few (measured at 24 to 128 requests of 2,048 keys: no split is 4 to 6 %
    of a layer faster than any split; at 16 requests two splits win, at 8 four, at one 12 to 16)."""
    slots, units = 2 * sm_count, max(1, n_dec * num_kv_heads)
    keys = max_kv_len if max_kv_len and max_kv_len > 0 else 2048
    if 2 * units > slots and keys <= 4096:
        return 1
    limit = max(1, min(32, -(-keys // 64)))
    walk = 0.02 * keys
    best, best_cost = 1, float("inf")
    for s in range(1, limit + 1):
        waves = -(-units * s // slots)
        cost = waves * (fixed_us + walk / s) + (5.0 + 0.25 * s if s > 1 else 0.0)
        if cost < best_cost:
            best, best_cost = s, cost
    return best


def decode_tma(mode) -> int:
    """The decode attention's keys and values by TMA (``cp.async.bulk.tensor`` page boxes, a few lanes
    issuing side by side; pages of 8, 16, 32, ... tokens) or by ``cp.async`` from every lane: 1 (the
    default) TMA for up to 16 requests, where it measured slightly faster, 2 or True always, 0 or False
    never.  Returns the setting before.  For tests and timing comparisons."""
    mode = 2 if mode is True else (0 if mode is False else int(mode))
    return int(lib().zi_attention_decode_tma(mode))


def decode_transposed_tile(on: bool) -> bool:
    """The decode attention's tile for groups of at most 8 query heads: with the keys on the MMA's rows
    (on, the default: half the MMAs and a quarter of the exponentials) or with the heads on them as
    for larger groups (off).  Returns the setting before.  For tests and timing comparisons."""
    return bool(lib().zi_attention_decode_transposed(1 if on else 0))


def decode_fused_ok(dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int, step) -> bool:
    """Whether a step can use :func:`attention_decode_fused`: bfloat16, every request brings
    one token, and the split-key decode kernel takes the shape."""
    if not (ATTENTION_BACKEND != "generic" and dtype == torch.bfloat16 and step.n_pf_tiles == 0
            and step.n_dec > 0 and step.n_dec == step.n_seqs and torch.cuda.is_available()
            and lib().zi_attention_mma_supported(num_heads, num_kv_heads, head_dim, 1)):
        return False
    # Worth it while all blocks run at once (few requests: the step is a chain of short
    # kernels and one kernel less counts).  With more blocks than fit, the work every block
    # repeats before it streams its keys costs more than the separate kernel (measured at 64 requests).
    return step.n_dec * num_kv_heads <= 2 * _sm_count(torch.device("cuda", torch.cuda.current_device()))


def attention_decode_fused(qkv, num_heads: int, num_kv_heads: int, head_dim: int, q_weight: Optional[torch.Tensor],
                           k_weight: Optional[torch.Tensor], eps: float, cos: Optional[torch.Tensor],
                           sin: Optional[torch.Tensor], k_cache: torch.Tensor, v_cache: torch.Tensor,
                           slots: torch.Tensor, block_tables: torch.Tensor, step, page_size: int,
                           window: Optional[int], scale: float) -> torch.Tensor:
    """q/k RMSNorm, rotary positions, the write of each token's key and value into its page
    and the attention itself in ONE kernel, for steps in which every request brings a single
    token.  ``qkv`` is the fused projection row as a tensor or as split-K partial sums."""
    L = lib()
    width = (num_heads + 2 * num_kv_heads) * head_dim
    if isinstance(qkv, Partials):
        T = qkv.shape[0]
        _need(qkv.shape[1] == width, "partial sums must have exactly the heads' width")
        src, src_stride, part, psplits, pz = None, 0, qkv.data, qkv.splits, T * width
        device = qkv.data.device
    else:
        T = qkv.shape[0]
        _need(qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1 and qkv.shape[1] >= width, "qkv rows are dense bfloat16")
        src, src_stride, part, psplits, pz = qkv, qkv.stride(0), None, 0, 0
        device = qkv.device
    _need(T == step.n_dec, "every request brings exactly one token")
    for wt in (q_weight, k_weight):
        if wt is not None:
            _need(wt.dtype == torch.float32 and wt.numel() == head_dim, "q/k norm weights are float32 [head_dim]")
    n_table = 0
    if cos is not None:
        _need(cos.shape == sin.shape and cos.shape[1] == head_dim // 2 and cos.dtype == torch.float32,
              "rotary tables are float32 [positions, head_dim/2]")
        n_table = cos.shape[0]
    _need(k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.dtype == torch.bfloat16
          and tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim), "cache pages are bfloat16 [pages, kv heads, page, d]")
    _i32(slots, "slots")
    out = torch.empty((T, num_heads * head_dim), dtype=torch.bfloat16, device=device)
    splits = decode_splits(step.n_dec, num_kv_heads, _sm_count(device), step.max_kv_len, fixed_us=8.0)
    need = L.zi_attention_decode_workspace_floats(step.n_dec, num_heads, num_kv_heads, head_dim, splits)
    ws = torch.empty((need,), dtype=torch.float32, device=device) if need else None
    work = _attention_work(step, True, num_heads, num_kv_heads, head_dim, 2) if _prof.ACTIVE is not None else (0, 0)
    with _prof.region("attention (decode, fused with q/k norm, rotary, cache write)", work[0] + _nb(part), work[1]):
        _check(L.zi_attention_decode_fused(
            _ptr(out), out.stride(0), _ptr(ws), _ptr(src), src_stride, _ptr(part), psplits, ctypes.c_longlong(pz),
            _ptr(q_weight), _ptr(k_weight), ctypes.c_float(eps), _ptr(cos), _ptr(sin), n_table, _ptr(step.positions),
            _ptr(slots), _ptr(k_cache), _ptr(v_cache), ctypes.c_longlong(k_cache.shape[0]), _ptr(block_tables),
            block_tables.stride(0), _ptr(step.cu_q),
            _ptr(step.kv_lens), _ptr(step.dec_seq), step.n_dec, num_heads, num_kv_heads, head_dim, page_size,
            int(window or 0), ctypes.c_float(scale), splits, _stream()), "attention (fused decode)")
    return out


# ------------------------------------------------------------------------ sampling
def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    R, V = logits.shape
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "logits are float32 with dense rows")
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    chunks = lib().zi_argmax_chunks(R, V)
    ws = torch.empty((2 * R * chunks,), dtype=torch.int32, device=logits.device) if chunks else None
    with _prof.region("argmax", lambda: R * V * 4):
        _check(lib().zi_argmax(_ptr(out), _ptr(logits), R, V, logits.stride(0), _ptr(ws), _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, seeds: torch.Tensor, draw_index: torch.Tensor,
           top_k: Optional[torch.Tensor] = None, top_p: Optional[torch.Tensor] = None,
           min_p: Optional[torch.Tensor] = None, repetition_penalty: Optional[torch.Tensor] = None,
           presence_penalty: Optional[torch.Tensor] = None, frequency_penalty: Optional[torch.Tensor] = None,
           count_rows: Optional[torch.Tensor] = None, counts: Optional[torch.Tensor] = None,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row.  Per-row parameters are device tensors: float32 for
    ``temperature``/``top_p``/``min_p``/penalties, int32 for ``top_k``,
    ``draw_index`` and ``count_rows``, int64 for ``seeds``.  ``counts`` [slots, V]
    int32 holds how often each token occurred in a request; the row named by
    ``count_rows`` is read for the penalties and incremented at the drawn token."""
    R, V = logits.shape
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "logits are float32 with dense rows")
    for t in (temperature, top_p, min_p, repetition_penalty, presence_penalty, frequency_penalty):
        if t is not None:
            _need(t.dtype == torch.float32 and t.numel() == R, "per-row float parameters are float32 [rows]")
    for t in (top_k, draw_index, count_rows):
        if t is not None:
            _need(t.dtype == torch.int32 and t.numel() == R, "per-row integer parameters are int32 [rows]")
    _need(seeds.dtype == torch.int64 and seeds.numel() == R, "seeds are int64 [rows]")
    if counts is not None:
        _need(counts.dtype == torch.int32 and counts.shape[1] == V and counts.is_contiguous(), "counts are int32 [slots, V]")
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    with _prof.region("sample", lambda: R * V * 4 * (2 if counts is not None else 1)):
        _check(lib().zi_sample(_ptr(out), _ptr(logits), R, V, logits.stride(0), _ptr(temperature), _ptr(top_k),
                               _ptr(top_p), _ptr(min_p), _ptr(repetition_penalty), _ptr(presence_penalty),
                               _ptr(frequency_penalty), _ptr(count_rows), _ptr(counts), _ptr(seeds), _ptr(draw_index),
                               _stream()), "sample")
    return out


def count_tokens(counts_row: torch.Tensor, tokens: torch.Tensor) -> None:
    _need(counts_row.dtype == torch.int32 and counts_row.is_contiguous(), "counts row is contiguous int32")
    _i32(tokens, "tokens")
    _check(lib().zi_count_tokens(_ptr(counts_row), _ptr(tokens), tokens.numel(), counts_row.numel(), _stream()),
           "count_tokens")
