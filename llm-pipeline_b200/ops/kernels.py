"""Python bindings of the CUDA entry points (``csrc/*.cu``), one function per kernel.

Arguments are CUDA tensors; the functions check types, contiguity and sizes, pass raw pointers
and the current stream to the library, and raise ``KernelError`` with the library's message when
an entry point refuses its arguments. There is no CPU implementation behind these functions: a
tensor that is not on a CUDA device is an error.
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional, Sequence

import torch

from .build import library

F32, BF16 = 0, 1
_P = ctypes.c_void_p
_I = ctypes.c_int
_L = ctypes.c_long
_F = ctypes.c_float


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported element type {dtype}; the kernels take float32 and bfloat16")


_SIGNATURES = {
    "llmp_embedding": [_P, _P, _I, _P, _I, _I, _I, _F, _P],
    "llmp_rope_tables": [_P, _P, _F, _P, _P, _I, _I, _P],
    "llmp_add_rmsnorm": [_P, _P, _P, _I, _P, _I, _F, _P, _I, _P, _I, _I, _P],
    "llmp_qkv_post": [_P, _I, _P, _I, _P, _P, _I, _F, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _P],
    "llmp_swiglu": [_P, _P, _I, _I, _I, _P],
    "llmp_gemm_simt": [_P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _L, _L, _L, _P],
    "llmp_gemm_skinny": [_P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _P],
    "llmp_gemm_tc": [_P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _P, _P],
    "llmp_gemm_stream": [_P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _P, _P],
    "llmp_gemm_stream_swiglu": [_P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _P, _P],
    "llmp_gemm_stream_tc": [_P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _P, _P],
    "llmp_paged_attention": [_P, _L, _P, _L, _P, _I, _I, _P, _I, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I,
                             _P, _P],
    "llmp_gemm_stream_fused": [_P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _I, _P, _I, _F, _F, _P, _L, _P, _I, _P, _L, _P, _P, _P],
    "llmp_decode_attention": [_P, _L, _P, _L, _P, _I, _I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _I, _F, _P, _L, _P, _I, _P, _P],
    "llmp_argmax": [_P, _L, _I, _I, _P, _P, _P],
    "llmp_repetition_penalty": [_P, _L, _I, _I, _P, _P, _P, _P],
    "llmp_sample": [_P, _L, _I, _I, _P, _P, _P, _P],
    "llmp_entropy": [_P, _L, _I, _I, _F, _P, _P],
    "llmp_bounded_wait_check": [_P, _I, _P, _P],
    "llmp_gemm_stream_chain": [_P, _I, _I, _P, _P, _P],
    "llmp_gemm_simt_batched": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _L, _L, _L, _L, _L, _L, _P],
    "llmp_embedding_norm": [_P, _P, _I, _P, _I, _F, _F, _P, _I, _I, _I, _P],
    "llmp_add_norm_mix": [_P, _P, _I, _P, _I, _F, _F, _P, _L, _P, _I, _P, _I, _F, _F, _P, _I, _P, _I, _I, _P],
    "llmp_poly_norm": [_P, _I, _L, _P, _F, _P, _I, _I, _I, _P],
    "llmp_softcap": [_P, _L, _F, _P],
    "llmp_min_gru": [_P, _P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _P],
    "llmp_latent_kv_post": [_P, _I, _L, _I, _I, _I, _I, _P, _I, _F, _P, _P, _I, _P, _P, _I, _P],
    "llmp_latent_attention": [_P, _L, _L, _P, _L, _L, _P, _I, _P, _I, _P, _P, _P, _L, _L, _I, _I, _I, _I, _I, _F, _P, _P],
    "llmp_latent_attention_mma": [_P, _L, _L, _P, _L, _L, _P, _P, _I, _P, _P, _P, _P, _P, _I, _P, _L, _L, _I, _I, _I, _I, _I, _F, _I,
                                  _I, _P, _P, _P],
    "llmp_latent_rows_post": [_P, _L, _P, _L, _I, _I, _I, _I, _P, _I, _F, _P, _P, _I, _I, _P, _I, _L, _P, _P, _I, _P],
    "llmp_capped_qkv_post": [_P, _L, _P, _I, _F, _I, _P, _I, _L, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "llmp_capped_attention": [_P, _L, _P, _I, _P, _I, _P, _P, _P, _P, _P, _L, _P, _L, _I, _I, _I, _I, _I, _I, _I, _I, _F, _F, _P],
    "llmp_capped_attention_mma": [_P, _L, _P, _L, _P, _P, _I, _P, _P, _P, _P, _I, _P, _P, _P, _L, _I, _I, _I, _I, _I, _I, _I, _F, _F, _I, _P],
    "llmp_selective_scan": [_P, _L, _P, _L, _P, _P, _P, _L, _P, _P, _P, _L, _P, _L, _L, _P, _P, _P, _P, _I, _L, _I, _I, _I, _P],
    "llmp_add_rmsnorm_multi": [_P, _P, _I, _P, _I, _P, _I, _P, _I, _I, _F, _P, _I, _L, _L, _P, _I, _I, _P],
    "llmp_gated_act": [_P, _I, _L, _P, _I, _L, _I, _I, _P],
    "llmp_sigmoid_gate": [_P, _P, _L, _P, _I, _L, _I, _P],
    "llmp_convert_rows": [_P, _L, _P, _I, _L, _I, _P],
    "llmp_route_topk": [_P, _I, _P, _I, _P, _P, _I, _I, _I, _I, _P, _P, _P],
    "llmp_expert_grouped": [_P, _P, _P, _P, _P, _F, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    "llmp_expert_rows": [_P, _P, _P, _I, _P, _P, _F, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "llmp_add_layernorm": [_P, _P, _I, _P, _I, _P, _P, _I, _F, _P, _I, _I, _I, _P, _P],
    "llmp_relu_squared": [_P, _P, _I, _L, _P],
    "llmp_add_scaled_rows": [_P, _P, _I, _P, _I, _I, _P],
    "llmp_diff_qkv_post": [_P, _I, _L, _I, _I, _I, _I, _P, _P, _I, _F, _P, _P, _I, _P, _P, _I, _I, _P],
    "llmp_diff_attention": [_P, _L, _P, _I, _P, _I, _P, _P, _P, _L, _I, _I, _I, _I, _I, _I, _I, _F, _F, _F, _F, _P],
    "llmp_diff_attention_mma": [_P, _L, _P, _L, _P, _P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _F, _F, _F,
                                _I, _I, _I, _P, _P, _P],
    "llmp_short_conv": [_P, _L, _P, _I, _P, _I, _P, _L, _L, _P, _P, _P, _P, _P, _L, _P, _I, _L, _L, _I, _I, _I, _I, _I, _I, _I, _P],
    "llmp_ssd_scan": [_P, _L, _P, _L, _P, _P, _P, _P, _L, _L, _P, _P, _P, _P, _L, _I, _I, _I, _I, _I, _P],
    "llmp_gated_group_norm": [_P, _L, _P, _L, _P, _P, _I, _L, _I, _I, _I, _I, _F, _P],
    "llmp_delta_prep": [_P, _L, _P, _L, _P, _L, _P, _L, _P, _P, _I, _I, _I, _I, _P],
    "llmp_delta_scan": [_P, _L, _P, _L, _P, _L, _P, _L, _P, _L, _P, _L, _L, _P, _P, _P, _P, _L, _I, _I, _I, _I, _I, _P],
    "llmp_sig_qkv_post": [_P, _L, _P, _I, _P, _P, _I, _P, _I, _L, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "llmp_sigmoid_attention": [_P, _L, _P, _I, _P, _I, _P, _P, _P, _P, _P, _L, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _F, _P],
    "llmp_sigmoid_attention_mma": [_P, _L, _P, _P, _I, _P, _P, _P, _P, _P, _I, _P, _P, _P, _L, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _F, _P],
    "llmp_xielu": [_P, _P, _I, _F, _F, _P, _I, _L, _I, _P],
    "llmp_scaled_sum": [_P, _F, _P, _F, _P, _L, _P],
}
_bound = {}
launch_count = 0   # kernels of this library launched so far (captured launches count once per capture)


def _fn(name: str):
    fn = _bound.get(name)
    if fn is None:
        lib = library()
        fn = getattr(lib, name)
        fn.argtypes = _SIGNATURES[name]
        fn.restype = ctypes.c_int
        _bound[name] = fn
    return fn


def _call(name: str, *args) -> None:
    global launch_count
    launch_count += 1
    rc = _fn(name)(*args)
    if rc != 0:
        lib = library()
        lib.llmp_last_error.restype = ctypes.c_char_p
        raise KernelError(lib.llmp_last_error().decode(errors="replace"))


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("a kernel was given a tensor that is not on a CUDA device; this engine has no CPU path")
    return t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream of the current device as a raw handle (the fast accessor where torch has it:
    ``torch.cuda.current_stream()`` costs about 15 microseconds a call, several milliseconds per eager step)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _need(cond: bool, message: str) -> None:
    if not cond:
        raise KernelError(message)


def _i32(t: torch.Tensor, name: str) -> None:
    _need(t.dtype == torch.int32 and t.is_contiguous(), f"{name} must be a contiguous int32 tensor")


def tokens_per_attention_tile(num_heads: int, num_kv_heads: int, dtype: torch.dtype = torch.float32,
                              head_dim: int = 0, page_size: int = 0) -> int:
    """Query tokens per tile of the general attention kernel that serves this type, head size and page
    size (0: not known, which rules out the kernels that depend on the page size)."""
    fn = library().llmp_attention_tokens_per_tile
    fn.argtypes = [_I, _I, _I, _I, _I]
    fn.restype = _I
    n = fn(num_heads, num_kv_heads, dtype_code(dtype), head_dim, page_size)
    _need(n > 0, f"{num_heads} query heads cannot share {num_kv_heads} key/value heads")
    return n


def attention_max_segments(num_heads: int, num_kv_heads: int, dtype: torch.dtype, head_dim: int, page_size: int) -> int:
    """How many items of the tile list may share the keys of one tile in the general attention kernel that serves
    these sizes (1: it takes whole tiles only)."""
    fn = library().llmp_attention_max_segments
    fn.argtypes = [_I, _I, _I, _I, _I]
    fn.restype = _I
    return int(fn(num_heads, num_kv_heads, dtype_code(dtype), head_dim, page_size))


ATTENTION_MAX_PLACES = 8192          # places for the sums of items that share a tile, per launch
_attention_counters: dict = {}
_place_floats: Optional[int] = None


def attention_place_floats() -> int:
    global _place_floats
    if _place_floats is None:
        fn = library().llmp_attention_place_floats
        fn.argtypes = []
        fn.restype = _L
        _place_floats = int(fn())
    return _place_floats


def attention_counters(device: torch.device, count: int) -> torch.Tensor:
    """Counters with which the items that share a tile find out who finishes last; every launch leaves them zero.
    One set per device, as for ``decode_counters``."""
    key = torch.device(device).index or 0
    counters = _attention_counters.get(key)
    if counters is None or counters.numel() < count:
        _need(not torch.cuda.is_current_stream_capturing(), "attention counters must exist before a graph is captured")
        counters = _attention_counters[key] = torch.zeros(max(count, 65536), dtype=torch.int32, device=device)
    return counters


def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """out[n, :] = float32(table[ids[n], :]) * scale"""
    _i32(ids, "ids")
    _need(table.dim() == 2 and table.is_contiguous(), "embedding table must be a contiguous matrix")
    _need(out.dtype == torch.float32 and out.is_contiguous() and out.shape == (ids.numel(), table.shape[1]),
          "embedding output must be float32 [tokens, hidden]")
    _call("llmp_embedding", _ptr(ids), _ptr(table), dtype_code(table.dtype), _ptr(out), ids.numel(),
          table.shape[1], table.shape[0], float(scale), _stream())
    return out


def rope_tables(positions: torch.Tensor, inv_freq: torch.Tensor, scaling: float, cos: torch.Tensor,
                sin: torch.Tensor) -> None:
    """cos/sin[n, j] = cos/sin(float(positions[n]) * inv_freq[j]) * scaling, all float32."""
    _i32(positions, "positions")
    half = inv_freq.numel()
    _need(inv_freq.dtype == torch.float32 and inv_freq.is_contiguous(), "inv_freq must be contiguous float32")
    for t in (cos, sin):
        _need(t.dtype == torch.float32 and t.is_contiguous() and t.shape == (positions.numel(), half),
              "rotary tables must be float32 [tokens, rotary_dim / 2]")
    _call("llmp_rope_tables", _ptr(positions), _ptr(inv_freq), float(scaling), _ptr(cos), _ptr(sin),
          positions.numel(), half, _stream())


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, delta_bias: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x = residual + delta (+ delta_bias); residual = x (unless ``rows`` selects rows);
    out = weight * (x * rsqrt(mean(x^2) + eps)).  residual is float32, delta/out have the compute type."""
    H = residual.shape[-1]
    _need(residual.dtype == torch.float32 and residual.is_contiguous() and residual.dim() == 2,
          "residual must be a contiguous float32 matrix")
    M = rows.numel() if rows is not None else residual.shape[0]
    _need(out.is_contiguous() and out.shape == (M, H), "norm output has the wrong shape")
    if delta is not None:
        _need(delta.dtype == out.dtype and delta.is_contiguous() and delta.shape == residual.shape,
              "delta must match the residual's shape and the output's type")
    _need(weight.numel() == H and weight.is_contiguous(), "norm weight has the wrong size")
    if delta_bias is not None:
        _need(delta_bias.numel() == H and delta_bias.is_contiguous(), "delta bias has the wrong size")
    if rows is not None:
        _i32(rows, "rows")
    _call("llmp_add_rmsnorm", _ptr(residual), _ptr(delta), _ptr(delta_bias),
          dtype_code(delta_bias.dtype) if delta_bias is not None else F32, _ptr(weight), dtype_code(weight.dtype),
          float(eps), _ptr(out), dtype_code(out.dtype), _ptr(rows), M, H, _stream())
    return out


# ---- the library product into a float32 residual ---------------------------------------------------------------------
_cublas = None
_CUDA_R_16BF, _CUDA_R_32F, _CUBLAS_COMPUTE_32F, _CUBLAS_OP_N, _CUBLAS_OP_T, _CUBLAS_GEMM_DEFAULT = 14, 0, 68, 0, 1, -1


def _cublas_gemm_ex():
    """cuBLAS's cublasGemmEx from the library that torch has loaded (None when it cannot be had)."""
    global _cublas
    if _cublas is None:
        _cublas = False
        for name in ("libcublas.so.12", "libcublas.so"):
            try:
                fn = ctypes.CDLL(name).cublasGemmEx
            except (OSError, AttributeError):
                continue
            fn.restype = ctypes.c_int
            fn.argtypes = [_P, _I, _I, _I, _I, _I, _P, _P, _I, _I, _P, _I, _I, _P, _P, _I, _I, _I, _I]
            _cublas = fn
            break
    return _cublas or None


_ONE = ctypes.c_float(1.0)
_ONE_REF = ctypes.byref(_ONE)


def library_add_product(residual: torch.Tensor, x: torch.Tensor, w: torch.Tensor) -> bool:
    """residual[M, N] (float32) += x[M, K] @ w[N, K]^T (bfloat16 operands, float32 sums) by the library's matrix
    product with the residual as its float32 C operand: the product is never rounded to bfloat16 and the norm kernel
    after it has nothing to add. On torch's cuBLAS handle and current stream, like ``torch.mm``; where the engine uses
    a library product for the rows of a prompt portion (the reference's ``nn.Linear`` is the same library,
    src/llm_pipeline/models/qwen3/custom_builder.py:124-131). False, and nothing done, when the operands are not of
    these types, not row-major, not 16-byte aligned, or the library cannot be had."""
    gemm = _cublas or _cublas_gemm_ex()
    M, K = x.shape
    N = w.shape[0]
    if (not gemm or residual.dtype != torch.float32 or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or M == 0 or
            not residual.is_cuda or x.stride(1) != 1 or w.stride(1) != 1 or residual.stride(1) != 1 or w.shape[1] != K or
            residual.shape != (M, N)):
        return False
    xp, wp, rp = x.data_ptr(), w.data_ptr(), residual.data_ptr()
    if (xp | wp | rp) % 16:
        return False
    # row-major residual[M, N] is column-major [N, M]: (w as [K, N] column-major, transposed) times (x as [K, M])
    rc = gemm(torch.cuda.current_blas_handle(), _CUBLAS_OP_T, _CUBLAS_OP_N, N, M, K, _ONE_REF, wp, _CUDA_R_16BF, w.stride(0),
              xp, _CUDA_R_16BF, x.stride(0), _ONE_REF, rp, _CUDA_R_32F, residual.stride(0), _CUBLAS_COMPUTE_32F,
              _CUBLAS_GEMM_DEFAULT)
    if rc != 0:
        raise KernelError(f"cublasGemmEx failed with status {rc}")
    return True


def qkv_post(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, *,
             bias: Optional[torch.Tensor], q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
             eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary_dim: int,
             slots: Optional[torch.Tensor], pages: Optional[torch.Tensor], page_size: int) -> None:
    """In place on qkv [N, (nq + 2 nkv) d]: bias, per-head RMSNorm of q and k, rotary; k and v are
    stored to their page slots (pages [P, 2, nkv, page_size, d])."""
    N = qkv.shape[0]
    _need(qkv.is_contiguous() and qkv.shape[1] == (num_heads + 2 * num_kv_heads) * head_dim,
          "qkv must be contiguous [tokens, (heads + 2 kv heads) * head_dim]")
    if pages is not None:
        _need(pages.dtype == qkv.dtype and pages.is_contiguous() and
              tuple(pages.shape[1:]) == (2, num_kv_heads, page_size, head_dim), "pages have the wrong layout")
        _need(slots is not None, "a page write needs slots")
    if slots is not None:
        _i32(slots, "slots")
        _need(slots.numel() == N, "one slot per token")
    w_dtype = F32
    if q_weight is not None:
        _need(k_weight is not None and q_weight.dtype == k_weight.dtype and q_weight.numel() == head_dim and
              k_weight.numel() == head_dim, "q/k norm weights must have head_dim entries of one type")
        w_dtype = dtype_code(q_weight.dtype)
    if rotary_dim:
        _need(cos is not None and sin is not None and cos.shape == (N, rotary_dim // 2) and cos.dtype == torch.float32
              and cos.is_contiguous() and sin.is_contiguous(), "rotary tables must be float32 [tokens, rotary_dim / 2]")
    if bias is not None:
        _need(bias.numel() == qkv.shape[1] and bias.is_contiguous(), "qkv bias has the wrong size")
    _call("llmp_qkv_post", _ptr(qkv), dtype_code(qkv.dtype), _ptr(bias),
          dtype_code(bias.dtype) if bias is not None else F32, _ptr(q_weight), _ptr(k_weight), w_dtype, float(eps),
          _ptr(cos), _ptr(sin), int(rotary_dim), _ptr(slots), _ptr(pages), N, num_heads, num_kv_heads, head_dim,
          int(page_size), _stream())


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[n, i] = silu(gate_up[n, i]) * gate_up[n, I + i]"""
    N, two_i = gate_up.shape
    _need(gate_up.is_contiguous() and out.is_contiguous() and out.shape == (N, two_i // 2) and
          out.dtype == gate_up.dtype and two_i % 2 == 0, "swiglu shapes do not match")
    _call("llmp_swiglu", _ptr(gate_up), _ptr(out), dtype_code(out.dtype), N, two_i // 2, _stream())
    return out


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T (+ bias) on the CUDA cores with float32 accumulation."""
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N), "gemm shapes do not match")
    _need(a.dtype == w.dtype, "gemm operands must have one type")
    _need(a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1, "gemm operands must be row-major")
    if bias is not None:
        _need(bias.numel() == N and bias.is_contiguous(), "gemm bias has the wrong size")
    _call("llmp_gemm_simt", _ptr(a), _ptr(w), _ptr(bias), dtype_code(bias.dtype) if bias is not None else F32,
          _ptr(out), dtype_code(a.dtype), dtype_code(out.dtype), M, N, K, a.stride(0), w.stride(0), out.stride(0),
          _stream())
    return out


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T for M <= 16, bfloat16 operands, bfloat16 or float32 output: the
    weight-streaming tensor-core kernel of the decode step."""
    M, K = x.shape
    N = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "gemm_skinny takes bfloat16 operands")
    _need(w.shape[1] == K and out.shape == (M, N), "gemm shapes do not match")
    _need(x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1, "gemm operands must be row-major")
    _call("llmp_gemm_skinny", _ptr(x), _ptr(w), _ptr(out), dtype_code(out.dtype), M, N, K, x.stride(0), w.stride(0),
          out.stride(0), _stream())
    return out


_error_flag: Optional[torch.Tensor] = None


def error_flag() -> torch.Tensor:
    """One int32 in pinned host memory that kernels with bounded waits set to 1 when a wait ran out.
    The device writes it through its mapped address; the host may read it after any synchronisation."""
    global _error_flag
    if _error_flag is None:
        _error_flag = torch.zeros(1, dtype=torch.int32).pin_memory()
    return _error_flag


def check_error_flag() -> None:
    if _error_flag is not None and int(_error_flag[0]) != 0:
        _error_flag[0] = 0
        raise KernelError("a kernel gave up waiting on one of its barriers (bounded wait ran out); its output is not valid")


def bounded_wait_check(limit: int = 1024) -> bool:
    """Self-check of the bounded waits: launches one thread that waits, with the kernels' own wait and a limit of
    ``limit`` tries, on a barrier that nothing completes. True when the wait gave up; ``check_error_flag()`` then raises
    after the next synchronisation, as it does when a wait of a real kernel runs out."""
    gave_up = torch.zeros(1, dtype=torch.int32, device="cuda")
    _call("llmp_bounded_wait_check", error_flag().data_ptr(), int(limit), _ptr(gave_up), _stream())
    return bool(int(gave_up.item()))


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T on the tcgen05 tensor cores (TMA loads, accumulator in tensor
    memory); bfloat16 operands, bfloat16 or float32 output."""
    M, K = x.shape
    N = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "gemm_tc takes bfloat16 operands")
    _need(w.shape[1] == K and out.shape == (M, N), "gemm shapes do not match")
    _need(x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1, "gemm operands must be row-major")
    _need(x.is_cuda and w.is_cuda and out.is_cuda, "gemm_tc takes CUDA tensors")
    _call("llmp_gemm_tc", _ptr(x), _ptr(w), _ptr(out), dtype_code(out.dtype), M, N, K, x.stride(0), w.stride(0),
          out.stride(0), error_flag().data_ptr(), _stream())
    return out


def gemm_stream_supports(M: int, N: int, K: int, ldx: int, ldw: int) -> bool:
    fn = library().llmp_gemm_stream_supports
    fn.argtypes = [_I, _I, _I, _L, _L]
    fn.restype = _I
    return bool(fn(M, N, K, ldx, ldw))


def gemm_stream(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T for at most 64 rows (see ``gemm_stream_supports``): one persistent block per SM streams its share of
    ``w`` through a ring of TMA boxes; bfloat16 operands, bfloat16 or float32 output, K a multiple of 64."""
    M, K = x.shape
    N = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "gemm_stream takes bfloat16 operands")
    _need(w.shape[1] == K and out.shape == (M, N), "gemm shapes do not match")
    _need(x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1, "gemm operands must be row-major")
    _need(x.is_cuda and w.is_cuda and out.is_cuda, "gemm_stream takes CUDA tensors")
    _call("llmp_gemm_stream", _ptr(x), _ptr(w), _ptr(out), dtype_code(out.dtype), M, N, K, x.stride(0), w.stride(0),
          out.stride(0), error_flag().data_ptr(), _stream())
    return out


def gemm_stream_tc_supports(M: int, N: int, K: int, ldx: int, ldw: int) -> bool:
    fn = library().llmp_gemm_stream_tc_supports
    fn.argtypes = [_I, _I, _I, _L, _L]
    fn.restype = _I
    return bool(fn(M, N, K, ldx, ldw))


def gemm_stream_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T for at most 64 rows: the weight stream of ``gemm_stream`` with the
    products by tcgen05.mma and the accumulator in tensor memory; bfloat16 operands, K a multiple of 64."""
    M, K = x.shape
    N = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "gemm_stream_tc takes bfloat16 operands")
    _need(w.shape[1] == K and out.shape == (M, N), "gemm shapes do not match")
    _need(x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1, "gemm operands must be row-major")
    _need(x.is_cuda and w.is_cuda and out.is_cuda, "gemm_stream_tc takes CUDA tensors")
    _call("llmp_gemm_stream_tc", _ptr(x), _ptr(w), _ptr(out), dtype_code(out.dtype), M, N, K, x.stride(0), w.stride(0),
          out.stride(0), error_flag().data_ptr(), _stream())
    return out


def gemm_stream_blocks(M: int, N: int, K: int, ldx: int, ldw: int) -> int:
    """Blocks that ``gemm_stream`` deals a product of these sizes out to (0: sizes it does not take)."""
    fn = library().llmp_gemm_stream_blocks
    fn.argtypes = [_I, _I, _I, _L, _L]
    fn.restype = _I
    return int(fn(M, N, K, ldx, ldw))


def gemm_stream_fused(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor], *, glu: bool = False,
                      in_sumsq: Optional[torch.Tensor] = None, in_parts: int = 0, in_width: int = 0, in_eps: float = 0.0,
                      residual: Optional[torch.Tensor] = None, norm_weight: Optional[torch.Tensor] = None,
                      xw: Optional[torch.Tensor] = None, out_sumsq: Optional[torch.Tensor] = None) -> None:
    """The streaming product (at most 8 rows of x) with the work of the RMSNorm around it folded in.

    ``in_sumsq`` [parts, 8] float32: the rows of ``x`` still lack the factor rsqrt(sum(in_sumsq[:in_parts, m]) / in_width +
    in_eps); the product is multiplied by it (with ``glu`` before the SwiGLU of ``w`` = [gate rows; up rows]).
    ``residual`` [M, N] float32: the product is added into it; ``xw`` [M, N] bfloat16 receives residual * norm_weight and
    ``out_sumsq`` [gemm_stream_blocks(...), 8] each block's sums of residual^2, which are what the next product takes as
    ``x`` and ``in_sumsq``; ``out`` is then not written and may be None."""
    M, K = x.shape
    N = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and M <= 8, "gemm_stream_fused takes up to 8 bfloat16 rows")
    _need(w.shape[1] == K and x.stride(1) == 1 and w.stride(1) == 1, "gemm operands must be row-major and match")
    if out is not None:
        _need(out.shape == (M, N // 2 if glu else N) and out.stride(1) == 1, "gemm output has the wrong shape")
    if in_sumsq is not None:
        _need(in_sumsq.dtype == torch.float32 and in_sumsq.is_contiguous() and in_sumsq.shape[1] == 8 and
              0 < in_parts <= in_sumsq.shape[0] and in_width > 0, "sums of squares must be [parts, 8] float32")
    if residual is not None:
        _need(not glu and out_sumsq is not None and xw is not None and norm_weight is not None,
              "the residual form needs a norm weight, xw and out_sumsq, and no SwiGLU")
        _need(residual.dtype == torch.float32 and residual.shape == (M, N) and residual.stride(1) == 1, "residual must be [M, N] float32")
        _need(xw.dtype == torch.bfloat16 and xw.shape == (M, N) and xw.stride(1) == 1, "xw must be [M, N] bfloat16")
        _need(norm_weight.numel() == N and norm_weight.is_contiguous() and norm_weight.dtype in (torch.float32, torch.bfloat16),
              "the norm weight must have N entries")
        _need(out_sumsq.dtype == torch.float32 and out_sumsq.is_contiguous() and out_sumsq.shape[1] == 8 and
              out_sumsq.shape[0] >= gemm_stream_blocks(M, N, K, x.stride(0), w.stride(0)) > 0, "out_sumsq must be [blocks, 8] float32")
    else:
        _need(out is not None, "a product that is no residual addend needs an output")
    _call("llmp_gemm_stream_fused", _ptr(x), _ptr(w), _ptr(out), dtype_code(out.dtype) if out is not None else BF16, M, N, K,
          x.stride(0), w.stride(0), out.stride(0) if out is not None else 0, N // 2 if glu else 0,
          _ptr(in_sumsq), int(in_parts), 1.0 / in_width if in_width else 0.0, float(in_eps),
          _ptr(residual), residual.stride(0) if residual is not None else 0, _ptr(norm_weight),
          dtype_code(norm_weight.dtype) if norm_weight is not None else F32, _ptr(xw), xw.stride(0) if xw is not None else 0,
          _ptr(out_sumsq), error_flag().data_ptr(), _stream())


class ChainPhase(ctypes.Structure):
    """One product of ``gemm_stream_chain`` as the library reads it (``LlmpChainPhase`` in csrc/gemm_stream_chain.cu)."""

    _fields_ = [("X", _P), ("W", _P), ("Y", _P), ("ldx", _L), ("ldw", _L), ("ldy", _L),
                ("N", _I), ("K", _I), ("out_dtype", _I), ("glu_rows", _I),
                ("in_sumsq", _P), ("in_parts", _I), ("in_inv_width", _F), ("in_eps", _F),
                ("residual", _P), ("ldr", _L), ("norm_w", _P), ("norm_w_dtype", _I),
                ("xw", _P), ("ldxw", _L), ("out_sumsq", _P)]


def chain_phase(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor], *, glu: bool = False,
                in_sumsq: Optional[torch.Tensor] = None, in_parts: int = 0, in_width: int = 0, in_eps: float = 0.0,
                residual: Optional[torch.Tensor] = None, norm_weight: Optional[torch.Tensor] = None,
                xw: Optional[torch.Tensor] = None, out_sumsq: Optional[torch.Tensor] = None) -> ChainPhase:
    """A phase of a chain, with the arguments of ``gemm_stream_fused``."""
    K = x.shape[1]
    N = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1 and w.shape[1] == K,
          "a chain takes row-major bfloat16 operands that match")
    phase = ChainPhase()
    phase.X, phase.W, phase.Y = _ptr(x), _ptr(w), _ptr(out)
    phase.ldx, phase.ldw, phase.ldy = x.stride(0), w.stride(0), out.stride(0) if out is not None else 0
    phase.N, phase.K, phase.out_dtype = N, K, dtype_code(out.dtype) if out is not None else BF16
    phase.glu_rows = N // 2 if glu else 0
    phase.in_sumsq, phase.in_parts = _ptr(in_sumsq), int(in_parts)
    phase.in_inv_width, phase.in_eps = (1.0 / in_width if in_width else 0.0), float(in_eps)
    phase.residual, phase.ldr = _ptr(residual), residual.stride(0) if residual is not None else 0
    phase.norm_w = _ptr(norm_weight)
    phase.norm_w_dtype = dtype_code(norm_weight.dtype) if norm_weight is not None else F32
    phase.xw, phase.ldxw = _ptr(xw), xw.stride(0) if xw is not None else 0
    phase.out_sumsq = _ptr(out_sumsq)
    return phase


_chain_counters: dict = {}
_chain_max_phases: Optional[int] = None


def gemm_stream_chain_max_phases() -> int:
    global _chain_max_phases
    if _chain_max_phases is None:
        fn = library().llmp_gemm_stream_chain_max_phases
        fn.argtypes = []
        fn.restype = _I
        _chain_max_phases = int(fn())
    return _chain_max_phases


def gemm_stream_chain_supports(phases: Sequence[ChainPhase], M: int) -> bool:
    fn = library().llmp_gemm_stream_chain_supports
    fn.argtypes = [_P, _I, _I]
    fn.restype = _I
    array = (ChainPhase * len(phases))(*phases)
    return bool(fn(ctypes.cast(array, _P), len(phases), M))


def gemm_stream_chain(phases: Sequence[ChainPhase], M: int, device: torch.device) -> None:
    """The products of ``phases`` (at most 8 rows of X each, every phase reading what the phase before wrote) in one
    persistent cooperative launch whose ring of weight boxes never drains between them; the results are those of
    ``gemm_stream_fused`` called phase by phase, bit for bit. The blocks tell each other through counters in global
    memory that a phase is complete; one set per device, so chains on a device must follow one another in one stream."""
    key = torch.device(device).index or 0
    counters = _chain_counters.get(key)
    if counters is None:
        _need(not torch.cuda.is_current_stream_capturing(), "the chain's counters must exist before a graph is captured")
        fn = library().llmp_gemm_stream_chain_counters
        fn.argtypes = []
        fn.restype = _I
        counters = _chain_counters[key] = torch.zeros(int(fn()), dtype=torch.int32, device=device)
    array = (ChainPhase * len(phases))(*phases)
    _call("llmp_gemm_stream_chain", ctypes.cast(array, _P), len(phases), int(M), _ptr(counters), error_flag().data_ptr(),
          _stream())


def gemm_stream_swiglu_supports(M: int, I: int, K: int, ldx: int, ldw: int) -> bool:
    fn = library().llmp_gemm_stream_swiglu_supports
    fn.argtypes = [_I, _I, _I, _L, _L]
    fn.restype = _I
    return bool(fn(M, I, K, ldx, ldw))


def gemm_stream_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[m, i] = silu(x[m] . w[i]) * (x[m] . w[I + i]) for ``w_gate_up`` = [gate rows; up rows] ([2 I, K]): the
    gate/up product of a SwiGLU feed-forward and its activation in one streaming kernel (at most 16 rows of x)."""
    M, K = x.shape
    I = w_gate_up.shape[0] // 2
    _need(x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16, "gemm_stream_swiglu takes bfloat16 operands")
    _need(w_gate_up.shape == (2 * I, K) and out.shape == (M, I), "gemm_stream_swiglu shapes do not match")
    _need(x.stride(1) == 1 and w_gate_up.stride(1) == 1 and out.stride(1) == 1, "gemm operands must be row-major")
    _need(x.is_cuda and w_gate_up.is_cuda and out.is_cuda, "gemm_stream_swiglu takes CUDA tensors")
    _call("llmp_gemm_stream_swiglu", _ptr(x), _ptr(w_gate_up), _ptr(out), dtype_code(out.dtype), M, I, K, x.stride(0),
          w_gate_up.stride(0), out.stride(0), error_flag().data_ptr(), _stream())
    return out


def paged_attention(q: torch.Tensor, q_stride: int, out: torch.Tensor, pages: torch.Tensor,
                    block_tables: torch.Tensor, q_start: torch.Tensor, ctx_len: torch.Tensor,
                    tile_req: torch.Tensor, tile_tok0: torch.Tensor, num_heads: int, num_kv_heads: int,
                    head_dim: int, page_size: int, window: int, scale: float, tokens_per_tile: int,
                    tile_seg: Optional[torch.Tensor] = None, tile_slot: Optional[torch.Tensor] = None,
                    places: int = 0) -> torch.Tensor:
    """Causal attention of the step's query rows over the paged keys and values (any portion sizes).
    ``tokens_per_tile`` is the step the tile list was built with (``tokens_per_attention_tile``).
    With ``tile_seg`` the list holds items that share the keys of a tile (see ``attention_max_segments``): item i is
    number ``tile_seg[i] & 255`` of ``tile_seg[i] >> 8`` consecutive items of its tile, and ``tile_slot[i]`` is the
    first of the tile's ``places`` (one per item) for their sums."""
    for name, t in (("block_tables", block_tables), ("q_start", q_start), ("ctx_len", ctx_len),
                    ("tile_req", tile_req), ("tile_tok0", tile_tok0)):
        _i32(t, name)
    _need(q.dtype == pages.dtype == out.dtype, "q, pages and out must have one type")
    _need(out.is_contiguous() and out.shape[1] == num_heads * head_dim, "attention output must be [tokens, heads * head_dim]")
    _need(pages.is_contiguous() and tuple(pages.shape[1:]) == (2, num_kv_heads, page_size, head_dim),
          "pages have the wrong layout")
    seg = slot = partials = counters = None
    if tile_seg is not None:
        _i32(tile_seg, "tile_seg")
        _i32(tile_slot, "tile_slot")
        _need(tile_seg.numel() == tile_req.numel() == tile_slot.numel() and 0 < places <= ATTENTION_MAX_PLACES,
              "tile_seg and tile_slot must have an entry per item, and the places a count within bounds")
        partials = torch.empty(places * num_kv_heads * attention_place_floats(), dtype=torch.float32, device=q.device)
        counters = attention_counters(q.device, places * num_kv_heads)
        seg, slot = tile_seg, tile_slot
    _call("llmp_paged_attention", _ptr(q), int(q_stride), _ptr(out), out.stride(0), _ptr(pages), pages.shape[0],
          dtype_code(q.dtype), _ptr(block_tables), block_tables.stride(0), _ptr(q_start), _ptr(ctx_len),
          _ptr(tile_req), _ptr(tile_tok0), _ptr(seg), _ptr(slot), _ptr(partials), _ptr(counters), tile_req.numel(),
          num_heads, num_kv_heads, head_dim, page_size, int(window), float(scale), int(tokens_per_tile),
          error_flag().data_ptr(), _stream())
    return out


def decode_scratch_floats(rows: int, num_heads: int, head_dim: int, max_ctx: int) -> int:
    fn = library().llmp_decode_scratch_floats
    fn.argtypes = [_I, _I, _I, _I]
    fn.restype = _L
    return int(fn(rows, num_heads, head_dim, max_ctx))


_decode_counters: dict = {}
DECODE_RANGE = 128                   # keys per fixed range of the decode attention kernels
DECODE_MAX_KEYS = 1024 * DECODE_RANGE   # the longest context the decode attention kernels take
_DECODE_LIST = os.environ.get("LLMP_B200_DECODE_LIST", "")


_sm_count: Optional[int] = None


def sm_count() -> int:
    global _sm_count
    if _sm_count is None:
        _sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _sm_count


def decode_prefers_list(longest: int, total: int, rows: int, num_kv_heads: int, sms: Optional[int] = None) -> bool:
    """Whether a decode step over ``rows`` requests that see ``total`` keys together, the longest ``longest``, is
    better served by the kernel that deals the key ranges of all requests out evenly over the SMs than by the one
    that gives every (request, key/value head) pair blocks of its own. The latter walks as many keys per block as
    the longest request needs with the up to 8 blocks a pair can get; the former the average, plus the adding up of
    shared sums through global memory (worth about a thousand keys of reading). Also with many more pairs than SMs:
    whole pairs per block then leave SMs idle in the last round (Qwen3-8B heads, 2,048 keys each: from 64 requests on)."""
    sms = sms or sm_count()
    pairs = rows * num_kv_heads
    if pairs > 2 * sms:
        return True
    blocks = 1
    while blocks < 8 and pairs * blocks * 2 <= sms:
        blocks *= 2
    own = longest * -(-pairs // sms) / blocks
    even = total * num_kv_heads / sms
    return own > 1.25 * even + 1024


def decode_counters(device: torch.device) -> torch.Tensor:
    """The counters with which the blocks of the streaming decode kernel that share a long request find out who
    finishes last. Every launch leaves them zero. One set per device: decode launches on a device must follow one
    another (one stream, or streams ordered by events), as they do in the engine. They are made outside a graph
    capture (the engine runs every shape once before it captures it)."""
    key = torch.device(device).index or 0
    counters = _decode_counters.get(key)
    if counters is None:
        _need(not torch.cuda.is_current_stream_capturing(), "decode counters must exist before a graph is captured")
        fn = library().llmp_decode_counters
        fn.argtypes = []
        fn.restype = _I
        counters = _decode_counters[key] = torch.zeros(int(fn()), dtype=torch.int32, device=device)
    return counters


def decode_attention(q: torch.Tensor, q_stride: int, out: torch.Tensor, pages: torch.Tensor,
                     block_tables: torch.Tensor, ctx_len: torch.Tensor, max_ctx: int, num_heads: int,
                     num_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float,
                     scratch: Optional[torch.Tensor] = None, uneven: bool = False) -> torch.Tensor:
    """Attention of one query row per request (row r belongs to request r, at position ctx_len[r] - 1)
    over the request's pages; keys are split into fixed ranges whose partial results go through
    ``scratch`` (float32, at least ``decode_scratch_floats(...)`` entries; allocated when None).
    ``uneven`` (see ``decode_prefers_list``) picks, where there is a choice, the kernel that deals the key ranges of
    all requests out evenly over the SMs instead of giving every request blocks of its own; the result is the same
    beyond rounding. ``LLMP_B200_DECODE_LIST=0`` or ``1`` overrides it."""
    if _DECODE_LIST in ("0", "1"):
        uneven = _DECODE_LIST == "1"
    _i32(block_tables, "block_tables")
    _i32(ctx_len, "ctx_len")
    R = ctx_len.numel()
    _need(q.dtype == pages.dtype == out.dtype, "q, pages and out must have one type")
    _need(out.is_contiguous() and out.shape == (R, num_heads * head_dim), "decode output must be [requests, heads * head_dim]")
    _need(pages.is_contiguous() and tuple(pages.shape[1:]) == (2, num_kv_heads, page_size, head_dim),
          "pages have the wrong layout")
    need = decode_scratch_floats(R, num_heads, head_dim, max_ctx)
    if scratch is None:
        scratch = torch.empty(need, dtype=torch.float32, device=q.device)
    _need(scratch.dtype == torch.float32 and scratch.is_contiguous() and scratch.numel() >= need,
          f"decode scratch must hold {need} float32 values")
    _call("llmp_decode_attention", _ptr(q), int(q_stride), _ptr(out), out.stride(0), _ptr(pages), pages.shape[0],
          dtype_code(q.dtype), _ptr(block_tables), block_tables.stride(0), _ptr(ctx_len), R, int(max_ctx), num_heads,
          num_kv_heads, head_dim, page_size, int(window), float(scale), _ptr(scratch), scratch.numel(),
          _ptr(decode_counters(q.device)), int(bool(uneven)), error_flag().data_ptr(), _stream())
    return out


def argmax(logits: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "logits must be float32 rows")
    _i32(out, "out")
    scratch = torch.empty(logits.shape[0] * 64, dtype=torch.int32, device=logits.device)   # slices' best values and indices
    _call("llmp_argmax", _ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1], _ptr(out), _ptr(scratch),
          _stream())
    return out


def repetition_penalty(logits: torch.Tensor, tokens: torch.Tensor, offsets: torch.Tensor, penalty: torch.Tensor) -> None:
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "logits must be float32 rows")
    _i32(tokens, "tokens")
    _i32(offsets, "offsets")
    _need(penalty.dtype == torch.float32 and penalty.numel() == logits.shape[0], "one penalty per row")
    _call("llmp_repetition_penalty", _ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1], _ptr(tokens),
          _ptr(offsets), _ptr(penalty), _stream())


def entropy(logits: torch.Tensor, temperature: float) -> torch.Tensor:
    """Entropy in nats of softmax(logits / temperature) for every row of float32 ``logits [rows, vocab]`` (the logits
    as they are when ``temperature`` is not positive); float32 ``[rows]``."""
    _need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1, "logits must be float32 rows")
    out = torch.empty(logits.shape[0], dtype=torch.float32, device=logits.device)
    _call("llmp_entropy", _ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1], float(temperature), _ptr(out),
          _stream())
    return out


def sample(logits: torch.Tensor, params: torch.Tensor, out: torch.Tensor, out_u: Optional[torch.Tensor] = None) -> torch.Tensor:
    """params: int32 [M, 8] rows {temperature, top_k, top_p, min_p, typical_p, seed low, seed high, step}
    with the float fields stored by bit pattern."""
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "logits must be float32 rows")
    _need(params.dtype == torch.int32 and params.is_contiguous() and params.shape == (logits.shape[0], 8),
          "sampling parameters must be int32 [rows, 8]")
    _i32(out, "out")
    _call("llmp_sample", _ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1], _ptr(params), _ptr(out),
          _ptr(out_u), _stream())
    return out


# ---- parts beyond the dense pre-norm decoder: norms around a sublayer, depth mixing, recurrent and latent mixers, experts ----
def gemm_batched(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[b, m, :] = a[b, m, :] @ w[b]^T for a [B, M, K], w [B, N, K], out [B, M, N] on the CUDA cores with float32 sums.
    Any of the three may be a view whose batches and rows lie apart (the heads of a [tokens, heads, size] tensor
    transposed to [heads, tokens, size]); only the last axis must be dense."""
    B, M, K = a.shape
    N = w.shape[1]
    _need(w.shape == (B, N, K) and out.shape == (B, M, N), "batched gemm shapes do not match")
    _need(a.dtype == w.dtype and a.stride(2) == 1 and w.stride(2) == 1 and out.stride(2) == 1,
          "batched gemm operands must have one type and a dense last axis")
    _call("llmp_gemm_simt_batched", _ptr(a), _ptr(w), _ptr(out), dtype_code(a.dtype), dtype_code(out.dtype), B, M, N, K,
          a.stride(1), w.stride(1), out.stride(1), a.stride(0), w.stride(0), out.stride(0), _stream())
    return out


def embedding_norm(ids: torch.Tensor, table: torch.Tensor, weight: torch.Tensor, offset: float, eps: float,
                   out: torch.Tensor) -> torch.Tensor:
    """out[n] = rms_norm(table[ids[n]]) * (offset + weight), float32."""
    _i32(ids, "ids")
    _need(table.dim() == 2 and table.is_contiguous(), "embedding table must be a contiguous matrix")
    _need(out.dtype == torch.float32 and out.is_contiguous() and out.shape == (ids.numel(), table.shape[1]),
          "embedding output must be float32 [tokens, hidden]")
    _need(weight.numel() == table.shape[1] and weight.is_contiguous(), "norm weight has the wrong size")
    _call("llmp_embedding_norm", _ptr(ids), _ptr(table), dtype_code(table.dtype), _ptr(weight), dtype_code(weight.dtype),
          float(offset), float(eps), _ptr(out), ids.numel(), table.shape[1], table.shape[0], _stream())
    return out


def add_norm_mix(residual: torch.Tensor, *, delta: Optional[torch.Tensor] = None, delta_weight: Optional[torch.Tensor] = None,
                 delta_offset: float = 0.0, delta_eps: float = 0.0, history: Optional[torch.Tensor] = None,
                 mix: Optional[torch.Tensor] = None, index: int = 0, weight: Optional[torch.Tensor] = None, offset: float = 0.0,
                 eps: float = 0.0, out: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """The residual stream's norm kernel in its general form, per row r (``rows`` selects rows and leaves the stream as it is):
    y = delta[r], normed by (delta_offset + delta_weight) if that is given; x = residual[r] + y; with ``history``
    [slots, tokens, width]: history[index][r] = x and x = sum_{j <= index} mix[j] history[j][r]; residual[r] = x;
    out = rms_norm(x) * (offset + weight) if ``out`` is given."""
    T, H = residual.shape
    _need(residual.dtype == torch.float32 and residual.is_contiguous(), "residual must be a contiguous float32 matrix")
    M = rows.numel() if rows is not None else T
    if delta is not None:
        _need(delta.is_contiguous() and delta.shape == residual.shape, "delta must match the residual's shape")
    if delta_weight is not None:
        _need(delta_weight.numel() == H and delta_weight.is_contiguous(), "the addend's norm weight has the wrong size")
    if history is not None:
        _need(history.dtype == torch.float32 and history.is_contiguous() and history.dim() == 3 and
              tuple(history.shape[1:]) == (T, H) and 0 <= index < history.shape[0], "history must be float32 [slots, tokens, width]")
        _need(mix is not None and mix.dtype == torch.float32 and mix.is_contiguous() and mix.numel() >= index + 1,
              "mixing weights must be float32, one per result so far")
    if out is not None:
        _need(out.is_contiguous() and out.shape == (M, H) and weight is not None and weight.numel() == H and weight.is_contiguous(),
              "norm output or weight has the wrong shape")
    if rows is not None:
        _i32(rows, "rows")
    _call("llmp_add_norm_mix", _ptr(residual), _ptr(delta), dtype_code(delta.dtype) if delta is not None else F32,
          _ptr(delta_weight), dtype_code(delta_weight.dtype) if delta_weight is not None else F32, float(delta_offset),
          float(delta_eps), _ptr(history), T * H, _ptr(mix), int(index), _ptr(weight),
          dtype_code(weight.dtype) if weight is not None else F32, float(offset), float(eps), _ptr(out),
          dtype_code(out.dtype) if out is not None else F32, _ptr(rows), M, H, _stream())
    return out


def poly_norm(z: torch.Tensor, act: torch.Tensor, eps: float, out: torch.Tensor) -> torch.Tensor:
    """out = a N(z) + b N(z^2) + c N(z^3) + e per row, N(v) = v / sqrt(mean(v^2) + eps); ``act`` = float32 (a, b, c, e)."""
    N, F = z.shape
    _need(z.stride(1) == 1 and out.is_contiguous() and out.shape == (N, F), "poly_norm shapes do not match")
    _need(act.dtype == torch.float32 and act.numel() == 4 and act.is_contiguous(), "poly_norm takes four float32 coefficients")
    _call("llmp_poly_norm", _ptr(z), dtype_code(z.dtype), z.stride(0), _ptr(act), float(eps), _ptr(out), dtype_code(out.dtype),
          N, F, _stream())
    return out


def softcap(logits: torch.Tensor, cap: float) -> torch.Tensor:
    """In place: logits = cap * tanh(logits / cap)."""
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "softcap takes contiguous float32 logits")
    _call("llmp_softcap", _ptr(logits), logits.numel(), float(cap), _stream())
    return logits


_gru_chunk: Optional[int] = None


def min_gru_chunk() -> int:
    """Tokens per chunk of the parallel form of ``min_gru``; portions longer than this need scratch."""
    global _gru_chunk
    if _gru_chunk is None:
        fn = library().llmp_min_gru_chunk
        fn.argtypes = []
        fn.restype = _I
        _gru_chunk = int(fn())
    return _gru_chunk


def min_gru(p: torch.Tensor, bias: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor, positions: torch.Tensor,
            state: torch.Tensor, out: torch.Tensor, max_q_len: int) -> torch.Tensor:
    """The minGRU recurrence over the step's tokens. ``p`` float32 [tokens, 3 W] (gate, candidate and output-gate
    products), ``bias`` float32 [2 W], ``state`` float32 [slots, 2, W] (see csrc/min_gru.cu), ``out`` [tokens, W]."""
    N, three_w = p.shape
    W = three_w // 3
    R = slots.numel()
    _need(p.dtype == torch.float32 and p.is_contiguous() and three_w == 3 * W, "min_gru takes float32 products [tokens, 3 W]")
    _need(bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == 2 * W, "min_gru takes float32 biases [2 W]")
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (2, W), "min_gru state must be float32 [slots, 2, W]")
    _need(out.is_contiguous() and out.shape == (N, W), "min_gru output has the wrong shape")
    for t, name in ((q_start, "q_start"), (slots, "slots"), (positions, "positions")):
        _i32(t, name)
    scratch = None
    chunk = min_gru_chunk()
    if max_q_len > chunk:
        scratch = torch.empty((3, R, -(-max_q_len // chunk), W), dtype=torch.float32, device=p.device)
    _call("llmp_min_gru", _ptr(p), _ptr(bias), _ptr(q_start), _ptr(slots), _ptr(positions), _ptr(state), _ptr(out),
          dtype_code(out.dtype), _ptr(scratch), R, W, int(max_q_len), _stream())
    return out


def latent_kv_post(qd: torch.Tensor, num_heads: int, dim: int, rot: int, rank: int, norm_weight: torch.Tensor, eps: float,
                   cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rot_dims: int, slots: Optional[torch.Tensor],
                   pages: Optional[torch.Tensor]) -> None:
    """In place on ``qd`` [tokens, heads (dim + rot) + rank + rot]: every head's last ``rot`` query entries are rotated;
    the row's last rank + rot entries become a cache row (the first ``rank`` RMS-normed with ``norm_weight``, the rest
    rotated) written to the token's slot of ``pages`` [pages, page_size, rank + rot]."""
    N = qd.shape[0]
    _need(qd.stride(1) == 1 and qd.shape[1] == num_heads * (dim + rot) + rank + rot, "latent_kv_post: the product has the wrong width")
    _need(norm_weight.numel() == rank and norm_weight.is_contiguous(), "latent norm weight has the wrong size")
    if rot_dims:
        _need(cos is not None and sin is not None and cos.shape == (N, rot_dims // 2) and cos.dtype == torch.float32 and
              cos.is_contiguous() and sin.is_contiguous(), "rotary tables must be float32 [tokens, rotated / 2]")
    if pages is not None:
        _need(pages.dtype == qd.dtype and pages.is_contiguous() and pages.shape[2] == rank + rot and slots is not None,
              "latent pages have the wrong layout")
        _i32(slots, "slots")
    _call("llmp_latent_kv_post", _ptr(qd), dtype_code(qd.dtype), qd.stride(0), num_heads, dim, rot, rank, _ptr(norm_weight),
          dtype_code(norm_weight.dtype), float(eps), _ptr(cos), _ptr(sin), int(rot_dims), _ptr(slots) if pages is not None else None,
          _ptr(pages), N, _stream())


def latent_attention(q_lat: torch.Tensor, q_rot: torch.Tensor, pages: torch.Tensor, tables: torch.Tensor,
                     token_request: torch.Tensor, positions: torch.Tensor, out: torch.Tensor, scale: float,
                     sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of rows (token, head) over latent cache rows. ``q_lat`` [tokens, heads, rank] and ``q_rot``
    [tokens, heads, rot] (views with a dense last axis), ``pages`` [pages, page_size, rank + rot], ``out`` [tokens,
    heads, rank]: the softmax-weighted sum of the visible rows' first ``rank`` entries. ``sink`` (float32 [heads]): exp(sink)
    joins each head's denominator."""
    _sink(sink, q_lat.shape[1])
    N, H, rank = q_lat.shape
    rot = q_rot.shape[2]
    _need(q_rot.shape[:2] == (N, H) and out.shape == (N, H, rank), "latent attention shapes do not match")
    _need(q_lat.stride(2) == 1 and (rot == 0 or q_rot.stride(2) == 1) and out.stride(2) == 1, "latent attention needs dense last axes")
    _need(q_lat.dtype == pages.dtype == out.dtype == q_rot.dtype, "latent attention operands must have one type")
    _need(pages.is_contiguous() and pages.dim() == 3 and pages.shape[2] == rank + rot, "latent pages have the wrong layout")
    _i32(tables, "tables"); _i32(token_request, "token_request"); _i32(positions, "positions")
    _call("llmp_latent_attention", _ptr(q_lat), q_lat.stride(0), q_lat.stride(1), _ptr(q_rot), q_rot.stride(0), q_rot.stride(1),
          _ptr(pages), dtype_code(pages.dtype), _ptr(tables), tables.shape[1], _ptr(token_request), _ptr(positions), _ptr(out),
          out.stride(0), out.stride(1), N, H, rank, rot, pages.shape[1], float(scale), _ptr(sink), _stream())
    return out


def _sink(sink: Optional[torch.Tensor], heads: int) -> None:
    _need(sink is None or (sink.dtype == torch.float32 and sink.numel() == heads and sink.is_contiguous()),
          "a sink is one float32 number per head")


def route_topk(h: torch.Tensor, w_router: torch.Tensor, top: int, ids: torch.Tensor, weights: torch.Tensor, *,
               softmax: bool = False, correction: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None) -> None:
    """ids[n, :], weights[n, :] = the ``top`` router outputs with the largest score (+ ``correction``, if given) and their
    scores without the correction; float32 logits. The score is sigmoid(logit), or with ``softmax`` the softmax over all
    router outputs. With ``gate`` (float32 [tokens]) the matrix has one row more than router outputs, and
    gate[n] = sigmoid(that row . h[n])."""
    N, Hd = h.shape
    E = w_router.shape[0] - (1 if gate is not None else 0)
    _need(h.is_contiguous() and w_router.dtype == torch.float32 and w_router.is_contiguous() and w_router.shape[1] == Hd,
          "the router matrix must be float32 [experts, width]")
    _need(ids.dtype == torch.int32 and ids.is_contiguous() and ids.shape == (N, top) and weights.dtype == torch.float32 and
          weights.is_contiguous() and weights.shape == (N, top), "route_topk outputs must be int32 and float32 [tokens, top]")
    if correction is not None:
        _need(correction.dtype == torch.float32 and correction.is_contiguous() and correction.numel() == E,
              "the router's correction must be float32 [router outputs]")
    if gate is not None:
        _need(gate.dtype == torch.float32 and gate.is_contiguous() and gate.numel() == N, "the gate must be float32 [tokens]")
    _call("llmp_route_topk", _ptr(h), dtype_code(h.dtype), _ptr(w_router), int(top), _ptr(ids), _ptr(weights), N, Hd, E,
          1 if softmax else 0, _ptr(correction), _ptr(gate), _stream())


EXPERT_FORMS = {"clamped": 0, "silu": 1}     # csrc/routed_experts.cu: expert_act


def expert_rows(h: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
                limit: float, out: torch.Tensor, form: str = "clamped") -> torch.Tensor:
    """out[n] = sum_k Wd[e] act(Wg[e] h[n], Wu[e] h[n], weights[n, k]) with e = ids[n, k], float32; ``form`` names the
    activation and where the weight enters (``EXPERT_FORMS``); an id from the number of experts on adds weights[n, k] h[n].
    ``w_gate_up`` [experts, 2 ff, width] (gate rows, then up rows), ``w_down`` [experts, width, ff]. Reads an expert once
    per token that chose it: for the few rows of a decode step."""
    N, Hd = h.shape
    E, two_f, _ = w_gate_up.shape
    F = two_f // 2
    top = ids.shape[1]
    _need(h.is_contiguous() and w_gate_up.is_contiguous() and w_down.is_contiguous() and w_gate_up.shape == (E, 2 * F, Hd) and
          w_down.shape == (E, Hd, F) and h.dtype == w_gate_up.dtype == w_down.dtype, "expert matrices have the wrong layout")
    _need(out.dtype == torch.float32 and out.is_contiguous() and out.shape == (N, Hd), "expert output must be float32 [tokens, width]")
    y = torch.empty((N * top, F), dtype=h.dtype, device=h.device)
    _call("llmp_expert_rows", _ptr(h), _ptr(w_gate_up), _ptr(w_down), dtype_code(h.dtype), _ptr(ids), _ptr(weights), float(limit),
          _ptr(y), _ptr(out), N, top, Hd, F, EXPERT_FORMS[form], E, _stream())
    return out


EXPERT_GROUPED_MIN_ROWS = 33         # (token, choice) pairs from which a step's experts run as grouped products


def expert_grouped_supports(dtype: torch.dtype, Hd: int, F: int) -> bool:
    if dtype != torch.bfloat16:
        return False
    fn = library().llmp_expert_grouped_supports
    fn.argtypes = [_I, _I]
    fn.restype = _I
    return bool(fn(Hd, F))


def expert_grouped(h: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
                   limit: float, out: torch.Tensor, form: str = "clamped", identity: int = 0) -> torch.Tensor:
    """``expert_rows`` for many rows (bfloat16): the pairs are sorted by expert on the device and the experts' products
    run as grouped tensor-core products that read an expert's rows once per 64 pairs."""
    N, Hd = h.shape
    E, two_f, _ = w_gate_up.shape
    F = two_f // 2
    top = ids.shape[1]
    _need(h.is_contiguous() and w_gate_up.is_contiguous() and w_down.is_contiguous() and w_gate_up.shape == (E, 2 * F, Hd) and
          w_down.shape == (E, Hd, F) and h.dtype == w_gate_up.dtype == w_down.dtype == torch.bfloat16, "expert matrices have the wrong layout")
    _need(out.dtype == torch.float32 and out.is_contiguous() and out.shape == (N, Hd), "expert output must be float32 [tokens, width]")
    fn = library().llmp_expert_grouped_rows
    fn.argtypes = [_I, _I]
    fn.restype = _L
    rows = int(fn(N * top, E))
    ints = torch.empty(3 * E + 1 + 2 * (rows // 64) + rows, dtype=torch.int32, device=h.device)
    y = torch.empty((rows, F), dtype=torch.bfloat16, device=h.device)
    pair_out = torch.empty((N * top, Hd), dtype=torch.float32, device=h.device) if top > 1 or identity else None
    _call("llmp_expert_grouped", _ptr(h), _ptr(w_gate_up), _ptr(w_down), _ptr(ids), _ptr(weights), float(limit), _ptr(ints), _ptr(y),
          _ptr(pair_out), _ptr(out), N, top, Hd, F, E, EXPERT_FORMS[form], int(identity), _stream())
    return out


def routed_experts(h: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
                   limit: float, out: torch.Tensor, form: str = "clamped", identity: int = 0) -> torch.Tensor:
    """The experts' work for a step's rows, by the kernel that suits their number: grouped tensor-core products for many
    bfloat16 rows, a warp per output entry (``expert_rows``) for the few rows of a decode step and for float32."""
    pairs = ids.numel()
    if pairs >= EXPERT_GROUPED_MIN_ROWS and expert_grouped_supports(h.dtype, h.shape[1], w_down.shape[2]):
        return expert_grouped(h, w_gate_up, w_down, ids, weights, limit, out, form, identity)
    return expert_rows(h, w_gate_up, w_down, ids, weights, limit, out, form)


LATENT_SEGMENT_KEYS = 256            # keys per segment when a step's rows are too few to fill the GPU (a multiple of the key tile)


def latent_mma_supports(dtype: torch.dtype, rank: int, rot: int, page_size: int) -> bool:
    """Whether the tensor-core latent attention kernel serves these sizes (bfloat16, sizes in multiples of 16)."""
    if dtype != torch.bfloat16:
        return False
    fn = library().llmp_latent_mma_supports
    fn.argtypes = [_I, _I, _I]
    fn.restype = _I
    return bool(fn(rank, rot, page_size))


def latent_mma_tokens_per_tile(num_heads: int) -> int:
    fn = library().llmp_latent_mma_tokens_per_tile
    fn.argtypes = [_I]
    fn.restype = _I
    return int(fn(num_heads))


def latent_attention_mma(q_lat: torch.Tensor, q_rot: torch.Tensor, pages: torch.Tensor, tables: torch.Tensor, q_start: torch.Tensor,
                         ctx_len: torch.Tensor, positions: torch.Tensor, tile_req: torch.Tensor, tile_tok0: torch.Tensor,
                         out: torch.Tensor, scale: float, segments: int = 0, sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``latent_attention`` on the tensor cores for bfloat16. ``tile_req``/``tile_tok0``: the work list (request and
    first token of every tile of ``latent_mma_tokens_per_tile`` tokens). ``segments`` > 0: the keys are cut into that many
    segments of ``LATENT_SEGMENT_KEYS``, each with blocks of its own, and a second kernel adds them up (for steps of few
    rows over long contexts; ``segments`` must cover the longest context)."""
    N, H, rank = q_lat.shape
    rot = q_rot.shape[2]
    _sink(sink, H)
    _need(q_lat.dtype == torch.bfloat16 and q_rot.dtype == torch.bfloat16 and pages.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
          "latent_attention_mma takes bfloat16")
    _need(q_rot.shape[:2] == (N, H) and out.shape == (N, H, rank) and q_lat.stride(2) == 1 and out.stride(2) == 1 and
          (rot == 0 or q_rot.stride(2) == 1), "latent attention shapes do not match")
    _need(pages.is_contiguous() and pages.dim() == 3 and pages.shape[2] == rank + rot, "latent pages have the wrong layout")
    for t, name in ((tables, "tables"), (q_start, "q_start"), (ctx_len, "ctx_len"), (positions, "positions"), (tile_req, "tile_req"),
                    (tile_tok0, "tile_tok0")):
        _i32(t, name)
    scratch = None
    if segments > 0:
        scratch = torch.empty(segments * N * H * (rank + 2), dtype=torch.float32, device=q_lat.device)
    _call("llmp_latent_attention_mma", _ptr(q_lat), q_lat.stride(0), q_lat.stride(1), _ptr(q_rot), q_rot.stride(0), q_rot.stride(1),
          _ptr(pages), _ptr(tables), tables.shape[1], _ptr(q_start), _ptr(ctx_len), _ptr(positions), _ptr(tile_req), _ptr(tile_tok0),
          tile_req.numel(), _ptr(out), out.stride(0), out.stride(1), N, H, rank, rot, pages.shape[1], float(scale),
          LATENT_SEGMENT_KEYS if segments > 0 else 0, int(segments), _ptr(scratch), _ptr(sink), _stream())
    return out


def add_layernorm(residual: torch.Tensor, delta: Optional[torch.Tensor], delta2: Optional[torch.Tensor], weight: torch.Tensor,
                  bias: torch.Tensor, eps: float, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """residual += delta + delta2 (float32, in place; either may be None), then out = layer norm of the rows with ``weight``
    and ``bias`` (variance = mean of the squared deviations), float32 statistics. With ``rows`` only those rows are normed
    into ``out`` and the residual is left as it is."""
    R, H = residual.shape
    _need(residual.dtype == torch.float32 and residual.is_contiguous(), "the residual must be contiguous float32")
    for d in (delta, delta2):
        if d is not None:
            _need(d.shape == residual.shape and d.is_contiguous(), "an addend must have the residual's shape")
            dtype_code(d.dtype)
    _need(weight.numel() == H and bias.numel() == H and weight.dtype == bias.dtype and weight.is_contiguous() and bias.is_contiguous(),
          "layer norm weight and bias must have the row's length and one type")
    count = R
    if rows is not None:
        _i32(rows, "rows")
        count = rows.numel()
    _need(out.shape == (count, H) and out.is_contiguous(), "layer norm output has the wrong shape")
    _call("llmp_add_layernorm", _ptr(residual), _ptr(delta), dtype_code(delta.dtype) if delta is not None else F32, _ptr(delta2),
          dtype_code(delta2.dtype) if delta2 is not None else F32, _ptr(weight), _ptr(bias), dtype_code(weight.dtype), float(eps),
          _ptr(out), dtype_code(out.dtype), count, H, _ptr(rows), _stream())
    return out


def relu_squared(z: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out = max(z, 0)^2"""
    _need(z.is_contiguous() and out.is_contiguous() and z.shape == out.shape and z.dtype == out.dtype, "relu_squared shapes do not match")
    _call("llmp_relu_squared", _ptr(z), _ptr(out), dtype_code(z.dtype), z.numel(), _stream())
    return out


def add_scaled_rows(out: torch.Tensor, x: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """out[n, :] += scales[n] * x[n, :] (float32 ``out`` and ``scales``)."""
    N, H = out.shape
    _need(out.dtype == torch.float32 and out.is_contiguous() and x.shape == out.shape and x.is_contiguous() and
          scales.dtype == torch.float32 and scales.is_contiguous() and scales.numel() == N, "add_scaled_rows shapes do not match")
    _call("llmp_add_scaled_rows", _ptr(out), _ptr(x), dtype_code(x.dtype), _ptr(scales), N, H, _stream())
    return out


def diff_qkv_post(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, dim: int, vdim: int, q_weight: torch.Tensor,
                  k_weight: torch.Tensor, eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary_dim: int,
                  slots: Optional[torch.Tensor], pages: Optional[torch.Tensor]) -> None:
    """In place on ``qkv`` [tokens, heads 2 dim | kv_heads 2 dim | kv_heads vdim] (two maps per head): every run of ``dim``
    entries of q and k is RMS-normed with ``q_weight`` / ``k_weight`` and its first ``rotary_dim`` entries rotated; q stays
    in place, k and v go to the token's slot of ``pages`` [pages, kv_heads, page_size, 2 dim + vdim]."""
    N = qkv.shape[0]
    _need(qkv.stride(1) == 1 and qkv.shape[1] == 2 * dim * (num_heads + num_kv_heads) + num_kv_heads * vdim,
          "diff_qkv_post: the product has the wrong width")
    _need(q_weight.numel() == dim and k_weight.numel() == dim and q_weight.dtype == k_weight.dtype and q_weight.is_contiguous() and
          k_weight.is_contiguous(), "q/k norm weights must have the key size and one type")
    if rotary_dim:
        _need(cos is not None and sin is not None and cos.shape == (N, rotary_dim // 2) and cos.dtype == torch.float32 and
              cos.is_contiguous() and sin.is_contiguous(), "rotary tables must be float32 [tokens, rotated / 2]")
    page_size = 0
    if pages is not None:
        _need(pages.dtype == qkv.dtype and pages.is_contiguous() and pages.dim() == 4 and pages.shape[1] == num_kv_heads and
              pages.shape[3] == 2 * dim + vdim and slots is not None, "differential attention pages have the wrong layout")
        _i32(slots, "slots")
        page_size = pages.shape[2]
    _call("llmp_diff_qkv_post", _ptr(qkv), dtype_code(qkv.dtype), qkv.stride(0), num_heads, num_kv_heads, dim, vdim, _ptr(q_weight),
          _ptr(k_weight), dtype_code(q_weight.dtype), float(eps), _ptr(cos), _ptr(sin), int(rotary_dim),
          _ptr(slots) if pages is not None else None, _ptr(pages), page_size, N, _stream())


def diff_attention(q: torch.Tensor, pages: torch.Tensor, tables: torch.Tensor, token_request: torch.Tensor, positions: torch.Tensor,
                   out: torch.Tensor, num_heads: int, num_kv_heads: int, dim: int, vdim: int, window: int, scale: float, lam: float,
                   eps: float, out_scale: float) -> torch.Tensor:
    """Differential attention of rows (token, head), any sizes, float32 or bfloat16: ``q`` [tokens, >= heads 2 dim] (a view
    with a dense last axis; head h's two queries at h 2 dim), ``pages`` [pages, kv_heads, page_size, 2 dim + vdim], ``out``
    [tokens, heads vdim] = rms_norm(a1 - lam a2) * out_scale per head, with a1, a2 the two maps' softmax-weighted sums of
    the values; ``window`` > 0: a token sees itself and the window - 1 tokens before it."""
    N = q.shape[0]
    _need(q.stride(1) == 1 and q.shape[1] >= 2 * dim * num_heads and out.shape == (N, num_heads * vdim) and out.stride(1) == 1,
          "differential attention shapes do not match")
    _need(q.dtype == pages.dtype == out.dtype, "differential attention operands must have one type")
    _need(pages.is_contiguous() and pages.dim() == 4 and pages.shape[1] == num_kv_heads and pages.shape[3] == 2 * dim + vdim,
          "differential attention pages have the wrong layout")
    _i32(tables, "tables"); _i32(token_request, "token_request"); _i32(positions, "positions")
    _call("llmp_diff_attention", _ptr(q), q.stride(0), _ptr(pages), dtype_code(pages.dtype), _ptr(tables), tables.shape[1],
          _ptr(token_request), _ptr(positions), _ptr(out), out.stride(0), N, num_heads, num_kv_heads, dim, vdim, pages.shape[2],
          int(window), float(scale), float(lam), float(eps), float(out_scale), _stream())
    return out


DIFF_SEGMENT_KEYS = 256              # keys per segment when a step's rows are too few to fill the GPU (a multiple of the key tile)


def diff_mma_supports(dtype: torch.dtype, dim: int, vdim: int, page_size: int) -> bool:
    """Whether the tensor-core differential attention kernel serves these sizes (bfloat16)."""
    if dtype != torch.bfloat16:
        return False
    fn = library().llmp_diff_mma_supports
    fn.argtypes = [_I, _I, _I]
    fn.restype = _I
    return bool(fn(dim, vdim, page_size))


def diff_mma_tokens_per_tile(num_heads: int, num_kv_heads: int) -> int:
    fn = library().llmp_diff_mma_tokens_per_tile
    fn.argtypes = [_I, _I]
    fn.restype = _I
    return int(fn(num_heads, num_kv_heads))


def diff_attention_mma(q: torch.Tensor, pages: torch.Tensor, tables: torch.Tensor, q_start: torch.Tensor, ctx_len: torch.Tensor,
                       positions: torch.Tensor, tile_req: torch.Tensor, tile_tok0: torch.Tensor, out: torch.Tensor, num_heads: int,
                       num_kv_heads: int, dim: int, vdim: int, window: int, scale: float, lam: float, eps: float, out_scale: float,
                       segments: int = 0, split: bool = False) -> torch.Tensor:
    """``diff_attention`` on the tensor cores for bfloat16. ``tile_req``/``tile_tok0``: the work list (request and first
    token of every tile of ``diff_mma_tokens_per_tile`` tokens). ``segments`` > 0: the keys are cut into that many segments
    of ``DIFF_SEGMENT_KEYS`` with blocks of their own, and the block of a tile that ends last adds them up (steps of few rows over many keys;
    ``segments`` must cover the longest context). ``split`` (with segments, every tile one token): the four warps of a
    block share a key tile (half of its keys and one map each) instead of three of them idling."""
    N = q.shape[0]
    _need(q.dtype == torch.bfloat16 and pages.dtype == torch.bfloat16 and out.dtype == torch.bfloat16, "diff_attention_mma takes bfloat16")
    _need(q.stride(1) == 1 and q.shape[1] >= 2 * dim * num_heads and out.shape == (N, num_heads * vdim) and out.stride(1) == 1,
          "differential attention shapes do not match")
    _need(pages.is_contiguous() and pages.dim() == 4 and pages.shape[1] == num_kv_heads and pages.shape[3] == 2 * dim + vdim,
          "differential attention pages have the wrong layout")
    for t, name in ((tables, "tables"), (q_start, "q_start"), (ctx_len, "ctx_len"), (positions, "positions"), (tile_req, "tile_req"),
                    (tile_tok0, "tile_tok0")):
        _i32(t, name)
    scratch = None
    # at most one counter per (tile, kv head, chunk of heads); asked for in every call, so that they exist before a step is
    # captured whose eager run needed no segments
    counters = attention_counters(q.device, tile_req.numel() * num_heads)
    if segments > 0:
        _need(not split or tile_req.numel() == N, "warps share a tile's keys only in steps of one token a request")
        scratch = torch.empty(segments * (2 if split else 1) * N * num_heads * 2 * (vdim + 2), dtype=torch.float32, device=q.device)
    _call("llmp_diff_attention_mma", _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(pages), _ptr(tables), tables.shape[1],
          _ptr(q_start), _ptr(ctx_len), _ptr(positions), _ptr(tile_req), _ptr(tile_tok0), tile_req.numel(), N, num_heads, num_kv_heads,
          dim, vdim, pages.shape[2], int(window), float(scale), float(lam), float(eps), float(out_scale),
          DIFF_SEGMENT_KEYS if segments > 0 else 0, int(segments), 1 if split and segments > 0 else 0, _ptr(scratch), _ptr(counters),
          _stream())
    return out


SHORT_CONV_MAX_TAPS = 8           # taps the short-convolution kernels hold in registers


def _state_views(state: torch.Tensor, offset: int, half: int, name: str):
    """A request's state slot is one float32 vector ``state[slot, :]``; a part keeps a piece of it that starts at ``offset``
    and holds two copies of ``half`` entries, which take turns by the parity of the last position written."""
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1, f"{name}: the state must be float32 [slots, entries]")
    _need(0 <= offset and offset + 2 * half <= state.shape[1], f"{name}: the state piece does not fit the slot")
    return state.data_ptr() + 4 * offset, state.stride(0), half


def short_conv(x: torch.Tensor, taps: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor, state_offset: int,
               q_start: torch.Tensor, slots: torch.Tensor, positions: torch.Tensor, token_request: torch.Tensor,
               out: Optional[torch.Tensor], max_q_len: int, silu: bool = True, add_input: bool = False,
               out_typed: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """Causal convolution over time per channel with its carried inputs: ``x`` float32 [tokens, C] (a view with a dense last
    axis), ``taps`` [C, K] (the last column multiplies the current token), ``bias`` [C] or None, ``out`` float32 [tokens, C]
    or None. The state piece holds two copies of the request's last K - 1 inputs [K - 1, C]. ``add_input``: the result is
    ``x + conv(x)`` with no activation. ``out_typed`` (float32 or bfloat16): the result once more as ``[parts, tokens,
    C / parts]`` or ``[tokens, C]``, the channels cut into equal runs that become matrices of their own."""
    N, C = x.shape
    K = taps.shape[1]
    _need(x.dtype == torch.float32 and x.stride(1) == 1, "short_conv takes float32 rows")
    _need(out is None or (out.dtype == torch.float32 and out.stride(1) == 1 and out.shape == (N, C)), "short_conv gives float32 rows")
    _need(out is not None or out_typed is not None, "short_conv needs an output")
    _need(taps.shape[0] == C and taps.is_contiguous() and (bias is None or (bias.numel() == C and bias.is_contiguous())),
          "short_conv: taps or bias have the wrong shape")
    _need(not (silu and add_input), "short_conv: one of SiLU and the added input")
    for t, name in ((q_start, "q_start"), (slots, "slots"), (positions, "positions"), (token_request, "token_request")):
        _i32(t, name)
    split, block, stride2 = C, 0, 0
    if out_typed is not None:
        _need(out_typed.is_contiguous() and out_typed.shape[-2] == N and out_typed.numel() == N * C and out_typed.dim() in (2, 3),
              "short_conv: the typed output must be [tokens, C] or [parts, tokens, C / parts]")
        split, stride2 = out_typed.shape[-1], out_typed.shape[-1]
        block = N * split
    ptr, slot_stride, half = _state_views(state, state_offset, (K - 1) * C, "short_conv")
    _call("llmp_short_conv", _ptr(x), x.stride(0), _ptr(taps), dtype_code(taps.dtype), _ptr(bias),
          dtype_code(bias.dtype) if bias is not None else F32, ptr, slot_stride, half, _ptr(q_start), _ptr(slots), _ptr(positions),
          _ptr(token_request), _ptr(out), out.stride(0) if out is not None else 0, _ptr(out_typed),
          dtype_code(out_typed.dtype) if out_typed is not None else F32, stride2, block, split, N, slots.numel(), C, K,
          2 if add_input else (1 if silu else 0), int(max_q_len), _stream())
    return out if out is not None else out_typed


def ssd_scan(xbc: torch.Tensor, dt: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor, d_skip: torch.Tensor,
             state: torch.Tensor, state_offset: int, q_start: torch.Tensor, slots: torch.Tensor, positions: torch.Tensor,
             y: torch.Tensor, heads: int, groups: int, state_size: int, vdim: int) -> torch.Tensor:
    """The state-space recurrence with a scalar decay per head and token (csrc/state_space.cu): ``xbc`` float32 [tokens,
    heads vdim + 2 groups state] = x | B | C, ``dt`` float32 [tokens, heads] (a view), the three per-head vectors float32,
    ``y`` float32 [tokens, heads vdim]. The state piece holds two copies of [heads, state, vdim]."""
    N = xbc.shape[0]
    _need(xbc.dtype == torch.float32 and xbc.stride(1) == 1 and xbc.shape[1] == heads * vdim + 2 * groups * state_size,
          "ssd_scan: x | B | C has the wrong width")
    _need(dt.dtype == torch.float32 and dt.stride(1) == 1 and dt.shape == (N, heads), "ssd_scan: dt must be float32 [tokens, heads]")
    _need(y.dtype == torch.float32 and y.stride(1) == 1 and y.shape == (N, heads * vdim), "ssd_scan: y has the wrong shape")
    for t in (dt_bias, a_log, d_skip):
        _need(t.dtype == torch.float32 and t.numel() == heads and t.is_contiguous(), "ssd_scan takes float32 vectors of one entry per head")
    for t, name in ((q_start, "q_start"), (slots, "slots"), (positions, "positions")):
        _i32(t, name)
    ptr, slot_stride, half = _state_views(state, state_offset, heads * state_size * vdim, "ssd_scan")
    _call("llmp_ssd_scan", _ptr(xbc), xbc.stride(0), _ptr(dt), dt.stride(0), _ptr(dt_bias), _ptr(a_log), _ptr(d_skip), ptr,
          slot_stride, half, _ptr(q_start), _ptr(slots), _ptr(positions), _ptr(y), y.stride(0), slots.numel(), heads, groups,
          state_size, vdim, _stream())
    return y


def gated_group_norm(y: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, group_size: int, eps: float,
                     gate_first: bool) -> torch.Tensor:
    """Rows cut into groups of ``group_size`` entries, each divided by its own root mean square. ``gate_first``: out =
    rms(y silu(gate)) * weight[column]; else out = rms(y) * weight[column within the group] * sigmoid(gate). ``y`` and
    ``gate`` float32 views, ``weight`` float32."""
    N, W = y.shape
    _need(y.dtype == torch.float32 and gate.dtype == torch.float32 and y.stride(1) == 1 and gate.stride(1) == 1 and gate.shape == (N, W),
          "gated_group_norm takes float32 rows and gates")
    _need(weight.dtype == torch.float32 and weight.is_contiguous() and weight.numel() == (W if gate_first else group_size),
          "gated_group_norm: the weight has the wrong size")
    _need(out.shape == (N, W) and out.stride(1) == 1, "gated_group_norm: the output has the wrong shape")
    _call("llmp_gated_group_norm", _ptr(y), y.stride(0), _ptr(gate), gate.stride(0), _ptr(weight), _ptr(out), dtype_code(out.dtype),
          out.stride(0), N, W, int(group_size), 0 if gate_first else 1, float(eps), _stream())
    return out


def delta_prep(q: torch.Tensor, k: torch.Tensor, decay: torch.Tensor, beta: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor,
               heads: int, qk_heads: int, dim: int) -> None:
    """In place, per token (csrc/delta_rule.cu): ``q`` and ``k`` float32 [tokens, qk_heads dim] become unit vectors per head (q also
    times dim^(-1/2)); ``decay`` float32 [tokens, heads dim] goes from its pre-activation to exp(-exp(a_log[head]) softplus(. +
    dt_bias)); ``beta`` float32 [tokens, heads] to its sigmoid. All four may be views with a dense last axis."""
    N = q.shape[0]
    for t, w, name in ((q, qk_heads * dim, "q"), (k, qk_heads * dim, "k"), (decay, heads * dim, "decay"), (beta, heads, "beta")):
        _need(t.dtype == torch.float32 and t.stride(1) == 1 and t.shape == (N, w), f"delta_prep: {name} must be float32 [tokens, {w}]")
    _need(a_log.dtype == torch.float32 and a_log.numel() == heads and a_log.is_contiguous() and dt_bias.dtype == torch.float32 and
          dt_bias.numel() == heads * dim and dt_bias.is_contiguous(), "delta_prep takes float32 A_log [heads] and dt_bias [heads dim]")
    _call("llmp_delta_prep", _ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(decay), decay.stride(0), _ptr(beta), beta.stride(0),
          _ptr(a_log), _ptr(dt_bias), N, heads, qk_heads, dim, _stream())


def delta_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, beta: torch.Tensor, state: torch.Tensor,
               state_offset: int, q_start: torch.Tensor, slots: torch.Tensor, positions: torch.Tensor, out: torch.Tensor,
               heads: int, qk_heads: int, dim: int, vdim: int) -> torch.Tensor:
    """The gated delta rule over the step's tokens, request by request (csrc/delta_rule.cu); inputs as ``delta_prep`` leaves
    them, ``v`` float32 [tokens, heads vdim], ``out`` float32 [tokens, heads vdim]. The state piece holds two copies of
    [heads, dim, vdim]."""
    N = q.shape[0]
    for t, w, name in ((q, qk_heads * dim, "q"), (k, qk_heads * dim, "k"), (v, heads * vdim, "v"), (decay, heads * dim, "decay"),
                       (beta, heads, "beta"), (out, heads * vdim, "out")):
        _need(t.dtype == torch.float32 and t.stride(1) == 1 and t.shape == (N, w), f"delta_scan: {name} must be float32 [tokens, {w}]")
    for t, name in ((q_start, "q_start"), (slots, "slots"), (positions, "positions")):
        _i32(t, name)
    ptr, slot_stride, half = _state_views(state, state_offset, heads * dim * vdim, "delta_scan")
    _call("llmp_delta_scan", _ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(v), v.stride(0), _ptr(decay), decay.stride(0),
          _ptr(beta), beta.stride(0), ptr, slot_stride, half, _ptr(q_start), _ptr(slots), _ptr(positions), _ptr(out), out.stride(0),
          slots.numel(), heads, qk_heads, dim, vdim, _stream())
    return out


def sig_qkv_post(qkv: torch.Tensor, bias: Optional[torch.Tensor], cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                 rotary_dim: int, q_out: torch.Tensor, slot_mapping: Optional[torch.Tensor], pages: Optional[torch.Tensor],
                 heads: int, kv_heads: int, dim: int, vdim: int) -> torch.Tensor:
    """After the float32 product [q | k | v] (csrc/sigmoid_attention.cu): bias, rotation of the first ``rotary_dim`` entries of
    every query and key head (entry i with i + rotary_dim / 2), queries to ``q_out`` [tokens, heads dim], the token's [k | v]
    rows to its page slot. ``pages``: [pages, kv_heads, page_size, dim + vdim]."""
    N = qkv.shape[0]
    width = (heads + kv_heads) * dim + kv_heads * vdim
    _need(qkv.dtype == torch.float32 and qkv.stride(1) == 1 and qkv.shape[1] == width, "sig_qkv_post takes the float32 product [q | k | v]")
    _need(bias is None or (bias.numel() == width and bias.is_contiguous()), "sig_qkv_post: the bias has the wrong size")
    _need(q_out.shape == (N, heads * dim) and q_out.stride(1) == 1, "sig_qkv_post: the query output has the wrong shape")
    if rotary_dim:
        _need(cos is not None and sin is not None and cos.dtype == torch.float32 and cos.shape == (N, rotary_dim // 2) and
              cos.is_contiguous() and sin.is_contiguous(), "sig_qkv_post: the rotation's tables must be float32 [tokens, rotary_dim / 2]")
    page_size = 0
    if pages is not None:
        _need(slot_mapping is not None and pages.dim() == 4 and pages.is_contiguous() and pages.shape[1] == kv_heads and
              pages.shape[3] == dim + vdim and pages.dtype == q_out.dtype, "sig_qkv_post: pages must be [pages, kv_heads, page_size, dim + vdim] of the queries' type")
        _i32(slot_mapping, "slot_mapping")
        page_size = pages.shape[2]
    _call("llmp_sig_qkv_post", _ptr(qkv), qkv.stride(0), _ptr(bias), dtype_code(bias.dtype) if bias is not None else F32, _ptr(cos),
          _ptr(sin), int(rotary_dim), _ptr(q_out), dtype_code(q_out.dtype), q_out.stride(0), _ptr(slot_mapping) if pages is not None else None,
          _ptr(pages), page_size, N, heads, kv_heads, dim, vdim, _stream())
    return q_out


SIGMOID_MAX_HEADS = 32             # query heads whose weights one block of the sigmoid attention kernel mixes
SIGMOID_SEGMENT_KEYS = 1024       # keys of a segment when a token's keys are shared among blocks (a multiple of the key tile)
SIGMOID_MMA_SEGMENT_KEYS = 128    # the same for the tensor-core kernel, whose blocks walk a tile of keys for up to 16 tokens at once
SIGMOID_MMA_LONG_SEGMENT_KEYS = 1024   # ranges of long prompts whose tiles are too few for two rounds of blocks
SIGMOID_MMA_ROWS = 16             # new tokens of a request in a tile of the tensor-core kernel


def sigmoid_attention(q: torch.Tensor, pages: torch.Tensor, tables: torch.Tensor, token_request: torch.Tensor, positions: torch.Tensor,
                      talk: torch.Tensor, head_bias: torch.Tensor, out: torch.Tensor, heads: int, kv_heads: int, dim: int, vdim: int,
                      scale: float, softcap: float, segments: int = 1) -> torch.Tensor:
    """Causal attention whose weights are sigmoid(capped score + head_bias[head]), mixed across heads by ``talk`` [heads, heads]
    before they meet the values, not normalised over keys (csrc/sigmoid_attention.cu). ``segments`` > 1: a token's keys are
    shared among that many blocks in fixed ranges of ``SIGMOID_SEGMENT_KEYS`` and the partial sums added in their order."""
    N = q.shape[0]
    _need(q.shape == (N, heads * dim) and q.stride(1) == 1 and out.shape == (N, heads * vdim) and out.stride(1) == 1 and
          q.dtype == out.dtype == pages.dtype, "sigmoid_attention: queries, pages and output must have one type and matching shapes")
    _need(pages.dim() == 4 and pages.is_contiguous() and pages.shape[1] == kv_heads and pages.shape[3] == dim + vdim,
          "sigmoid_attention: pages must be [pages, kv_heads, page_size, dim + vdim]")
    _need(talk.dtype == torch.float32 and talk.is_contiguous() and talk.shape == (heads, heads) and head_bias.dtype == torch.float32 and
          head_bias.is_contiguous() and head_bias.numel() == heads, "sigmoid_attention takes a float32 head mix [heads, heads] and bias [heads]")
    _need(tables.dtype == torch.int32 and tables.dim() == 2 and tables.stride(1) == 1, "block tables must be int32 [requests, width]")
    _need(tables.is_contiguous(), "block tables must be contiguous")
    _i32(token_request, "token_request")
    _i32(positions, "positions")
    partial = None
    if segments > 1:
        partial = torch.empty((N, segments, heads * vdim), dtype=torch.float32, device=q.device)
    _call("llmp_sigmoid_attention", _ptr(q), q.stride(0), _ptr(pages), dtype_code(q.dtype), _ptr(tables), tables.shape[1],
          _ptr(token_request), _ptr(positions), _ptr(talk), _ptr(head_bias), _ptr(out), out.stride(0), _ptr(partial), int(segments),
          SIGMOID_SEGMENT_KEYS, N, heads, kv_heads, dim, vdim, pages.shape[2], float(scale), float(softcap or 0.0), _stream())
    return out


def sigmoid_attention_mma_supports(dtype: torch.dtype, heads: int, kv_heads: int, dim: int, vdim: int) -> bool:
    """Whether the tensor-core kernel has an instance for these sizes (bfloat16, up to 16 heads, head sizes 16, 32, 64, 96 or 128)."""
    if dtype != torch.bfloat16:
        return False
    fn = library().llmp_sigmoid_attention_mma_supports
    fn.argtypes = [_I, _I, _I, _I]
    fn.restype = ctypes.c_int
    return bool(fn(int(heads), int(kv_heads), int(dim), int(vdim)))


def sigmoid_attention_mma(q: torch.Tensor, pages: torch.Tensor, tables: torch.Tensor, q_start: torch.Tensor, ctx_len: torch.Tensor,
                          positions: torch.Tensor, tile_req: torch.Tensor, tile_tok0: torch.Tensor, talk: torch.Tensor,
                          head_bias: torch.Tensor, out: torch.Tensor, heads: int, kv_heads: int, dim: int, vdim: int, scale: float,
                          softcap: float, segments: int = 1, segment_keys: int = 0) -> torch.Tensor:
    """``sigmoid_attention`` on the tensor cores for bfloat16 (csrc/sigmoid_attention_mma.cu). ``tile_req``/``tile_tok0``: the
    work list (request and first new token of every tile of ``SIGMOID_MMA_ROWS`` tokens), in the order of the keys a tile
    sees. ``segments`` > 1: fixed ranges of ``segment_keys`` keys (a multiple of 32; ``SIGMOID_MMA_SEGMENT_KEYS`` when 0) go to
    blocks of their own."""
    N = q.shape[0]
    _need(q.dtype == out.dtype == pages.dtype == torch.bfloat16 and q.shape == (N, heads * dim) and q.stride(1) == 1 and
          out.shape == (N, heads * vdim) and out.stride(1) == 1, "sigmoid_attention_mma takes bfloat16 queries, pages and output of matching shapes")
    _need(pages.dim() == 4 and pages.is_contiguous() and pages.shape[1] == kv_heads and pages.shape[3] == dim + vdim,
          "sigmoid_attention_mma: pages must be [pages, kv_heads, page_size, dim + vdim]")
    _need(talk.dtype == torch.float32 and talk.is_contiguous() and talk.shape == (heads, heads) and head_bias.dtype == torch.float32 and
          head_bias.is_contiguous() and head_bias.numel() == heads, "sigmoid_attention_mma takes a float32 head mix [heads, heads] and bias [heads]")
    _need(tables.dtype == torch.int32 and tables.dim() == 2 and tables.is_contiguous(), "block tables must be dense int32 [requests, width]")
    for t, name in ((q_start, "q_start"), (ctx_len, "ctx_len"), (positions, "positions"), (tile_req, "tile_req"), (tile_tok0, "tile_tok0")):
        _i32(t, name)
    _need(tile_req.numel() == tile_tok0.numel(), "sigmoid_attention_mma: the work list's columns differ in length")
    partial = None
    if segments > 1:
        partial = torch.empty((N, segments, heads * vdim), dtype=torch.float32, device=q.device)
    _call("llmp_sigmoid_attention_mma", _ptr(q), q.stride(0), _ptr(pages), _ptr(tables), tables.shape[1], _ptr(q_start), _ptr(ctx_len),
          _ptr(positions), _ptr(tile_req), _ptr(tile_tok0), tile_req.numel(), _ptr(talk), _ptr(head_bias), _ptr(out), out.stride(0),
          _ptr(partial), int(segments), int(segment_keys) or SIGMOID_MMA_SEGMENT_KEYS, N, heads, kv_heads, dim, vdim, pages.shape[2], float(scale),
          float(softcap or 0.0), _stream())
    return out


def xielu(z: torch.Tensor, bias: Optional[torch.Tensor], a_pos: float, a_neg: float, out: torch.Tensor) -> torch.Tensor:
    """out = f(z + bias) with f(v) = a_pos v^2 + v / 2 for v > 0 and a_neg (exp(v) - 1 - v) + v / 2 otherwise; ``z`` float32."""
    N, F = z.shape
    _need(z.dtype == torch.float32 and z.is_contiguous() and out.is_contiguous() and out.shape == (N, F), "xielu takes dense float32 rows")
    _need(bias is None or (bias.numel() == F and bias.is_contiguous()), "xielu: the bias has the wrong size")
    _call("llmp_xielu", _ptr(z), _ptr(bias), dtype_code(bias.dtype) if bias is not None else F32, float(a_pos), float(a_neg), _ptr(out),
          dtype_code(out.dtype), N, F, _stream())
    return out


def scaled_sum(a: torch.Tensor, scale_a: float, b: torch.Tensor, scale_b: float, out: torch.Tensor) -> torch.Tensor:
    """out = scale_a a + scale_b b, all float32 and dense."""
    _need(a.dtype == b.dtype == out.dtype == torch.float32 and a.is_contiguous() and b.is_contiguous() and out.is_contiguous() and
          a.shape == b.shape == out.shape, "scaled_sum takes dense float32 tensors of one shape")
    _call("llmp_scaled_sum", _ptr(a), float(scale_a), _ptr(b), float(scale_b), _ptr(out), a.numel(), _stream())
    return out


# ---- kernels of the capped window attention, the selective scan, the several-weight norm and small activations -------
def latent_rows_post(q: torch.Tensor, dkv: Optional[torch.Tensor], heads: int, dim: int, rot: int, rank: int,
                     norm_weight: Optional[torch.Tensor], eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                     rot_dims: int, interleaved: bool, q_out: torch.Tensor, slot_mapping: Optional[torch.Tensor],
                     pages: Optional[torch.Tensor]) -> torch.Tensor:
    """After the float32 products of a latent attention layer (csrc/latent_attention.cu): ``q`` [tokens, heads (dim + rot)]
    leaves in the compute type with every head's rotated part rotated; ``dkv`` [tokens, rank + rot] (None: the layer reads
    another layer's rows) becomes the cache row [rms_norm(latent) * weight | rotated shared key part] in the token's page
    slot. ``interleaved``: entry 2i turns with entry 2i + 1, else entry i with entry i + rot_dims / 2."""
    N = q.shape[0]
    _need(q.dtype == torch.float32 and q.stride(1) == 1 and q.shape[1] == heads * (dim + rot), "latent_rows_post takes the float32 queries")
    _need(q_out.shape == (N, heads * (dim + rot)) and q_out.stride(1) == 1, "latent_rows_post: the query output has the wrong shape")
    if rot_dims:
        _need(cos is not None and sin is not None and cos.dtype == torch.float32 and cos.shape == (N, rot_dims // 2) and
              cos.is_contiguous() and sin.is_contiguous(), "latent_rows_post: the rotation's tables must be float32 [tokens, rot_dims / 2]")
    writes = dkv is not None and pages is not None
    if writes:
        _need(dkv.dtype == torch.float32 and dkv.stride(1) == 1 and dkv.shape == (N, rank + rot), "latent_rows_post takes the float32 row [latent | key part]")
        _need(pages.is_contiguous() and pages.dim() == 3 and pages.shape[2] == rank + rot and pages.dtype == q_out.dtype,
              "latent pages have the wrong layout")
        _need(norm_weight is not None and norm_weight.numel() == rank and norm_weight.is_contiguous(), "the latent's norm weight has the wrong size")
        _i32(slot_mapping, "slot_mapping")
    _call("llmp_latent_rows_post", _ptr(q), q.stride(0), _ptr(dkv) if writes else None, dkv.stride(0) if writes else 0, heads, dim, rot, rank,
          _ptr(norm_weight) if writes else None, dtype_code(norm_weight.dtype) if writes else F32, float(eps), _ptr(cos), _ptr(sin),
          int(rot_dims), 1 if interleaved else 0, _ptr(q_out), dtype_code(q_out.dtype), q_out.stride(0),
          _ptr(slot_mapping) if writes else None, _ptr(pages) if writes else None, N, _stream())
    return q_out


def capped_qkv_post(qkv: torch.Tensor, bias: Optional[torch.Tensor], value_norm_eps: Optional[float], q_out: torch.Tensor,
                    slot_mapping: Optional[torch.Tensor], pages: Optional[torch.Tensor], heads: int, kv_heads: int, dim: int,
                    vdim: int) -> torch.Tensor:
    """After the float32 product [q | k | v] (csrc/capped_attention.cu): bias, every value head divided by its root mean
    square (``value_norm_eps`` not None), queries to ``q_out`` [tokens, heads dim], the token's [k | v] rows to its page slot.
    ``pages``: [pages, kv_heads, page_size, dim + vdim]."""
    N = qkv.shape[0]
    width = (heads + kv_heads) * dim + kv_heads * vdim
    _need(qkv.dtype == torch.float32 and qkv.stride(1) == 1 and qkv.shape[1] == width, "capped_qkv_post takes the float32 product [q | k | v]")
    _need(bias is None or (bias.numel() == width and bias.is_contiguous()), "capped_qkv_post: the bias has the wrong size")
    _need(q_out.shape == (N, heads * dim) and q_out.stride(1) == 1, "capped_qkv_post: the query output has the wrong shape")
    page_size = 0
    if pages is not None:
        _need(slot_mapping is not None and pages.dim() == 4 and pages.is_contiguous() and pages.shape[1] == kv_heads and
              pages.shape[3] == dim + vdim and pages.dtype == q_out.dtype, "capped_qkv_post: pages must be [pages, kv_heads, page_size, dim + vdim] of the queries' type")
        _i32(slot_mapping, "slot_mapping")
        page_size = pages.shape[2]
    _call("llmp_capped_qkv_post", _ptr(qkv), qkv.stride(0), _ptr(bias), dtype_code(bias.dtype) if bias is not None else F32,
          float(value_norm_eps or 0.0), 0 if value_norm_eps is None else 1, _ptr(q_out), dtype_code(q_out.dtype), q_out.stride(0),
          _ptr(slot_mapping) if pages is not None else None, _ptr(pages), page_size, N, heads, kv_heads, dim, vdim, _stream())
    return q_out


def capped_attention(q: torch.Tensor, pages: torch.Tensor, tables: torch.Tensor, token_request: torch.Tensor, positions: torch.Tensor,
                     out: torch.Tensor, num_heads: int, num_kv_heads: int, dim: int, vdim: int, window: int, keep_first: int,
                     scale: float, softcap: float, slopes: Optional[torch.Tensor] = None, sink: Optional[torch.Tensor] = None,
                     gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Softmax attention of rows (token, head), any sizes, float32 or bfloat16 (csrc/capped_attention.cu): ``q`` [tokens, heads
    dim], ``pages`` [pages, kv_heads, page_size, dim + vdim], ``out`` [tokens, heads vdim]. A token sees the ``window`` keys up
    to itself (0: all) and the first ``keep_first`` keys; a score is capped (``softcap`` > 0) and loses ``slopes[h]`` times the
    distance; exp(``sink[h]``) joins the denominator; the result is multiplied by sigmoid(``gate``) (float32 [tokens, heads vdim],
    a view)."""
    N = q.shape[0]
    _need(q.stride(1) == 1 and q.shape[1] == num_heads * dim and out.shape == (N, num_heads * vdim) and out.stride(1) == 1,
          "capped attention shapes do not match")
    _need(q.dtype == pages.dtype == out.dtype, "capped attention operands must have one type")
    _need(pages.is_contiguous() and pages.dim() == 4 and pages.shape[1] == num_kv_heads and pages.shape[3] == dim + vdim,
          "capped attention pages have the wrong layout")
    _sink(sink, num_heads); _sink(slopes, num_heads)
    _need(gate is None or (gate.dtype == torch.float32 and gate.shape == (N, num_heads * vdim) and gate.stride(1) == 1),
          "the gate must be float32 [tokens, heads vdim]")
    _i32(tables, "tables"); _i32(token_request, "token_request"); _i32(positions, "positions")
    _call("llmp_capped_attention", _ptr(q), q.stride(0), _ptr(pages), dtype_code(pages.dtype), _ptr(tables), tables.shape[1],
          _ptr(token_request), _ptr(positions), _ptr(slopes), _ptr(sink), _ptr(gate), gate.stride(0) if gate is not None else 0,
          _ptr(out), out.stride(0), N, num_heads, num_kv_heads, dim, vdim, pages.shape[2], int(window), int(keep_first),
          float(scale), float(softcap), _stream())
    return out


def capped_mma_supports(dtype: torch.dtype, dim: int, vdim: int) -> bool:
    """Whether the tensor-core capped attention kernel serves these sizes (bfloat16)."""
    if dtype != torch.bfloat16:
        return False
    fn = library().llmp_capped_mma_supports
    fn.argtypes = [_I, _I]
    fn.restype = _I
    return bool(fn(dim, vdim))


def capped_mma_tokens_per_tile(num_heads: int, num_kv_heads: int) -> int:
    fn = library().llmp_capped_mma_tokens_per_tile
    fn.argtypes = [_I, _I]
    fn.restype = _I
    return int(fn(num_heads, num_kv_heads))


def capped_attention_mma(q: torch.Tensor, pages: torch.Tensor, tables: torch.Tensor, q_start: torch.Tensor, ctx_len: torch.Tensor,
                         tile_req: torch.Tensor, tile_tok0: torch.Tensor, out: torch.Tensor, num_heads: int, num_kv_heads: int, dim: int,
                         vdim: int, window: int, keep_first: int, scale: float, softcap: float, slopes: Optional[torch.Tensor] = None,
                         sink: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None, split: bool = False) -> torch.Tensor:
    """``capped_attention`` on the tensor cores for bfloat16 (csrc/capped_attention_mma.cu). ``tile_req``/``tile_tok0``: the work
    list (request and first token of every tile of ``capped_mma_tokens_per_tile`` tokens). ``split``: every tile is one token,
    and the four warps of a block share its keys."""
    N = q.shape[0]
    _need(q.dtype == torch.bfloat16 and pages.dtype == torch.bfloat16 and out.dtype == torch.bfloat16, "capped_attention_mma takes bfloat16")
    _need(q.stride(1) == 1 and q.shape[1] == num_heads * dim and out.shape == (N, num_heads * vdim) and out.stride(1) == 1,
          "capped attention shapes do not match")
    _need(pages.is_contiguous() and pages.dim() == 4 and pages.shape[1] == num_kv_heads and pages.shape[3] == dim + vdim,
          "capped attention pages have the wrong layout")
    _sink(sink, num_heads); _sink(slopes, num_heads)
    _need(gate is None or (gate.dtype == torch.float32 and gate.shape == (N, num_heads * vdim) and gate.stride(1) == 1),
          "the gate must be float32 [tokens, heads vdim]")
    for t, name in ((tables, "tables"), (q_start, "q_start"), (ctx_len, "ctx_len"), (tile_req, "tile_req"), (tile_tok0, "tile_tok0")):
        _i32(t, name)
    _need(not split or tile_req.numel() == N, "warps share a tile's keys only in steps of one token a request")
    _call("llmp_capped_attention_mma", _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(pages), _ptr(tables), tables.shape[1],
          _ptr(q_start), _ptr(ctx_len), _ptr(tile_req), _ptr(tile_tok0), tile_req.numel(), _ptr(slopes), _ptr(sink), _ptr(gate),
          gate.stride(0) if gate is not None else 0, num_heads, num_kv_heads, dim, vdim, pages.shape[2], int(window), int(keep_first),
          float(scale), float(softcap), 1 if split else 0, _stream())
    return out


SELECTIVE_SCAN_MAX_STATES = 256


def selective_scan(x: torch.Tensor, dt: torch.Tensor, dt_bias: torch.Tensor, b: torch.Tensor, c: torch.Tensor, a: torch.Tensor,
                   d_skip: torch.Tensor, z: Optional[torch.Tensor], state: torch.Tensor, state_offset: int, q_start: torch.Tensor,
                   slots: torch.Tensor, positions: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """The selective state-space recurrence with a decay per channel and state entry (csrc/selective_scan.cu): float32 rows
    ``x``, ``dt`` [tokens, inner] (dt before bias and softplus), ``b``, ``c`` [tokens, states] (views of one matrix), ``a`` [inner,
    states] (negative), ``d_skip``, ``dt_bias`` [inner], ``z`` [tokens, inner] or None; ``out`` [tokens, inner] = y * silu(z) in the
    compute type. The state piece holds two copies of [inner, states]."""
    N, inner = x.shape
    states = a.shape[1]
    for t, name in ((x, "x"), (dt, "dt"), (b, "B"), (c, "C")) + (((z, "z"),) if z is not None else ()):
        _need(t.dtype == torch.float32 and t.stride(1) == 1 and t.shape[0] == N, f"selective_scan: {name} must be float32 rows")
    _need(dt.shape == (N, inner) and b.shape == (N, states) and c.shape == (N, states) and b.stride(0) == c.stride(0) and
          (z is None or z.shape == (N, inner)), "selective_scan: shapes do not match")
    for t in (dt_bias, d_skip, a):
        _need(t.dtype == torch.float32 and t.is_contiguous(), "selective_scan: the layer's vectors must be float32")
    _need(dt_bias.numel() == inner and d_skip.numel() == inner and a.shape == (inner, states), "selective_scan: the layer's vectors have the wrong size")
    _need(out.shape == (N, inner) and out.stride(1) == 1, "selective_scan: the output has the wrong shape")
    for t, name in ((q_start, "q_start"), (slots, "slots"), (positions, "positions")):
        _i32(t, name)
    ptr, slot_stride, half = _state_views(state, state_offset, inner * states, "selective_scan")
    _call("llmp_selective_scan", _ptr(x), x.stride(0), _ptr(dt), dt.stride(0), _ptr(dt_bias), _ptr(b), _ptr(c), b.stride(0), _ptr(a),
          _ptr(d_skip), _ptr(z), z.stride(0) if z is not None else 0, ptr, slot_stride, half, _ptr(q_start), _ptr(slots),
          _ptr(positions), _ptr(out), dtype_code(out.dtype), out.stride(0), slots.numel(), inner, states, _stream())
    return out


def add_rmsnorm_multi(residual: torch.Tensor, first: Optional[torch.Tensor], second: Optional[torch.Tensor],
                      bias: Optional[torch.Tensor], weights: torch.Tensor, eps: float, out: torch.Tensor,
                      rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """residual += (first + bias) + second (float32, in place; each may be None), then ``out[j]`` = the RMS norm of the rows
    times ``weights[j]``, for every row of ``weights`` [k, width]; ``out`` [rows, k width] (the k results of a row side by
    side), float32 or the compute type. With ``rows`` only those rows are normed and the residual stays as it is."""
    R, D = residual.shape
    _need(residual.dtype == torch.float32 and residual.is_contiguous(), "the residual must be contiguous float32")
    for d in (first, second):
        if d is not None:
            _need(d.shape == residual.shape and d.is_contiguous(), "an addend must have the residual's shape")
    _need(weights.dim() == 2 and weights.shape[1] == D and weights.is_contiguous(), "norm weights must be [k, width]")
    _need(bias is None or (bias.numel() == D and bias.is_contiguous()), "the addend's bias has the wrong size")
    k = weights.shape[0]
    M = rows.numel() if rows is not None else R
    _need(out.is_contiguous() and out.shape == (M, k * D), "norm output must be [rows, k width]")
    if rows is not None:
        _i32(rows, "rows")
    code = lambda t: dtype_code(t.dtype) if t is not None else F32   # noqa: E731
    _call("llmp_add_rmsnorm_multi", _ptr(residual), _ptr(first), code(first), _ptr(second), code(second), _ptr(bias), code(bias),
          _ptr(weights), dtype_code(weights.dtype), k, float(eps), _ptr(out), dtype_code(out.dtype), D, k * D, _ptr(rows), M, D, _stream())
    return out


def gated_act(gate_up: torch.Tensor, out: torch.Tensor, act: str = "gelu_tanh") -> torch.Tensor:
    """out = act(gate) * up for rows [gate | up] (float32 or the compute type), act "gelu_tanh" or "silu"; float32 arithmetic."""
    M, F2 = gate_up.shape
    _need(gate_up.stride(1) == 1 and out.is_contiguous() and out.shape == (M, F2 // 2) and F2 % 2 == 0, "gated_act shapes do not match")
    _need(act in ("gelu_tanh", "silu"), f"gated_act: unknown activation {act!r}")
    _call("llmp_gated_act", _ptr(gate_up), dtype_code(gate_up.dtype), gate_up.stride(0), _ptr(out), dtype_code(out.dtype), M, F2 // 2,
          1 if act == "gelu_tanh" else 0, _stream())
    return out


def sigmoid_gate(x: torch.Tensor, gate: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = x * sigmoid(gate): ``x`` dense rows of the compute type, ``gate`` float32 rows (a view)."""
    out = x if out is None else out
    _need(x.is_contiguous() and out.is_contiguous() and out.shape == x.shape and out.dtype == x.dtype and x.dim() == 2, "sigmoid_gate takes dense rows")
    _need(gate.dtype == torch.float32 and gate.shape == x.shape and gate.stride(1) == 1, "the gate must be float32 rows of the same shape")
    _call("llmp_sigmoid_gate", _ptr(x), _ptr(gate), gate.stride(0), _ptr(out), dtype_code(x.dtype), x.shape[0], x.shape[1], _stream())
    return out


def convert_rows(x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """Float32 rows (a view with a dense last axis) as dense rows of ``out``'s type."""
    _need(x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1 and out.is_contiguous() and out.shape == x.shape, "convert_rows shapes do not match")
    _call("llmp_convert_rows", _ptr(x), x.stride(0), _ptr(out), dtype_code(out.dtype), x.shape[0], x.shape[1], _stream())
    return out
