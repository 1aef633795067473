"""Python face of the CUDA kernels: one thin function per exported entry point.

The shared library is compiled from ``cuinfer_b200/csrc`` on first use (see ``csrc/build.py``) and
loaded with ctypes.  Every function takes torch CUDA tensors, checks dtypes, shapes and contiguity,
and launches on torch's current stream, so that calls are ordered with torch's own work and are
recorded when a CUDA graph is being captured.  There is no CPU or library fallback: if the library
cannot be built or loaded, or a tensor is not on a CUDA device, the call raises.
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import Optional

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}

_lib_handle: Optional[ctypes.CDLL] = None
_lib_lock = threading.Lock()

# Number of kernel launches issued through this module (each wrapper call launches one kernel unless
# it says otherwise).  The benchmark reads it.
launch_count = 0


class KernelError(RuntimeError):
    pass


def library() -> ctypes.CDLL:
    """The loaded kernel library; built first if it is missing or stale."""
    global _lib_handle
    if _lib_handle is not None:
        return _lib_handle
    with _lib_lock:
        if _lib_handle is not None:
            return _lib_handle
        try:
            path = _build.build(verbose=True)
            lib = ctypes.CDLL(path)
        except Exception as exc:  # noqa: BLE001 - anything here means the product path cannot run
            raise KernelError(
                "the CUDA kernel library of cuinfer_b200 is not available, and there is no fallback: "
                f"{type(exc).__name__}: {exc}"
            ) from exc
        lib.cib_last_error.restype = ctypes.c_char_p
        _declare(lib)
        lib.cib_set_prompt_pdl.argtypes = [ctypes.c_int]
        lib.cib_set_prompt_pdl.restype = None
        lib.cib_set_prompt_pdl(1 if os.environ.get("CUINFER_B200_PROMPT_PDL", "1") != "0" and os.environ.get("CUINFER_B200_PDL", "1") != "0" else 0)
        _lib_handle = lib
        return lib


def library_path() -> str:
    library()
    return _build.library_path()


_P, _I, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


def _declare(lib: ctypes.CDLL) -> None:
    sig = {
        "cib_embedding_gather": [_P, _P, _I, _P, _I, _I, _I, _P, _F, _I, _P],
        "cib_sandwich_layernorm": [_P, _P, _I, _P, _P, _F, _P, _P, _P, _F, _I, _P, _I, _I, _I, _P],
        "cib_relu_squared": [_P, _P, _I, ctypes.c_longlong, _P],
        "cib_sigmoid_gate": [_P, _I, _P, _I, _P, _I, _I, _I, _P],
        "cib_latent_prep": [_P, _I, _I, _I, _I, _I, _I, _I, _P, _P, _I, _F, _P, _P, _I, _F, _P, _P, ctypes.c_longlong, _P, _I, _I, _P],
        "cib_latent_attention_generic": [_P, _I, _I, _P, _I, _I, _I, _P, _I, _P, _I, _I, _P, _I, _P, _P, _P, _P, _P, _I, _F, _P, _I,
                                         _I, _I, _I, _I, _F, _I, _P],
        "cib_latent_attention_mma": [_P, _I, _P, _I, _I, _P, _I, _P, _P, _I, _I, _P, _I, _P, _P, _I, _I, _I, _P, _I, _P, _I, _I, _I, _I,
                                     _F, _I, _F, _I, _P],
        "cib_gemm_generic_batched": [_P, _I, ctypes.c_longlong, _P, _I, ctypes.c_longlong, _I, _P, _I, ctypes.c_longlong, _I,
                                     _I, _I, _I, _I, _P],
        "cib_moe_table_gate_up": [_P, _I, _I, _P, _P, _I, _I, _I, _P, _P, _I, _I, _I, _I, _F, _P],
        "cib_moe_table_grouped": [_P, _I, _P, _P, _I, _I, _I, _P, _P, _P, _I, _F, _P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _F, _P],
        "cib_moe_table_down": [_P, _I, _P, _P, _I, _I, _I, _P, _P, _I, _F, _P, _P, _I, _P, _I, _I, _I, _P],
        "cib_window_attention_prep": [_P, _I, _I, _P, _P, _P, _I, _F, _I, _I, _I, _I, _P, _I, _P, _I, _P, ctypes.c_longlong, _I, _I,
                                      _P, _P, _P, _I, _I, _I, _I, _F, _I, _I, _F, _P],
        "cib_window_attention_generic": [_P, _I, _I, _P, _I, _P, _I, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _F, _I, _I, _I, _P, _P, _P],
        "cib_window_attention_mma": [_P, _I, _P, _I, _P, _I, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _F, _F, _I, _I, _I, _P, _I, _I, _I, _P, _P, _P],
        "cib_hyper_stream": [_P, _P, _I, _P, _P, _P, _P, _I, _F, _P, _I, _P, _I, _I, _I, _P],
        "cib_hyper_gather": [_P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _P],
        "cib_mlstm_scan": [_P, _P, _P, _I, _I, _P, _I, _P, _P, _I, _F, _F, _F, _P, _P, _P, _I, _I, _I, _P, _I, _I, _I, _P],
        "cib_delta_prep": [_P, _I, _I, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _F, _P, _I, _P],
        "cib_delta_scan": [_P, _I, _P, _I, _P, _P, _I, _P, _P, _P, _I, _I, _I, _P, _I, _I, _I, _P],
        "cib_head_rms_gate": [_P, _P, _I, _I, _P, _I, _I, _F, _I, _P, _I, _I, _I, _P],
        "cib_router_topk": [_P, _I, _I, _I, _P, _P, _I, _P],
        "cib_router_scored_topk": [_P, _I, _I, _I, _P, _I, _I, _F, _P, _P, _I, _P],
        "cib_rms_stream": [_P, _P, _I, _P, _I, _F, _P, _I, _F, _P, _P, _I, _I, _I, _P],
        "cib_gelu_tanh": [_P, _P, _I, _P, _I, _P, _I, _I, _I, _P],
        "cib_add_rmsnorm": [_P, _P, _I, _P, _I, _F, _P, _I, _I, _I, _P],
        "cib_gather_rows": [_P, _P, _I, _P, _P, _I, _I, _I, _P],
        "cib_silu_mul": [_P, _P, _I, _I, _I, _I, _P],
        "cib_qk_norm_rope_kv_write": [_P, _I, _I, _P, _P, _P, _P, _I, _I, _F, _P, _I, _I, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P],
        "cib_paged_attention_generic": [_P, _I, _I, _P, _I, _P, _I, _I, _P, _I, _P, _P, _P, _I, _I, _I, _I, _F, _I, _P],
        "cib_paged_attention_decode": [_P, _I, _P, _I, _P, _I, _I, _P, _I, _P, _I, _I, _I, _I, _F, _I, _I, _P, _P, _I, _P, _P, ctypes.c_longlong, _P],
        "cib_paged_attention_prefill": [_P, _I, _P, _I, _P, _I, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P],
        "cib_attention_tcgen05": [_P, _I, _P, _I, _P, _I, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P, _P, _P],
        "cib_gemm_skinny": [_P, _I, _I, _I, _P, _I, _P, _P, _I, _P, _I, _F, _P, _P, _I, _I, _I, _I, _I, _P, ctypes.c_longlong, _P],
        "cib_gemm_tcgen05": [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _P, _P],
        "cib_gemm_wstream": [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _P, _P],
        "cib_gemm_generic": [_P, _I, _P, _I, _I, _P, _I, _I, _I, _I, _I, _P],
        "cib_sample": [_P, _I, _I, _I, _P, _P, _P],
        "cib_argmax_rows": [_P, _I, _I, _I, _P, _P],
        "cib_selftest_bounded_wait": [ctypes.c_longlong, _P, _P, _P],
        "cib_fill_random": [_P, _I, ctypes.c_longlong, ctypes.c_ulonglong, ctypes.c_double, ctypes.c_double, _F, _I, _P],
    }
    for name, argtypes in sig.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = _I
    lib.cib_moe_table_grouped_supports.argtypes = [_I, _I, _I]
    lib.cib_moe_table_grouped_supports.restype = _I
    lib.cib_moe_table_grouped_workspace_ints.argtypes = [_I, _I, _I]
    lib.cib_moe_table_grouped_workspace_ints.restype = ctypes.c_longlong
    lib.cib_window_attention_mma_supports.argtypes = [_I, _I, _I, _I]
    lib.cib_window_attention_mma_supports.restype = _I
    lib.cib_latent_attention_mma_supports.argtypes = [_I, _I, _I]
    lib.cib_latent_attention_mma_supports.restype = _I
    lib.cib_latent_attention_mma_tiles.argtypes = [_P, _I, _I, _I]
    lib.cib_latent_attention_mma_tiles.restype = _I
    lib.cib_paged_attention_decode_supports.argtypes = [_I, _I, _I]
    lib.cib_paged_attention_decode_supports.restype = _I
    lib.cib_gemm_tcgen05_supports.argtypes = [_I, _I, _I]
    lib.cib_gemm_tcgen05_supports.restype = _I
    lib.cib_attention_tcgen05_supports.argtypes = [_I, _I, _I, _I]
    lib.cib_attention_tcgen05_supports.restype = _I
    lib.cib_gemm_wstream_supports.argtypes = [_I, _I, _I]
    lib.cib_gemm_wstream_supports.restype = _I
    lib.cib_gemm_skinny_supports.argtypes = [_I, _I, _I, _I]
    lib.cib_gemm_skinny_supports.restype = _I
    lib.cib_paged_attention_prefill_supports.argtypes = [_I, _I, _I]
    lib.cib_paged_attention_prefill_supports.restype = _I
    lib.cib_paged_attention_decode_scratch_floats.argtypes = [_I, _I, _I, _I]
    lib.cib_paged_attention_decode_scratch_floats.restype = ctypes.c_longlong


def _check(rc: int, name: str) -> None:
    if rc != 0:
        msg = library().cib_last_error()
        raise KernelError(f"{name} failed ({rc}): {msg.decode() if msg else 'no message'}")


# torch's current stream as a raw pointer.  The private accessors skip the construction of a Stream object, which is
# a microsecond and a half on every launch; without them the public call is used.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def _code(t: torch.Tensor, what: str) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise KernelError(f"{what}: dtype {t.dtype} is not supported (float32 or bfloat16)") from None


def _cuda(t: torch.Tensor, what: str, dtype: torch.dtype | None = None, contiguous: bool = True) -> int:
    if not t.is_cuda:
        raise KernelError(f"{what} must be a CUDA tensor; cuinfer_b200 has no CPU path")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what} must be {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")
    return t.data_ptr()


def _count() -> None:
    global launch_count
    launch_count += 1


# ---- row-wise kernels ----------------------------------------------------------------------------

def embedding_gather(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, bad_flag: torch.Tensor | None = None,
                     scale: float = 1.0) -> None:
    """out[t] = table[ids[t]] * scale as float32 rows; an ``out`` of shape [T, S, H] gets the row S times (a residual
    of several streams starts with every stream equal)."""
    T = ids.numel()
    V, H = table.shape
    copies = out.shape[1] if out.dim() == 3 else 1
    if out.shape not in ((T, H), (T, copies, H)):
        raise KernelError(f"embedding_gather: out must be [{T}, {H}] or [{T}, S, {H}], got {list(out.shape)}")
    rc = library().cib_embedding_gather(
        _cuda(ids, "ids", torch.int32), _cuda(table, "table"), _code(table, "table"), _cuda(out, "out", torch.float32),
        T, H, V, _cuda(bad_flag, "bad_flag", torch.int32) if bad_flag is not None else None, float(scale), copies, _stream())
    _check(rc, "embedding_gather")
    _count()


def add_rmsnorm(residual: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor | None, eps: float,
                out: torch.Tensor | None) -> None:
    """residual += delta (if given); out = rmsnorm(residual) * weight (if out given)."""
    rows, H = residual.shape
    if delta is not None and delta.shape != residual.shape:
        raise KernelError(f"add_rmsnorm: delta {list(delta.shape)} does not match residual {list(residual.shape)}")
    if out is not None:
        if out.shape != residual.shape:
            raise KernelError(f"add_rmsnorm: out {list(out.shape)} does not match residual {list(residual.shape)}")
        if weight is None or weight.numel() != H:
            raise KernelError(f"add_rmsnorm: weight must have {H} elements")
    rc = library().cib_add_rmsnorm(
        _cuda(residual, "residual", torch.float32),
        _cuda(delta, "delta") if delta is not None else None, _code(delta, "delta") if delta is not None else 0,
        _cuda(weight, "weight") if weight is not None else None, _code(weight, "weight") if weight is not None else 0,
        float(eps), _cuda(out, "out") if out is not None else None, _code(out, "out") if out is not None else 0,
        rows, H, _stream())
    _check(rc, "add_rmsnorm")
    _count()


def sandwich_layernorm(residual: torch.Tensor, y: torch.Tensor | None, post: tuple | None, extra: torch.Tensor | None,
                       pre: tuple | None, out: torch.Tensor | None) -> None:
    """One pass over the 32-bit residual rows: ``residual += post-norm(y)`` (``post = (gain, bias, eps)``; a plain
    ``+= y`` when ``post`` is None), ``residual += extra``, ``out = norm(residual)`` with ``pre = (gain, bias, eps)``.
    Every part may be left out.  Layer norm with gain and bias, 32-bit statistics."""
    rows, H = residual.shape
    vecs = [v for pair in (post, pre) if pair is not None for v in pair[:2]]
    if any(v.numel() != H for v in vecs) or len({v.dtype for v in vecs}) > 1:
        raise KernelError(f"layernorm: gains and biases must have {H} elements and one dtype")
    for name, t in (("y", y), ("extra", extra), ("out", out)):
        if t is not None and t.shape != residual.shape:
            raise KernelError(f"layernorm: {name} {list(t.shape)} does not match residual {list(residual.shape)}")
    if post is not None and y is None:
        raise KernelError("layernorm: an output norm needs rows to norm")
    if out is not None and pre is None:
        raise KernelError("layernorm: out needs the norm's gain and bias")
    vd = _code(vecs[0], "gain") if vecs else 0
    rc = library().cib_sandwich_layernorm(
        _cuda(residual, "residual", torch.float32), _cuda(y, "y") if y is not None else None, _code(y, "y") if y is not None else 0,
        _cuda(post[0], "post gain") if post else None, _cuda(post[1], "post bias") if post else None, float(post[2]) if post else 0.0,
        _cuda(extra, "extra", torch.float32) if extra is not None else None,
        _cuda(pre[0], "gain") if pre else None, _cuda(pre[1], "bias") if pre else None, float(pre[2]) if pre else 0.0, vd,
        _cuda(out, "out") if out is not None else None, _code(out, "out") if out is not None else 0, rows, H, _stream())
    _check(rc, "sandwich_layernorm")
    _count()


def relu_squared(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = max(x, 0) ** 2, element by element."""
    if out.shape != x.shape or out.dtype != x.dtype:
        raise KernelError("relu_squared: out does not fit x")
    rc = library().cib_relu_squared(_cuda(x, "x"), _cuda(out, "out"), _code(x, "x"), x.numel(), _stream())
    _check(rc, "relu_squared")
    _count()


def sigmoid_gate(x: torch.Tensor, gate: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, j] = x[t, j] * sigmoid(gate[t, j]); x and gate may be column ranges of wider rows."""
    rows, cols = x.shape
    if gate.shape != x.shape or out.shape != x.shape or not (x.dtype == gate.dtype == out.dtype):
        raise KernelError("sigmoid_gate: x, gate and out must have one shape and dtype")
    if x.stride(1) != 1 or gate.stride(1) != 1:
        raise KernelError("sigmoid_gate: rows must be dense")
    rc = library().cib_sigmoid_gate(_cuda(x, "x", contiguous=False), x.stride(0), _cuda(gate, "gate", contiguous=False),
                                    gate.stride(0), _cuda(out, "out"), _code(x, "x"), rows, cols, _stream())
    _check(rc, "sigmoid_gate")
    _count()


def gather_rows(residual: torch.Tensor, delta: torch.Tensor | None, indices: torch.Tensor, out: torch.Tensor) -> None:
    """out[s] = residual[indices[s]] (+ delta[indices[s]]), float32."""
    rows, H = residual.shape
    S = indices.numel()
    if out.shape != (S, H):
        raise KernelError(f"gather_rows: out must be [{S}, {H}]")
    rc = library().cib_gather_rows(
        _cuda(residual, "residual", torch.float32),
        _cuda(delta, "delta") if delta is not None else None, _code(delta, "delta") if delta is not None else 0,
        _cuda(indices, "indices", torch.int32), _cuda(out, "out", torch.float32), S, H, rows, _stream())
    _check(rc, "gather_rows")
    _count()


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, gelu: bool = False) -> None:
    """out[t, j] = silu(gate_up[t, j]) * gate_up[t, I + j]; ``gelu``: the tanh form of GELU in the place of SiLU."""
    rows, two_i = gate_up.shape
    inter = two_i // 2
    if two_i != 2 * inter or out.shape != (rows, inter) or out.dtype != gate_up.dtype:
        raise KernelError(f"silu_mul: gate_up {list(gate_up.shape)} / out {list(out.shape)} do not fit")
    rc = library().cib_silu_mul(_cuda(gate_up, "gate_up"), _cuda(out, "out"), _code(gate_up, "gate_up"), rows, inter, 1 if gelu else 0, _stream())
    _check(rc, "silu_mul")
    _count()


# ---- attention -------------------------------------------------------------------------------------

def qk_norm_rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, slot_mapping: torch.Tensor | None,
                          q_weight: torch.Tensor | None, k_weight: torch.Tensor | None, eps: float,
                          rope_table: torch.Tensor | None, rotary_dim: int, cache: torch.Tensor | None,
                          num_q_heads: int, num_kv_heads: int, head_dim: int) -> None:
    """Per-head RMSNorm (if weights are given) and rotary encoding (if a table is given) of the query and
    key heads of the packed ``qkv`` rows; queries are rewritten in place, keys and values are written to
    ``cache[page, 0|1, kv head, slot, :]`` (if a cache is given)."""
    T, stride = qkv.shape
    has_norm = q_weight is not None
    if has_norm and (k_weight is None or q_weight.dtype != k_weight.dtype):
        raise KernelError("qk_norm_rope: q and k norm weights must both be given, in one dtype")
    write_cache = cache is not None
    if write_cache:
        if cache.dim() != 5 or cache.shape[1] != 2 or cache.shape[2] != num_kv_heads or cache.shape[4] != head_dim:
            raise KernelError(f"qk_norm_rope: cache must be [pages, 2, {num_kv_heads}, page_size, {head_dim}], got {list(cache.shape)}")
        if cache.dtype != qkv.dtype:
            raise KernelError("qk_norm_rope: cache and qkv must have one dtype")
        if slot_mapping is None:
            raise KernelError("qk_norm_rope: a cache write needs slot_mapping")
    if rope_table is not None and (rope_table.dim() != 3 or rope_table.shape[1] * 2 != rotary_dim or rope_table.shape[2] != 2):
        raise KernelError(f"qk_norm_rope: rope table must be [positions, {rotary_dim // 2}, 2], got {list(rope_table.shape)}")
    rc = library().cib_qk_norm_rope_kv_write(
        _cuda(qkv, "qkv"), _code(qkv, "qkv"), stride, _cuda(positions, "positions", torch.int32),
        _cuda(slot_mapping, "slot_mapping", torch.int32) if slot_mapping is not None else None,
        _cuda(q_weight, "q_weight") if has_norm else None, _cuda(k_weight, "k_weight") if has_norm else None,
        _code(q_weight, "q_weight") if has_norm else 0, 1 if has_norm else 0, float(eps),
        _cuda(rope_table, "rope_table", torch.float32) if rope_table is not None else None,
        rotary_dim if rope_table is not None else 0, rope_table.shape[0] if rope_table is not None else 0,
        _cuda(cache, "cache") if write_cache else None, cache.shape[0] if write_cache else 0,
        cache.shape[3] if write_cache else 0, T, num_q_heads, num_kv_heads, head_dim, 1 if write_cache else 0,
        1 if use_pdl else 0, _stream())
    _check(rc, "qk_norm_rope_kv_write")
    _count()


def paged_attention_generic(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                            query_start_loc: torch.Tensor, seq_lens: torch.Tensor, token_request: torch.Tensor,
                            num_q_heads: int, num_kv_heads: int, head_dim: int, scale: float, window: int = 0) -> None:
    """Causal attention of the packed query rows ``q[:, :nq*d]`` over the paged cache; out[T, nq*d]."""
    T = q.shape[0]
    if q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("paged_attention: q and out rows must be dense")
    if out.shape != (T, num_q_heads * head_dim) or out.dtype != q.dtype or cache.dtype != q.dtype:
        raise KernelError("paged_attention: out/cache do not fit q")
    rc = library().cib_paged_attention_generic(
        _cuda(q, "q", contiguous=False), _code(q, "q"), q.stride(0), _cuda(out, "out", contiguous=False), out.stride(0),
        _cuda(cache, "cache"), cache.shape[0], cache.shape[3],
        _cuda(block_table, "block_table", torch.int32), block_table.stride(0),
        _cuda(query_start_loc, "query_start_loc", torch.int32), _cuda(seq_lens, "seq_lens", torch.int32),
        _cuda(token_request, "token_request", torch.int32), T, num_q_heads, num_kv_heads, head_dim, float(scale),
        int(window), _stream())
    _check(rc, "paged_attention_generic")
    _count()


def latent_prep(proj: torch.Tensor, q_off: int, rq: int, kv_off: int, rk: int, dr: int, q_gain: torch.Tensor,
                kv_gain: torch.Tensor, eps: float, positions: torch.Tensor, freq: torch.Tensor | None, rot_dims: int,
                slot_mapping: torch.Tensor | None, cache: torch.Tensor | None, cq_out: torch.Tensor | None,
                rot_gain: float = 1.0) -> None:
    """Per token of the stacked down-projection rows ``proj``: RMS norm of the query latent (columns q_off..+rq) into
    ``cq_out`` (None, with ``q_gain`` None and ``rq`` 0: the rows hold no query latent); RMS norm of the key/value latent
    (kv_off..+rk) and interleaved rotary encoding of the ``dr`` columns after it (cosine and sine times ``rot_gain``),
    both written to the token's slot of ``cache[page, 0, 0, slot, rk + dr]`` (if a cache is given)."""
    T, stride = proj.shape
    if cq_out is None:
        if rq != 0 or q_gain is not None:
            raise KernelError("latent_prep: a query latent needs a place for its norm")
        q_gain = kv_gain
    elif cq_out.shape != (T, rq) or cq_out.dtype != proj.dtype or cq_out.stride(1) != 1:
        raise KernelError("latent_prep: rows do not fit")
    if proj.stride(1) != 1:
        raise KernelError("latent_prep: rows do not fit")
    if (cq_out is not None and q_gain.numel() != rq) or kv_gain.numel() != rk or q_gain.dtype != kv_gain.dtype:
        raise KernelError("latent_prep: gains do not fit the latents")
    slots = 0
    if cache is not None:
        if cache.dim() != 5 or tuple(cache.shape[1:3]) != (1, 1) or cache.shape[4] != rk + dr or cache.dtype != proj.dtype:
            raise KernelError(f"latent_prep: cache must be [pages, 1, 1, page_size, {rk + dr}] of the rows' dtype, got {list(cache.shape)}")
        if slot_mapping is None:
            raise KernelError("latent_prep: a cache write needs slot_mapping")
        slots = cache.shape[0] * cache.shape[3]
    rc = library().cib_latent_prep(
        _cuda(proj, "proj", contiguous=False), _code(proj, "proj"), proj.stride(0), q_off, rq, kv_off, rk, dr,
        _cuda(q_gain, "q_gain"), _cuda(kv_gain, "kv_gain"), _code(q_gain, "q_gain"), float(eps),
        _cuda(positions, "positions", torch.int32), _cuda(freq, "freq", torch.float32) if freq is not None else None,
        rot_dims if freq is not None else 0, float(rot_gain),
        _cuda(slot_mapping, "slot_mapping", torch.int32) if cache is not None else None,
        _cuda(cache, "cache") if cache is not None else None, slots,
        _cuda(cq_out, "cq_out", contiguous=False) if cq_out is not None else None,
        cq_out.stride(0) if cq_out is not None else 0, T, _stream())
    _check(rc, "latent_prep")
    _count()


def latent_attention_generic(q_abs: torch.Tensor, q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor,
                             block_table: torch.Tensor, query_start_loc: torch.Tensor, seq_lens: torch.Tensor,
                             token_request: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor | None, rot_dims: int,
                             sinks: torch.Tensor | None, num_heads: int, dn: int, rk: int, dr: int, scale: float,
                             window: int = 0, rot_gain: float = 1.0) -> None:
    """Causal multi-query attention over cached latent rows ``[c | k_rot]``: ``q_abs[T, H*rk]`` are the queries with the
    key up-projection folded in, ``q[T, H*(dn+dr)]`` holds each head's rotary part (encoded by the kernel), ``out[T, H*rk]``
    the weighted sums of the latents.  ``sinks[H]``: per-head scores that only join the softmax denominator.
    ``window`` w > 0: query i sees key j only when ``i - j < w``; ``rot_gain``: a factor on the rotation's cosine and sine."""
    T = q.shape[0]
    if q_abs.shape != (T, num_heads * rk) or out.shape != (T, num_heads * rk) or q.shape[1] != num_heads * (dn + dr):
        raise KernelError("latent_attention: q_abs / q / out do not fit the sizes")
    if q_abs.stride(1) != 1 or q.stride(1) != 1 or out.stride(1) != 1 or out.dtype != q.dtype or cache.dtype != q.dtype:
        raise KernelError("latent_attention: rows must be dense and of one dtype")
    if cache.dim() != 5 or tuple(cache.shape[1:3]) != (1, 1) or cache.shape[4] != rk + dr:
        raise KernelError(f"latent_attention: cache must be [pages, 1, 1, page_size, {rk + dr}], got {list(cache.shape)}")
    if sinks is not None and sinks.numel() != num_heads:
        raise KernelError("latent_attention: one sink per head")
    rc = library().cib_latent_attention_generic(
        _cuda(q_abs, "q_abs", contiguous=False), _code(q_abs, "q_abs"), q_abs.stride(0), _cuda(q, "q", contiguous=False),
        _code(q, "q"), q.stride(0), dn, _cuda(out, "out", contiguous=False), out.stride(0), _cuda(cache, "cache"),
        cache.shape[0], cache.shape[3], _cuda(block_table, "block_table", torch.int32), block_table.stride(0),
        _cuda(query_start_loc, "query_start_loc", torch.int32), _cuda(seq_lens, "seq_lens", torch.int32),
        _cuda(token_request, "token_request", torch.int32), _cuda(positions, "positions", torch.int32),
        _cuda(freq, "freq", torch.float32) if freq is not None else None, rot_dims if freq is not None else 0, float(rot_gain),
        _cuda(sinks, "sinks") if sinks is not None else None, _code(sinks, "sinks") if sinks is not None else 0,
        T, num_heads, rk, dr, float(scale), int(window), _stream())
    _check(rc, "latent_attention_generic")
    _count()


def latent_attention_mma_supports(rk: int, dr: int, dn: int) -> bool:
    return bool(library().cib_latent_attention_mma_supports(rk, dr, dn))


def latent_attention_splits(row_tiles: int, head_blocks: int, max_seq_len: int, ctas: int = 296) -> int:
    """Over how many CTAs the keys of one query tile are split: enough to occupy the GPU when the tiles alone do not (a
    decode step), each split keeping at least 64 keys."""
    base = max(1, row_tiles * head_blocks)
    if base >= ctas // 2:
        return 1
    return max(1, min(ctas // base, max_seq_len // 64, 64))


def latent_attention_mma(q_abs: torch.Tensor, q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor,
                         block_table: torch.Tensor, query_start_loc: torch.Tensor, seq_lens: torch.Tensor,
                         query_lens: list, freq: torch.Tensor | None, rot_dims: int, sinks: torch.Tensor | None,
                         num_heads: int, dn: int, rk: int, dr: int, scale: float, max_seq_len: int,
                         decode_only: bool = False, window: int = 0, rot_gain: float = 1.0) -> None:
    """The bfloat16 tensor-core form of :func:`latent_attention_generic` (same operands, ``q_abs`` in bfloat16).  ``query_lens``: tokens per request as host integers, an upper bound in a captured step (CTAs that find
    no request leave); ``max_seq_len``: the longest context, which decides how a decode step's keys are split;
    ``decode_only``: every request brings one token (query tiles of 32 rows then, when the heads fit)."""
    T = q.shape[0]
    R = seq_lens.numel()
    if q_abs.shape != (T, num_heads * rk) or out.shape != (T, num_heads * rk) or q.shape[1] != num_heads * (dn + dr):
        raise KernelError("latent_attention: q_abs / q / out do not fit the sizes")
    for name, t in (("q_abs", q_abs), ("q", q), ("out", out), ("cache", cache)):
        if t.dtype != torch.bfloat16 or t.stride(-1) != 1:
            raise KernelError(f"latent_attention_mma: {name} must be bfloat16 with dense rows")
    if cache.dim() != 5 or tuple(cache.shape[1:3]) != (1, 1) or cache.shape[4] != rk + dr:
        raise KernelError(f"latent_attention: cache must be [pages, 1, 1, page_size, {rk + dr}], got {list(cache.shape)}")
    if sinks is not None and (sinks.numel() != num_heads or sinks.dtype != torch.float32):
        raise KernelError("latent_attention_mma: one 32-bit sink per head")
    lib = library()
    lens = (ctypes.c_int * len(query_lens))(*query_lens)
    tile_rows = 32 if decode_only and num_heads <= 32 else 64
    tiles = lib.cib_latent_attention_mma_tiles(lens, len(query_lens), num_heads, tile_rows)
    head_blocks = -(-num_heads // 64) if num_heads > 64 else 1
    # with a window a query tile reads at most the window and its own tokens' keys
    reach = min(max_seq_len, window + tile_rows) if window else max_seq_len
    splits = latent_attention_splits(tiles, head_blocks, reach)
    scratch = torch.empty(T * num_heads * splits * (rk + 2), dtype=torch.float32, device=q.device) if splits > 1 else None
    rc = lib.cib_latent_attention_mma(
        _cuda(q_abs, "q_abs", contiguous=False), q_abs.stride(0), _cuda(q, "q", contiguous=False), q.stride(0), dn,
        _cuda(out, "out", contiguous=False), out.stride(0), _cuda(scratch, "scratch") if scratch is not None else None,
        _cuda(cache, "cache"), cache.shape[0], cache.shape[3], _cuda(block_table, "block_table", torch.int32),
        block_table.stride(0), _cuda(query_start_loc, "query_start_loc", torch.int32), _cuda(seq_lens, "seq_lens", torch.int32),
        R, tiles, tile_rows, _cuda(freq, "freq", torch.float32) if freq is not None else None, rot_dims if freq is not None else 0,
        _cuda(sinks, "sinks") if sinks is not None else None, T, num_heads, rk, dr, float(scale), splits, float(rot_gain),
        int(window), _stream())
    _check(rc, "latent_attention_mma")
    _count()
    if splits > 1:
        _count()


_decode_counters: dict = {}
_retired: list = []


def paged_attention_decode_supports(head_dim: int, num_q_heads: int, num_kv_heads: int) -> bool:
    return bool(library().cib_paged_attention_decode_supports(head_dim, num_q_heads, num_kv_heads))


# CUINFER_B200_DECODE_TMA=0 keeps the decode attention kernel on its cp.async path (for comparisons).
decode_tma = os.environ.get("CUINFER_B200_DECODE_TMA", "1") != "0"


DECODE_TMA_MIN_KEYS = int(os.environ.get("CUINFER_B200_DECODE_TMA_MIN_KEYS", "1024"))      # keys per CTA from which the TMA path of the decode kernel pays inside a step (measured)


def decode_tma_takes(page_size: int, head_dim: int, window: int) -> bool:
    """Whether the decode attention can stream its keys and values as TMA page boxes for this cache layout (else
    cp.async only): whole 16-slot blocks inside a page, 64-column panels, no window."""
    return decode_tma and page_size % 16 == 0 and head_dim % 64 == 0 and window <= 0


def decode_uses_tma(max_seq_len: int, splits: int) -> bool:
    """The TMA path streams faster, but it starts later after the kernel before it in a step (the cp.async path asks
    for its first blocks before that kernel has ended): timed alone it wins at every size, inside a decode step only
    for long streams per CTA (batch 1 with 26 CTAs of 160 keys per head: 919 tokens/s against 974 on cp.async)."""
    return -(-max_seq_len // splits) >= DECODE_TMA_MIN_KEYS


def decode_slots(head_dim: int) -> int:
    """CTAs of the decode attention kernel that the GPU runs at a time: its key and value rings take 768 bytes per
    value of the head size, so one CTA per SM at head size 256, two at 128, and three (by registers) below."""
    return 148 * (1 if head_dim > 128 else 2 if head_dim > 64 else 3)


def decode_splits(num_requests: int, num_kv_heads: int, max_seq_len: int, slots: int = 296, tma: bool = False,
                  head_dim: int = 128) -> int:
    """How many CTAs share the keys of one (request, kv head).  ``tma``: the cache layout allows the TMA path, which
    a split then takes if it leaves a CTA ``DECODE_TMA_MIN_KEYS`` keys or more.

    The GPU runs ``slots`` CTAs of this kernel at a time (two on each of the 148 SMs); a CTA's four warps take
    16-key blocks in turn, so a CTA's share counts in steps of 64 keys.  A launch is estimated, in nanoseconds, round
    of CTAs by round: a round of n CTAs takes keys per CTA x (the larger of a CTA's own pace per key and n x 0.072, the
    memory's pace when n CTAs stream at once) plus a fixed cost for a CTA's start and its partial results; splitting
    adds 3000 for the combine and 40 per split.  A CTA's own pace is 16 per key and 3000 fixed on the TMA path, 18 and
    4000 on the cp.async path.  The constants were fitted to timings at batch 1 to 128 with 300 to 9000 keys of head
    size 128 (largest miss 1.7 us, 9 % r.m.s. error of the estimate); for another head size the costs per key scale
    with the bytes of a key.  The smallest estimate wins.
    """
    pairs = max(1, num_requests * num_kv_heads)
    width = head_dim / 128.0
    best, best_cost = 1, None
    for s in range(1, 65):
        keys = -(-(-(-max_seq_len // s)) // 64) * 64
        if s > 1 and (s - 1) * keys >= max_seq_len:
            continue                                   # the last CTA would get nothing: a smaller s does the same
        per_key, fixed = (16.0 * width, 3000.0) if tma and decode_uses_tma(max_seq_len, s) else (18.0 * width, 4000.0)
        full, rest = divmod(pairs * s, slots)
        cost = full * (keys * max(per_key, 0.072 * width * slots) + fixed)
        if rest:
            cost += keys * max(per_key, 0.072 * width * rest) + fixed
        if s > 1:
            cost += 3000.0 + 40.0 * s
        if best_cost is None or cost < best_cost:
            best, best_cost = s, cost
    return best


# A kernel of the decode chain may ask for the weights of the kernel after it to be fetched into the L2 while it runs.
# That pays where the chain is bound by latencies and the weights are small beside the 126 MB L2 (every matrix of the
# 0.6B layer sizes is under 13 MB).  Matrices of 33 to 200 MB (the 8B layer sizes) would compete with the running
# kernel's own stream and could not stay in the L2 until they are used, so larger ones are not asked for.
L2_HINT_MAX_BYTES = 16 << 20


def _l2_hint(warm: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    if warm is None or warm.numel() * warm.element_size() > L2_HINT_MAX_BYTES:
        return None
    return warm


def paged_attention_decode(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                           seq_lens: torch.Tensor, num_q_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                           window: int, splits: int, tma: bool | None = None, warm: torch.Tensor | None = None) -> None:
    """bfloat16 attention of one query token per request (``q[r, :nq*d]``) over the paged cache, the keys of
    every (request, kv head) split over ``splits`` CTAs.  Allocates the partial-result scratch with torch.
    ``tma``: let the kernel fetch the cache through TMA where the geometry allows it (default: yes).  That path
    streams faster but starts slower, so callers that know the keys per CTA pass False for short streams.
    ``warm``: a tensor that the kernel after this one reads first; fetched into the L2 when the stream of keys ends."""
    R = q.shape[0]
    warm = _l2_hint(warm)
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError("paged_attention_decode: bfloat16 only")
    if q.stride(1) != 1 or out.stride(1) != 1 or out.shape != (R, num_q_heads * head_dim):
        raise KernelError("paged_attention_decode: q/out rows must be dense and out [R, nq*d]")
    scratch = None
    counters = None
    if splits > 1:
        n = library().cib_paged_attention_decode_scratch_floats(R, num_q_heads, head_dim, splits)
        scratch = torch.empty(n, dtype=torch.float32, device=q.device)
        need = R * num_kv_heads
        counters = _decode_counters.get(q.device.index)
        if counters is None or counters.numel() < need:
            if torch.cuda.is_current_stream_capturing():
                raise KernelError("paged_attention_decode: the split counters must exist before a graph capture "
                                  "(run the step once eagerly first)")
            if counters is not None:
                _retired.append(counters)      # a captured graph may still point at the old buffer
            counters = torch.zeros(max(need, 4096), dtype=torch.int32, device=q.device)
            _decode_counters[q.device.index] = counters
    rc = library().cib_paged_attention_decode(
        _cuda(q, "q", contiguous=False), q.stride(0), _cuda(out, "out", contiguous=False), out.stride(0),
        _cuda(cache, "cache"), cache.shape[0], cache.shape[3], _cuda(block_table, "block_table", torch.int32),
        block_table.stride(0), _cuda(seq_lens, "seq_lens", torch.int32), R, num_q_heads, num_kv_heads, head_dim,
        float(scale), int(window), int(splits), scratch.data_ptr() if scratch is not None else None,
        counters.data_ptr() if counters is not None else None, 1 if use_pdl else 0,
        _error_flag(q.device).data_ptr() if decode_tma and tma is not False else None,
        warm.data_ptr() if warm is not None else None, warm.numel() * warm.element_size() if warm is not None else 0,
        _stream())
    _check(rc, "paged_attention_decode")
    note_flagged_launch()
    _count()


def paged_attention_prefill_supports(head_dim: int, num_q_heads: int, num_kv_heads: int) -> bool:
    return bool(library().cib_paged_attention_prefill_supports(head_dim, num_q_heads, num_kv_heads))


def paged_attention_prefill(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                            query_start_loc: torch.Tensor, seq_lens: torch.Tensor, query_lens_host, num_q_heads: int,
                            num_kv_heads: int, head_dim: int, scale: float, window: int = 0) -> None:
    """bfloat16 tensor-core attention for any mix of prompt portions and decoded tokens.
    ``query_lens_host``: tokens each request brings in this step (host ints), to size the grid."""
    T = q.shape[0]
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError("paged_attention_prefill: bfloat16 only")
    if q.stride(1) != 1 or out.stride(1) != 1 or out.shape != (T, num_q_heads * head_dim):
        raise KernelError("paged_attention_prefill: q/out rows must be dense and out [T, nq*d]")
    g = num_q_heads // num_kv_heads
    # CTAs take 64-row tiles one by one, or in pairs (tile p with tile t-1-p: equal work under the causal mask)
    # when the pairs alone still fill the GPU
    paired = sum(((n * g + 63) // 64 + 1) // 2 for n in query_lens_host)
    pair = 1 if paired * num_kv_heads >= 200 else 0
    tiles = paired if pair else sum((n * g + 63) // 64 for n in query_lens_host)
    rc = library().cib_paged_attention_prefill(
        _cuda(q, "q", contiguous=False), q.stride(0), _cuda(out, "out", contiguous=False), out.stride(0),
        _cuda(cache, "cache"), cache.shape[0], cache.shape[3], _cuda(block_table, "block_table", torch.int32),
        block_table.stride(0), _cuda(query_start_loc, "query_start_loc", torch.int32),
        _cuda(seq_lens, "seq_lens", torch.int32), len(query_lens_host), tiles, num_q_heads, num_kv_heads, head_dim,
        float(scale), int(window), pair, _stream())
    _check(rc, "paged_attention_prefill")
    _count()


# ---- matrix product ----------------------------------------------------------------------------------

def gemm_generic(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T with 32-bit FMA accumulation, any sizes."""
    M, K = a.shape
    N, K2 = w.shape
    if K != K2 or out.shape != (M, N) or a.dtype != w.dtype:
        raise KernelError(f"gemm: a {list(a.shape)} {a.dtype}, w {list(w.shape)} {w.dtype}, out {list(out.shape)} do not fit")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm: rows must be dense")
    rc = library().cib_gemm_generic(
        _cuda(a, "a", contiguous=False), a.stride(0), _cuda(w, "w", contiguous=False), w.stride(0), _code(a, "a"),
        _cuda(out, "out", contiguous=False), out.stride(0), _code(out, "out"), M, N, K, _stream())
    _check(rc, "gemm_generic")
    _count()


def gemm_generic_batched(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[b, M, N] = a[b, M, K] @ w[b, N, K]^T for every b, 32-bit FMA accumulation, any sizes.  The three tensors
    may be strided views (heads side by side inside wider rows); only their last axis must be dense."""
    B, M, K = a.shape
    B2, N, K2 = w.shape
    if B != B2 or K != K2 or out.shape != (B, M, N) or a.dtype != w.dtype:
        raise KernelError(f"gemm: a {list(a.shape)} {a.dtype}, w {list(w.shape)} {w.dtype}, out {list(out.shape)} do not fit")
    if a.stride(2) != 1 or w.stride(2) != 1 or out.stride(2) != 1:
        raise KernelError("gemm: rows must be dense")
    rc = library().cib_gemm_generic_batched(
        _cuda(a, "a", contiguous=False), a.stride(1), a.stride(0), _cuda(w, "w", contiguous=False), w.stride(1), w.stride(0),
        _code(a, "a"), _cuda(out, "out", contiguous=False), out.stride(1), out.stride(0), _code(out, "out"), M, N, K, B, _stream())
    _check(rc, "gemm_generic_batched")
    _count()


# (token, choice) rows from which the experts' products run grouped by expert on the tensor cores; below, a token's
# experts are streamed once per token (a decode step)
MOE_GROUPED_MIN_ROWS = 128


def moe_table_feed_forward(h: torch.Tensor, ids: torch.Tensor | None, table: torch.Tensor, gate_up: torch.Tensor,
                           down: torch.Tensor, base: torch.Tensor | None, out: torch.Tensor,
                           weights: torch.Tensor | None = None, clamp_limit: float | None = None, activation: str | None = None,
                           base_gate: torch.Tensor | None = None) -> None:
    """out[t] = base[t] + (1/top) * sum over k of expert(table[ids[t], k])(h[t]) with gated experts
    (``ids`` None: the table has a row per row of ``h`` — experts chosen by a router; ``weights`` float32 [T, top]:
    a weight per choice instead of 1/top; ``clamp_limit``: the experts' activation is
    ``g * sigmoid(1.702 g) * (u + 1)`` with ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)``)
    ``down_e(silu(gate_e h) * up_e h)``; ``gate_up[E, 2 ff, W]`` (gate rows first), ``down[E, W, ff]``, ``table[V, top]``.
    ``activation="relu2"``: experts without a gate, ``down_e(relu(up_e h) ** 2)``, whose first matrix is ``[E, ff, W]``.
    ``base_gate`` float32 [T] (any stride): ``base[t]`` is multiplied by ``sigmoid(base_gate[t])`` as it is added.
    Few rows, 32-bit, or sizes that are not multiples of 32: two launches (a matrix-vector product per token and
    choice).  Many bfloat16 rows: grouped by expert (see ``MOE_GROUPED_MIN_ROWS``)."""
    T, W = h.shape
    if activation not in (None, "relu2"):
        raise KernelError(f"moe_table: activation {activation!r} is not one of the experts' forms")
    E, two_ff, W2 = gate_up.shape
    ff = two_ff if activation == "relu2" else two_ff // 2
    V, top = table.shape
    if W2 != W or down.shape != (E, W, ff) or out.shape != (T, W) or not (h.dtype == gate_up.dtype == down.dtype == out.dtype):
        raise KernelError("moe_table: weights, rows and out do not fit")
    if h.stride(1) != 1 or (base is not None and (base.shape != (T, W) or base.stride(1) != 1 or base.dtype != h.dtype)):
        raise KernelError("moe_table: rows must be dense and of one dtype")
    if ids is None and V != T:
        raise KernelError("moe_table: without token ids the table needs a row per row of h")
    if weights is not None and weights.shape != (T, top):
        raise KernelError("moe_table: weights must be [rows, top]")
    p_ids = _cuda(ids, "ids", torch.int32) if ids is not None else None
    p_w = _cuda(weights, "weights", torch.float32) if weights is not None else None
    act_kind, limit = (1, float(clamp_limit)) if clamp_limit is not None else (0, 0.0)
    if activation == "relu2":
        act_kind, limit = 2, 0.0
    if base_gate is not None and (base is None or base_gate.shape != (T,)):
        raise KernelError("moe_table: a gate for base needs base and one number per row")
    p_bg = _cuda(base_gate, "base_gate", torch.float32, contiguous=False) if base_gate is not None else None
    bg_stride = base_gate.stride(0) if base_gate is not None else 0
    lib = library()
    if (h.dtype == torch.bfloat16 and T * top >= MOE_GROUPED_MIN_ROWS and h.stride(0) % 8 == 0
            and lib.cib_moe_table_grouped_supports(W, ff, E)):
        # many rows: sorted by expert on the device, one tensor-core product per expert group (four launches)
        act = torch.empty((T * top, ff), dtype=h.dtype, device=h.device)
        y = torch.empty((T * top, W), dtype=h.dtype, device=h.device)
        ints = torch.empty(lib.cib_moe_table_grouped_workspace_ints(T, top, E), dtype=torch.int32, device=h.device)
        rc = lib.cib_moe_table_grouped(
            _cuda(h, "h", contiguous=False), h.stride(0), p_ids, _cuda(table, "table", torch.int32), V, top, E,
            _cuda(gate_up, "gate_up"), _cuda(down, "down"), _cuda(base, "base", contiguous=False) if base is not None else None,
            base.stride(0) if base is not None else 0, 1.0 / top, p_w, p_bg, bg_stride, _cuda(out, "out"), _cuda(act, "act"), _cuda(y, "y"),
            _cuda(ints, "ints"), T, W, ff, act_kind, limit, _stream())
        _check(rc, "moe_table_grouped")
        for _ in range(4):
            _count()
        return
    act = torch.empty((T, top, ff), dtype=h.dtype, device=h.device)
    rc = lib.cib_moe_table_gate_up(_cuda(h, "h", contiguous=False), h.stride(0), _code(h, "h"), p_ids,
                                   _cuda(table, "table", torch.int32), V, top, E, _cuda(gate_up, "gate_up"), _cuda(act, "act"),
                                   T, W, ff, act_kind, limit, _stream())
    _check(rc, "moe_table_gate_up")
    rc = lib.cib_moe_table_down(_cuda(act, "act"), _code(act, "act"), p_ids, _cuda(table, "table", torch.int32),
                                V, top, E, _cuda(down, "down"), _cuda(base, "base", contiguous=False) if base is not None else None,
                                base.stride(0) if base is not None else 0, 1.0 / top, p_w, p_bg, bg_stride, _cuda(out, "out"), T, W, ff, _stream())
    _check(rc, "moe_table_down")
    _count()
    _count()


# Programmatic dependent launch for the kernels that support it: such a kernel may start, and prefetch its
# weights, while the kernel before it in the stream is still running; it reads that kernel's results only after
# `griddepcontrol.wait`.  CUINFER_B200_PDL=0 switches it off.
use_pdl = os.environ.get("CUINFER_B200_PDL", "1") != "0"

EPILOGUE_BF16, EPILOGUE_F32, EPILOGUE_SILU_PAIR = 0, 1, 2
EPILOGUE_GELU_PAIR = 3          # as the SiLU pair, with the tanh form of GELU as the gate


def gemm_skinny_supports(M: int, N: int, K: int, with_norm: bool = False) -> bool:
    return bool(library().cib_gemm_skinny_supports(M, N, K, 1 if with_norm else 0))


def gemm_skinny(w: torch.Tensor, out: torch.Tensor, *, act: torch.Tensor | None = None,
                residual: torch.Tensor | None = None, pending: torch.Tensor | None = None,
                norm_weight: torch.Tensor | None = None, eps: float = 0.0, residual_out: torch.Tensor | None = None,
                silu_pair: bool = False, warm: torch.Tensor | None = None) -> None:
    """out = act @ w^T for at most 16 rows, bfloat16 weights.  ``warm``: a tensor that the kernel after this one
    reads first (its weights); the kernel asks for it to be fetched into the L2 while it runs.

    Either ``act`` [M, K] is given, or ``residual`` (float32 [M, K]) with optional ``pending``: then the rows are
    RMSNorm(residual + pending) * norm_weight, computed in the kernel, and ``residual_out`` (another buffer)
    receives residual + pending.  ``silu_pair``: ``w`` is [2I, K] = gates then ups and out [M, I] = silu(g) * u.
    ``out`` float32 selects the 32-bit store."""
    N, K = w.shape
    M = out.shape[0]
    warm = _l2_hint(warm)
    if w.dtype != torch.bfloat16 or w.stride(1) != 1:
        raise KernelError("gemm_skinny: weights must be bfloat16 with dense rows")
    if silu_pair:
        epi = EPILOGUE_GELU_PAIR if silu_pair == "gelu_tanh" else EPILOGUE_SILU_PAIR
        if out.dtype != torch.bfloat16 or out.shape[1] * 2 != N:
            raise KernelError("gemm_skinny: a gate/up pair writes bfloat16 [M, N/2]")
    else:
        if out.shape[1] != N:
            raise KernelError(f"gemm_skinny: out must be [M, {N}]")
        epi = EPILOGUE_F32 if out.dtype == torch.float32 else EPILOGUE_BF16
        if out.dtype not in (torch.float32, torch.bfloat16):
            raise KernelError("gemm_skinny: out must be bfloat16 or float32")
    if out.stride(1) != 1:
        raise KernelError("gemm_skinny: out rows must be dense")
    if act is not None:
        if act.dtype != torch.bfloat16 or act.shape != (M, K) or act.stride(1) != 1:
            raise KernelError("gemm_skinny: act must be bfloat16 [M, K] with dense rows")
    else:
        if residual is None or residual.dtype != torch.float32 or residual.shape != (M, K) or not residual.is_contiguous():
            raise KernelError("gemm_skinny: residual must be contiguous float32 [M, K]")
        if pending is not None and (pending.shape != (M, K) or not pending.is_contiguous()):
            raise KernelError("gemm_skinny: pending must be contiguous [M, K]")
        if norm_weight is None or norm_weight.numel() != K:
            raise KernelError("gemm_skinny: the norm needs K weights")
        if residual_out is not None and (residual_out.shape != (M, K) or residual_out.dtype != torch.float32
                                         or residual_out.data_ptr() == residual.data_ptr()):
            raise KernelError("gemm_skinny: residual_out must be another float32 [M, K] buffer")
    rc = library().cib_gemm_skinny(
        _cuda(w, "w", contiguous=False), w.stride(0), N, K,
        _cuda(act, "act", contiguous=False) if act is not None else None, act.stride(0) if act is not None else 0,
        _cuda(residual, "residual") if residual is not None else None,
        _cuda(pending, "pending") if pending is not None else None, _code(pending, "pending") if pending is not None else 0,
        _cuda(norm_weight, "norm_weight") if norm_weight is not None else None,
        _code(norm_weight, "norm_weight") if norm_weight is not None else 0, float(eps),
        _cuda(residual_out, "residual_out") if residual_out is not None else None,
        _cuda(out, "out", contiguous=False), out.stride(0), M, epi, N // 2 if silu_pair else 0, 1 if use_pdl else 0,
        warm.data_ptr() if warm is not None else None, warm.numel() * warm.element_size() if warm is not None else 0,
        _stream())
    _check(rc, "gemm_skinny")
    _count()


_error_flags: dict = {}


def _error_flag(device: torch.device) -> torch.Tensor:
    """One int per device that kernels with bounded waits raise instead of hanging."""
    flag = _error_flags.get(device.index)
    if flag is None:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the device error flag must exist before a graph capture (run the step once eagerly first)")
        flag = torch.zeros(1, dtype=torch.int32, device=device)
        _error_flags[device.index] = flag
    return flag


_flagged_launches = 0
_unchecked_steps = 0
CHECK_EVERY = 32          # a captured step that is replayed is looked at this often, not after every replay


def note_flagged_launch(replayed: bool = False) -> None:
    """Record that a kernel with bounded waits has run.  ``replayed``: it ran as part of a replayed CUDA graph, which
    happens every decode step; the flag is then read only every ``CHECK_EVERY`` steps (and whenever ``force`` is given),
    so that a step does not pay a device-to-host read for it."""
    global _flagged_launches, _unchecked_steps
    if replayed:
        _unchecked_steps += 1
    else:
        _flagged_launches += 1


def check_error_flags(force: bool = False) -> None:
    """Raise if a kernel gave up on a bounded wait since the last check.  Reads one int per device (which
    synchronises), but only if such a kernel was launched since the last check."""
    global _flagged_launches, _unchecked_steps
    if _flagged_launches == 0 and not (_unchecked_steps >= CHECK_EVERY or (force and _unchecked_steps)):
        return
    _flagged_launches = 0
    _unchecked_steps = 0
    for index, flag in _error_flags.items():
        code = int(flag.item())
        if code:
            flag.zero_()
            raise KernelError(f"a kernel on cuda:{index} gave up waiting on a barrier (code {code}); its results are invalid")


def selftest_bounded_wait(limit_cycles: int = 1_000_000, device: torch.device | str = "cuda:0",
                          gave_up: torch.Tensor | None = None) -> None:
    """Run the kernels' bounded mbarrier wait on a barrier that never completes (it gives up after ``limit_cycles``
    and raises the device's error word); the next ``check_error_flags`` must then raise.  For tests of the failure
    path: a healthy kernel never takes it."""
    device = torch.device(device)
    rc = library().cib_selftest_bounded_wait(int(limit_cycles), _error_flag(device).data_ptr(),
                                             _cuda(gave_up, "gave_up", torch.int32) if gave_up is not None else None, _stream())
    _check(rc, "selftest_bounded_wait")
    note_flagged_launch()
    _count()


def attention_tcgen05_supports(head_dim: int, num_q_heads: int, num_kv_heads: int, page_size: int) -> bool:
    return bool(library().cib_attention_tcgen05_supports(head_dim, num_q_heads, num_kv_heads, page_size))


def attention_tcgen05(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                      query_start_loc: torch.Tensor, seq_lens: torch.Tensor, query_lens_host, num_q_heads: int,
                      num_kv_heads: int, head_dim: int, scale: float, window: int = 0, *, joined: bool = False,
                      sinks: torch.Tensor | None = None) -> None:
    """bfloat16 attention for prompt portions on tcgen05 tensor cores (head size 128, pages of 8, 16, 32, ...
    slots): scores and output accumulate in tensor memory, keys and values come page by page through TMA.
    ``cache`` is ``[pages, 2, kv heads, page, 128]`` (keys, values) or, with ``joined``, ``[pages, 1, kv heads, page, 256]``
    with a token's key and value side by side; ``sinks`` float32 [query heads]: ``exp(sink)`` joins a row's denominator."""
    T = q.shape[0]
    planes, row = (1, 2 * head_dim) if joined else (2, head_dim)
    if cache.dim() != 5 or cache.shape[1] != planes or cache.shape[2] != num_kv_heads or cache.shape[4] != row:
        raise KernelError(f"attention_tcgen05: cache must be [pages, {planes}, {num_kv_heads}, page, {row}], got {list(cache.shape)}")
    if sinks is not None and (sinks.dtype != torch.float32 or sinks.numel() != num_q_heads):
        raise KernelError("attention_tcgen05: one 32-bit sink per query head")
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError("attention_tcgen05: bfloat16 only")
    if q.stride(1) != 1 or out.stride(1) != 1 or out.shape != (T, num_q_heads * head_dim) or not cache.is_contiguous():
        raise KernelError("attention_tcgen05: q/out rows must be dense, out [T, nq*d], cache contiguous")
    g = num_q_heads // num_kv_heads
    tiles = sum((n * g + 127) // 128 for n in query_lens_host)
    rc = library().cib_attention_tcgen05(
        _cuda(q, "q", contiguous=False), q.stride(0), _cuda(out, "out", contiguous=False), out.stride(0),
        _cuda(cache, "cache"), cache.shape[0], cache.shape[3], _cuda(block_table, "block_table", torch.int32),
        block_table.stride(0), _cuda(query_start_loc, "query_start_loc", torch.int32),
        _cuda(seq_lens, "seq_lens", torch.int32), len(query_lens_host), tiles, num_q_heads, num_kv_heads, head_dim,
        float(scale), int(window), 1 if joined else 0, _cuda(sinks, "sinks") if sinks is not None else None,
        _error_flag(q.device).data_ptr(), _stream())
    _check(rc, "attention_tcgen05")
    note_flagged_launch()
    _count()


def gemm_wstream_supports(M: int, N: int, K: int) -> bool:
    return bool(library().cib_gemm_wstream_supports(M, N, K))


def gemm_wstream(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, silu_pair: bool = False) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T for up to 128 rows on tcgen05 tensor cores with the weights as the streamed
    128-row operand (bfloat16 in, bfloat16 or float32 out).  ``silu_pair``: w holds N/2 gate rows then N/2 up rows and
    out[M, N/2] = silu(gate) * up (bfloat16)."""
    M, K = a.shape
    N, K2 = w.shape
    out_cols = N // 2 if silu_pair else N
    if K != K2 or out.shape != (M, out_cols) or a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"gemm_wstream: a {list(a.shape)} {a.dtype}, w {list(w.shape)} {w.dtype}, out {list(out.shape)} do not fit")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1 or out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("gemm_wstream: rows must be dense and out bfloat16 or float32")
    if silu_pair and (N % 2 or out.dtype != torch.bfloat16):
        raise KernelError("gemm_wstream: the gated epilogue needs an even N and a bfloat16 result")
    epilogue = 2 if silu_pair else (1 if out.dtype == torch.float32 else 0)
    rc = library().cib_gemm_wstream(
        _cuda(a, "a", contiguous=False), a.stride(0), _cuda(w, "w", contiguous=False), w.stride(0),
        _cuda(out, "out", contiguous=False), out.stride(0), epilogue, M, N, K, 1 if use_pdl else 0,
        _error_flag(a.device).data_ptr(), _stream())
    _check(rc, "gemm_wstream")
    note_flagged_launch()
    _count()


def gemm_tcgen05_supports(M: int, N: int, K: int) -> bool:
    return bool(library().cib_gemm_tcgen05_supports(M, N, K))


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, silu_pair: bool = False) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T on tcgen05 tensor cores (bfloat16 in, bfloat16 or float32 out).
    ``silu_pair``: w holds N/2 gate rows then N/2 up rows and out[M, N/2] = silu(gate) * up (bfloat16)."""
    M, K = a.shape
    N, K2 = w.shape
    out_cols = N // 2 if silu_pair else N
    if K != K2 or out.shape != (M, out_cols) or a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"gemm_tcgen05: a {list(a.shape)} {a.dtype}, w {list(w.shape)} {w.dtype}, out {list(out.shape)} do not fit")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1 or out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("gemm_tcgen05: rows must be dense and out bfloat16 or float32")
    if silu_pair and (N % 2 or out.dtype != torch.bfloat16 or out.stride(0) % 8 or out.data_ptr() % 16):
        raise KernelError("gemm_tcgen05: the gated epilogue needs an even N and 16-byte aligned bfloat16 rows")
    rc = library().cib_gemm_tcgen05(
        _cuda(a, "a", contiguous=False), a.stride(0), _cuda(w, "w", contiguous=False), w.stride(0),
        _cuda(out, "out", contiguous=False), out.stride(0), 1 if out.dtype == torch.float32 else 0,
        (2 if silu_pair == "gelu_tanh" else 1) if silu_pair else 0, M, N, K, _error_flag(a.device).data_ptr(), _stream())
    _check(rc, "gemm_tcgen05")
    note_flagged_launch()
    _count()


# ---- random weights ------------------------------------------------------------------------------------

def fill_random(out: torch.Tensor, key: int, mean: float, std: float, factor: float = 1.0, via_bf16: bool = False) -> None:
    """out.flat[i] = factor * (mean + std * z(key, i)), z approximately standard normal and a function of (key, i)
    alone (``cuinfer_b200.weights.random_init.counter_normal`` computes the same values on the host)."""
    rc = library().cib_fill_random(_cuda(out, "out"), _code(out, "out"), out.numel(), int(key) & 0xFFFFFFFFFFFFFFFF,
                                   float(mean), float(std), float(factor), 1 if via_bf16 else 0, _stream())
    _check(rc, "fill_random")
    _count()


# ---- sampling ----------------------------------------------------------------------------------------

def argmax_rows(logits: torch.Tensor, out_ids: torch.Tensor) -> None:
    """out_ids[s] = index of the largest of logits[s] (float32), ties to the lowest index: greedy sampling of every row."""
    S, V = logits.shape
    if logits.stride(1) != 1 or out_ids.numel() < S:
        raise KernelError("argmax_rows: logits rows must be dense and out_ids hold a row each")
    rc = library().cib_argmax_rows(_cuda(logits, "logits", torch.float32, contiguous=False), logits.stride(0), S, V,
                                   _cuda(out_ids, "out_ids", torch.int32), _stream())
    _check(rc, "argmax_rows")
    _count()


def sample(logits: torch.Tensor, params: torch.Tensor, out_ids: torch.Tensor) -> None:
    """out_ids[s] = token drawn from logits[s]; params[s] = (temperature, top_k as int bits, top_p, u)."""
    S, V = logits.shape
    if logits.stride(1) != 1:
        raise KernelError("sample: logits rows must be dense")
    if params.numel() * params.element_size() < S * 16:
        raise KernelError("sample: params must hold 16 bytes per row")
    rc = library().cib_sample(_cuda(logits, "logits", torch.float32, contiguous=False), logits.stride(0), S, V,
                              _cuda(params, "params"), _cuda(out_ids, "out_ids", torch.int32), _stream())
    _check(rc, "sample")
    _count()


# ---- RMS norms around the residual sum, GELU ---------------------------------------------------------------------------

def rms_stream(residual: torch.Tensor, delta: torch.Tensor | None, post: tuple | None, pre: tuple | None,
               out: torch.Tensor | None, raw: torch.Tensor | None = None) -> None:
    """One pass over the 32-bit residual rows: ``residual += rmsnorm(delta) * post_gain`` (``post = (gain, eps)``; a plain
    ``+= delta`` when ``post`` is None), ``raw = residual`` rounded to its dtype, ``out = rmsnorm(residual) * gain``
    with ``pre = (gain, eps)``.  Every part may be left out."""
    rows, H = residual.shape
    for name, t in (("delta", delta), ("out", out), ("raw", raw)):
        if t is not None and t.shape != residual.shape:
            raise KernelError(f"rms_stream: {name} {list(t.shape)} does not match residual {list(residual.shape)}")
    if out is not None and raw is not None and out.dtype != raw.dtype:
        raise KernelError("rms_stream: out and raw must have one dtype")
    if (post is not None and post[0].numel() != H) or (pre is not None and pre[0].numel() != H):
        raise KernelError(f"rms_stream: gains must have {H} elements")
    if out is not None and pre is None:
        raise KernelError("rms_stream: out needs the norm's gain")
    target = out if out is not None else raw
    rc = library().cib_rms_stream(
        _cuda(residual, "residual", torch.float32), _cuda(delta, "delta") if delta is not None else None,
        _code(delta, "delta") if delta is not None else 0,
        _cuda(post[0], "post gain") if post else None, _code(post[0], "post gain") if post else 0, float(post[1]) if post else 0.0,
        _cuda(pre[0], "gain") if pre else None, _code(pre[0], "gain") if pre else 0, float(pre[1]) if pre else 0.0,
        _cuda(out, "out") if out is not None else None, _cuda(raw, "raw") if raw is not None else None,
        _code(target, "out") if target is not None else 0, rows, H, _stream())
    _check(rc, "rms_stream")
    _count()


def gelu_tanh(x: torch.Tensor, out: torch.Tensor, table: torch.Tensor | None = None, ids: torch.Tensor | None = None) -> None:
    """out = gelu_tanh(x) element by element; with ``table`` [V, cols] (rows may be a column range of wider rows) and
    ``ids`` [rows], each row is also multiplied by ``table[ids[row]]``."""
    rows, cols = x.shape
    if out.shape != x.shape or out.dtype != x.dtype or not x.is_contiguous():
        raise KernelError("gelu_tanh: out does not fit x")
    if table is not None and (ids is None or table.shape[1] != cols or table.dtype != x.dtype or table.stride(1) != 1):
        raise KernelError("gelu_tanh: the table does not fit x")
    rc = library().cib_gelu_tanh(
        _cuda(x, "x"), _cuda(table, "table", contiguous=False) if table is not None else None,
        table.stride(0) if table is not None else 0, _cuda(ids, "ids", torch.int32) if table is not None else None,
        table.shape[0] if table is not None else 0, _cuda(out, "out"), _code(x, "x"), rows, cols, _stream())
    _check(rc, "gelu_tanh")
    _count()


def router_topk(logits: torch.Tensor, top: int, choice: torch.Tensor, weight: torch.Tensor) -> None:
    """From float32 logits [T, E]: ``choice`` int32 [T, top] (largest logits first, the lower index wins a tie) and
    ``weight`` float32 [T, top], the softmax over the chosen logits."""
    T, E = logits.shape
    if choice.shape != (T, top) or weight.shape != (T, top) or logits.stride(1) != 1:
        raise KernelError("router_topk: shapes do not fit")
    rc = library().cib_router_topk(_cuda(logits, "logits", torch.float32, contiguous=False), logits.stride(0), E, top,
                                   _cuda(choice, "choice", torch.int32), _cuda(weight, "weight", torch.float32), T, _stream())
    _check(rc, "router_topk")
    _count()


def router_scored_topk(logits: torch.Tensor, top: int, choice: torch.Tensor, weight: torch.Tensor, *,
                       correction: torch.Tensor | None = None, groups: int = 1, keep: int = 1, scale: float = 1.0) -> None:
    """From float32 logits [T, E] with scores ``s = sigmoid(logits)``: ``choice`` int32 [T, top], the experts with the
    largest ``s + correction`` (float32 [E], None: no correction; the lower index wins a tie) among the ``keep`` of
    ``groups`` equal groups of neighbouring experts whose two largest ``s + correction`` sum highest; ``weight`` float32
    [T, top] = ``scale * s`` of the chosen, not renormalised."""
    T, E = logits.shape
    if choice.shape != (T, top) or weight.shape != (T, top) or logits.stride(1) != 1:
        raise KernelError("router_scored_topk: shapes do not fit")
    if correction is not None and (correction.dtype != torch.float32 or correction.numel() != E):
        raise KernelError("router_scored_topk: the correction must be float32 with a number per expert")
    rc = library().cib_router_scored_topk(_cuda(logits, "logits", torch.float32, contiguous=False), logits.stride(0), E, top,
                                          _cuda(correction, "correction") if correction is not None else None, int(groups),
                                          int(keep), float(scale), _cuda(choice, "choice", torch.int32),
                                          _cuda(weight, "weight", torch.float32), T, _stream())
    _check(rc, "router_scored_topk")
    _count()


# ---- attention with a capped score and a window that keeps the first tokens ---------------------------------------------------

def _f32_vec(t: torch.Tensor | None, n: int, what: str):
    """Pointer of an optional float32 vector of ``n`` values (None -> null)."""
    if t is None:
        return None
    if t.dtype != torch.float32 or t.numel() != n:
        raise KernelError(f"{what} must be float32 with {n} values, got {t.dtype} with {t.numel()}")
    return _cuda(t, what)


def window_attention_prep(qkv: torch.Tensor, positions: torch.Tensor, slot_mapping: torch.Tensor | None,
                          freq: torch.Tensor | None, rot_dims: int, eps: float, num_heads: int, num_kv_heads: int, dim: int,
                          vdim: int, v_first: torch.Tensor | None, mix: torch.Tensor | None, cache: torch.Tensor | None, *,
                          bias: torch.Tensor | None = None, norm: bool = True, q_gain: torch.Tensor | None = None,
                          k_gain: torch.Tensor | None = None, norm_first: bool = False, rot_half: bool = False,
                          q_temp: tuple | None = None, value_from_key: bool = False, rot_gain: float = 1.0) -> None:
    """On the packed rows ``[q | k | v]``: ``bias`` (float32, one value per column) is added; rotary encoding of the
    first ``rot_dims`` values of every query and key head (32-bit angle ``pos * freq[i]``; neighbouring pairs, or with
    ``rot_half`` the pairs (i, i + rot_dims / 2)); with ``norm`` every query and key head is divided by its root mean
    square and multiplied by ``q_gain`` / ``k_gain`` (float32 [dim], None: no gain), after the rotation or, with
    ``norm_first``, before it; ``q_temp = (coef, every)`` multiplies the queries by
    ``1 + coef * ln(floor((pos + 1) / every) + 1)``.  ``value_from_key``: the rows are ``[q | k]`` and a token's value is
    its key as it stands before norm and rotation (``vdim == dim``).  ``rot_gain``: a factor on the rotation's cosine and
    sine.  Queries are rewritten in place; keys and values
    (``(1 - mix) * v + mix * v_first`` when both are given) go to ``cache[page, 0, kv head, slot, dim + vdim]``."""
    T, stride = qkv.shape
    columns = (num_heads + num_kv_heads) * dim + (0 if value_from_key else num_kv_heads * vdim)
    if value_from_key and (vdim != dim or v_first is not None):
        raise KernelError("window_attention_prep: values taken from the keys have the keys' size and are not mixed")
    if stride < columns or qkv.stride(1) != 1:
        raise KernelError("window_attention_prep: rows are too short")
    if cache is not None:
        if cache.dim() != 5 or cache.shape[1] != 1 or cache.shape[2] != num_kv_heads or cache.shape[4] != dim + vdim or cache.dtype != qkv.dtype:
            raise KernelError(f"window_attention_prep: cache must be [pages, 1, {num_kv_heads}, page, {dim + vdim}] of the rows' dtype")
        if slot_mapping is None:
            raise KernelError("window_attention_prep: a cache write needs slot_mapping")
    if (v_first is None) != (mix is None):
        raise KernelError("window_attention_prep: mixing needs both the values and the factor")
    if v_first is not None and (v_first.shape != (T, num_kv_heads * vdim) or v_first.dtype != qkv.dtype or v_first.stride(1) != 1):
        raise KernelError("window_attention_prep: v_first does not fit")
    rc = library().cib_window_attention_prep(
        _cuda(qkv, "qkv", contiguous=False), _code(qkv, "qkv"), qkv.stride(0), _cuda(positions, "positions", torch.int32),
        _cuda(slot_mapping, "slot_mapping", torch.int32) if cache is not None else None,
        _cuda(freq, "freq", torch.float32) if freq is not None and rot_dims else None, rot_dims if freq is not None else 0,
        float(eps), num_heads, num_kv_heads, dim, vdim,
        _cuda(v_first, "v_first", contiguous=False) if v_first is not None else None, v_first.stride(0) if v_first is not None else 0,
        _cuda(mix, "mix") if mix is not None else None, _code(mix, "mix") if mix is not None else 0,
        _cuda(cache, "cache") if cache is not None else None, cache.shape[0] * cache.shape[3] if cache is not None else 0,
        cache.shape[3] if cache is not None else 1, T,
        _f32_vec(bias, columns, "bias"), _f32_vec(q_gain, dim, "q_gain"), _f32_vec(k_gain, dim, "k_gain"), 1 if norm else 0,
        1 if norm_first else 0, 1 if rot_half else 0, 1 if q_temp else 0, float(q_temp[0]) if q_temp else 0.0,
        int(q_temp[1]) if q_temp else 1, 1 if value_from_key else 0, float(rot_gain), _stream())
    _check(rc, "window_attention_prep")
    _count()


def window_attention_generic(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                             positions: torch.Tensor, token_request: torch.Tensor, num_heads: int, num_kv_heads: int,
                             dim: int, vdim: int, scale: float, softcap: float, window: int, keep_first: int, *,
                             chunked: bool = False, slopes: torch.Tensor | None = None, sinks: torch.Tensor | None = None) -> None:
    """Attention of the query rows ``q[:, :H * dim]`` over the paged cache of [key | value] rows; ``out`` [T, H * vdim].
    ``softcap`` 0: no cap; ``window`` 0: every earlier key; ``chunked``: the window is a chunk, key j is seen when
    ``j // window == i // window``; ``slopes`` (float32 [H]): ``score -= slope * (i - j)``; ``sinks`` (float32 [H]): a
    score per head that joins the softmax's denominator and nothing else."""
    T = q.shape[0]
    if q.stride(1) != 1 or out.shape != (T, num_heads * vdim) or out.dtype != q.dtype or cache.dtype != q.dtype or not out.is_contiguous():
        raise KernelError("window_attention: out/cache do not fit q")
    rc = library().cib_window_attention_generic(
        _cuda(q, "q", contiguous=False), _code(q, "q"), q.stride(0), _cuda(out, "out"), out.stride(0), _cuda(cache, "cache"),
        cache.shape[0], cache.shape[3], _cuda(block_table, "block_table", torch.int32, contiguous=False), block_table.stride(0),
        _cuda(positions, "positions", torch.int32), _cuda(token_request, "token_request", torch.int32), T, num_heads,
        num_kv_heads, dim, vdim, float(scale), float(softcap or 0.0), int(window or 0), int(keep_first or 0),
        1 if chunked and window else 0, _f32_vec(slopes, num_heads, "slopes"), _f32_vec(sinks, num_heads, "sinks"), _stream())
    _check(rc, "window_attention_generic")
    _count()


def window_attention_mma_supports(dim: int, vdim: int, num_heads: int, num_kv_heads: int) -> bool:
    return bool(library().cib_window_attention_mma_supports(dim, vdim, num_heads, num_kv_heads))


def window_attention_mma(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                         query_start_loc: torch.Tensor, seq_lens: torch.Tensor, query_lens, num_heads: int, num_kv_heads: int,
                         dim: int, vdim: int, scale: float, softcap: float, window: int, keep_first: int, splits: int = 1, *,
                         chunked: bool = False, slopes: torch.Tensor | None = None, sinks: torch.Tensor | None = None) -> None:
    """The same attention on the tensor cores (bfloat16; key sizes 64 or 128, value sizes 32, 64 or 128).  ``query_lens``:
    tokens per request as host integers, or an upper bound that holds for every batch a captured step replays; they size
    the launch only.  ``splits`` > 1: the key tiles of every row tile are shared out to so many CTAs and a second kernel
    merges their partial results (decode steps over long windows, where a request has one row tile per key head).
    ``chunked``, ``slopes``, ``sinks``: as for the all-sizes kernel."""
    T = q.shape[0]
    if q.dtype != torch.bfloat16 or q.stride(1) != 1 or out.shape != (T, num_heads * vdim) or out.dtype != q.dtype or cache.dtype != q.dtype:
        raise KernelError("window_attention_mma: bfloat16 rows, out [T, H * vdim]")
    g = num_heads // num_kv_heads
    tiles = sum((n * g + 63) // 64 for n in query_lens)
    few_rows = all(n * g <= 16 for n in query_lens)      # a decode step: the warps of a tile share out its keys, not its rows
    splits = max(1, min(int(splits), 64))
    partial = torch.empty((T * num_heads, splits, vdim + 2), dtype=torch.float32, device=q.device) if splits > 1 else None
    rc = library().cib_window_attention_mma(
        _cuda(q, "q", contiguous=False), q.stride(0), _cuda(out, "out"), out.stride(0), _cuda(cache, "cache"), cache.shape[0],
        cache.shape[3], _cuda(block_table, "block_table", torch.int32, contiguous=False), block_table.stride(0),
        _cuda(query_start_loc, "query_start_loc", torch.int32), _cuda(seq_lens, "seq_lens", torch.int32), seq_lens.numel(), tiles,
        num_heads, num_kv_heads, dim, vdim, float(scale), float(softcap or 0.0), int(window or 0), int(keep_first or 0), splits,
        _cuda(partial, "partial") if partial is not None else None, T, 1 if chunked and window else 0, 1 if few_rows else 0,
        _f32_vec(slopes, num_heads, "slopes"), _f32_vec(sinks, num_heads, "sinks"), _stream())
    _check(rc, "window_attention_mma")
    _count()
    if splits > 1:
        _count()


# ---- mixers with a matrix state ------------------------------------------------------------------------------------------------

def mlstm_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gates: torch.Tensor, i_bias: torch.Tensor,
               f_bias: torch.Tensor, cap: float, q_scale: float, state: torch.Tensor, query_start_loc: torch.Tensor,
               state_slots: torch.Tensor, out: torch.Tensor, num_heads: int, dim: int, vdim: int, floor: float = 1e-6) -> None:
    """The matrix memory with exponential gates over every request's rows, from and to its state slot.  ``q``, ``k``, ``v``
    are column ranges of the same packed rows; ``gates`` float32 [T, 2H] (input then forget pre-activations; overwritten
    with the gates themselves by a first launch, before the scan walks the tokens);
    ``state`` float32 [slots, H, dim * vdim + dim + 1]; ``out`` float32 [T, H * vdim]."""
    T = out.shape[0]
    R = state_slots.numel()
    if not (q.stride(0) == k.stride(0) == v.stride(0)) or not (q.dtype == k.dtype == v.dtype) or q.stride(1) != 1:
        raise KernelError("mlstm_scan: q, k and v must be column ranges of the same rows")
    if state.shape[1:] != (num_heads, dim * vdim + dim + 1) or gates.shape != (T, 2 * num_heads) or out.shape != (T, num_heads * vdim):
        raise KernelError("mlstm_scan: state, gates or out do not fit")
    if i_bias.dtype != f_bias.dtype:
        raise KernelError("mlstm_scan: the biases must have one dtype")
    rc = library().cib_mlstm_scan(
        _cuda(q, "q", contiguous=False), _cuda(k, "k", contiguous=False), _cuda(v, "v", contiguous=False), _code(q, "q"), q.stride(0),
        _cuda(gates, "gates", torch.float32), gates.stride(0), _cuda(i_bias, "i_bias"), _cuda(f_bias, "f_bias"), _code(i_bias, "i_bias"),
        float(cap), float(q_scale), float(floor), _cuda(state, "state", torch.float32),
        _cuda(query_start_loc, "query_start_loc", torch.int32), _cuda(state_slots, "state_slots", torch.int32), state.shape[0], R, T,
        _cuda(out, "out", torch.float32), num_heads, dim, vdim, _stream())
    _check(rc, "mlstm_scan")
    _count()
    _count()


def delta_prep(x: torch.Tensor, taps: torch.Tensor, conv_state: torch.Tensor, query_start_loc: torch.Tensor,
               token_request: torch.Tensor, state_slots: torch.Tensor, num_kv_heads: int, num_heads: int, dim: int, vdim: int,
               unit_eps: float, q_scale: float, out: torch.Tensor) -> None:
    """Short causal convolution + SiLU over the channels ``[q | k | v]`` of the packed rows ``x`` (continuing from, and
    updating, each request's ``conv_state`` float32 [slots, taps - 1, C]), then unit q and k heads, q times ``q_scale``;
    ``out`` float32 [T, C].  Two launches."""
    T = x.shape[0]
    C = 2 * num_kv_heads * dim + num_heads * vdim
    K = taps.shape[1]
    if taps.shape != (C, K) or taps.dtype != x.dtype or out.shape != (T, C) or x.stride(1) != 1 or x.shape[1] < C:
        raise KernelError("delta_prep: taps, rows or out do not fit")
    if conv_state.shape[1:] != (max(K - 1, 1), C):
        raise KernelError("delta_prep: conv_state must be [slots, taps - 1, channels]")
    rc = library().cib_delta_prep(
        _cuda(x, "x", contiguous=False), _code(x, "x"), x.stride(0), _cuda(taps, "taps"), K, _cuda(conv_state, "conv_state", torch.float32),
        _cuda(query_start_loc, "query_start_loc", torch.int32), _cuda(token_request, "token_request", torch.int32),
        _cuda(state_slots, "state_slots", torch.int32), conv_state.shape[0], state_slots.numel(), num_kv_heads, num_heads, dim, vdim,
        float(unit_eps), float(q_scale), _cuda(out, "out", torch.float32), T, _stream())
    _check(rc, "delta_prep")
    _count()
    _count()


def delta_scan(qkv: torch.Tensor, gates: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor, state: torch.Tensor,
               query_start_loc: torch.Tensor, state_slots: torch.Tensor, out: torch.Tensor, num_kv_heads: int, num_heads: int,
               dim: int, vdim: int) -> None:
    """The gated delta rule over every request's rows.  ``qkv`` float32 [T, C] from ``delta_prep``; ``gates`` float32
    [T, 2H] (beta then decay pre-activations; overwritten with beta and the decay by a first launch); ``state`` float32 [slots, H, dim * vdim]; ``out`` float32 [T, H * vdim]."""
    T = qkv.shape[0]
    if state.shape[1:] != (num_heads, dim * vdim) or gates.shape != (T, 2 * num_heads) or out.shape != (T, num_heads * vdim):
        raise KernelError("delta_scan: state, gates or out do not fit")
    if a_log.dtype != dt_bias.dtype:
        raise KernelError("delta_scan: the per-head vectors must have one dtype")
    rc = library().cib_delta_scan(
        _cuda(qkv, "qkv", torch.float32), num_kv_heads, _cuda(gates, "gates", torch.float32), gates.stride(0), _cuda(a_log, "a_log"),
        _cuda(dt_bias, "dt_bias"), _code(a_log, "a_log"), _cuda(state, "state", torch.float32),
        _cuda(query_start_loc, "query_start_loc", torch.int32), _cuda(state_slots, "state_slots", torch.int32), state.shape[0],
        state_slots.numel(), T, _cuda(out, "out", torch.float32), num_heads, dim, vdim, _stream())
    _check(rc, "delta_scan")
    _count()
    _count()


def head_rms_gate(o: torch.Tensor, gate: torch.Tensor, gain: torch.Tensor, eps: float, silu: bool, out: torch.Tensor,
                  num_heads: int, vdim: int) -> None:
    """out[t, h, :] = rmsnorm(o[t, h, :]) * gain * act(gate[t, h, :]); ``gain`` has ``vdim`` elements (shared by the heads)
    or ``H * vdim``; act is SiLU or the sigmoid; ``o`` float32, ``gate`` a column range of the packed rows."""
    T = o.shape[0]
    if o.shape != (T, num_heads * vdim) or out.shape != o.shape or gate.shape != o.shape or gate.stride(1) != 1 or gate.dtype != out.dtype:
        raise KernelError("head_rms_gate: shapes do not fit")
    if gain.numel() not in (vdim, num_heads * vdim):
        raise KernelError("head_rms_gate: the gain must have vdim or heads * vdim elements")
    rc = library().cib_head_rms_gate(
        _cuda(o, "o", torch.float32), _cuda(gate, "gate", contiguous=False), _code(gate, "gate"), gate.stride(0), _cuda(gain, "gain"),
        _code(gain, "gain"), 1 if gain.numel() != vdim else 0, float(eps), 1 if silu else 0,
        _cuda(out, "out"), num_heads, vdim, T, _stream())
    _check(rc, "head_rms_gate")
    _count()


# ---- a residual of several streams ---------------------------------------------------------------------------------------------

def hyper_stream(streams: torch.Tensor, y: torch.Tensor | None, write: tuple | None, read: torch.Tensor | None,
                 norm: tuple | None, out: torch.Tensor | None, read_out: torch.Tensor | None = None) -> None:
    """One pass over the 32-bit residual streams ``[T, S, W]``.  ``write = (mix [S, S], out [S])`` with the sub-layer
    output ``y`` [T, W]: every stream is rewritten from the old ones, ``x_t = sum_s mix[s, t] x_s + out[t] y``.
    ``read`` [S]: the next sub-layer's input ``u = sum_t read[t] x_t``; ``out`` gets its RMS norm times the gain
    (``norm = (gain or None, eps)``) in its dtype and ``read_out`` (float32) the row ``u`` itself.  Coefficients are
    float32."""
    T, S, W = streams.shape
    if (y is None) != (write is None):
        raise KernelError("hyper_stream: a write needs the sub-layer's output and its coefficients")
    if y is not None and (y.shape != (T, W) or not y.is_contiguous()):
        raise KernelError(f"hyper_stream: y must be [{T}, {W}], got {list(y.shape)}")
    if (out is not None or read_out is not None) and read is None:
        raise KernelError("hyper_stream: a read needs its coefficients")
    if out is not None and (norm is None or out.shape != (T, W)):
        raise KernelError("hyper_stream: the normed rows need (gain, eps) and the shape [T, W]")
    if read_out is not None and read_out.shape != (T, W):
        raise KernelError("hyper_stream: read_out must be [T, W]")
    gain = norm[0] if norm else None
    if gain is not None and gain.numel() != W:
        raise KernelError(f"hyper_stream: the gain must have {W} values")
    rc = library().cib_hyper_stream(
        _cuda(streams, "streams", torch.float32), _cuda(y, "y") if y is not None else None, _code(y, "y") if y is not None else 0,
        _f32_vec(write[0], S * S, "mix") if write else None, _f32_vec(write[1], S, "out coefficients") if write else None,
        _f32_vec(read, S, "read coefficients"), _cuda(gain, "gain") if gain is not None else None,
        _code(gain, "gain") if gain is not None else 0, float(norm[1]) if norm else 0.0,
        _cuda(out, "out") if out is not None else None, _code(out, "out") if out is not None else 0,
        _cuda(read_out, "read_out", torch.float32) if read_out is not None else None, S, W, T, _stream())
    _check(rc, "hyper_stream")
    _count()


def hyper_gather(streams: torch.Tensor, y: torch.Tensor | None, write: tuple | None, indices: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = the sum over the streams of token ``indices[r]``, after the outstanding write ``(y, (mix, out))`` if
    there is one; the other tokens' rows are not touched."""
    T, S, W = streams.shape
    n = indices.numel()
    if out.shape != (n, W) or (y is None) != (write is None) or (y is not None and y.shape != (T, W)):
        raise KernelError("hyper_gather: shapes do not fit")
    rc = library().cib_hyper_gather(
        _cuda(streams, "streams", torch.float32), _cuda(y, "y") if y is not None else None, _code(y, "y") if y is not None else 0,
        _f32_vec(write[0], S * S, "mix") if write else None, _f32_vec(write[1], S, "out coefficients") if write else None,
        _cuda(indices, "indices", torch.int32), _cuda(out, "out", torch.float32), S, W, T, n, _stream())
    _check(rc, "hyper_gather")
    _count()
