"""Python face of the CUDA kernels in ``csrc/``.

Every function checks what it is given (device, dtype, shape, contiguity),
refuses what the kernel does not take with a clear message, and launches on
torch's current CUDA stream.  There is no other implementation behind these
functions: without a CUDA device, ``nvcc`` or a successful build they raise.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import os

import torch

from .csrc.build import load_library

c_int, c_long, c_float, c_void_p = ctypes.c_int, ctypes.c_long, ctypes.c_float, ctypes.c_void_p


class KernelError(RuntimeError):
    pass


_SIGNATURES = {
    "ib_embedding_gather": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p],
    "ib_rms_norm_rows": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p],
    "ib_add_cast": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "ib_logit_scale_softcap": [c_void_p, c_long, c_float, c_float, c_void_p],
    "ib_resolve_tokens": [c_void_p, c_int, c_void_p, c_int, c_void_p],
    "ib_add_rms_norm": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
    "ib_silu_gate": [c_void_p, c_void_p, c_int, c_int, c_void_p],
    "ib_act_to_float": [c_void_p, c_void_p, c_long, c_void_p],
    "ib_qk_norm_rope_store": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_float,
                              c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                              c_void_p, c_void_p, c_void_p, c_void_p],
    "ib_paged_attention_generic": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
                                   c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p],
    "ib_gemm_tn_simt": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_long, c_long,
                        c_long, c_void_p],
    "ib_paged_attention_mma": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                               c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_int, c_int,
                               c_void_p, c_void_p, c_void_p],
    "ib_paged_attention_tcgen05": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
                                   c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p,
                                   c_void_p],
    "ib_attention_tcgen05_error": [c_int],
    "ib_paged_attention_pair_tcgen05": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
                                        c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p,
                                        c_void_p],
    "ib_attention_pair_tcgen05_error": [c_int],
    "ib_row_fault": [c_int],
    "ib_row_fault_async": [c_void_p, c_void_p],
    "ib_attention_tcgen05_error_async": [c_void_p, c_void_p],
    "ib_attention_pair_tcgen05_error_async": [c_void_p, c_void_p],
    "ib_attention_decode_error_async": [c_void_p, c_void_p],
    "ib_paged_attention_decode": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int,
                                  c_int, c_int, c_float, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_void_p, c_void_p],
    "ib_attention_decode_error": [c_int],
    "ib_argmax": [c_void_p, c_void_p, c_int, c_int, c_long, c_void_p, c_void_p],
    "ib_penalties": [c_void_p, c_long, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                     c_void_p],
    "ib_sample": [c_void_p, c_long, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                  c_int, c_void_p, c_void_p],
}

_LIBS = {}


def _core(act_dtype: torch.dtype):
    """The core library built for this activation dtype, with argument types set."""
    if act_dtype == torch.float32:
        name = "core_f32"
    elif act_dtype == torch.bfloat16:
        name = "core_bf16"
    else:
        raise KernelError(f"activations must be float32 or bfloat16, got {act_dtype}")
    lib = _LIBS.get(name)
    if lib is None:
        lib = load_library(name)
        for fn, args in _SIGNATURES.items():
            f = getattr(lib, fn)
            f.argtypes = args
            f.restype = c_int
        _LIBS[name] = lib
    return lib


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_DEVICE_INDEX = None


def _stream() -> int:
    """The current CUDA stream's handle (the short way where this torch has it: a launch asks for it every time)."""
    global _DEVICE_INDEX
    if _RAW_STREAM is not None:
        if _DEVICE_INDEX is None:
            _DEVICE_INDEX = torch.cuda.current_device()   # one process drives one GPU
        return _RAW_STREAM(_DEVICE_INDEX)
    return torch.cuda.current_stream().cuda_stream


_LAUNCHES = 0


def launch_count() -> int:
    """Kernel launches of this package's own libraries so far (library matrix products are not counted)."""
    return _LAUNCHES


def count_launches(n: int):
    """Add the kernels of a replayed CUDA graph to the count."""
    global _LAUNCHES
    _LAUNCHES += n


def _check(code: int, what: str):
    global _LAUNCHES
    if code == 0:
        _LAUNCHES += 1
        return
    if code == -1:
        raise KernelError(f"{what}: these sizes are not supported by the kernel")
    if code == -2:
        raise KernelError(f"{what}: invalid argument")
    raise KernelError(f"{what}: CUDA launch failed with error {code}")


def _need(t: Optional[torch.Tensor], name: str, dtypes, ndim: Optional[int] = None, optional: bool = False):
    if t is None:
        if optional:
            return
        raise KernelError(f"{name} is required")
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (the kernels have no CPU implementation), got {t.device}")
    if t.dtype not in dtypes:
        raise KernelError(f"{name} must have dtype in {dtypes}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{name} must have {ndim} dimensions, got shape {tuple(t.shape)}")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous, got strides {t.stride()} for shape {tuple(t.shape)}")


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


_W = (torch.float32, torch.bfloat16)
_I = (torch.int32,)


def embedding_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, act_dtype: torch.dtype,
                     scale: float = 1.0):
    """out[r, :] = table[ids[r], :] * scale as float32."""
    _need(table, "table", _W, 2)
    _need(ids, "ids", _I, 1)
    _need(out, "out", (torch.float32,), 2)
    n, width = out.shape
    if ids.shape[0] != n or table.shape[1] != width:
        raise KernelError(f"embedding_gather: ids {tuple(ids.shape)}, table {tuple(table.shape)}, out {tuple(out.shape)}")
    _check(_core(act_dtype).ib_embedding_gather(_p(table), int(table.dtype == torch.float32), _p(ids), _p(out), n,
                                                width, table.shape[0], float(scale), _stream()), "embedding_gather")


def resolve_tokens(ids: torch.Tensor, carry: torch.Tensor, act_dtype: torch.dtype):
    """ids[i] = carry[-1 - ids[i]] wherever ids[i] < 0: a step's description names tokens that an earlier step
    sampled and the host has not read yet by their place in that step's output."""
    _need(ids, "ids", _I, 1)
    _need(carry, "carry", _I, 1)
    _check(_core(act_dtype).ib_resolve_tokens(_p(ids), ids.shape[0], _p(carry), carry.shape[0], _stream()),
           "resolve_tokens")


def add_rms_norm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                 out: torch.Tensor, rows: Optional[torch.Tensor] = None):
    """residual += delta (float32, in place when ``rows`` is None); out = rms_norm(residual) * weight.

    With ``rows`` (int32 [W]) only those rows are read and out has W rows; nothing is written back.
    """
    act = out.dtype
    _need(residual, "residual", (torch.float32,), 2)
    _need(delta, "delta", (act,), 2, optional=True)
    _need(weight, "weight", _W, 1)
    _need(out, "out", _W, 2)
    _need(rows, "rows", _I, 1, optional=True)
    n, width = residual.shape
    n_out = n if rows is None else rows.shape[0]
    if weight.shape[0] != width or out.shape != (n_out, width) or (delta is not None and delta.shape != residual.shape):
        raise KernelError(f"add_rms_norm: residual {tuple(residual.shape)}, weight {tuple(weight.shape)}, "
                          f"out {tuple(out.shape)}, delta {None if delta is None else tuple(delta.shape)}")
    _check(_core(act).ib_add_rms_norm(_p(residual), _p(delta), _p(weight), int(weight.dtype == torch.float32),
                                      _p(out), _p(rows), n_out, width, float(eps), _stream()), "add_rms_norm")


def rms_norm_rows(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor):
    """out = rms_norm(x) * weight for rows in the activation dtype (a norm on a sub-layer's output)."""
    act = out.dtype
    _need(x, "x", (act,), 2)
    _need(weight, "weight", _W, 1)
    _need(out, "out", _W, 2)
    if out.shape != x.shape or weight.shape[0] != x.shape[1]:
        raise KernelError(f"rms_norm_rows: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    _check(_core(act).ib_rms_norm_rows(_p(x), _p(weight), int(weight.dtype == torch.float32), _p(out), x.shape[0],
                                       x.shape[1], float(eps), _stream()), "rms_norm_rows")


def add_cast(residual: torch.Tensor, delta: Optional[torch.Tensor], out: torch.Tensor,
             rows: Optional[torch.Tensor] = None):
    """residual += delta (float32, in place when ``rows`` is None); out = residual in the activation dtype:
    what a sub-layer without a norm reads."""
    act = out.dtype
    _need(residual, "residual", (torch.float32,), 2)
    _need(delta, "delta", (act,), 2, optional=True)
    _need(out, "out", _W, 2)
    _need(rows, "rows", _I, 1, optional=True)
    n, width = residual.shape
    n_out = n if rows is None else rows.shape[0]
    if out.shape != (n_out, width) or (delta is not None and delta.shape != residual.shape):
        raise KernelError(f"add_cast: residual {tuple(residual.shape)}, out {tuple(out.shape)}, "
                          f"delta {None if delta is None else tuple(delta.shape)}")
    _check(_core(act).ib_add_cast(_p(residual), _p(delta), _p(out), _p(rows), n_out, width, _stream()), "add_cast")


def logit_scale_softcap(logits: torch.Tensor, scale: float, softcap: Optional[float], act_dtype: torch.dtype):
    """In place on float32 logits: x *= scale, then x = cap * tanh(x / cap) where a cap is given."""
    _need(logits, "logits", (torch.float32,), 2)
    if softcap is not None and not softcap > 0:
        raise KernelError(f"logit_scale_softcap: the cap must be positive, got {softcap}")
    _check(_core(act_dtype).ib_logit_scale_softcap(_p(logits), logits.numel(), float(scale),
                                                   float(softcap) if softcap else 0.0, _stream()),
           "logit_scale_softcap")


def silu_gate(gate_up: torch.Tensor, out: torch.Tensor):
    """out[r, j] = silu(gate_up[r, j]) * gate_up[r, inner + j]."""
    act = out.dtype
    _need(gate_up, "gate_up", (act,), 2)
    _need(out, "out", _W, 2)
    n, inner = out.shape
    if gate_up.shape != (n, 2 * inner):
        raise KernelError(f"silu_gate: gate_up {tuple(gate_up.shape)} does not match out {tuple(out.shape)}")
    _check(_core(act).ib_silu_gate(_p(gate_up), _p(out), n, inner, _stream()), "silu_gate")


def qk_norm_rope_store(qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, store_kv: bool,
                       q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                       cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rot_dim: int,
                       positions: torch.Tensor, row_request: torch.Tensor, block_table: Optional[torch.Tensor],
                       k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor], q_out: torch.Tensor,
                       interleaved: bool = False):
    """Per-head norm of q and k, rotation by position, q to ``q_out``, k and v into their pages.  Element ``i`` of
    a head's first ``rot_dim / 2`` turns with element ``i + rot_dim / 2``; ``interleaved``: element ``2i`` with ``2i + 1``.

    qkv [N, (n_heads + 2 n_kv_heads) * d] (queries only when ``store_kv`` is False);
    pages [n_pages, n_kv_heads, page_size, d]; block_table int32 [R, max_pages].
    """
    act = q_out.dtype
    _need(qkv, "qkv", (act,), 2)
    _need(q_out, "q_out", _W, 3)
    _need(positions, "positions", _I, 1)
    _need(row_request, "row_request", _I, 1)
    n = qkv.shape[0]
    cols = (n_heads + (2 * n_kv_heads if store_kv else 0)) * head_dim
    if qkv.shape[1] != cols or q_out.shape != (n, n_heads, head_dim) or positions.shape[0] != n \
            or row_request.shape[0] != n:
        raise KernelError(f"qk_norm_rope_store: qkv {tuple(qkv.shape)} (want {cols} columns), q_out "
                          f"{tuple(q_out.shape)}, positions {tuple(positions.shape)}")
    wdt = None
    for name, w in (("q_weight", q_weight), ("k_weight", k_weight)):
        _need(w, name, _W, 1, optional=True)
        if w is not None:
            if w.shape[0] != head_dim:
                raise KernelError(f"{name} has {w.shape[0]} elements, head_dim is {head_dim}")
            if wdt is not None and w.dtype != wdt:
                raise KernelError("q_weight and k_weight must have the same dtype")
            wdt = w.dtype
    table_rows = 0
    if rot_dim:
        _need(cos, "cos", (torch.float32,), 2)
        _need(sin, "sin", (torch.float32,), 2)
        if cos.shape[1] != rot_dim // 2 or sin.shape != cos.shape:
            raise KernelError(f"rotation tables {tuple(cos.shape)} do not match rot_dim {rot_dim}")
        table_rows = cos.shape[0]
    max_pages = page_size = n_pages = 0
    if store_kv:
        _need(block_table, "block_table", _I, 2)
        _need(k_pages, "k_pages", (act,), 4)
        _need(v_pages, "v_pages", (act,), 4)
        n_pages, nkv, page_size, d = k_pages.shape
        if (nkv, d) != (n_kv_heads, head_dim) or v_pages.shape != k_pages.shape:
            raise KernelError(f"cache pages {tuple(k_pages.shape)} do not match {n_kv_heads} heads of {head_dim}")
        max_pages = block_table.shape[1]
    _check(_core(act).ib_qk_norm_rope_store(
        _p(qkv), cols, n, n_heads, n_kv_heads, head_dim, int(store_kv), _p(q_weight), _p(k_weight),
        int(wdt == torch.float32), float(eps), _p(cos) if rot_dim else None, _p(sin) if rot_dim else None, rot_dim,
        int(bool(interleaved)), table_rows, _p(positions), _p(row_request), _p(block_table) if store_kv else None, max_pages, page_size,
        n_pages, _p(k_pages) if store_kv else None, _p(v_pages) if store_kv else None, _p(q_out), _stream()),
        "qk_norm_rope_store")


def row_fault(act_dtype: torch.dtype, reset: bool = True) -> Optional[int]:
    """The first row that a kernel left out because its position lay outside the rotation tables (None if
    there was none).  Waits for the device."""
    v = _core(act_dtype).ib_row_fault(int(reset))
    if v < 0:
        raise KernelError(f"row_fault: CUDA error {-v}")
    return None if v == 0 else v - 1


def paged_attention_generic(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                            row_request: torch.Tensor, positions: torch.Tensor, scale: float, window: Optional[int],
                            out: torch.Tensor):
    """out[r, h*d:(h+1)*d] = attention of token r's head h over its request's cached keys lo..pos."""
    act = out.dtype
    _need(q, "q", (act,), 3)
    _need(k_pages, "k_pages", (act,), 4)
    _need(v_pages, "v_pages", (act,), 4)
    _need(block_table, "block_table", _I, 2)
    _need(row_request, "row_request", _I, 1)
    _need(positions, "positions", _I, 1)
    _need(out, "out", _W, 2)
    n, nh, d = q.shape
    n_pages, nkv, page_size, dk = k_pages.shape
    if dk != d or v_pages.shape != k_pages.shape or out.shape != (n, nh * d) or nh % nkv:
        raise KernelError(f"paged_attention: q {tuple(q.shape)}, pages {tuple(k_pages.shape)}, out {tuple(out.shape)}")
    if d > 512:
        raise KernelError(f"paged_attention: head_dim {d} is larger than 512, the largest the kernel takes")
    _check(_core(act).ib_paged_attention_generic(
        _p(q), _p(k_pages), _p(v_pages), _p(block_table), block_table.shape[1], page_size, n_pages, _p(row_request),
        _p(positions), n, nh, nkv, d, float(scale), int(window) if window else 0, _p(out), _stream()),
        "paged_attention_generic")


def gemm_tn_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, act_dtype: torch.dtype):
    """out = x @ w.T with 32-bit fused multiply-adds in ascending k (no tensor cores)."""
    _need(x, "x", _W, 2)
    _need(w, "w", _W, 2)
    _need(out, "out", _W, 2)
    n, k = x.shape
    m = w.shape[0]
    if w.shape[1] != k or out.shape != (n, m):
        raise KernelError(f"gemm: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    code = _core(act_dtype).ib_gemm_tn_simt(_p(x), int(x.dtype == torch.float32), _p(w),
                                            int(w.dtype == torch.float32), _p(out), int(out.dtype == torch.float32),
                                            n, m, k, k, k, m, _stream())
    if code == -1:
        raise KernelError(f"gemm: no kernel for x {x.dtype}, w {w.dtype}, out {out.dtype} with activations {act_dtype}")
    _check(code, "gemm_tn_simt")


def argmax(logits: torch.Tensor, out: torch.Tensor, act_dtype: torch.dtype = torch.float32):
    """out[r] = index of the largest logit of row r (lowest index among equals).  ``act_dtype`` only
    selects which of the two builds of the kernel library serves the call."""
    _need(logits, "logits", (torch.float32,), 2)
    _need(out, "out", _I, 1)
    if out.shape[0] != logits.shape[0]:
        raise KernelError(f"argmax: logits {tuple(logits.shape)}, out {tuple(out.shape)}")
    rows, vocab = logits.shape
    scratch = None
    if vocab > ARGMAX_CHUNK:  # the vocabulary is cut into chunks so that few rows still fill the machine
        scratch = torch.empty((rows, (vocab + ARGMAX_CHUNK - 1) // ARGMAX_CHUNK), dtype=torch.int64,
                              device=logits.device)
    _check(_core(act_dtype).ib_argmax(_p(logits), _p(out), rows, vocab, vocab, _p(scratch), _stream()), "argmax")


_MM_F32_OUT = None  # does this torch give float32 results from a bfloat16 product?


def gemm_tn_bf16(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor):
    """out = x @ w.T for bfloat16 x and w on the tensor cores with float32 accumulation.

    The product itself is the vendor library's (cuBLASLt through ``torch.mm``), as the reference
    calls cuBLAS for every matrix product (candle-core/src/cuda_backend/mod.rs:2260-2310).
    ``out`` may be bfloat16 or float32.
    """
    global _MM_F32_OUT
    _need(x, "x", (torch.bfloat16,), 2)
    _need(w, "w", (torch.bfloat16,), 2)
    _need(out, "out", _W, 2)
    if w.shape[1] != x.shape[1] or out.shape != (x.shape[0], w.shape[0]):
        raise KernelError(f"gemm: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if out.dtype == torch.bfloat16:
        torch.mm(x, w.t(), out=out)
        return
    if _MM_F32_OUT is None:
        try:
            torch.mm(x[:1], w[:8].t(), out_dtype=torch.float32)
            _MM_F32_OUT = True
        except (TypeError, RuntimeError):
            _MM_F32_OUT = False
    if _MM_F32_OUT:
        torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
    else:
        gemm_tn_simt(x, w, out, torch.bfloat16)


SSQ_LD = 32   # tokens per part of a list of sums of squares (csrc/gemm_tcgen05.cu)


@dataclass
class ScaledRows:
    """Rows with an RMS norm folded in: ``x`` holds (stream * norm weight) as bfloat16, ``ssq[:n_parts, :rows]`` the
    parts of the stream's sums of squares per row.  The norm's output is x / sqrt(sum(ssq) / width + eps) per row;
    a product that reads ``x`` applies that factor to its result instead (see csrc/gemm_tcgen05.cu)."""

    x: torch.Tensor
    ssq: torch.Tensor
    n_parts: int
    eps: float
    width: int

    @property
    def shape(self):
        return self.x.shape

    @property
    def device(self):
        return self.x.device


@dataclass
class ResidualSink:
    """Where a product's result goes when the addition to the residual stream and the norm that follows are folded
    into its read-back: it is added to ``residual`` (float32, in place) and handed on as :class:`ScaledRows` of the
    norm with weight ``weight`` and ``eps``."""

    residual: torch.Tensor
    weight: torch.Tensor
    eps: float


def folded_norm_supported(n_rows: int, act_dtype: torch.dtype, w: torch.Tensor) -> bool:
    """Whether a product of ``n_rows`` rows with weight ``w`` can take scaled rows or feed a sink: the bfloat16 tcgen05
    product for a few rows does."""
    return (act_dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and n_rows <= min(TCGEN05_MAX_TOKENS, SSQ_LD)
            and w.shape[1] % 8 == 0 and w.data_ptr() % 16 == 0)


# ---- chains of products ---------------------------------------------------------------------------------------
# In a step of a few rows the products whose norms are folded in follow one another without any other kernel between
# them: o projection (sink) -> gate/up (scaled rows) -> down (sink) -> the next layer's q/k/v (scaled rows).
# csrc/gemm_chain.cu runs up to four such products as ONE persistent cooperative kernel whose producers keep streaming
# the next product's weights while the CTAs meet between two products.  On a B200 it came out a little slower than the
# products launched one by one under programmatic dependent launch (a meeting of 148 CTAs through global memory costs
# 5 to 6 us, as much as a kernel's ends), so the parts do not use it; it stands here as a kernel of its own with its
# tests, for shapes and machines where the balance is another.
_CHAIN_WS = {}       # device index -> (workspace, counters, number of CTAs)


class _ChainProduct(ctypes.Structure):
    _fields_ = [("x", c_void_p), ("ldx", c_long), ("w", c_void_p), ("ldw", c_long), ("y", c_void_p), ("ldy", c_long),
                ("n_out", c_int), ("k", c_int), ("gated", c_int),
                ("in_ssq", c_void_p), ("n_in_parts", c_int), ("in_eps", c_float), ("in_width", c_int),
                ("residual", c_void_p), ("ld_res", c_long), ("sink_w", c_void_p), ("sink_w_is_f32", c_int),
                ("out_ssq", c_void_p)]


def _chain_workspace(device: torch.device):
    idx = device.index if device.index is not None else torch.cuda.current_device()
    ws = _CHAIN_WS.get(idx)
    if ws is None:
        lib = _gemm_lib()
        sms = torch.cuda.get_device_properties(idx).multi_processor_count
        # (the kernel needs the workspace filled with its "not yet" value and the counters zero, and leaves them so)
        ws = (torch.full((lib.ib_gemm_chain_workspace_floats(sms),), lib.ib_gemm_chain_workspace_fill(),
                         dtype=torch.int32, device=device).view(torch.float32),
              torch.zeros((lib.ib_gemm_chain_max_products() + 1,), dtype=torch.int32, device=device), sms)
        _CHAIN_WS[idx] = ws
    return ws


class ProductChain:
    """Up to four products of a few bfloat16 rows (at most 16) that are launched as one kernel by :meth:`launch`.

    ``linear`` and ``gated_linear`` take what the functions of the same names take, ``x`` a tensor or
    :class:`ScaledRows`; a product's output tensor may be the input of a later product of the chain (that is what the
    chain is for) and holds nothing before the launch."""

    def __init__(self):
        self._products = []    # (structure, rows, device, units, what keeps the tensors alive)

    def linear(self, x, w: torch.Tensor, out: torch.Tensor, sink: Optional["ResidualSink"] = None):
        return self._add(x, w, out, sink, gated=False)

    def gated_linear(self, x, w_gate_up: torch.Tensor, out: torch.Tensor):
        if w_gate_up.shape[0] != 2 * out.shape[1] or out.shape[1] % 64 != 0:
            raise KernelError(f"chain: gate/up weights {tuple(w_gate_up.shape)} for out {tuple(out.shape)} "
                              f"(the inner width must be a multiple of 64)")
        self._add(x, w_gate_up, out, None, gated=True)

    def _add(self, x, w, out, sink, gated):
        lib = _gemm_lib()
        if len(self._products) >= lib.ib_gemm_chain_max_products():
            raise KernelError(f"chain: at most {lib.ib_gemm_chain_max_products()} products")
        xt, scaled = _scaled_args(x)
        _need(xt, "x", (torch.bfloat16,), 2)
        _need(w, "w", (torch.bfloat16,), 2)
        _need(out, "out", (torch.bfloat16,), 2)
        n, k = xt.shape
        m = out.shape[1]
        if n > 16 or k % 8 != 0:
            raise KernelError(f"chain: {n} rows of width {k} (at most 16 rows, a width that is a multiple of 8)")
        if w.shape != ((2 * m if gated else m), k) or out.shape[0] != n:
            raise KernelError(f"chain: x {tuple(xt.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
        if self._products and (self._products[0][1] != n or self._products[0][2] != out.device):
            raise KernelError("chain: all products have the same rows on the same device")
        prod = _ChainProduct(x=_p(xt), ldx=k, w=_p(w), ldw=k, y=_p(out), ldy=m, n_out=m, k=k, gated=int(gated),
                             in_ssq=scaled[0], n_in_parts=scaled[1], in_eps=scaled[2], in_width=scaled[3])
        result, keep = None, [xt, w, out, x]
        if sink is not None:
            _need(sink.residual, "residual", (torch.float32,), 2)
            _need(sink.weight, "sink weight", _W, 1)
            if sink.residual.shape != (n, m) or sink.weight.shape[0] != m or gated:
                raise KernelError(f"chain: residual {tuple(sink.residual.shape)} and norm weight "
                                  f"{tuple(sink.weight.shape)} do not match the result {(n, m)}")
            parts = lib.ib_gemm_chain_ssq_parts(m)
            ssq = torch.empty((parts, SSQ_LD), dtype=torch.float32, device=out.device)
            prod.residual, prod.ld_res, prod.sink_w = _p(sink.residual), m, _p(sink.weight)
            prod.sink_w_is_f32, prod.out_ssq = int(sink.weight.dtype == torch.float32), _p(ssq)
            result = ScaledRows(out, ssq, parts, float(sink.eps), m)
            keep += [sink.residual, sink.weight, ssq]
        units = ((m // 64) if gated else (m + 127) // 128) * ((k + 63) // 64)
        self._products.append((prod, n, out.device, units, keep))
        return result

    def launch(self):
        if not self._products:
            return
        products, self._products = self._products, []
        n_tok, device = products[0][1], products[0][2]
        scratch, counters, sms = _chain_workspace(device)
        grid = min([sms] + [p[3] for p in products])
        arr = (_ChainProduct * len(products))(*[p[0] for p in products])
        code = _gemm_lib().ib_gemm_chain(arr, len(products), n_tok, _p(scratch), _p(counters), grid, _stream())
        if code == -1:
            raise KernelError("chain: these sizes are not supported (up to 16 rows, K a multiple of 8, gated widths a "
                              "multiple of 64)")
        _check(code, "chain of products")


def linear(x, w: torch.Tensor, out: torch.Tensor, act_dtype: torch.dtype, sink: Optional[ResidualSink] = None):
    """out = x @ w.T in the precision that ``act_dtype`` and the weight's own dtype ask for.  ``x`` may be
    :class:`ScaledRows`; with ``sink`` the result is added to the residual stream and ``out`` receives the stream times
    the next norm's weight: the returned :class:`ScaledRows` (else None) stand for that norm's output."""
    if isinstance(x, ScaledRows) or sink is not None:
        rows = x.shape[0]
        if not folded_norm_supported(rows, act_dtype, w):
            raise KernelError(f"linear: {rows} rows of {act_dtype} with a {w.dtype} weight cannot take folded norms; "
                              f"ask folded_norm_supported first")
        return gemm_tn_tcgen05(x, w, out, sink=sink)
    if act_dtype == torch.float32 or w.dtype == torch.float32:
        gemm_tn_simt(x, w, out, act_dtype)
    elif x.shape[0] <= TCGEN05_MAX_TOKENS and tcgen05_gemm_supported(x, w):
        gemm_tn_tcgen05(x, w, out)
    else:
        gemm_tn_bf16(x, w, out)
    return None


def gated_linear(x, w_gate_up: torch.Tensor, out: torch.Tensor, act_dtype: torch.dtype):
    """out = silu(x @ gate.T) * (x @ up.T), ``w_gate_up`` [2 * inner, k] holding the gate matrix above the up
    matrix.  A few bfloat16 rows run as one tcgen05 kernel; everything else as the product and the gate kernel.
    ``x`` may be :class:`ScaledRows` (a few bfloat16 rows only)."""
    inner = out.shape[1]
    if w_gate_up.shape[0] != 2 * inner:
        raise KernelError(f"gated_linear: weights {tuple(w_gate_up.shape)} do not match out {tuple(out.shape)}")
    if isinstance(x, ScaledRows):
        if not folded_norm_supported(x.shape[0], act_dtype, w_gate_up) or x.shape[0] > SWIGLU_MAX_TOKENS:
            raise KernelError("gated_linear: these rows cannot take a folded norm; ask folded_norm_supported first")
        gemm_swiglu_tcgen05(x, w_gate_up, out)
        return
    if act_dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 \
            and x.shape[0] <= min(TCGEN05_MAX_TOKENS, SWIGLU_MAX_TOKENS) \
            and tcgen05_gemm_supported(x, w_gate_up):
        gemm_swiglu_tcgen05(x, w_gate_up, out)
        return
    gu = torch.empty((x.shape[0], 2 * inner), dtype=act_dtype, device=x.device)
    linear(x, w_gate_up, gu, act_dtype)
    silu_gate(gu, out)


ARGMAX_CHUNK = 8192      # vocabulary entries per block of the two-stage argmax
MMA_KEYS = 64          # keys per tile of the tensor-core attention kernel
MMA_TARGET_CTAS = 1184  # four waves of 2 resident CTAs on 148 SMs: many small CTAs even out the last wave


def mma_attention_supported(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int, page_size: int) -> bool:
    return (dtype == torch.bfloat16 and head_dim in (64, 128, 256) and MMA_KEYS % page_size == 0
            and n_heads % n_kv_heads == 0 and n_heads // n_kv_heads <= 16)


def decode_splits(n_requests: int, n_kv_heads: int, max_kv_len: int) -> int:
    """How many ways the decode form cuts each request's keys: enough CTAs to fill the machine several
    times over, but at least four 64-key tiles for each of them."""
    tiles = max(1, (max_kv_len + MMA_KEYS - 1) // MMA_KEYS)
    want = (MMA_TARGET_CTAS + n_requests * n_kv_heads - 1) // (n_requests * n_kv_heads)
    return max(1, min(want, tiles // 4))


def paged_attention_mma(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                        tile_req: torch.Tensor, tile_row0: torch.Tensor, n_tiles: int, q_start: torch.Tensor,
                        positions: torch.Tensor, scale: float, window: Optional[int], out: torch.Tensor,
                        decode_form: bool, n_splits: int = 1):
    """Tensor-core attention over the pages (bfloat16).  Prefill form: tile i holds up to 64/G tokens of request
    tile_req[i] from row tile_row0[i].  Decode form: every tile is one token; its keys are cut ``n_splits`` ways
    and merged through float32 scratch."""
    bf = (torch.bfloat16,)
    _need(q, "q", bf, 3)
    _need(k_pages, "k_pages", bf, 4)
    _need(v_pages, "v_pages", bf, 4)
    _need(out, "out", bf, 2)
    for name, t in (("block_table", block_table),):
        _need(t, name, _I, 2)
    for name, t in (("tile_req", tile_req), ("tile_row0", tile_row0), ("q_start", q_start), ("positions", positions)):
        _need(t, name, _I, 1)
    n, nh, d = q.shape
    n_pages, nkv, page_size, dk = k_pages.shape
    if dk != d or v_pages.shape != k_pages.shape or out.shape != (n, nh * d):
        raise KernelError(f"paged_attention_mma: q {tuple(q.shape)}, pages {tuple(k_pages.shape)}, out {tuple(out.shape)}")
    if not mma_attention_supported(q.dtype, nh, nkv, d, page_size):
        raise KernelError(f"paged_attention_mma takes head_dim 64/128/256, a page size that divides {MMA_KEYS} and at "
                          f"most 16 query heads per key/value head; got head_dim {d}, page size {page_size}, "
                          f"{nh}/{nkv} heads")
    if tile_req.shape[0] < n_tiles or tile_row0.shape[0] < n_tiles:
        raise KernelError("paged_attention_mma: tile arrays are shorter than n_tiles")
    part_o = part_ml = None
    if decode_form and n_splits > 1:
        part_o = torch.empty((n, nh, n_splits, d), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n, nh, n_splits, 2), dtype=torch.float32, device=q.device)
    _check(_core(torch.bfloat16).ib_paged_attention_mma(
        _p(q), _p(k_pages), _p(v_pages), _p(block_table), block_table.shape[1], page_size, n_pages, _p(tile_req),
        _p(tile_row0), n_tiles, _p(q_start), _p(positions), n, nh, nkv, d, float(scale), int(window) if window else 0,
        _p(out), int(decode_form), int(n_splits), _p(part_o), _p(part_ml), _stream()), "paged_attention_mma")


_DECODE_COUNTERS = {}  # device index -> zeroed int32 counters of the decode attention kernel


def tma_decode_attention_supported(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int, page_size: int) -> bool:
    return (dtype == torch.bfloat16 and head_dim == 128 and page_size >= 8 and MMA_KEYS % page_size == 0
            and n_heads % n_kv_heads == 0 and n_heads // n_kv_heads <= 16)


DECODE_RESIDENT_CTAS = 296  # two CTAs of the decode attention kernel fit on each of the 148 SMs


def decode_slices(n_requests: int, n_kv_heads: int, max_kv_len: int):
    """(max_splits, min_tiles) for :func:`paged_attention_decode`: the slices per request that the decode kernel's
    grid provides, and how the kernel picks a request's slices from its real length.

    Few requests: as many slices as still run as one wave of resident CTAs, because a CTA's fixed start-up cost
    is paid once per wave; a request uses as many as leave each slice four tiles.  Between one and one and a half
    waves of (request, head group) pairs the second wave would be nearly empty and as long as the first: three or two
    slices make four or three nearly full waves of shorter CTAs (measured at 2,048 keys: 40 requests 88 us against
    99 with one slice, 48 requests 92 against 99; inside a step of 48 requests of 8,192 keys 347 us per layer against
    400).  More pairs: one slice (at 2,048 keys 64 requests take 102 us with one slice and 115 to 123 with two to
    four; 64 requests of 8,192 keys in four slices, which would fill seven waves, take 438 us per layer inside a step
    against 421 with one)."""
    tiles = max(1, (max_kv_len + MMA_KEYS - 1) // MMA_KEYS)
    pairs = max(1, n_requests * n_kv_heads)
    most = max(1, (tiles + 3) // 4)
    room = DECODE_RESIDENT_CTAS
    if pairs <= room:
        return max(1, min(most, room // pairs)), 4
    if pairs * 3 <= 4 * room:
        return min(most, 3), 4
    if pairs * 2 <= 3 * room:
        return min(most, 2), 4
    return 1, 4


def decode_max_splits(n_requests: int, n_kv_heads: int, max_kv_len: int) -> int:
    return decode_slices(n_requests, n_kv_heads, max_kv_len)[0]


def paged_attention_decode(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                           positions: torch.Tensor, scale: float, window: Optional[int], out: torch.Tensor,
                           max_splits: int, rows: Optional[torch.Tensor] = None, reqs: Optional[torch.Tensor] = None,
                           min_tiles: int = 4):
    """Attention of one new token per request (row r = request r) over its pages: TMA-fed key/value tiles, split
    over the keys, merged by the slice that finishes last (bfloat16, head_dim 128).  With ``rows`` and ``reqs``
    (int32, equally long) only the rows named are worked on, row ``rows[i]`` being a single token of request
    ``reqs[i]``; a negative row is skipped.  The other rows of ``out`` are left alone.  A request is cut into as
    many slices as leave each ``min_tiles`` tiles of 64 keys (at most ``max_splits``)."""
    bf = (torch.bfloat16,)
    _need(q, "q", bf, 3)
    _need(k_pages, "k_pages", bf, 4)
    _need(v_pages, "v_pages", bf, 4)
    _need(out, "out", bf, 2)
    _need(block_table, "block_table", _I, 2)
    _need(positions, "positions", _I, 1)
    n_q, nh, d = q.shape
    n_pages, nkv, page_size, dk = k_pages.shape
    _need(rows, "rows", _I, 1, optional=True)
    _need(reqs, "reqs", _I, 1, optional=True)
    if (rows is None) != (reqs is None) or (rows is not None and rows.shape != reqs.shape):
        raise KernelError("paged_attention_decode: rows and reqs come together and are equally long")
    n = n_q if rows is None else rows.shape[0]
    if dk != d or v_pages.shape != k_pages.shape or out.shape != (n_q, nh * d) or positions.shape[0] != n_q \
            or (rows is None and block_table.shape[0] < n):
        raise KernelError(f"paged_attention_decode: q {tuple(q.shape)}, pages {tuple(k_pages.shape)}, out {tuple(out.shape)}")
    if n == 0:
        return
    if not tma_decode_attention_supported(q.dtype, nh, nkv, d, page_size):
        raise KernelError(f"paged_attention_decode takes head_dim 128, a page size of 8..64 that divides 64 and at most "
                          f"16 query heads per key/value head; got head_dim {d}, page size {page_size}, {nh}/{nkv} heads")
    idx = q.device.index if q.device.index is not None else torch.cuda.current_device()
    counters = _DECODE_COUNTERS.get(idx)
    if counters is None or counters.numel() < n * nkv:
        counters = torch.zeros((max(65536, n * nkv),), dtype=torch.int32, device=q.device)
        _DECODE_COUNTERS[idx] = counters
    part_o = part_ml = None
    if max_splits > 1:
        part_o = torch.empty((n, nh, max_splits, d), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n, nh, max_splits, 2), dtype=torch.float32, device=q.device)
    _check(_core(torch.bfloat16).ib_paged_attention_decode(
        _p(q), _p(k_pages), _p(v_pages), _p(block_table), block_table.shape[1], page_size, n_pages, _p(positions), n,
        nh, nkv, d, float(scale), int(window) if window else 0, _p(out), int(max_splits), int(min_tiles), _p(part_o),
        _p(part_ml), _p(counters), _p(rows), _p(reqs), _stream()), "paged_attention_decode")


def attention_decode_error(reset: bool = True) -> int:
    """0, or the code of the first bounded wait that ran out in the decode attention kernel (synchronises)."""
    return _core(torch.bfloat16).ib_attention_decode_error(int(reset))


TC_ROWS = 128  # query rows per tile of the tcgen05 attention kernel


def tcgen05_attention_supported(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int, page_size: int) -> bool:
    g = n_heads // max(n_kv_heads, 1)
    return (dtype == torch.bfloat16 and head_dim == 128 and page_size >= 8 and 128 % page_size == 0
            and n_heads % n_kv_heads == 0 and 1 <= g <= TC_ROWS)


def paged_attention_tcgen05(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                            tile_req: torch.Tensor, tile_row0: torch.Tensor, n_tiles: int, q_start: torch.Tensor,
                            positions: torch.Tensor, scale: float, window: Optional[int], out: torch.Tensor):
    """Attention of prompt portions on tcgen05 tensor cores (bfloat16, head_dim 128): tile i holds up to
    128/G tokens of request tile_req[i] from row tile_row0[i]; Q, K, V by TMA, scores and P V in tensor memory."""
    bf = (torch.bfloat16,)
    _need(q, "q", bf, 3)
    _need(k_pages, "k_pages", bf, 4)
    _need(v_pages, "v_pages", bf, 4)
    _need(out, "out", bf, 2)
    _need(block_table, "block_table", _I, 2)
    for name, t in (("tile_req", tile_req), ("tile_row0", tile_row0), ("q_start", q_start), ("positions", positions)):
        _need(t, name, _I, 1)
    n, nh, d = q.shape
    n_pages, nkv, page_size, dk = k_pages.shape
    if dk != d or v_pages.shape != k_pages.shape or out.shape != (n, nh * d):
        raise KernelError(f"paged_attention_tcgen05: q {tuple(q.shape)}, pages {tuple(k_pages.shape)}, out {tuple(out.shape)}")
    if not tcgen05_attention_supported(q.dtype, nh, nkv, d, page_size):
        raise KernelError(f"paged_attention_tcgen05 takes head_dim 128, a page size of 8..128 that divides 128 and a "
                          f"group size of at most 128; got head_dim {d}, page size {page_size}, {nh}/{nkv} heads")
    _check(_core(torch.bfloat16).ib_paged_attention_tcgen05(
        _p(q), _p(k_pages), _p(v_pages), _p(block_table), block_table.shape[1], page_size, n_pages, _p(tile_req),
        _p(tile_row0), n_tiles, _p(q_start), _p(positions), n, nh, nkv, d, float(scale), int(window) if window else 0,
        _p(out), _stream()), "paged_attention_tcgen05")


TC_PAIR_ROWS = 256  # query rows per tile of the tcgen05 attention kernel with two query tiles per CTA
PAIR_MIN_CTAS = 128  # that kernel serves steps with at least this many of its CTAs (fewer leave SMs without work)


def pair_tile_tokens(n_heads: int, n_kv_heads: int) -> int:
    """Tokens that a tile of the kernel with two query tiles holds: each query tile takes as many whole tokens (all
    heads of the group) as fit into its 128 rows."""
    return 2 * ((TC_PAIR_ROWS // 2) // (n_heads // n_kv_heads))


def tcgen05_pair_attention_supported(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int,
                                     page_size: int) -> bool:
    g = n_heads // max(n_kv_heads, 1)
    return (dtype == torch.bfloat16 and head_dim == 128 and page_size >= 8 and 128 % page_size == 0
            and n_heads % n_kv_heads == 0 and 1 <= g <= 128)


def paged_attention_pair_tcgen05(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                                 block_table: torch.Tensor, tile_req: torch.Tensor, tile_row0: torch.Tensor, n_tiles: int,
                                 q_start: torch.Tensor, positions: torch.Tensor, scale: float, window: Optional[int],
                                 out: torch.Tensor):
    """Attention of prompt portions on tcgen05 tensor cores with two query tiles per CTA that take turns
    (bfloat16, head_dim 128): tile i holds up to ``pair_tile_tokens`` tokens of request tile_req[i] from row
    tile_row0[i]; the probabilities go to the second product through tensor memory, where the output is
    accumulated too."""
    bf = (torch.bfloat16,)
    _need(q, "q", bf, 3)
    _need(k_pages, "k_pages", bf, 4)
    _need(v_pages, "v_pages", bf, 4)
    _need(out, "out", bf, 2)
    _need(block_table, "block_table", _I, 2)
    for name, t in (("tile_req", tile_req), ("tile_row0", tile_row0), ("q_start", q_start), ("positions", positions)):
        _need(t, name, _I, 1)
    n, nh, d = q.shape
    n_pages, nkv, page_size, dk = k_pages.shape
    if dk != d or v_pages.shape != k_pages.shape or out.shape != (n, nh * d):
        raise KernelError(f"paged_attention_pair_tcgen05: q {tuple(q.shape)}, pages {tuple(k_pages.shape)}, "
                          f"out {tuple(out.shape)}")
    if not tcgen05_pair_attention_supported(q.dtype, nh, nkv, d, page_size):
        raise KernelError(f"paged_attention_pair_tcgen05 takes head_dim 128, a page size of 8..128 that divides 128 and "
                          f"a group size of at most 128; got head_dim {d}, page size {page_size}, {nh}/{nkv} heads")
    _check(_core(torch.bfloat16).ib_paged_attention_pair_tcgen05(
        _p(q), _p(k_pages), _p(v_pages), _p(block_table), block_table.shape[1], page_size, n_pages, _p(tile_req),
        _p(tile_row0), n_tiles, _p(q_start), _p(positions), n, nh, nkv, d, float(scale), int(window) if window else 0,
        _p(out), _stream()), "paged_attention_pair_tcgen05")


def attention_pair_tcgen05_error(reset: bool = True) -> int:
    """0, or the code of the first bounded wait that ran out in the kernel above (synchronises)."""
    return _core(torch.bfloat16).ib_attention_pair_tcgen05_error(int(reset))


def attention_tcgen05_error(reset: bool = True) -> int:
    """0, or the code of the first bounded wait that ran out in the tcgen05 attention kernel (synchronises)."""
    return _core(torch.bfloat16).ib_attention_tcgen05_error(int(reset))


def paged_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                    ctx, scale: float, window: Optional[int], out: torch.Tensor):
    """Attention of every row of the step over its request's pages; picks the kernel for the sizes.

    ``ctx`` is the step's :class:`~inferrs_b200.engine.batch.StepContext` (row_request, positions
    and what the faster kernels need to cut the work).
    """
    n, nh, d = q.shape
    nkv, page_size = k_pages.shape[1], k_pages.shape[2]
    if not mma_attention_supported(q.dtype, nh, nkv, d, page_size):
        paged_attention_generic(q, k_pages, v_pages, block_table, ctx.row_request, ctx.positions, scale, window, out)
        return
    # Prompt portions: tiles of 256 rows (two query tiles per CTA) where they still give every SM a CTA, else
    # tiles of 128 rows.  A step that stands for a padded one (before its graph is captured) says so.
    pair_tokens = pair_tile_tokens(nh, nkv)
    rows_for_dispatch = ctx.extra.get("dispatch_rows", ctx.n_rows)
    pair = tcgen05_pair_attention_supported(q.dtype, nh, nkv, d, page_size) \
        and (rows_for_dispatch // pair_tokens) * nkv >= PAIR_MIN_CTAS
    prefill_kernel = paged_attention_pair_tcgen05 if pair else paged_attention_tcgen05
    prefill_tokens = pair_tokens if pair else TC_ROWS // (nh // nkv)
    if ctx.decode_only and tma_decode_attention_supported(q.dtype, nh, nkv, d, page_size):
        max_splits, min_tiles = decode_slices(ctx.n_requests, nkv, ctx.max_kv_len)
        paged_attention_decode(q, k_pages, v_pages, block_table, ctx.positions, scale, window, out, max_splits,
                               min_tiles=min_tiles)
    elif ctx.decode_only:
        # one row per request: the rows are the tiles
        splits = decode_splits(ctx.n_requests, nkv, ctx.max_kv_len)
        paged_attention_mma(q, k_pages, v_pages, block_table, ctx.row_request, ctx.q_start, ctx.n_requests,
                            ctx.q_start, ctx.positions, scale, window, out, True, splits)
    elif tcgen05_attention_supported(q.dtype, nh, nkv, d, page_size) \
            and tma_decode_attention_supported(q.dtype, nh, nkv, d, page_size):
        # portions of prompts and single tokens side by side: the single tokens go to the decode kernel (a tile
        # of the prefill kernel would hold one token of 32), the portions to the prefill kernel
        rows, reqs, n_single = ctx.single_rows()
        if n_single > 0:
            max_splits, min_tiles = decode_slices(n_single, nkv, ctx.max_kv_len)
            paged_attention_decode(q, k_pages, v_pages, block_table, ctx.positions, scale, window, out, max_splits,
                                   rows, reqs, min_tiles=min_tiles)
        tile_req, tile_row0, n_tiles = ctx.attention_tiles(prefill_tokens, portions_only=True)
        if n_tiles > 0:
            prefill_kernel(q, k_pages, v_pages, block_table, tile_req, tile_row0, n_tiles, ctx.q_start,
                           ctx.positions, scale, window, out)
    elif tcgen05_attention_supported(q.dtype, nh, nkv, d, page_size):
        tile_req, tile_row0, n_tiles = ctx.attention_tiles(prefill_tokens)
        prefill_kernel(q, k_pages, v_pages, block_table, tile_req, tile_row0, n_tiles, ctx.q_start,
                       ctx.positions, scale, window, out)
    else:
        tile_req, tile_row0, n_tiles = ctx.attention_tiles(MMA_KEYS // (nh // nkv))
        paged_attention_mma(q, k_pages, v_pages, block_table, tile_req, tile_row0, n_tiles, ctx.q_start,
                            ctx.positions, scale, window, out, False)


def penalties(logits: torch.Tensor, prev: torch.Tensor, n_prev: torch.Tensor, repetition: torch.Tensor,
              frequency: torch.Tensor, presence: torch.Tensor, act_dtype: torch.dtype = torch.float32):
    """In place on float32 logits [R, V]: repetition, frequency and presence penalties for the tokens in
    each row's window ``prev[r, :n_prev[r]]`` (int32)."""
    _need(logits, "logits", (torch.float32,), 2)
    _need(prev, "prev", _I, 2)
    _need(n_prev, "n_prev", _I, 1)
    r = logits.shape[0]
    for name, t in (("repetition", repetition), ("frequency", frequency), ("presence", presence)):
        _need(t, name, (torch.float32,), 1)
        if t.shape[0] != r:
            raise KernelError(f"penalties: {name} has {t.shape[0]} entries for {r} rows")
    if prev.shape[0] != r or n_prev.shape[0] != r:
        raise KernelError(f"penalties: prev {tuple(prev.shape)}, n_prev {tuple(n_prev.shape)} for {r} rows")
    _check(_core(act_dtype).ib_penalties(_p(logits), logits.shape[1], r, logits.shape[1], _p(prev), prev.shape[1],
                                         _p(n_prev), _p(repetition), _p(frequency), _p(presence), _stream()),
           "penalties")


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           min_p: torch.Tensor, uniform: torch.Tensor, out: torch.Tensor, act_dtype: torch.dtype = torch.float32,
           cluster: int = 0):
    """One token per row of float32 logits [R, V]: largest logit where temperature < 1e-5, else
    temperature, top-k, top-p, min-p and the inverse-CDF walk with the row's random number ``uniform``.
    ``cluster``: CTAs that share a row (1, 2, 4 or 8; 0 lets the kernel library choose by the number of rows)."""
    _need(logits, "logits", (torch.float32,), 2)
    r = logits.shape[0]
    for name, t, dt in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
                        ("top_p", top_p, torch.float32), ("min_p", min_p, torch.float32),
                        ("uniform", uniform, torch.float32), ("out", out, torch.int32)):
        _need(t, name, (dt,), 1)
        if t.shape[0] != r:
            raise KernelError(f"sample: {name} has {t.shape[0]} entries for {r} rows")
    scratch = torch.empty((r, logits.shape[1]), dtype=torch.float32, device=logits.device)
    _check(_core(act_dtype).ib_sample(_p(logits), logits.shape[1], r, logits.shape[1], _p(temperature), _p(top_k),
                                      _p(top_p), _p(min_p), _p(uniform), _p(scratch), int(cluster), _p(out), _stream()),
           "sample")


_GEMM_LIB = None


def _gemm_lib():
    global _GEMM_LIB
    if _GEMM_LIB is None:
        lib = load_library("gemm_bf16")
        lib.ib_gemm_tn_tcgen05.argtypes = [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int,
                                           c_int, c_int, c_void_p]
        lib.ib_gemm_tn_tcgen05.restype = c_int
        lib.ib_gemm_swiglu_tcgen05.argtypes = [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int,
                                               c_void_p]
        lib.ib_gemm_swiglu_tcgen05.restype = c_int
        lib.ib_gemm_tn_tcgen05_folded.argtypes = [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int,
                                                  c_int, c_void_p, c_int, c_float, c_int, c_void_p, c_long, c_void_p,
                                                  c_int, c_void_p, c_void_p]
        lib.ib_gemm_tn_tcgen05_folded.restype = c_int
        lib.ib_gemm_swiglu_tcgen05_folded.argtypes = [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int,
                                                      c_int, c_void_p, c_int, c_float, c_int, c_void_p]
        lib.ib_gemm_swiglu_tcgen05_folded.restype = c_int
        lib.ib_gemm_tcgen05_ssq_parts.argtypes = [c_int, c_int, c_int, c_int]
        lib.ib_gemm_tcgen05_ssq_parts.restype = c_int
        lib.ib_gemm_chain.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p]
        lib.ib_gemm_chain.restype = c_int
        lib.ib_gemm_chain_workspace_floats.argtypes = [c_int]
        lib.ib_gemm_chain_workspace_floats.restype = c_long
        lib.ib_gemm_chain_workspace_fill.argtypes = []
        lib.ib_gemm_chain_workspace_fill.restype = c_int
        lib.ib_gemm_chain_max_products.argtypes = []
        lib.ib_gemm_chain_max_products.restype = c_int
        lib.ib_gemm_chain_ssq_parts.argtypes = [c_int]
        lib.ib_gemm_chain_ssq_parts.restype = c_int
        lib.ib_gemm_chain_set_pdl.argtypes = [c_int]
        lib.ib_gemm_chain_set_pdl.restype = None
        lib.ib_gemm_chain_error.argtypes = [c_int]
        lib.ib_gemm_chain_error.restype = c_int
        lib.ib_gemm_chain_error_async.argtypes = [c_void_p, c_void_p]
        lib.ib_gemm_chain_error_async.restype = c_int
        lib.ib_gemm_tcgen05_error.argtypes = [c_int]
        lib.ib_gemm_tcgen05_error.restype = c_int
        lib.ib_gemm_tcgen05_error_async.argtypes = [c_void_p, c_void_p]
        lib.ib_gemm_tcgen05_error_async.restype = c_int
        _GEMM_LIB = lib
    return _GEMM_LIB


def tcgen05_gemm_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """TMA needs 16-byte aligned bases and row strides: K a multiple of 8 for bfloat16."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def _scaled_args(x):
    if isinstance(x, ScaledRows):
        _need(x.ssq, "ssq", (torch.float32,), 2)
        if x.ssq.shape[1] != SSQ_LD or x.ssq.shape[0] < x.n_parts or x.n_parts <= 0:
            raise KernelError(f"scaled rows: {x.n_parts} parts do not fit a list of shape {tuple(x.ssq.shape)}")
        return x.x, (_p(x.ssq), int(x.n_parts), float(x.eps), int(x.width))
    return x, (None, 0, 0.0, 0)


def gemm_tn_tcgen05(x, w: torch.Tensor, out: torch.Tensor, split_k: int = 0, sink: Optional[ResidualSink] = None):
    """out = x @ w.T with TMA-fed tcgen05 MMAs: W is the 128-row operand, the tokens are the N dimension.
    ``split_k`` 0 lets the kernel library choose how many CTAs of a cluster share one output tile.  ``x`` may be
    :class:`ScaledRows` and the result may go to a :class:`ResidualSink` (both: up to 32 rows, bfloat16 out); with a
    sink the :class:`ScaledRows` that stand for the next norm's output are returned."""
    xt, scaled = _scaled_args(x)
    _need(xt, "x", (torch.bfloat16,), 2)
    _need(w, "w", (torch.bfloat16,), 2)
    _need(out, "out", _W, 2)
    n, k = xt.shape
    m = w.shape[0]
    if w.shape[1] != k or out.shape != (n, m):
        raise KernelError(f"gemm: x {tuple(xt.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    lib = _gemm_lib()
    if scaled[0] is None and sink is None:
        code = lib.ib_gemm_tn_tcgen05(_p(xt), k, _p(w), k, _p(out), m, int(out.dtype == torch.float32), n, m, k, split_k,
                                      _stream())
        if code == -1:
            raise KernelError(f"gemm_tn_tcgen05: K={k} must be a multiple of 8 and the bases 16-byte aligned")
        _check(code, "gemm_tn_tcgen05")
        return None
    if out.dtype != torch.bfloat16:
        raise KernelError("gemm_tn_tcgen05: the folded forms store bfloat16")
    result, sink_args = None, (None, 0, None, 0, None)
    if sink is not None:
        _need(sink.residual, "residual", (torch.float32,), 2)
        _need(sink.weight, "sink weight", _W, 1)
        if sink.residual.shape != (n, m) or sink.weight.shape[0] != m:
            raise KernelError(f"gemm: residual {tuple(sink.residual.shape)} and norm weight {tuple(sink.weight.shape)} "
                              f"do not match the result {(n, m)}")
        parts = lib.ib_gemm_tcgen05_ssq_parts(n, m, k, split_k)
        if parts <= 0:
            raise KernelError(f"gemm_tn_tcgen05: {n} rows take no sink")
        ssq = torch.empty((parts, SSQ_LD), dtype=torch.float32, device=out.device)
        sink_args = (_p(sink.residual), m, _p(sink.weight), int(sink.weight.dtype == torch.float32), _p(ssq))
        result = ScaledRows(out, ssq, parts, float(sink.eps), m)
    code = lib.ib_gemm_tn_tcgen05_folded(_p(xt), k, _p(w), k, _p(out), m, n, m, k, split_k, *scaled, *sink_args, _stream())
    if code == -1:
        raise KernelError(f"gemm_tn_tcgen05: the folded forms take up to {SSQ_LD} rows, K={k} a multiple of 8 and "
                          f"16-byte aligned bases")
    _check(code, "gemm_tn_tcgen05 (folded)")
    return result


def gemm_swiglu_tcgen05(x, w_gate_up: torch.Tensor, out: torch.Tensor):
    """out[t, f] = silu(x[t] . w[f]) * (x[t] . w[inner + f]): both products of a gated feed-forward and the gate
    in one tcgen05 kernel (up to 64 gate rows and the same up rows per tile).  Up to 32 rows of x, which may be
    :class:`ScaledRows`."""
    xt, scaled = _scaled_args(x)
    _need(xt, "x", (torch.bfloat16,), 2)
    _need(w_gate_up, "w_gate_up", (torch.bfloat16,), 2)
    _need(out, "out", (torch.bfloat16,), 2)
    n, k = xt.shape
    inner = out.shape[1]
    if w_gate_up.shape != (2 * inner, k) or out.shape[0] != n:
        raise KernelError(f"gemm_swiglu: x {tuple(xt.shape)}, w {tuple(w_gate_up.shape)}, out {tuple(out.shape)}")
    code = _gemm_lib().ib_gemm_swiglu_tcgen05_folded(_p(xt), k, _p(w_gate_up), k, _p(out), inner, n, inner, k, *scaled,
                                                     _stream())
    if code == -1:
        raise KernelError(f"gemm_swiglu_tcgen05: at most 32 rows (got {n}), K={k} a multiple of 8, 16-byte aligned bases")
    _check(code, "gemm_swiglu_tcgen05")


def gemm_tcgen05_set_pdl(on: bool):
    """Let tcgen05 products start before their predecessor in the stream has finished (they prefetch weights and
    wait for the predecessor before touching anything else).  Only safe among kernels that all wait likewise."""
    _gemm_lib().ib_gemm_tcgen05_set_pdl(int(bool(on)))
    _gemm_lib().ib_gemm_chain_set_pdl(int(bool(on)))


def gemm_tcgen05_set_even_tiles(on: bool):
    """Whether a tcgen05 product whose CTAs all run at once cuts its tiles lower than the MMA so that every SM gets
    the same number of them (default) or keeps every tile at the MMA's height."""
    lib = _gemm_lib()
    lib.ib_gemm_tcgen05_set_even_tiles.argtypes = [c_int]
    lib.ib_gemm_tcgen05_set_even_tiles.restype = None
    lib.ib_gemm_tcgen05_set_even_tiles(int(bool(on)))


def gemm_tcgen05_tile_rows(n_rows: int, n_out: int, k: int, split_k: int = 0, gated: bool = False) -> int:
    """Rows of the weight matrix per tile (of each of the two matrices in the gated form) that a tcgen05 product of
    these sizes takes: the MMA's 128 (64), or fewer where that spreads the product evenly over the SMs."""
    lib = _gemm_lib()
    lib.ib_gemm_tcgen05_tile_rows.argtypes = [c_int, c_int, c_int, c_int, c_int]
    lib.ib_gemm_tcgen05_tile_rows.restype = c_int
    return int(lib.ib_gemm_tcgen05_tile_rows(n_rows, n_out, k, split_k, int(gated)))


def set_pdl(on: bool, act_dtype: torch.dtype = torch.bfloat16):
    """Programmatic dependent launch for every kernel of the package launched from now on: a kernel may start
    while the one before it in the stream still runs, does what needs no input (barrier set-up, fetching
    weights) and waits for the earlier kernel before it reads or writes anything else.  Used while a decode
    step is captured into a CUDA graph; library kernels in between simply keep plain stream order."""
    lib = _core(act_dtype)
    lib.ib_set_pdl.argtypes = [c_int]
    lib.ib_set_pdl.restype = None
    lib.ib_set_pdl(int(bool(on)))
    if act_dtype == torch.bfloat16:
        gemm_tcgen05_set_pdl(on)


# up to this many rows the own tcgen05 product is the faster one in a decode step (the environment variable is
# there for measuring other thresholds)
TCGEN05_MAX_TOKENS = int(os.environ.get("INFERRS_B200_TCGEN05_MAX_TOKENS", "16"))
SWIGLU_MAX_TOKENS = 32  # rows that the fused gate/up kernel takes


def gemm_tcgen05_error(reset: bool = True) -> int:
    """0, or the code of the first bounded wait that ran out in a tcgen05 GEMM (synchronises with the device)."""
    return _gemm_lib().ib_gemm_tcgen05_error(int(reset))


def gemm_chain_error(reset: bool = True) -> int:
    """0, or the code of the first bounded wait that ran out in a chain of products (synchronises)."""
    code = _gemm_lib().ib_gemm_chain_error(int(reset))
    if code != 0 and reset:
        _CHAIN_WS.clear()    # a chain that gave up may have left marks in its workspace: the next chain gets a fresh one
    return code


# ---- the kernels' error words, all of them ------------------------------------------------------------------
# A bounded wait that ran out, or a row whose position lay outside the rotation tables, leaves a code in a word
# on the device.  The functions above read one word each and wait for the device; these read all of them the way
# a serving loop wants it: asked for in stream order, read later from pinned memory.
ERROR_WORDS = ("a row's position outside the rotation tables", "prefill attention (tcgen05)",
               "prefill attention (two query tiles)", "decode attention", "matrix product (tcgen05)",
               "chain of matrix products")


def error_words_async(host: torch.Tensor, act_dtype: torch.dtype):
    """Ask for every error word of the kernel libraries, in the order of ``ERROR_WORDS``, to be copied into ``host``
    (pinned int32, at least ``len(ERROR_WORDS)`` long) behind the work that the current stream holds.  The caller
    records an event after this call and reads ``host`` once the event has come."""
    if host.dtype != torch.int32 or host.numel() < len(ERROR_WORDS) or not host.is_pinned():
        raise KernelError("error_words_async wants a pinned int32 tensor with room for every word")
    core, stream, at = _core(act_dtype), _stream(), host.data_ptr()
    calls = [core.ib_row_fault_async, core.ib_attention_tcgen05_error_async,
             core.ib_attention_pair_tcgen05_error_async, core.ib_attention_decode_error_async]
    if act_dtype == torch.bfloat16:
        calls += [_gemm_lib().ib_gemm_tcgen05_error_async, _gemm_lib().ib_gemm_chain_error_async]
    else:
        host[len(calls):len(ERROR_WORDS)] = 0
    for i, fn in enumerate(calls):
        code = fn(at + 4 * i, stream)
        if code != 0:
            raise KernelError(f"error_words_async: CUDA error {code}")


def reset_error_words(act_dtype: torch.dtype) -> dict:
    """Read every error word now (waits for the device), clear them, and put the decode attention's counters back
    to zero (a wait that ran out may have left a slice uncounted).  Returns {name: code} of the words that were set."""
    found = {}
    row = row_fault(act_dtype, reset=True)
    if row is not None:
        found[ERROR_WORDS[0]] = row + 1
    if act_dtype == torch.bfloat16:
        for name, fn in zip(ERROR_WORDS[1:], (attention_tcgen05_error, attention_pair_tcgen05_error,
                                              attention_decode_error, gemm_tcgen05_error, gemm_chain_error)):
            v = fn(True)
            if v:
                found[name] = v
    for counters in _DECODE_COUNTERS.values():
        counters.zero_()
    return found
