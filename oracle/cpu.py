"""ctypes front end of the CPU parity oracle (``liboracle.so``).  TEST INFRASTRUCTURE ONLY.

Only the tests, ``__graft_entry__.smoke`` and the benchmark's CPU-baseline legs may
import this module; the product package never does.  All functions take and return
CPU torch tensors.  The arithmetic lives in ``oracle.c``; each wrapper names the
reference code (paths relative to the reference project) that it restates.
"""

from __future__ import annotations

import ctypes
import subprocess
from functools import lru_cache
from pathlib import Path

import torch

_HERE = Path(__file__).resolve().parent
_OUT_KIND = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def build() -> Path:
    """Compile ``liboracle.so`` beside its source if it is missing or stale."""
    library = _HERE / "liboracle.so"
    source = _HERE / "oracle.c"
    if not library.exists() or library.stat().st_mtime < source.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "liboracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return library


@lru_cache(maxsize=1)
def _lib():
    lib = ctypes.CDLL(str(build()))
    lib.oracle_threads.restype = ctypes.c_int
    for name in ("oracle_int8_gemm", "oracle_route", "oracle_swiglu_quantize", "oracle_quantize_rows",
                 "oracle_ragged_gemm", "oracle_combine"):
        getattr(lib, name).restype = ctypes.c_int
    return lib


def threads() -> int:
    return int(_lib().oracle_threads())


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def _i64(v):
    return ctypes.c_int64(int(v))


def int8_gemm(a, b, scale_a, scale_b, group_size, output_dtype=torch.float32,
              return_partials=False):
    """Grouped W8A8 GEMM; restates ``src/grain_gemm/kernels/triton.py:28-51``.

    Accepts any strides.  Returns the result in ``output_dtype``; with
    ``return_partials`` also the INT32 group dots as ``[M, N, ceil(K/G)]``.
    """
    m, k = a.shape
    n = b.shape[1]
    groups = (k + group_size - 1) // group_size
    out = torch.zeros((m, n), dtype=torch.float32)
    partials = torch.zeros((m, n, groups), dtype=torch.int32) if return_partials else None
    status = _lib().oracle_int8_gemm(
        _p(a), _p(b), _p(scale_a), _p(scale_b), _p(out), _p(partials),
        _i64(m), _i64(n), _i64(k),
        _i64(a.stride(0)), _i64(a.stride(1)), _i64(b.stride(0)), _i64(b.stride(1)),
        _i64(scale_a.stride(0)), _i64(scale_a.stride(1)),
        _i64(scale_b.stride(0)), _i64(scale_b.stride(1)),
        ctypes.c_int(group_size), ctypes.c_int(_OUT_KIND[output_dtype]))
    if status:
        raise RuntimeError(f"oracle_int8_gemm failed with status {status}")
    result = out.to(output_dtype)
    return (result, partials) if return_partials else result


class Routes:
    """Routing metadata; field meaning as ``src/grain_gemm/kernels/moe.py:20-45``."""

    def __init__(self, order, inverse, counts, offsets, effective_ids, statistics,
                 tokens, top_k, experts):
        self.order, self.inverse, self.counts = order, inverse, counts
        self.offsets, self.effective_ids, self.statistics = offsets, effective_ids, statistics
        self.tokens, self.top_k, self.experts = tokens, top_k, experts


def route(topk_ids, num_experts, token_mask=None):
    """Stable routing sort; restates ``src/grain_gemm/kernels/moe.py:222-291``."""
    tokens, top_k = topk_ids.shape
    slots = tokens * top_k
    ids = topk_ids.contiguous()
    mask = token_mask.contiguous().to(torch.uint8) if token_mask is not None else None
    effective = torch.empty((slots,), dtype=ids.dtype)
    order = torch.empty((slots,), dtype=torch.int64)
    inverse = torch.empty((slots,), dtype=torch.int32)
    counts = torch.empty((num_experts,), dtype=torch.int32)
    offsets = torch.empty((num_experts + 1,), dtype=torch.int32)
    statistics = torch.empty((3,), dtype=torch.int32)
    status = _lib().oracle_route(
        _p(ids), ctypes.c_int(int(ids.dtype == torch.int64)), _p(mask),
        _i64(tokens), _i64(top_k), _i64(num_experts),
        _p(effective), _p(order), _p(inverse), _p(counts), _p(offsets), _p(statistics))
    if status:
        raise RuntimeError(f"oracle_route failed with status {status}")
    return Routes(order, inverse, counts, offsets, effective, statistics,
                  tokens, top_k, num_experts)


def silu(values):
    """``v / (1 + expf(-v))`` in FP32 with the host C library's ``expf``
    (the SwiGLU formula of ``src/grain_gemm/kernels/moe.py:594``)."""
    source = values.float().contiguous()
    out = torch.empty_like(source)
    _lib().oracle_silu.restype = None
    _lib().oracle_silu(_p(source), _p(out), _i64(source.numel()))
    return out


def swiglu_quantize(gate_up, valid_rows=None, gate_up_layout="split", silu_table=None):
    """SwiGLU + G256 requantisation; restates ``src/grain_gemm/kernels/moe.py:564-601``.

    ``gate_up`` is ``[rows, 2I]`` in BF16/FP16/FP32 (the already rounded GEMM output).
    ``silu_table`` (65536 FP32 values indexed by the 16-bit pattern of ``gate_up``'s dtype)
    replaces the evaluation of ``gate / (1 + expf(-gate))`` by a lookup.
    """
    rows, twice = gate_up.shape
    inter = twice // 2
    values = gate_up.float().contiguous()
    q = torch.empty((rows, inter), dtype=torch.int8)
    s = torch.empty((rows, inter // 256), dtype=torch.float32)
    table = None
    if silu_table is not None:
        if gate_up.dtype not in (torch.bfloat16, torch.float16):
            raise ValueError("a SiLU table needs 16-bit gate/up values")
        table = silu_table.float().contiguous()
        assert table.numel() == 65536
    status = _lib().oracle_swiglu_quantize(
        _p(values), _i64(rows), _i64(rows if valid_rows is None else valid_rows), _i64(inter),
        ctypes.c_int(int(gate_up_layout == "interleaved")), _p(q), _p(s), _p(table),
        ctypes.c_int(_OUT_KIND[gate_up.dtype] if table is not None else 0))
    if status:
        raise RuntimeError(f"oracle_swiglu_quantize failed with status {status}")
    return q, s


def router_topk(logits, top_k):
    """Router front-end: logits -> softmax -> top-k -> renormalise, as the reference's callers do
    it before ``moe_ffn`` (``benchmarks/bench_moe_ffn.py:283-285``, ``docs/moe_ffn.md:5-7``).

    Ids in descending order of logit, ties to the lower id; weights
    ``exp(l_i - l_max) / sum_selected exp(l_j - l_max)`` with the sum taken in selection order.
    """
    values = logits.float()
    order = torch.argsort(-values, dim=-1, stable=True)[:, :top_k]
    selected = values.gather(1, order)
    weights = torch.exp(selected - selected[:, :1])
    total = torch.zeros_like(weights[:, 0])
    for r in range(top_k):
        total = total + weights[:, r]
    return weights / total[:, None], order


def quantize_rows(x, group_size=256):
    """Entry quantiser; restates ``quantize_rows`` (``src/grain_gemm/kernels/moe.py:321-356``).

    ``x`` is ``[..., K]`` in BF16/FP16/FP32; returns INT8 data of the same shape and FP32
    scales ``[..., K / group_size]``.
    """
    width = x.shape[-1]
    values = x.float().contiguous().reshape(-1, width)
    rows = values.shape[0]
    q = torch.empty((rows, width), dtype=torch.int8)
    s = torch.empty((rows, width // group_size), dtype=torch.float32)
    status = _lib().oracle_quantize_rows(_p(values), _i64(rows), _i64(width), _i64(group_size),
                                         _p(q), _p(s))
    if status:
        raise RuntimeError(f"oracle_quantize_rows failed with status {status}")
    return q.reshape(x.shape), s.reshape(*x.shape[:-1], width // group_size)


def ragged_gemm(a, w_linear, scale_a, scale_b, routes, output_dtype, source_is_token):
    """All experts' grouped GEMMs over the sorted slots; restates
    ``src/grain_gemm/kernels/moe.py:359-415``.  ``w_linear`` is ``[E, N, K]`` contiguous.
    Rows of invalid slots are returned as zero."""
    experts, n, k = w_linear.shape
    slots = routes.tokens * routes.top_k
    out = torch.zeros((slots, n), dtype=torch.float32)
    a, w_linear = a.contiguous(), w_linear.contiguous()
    scale_a, scale_b = scale_a.contiguous(), scale_b.contiguous()
    status = _lib().oracle_ragged_gemm(
        _p(a), _p(scale_a), _p(w_linear), _p(scale_b), _p(routes.order), _p(routes.offsets),
        _p(out), _i64(experts), _i64(n), _i64(k), _i64(routes.top_k),
        ctypes.c_int(int(source_is_token)), ctypes.c_int(_OUT_KIND[output_dtype]))
    if status:
        raise RuntimeError(f"oracle_ragged_gemm failed with status {status}")
    return out.to(output_dtype)


def combine(expert_output, topk_weights, routes, output_dtype):
    """Top-k weighted FP32 reduction; restates ``src/grain_gemm/kernels/moe.py:634-653``."""
    tokens, top_k = routes.tokens, routes.top_k
    h = expert_output.shape[-1]
    values = expert_output.float().contiguous()
    weights = topk_weights.float().contiguous()
    out = torch.zeros((tokens, h), dtype=torch.float32)
    status = _lib().oracle_combine(_p(values), _p(weights), _p(routes.inverse), _p(out),
                                   _i64(tokens), _i64(top_k), _i64(h),
                                   ctypes.c_int(_OUT_KIND[output_dtype]))
    if status:
        raise RuntimeError(f"oracle_combine failed with status {status}")
    return out.to(output_dtype)


def moe_ffn(hidden_states, w_gate_up, w_down, topk_weights, topk_ids, *, scale_x,
            scale_gate_up, scale_down, token_mask=None, output_dtype=torch.bfloat16,
            gate_up_layout="split", return_stages=False, silu_table=None):
    """Full pre-routed INT8 G256 MoE FFN; stage order of ``src/grain_gemm/moe.py:296-346``.

    ``w_gate_up`` ``[E,H,2I]`` and ``w_down`` ``[E,I,H]`` are the logical (transposed)
    views the public API takes.
    """
    experts = w_gate_up.shape[0]
    routes = route(topk_ids, experts, token_mask)
    valid = int(routes.offsets[-1])
    w1 = w_gate_up.transpose(-2, -1).contiguous()
    w2 = w_down.transpose(-2, -1).contiguous()
    gate_up = ragged_gemm(hidden_states, w1, scale_x, scale_gate_up, routes,
                          output_dtype, source_is_token=True)
    qh, sh = swiglu_quantize(gate_up, valid, gate_up_layout, silu_table)
    expert_out = ragged_gemm(qh, w2, sh, scale_down, routes, output_dtype,
                             source_is_token=False)
    out = combine(expert_out, topk_weights, routes, output_dtype)
    if return_stages:
        return out, dict(routes=routes, gate_up=gate_up, qh=qh, sh=sh, expert_out=expert_out)
    return out


def fmaf(x, y, z):
    """Element-wise exact FP32 fused multiply-add on numpy float32 arrays."""
    import numpy as np
    x, y, z = np.broadcast_arrays(np.asarray(x, np.float32), np.asarray(y, np.float32),
                                  np.asarray(z, np.float32))
    x, y, z = (np.ascontiguousarray(v) for v in (x, y, z))
    out = np.empty_like(x)
    _lib().oracle_fmaf.restype = None
    _lib().oracle_fmaf(ctypes.c_void_p(x.ctypes.data), ctypes.c_void_p(y.ctypes.data),
                       ctypes.c_void_p(z.ctypes.data), ctypes.c_void_p(out.ctypes.data),
                       _i64(x.size))
    return out
