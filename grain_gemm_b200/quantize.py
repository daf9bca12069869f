"""The steps immediately before the two hot paths: activation quantisation and weight
preparation, with the reference's names and conventions.

* ``quantize_rows`` mirrors ``quantize_rows`` of ``src/grain_gemm/kernels/moe.py:344-356`` of
  the reference (symmetric INT8, one FP32 scale per row and K group) and runs the CUDA kernel
  behind ``gg_quantize_rows``.
* ``route_topk`` is the router front-end (logits -> softmax -> top-k -> renormalise) that the
  reference leaves to its callers (``benchmarks/bench_moe_ffn.py:283-285``).
* ``prepare_weight`` and ``interleave_gate_up`` restate the preparation recipes of the
  reference's ``docs/moe_ffn.md:119-133`` and ``docs/moe_interleaved.md:32-40``; they run once,
  outside the forward pass, as plain tensor operations.
"""

from __future__ import annotations

import torch

from . import _loader


def quantize_rows(x, group_size=256, *, rows_per_program=4):
    """Quantize contiguous floating rows; return INT8 data and FP32 row scales.

    ``x`` is ``[..., K]`` (FP32, BF16 or FP16, contiguous, on a B200), ``K`` a multiple of 256
    and ``group_size`` one of 32, 64, 128, 256.  Returns ``(q, scales)`` with ``q`` INT8 of
    ``x``'s shape and ``scales`` FP32 ``[..., K // group_size]``:
    ``scale = max(|x|_group, 1e-12) / 127`` and ``q = clamp(rint(x / scale), -127, 127)``.
    ``rows_per_program`` is accepted for signature compatibility and ignored.
    """
    del rows_per_program
    if not isinstance(x, torch.Tensor) or x.dim() < 1:
        raise ValueError("x must be a tensor with at least one dimension")
    if x.dtype not in _loader.OUT_DTYPE:
        raise ValueError("x must be torch.float32, torch.bfloat16 or torch.float16")
    if group_size not in (32, 64, 128, 256):
        raise ValueError("group_size must be one of 32, 64, 128 or 256")
    width = x.shape[-1]
    if width == 0 or width % 256:
        raise ValueError("the last dimension must be a positive multiple of 256")
    if x.device.type != "cuda":
        raise ValueError("x must be a CUDA tensor")
    if not x.is_contiguous():
        raise ValueError("x must be contiguous")
    if torch.cuda.get_device_capability(x.device) != (10, 0):
        raise RuntimeError("this build of quantize_rows requires an NVIDIA B200 (sm_100) GPU")
    rows = x.numel() // width
    quantized = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    scales = torch.empty((*x.shape[:-1], width // group_size), dtype=torch.float32, device=x.device)
    if rows:
        lib = _loader.library()
        with torch.cuda.device(x.device):
            _loader.check(lib.gg_quantize_rows(
                _loader.pointer(x), _loader.OUT_DTYPE[x.dtype], rows, width, group_size,
                _loader.pointer(quantized), _loader.pointer(scales),
                _loader.stream_pointer(x.device)), "gg_quantize_rows")
    return quantized, scales


def route_topk(logits, top_k, *, ids_dtype=torch.int64):
    """Router front-end: the ``top_k`` experts of every token and their routing weights.

    ``logits`` is ``[T, E]`` (FP32, BF16 or FP16, contiguous, finite, ``E <= 1024``).  Returns
    ``(topk_weights [T, top_k] FP32, topk_ids [T, top_k])`` ready for ``moe_ffn``: ids in
    descending order of logit (ties to the lower id) and ``softmax(logits)`` of the selected
    experts renormalised to sum to one.
    """
    if not isinstance(logits, torch.Tensor) or logits.dim() != 2:
        raise ValueError("logits must be a [T, E] tensor")
    if logits.dtype not in _loader.OUT_DTYPE:
        raise ValueError("logits must be torch.float32, torch.bfloat16 or torch.float16")
    tokens, experts = logits.shape
    if not 0 < top_k <= experts or experts > 1024:
        raise ValueError("need 0 < top_k <= E <= 1024")
    if ids_dtype not in (torch.int32, torch.int64):
        raise ValueError("ids_dtype must be torch.int32 or torch.int64")
    if logits.device.type != "cuda" or not logits.is_contiguous():
        raise ValueError("logits must be a contiguous CUDA tensor")
    weights = torch.empty((tokens, top_k), dtype=torch.float32, device=logits.device)
    ids = torch.empty((tokens, top_k), dtype=ids_dtype, device=logits.device)
    if tokens:
        lib = _loader.library()
        with torch.cuda.device(logits.device):
            _loader.check(lib.gg_moe_topk(
                _loader.pointer(logits), _loader.OUT_DTYPE[logits.dtype], tokens, experts, top_k,
                _loader.pointer(weights), _loader.pointer(ids), int(ids_dtype == torch.int64),
                _loader.stream_pointer(logits.device)), "gg_moe_topk")
    return weights, ids


def route_topk_routes(logits, top_k, *, token_mask=None, ids_dtype=torch.int64, tile_rows=128):
    """``route_topk`` and ``moe.prepare_routes`` together: ``(topk_weights, topk_ids, routes)``.

    For decode-sized problems (``T * top_k <= 1024``) both steps run in ONE kernel launch
    (``gg_moe_route_topk``: the CTA that selects the experts sorts the assignments it has just
    written); larger problems make the two calls.  Pass ``routes`` on to
    ``moe_ffn(..., routes=routes)`` to skip its own routing.  Results are identical either way.
    """
    from . import moe
    if not isinstance(logits, torch.Tensor) or logits.dim() != 2:
        raise ValueError("logits must be a [T, E] tensor")
    tokens, experts = logits.shape
    fused = (0 < tokens * top_k <= 1024 and 0 < top_k <= experts <= 1024
             and logits.dtype in _loader.OUT_DTYPE and logits.device.type == "cuda"
             and logits.is_contiguous() and ids_dtype in (torch.int32, torch.int64))
    if not fused:
        weights, ids = route_topk(logits, top_k, ids_dtype=ids_dtype)
        return weights, ids, moe.prepare_routes(ids, experts, token_mask, tile_rows=tile_rows)
    device = logits.device
    slots = tokens * top_k
    weights = torch.empty((tokens, top_k), dtype=torch.float32, device=device)
    ids = torch.empty((tokens, top_k), dtype=ids_dtype, device=device)
    effective_ids = torch.empty((slots,), dtype=ids_dtype, device=device)
    order = torch.empty((slots,), dtype=torch.int64, device=device)
    inverse = torch.empty((slots,), dtype=torch.int32, device=device)
    counts = torch.empty((experts,), dtype=torch.int32, device=device)
    offsets = torch.empty((experts + 1,), dtype=torch.int32, device=device)
    statistics = torch.empty((3,), dtype=torch.int32, device=device)
    mask = None if token_mask is None else token_mask.contiguous()
    lib = _loader.library()
    with torch.cuda.device(device):
        _loader.check(lib.gg_moe_route_topk(
            _loader.pointer(logits), _loader.OUT_DTYPE[logits.dtype], _loader.pointer(mask), tokens,
            experts, top_k, _loader.pointer(weights), _loader.pointer(ids),
            int(ids_dtype == torch.int64), _loader.pointer(effective_ids), _loader.pointer(order),
            _loader.pointer(inverse), _loader.pointer(counts), _loader.pointer(offsets),
            _loader.pointer(statistics), _loader.stream_pointer(device)), "gg_moe_route_topk")
        routes = moe.Routes(order, counts, offsets, inverse, effective_ids, statistics, tokens,
                            top_k, experts)
        if tile_rows:
            routes = moe.prepare_tiles(routes, tile_rows)
    return weights, ids, routes


def prepare_weight(linear_weight, group_size=256):
    """Quantise Linear-format weights ``[E, N, K]`` (or ``[N, K]``) once, outside forward.

    Returns ``(q, scales)``: ``q`` is the INT8 *logical* GEMM weight ``[E, K, N]`` as a
    transposed view of contiguous Linear storage (stride ``(N*K, 1, K)``, what ``moe_ffn`` and
    ``int8_gemm`` take as B), ``scales`` is contiguous FP32 ``[E, K // group_size, N]``.
    """
    if linear_weight.dim() not in (2, 3):
        raise ValueError("linear_weight must be [N, K] or [E, N, K]")
    if linear_weight.device.type == "cuda" and linear_weight.shape[-1] % 256 == 0:
        source = linear_weight if linear_weight.dtype in _loader.OUT_DTYPE else linear_weight.float()
        q, scales = quantize_rows(source.contiguous(), group_size)
    else:
        k = linear_weight.shape[-1]
        if k % group_size:
            raise ValueError("K must be a multiple of group_size")
        blocks = linear_weight.float().reshape(*linear_weight.shape[:-1], k // group_size, group_size)
        scales = blocks.abs().amax(-1).clamp_min(1e-12) / 127
        q = (blocks / scales[..., None]).round().clamp(-127, 127).to(torch.int8)
        q = q.reshape(linear_weight.shape).contiguous()
    return q.transpose(-2, -1), scales.transpose(-2, -1).contiguous()


def interleave_gate_up(w_gate_up, scale_gate_up):
    """Reorder a split ``[gate | up]`` checkpoint to ``[g0, u0, g1, u1, ...]`` once.

    ``w_gate_up`` is ``[E, H, 2I]`` as a transposed view of Linear storage, ``scale_gate_up``
    contiguous ``[E, H // 256, 2I]``; the results have the same layouts and are what
    ``moe_ffn(..., gate_up_layout="interleaved")`` expects.
    """
    inter = w_gate_up.shape[-1] // 2
    channels = torch.arange(inter, device=w_gate_up.device)
    order = torch.stack((channels, channels + inter), dim=-1).reshape(-1)
    linear_weight = w_gate_up.transpose(-2, -1)
    return (linear_weight.index_select(-2, order).contiguous().transpose(-2, -1),
            scale_gate_up.index_select(-1, order).contiguous())
