"""Inference-only INT8 G256 MoE FFN: the ``grain_gemm.moe_ffn`` API on B200.

Signature, validation and stage semantics follow the reference's ``src/grain_gemm/moe.py``
(``_validate`` :19-93, ``moe_ffn`` :181-347) and ``src/grain_gemm/kernels/moe.py``
(``Routes`` :20-45, ``prepare_routes`` :222-291, ``swiglu_quantize`` :604-631, ``combine``
:656-676).  The stages run as four hand-written sm_100a kernels behind the C ABI:

1. route / stable sort                      (``gg_moe_route`` + ``gg_moe_tiles``)
2. gathered Gate/Up + rounding + SwiGLU + G256 requantisation   (``gg_moe_gate_up``)
3. grouped Down projection over the sorted slots                (``gg_moe_down``)
4. top-k weighted combine                                       (``gg_moe_combine``)

Intermediates use the ragged sorted-slot layout (``[S, I]`` INT8 + ``[S, I/256]`` scales,
``[S, H]`` expert outputs), never a capacity-padded ``[E, C, *]`` one.  Stage 2 has two ways
to fetch token rows: by default a copy kernel first writes them in sorted-slot order (one
tiled TMA box per operand slab, the faster way on B200); ``variant='tensor_core_gather'``
reads ``hidden_states`` directly with TMA row gathers, without any copy in expert order.
"""

from __future__ import annotations

import threading
from dataclasses import dataclass

import torch

from . import _loader
from .gemm import _check_backend

TENSOR_CORE_TILE_ROWS = 128
CUDA_CORE_TILE_ROWS = 32


# Validation contract (_stride, _validate) restated from the reference's
# src/grain_gemm/moe.py:7-93 (Apache-2.0): same checks, order, exception types and messages.
def _stride(shape, column_major=False):
    if column_major:
        e, k, n = shape
        return (k * n, 1, k)
    result = []
    product = 1
    for dimension in reversed(shape):
        result.append(product)
        product *= dimension
    return tuple(reversed(result))


def _validate(hidden_states, w_gate_up, w_down, topk_weights, topk_ids,
              scale_x, scale_gate_up, scale_down, token_mask, group_size, activation,
              backend, output_dtype, gate_up_layout="split"):
    if type(group_size) is not int or group_size != 256:
        raise ValueError("moe_ffn currently requires group_size=256")
    if activation != "swiglu":
        raise ValueError("moe_ffn currently requires activation='swiglu'")
    if gate_up_layout not in ("split", "interleaved"):
        raise ValueError("gate_up_layout must be 'split' or 'interleaved'")
    _check_backend(backend)
    if not isinstance(hidden_states, torch.Tensor) or hidden_states.ndim != 2:
        raise ValueError("hidden_states must be a two-dimensional tensor [T, H]")
    if not isinstance(w_gate_up, torch.Tensor) or w_gate_up.ndim != 3:
        raise ValueError("w_gate_up must be a three-dimensional tensor [E, H, 2I]")
    if not isinstance(w_down, torch.Tensor) or w_down.ndim != 3:
        raise ValueError("w_down must be a three-dimensional tensor [E, I, H]")
    if not isinstance(topk_ids, torch.Tensor) or topk_ids.ndim != 2:
        raise ValueError("topk_ids must be a two-dimensional tensor [T, R]")
    tokens, hidden = hidden_states.shape
    experts, weight_hidden, twice_intermediate = w_gate_up.shape
    intermediate = twice_intermediate // 2
    routes = topk_ids.shape[1]
    if (experts <= 0 or hidden <= 0 or twice_intermediate <= 0
            or twice_intermediate % 2 or weight_hidden != hidden):
        raise ValueError("w_gate_up must have shape [E, H, 2I] with positive E, H, I")
    if hidden % group_size or intermediate % group_size:
        raise ValueError("H and I must be positive multiples of group_size=256")
    if not 1 <= routes <= experts:
        raise ValueError("top-k R must satisfy 1 <= R <= E")
    if output_dtype not in (torch.bfloat16, torch.float16):
        raise ValueError("output_dtype must be torch.bfloat16 or torch.float16")
    specs = [
        ("hidden_states", hidden_states, (tokens, hidden), (torch.int8,), False),
        ("scale_x", scale_x, (tokens, hidden // group_size), (torch.float32,), False),
        ("w_gate_up", w_gate_up, (experts, hidden, 2 * intermediate), (torch.int8,), True),
        ("w_down", w_down, (experts, intermediate, hidden), (torch.int8,), True),
        ("topk_weights", topk_weights, (tokens, routes), (torch.float32,), False),
        ("topk_ids", topk_ids, (tokens, routes), (torch.int32, torch.int64), False),
        ("scale_gate_up", scale_gate_up, (experts, hidden // group_size, 2 * intermediate),
         (torch.float32,), False),
        ("scale_down", scale_down, (experts, intermediate // group_size, hidden),
         (torch.float32,), False),
    ]
    if token_mask is not None:
        specs.append(("token_mask", token_mask, (tokens,), (torch.bool,), False))
    for name, tensor, shape, dtypes, column_major in specs:
        if not isinstance(tensor, torch.Tensor):
            raise TypeError(f"{name} must be a torch.Tensor")
        if tensor.layout != torch.strided or tuple(tensor.shape) != shape:
            raise ValueError(f"{name} must have shape {shape} and strided layout")
        if tensor.dtype not in dtypes:
            raise TypeError(f"{name} must have dtype {dtypes}")
        wanted_stride = _stride(shape, column_major)
        # A dimension of size one is never stepped through, whatever stride torch kept for it.
        if (any(size > 1 and actual != wanted for size, actual, wanted in
                zip(shape, tensor.stride(), wanted_stride))
                or (tensor.numel() and any(s <= 0 for s in tensor.stride()))):
            raise ValueError(f"{name} must have stride {wanted_stride}, got {tensor.stride()}")
        if tensor.device != hidden_states.device or tensor.device.type != "cuda":
            raise ValueError(f"{name} must be on the same CUDA device as hidden_states")
        # The kernels address weights and their scales with 64-bit offsets (E * 2I and E * H
        # rows must fit 32 bits), so the reference's 2^31-element limit applies only to the
        # per-token tensors; the 256-expert, H=7168 configuration fits one GPU.
        weight_like = name in ("w_gate_up", "w_down", "scale_gate_up", "scale_down")
        if tensor.numel() > 2**31 - 1 and not (
                weight_like and tensor.shape[0] * max(tensor.shape[1], tensor.shape[2]) < 2**31):
            raise ValueError(f"{name} exceeds the supported 32-bit indexing range")
        if torch.is_grad_enabled() and tensor.requires_grad:
            raise ValueError("moe_ffn is inference-only; use torch.no_grad() for tensors requiring gradients")
    if tokens * routes > 2**31 - 1:
        raise ValueError("the expanded token count exceeds the supported indexing range")
    if tokens * routes * max(hidden, 2 * intermediate) > 2**31 - 1:
        raise ValueError("the expanded MoE workspace exceeds the supported indexing range")
    if torch.cuda.get_device_capability(hidden_states.device) != (10, 0):
        raise RuntimeError("this build of moe_ffn requires an NVIDIA B200 (sm_100) GPU")
    return tokens, hidden, intermediate, experts, routes


class MoEWorkspace:
    """Reusable device buffers for the intermediates of ``moe_ffn``.

    Without one every call allocates about ten tensors (routing metadata, the tile list,
    ``qh``/``sh``, the Gate/Up scratch, the expert outputs); a serving loop passes the same
    workspace to every call instead and the buffers are only (re)allocated when a shape, dtype
    or device changes.  A buffer is reused by the next call on the same stream, so the tensors
    a call got from the workspace are only valid until the next call that uses it; the result
    of ``moe_ffn`` is never taken from the workspace.  Not thread-safe: one workspace per stream.
    """

    def __init__(self):
        self._buffers = {}

    def get(self, name, shape, dtype, device):
        shape = tuple(int(d) for d in shape)
        tensor = self._buffers.get(name)
        if (tensor is None or tuple(tensor.shape) != shape or tensor.dtype != dtype
                or tensor.device != torch.device(device)):
            tensor = torch.empty(shape, dtype=dtype, device=device)
            self._buffers[name] = tensor
        return tensor

    def nbytes(self):
        return sum(t.numel() * t.element_size() for t in self._buffers.values())


def _buffer(workspace, name, shape, dtype, device):
    if workspace is None:
        return torch.empty(shape, dtype=dtype, device=device)
    return workspace.get(name, shape, dtype, device)


@dataclass(frozen=True)
class Routes:
    """GPU-resident routing metadata; valid assignments occupy a sorted prefix.

    ``order[slot]`` is the flattened ``[token, top-k]`` assignment at a sorted slot (the
    invalid tail keeps its original order too); ``inverse[assignment]`` is its slot or -1;
    ``offsets[E]`` is the number of valid assignments; ``statistics`` holds the count of
    unmasked out-of-range ids, the largest expert count and the valid total.
    ``tile_expert`` / ``tile_row`` list the row tiles of ``tile_rows`` rows the grouped
    kernels walk (expert -1 marks an unused entry).
    """

    order: torch.Tensor
    counts: torch.Tensor
    offsets: torch.Tensor
    inverse: torch.Tensor
    effective_ids: torch.Tensor
    statistics: torch.Tensor
    tokens: int
    top_k: int
    experts: int
    tile_rows: int = 0
    tile_expert: torch.Tensor | None = None
    tile_row: torch.Tensor | None = None


def prepare_routes(topk_ids, num_experts, token_mask=None, tile_rows=TENSOR_CORE_TILE_ROWS,
                   workspace=None):
    """Stable sort of the assignments by expert plus per-expert metadata, all on the GPU.

    Out-of-range ids and masked tokens get key E and sort to the tail.  ``tile_rows=0``
    skips the row-tile list.  ``token_mask`` may be BOOL or UINT8.
    """
    lib = _loader.library()
    tokens, top_k = topk_ids.shape
    slots = tokens * top_k
    device = topk_ids.device
    ids = topk_ids if topk_ids.is_contiguous() else topk_ids.contiguous()
    mask = None
    if token_mask is not None:
        mask = token_mask if token_mask.is_contiguous() else token_mask.contiguous()
    effective_ids = _buffer(workspace, "effective_ids", (slots,), ids.dtype, device)
    order = _buffer(workspace, "order", (slots,), torch.int64, device)
    inverse = _buffer(workspace, "inverse", (slots,), torch.int32, device)
    counts = _buffer(workspace, "counts", (num_experts,), torch.int32, device)
    offsets = _buffer(workspace, "offsets", (num_experts + 1,), torch.int32, device)
    statistics = _buffer(workspace, "statistics", (3,), torch.int32, device)
    workspace_bytes = lib.gg_moe_route_workspace_bytes(tokens, top_k, num_experts)
    scratch = (_buffer(workspace, "route_scratch", (workspace_bytes,), torch.uint8, device)
               if workspace_bytes else None)
    stream = _loader.stream_pointer(device)
    _loader.check(lib.gg_moe_route(
        _loader.pointer(ids), int(ids.dtype == torch.int64), _loader.pointer(mask),
        tokens, top_k, num_experts, _loader.pointer(effective_ids), _loader.pointer(order),
        _loader.pointer(inverse), _loader.pointer(counts), _loader.pointer(offsets),
        _loader.pointer(statistics), _loader.pointer(scratch), workspace_bytes, stream),
        "gg_moe_route")
    routes = Routes(order, counts, offsets, inverse, effective_ids, statistics,
                    tokens, top_k, num_experts)
    return prepare_tiles(routes, tile_rows, workspace) if tile_rows else routes


def prepare_tiles(routes, tile_rows, workspace=None):
    """Return ``routes`` with the row-tile list for tiles of ``tile_rows`` rows added."""
    if routes.tile_rows == tile_rows and routes.tile_expert is not None:
        return routes
    lib = _loader.library()
    device = routes.offsets.device
    capacity = lib.gg_moe_tile_capacity(routes.tokens * routes.top_k, routes.experts, tile_rows)
    tiles = _buffer(workspace, "tiles", (2, max(capacity, 1)), torch.int32, device)
    _loader.check(lib.gg_moe_tiles(
        _loader.pointer(routes.offsets), routes.experts, tile_rows, capacity,
        _loader.pointer(tiles[0]), _loader.pointer(tiles[1]), _loader.stream_pointer(device)),
        "gg_moe_tiles")
    return Routes(routes.order, routes.counts, routes.offsets, routes.inverse,
                  routes.effective_ids, routes.statistics, routes.tokens, routes.top_k,
                  routes.experts, tile_rows, tiles[0], tiles[1])


def gate_up_swiglu_quantize(hidden_states, scale_x, w1_linear, scale_gate_up, routes, *,
                            output_dtype=torch.bfloat16, gate_up_layout="split", row_gather=False,
                            workspace=None):
    """Stage 2: ``qh[S, I]`` INT8 and ``sh[S, I/256]`` FP32 for the valid sorted slots.

    ``w1_linear`` is the contiguous Linear view ``[E, 2I, H]``.  Rows of invalid slots are
    left unwritten; nothing downstream reads them.  ``row_gather`` makes the fused kernel read
    the token rows straight from ``hidden_states`` by TMA row gathers instead of from a copy in
    sorted order (same bits; the copy is faster on B200 and is the default).
    """
    lib = _loader.library()
    experts, twice_intermediate, hidden = w1_linear.shape
    intermediate = twice_intermediate // 2
    slots = routes.tokens * routes.top_k
    device = hidden_states.device
    qh = _buffer(workspace, "qh", (slots, intermediate), torch.int8, device)
    sh = _buffer(workspace, "sh", (slots, intermediate // 256), torch.float32, device)
    with torch.cuda.device(device):
        scratch_bytes = lib.gg_moe_gate_up_scratch_bytes(slots, hidden, intermediate,
                                                         routes.tile_rows, int(row_gather))
    scratch = _buffer(workspace, "gate_up_scratch", (max(scratch_bytes, 16),), torch.uint8, device)
    _loader.check(lib.gg_moe_gate_up(
        _loader.pointer(hidden_states), _loader.pointer(scale_x), _loader.pointer(w1_linear),
        _loader.pointer(scale_gate_up), _loader.pointer(routes.order),
        _loader.pointer(routes.offsets), _loader.pointer(routes.tile_expert),
        _loader.pointer(routes.tile_row), routes.tile_expert.numel(), routes.tile_rows,
        _loader.pointer(qh), _loader.pointer(sh), _loader.pointer(scratch),
        routes.tokens, routes.top_k, experts, hidden, intermediate,
        int(gate_up_layout == "interleaved"), _loader.OUT_DTYPE[output_dtype], int(row_gather),
        _loader.stream_pointer(device)), "gg_moe_gate_up")
    return qh, sh


def down_projection(qh, sh, w2_linear, scale_down, routes, *, output_dtype=torch.bfloat16,
                    row_destination=None, workspace=None):
    """Stage 3: ``expert_output[S, H]`` for the valid sorted slots (``w2_linear`` ``[E, H, I]``).

    With ``row_destination`` (INT64 ``[S]`` device addresses, tensor-core path) every row is
    stored at its own address instead and nothing is returned.
    """
    lib = _loader.library()
    experts, hidden, intermediate = w2_linear.shape
    slots = routes.tokens * routes.top_k
    out = (_buffer(workspace, "expert_output", (slots, hidden), output_dtype, qh.device)
           if row_destination is None else None)
    _loader.check(lib.gg_moe_down(
        _loader.pointer(qh), _loader.pointer(sh), _loader.pointer(w2_linear),
        _loader.pointer(scale_down), _loader.pointer(routes.offsets),
        _loader.pointer(routes.tile_expert), _loader.pointer(routes.tile_row),
        routes.tile_expert.numel(), routes.tile_rows, _loader.pointer(out),
        _loader.pointer(row_destination), slots, experts,
        hidden, intermediate, _loader.OUT_DTYPE[output_dtype],
        _loader.stream_pointer(qh.device)), "gg_moe_down")
    return out


def combine(expert_output, topk_weights, routes, *, output_dtype=torch.bfloat16):
    """Stage 4: apply the supplied routing weights and reduce in FP32 to ``[T, H]``."""
    lib = _loader.library()
    hidden = expert_output.shape[-1]
    out = torch.empty((routes.tokens, hidden), dtype=output_dtype, device=expert_output.device)
    weights = topk_weights if topk_weights.is_contiguous() else topk_weights.contiguous()
    _loader.check(lib.gg_moe_combine(
        _loader.pointer(expert_output), _loader.pointer(weights), _loader.pointer(routes.inverse),
        _loader.pointer(out), routes.tokens, routes.top_k, hidden,
        _loader.OUT_DTYPE[output_dtype], _loader.stream_pointer(expert_output.device)),
        "gg_moe_combine")
    return out


_HOST = threading.local()


def _statistics_readback(statistics, count=3, slot="statistics"):
    """Start handing ``count`` integers of ``statistics`` to pinned host memory.

    Returns ``(host_tensor, event)``; the event completes as soon as the kernels before it have
    run, so a caller that first launches the remaining stages and only then waits on it never
    leaves the GPU idle.  The integers are stored by a kernel (``gg_report_to_host``), not by
    a copy: a device-to-host copy would queue behind whatever large transfer the application
    has on the copy engine (the previous call's result on its way to the host, say), and the
    stream, and with it the remaining stages, would wait for it.  One pinned buffer per thread,
    device and ``slot`` is reused: a call's readback is consumed before the same thread can
    start another call.
    """
    from . import _loader
    buffers = getattr(_HOST, "buffers", None)
    if buffers is None:
        buffers = _HOST.buffers = {}
    key = (statistics.device.index, slot, count)
    if key not in buffers:
        buffers[key] = torch.empty((count,), dtype=torch.int32, pin_memory=True)
    host = buffers[key]
    status = _loader.library().gg_report_to_host(
        _loader.pointer(statistics), count, host.data_ptr(), _loader.stream_pointer(statistics.device))
    if status != 0:
        # Host memory the device cannot address: fall back to the copy engine.
        host.copy_(statistics.reshape(-1)[:count], non_blocking=True)
    event = torch.cuda.Event()
    event.record()
    return host, event


def _tensor_core_ready(*tensors):
    return all(t.data_ptr() % 16 == 0 for t in tensors)


def moe_ffn(hidden_states, w_gate_up, w_down, topk_weights, topk_ids, *,
            scale_x, scale_gate_up, scale_down, group_size=256, activation="swiglu",
            token_mask=None, output_dtype=torch.bfloat16, backend="auto",
            gate_up_layout="split", variant="auto", workspace=None, routes=None):
    """Run a complete pre-routed INT8 G256 MoE FFN on the current CUDA stream.

    ``w_gate_up[E,H,2I]`` and ``w_down[E,I,H]`` are transposed views of contiguous
    Linear-format INT8 weights (strides ``(H*2I,1,H)`` / ``(I*H,1,I)``); FP32 scales are
    contiguous ``[E,H/256,2I]`` and ``[E,I/256,H]``.  ``gate_up_layout`` is ``'split'``
    (``[g0..gI-1,u0..uI-1]``) or ``'interleaved'`` (``[g0,u0,g1,u1,...]``) for both the
    weight's and the scale's last dimension.  Inputs ``[T,H]`` are INT8 with contiguous
    FP32 ``scale_x[T,H/256]``; route scores ``[T,R]`` are FP32 and used as supplied;
    expert ids are INT32/INT64.  Masked tokens return zero.  Every GEMM accumulates group
    dots in INT32 and scaled sums in FP32 and rounds once to ``output_dtype``; SwiGLU
    activations are requantised per row and 256-channel group with
    ``amax.clamp_min(1e-12)/127``, nearest-even rounding and clipping to [-127,127].

    Eager calls read three integers back to reject unmasked ids outside ``[0,E)`` with a
    ``ValueError`` (the copy overlaps the remaining stages; the call returns or raises once
    routing has run); under CUDA-graph capture that check is skipped.  ``variant`` is
    ``'auto'``, ``'tensor_core'``, ``'tensor_core_gather'`` (the fused Gate/Up kernel fetches
    token rows by TMA row gathers, no copy in expert order) or ``'cuda_core'``.  ``workspace``
    (a ``MoEWorkspace``) makes repeated calls reuse their intermediate buffers.  ``routes``
    (from ``prepare_routes`` or ``route_topk_routes`` on the same ids and mask) skips stage 1.
    """
    tokens, hidden, intermediate, experts, top_k = _validate(
        hidden_states, w_gate_up, w_down, topk_weights, topk_ids,
        scale_x, scale_gate_up, scale_down, token_mask, group_size, activation, backend,
        output_dtype, gate_up_layout)
    if variant not in ("auto", "tensor_core", "tensor_core_gather", "cuda_core"):
        raise ValueError("variant must be 'auto', 'tensor_core', 'tensor_core_gather' or 'cuda_core'")
    with torch.cuda.device(hidden_states.device):
        capturing = torch.cuda.is_current_stream_capturing()
        if tokens == 0:
            return torch.zeros(hidden_states.shape, device=hidden_states.device, dtype=output_dtype)
        w1_linear = w_gate_up.transpose(-2, -1)
        w2_linear = w_down.transpose(-2, -1)
        aligned = _tensor_core_ready(hidden_states, w_gate_up, w_down)
        if variant.startswith("tensor_core") and not aligned:
            raise ValueError(f"variant='{variant}' requires 16-byte-aligned hidden_states and weights")
        tile_rows = (CUDA_CORE_TILE_ROWS if variant == "cuda_core" or not aligned
                     else TENSOR_CORE_TILE_ROWS)
        if routes is None:
            routes = prepare_routes(topk_ids, experts, token_mask, tile_rows=tile_rows,
                                    workspace=workspace)
        else:
            if (routes.tokens, routes.top_k, routes.experts) != (tokens, top_k, experts):
                raise ValueError("routes were prepared for other topk_ids or another expert count")
            routes = prepare_tiles(routes, tile_rows, workspace)
        # The check for unmasked ids outside [0, E) reads three integers back.  Its copy is
        # started now and awaited after the remaining stages are in the stream (they are safe
        # for any ids: invalid assignments sort to the ignored tail), so the GPU never waits
        # for the host between routing and Gate/Up.
        readback = None if capturing else _statistics_readback(routes.statistics)
        qh, sh = gate_up_swiglu_quantize(
            hidden_states, scale_x, w1_linear, scale_gate_up, routes,
            output_dtype=output_dtype, gate_up_layout=gate_up_layout,
            row_gather=variant == "tensor_core_gather", workspace=workspace)
        expert_output = down_projection(qh, sh, w2_linear, scale_down, routes,
                                        output_dtype=output_dtype, workspace=workspace)
        out = combine(expert_output, topk_weights, routes, output_dtype=output_dtype)
        if readback is not None:
            host, event = readback
            event.synchronize()
            if int(host[0]):
                raise ValueError("unmasked topk_ids must be in [0, E)")
        return out
