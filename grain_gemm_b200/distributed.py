"""Expert-parallel ``moe_ffn`` and the N-sharded GEMM over one node of B200s.

The reference has no distributed code; this module adds the partitioning its operators
allow without changing their arithmetic:

* ``moe_ffn_expert_parallel``: experts are split contiguously over the ranks (expert ``e``
  lives on rank ``e // (E / W)``), tokens are sharded per rank.  One exchange step each way.
  Out: every rank sends each token row, its scales and its per-slot local expert indices once
  to every rank that holds at least one of the token's experts (the (token, rank) pairs are
  sorted by rank with the routing kernel) with NCCL ``all_to_all_single``; the receiving rank
  runs stages 1-3 of the FFN on those tokens with its own experts.  Back: the expert outputs
  travel per assignment, grouped by home rank in (token, slot) order, and the home rank
  combines them in slot order.  Each assignment is computed from the same inputs by the same
  kernels as on one GPU, and the combine adds the slots in the same order, so the result
  equals the single-GPU result bit for bit.  Remote rows always land in local memory first;
  kernels only ever read local memory.
* ``int8_gemm_n_sharded``: a rank owns a block of B's columns (and of ``scale_b`` and C);
  A and ``scale_a`` are replicated.  Column blocks are independent, so there is no
  data-path collective; ``gather=True`` all-gathers C when the caller wants it whole.
  K is never sharded: that would need an FP32 reduction and break the group-order ``fmaf``.

``stages`` makes the local computation pluggable so that the exchange logic can be tested on
CPU ranks (gloo) with a CPU implementation of the stages; the default is the CUDA path.

``moe_ffn_expert_parallel`` has two exchange mechanisms:

* NCCL ``all_to_all_single`` both ways (the default without an ``exchange`` argument);
* ``PeerExchange``: every rank owns a receive area in device memory that all ranks of the node
  map (CUDA IPC over NVLink).  The dispatch kernel stores token rows straight into the
  destination ranks' areas, one small count all-gather orders "everything has arrived", the
  local experts run on the received rows, and the Down projection stores every result row from
  inside the GEMM straight into the home rank's area (``row_destination``), so the return trip
  overlaps the tensor-core work tile by tile; one tiny all-reduce orders "all results are
  home" before the combine.  No host synchronisation, no per-call allocation, the same bits.
"""

from __future__ import annotations

import ctypes
from types import SimpleNamespace

import torch
import torch.distributed as dist


class CudaStages:
    """Local stages backed by the C-ABI kernels."""

    def route(self, keys, num_keys, token_mask=None):
        from . import moe
        return moe.prepare_routes(keys, num_keys, token_mask, tile_rows=0)

    def expert_ffn(self, x, scale_x, expert_ids, valid, w_gate_up, w_down, scale_gate_up,
                   scale_down, output_dtype, gate_up_layout):
        """FFN of the received tokens through this rank's experts.

        ``x [m, H]`` / ``scale_x`` are the received token rows, ``expert_ids [m, R]`` their
        local expert indices with ``E_local`` marking the slots that belong to other ranks.
        Returns the expert outputs of the ``valid`` real assignments as ``[valid, H]`` in
        flattened ``(token, slot)`` order, which is the order the home ranks expect.
        """
        from . import moe
        tokens, top_k = expert_ids.shape
        experts = w_gate_up.shape[0]
        if tokens == 0 or valid == 0:
            return torch.empty((0, x.shape[1]), dtype=output_dtype, device=x.device)
        aligned = all(t.data_ptr() % 16 == 0 for t in (x, w_gate_up, w_down))
        routes = moe.prepare_routes(expert_ids, experts, None,
                                    tile_rows=moe.TENSOR_CORE_TILE_ROWS if aligned
                                    else moe.CUDA_CORE_TILE_ROWS)
        qh, sh = moe.gate_up_swiglu_quantize(
            x, scale_x, w_gate_up.transpose(-2, -1), scale_gate_up, routes,
            output_dtype=output_dtype, gate_up_layout=gate_up_layout)
        sorted_out = moe.down_projection(qh, sh, w_down.transpose(-2, -1), scale_down, routes,
                                         output_dtype=output_dtype)
        # Real assignments in flattened order: a stable sort with one key puts them first.
        foreign = (expert_ids >= experts).reshape(-1, 1).to(torch.int32)
        flattened = moe.prepare_routes(foreign, 1, None, tile_rows=0).order[:valid]
        return sorted_out.index_select(0, routes.inverse.index_select(0, flattened).long())

    def combine(self, rows, topk_weights, routes, output_dtype):
        from . import moe
        return moe.combine(rows, topk_weights, routes, output_dtype=output_dtype)


def _all_to_all_rows(send, send_counts, recv_counts, group):
    """Variable-sized row exchange; ``send`` rows are grouped by destination rank."""
    received = torch.empty((int(sum(recv_counts)),) + tuple(send.shape[1:]), dtype=send.dtype,
                           device=send.device)
    dist.all_to_all_single(received, send, output_split_sizes=list(recv_counts),
                           input_split_sizes=list(send_counts), group=group)
    return received


def moe_ffn_expert_parallel(hidden_states, w_gate_up, w_down, topk_weights, topk_ids, *,
                            scale_x, scale_gate_up, scale_down, num_experts, token_mask=None,
                            output_dtype=torch.bfloat16, gate_up_layout="split", group=None,
                            stages=None, exchange=None, marks=None):
    """Expert-parallel FFN for this rank's tokens.

    ``hidden_states [T_local, H]``, ``scale_x``, ``topk_weights``, ``topk_ids`` (global expert
    ids in ``[0, num_experts)``) and ``token_mask`` describe the local tokens;
    ``w_gate_up [E_local, H, 2I]``, ``w_down [E_local, I, H]`` and their scales are this
    rank's experts ``[rank * E_local, (rank + 1) * E_local)``, in the layouts ``moe_ffn`` takes.
    Returns ``[T_local, H]`` in ``output_dtype``.  Raises ``ValueError`` when an unmasked id is
    outside ``[0, num_experts)`` on any rank, and ``RuntimeError`` when the row counts that
    arrive do not match the counts that were announced.  ``exchange`` (a ``PeerExchange``)
    replaces the NCCL all-to-alls by stores into peer memory fused into the dispatch and Down
    kernels; the result is bit-identical.
    """
    if exchange is not None:
        if exchange.local_experts * exchange.world != num_experts or \
                exchange.output_dtype != output_dtype:
            raise ValueError("the exchange was created for another expert count or output type")
        return _peer_step(exchange, hidden_states, w_gate_up, w_down, topk_weights, topk_ids,
                          scale_x, scale_gate_up, scale_down, token_mask, gate_up_layout, marks)
    stages = stages or CudaStages()
    world = dist.get_world_size(group)
    local_experts = w_gate_up.shape[0]
    if local_experts * world != num_experts:
        raise ValueError(f"num_experts={num_experts} must equal E_local={local_experts} x world={world}")
    tokens, hidden = hidden_states.shape
    top_k = topk_ids.shape[1]
    device = hidden_states.device

    # 1. Sort the local assignments by destination rank (for the way back), and the
    #    (token, rank) pairs a token has at least one expert on (for the way out): a token row
    #    crosses the link once per destination rank, not once per assignment.  Out-of-range ids
    #    keep a key outside [0, W) so that the routing statistics count them as on one GPU.
    in_range = (topk_ids >= 0) & (topk_ids < num_experts)
    destination = torch.where(in_range, topk_ids // local_experts,
                              torch.full_like(topk_ids, world))
    routes = stages.route(destination.contiguous(), world, token_mask)
    reachable = destination if token_mask is None else torch.where(
        token_mask.reshape(-1, 1).to(torch.bool), destination, torch.full_like(destination, world))
    member = torch.zeros((tokens, world + 1), dtype=torch.bool, device=device)
    member.scatter_(1, reachable.long(), True)
    ranks = torch.arange(world, dtype=topk_ids.dtype, device=device).expand(tokens, world)
    pair_keys = torch.where(member[:, :world], ranks, torch.full_like(ranks, world))
    pairs = stages.route(pair_keys.contiguous(), world, None)

    # 2. Announce per-destination token and assignment counts (and any invalid id).
    counts = torch.cat([pairs.counts.to(torch.int64), routes.counts.to(torch.int64),
                        routes.statistics[:1].to(torch.int64)])
    announced = torch.empty((world, 2 * world + 1), dtype=torch.int64, device=device)
    dist.all_gather_into_tensor(announced, counts.reshape(1, -1), group=group)
    announced = announced.cpu()
    if int(announced[:, 2 * world].sum()):
        raise ValueError("unmasked topk_ids must be in [0, E)")
    rank = dist.get_rank(group)
    send_tokens = announced[rank, :world].tolist()
    recv_tokens = announced[:, rank].tolist()
    send_assignments = announced[rank, world:2 * world].tolist()
    recv_assignments = announced[:, world + rank].tolist()
    sent_tokens = int(sum(send_tokens))
    valid = int(sum(send_assignments))

    # 3. Dispatch: token rows, their scales and, per token, the local expert index of each of
    #    its slots on the destination rank (E_local marks slots that live elsewhere).
    pair = pairs.order[:sent_tokens]
    source_token = pair // world
    pair_rank = (pair % world).reshape(-1, 1)
    send_x = hidden_states.index_select(0, source_token)
    send_scale = scale_x.index_select(0, source_token)
    token_ids = topk_ids.index_select(0, source_token)
    on_rank = reachable.index_select(0, source_token) == pair_rank
    send_expert = torch.where(on_rank, token_ids - pair_rank * local_experts,
                              torch.full_like(token_ids, local_experts)).to(torch.int32)
    recv_x = _all_to_all_rows(send_x, send_tokens, recv_tokens, group)
    recv_scale = _all_to_all_rows(send_scale, send_tokens, recv_tokens, group)
    recv_expert = _all_to_all_rows(send_expert, send_tokens, recv_tokens, group)
    if recv_x.shape[0] != sum(recv_tokens) or recv_expert.shape[0] != recv_x.shape[0]:
        raise RuntimeError("expert-parallel dispatch delivered a different number of rows than announced")

    # 4. Local experts on the received tokens (stages 1-3 of the FFN); outputs of the real
    #    assignments in (source rank, token, slot) order.
    computed = stages.expert_ffn(recv_x, recv_scale, recv_expert, int(sum(recv_assignments)),
                                 w_gate_up, w_down, scale_gate_up, scale_down, output_dtype,
                                 gate_up_layout)

    # 5. Return the expert outputs to the ranks that own the tokens, then combine at home.
    returned = _all_to_all_rows(computed, recv_assignments, send_assignments, group)
    if returned.shape[0] != valid:
        raise RuntimeError("expert-parallel combine delivered a different number of rows than sent")
    if valid == 0:
        return torch.zeros((tokens, hidden), dtype=output_dtype, device=device)
    return stages.combine(returned, topk_weights, routes, output_dtype)


class _DeviceMemory:
    """Raw device memory as something ``torch.as_tensor`` accepts (CUDA array interface)."""

    def __init__(self, address, nbytes):
        self.__cuda_array_interface__ = {"shape": (int(nbytes),), "typestr": "|u1",
                                         "data": (int(address), False), "version": 2}


def _align(value, to=256):
    return (value + to - 1) // to * to


class PeerExchange:
    """One rank's side of the expert-parallel exchange over peer memory.

    Holds this rank's receive area (token rows, scales, local expert indices and home token
    index of up to ``capacity`` tokens from each of ``world`` ranks, plus the ``home_out``
    block the other ranks write this rank's results into), the device addresses of every
    rank's area, and the per-call scratch, all allocated once.  ``capacity`` is the largest
    number of tokens a rank will pass per call.

    ``PeerExchange.create(group, ...)`` builds the exchange of a process group: the areas are
    shared between the processes with CUDA IPC handles (one node).  ``PeerExchange.local_ranks``
    builds ``world`` exchanges inside one process on one GPU, which run the same kernels against
    the same addresses without any collective; tests use it to cover the whole path on a single
    GPU.
    """

    def __init__(self, *, rank, world, capacity, hidden, top_k, local_experts, output_dtype,
                 device, group=None):
        from . import _loader, moe
        self.rank, self.world, self.capacity = rank, world, capacity
        self.hidden, self.top_k, self.local_experts = hidden, top_k, local_experts
        self.output_dtype, self.device, self.group = output_dtype, torch.device(device), group
        rows = world * capacity
        groups = hidden // 256
        sections = [("recv_x", rows * hidden), ("recv_scale", rows * groups * 4),
                    ("recv_ids", rows * top_k * 4), ("recv_src", rows * 4),
                    ("home_out", capacity * top_k * hidden * 2)]
        self.offsets, total = {}, 0
        for name, size in sections:
            self.offsets[name] = total
            total += _align(size)
        self.area_bytes = total
        self._lib = _loader.library()
        with torch.cuda.device(self.device):
            pointer = ctypes.c_void_p()
            _loader.check(self._lib.gg_peer_alloc(total, ctypes.byref(pointer)), "gg_peer_alloc")
        self.base = pointer.value
        self._imported = []
        area = torch.as_tensor(_DeviceMemory(self.base, total), device=self.device)
        view = lambda name, size, dtype, shape: area[self.offsets[name]:self.offsets[name] + size] \
            .view(dtype).view(shape)
        self.recv_x = view("recv_x", rows * hidden, torch.int8, (rows, hidden))
        self.recv_scale = view("recv_scale", rows * groups * 4, torch.float32, (rows, groups))
        self.recv_ids = view("recv_ids", rows * top_k * 4, torch.int32, (rows, top_k))
        self.recv_src = view("recv_src", rows * 4, torch.int32, (rows,))
        self.home_out = view("home_out", capacity * top_k * hidden * 2, output_dtype,
                             (capacity * top_k, hidden))
        self.recv_src.fill_(0)
        make = lambda shape, dtype: torch.zeros(shape, dtype=dtype, device=self.device)
        self.position = make((capacity, world), torch.int32)
        self.counts = make((world + 1,), torch.int32)
        self.counts_all = make((world, world + 1), torch.int32)
        self.home_inverse = make((capacity * top_k,), torch.int32)
        self.row_mask = make((rows,), torch.uint8)
        self.row_destination = make((rows * top_k,), torch.int64)
        self.flags = make((2,), torch.int32)           # [0] = a kernel refused an index
        self.report = make((world + 2,), torch.int32)  # invalid-id counts per rank, then flags
        self.tables = None
        self.workspace = moe.MoEWorkspace()

    # -- construction ----------------------------------------------------------------------

    def _set_peer_bases(self, bases):
        table = lambda name: torch.tensor([b + self.offsets[name] for b in bases],
                                          dtype=torch.int64, device=self.device)
        self.tables = {name: table(name) for name in self.offsets}

    @classmethod
    def create(cls, group, *, capacity, hidden, top_k, local_experts,
               output_dtype=torch.bfloat16, device=None):
        """The exchange of this rank in ``group`` (all ranks on one node, NCCL backend)."""
        from . import _loader
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        self = cls(rank=rank, world=world, capacity=capacity, hidden=hidden, top_k=top_k,
                   local_experts=local_experts, output_dtype=output_dtype, device=device,
                   group=group)
        handle = ctypes.create_string_buffer(64)
        with torch.cuda.device(self.device):
            _loader.check(self._lib.gg_peer_export(ctypes.c_void_p(self.base), handle),
                          "gg_peer_export")
        handles = [None] * world
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        bases = []
        with torch.cuda.device(self.device):
            for peer, raw in enumerate(handles):
                if peer == rank:
                    bases.append(self.base)
                    continue
                pointer = ctypes.c_void_p()
                _loader.check(self._lib.gg_peer_import(ctypes.create_string_buffer(raw, 64),
                                                       ctypes.byref(pointer)), "gg_peer_import")
                self._imported.append(pointer.value)
                bases.append(pointer.value)
        self._set_peer_bases(bases)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)
        return self

    @classmethod
    def local_ranks(cls, world, *, capacity, hidden, top_k, local_experts,
                    output_dtype=torch.bfloat16, device="cuda"):
        """``world`` exchanges inside this process on one GPU, addressing each other directly."""
        ranks = [cls(rank=r, world=world, capacity=capacity, hidden=hidden, top_k=top_k,
                     local_experts=local_experts, output_dtype=output_dtype, device=device)
                 for r in range(world)]
        for exchange in ranks:
            exchange._set_peer_bases([peer.base for peer in ranks])
        return ranks

    def close(self):
        """Unmap the peers' areas and free this rank's.  Call on every rank, after a barrier."""
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            for pointer in self._imported:
                self._lib.gg_peer_release(ctypes.c_void_p(pointer))
            self._imported = []
            if self.base:
                for name in ("recv_x", "recv_scale", "recv_ids", "recv_src", "home_out"):
                    setattr(self, name, None)
                self._lib.gg_peer_free(ctypes.c_void_p(self.base))
                self.base = 0

    # -- the three phases of a step ----------------------------------------------------------

    def dispatch(self, hidden_states, scale_x, topk_ids, token_mask=None):
        """Plan and send: every token row goes once to every rank that owns one of its experts.
        Returns this rank's ``counts`` (rows per destination, then the invalid-id count)."""
        from . import _loader
        tokens = hidden_states.shape[0]
        if tokens > self.capacity or hidden_states.shape[1] != self.hidden \
                or topk_ids.shape[1] != self.top_k:
            raise ValueError("PeerExchange: token count, hidden size or top-k exceed what the "
                             "exchange was created for")
        ids = topk_ids if topk_ids.is_contiguous() else topk_ids.contiguous()
        mask = None if token_mask is None else token_mask.contiguous()
        experts = self.local_experts * self.world
        stream = _loader.stream_pointer(self.device)
        is_i64 = int(ids.dtype == torch.int64)
        _loader.check(self._lib.gg_ep_plan(
            _loader.pointer(ids), is_i64, _loader.pointer(mask), tokens, self.top_k, experts,
            self.world, self.local_experts, _loader.pointer(self.position),
            _loader.pointer(self.counts), _loader.pointer(self.home_inverse), stream), "gg_ep_plan")
        _loader.check(self._lib.gg_ep_dispatch(
            _loader.pointer(hidden_states), _loader.pointer(scale_x), _loader.pointer(ids), is_i64,
            _loader.pointer(mask), _loader.pointer(self.position), tokens, self.top_k, experts,
            self.world, self.local_experts, self.hidden, self.rank, self.capacity,
            _loader.pointer(self.tables["recv_x"]), _loader.pointer(self.tables["recv_scale"]),
            _loader.pointer(self.tables["recv_ids"]), _loader.pointer(self.tables["recv_src"]),
            _loader.pointer(self.flags), stream), "gg_ep_dispatch")
        return self.counts

    def experts(self, counts_all, w_gate_up, w_down, scale_gate_up, scale_down, gate_up_layout,
                mark=None):
        """Stages 1-3 on the rows that arrived; Down stores each result row into the home
        rank's ``home_out``.  ``counts_all`` is the all-gathered ``[world, world + 1]`` matrix.
        ``mark``, a callable, is invoked after routing and after Gate/Up (timing events)."""
        from . import _loader, moe
        stream = _loader.stream_pointer(self.device)
        _loader.check(self._lib.gg_ep_row_mask(
            _loader.pointer(counts_all), self.world, self.rank, self.capacity,
            _loader.pointer(self.row_mask), stream), "gg_ep_row_mask")
        routes = moe.prepare_routes(self.recv_ids, self.local_experts, self.row_mask,
                                    tile_rows=moe.TENSOR_CORE_TILE_ROWS, workspace=self.workspace)
        if mark is not None:
            mark()
        qh, sh = moe.gate_up_swiglu_quantize(
            self.recv_x, self.recv_scale, w_gate_up.transpose(-2, -1), scale_gate_up, routes,
            output_dtype=self.output_dtype, gate_up_layout=gate_up_layout, workspace=self.workspace)
        if mark is not None:
            mark()
        _loader.check(self._lib.gg_ep_row_destination(
            _loader.pointer(routes.order), _loader.pointer(routes.offsets), self.local_experts,
            self.top_k, self.capacity, self.world, self.hidden, _loader.OUT_DTYPE[self.output_dtype],
            _loader.pointer(self.recv_src), _loader.pointer(self.tables["home_out"]),
            _loader.pointer(self.row_destination), _loader.pointer(self.flags), stream),
            "gg_ep_row_destination")
        moe.down_projection(qh, sh, w_down.transpose(-2, -1), scale_down, routes,
                            output_dtype=self.output_dtype, row_destination=self.row_destination)

    def combine(self, topk_weights):
        """Top-k weighted sum of this rank's tokens from ``home_out`` (slot order)."""
        from . import moe
        tokens = topk_weights.shape[0]
        routes = SimpleNamespace(inverse=self.home_inverse, tokens=tokens, top_k=self.top_k)
        return moe.combine(self.home_out[:tokens * self.top_k], topk_weights, routes,
                           output_dtype=self.output_dtype)


def _peer_step(exchange, hidden_states, w_gate_up, w_down, topk_weights, topk_ids, scale_x,
               scale_gate_up, scale_down, token_mask, gate_up_layout, marks=None):
    """One expert-parallel FFN through ``exchange`` (see ``PeerExchange``).  ``marks``, a list,
    receives timing events at the phase boundaries (start, dispatched, counts gathered, routed,
    Gate/Up done, Down done, results home, combined)."""
    world, group = exchange.world, exchange.group

    def mark():
        if marks is not None:
            event = torch.cuda.Event(enable_timing=True)
            event.record()
            marks.append(event)

    mark()
    aligned = all(t.data_ptr() % 16 == 0 for t in (hidden_states, w_gate_up, w_down))
    if not aligned:
        raise ValueError("the peer exchange needs 16-byte-aligned hidden_states and weights")
    counts = exchange.dispatch(hidden_states, scale_x, topk_ids, token_mask)
    mark()
    # Counts of every rank; the collective also orders "every rank's rows have arrived".
    if world > 1:
        dist.all_gather_into_tensor(exchange.counts_all, counts.reshape(1, -1), group=group)
    else:
        exchange.counts_all.copy_(counts.reshape(1, -1))
    mark()
    exchange.experts(exchange.counts_all, w_gate_up, w_down, scale_gate_up, scale_down,
                     gate_up_layout, mark=mark if marks is not None else None)
    mark()
    # "All results are home" (and any refused index on any rank) before the combine.
    if world > 1:
        dist.all_reduce(exchange.flags, group=group)
    mark()
    # Invalid ids and refused indices are read back while the combine runs (not under capture).
    capturing = torch.cuda.is_current_stream_capturing()
    if not capturing:
        from . import moe
        exchange.report[:world].copy_(exchange.counts_all[:, world])
        exchange.report[world:].copy_(exchange.flags)
        host, event = moe._statistics_readback(exchange.report, world + 2, slot="expert_parallel")
    out = exchange.combine(topk_weights)
    mark()
    if not capturing:
        event.synchronize()
        if int(host[world]):
            exchange.flags.zero_()
            raise RuntimeError("expert-parallel exchange: a kernel refused an out-of-range row index")
        if int(host[:world].sum()):
            raise ValueError("unmasked topk_ids must be in [0, E)")
    return out


def run_local_ranks(exchanges, cases, token_masks=None):
    """Run one expert-parallel step of every rank of ``PeerExchange.local_ranks`` in this process.

    ``cases[r]`` holds rank r's ``moe_ffn_expert_parallel`` tensors.  The phases run rank by
    rank (dispatch of all ranks, then the experts of all ranks, then the combines), which is
    the order the collectives of the multi-process path enforce.  Returns the per-rank outputs.
    """
    world = len(exchanges)
    masks = token_masks or [None] * world
    counts = [ex.dispatch(case["hidden_states"], case["scale_x"], case["topk_ids"], mask)
              for ex, case, mask in zip(exchanges, cases, masks)]
    counts_all = torch.stack(counts).contiguous()
    if int(counts_all[:, world].sum()):
        raise ValueError("unmasked topk_ids must be in [0, E)")
    for ex, case in zip(exchanges, cases):
        ex.experts(counts_all, case["w_gate_up"], case["w_down"], case["scale_gate_up"],
                   case["scale_down"], case.get("gate_up_layout", "split"))
    outputs = [ex.combine(case["topk_weights"]) for ex, case in zip(exchanges, cases)]
    if any(int(ex.flags[0]) for ex in exchanges):
        raise RuntimeError("expert-parallel exchange: a kernel refused an out-of-range row index")
    return outputs


def int8_gemm_n_sharded(a, b_local, scale_a, scale_b_local, *, group_size=256,
                        output_dtype=torch.bfloat16, group=None, gather=False):
    """``int8_gemm`` with B, ``scale_b`` and C split along N over the ranks of ``group``.

    Every rank passes the full ``a``/``scale_a`` and its own column block.  Returns the local
    block of C, or the whole C (column blocks concatenated in rank order) when ``gather``.
    """
    from .gemm import int8_gemm
    local = int8_gemm(a, b_local, scale_a, scale_b_local, group_size=group_size,
                      output_dtype=output_dtype)
    if not gather:
        return local
    world = dist.get_world_size(group)
    blocks = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(blocks, local.contiguous(), group=group)
    return torch.cat(blocks, dim=1)
