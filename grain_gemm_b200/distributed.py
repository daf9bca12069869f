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
"""

from __future__ import annotations

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
                            stages=None):
    """Expert-parallel FFN for this rank's tokens.

    ``hidden_states [T_local, H]``, ``scale_x``, ``topk_weights``, ``topk_ids`` (global expert
    ids in ``[0, num_experts)``) and ``token_mask`` describe the local tokens;
    ``w_gate_up [E_local, H, 2I]``, ``w_down [E_local, I, H]`` and their scales are this
    rank's experts ``[rank * E_local, (rank + 1) * E_local)``, in the layouts ``moe_ffn`` takes.
    Returns ``[T_local, H]`` in ``output_dtype``.  Raises ``ValueError`` when an unmasked id is
    outside ``[0, num_experts)`` on any rank, and ``RuntimeError`` when the row counts that
    arrive do not match the counts that were announced.
    """
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
