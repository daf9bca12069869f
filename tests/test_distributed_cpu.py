"""Expert-parallel exchange logic on CPU ranks (gloo, world size 2).

The local stages are the CPU oracle here, so these tests cover the host-side logic of
``grain_gemm_b200.distributed``: destination sorting of assignments and of (token, rank)
pairs, count exchange, token-level dispatch, per-assignment return and the home combine.  The expert-parallel result must equal the single-process result bit for
bit, and a bad id on one rank must raise on every rank before anything is exchanged.
"""

import os
import socket
import sys
import traceback
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

from oracle import cpu as oracle  # noqa: E402


class OracleStages:
    """CPU stand-in for the CUDA stages, same interface as distributed.CudaStages."""

    def route(self, keys, num_keys, token_mask=None):
        return oracle.route(keys, num_keys, token_mask)

    def expert_ffn(self, x, scale_x, expert_ids, valid, w_gate_up, w_down, scale_gate_up,
                   scale_down, output_dtype, gate_up_layout):
        experts = w_gate_up.shape[0]
        token, slot = torch.nonzero(expert_ids < experts, as_tuple=True)   # flattened order
        assert token.numel() == valid
        if valid == 0:
            return torch.empty((0, x.shape[1]), dtype=output_dtype)
        return oracle.moe_ffn(x[token], w_gate_up, w_down, torch.ones((valid, 1)),
                              expert_ids[token, slot].reshape(valid, 1).long(),
                              scale_x=scale_x[token], scale_gate_up=scale_gate_up,
                              scale_down=scale_down, output_dtype=output_dtype,
                              gate_up_layout=gate_up_layout)

    def combine(self, rows, topk_weights, routes, output_dtype):
        return oracle.combine(rows, topk_weights, routes, output_dtype)


def full_case(tokens=24, hidden=256, inter=256, experts=6, top_k=3, seed=11):
    generator = torch.Generator().manual_seed(seed)
    x = torch.randint(-127, 128, (tokens, hidden), dtype=torch.int8, generator=generator)
    scale_x = (0.5 + torch.rand((tokens, 1), generator=generator)) / 127
    w1 = torch.randint(-127, 128, (experts, 2 * inter, hidden), dtype=torch.int8, generator=generator)
    w2 = torch.randint(-127, 128, (experts, hidden, inter), dtype=torch.int8, generator=generator)
    s1 = (0.5 + torch.rand((experts, 1, 2 * inter), generator=generator)) * (3 / hidden) ** 0.5 / 127
    s2 = (0.5 + torch.rand((experts, 1, hidden), generator=generator)) * (3 / inter) ** 0.5 / 127
    weights, ids = torch.softmax(torch.randn((tokens, experts), generator=generator), -1).topk(top_k)
    mask = torch.rand((tokens,), generator=generator) > 0.2
    return dict(hidden_states=x, w_gate_up=w1.transpose(-2, -1), w_down=w2.transpose(-2, -1),
                topk_weights=weights.contiguous(), topk_ids=ids.contiguous(), scale_x=scale_x,
                scale_gate_up=s1, scale_down=s2, token_mask=mask)


def shard(case, rank, world):
    tokens = case["hidden_states"].shape[0] // world
    experts = case["w_gate_up"].shape[0] // world
    rows = slice(rank * tokens, (rank + 1) * tokens)
    block = slice(rank * experts, (rank + 1) * experts)
    out = {}
    for name, value in case.items():
        if name in ("w_gate_up", "w_down", "scale_gate_up", "scale_down"):
            out[name] = value[block]
        else:
            out[name] = value[rows]
    return out


def worker(rank, world, port, scenario, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from grain_gemm_b200 import distributed
        case = full_case()
        if scenario == "one_sided":
            case["topk_ids"] = case["topk_ids"] % 3   # every expert used lives on rank 0
        if scenario == "invalid_id":
            case["token_mask"][:] = True
            case["topk_ids"][1, 0] = 6           # token 1 belongs to rank 0 only
        local = shard(case, rank, world)
        try:
            out = distributed.moe_ffn_expert_parallel(
                **local, num_experts=case["w_gate_up"].shape[0], stages=OracleStages())
            results[rank] = ("ok", out.float())
        except ValueError as error:
            results[rank] = ("ValueError", str(error))
        dist.destroy_process_group()
    except Exception:  # pragma: no cover - surfaced by the parent
        results[rank] = ("crash", traceback.format_exc())


def run_scenario(scenario, world=2):
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(worker, args=(world, port, scenario, results), nprocs=world, join=True)
    return dict(results)


def test_expert_parallel_equals_single_process_bit_for_bit():
    results = run_scenario("plain")
    assert all(results[r][0] == "ok" for r in range(2)), results
    case = full_case()
    expected = oracle.moe_ffn(**case).float()
    actual = torch.cat([results[0][1], results[1][1]])
    assert torch.equal(actual, expected)
    assert actual[~case["token_mask"]].abs().sum() == 0


def test_rank_without_incoming_tokens():
    """All assignments go to rank 0's experts: rank 1 receives nothing and still takes part in
    every collective; repeated experts within a token travel as one row."""
    results = run_scenario("one_sided")
    assert all(results[r][0] == "ok" for r in range(2)), results
    case = full_case()
    case["topk_ids"] = case["topk_ids"] % 3
    expected = oracle.moe_ffn(**case).float()
    assert torch.equal(torch.cat([results[0][1], results[1][1]]), expected)


def test_invalid_id_on_one_rank_raises_everywhere():
    results = run_scenario("invalid_id")
    for rank in range(2):
        assert results[rank][0] == "ValueError", results[rank]
        assert "topk_ids" in results[rank][1]
