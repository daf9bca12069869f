"""Expert-parallel moe_ffn: bit-identical to the single-GPU result.

Two exchange mechanisms are covered: NCCL all-to-all and stores into peer memory
(``PeerExchange``).  The peer path is also run with all ranks inside one process on one GPU
(``PeerExchange.local_ranks``): the same kernels write to the same kind of addresses, only the
collectives are replaced by running the phases rank by rank, so a single-GPU box still checks
the plan, dispatch, row-mask, row-destination and Down-to-destination kernels bit for bit.
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

pytestmark = pytest.mark.gpu


EP_TEST = dict(tokens=768, hidden=1024, inter=512, experts=16, top_k=4, layout="split", biased=True)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("layout", ["split", "interleaved"])
def test_peer_exchange_with_all_ranks_on_one_gpu_matches_single_gpu_bits(world, layout):
    import bench_moe
    from grain_gemm_b200 import _loader, distributed, moe
    device = torch.device("cuda")
    bench_moe.CONFIGS["ep_test"] = dict(EP_TEST, layout=layout)
    whole = bench_moe.make_case("ep_test", device)
    generator = torch.Generator().manual_seed(world)
    mask = (torch.rand((768,), generator=generator) > 0.15).to(device)
    whole["topk_ids"][5, 1] = 77          # out of range, but on a masked token
    mask[5] = False
    single = moe.moe_ffn(**whole, token_mask=mask)
    tokens = 768 // world
    exchanges = distributed.PeerExchange.local_ranks(
        world, capacity=tokens, hidden=1024, top_k=4, local_experts=16 // world, device=device)
    try:
        cases = [bench_moe.make_case("ep_test", device, rank=r, world=world) for r in range(world)]
        for r, case in enumerate(cases):
            case["topk_ids"] = whole["topk_ids"][r * tokens:(r + 1) * tokens].contiguous()
        masks = [mask[r * tokens:(r + 1) * tokens].contiguous() for r in range(world)]
        for repeat in range(2):           # the areas are reused from call to call
            outputs = distributed.run_local_ranks(exchanges, cases, masks)
            for r in range(world):
                assert torch.equal(outputs[r], single[r * tokens:(r + 1) * tokens]), (r, repeat)
        # An unmasked invalid id on one rank is reported.
        cases[world - 1]["topk_ids"][3, 0] = 16
        masks[world - 1][3] = True
        with pytest.raises(ValueError, match="topk_ids"):
            distributed.run_local_ranks(exchanges, cases, masks)
    finally:
        for exchange in exchanges:
            exchange.close()
    assert _loader.device_status() == 0


def captured_step(distributed, exchange, static):
    """Capture one expert-parallel step over the tensors of ``static`` into a CUDA graph."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):                # warm-up: buffers of the workspace, function attributes
            distributed.moe_ffn_expert_parallel(**static, exchange=exchange)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = distributed.moe_ffn_expert_parallel(**static, exchange=exchange)
    return graph, out


def test_peer_exchange_step_replays_from_a_cuda_graph_with_new_routing():
    """The peer-memory step has no host read-back on its path, so a whole step (plan, dispatch,
    routing, Gate/Up, Down into home_out, combine) is one CUDA graph; replays follow the token
    rows, ids and weights written into the captured tensors."""
    import bench_moe
    from grain_gemm_b200 import _loader, distributed, moe
    device = torch.device("cuda")
    bench_moe.CONFIGS["ep_test"] = dict(EP_TEST)
    case = bench_moe.make_case("ep_test", device)
    exchange = distributed.PeerExchange.local_ranks(
        1, capacity=768, hidden=1024, top_k=4, local_experts=16, device=device)[0]
    try:
        static = dict(case, num_experts=16)
        graph, out = captured_step(distributed, exchange, static)
        generator = torch.Generator(device="cuda").manual_seed(11)
        for repeat in range(3):
            ids = torch.randint(0, 16, (768, 4), device=device, generator=generator,
                                dtype=case["topk_ids"].dtype)
            x = torch.randint(-127, 128, (768, 1024), device=device, generator=generator,
                              dtype=torch.int8)
            static["topk_ids"].copy_(ids)
            static["hidden_states"].copy_(x)
            graph.replay()
            expected = moe.moe_ffn(**case)          # `case` shares the captured tensors
            assert torch.equal(out, expected), repeat
    finally:
        exchange.close()
    assert _loader.device_status() == 0


def worker(rank, world, port, results, from_graph=False):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    try:
        torch.cuda.set_device(rank)
        device = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
        import bench_moe
        from grain_gemm_b200 import _loader, distributed, moe
        bench_moe.CONFIGS["ep_test"] = dict(EP_TEST)
        local = bench_moe.make_case("ep_test", device, rank=rank, world=world)
        # The same tokens through all experts on this GPU alone.
        whole = bench_moe.make_case("ep_test", device, rank=0, world=1)
        tokens = 768 // world
        rows = slice(rank * tokens, (rank + 1) * tokens)
        for name in ("hidden_states", "scale_x", "topk_weights", "topk_ids"):
            assert torch.equal(whole[name][rows], local[name]), name
        single = moe.moe_ffn(**whole)
        via_nccl = distributed.moe_ffn_expert_parallel(**local, num_experts=16)
        exchange = distributed.PeerExchange.create(
            dist.group.WORLD, capacity=tokens, hidden=1024, top_k=4, local_experts=16 // world)
        via_peers = [distributed.moe_ffn_expert_parallel(**local, num_experts=16, exchange=exchange)
                     for _ in range(3)]
        torch.cuda.synchronize()
        replays = []
        if from_graph:
            # The same step from a CUDA graph (the two small collectives are captured with it).
            graph, captured_out = captured_step(distributed, exchange, dict(local, num_experts=16))
            for _ in range(2):
                captured_out.zero_()
                graph.replay()
                torch.cuda.synchronize()
                replays.append(bool(torch.equal(captured_out, single[rows])))
            del graph
        results[rank] = ("ok", bool(torch.equal(via_nccl, single[rows])),
                         all(bool(torch.equal(out, single[rows])) for out in via_peers)
                         and all(replays), _loader.device_status())
        dist.barrier()
        exchange.close()
        dist.barrier()
        dist.destroy_process_group()
    except Exception:  # pragma: no cover - surfaced by the parent
        results[rank] = ("crash", traceback.format_exc())


@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_matches_single_gpu_bits(world):
    """One process per GPU: NCCL all-to-all and the peer-memory exchange against one GPU."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    results = mp.Manager().dict()
    mp.spawn(worker, args=(world, port, results), nprocs=world, join=True)
    for rank in range(world):
        assert results[rank] == ("ok", True, True, 0), results[rank]


def test_expert_parallel_step_replays_from_a_cuda_graph_on_two_gpus():
    """The peer-memory step with its count all-gather and its 2-int all-reduce inside one CUDA
    graph per rank; replays are bit-identical to one GPU."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    results = mp.Manager().dict()
    mp.spawn(worker, args=(2, port, results, True), nprocs=2, join=True)
    for rank in range(2):
        assert results[rank] == ("ok", True, True, 0), results[rank]
