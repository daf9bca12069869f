"""Expert-parallel moe_ffn on two GPUs (NCCL): bit-identical to the single-GPU result."""

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


def worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    try:
        torch.cuda.set_device(rank)
        device = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
        import bench_moe
        from grain_gemm_b200 import _loader, distributed, moe
        bench_moe.CONFIGS["ep_test"] = dict(tokens=768, hidden=1024, inter=512, experts=16,
                                            top_k=4, layout="split", biased=True)
        local = bench_moe.make_case("ep_test", device, rank=rank, world=world)
        out = distributed.moe_ffn_expert_parallel(**local, num_experts=16)
        # The same tokens through all experts on this GPU alone.
        whole = bench_moe.make_case("ep_test", device, rank=0, world=1)
        tokens = 768 // world
        rows = slice(rank * tokens, (rank + 1) * tokens)
        for name in ("hidden_states", "scale_x", "topk_weights", "topk_ids"):
            assert torch.equal(whole[name][rows], local[name]), name
        single = moe.moe_ffn(**whole)
        results[rank] = ("ok", bool(torch.equal(out, single[rows])), _loader.device_status())
        dist.barrier()
        dist.destroy_process_group()
    except Exception:  # pragma: no cover - surfaced by the parent
        results[rank] = ("crash", traceback.format_exc())


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_expert_parallel_matches_single_gpu_bits():
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    results = mp.Manager().dict()
    mp.spawn(worker, args=(2, port, results), nprocs=2, join=True)
    for rank in range(2):
        assert results[rank] == ("ok", True, 0), results[rank]
