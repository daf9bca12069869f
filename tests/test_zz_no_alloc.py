"""Routing through the entry point that allocates nothing.

Some hosts of the library cannot allocate device memory where routing runs (a server
that hands out its whole memory budget at start-up, a plugin without an allocator, a loop
that must avoid the device-wide synchronisation an allocation implies), so they cannot give
``gg_moe_route`` its workspace.  ``gg_moe_route_noalloc`` keeps that scratch in a fixed
2 MiB array inside the library instead.  This test calls it through the C ABI twice in a
row, with different routing problems, and checks every output against ``gg_moe_route`` run
on a caller-provided workspace: routing is integer work, so the outputs must be identical.
The second call also shows that what the first call left in the shared scratch does not
leak into the next result.  The file name sorts last so that a run that stops at the first
failure has already run every other test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _route(lib, loader, ids, mask, experts, static_scratch):
    tokens, top_k = ids.shape
    slots = tokens * top_k
    device = ids.device
    outputs = dict(
        effective_ids=torch.full((slots,), -7, dtype=ids.dtype, device=device),
        order=torch.full((slots,), -7, dtype=torch.int64, device=device),
        inverse=torch.full((slots,), -7, dtype=torch.int32, device=device),
        counts=torch.full((experts,), -7, dtype=torch.int32, device=device),
        offsets=torch.full((experts + 1,), -7, dtype=torch.int32, device=device),
        statistics=torch.full((3,), -7, dtype=torch.int32, device=device),
    )
    common = [loader.pointer(ids), int(ids.dtype == torch.int64), loader.pointer(mask),
              tokens, top_k, experts] + [loader.pointer(outputs[name]) for name in outputs]
    stream = loader.stream_pointer(device)
    if static_scratch:
        status = lib.gg_moe_route_noalloc(*common, stream)
    else:
        size = lib.gg_moe_route_workspace_bytes(tokens, top_k, experts)
        workspace = torch.empty((max(size, 1),), dtype=torch.uint8, device=device)
        status = lib.gg_moe_route(*common, loader.pointer(workspace), size, stream)
    assert status == 0, lib.gg_error_string(status)
    torch.cuda.synchronize(device)
    return {name: tensor.cpu() for name, tensor in outputs.items()}


def test_noalloc_routing_matches_workspace_routing_twice_in_a_row():
    from grain_gemm_b200 import _loader

    lib = _loader.library()
    generator = torch.Generator().manual_seed(99)
    problems = [
        # multi-chunk problem with masked tokens and out-of-range ids (uses the static scratch)
        (torch.randint(-3, 260, (4099, 8), generator=generator).to(torch.int32), True, 256),
        # different shape and id width right after it, reusing the same scratch
        (torch.randint(0, 40, (2500, 3), generator=generator).to(torch.int64), False, 40),
    ]
    for ids, with_mask, experts in problems:
        mask = (torch.rand((ids.shape[0],), generator=generator) > 0.2) if with_mask else None
        ids_gpu = ids.cuda()
        mask_gpu = mask.cuda() if mask is not None else None
        expected = _route(lib, _loader, ids_gpu, mask_gpu, experts, static_scratch=False)
        actual = _route(lib, _loader, ids_gpu, mask_gpu, experts, static_scratch=True)
        for name in expected:
            assert torch.equal(actual[name], expected[name]), name
    assert _loader.device_status() == 0


def test_noalloc_routing_rejects_problems_beyond_its_capacity():
    from grain_gemm_b200 import _loader

    lib = _loader.library()
    capacity = lib.gg_moe_route_noalloc_capacity_bytes()
    assert capacity == 2 * 1024 * 1024
    tokens, top_k, experts = 131072, 8, 4094          # 1024 chunks x 4096 ints > capacity
    assert lib.gg_moe_route_workspace_bytes(tokens, top_k, experts) > capacity
    null = ctypes.c_void_p(0)
    status = lib.gg_moe_route_noalloc(null, 0, null, tokens, top_k, experts, null, null, null,
                                      null, null, null, null)
    assert status == -20001
    assert b"static scratch" in lib.gg_error_string(status)
