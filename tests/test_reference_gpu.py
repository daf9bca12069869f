"""The CUDA path against the reference itself, run on the same GPU.

On a B200 the reference's own GPU path is its Triton backend (``auto`` selects it for compute
capability 10.0).  When the reference is installed beside the oracle (``oracle/make_ref.py``
puts it into the git-ignored ``oracle/_ref``), these tests call its Triton kernels on identical
seeded inputs and compare bit for bit at sizes no CPU oracle reaches: full 8192-wide GEMM
outputs in BF16 and FP32, and every stage of ``moe_ffn`` (routing metadata, quantised
activations and scales - the one place where libdevice ``expf`` is evaluated -, the Down
projection) on the decode, prefill and expert-parallel-sized configurations.  Only the final
combine is compared at a tolerance: the reference adds the top-k slots with a tree reduction
(``tl.sum``), this library in slot order, so an FP32 sum may differ in its last bit and flip a
BF16 rounding (counted and bounded below).  Skipped when the reference is not installed.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def reference():
    from oracle import make_ref
    module = make_ref.load()
    if module is None:
        pytest.skip("the reference is not installed in oracle/_ref (python oracle/make_ref.py)")
    import importlib
    kernels = importlib.import_module("grain_gemm_reference.kernels.moe")
    return module, kernels


@pytest.fixture(scope="module")
def ours():
    from grain_gemm_b200 import _loader, gemm, moe
    yield gemm, moe
    assert _loader.device_status() == 0


def gemm_inputs(m, n, k, g, seed):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randint(-127, 128, (m, k), dtype=torch.int8, device="cuda", generator=gen)
    w = torch.randint(-127, 128, (n, k), dtype=torch.int8, device="cuda", generator=gen)
    q = (k + g - 1) // g
    sa = torch.exp(-5 + 0.5 * torch.randn((m, q), device="cuda", generator=gen))
    sb = torch.exp(-5 + 0.5 * torch.randn((q, n), device="cuda", generator=gen))
    return a, w.t(), sa, sb


@pytest.mark.parametrize("m,n,k,g", [(8192, 8192, 8192, 256), (1024, 8192, 8192, 32),
                                     (128, 8192, 8192, 64), (16, 8192, 8192, 128),
                                     (1, 8192, 8192, 256), (512, 4096, 4000, 256)])
def test_gemm_equals_reference_triton_bits(reference, ours, m, n, k, g):
    module, _ = reference
    gemm, _ = ours
    a, b, sa, sb = gemm_inputs(m, n, k, g, 2026 + g + m)
    for dtype in (torch.bfloat16, torch.float32):
        expected = module.int8_gemm(a, b, sa, sb, group_size=g, output_dtype=dtype, backend="triton")
        actual = gemm.int8_gemm(a, b, sa, sb, group_size=g, output_dtype=dtype)
        assert torch.equal(actual, expected), (m, n, k, g, dtype)


@pytest.mark.parametrize("name", ["decode_small", "interleaved_decode", "interleaved_prefill",
                                  "large_rank_share", "large_quarter"])
def test_moe_stages_equal_reference_triton_bits(reference, ours, name):
    """`large_quarter` is a quarter of the 16384-token, 256-expert configuration (4096 tokens, 64
    experts of the same shape): the reference addresses weights with 32-bit offsets and rejects
    tensors of 2^31 elements or more (src/grain_gemm/moe.py:82-83), so it cannot run the whole
    configuration on one GPU, which this library can."""
    import bench_moe
    module, kernels = reference
    _, moe = ours
    bench_moe.CONFIGS["large_quarter"] = dict(tokens=4096, hidden=7168, inter=2048, experts=64,
                                              top_k=8, layout="split", biased=False)
    case = bench_moe.make_case(name, torch.device("cuda"))
    layout = case["gate_up_layout"]
    experts = case["w_gate_up"].shape[0]
    w1 = case["w_gate_up"].transpose(-2, -1)
    w2 = case["w_down"].transpose(-2, -1)

    expected_routes = kernels.prepare_routes(case["topk_ids"], experts, None)
    routes = moe.prepare_routes(case["topk_ids"], experts, None)
    for field in ("order", "inverse", "counts", "offsets", "effective_ids", "statistics"):
        assert torch.equal(getattr(routes, field), getattr(expected_routes, field)), field
    valid = int(routes.offsets[-1])

    gate_up = kernels.ragged_gemm(case["hidden_states"], w1, case["scale_x"], case["scale_gate_up"],
                                  expected_routes, output_dtype=torch.bfloat16, source_is_token=True)
    expected_q, expected_s = kernels.swiglu_quantize(gate_up, routes=expected_routes,
                                                     gate_up_layout=layout)
    del gate_up
    qh, sh = moe.gate_up_swiglu_quantize(case["hidden_states"], case["scale_x"], w1,
                                         case["scale_gate_up"], routes, gate_up_layout=layout)
    assert torch.equal(sh[:valid], expected_s[:valid])
    assert torch.equal(qh[:valid], expected_q[:valid])

    expected_out = kernels.ragged_gemm(expected_q, w2, expected_s, case["scale_down"],
                                       expected_routes, output_dtype=torch.bfloat16)
    expert_out = moe.down_projection(qh, sh, w2, case["scale_down"], routes)
    assert torch.equal(expert_out[:valid], expected_out[:valid])

    expected_final = kernels.combine(expected_out, case["topk_weights"], expected_routes,
                                     output_dtype=torch.bfloat16)
    final = moe.combine(expert_out, case["topk_weights"], routes)
    differing = (final != expected_final)
    fraction = differing.float().mean().item()
    print(f"{name}: {int(differing.sum())} of {final.numel()} final BF16 values differ from the "
          f"reference's tree-order combine ({fraction:.2e})")
    assert fraction < 2e-2
    torch.testing.assert_close(final.float(), expected_final.float(), rtol=1e-2, atol=1e-2)
    # The whole public call gives what the stages gave.
    assert torch.equal(moe.moe_ffn(**case), final)
