"""Parity of the CUDA GEMM (through the C ABI) with the CPU oracle and the golden fixtures.

Bar: bit-exact FP32/BF16/FP16 outputs against the oracle's fmaf chain (which is itself
bit-identical to the reference's Triton kernel on the golden fixtures), bit-exact INT32
group partials, and the reference's zero-tolerance known-answer cases.
"""

import pytest
import torch

from conftest import load_golden
from oracle import cpu as oracle

pytestmark = pytest.mark.gpu

TC_VARIANTS = ["tc_n256", "tc_n128", "tc_n64", "tc_pair_n256", "tc_pair_n128"]
ALL_VARIANTS = ["simt"] + TC_VARIANTS


@pytest.fixture(scope="module")
def gg():
    from grain_gemm_b200 import _loader, gemm
    assert _loader.is_available(), "libgrain_b200.so must be built for the GPU tests"
    yield gemm
    assert _loader.device_status() == 0, "a kernel reported a bounded-wait timeout"


def linear_case(m, n, k, g, seed, scale="uniform"):
    gen = torch.Generator().manual_seed(seed)
    a = torch.randint(-127, 128, (m, k), dtype=torch.int8, generator=gen)
    w = torch.randint(-127, 128, (n, k), dtype=torch.int8, generator=gen)
    q = (k + g - 1) // g
    if scale == "uniform":
        sa = (0.5 + torch.rand((m, q), generator=gen)) / 127
        sb = (0.5 + torch.rand((q, n), generator=gen)) / 127
    else:
        sa = torch.exp(-5 + 0.5 * torch.randn((m, q), generator=gen))
        sb = torch.exp(-5 + 0.5 * torch.randn((q, n), generator=gen))
    return a, w.t(), sa, sb


def run(gg, tensors, g, dtype, variant="auto"):
    a, b, sa, sb = (t.cuda() for t in tensors)
    # .cuda() keeps the strides of the Linear-format (transposed) weight view.
    return gg.int8_gemm(a, b, sa, sb, group_size=g, output_dtype=dtype, variant=variant).cpu()


@pytest.mark.parametrize("name", ["tails_g32", "tails_g64", "tails_g128", "tails_g256",
                                  "views_transposed", "views_sliced", "linear_weights"])
def test_golden_fixtures_bit_exact(gg, name):
    case = load_golden(f"gemm_{name}")
    g = case["group_size"]
    a, b, sa, sb = case["a"], case["b"], case["scale_a"], case["scale_b"]
    if name == "views_transposed":
        a, b, sa, sb = (t.t().contiguous().t() for t in (a, b, sa, sb))
    if name == "linear_weights":
        b = b.t().contiguous().t()
    actual = run(gg, (a, b, sa, sb), g, torch.float32)
    assert torch.equal(actual, case["triton_fp32"])
    torch.testing.assert_close(actual, case["reference_fp64"], rtol=1e-5, atol=1e-3)


def test_sliced_views_with_storage_offset(gg):
    case = load_golden("gemm_views_sliced")

    def sliced(t):
        backing = torch.zeros((2 * t.shape[0] + 1, 2 * t.shape[1] + 1), dtype=t.dtype).cuda()
        view = backing[1::2, 1::2]
        view.copy_(t)
        return view

    a, b, sa, sb = (sliced(case[k]) for k in ("a", "b", "scale_a", "scale_b"))
    assert all(not t.is_contiguous() and t.storage_offset() > 0 for t in (a, b, sa, sb))
    actual = gg.int8_gemm(a, b, sa, sb, group_size=128, output_dtype=torch.float32).cpu()
    assert torch.equal(actual, case["triton_fp32"])


@pytest.mark.parametrize("variant", ALL_VARIANTS)
def test_cancellation_needs_one_rounding_and_a_fused_add(gg, variant):
    case = load_golden("gemm_cancellation")
    tensors = (case["a"], case["b"].t().contiguous().t(), case["scale_a"], case["scale_b"])
    for dtype in (torch.float32, torch.bfloat16):
        actual = run(gg, tensors, 256, dtype, variant)
        assert torch.equal(actual.float(), torch.full((32, 64), 2.0 ** -36))


@pytest.mark.parametrize("variant", ALL_VARIANTS)
@pytest.mark.parametrize("g", [32, 64, 128, 256])
def test_random_linear_layout_bit_exact(gg, variant, g):
    m, n, k = 300, 520, 4 * g + 160 if g >= 128 else 1024 + 32
    tensors = linear_case(m, n, k, g, seed=2026 + g)
    for dtype in (torch.float32, torch.bfloat16, torch.float16):
        expected = oracle.int8_gemm(*tensors, g, dtype)
        actual = run(gg, tensors, g, dtype, variant)
        assert torch.equal(actual, expected), (variant, g, dtype)


@pytest.mark.parametrize("seed", range(6))
def test_random_shapes_dtypes_and_variants_bit_exact(gg, seed):
    """Seeded sweep over ragged M/N/K, all group sizes, output types and variants: the C tile
    leaves through a quad exchange and 16-byte stores, so N tails, unaligned row pitches
    (N not a multiple of 8) and FP32 output each take their own path."""
    import random
    rng = random.Random(seed)
    for _ in range(12):
        m = rng.choice([1, 3, 17, 100, 128, 129, 255, 300, 513])
        n = rng.choice([8, 24, 72, 136, 200, 256, 264, 520])
        g = rng.choice([32, 64, 128, 256])
        k = rng.choice([16, 48, 128, 272, 512, 768, 1040])
        dtype = rng.choice([torch.float32, torch.bfloat16, torch.float16])
        variant = rng.choice(ALL_VARIANTS + ["auto"])
        a, b, sa, sb = linear_case(m, n, k, g, seed * 100 + m + n + k, scale="lognormal")
        expected = oracle.int8_gemm(a, b, sa, sb, g, dtype)
        out = torch.empty((m, n), dtype=dtype, device="cuda")
        gg.launch(a.cuda(), b.cuda(), sa.cuda(), sb.cuda(), out, g, variant)
        assert torch.equal(out.cpu(), expected), (m, n, k, g, dtype, variant)


@pytest.mark.parametrize("variant", TC_VARIANTS)
def test_int32_group_partials_bit_exact_on_tensor_cores(gg, variant):
    """Unit scales on one group at a time expose float(partial) exactly (|p| <= 2^22)."""
    m, n, k, g = 256, 512, 1024, 256
    a, b, _, _ = linear_case(m, n, k, g, seed=7)
    a[0, :256] = -128
    b[:256, 0] = -128          # extreme product (-128 * -128) * 256 = 2^22
    _, partials = oracle.int8_gemm(a, b, torch.ones((m, 4)), torch.ones((4, n)), g,
                                   torch.float32, return_partials=True)
    assert partials[0, 0, 0] == 2 ** 22
    for group in range(4):
        sa = torch.zeros((m, 4))
        sa[:, group] = 1
        actual = run(gg, (a, b, sa, torch.ones((4, n))), g, torch.float32, variant)
        assert torch.equal(actual, partials[..., group].float())


def test_partials_entry_point_bit_exact(gg):
    tensors = linear_case(70, 90, 400, 64, seed=3)
    expected, partials = oracle.int8_gemm(*tensors, 64, torch.float32, return_partials=True)
    a, b, sa, sb = (t.cuda() for t in tensors)
    actual, actual_partials = gg.int8_gemm_partials(a, b, sa, sb, group_size=64)
    assert torch.equal(actual_partials.cpu(), partials)
    assert torch.equal(actual.cpu(), expected)


@pytest.mark.parametrize("g", [32, 64, 128, 256])
def test_int8_extrema_accumulate_without_overflow(gg, g):
    k = g + 7
    a = torch.tensor([-128, 127], dtype=torch.int8)[:, None].expand(2, k).contiguous()
    b = torch.tensor([-128, 127], dtype=torch.int8)[None, :].expand(k, 2).contiguous()
    ones = torch.ones((2, 2))
    actual = run(gg, (a, b, ones, ones), g, torch.float32)
    assert torch.equal(actual, (a.double() @ b.double()).float())


def test_signed_and_zero_scales_exact(gg):
    a = torch.ones((3, 69), dtype=torch.int8)
    b = torch.cat([torch.full((length, 4), value, dtype=torch.int8)
                   for length, value in [(32, 1), (32, -2), (5, 3)]])
    sa = torch.tensor([[1, -8, 0], [2, 0, 1], [-0.5, 2, 4]])
    sb = torch.tensor([[0.5, -2, 0, 1], [-4, 1, 0.25, 2], [2, 0.5, -1, 0]])
    actual = run(gg, (a, b, sa, sb), 32, torch.float32)
    expected = torch.zeros((3, 4), dtype=torch.float64)
    for group, (start, stop) in enumerate([(0, 32), (32, 64), (64, 69)]):
        partial = a[:, start:stop].double() @ b[start:stop].double()
        expected += partial * sa[:, group, None].double() * sb[group, None, :].double()
    assert torch.equal(actual, expected.float())


@pytest.mark.parametrize("variant", ["tc_n256", "tc_pair_n256"])
def test_endpoint_pattern_with_signed_scales(gg, variant):
    rows = torch.arange(256)[:, None]
    cols = torch.arange(128)[:, None]
    groups = torch.arange(3)[None, :]
    endpoints = torch.tensor([-128, 127], dtype=torch.int8)
    a = endpoints[(rows + groups) % 2].repeat_interleave(256, dim=1)
    w = endpoints[(cols + groups // 2) % 2].repeat_interleave(256, dim=1)
    sa = torch.tensor([0, 0.125, -0.5, 1])[(rows + 2 * groups) % 4]
    sb = torch.tensor([-0.25, 0, 0.5, 2])[(cols + 3 * groups) % 4].t().contiguous()
    expected = oracle.int8_gemm(a, w.t(), sa, sb, 256, torch.bfloat16)
    actual = run(gg, (a, w.t(), sa, sb), 256, torch.bfloat16, variant)
    assert torch.equal(actual, expected)


def test_closed_form_constant_inputs(gg):
    m, n, k = 384, 640, 1280
    a = torch.full((m, k), -128, dtype=torch.int8)
    w = torch.full((n, k), 127, dtype=torch.int8)
    sa = torch.full((m, 5), 0.125)
    sb = torch.full((5, n), 0.25)
    actual = run(gg, (a, w.t(), sa, sb), 256, torch.float32)
    assert torch.equal(actual, torch.full((m, n), -128.0 * 127 * k * 0.125 * 0.25))


def test_base_config_and_ragged_k(gg):
    # The CPU-runnable base case (256 x 4096 x 4096, G256, FP32) and the ragged K = 4000 case.
    for (m, n, k), dtype, scale in (((256, 4096, 4096), torch.float32, "uniform"),
                                    ((512, 4096, 4000), torch.bfloat16, "lognormal")):
        tensors = linear_case(m, n, k, 256, seed=2026, scale=scale)
        expected = oracle.int8_gemm(*tensors, 256, dtype)
        assert torch.equal(run(gg, tensors, 256, dtype), expected)


@pytest.mark.parametrize("g", [32, 64, 128, 256])
@pytest.mark.parametrize("m,n,k", [(1, 2048, 4096), (16, 4096, 4000), (32, 1000, 2080), (7, 8192, 8192)])
def test_split_k_for_skinny_m_is_bit_exact(gg, m, n, k, g):
    """K split over the SMs with the INT32 dots folded in group order afterwards."""
    tensors = linear_case(m, n, k, g, seed=m + g, scale="lognormal")
    for dtype in (torch.float32, torch.bfloat16):
        expected = oracle.int8_gemm(*tensors, g, dtype)
        assert torch.equal(run(gg, tensors, g, dtype, "tc_splitk"), expected)
    a, b, _, _ = (t.cuda() for t in tensors)
    config = gg.get_kernel_config(a, b, group_size=g)
    # The library's own rule splits K for these shapes (one or two rows stream the weights on
    # CUDA cores instead); a measured table entry may overrule it.
    assert config["variant"] == ("gemv" if m == 1 else "tc_splitk") or config["policy"] == "sm100_table"


@pytest.mark.parametrize("g", [32, 64, 128, 256])
@pytest.mark.parametrize("m,n,k", [(1, 2048, 4096), (2, 37, 4000), (3, 1000, 2080), (4, 8192, 8192),
                                   (5, 520, 16), (8, 4096, 7168), (1, 7, 272)])
def test_weight_streaming_kernel_for_a_handful_of_rows_is_bit_exact(gg, m, n, k, g):
    """The CUDA-core kernel for M <= 8 (dp4a dots per group, ordered fold): ragged N, K tails
    that end inside a group and inside a lane's range, every group size and output type."""
    tensors = linear_case(m, n, k, g, seed=3 * m + g, scale="lognormal")
    for dtype in (torch.float32, torch.bfloat16, torch.float16):
        expected = oracle.int8_gemm(*tensors, g, dtype)
        assert torch.equal(run(gg, tensors, g, dtype, "gemv"), expected)
    a, b, _, _ = (t.cuda() for t in tensors)
    if m == 1:
        config = gg.get_kernel_config(a, b, group_size=g)
        assert config["variant"] == "gemv" or config["policy"] == "sm100_table"
    # More than eight rows, or a K that is not a whole number of 16-byte chunks, is refused.
    with pytest.raises(RuntimeError):
        run(gg, linear_case(9, 64, 256, g, seed=1, scale="lognormal"), g, torch.float32, "gemv")
    with pytest.raises(RuntimeError):
        run(gg, linear_case(2, 64, 264, g, seed=1, scale="lognormal"), g, torch.float32, "gemv")


@pytest.mark.parametrize("g", [32, 256])
@pytest.mark.parametrize("m", [9, 33, 64, 65])
def test_tiles_with_whole_warps_of_missing_rows_are_bit_exact(gg, m, g):
    """Promotion warps whose 32 rows lie beyond M hand their accumulator buffer straight back;
    the warps that have rows must not notice (9, 33, 64 and 65 rows: one to three such warps)."""
    tensors = linear_case(m, 520, 1040, g, seed=m + g, scale="lognormal")
    for dtype in (torch.float32, torch.bfloat16):
        expected = oracle.int8_gemm(*tensors, g, dtype)
        for variant in ("tc_n64", "tc_n256"):
            assert torch.equal(run(gg, tensors, g, dtype, variant), expected), (m, g, dtype, variant)


@pytest.mark.parametrize("m", [1, 16, 128])
def test_skinny_m(gg, m):
    tensors = linear_case(m, 2048, 2048, 128, seed=m, scale="lognormal")
    expected = oracle.int8_gemm(*tensors, 128, torch.bfloat16)
    assert torch.equal(run(gg, tensors, 128, torch.bfloat16), expected)


def test_full_size_linearity_property(gg):
    """8192^3 is too large for the CPU oracle: check sampled rows against it and the
    homogeneity property C(2*sa) == 2*C(sa), which is exact in binary floating point."""
    m = n = k = 8192
    gen = torch.Generator(device="cuda").manual_seed(5)
    a = torch.randint(-127, 128, (m, k), dtype=torch.int8, device="cuda", generator=gen)
    w = torch.randint(-127, 128, (n, k), dtype=torch.int8, device="cuda", generator=gen)
    sa = torch.exp(-5 + 0.5 * torch.randn((m, 32), device="cuda", generator=gen))
    sb = torch.exp(-5 + 0.5 * torch.randn((32, n), device="cuda", generator=gen))
    out = gg.int8_gemm(a, w.t(), sa, sb, group_size=256, output_dtype=torch.float32)
    doubled = gg.int8_gemm(a, w.t(), sa * 2, sb, group_size=256, output_dtype=torch.float32)
    assert torch.equal(doubled, out * 2)
    rows = torch.tensor([0, 127, 128, 4095, 8191])
    cols = torch.arange(0, n, 61)
    expected = oracle.int8_gemm(a[rows].cpu(), w[cols].cpu().t(), sa[rows].cpu(),
                                sb[:, cols].cpu().contiguous(), 256, torch.float32)
    assert torch.equal(out[rows][:, cols].cpu(), expected)


@pytest.mark.parametrize("g", [32, 64, 128, 256])
@pytest.mark.parametrize("m", [1, 16, 128, 1024, 8192])
def test_sweep_k8192_n8192_sampled_rows_bit_exact(gg, g, m):
    """The sweep G in {32, 64, 128, 256} x M in {1, 16, 128, 1024, 8192} at K = N = 8192 with
    lognormal scales, BF16 and FP32 outputs, whichever variant `auto` picks for the shape:
    sampled rows (all of them for M <= 16) over all 8192 columns against the oracle."""
    n = k = 8192
    gen = torch.Generator(device="cuda").manual_seed(2026 + g + m)
    a = torch.randint(-127, 128, (m, k), dtype=torch.int8, device="cuda", generator=gen)
    w = torch.randint(-127, 128, (n, k), dtype=torch.int8, device="cuda", generator=gen)
    q = k // g
    sa = torch.exp(-5 + 0.5 * torch.randn((m, q), device="cuda", generator=gen))
    sb = torch.exp(-5 + 0.5 * torch.randn((q, n), device="cuda", generator=gen))
    rows = torch.arange(m) if m <= 16 else torch.tensor(sorted({0, 1, 127, m // 2 + 5, m - 129, m - 1}))
    w_cpu, sb_cpu = w.cpu(), sb.cpu()
    a_rows, sa_rows = a[rows.cuda()].cpu(), sa[rows.cuda()].cpu()
    for dtype in (torch.bfloat16, torch.float32):
        out = gg.int8_gemm(a, w.t(), sa, sb, group_size=g, output_dtype=dtype)
        expected = oracle.int8_gemm(a_rows, w_cpu.t(), sa_rows, sb_cpu, g, dtype)
        assert torch.equal(out[rows.cuda()].cpu(), expected), (g, m, dtype)


def test_large_row_major_b_is_repacked_for_the_tensor_cores(gg):
    """A contiguous [K, N] B (N fastest) must not fall off a performance cliff: it is copied
    to K-contiguous storage once and gives the same bits as the Linear-format view."""
    m, n, k = 512, 2048, 4096
    a, b, sa, sb = linear_case(m, n, k, 256, seed=21)
    expected = oracle.int8_gemm(a, b, sa, sb, 256, torch.bfloat16)
    row_major = b.contiguous().cuda()
    assert row_major.stride() == (n, 1)
    out = gg.int8_gemm(a.cuda(), row_major, sa.cuda(), sb.cuda(), group_size=256)
    assert torch.equal(out.cpu(), expected)
    column_major_a = a.t().contiguous().t().cuda()
    assert column_major_a.stride() == (1, m)
    out = gg.int8_gemm(column_major_a, b.cuda(), sa.cuda(), sb.cuda(), group_size=256)
    assert torch.equal(out.cpu(), expected)


def test_zero_sized_and_config_description(gg):
    a = torch.zeros((0, 64), dtype=torch.int8, device="cuda")
    b = torch.zeros((64, 8), dtype=torch.int8, device="cuda")
    out = gg.int8_gemm(a, b, torch.ones((0, 1), device="cuda"), torch.ones((1, 8), device="cuda"))
    assert out.shape == (0, 8) and out.dtype == torch.bfloat16
    a, b, _, _ = (t.cuda() for t in linear_case(8192, 8192, 512, 256, seed=1))
    config = gg.get_kernel_config(a, b, group_size=256)
    assert config["backend"] == "cuda" and config["policy"] in ("sm100_native", "sm100_table")
    assert config["compute_capability"] == [10, 0] and config["tensor_cores"]
    config = gg.get_kernel_config(a, b.contiguous(), group_size=256)
    assert config["tensor_cores"] and config["repacked_b"] and not config["repacked_a"]
    config = gg.get_kernel_config(a[:16, :64], b[:64, :24].contiguous(), group_size=32)
    assert config["variant"] == "simt" and not config["repacked_b"]
    with pytest.raises(ValueError, match="stride"):
        gg.int8_gemm(a[:1].expand(8192, 512), b, torch.ones((8192, 2), device="cuda"),
                     torch.ones((2, 8192), device="cuda"))


def test_streams_and_graph_replay_read_updated_inputs(gg):
    tensors = [t.cuda() for t in linear_case(256, 128, 768, 256, seed=9)]
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(3):
            gg.int8_gemm(*tensors, group_size=256, output_dtype=torch.float32)
    torch.cuda.current_stream().wait_stream(stream)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        actual = gg.int8_gemm(*tensors, group_size=256, output_dtype=torch.float32)
    graph.replay()
    expected = oracle.int8_gemm(*(t.cpu() for t in tensors), 256, torch.float32)
    assert torch.equal(actual.cpu(), expected)
    a, b, sa, sb = tensors
    a.fill_(1)
    b.fill_(-2)
    sa.fill_(0.125)
    sb.fill_(-0.25)
    graph.replay()
    assert torch.equal(actual.cpu(), torch.full((256, 128), 48.0))
    with torch.cuda.stream(stream):
        a.fill_(-7)
        b.fill_(5)
        sb.fill_(0.25)
        streamed = gg.int8_gemm(*tensors, group_size=256, output_dtype=torch.float32)
    torch.cuda.current_stream().wait_stream(stream)
    assert torch.equal(streamed.cpu(), torch.full((256, 128), -840.0))


def test_reference_native_entry_point_alias(gg):
    from grain_gemm_b200 import _loader
    a, b, sa, sb = (t.cuda() for t in linear_case(256, 512, 768, 256, seed=11))
    out = torch.empty((256, 512), dtype=torch.bfloat16, device="cuda")
    weights = b.t()
    assert weights.is_contiguous()
    status = _loader.library().grain_cute_g256(
        _loader.pointer(a), _loader.pointer(weights), _loader.pointer(sa), _loader.pointer(sb),
        _loader.pointer(out), 256, 512, 768, 27, _loader.stream_pointer(a.device))
    assert status == 0
    expected = oracle.int8_gemm(a.cpu(), b.cpu(), sa.cpu(), sb.cpu(), 256, torch.bfloat16)
    assert torch.equal(out.cpu(), expected)
