"""Parity of the CUDA MoE stages (through the C ABI) with the CPU oracle and golden fixtures.

Every stage is compared bit for bit: routing metadata, the quantised activations and their
scales, the Down projection and the combine.  The one place where host and device arithmetic
can differ is ``expf`` inside SiLU.  The CUDA path evaluates SiLU once per 16-bit gate pattern
into a 65536-entry table (``gg_moe_silu_table``); ``test_silu_table_against_host_formula``
compares that table with the host formula entry by entry and lists the patterns that differ,
and the stage tests hand the GPU's table to the oracle, so that everything downstream of it
must agree exactly.  Final outputs are also checked against the table-free oracle at
rtol 1e-3 / atol 1e-2 after BF16/FP16 rounding.
"""

import pytest
import torch

from conftest import load_golden
from oracle import cpu as oracle

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-3, 1e-2


@pytest.fixture(scope="module")
def moe():
    from grain_gemm_b200 import _loader, moe
    assert _loader.is_available(), "libgrain_b200.so must be built for the GPU tests"
    yield moe
    assert _loader.device_status() == 0, "a kernel reported a bounded-wait timeout"


_TABLES = {}


def gpu_silu_table(dtype):
    """The library's SiLU table for `dtype` (BF16/FP16), read back to the host."""
    if dtype not in _TABLES:
        from grain_gemm_b200 import _loader
        table = torch.empty((65536,), dtype=torch.float32, device="cuda")
        _loader.check(_loader.library().gg_moe_silu_table(
            _loader.pointer(table), _loader.OUT_DTYPE[dtype], _loader.stream_pointer(table.device)),
            "gg_moe_silu_table")
        _TABLES[dtype] = table.cpu()
    return _TABLES[dtype]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_silu_table_against_host_formula(moe, dtype):
    """Entry by entry: the GPU's silu(v) for every 16-bit pattern against the host's
    v / (1 + expf(-v)).  CUDA's expf and the host C library's may round differently in the last
    place; the differing patterns are enumerated here (and printed), each within a few units in
    the last place (at most 4 seen), so the set on which the two arithmetics disagree is known, finite and small
    (856 BF16 and 5701 FP16 patterns on the first B200 this ran on)."""
    table = gpu_silu_table(dtype)
    patterns = torch.arange(65536, dtype=torch.int32).to(torch.int16)
    values = patterns.view(dtype).float()
    host = oracle.silu(values)
    finite = torch.isfinite(values)
    assert torch.equal(torch.isnan(table), torch.isnan(host))
    same = (table.view(torch.int32) == host.view(torch.int32)) | torch.isnan(host)
    differing = torch.nonzero(~same).flatten()
    ulps = (table.view(torch.int32)[differing] - host.view(torch.int32)[differing]).abs()
    print(f"silu table ({dtype}): {differing.numel()} of 65536 patterns differ from the host "
          f"formula: {[hex(int(b)) for b in differing[:64]]}{' ...' if differing.numel() > 64 else ''}")
    assert finite[differing].all()
    assert differing.numel() < 7864           # under 12 % of the patterns
    assert ulps.numel() == 0 or int(ulps.max()) <= 8
    # Known answers that involve no rounding: silu(+0) = 0 and silu(+inf) = inf.
    infinity = int(torch.tensor([float("inf")]).to(dtype).view(torch.int16))
    assert table[0] == 0 and table[infinity] == float("inf")


def assert_routes_equal(routes, expected):
    for field in ("order", "inverse", "counts", "offsets", "effective_ids", "statistics"):
        actual = getattr(routes, field).cpu()
        wanted = getattr(expected, field) if not isinstance(expected, dict) else expected[field]
        assert actual.dtype == wanted.dtype, field
        assert torch.equal(actual, wanted), field


@pytest.mark.parametrize("name", ["mixed", "all_masked", "e32_t1031", "e64_t1031", "e65_t1031",
                                  "e128_top8_int32"])
def test_routes_match_reference_fixtures(moe, name):
    case = load_golden(f"routes_{name}")
    mask = case["mask"].bool().cuda() if "mask" in case else None
    routes = moe.prepare_routes(case["ids"].cuda(), case["experts"], mask, tile_rows=0)
    assert_routes_equal(routes, case)


@pytest.mark.parametrize("tokens,top_k,experts,dtype", [
    (0, 3, 5, torch.int64), (1, 1, 1, torch.int32), (128, 8, 128, torch.int32),
    (1024, 1, 7, torch.int64), (1025, 1, 7, torch.int64), (512, 8, 128, torch.int64),
    (16384, 8, 256, torch.int32), (4096, 2, 8, torch.int64), (3000, 5, 1000, torch.int32),
    (8192, 1, 511, torch.int32), (1366, 6, 33, torch.int64), (2048, 4, 512, torch.int32)])
def test_routes_match_oracle(moe, tokens, top_k, experts, dtype):
    gen = torch.Generator().manual_seed(tokens + experts)
    ids = torch.randint(-2, experts + 2, (tokens, top_k), generator=gen).to(dtype)
    mask = torch.rand((tokens,), generator=gen) > 0.1
    for m in (None, mask):
        expected = oracle.route(ids, experts, m)
        routes = moe.prepare_routes(ids.cuda(), experts, m.cuda() if m is not None else None,
                                    tile_rows=0)
        assert_routes_equal(routes, expected)


@pytest.mark.parametrize("count", [9, 2500])
def test_tile_list(moe, count):
    """The tile list is a scan over the experts, 1024 at a time: few and many experts."""
    gen = torch.Generator().manual_seed(4)
    ids = torch.randint(0, count, (700, 2), generator=gen)
    for tile_rows in (32, 128):
        routes = moe.prepare_routes(ids.cuda(), count, None, tile_rows=tile_rows)
        offsets = routes.offsets.cpu().tolist()
        experts, rows = [], []
        for e in range(count):
            for start in range(offsets[e], offsets[e + 1], tile_rows):
                experts.append(e)
                rows.append(start)
        used = len(experts)
        assert routes.tile_expert.numel() == (1400 + tile_rows - 1) // tile_rows + count
        assert routes.tile_expert[:used].cpu().tolist() == experts
        assert routes.tile_row[:used].cpu().tolist() == rows
        assert (routes.tile_expert[used:] < 0).all()


def make_case(tokens, hidden, inter, experts, top_k, *, seed=2026, layout="split",
              dtype=torch.bfloat16, biased=False, mask=False, ids_dtype=torch.int64):
    """Seeded synthetic MoE case: uniform INT8 values, uniform positive scales, softmax top-k."""
    gen = torch.Generator().manual_seed(seed)
    x = torch.randint(-127, 128, (tokens, hidden), dtype=torch.int8, generator=gen)
    scale_x = (0.5 + torch.rand((tokens, hidden // 256), generator=gen)) / 127
    logits = torch.randn((tokens, experts), generator=gen)
    if biased:
        logits[:, 0] += 2
    weights, ids = torch.softmax(logits, dim=-1).topk(top_k, dim=-1)
    weights = (weights / weights.sum(-1, keepdim=True)).float().contiguous()
    w1 = torch.randint(-127, 128, (experts, 2 * inter, hidden), dtype=torch.int8, generator=gen)
    w2 = torch.randint(-127, 128, (experts, hidden, inter), dtype=torch.int8, generator=gen)
    w1[:, :, 0], w1[:, :, 1] = -128, 127
    s1 = (0.5 + torch.rand((experts, hidden // 256, 2 * inter), generator=gen)) * (3 / hidden) ** 0.5 / 127
    s2 = (0.5 + torch.rand((experts, inter // 256, hidden), generator=gen)) * (3 / inter) ** 0.5 / 127
    s1[:, :, ::11] *= -1
    s1[:, :, 5::17] = 0
    if layout == "interleaved":
        # Column order [g0, u0, g1, u1, ...] of the same logical weights.
        permutation = torch.stack([torch.arange(inter), inter + torch.arange(inter)], 1).reshape(-1)
        w1 = w1[:, permutation].contiguous()
        s1 = s1[:, :, permutation].contiguous()
    case = dict(hidden_states=x, w_gate_up=w1.transpose(-2, -1), w_down=w2.transpose(-2, -1),
                topk_weights=weights, topk_ids=ids.to(ids_dtype).contiguous(), scale_x=scale_x,
                scale_gate_up=s1, scale_down=s2, output_dtype=dtype, gate_up_layout=layout)
    if mask:
        case["token_mask"] = torch.rand((tokens,), generator=gen) > 0.2
    return case


def to_cuda(case):
    return {k: v.cuda() if isinstance(v, torch.Tensor) else v for k, v in case.items()}


def run_stages(moe, case, variant):
    """Run the CUDA stages one by one and check each against the oracle on the same inputs."""
    dev = to_cuda(case)
    dtype, layout = case["output_dtype"], case["gate_up_layout"]
    experts = case["w_gate_up"].shape[0]
    tile_rows = 32 if variant == "cuda_core" else 128
    mask = case.get("token_mask")
    routes = moe.prepare_routes(dev["topk_ids"], experts, dev.get("token_mask"), tile_rows=tile_rows)
    expected_routes = oracle.route(case["topk_ids"], experts, mask)
    assert_routes_equal(routes, expected_routes)
    valid = int(expected_routes.offsets[-1])

    w1 = dev["w_gate_up"].transpose(-2, -1)
    w2 = dev["w_down"].transpose(-2, -1)
    qh, sh = moe.gate_up_swiglu_quantize(dev["hidden_states"], dev["scale_x"], w1,
                                         dev["scale_gate_up"], routes, output_dtype=dtype,
                                         gate_up_layout=layout,
                                         row_gather=variant == "tensor_core_gather")
    gate_up = oracle.ragged_gemm(case["hidden_states"], case["w_gate_up"].transpose(-2, -1),
                                 case["scale_x"], case["scale_gate_up"], expected_routes, dtype,
                                 source_is_token=True)
    expected_q, expected_s = oracle.swiglu_quantize(gate_up, valid, layout,
                                                    silu_table=gpu_silu_table(dtype))
    assert torch.equal(sh.cpu()[:valid], expected_s[:valid])
    assert torch.equal(qh.cpu()[:valid], expected_q[:valid])

    # Down and combine, on the (identical) quantised activations.
    expert_out = moe.down_projection(qh, sh, w2, dev["scale_down"], routes, output_dtype=dtype)
    expected_out = oracle.ragged_gemm(qh.cpu(), case["w_down"].transpose(-2, -1), sh.cpu(),
                                      case["scale_down"], expected_routes, dtype,
                                      source_is_token=False)
    assert torch.equal(expert_out.cpu()[:valid], expected_out[:valid])
    out = moe.combine(expert_out, dev["topk_weights"], routes, output_dtype=dtype)
    expected_final = oracle.combine(expert_out.cpu(), case["topk_weights"], expected_routes, dtype)
    assert torch.equal(out.cpu(), expected_final)
    return out.cpu()


SMALL_CASES = [
    dict(tokens=7, hidden=512, inter=256, experts=5, top_k=3),
    dict(tokens=129, hidden=512, inter=512, experts=4, top_k=4, mask=True),
    dict(tokens=300, hidden=1024, inter=768, experts=16, top_k=2, layout="interleaved", biased=True),
    dict(tokens=64, hidden=256, inter=256, experts=3, top_k=1, dtype=torch.float16,
         ids_dtype=torch.int32),
]


@pytest.mark.parametrize("variant", ["cuda_core", "tensor_core", "tensor_core_gather"])
@pytest.mark.parametrize("spec", SMALL_CASES, ids=lambda s: "-".join(f"{k}{v}" for k, v in s.items()))
def test_stages_against_oracle(moe, spec, variant):
    case = make_case(**spec)
    staged = run_stages(moe, case, variant)
    full = moe.moe_ffn(**to_cuda(case), variant=variant).cpu()
    assert torch.equal(full, staged)
    exact = oracle.moe_ffn(**case, silu_table=gpu_silu_table(case["output_dtype"]))
    assert torch.equal(full, exact)
    expected = oracle.moe_ffn(**{k: v for k, v in case.items()})
    torch.testing.assert_close(full.float(), expected.float(), rtol=RTOL, atol=ATOL)
    if "token_mask" in case:
        assert full[~case["token_mask"]].abs().sum() == 0


@pytest.mark.parametrize("label,dtype", [("bf16", torch.bfloat16), ("fp16", torch.float16)])
@pytest.mark.parametrize("variant", ["cuda_core", "tensor_core"])
def test_reference_fixture_case(moe, label, dtype, variant):
    """The reference's own 7-token case (extrema weights, zero scales, repeated experts)."""
    case = load_golden(f"moe_small_{label}")
    tensors = dict(
        hidden_states=case["hidden_states"],
        w_gate_up=case["w_gate_up"].transpose(-2, -1).contiguous().transpose(-2, -1),
        w_down=case["w_down"].transpose(-2, -1).contiguous().transpose(-2, -1),
        topk_weights=case["topk_weights"], topk_ids=case["topk_ids"], scale_x=case["scale_x"],
        scale_gate_up=case["scale_gate_up"], scale_down=case["scale_down"])
    actual = moe.moe_ffn(**to_cuda(tensors), output_dtype=dtype, variant=variant).cpu()
    # The reference's own tolerance for its FP64-approximated CPU check ...
    torch.testing.assert_close(actual.float(), case["expected"], rtol=0.015, atol=0.025)
    # ... and the tighter bar against the exact-fmaf oracle.
    expected = oracle.moe_ffn(**tensors, output_dtype=dtype)
    torch.testing.assert_close(actual.float(), expected.float(), rtol=RTOL, atol=ATOL)
    mask = case["token_mask"].bool()
    masked = moe.moe_ffn(**to_cuda(tensors), token_mask=mask.cuda(), output_dtype=dtype,
                         variant=variant).cpu()
    torch.testing.assert_close(masked.float(), case["expected_masked"], rtol=0.015, atol=0.025)
    assert masked[~mask].abs().sum() == 0


def test_masked_rows_may_hold_nan_and_out_of_range_ids(moe):
    case = make_case(129, 512, 256, 4, 4, mask=True)
    masked = ~case["token_mask"]
    case["scale_x"][masked] = float("nan")
    case["topk_weights"][masked] = float("nan")
    case["topk_ids"][masked] = torch.tensor([2**40, -(2**40), 2**63 - 1, -(2**63)])
    actual = moe.moe_ffn(**to_cuda(case)).cpu()
    assert torch.isfinite(actual.float()).all()
    assert actual[masked].abs().sum() == 0
    expected = oracle.moe_ffn(**case)
    torch.testing.assert_close(actual.float(), expected.float(), rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("variant", ["cuda_core", "tensor_core"])
def test_all_tokens_masked_returns_zeros(moe, variant):
    case = make_case(70, 512, 256, 4, 2)
    case["token_mask"] = torch.zeros((70,), dtype=torch.bool)
    case["scale_x"][:] = float("nan")
    actual = moe.moe_ffn(**to_cuda(case), variant=variant).cpu()
    assert actual.shape == (70, 512) and actual.abs().sum() == 0


def test_unmasked_invalid_ids_raise(moe):
    case = make_case(8, 256, 256, 4, 2)
    case["topk_ids"][3, 1] = 4
    with pytest.raises(ValueError, match="topk_ids"):
        moe.moe_ffn(**to_cuda(case))


@pytest.mark.parametrize("layout", ["split", "interleaved"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fused_gate_up_equals_unfused_bits(moe, layout, dtype):
    """The fused epilogue divides with an FMA sequence, the stand-alone SwiGLU kernel with
    the library division; codes and scales must agree bit for bit, also for rows whose gate
    values are zero, huge (exp overflows, quotient -0) or far beyond the FMA sequence's range."""
    case = make_case(1500, 512, 1024, 6, 2, layout=layout, dtype=dtype, seed=11)
    case["scale_x"][0:40] = 0.0          # gate = up = 0
    case["scale_x"][40:80] *= 300.0      # |gate| in the hundreds: exp(-gate) overflows
    case["scale_x"][80:120] *= 1.0e-30   # tiny numerators
    case["scale_x"][120:160] *= 30.0     # around the range test of the FMA sequence
    dev = to_cuda(case)
    experts = case["w_gate_up"].shape[0]
    w1 = dev["w_gate_up"].transpose(-2, -1)
    results = []
    for tile_rows in (128, 32):
        routes = moe.prepare_routes(dev["topk_ids"], experts, None, tile_rows=tile_rows)
        qh, sh = moe.gate_up_swiglu_quantize(dev["hidden_states"], dev["scale_x"], w1,
                                             dev["scale_gate_up"], routes, output_dtype=dtype,
                                             gate_up_layout=layout)
        valid = int(routes.offsets[-1])
        results.append((qh[:valid].cpu(), sh[:valid].cpu()))
    assert torch.equal(results[0][0], results[1][0])
    assert torch.equal(results[0][1], results[1][1])
    assert results[0][0].abs().max() == 127


@pytest.mark.parametrize("hidden", [256, 512])
def test_fused_gate_up_many_items_per_cta_with_short_k(moe, hidden):
    """H = 256 / 512 gives one or two K groups per sub-tile, so a fast warp reaches the next
    work item while its partner half still reads the row maxima both exchange through shared
    memory; with several hundred work items every CTA walks several items back to back.
    Codes and scales must equal the unfused kernels' bit for bit."""
    case = make_case(12000, hidden, 512, 6, 2, seed=23)
    dev = to_cuda(case)
    w1 = dev["w_gate_up"].transpose(-2, -1)
    results = []
    for tile_rows in (128, 32):
        routes = moe.prepare_routes(dev["topk_ids"], 6, None, tile_rows=tile_rows)
        if tile_rows == 128:
            used = int((routes.tile_expert >= 0).sum())
            assert used * (512 // 256) > 300
        qh, sh = moe.gate_up_swiglu_quantize(dev["hidden_states"], dev["scale_x"], w1,
                                             dev["scale_gate_up"], routes)
        valid = int(routes.offsets[-1])
        results.append((qh[:valid].cpu(), sh[:valid].cpu()))
    assert torch.equal(results[0][0], results[1][0])
    assert torch.equal(results[0][1], results[1][1])


def test_row_gather_equals_presorted_rows_bits(moe):
    """The fused Gate/Up kernel fetching token rows by TMA row gathers from the original
    activations gives the bits of the default mode (rows copied into sorted order first), on a
    case with several row tiles per expert, ragged last tiles and masked tokens."""
    case = make_case(3000, 1024, 512, 7, 3, seed=31, mask=True)
    dev = to_cuda(case)
    default = moe.moe_ffn(**dev, variant="tensor_core")
    gathered = moe.moe_ffn(**dev, variant="tensor_core_gather")
    assert torch.equal(default, gathered)


def test_interleaved_equals_split_bits(moe):
    split = make_case(200, 512, 512, 6, 2, layout="split", seed=5)
    inter = make_case(200, 512, 512, 6, 2, layout="interleaved", seed=5)
    a = moe.moe_ffn(**to_cuda(split)).cpu()
    b = moe.moe_ffn(**to_cuda(inter)).cpu()
    assert torch.equal(a, b)


def check_against_oracle(actual, case):
    """Bit-exact against the oracle given the GPU's SiLU table, and within the stated
    tolerance of the oracle that evaluates SiLU with the host's expf."""
    dtype = case.get("output_dtype", torch.bfloat16)
    exact = oracle.moe_ffn(**case, silu_table=gpu_silu_table(dtype))
    assert torch.equal(actual, exact)
    expected = oracle.moe_ffn(**case)
    torch.testing.assert_close(actual.float(), expected.float(), rtol=RTOL, atol=ATOL)


def test_config_decode_small(moe):
    """T=512, H=2048, I=768, E=128, top-8, split layout, BF16."""
    case = make_case(512, 2048, 768, 128, 8)
    check_against_oracle(moe.moe_ffn(**to_cuda(case)).cpu(), case)


def test_config_interleaved_decode(moe):
    """H=4096, I=14336, E=8, top-2, T=16, one expert biased, interleaved layout."""
    case = make_case(16, 4096, 14336, 8, 2, layout="interleaved", biased=True)
    check_against_oracle(moe.moe_ffn(**to_cuda(case)).cpu(), case)


def sampled_token_case(case, tokens, experts):
    """The sub-problem of `tokens` (CPU tensors) on the experts those tokens use."""
    index = tokens.cuda()
    ids = case["topk_ids"][index].cpu()
    used = torch.unique(ids)
    remap = torch.full((experts,), -1, dtype=torch.int64)
    remap[used] = torch.arange(used.numel())
    return dict(
        hidden_states=case["hidden_states"][index].cpu(),
        scale_x=case["scale_x"][index].cpu(),
        topk_weights=case["topk_weights"][index].cpu(),
        topk_ids=remap[ids],
        w_gate_up=case["w_gate_up"][used.cuda()].cpu(),
        w_down=case["w_down"][used.cuda()].cpu(),
        scale_gate_up=case["scale_gate_up"][used.cuda()].cpu(),
        scale_down=case["scale_down"][used.cuda()].cpu(),
        gate_up_layout=case.get("gate_up_layout", "split"))


def test_config_interleaved_prefill_sampled_tokens(moe):
    """H=4096, I=14336, E=8, top-2, T=4096, one expert biased, interleaved layout: sampled
    tokens against the oracle, bit for bit."""
    import bench_moe

    case = bench_moe.make_case("interleaved_prefill", torch.device("cuda"))
    out = moe.moe_ffn(**case)
    tokens = torch.tensor([0, 1, 255, 2048, 3000, 4095])
    sub = sampled_token_case(case, tokens, 8)
    check_against_oracle(out[tokens.cuda()].cpu(), sub)
    counts = torch.bincount(case["topk_ids"].flatten().cpu(), minlength=8)
    assert counts[0] > 2 * counts[1:].float().mean()          # the biased expert is loaded more


def test_config_large_sampled_tokens_and_properties(moe):
    """T=16384, H=7168, I=2048, E=256, top-8 is far beyond the CPU oracle: check sampled tokens
    against it (on the experts those tokens use) and two size-independent properties:
    doubling every routing weight doubles the output exactly, and zero weights give zero."""
    import bench_moe

    case = bench_moe.make_case("large", torch.device("cuda"))
    out = moe.moe_ffn(**case)
    doubled = moe.moe_ffn(**{**case, "topk_weights": case["topk_weights"] * 2})
    assert torch.equal(doubled.float(), out.float() * 2)
    zeroed = moe.moe_ffn(**{**case, "topk_weights": torch.zeros_like(case["topk_weights"])})
    assert zeroed.abs().sum() == 0

    tokens = torch.tensor([0, 1, 4097, 8191, 12345, 16383])
    sub = sampled_token_case(case, tokens, 256)
    check_against_oracle(out[tokens.cuda()].cpu(), sub)


def test_graph_replay_with_changed_routes(moe):
    case = to_cuda(make_case(64, 512, 256, 8, 2))
    kwargs = {k: v for k, v in case.items()}
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(2):
            moe.moe_ffn(**kwargs)
    torch.cuda.current_stream().wait_stream(stream)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        captured = moe.moe_ffn(**kwargs)
    graph.replay()
    assert torch.equal(captured, moe.moe_ffn(**kwargs))
    case["topk_ids"].copy_((case["topk_ids"] + 3) % 8)
    graph.replay()
    assert torch.equal(captured, moe.moe_ffn(**kwargs))
