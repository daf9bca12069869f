"""Entry quantiser and weight preparation on the GPU, through the C ABI, against the oracle."""

import pytest
import torch

from oracle import cpu as oracle
from tests.conftest import load_golden

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def quantize():
    from grain_gemm_b200 import quantize as module
    return module


def test_reference_vectors(quantize):
    case = load_golden("quantizer_known")
    q, s = quantize.quantize_rows(case["x"].cuda())
    assert torch.equal(q.cpu(), case["q"])
    assert torch.equal(s.cpu(), case["s"])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("group", [32, 64, 128, 256])
def test_random_rows_bit_exact(quantize, dtype, group):
    gen = torch.Generator().manual_seed(group)
    x = (torch.randn((37, 3, 1024), generator=gen) * 3).to(dtype)
    x[0, 0, :256] = 0                         # all-zero group: scale 1e-12 / 127, codes 0
    x[1, 1, 5] = 1.0e30 if dtype != torch.float16 else 6.0e4
    x[2, 2, 256:512] = 1.0e-30 if dtype != torch.float16 else 6.0e-8
    q, s = quantize.quantize_rows(x.cuda(), group)
    expected_q, expected_s = oracle.quantize_rows(x, group)
    assert q.shape == x.shape and s.shape == (37, 3, 1024 // group)
    assert torch.equal(s.cpu(), expected_s)
    assert torch.equal(q.cpu(), expected_q)
    assert int(q.abs().max()) == 127


def test_ties_round_to_even_and_clamp(quantize):
    x = torch.zeros((1, 256))
    x[0, 0] = 127.0                            # scale exactly 1
    x[0, 1:7] = torch.tensor([0.5, 1.5, 2.5, -0.5, -1.5, -2.5])
    q, s = quantize.quantize_rows(x.cuda())
    assert s.item() == 1.0
    assert q[0, :7].tolist() == [127, 0, 2, 2, 0, -2, -2]


def test_empty_and_argument_errors(quantize):
    q, s = quantize.quantize_rows(torch.empty((0, 512), device="cuda"))
    assert q.shape == (0, 512) and s.shape == (0, 2)
    with pytest.raises(ValueError, match="multiple of 256"):
        quantize.quantize_rows(torch.zeros((4, 100), device="cuda"))
    with pytest.raises(ValueError, match="group_size"):
        quantize.quantize_rows(torch.zeros((4, 256), device="cuda"), 48)
    with pytest.raises(ValueError, match="contiguous"):
        quantize.quantize_rows(torch.zeros((256, 4), device="cuda").t())
    with pytest.raises(ValueError, match="float"):
        quantize.quantize_rows(torch.zeros((4, 256), dtype=torch.int8, device="cuda"))


def test_quantised_rows_feed_the_gemm(quantize):
    """Quantise activations and weights with the helpers and run int8_gemm on the result."""
    from grain_gemm_b200 import int8_gemm
    gen = torch.Generator().manual_seed(9)
    x = torch.randn((64, 512), generator=gen)
    weight = torch.randn((128, 512), generator=gen) / 512 ** 0.5      # Linear [N, K]
    qx, sx = quantize.quantize_rows(x.cuda())
    qw, sw = quantize.prepare_weight(weight.cuda())
    assert qw.shape == (512, 128) and qw.stride() == (1, 512) and sw.shape == (2, 128)
    out = int8_gemm(qx, qw, sx, sw, output_dtype=torch.float32)
    expected = oracle.int8_gemm(qx.cpu(), qw.cpu(), sx.cpu(), sw.cpu(), 256, torch.float32)
    assert torch.equal(out.cpu(), expected)
    torch.testing.assert_close(out.cpu(), x @ weight.t(), rtol=0.05, atol=0.05)


def test_prepare_weight_and_interleave(quantize):
    gen = torch.Generator().manual_seed(4)
    weight = torch.randn((3, 512, 256), generator=gen)                # [E, 2I, H]
    q, s = quantize.prepare_weight(weight.cuda())
    q_cpu, s_cpu = quantize.prepare_weight(weight)
    assert q.shape == (3, 256, 512) and q.stride() == (512 * 256, 1, 256)
    assert s.shape == (3, 1, 512) and s.is_contiguous()
    assert torch.equal(q.cpu(), q_cpu) and torch.equal(s.cpu(), s_cpu)
    qi, si = quantize.interleave_gate_up(q, s)
    inter = 256
    assert qi.stride() == q.stride()
    assert torch.equal(qi[..., 0::2], q[..., :inter]) and torch.equal(qi[..., 1::2], q[..., inter:])
    assert torch.equal(si[..., 0::2], s[..., :inter]) and torch.equal(si[..., 1::2], s[..., inter:])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("experts,top_k", [(8, 2), (128, 8), (256, 8), (1000, 6), (40, 40)])
def test_router_front_end(quantize, dtype, experts, top_k):
    gen = torch.Generator().manual_seed(experts + top_k)
    logits = (torch.randn((333, experts), generator=gen) * 2).to(dtype)
    logits[5, :] = 0.25                       # all tied: the lowest ids win, in order
    weights, ids = quantize.route_topk(logits.cuda(), top_k)
    expected_weights, expected_ids = oracle.router_topk(logits, top_k)
    assert torch.equal(ids.cpu(), expected_ids)
    assert ids[5].tolist() == list(range(top_k))
    torch.testing.assert_close(weights.cpu(), expected_weights, rtol=2e-6, atol=1e-9)
    torch.testing.assert_close(weights.sum(-1).cpu(), torch.ones(333), rtol=1e-6, atol=0)
    reference = torch.softmax(logits.float(), -1).gather(1, expected_ids)
    torch.testing.assert_close(weights.cpu(), reference / reference.sum(-1, keepdim=True),
                               rtol=1e-5, atol=1e-9)
    small, small_ids = quantize.route_topk(logits.cuda(), top_k, ids_dtype=torch.int32)
    assert small_ids.dtype == torch.int32 and torch.equal(small_ids.long().cpu(), expected_ids)


def test_router_output_feeds_moe_ffn(quantize):
    from grain_gemm_b200 import moe_ffn
    gen = torch.Generator().manual_seed(21)
    tokens, hidden, inter, experts, top_k = 50, 512, 256, 6, 2
    x, sx = quantize.quantize_rows(torch.randn((tokens, hidden), generator=gen).cuda())
    w1, s1 = quantize.prepare_weight((torch.randn((experts, 2 * inter, hidden), generator=gen) / hidden ** 0.5).cuda())
    w2, s2 = quantize.prepare_weight((torch.randn((experts, hidden, inter), generator=gen) / inter ** 0.5).cuda())
    weights, ids = quantize.route_topk(torch.randn((tokens, experts), generator=gen).cuda(), top_k)
    out = moe_ffn(x, w1, w2, weights, ids, scale_x=sx, scale_gate_up=s1, scale_down=s2)
    expected = oracle.moe_ffn(x.cpu(), w1.cpu(), w2.cpu(), weights.cpu(), ids.cpu(), scale_x=sx.cpu(),
                              scale_gate_up=s1.cpu(), scale_down=s2.cpu())
    torch.testing.assert_close(out.float().cpu(), expected.float(), rtol=1e-3, atol=1e-2)


@pytest.mark.parametrize("tokens,experts,top_k", [(16, 8, 2), (128, 128, 8), (100, 1000, 10),
                                                  (1024, 64, 1), (512, 128, 8)])
def test_router_and_routing_in_one_launch(quantize, tokens, experts, top_k):
    """Decode-sized problems run top-k and the routing sort in one kernel; ids, weights and all
    routing metadata equal those of the two separate calls (the last case is too large for the
    fused kernel and takes the two calls inside the helper)."""
    from grain_gemm_b200 import moe
    gen = torch.Generator().manual_seed(tokens + experts)
    logits = (torch.randn((tokens, experts), generator=gen) * 2).cuda()
    mask = (torch.rand((tokens,), generator=gen) > 0.2).cuda()
    for dtype in (torch.int64, torch.int32):
        weights, ids, routes = quantize.route_topk_routes(logits, top_k, token_mask=mask,
                                                          ids_dtype=dtype)
        expected_weights, expected_ids = quantize.route_topk(logits, top_k, ids_dtype=dtype)
        expected = moe.prepare_routes(expected_ids, experts, mask)
        assert torch.equal(ids, expected_ids) and torch.equal(weights, expected_weights)
        for field in ("order", "inverse", "counts", "offsets", "effective_ids", "statistics",
                      "tile_expert", "tile_row"):
            assert torch.equal(getattr(routes, field), getattr(expected, field)), field


def test_moe_ffn_accepts_prepared_routes(quantize):
    from grain_gemm_b200 import moe_ffn
    gen = torch.Generator().manual_seed(22)
    tokens, hidden, inter, experts, top_k = 60, 512, 256, 6, 2
    x, sx = quantize.quantize_rows(torch.randn((tokens, hidden), generator=gen).cuda())
    w1, s1 = quantize.prepare_weight((torch.randn((experts, 2 * inter, hidden), generator=gen) / hidden ** 0.5).cuda())
    w2, s2 = quantize.prepare_weight((torch.randn((experts, hidden, inter), generator=gen) / inter ** 0.5).cuda())
    logits = torch.randn((tokens, experts), generator=gen).cuda()
    weights, ids, routes = quantize.route_topk_routes(logits, top_k)
    plain = moe_ffn(x, w1, w2, weights, ids, scale_x=sx, scale_gate_up=s1, scale_down=s2)
    routed = moe_ffn(x, w1, w2, weights, ids, scale_x=sx, scale_gate_up=s1, scale_down=s2,
                     routes=routes)
    assert torch.equal(plain, routed)
