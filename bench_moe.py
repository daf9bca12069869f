"""Synthetic MoE FFN workloads and their timing (used by ``bench.py`` and the GPU tests).

Configurations: ``decode_small`` (T=512, H=2048, I=768, E=128, top-8,
split), ``interleaved_decode`` / ``interleaved_prefill`` (H=4096, I=14336, E=8, top-2, T=16 /
4096, one expert biased, interleaved gate/up) and ``large`` (T=16384, H=7168, I=2048, E=256,
top-8), the expert-parallel case, and ``large_rank_share`` (T=2048, E=32 of the same shape: the
experts and rows one rank of eight holds, small enough to profile).  All tensors are generated on the device from seeds, so that
every expert-parallel rank can materialise only its own experts: expert ``e`` always gets the
same weights whatever the world size.
"""

from __future__ import annotations

import torch

CONFIGS = {
    "decode_small": dict(tokens=512, hidden=2048, inter=768, experts=128, top_k=8,
                         layout="split", biased=False),
    "interleaved_decode": dict(tokens=16, hidden=4096, inter=14336, experts=8, top_k=2,
                               layout="interleaved", biased=True),
    "interleaved_prefill": dict(tokens=4096, hidden=4096, inter=14336, experts=8, top_k=2,
                                layout="interleaved", biased=True),
    "large": dict(tokens=16384, hidden=7168, inter=2048, experts=256, top_k=8,
                  layout="split", biased=False),
    "large_rank_share": dict(tokens=2048, hidden=7168, inter=2048, experts=32, top_k=8,
                             layout="split", biased=False),
}


def expert_weights(expert, hidden, inter, device, seed=2026):
    """INT8 weights and G256 scales of one expert: Linear W1 [2I,H], W2 [H,I]."""
    generator = torch.Generator(device=device).manual_seed(seed * 100003 + expert)
    w1 = torch.randint(-127, 128, (2 * inter, hidden), dtype=torch.int8, device=device,
                       generator=generator)
    w2 = torch.randint(-127, 128, (hidden, inter), dtype=torch.int8, device=device,
                       generator=generator)
    s1 = (0.5 + torch.rand((hidden // 256, 2 * inter), device=device, generator=generator)) \
        * (3.0 / hidden) ** 0.5 / 127
    s2 = (0.5 + torch.rand((inter // 256, hidden), device=device, generator=generator)) \
        * (3.0 / inter) ** 0.5 / 127
    return w1, w2, s1, s2


def make_weights(first_expert, num_experts, hidden, inter, device):
    w1 = torch.empty((num_experts, 2 * inter, hidden), dtype=torch.int8, device=device)
    w2 = torch.empty((num_experts, hidden, inter), dtype=torch.int8, device=device)
    s1 = torch.empty((num_experts, hidden // 256, 2 * inter), dtype=torch.float32, device=device)
    s2 = torch.empty((num_experts, inter // 256, hidden), dtype=torch.float32, device=device)
    for local in range(num_experts):
        w1[local], w2[local], s1[local], s2[local] = expert_weights(
            first_expert + local, hidden, inter, device)
    return w1, w2, s1, s2


TOKEN_BLOCK = 16


def make_tokens(first_token, num_tokens, hidden, experts, top_k, biased, device, seed=2026):
    """Quantised activations and routing of tokens [first_token, first_token + num_tokens).

    Tokens are generated in blocks of TOKEN_BLOCK from a seed that depends only on the block
    index, so a shard reproduces exactly the tokens the whole batch would hold."""
    if first_token % TOKEN_BLOCK or num_tokens % TOKEN_BLOCK:
        raise ValueError(f"token ranges must be multiples of {TOKEN_BLOCK}")
    x = torch.empty((num_tokens, hidden), dtype=torch.int8, device=device)
    scale_x = torch.empty((num_tokens, hidden // 256), dtype=torch.float32, device=device)
    logits = torch.empty((num_tokens, experts), dtype=torch.float32, device=device)
    generator = torch.Generator(device=device)
    for block in range(num_tokens // TOKEN_BLOCK):
        generator.manual_seed(seed * 7919 + first_token // TOKEN_BLOCK + block)
        rows = slice(block * TOKEN_BLOCK, (block + 1) * TOKEN_BLOCK)
        x[rows] = torch.randint(-127, 128, (TOKEN_BLOCK, hidden), dtype=torch.int8, device=device,
                                generator=generator)
        scale_x[rows] = (0.5 + torch.rand((TOKEN_BLOCK, hidden // 256), device=device,
                                          generator=generator)) / 127
        logits[rows] = torch.randn((TOKEN_BLOCK, experts), device=device, generator=generator)
    if biased:
        logits[:, 0] += 2
    weights, ids = torch.softmax(logits, dim=-1).topk(top_k, dim=-1)
    weights = (weights / weights.sum(-1, keepdim=True)).float().contiguous()
    return x, scale_x, weights, ids.contiguous()


def make_case(name, device, *, rank=0, world=1):
    """This rank's shard of a configuration: tokens T/world, experts E/world."""
    config = CONFIGS[name]
    tokens, experts = config["tokens"], config["experts"]
    if tokens % world or experts % world:
        raise ValueError(f"{name}: tokens and experts must divide by the world size {world}")
    local_tokens, local_experts = tokens // world, experts // world
    w1, w2, s1, s2 = make_weights(rank * local_experts, local_experts, config["hidden"],
                                  config["inter"], device)
    if config["layout"] == "interleaved":
        inter = config["inter"]
        order = torch.stack([torch.arange(inter), inter + torch.arange(inter)], 1).reshape(-1)
        order = order.to(device)
        w1 = w1[:, order].contiguous()
        s1 = s1[:, :, order].contiguous()
    x, scale_x, weights, ids = make_tokens(rank * local_tokens, local_tokens, config["hidden"],
                                           experts, config["top_k"], config["biased"], device)
    return dict(hidden_states=x, w_gate_up=w1.transpose(-2, -1), w_down=w2.transpose(-2, -1),
                topk_weights=weights, topk_ids=ids, scale_x=scale_x, scale_gate_up=s1,
                scale_down=s2, gate_up_layout=config["layout"])


def useful_ops(name):
    c = CONFIGS[name]
    return 6.0 * c["tokens"] * c["top_k"] * c["hidden"] * c["inter"]


def algorithmic_bytes(name, active_experts=None):
    """Byte model of one FFN pass: weights and scales of the experts touched, x, the INT8
    intermediate written and read, the expert outputs written and read, and the result."""
    c = CONFIGS[name]
    t, h, i, e, r = c["tokens"], c["hidden"], c["inter"], c["experts"], c["top_k"]
    s = t * r
    active = min(e, s) if active_experts is None else active_experts
    weights = active * 3 * h * i + 4 * active * (h // 256 * 2 * i + i // 256 * h)
    return weights + t * h + 4 * t * h // 256 + 2 * (s * i + 4 * s * i // 256) + 2 * 2 * s * h + 2 * t * h


def time_stages(case, steps, warmup):
    """Per-stage and total device time (ms per call) of the single-GPU FFN."""
    from grain_gemm_b200 import moe

    device = case["hidden_states"].device
    experts = case["w_gate_up"].shape[0]
    w1 = case["w_gate_up"].transpose(-2, -1)
    w2 = case["w_down"].transpose(-2, -1)
    events = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(steps)]

    def one(marks=None):
        if marks:
            marks[0].record()
        routes = moe.prepare_routes(case["topk_ids"], experts, None)
        if marks:
            marks[1].record()
        qh, sh = moe.gate_up_swiglu_quantize(case["hidden_states"], case["scale_x"], w1,
                                             case["scale_gate_up"], routes,
                                             gate_up_layout=case["gate_up_layout"])
        if marks:
            marks[2].record()
        eo = moe.down_projection(qh, sh, w2, case["scale_down"], routes)
        if marks:
            marks[3].record()
        out = moe.combine(eo, case["topk_weights"], routes)
        if marks:
            marks[4].record()
        return out

    for _ in range(warmup):
        one()
    torch.cuda.synchronize(device)
    for marks in events:
        one(marks)
    torch.cuda.synchronize(device)
    names = ["route", "gate_up", "down", "combine"]
    result = {}
    for index, stage in enumerate(names):
        times = sorted(marks[index].elapsed_time(marks[index + 1]) for marks in events)
        result[stage] = times[len(times) // 2]
    totals = sorted(marks[0].elapsed_time(marks[4]) for marks in events)
    result["total"] = totals[len(totals) // 2]
    return result
