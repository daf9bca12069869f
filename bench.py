"""Benchmark of the hot paths: prints ONE JSON line (rank 0).

Headline workload (N = 1): the W8A8 G256 GEMM at M = N = K = 8192 with BF16 output
(seeded synthetic INT8 operands uniform in [-127, 127], lognormal FP32 scales), metric
``g256_gemm_effective_int8_tops`` = 2*M*N*K / t.  A step is one GEMM over inputs resident in
HBM.  ``e2e`` is the same metric through the public ``int8_gemm`` call with HOST (pinned)
operands: every step's host-to-device copies of A, B and the scales and the device-to-host
read of C are inside the timed region; consecutive steps are pipelined over a copy-in, a
compute and a copy-out stream (two device buffer sets), so the rate is that of the slowest leg.

N > 1 (``torchrun``): the GEMM is sharded along N with no data-path collective (every rank
owns its own 8192-column block of B and of C; A and scale_a are replicated), weak scaling;
the MoE FFN timed beside it (``--moe-config``, reported under ``"moe"``) is expert-parallel:
token rows and results travel through peer memory from inside the dispatch and Down kernels
(``PeerExchange``), with the NCCL all-to-all path timed next to it (``nccl_all_to_all_ms``).
The ``moe`` block carries its own roofline, CPU baseline, end-to-end figure, per-phase times
and, at N > 1, a bit-identity check of the expert-parallel result against one GPU.

``reference_gpu_triton`` (N = 1, when ``oracle/make_ref.py`` has installed the reference beside
the oracle) times the reference's own Triton path on this GPU on the same operands: context for
what a B200 user of the reference gets today, outside every timed region of this library.

``--impl reference`` times the reference's CPU path for the same metric: the CPU oracle
(``oracle/``, a restatement of the reference's arithmetic; the reference ships no compiled
CPU implementation) on the whole workload, all host threads.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# DRAM traffic of one launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum
# from the ncu capture summarised in profiles/); None until a capture exists for the workload.
NCU_TRAFFIC_BYTES = {"gemm_g256_m8192_n8192_k8192_bf16": 250927360 + 119968000}


def parse():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    # 50 steps: the burst regime of the kernel timed alone (`roofline.peak` is the burst figure
    # too); the seconds-long rate under the power cap is reported beside it under `sustained`.
    parser.add_argument("--steps", type=int, default=50)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--moe-config", default="large",
                        help="MoE FFN configuration timed beside the GEMM ('none' skips it)")
    parser.add_argument("--moe-steps", type=int, default=10)
    parser.add_argument("--only-moe", action="store_true",
                        help="time only the MoE FFN and print its report as the JSON line")
    parser.add_argument("--m", type=int, default=8192)
    parser.add_argument("--n", type=int, default=8192)
    parser.add_argument("--k", type=int, default=8192)
    parser.add_argument("--group-size", type=int, default=256)
    parser.add_argument("--variant", default="auto")
    parser.add_argument("--skip-cpu-baseline", action="store_true")
    parser.add_argument("--skip-e2e", action="store_true")
    parser.add_argument("--sweep", action="store_true",
                        help="measure every tensor-core variant over the shape grid and write the "
                             "shape -> variant table the package loads (one GPU)")
    parser.add_argument("--sweep-output", default=str(ROOT / "grain_gemm_b200" / "configs"
                                                      / "b200_sm100_variants.json"))
    parser.add_argument("--skip-sustained", action="store_true")
    parser.add_argument("--skip-library-probe", action="store_true")
    parser.add_argument("--skip-reference-gpu", action="store_true",
                        help="do not time the reference's own Triton path on this GPU (context)")
    return parser.parse_args()


def reference_gpu_module():
    try:
        from oracle import make_ref
        return make_ref.load()
    except Exception:  # the reference is optional context
        return None


def time_calls(call, start, stop, warmup=3, steps=5):
    for _ in range(warmup):
        call()
    torch.cuda.synchronize()
    start.record()
    for _ in range(steps):
        call()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / steps


def reference_gpu_triton_gemm(a, b, scale_a, scale_b, g, start, stop):
    """The reference's int8_gemm(backend="triton") on the bench's own operands."""
    module = reference_gpu_module()
    if module is None:
        return None
    m, k = a.shape
    n = b.shape[1]
    try:
        ms = time_calls(lambda: module.int8_gemm(a, b, scale_a, scale_b, group_size=g,
                                                 output_dtype=torch.bfloat16, backend="triton"),
                        start, stop)
    except Exception as error:
        return {"gemm_unavailable": str(error).splitlines()[0][:200]}
    return {"gemm_ms_per_step": ms, "gemm_value": 2.0 * m * n * k / (ms * 1e-3) / 1e12,
            "gemm_unit": "TOPS", "note": "the reference's Triton backend on this GPU, same operands; "
                                         "context, not the reference arm"}


def reference_gpu_triton_moe(device, name="large_rank_share"):
    """Both libraries' moe_ffn on one expert-parallel rank's share of the large configuration:
    the reference addresses weights with 32-bit offsets and cannot hold all 256 experts."""
    module = reference_gpu_module()
    if module is None:
        return {}
    import bench_moe
    from grain_gemm_b200 import moe
    case = bench_moe.make_case(name, device)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    try:
        reference_ms = time_calls(lambda: module.moe_ffn(backend="triton", **case), start, stop)
    except Exception as error:
        return {"moe_unavailable": str(error).splitlines()[0][:200]}
    ours_ms = time_calls(lambda: moe.moe_ffn(**case), start, stop)
    tokens = case["hidden_states"].shape[0]
    return {"moe_config": name, "moe_ms_per_step": reference_ms,
            "moe_value": tokens / (reference_ms * 1e-3), "moe_unit": "tokens/s",
            "moe_this_library_ms_per_step": ours_ms}


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return dict(hbm_gbs=data["hbm_gbs"], bf16_tflops=data["bf16_tflops"],
                    bf16_tflops_sustained=data.get("bf16_tflops_sustained"), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.device_index = device_index
        self.process = None
        self.lines = []
        self.skip = 0

    def __enter__(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "20", "-i", str(self.device_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            # nvidia-smi needs a moment to start (longer on an 8-GPU box): wait for its first
            # line so that a short timed region is still sampled.
            deadline = time.time() + 5.0
            while not self.lines and time.time() < deadline:
                time.sleep(0.01)
            self.skip = len(self.lines)
        except OSError:
            self.process = None
        return self

    def _read(self):
        for line in self.process.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.process is not None:
            time.sleep(0.15)
            self.process.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        clocks, maxima, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        # Lines read before the timed region began describe an idle GPU; use them only when the
        # region was too short to be sampled at all.
        lines = self.lines[self.skip:] or self.lines
        for line in lines:
            fields = [f.strip() for f in line.split(",")]
            if len(fields) < 9:
                continue
            try:
                clocks.append(float(fields[1]))
                maxima.append(float(fields[2]))
            except ValueError:
                continue
            for name, value in zip(names, fields[5:9]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        clocks.sort()
        return {"sm_mhz": clocks[len(clocks) // 2], "sm_max_mhz": max(maxima),
                "reasons": sorted(reasons), "samples": len(clocks)}


def make_gemm_inputs(m, n, k, group, seed, device, weight_seed=None):
    """A [m,k] and scale_a from `seed`; Linear-format weights [n,k] and scale_b from
    `weight_seed` (so that ranks can share A and own different column blocks of B)."""
    groups = (k + group - 1) // group
    generator = torch.Generator(device=device).manual_seed(seed)
    a = torch.randint(-127, 128, (m, k), dtype=torch.int8, device=device, generator=generator)
    scale_a = torch.exp(-5 + 0.5 * torch.randn((m, groups), device=device, generator=generator))
    generator = torch.Generator(device=device).manual_seed(seed + 1 if weight_seed is None else weight_seed)
    w = torch.randint(-127, 128, (n, k), dtype=torch.int8, device=device, generator=generator)
    scale_b = torch.exp(-5 + 0.5 * torch.randn((groups, n), device=device, generator=generator))
    return a, w, scale_a, scale_b


def gemm_bytes(m, n, k, group, out_bytes=2):
    groups = (k + group - 1) // group
    return m * k + n * k + 4 * m * groups + 4 * groups * n + out_bytes * m * n


def use_all_host_threads():
    """The launcher of multi-rank runs exports OMP_NUM_THREADS=1; the CPU arms use every core.
    Must run before the oracle library (OpenMP) is loaded."""
    cores = os.cpu_count() or 1
    os.environ["OMP_NUM_THREADS"] = str(cores)
    torch.set_num_threads(cores)
    return cores


def cpu_gemm_sample(m, n, k, group, budget_seconds=10.0):
    """Times the CPU oracle on the workload, or on a row sample sized for about
    `budget_seconds` of work when the whole of it would take longer; returns
    (TOPS, seconds, rows, threads)."""
    use_all_host_threads()
    from oracle import cpu as oracle
    probe_rows = 8
    a, w, scale_a, scale_b = make_gemm_inputs(m, n, k, group, 2026, "cpu")
    b = w.t()
    start = time.perf_counter()
    oracle.int8_gemm(a[:probe_rows], b, scale_a[:probe_rows], scale_b, group, torch.bfloat16)
    probe = time.perf_counter() - start
    rows = int(max(probe_rows, min(a.shape[0], budget_seconds / max(probe, 1e-6) * probe_rows)))
    start = time.perf_counter()
    oracle.int8_gemm(a[:rows], b, scale_a[:rows], scale_b, group, torch.bfloat16)
    elapsed = time.perf_counter() - start
    return 2.0 * rows * n * k / elapsed / 1e12, elapsed, rows, oracle.threads()


def run_reference_arm(args, rank):
    """The reference's CPU path (oracle port) on a bounded sample, rank 0 only."""
    if rank != 0:
        return
    m, n, k, g = args.m, args.n, args.k, args.group_size
    samples = []
    for _ in range(max(1, min(args.steps, 3))):
        samples.append(cpu_gemm_sample(m, n, k, g, budget_seconds=30.0))
    samples.sort(key=lambda item: item[0])
    value, seconds, rows, threads = samples[len(samples) // 2]
    times = samples
    sample = (f"all {rows} rows" if rows == m else f"{rows} of {m} rows of A") + \
        f" against the full B (N={n}, K={k}); TOPS = 2*rows*N*K/t"
    line = {
        "impl": "reference", "metric": "g256_gemm_effective_int8_tops", "value": value,
        "unit": "TOPS", "n_gpus": args.gpus, "steps": len(times), "warmup": args.warmup,
        "ms_per_step": seconds * 1e3 * (m / rows), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": f"gemm_g{g}_m{m}_n{n}_k{k}_bf16", "sampled_rows": rows},
        "cpu_baseline": {"value": value, "unit": "TOPS", "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


class HostPipeline:
    """End-to-end loop with host operands: every step copies its inputs from pinned host memory,
    runs ``compute(device_inputs)`` through the public API and copies the result back.  The
    three legs of consecutive steps overlap (copy-in stream, compute stream, copy-out stream,
    two sets of device buffers), as a serving loop would run them: PCIe is full duplex, so the
    step rate is set by the slowest leg, not by the sum."""

    def __init__(self, host_inputs, host_out, compute, device):
        self.host_inputs, self.host_out, self.compute_fn, self.device = host_inputs, host_out, compute, device
        self.copy_in, self.copy_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
        self.sets = [dict(inputs=[torch.empty_like(t, device=device) for t in host_inputs],
                          loaded=torch.cuda.Event(), computed=torch.cuda.Event(),
                          drained=torch.cuda.Event(), result=None) for _ in range(2)]

    def step(self, index):
        buffers = self.sets[index % 2]
        compute = torch.cuda.current_stream(self.device)
        with torch.cuda.stream(self.copy_in):
            self.copy_in.wait_event(buffers["computed"])   # the set's previous step has read it
            for target, source in zip(buffers["inputs"], self.host_inputs):
                target.copy_(source, non_blocking=True)
            buffers["loaded"].record(self.copy_in)
        compute.wait_event(buffers["loaded"])
        compute.wait_event(buffers["drained"])             # the set's previous result has left
        result = self.compute_fn(buffers["inputs"])
        result.record_stream(self.copy_out)
        buffers["result"] = result
        buffers["computed"].record(compute)
        with torch.cuda.stream(self.copy_out):
            self.copy_out.wait_event(buffers["computed"])
            self.host_out.copy_(result, non_blocking=True)
            buffers["drained"].record(self.copy_out)

    def run(self, steps, first=0):
        for index in range(first, first + steps):
            self.step(index)
        compute = torch.cuda.current_stream(self.device)
        compute.wait_stream(self.copy_out)
        compute.wait_stream(self.copy_in)


# Per-launch DRAM traffic of the two MoE GEMM stages on the large configuration, scaled from the
# ncu captures of one rank's share (T = 2048, 32 experts; profiles/): traffic there is weight
# dominated and grows with the number of experts touched, i.e. by 8 for all 256 experts.
MOE_NCU_TRAFFIC_BYTES = {"large": {"gate_up": 8 * (1.145490e9 + 34.562816e6),
                                   "down": 8 * (539.494144e6 + 215.468032e6)}}


def cpu_moe_sample(name, case, device, experts_sampled=4):
    """Times the CPU oracle on the assignments of the first `experts_sampled` experts of the
    workload (their token rows through Gate/Up, SwiGLU, requantisation and Down), all host
    threads; returns (tokens/s equivalent, seconds, assignments, threads)."""
    use_all_host_threads()
    from oracle import cpu as oracle
    config = bench_moe_config(name)
    ids = case["topk_ids"].cpu()
    token, slot = torch.nonzero(ids < experts_sampled, as_tuple=True)
    if token.numel() == 0:
        return None
    sub = dict(
        hidden_states=case["hidden_states"][token.to(device)].cpu(),
        scale_x=case["scale_x"][token.to(device)].cpu(),
        topk_weights=torch.ones((token.numel(), 1)),
        topk_ids=ids[token, slot].reshape(-1, 1).long(),
        w_gate_up=case["w_gate_up"][:experts_sampled].cpu(),
        w_down=case["w_down"][:experts_sampled].cpu(),
        scale_gate_up=case["scale_gate_up"][:experts_sampled].cpu(),
        scale_down=case["scale_down"][:experts_sampled].cpu(),
        gate_up_layout=case.get("gate_up_layout", "split"))
    start = time.perf_counter()
    oracle.moe_ffn(**sub)
    seconds = time.perf_counter() - start
    assignments = int(token.numel())
    return assignments / config["top_k"] / seconds, seconds, assignments, oracle.threads()


def bench_moe_config(name):
    import bench_moe
    return bench_moe.CONFIGS[name]


def run_moe(args, rank, world, device, barrier):
    """Times the MoE FFN: single GPU at world == 1, expert parallel beyond (peer-memory exchange;
    the NCCL all-to-all path is timed beside it).  Returns the rank-0 report (None elsewhere)."""
    import torch.distributed as dist

    import bench_moe
    from grain_gemm_b200 import distributed, moe

    name = args.moe_config
    config = bench_moe.CONFIGS[name]
    case = bench_moe.make_case(name, device, rank=rank, world=world)
    local_tokens = config["tokens"] // world
    workspace = moe.MoEWorkspace()
    exchange, exchange_error = None, None
    if world > 1:
        # Peer mappings need CUDA IPC between the ranks' processes; where a host does not allow
        # it, every rank falls back to the NCCL all-to-all path together and the line says so.
        try:
            exchange = distributed.PeerExchange.create(
                dist.group.WORLD, capacity=local_tokens, hidden=config["hidden"],
                top_k=config["top_k"], local_experts=config["experts"] // world)
        except Exception as error:   # noqa: BLE001 - reported in the JSON line
            exchange_error = f"{type(error).__name__}: {error}"[:200]
        usable = torch.tensor([int(exchange is not None)], device=device)
        dist.all_reduce(usable, op=dist.ReduceOp.MIN)
        if not int(usable.item()) and exchange is not None:
            exchange.close()
            exchange = None

    def step(tensors, marks=None, nccl=False):
        if world == 1:
            return moe.moe_ffn(**tensors, workspace=workspace)
        return distributed.moe_ffn_expert_parallel(
            **tensors, num_experts=config["experts"], exchange=None if nccl else exchange,
            marks=marks)

    def timed(loop_steps, **kwargs):
        for _ in range(3):
            step(case, **kwargs)
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(loop_steps):
            step(case, **kwargs)
        stop.record()
        barrier()
        value = torch.tensor([start.elapsed_time(stop) / loop_steps], device=device)
        if world > 1:
            dist.all_reduce(value, op=dist.ReduceOp.MAX)
        return float(value.item())

    steps = max(1, args.moe_steps)
    with ClockSampler(device.index) as sampler:
        ms = timed(steps)
    nccl_ms = timed(steps, nccl=True) if world > 1 else None

    # Phase times of the expert-parallel step (rank 0's events; no extra synchronisation).
    phases = None
    if exchange is not None:
        names = ["plan_and_dispatch", "count_all_gather", "mask_and_route", "gather_and_gate_up",
                 "down_into_home_ranks", "results_home_all_reduce", "combine"]
        totals = [0.0] * len(names)
        for _ in range(steps):
            marks = []
            step(case, marks=marks)
            torch.cuda.synchronize()
            for index in range(len(names)):
                totals[index] += marks[index].elapsed_time(marks[index + 1])
        phases = {n: t / steps for n, t in zip(names, totals)}
        barrier()

    # Bit identity of the expert-parallel result with one GPU, on a problem small enough for
    # every rank to hold all experts (outside the timed regions).
    identical = None
    if world > 1:
        bench_moe.CONFIGS["ep_check"] = dict(tokens=768, hidden=1024, inter=512, experts=16, top_k=4,
                                             layout=config["layout"], biased=True)
        if 768 % world == 0 and 16 % world == 0:
            small = bench_moe.make_case("ep_check", device, rank=rank, world=world)
            whole = bench_moe.make_case("ep_check", device)
            rows = slice(rank * (768 // world), (rank + 1) * (768 // world))
            single = moe.moe_ffn(**whole)[rows]
            check = None
            if exchange is not None:
                check = distributed.PeerExchange.create(dist.group.WORLD, capacity=768 // world,
                                                        hidden=1024, top_k=4,
                                                        local_experts=16 // world)
            via_nccl = distributed.moe_ffn_expert_parallel(**small, num_experts=16)
            via_peers = via_nccl if check is None else distributed.moe_ffn_expert_parallel(
                **small, num_experts=16, exchange=check)
            same = torch.tensor([int(torch.equal(via_peers, single) and torch.equal(via_nccl, single))],
                                device=device)
            dist.all_reduce(same, op=dist.ReduceOp.MIN)
            identical = bool(same.item())
            barrier()
            if check is not None:
                check.close()

    # End to end: the per-token inputs come from pinned host memory, the result goes back.
    token_names = ("hidden_states", "scale_x", "topk_weights", "topk_ids")
    host = {n: case[n].cpu().pin_memory() for n in token_names}
    host_out = torch.empty(case["hidden_states"].shape, dtype=torch.bfloat16).pin_memory()

    def from_device_inputs(inputs):
        tensors = dict(case)
        tensors.update(zip(token_names, inputs))
        return step(tensors)

    pipeline = HostPipeline([host[n] for n in token_names], host_out, from_device_inputs, device)
    pipeline.run(2)
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    pipeline.run(steps, first=2)
    stop.record()
    barrier()
    e2e_elapsed = torch.tensor([start.elapsed_time(stop) / steps], device=device)
    if world > 1:
        dist.all_reduce(e2e_elapsed, op=dist.ReduceOp.MAX)
    # Same number of back-to-back calls as the timed loop, so that the stage sum and the call
    # time are taken at comparable clocks (the part is power-managed).
    stages = bench_moe.time_stages(case, steps=steps, warmup=3) if world == 1 else None
    cpu = None
    if rank == 0 and world == 1 and not args.skip_cpu_baseline:
        cpu = cpu_moe_sample(name, case, device)
    exchange_used = exchange is not None
    if exchange is not None:
        barrier()
        exchange.close()
    if rank != 0:
        return None
    e2e_ms = float(e2e_elapsed.item())
    tokens = config["tokens"]
    peaks = measured_peaks()
    int8_peak = 2.0 * peaks["bf16_tflops"]
    useful_tops = bench_moe.useful_ops(name) / (ms * 1e-3) / 1e12
    traffic = MOE_NCU_TRAFFIC_BYTES.get(name)
    roofline = {
        "bound": "tensor", "achieved": useful_tops / world, "peak": int8_peak, "unit": "TFLOP/s",
        "frac": useful_tops / world / int8_peak,
        "traffic": sum(traffic.values()) if traffic else None,
        "peak_source": f"2 x bf16_tflops burst ({peaks['source']}); MEASURED_PEAKS has no INT8 entry",
        "algorithmic_ops_per_step": bench_moe.useful_ops(name),
        "algorithmic_bytes_per_step": bench_moe.algorithmic_bytes(name),
        "hbm_time_floor_ms": bench_moe.algorithmic_bytes(name) / (peaks["hbm_gbs"] * 1e9) * 1e3 / world,
    }
    if stages is not None:
        t, r, h, i = config["tokens"], config["top_k"], config["hidden"], config["inter"]
        roofline["stage_frac"] = {
            "gate_up": 4.0 * t * r * h * i / (stages["gate_up"] * 1e-3) / 1e12 / int8_peak,
            "down": 2.0 * t * r * h * i / (stages["down"] * 1e-3) / 1e12 / int8_peak,
            "combine_hbm": (2.0 * t * r * h + 2.0 * t * h) / (stages["combine"] * 1e-3) / 1e9
            / peaks["hbm_gbs"],
        }
    report = {
        "metric": "moe_ffn_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": steps, "ms_per_step": ms, "scaling": "strong",
        "useful_tops": useful_tops,
        "config": {"workload": f"moe_{name}", **{k: v for k, v in config.items()},
                   "parallelism": "single" if world == 1 else
                   (f"ep{world}_peer_memory_exchange" if exchange_used else f"ep{world}_nccl_all_to_all")},
        "roofline": roofline, "clocks": sampler.summary(),
        "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s",
                "h2d_bytes_per_step": world * sum(t.numel() * t.element_size() for t in host.values()),
                "d2h_bytes_per_step": world * host_out.numel() * host_out.element_size(),
                "ms_per_step": e2e_ms},
        # route (3), tiles, statistics report, row copy, SiLU table, Gate/Up, Down, combine;
        # the expert-parallel step adds plan, dispatch, row mask and row destinations (its two
        # small copies into the report buffer and its two NCCL collectives are not counted).
        "gpu_launches_per_step": 10 if world == 1 else 14,
    }
    if stages is not None:
        report["stage_ms"] = stages
    if exchange_error is not None:
        report["peer_exchange_unavailable"] = exchange_error
    if phases is not None:
        report["phases_ms"] = phases
        report["nccl_all_to_all_ms"] = nccl_ms
        report["ep_bit_identical"] = identical
    if cpu is not None:
        value, seconds, assignments, threads = cpu
        report["cpu_baseline"] = {
            "value": value, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"{assignments} assignments (those of the first 4 experts) through Gate/Up, "
                      f"SwiGLU, requantisation and Down in {seconds:.2f} s; tokens = assignments / top_k"}
    return report


SWEEP_M = [1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192]
SWEEP_NK = [(8192, 8192), (4096, 4096), (4096, 7168), (7168, 2048), (28672, 4096), (4096, 14336)]
SWEEP_VARIANTS = ["tc_n256", "tc_n128", "tc_n64", "tc_pair_n256", "tc_pair_n128", "tc_splitk", "gemv"]


def run_sweep(args, device):
    """Times every variant on M x (N, K) x G and writes, per (G, N, K), the fastest variant for
    each M bucket (the table ``get_kernel_config`` / ``int8_gemm`` consult).  Launches are
    replayed from a CUDA graph, so that microsecond kernels are not timed by the host's launch
    rate, and walk through several copies of the weights (more than the L2 holds), as the
    layers of a model would."""
    from grain_gemm_b200 import _loader, gemm

    lib = _loader.library()
    shapes, timings = {}, {}
    side = torch.cuda.Stream(device)
    for g in (256, 128, 64, 32):
        for n, k in SWEEP_NK:
            rows = []
            copies = max(1, min(8, int(140e6 // (n * k)) + 1))
            weights = [make_gemm_inputs(1, n, k, g, 7 + c, device)[1] for c in range(copies)]
            for m in SWEEP_M:
                a, _, scale_a, scale_b = make_gemm_inputs(m, n, k, g, 7, device)
                out = torch.empty((m, n), dtype=torch.bfloat16, device=device)
                best = None
                for variant in SWEEP_VARIANTS:
                    if variant == "tc_splitk" and not lib.gg_int8_gemm_workspace_bytes(m, n, k, g):
                        continue
                    if variant.startswith("tc_pair") and m <= 128:
                        continue
                    if variant == "gemv" and m > 8:
                        continue
                    try:
                        for w in weights[:2]:
                            gemm.launch(a, w.t(), scale_a, scale_b, out, g, variant)
                    except RuntimeError:
                        continue
                    torch.cuda.synchronize()
                    rounds = max(1, (12 if m * n * k < 2 ** 36 else 3) // copies)
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.stream(side):
                        with torch.cuda.graph(graph, stream=side):
                            for _ in range(rounds):
                                for w in weights:
                                    gemm.launch(a, w.t(), scale_a, scale_b, out, g, variant)
                    graph.replay()
                    torch.cuda.synchronize()
                    start, stop = (torch.cuda.Event(enable_timing=True) for _ in range(2))
                    start.record()
                    graph.replay()
                    stop.record()
                    torch.cuda.synchronize()
                    microseconds = start.elapsed_time(stop) / (rounds * copies) * 1e3
                    del graph
                    timings[f"{g}:{n}:{k}:{m}:{variant}"] = round(microseconds, 2)
                    if best is None or microseconds < best[0]:
                        best = (microseconds, variant)
                if best is not None:
                    if rows and rows[-1][1] == best[1]:
                        rows[-1][0] = m
                    else:
                        rows.append([m, best[1]])
                del a, scale_a, scale_b, out
            del weights
            if rows:
                rows[-1][0] = 2 ** 31 - 1
                shapes[f"{g}:{n}:{k}"] = rows
    table = {"device": torch.cuda.get_device_name(device), "measured_with": "bench.py --sweep",
             "key": "G:N:K -> [[largest M, variant], ...] in ascending M", "shapes": shapes,
             "microseconds": timings}
    output = Path(args.sweep_output)
    output.parent.mkdir(parents=True, exist_ok=True)
    output.write_text(json.dumps(table, indent=1) + "\n")
    print(json.dumps({"sweep": str(output), "shapes": len(shapes), "timings": len(timings)}))


def main():
    args = parse()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    import torch.distributed as dist
    from grain_gemm_b200 import _loader, gemm

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.sweep:
        if world != 1:
            raise SystemExit("--sweep runs on one GPU")
        run_sweep(args, device)
        return

    if args.only_moe:
        report = run_moe(args, rank, world, device, barrier)
        if rank == 0:
            report.update({"warmup": 3, "higher_is_better": True, "vs_baseline": None,
                           "dtype": "int8", "data": "synthetic"})
            print(json.dumps(report))
        if world > 1:
            dist.destroy_process_group()
        return

    m, n, k, g = args.m, args.n, args.k, args.group_size
    # Rank r owns columns [r*n, (r+1)*n) of B, scale_b and C; A and scale_a are replicated.
    a, w, scale_a, scale_b = make_gemm_inputs(m, n, k, g, 2026, device, weight_seed=3000 + rank)
    b = w.t()
    out = torch.empty((m, n), dtype=torch.bfloat16, device=device)
    workload = f"gemm_g{g}_m{m}_n{n * world}_k{k}_bf16"

    def step():
        gemm.launch(a, b, scale_a, scale_b, out, g, args.variant)

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as sampler:
        barrier()
        start.record()
        for _ in range(args.steps):
            step()
        stop.record()
        barrier()
    elapsed_ms = start.elapsed_time(stop)
    if world > 1:
        reduced = torch.tensor([elapsed_ms], device=device)
        dist.all_reduce(reduced, op=dist.ReduceOp.MAX)
        elapsed_ms = float(reduced.item())
    ms_per_step = elapsed_ms / args.steps
    status = _loader.device_status(device)
    if status:
        raise SystemExit(f"a kernel reported device status {status:#x}")
    tops = 2.0 * m * n * world * k / (ms_per_step * 1e-3) / 1e12
    kernel_name = gemm.get_kernel_config(a, b, group_size=g)["variant"]

    # Sustained rate: at least two seconds of back-to-back launches, with its own clock record
    # (the part runs into its power limit; the burst figure above does not show that).
    sustained = None
    if not args.skip_sustained:
        sustained_steps = max(args.steps, int(2.2 / (ms_per_step * 1e-3)))
        with ClockSampler(local_rank) as sustained_sampler:
            barrier()
            start.record()
            for _ in range(sustained_steps):
                step()
            stop.record()
            barrier()
        sustained_ms = start.elapsed_time(stop)
        if world > 1:
            reduced = torch.tensor([sustained_ms], device=device)
            dist.all_reduce(reduced, op=dist.ReduceOp.MAX)
            sustained_ms = float(reduced.item())
        sustained_ms /= sustained_steps
        sustained = {"steps": sustained_steps, "ms_per_step": sustained_ms,
                     "value": 2.0 * m * n * world * k / (sustained_ms * 1e-3) / 1e12, "unit": "TOPS",
                     "clocks": sustained_sampler.summary()}

    # Same-box context: the library INT8 GEMM (cuBLASLt through torch._int_mm; INT32 output, no
    # scales, no promotion), a library call timed the same way.
    library_probe = None
    if world == 1 and m > 16 and not args.skip_library_probe:
        try:
            for _ in range(3):
                torch._int_mm(a, b)
            barrier()
            start.record()
            for _ in range(10):
                torch._int_mm(a, b)
            stop.record()
            barrier()
            probe_ms = start.elapsed_time(stop) / 10
            library_probe = {"call": "torch._int_mm", "ms_per_step": probe_ms,
                             "value": 2.0 * m * n * k / (probe_ms * 1e-3) / 1e12, "unit": "TOPS",
                             "note": "INT32 output, no group scales: context, not the same operator"}
        except RuntimeError as error:
            library_probe = {"call": "torch._int_mm", "unavailable": str(error).splitlines()[0][:200]}

    # Same-box context: what a B200 user of the reference gets today (its `auto` backend selects
    # its Triton kernels on compute capability 10.0).  Only when the reference is installed
    # beside the oracle; never part of a timed region of this library.
    reference_gpu = None
    if world == 1 and m > 16 and not args.skip_reference_gpu:
        reference_gpu = reference_gpu_triton_gemm(a, b, scale_a, scale_b, g, start, stop)

    # End to end through the public API with host operands.
    e2e = None
    if not args.skip_e2e:
        host = [t.cpu().pin_memory() for t in (a, w, scale_a, scale_b)]
        host_out = torch.empty((m, n), dtype=torch.bfloat16).pin_memory()
        h2d = sum(t.numel() * t.element_size() for t in host)
        d2h = host_out.numel() * host_out.element_size()

        pipeline = HostPipeline(
            host, host_out,
            lambda t: gemm.int8_gemm(t[0], t[1].t(), t[2], t[3], group_size=g,
                                     output_dtype=torch.bfloat16), device)
        e2e_steps = max(4, min(args.steps, 10))
        pipeline.run(2)
        barrier()
        start.record()
        pipeline.run(e2e_steps, first=2)
        stop.record()
        barrier()
        e2e_ms = start.elapsed_time(stop)
        if world > 1:
            reduced = torch.tensor([e2e_ms], device=device)
            dist.all_reduce(reduced, op=dist.ReduceOp.MAX)
            e2e_ms = float(reduced.item())
        e2e_ms /= e2e_steps
        e2e = {"value": 2.0 * m * n * world * k / (e2e_ms * 1e-3) / 1e12, "unit": "TOPS",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms}

    moe_result = None
    if args.moe_config != "none":
        del a, w, scale_a, scale_b, out
        torch.cuda.empty_cache()
        moe_result = run_moe(args, rank, world, device, barrier)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = measured_peaks()
    int8_peak = 2.0 * peaks["bf16_tflops"]
    per_gpu_tops = tops / world
    roofline = {
        "bound": "tensor", "achieved": per_gpu_tops, "peak": int8_peak, "unit": "TFLOP/s",
        "frac": per_gpu_tops / int8_peak,
        "traffic": NCU_TRAFFIC_BYTES.get(f"gemm_g{g}_m{m}_n{n}_k{k}_bf16"),
        "peak_source": f"2 x bf16_tflops burst ({peaks['source']}); MEASURED_PEAKS has no INT8 entry",
        "frac_of_nominal_4500": per_gpu_tops / 4500.0,
        "algorithmic_ops_per_launch": 2.0 * m * n * k,
        "algorithmic_bytes_per_launch": gemm_bytes(m, n, k, g),
        "kernel": kernel_name,
    }
    line = {
        "metric": "g256_gemm_effective_int8_tops", "value": tops, "unit": "TOPS", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic",
        "config": {"workload": workload, "group_size": g, "output": "bf16",
                   "sharding": "replicas" if world == 1 else f"n_sharded_x{world}",
                   "l2": "inputs_larger_than_l2 (A + B + C = 256 MiB per GPU, no flush)"},
        "roofline": roofline, "clocks": sampler.summary(), "gpu_launches": args.steps,
    }
    if e2e is not None:
        line["e2e"] = e2e
    if sustained is not None:
        if peaks.get("bf16_tflops_sustained"):
            sustained["frac_of_2x_bf16_sustained"] = (sustained["value"] / world
                                                      / (2.0 * peaks["bf16_tflops_sustained"]))
        mhz = sustained["clocks"].get("sm_mhz")
        sustained["ms_times_median_sm_mhz"] = sustained["ms_per_step"] * mhz if mhz else None
        line["sustained"] = sustained
    if library_probe is not None:
        line["int8_library_probe"] = library_probe
    if reference_gpu is not None:
        if world == 1 and args.moe_config != "none":
            reference_gpu.update(reference_gpu_triton_moe(device))
        line["reference_gpu_triton"] = reference_gpu
    if moe_result is not None:
        line["moe"] = moe_result
    if world == 1 and not args.skip_cpu_baseline:
        cpu_tops, seconds, rows, threads = cpu_gemm_sample(m, n, k, g)
        line["cpu_baseline"] = {
            "value": cpu_tops, "unit": "TOPS", "cores": threads, "kind": "port",
            "sample": (f"all {rows} rows" if rows == m else f"{rows} of {m} rows of A")
            + f" against the full B ({seconds:.2f} s)"}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
