"""Generate the golden fixtures in this folder from the reference project itself.

Run once, in a container that has the reference checked out; its location comes from the
environment:

    GRAIN_REFERENCE_DIR=<reference checkout> python tests/golden/make_golden.py

Two sources are used, both the reference's own code, unmodified:

* its CPU oracles in ``tests/test_int8_gemm.py`` (``inputs``, ``reference``) and
  ``tests/test_moe_ffn.py`` (``make_case``, ``reference``, ``quantize_rows_cpu``);
* its Triton kernels (``kernels/triton.py``, ``kernels/moe.py``) executed on CPU
  tensors by Triton's interpreter (``TRITON_INTERPRET=1``).  The interpreter's
  ``fma`` is an unfused multiply-add, so it is replaced here by an exact
  ``fmaf`` to keep the kernels' documented fused semantics; integer kernels
  (routing) need no patch.  The SwiGLU/requantisation and combine kernels call libdevice
  (``div_rn``, ``nearbyint``, ``exp``), which the interpreter cannot run: IEEE stand-ins on
  float32 arrays replace them (``libdevice_stand_ins``), and the fixture carries silu of every
  BF16 value as computed with them, so that a test can take the exponential out of the
  comparison.

``python tests/golden/make_golden.py stages`` (or ``gemm``, ``routing``, ``moe``) regenerates one
family.

The fixtures are small ``.npz`` files; the tests never need the reference.
"""

import os
import sys
from pathlib import Path

os.environ["TRITON_INTERPRET"] = "1"
if "GRAIN_REFERENCE_DIR" not in os.environ:
    raise SystemExit("set GRAIN_REFERENCE_DIR to the reference checkout")
REFERENCE = Path(os.environ["GRAIN_REFERENCE_DIR"])
sys.path.insert(0, str(REFERENCE / "src"))
sys.path.insert(0, str(REFERENCE / "tests"))
# Behind the reference on the path: this repository's optional `grain_gemm` drop-in package must
# not shadow the reference's package of the same name.
sys.path.append(str(Path(__file__).resolve().parents[2]))

import numpy as np
import torch

# The reference asks the device for its capability when choosing the routing
# variant; there is no device here, so answer as a B200 would.
torch.cuda.get_device_capability = lambda *args, **kwargs: (10, 0)

import triton.runtime.interpreter as interpreter
from oracle import cpu as oracle

HERE = Path(__file__).resolve().parent


def _exact_fma(self, x, y, z):
    result = oracle.fmaf(x.data, y.data, z.data)
    return interpreter.TensorHandle(result.reshape(np.broadcast(x.data, y.data, z.data).shape),
                                    x.dtype.scalar)


interpreter.InterpreterBuilder.create_fma = _exact_fma

import test_int8_gemm as ref_gemm_tests
import test_moe_ffn as ref_moe_tests
from grain_gemm.kernels import moe as ref_moe_kernels
from grain_gemm.kernels import triton as ref_triton

PORTABLE = dict(block_m=32, block_n=64, num_warps=4, num_stages=2, swizzle=8)


def save(name, **arrays):
    converted = {}
    for key, value in arrays.items():
        if isinstance(value, torch.Tensor):
            if value.dtype in (torch.bfloat16, torch.float16):
                value = value.float()
            value = value.contiguous().numpy()
        converted[key] = np.asarray(value)
    np.savez_compressed(HERE / f"{name}.npz", **converted)
    print("wrote", name, {k: v.shape for k, v in converted.items()})


def triton_gemm(a, b, sa, sb, group_size):
    out = torch.empty((a.shape[0], b.shape[1]), dtype=torch.float32)
    ref_triton.launch(a, b, sa, sb, out, group_size, PORTABLE)
    return out


def gemm_fixtures():
    cases = [(f"tails_g{g}", 19, 37, 2 * g + 13, g, "contiguous") for g in (32, 64, 128, 256)]
    cases += [("views_transposed", 33, 65, 269, 128, "transposed"),
              ("views_sliced", 33, 65, 269, 128, "sliced"),
              ("linear_weights", 64, 128, 768, 256, "column_major_b")]
    for name, m, n, k, g, layout in cases:
        a, b, sa, sb = ref_gemm_tests.inputs(m, n, k, g, layout=layout)
        expected = ref_gemm_tests.reference(a, b, sa, sb, g)
        fused = triton_gemm(a, b, sa, sb, g)
        save(f"gemm_{name}", a=a, b=b, scale_a=sa, scale_b=sb, group_size=g,
             reference_fp64=expected, triton_fp32=fused)
    # The cancellation case of the reference's tests: -1 + 4097 * f32(1/4097) = 2^-36
    # only when the scale product is rounded once and then fused into the sum.
    a = torch.zeros((32, 512), dtype=torch.int8)
    w = torch.zeros((64, 512), dtype=torch.int8)
    a[:, 0], w[:, 0] = -1, 1
    a[:, 256], w[:, 256] = 127, 32
    a[:, 257], w[:, 257] = 1, 33
    sa = torch.ones((32, 2))
    sb = torch.ones((2, 64))
    sb[1] = 1 / 4097
    save("gemm_cancellation", a=a, b=w.t(), scale_a=sa, scale_b=sb, group_size=256,
         triton_fp32=triton_gemm(a, w.t(), sa, sb, 256))


def routes_dict(routes):
    return dict(order=routes.order, inverse=routes.inverse, counts=routes.counts,
                offsets=routes.offsets, effective_ids=routes.effective_ids,
                statistics=routes.statistics)


def routing_fixtures():
    ids, mask = ref_moe_tests.routing_fixture_cpu()
    for dtype in (torch.int64,):
        routes = ref_moe_kernels.prepare_routes(ids.to(dtype), 5, mask, include_tiles=False)
        save("routes_mixed", ids=ids, mask=mask, experts=5, **routes_dict(routes))
    routes = ref_moe_kernels.prepare_routes(ids, 5, torch.zeros(4, dtype=torch.bool),
                                            include_tiles=False)
    save("routes_all_masked", ids=ids, mask=torch.zeros(4, dtype=torch.bool), experts=5,
         **routes_dict(routes))
    for experts, tokens in ((32, 1031), (64, 1031), (65, 1031)):
        ids = ((torch.arange(tokens, dtype=torch.int64) * 17 + 11) % experts).reshape(-1, 1)
        mask = torch.arange(tokens) % 11 != 0
        for token, value in ((1, 2**40), (255, -(2**40)), (256, experts),
                             (1024, 2**63 - 1), (1030, -(2**63))):
            ids[token, 0] = value
        routes = ref_moe_kernels.prepare_routes(ids, experts, mask, include_tiles=False)
        save(f"routes_e{experts}_t{tokens}", ids=ids, mask=mask, experts=experts,
             **routes_dict(routes))
    generator = torch.Generator().manual_seed(7)
    ids = torch.randint(0, 128, (300, 8), generator=generator, dtype=torch.int32)
    routes = ref_moe_kernels.prepare_routes(ids, 128, None, include_tiles=False)
    save("routes_e128_top8_int32", ids=ids, experts=128, **routes_dict(routes))


def moe_fixtures():
    for label, dtype in (("bf16", torch.bfloat16), ("fp16", torch.float16)):
        case = ref_moe_tests.make_case(dtype=dtype, device="cpu")
        expected = ref_moe_tests.reference(case)
        masked = dict(case)
        masked["token_mask"] = torch.tensor([True, False, True, True, False, True, True])
        expected_masked = ref_moe_tests.reference(masked)
        arrays = {k: v for k, v in case.items() if isinstance(v, torch.Tensor)}
        # Gathered ragged Gate/Up GEMM through the reference's Triton kernel.  FP32 output:
        # the interpreter truncates FP32 -> BF16 instead of rounding to nearest even.
        routes = ref_moe_kernels.prepare_routes(case["topk_ids"], 5, None, include_tiles=True)
        w1 = case["w_gate_up"].transpose(-2, -1)
        gate_up = ref_moe_kernels.ragged_gemm(
            case["hidden_states"], w1, case["scale_x"], case["scale_gate_up"], routes,
            output_dtype=torch.float32, source_is_token=True)
        save(f"moe_small_{label}", expected=expected, expected_masked=expected_masked,
             token_mask=masked["token_mask"], triton_gate_up=gate_up,
             triton_order=routes.order, triton_offsets=routes.offsets, **arrays)
    # Activation quantiser known answers (ties to even, all-zero group, clamp).
    x = torch.zeros((4, 512))
    x[:, 0] = 127
    x[:, 256] = 127
    x[0, 1:7] = torch.tensor([0.5, 1.5, 2.5, -0.5, -1.5, -2.5])
    x[1, 256:] = 0
    x[2, 5] = -300
    q, s = ref_moe_tests.quantize_rows_cpu(x)
    save("quantizer_known", x=x, q=q, s=s)


def libdevice_stand_ins():
    """The stage kernels call libdevice (``div_rn``, ``exp``, ``nearbyint``), which the interpreter
    cannot run.  Stand-ins with the same IEEE meaning on float32 numpy arrays: a correctly
    rounded division, round-half-even, and the interpreter's own ``tl.exp``."""
    import triton.language as tl

    def elementwise(function):
        def call(*operands, _semantic=None, **unused):
            arrays = [o.handle.data if isinstance(o, tl.tensor) else np.float32(o) for o in operands]
            first = next(o for o in operands if isinstance(o, tl.tensor))
            result = np.asarray(function(*arrays), dtype=np.float32)
            return tl.tensor(interpreter.TensorHandle(result, tl.float32), first.type)
        return call

    ref_moe_kernels.libdevice.div_rn = elementwise(
        lambda a, b: np.divide(np.asarray(a, np.float32), np.asarray(b, np.float32)))
    ref_moe_kernels.libdevice.nearbyint = elementwise(np.rint)
    ref_moe_kernels.libdevice.exp = elementwise(
        lambda x: np.exp(np.asarray(x, np.float32)))


def interpreter_silu_table():
    """silu of every BF16 value with the operations the stand-ins use (numpy's float32 ``exp``,
    not libdevice's): entry b = g / (1 + exp(-g)) for the value with bit
    pattern b.  Handing this table to the oracle removes the one library call the two sides
    cannot share and leaves everything else of the stage to be compared bit for bit."""
    bits = np.arange(65536, dtype=np.uint32) << 16
    gate = bits.view(np.float32)
    with np.errstate(over="ignore", invalid="ignore"):
        return (gate / (np.float32(1) + np.exp(-gate))).astype(np.float32)


def stage_fixtures():
    """The reference's ``swiglu_quantize`` and ``combine`` Triton kernels (kernels/moe.py:564-601,
    634-653) under the interpreter, on inputs of their own (BF16 gate/up rows, BF16 expert
    outputs), both layouts, ragged routes with an empty expert and masked tokens."""
    libdevice_stand_ins()
    generator = torch.Generator().manual_seed(11)
    tokens, top_k, experts, inter, hidden = 37, 3, 6, 512, 256
    ids = torch.randint(0, experts - 1, (tokens, top_k), generator=generator)   # expert 5 empty
    mask = torch.rand((tokens,), generator=generator) > 0.2
    routes = ref_moe_kernels.prepare_routes(ids, experts, mask, include_tiles=False)
    slots = tokens * top_k
    gate_up = (3.0 * torch.randn((slots, 2 * inter), generator=generator)).to(torch.bfloat16)
    gate_up[0, :8] = torch.tensor([0.0, -0.0, 1.0, -1.0, 20.0, -20.0, 88.0, -88.0]).to(torch.bfloat16)
    gate_up[1, :inter] = 0                         # a row whose activations are all zero
    table = interpreter_silu_table()
    arrays = dict(ids=ids, mask=mask, experts=experts, gate_up=gate_up, silu_table=table,
                  offsets=routes.offsets, inverse=routes.inverse)
    for layout in ("split", "interleaved"):
        q, scales = ref_moe_kernels.swiglu_quantize(gate_up, routes=routes, gate_up_layout=layout)
        arrays[f"q_{layout}"] = q
        arrays[f"scale_{layout}"] = scales
    expert_out = torch.randn((slots, hidden), generator=generator).to(torch.bfloat16)
    weights = torch.rand((tokens, top_k), generator=generator)
    # FP32 output: the interpreter truncates FP32 -> BF16 instead of rounding to nearest even.
    combined = ref_moe_kernels.combine(expert_out, weights, routes, output_dtype=torch.float32)
    save("moe_stages", expert_out=expert_out, topk_weights=weights, combined_fp32=combined, **arrays)


if __name__ == "__main__":
    only = sys.argv[1:]
    for name, make in (("gemm", gemm_fixtures), ("routing", routing_fixtures), ("moe", moe_fixtures),
                       ("stages", stage_fixtures)):
        if not only or name in only:
            make()
