"""W8A8 GEMM with per-row x per-column K-group scales: the ``grain_gemm.int8_gemm`` API on B200.

Same signature, validation order, exception types and messages as the reference's
``src/grain_gemm/gemm.py`` (``_validate`` :13-50, ``get_kernel_config`` :84-178, ``int8_gemm``
:181-220 there).  The dispatch collapses to one backend: hand-written sm_100a CUDA behind the
C ABI of ``libgrain_b200.so``.  There is no Triton path and no CPU fallback.
"""

from __future__ import annotations

import json
from functools import lru_cache
from pathlib import Path

import torch

from . import _loader

_TABLE = Path(__file__).resolve().parent / "configs" / "b200_sm100_variants.json"


@lru_cache(maxsize=1)
def _variant_table():
    """Measured shape -> variant table (``bench.py --sweep`` writes it), like the reference's
    per-GPU dispatch tables (``src/grain_gemm/gemm.py:53-69``, ``kernels/configs/*.json``).

    Keys are ``"G:N:K"``; each entry lists ``[m_upper_bound, variant]`` pairs in ascending
    order of M.  A missing file or shape leaves the choice to the library's own rule."""
    try:
        data = json.loads(_TABLE.read_text())
    except (OSError, ValueError):
        return {}
    return {key: [(int(bound), str(name)) for bound, name in rows]
            for key, rows in data.get("shapes", {}).items()}


def _table_variant(m, n, k, group_size):
    """Variant the measured table names for this shape, or None."""
    rows = _variant_table().get(f"{group_size}:{n}:{k}")
    if not rows:
        return None
    for bound, name in rows:
        if m <= bound:
            return name
    return rows[-1][1]

_BACKENDS = ("auto", "cuda")
_FOREIGN_BACKENDS = ("triton", "cutlass")


def _check_backend(backend):
    if backend in _FOREIGN_BACKENDS:
        raise ValueError(f"backend='{backend}' does not exist in the B200 build; "
                         "use 'auto' or 'cuda' (hand-written sm_100a kernels)")
    if backend not in _BACKENDS:
        raise ValueError("backend must be 'auto', 'triton', 'cuda', or 'cutlass'")


# Validation contract restated from the reference's src/grain_gemm/gemm.py:13-50 (Apache-2.0):
# same checks, order, exception types and messages, so callers and their tests port unchanged.
def _validate(a, b, scale_a, scale_b, group_size, output_dtype):
    if type(group_size) is not int or group_size not in (32, 64, 128, 256):
        raise ValueError("group_size must be one of 32, 64, 128, or 256")
    if output_dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise TypeError("output_dtype must be torch.float32, torch.float16, or torch.bfloat16")
    tensors = (("a", a), ("b", b), ("scale_a", scale_a), ("scale_b", scale_b))
    for name, tensor in tensors:
        if not isinstance(tensor, torch.Tensor):
            raise TypeError(f"{name} must be a torch.Tensor")
        if tensor.layout != torch.strided or tensor.ndim != 2:
            raise ValueError(f"{name} must be a two-dimensional strided tensor")
        expected = torch.int8 if name in ("a", "b") else torch.float32
        if tensor.dtype != expected:
            raise TypeError(f"{name} must have dtype {expected}")
    m, k = a.shape
    n = b.shape[1]
    if b.shape[0] != k:
        raise ValueError("a.shape[1] must equal b.shape[0] (the K dimension)")
    groups = (k + group_size - 1) // group_size
    for name, tensor, shape in (("scale_a", scale_a, (m, groups)),
                                ("scale_b", scale_b, (groups, n))):
        if tensor.shape != shape:
            raise ValueError(f"{name} must have shape {shape}, got {tuple(tensor.shape)}")
    for name, tensor in tensors:
        if tensor.device != a.device:
            raise ValueError(f"{name} must be on the same device as a ({a.device})")
        if tensor.device.type != "cuda":
            raise ValueError(f"{name} must be a CUDA tensor")
        if tensor.numel() and any(s <= 0 for s in tensor.stride()):
            raise ValueError(f"{name} must have positive strides")
        if tensor.numel() and sum((d - 1) * s for d, s in zip(tensor.shape, tensor.stride())) > 2**31 - 1:
            raise ValueError(f"{name} exceeds the supported 32-bit relative element offsets")
    if m * n > 2**31:
        raise ValueError("output exceeds the supported 32-bit relative element offsets")
    if torch.cuda.get_device_capability(a.device) != (10, 0):
        raise ValueError("this build of GrainGEMM requires an NVIDIA B200 (sm_100) GPU")
    return m, n, k


def _operand_strides(a, b):
    """Element strides of A [M,K] and B [K,N]; a dimension of size one is never stepped
    through, so its stride is replaced by one the tensor-core path accepts."""
    m, k = a.shape
    n = b.shape[1]
    a_sm, a_sk = a.stride()
    b_sk, b_sn = b.stride()
    if k == 1:
        a_sk = b_sk = 1
    if m == 1:
        a_sm = -(-(k * a_sk) // 16) * 16
    if n == 1:
        b_sn = -(-(k * b_sk) // 16) * 16
    return a_sm, a_sk, b_sk, b_sn


def _select(a, b, result, group_size, output_dtype):
    m, k = a.shape
    n = b.shape[1]
    return _loader.library().gg_int8_gemm_select(
        _loader.pointer(a), _loader.pointer(b), _loader.pointer(result), m, n, k,
        *_operand_strides(a, b),
        result.stride(0) if result is not None else n,
        group_size, _loader.OUT_DTYPE[output_dtype])


def get_kernel_config(a, b, *, group_size=256, output_dtype=torch.bfloat16,
                      scale_a=None, scale_b=None, backend="auto"):
    """Describe the kernel ``int8_gemm`` would launch, without launching it.

    Returns a dict with ``policy``, ``compute_capability``, ``backend`` and the
    tile description (``variant``, ``block_m``, ``block_n``, ``cta_group``), like the
    reference's ``get_kernel_config`` does for its own backends.
    """
    _check_backend(backend)
    capability = torch.cuda.get_device_capability(a.device)
    m, k = a.shape
    n = b.shape[1]
    repack_a, repack_b = _repack_plan(a, b)
    with torch.cuda.device(a.device):
        if repack_a or repack_b:
            # Describe the launch on the repacked (K-contiguous, aligned) operands.
            aligned = _loader._VOID(256)
            a_strides = (k, 1) if repack_a else a.stride()
            b_strides = (1, k) if repack_b else b.stride()
            variant = _loader.library().gg_int8_gemm_select(
                aligned if repack_a else _loader.pointer(a),
                aligned if repack_b else _loader.pointer(b), None, m, n, k,
                a_strides[0], a_strides[1], b_strides[0], b_strides[1], n, group_size,
                _loader.OUT_DTYPE[output_dtype])
        else:
            variant = _select(a, b, None, group_size, output_dtype)
    name = _loader.VARIANT_NAMES[variant]
    policy = "sm100_native"
    tabled = _table_variant(m, n, k, group_size)
    if tabled is not None and (name.startswith("tc") or name == "gemv"):
        name, policy = tabled, "sm100_table"
    pair = name.startswith("tc_pair")
    block_n = (256 if name == "tc_splitk" else int(name.split("_n", 1)[1].split("_")[0])
               if name.startswith("tc") else 8 if name == "gemv" else 32)
    block_m = ((256 if pair else 128) if name.startswith("tc") else 8 if name == "gemv" else 32)
    return dict(policy=policy, compute_capability=list(capability), backend="cuda",
                variant=name, block_m=block_m,
                block_n=block_n, cta_group=2 if pair else 1,
                tensor_cores=name.startswith("tc"), repacked_a=repack_a, repacked_b=repack_b)


_REPACK_MIN_OPS = 1 << 32


def _repack_plan(a, b):
    """(repack A?, repack B?) for the rule described in ``_tensor_core_operands``."""
    m, k = a.shape
    n = b.shape[1]
    if 2 * m * n * k < _REPACK_MIN_OPS or k % 16:
        return False, False
    return (a.stride(1) != 1 or a.stride(0) % 16 != 0 or a.data_ptr() % 16 != 0,
            b.stride(0) != 1 or b.stride(1) % 16 != 0 or b.data_ptr() % 16 != 0)


def _tensor_core_operands(a, b):
    """Operands in the layout the tensor-core path reads (K contiguous, 16-byte aligned rows).

    Any positive-stride view is accepted by the CUDA-core kernel, but that kernel is two orders
    of magnitude slower on large problems.  For those, an operand whose K direction is not
    contiguous (a row-major ``[K, N]`` B, a transposed A) or whose rows are not 16-byte aligned
    is copied once into K-contiguous storage; the arithmetic and the result do not change.
    """
    repack_a, repack_b = _repack_plan(a, b)
    if repack_a:
        a = a.contiguous()
    if repack_b:
        b = b.t().contiguous().t()
    return a, b


def _tc_ready(a, b):
    """Operands the tensor-core variants accept (K contiguous, 16-byte aligned rows)."""
    a_sm, a_sk, b_sk, b_sn = _operand_strides(a, b)
    k = a.shape[1]
    return (a_sk == 1 and b_sk == 1 and a_sm % 16 == 0 and b_sn % 16 == 0 and a_sm >= k
            and b_sn >= k and a.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0)


def launch(a, b, scale_a, scale_b, out, group_size, variant="auto"):
    """Launch the GEMM on torch's current stream (arguments already validated)."""
    m, k = a.shape
    n = b.shape[1]
    if variant == "auto":
        a, b = _tensor_core_operands(a, b)
        tabled = _table_variant(m, n, k, group_size)
        if tabled is not None and _tc_ready(a, b):
            variant = tabled
    lib = _loader.library()
    workspace, workspace_bytes = None, 0
    if variant in ("auto", "tc_splitk"):
        # Skinny problems split K over the SMs through a caller-owned INT32 workspace.
        workspace_bytes = lib.gg_int8_gemm_workspace_bytes(m, n, k, group_size)
        if workspace_bytes:
            workspace = torch.empty((workspace_bytes,), dtype=torch.uint8, device=a.device)
    status = lib.gg_int8_gemm_ws(
        _loader.pointer(a), _loader.pointer(b), _loader.pointer(scale_a), _loader.pointer(scale_b),
        _loader.pointer(out), m, n, k,
        *_operand_strides(a, b),
        scale_a.stride(0), scale_a.stride(1), scale_b.stride(0), scale_b.stride(1),
        out.stride(0), group_size, _loader.OUT_DTYPE[out.dtype], _loader.VARIANTS[variant],
        _loader.pointer(workspace), workspace_bytes, _loader.stream_pointer(a.device))
    _loader.check(status, "gg_int8_gemm")
    return out


def int8_gemm(a, b, scale_a, scale_b, *, group_size=256,
              output_dtype=torch.bfloat16, backend="auto", variant="auto"):
    """Compute INT8 A[M,K] @ B[K,N] with independent row/column K-group scales.

    FP32 scale shapes are [M, ceil(K/G)] and [ceil(K/G), N].  Each G-element dot product
    accumulates in INT32, then contributes to an FP32 scaled sum by one fused multiply-add
    per group; the result is cast once to BF16 (default), FP16 or FP32.  G can be
    32/64/128/256.  Positive-stride views and M/N/K tails are supported without packing:
    operands whose K direction is contiguous and 16-byte aligned run on the tensor cores,
    everything else on a CUDA-core kernel with identical arithmetic.  ``variant`` pins a
    kernel variant (see ``_loader.VARIANTS``) and is meant for tests and benchmarks.
    """
    _check_backend(backend)
    m, n, k = _validate(a, b, scale_a, scale_b, group_size, output_dtype)
    with torch.cuda.device(a.device):
        if m == 0 or n == 0 or k == 0:
            return torch.zeros((m, n), device=a.device, dtype=output_dtype)
        result = torch.empty((m, n), device=a.device, dtype=output_dtype)
        launch(a, b, scale_a, scale_b, result, group_size, variant)
    return result


def int8_gemm_partials(a, b, scale_a, scale_b, *, group_size=256):
    """Test aid: FP32 result and the INT32 group dots ``[M, N, ceil(K/G)]`` (CUDA cores)."""
    m, n, k = _validate(a, b, scale_a, scale_b, group_size, torch.float32)
    groups = (k + group_size - 1) // group_size
    with torch.cuda.device(a.device):
        result = torch.empty((m, n), device=a.device, dtype=torch.float32)
        partials = torch.empty((m, n, groups), device=a.device, dtype=torch.int32)
        status = _loader.library().gg_int8_gemm_partials(
            _loader.pointer(a), _loader.pointer(b), _loader.pointer(scale_a),
            _loader.pointer(scale_b), _loader.pointer(result), _loader.pointer(partials), m, n, k,
            a.stride(0), a.stride(1), b.stride(0), b.stride(1),
            scale_a.stride(0), scale_a.stride(1), scale_b.stride(0), scale_b.stride(1),
            group_size, _loader.stream_pointer(a.device))
        _loader.check(status, "gg_int8_gemm_partials")
    return result, partials
