"""The C-ABI library loads without a GPU and exports what include/grain_gemm_b200.h declares."""

import ctypes
import re
from pathlib import Path

import pytest
import torch

import grain_gemm_b200
from grain_gemm_b200 import _loader, build

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def library():
    build.build_library()
    return _loader.library()


def declared_functions():
    text = (ROOT / "include" / "grain_gemm_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"\b((?:gg|grain)_[a-z0-9_]+)\s*\(", text))


def test_header_and_binding_agree(library):
    declared = declared_functions()
    assert declared == set(_loader.EXPORTS)
    raw = ctypes.CDLL(str(build.LIBRARY))
    for name in declared:
        assert hasattr(raw, name), name


def test_abi_version_and_error_strings(library):
    assert library.gg_abi_version() == build.ABI_VERSION
    assert library.gg_error_string(0) == b"success"
    assert b"invalid" in library.gg_error_string(1)
    assert b"CUresult 1" in library.gg_error_string(-10001)
    assert library.grain_cuda_error_string(0) == b"success"


def test_host_side_size_queries(library):
    assert library.gg_moe_tile_capacity(4096, 128, 128) == 4096 // 128 + 128
    assert library.gg_moe_tile_capacity(1, 5, 32) == 6
    assert library.gg_moe_route_workspace_bytes(16, 2, 8) == 0
    chunks = (512 * 8 + 1023) // 1024
    assert library.gg_moe_route_workspace_bytes(512, 8, 128) == chunks * 130 * 4


def test_null_pointers_are_rejected_before_any_launch(library):
    """Argument errors come back as cudaErrorInvalidValue (1) from the host-side checks, for
    the single-CTA routing path too (it once reached its kernel with NULL outputs)."""
    null = ctypes.c_void_p(0)
    fake = ctypes.c_void_p(256)     # never dereferenced: the call fails on the NULL arguments
    for tokens, top_k in ((4, 2), (1024, 1), (2048, 8)):
        assert library.gg_moe_route(null, 0, null, tokens, top_k, 8, fake, fake, fake, fake, fake,
                                    fake, null, 0, null) == 1
        assert library.gg_moe_route(fake, 0, null, tokens, top_k, 8, fake, null, fake, fake, fake,
                                    fake, null, 0, null) == 1
        assert library.gg_moe_route_noalloc(fake, 0, null, tokens, top_k, 8, fake, fake, null, fake,
                                            fake, fake, null) == 1
    assert library.gg_moe_combine(null, fake, fake, fake, 4, 2, 256, 1, null) == 1
    assert library.gg_selftest_wait_timeout(0, fake, null) == 1
    assert library.gg_moe_silu_table(null, 1, null) == 1
    assert library.gg_moe_silu_table(fake, 0, null) == 1
    assert library.gg_report_to_host(null, 3, fake, null) == 1
    assert library.gg_report_to_host(fake, 3, null, null) == 1
    assert library.gg_report_to_host(fake, 1025, fake, null) == 1
    assert library.gg_report_to_host(null, 0, null, null) == 0      # nothing to report


def test_stale_library_is_refused(library, monkeypatch):
    monkeypatch.setattr(build, "source_hashes", lambda: {"abi.cu": "different"})
    _loader.library.cache_clear()
    try:
        with pytest.raises(RuntimeError, match="does not match"):
            _loader.library()
        assert not _loader.is_available()
    finally:
        monkeypatch.undo()
        _loader.library.cache_clear()
    assert _loader.is_available()


def test_public_names():
    assert set(grain_gemm_b200.__all__) >= {"int8_gemm", "get_kernel_config", "moe_ffn"}
    assert callable(grain_gemm_b200.int8_gemm) and callable(grain_gemm_b200.moe_ffn)
    with pytest.raises(AttributeError):
        grain_gemm_b200.nothing


# ---- argument contract of the public API that needs no device (reference: gemm.py:13-50) ----

def _cpu_gemm_args():
    a = torch.zeros((4, 64), dtype=torch.int8)
    b = torch.zeros((64, 8), dtype=torch.int8)
    return a, b, torch.ones((4, 2)), torch.ones((2, 8))


def test_gemm_argument_errors_without_a_device():
    from grain_gemm_b200 import int8_gemm
    a, b, sa, sb = _cpu_gemm_args()
    with pytest.raises(ValueError, match="backend"):
        int8_gemm(a, b, sa, sb, group_size=32, backend="fastest")
    with pytest.raises(ValueError, match="does not exist"):
        int8_gemm(a, b, sa, sb, group_size=32, backend="triton")
    with pytest.raises(ValueError, match="group_size"):
        int8_gemm(a, b, sa, sb, group_size=48)
    with pytest.raises(ValueError, match="group_size"):
        int8_gemm(a, b, sa, sb, group_size=True)
    with pytest.raises(TypeError, match="output_dtype"):
        int8_gemm(a, b, sa, sb, group_size=32, output_dtype=torch.float64)
    with pytest.raises(TypeError, match="dtype"):
        int8_gemm(a.float(), b, sa, sb, group_size=32)
    with pytest.raises(ValueError, match="K dimension"):
        int8_gemm(a, b[:32], sa, sb, group_size=32)
    with pytest.raises(ValueError, match="scale_a must have shape"):
        int8_gemm(a, b, sa[:, :1], sb, group_size=32)
    with pytest.raises(ValueError, match="two-dimensional"):
        int8_gemm(a[0], b, sa, sb, group_size=32)
    with pytest.raises(ValueError, match="CUDA"):
        int8_gemm(a, b, sa, sb, group_size=32)


def test_moe_argument_errors_without_a_device():
    from grain_gemm_b200 import moe_ffn
    t, h, i, e, r = 3, 256, 256, 4, 2
    case = dict(
        hidden_states=torch.zeros((t, h), dtype=torch.int8),
        w_gate_up=torch.zeros((e, 2 * i, h), dtype=torch.int8).transpose(-2, -1),
        w_down=torch.zeros((e, h, i), dtype=torch.int8).transpose(-2, -1),
        topk_weights=torch.ones((t, r)),
        topk_ids=torch.zeros((t, r), dtype=torch.int64),
        scale_x=torch.ones((t, 1)),
        scale_gate_up=torch.ones((e, 1, 2 * i)),
        scale_down=torch.ones((e, 1, h)),
    )
    with pytest.raises(ValueError, match="group_size=256"):
        moe_ffn(**case, group_size=128)
    with pytest.raises(ValueError, match="swiglu"):
        moe_ffn(**case, activation="gelu")
    with pytest.raises(ValueError, match="gate_up_layout"):
        moe_ffn(**case, gate_up_layout="packed")
    with pytest.raises(ValueError, match="output_dtype"):
        moe_ffn(**case, output_dtype=torch.float32)
    bad = dict(case, topk_ids=torch.zeros((t, e + 1), dtype=torch.int64),
               topk_weights=torch.ones((t, e + 1)))
    with pytest.raises(ValueError, match="top-k"):
        moe_ffn(**bad)
    with pytest.raises(ValueError, match="CUDA"):
        moe_ffn(**case)


def test_measured_variant_table_is_well_formed():
    """The shipped shape -> variant table: known variant names, ascending M bounds that end
    open, one entry per (G, N, K) key, and the weight-streaming kernel only where it can run."""
    import json
    from pathlib import Path
    table = json.loads((Path(grain_gemm_b200.__file__).parent / "configs"
                        / "b200_sm100_variants.json").read_text())
    assert table["shapes"]
    for key, rows in table["shapes"].items():
        group, n, k = (int(part) for part in key.split(":"))
        assert group in (32, 64, 128, 256) and n > 0 and k > 0
        bounds = [bound for bound, _ in rows]
        assert bounds == sorted(bounds) and len(set(bounds)) == len(bounds)
        assert bounds[-1] == 2 ** 31 - 1
        for bound, name in rows:
            assert name in _loader.VARIANTS and name != "auto", (key, name)
            if name == "gemv":
                assert bound <= 8 and k % 16 == 0, (key, bound)
            if name == "tc_splitk":
                assert bound <= 32, (key, bound)
