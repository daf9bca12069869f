"""GrainGEMM's two hot paths on NVIDIA B200: ``int8_gemm`` and ``moe_ffn``.

The public names match the reference package (``src/grain_gemm/__init__.py:4`` there);
attributes are resolved lazily so that importing the package does not import torch.
"""

__version__ = "0.1.0"
__all__ = ["__version__", "get_kernel_config", "int8_gemm", "moe_ffn", "quantize_rows",
           "prepare_weight", "interleave_gate_up", "route_topk", "route_topk_routes"]


def __getattr__(name):
    if name in ("int8_gemm", "get_kernel_config"):
        from . import gemm
        return getattr(gemm, name)
    if name == "moe_ffn":
        from .moe import moe_ffn
        return moe_ffn
    if name in ("quantize_rows", "prepare_weight", "interleave_gate_up", "route_topk",
                "route_topk_routes"):
        from . import quantize
        return getattr(quantize, name)
    raise AttributeError(f"module 'grain_gemm_b200' has no attribute '{name}'")
