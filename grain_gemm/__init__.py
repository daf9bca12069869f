"""Optional drop-in name: ``import grain_gemm`` resolves to the B200 build.

The reference package is called ``grain_gemm`` (``src/grain_gemm/__init__.py:3-17`` there) and
exports ``int8_gemm``, ``get_kernel_config``, ``moe_ffn`` and ``__version__`` lazily.  Code
written against it keeps working unchanged when this directory is on ``sys.path`` instead of
the reference: every public name is forwarded to ``grain_gemm_b200``.  Do not install both.
"""

import grain_gemm_b200 as _implementation

__version__ = _implementation.__version__
__all__ = list(_implementation.__all__)


def __getattr__(name):
    if name in __all__:
        return getattr(_implementation, name)
    raise AttributeError(f"module 'grain_gemm' has no attribute {name!r}")
