"""B200-native EXL3 fused dequant-matmul path behind the reference's linear-module API.

The package is a thin host side over ``libexl3b200.so`` (hand-written sm_100a CUDA
kernels behind a C ABI, see ``include/exl3_b200.h``).  Importing it needs no GPU;
calling any op needs the built library and a CUDA device — there is no fallback.
"""

from .layer import CodebookMode, EXL3Layer, codebook_mode_from_flags  # noqa: F401

__version__ = "0.1.0"


_LAZY = {
    "EXL3Linear": ".linear",
    "FusedEXL3Group": ".fused",
    "FusedEXL3Sibling": ".fused",
    "EXL3MLPMonolith": ".mlp",
    "EXL3SwitchGLU": ".moe",
    "EXL3MoEBlock": ".moe",
    "EXL3Gemma4MoEBlock": ".moe",
    "EXL3Checkpoint": ".loader",
    "load_exl3_layer": ".loader",
    "list_exl3_layers": ".loader",
}


def __getattr__(name: str):
    # torch-dependent modules load lazily so that `import ponyexl3_b200` stays cheap
    import importlib

    if name in _LAZY:
        return getattr(importlib.import_module(_LAZY[name], __name__), name)
    raise AttributeError(name)
