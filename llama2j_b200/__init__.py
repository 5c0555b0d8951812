"""B200-native drop-in for llama2j's `--mode CUDA` token-decode path.

The package is a thin host layer over libl2j_b200.so (hand-written sm_100a kernels behind a C ABI,
include/l2j_b200.h).  There is no CPU compute path in here.
"""
from .model_files import ModelConfig  # noqa: F401
from .layer_allocation import LayerAllocation  # noqa: F401

__all__ = ["ModelConfig", "LayerAllocation"]
