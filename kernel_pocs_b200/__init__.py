"""B200-native (sm_100a) implementation of the fused SwiGLU activation path of
Forge-researchlab/kernel-POCs (kernels/swiglu): hand-written CUDA kernels behind a C ABI,
with a host side that mirrors the reference's operator interface name for name."""
from .swiglu import ForgePackedSwiGLUFunction
from .swiglu import ForgeSwiGLUFunction
from .swiglu import swiglu
from .swiglu import swiglu_backward
from .swiglu import swiglu_forward
from .swiglu import swiglu_packed
from .swiglu import swiglu_packed_backward
from .swiglu import swiglu_packed_forward
from .swiglu import torch_swiglu_packed_reference
from .swiglu import torch_swiglu_reference

__all__ = [
    "ForgeSwiGLUFunction",
    "ForgePackedSwiGLUFunction",
    "swiglu",
    "swiglu_backward",
    "swiglu_forward",
    "swiglu_packed",
    "swiglu_packed_backward",
    "swiglu_packed_forward",
    "torch_swiglu_packed_reference",
    "torch_swiglu_reference",
]
