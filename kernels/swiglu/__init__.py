"""Drop-in import path: ``from kernels.swiglu import swiglu`` resolves to the sm_100a
implementation, with the same ten public names the reference package exports
(kernels/swiglu/__init__.py:1-23 of Forge-researchlab/kernel-POCs)."""
from kernel_pocs_b200.swiglu import ForgePackedSwiGLUFunction
from kernel_pocs_b200.swiglu import ForgeSwiGLUFunction
from kernel_pocs_b200.swiglu import swiglu
from kernel_pocs_b200.swiglu import swiglu_backward
from kernel_pocs_b200.swiglu import swiglu_forward
from kernel_pocs_b200.swiglu import swiglu_packed
from kernel_pocs_b200.swiglu import swiglu_packed_backward
from kernel_pocs_b200.swiglu import swiglu_packed_forward
from kernel_pocs_b200.swiglu import torch_swiglu_packed_reference
from kernel_pocs_b200.swiglu import torch_swiglu_reference

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
