"""Drop-in import path for the GeGLU activation: ``from kernels.geglu import geglu`` resolves to the
sm_100a implementation.  Exports the activation-level names of the reference package
(kernels/geglu/__init__.py of Forge-researchlab/kernel-POCs); its MLP-level helpers are not provided."""
from kernel_pocs_b200.geglu import ForgeGEGLUFunction
from kernel_pocs_b200.geglu import ForgePackedGEGLUFunction
from kernel_pocs_b200.geglu import geglu
from kernel_pocs_b200.geglu import geglu_backward
from kernel_pocs_b200.geglu import geglu_forward
from kernel_pocs_b200.geglu import geglu_packed
from kernel_pocs_b200.geglu import geglu_packed_backward
from kernel_pocs_b200.geglu import geglu_packed_forward
from kernel_pocs_b200.geglu import torch_geglu_packed_reference
from kernel_pocs_b200.geglu import torch_geglu_reference

__all__ = [
    "ForgeGEGLUFunction",
    "ForgePackedGEGLUFunction",
    "geglu",
    "geglu_backward",
    "geglu_forward",
    "geglu_packed",
    "geglu_packed_backward",
    "geglu_packed_forward",
    "torch_geglu_packed_reference",
    "torch_geglu_reference",
]
