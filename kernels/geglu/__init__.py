"""Drop-in import path for the GeGLU activation: ``from kernels.geglu import geglu`` resolves to the
sm_100a implementation.  Exports the fourteen names of the reference package
(kernels/geglu/__init__.py of Forge-researchlab/kernel-POCs)."""
from kernel_pocs_b200.geglu import ForgeGEGLUFunction
from kernel_pocs_b200.geglu import ForgePackedGEGLUFunction
from kernel_pocs_b200.geglu import geglu
from kernel_pocs_b200.geglu import geglu_backward
from kernel_pocs_b200.geglu import geglu_forward
from kernel_pocs_b200.geglu import geglu_mlp
from kernel_pocs_b200.geglu import geglu_packed
from kernel_pocs_b200.geglu import geglu_packed_backward
from kernel_pocs_b200.geglu import geglu_packed_forward
from kernel_pocs_b200.geglu import pack_geglu_gate_up_bias
from kernel_pocs_b200.geglu import pack_geglu_gate_up_weight
from kernel_pocs_b200.geglu import torch_geglu_mlp_reference
from kernel_pocs_b200.geglu import torch_geglu_packed_reference
from kernel_pocs_b200.geglu import torch_geglu_reference

__all__ = [
    "ForgeGEGLUFunction",
    "ForgePackedGEGLUFunction",
    "geglu",
    "geglu_backward",
    "geglu_forward",
    "geglu_mlp",
    "geglu_packed",
    "geglu_packed_backward",
    "geglu_packed_forward",
    "pack_geglu_gate_up_bias",
    "pack_geglu_gate_up_weight",
    "torch_geglu_mlp_reference",
    "torch_geglu_packed_reference",
    "torch_geglu_reference",
]
