"""Model-level adapter for the SwiGLU path and its GeGLU sibling: ``patch(model)`` / ``unpatch(model)``.

Covers the part of the reference's ``forge.patch`` that calls this path
(forge/forge/patching/core.py:152-267 for the orchestration, qwen3.py:49-50 and gemma.py:31-32 for the class
mappings, kernels/basic.py:88-104 and :49-85 for the closures): every ``Qwen2MLP`` / ``Qwen3MLP`` instance of a
Hugging Face model gets the forward ``down_proj(swiglu(gate_proj(x), up_proj(x)))``, every ``GemmaMLP`` /
``Gemma2MLP`` the forward ``down_proj(geglu(gate_proj(x), up_proj(x), approximate))`` with the GELU form read
from the model's config, bound to the CUDA kernels of this package, with the original bound method kept for a
bit-exact ``unpatch``.  Book-keeping attributes
(``_forge_patched``, ``_forge_originals``, ``_forge_patched_counts``, ``_forge_arch``) and error types follow the
reference.  The other kernels of the reference's registry (rmsnorm, rope, embedding, cross entropy, LoRA)
are not part of this package; asking for them raises ``KeyError``.

``"lora_mlp"`` is the reference's adapter for PEFT-wrapped MLPs (kernels/lora.py:147-188): it accepts a module only
when its three projections carry an active, unmerged LoRA adapter without dropout, and then routes the activation
through ``swiglu`` / ``geglu`` while the wrapped projections compute their own adapter terms; any other module is left
to the next kernel in the list.  PEFT itself is not needed: the wrappers are recognised by their attributes
(``base_layer``, ``lora_A``, ``lora_B``, ``scaling``, ``lora_dropout``).  ``"lora_mlp_fused"`` (opt-in, not in the
reference's final mapping) goes further for bias-free bf16 MLPs, SiLU or GELU: the whole block runs through ``LoRAMLP`` of
``lora_mlp`` (projections, adapters and SwiGLU in one tcgen05 launch; hand-written backward).

One kernel is added that the reference does not have: ``"fused_gate_up"`` replaces the two projection GEMMs
and the activation by the single tcgen05 kernel of ``fused_mlp`` (SiLU) or ``geglu`` (GELU) when the module's
projections are plain bias-free bf16 ``nn.Linear`` layers (otherwise the module is left to the next kernel in the
list).  It is opt-in: ``patch(model, kernels=["fused_gate_up", "swiglu"])`` or ``[..., "geglu"]``.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional

import torch

from .fused_mlp import fused_gate_up_swiglu
from .geglu import FusedGateUpGEGLUFunction, geglu
from .swiglu import swiglu

# model_type -> (MLP class names, kernels tried by default)
ARCHITECTURES = {
    "qwen2": (("Qwen2MLP", "Qwen3MLP"), ("lora_mlp", "swiglu")),
    "qwen3": (("Qwen2MLP", "Qwen3MLP"), ("lora_mlp", "swiglu")),
    "gemma": (("GemmaMLP", "Gemma2MLP"), ("lora_mlp", "geglu")),
    "gemma2": (("GemmaMLP", "Gemma2MLP"), ("lora_mlp", "geglu")),
}
SUPPORTED_MODEL_TYPES = tuple(ARCHITECTURES)
GELU_EXACT = ("gelu", "gelu_python")
GELU_TANH = ("gelu_pytorch_tanh", "gelu_new")


class SkipPatch(Exception):
    """Raised by a forward factory that does not apply to a module; the next kernel is tried."""


def _model_config(model):
    config = getattr(model, "config", None)
    if config is None:
        inner = getattr(getattr(model, "base_model", None), "model", None)
        config = getattr(inner, "config", None)
    if config is None:
        raise ValueError("patch: model does not expose a Hugging Face config.")
    return config


def _activation_name(module) -> str:
    """``hidden_activation`` (Gemma) or ``hidden_act`` of the module's config; ``"silu"`` when it has neither."""
    cfg = getattr(module, "config", None)
    name = None
    if cfg is not None:
        name = getattr(cfg, "hidden_activation", None) or getattr(cfg, "hidden_act", None)
    return name or "silu"


def _gelu_form(module) -> str:
    """``"tanh"`` or ``"none"`` for ``geglu(..., approximate=...)``, inferred as the reference does
    (forge/forge/patching/kernels/basic.py:58-78)."""
    name = _activation_name(module)
    if name in GELU_EXACT:
        return "none"
    if name in GELU_TANH:
        return "tanh"
    raise NotImplementedError(f"patch: the geglu kernel cannot infer the GELU variant for hidden_activation={name!r}")


def make_swiglu_forward(module) -> Callable:
    if _activation_name(module) != "silu":
        raise NotImplementedError(
            f"patch: the swiglu kernel only supports activation='silu', got {_activation_name(module)!r}"
        )

    def forward(x):
        return module.down_proj(swiglu(module.gate_proj(x), module.up_proj(x)))

    return forward


def make_geglu_forward(module) -> Callable:
    approximate = _gelu_form(module)

    def forward(x):
        return module.down_proj(geglu(module.gate_proj(x), module.up_proj(x), approximate=approximate))

    return forward


def make_fused_gate_up_forward(module) -> Callable:
    act = _activation_name(module)
    if act != "silu" and act not in GELU_EXACT + GELU_TANH:
        raise SkipPatch
    for proj in (module.gate_proj, module.up_proj):
        if type(proj) is not torch.nn.Linear or proj.bias is not None or proj.weight.dtype != torch.bfloat16:
            raise SkipPatch
    n, k = module.gate_proj.weight.shape
    if k % 8 or n % 16:
        raise SkipPatch

    # weights are read at call time, so optimiser updates and .to() moves are seen
    if act == "silu":
        def forward(x):
            return module.down_proj(fused_gate_up_swiglu(x, module.gate_proj.weight, module.up_proj.weight))
    else:
        approximate = _gelu_form(module)

        def forward(x):
            return module.down_proj(
                FusedGateUpGEGLUFunction.apply(x, module.gate_proj.weight, module.up_proj.weight, approximate))

    return forward


def _active_adapter(linear):
    """Name of the LoRA adapter a PEFT-style wrapped linear would apply, or ``None``."""
    lora_a, lora_b = getattr(linear, "lora_A", None), getattr(linear, "lora_B", None)
    if not lora_a or not lora_b:
        return None
    active = getattr(linear, "active_adapters", None)
    if active is None:
        active = getattr(linear, "active_adapter", None)
    if callable(active):
        active = active()
    if isinstance(active, str):
        active = [active]
    for name in (active or list(lora_a.keys())):
        if name in lora_a and name in lora_b:
            return name
    return None


def _lora_parts(linear, allow_bias: bool = False):
    """``(W, A, B, scaling, bias)`` of a wrapped linear whose adapter can be applied exactly by a fused kernel
    (active, not merged, not disabled, no dropout); ``SkipPatch`` otherwise.  Same policy as the reference's
    ``_lora_tensors`` (forge/forge/patching/kernels/lora.py:54-79)."""
    name = _active_adapter(linear)
    if name is None or getattr(linear, "disable_adapters", False) or getattr(linear, "merged", False):
        raise SkipPatch
    base = getattr(linear, "base_layer", linear)
    bias = getattr(base, "bias", None)
    if bias is not None and not allow_bias:
        raise SkipPatch
    dropouts = getattr(linear, "lora_dropout", {})
    dropout = dropouts[name] if name in dropouts else None
    if dropout is not None and not isinstance(dropout, torch.nn.Identity) and float(getattr(dropout, "p", 0.0)) != 0.0:
        raise SkipPatch
    scaling = getattr(linear, "scaling", {})
    return base.weight, linear.lora_A[name].weight, linear.lora_B[name].weight, float(scaling.get(name, 1.0)), bias


def make_lora_mlp_forward(module) -> Callable:
    for proj in (module.gate_proj, module.up_proj, module.down_proj):
        _lora_parts(proj, allow_bias=True)
    act = _activation_name(module)
    if act == "silu":
        return make_swiglu_forward(module)
    if act in GELU_EXACT + GELU_TANH:
        return make_geglu_forward(module)
    raise SkipPatch


def make_lora_mlp_fused_forward(module) -> Callable:
    act = _activation_name(module)
    if act == "silu":
        activation = "silu"
    elif act in GELU_TANH:
        activation = "gelu_tanh"
    elif act in GELU_EXACT:
        activation = "gelu_exact"
    else:
        raise SkipPatch
    for proj in (module.gate_proj, module.up_proj, module.down_proj):
        w, a, b, _, _ = _lora_parts(proj)
        # LoRAMLP differentiates the adapters and the input only: the base weights must be frozen
        if not (w.dtype == a.dtype == b.dtype == torch.bfloat16) or w.requires_grad:
            raise SkipPatch
    from .lora_mlp import LoRAMLP

    # what the block does when its adapters cannot be folded in at call time: route through the (wrapped)
    # projections, as the reference's own patched forward does
    routed = make_swiglu_forward(module) if activation == "silu" else make_geglu_forward(module)

    def forward(x):
        # tensors are looked up at call time: optimiser steps, .to() moves and adapter switches are seen
        try:
            wg, ag, bg, sg, _ = _lora_parts(module.gate_proj)
            wu, au, bu, su, _ = _lora_parts(module.up_proj)
            wd, ad, bd, sd, _ = _lora_parts(module.down_proj)
        except SkipPatch:
            # adapters disabled or merged after patch() (e.g. inside PEFT's ``with model.disable_adapter():``)
            return routed(x)
        return LoRAMLP.apply(x, wg, ag, bg, sg, wu, au, bu, su, wd, ad, bd, sd, activation)

    return forward


FORWARD_MAKERS: Dict[str, Callable] = {
    "swiglu": make_swiglu_forward,
    "geglu": make_geglu_forward,
    "fused_gate_up": make_fused_gate_up_forward,
    "lora_mlp": make_lora_mlp_forward,
    "lora_mlp_fused": make_lora_mlp_fused_forward,
}


def patch(model, kernels: Optional[List[str]] = None):
    """Rebinds the MLP forwards of ``model`` in place and returns it.

    ``kernels``: ordered list of kernel names to try per MLP; the first whose factory accepts the module
    wins.  ``None`` means the reference's mapping: ``["lora_mlp", "swiglu"]`` for Qwen2 / Qwen3 (qwen3.py:49-50) and
    ``["lora_mlp", "geglu"]`` for Gemma / Gemma 2 (gemma.py:31-32).
    """
    if getattr(model, "_forge_patched", False):
        raise RuntimeError("Model already patched. Call unpatch(model) first.")
    model_type = getattr(_model_config(model), "model_type", None)
    if model_type not in SUPPORTED_MODEL_TYPES:
        raise ValueError(
            f"patch: no mapping for model_type={model_type!r}. Supported: {sorted(SUPPORTED_MODEL_TYPES)}."
        )
    mlp_classes, default_kernels = ARCHITECTURES[model_type]
    wanted = list(default_kernels if kernels is None else kernels)
    for name in wanted:  # validate before touching any module
        if name not in FORWARD_MAKERS:
            raise KeyError(f"patch: unknown kernel {name!r}. Known: {sorted(FORWARD_MAKERS)}.")

    originals: dict = {}
    counts: Dict[str, int] = {}
    for _name, module in model.named_modules():
        if type(module).__name__ not in mlp_classes:
            continue
        for name in wanted:
            try:
                new_forward = FORWARD_MAKERS[name](module)
            except SkipPatch:
                continue
            originals[id(module)] = (module, module.forward)
            module.forward = new_forward
            counts[name] = counts.get(name, 0) + 1
            break

    model._forge_originals = originals
    model._forge_patched = True
    model._forge_patched_counts = counts
    model._forge_arch = model_type
    return model


def unpatch(model):
    """Restores the original forwards; a no-op on a model that is not patched."""
    if not getattr(model, "_forge_patched", False):
        return model
    for module, original in model._forge_originals.values():
        module.forward = original
    for attr in ("_forge_originals", "_forge_patched", "_forge_patched_counts", "_forge_arch"):
        if hasattr(model, attr):
            delattr(model, attr)
    return model
