"""Model-level drop-in: patch()/unpatch() on a randomly initialised tiny Qwen3 (no checkpoint needed).

CPU tests cover the orchestration (what gets rebound, book-keeping, error types, bit-exact unpatch);
the GPU tests apply the acceptance criteria of the reference's verify_patch_qwen3.py:186-201 to the
logits of the patched model -- NaN-free, same shape, max-abs difference < 1.0, cosine > 0.999 -- and its
requirement that unpatch restores the original outputs bit for bit (:219-225), plus gradient agreement in
the spirit of verify_qwen_patch_backward.py:187-204 (loss difference and gradient cosine).
"""
import pytest
import torch

from kernel_pocs_b200 import _lib, patching

transformers = pytest.importorskip("transformers")


def tiny_qwen3(dtype=torch.float32, device="cpu", layers=2):
    cfg = transformers.Qwen3Config(
        vocab_size=512, hidden_size=128, intermediate_size=384, num_hidden_layers=layers, num_attention_heads=4,
        num_key_value_heads=2, head_dim=32, max_position_embeddings=128, tie_word_embeddings=False,
    )
    torch.manual_seed(0)
    return transformers.Qwen3ForCausalLM(cfg).to(device=device, dtype=dtype)


def tiny_gemma2(dtype=torch.float32, device="cpu", layers=2, act="gelu_pytorch_tanh"):
    cfg = transformers.Gemma2Config(
        vocab_size=512, hidden_size=128, intermediate_size=384, num_hidden_layers=layers, num_attention_heads=4,
        num_key_value_heads=2, head_dim=32, max_position_embeddings=128, hidden_activation=act,
    )
    torch.manual_seed(0)
    return transformers.Gemma2ForCausalLM(cfg).to(device=device, dtype=dtype)


class FakeLoraLinear(torch.nn.Module):
    """A linear layer wrapped the way PEFT's LoRA wraps it, as far as patch() looks: ``base_layer`` (frozen),
    ``lora_A`` / ``lora_B`` module dicts keyed by adapter name, ``scaling`` and ``lora_dropout`` dicts, the
    ``merged`` / ``disable_adapters`` flags and ``active_adapters``."""

    def __init__(self, base: torch.nn.Linear, r: int = 8, alpha: float = 16.0, dropout: float = 0.0, name="default"):
        super().__init__()
        self.base_layer = base
        base.weight.requires_grad_(False)
        self.lora_A = torch.nn.ModuleDict({name: torch.nn.Linear(base.in_features, r, bias=False)})
        self.lora_B = torch.nn.ModuleDict({name: torch.nn.Linear(r, base.out_features, bias=False)})
        torch.nn.init.normal_(self.lora_B[name].weight, std=0.05)  # non-zero, so that the adapters matter
        self.scaling = {name: alpha / r}
        self.lora_dropout = torch.nn.ModuleDict(
            {name: torch.nn.Dropout(dropout) if dropout else torch.nn.Identity()})
        self.active_adapters = [name]
        self.merged = False
        self.disable_adapters = False

    def forward(self, x):
        a = self.active_adapters[0]
        if self.disable_adapters:
            return self.base_layer(x)
        return self.base_layer(x) + self.scaling[a] * self.lora_B[a](self.lora_A[a](self.lora_dropout[a](x)))


def wrap_mlps(model, **kw):
    torch.manual_seed(1)
    for m in model.modules():
        if type(m).__name__.endswith("MLP"):
            for proj in ("gate_proj", "up_proj", "down_proj"):
                setattr(m, proj, FakeLoraLinear(getattr(m, proj), **kw))
    return model


def test_lora_wrapped_mlps_take_the_lora_kernel():
    model = wrap_mlps(tiny_qwen3())
    patching.patch(model)
    assert model._forge_patched_counts == {"lora_mlp": 2}
    patching.unpatch(model)
    # adapters that a fused path could not apply exactly (dropout, merged) leave the module to the next kernel
    model = wrap_mlps(tiny_qwen3(), dropout=0.1)
    patching.patch(model)
    assert model._forge_patched_counts == {"swiglu": 2}
    patching.unpatch(model)
    model = wrap_mlps(tiny_qwen3())
    next(m for m in model.modules() if type(m).__name__ == "Qwen3MLP").up_proj.merged = True
    patching.patch(model)
    assert model._forge_patched_counts == {"lora_mlp": 1, "swiglu": 1}
    patching.unpatch(model)
    # the one-launch kernel takes bf16 only: fp32 wrappers fall through
    model = wrap_mlps(tiny_qwen3())
    patching.patch(model, kernels=["lora_mlp_fused", "lora_mlp", "swiglu"])
    assert model._forge_patched_counts == {"lora_mlp": 2}
    gemma = wrap_mlps(tiny_gemma2())
    patching.patch(gemma)
    assert gemma._forge_patched_counts == {"lora_mlp": 2}


def test_gemma_mlps_get_the_geglu_forward():
    model = tiny_gemma2()
    mlps = [m for m in model.modules() if type(m).__name__ == "Gemma2MLP"]
    patching.patch(model)
    assert model._forge_arch == "gemma2" and model._forge_patched_counts == {"geglu": len(mlps)} and len(mlps) == 2
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        model(torch.randint(0, 512, (1, 8)))
    patching.unpatch(model)
    ids = torch.randint(0, 512, (1, 8))
    assert torch.equal(model(ids).logits, tiny_gemma2()(ids).logits)
    # the GELU form comes from the config; an activation that is not a GELU is refused
    assert patching._gelu_form(mlps[0]) == "tanh"
    assert patching._gelu_form([m for m in tiny_gemma2(act="gelu").modules() if type(m).__name__ == "Gemma2MLP"][0]) == "none"
    odd = tiny_gemma2(act="relu")
    with pytest.raises(NotImplementedError, match="cannot infer the GELU variant"):
        patching.patch(odd)


def test_patch_rebinds_every_mlp_and_unpatch_restores_them():
    model = tiny_qwen3()
    mlps = [m for m in model.modules() if type(m).__name__ == "Qwen3MLP"]
    originals = [m.forward for m in mlps]
    assert patching.patch(model) is model
    assert model._forge_patched and model._forge_arch == "qwen3"
    assert model._forge_patched_counts == {"swiglu": len(mlps)} and len(mlps) == 2
    assert all(m.forward is not o for m, o in zip(mlps, originals))
    with pytest.raises(RuntimeError, match="already patched"):
        patching.patch(model)
    # the patched forward reaches the CUDA-only operator: on CPU tensors it must refuse, not compute
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        model(torch.randint(0, 512, (1, 8)))
    patching.unpatch(model)
    assert not hasattr(model, "_forge_patched") and not hasattr(model, "_forge_originals")
    assert all(m.forward == o for m, o in zip(mlps, originals))
    ids = torch.randint(0, 512, (1, 8))
    assert torch.equal(model(ids).logits, tiny_qwen3()(ids).logits)
    assert patching.unpatch(model) is model  # idempotent


def test_patch_validates_before_mutating():
    model = tiny_qwen3()
    with pytest.raises(KeyError, match="unknown kernel"):
        patching.patch(model, kernels=["swiglu", "rmsnorm"])
    assert not getattr(model, "_forge_patched", False)
    model.config.model_type = "gpt2"
    with pytest.raises(ValueError, match="no mapping for model_type"):
        patching.patch(model)
    # fp32 projections are not eligible for the fused GEMM: the module falls through to swiglu
    model = tiny_qwen3()
    patching.patch(model, kernels=["fused_gate_up", "swiglu"])
    assert model._forge_patched_counts == {"swiglu": 2}


@pytest.mark.gpu
def test_fused_lora_forward_survives_adapters_disabled_after_patching():
    """``with model.disable_adapter():`` after patch(): the one-launch LoRA forward can no longer fold the adapters
    in, so it must route through the wrapped projections (like the reference's own patched forward) instead of
    letting its skip signal escape from ``module.forward``."""
    model = wrap_mlps(tiny_qwen3(layers=2)).to(device="cuda", dtype=torch.bfloat16)
    ids = torch.randint(0, 512, (2, 32), device="cuda", generator=torch.Generator(device="cuda").manual_seed(2))
    wrappers = [m for m in model.modules() if isinstance(m, FakeLoraLinear)]
    for w in wrappers:
        w.disable_adapters = True
    with torch.no_grad():
        want = model(ids).logits
    for w in wrappers:
        w.disable_adapters = False
    patching.patch(model, kernels=["lora_mlp_fused", "swiglu"])
    assert model._forge_patched_counts == {"lora_mlp_fused": 2}
    with torch.no_grad():
        with_adapters = model(ids).logits
    for w in wrappers:
        w.disable_adapters = True
    with torch.no_grad():
        got = model(ids).logits
    assert float((got.float() - want.float()).abs().max()) < 1.0
    assert float(torch.nn.functional.cosine_similarity(got.float().flatten(), want.float().flatten(), dim=0)) > 0.999
    assert not torch.equal(got, with_adapters)


@pytest.mark.gpu
@pytest.mark.parametrize("make,kernels,expected", [
    (tiny_qwen3, None, "swiglu"), (tiny_qwen3, ["fused_gate_up", "swiglu"], "fused_gate_up"),
    (tiny_gemma2, None, "geglu"), (tiny_gemma2, ["fused_gate_up", "geglu"], "fused_gate_up"),
    (lambda *a, **k: tiny_gemma2(*a, act="gelu", **k), ["fused_gate_up", "geglu"], "fused_gate_up"),
    (lambda dtype, device, layers: wrap_mlps(tiny_qwen3(layers=layers)).to(device=device, dtype=dtype), None, "lora_mlp"),
    (lambda dtype, device, layers: wrap_mlps(tiny_qwen3(layers=layers)).to(device=device, dtype=dtype),
     ["lora_mlp_fused", "swiglu"], "lora_mlp_fused"),
    (lambda dtype, device, layers: wrap_mlps(tiny_gemma2(layers=layers)).to(device=device, dtype=dtype), None, "lora_mlp"),
    (lambda dtype, device, layers: wrap_mlps(tiny_gemma2(layers=layers)).to(device=device, dtype=dtype),
     ["lora_mlp_fused", "geglu"], "lora_mlp_fused"),
    (lambda dtype, device, layers: wrap_mlps(tiny_gemma2(layers=layers, act="gelu")).to(device=device, dtype=dtype),
     ["lora_mlp_fused", "geglu"], "lora_mlp_fused"),
])
def test_patched_logits_and_gradients_match(make, kernels, expected):
    model = make(torch.bfloat16, "cuda", layers=3)
    ids = torch.randint(0, 512, (4, 64), device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))

    def run():
        model.zero_grad(set_to_none=True)
        out = model(ids, labels=ids)
        out.loss.backward()
        grads = torch.cat([p.grad.float().flatten() for p in model.parameters() if p.grad is not None])
        return out.logits.detach().clone(), out.loss.detach().clone(), grads

    base_logits, base_loss, base_grads = run()
    launches = _lib.launch_count() + _lib.lib.swiglu_b200_gemm_launch_count()
    patching.patch(model, kernels=kernels)
    assert model._forge_patched_counts == {expected: 3}
    logits, loss, grads = run()
    assert _lib.launch_count() + _lib.lib.swiglu_b200_gemm_launch_count() > launches, "no kernel of this library ran"
    assert logits.shape == base_logits.shape and bool(torch.isfinite(logits).all())
    assert float((logits.float() - base_logits.float()).abs().max()) < 1.0
    cos = torch.nn.functional.cosine_similarity(logits.float().flatten(), base_logits.float().flatten(), dim=0)
    assert float(cos) > 0.999
    assert abs(float(loss) - float(base_loss)) <= 2e-2
    assert float(torch.nn.functional.cosine_similarity(grads, base_grads, dim=0)) >= 0.999
    patching.unpatch(model)
    again_logits, _, _ = run()
    assert torch.equal(again_logits, base_logits)
