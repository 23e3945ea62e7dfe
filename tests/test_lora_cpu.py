"""LoRA on CPU: adapter math against the dense statement, merge / unmerge, injection by target patterns, freezing,
conv adapters, named adapters, serialisation. (The fused GPU path is covered by tests/test_lora_gpu.py.)"""
import copy

import pytest
import torch
import torch.nn as nn

from ml_framework_b200.nn import lora as R


class Block(nn.Module):
    def __init__(self):
        super().__init__()
        self.q_proj, self.k_proj, self.v_proj = nn.Linear(16, 16), nn.Linear(16, 16), nn.Linear(16, 16, bias=False)
        self.mlp = nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 16))
        self.conv = nn.Conv2d(2, 4, 3, padding=1)

    def forward(self, x):
        return self.mlp(self.q_proj(x) + self.k_proj(x) + self.v_proj(x))


def test_config_validation_presets_and_target_matching():
    for bad in (dict(rank=0), dict(alpha=0), dict(dropout=1.0), dict(bias="some"), dict(lora_type="x")):
        with pytest.raises(ValueError):
            R.LoraConfig(**bad).validate()
    assert R.LoraConfig(rank=8, alpha=16).scaling == 2.0
    assert R.LoraConfig(rank=16, alpha=16, lora_type="scaled").scaling == 4.0
    assert "o_proj" in R.LoraConfig.for_llama().target_modules and R.LoraConfig.for_gpt(4).alpha == 8
    assert R.LoraConfig.for_bert().target_modules == ("query", "value")
    assert R.matches_target("blocks.0.q_proj", ["q_proj"]) and R.matches_target("blocks.0.attn.qkv", ["attn.qkv"])
    assert R.matches_target("blocks.3.mlp.fc1", ["*.mlp.fc?"]) and R.matches_target("head", ["h*"])
    assert not R.matches_target("blocks.0.k_proj", ["q_proj", "v_proj"]) and not R.matches_target("xq_proj", ["q_proj"])


def test_lora_linear_math_merge_unmerge_and_gradients():
    torch.manual_seed(0)
    base = nn.Linear(12, 20)
    dense = copy.deepcopy(base)
    m = R.LoraLinear(base, R.LoraConfig(rank=4, alpha=8))
    x = torch.randn(5, 12)
    assert torch.allclose(m(x), dense(x))                              # B starts at zero: the adapter is the identity
    with torch.no_grad():
        m.lora_B.copy_(torch.randn(4, 12) * 0.3)
    want = dense(x) + (x @ m.lora_B.t() @ m.lora_A.t()) * 2.0
    assert torch.allclose(m(x), want, atol=1e-6)
    assert torch.allclose(m.delta_weight(), 2.0 * m.lora_A @ m.lora_B)
    assert not base.weight.requires_grad and not base.bias.requires_grad and m.lora_A.requires_grad
    m(x).sum().backward()
    assert base.weight.grad is None and m.lora_A.grad is not None and m.lora_B.grad is not None
    # gradient of B against autograd on the dense statement
    A, B = m.lora_A.detach().clone(), m.lora_B.detach().clone().requires_grad_(True)
    (dense(x) + (x @ B.t() @ A.t()) * 2.0).sum().backward()
    assert torch.allclose(m.lora_B.grad, B.grad, atol=1e-6)
    m.merge()
    assert m.merged and torch.allclose(m(x), want, atol=1e-5) and torch.allclose(base.weight, dense.weight + m.delta_weight(), atol=1e-6)
    m.merge()                                                          # idempotent
    assert torch.allclose(base.weight, dense.weight + m.delta_weight(), atol=1e-6)
    m.unmerge()
    assert not m.merged and torch.allclose(base.weight, dense.weight, atol=1e-6) and torch.allclose(m(x), want, atol=1e-5)
    m.enabled = False
    assert torch.allclose(m(x), dense(x))
    keep = R.LoraLinear(nn.Linear(4, 4), R.LoraConfig(rank=2, bias="lora_only"))
    assert keep.base.bias.requires_grad and not keep.base.weight.requires_grad
    drop = R.LoraLinear(nn.Linear(4, 4), R.LoraConfig(rank=2, dropout=0.5))
    drop.eval()
    assert torch.allclose(drop(torch.ones(2, 4)), drop.base(torch.ones(2, 4)))


def test_lora_conv2d_matches_merged_convolution():
    torch.manual_seed(1)
    base = nn.Conv2d(3, 6, 3, padding=1)
    dense = copy.deepcopy(base)
    m = R.LoRAConv2d(base, R.LoraConfig(rank=2, alpha=4))
    with torch.no_grad():
        m.lora_B.copy_(torch.randn_like(m.lora_B) * 0.2)
    x = torch.randn(2, 3, 8, 8)
    y = m(x)
    assert not torch.allclose(y, dense(x))
    m.merge()
    assert torch.allclose(m(x), y, atol=1e-5) and torch.allclose(nn.functional.conv2d(x, base.weight, base.bias, padding=1), y, atol=1e-5)
    m.unmerge()
    assert torch.allclose(base.weight, dense.weight, atol=1e-6)


def test_injector_freeze_remove_and_parameter_listing():
    torch.manual_seed(2)
    model = Block()
    ref = copy.deepcopy(model)
    wrapped = R.LoraInjector.inject(model, R.LoraConfig(rank=4, target_modules=("q_proj", "v_proj", "conv", "mlp.0")))
    assert sorted(wrapped) == ["conv", "mlp.0", "q_proj", "v_proj"]
    assert isinstance(model.q_proj, R.LoraLinear) and isinstance(model.conv, R.LoRAConv2d) and isinstance(model.k_proj, nn.Linear)
    assert R.LoraInjector.inject(model, R.LoraConfig(rank=4, target_modules=("q_proj",))) == []      # already wrapped
    R.freeze_base(model)
    trainable = [n for n, p in model.named_parameters() if p.requires_grad]
    assert trainable and all("lora_" in n for n in trainable) and len(R.lora_parameters(model)) == 8
    x = torch.randn(3, 16)
    assert torch.allclose(model(x), ref(x), atol=1e-6)
    with torch.no_grad():
        for p in R.lora_parameters(model):
            p.add_(0.05)
    changed = model(x)
    assert not torch.allclose(changed, ref(x))
    assert R.LoraInjector.remove(model, merge=True) == 4 and isinstance(model.q_proj, nn.Linear)
    assert torch.allclose(model(x), changed, atol=1e-5) and R.LoraInjector.get_lora_layers(model) == {}
    m2 = R.apply_lora(Block())
    assert set(R.LoraInjector.get_lora_layers(m2)) == {"q_proj", "v_proj"}
    assert all(p.requires_grad == ("lora_" in n) for n, p in m2.named_parameters())


def test_named_adapters_manager_and_serializer(tmp_path):
    torch.manual_seed(3)
    model = R.apply_lora(Block(), R.LoraConfig(rank=2, target_modules=("q_proj", "k_proj")))
    x = torch.randn(4, 16)
    base_out = model(x)                                                 # B = 0: the plain model
    with torch.no_grad():
        for p in R.lora_parameters(model):
            p.normal_(0, 0.2)
    a = R.LoraAdapter.from_model("style-a", model)
    out_a = model(x)
    with torch.no_grad():
        for p in R.lora_parameters(model):
            p.normal_(0, 0.2)
    b = R.LoraAdapter.from_model("style-b", model)
    out_b = model(x)
    mgr = R.AdapterManager(model)
    mgr.load_adapter(a)
    mgr.load_adapter(b, activate=True)
    assert mgr.active == "style-b" and torch.allclose(model(x), out_b, atol=1e-6) and mgr.list_adapters() == ["style-a", "style-b"]
    mgr.activate("style-a")
    assert torch.allclose(model(x), out_a, atol=1e-6)
    mgr.deactivate()
    assert mgr.active is None and torch.allclose(model(x), base_out, atol=1e-6)
    with pytest.raises(ValueError):
        mgr.load_adapter(a)
    with pytest.raises(KeyError):
        mgr.set_active_adapter("nope")
    mgr.activate("style-b")
    mgr.unload("style-b")
    assert mgr.active is None and mgr.list_adapters() == ["style-a"]
    path = str(tmp_path / "ad" / "a.pt")
    R.AdapterSerializer.save(a, path)
    back = R.AdapterSerializer.load(path)
    assert back.name == "style-a" and back.config.rank == 2 and back.config.target_modules == ("q_proj", "k_proj")
    fresh = R.apply_lora(copy.deepcopy(Block()), back.config)
    fresh.load_state_dict({k: v for k, v in model.state_dict().items() if "lora_" not in k}, strict=False)
    back.apply_to(fresh)
    assert torch.allclose(fresh(x), out_a, atol=1e-6)
    R.AdapterSerializer.save_json(a, str(tmp_path / "a.json"))
    import json
    j = json.load(open(tmp_path / "a.json"))
    assert j["name"] == "style-a" and set(j["weights"]) == {"q_proj", "k_proj"} and len(j["weights"]["q_proj"]["lora_A"]) == 16
    torch.save({"format": "other"}, str(tmp_path / "x.pt"))
    with pytest.raises(ValueError):
        R.AdapterSerializer.load(str(tmp_path / "x.pt"))
    other = R.apply_lora(Block(), R.LoraConfig(rank=2, target_modules=("v_proj",)))
    with pytest.raises(KeyError):
        a.apply_to(other)
    with pytest.raises(ValueError):
        R.LoraAdapter.from_model("none", Block())
