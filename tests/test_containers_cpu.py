"""Sequential container, tree access by path, hierarchical wrappers, gradient hooks, Conv2d."""
import pytest
import torch
import torch.nn as nn

from ml_framework_b200.nn import containers as C


def test_sequential_module_edits_in_place():
    s = C.SequentialModule([nn.Linear(4, 4)], name="net").add(nn.ReLU()).add(nn.Linear(4, 2))
    assert s.count == 3 and len(s) == 3 and isinstance(s.get_module(1), nn.ReLU)
    s.insert(1, nn.Tanh())
    assert [type(m).__name__ for m in s] == ["Linear", "Tanh", "ReLU", "Linear"]
    x = torch.randn(3, 4)
    assert torch.allclose(s(x), s.layers[3](torch.relu(torch.tanh(s.layers[0](x)))))
    assert isinstance(s.remove_at(1), nn.Tanh) and s.count == 3 and len(list(s.parameters())) == 4
    for bad in (lambda: s.insert(9, nn.ReLU()), lambda: s.remove_at(3)):
        with pytest.raises(IndexError):
            bad()
    with pytest.raises(TypeError):
        s.add("relu")
    s.clear()
    assert s.count == 0 and torch.equal(s(x), x) and s.get_modules() == []


def test_tree_access_by_path():
    net = nn.Sequential(nn.Sequential(nn.Linear(2, 2), nn.ReLU()), nn.Linear(2, 1))
    assert C.get_child(net, "") is net and C.get_child(net, "0.1") is net[0][1] and C.parent_of(net, "0.1") is net[0] and C.parent_of(net, "") is None
    old = C.replace_child(net, "0.1", nn.Tanh())
    assert isinstance(old, nn.ReLU) and isinstance(net[0][1], nn.Tanh)
    with pytest.raises(KeyError):
        C.get_child(net, "0.7")
    with pytest.raises(KeyError):
        C.replace_child(net, "5", nn.ReLU())
    with pytest.raises(ValueError):
        C.replace_child(net, "", nn.ReLU())
    assert [(n, d) for n, _, d in C.walk(net, max_depth=1)] == [("", 0), ("0", 1), ("1", 1)] and C.depth_of("a.b.c") == 3
    assert C.set_requires_grad(net, False, "0") == 2 and not net[0][0].weight.requires_grad and net[1].weight.requires_grad


def test_hierarchical_wrappers():
    root = C.ModuleContainer("root")
    a, b = C.HierarchicalWrapper(nn.Linear(3, 3), "a"), C.HierarchicalWrapper(nn.ReLU(), "b")
    root.add_child(a)
    root.add_child(b)
    assert a.parent is root and a.path == "root.a" and a.module_type == "Linear" and [c.name for c in root.children_nodes()] == ["a", "b"]
    x = torch.randn(2, 3)
    assert torch.allclose(root(x), torch.relu(a.module(x))) and len(list(root.parameters())) == 2
    c = C.HierarchicalWrapper(nn.Tanh(), "whatever")
    root.replace_child("b", c)
    assert c.name == "b" and c.parent is root and b.parent is None and torch.allclose(root(x), torch.tanh(a.module(x)))
    with pytest.raises(KeyError):
        root.add_child(C.HierarchicalWrapper(nn.ReLU(), "a"))
    with pytest.raises(KeyError):
        root.get_child("zzz")
    assert root.get_child("a") is a


def test_gradient_hooks_fire_during_backward():
    reg = C.GradientHookRegistry()
    lin = nn.Linear(2, 1)
    ready = []
    reg.register(lin.weight, lambda g: g * 10, "w")
    reg.register_ready(lin.weight, lambda p: ready.append(p.grad.clone()))
    lin(torch.ones(1, 2)).sum().backward()
    assert torch.equal(lin.weight.grad, torch.full((1, 2), 10.0)) and torch.equal(ready[0], lin.weight.grad) and len(reg) == 2
    assert reg.has_hook(lin.weight) and not reg.has_hook(lin.bias) and reg.remove(lin.weight) == 2
    lin.weight.grad = None
    lin(torch.ones(1, 2)).sum().backward()
    assert torch.equal(lin.weight.grad, torch.ones(1, 2)) and len(ready) == 1
    with pytest.raises(ValueError):
        reg.register(torch.zeros(1), lambda g: g)
    reg.register(lin.bias, lambda g: None)
    reg.clear()
    assert len(reg) == 0


def test_conv2d_matches_torch_and_reports_its_output_shape():
    torch.manual_seed(0)
    c = C.Conv2d(4, 6, 3, stride=2, padding=1, groups=2)
    x = torch.randn(2, 4, 9, 7)
    y = c(x)
    assert y.shape == (2, 6, *c.output_shape(9, 7)) == (2, 6, 5, 4)
    assert torch.allclose(y, torch.nn.functional.conv2d(x, c.weight, c.bias, 2, 1, 1, 2)) and c.weight.shape == (6, 2, 3, 3)
    y.sum().backward()
    assert c.weight.grad is not None and C.Conv2d(1, 1, (1, 3), bias=False).bias is None
    with pytest.raises(ValueError):
        c(torch.randn(2, 3, 9, 7))
    with pytest.raises(ValueError):
        C.Conv2d(3, 6, 3, groups=2)
