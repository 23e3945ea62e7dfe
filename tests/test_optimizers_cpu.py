"""AdamW / SGD on CPU against torch.optim on the same gradients; learning-rate access, scheduler hook, state round
trips, flat buffers, bf16 parameters with an fp32 master copy, the found-inf skip."""
import copy

import pytest
import torch
import torch.nn as nn

from ml_framework_b200.optim.optimizers import SGD, Adam, AdamW
from ml_framework_b200.optim.schedulers import StepDecay
from ml_framework_b200.parallel.flat import FlatParams


def _model():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(6, 8), nn.Tanh(), nn.Linear(8, 3))


def _run(opt_ours, opt_ref, m_ours, m_ref, steps=6):
    g = torch.Generator().manual_seed(1)
    for _ in range(steps):
        x = torch.randn(5, 6, generator=g)
        for m, o in ((m_ours, opt_ours), (m_ref, opt_ref)):
            o.zero_grad()
            m(x).pow(2).mean().backward()
            o.step()
    for a, b in zip(m_ours.parameters(), m_ref.parameters()):
        assert torch.allclose(a, b, atol=1e-6), (a - b).abs().max()


@pytest.mark.parametrize("amsgrad", [False, True])
def test_adamw_matches_torch(amsgrad):
    a, b = _model(), _model()
    _run(AdamW(a.parameters(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, amsgrad=amsgrad),
         torch.optim.AdamW(b.parameters(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, amsgrad=amsgrad), a, b)
    assert issubclass(Adam, AdamW)
    for bad in (dict(lr=-1.0), dict(eps=-1e-8), dict(betas=(1.0, 0.9)), dict(weight_decay=-0.1)):
        with pytest.raises(ValueError):
            AdamW(_model().parameters(), **bad)


@pytest.mark.parametrize("momentum,wd", [(0.0, 0.0), (0.9, 0.0), (0.9, 0.05)])
def test_sgd_matches_torch(momentum, wd):
    a, b = _model(), _model()
    _run(SGD(a.parameters(), lr=0.05, momentum=momentum, weight_decay=wd),
         torch.optim.SGD(b.parameters(), lr=0.05, momentum=momentum, weight_decay=wd), a, b)


def test_flat_buffer_lr_scheduler_hook_and_state_round_trip():
    m = _model()
    ref = copy.deepcopy(m)
    flat = FlatParams(list(m.parameters()))
    opt = AdamW(flat, lr=0.1, weight_decay=0.0)
    assert opt.get_learning_rate() == 0.1
    opt.set_learning_rate(0.01)
    opt.set_scheduler(StepDecay(0.01, 2, 0.5))
    tor = torch.optim.AdamW(ref.parameters(), lr=0.01, weight_decay=0.0)
    sch = torch.optim.lr_scheduler.StepLR(tor, 2, 0.5)
    g = torch.Generator().manual_seed(2)
    for step in range(5):
        x = torch.randn(4, 6, generator=g)
        opt.zero_grad()
        m(x).pow(2).mean().backward()
        flat.gather_missing_grads()
        opt.step()
        tor.zero_grad()
        ref(x).pow(2).mean().backward()
        tor.step()
        sch.step()
        assert opt.lr == pytest.approx(tor.param_groups[0]["lr"])
    for a, b in zip(m.parameters(), ref.parameters()):
        assert torch.allclose(a, b, atol=1e-6)
    sd = opt.state_dict()
    assert sd["type"] == "AdamW" and sd["step"] == 5 and len(sd["segments"]) == 1
    m2 = _model()
    opt2 = AdamW(FlatParams(list(m2.parameters())), lr=1.0)
    opt2.load_state_dict(sd)
    assert opt2.step_count == 5 and opt2.lr == opt.lr
    for a, b in zip(m.parameters(), m2.parameters()):
        assert torch.equal(a, b)                                         # parameters come back with the state
    with pytest.raises(ValueError):
        AdamW(_model()[0].parameters()).load_state_dict(sd)             # another layout
    s = SGD(_model().parameters(), lr=0.1, momentum=0.9)
    ssd = s.state_dict()
    assert ssd["type"] == "SGD" and ssd["segments"][0]["m"] is not None
    s2 = SGD(_model().parameters(), lr=0.5, momentum=0.1)
    s2.load_state_dict(ssd)
    assert s2.lr == 0.1 and s2.momentum == 0.9


def test_bf16_parameters_keep_an_fp32_master_and_found_inf_skips():
    torch.manual_seed(3)
    w = nn.Parameter(torch.randn(64).to(torch.bfloat16))
    master = w.detach().float().clone()
    opt = AdamW([w], lr=1e-3, weight_decay=0.0)
    seg = opt.segments[0]
    assert seg.needs_master and seg.master.dtype == torch.float32
    for _ in range(20):                                                 # 20 steps of 1e-3 on values of size ~1: below one bf16 step each
        w.grad = torch.ones_like(w)
        opt.step()
    assert torch.allclose(seg.master, master - 20 * 1e-3, atol=1e-4)   # the master moved by the exact sum ...
    assert torch.equal(w.detach(), seg.master.to(torch.bfloat16))       # ... and the bf16 copy is its rounding
    before = seg.master.clone()
    w.grad = torch.full_like(w, float("inf"))
    opt.step(found_inf=torch.tensor([1], dtype=torch.int32))
    assert torch.equal(seg.master, before)                              # the overflow flag skips the update
    opt.step(inv_scale=torch.tensor(0.5), grad_scale=2.0)               # scale factors multiply the gradient
    frozen = nn.Parameter(torch.ones(2), requires_grad=False)
    assert len(AdamW([frozen, nn.Parameter(torch.ones(2))]).segments) == 1
    o = SGD([nn.Parameter(torch.ones(2))], lr=0.1)
    o.step()                                                            # no gradient yet: nothing happens
    assert o.step_count == 1
