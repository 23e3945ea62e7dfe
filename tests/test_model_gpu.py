"""End-to-end: the GPT and Llama blocks on the native kernels against the same modules run in
fp32 PyTorch on the same weights, and a few optimisation steps through the engine."""
import copy

import pytest
import torch

from ml_framework_b200.engine import EngineConfig, TrainEngine
from ml_framework_b200.models import GPT, GPTConfig, Llama, LlamaConfig

pytestmark = pytest.mark.gpu


def _grads_close(m_native, m_ref, flat, tol):
    worst = 0.0
    for (n, p), (_, q) in zip(m_native.named_parameters(), m_ref.named_parameters()):
        g = p.main_grad.float() if getattr(p, "main_grad", None) is not None else p.grad.float()
        r = q.grad.float()
        err = (g - r).abs().max().item() / (r.abs().max().item() + 1e-6)
        worst = max(worst, err)
        assert err < tol, f"{n}: rel err {err}"
    return worst


@pytest.mark.parametrize("family", ["gpt", "llama"])
def test_model_fwd_bwd_matches_fp32(family):
    torch.manual_seed(0)
    dev = "cuda"
    if family == "gpt":
        cfg = GPTConfig.tiny()
        model = GPT(cfg, dtype=torch.bfloat16, device=dev)
    else:
        cfg = LlamaConfig.tiny()
        model = Llama(cfg, dtype=torch.bfloat16, device=dev)
    ref = copy.deepcopy(model).float()
    from ml_framework_b200.parallel.flat import FlatParams
    flat = FlatParams(list(dict.fromkeys(model.parameters())))
    ids = torch.randint(0, cfg.vocab_size, (2, 256), device=dev)
    tgt = torch.randint(0, cfg.vocab_size, (2, 256), device=dev)
    loss = model(ids, tgt)
    loss.backward()
    flat.gather_missing_grads()
    loss_ref = ref(ids, tgt)
    loss_ref.backward()
    assert abs(loss.item() - loss_ref.item()) < 3e-2 * abs(loss_ref.item())
    _grads_close(model, ref, flat, 8e-2)


def test_engine_trains():
    torch.manual_seed(1)
    cfg = GPTConfig.tiny()
    model = GPT(cfg, dtype=torch.bfloat16, device="cuda")
    eng = TrainEngine(model, EngineConfig(strategy="none", lr=2e-3))
    ids = torch.randint(0, cfg.vocab_size, (2, 256), device="cuda")
    tgt = torch.randint(0, cfg.vocab_size, (2, 256), device="cuda")
    losses = [float(eng.step(ids, tgt)) for _ in range(8)]
    assert losses[-1] < losses[0] - 0.5, losses
    assert eng.scaler.get_stats().skipped_steps == 0


def test_fsdp_parameter_offload_with_prefetch_trains_like_resident_shards():
    """One GPU, parameter shards in pinned host memory brought back by the prefetch manager two units ahead,
    optimizer update unit by unit through a staging buffer: same losses as with resident shards."""
    import copy
    from ml_framework_b200.amp.grad_scaler import DynamicLossScaler, DynamicScalerConfig
    from ml_framework_b200.parallel.fsdp import FSDP, FSDPConfig, FSDPCpuOffloadConfig
    cfg = GPTConfig(n_layers=4, d_model=256, n_heads=2, d_ff=1024, vocab_size=1000, max_seq=128)
    torch.manual_seed(0)
    base = GPT(cfg, dtype=torch.bfloat16, device="cuda")
    ids = torch.randint(0, cfg.vocab_size, (2, 128), device="cuda")
    tgt = torch.randint(0, cfg.vocab_size, (2, 128), device="cuda")
    out = {}
    for name, off in (("resident", None), ("offload", FSDPCpuOffloadConfig(enabled=True, offload_optimizer_states=False,
                                                                            offload_parameters=True, prefetch_steps=2))):
        fs = FSDP(copy.deepcopy(base), FSDPConfig(cpu_offload=off) if off else FSDPConfig(), None,
                  optimizer_kwargs=dict(lr=1e-3, betas=(0.9, 0.95), eps=1e-6, weight_decay=0.01))
        scaler = DynamicLossScaler(DynamicScalerConfig(initial_scale=1024.0), device="cuda")
        out[name] = [float(fs.train_step(ids, tgt, scaler)) for _ in range(5)]
        if off:
            assert fs.param_shards.device.type == "cpu" and fs.prefetch.hits > 0
    torch.cuda.synchronize()
    for a, b in zip(out["resident"], out["offload"]):
        assert abs(a - b) < 2e-2 * abs(a), out
    assert out["offload"][-1] < out["offload"][0]
