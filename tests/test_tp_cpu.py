"""Tensor-parallel layers on simulated ranks: forward equals the dense layer, backward equals the
dense gradients (including dX through the column layer), sequence-parallel variants, vocabulary-
parallel loss, model conversion, DeviceMesh rules."""
import copy

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from ml_framework_b200.dist.mesh import DeviceMesh, ParallelismDimension
from ml_framework_b200.dist.process_group import run_fake_world
from ml_framework_b200.parallel import tensor_parallel as tpm


def test_device_mesh_rules():
    m = DeviceMesh((2, 4), rank=5)          # data=2, tensor=4, row-major, last dim fastest
    assert m.coord.coords == (1, 1) and m.coord_to_rank((1, 1)) == 5
    assert m.tp_group_ranks() == [4, 5, 6, 7] and m.dp_group_ranks() == [1, 5]
    assert m.tp_world_size == 4 and m.dp_world_size == 2 and m.tp_rank == 1 and m.dp_rank == 1
    assert m.ranks_with_index(ParallelismDimension.TENSOR, 0) == [0, 4]
    assert m.all_groups(1) == [[0, 1, 2, 3], [4, 5, 6, 7]]
    m3 = DeviceMesh((2, 2, 2), rank=3)
    assert m3.coord.coords == (0, 1, 1) and m3.pp_group_ranks() == [2, 3] and m3.pp_world_size == 2
    for r in range(8):
        assert m3.coord_to_rank(m3.rank_to_coord(r)) == r
    with pytest.raises(ValueError):
        DeviceMesh((2, 2), rank=4)
    with pytest.raises(ValueError):
        m.coord_to_rank((2, 0))


@pytest.mark.parametrize("sp", [False, True])
def test_column_row_mlp_matches_dense(sp):
    W, T, D, H = 4, 8, 16, 32
    torch.manual_seed(0)
    w1, b1 = torch.randn(H, D) * 0.3, torch.randn(H) * 0.1
    w2, b2 = torch.randn(D, H) * 0.3, torch.randn(D) * 0.1
    x = torch.randn(T, D)
    dy = torch.randn(T, D)
    xr = x.clone().requires_grad_()
    w1r, b1r, w2r, b2r = [t.clone().requires_grad_() for t in (w1, b1, w2, b2)]
    yr = F.linear(F.gelu(F.linear(xr, w1r, b1r), approximate="tanh"), w2r, b2r)
    yr.backward(dy)

    def run(pg):
        tp = tpm.TPContext(pg, None, fused=False)
        fc1 = tpm.ColumnParallelLinear(D, H, True, sequence_parallel=sp, tp=tp)
        fc2 = tpm.RowParallelLinear(H, D, True, sequence_parallel=sp, tp=tp)
        r = pg.rank
        with torch.no_grad():
            fc1.weight.copy_(w1.chunk(W, 0)[r]); fc1.bias.copy_(b1.chunk(W, 0)[r])
            fc2.weight.copy_(w2.chunk(W, 1)[r]); fc2.bias.copy_(b2)
        xin = (x.chunk(W, 0)[r] if sp else x).clone().requires_grad_()
        y = fc2(F.gelu(fc1(xin), approximate="tanh"))
        y.backward(dy.chunk(W, 0)[r] if sp else dy)
        return y.detach(), xin.grad, fc1.weight.grad, fc1.bias.grad, fc2.weight.grad, fc2.bias.grad
    outs = run_fake_world(W, run)
    y = torch.cat([o[0] for o in outs]) if sp else outs[0][0]
    dx = torch.cat([o[1] for o in outs]) if sp else outs[0][1]
    assert torch.allclose(y, yr, atol=1e-5) and torch.allclose(dx, xr.grad, atol=1e-5)
    assert torch.allclose(torch.cat([o[2] for o in outs]), w1r.grad, atol=1e-5)
    assert torch.allclose(torch.cat([o[3] for o in outs]), b1r.grad, atol=1e-5)
    assert torch.allclose(torch.cat([o[4] for o in outs], 1), w2r.grad, atol=1e-5)
    b2g = sum(o[5] for o in outs) if sp else outs[0][5]      # SP: each rank saw its token shard only
    assert torch.allclose(b2g, b2r.grad, atol=1e-5)


def test_shape_validation_and_gather_output():
    def run(pg):
        tp = tpm.TPContext(pg, None, fused=False)
        with pytest.raises(ValueError):
            tpm.ColumnParallelLinear(8, 10, tp=tp)
        with pytest.raises(ValueError):
            tpm.RowParallelLinear(10, 8, tp=tp)
        col = tpm.ColumnParallelLinear(8, 12, False, gather_output=True, tp=tp)
        assert col.local_weight_shape() == (4, 8)
        return col(torch.ones(2, 8)).shape
    assert run_fake_world(3, run) == [torch.Size([2, 12])] * 3


def test_vocab_parallel_loss_and_embedding():
    W, T, D, V = 2, 6, 8, 10
    torch.manual_seed(1)
    h = torch.randn(T, D)
    w = torch.randn(12, D)       # padded vocabulary 12, 10 valid
    tg = torch.randint(0, V, (T,))
    hr, wr = h.clone().requires_grad_(), w.clone().requires_grad_()
    F.cross_entropy(F.linear(hr, wr)[:, :V], tg).backward()
    ref_loss = F.cross_entropy(F.linear(h, w)[:, :V], tg)

    def run(pg):
        tp = tpm.TPContext(pg, None, fused=False)
        hh = h.clone().requires_grad_()
        ws = w.chunk(W, 0)[pg.rank].clone().requires_grad_()
        loss = tpm.vocab_parallel_lm_loss(hh, ws, tg, tp, V)
        loss.backward()
        emb = tpm.VocabParallelEmbedding(12, D, tp)
        with torch.no_grad():
            emb.weight.copy_(w.chunk(W, 0)[pg.rank])
        return loss.item(), hh.grad, ws.grad, emb(tg)
    outs = run_fake_world(W, run)
    assert abs(outs[0][0] - ref_loss.item()) < 1e-5
    assert torch.allclose(outs[0][1], hr.grad, atol=1e-5)
    assert torch.allclose(torch.cat([o[2] for o in outs]), wr.grad, atol=1e-5)
    assert torch.allclose(outs[1][3], w[tg], atol=1e-6)


def test_converter_and_analyzer():
    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.fc1, self.fc2, self.other = nn.Linear(8, 16), nn.Linear(16, 8), nn.Linear(8, 3)

        def forward(self, x):
            return self.other(self.fc2(torch.relu(self.fc1(x))))
    torch.manual_seed(2)
    dense = Net()
    x = torch.randn(4, 8)
    want = dense(x)
    rep = tpm.TPModelAnalyzer().analyze(dense, 2)
    kinds = {a.name: a.parallelism for a in rep}
    assert kinds == {"fc1": "column", "fc2": "row", "other": "replicate"}
    est = tpm.TPMemoryEstimator.estimate(rep)
    assert 0.3 < est["savings"] < 0.5

    def run(pg):
        tp = tpm.TPContext(pg, None, fused=False)
        m = tpm.TPModelConverter(tp).convert(copy.deepcopy(dense))
        assert isinstance(m.fc1, tpm.ColumnParallelLinear) and isinstance(m.fc2, tpm.RowParallelLinear)
        return m(x)
    for y in run_fake_world(2, run):
        assert torch.allclose(y, want, atol=1e-5)


def test_llama_tp_sequence_parallel_matches_plain_tensor_parallel():
    """Same weight shards, same batch: the sequence-parallel model (token-sharded residual stream, reduce-scatter /
    all-gather pairs, head fed from token shards) must give the loss and every gradient of the plain tensor-parallel
    model (replicated activations, all-reduces). Norm scales see token shards under SP: their gradients match after
    the sum over the group."""
    from ml_framework_b200.models.llama import LlamaConfig
    from ml_framework_b200.models.llama_tp import LlamaTP
    cfg = LlamaConfig(n_layers=2, d_model=32, n_heads=4, n_kv_heads=2, head_dim=8, d_ff=64, vocab_size=50, max_seq=16)
    W = 2
    ids = torch.randint(0, 50, (2, 8), generator=torch.Generator().manual_seed(5))
    tgt = torch.randint(0, 50, (2, 8), generator=torch.Generator().manual_seed(6))

    def run(pg):
        out = {}
        for sp in (False, True):
            tp = tpm.TPContext(pg, None, fused=False)
            m = LlamaTP(cfg, tp, sequence_parallel=sp, dtype=torch.float32)
            # ranks are threads here and share torch's global generator: fill the shards from per-rank generators
            g = torch.Generator().manual_seed(10 + pg.rank)
            gr = torch.Generator().manual_seed(99)
            rep = {id(p) for p in m.replicated_parameters()}
            with torch.no_grad():
                for p in m.parameters():
                    if id(p) in rep:
                        p.copy_(1.0 + 0.1 * torch.randn(p.shape, generator=gr))
                    else:
                        p.copy_(0.08 * torch.randn(p.shape, generator=g))
            loss = m(ids, tgt)
            loss.backward()
            m.sync_replicated_grads()
            out[sp] = (loss.item(), {n: p.grad.clone() for n, p in m.named_parameters()})
        return out
    for res in run_fake_world(W, run):
        (l0, g0), (l1, g1) = res[False], res[True]
        assert abs(l0 - l1) < 1e-5
        for n in g0:
            assert torch.allclose(g0[n], g1[n], atol=2e-5, rtol=1e-4), (n, (g0[n] - g1[n]).abs().max())


def test_tp_gradient_manager_flat_path_averages_over_the_data_parallel_group():
    """TP x DP: each data-parallel replica holds the same shard; gradients of different micro-batches are averaged over
    the data-parallel group through the flat, bucketed, hook-driven reducer (several buckets)."""
    W = 2

    def make():                                                  # fake ranks are threads: no use of the global generator
        g = torch.Generator().manual_seed(0)
        lin1, lin2 = nn.Linear(16, 32), nn.Linear(32, 16)
        with torch.no_grad():
            for p in list(lin1.parameters()) + list(lin2.parameters()):
                p.copy_(torch.randn(p.shape, generator=g) * 0.2)
        return lin1, lin2

    def run(dp_pg):
        lin1, lin2 = make()
        gm = tpm.TPGradientManager(tpm.TPContext(None, None, False), dp_pg)
        params = list(lin1.parameters()) + list(lin2.parameters())
        flat = gm.attach_flat(params, bucket_size_mb=0.002, fused=True)      # CPU tensors: process-group all-reduces
        assert gm.reducer is not None and len(gm.reducer.ranges) >= 2
        g = torch.Generator().manual_seed(100 + dp_pg.rank)
        outs = []
        for step in range(2):
            flat.zero_grad()
            x = torch.randn(8, 16, generator=g)
            lin2(torch.relu(lin1(x))).pow(2).mean().backward()
            gm.synchronize_gradients(params)
            outs.append([p.main_grad.clone() for p in params])
        gm.close()
        return outs

    res = run_fake_world(W, run)
    for step in range(2):
        for k in range(4):
            assert torch.allclose(res[0][step][k], res[1][step][k], atol=1e-6)           # replicas agree
    # and the agreed value is the mean of the per-replica gradients
    gens = [torch.Generator().manual_seed(100 + r) for r in range(W)]
    for step in range(2):
        want = None
        for r in range(W):
            lin1, lin2 = make()
            x = torch.randn(8, 16, generator=gens[r])
            lin2(torch.relu(lin1(x))).pow(2).mean().backward()
            gr = [p.grad / W for p in list(lin1.parameters()) + list(lin2.parameters())]
            want = gr if want is None else [a + b for a, b in zip(want, gr)]
        for k in range(4):
            assert torch.allclose(res[0][step][k], want[k], atol=1e-5), (step, k)
