"""Tensor-parallel factories, rank-conditional execution, tensor-returning group facade, mesh-aware context (simulated ranks)."""
import pytest
import torch
import torch.nn as nn

from ml_framework_b200.dist.mesh import DeviceMesh
from ml_framework_b200.dist.process_group import ReduceOp, run_fake_world
from ml_framework_b200.parallel import tp_api as T
from ml_framework_b200.parallel.tensor_parallel import TPContext


def test_factories_build_sharded_layers_that_match_a_dense_model():
    W, d, hid = 2, 8, 16

    def run(pg):
        tp = TPContext(pg, None, False)
        qkv = T.ColumnParallelLinearFactory.create_for_attention(d, n_heads=4, n_kv_heads=2, head_dim=2, tp=tp)
        out = T.RowParallelLinearFactory.create_for_attention_output(d, 4, head_dim=2, tp=tp)
        up = T.ColumnParallelLinearFactory.create_for_mlp_hidden(d, hid, gated=True, tp=tp)
        down = T.RowParallelLinearFactory.create_for_mlp_output(hid, d, tp=tp)
        mlp = T.TPMLPFactory.create_mlp_block(d, hid, "relu", tp=tp)
        shapes = [tuple(m.weight.shape) for m in (qkv, out, up, down, mlp.fc1, mlp.fc2)]
        g = torch.Generator().manual_seed(0)
        w1, b1, w2, b2 = torch.randn(hid, d, generator=g), torch.randn(hid, generator=g), torch.randn(d, hid, generator=g), torch.randn(d, generator=g)
        with torch.no_grad():
            mlp.fc1.weight.copy_(w1.chunk(W, 0)[pg.rank]); mlp.fc1.bias.copy_(b1.chunk(W, 0)[pg.rank])
            mlp.fc2.weight.copy_(w2.chunk(W, 1)[pg.rank]); mlp.fc2.bias.copy_(b2)
        x = torch.randn(3, d, generator=g)
        y = T.TPMLPFactory.forward_mlp(mlp, x)
        want = torch.relu(x @ w1.t() + b1) @ w2.t() + b2
        errs = []
        for bad in (lambda: T.ColumnParallelLinearFactory.create_for_attention(d, n_heads=3, tp=tp), lambda: T.TPMLPFactory.create_mlp_block(d, hid, "swish", tp=tp)):
            try:
                bad()
            except ValueError as e:
                errs.append(str(e))
        return shapes, torch.allclose(y, want, atol=1e-5), errs
    for shapes, ok, errs in run_fake_world(W, run):
        assert shapes == [(8, 8), (8, 4), (16, 8), (8, 8), (8, 8), (8, 8)] and ok and len(errs) == 2 and "do not split" in errs[0]


def test_conv_bottleneck_matches_dense_convolutions():
    W = 2

    def run(pg):
        tp = TPContext(pg, None, False)
        blk = T.TPConv2dFactory.create_bottleneck(4, 6, 4, 3, tp=tp)
        g = torch.Generator().manual_seed(1)
        w1, b1, w2, b2 = torch.randn(6, 4, 3, 3, generator=g), torch.randn(6, generator=g), torch.randn(4, 6, 3, 3, generator=g), torch.randn(4, generator=g)
        c1, c2 = blk[0], blk[2]
        with torch.no_grad():
            c1.conv.weight.copy_(w1.chunk(W, 0)[pg.rank]); c1.conv.bias.copy_(b1.chunk(W, 0)[pg.rank])
            c2.conv.weight.copy_(w2.chunk(W, 1)[pg.rank])
            c2.bias.copy_(b2)
        x = torch.randn(2, 4, 5, 5, generator=g)
        want = torch.nn.functional.conv2d(torch.relu(torch.nn.functional.conv2d(x, w1, b1, padding=1)), w2, b2, padding=1)
        return torch.allclose(blk(x), want, atol=1e-4)
    assert all(run_fake_world(W, run))


def test_tp_state_and_group_facade():
    def run(pg):
        tp = TPContext(pg, None, False)
        st, grp = T.TPState(tp), T.TensorParallelGroup(tp)
        on1 = st.execute_on_rank(1, lambda: "one")
        master = st.execute_on_master(lambda a: a * 2, 21)
        everywhere = st.execute_on_all(lambda r: r * 10, barrier=True)
        shared = st.broadcast_from_master({"lr": 0.1} if st.is_master else "ignored")
        t = torch.full((2,), float(pg.rank + 1))
        ar, ag = grp.all_reduce(t), grp.all_gather(t.view(1, 2), dim=-1)
        rs = grp.reduce_scatter(torch.arange(4.0))
        bc = grp.broadcast(t, root=1)
        grp.barrier()
        try:
            st.execute_on_rank(5, lambda: None)
            bad = False
        except ValueError:
            bad = True
        return on1, master, everywhere, shared, t.tolist(), ar.tolist(), tuple(ag.shape), rs.tolist(), bc.tolist(), bad, grp.size
    r0, r1 = run_fake_world(2, run)
    assert (r0[0], r1[0]) == (None, "one") and (r0[1], r1[1]) == (42, None) and (r0[2], r1[2]) == (0, 10) and r0[3] == r1[3] == {"lr": 0.1}
    assert r0[4] == [1.0, 1.0] and r0[5] == [3.0, 3.0] and r0[6] == (1, 4) and r0[7] == [0.0, 2.0] and r1[7] == [4.0, 6.0] and r0[8] == [2.0, 2.0] and r0[9] and r0[10] == 2
    solo = T.TensorParallelGroup(TPContext(None, None, False))
    x = torch.ones(3)
    assert solo.all_reduce(x) is not x and torch.equal(solo.all_gather(x), x) and torch.equal(solo.reduce_scatter(x), x) and solo.size == 1
    assert T.TPState(TPContext(None, None, False)).broadcast_from_master(7) == 7


def test_mesh_context_and_layer_factory():
    def run(pg):
        mesh = DeviceMesh((1, 2), pg.rank)                       # data x tensor
        ctx = T.TensorParallelMeshContext.initialize_with_mesh(mesh, tp_group=pg)
        f = T.TPMeshLayerFactory(ctx)
        col, row, mlp = f.column_linear(8, 12), f.row_linear(12, 8), f.mlp(8, 16)
        gm = ctx.gradient_manager()
        return (ctx.tp_rank, ctx.dp_rank, ctx.state.tp_world_size(), ctx.state.dp_world_size(), ctx.state.is_master_rank(),
                tuple(col.weight.shape), tuple(row.weight.shape), tuple(mlp.fc1.weight.shape), gm.dp is None, ctx.state.describe(),
                ctx.state.execute_on_master(lambda: "m"))
    r0, r1 = run_fake_world(2, run)
    assert r0[:5] == (0, 0, 2, 1, True) and r1[:5] == (1, 0, 2, 1, False) and r0[5:8] == ((6, 8), (8, 6), (8, 8)) and r0[8]
    assert r1[9] == "rank 1: tp 1/2, dp 0/1, pp 0/1" and (r0[10], r1[10]) == ("m", None)
    solo = T.TensorParallelMeshContext(DeviceMesh((1, 1), 0))
    assert solo.tp.world == 1 and solo.tp_group is None and solo.dp_group is None
