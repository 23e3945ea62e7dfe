"""GPU numerics of the int8 quantisation kernels and the mobile runtime's operator kernels against plain
PyTorch fp32 statements of the same ops; CUDA-graph capture / replay of a kernel sequence."""
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def test_quant_kernels_match_reference():
    from ml_framework_b200.quantization import core as Q
    torch.manual_seed(0)
    for dtype in (torch.float32, torch.bfloat16):
        x = (torch.randn(257, 130, device="cuda") * 3).to(dtype)
        xc = x.cpu()
        for axis, mode in ((None, Q.QuantizationMode.SYMMETRIC), (0, Q.QuantizationMode.ASYMMETRIC), (1, Q.QuantizationMode.SYMMETRIC)):
            if axis is None:
                lo, hi = Q.tensor_minmax(x)
                assert float(lo) == float(xc.float().min()) and float(hi) == float(xc.float().max())
            else:
                lo, hi = xc.float().amin(1 - axis), xc.float().amax(1 - axis)
            qp = Q.compute_qparams(lo.cpu(), hi.cpu(), mode, axis=axis)
            q_gpu, q_cpu = Q.quantize(x, qp), Q.quantize(xc, qp)
            assert (q_gpu.cpu().int() - q_cpu.int()).abs().max() <= 1                 # x / s rounding may differ by one ulp at ties
            assert ((q_gpu.cpu() != q_cpu).float().mean()) < 1e-3
            d_gpu = Q.dequantize(q_gpu, qp, dtype)
            assert torch.allclose(d_gpu.cpu().float(), Q.dequantize(q_gpu.cpu(), qp, dtype).float(), rtol=1e-2, atol=1e-6)
            fq, mask = Q.fake_quantize(x, qp, want_mask=True)
            fq_ref, mask_ref = Q.fake_quantize(xc, qp, want_mask=True)
            assert (fq.cpu().float() - fq_ref.float()).abs().max() <= float(qp.scale.max()) * 1.01
            assert (mask.cpu() != mask_ref).float().mean() < 1e-3
    lin = nn.Linear(128, 64).cuda().bfloat16()
    xin = torch.randn(32, 128, device="cuda", dtype=torch.bfloat16)
    ql = Q.QuantizedLinear(lin)
    assert Q.sqnr_db(lin(xin), ql(xin)) > 25


def test_mobile_kernels_match_torch():
    from ml_framework_b200.mobile import runtime as R
    torch.manual_seed(0)
    net = nn.Sequential(nn.Conv2d(3, 20, 3, padding=1), nn.BatchNorm2d(20), nn.ReLU(), nn.MaxPool2d(2), nn.Conv2d(20, 33, 5, stride=2, padding=2, groups=1),
                        nn.ReLU(), nn.Conv2d(33, 33, 3, padding=2, dilation=2, groups=33), nn.AvgPool2d(3, 2, 1), nn.BatchNorm2d(33),
                        nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.Linear(33, 17), nn.ReLU(), nn.Linear(17, 10), nn.Softmax(-1)).eval()
    for m in net:
        if isinstance(m, nn.BatchNorm2d):
            m.running_mean.normal_()
            m.running_var.uniform_(0.5, 2)
    x = torch.randn(3, 3, 37, 41)
    ref = net(x)
    for optimise in (False, True):
        mm = R.convert_sequential(net, (1, 3, 37, 41))
        if optimise:
            mm = R.optimize(mm)
        rt = R.MobileRuntime("cuda").load_model(mm)
        for _ in range(2):                                   # second call runs on recycled buffers
            out = rt.predict(x)[0]
        assert torch.allclose(out.cpu(), ref, atol=2e-4, rtol=1e-3), (out.cpu() - ref).abs().max()
    assert rt.pool.hits > 0


def test_cuda_graph_manager_captures_and_replays():
    from ml_framework_b200.hal.cuda_graphs import CUDAGraphManager, GraphMemoryPool
    from ml_framework_b200.ops.gemm import gemm
    w = torch.randn(256, 128, device="cuda").bfloat16()

    def fn(x):
        return torch.relu(gemm(x, w).float())
    mgr = CUDAGraphManager()
    outs = []
    for i in range(6):
        x = torch.randn(64, 128, device="cuda").bfloat16()
        y = mgr.run("mlp", fn, x)
        torch.cuda.synchronize()
        assert torch.allclose(y, torch.relu((x.float() @ w.float().t())), atol=0.5, rtol=5e-2)
    st = mgr.stats()
    assert st["graphs"] == 1 and st["replays"] >= 2
    pool = GraphMemoryPool(1 << 20)
    a = pool.allocate((128, 4), torch.bfloat16)
    assert a.is_cuda and a.data_ptr() % 256 == 0


def test_gpu_quantization_backend_int8_matmul_on_the_tensor_cores():
    from ml_framework_b200.quantization.backends import B200Backend, BackendFactory
    from ml_framework_b200.quantization.core import compute_qparams
    BackendFactory.clear_cache()
    be = BackendFactory.create_default()
    assert isinstance(be, B200Backend) and be.get_name() == "GPU"
    torch.manual_seed(0)
    a, b = torch.randn(256, 512, device="cuda"), torch.randn(512, 384, device="cuda")
    qa, qb = compute_qparams(a.min(), a.max()), compute_qparams(b.min(), b.max())
    ia, ib = be.quantize(a, qa), be.quantize(b, qb)
    y = be.matmul_int8(ia, ib, float(qa.scale * qb.scale))
    exact = (ia.to(torch.int32).cpu() @ ib.to(torch.int32).cpu()).float().cuda() * float(qa.scale * qb.scale)
    assert torch.allclose(y, exact, atol=1e-3, rtol=1e-4)          # int8 products accumulate exactly in fp32 up to rounding
    ref = a @ b
    assert (y - ref).abs().max() < 0.08 * ref.abs().max()          # int8 quantisation error of a 512-term dot product
