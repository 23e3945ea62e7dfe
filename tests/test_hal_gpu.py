"""Native CUDA runtime binding and graph validation over real captures."""
import ctypes as C

import pytest
import torch

from ml_framework_b200.hal import cuda_rt
from ml_framework_b200.hal.cuda_graphs import CaptureOptions, CUDAGraphManager, GraphValidator, ValidationSeverity

pytestmark = pytest.mark.gpu


def test_runtime_binding_devices_memory_streams_events():
    assert cuda_rt.device_count() >= 1
    props = cuda_rt.device_properties(cuda_rt.current_device())
    assert props["multiprocessors"] > 0 and props["compute_capability"][0] >= 9 and props["total_memory_mib"] > 1000
    free, total = cuda_rt.mem_info()
    assert 0 < free <= total
    n = 1 << 20
    dev, host = cuda_rt.DeviceBuffer(n), cuda_rt.DeviceBuffer(n, pinned_host=True)
    st = cuda_rt.Stream()
    e0, e1 = cuda_rt.Event(), cuda_rt.Event()
    e0.record(st)
    dev.memset(0x5A, st)
    cuda_rt.memcpy(host.ptr, dev.ptr, n, "d2h", st)
    e1.record(st)
    e1.synchronize()
    assert e1.query() and st.query() and e0.elapsed_ms(e1) >= 0.0
    buf = (C.c_ubyte * 16).from_address(host.ptr)
    assert list(buf) == [0x5A] * 16
    other = cuda_rt.Stream()
    other.wait_event(e1)
    other.synchronize()
    for o in (dev, host, st, other, e0, e1):
        o.close()
    with pytest.raises(cuda_rt.CudaRuntimeError):
        cuda_rt.DeviceBuffer(1 << 60)
    cuda_rt.synchronize()


def test_native_capture_node_census_and_replay():
    n = 4096
    a, b = cuda_rt.DeviceBuffer(n), cuda_rt.DeviceBuffer(n)
    st = cuda_rt.Stream()
    st.begin_capture("thread_local")
    assert st.is_capturing()
    a.memset(7, st)
    cuda_rt.memcpy(b.ptr, a.ptr, n, "d2d", st)
    g = st.end_capture()
    kinds = g.node_kinds()
    assert sorted(kinds) == ["memcpy", "memset"]
    v = GraphValidator()
    assert [i for i in v.validate_graph(g) if i.severity == ValidationSeverity.ERROR] == []
    ex = g.instantiate()
    b.memset(0)
    cuda_rt.synchronize()
    ex.launch(st)
    st.synchronize()
    out = torch.empty(n, dtype=torch.uint8, device="cuda")
    cuda_rt.memcpy(out.data_ptr(), b.ptr, n, "d2d")
    assert int(out.min()) == 7 and int(out.max()) == 7
    # an empty capture is rejected by the validator
    st.begin_capture("thread_local")
    empty = st.end_capture()
    assert any(i.rule == "EmptyGraph" for i in v.validate_graph(empty))
    for o in (ex, g, empty, st, a, b):
        o.close()


def test_manager_validates_the_real_capture_of_a_kernel_sequence():
    from ml_framework_b200.ops import native
    mgr = CUDAGraphManager(CaptureOptions(warmup_iterations=1))
    x = torch.randn(1024, 256, device="cuda").to(torch.bfloat16)
    w = torch.ones(256, device="cuda", dtype=torch.bfloat16)

    def fn(t):
        return native.norm_fwd(t, w, None, 1e-5, True, want_stats=False)[0]

    want = fn(x).clone()
    for _ in range(3):
        out = mgr.run("norm", fn, x)
    cg = next(iter(mgr._graphs.values()))
    assert cg.replays >= 1 and "kernel" in cg.node_kinds
    assert not any(i.severity == ValidationSeverity.ERROR for i in cg.issues)
    assert torch.allclose(out.float(), want.float(), atol=1e-2)
