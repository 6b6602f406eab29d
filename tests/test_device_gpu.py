"""Runtime behaviour on a real device: device selection, copies, streams, events, allocator
statistics, pinned memory, RNG, the CUDA-alias fallback.  Modelled on the reference's
tests/unittest/core/test_device.py:19-909 and test_memory.py:28-398."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_device_basics(bw, dev):
    assert bw.is_available() and bw.device_count() >= 1
    bw.set_device(0)
    assert bw.current_device() == 0
    with bw.device(0):
        assert bw.current_device() == 0
    name = bw.get_device_name(0)
    assert isinstance(name, str) and len(name) > 0
    major, minor = bw.get_device_capability(0)
    assert (major, minor) >= (10, 0), f"expected sm_100+, got {major}.{minor}"
    p = bw.get_device_properties(0)
    assert p.multi_processor_count > 0 and p.total_memory > 0
    bw.synchronize()


def test_roundtrip_and_casts(bw, dev):
    x = torch.randn(1000, 37)
    d = x.to(dev)
    assert d.device.type == "blackwell" and d.is_blackwell
    assert torch.equal(d.cpu(), x)
    assert torch.equal(d.to(torch.bfloat16).cpu(), x.to(torch.bfloat16))
    assert torch.equal(d.to(torch.float16).float().cpu(), x.to(torch.float16).float())
    # strided / transposed copies
    assert torch.equal(d.t().contiguous().cpu(), x.t().contiguous())
    assert torch.equal(d[::2, 1::3].cpu(), x[::2, 1::3])
    y = torch.empty(37, 1000, device=dev)
    y.copy_(d.t())
    assert torch.equal(y.cpu(), x.t())
    # host strided -> device
    z = x[:, ::2].to(dev)
    assert torch.equal(z.cpu(), x[:, ::2])
    # int / bool dtypes go through the generic route
    i = torch.arange(100).to(dev)
    assert torch.equal((i * 2).cpu(), torch.arange(100) * 2)
    assert float(d.sum().cpu()) == pytest.approx(float(x.sum()), rel=1e-4)
    assert d.sum().item() == pytest.approx(x.sum().item(), rel=1e-4)


def test_views_and_resize(bw, dev):
    x = torch.arange(24, dtype=torch.float32).to(dev)
    v = x.view(2, 3, 4)
    assert v.data_ptr() == x.data_ptr()
    assert torch.equal(v.permute(2, 0, 1).cpu(), torch.arange(24.).view(2, 3, 4).permute(2, 0, 1))
    assert torch.equal(x.as_strided((3, 2), (4, 1), 2).cpu(), torch.arange(24.).as_strided((3, 2), (4, 1), 2))
    assert torch.equal(x.unfold(0, 4, 4).cpu(), torch.arange(24.).unfold(0, 4, 4))
    x.resize_(30)
    assert x.numel() == 30 and torch.equal(x[:24].cpu(), torch.arange(24.))
    e = torch.empty(0, device=dev)
    e.set_(x.untyped_storage(), 0, (5,), (1,))
    assert torch.equal(e.cpu(), torch.arange(5.))


def test_streams_and_events(bw, dev):
    s0 = bw.current_stream()
    assert s0 == bw.default_stream() and s0.cuda_stream == 0
    s1 = bw.Stream()
    s2 = bw.Stream(priority=-1)
    assert s1 != s0 and s1.cuda_stream != 0
    lo, hi = bw.Stream.priority_range()
    assert lo == 0 and hi <= 0
    assert s2.priority in (hi, 0, -1)
    with bw.stream(s1):
        assert bw.current_stream() == s1
        a = torch.ones(1 << 20, device=dev)
        b = a * 2
        ev = s1.record_event()
    assert bw.current_stream() == s0
    s0.wait_event(ev)
    s0.wait_stream(s1)
    assert float(b.sum()) == 2 * (1 << 20)
    start, end = bw.Event(enable_timing=True), bw.Event(enable_timing=True)
    start.record()
    bw._sleep(2_000_000)
    end.record()
    end.synchronize()
    assert start.elapsed_time(end) > 0.1
    assert end.query() is True
    s1.synchronize()
    assert s1.query() is True
    ext = bw.ExternalStream(s1.cuda_stream)
    assert ext.cuda_stream == s1.cuda_stream


def test_record_stream_delays_reuse(bw, dev):
    s = bw.Stream()
    x = torch.empty(8 << 20, dtype=torch.uint8, device=dev)
    ptr = x.data_ptr()
    with bw.stream(s):
        bw._sleep(50_000_000)  # keep the side stream busy ~25 ms
        x.record_stream(s)
    del x
    y = torch.empty(8 << 20, dtype=torch.uint8, device=dev)
    assert y.data_ptr() != ptr, "block was recycled while another stream may still use it"
    s.synchronize()
    del y
    bw.synchronize()


def test_memory_stats(bw, dev):
    bw.synchronize()
    bw.empty_cache()
    base = bw.memory_allocated()
    x = torch.empty(64 << 20, dtype=torch.uint8, device=dev)
    assert bw.memory_allocated() - base == 64 << 20
    assert bw.memory_reserved() >= 64 << 20
    assert bw.max_memory_allocated() >= base + (64 << 20)
    del x
    assert bw.memory_allocated() == base
    assert bw.memory_reserved() >= 64 << 20  # cached
    bw.empty_cache()
    free, total = bw.mem_get_info()
    assert 0 < free <= total
    st = bw.memory_stats()
    assert "allocated_bytes.all.peak" in st and "num_ooms" in st
    assert "blackwell memory summary" in bw.memory_summary()
    snap = bw.memory_snapshot()
    assert isinstance(snap, list)
    assert bw.get_allocator_backend() in ("native", "unified", "cudaMallocAsync")


def test_oom_is_reported(bw, dev):
    free, total = bw.mem_get_info()
    with pytest.raises(torch.OutOfMemoryError):
        torch.empty(total * 2, dtype=torch.uint8, device=dev)
    assert bw.memory_stats()["num_ooms"] >= 1
    # the context is still healthy
    assert float(torch.ones(4, device=dev).sum()) == 4.0


def test_pinned_memory(bw, dev):
    h = torch.randn(1 << 16).pin_memory()
    assert h.is_pinned()
    d = h.to(dev, non_blocking=True)
    back = torch.empty_like(h).pin_memory()
    back.copy_(d, non_blocking=True)
    bw.synchronize()
    assert torch.equal(back, h)
    assert bw.host_memory_stats()["allocations"] >= 2


def test_rng_reproducible(bw, dev):
    bw.manual_seed(123)
    a = torch.randn(1000, device=dev)
    u = torch.rand(1000, device=dev)
    st = bw.get_rng_state()
    b = torch.randn(1000, device=dev)
    bw.manual_seed(123)
    a2 = torch.randn(1000, device=dev)
    assert torch.equal(a.cpu(), a2.cpu())
    bw.set_rng_state(st)
    b2 = torch.randn(1000, device=dev)
    assert torch.equal(b.cpu(), b2.cpu())
    assert abs(float(a.mean())) < 0.2 and 0.8 < float(a.std()) < 1.2
    assert 0.4 < float(u.mean()) < 0.6 and float(u.min()) >= 0 and float(u.max()) <= 1
    torch.manual_seed(7)
    c = torch.randn(10, device=dev)
    torch.manual_seed(7)
    assert torch.equal(c.cpu(), torch.randn(10, device=dev).cpu())


def test_fallback_ops_share_memory(bw, dev):
    bw.reset_fallback_counts()
    x = torch.randn(257, 33)
    d = x.to(dev)
    v, i = d.sort(dim=1)
    rv, ri = x.sort(dim=1)
    assert torch.equal(v.cpu(), rv)
    assert v.device.type == "blackwell"
    assert torch.allclose(torch.cumsum(d, 0).cpu(), torch.cumsum(x, 0), atol=1e-4, rtol=1e-4)
    m = d > 0
    assert m.dtype == torch.bool and torch.equal(m.cpu(), x > 0)
    assert torch.equal(d[m].cpu(), x[x > 0])
    w = torch.where(m, d, torch.zeros_like(d))
    assert torch.equal(w.cpu(), torch.where(x > 0, x, torch.zeros_like(x)))
    d.clamp_(min=-0.5, max=0.5)  # in-place through the fallback writes the original memory
    assert torch.equal(d.cpu(), x.clamp(-0.5, 0.5))
    out = torch.empty(0, device=dev)
    torch.mul(d, d, out=out)      # out= resize
    assert out.shape == d.shape
    # operators without a hand-written kernel (here: a matrix inverse, a complex product) take the fallback: the
    # library kernel runs on the same memory, in place / out= semantics included
    a = (torch.eye(6) * 2 + torch.randn(6, 6) * 0.1)
    inv = torch.linalg.inv(a.to(dev))
    assert inv.device.type == "blackwell" and torch.allclose(inv.cpu(), torch.linalg.inv(a), atol=1e-4)
    z = torch.randn(5, dtype=torch.complex64)
    zd = z.to(dev)
    zd.mul_(zd)
    assert torch.allclose(zd.cpu(), z * z)
    assert any("linalg_inv" in k for k in bw.fallback_counts()), bw.fallback_counts()


def test_serialization_roundtrip(bw, dev, tmp_path):
    x = torch.randn(5, 7, device=dev)
    f = tmp_path / "t.pt"
    torch.save({"x": x}, f)
    y = torch.load(f)
    assert y["x"].device.type == "blackwell" and torch.equal(y["x"].cpu(), x.cpu())
    z = torch.load(f, map_location="cpu")
    assert z["x"].device.type == "cpu"
    # a CUDA-tagged checkpoint maps onto the device
    torch.save({"c": torch.randn(3)}, f)
    w = torch.load(f, map_location="blackwell:0")
    assert w["c"].device.type == "blackwell"


def test_module_and_autocast(bw, dev):
    lin = torch.nn.Linear(64, 32).blackwell()
    x = torch.randn(16, 64, device=dev)
    with torch.autocast("blackwell", dtype=torch.bfloat16):
        y = lin(x)
        assert y.dtype == torch.bfloat16
        s = torch.softmax(y, -1)
        assert s.dtype == torch.float32
    ref = torch.nn.functional.linear(x.cpu(), lin.weight.detach().cpu(), lin.bias.detach().cpu())
    assert torch.allclose(y.float().cpu(), ref, atol=5e-2, rtol=5e-2)


def test_legacy_autograd_profiler_uses_device_stubs(bw, dev):
    """torch.autograd.profiler with use_device='blackwell' times operators through the backend's profiler stubs
    (skipped where this torch build no longer offers the legacy, non-Kineto profiler)."""
    x = torch.randn(512, 512, device=dev)
    try:
        with torch.autograd.profiler.profile(use_device="blackwell", use_kineto=False) as prof:
            for _ in range(3):
                (x @ x).relu_()
            bw.synchronize()
        table = prof.key_averages().table(sort_by="self_cpu_time_total", row_limit=5)
    except (RuntimeError, AssertionError, TypeError, ValueError) as e:
        pytest.skip(f"legacy autograd profiler unavailable here: {e}")
    assert "aten::mm" in table


def test_legacy_typed_tensor_classes_on_device(bw, dev):
    t = bw.FloatTensor(2, 3)
    assert t.shape == (2, 3) and t.dtype == torch.float32 and t.device.type == "blackwell"
    assert isinstance(t, bw.FloatTensor) and not isinstance(t, bw.HalfTensor)
    h = bw.HalfTensor([1.0, 2.0, 3.0])
    assert isinstance(h, bw.HalfTensor) and h.cpu().tolist() == [1.0, 2.0, 3.0]
    assert isinstance(bw.LongTensor(torch.arange(4)), bw.LongTensor)
    assert bw.BFloat16Tensor().numel() == 0


def test_cpp_example_runs(bw):
    import os
    import subprocess

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run(["make", "-C", os.path.join(root, "examples", "cpp")], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    r = subprocess.run([os.path.join(root, "examples", "cpp", "rmsnorm_example")], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "max abs error" in r.stdout


def test_stream_guards_and_event_cache(bw, dev):
    """MultiStreamGuard / OptionalStreamGuard set and restore the current streams; finished events are reused."""
    a, b = bw.Stream(), bw.Stream()
    before = bw.current_stream().stream_id
    inside, after = bw._C._multi_stream_guard_probe([(a.stream_id, a.device_index)])
    assert inside == [a.stream_id] and after == [before]
    hits0, _ = bw._C._event_cache_stats()
    cur = bw.current_stream()
    for _ in range(4):
        e = bw._C._IpcEvent(interprocess=False)      # the runtime's own event class
        e.record(cur.stream_id, cur.device_index)
        e.synchronize()
        del e                                        # goes back to the cache, the next one reuses it
    assert bw._C._event_cache_stats()[0] >= hits0 + 3


def test_current_blas_handle(bw, dev):
    h = bw.current_blas_handle()
    assert isinstance(h, int) and h != 0


def test_fft_plan_cache(bw, dev):
    cache = torch.backends.blackwell.fft_plan_cache[bw.current_device()]
    cache.clear()
    x = torch.randn(8, 256, device=dev)
    y = torch.fft.rfft(x)
    assert torch.allclose(torch.view_as_real(y).cpu(), torch.view_as_real(torch.fft.rfft(x.cpu())), atol=1e-3)
    assert cache.size >= 1
    cache.max_size = 8
    assert cache.max_size == 8


def test_memory_snapshot_pickle_format(bw, dev, tmp_path):
    """The dumped snapshot has the layout torch's memory visualiser reads: segments with blocks, device traces."""
    import pickle

    bw._record_memory_history(True, 1000, stacks="cpp")
    keep = [torch.empty(1 << 20, device=dev) for _ in range(3)]
    del keep[1]
    path = str(tmp_path / "snap.pickle")
    bw._dump_snapshot(path)
    bw._record_memory_history(None)
    snap = pickle.load(open(path, "rb"))
    assert set(snap) >= {"segments", "device_traces"}
    seg = snap["segments"][0]
    assert {"address", "total_size", "allocated_size", "stream", "segment_type", "blocks"} <= set(seg)
    assert {"size", "requested_size", "state"} <= set(seg["blocks"][0])
    actions = {t["action"] for t in snap["device_traces"][bw.current_device()]}
    assert {"alloc", "free_requested"} <= actions or {"alloc", "free_completed"} <= actions
    allocs = [t for t in snap["device_traces"][bw.current_device()] if t["action"] == "alloc"]
    assert allocs and len(allocs[-1].get("frames", "")) > 20        # the call site's frames were recorded


def test_telemetry_and_legacy_storage(bw, dev):
    s = bw.FloatStorage(16)
    assert s.device.type == "blackwell" and s.dtype == torch.float32 and len(s) == 16
    assert bw.current_blaslt_handle() != 0
    assert bw.cudart().cudaMemGetInfo(0)[1] > (100 << 30)
    try:
        t, p, c = bw.temperature(), bw.power_draw(), bw.clock_rate()
    except (RuntimeError, ModuleNotFoundError):
        pytest.skip("NVML is not reachable in this container")
    assert 0 < t < 120 and p > 0 and 0 < c <= 2500
    assert 0 <= bw.utilization() <= 100
    assert "GPU:0" in bw.list_gpu_processes()
