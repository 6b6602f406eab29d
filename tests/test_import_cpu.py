"""Import-time behaviour on any host (no GPU needed): backend naming, module registration,
generated Tensor/Module methods, allocator configuration parser, lazy-init errors."""
import pytest
import torch


def test_backend_named_and_registered(bw):
    assert torch._C._get_privateuse1_backend_name() == "blackwell"
    assert torch.blackwell is bw
    d = torch.device("blackwell:1")
    assert d.type == "blackwell" and d.index == 1
    assert bw._C._device_type_enum() == 20


def test_generated_methods(bw):
    assert hasattr(torch.Tensor, "blackwell") and hasattr(torch.Tensor, "is_blackwell")
    assert hasattr(torch.nn.Module, "blackwell")
    assert hasattr(torch.UntypedStorage, "blackwell")
    assert torch.zeros(1).is_blackwell is False


def test_api_surface(bw):
    for name in ["device", "device_of", "set_device", "current_device", "is_available", "device_count",
                 "synchronize", "get_device_name", "get_device_capability", "get_device_properties",
                 "can_device_access_peer", "Stream", "Event", "ExternalStream", "StreamContext", "stream",
                 "current_stream", "default_stream", "set_stream", "empty_cache", "memory_stats",
                 "memory_allocated", "max_memory_allocated", "memory_reserved", "mem_get_info",
                 "set_per_process_memory_fraction", "memory_summary", "memory_snapshot", "MemPool",
                 "use_mem_pool", "change_current_allocator", "manual_seed", "manual_seed_all", "get_rng_state",
                 "set_rng_state", "seed", "initial_seed", "BlackwellGraph", "graph", "graph_pool_handle",
                 "make_graphed_callables", "update_graph_with_profile", "is_current_stream_capturing", "amp", "_lazy_init", "_sleep",
                 "use_unified_cpu_allocator", "get_allocator_backend", "ipc_collect", "OutOfMemoryError"]:
        assert hasattr(bw, name), name
    assert bw.get_arch_list() == ["sm_100a"]
    assert bw.amp.get_amp_supported_dtype() == [torch.float16, torch.bfloat16]


def test_not_available_is_clean(bw):
    if bw.is_available():
        pytest.skip("a device is present")
    assert bw.device_count() == 0
    assert not bw.is_initialized()
    with pytest.raises(RuntimeError, match="no device found|No blackwell"):
        torch.empty(1, device="blackwell")
    assert bw.memory_stats() == {}
    bw.empty_cache()  # no-op before init
    bw.manual_seed(1)  # queued, must not raise


def test_allocator_config_parser(bw):
    c = bw._C._parse_allocator_config("max_split_size_mb:128, garbage_collection_threshold:0.8,"
                                      "roundup_power2_divisions:4,expandable_segments:True,backend:unified,cpu:unified")
    assert c["max_split_size"] == 128 << 20
    assert abs(c["garbage_collection_threshold"] - 0.8) < 1e-9
    assert c["roundup_power2_divisions"] == 4 and c["expandable_segments"] is True
    assert c["backend"] == "unified" and c["cpu_unified"] is True
    for bad in ["max_split_size_mb:10", "bogus:1", "backend:foo", "garbage_collection_threshold:1.5",
                "roundup_power2_divisions:3", "nocolon"]:
        with pytest.raises(RuntimeError):
            bw._C._parse_allocator_config(bad)


def test_custom_ops_declared(bw):
    for op in ["rope", "swiglu", "swiglu_backward", "silu_mul", "silu_mul_backward", "cross_entropy_fwd",
               "cross_entropy_bwd", "cross_entropy_bwd_", "online_softmax_stats", "vocab_parallel_ce_finish",
               "rms_norm_residual", "multi_tensor_l2norm", "multi_tensor_scale_", "multi_tensor_lamb_"]:
        assert hasattr(torch.ops.blackwell, op), op


def test_amp_autocast_context_constructs(bw):
    ctx = bw.amp.autocast(dtype=torch.bfloat16)
    assert ctx.device == "blackwell" and ctx.fast_dtype == torch.bfloat16


def test_fake_tensor_rules(bw):
    from torch._subclasses.fake_tensor import FakeTensorMode

    with FakeTensorMode():
        x = torch.empty(4, 64, device="meta")
    # shape rules are plain functions: call them on meta tensors
    y = torch.ops.blackwell.swiglu(torch.empty(4, 64, device="meta"))
    assert y.shape == (4, 32)
    l, lse = torch.ops.blackwell.cross_entropy_fwd(torch.empty(8, 100, device="meta"), torch.empty(8, dtype=torch.long, device="meta"))
    assert l.shape == (8,) and l.dtype == torch.float32


def test_legacy_typed_tensor_classes(bw):
    for name, dt in [("FloatTensor", torch.float32), ("HalfTensor", torch.float16), ("BFloat16Tensor", torch.bfloat16),
                     ("LongTensor", torch.int64), ("BoolTensor", torch.bool), ("DoubleTensor", torch.float64)]:
        cls = getattr(torch.blackwell, name)
        assert cls.dtype == dt and cls.is_blackwell
        assert not isinstance(torch.zeros(1, dtype=dt), cls)        # a CPU tensor is not a device tensor
    assert repr(bw.FloatTensor) == "<class 'torch.blackwell.FloatTensor'>"


def test_small_api_surface(bw):
    import torch

    assert bw.get_gencode_flags() == "-gencode arch=compute_100a,code=sm_100a"
    assert bw.FloatStorage.dtype == torch.float32 and bw.BFloat16Storage.dtype == torch.bfloat16
    for name in ("utilization", "temperature", "power_draw", "clock_rate", "memory_usage", "list_gpu_processes",
                 "current_blas_handle", "current_blaslt_handle", "cudart", "ipc_collect", "get_pool_checkpoint"):
        assert callable(getattr(bw, name)), name
