"""The allocation-free L2-norm entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory when they need a gradient norm (a host
application that owns all device memory and exposes no allocator, a diagnostic path that runs when the
allocator itself has failed).  ``b200_multi_tensor_l2norm_static`` serves them from a fixed array inside
the library.  This test drives it with ctypes -- no torch operator in between -- twice in a row, and
compares it with the ordinary entry point (caller-provided scratch) on the same inputs.
Collected last on purpose (file name), so a failure here cannot hide other tests under ``-x``.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

B200_F32, B200_BF16 = 0, 1


def _lib():
    import torch_musa_b200 as bw

    path = os.path.join(os.path.dirname(bw.__file__), "libb200_kernels.so")
    lib = ctypes.CDLL(path)
    lib.b200_multi_tensor_l2norm_static.restype = ctypes.c_int
    lib.b200_multi_tensor_l2norm_static.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_void_p),
                                                    ctypes.POINTER(ctypes.c_int64), ctypes.c_void_p, ctypes.c_void_p,
                                                    ctypes.c_void_p]
    lib.b200_multi_tensor_l2norm.restype = ctypes.c_int
    lib.b200_multi_tensor_l2norm.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_void_p),
                                             ctypes.POINTER(ctypes.c_int64), ctypes.c_void_p, ctypes.c_void_p,
                                             ctypes.c_void_p, ctypes.c_void_p]
    lib.b200_multi_tensor_l2norm_scratch_floats.restype = ctypes.c_size_t
    lib.b200_multi_tensor_l2norm_scratch_floats.argtypes = [ctypes.c_int]
    return lib


def _args(tensors):
    n = len(tensors)
    ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in tensors])
    numels = (ctypes.c_int64 * n)(*[t.numel() for t in tensors])
    return n, ptrs, numels


@pytest.mark.parametrize("dtype,code", [(torch.float32, B200_F32), (torch.bfloat16, B200_BF16)])
def test_static_l2norm_matches_regular_entry_point(bw, dev, dtype, code):
    lib = _lib()
    bw.set_device(0)
    stream = bw.current_stream().cuda_stream
    for round_ in range(2):  # two calls in a row share the library's array
        torch.manual_seed(round_)
        tensors = [torch.randn(n, device=dev).to(dtype) for n in (3, 1000, 70001, 5 << 20, 17)]
        n, ptrs, numels = _args(tensors)
        tot_s = torch.zeros(1, device=dev)
        per_s = torch.zeros(n, device=dev)
        rc = lib.b200_multi_tensor_l2norm_static(n, code, ptrs, numels, tot_s.data_ptr(), per_s.data_ptr(), stream)
        assert rc == 0, rc
        tot_r = torch.zeros(1, device=dev)
        per_r = torch.zeros(n, device=dev)
        scratch = torch.empty(lib.b200_multi_tensor_l2norm_scratch_floats(n), device=dev)
        rc = lib.b200_multi_tensor_l2norm(n, code, ptrs, numels, tot_r.data_ptr(), per_r.data_ptr(),
                                          scratch.data_ptr(), stream)
        assert rc == 0, rc
        bw.synchronize()
        assert torch.allclose(per_s.cpu(), per_r.cpu(), rtol=1e-6, atol=0)
        assert torch.allclose(tot_s.cpu(), tot_r.cpu(), rtol=1e-6, atol=0)
        ref = torch.stack([t.cpu().double().norm() for t in tensors]).float()  # fp64 oracle: a 5M-element fp32 sum drifts
        assert torch.allclose(per_s.cpu(), ref, rtol=1e-4)
        assert float(tot_s) == pytest.approx(float(ref.norm()), rel=1e-4)


def test_static_l2norm_rejects_oversize_lists(bw, dev):
    lib = _lib()
    bw.set_device(0)
    t = torch.ones(8, device=dev)
    n = 1025
    ptrs = (ctypes.c_void_p * n)(*([t.data_ptr()] * n))
    numels = (ctypes.c_int64 * n)(*([8] * n))
    out = torch.zeros(1, device=dev)
    rc = lib.b200_multi_tensor_l2norm_static(n, B200_F32, ptrs, numels, out.data_ptr(), None, 0)
    assert rc == 1  # cudaErrorInvalidValue: refused before anything is launched
    bw.synchronize()
    assert float(out) == 0.0


@pytest.mark.parametrize("n_tensors", [300, 1024])
def test_static_l2norm_many_tensors_without_per_tensor_output(bw, dev, n_tensors):
    """The cases that depend on the fixed sizing: several clean-up batches (more than 128 tensors), the 1024-tensor
    boundary, and no per-tensor output (the per-tensor norms then live in the array's last n floats)."""
    lib = _lib()
    bw.set_device(0)
    stream = bw.current_stream().cuda_stream
    torch.manual_seed(n_tensors)
    sizes = [1 + (i * 37) % 513 for i in range(n_tensors)]
    sizes[7] = 300001                                   # one tensor that spans many chunks
    tensors = [torch.randn(s, device=dev) for s in sizes]
    n, ptrs, numels = _args(tensors)
    for _ in range(2):
        tot = torch.zeros(1, device=dev)
        rc = lib.b200_multi_tensor_l2norm_static(n, B200_F32, ptrs, numels, tot.data_ptr(), None, stream)
        assert rc == 0, rc
        bw.synchronize()
        ref = torch.cat([t.cpu().double().reshape(-1) for t in tensors]).norm()
        assert float(tot) == pytest.approx(float(ref), rel=1e-5)
