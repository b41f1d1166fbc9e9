"""nvfp4_tensor_amax_f32_static_scratch (the entry that allocates nothing) against
nvfp4_tensor_amax_f32, through the C ABI.  Collected last on purpose: it has to pass both alone
and after every other GPU test has used the library in the same process."""
import ctypes

import numpy as np
import pytest
import torch

import __graft_entry__ as entry

pytestmark = pytest.mark.gpu

MAX_ELEMENTS = 1 << 26


def _lib():
    pkg = entry.load_package()
    return pkg, pkg.library()


def _pair(lib, x, out_static, out_ref):
    """Both entries on the current stream; returns (static, existing) results."""
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    n = x.numel()
    chunks = torch.empty(max(1, (n + 1023) // 1024), dtype=torch.float32, device=x.device)
    rc = lib.nvfp4_tensor_amax_f32_static_scratch(stream, ctypes.c_void_p(x.data_ptr()),
                                                  ctypes.c_void_p(out_static.data_ptr()), n)
    assert rc == 0, lib.nvfp4_last_error()
    rc = lib.nvfp4_tensor_amax_f32(stream, ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(chunks.data_ptr()),
                                   ctypes.c_void_p(out_ref.data_ptr()), n)
    assert rc == 0, lib.nvfp4_last_error()
    torch.cuda.synchronize()
    return out_static.cpu().numpy().copy(), out_ref.cpu().numpy().copy()


def test_static_scratch_matches_existing_entry_on_consecutive_calls():
    _, lib = _lib()
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(77)
    out_static = torch.full((1,), -1.0, dtype=torch.float32, device=dev)
    out_ref = torch.full((1,), -2.0, dtype=torch.float32, device=dev)
    # a large tensor first, then smaller ones: stale slots of the earlier call must not leak
    sizes = [(1 << 22) + 3, 1024 * 37 + 5, 1000, 1, 16 * 1024, (1 << 20)]
    for i, n in enumerate(sizes):
        x = torch.randn(n, generator=gen, dtype=torch.float32) * (10.0 ** (2 - i))
        x[(n * 2) // 3] = -float(3 * abs(x).max())  # the maximum sits on a negative value
        a, b = _pair(lib, x.to(dev), out_static, out_ref)
        assert a.tobytes() == b.tobytes(), (n, a, b)
        assert a[0] == np.abs(x.numpy()).max()
    # the same input twice in a row gives the same answer
    x = torch.randn(123457, generator=gen, dtype=torch.float32).to(dev)
    first, ref = _pair(lib, x, out_static, out_ref)
    second, _ = _pair(lib, x, out_static, out_ref)
    assert first.tobytes() == second.tobytes() == ref.tobytes()


def test_static_scratch_unaligned_and_empty():
    _, lib = _lib()
    dev = torch.device("cuda:0")
    out_static = torch.full((1,), -1.0, dtype=torch.float32, device=dev)
    out_ref = torch.full((1,), -2.0, dtype=torch.float32, device=dev)
    base = torch.randn(8192 + 1, generator=torch.Generator().manual_seed(5), dtype=torch.float32).to(dev)
    a, b = _pair(lib, base[1:], out_static, out_ref)  # 4-byte aligned only
    assert a.tobytes() == b.tobytes()
    a, b = _pair(lib, base[:0], out_static, out_ref)
    assert a[0] == 0.0 and b[0] == 0.0


def test_static_scratch_rejects_oversize():
    pkg, lib = _lib()
    dev = torch.device("cuda:0")
    out = torch.full((1,), -1.0, dtype=torch.float32, device=dev)
    x = torch.zeros(16, dtype=torch.float32, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # the size is checked before anything is launched, so the small buffer is never read
    rc = lib.nvfp4_tensor_amax_f32_static_scratch(stream, ctypes.c_void_p(x.data_ptr()),
                                                  ctypes.c_void_p(out.data_ptr()), MAX_ELEMENTS + 1)
    assert rc == 1
    assert b"exceeds the built-in scratch" in lib.nvfp4_last_error()
    torch.cuda.synchronize()
    assert out.item() == -1.0
    with pytest.raises(pkg.Nvfp4Error):  # the Python mirror turns the code into an exception
        pkg._call("nvfp4_tensor_amax_f32_static_scratch", stream, ctypes.c_void_p(x.data_ptr()),
                  ctypes.c_void_p(out.data_ptr()), MAX_ELEMENTS + 1)


def test_static_scratch_at_the_limit():
    pkg, lib = _lib()
    dev = torch.device("cuda:0")
    out_static = torch.empty(1, dtype=torch.float32, device=dev)
    out_ref = torch.empty(1, dtype=torch.float32, device=dev)
    x = torch.zeros(MAX_ELEMENTS, dtype=torch.float32, device=dev)
    x[MAX_ELEMENTS - 1] = -7.5
    x[12345] = 7.25
    a, b = _pair(lib, x, out_static, out_ref)
    assert a.tobytes() == b.tobytes() and a[0] == 7.5
    q = pkg.Nvfp4QuantModule()
    assert q.tensor_amax_f32_static_scratch(x, out_static).item() == 7.5
