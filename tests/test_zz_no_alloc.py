"""Allocation-free GLA forward (libtriune_noalloc.so), called through its exported C symbol.

Some callers of this library cannot allocate device memory while they run: a serving loop that was given a fixed
memory plan, a plugin that receives a device but no allocator, or code that must not pay the device-wide
synchronisation of a cudaMalloc in the middle of a request. For them ``triune_gla_forward_noalloc`` runs the same
kernels as the regular entry point with the scratch taken from an array built into the library. This test calls
it twice in a row (the array keeps the previous call's contents, so the second call checks that nothing stale
leaks through) and compares both results with the regular, allocating entry point.

The file name sorts last on purpose: with ``pytest -x`` every other test has already run when this one starts.
"""

import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "triune_b200", "libtriune_noalloc.so")


def _load():
    if not os.path.exists(LIB):
        pytest.skip("libtriune_noalloc.so is not built")
    lib = ctypes.CDLL(LIB)
    vp = ctypes.c_void_p
    lib.triune_gla_forward_noalloc.restype = ctypes.c_int
    lib.triune_gla_forward_noalloc.argtypes = [vp, vp, vp, vp, vp, vp, vp, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                               ctypes.c_int, vp, vp]
    lib.triune_gla_noalloc_scratch_bytes.restype = ctypes.c_ulonglong
    return lib


def _call(lib, q, k, v, g, init, B, T, H):
    out = torch.empty(B * T, H * 64, device=q.device, dtype=torch.bfloat16)
    fin = torch.empty(B * H, 64, 64, device=q.device, dtype=torch.float32)
    status = torch.full((1,), -1, dtype=torch.int32).pin_memory()
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.triune_gla_forward_noalloc(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), out.data_ptr(),
                                        fin.data_ptr(), init.data_ptr() if init is not None else None, B, T, H, 1,
                                        status.data_ptr(), stream)
    torch.cuda.synchronize()
    return rc, out, fin, int(status.item())


def test_noalloc_entry_matches_regular_entry_twice():
    from triune_b200 import _ext

    lib = _load()
    assert lib.triune_gla_noalloc_scratch_bytes() < 16 * 1024 * 1024
    dev = torch.device("cuda", 0)
    e = _ext.ext()
    for call, (B, T, H, seed, with_init) in enumerate(((2, 256, 3, 1, False), (1, 128, 2, 2, True))):
        torch.manual_seed(seed)
        q, k, v, g = (torch.randn(B * T, H * 64, device=dev).to(torch.bfloat16) for _ in range(4))
        q, k = q.abs() * 0.2, k.abs() * 0.2
        init = (torch.randn(B * H, 64, 64, device=dev) * 0.1) if with_init else None
        ref_out = torch.empty(B * T, H * 64, device=dev, dtype=torch.bfloat16)
        _, _, ref_fin, ref_status = e.gla_fwd(q, 0, k, 0, v, 0, g, 0, ref_out, 0, init, B, T, H, True)
        torch.cuda.synchronize()
        assert int(ref_status.item()) == 0
        rc, out, fin, status = _call(lib, q, k, v, g, init, B, T, H)
        assert rc == 0 and status == 0, (call, rc, status)
        scale = float(ref_out.float().abs().max().clamp_min(1e-6))
        assert float((out.float() - ref_out.float()).abs().max()) <= 2e-2 * scale, call
        fscale = float(ref_fin.abs().max().clamp_min(1e-6))
        assert float((fin - ref_fin.view_as(fin)).abs().max()) <= 2e-2 * fscale, call


def test_noalloc_entry_rejects_oversized_and_bad_arguments():
    lib = _load()
    dev = torch.device("cuda", 0)
    x = torch.zeros(64, 64, device=dev, dtype=torch.bfloat16)
    fin = torch.zeros(1, 64, 64, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    args = (x.data_ptr(),) * 4 + (x.data_ptr(), fin.data_ptr(), None)
    assert lib.triune_gla_forward_noalloc(*args, 64, 64 * 64, 1, 1, None, stream) == -2  # 4096 chunks > 512
    assert lib.triune_gla_forward_noalloc(*args, 1, 100, 1, 1, None, stream) == -1       # T not a multiple of 64
    torch.cuda.synchronize()


def test_noalloc_entry_at_the_scratch_limit():
    """Exactly 512 chunks (the whole built-in array) must work and agree with the regular entry; one chunk more is
    refused with -2 before anything is launched."""
    from triune_b200 import _ext

    lib = _load()
    dev = torch.device("cuda", 0)
    e = _ext.ext()
    B, T, H = 4, 4096, 2  # 4 * 2 * 64 = 512 chunks
    torch.manual_seed(3)
    q, k, v, g = (torch.randn(B * T, H * 64, device=dev).to(torch.bfloat16) for _ in range(4))
    q, k = q.abs() * 0.2, k.abs() * 0.2
    ref_out = torch.empty(B * T, H * 64, device=dev, dtype=torch.bfloat16)
    _, _, ref_fin, ref_status = e.gla_fwd(q, 0, k, 0, v, 0, g, 0, ref_out, 0, None, B, T, H, True)
    torch.cuda.synchronize()
    assert int(ref_status.item()) == 0
    rc, out, fin, status = _call(lib, q, k, v, g, None, B, T, H)
    assert rc == 0 and status == 0
    scale = float(ref_out.float().abs().max().clamp_min(1e-6))
    assert float((out.float() - ref_out.float()).abs().max()) <= 2e-2 * scale
    fscale = float(ref_fin.abs().max().clamp_min(1e-6))
    assert float((fin - ref_fin.view_as(fin)).abs().max()) <= 2e-2 * fscale
    # 513 chunks: B=513, T=64, H=1
    x = torch.zeros(64, 64, device=dev, dtype=torch.bfloat16)
    f1 = torch.zeros(1, 64, 64, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    args = (x.data_ptr(),) * 4 + (x.data_ptr(), f1.data_ptr(), None)
    assert lib.triune_gla_forward_noalloc(*args, 513, 64, 1, 1, None, stream) == -2
    torch.cuda.synchronize()


def test_noalloc_entry_on_a_second_device():
    """The scratch address and the kernels' shared-memory attributes are per device: the first call on another GPU
    of the same process has to set them up again."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two visible GPUs")
    from triune_b200 import _ext

    lib = _load()
    e = _ext.ext()
    B, T, H = 1, 128, 2
    for ordinal in (0, 1):
        dev = torch.device("cuda", ordinal)
        with torch.cuda.device(dev):
            torch.manual_seed(4 + ordinal)
            q, k, v, g = (torch.randn(B * T, H * 64, device=dev).to(torch.bfloat16) for _ in range(4))
            q, k = q.abs() * 0.2, k.abs() * 0.2
            ref_out = torch.empty(B * T, H * 64, device=dev, dtype=torch.bfloat16)
            _, _, ref_fin, _ = e.gla_fwd(q, 0, k, 0, v, 0, g, 0, ref_out, 0, None, B, T, H, True)
            rc, out, fin, status = _call(lib, q, k, v, g, None, B, T, H)
            assert rc == 0 and status == 0, ordinal
            scale = float(ref_out.float().abs().max().clamp_min(1e-6))
            assert float((out.float() - ref_out.float()).abs().max()) <= 2e-2 * scale, ordinal
