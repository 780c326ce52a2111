"""The allocation-free RMSNorm-backward entry point, called through its exported
C symbol the way an embedding host would (no torch allocation inside the call),
against the regular launcher.

Such hosts pre-partition device memory at start-up and cannot let a library
call cudaMalloc later; they pass inputs and outputs and rely on the workspace
that ships inside the library image.  Two calls in a row with different data
check that what the first call left in the shared workspace does not leak into
the second.  This file is collected last on purpose.
"""
import ctypes as C

import pytest
import torch

from chaoscontrol_b200.ops import _lib

pytestmark = pytest.mark.gpu


def _sym():
    lib = C.CDLL(str(_lib.lib_path()))
    fn = lib.ccb_rmsnorm_bwd_noalloc
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                   C.c_int64, C.c_int64, C.c_void_p]
    fn.restype = C.c_int
    err = lib.ccb_last_error
    err.restype = C.c_char_p
    return fn, err


def _inputs(R, D, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(R, D, device="cuda", generator=g).bfloat16()
    w = (torch.rand(D, device="cuda", generator=g) + 0.5).bfloat16()
    go = torch.randn(R, D, device="cuda", generator=g).bfloat16()
    inv = torch.rsqrt((x.float() ** 2).mean(-1) + 1e-6)
    return x, w, go, inv


def _regular(x, w, go, inv):
    L = _lib.lib()
    R, D = x.shape
    gx = torch.empty_like(x)
    nb = int(L.ccb_rmsnorm_bwd_blocks(R))
    part = torch.empty(nb, D, dtype=torch.float32, device="cuda")
    gw = torch.empty(D, dtype=torch.float32, device="cuda")
    _lib.check(L.ccb_rmsnorm_bwd(x.data_ptr(), w.data_ptr(), go.data_ptr(), inv.data_ptr(),
                                 gx.data_ptr(), part.data_ptr(), gw.data_ptr(), R, D,
                                 _lib.stream_ptr()), "rmsnorm_bwd")
    return gx, gw


def _check_pair(fn, err, R, D, seed, *, measure_free: bool):
    x, w, go, inv = _inputs(R, D, seed)
    ref_gx, ref_gw = _regular(x, w, go, inv)
    gx = torch.empty_like(x)
    gw = torch.empty(D, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    # the call goes straight to the CUDA runtime, so torch's allocator statistics cannot see what it
    # does: ask the driver how much device memory is free before and after instead (cudaMemGetInfo)
    free_before = torch.cuda.mem_get_info()[0]
    rc = fn(x.data_ptr(), w.data_ptr(), go.data_ptr(), inv.data_ptr(), gx.data_ptr(),
            gw.data_ptr(), R, D, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, err().decode()
    torch.cuda.synchronize()
    if measure_free:
        assert torch.cuda.mem_get_info()[0] == free_before, "the allocation-free entry point changed free memory"
    assert torch.allclose(gx.float(), ref_gx.float(), rtol=2e-2, atol=2e-2)
    assert torch.allclose(gw, ref_gw, rtol=1e-3, atol=1e-2 * max(1.0, (R / 4096) ** 0.5))
    # and against the plain fp32 formula
    xh = x.float() * inv[:, None]
    exp_gw = (go.float() * xh).sum(0)
    assert torch.allclose(gw, exp_gw, rtol=2e-2, atol=0.5 * max(1.0, (R / 4096) ** 0.5))


def test_noalloc_rmsnorm_bwd_matches_regular_twice():
    fn, err = _sym()
    # first call on this device: looks up the built-in workspace (and may load the module lazily),
    # so free memory is only compared on the calls after it
    _check_pair(fn, err, 256, 128, 9, measure_free=False)
    for seed, (R, D) in enumerate([(4096, 256), (1000, 512)]):
        _check_pair(fn, err, R, D, seed, measure_free=True)


def test_noalloc_largest_problem_fills_the_whole_workspace():
    """65 536 rows x 1 024 channels uses every slot of the 1 MiB built-in array."""
    fn, err = _sym()
    _check_pair(fn, err, 65536, 1024, 5, measure_free=True)


def test_noalloc_rejects_oversize():
    fn, err = _sym()
    x, w, go, inv = _inputs(8, 64, 3)
    rc = fn(x.data_ptr(), w.data_ptr(), go.data_ptr(), inv.data_ptr(), x.data_ptr(), inv.data_ptr(),
            65537, 64, None)
    assert rc != 0 and b"exceeds" in err()
    rc = fn(x.data_ptr(), w.data_ptr(), go.data_ptr(), inv.data_ptr(), x.data_ptr(), inv.data_ptr(),
            8, 2048, None)
    assert rc != 0 and b"unsupported" in err()
    rc = fn(x.data_ptr(), w.data_ptr(), go.data_ptr(), inv.data_ptr(), x.data_ptr(), inv.data_ptr(),
            8, 63, None)                                   # odd channel count
    assert rc != 0 and b"unsupported" in err()
