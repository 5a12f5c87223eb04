"""The allocation-free RMSNorm backward entry point, called through its exported C symbol.

Some callers may not allocate device memory at all (a serving loop with a fixed memory budget, a
process whose device memory belongs to another allocator). For them the library keeps the fp32
scratch of the weight gradient inside its own image; this test checks that the entry point gives
the same dx and dw as the regular one, twice in a row (the second call meets the first call's
left-overs in the shared scratch), and that it refuses rows wider than its scratch.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from rocm_systems_b200 import _lib

    lib = _lib.load()
    vp, ll, i32 = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
    lib.b200ops_rmsnorm_bwd_noalloc.argtypes = [vp, vp, vp, vp, vp, vp, ll, i32, vp]
    lib.b200ops_rmsnorm_bwd_noalloc.restype = i32
    lib.b200ops_rmsnorm_bwd_noalloc_error.restype = ctypes.c_char_p
    lib.b200ops_rmsnorm_bwd.argtypes = [vp, vp, vp, vp, vp, vp, ll, i32, vp]
    lib.b200ops_rmsnorm_bwd.restype = i32
    return lib


def test_noalloc_matches_regular_entry_point_twice():
    lib = _lib()
    torch.cuda.set_device(0)
    s = torch.cuda.current_stream().cuda_stream
    for call, (T, H) in enumerate([(96, 4096), (33, 1024)]):  # the second call is narrower: stale tail in the scratch
        g = torch.Generator(device="cuda").manual_seed(100 + call)
        x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
        w = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).to(torch.bfloat16)
        dy = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5).contiguous()
        # regular entry point: the caller brings the fp32 accumulator
        dx_ref = torch.empty_like(x)
        dw32 = torch.zeros(H, dtype=torch.float32, device="cuda")
        assert lib.b200ops_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx_ref.data_ptr(), dw32.data_ptr(), T, H, s) == 0
        dw_ref = dw32.to(torch.bfloat16)
        # allocation-free entry point: outputs only
        dx = torch.empty_like(x)
        dw = torch.empty(H, dtype=torch.bfloat16, device="cuda")
        rc = lib.b200ops_rmsnorm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), T, H, s)
        assert rc == 0, lib.b200ops_rmsnorm_bwd_noalloc_error().decode()
        torch.cuda.synchronize()
        assert torch.equal(dx, dx_ref)
        # fp32 atomics add in a different order from run to run: compare within the tolerance of the other kernel tests
        assert torch.allclose(dw.float(), dw_ref.float(), rtol=3e-2, atol=3e-2)


def test_noalloc_refuses_rows_wider_than_its_scratch():
    lib = _lib()
    torch.cuda.set_device(0)
    z = torch.zeros(8, device="cuda")
    rc = lib.b200ops_rmsnorm_bwd_noalloc(z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), 1, 16384, 0)
    assert rc == -2
    assert b"at most 8192" in lib.b200ops_rmsnorm_bwd_noalloc_error()
