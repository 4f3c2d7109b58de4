"""The allocation-free RMSNorm backward, called through its exported C symbol, against the regular operator.
Named so that it is collected after the other GPU tests; it also passes when run alone."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


@pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a GPU")
def test_static_scratch_rmsnorm_bwd_matches_regular_entry_point():
    from verl_b200.ops import native

    lib, ops = native.cdll(), native.ops()
    fn = lib.vb_rmsnorm_bwd_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int] * 3 + [ctypes.c_void_p]
    lib.vb_rmsnorm_bwd_static_strerror.restype = ctypes.c_char_p
    lib.vb_rmsnorm_bwd_static_strerror.argtypes = [ctypes.c_int]
    dev = torch.device("cuda", 0)
    torch.manual_seed(3)
    # calls in a row on shrinking and growing problems: two, one and four 16-byte packets per thread, the largest row
    # length the buffer covers, and fewer rows than blocks
    for call, (T, H) in enumerate([(1000, 3584), (77, 1024), (300, 8192), (5, 5120)]):
        x, dy, dres = (torch.randn(T, H, device=dev).bfloat16() for _ in range(3))
        w = (torch.rand(H, device=dev) + 0.5).bfloat16()
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
        dw_ref = torch.full((H,), 0.25, device=dev)
        dx_ref = ops.rmsnorm_bwd(dy, x, w, rstd, dres, dw_ref, True)
        dw = torch.full((H,), 0.25, device=dev)
        dx = torch.empty_like(x)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated(dev)
        rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres.data_ptr(), dx.data_ptr(), dw.data_ptr(),
                T, H, 1, torch.cuda.current_stream(dev).cuda_stream)
        assert rc == 0, lib.vb_rmsnorm_bwd_static_strerror(rc).decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated(dev) == before
        assert _rel(dx, dx_ref) < 1e-2 and _rel(dw, dw_ref) < 1e-4, (call, _rel(dx, dx_ref), _rel(dw, dw_ref))
        # overwrite mode and no incoming residual gradient
        dw2, dw2_ref = torch.empty(H, device=dev), torch.zeros(H, device=dev)
        dx2_ref = ops.rmsnorm_bwd(dy, x, w, rstd, None, dw2_ref, False)
        rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), None, dx.data_ptr(), dw2.data_ptr(), T, H, 0,
                torch.cuda.current_stream(dev).cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert _rel(dx, dx2_ref) < 1e-2 and _rel(dw2, dw2_ref) < 1e-4
    # no rows: dw is zeroed in overwrite mode, kept in accumulate mode, dx is not touched
    H = 1024
    t = torch.zeros(8, H, device=dev).bfloat16()
    r1 = torch.ones(8, device=dev)
    dw0 = torch.full((H,), 3.0, device=dev)
    sentinel = torch.full((8, H), 7.0, device=dev).bfloat16()
    args = (t.data_ptr(), t.data_ptr(), t[0].data_ptr(), r1.data_ptr(), None, sentinel.data_ptr(), dw0.data_ptr())
    assert fn(*args, 0, H, 1, torch.cuda.current_stream(dev).cuda_stream) == 0
    torch.cuda.synchronize()
    assert bool((dw0 == 3.0).all())
    assert fn(*args, 0, H, 0, torch.cuda.current_stream(dev).cuda_stream) == 0
    torch.cuda.synchronize()
    assert bool((dw0 == 0.0).all()) and bool((sentinel == 7.0).all())
    # null and misaligned pointers are turned away on the host (codes -5 / -6); nothing is launched
    good = [t.data_ptr(), t.data_ptr(), t[0].data_ptr(), r1.data_ptr(), None, sentinel.data_ptr(), dw0.data_ptr()]
    for i in (0, 1, 2, 3, 5, 6):
        bad = list(good)
        bad[i] = None
        rc = fn(*bad, 8, H, 0, None)
        assert rc == -5 and b"null" in lib.vb_rmsnorm_bwd_static_strerror(rc)
    for i in (0, 1, 2, 4, 5):
        bad = list(good)
        bad[i] = t.data_ptr() + 2  # one bf16 element off a 16-byte boundary
        rc = fn(*bad, 8, H, 0, None)
        assert rc == -6 and b"aligned" in lib.vb_rmsnorm_bwd_static_strerror(rc)
    torch.cuda.synchronize()
    # sizes beyond the built-in buffer are refused with a message, nothing is launched
    for H_bad, code in ((8200, -2), (16384, -2), (1001, -1)):
        rc = fn(None, None, None, None, None, None, None, 4, H_bad, 0, None)
        assert rc == code and b"vb_rmsnorm_bwd_static" in lib.vb_rmsnorm_bwd_static_strerror(rc)
