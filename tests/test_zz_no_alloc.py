"""The allocation-free C entry point for RMSNorm backward, called through the
exported symbol with raw pointers, against the module's ordinary entry point.
Collected last (file name) so that it also runs after everything else has
used the device."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    import torchcomms_b200
    from torchcomms_b200 import _comms

    lib = ctypes.CDLL(_comms.__file__)
    fn = lib.b200c_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.b200c_noalloc_strerror.restype = ctypes.c_char_p
    lib.b200c_noalloc_strerror.argtypes = [ctypes.c_int]
    return lib, fn


def _inputs(rows, cols, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, cols, generator=g, device="cuda").to(torch.bfloat16)
    dy = torch.randn(rows, cols, generator=g, device="cuda").to(torch.bfloat16)
    w = (1.0 + 0.1 * torch.randn(cols, generator=g, device="cuda")).to(torch.bfloat16)
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5)
    return dy, x, w, rstd


@pytest.mark.parametrize("rows,cols", [(64, 512), (1000, 4096), (4096, 8192)])
def test_matches_ordinary_entry_point_twice(rows, cols):
    from torchcomms_b200 import _comms

    lib, fn = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):  # two calls in a row reuse the same fixed scratch
        dy, x, w, rstd = _inputs(rows, cols, 77 + call)
        dx = torch.empty_like(x)
        dw = torch.empty_like(w)
        rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), rows, cols, stream)
        assert rc == 0, lib.b200c_noalloc_strerror(rc).decode()
        ref_dx, ref_dw = _comms.ops.rmsnorm_bwd(dy, x, w, rstd)
        torch.cuda.synchronize()
        torch.testing.assert_close(dx.float(), ref_dx.float(), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(dw.float(), ref_dw.float(), rtol=2e-2, atol=2e-2)
        # and both agree with plain PyTorch in fp32
        xf, dyf, wf = x.float(), dy.float(), w.float()
        xhat = xf * rstd[:, None]
        g = dyf * wf
        exp_dx = rstd[:, None] * (g - xhat * (g * xhat).mean(-1, keepdim=True))
        torch.testing.assert_close(dx.float(), exp_dx, rtol=3e-2, atol=3e-2)
        exp_dw = (dyf * xhat).sum(0)
        torch.testing.assert_close(dw.float(), exp_dw, rtol=3e-2, atol=0.02 * float(exp_dw.abs().max()) + 0.05)


def test_rejects_shapes_beyond_the_fixed_scratch():
    lib, fn = _lib()
    t = torch.zeros(16, device="cuda")
    p = t.data_ptr()
    rc = fn(p, p, p, p, p, p, 4, 8192 + 8, None)
    assert rc == -1
    assert b"8192" in lib.b200c_noalloc_strerror(rc)
    assert fn(p, p, p, p, p, p, 0, 512, None) == -2
    assert fn(p, p, p, p, p, p, 4, 500, None) == -2
    assert fn(None, p, p, p, p, p, 4, 512, None) == -2
    torch.cuda.synchronize()
