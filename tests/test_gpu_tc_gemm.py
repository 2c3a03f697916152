"""tcgen05 / TMEM GEMM against a PyTorch fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (128, 256, 256), (256, 512, 1024), (300, 384, 512), (300, 264, 200), (1024, 7168, 2048),
                                   (4096, 4096, 4096)])
def test_gemm_bf16_nt(m, n, k):
    from torchcomms_b200 import _comms

    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    a = (torch.randn(m, k, generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    b = (torch.randn(n, k, generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    c, status = _comms.ops.gemm_bf16_nt(a, b)
    torch.cuda.synchronize()
    assert int(status[0]) == 0, "a bounded wait inside the kernel ran out"
    ref = a.float() @ b.float().t()
    torch.testing.assert_close(c.float(), ref, rtol=2e-2, atol=2e-2 * (k ** 0.5))


@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (512, 512, 1024), (300, 264, 200), (1024, 7168, 2048), (4096, 4096, 4096),
                                   (8192, 1792, 512)])
def test_gemm_bf16_nt_cta_pairs(m, n, k):
    """Same product on clusters of two CTAs (tcgen05 cta_group::2)."""
    from torchcomms_b200 import _comms

    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    a = (torch.randn(m, k, generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    b = (torch.randn(n, k, generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    for _ in range(2):
        c, status = _comms.ops.gemm_bf16_nt_pair(a, b)
        torch.cuda.synchronize()
        assert int(status[0]) == 0, "a bounded wait inside the kernel ran out"
        ref = a.float() @ b.float().t()
        torch.testing.assert_close(c.float(), ref, rtol=2e-2, atol=2e-2 * (k ** 0.5))
