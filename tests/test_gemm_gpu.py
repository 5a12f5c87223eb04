"""The hand-written tcgen05 GEMM against an fp32 PyTorch reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K,bn", [(128, 256, 64, 256), (128, 128, 128, 128), (256, 512, 256, 0), (300, 520, 200, 0),
                                      (1024, 1024, 1024, 256), (1024, 1024, 1024, 128), (4096, 6144, 4096, 0)])
def test_gemm_bf16_tn_matches_fp32(M, N, K, bn):
    from rocm_systems_b200.ops import train_ops as ops

    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
    out = ops.gemm_bf16_tn(a, b, bn=bn)
    torch.cuda.synchronize()
    assert ops.gemm_take_error() == 0
    ref = a.float() @ b.float().t()
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 1e-2 * scale + 1e-2, (err, scale)
