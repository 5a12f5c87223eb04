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


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K,bn", [(256, 256, 64, 256), (256, 128, 128, 128), (512, 512, 256, 0), (304, 520, 200, 0), (1000, 328, 72, 0),
                                      (1024, 1024, 1024, 256), (1024, 1024, 1024, 128), (4096, 6144, 4096, 0)])
def test_gemm_on_cta_pairs_matches_fp32_for_every_operand_order(M, N, K, bn, ta, tb):
    """The CTA-pair kernel with each operand stored K-major (row-major [rows, K]) or MN-major (the transpose view of a
    row-major [K, rows]): the forward, input-gradient and weight-gradient forms of a linear layer."""
    from rocm_systems_b200.ops import train_ops as ops

    torch.manual_seed(M + N + K)
    a = (torch.randn(K, M, device="cuda").to(torch.bfloat16).t() if ta else torch.randn(M, K, device="cuda").to(torch.bfloat16))
    b = (torch.randn(K, N, device="cuda").to(torch.bfloat16).t() if tb else torch.randn(N, K, device="cuda").to(torch.bfloat16))
    out = ops.gemm(a, b, bn=bn)
    torch.cuda.synchronize()
    assert ops.gemm_take_error() == 0
    ref = a.float() @ b.float().t()
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 1e-2 * scale + 1e-2, (err, scale)


def test_gemm_on_cta_pairs_writes_into_a_strided_view():
    from rocm_systems_b200.ops import train_ops as ops

    torch.manual_seed(5)
    a = torch.randn(384, 256, device="cuda").to(torch.bfloat16)
    b = torch.randn(200, 256, device="cuda").to(torch.bfloat16)
    big = torch.full((384, 512), 7.0, dtype=torch.bfloat16, device="cuda")
    ops.gemm(a, b, out=big[:, 64:264])
    torch.cuda.synchronize()
    assert ops.gemm_take_error() == 0
    ref = a.float() @ b.float().t()
    assert (big[:, 64:264].float() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item() + 1e-2
    assert bool((big[:, :64] == 7).all()) and bool((big[:, 264:] == 7).all())     # nothing outside the view was written
