"""The block-scaled fp8 contract (rocm_systems_b200/ops/fp8.py) stated in PyTorch: quantise -> dequantise error bounds,
scale layouts, and the block-by-block GEMM against the GEMM of the dequantised operands."""
import torch

from rocm_systems_b200.ops import fp8


def test_activation_scales_are_block_major_and_bound_the_error():
    torch.manual_seed(0)
    x = torch.randn(70, 384) * torch.logspace(-3, 2, 70).unsqueeze(1)      # rows of very different magnitude
    q, s = fp8.ref_quantize_act(x.to(torch.bfloat16))
    assert q.dtype == torch.float8_e4m3fn and tuple(s.shape) == (3, 70)
    back = fp8.ref_dequantize_act(q, s)
    amax = x.to(torch.bfloat16).float().view(70, 3, 128).abs().amax(-1)
    # e4m3 keeps 3 mantissa bits: relative step 2^-3 at worst, half of it after rounding; values far below the block's
    # maximum fall into the subnormal grid, whose step is amax / 448 * 2^-9... bounded by amax * 2^-4 overall
    err = (back - x.to(torch.bfloat16).float()).view(70, 3, 128).abs().amax(-1)
    assert (err <= amax * 2 ** -4 + 1e-12).all()
    assert torch.allclose(s.t() * 448.0, amax.clamp_min(1e-10), rtol=1e-6)
    assert float(q.float().abs().max()) == 448.0                               # every block uses the whole range


def test_weight_scales_cover_ragged_last_block():
    torch.manual_seed(1)
    w = torch.randn(200, 256).to(torch.bfloat16)                              # 200 rows: second block has 72 live rows
    q, s = fp8.ref_quantize_weight(w)
    assert tuple(q.shape) == (200, 256) and tuple(s.shape) == (2, 2)
    back = fp8.ref_dequantize_weight(q, s)
    assert float((back - w.float()).abs().max()) <= float(w.float().abs().max()) * 2 ** -4
    blk = w.float()[128:, :128]
    assert torch.allclose(s[1, 0] * 448.0, blk.abs().max(), rtol=1e-6)        # padding rows did not change the scale


def test_blockwise_gemm_equals_gemm_of_dequantised_operands():
    torch.manual_seed(2)
    x = torch.randn(96, 512).to(torch.bfloat16)
    w = (torch.randn(160, 512) * 0.05).to(torch.bfloat16)
    xq, xs = fp8.ref_quantize_act(x)
    wq, ws = fp8.ref_quantize_weight(w)
    got = fp8.ref_gemm(xq, xs, wq, ws).float()
    want = fp8.ref_dequantize_act(xq, xs) @ fp8.ref_dequantize_weight(wq, ws).t()
    assert torch.allclose(got, want, rtol=2e-2, atol=2e-2)                   # bf16 rounding of the result only
    exact = x.float() @ w.float().t()
    rel = float((got - exact).norm() / exact.norm())
    assert rel < 0.05, rel                                                     # fp8 quantisation noise of both operands


def test_tensor_parallel_fp8_mlp_oracle_tracks_the_exact_mlp():
    """Two ranks' partials from the fp8 oracle of the fused tensor-parallel MLP, summed, against the same MLP in fp32:
    the per-tile gate/up interleave, the second quantisation of the activations and the bf16 partials together cost a few
    per cent, not more."""
    from rocm_systems_b200.parallel.tp import fp8_mlp_partial_oracle, interleave_gate_up

    torch.manual_seed(3)
    M, H, F, n = 64, 256, 128, 2
    x = torch.randn(M, H).to(torch.bfloat16)
    exact = torch.zeros(M, H)
    total = torch.zeros(M, H)
    for r in range(n):
        wg = (torch.randn(F, H) * 0.05).to(torch.bfloat16)
        wu = (torch.randn(F, H) * 0.05).to(torch.bfloat16)
        w2 = (torch.randn(H, F) * 0.05).to(torch.bfloat16)
        w13 = interleave_gate_up(wg, wu, 128)
        assert torch.equal(w13[:64], wg[:64]) and torch.equal(w13[64:128], wu[:64]) and torch.equal(w13[128:192], wg[64:])
        part = fp8_mlp_partial_oracle(x, wg, wu, w2)
        assert part.dtype == torch.bfloat16 and tuple(part.shape) == (M, H)
        total += part.float()
        exact += (torch.nn.functional.silu(x.float() @ wg.float().t()) * (x.float() @ wu.float().t())) @ w2.float().t()
    err = (total - exact).abs().max().item()
    assert err <= 0.06 * exact.abs().max().item()
