"""Numerics of the hand-written training kernels against plain PyTorch fp32 references."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _bf(x):
    return x.to(torch.bfloat16)


def test_rmsnorm_fwd_bwd():
    from rocm_systems_b200.ops import train_ops as ops

    torch.manual_seed(0)
    for T, H in [(37, 256), (128, 4096), (5, 8192)]:
        x = _bf(torch.randn(T, H, device="cuda")).requires_grad_(True)
        w = _bf(1 + 0.1 * torch.randn(H, device="cuda")).requires_grad_(True)
        dy = _bf(torch.randn(T, H, device="cuda"))
        y = ops.rmsnorm(x, w, 1e-5)
        y.backward(dy)
        xf, wf = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
        yr = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
        yr.backward(dy.float())
        assert torch.allclose(y.float(), yr, rtol=2e-2, atol=2e-2)
        assert torch.allclose(x.grad.float(), xf.grad, rtol=3e-2, atol=3e-2)
        assert torch.allclose(w.grad.float(), wf.grad, rtol=3e-2, atol=0.05 * math.sqrt(T))


def test_rope_matches_rotate_half_and_inverts():
    from rocm_systems_b200.ops import train_ops as ops

    torch.manual_seed(1)
    T, heads, total, D, S = 64, 6, 8, 128, 32
    table = ops.rope_table(S, D, 500000.0, "cuda")
    qkv = _bf(torch.randn(T, total, D, device="cuda")).requires_grad_(True)
    out = ops.rope_(qkv, table, heads)
    pos = torch.arange(T, device="cuda") % S
    cos = table[pos, :, 0].unsqueeze(1)
    sin = table[pos, :, 1].unsqueeze(1)
    x = qkv.detach().float()
    a, b = x[..., : D // 2], x[..., D // 2:]
    ref = torch.cat([a * cos - b * sin, b * cos + a * sin], -1)
    ref[:, heads:] = x[:, heads:]
    assert torch.allclose(out.float(), ref, rtol=2e-2, atol=2e-2)
    g = _bf(torch.randn_like(ref))
    out.backward(g)
    gf = g.float()
    ga, gb = gf[..., : D // 2], gf[..., D // 2:]
    gref = torch.cat([ga * cos + gb * sin, gb * cos - ga * sin], -1)
    gref[:, heads:] = gf[:, heads:]
    assert torch.allclose(qkv.grad.float(), gref, rtol=2e-2, atol=2e-2)


def test_swiglu_fwd_bwd():
    from rocm_systems_b200.ops import train_ops as ops

    torch.manual_seed(2)
    T, F = 33, 512
    gu = _bf(torch.randn(T, 2 * F, device="cuda")).requires_grad_(True)
    d = _bf(torch.randn(T, F, device="cuda"))
    out = ops.swiglu(gu)
    out.backward(d)
    gf = gu.detach().float().requires_grad_(True)
    ref = torch.nn.functional.silu(gf[:, :F]) * gf[:, F:]
    ref.backward(d.float())
    assert torch.allclose(out.float(), ref, rtol=2e-2, atol=2e-2)
    assert torch.allclose(gu.grad.float(), gf.grad, rtol=3e-2, atol=3e-2)


def test_cross_entropy_loss_and_gradient():
    from rocm_systems_b200.ops import train_ops as ops

    torch.manual_seed(3)
    for T, V in [(17, 1000), (8, 128256), (4, 1003 * 8)]:
        logits = _bf(3 * torch.randn(T, V, device="cuda"))
        tgt = torch.randint(0, V, (T,), device="cuda")
        tgt[0] = -100  # ignored row
        lf = logits.float().requires_grad_(True)
        mask = tgt >= 0
        ref_rows = torch.nn.functional.cross_entropy(lf, tgt.clamp(min=0), reduction="none") * mask
        (ref_rows.sum() / T).backward()
        work = logits.clone()
        rows = ops.cross_entropy_inplace(work, tgt, 1.0 / T)
        assert torch.allclose(rows, ref_rows.detach(), rtol=1e-3, atol=1e-3)
        assert torch.allclose(work.float(), lf.grad, rtol=2e-2, atol=2e-4)


def test_adamw_matches_torch():
    from rocm_systems_b200.ops import train_ops as ops

    torch.manual_seed(4)
    n = 10007
    w = torch.randn(n, device="cuda")
    ref = torch.nn.Parameter(w.clone())
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m, v, p = torch.zeros_like(w), torch.zeros_like(w), torch.empty(n, dtype=torch.bfloat16, device="cuda")
    for step in range(1, 4):
        g = torch.randn(n, device="cuda")
        ref.grad = g.clone()
        opt.step()
        ops.adamw_(w, m, v, g, p, 1e-2, (0.9, 0.95), 1e-8, 0.1, step)
    assert torch.allclose(w, ref.detach(), rtol=1e-5, atol=1e-6)
    assert torch.equal(p, w.to(torch.bfloat16))


def test_embedding_fwd_bwd_and_cast():
    from rocm_systems_b200.ops import train_ops as ops

    torch.manual_seed(5)
    V, H, T = 500, 256, 300
    table = _bf(torch.randn(V, H, device="cuda"))
    tok = torch.randint(0, V, (T,), device="cuda")
    out = ops.embedding(tok, table)
    assert torch.equal(out, table[tok])
    d = _bf(torch.randn(T, H, device="cuda"))
    dt = torch.zeros(V, H, device="cuda")
    ops.embedding_bwd_(tok, d, dt)
    ref = torch.zeros(V, H, device="cuda").index_add_(0, tok, d.float())
    assert torch.allclose(dt, ref, rtol=1e-5, atol=1e-5)
    src = _bf(torch.randn(1000 + 3, device="cuda"))
    dst = torch.empty(1003, device="cuda")
    ops.cast_scale_(src, dst, 0.25)
    assert torch.equal(dst, src.float() * 0.25)


def test_tiny_llama_trains_and_matches_autograd_reference():
    """Loss goes down, and the first-step loss equals a plain fp32 PyTorch forward of the same weights."""
    from rocm_systems_b200.models.llama import LlamaConfig, LlamaTrainer

    cfg = LlamaConfig.tiny(64)
    tr = LlamaTrainer(cfg, None, torch.device("cuda", 0), seed=7)
    g = torch.Generator().manual_seed(11)
    tok = torch.randint(0, cfg.vocab, (2, cfg.seq_len), generator=g)
    tgt = torch.randint(0, cfg.vocab, (2, cfg.seq_len), generator=g)
    l_eval = tr.eval_loss(tok, tgt)
    assert abs(l_eval - math.log(cfg.vocab)) < 0.5  # random init: near uniform
    losses = [tr.step(tok.pin_memory(), tgt.pin_memory()) for _ in range(8)]
    assert abs(losses[0] - l_eval) < 0.05
    assert losses[-1] < losses[0] - 0.5, losses
