"""Whole-model gradient check of the Llama trainer against plain PyTorch autograd in fp32.

The trainer applies AdamW behind every unit's backward and never exposes a gradient. With zero moments the first
update of a weight is ``lr * g / (|g| + eps)`` (plus a negligible decay term): its sign is the sign of the gradient.
So after one step the sign of ``before - after`` of every fp32 master weight must agree with the sign of the gradient
that autograd computes on an fp32 restatement of the same architecture with the same initial weights, wherever that
gradient is well above the bf16 noise of the training kernels. One wrong backward kernel, one mis-wired gradient view
or one transposed weight shows up as a sign agreement near 50 % for that parameter.
"""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _reference_grads(cfg, weights, tok, tgt, dtype=torch.float64):
    """fp32 autograd of the same decoder: rotate-half RoPE on q and k, grouped-query causal attention, SwiGLU with gate
    rows then up rows, RMSNorm, untied head, mean cross-entropy."""
    d, nh, nkv = cfg.head_dim, cfg.heads, cfg.kv_heads
    W = {k: v.detach().to(dtype).requires_grad_(True) for k, v in weights.items()}
    B, S = tok.shape
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, d, 2, device=tok.device, dtype=torch.float64) / d))
    ang = torch.outer(torch.arange(S, device=tok.device, dtype=torch.float64), inv)
    cos, sin = ang.cos()[None, :, None, :].to(dtype), ang.sin()[None, :, None, :].to(dtype)

    def norm(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.eps) * w

    def rope(x):
        a, b = x[..., : d // 2], x[..., d // 2:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)

    x = W["embed.tok"][tok]
    for i in range(cfg.layers):
        p = lambda n: W[f"layer{i}.{n}"]
        qkv = (norm(x, p("attn_norm")) @ p("wqkv").t()).view(B, S, nh + 2 * nkv, d)
        q, k, v = rope(qkv[:, :, :nh]), rope(qkv[:, :, nh:nh + nkv]), qkv[:, :, nh + nkv:]
        rep = nh // nkv
        a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2).repeat_interleave(rep, 1), v.transpose(1, 2).repeat_interleave(rep, 1),
                                           is_causal=True)
        x = x + a.transpose(1, 2).reshape(B, S, nh * d) @ p("wo").t()
        gu = norm(x, p("mlp_norm")) @ p("w13").t()
        x = x + (F.silu(gu[..., : cfg.ffn]) * gu[..., cfg.ffn:]) @ p("w2").t()
    logits = norm(x, W["head.norm"]) @ W["head.out"].t()
    loss = F.cross_entropy(logits.view(B * S, -1), tgt.reshape(-1))
    loss.backward()
    return float(loss), {k: v.grad for k, v in W.items()}


@pytest.mark.parametrize("shape", ["tiny", "wide", "one_layer_of_8b"])
def test_first_update_follows_the_autograd_gradient(shape):
    from rocm_systems_b200.models.llama import LlamaConfig, LlamaTrainer
    from rocm_systems_b200.parallel.fsdp import AdamWConfig

    batch, ref_dtype = 2, torch.float64
    if shape == "tiny":
        cfg = LlamaConfig.tiny(64)
    elif shape == "one_layer_of_8b":  # every kernel at the sizes of the benchmark: vocabulary 128256, FFN 14336, 4096 positions
        cfg = LlamaConfig(layers=1)
        batch, ref_dtype = 1, torch.float32
    else:  # rows of 4096 channels, 128-wide heads, grouped queries: the kernel configurations of the 8B model
        cfg = LlamaConfig(vocab=4096, hidden=4096, layers=2, heads=32, kv_heads=8, ffn=1024, seq_len=256)
    dev = torch.device("cuda", 0)
    tr = LlamaTrainer(cfg, None, dev, opt=AdamWConfig(lr=1e-3, weight_decay=0.0), seed=5)
    g = torch.Generator().manual_seed(3)
    tok = torch.randint(0, cfg.vocab, (batch, cfg.seq_len), generator=g).to(dev)
    tgt = torch.randint(0, cfg.vocab, (batch, cfg.seq_len), generator=g).to(dev)
    units = [tr.embed, *tr.layers, tr.head]
    before = {}
    for u in units:
        for s in u.specs:
            o = u.offsets[s.name]
            before[f"{u.name}.{s.name}"] = u.master[o:o + s.numel].view(*s.shape).clone()
    # the reference sees the weights the kernels see: the bf16 working copy
    seen = {k: v.to(torch.bfloat16).float() for k, v in before.items()}
    ref_loss, grads = _reference_grads(cfg, seen, tok, tgt, ref_dtype)
    del seen
    loss = tr.step(tok, tgt)
    torch.cuda.synchronize()
    assert abs(loss - ref_loss) < 0.02 * max(1.0, ref_loss), (loss, ref_loss)
    worst = []
    for u in units:
        for s in u.specs:
            name = f"{u.name}.{s.name}"
            o = u.offsets[s.name]
            delta = before[name] - u.master[o:o + s.numel].view(*s.shape)      # = lr * g / (|g| + eps)
            gr = grads[name].float()
            big = gr.abs() > 0.2 * gr.abs().max()                                # well above the bf16 noise of the kernels
            assert int(big.sum()) > 0, name
            agree = float((torch.sign(delta[big]) == torch.sign(gr[big])).float().mean())
            moved = float((delta[big].abs() > 0.5e-3).float().mean())          # and the step has the size AdamW gives it
            worst.append((agree, moved, name))
    bad = [w for w in worst if w[0] < 0.98 or w[1] < 0.98]
    assert not bad, f"sign agreement / moved fraction too low for {bad}"
