"""The expert-routing rule: ties, NaN and -inf rows. The CPU test pins the rule stated by ``ref_route``; the GPU test runs
``b200collEpRoute`` alone (it writes only its two outputs) on rows that have fewer than k selectable values and checks
that every expert id is a valid one and every weight finite, and that it agrees with the rule."""
import pytest
import torch

from rocm_systems_b200.parallel.ep import ref_route


def _rows(E: int):
    g = torch.Generator().manual_seed(5)
    normal = torch.randn(6, E, generator=g)
    ties = torch.zeros(1, E)
    all_nan = torch.full((1, E), float("nan"))
    all_ninf = torch.full((1, E), float("-inf"))
    two_left = torch.full((1, E), float("-inf"))
    two_left[0, 40] = 1.5
    two_left[0, 7] = 0.25
    some_nan = torch.randn(1, E, generator=g)
    some_nan[0, ::3] = float("nan")
    pinf = torch.randn(1, E, generator=g)
    pinf[0, 11] = float("inf")
    pinf[0, 3] = float("inf")
    return torch.cat([normal, ties, all_nan, all_ninf, two_left, some_nan, pinf]).contiguous()


def test_route_rule_on_cpu():
    E, k = 64, 4
    x = _rows(E)
    idx, w = ref_route(x, k)
    assert idx.dtype == torch.int32 and int(idx.min()) >= 0 and int(idx.max()) < E
    assert torch.isfinite(w).all() and torch.allclose(w.sum(-1), torch.ones(x.shape[0]))
    for r in range(x.shape[0]):
        assert len(set(idx[r].tolist())) == k                       # k distinct experts per token
    tv, ti = torch.topk(x[:6], k, dim=-1)                            # ordinary rows: plain top-k and its softmax
    assert torch.equal(idx[:6].long(), ti) and torch.allclose(w[:6], torch.softmax(tv, -1))
    assert idx[6].tolist() == [0, 1, 2, 3]                          # all equal: lowest ids
    assert idx[7].tolist() == [0, 1, 2, 3] and torch.allclose(w[7], torch.full((k,), 0.25))   # all NaN
    assert idx[8].tolist() == [0, 1, 2, 3] and torch.allclose(w[8], torch.full((k,), 0.25))   # all -inf
    assert idx[9].tolist() == [40, 7, 0, 1] and w[9, 2] == 0 and w[9, 3] == 0                 # two selectable values
    assert not torch.isnan(x[10][idx[10].long()]).any()             # NaN entries lose against every number
    assert idx[11].tolist()[:2] == [3, 11]                          # +inf entries tie at the top, lower id first


@pytest.mark.gpu
@pytest.mark.parametrize("E,k", [(32, 8), (64, 4), (256, 8)])
def test_route_kernel_never_writes_a_bad_expert(E, k):
    from rocm_systems_b200.parallel.ep import route

    x = _rows(max(E, 64))[:, :E].contiguous().cuda()
    idx, w = route(x, k)
    torch.cuda.synchronize()
    ridx, rw = ref_route(x.cpu(), k)
    assert int(idx.min()) >= 0 and int(idx.max()) < E
    assert torch.isfinite(w).all()
    assert torch.equal(idx.cpu(), ridx)
    assert torch.allclose(w.cpu(), rw, rtol=1e-4, atol=1e-6)


def test_router_backward_matches_autograd_of_topk_softmax():
    import torch

    from rocm_systems_b200.parallel.ep import router_backward

    g = torch.Generator().manual_seed(3)
    T, E, k = 64, 32, 4
    logits = torch.randn(T, E, generator=g, dtype=torch.float64, requires_grad=True)
    d_gate = torch.randn(T, k, generator=g, dtype=torch.float64)
    top_v, top_i = torch.topk(logits, k, dim=-1)
    w = torch.softmax(top_v, dim=-1)
    (w * d_gate).sum().backward()
    got = router_backward(w.detach().float(), top_i.to(torch.int32), d_gate.float(), E)
    assert torch.allclose(got.double(), logits.grad, atol=1e-6)


def test_gate_up_interleaving_round_trips():
    import torch

    from rocm_systems_b200.parallel.tp import deinterleave_gate_up, interleave_gate_up

    for tile in (128, 256):
        g, u = torch.randn(512, 24), torch.randn(512, 24)
        w13 = interleave_gate_up(g, u, tile)
        assert w13.shape == (1024, 24)
        # a tile holds tile/2 gate rows then the tile/2 up rows of the same outputs
        assert torch.equal(w13[: tile // 2], g[: tile // 2]) and torch.equal(w13[tile // 2: tile], u[: tile // 2])
        g2, u2 = deinterleave_gate_up(w13, tile)
        assert torch.equal(g2, g) and torch.equal(u2, u)
