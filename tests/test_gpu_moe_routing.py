"""GPU tests of MoE routing / permutation / combine.  Parity is UNPINNED in the reference
(it has no router or permutation); the oracle is the torch definition on the CPU."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from layerstormgemmkernels_b200 import ops as _ops
    return _ops


def oracle_route(logits, k):
    p = torch.softmax(logits.float(), -1)
    w, idx = torch.topk(p, k)
    return idx.to(torch.int32), w / w.sum(-1, keepdim=True)


def oracle_permutation(idx, E):
    flat = idx.flatten().to(torch.int64)
    perm = torch.sort(flat, stable=True).indices.to(torch.int32)
    offs = torch.zeros(E + 1, dtype=torch.int32)
    offs[1:] = torch.cumsum(torch.bincount(flat, minlength=E), 0).to(torch.int32)
    inv = torch.empty_like(perm)
    inv[perm.long()] = torch.arange(perm.numel(), dtype=torch.int32)
    return offs, perm, inv


@pytest.mark.parametrize("T,E,k", [(1, 128, 8), (64, 128, 8), (4096, 128, 8), (4096, 8, 2), (33, 60, 4), (5, 4, 4)])
def test_route_permute_combine(ops, T, E, k):
    g = torch.Generator().manual_seed(T + E)
    logits = torch.randn(T, E, generator=g)
    idx, w = ops.moe_route(logits.cuda(), k)
    ridx, rw = oracle_route(logits, k)
    assert torch.equal(idx.cpu(), ridx)
    torch.testing.assert_close(w.cpu(), rw, rtol=2e-6, atol=1e-7)

    offs, perm, inv = ops.moe_permutation(idx, E)
    roffs, rperm, rinv = oracle_permutation(ridx, E)
    assert torch.equal(offs.cpu(), roffs)
    assert torch.equal(perm.cpu(), rperm)
    assert torch.equal(inv.cpu(), rinv)

    H = 256
    hidden = torch.randn(T, H, generator=g).to(torch.bfloat16)
    xp = ops.moe_permute(hidden.cuda(), perm, k)
    assert torch.equal(xp.cpu(), hidden[(rperm // k).long()])

    y = torch.randn(T * k, H, generator=g).to(torch.bfloat16)
    out = ops.moe_unpermute(y.cuda(), inv, w)
    ref = (y.float()[rinv.long()].view(T, k, H) * w.cpu().view(T, k, 1)).sum(1)
    torch.testing.assert_close(out.float().cpu(), ref, rtol=2.0 ** -7, atol=1e-3)


def test_permutation_with_skewed_routing(ops):
    """All tokens to two experts, many empty experts."""
    T, E, k = 300, 16, 2
    idx = torch.stack([torch.full((T,), 3), torch.full((T,), 11)], 1).to(torch.int32)
    offs, perm, inv = ops.moe_permutation(idx.cuda(), E)
    roffs, rperm, rinv = oracle_permutation(idx, E)
    assert torch.equal(offs.cpu(), roffs) and torch.equal(perm.cpu(), rperm) and torch.equal(inv.cpu(), rinv)


@pytest.mark.parametrize("world,per,seed", [(2, 64, 0), (4, 3, 1), (8, 16, 2), (1, 5, 3)])
def test_ep_expert_order_matches_definition(ops, world, per, seed):
    """Regrouping of rows received by (source, expert) into (expert, source): against the
    definition written with numpy; empty blocks included."""
    rng = np.random.default_rng(seed)
    counts = rng.integers(0, 40, size=(world, per)).astype(np.int32)
    counts[rng.random((world, per)) < 0.3] = 0
    rows = int(counts.sum())
    offs, order, inv = ops.ep_expert_order(torch.from_numpy(counts).cuda(), world, per, rows)
    starts = np.zeros(world * per + 1, np.int64)
    starts[1:] = np.cumsum(counts.reshape(-1))
    exp = []
    for e in range(per):
        for s in range(world):
            b = s * per + e
            exp.extend(range(starts[b], starts[b] + counts[s, e]))
    exp = np.array(exp, dtype=np.int32)
    assert np.array_equal(order.cpu().numpy(), exp)
    assert np.array_equal(inv.cpu().numpy()[exp], np.arange(rows, dtype=np.int32))
    exp_offs = np.zeros(per + 1, np.int32)
    exp_offs[1:] = np.cumsum(counts.sum(0))
    assert np.array_equal(offs.cpu().numpy(), exp_offs)
