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


@pytest.mark.parametrize("world,E,T,k", [(2, 8, 40, 2), (4, 16, 64, 4), (1, 4, 10, 2), (2, 128, 512, 8)])
def test_ep_peer_exchange_kernels_emulated_ranks(ops, world, E, T, k):
    """The peer-memory exchange kernels (publish counts, plan, send rows, return rows) with the
    ranks emulated one after the other on this GPU: every 'peer' buffer is a local tensor, so
    the index arithmetic of a whole layer is checked without a second GPU.  The expert block
    is replaced by y = x * (global expert id + 1)."""
    from layerstormgemmkernels_b200 import capi
    lib = capi.lib
    H, P, per = 64, T * k, E // world
    cap = P * world            # worst case: everything lands on one rank
    st = torch.cuda.current_stream().cuda_stream
    g = torch.Generator().manual_seed(world * 100 + E)
    dev = "cuda"
    hidden = [torch.randn(T, H, generator=g).to(torch.bfloat16).to(dev) for _ in range(world)]
    logits = [torch.randn(T, E, generator=g).to(dev) for _ in range(world)]
    counts = [torch.zeros(world, E, dtype=torch.int32, device=dev) for _ in range(world)]
    recv = [torch.zeros(cap, H, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    back = [torch.zeros(P, H, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    ptrs = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=dev)
    cp, rp, bp = ptrs(counts), ptrs(recv), ptrs(back)
    routed = []
    for r in range(world):
        idx, w = ops.moe_route(logits[r], k)
        offs, perm, inv = ops.moe_permutation(idx, E)
        routed.append((idx, w, offs, perm, inv))
        capi.check(lib.lsg_ep_publish_counts(offs.data_ptr(), E, r, world, cp.data_ptr(), st))
    plans = []
    for r in range(world):
        sb = torch.empty(E, dtype=torch.int32, device=dev)
        lo = torch.empty(per + 1, dtype=torch.int32, device=dev)
        ds = torch.empty(E, dtype=torch.int32, device=dev)
        rb = torch.empty(E, dtype=torch.int32, device=dev)
        info = torch.zeros(2, dtype=torch.int32, device=dev)
        capi.check(lib.lsg_ep_plan(counts[r].data_ptr(), r, world, E, cap, sb.data_ptr(), lo.data_ptr(),
                                   ds.data_ptr(), rb.data_ptr(), info.data_ptr(), st))
        plans.append((sb, lo, ds, rb, info))
        idx, w, offs, perm, inv = routed[r]
        capi.check(lib.lsg_ep_send_rows(hidden[r].data_ptr(), perm.data_ptr(), offs.data_ptr(), sb.data_ptr(), P, k,
                                        H, E, world, rp.data_ptr(), cap, st))
    for r in range(world):
        sb, lo, ds, rb, info = plans[r]
        assert info.tolist()[1] == 0
        lo_h = lo.cpu().numpy()
        # rows this rank received = all pairs routed to its experts
        expected_rows = sum(int((routed[s][0] // per == r).sum().item()) for s in range(world))
        assert int(lo_h[-1]) == expected_rows == info.tolist()[0]
        y = recv[r].clone()
        for el in range(per):
            y[lo_h[el]:lo_h[el + 1]] = (y[lo_h[el]:lo_h[el + 1]].float() * (r * per + el + 1)).to(torch.bfloat16)
        capi.check(lib.lsg_ep_return_rows(y.data_ptr(), ds.data_ptr(), rb.data_ptr(), info.data_ptr(), world, per, H,
                                          cap, bp.data_ptr(), st))
    torch.cuda.synchronize()
    for r in range(world):
        idx, w, offs, perm, inv = routed[r]
        pair = perm.cpu().numpy()                      # sorted row -> pair index
        e_of_row = idx.reshape(-1).cpu().numpy()[pair]
        tok = pair // k
        exp = (hidden[r].float().cpu()[tok] * torch.from_numpy((e_of_row + 1).astype(np.float32))[:, None]).to(torch.bfloat16)
        assert torch.equal(back[r].cpu(), exp)
