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


@pytest.mark.parametrize("T,E,k", [(1, 128, 8), (64, 128, 8), (4096, 128, 8), (4096, 8, 2), (33, 60, 4), (5, 4, 4),
                                   (128, 128, 8), (129, 128, 8), (32, 1024, 8)])   # 1024 pairs: last one-CTA case
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
                                        H, E, world, rp.data_ptr(), cap, back[r].data_ptr(), st))
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


def test_ep_peer_exchange_overflow_is_clamped_and_reported(ops):
    """Receive buffers smaller than what the ranks send: every offset the plan writes stays
    within the capacity, rows that do not fit are dropped at the sender and their slots of the
    return buffer cleared, nothing is written past the buffers (canary rows), and the device
    status word reports code 7.  Ranks emulated one after the other on this GPU."""
    from layerstormgemmkernels_b200 import capi
    lib = capi.lib
    world, E, T, k, H = 2, 8, 64, 2, 64
    P, per = T * k, E // world
    cap = 40                                     # far below the ~64 rows each rank receives
    canary = 8
    st = torch.cuda.current_stream().cuda_stream
    g = torch.Generator().manual_seed(7)
    dev = "cuda"
    hidden = [torch.randn(T, H, generator=g).to(torch.bfloat16).to(dev) for _ in range(world)]
    logits = [torch.randn(T, E, generator=g).to(dev) for _ in range(world)]
    counts = [torch.zeros(world, E, dtype=torch.int32, device=dev) for _ in range(world)]
    recv = [torch.full((cap + canary, H), 7.0, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    back = [torch.full((P + canary, H), 9.0, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    ptrs = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=dev)
    cp, rp, bp = ptrs(counts), ptrs(recv), ptrs(back)
    assert capi.device_status() == 0
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
                                        H, E, world, rp.data_ptr(), cap, back[r].data_ptr(), st))
    dropped_total = 0
    for r in range(world):
        sb, lo, ds, rb, info = plans[r]
        rows, flag = info.tolist()
        assert flag == 1 and rows <= cap
        lo_h = lo.cpu().numpy()
        assert (np.diff(lo_h) >= 0).all() and lo_h[-1] == rows and lo_h.max() <= cap
        assert int(ds.max().item()) <= cap
        # the expert block on the clamped offsets: a grouped GEMM call must stay inside its rows
        y = recv[r][:cap].clone()
        capi.check(lib.lsg_ep_return_rows(y.data_ptr(), ds.data_ptr(), rb.data_ptr(), info.data_ptr(), world, per, H,
                                          cap, bp.data_ptr(), st))
    torch.cuda.synchronize()
    for r in range(world):
        assert torch.all(recv[r][cap:] == 7.0), "rows were written past the receive buffer"
        assert torch.all(back[r][P:] == 9.0), "rows were written past the return buffer"
        # every slot of the return buffer was either filled by a peer or cleared by the sender
        idx, w, offs, perm, inv = routed[r]
        tok = perm.cpu().numpy() // k
        got = back[r][:P].cpu()
        exp = hidden[r].cpu()[tok]
        same = (got == exp).all(dim=1)
        zero = (got == 0).all(dim=1)
        assert bool((same | zero).all())
        dropped_total += int((zero & ~same).sum())
    assert dropped_total > 0
    assert capi.device_status() == 7             # expert-parallel overflow, read and cleared
    assert capi.device_status() == 0


def test_grouped_gemm_ignores_offsets_past_its_rows(ops):
    """Expert offsets that run past the rows of the call (what an overflowed exchange would
    have produced without the clamp): the tensor-core grouped GEMM must not touch anything
    beyond its total_tokens rows."""
    from layerstormgemmkernels_b200 import capi, quantize as Q
    E, N, K, T = 4, 256, 512, 300
    rng = np.random.default_rng(3)
    Ws = [torch.from_numpy(Q.quantize_q4_k((rng.standard_normal((N, K)) * 0.02).astype(np.float32))).cuda()
          for _ in range(E)]
    b_ptrs = torch.tensor([w.data_ptr() for w in Ws], dtype=torch.int64, device="cuda")
    A = torch.randn(T, K, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).cuda()
    good = torch.tensor([0, 100, 100, 220, 300], dtype=torch.int32, device="cuda")
    bad = torch.tensor([0, 100, 100, 220, 900], dtype=torch.int32, device="cuda")     # last expert claims 680 rows
    ref = ops.gguf_grouped_gemm(A, good, b_ptrs, capi.Q4_K, 1, N, K, force=2)
    out = torch.full((T + 64, N), 3.0, dtype=torch.bfloat16, device="cuda")
    ops.gguf_grouped_gemm(A, bad, b_ptrs, capi.Q4_K, 1, N, K, force=2, out=out[:T])
    torch.cuda.synchronize()
    assert torch.all(out[T:] == 3.0), "the GEMM wrote past its rows"
    assert torch.equal(out[:T], ref)
    assert capi.device_status() == 0


def test_flag_barrier_emulated_ranks_and_timeout(ops):
    """lsg_ep_barrier with two ranks emulated on this GPU (flag arrays are local tensors).
    A kernel never waits for a kernel launched after it here: rank 1 arrives without waiting,
    then rank 0 arrives and waits (succeeds at once), then rank 1 waits.  After that rank 0
    arrives at a second barrier that rank 1 never reaches: with a short limit the wait gives
    up, the status word reports code 6, and the context stays usable."""
    from layerstormgemmkernels_b200 import capi
    lib = capi.lib
    world = 2
    flags = [torch.zeros(world + 1, dtype=torch.int32, device="cuda") for _ in range(world)]
    ptrs = torch.tensor([f.data_ptr() for f in flags], dtype=torch.int64, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    assert capi.device_status() == 0
    capi.check(lib.lsg_ep_barrier(ptrs.data_ptr(), 1, world, 1, st))     # rank 1 arrives
    capi.check(lib.lsg_ep_barrier(ptrs.data_ptr(), 0, world, 3, st))     # rank 0 arrives and waits
    capi.check(lib.lsg_ep_barrier(ptrs.data_ptr(), 1, world, 2, st))     # rank 1 waits
    assert capi.device_status() == 0
    assert flags[0].tolist() == [1, 1, 1] and flags[1].tolist() == [1, 1, 1]
    capi.check(lib.lsg_set_wait_limit_cycles(500000))                     # a quarter of a millisecond
    try:
        capi.check(lib.lsg_ep_barrier(ptrs.data_ptr(), 0, world, 3, st))  # rank 1 never comes
        assert capi.device_status() == 6
    finally:
        capi.check(lib.lsg_set_wait_limit_cycles(0))
    assert capi.device_status() == 0
    assert float(torch.ones(4, device="cuda").sum().item()) == 4.0
    with pytest.raises(ValueError):
        capi.check(lib.lsg_ep_barrier(ptrs.data_ptr(), 2, world, 3, st))
