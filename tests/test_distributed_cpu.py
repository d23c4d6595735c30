"""CPU tests (gloo, world size 2) of the multi-GPU host logic: expert-parallel dispatch /
combine and the column-split gather.  The GEMMs are replaced by plain torch matmuls here;
what is checked is the routing of rows between ranks."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _torch_route(logits, k):
    p = torch.softmax(logits.float(), -1)
    w, idx = torch.topk(p, k)
    return idx.to(torch.int32), w / w.sum(-1, keepdim=True)


def _torch_permutation(idx, E):
    flat = idx.flatten().to(torch.int64)
    perm = torch.sort(flat, stable=True).indices.to(torch.int32)
    offs = torch.zeros(E + 1, dtype=torch.int32)
    offs[1:] = torch.cumsum(torch.bincount(flat, minlength=E), 0).to(torch.int32)
    inv = torch.empty_like(perm)
    inv[perm.long()] = torch.arange(perm.numel(), dtype=torch.int32)
    return offs, perm, inv


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from layerstormgemmkernels_b200 import distributed as D
        E, k, H, I = 8, 2, 16, 24
        T_local = 5 + 3 * rank                   # ragged token counts per rank
        g = torch.Generator().manual_seed(100)   # same weights on every rank
        W1 = torch.randn(E, I, H, generator=g)
        W2 = torch.randn(E, H, I, generator=g)
        g2 = torch.Generator().manual_seed(7 + rank)
        hidden = torch.randn(T_local, H, generator=g2)
        logits = torch.randn(T_local, E, generator=g2)
        if rank == 1:
            logits[:, 0:4] = -50.0               # rank 1 never routes to rank 0's experts
        e0, e1 = D.expert_range(rank, world, E)

        def ffn(rows, offs):
            out = torch.empty_like(rows)
            for el in range(e1 - e0):
                s, t = int(offs[el]), int(offs[el + 1])
                out[s:t] = torch.relu(rows[s:t] @ W1[e0 + el].T) @ W2[e0 + el].T
            return out

        out = D.ep_moe_layer(
            hidden, logits, k, E, ffn, _torch_route, _torch_permutation,
            lambda h, perm, kk: h[(perm // kk).long()],
            lambda y, inv, w: (y[inv.long()].view(w.shape[0], w.shape[1], -1) * w.unsqueeze(-1)).sum(1))

        # single-process reference
        idx, w = _torch_route(logits, k)
        ref = torch.zeros_like(hidden)
        for t in range(T_local):
            for s in range(k):
                e = int(idx[t, s])
                ref[t] += w[t, s] * (torch.relu(hidden[t] @ W1[e].T) @ W2[e].T)
        ok_moe = torch.allclose(out, ref, rtol=1e-4, atol=1e-4)

        # column split
        N, M = 512, 3
        n0, n1 = D.column_slab(rank, world, N)
        full = torch.arange(M * N, dtype=torch.float32).reshape(M, N)
        gathered = D.column_split_gather(full[:, n0:n1].contiguous())
        ok_col = torch.equal(gathered, full)
        results[rank] = (ok_moe, ok_col)
    finally:
        dist.destroy_process_group()


def test_expert_parallel_and_column_split_world2():
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        for r in range(world):
            assert results[r] == (True, True), (r, results[r])


def test_expert_range_and_slabs():
    from layerstormgemmkernels_b200 import distributed as D
    assert D.expert_range(3, 8, 128) == (48, 64)
    assert D.column_slab(7, 8, 14336) == (12544, 14336)
    with pytest.raises(ValueError):
        D.expert_range(0, 3, 128)
    with pytest.raises(ValueError):
        D.column_slab(0, 3, 14336)


def _worker_bad_offsets(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from layerstormgemmkernels_b200 import distributed as D
        E, rows = 4, 6
        good = torch.tensor([0, 2, 3, 5, 6], dtype=torch.int32)
        bad = torch.tensor([0, 2, 3, 5, 9], dtype=torch.int32)      # ends past the rank's 6 rows
        offs = bad if rank == 1 else good
        try:
            D.make_ep_plan(offs, E, rows=rows)
            results[rank] = "no error"
        except D.EpExchangeError as exc:
            results[rank] = str(exc)
        # the group is still usable afterwards: the good offsets go through on both ranks
        plan = D.make_ep_plan(good, E, rows=rows)
        results[f"{rank}_after"] = plan.recv_rows
    finally:
        dist.destroy_process_group()


def test_inconsistent_expert_offsets_raise_on_every_rank_before_any_row_moves():
    """One rank's offsets do not end at its row count.  The verdict travels with the counts, so
    BOTH ranks raise (naming rank 1) instead of one of them entering a row exchange alone, and
    the next layer works."""
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        procs = [ctx.Process(target=_worker_bad_offsets, args=(r, world, port, results)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        for r in range(world):
            assert "rank(s) [1]" in results[r], results[r]
        # each rank keeps 3 rows for its own experts and receives the peer's 3 (rank 0: experts 0-1)
        assert results["0_after"] == 6 and results["1_after"] == 6


def _worker_peer_leaves(rank, world, port, results):
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    from layerstormgemmkernels_b200 import distributed as D
    E, rows = 4, 6
    good = torch.tensor([0, 2, 3, 5, 6], dtype=torch.int32)
    D.make_ep_plan(good, E, rows=rows)               # step 1: both ranks
    if rank == 1:
        results[rank] = "left"
        return                                       # leaves between steps, nothing in flight
    try:
        D.make_ep_plan(good, E, rows=rows)           # step 2: the peer is gone
        results[rank] = "no error"
    except D.EpExchangeError as exc:
        results[rank] = "EpExchangeError"
    except Exception as exc:                         # noqa: BLE001
        results[rank] = f"other: {type(exc).__name__}"


def test_a_rank_that_leaves_between_steps_ends_the_next_exchange_with_a_clean_error():
    """The failure is made on the host: rank 1 returns after a completed step.  Rank 0's next
    count exchange ends within the process group's short timeout (or at once, on a closed
    connection) with EpExchangeError, not with a hang."""
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        procs = [ctx.Process(target=_worker_peer_leaves, args=(r, world, port, results)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(90)
            assert not p.is_alive()
        assert results[1] == "left"
        assert results[0] == "EpExchangeError", results[0]
