"""Host-side logic of the expert-parallel exchange on CPU ranks (gloo, world size 2 and 4): the
split sizes and the regrouping of received rows by local expert."""
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


def _worker(rank, world, port, E, k, T, fail_rank):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from analog_moe.ep import make_plan
        from oracle import cvmm_oracle as O
        g = torch.Generator().manual_seed(100 + rank)
        logits = torch.randn(T + 3 * rank, E, generator=g)
        if rank == 0:
            logits[:, E - 1] = -60.0           # nobody on rank 0 picks the last expert
        s = O.select_sort(logits, k)
        plan = make_plan(s.expert_offsets, world)
        El = E // world
        P = s.sel.numel()
        assert sum(plan.send_splits) == P
        # rows tagged (source rank, global expert, position in the source's sorted list)
        rows = torch.stack([torch.full((P,), rank), s.sel.long(), torch.arange(P)], 1).double()
        recv = torch.empty(plan.n_recv, 3, dtype=torch.float64)
        dist.all_to_all_single(recv, rows, plan.recv_splits, plan.send_splits)
        srt = recv[plan.local_order.long()]
        # every received row belongs to one of this rank's experts, the regrouped list is sorted by
        # local expert, stable in (source rank, source position), and local_sel/offsets describe it
        assert torch.equal(srt[:, 1].long() - rank * El, plan.local_sel.long())
        assert bool((plan.local_sel[1:] >= plan.local_sel[:-1]).all())
        key = srt[:, 1] * 1e8 + srt[:, 0] * 1e6 + srt[:, 2]
        assert bool((key[1:] > key[:-1]).all())
        counts = torch.bincount(plan.local_sel.long(), minlength=El)
        assert torch.equal(plan.local_offsets[1:].long(), torch.cumsum(counts, 0))
        assert sorted(plan.local_order.tolist()) == list(range(plan.n_recv))
        # total conservation
        tot = torch.tensor([P, plan.n_recv])
        dist.all_reduce(tot)
        assert int(tot[0]) == int(tot[1])
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,E,k", [(2, 8, 2), (4, 8, 3)])
def test_exchange_plan_over_gloo(world, E, k):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, E, k, 37, -1), nprocs=world, join=True)


def test_plan_from_counts_handles_empty_rank():
    from analog_moe.ep import plan_from_counts
    send = torch.tensor([[3, 0], [0, 0]])
    recv = torch.zeros(2, 2, dtype=torch.int32)
    p = plan_from_counts(send, recv)
    assert p.n_recv == 0 and p.local_order.numel() == 0 and p.local_offsets.tolist() == [0, 0, 0]
    assert p.send_splits == [3, 0]


def _step_plan_worker(rank, world, port, E, k, T):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from analog_moe.ep import step_plan
        from oracle import cvmm_oracle as O
        g = torch.Generator().manual_seed(7 + rank)
        logits = torch.randn(T + 5 * rank, E, generator=g)
        s = O.select_sort(logits, k)
        El = E // world
        P = s.sel.numel()
        counts = (s.expert_offsets[1:] - s.expert_offsets[:-1]).to(torch.int32).view(world, El)
        plan = step_plan(counts, rank)
        assert sum(plan.send_n) == P and plan.send_off[0] == 0
        assert plan.p_max == max((T + 5 * r) * k for r in range(world))
        assert torch.equal(plan.recv_counts[rank], counts[rank])            # what this rank keeps for itself
        # emulate the stores of the device-driven exchange with an all-to-all of tagged rows and check that the block
        # starts the plan predicts are where the rows land
        rows = torch.stack([torch.full((P,), rank), torch.arange(P)], 1).double()
        recv = torch.empty(plan.n_recv, 2, dtype=torch.float64)
        dist.all_to_all_single(recv, rows, plan.recv_n, plan.send_n)
        for src in range(world):
            blk = recv[plan.recv_off[src]:plan.recv_off[src] + plan.recv_n[src]]
            assert bool((blk[:, 0] == src).all())
        # off_in / back_off: every rank publishes them, the owner checks its side
        mine = torch.tensor([plan.off_in, plan.back_off, plan.send_off, plan.recv_off], dtype=torch.int64)
        everyone = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(everyone, mine)
        for src in range(world):
            assert int(everyone[src][0][rank]) == plan.recv_off[src]         # source's off_in at me = my recv_off[source]
            assert int(everyone[src][2][rank]) == plan.back_off[src]         # my back_off[source] = source's send_off[me]
            if plan.recv_n[src]:
                assert float(recv[plan.recv_off[src], 1]) == float(everyone[src][2][rank])
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,E,k", [(2, 8, 2), (4, 16, 3)])
def test_step_plan_block_starts_over_gloo(world, E, k):
    mp.spawn(_step_plan_worker, args=(world, _free_port(), E, k, 29), nprocs=world, join=True)
