"""Failure detection without faulting anything.

CPU ranks over gloo: an exchange whose counts were corrupted on one rank is refused by all ranks together before any
row moves; a rank that leaves between steps is noticed by the others on the host, through the store, before their
next step.  One GPU test: a device-side wait that nothing ends gives up after its limit, records
AMOE_ERR_WAIT_LIMIT in the status word and returns - the context stays usable.
"""
import os
import socket
import tempfile

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


def _mismatch_worker(rank, world, port, bad_rank, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from analog_moe.ep import step_plan
        from analog_moe.health import ExchangeMismatchError
        from oracle import cvmm_oracle as O
        E, k, T = 4 * world, 2, 40 + rank
        s = O.select_sort(torch.randn(T, E, generator=torch.Generator().manual_seed(rank)), k)
        counts = (s.expert_offsets[1:] - s.expert_offsets[:-1]).to(torch.int32).view(world, E // world)
        good = step_plan(counts, rank, expect_rows=T * k)            # consistent counts pass on every rank
        assert sum(good.send_n) == T * k
        if rank == bad_rank:
            counts = counts.clone()
            counts[0, 0] += 3                                         # the injected fault: a corrupted count message
        try:
            step_plan(counts, rank, expect_rows=T * k)
            result = "no error"
        except ExchangeMismatchError as exc:
            result = "mismatch" + (" (this one)" if "this one" in str(exc) else "")
        with open(os.path.join(out, f"r{rank}"), "w") as f:
            f.write(result)
    finally:
        dist.destroy_process_group()


def test_corrupted_counts_are_refused_by_every_rank():
    world = 3
    with tempfile.TemporaryDirectory() as out:
        mp.spawn(_mismatch_worker, args=(world, _free_port(), 1, out), nprocs=world, join=True)
        res = [open(os.path.join(out, f"r{r}")).read() for r in range(world)]
    assert res == ["mismatch", "mismatch (this one)", "mismatch"]


def _leaver_worker(rank, world, store_path, out):
    from analog_moe.health import PeerLostError, StepHeartbeat
    store = dist.FileStore(store_path, world)
    hb = StepHeartbeat(store, rank, world, timeout_s=3.0)
    log = []
    try:
        for step in range(4):
            if rank == 1 and step == 2:
                hb.leave()                      # between steps: nothing of this rank is in flight
                log.append("left")
                break
            hb.announce(step)
            hb.check(step)                      # every peer is about to run the same step
            log.append(f"step {step}")
    except PeerLostError as exc:
        log.append("peer lost: " + str(exc))
    with open(os.path.join(out, f"r{rank}"), "w") as f:
        f.write("\n".join(log))


def test_a_rank_that_leaves_between_steps_is_noticed_on_the_host():
    world = 3
    with tempfile.TemporaryDirectory() as out:
        mp.spawn(_leaver_worker, args=(world, os.path.join(out, "store"), out), nprocs=world, join=True)
        res = [open(os.path.join(out, f"r{r}")).read().splitlines() for r in range(world)]
    assert res[1] == ["step 0", "step 1", "left"]
    for r in (0, 2):
        assert res[r][:2] == ["step 0", "step 1"]
        assert res[r][2].startswith("peer lost: rank 1 left the group before step 2")


def _silent_worker(rank, world, store_path, out):
    from analog_moe.health import PeerLostError, StepHeartbeat
    store = dist.FileStore(store_path, world)
    hb = StepHeartbeat(store, rank, world, timeout_s=0.5)
    msg = "ok"
    if rank == 0:
        hb.announce(0)
        try:
            hb.check(0)                         # rank 1 never announces anything
        except PeerLostError as exc:
            msg = str(exc)
    with open(os.path.join(out, f"r{rank}"), "w") as f:
        f.write(msg)


def test_a_silent_rank_times_out():
    with tempfile.TemporaryDirectory() as out:
        mp.spawn(_silent_worker, args=(2, os.path.join(out, "store"), out), nprocs=2, join=True)
        assert "rank 1 did not announce step 0" in open(os.path.join(out, "r0")).read()


@pytest.mark.gpu
def test_bounded_device_wait_gives_up_and_reports():
    import ctypes as C
    from analog_moe import _cabi, ops
    lib = _cabi.lib
    dev = torch.device("cuda:0")
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    rc = lib.amoe_selftest_bounded_wait(status.data_ptr(), 2_000_000, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    host = (C.c_int32 * 4)()
    code = lib.amoe_read_device_status(status.data_ptr(), C.byref(host), torch.cuda.current_stream().cuda_stream)
    assert code == 9 and host[0] == 9 and host[1] == 99          # AMOE_ERR_WAIT_LIMIT at the self-test's wait
    with pytest.raises(_cabi.AmoeError):
        ops.raise_on_device_status(status, "self-test")
    # the context is intact: a real kernel runs afterwards
    r = ops.select_sort(torch.randn(64, 8, device=dev), 2)
    assert int(r.expert_offsets[-1]) == 128
