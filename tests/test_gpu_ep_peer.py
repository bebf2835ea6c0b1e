"""Pieces of the expert-parallel step that touch other ranks' memory, with the ranks emulated on one GPU (one buffer per
rank, the "peer" pointers are local; nothing here waits for another launch):
  * gradient rows sent as fp16 with a power-of-two scale per row (amoe_ep_put_f16) give, through the operand pre-pass,
    the tiles that the fp32 rows give;
  * the small exchange (amoe_ep_share) on one rank, and its bounded wait when a rank never arrives."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(G, E, k, N, dev, seed):
    from analog_moe import ops
    El = E // G
    Ts = [130 + 29 * r for r in range(G)]
    g = torch.Generator().manual_seed(seed)
    logits = [torch.randn(T, E, generator=g) for T in Ts]
    logits[0][:, E - 1] = -50.0
    routes = [ops.select_sort(l.to(dev), k) for l in logits]
    counts = torch.stack([(r.expert_offsets[1:] - r.expert_offsets[:-1]).view(G, El) for r in routes]).contiguous()
    plans = [ops.ep_plan(counts, r) for r in range(G)]
    gys = [(torch.randn(T, N, generator=g) * (3e-3 * (r + 1))).to(dev) for r, T in enumerate(Ts)]   # a different scale per rank
    gates = [torch.rand(T * k, generator=g).to(dev) for T in Ts]
    return El, Ts, routes, counts, plans, gys, gates


@pytest.mark.parametrize("G,E,k", [(2, 8, 2), (4, 8, 4)])
def test_fp16_gradient_rows_give_the_tiles_of_the_fp32_rows(G, E, k):
    from analog_moe import ops, _cabi
    from analog_moe._cabi import lib, stream_ptr
    dev = torch.device("cuda:0")
    N = 128
    El, Ts, routes, counts, plans, gys, gates = _setup(G, E, k, N, dev, 5)
    p_cap = max(T * k for T in Ts)
    cap = G * p_cap
    recv32 = [torch.zeros(cap, N, device=dev) for _ in range(G)]
    recv16 = [torch.zeros(cap, N, device=dev, dtype=torch.float16) for _ in range(G)]
    rmax = [torch.zeros(cap, device=dev) for _ in range(G)]
    p32 = torch.tensor([t.data_ptr() for t in recv32], dtype=torch.int64, device=dev)
    p16 = torch.tensor([t.data_ptr() for t in recv16], dtype=torch.int64, device=dev)
    pm = torch.tensor([t.data_ptr() for t in rmax], dtype=torch.int64, device=dev)
    status = ops.new_status(dev)
    for r in range(G):
        P = Ts[r] * k
        assert lib.amoe_ep_put(gys[r].data_ptr(), 0, N, N, Ts[r], routes[r].slot_index.data_ptr(), k, gates[r].data_ptr(), P,
                               routes[r].sel.data_ptr(), El, plans[r].data_ptr(), p32.data_ptr(), G, cap, status.data_ptr(),
                               stream_ptr()) == 0
        assert lib.amoe_ep_put_f16(gys[r].data_ptr(), N, N, Ts[r], routes[r].slot_index.data_ptr(), k, gates[r].data_ptr(), P,
                                   routes[r].sel.data_ptr(), El, plans[r].data_ptr(), p16.data_ptr(), pm.data_ptr(), G, cap,
                                   status.data_ptr(), stream_ptr()) == 0
    torch.cuda.synchronize()
    ops.raise_on_device_status(status, "exchange")
    # the bound every rank would share: max|gy| * max|gate| over the ranks
    glob = torch.stack([ops.tensor_absmax(gys[r]) * ops.tensor_absmax(gates[r].view(-1, 1)) for r in range(G)]).max().reshape(1)
    prec = _cabi.PREC_F16X1
    for d in range(G):
        R = int(plans[d][0])
        assert torch.equal(rmax[d][:R], recv32[d][:R].abs().amax(1))          # the maxima are those of the fp32 rows
        order, offsets = ops.ep_local_plan_dev(plans[d], G, El, cap)
        want, _ = ops.operand_tiles(recv32[d], order, offsets, El, prec, P=cap, dac=False, g_absmax=glob)
        got, _ = ops.operand_tiles(recv16[d], order, offsets, El, prec, P=cap, dac=False, g_absmax=glob, row_absmax=rmax[d])
        torch.cuda.synchronize()
        # rows of the tiles that exist (the tile arrays are not cleared past the last tile)
        n_tiles = int(((offsets[1:] - offsets[:-1] + 127) // 128).sum())
        a = want.hi[:, :n_tiles * 128].view(torch.float16).float()     # (the arrays are typed bf16, the fp16 precision stores halves)
        b = got.hi[:, :n_tiles * 128].view(torch.float16).float()
        # identical except where the value is subnormal in fp16 (rounded twice on the way): one subnormal step at most
        assert float((a - b).abs().max()) <= 2.0 ** -24
        assert float((a != b).float().mean()) < 1e-4
        assert float(a.abs().max()) >= 16.0                                    # the scale put the rows into fp16's range


def test_small_exchange_on_one_rank_and_its_bounded_wait():
    from analog_moe import ops
    from analog_moe._cabi import lib, stream_ptr
    dev = torch.device("cuda:0")
    slot_bytes = 64
    # one rank: the payload comes back, the epoch advances, slots alternate
    slots = torch.zeros(2 * 1 * slot_bytes, dtype=torch.uint8, device=dev)
    flags = torch.zeros(4, dtype=torch.int32, device=dev)
    epoch = torch.zeros(1, dtype=torch.int32, device=dev)
    sp = torch.tensor([slots.data_ptr()], dtype=torch.int64, device=dev)
    fp = torch.tensor([flags.data_ptr()], dtype=torch.int64, device=dev)
    status = ops.new_status(dev)
    for step in range(3):
        val = torch.arange(5, dtype=torch.int32, device=dev) + 10 * step
        out = torch.full((1, 5), -1, dtype=torch.int32, device=dev)
        assert lib.amoe_ep_share(val.data_ptr(), 20, sp.data_ptr(), slot_bytes, fp.data_ptr(), epoch.data_ptr(), 0, 1,
                                 out.data_ptr(), 1000, status.data_ptr(), stream_ptr()) == 0
        torch.cuda.synchronize()
        assert torch.equal(out[0], val) and int(epoch[0]) == step + 1 and int(flags[0]) == step + 1
    ops.raise_on_device_status(status, "exchange")
    # two ranks of which the second never arrives (its flag in this rank's array stays zero): the wait runs out,
    # the status word says so, the kernel returns and the context stays usable
    slots2 = [torch.zeros(2 * 2 * slot_bytes, dtype=torch.uint8, device=dev) for _ in range(2)]
    flags2 = [torch.zeros(4, dtype=torch.int32, device=dev) for _ in range(2)]
    epoch2 = torch.zeros(1, dtype=torch.int32, device=dev)
    sp2 = torch.tensor([t.data_ptr() for t in slots2], dtype=torch.int64, device=dev)
    fp2 = torch.tensor([t.data_ptr() for t in flags2], dtype=torch.int64, device=dev)
    val = torch.arange(4, dtype=torch.int32, device=dev)
    out = torch.full((2, 4), -1, dtype=torch.int32, device=dev)
    assert lib.amoe_ep_share(val.data_ptr(), 16, sp2.data_ptr(), slot_bytes, fp2.data_ptr(), epoch2.data_ptr(), 0, 2,
                             out.data_ptr(), 2000, status.data_ptr(), stream_ptr()) == 0
    torch.cuda.synchronize()
    host = (C.c_int32 * 4)()
    assert lib.amoe_read_device_status(status.data_ptr(), C.byref(host), stream_ptr()) == 9        # AMOE_ERR_WAIT_LIMIT
    assert host[1] == 55 and host[2] == 1                                                           # waiting for rank 1
    assert int(flags2[1][0]) == 1                      # this rank did arrive at the other one
    assert bool((out == -1).all())                     # nothing handed out after a wait that gave up
    assert float(torch.ones(8, device=dev).sum()) == 8.0
