"""Expert-parallel layer on 2 GPUs (NCCL) against the single-GPU layer holding all experts."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, prec):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", AMOE_PRECISION=prec)
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from analog_moe import AnalogSigmaMoELayer, TorchInferenceRPUConfig
        from analog_moe.ep import ExpertParallelAnalogSigmaMoELayer
        D, F, E, k, T = 128, 64, 8, 2, 200 + 17 * rank
        cfg = TorchInferenceRPUConfig()
        cfg.forward.out_res, cfg.forward.out_bound = 254.0, 12.0      # DAC + ADC, no noise
        cfg.pre_post.input_range.decay = 0.0
        torch.manual_seed(0)
        dense = AnalogSigmaMoELayer(cfg, d_model=D, n_experts=E, expert_size=F, k=k).to(dev).eval()
        with torch.no_grad():
            dense.input_range.copy_(torch.linspace(2.0, 3.5, 2 * E).view(2, E))
        ep = ExpertParallelAnalogSigmaMoELayer(cfg, group=dist.group.WORLD, d_model=D, n_experts=E, expert_size=F,
                                               k=k).to(dev).eval()
        ep.load_global_weights(dense.keys.data, dense.values.data, dense.expert_sel.weight.data, dense.input_range.data)
        g = torch.Generator().manual_seed(10 + rank)
        x1 = torch.randn(1, T, D, generator=g).to(dev).requires_grad_()
        x2 = x1.detach().clone().requires_grad_()
        gy = torch.randn(1, T, D, generator=g).to(dev)
        y1, _ = dense(x1)
        (y1 * gy).sum().backward()
        y2, _ = ep(x2)
        (y2 * gy).sum().backward()
        # same kernels on both sides; in the fp16 precision the gradient scalar differs (max|g| over different row sets)
        tol = 1e-4 if prec == "split" else 5e-4
        assert float((y1 - y2).abs().max()) <= tol * max(1.0, float(y1.abs().max()))
        assert float((x1.grad - x2.grad).abs().max()) <= tol * max(1.0, float(x1.grad.abs().max()))
        # the owner's weight / input-range gradients equal the sum over ranks of the dense layers' gradients
        El = E // world
        sl = slice(rank * El, (rank + 1) * El)
        for name in ("keys", "values"):
            full = getattr(dense, name).grad.clone()
            dist.all_reduce(full)
            got = getattr(ep, name).grad
            assert float((full[sl] - got).abs().max()) <= tol * max(1.0, float(full.abs().max())), name
        full = dense.input_range.grad.clone()
        dist.all_reduce(full)
        assert float((full[:, sl] - ep.input_range.grad).abs().max()) <= tol * max(1.0, float(full.abs().max()))
        # router gradient: replicated parameter, compare the all-reduced gradients
        a, b = dense.expert_sel.weight.grad.clone(), ep.expert_sel.weight.grad.clone()
        dist.all_reduce(a)
        dist.all_reduce(b)
        assert float((a - b).abs().max()) <= tol * max(1.0, float(a.abs().max()))
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.parametrize("prec", ["split", "f16"])
def test_expert_parallel_matches_dense_on_two_gpus(prec):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    mp.spawn(_worker, args=(2, _free_port(), prec), nprocs=2, join=True)


def _worker_noise_and_decay(rank, world, port):
    """Weight noise: the owner draws, for its experts, exactly the noise a layer holding all experts draws (global
    expert id in the Philox counter), so ranks differ from each other.  Decay term: its threshold is the kept fraction
    over ALL routed pairs, summed over the ranks on the device - equal to the dense layer's under skewed routing."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", AMOE_PRECISION="split")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from analog_moe import AnalogSigmaMoELayer, TorchInferenceRPUConfig, WeightModifierType, ops, _cabi
        from analog_moe.ep import ExpertParallelAnalogSigmaMoELayer
        D, F, E, k, T = 128, 64, 8, 2, 256
        El = E // world
        # ---- weight noise of the owner == the dense layer's for the same experts
        torch.manual_seed(0)
        W = torch.randn(E, D, F, device=dev) / D ** 0.5
        kw = dict(noise_std=0.05, noise_per_channel=True, seed=77, offset=3, need_w_out=True)
        full = ops.weight_prepass(W, _cabi.PREC_FP32_SIMT, **kw).w
        mine = ops.weight_prepass(W[rank * El:(rank + 1) * El].contiguous(), _cabi.PREC_FP32_SIMT, expert_base=rank * El, **kw).w
        assert torch.equal(mine, full[rank * El:(rank + 1) * El])
        other = ops.weight_prepass(W[rank * El:(rank + 1) * El].contiguous(), _cabi.PREC_FP32_SIMT, expert_base=0, **kw).w
        assert (rank == 0) == bool(torch.equal(other, mine))
        # ---- decay with skewed routing, ranges low enough that a few per cent of the inputs clip
        cfg = TorchInferenceRPUConfig()
        cfg.forward.out_res, cfg.forward.out_bound = 254.0, 12.0
        cfg.pre_post.input_range.decay = 0.02
        cfg.pre_post.input_range.input_min_percentage = 0.9
        torch.manual_seed(0)
        dense = AnalogSigmaMoELayer(cfg, d_model=D, n_experts=E, expert_size=F, k=k).to(dev).train()
        with torch.no_grad():
            dense.input_range.copy_(torch.linspace(1.8, 3.0, 2 * E).view(2, E))
        ep = ExpertParallelAnalogSigmaMoELayer(cfg, group=dist.group.WORLD, d_model=D, n_experts=E, expert_size=F,
                                               k=k).to(dev).train()
        ep.load_global_weights(dense.keys.data, dense.values.data, dense.expert_sel.weight.data, dense.input_range.data)
        bias = -1.2 * torch.log(torch.arange(1, E + 1, device=dev, dtype=torch.float32)) * 1.6
        dense.router_bias = ep.router_bias = bias          # rank 0's experts get most of the rows
        # all ranks must see the same global kept fraction: give every rank the same tokens
        g = torch.Generator().manual_seed(4)
        x1 = torch.randn(1, T, D, generator=g).to(dev).requires_grad_()
        x2 = x1.detach().clone().requires_grad_()
        gy = torch.randn(1, T, D, generator=g).to(dev)
        y1, _ = dense(x1)
        (y1 * gy).sum().backward()
        y2, _ = ep(x2)
        (y2 * gy).sum().backward()
        full = dense.input_range.grad.clone()
        dist.all_reduce(full)                              # identical tokens on every rank: world x the dense gradient
        sl = slice(rank * El, (rank + 1) * El)
        err = float((full[:, sl] - ep.input_range.grad).abs().max())
        assert err <= 1e-4 * max(1.0, float(full.abs().max())), err
        # the decay term is really in there: without it the gradient differs
        cfg.pre_post.input_range.decay = 0.0
        dense.zero_grad()
        x3 = x1.detach().clone().requires_grad_()
        y3, _ = dense(x3)
        (y3 * gy).sum().backward()
        assert float((dense.input_range.grad * world - full).abs().max()) > 1e-3
    finally:
        dist.barrier()
        dist.destroy_process_group()


def test_expert_parallel_weight_noise_and_decay_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    mp.spawn(_worker_noise_and_decay, args=(2, _free_port()), nprocs=2, join=True)
