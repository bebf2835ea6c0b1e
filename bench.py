#!/usr/bin/env python
"""Benchmark of the analog CVMM hot path: one sigma-MoE analog layer, forward + backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config c2]

Prints ONE JSON line (rank 0).  `value` is tokens/s over all GPUs with inputs resident in HBM;
`e2e` is the same step fed from pinned host buffers with the result copied back; `roofline`
describes the dominant kernel (tensor-core bound) timed with CUDA events in a separate pass;
`cpu_baseline` is the CPU restatement of the reference's arithmetic timed on this box's cores.
With --impl reference the CPU restatement is the thing measured (the reference has no CPU path
of its own for this layer and its GPU path needs packages that are not installed).
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "analog-moe_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch  # noqa: E402

# benchmark configs: T tokens per GPU, k, D, F, E, dtype, analog settings
CONFIGS = {
    "c1": dict(T=512, k=2, D=256, F=64, E=8, dtype="fp32", out_noise=0.0, w_noise=0.0, adc=True, bwd=True),
    "c2": dict(T=8192, k=4, D=1024, F=128, E=16, dtype="fp32", out_noise=0.04, w_noise=0.02, adc=True, bwd=True),
    "c3": dict(T=32768, k=8, D=2048, F=256, E=64, dtype="bf16", out_noise=0.0, w_noise=0.0, adc=True, bwd=False),
    "c4": dict(T=16384, k=4, D=1024, F=128, E=32, dtype="fp32", out_noise=0.04, w_noise=0.02, adc=True, bwd=True,
               zipf=1.2),
    "c5": dict(T=8192, k=6, D=1536, F=192, E=48, dtype="bf16", out_noise=0.02, w_noise=0.01, adc=True, bwd=True,
               out_res=62.0),
}


def ncu_traffic(config):
    """DRAM bytes (read + write) per launch of each library call, as ncu measured them: read from the JSON file that
    sits beside the ncu summary of the same capture (null for configurations without a capture)."""
    path = os.path.join(ROOT, "profiles", f"dram_traffic_{config}.json")
    if not os.path.exists(path):
        return {}
    return json.load(open(path)).get("bytes_per_launch", {})


OUT_BOUND = 12.0     # ADC clip in units of the column weight maximum (aihwkit's default out_bound)
SEED = 1234


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(hbm=d["hbm_gbs"], tf=d["bf16_tflops"], tf_sustained=d.get("bf16_tflops_sustained"), src="measured")
    return dict(hbm=6650.0, tf=1590.0, tf_sustained=1400.0, src="fallback")


class ClockSampler(threading.Thread):
    """Reads SM clock and throttle reasons through NVML while the timed region runs (read-only)."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.stop_flag, self.ok = index, [], False, False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.max = None

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        while not self.stop_flag:
            try:
                self.samples.append((nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM),
                                     nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                                     if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons")
                                     else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)))
            except Exception:
                pass
            time.sleep(0.01)

    def result(self):
        if not self.ok or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max, "reasons": ["unavailable"]}
        clocks = sorted(s[0] for s in self.samples)
        bits = 0
        for _, r in self.samples:
            bits |= r
        names = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
                 0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
                 0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}
        return {"sm_mhz": clocks[len(clocks) // 2], "sm_max_mhz": self.max,
                "reasons": [n for b, n in names.items() if bits & b and n != "gpu_idle"], "samples": len(clocks)}


def make_inputs(cfg, seed, device, dtype, n_sets):
    g = torch.Generator().manual_seed(seed)
    T, D = cfg["T"], cfg["D"]
    xs = [torch.randn(1, T, D, generator=g).to(dtype) for _ in range(n_sets)]
    gys = [torch.randn(1, T, D, generator=g).to(dtype) for _ in range(n_sets)]
    return xs, gys


def build_layer(cfg, device, dtype, precision, n_experts_local=None, ep_group=None):
    from analog_moe import AnalogSigmaMoELayer, TorchInferenceRPUConfig, WeightModifierType
    rc = TorchInferenceRPUConfig()
    rc.forward.inp_res = 254.0
    rc.forward.out_res = cfg.get("out_res", 254.0) if cfg["adc"] else -1.0
    rc.forward.out_bound = OUT_BOUND if cfg["adc"] else -1.0
    rc.forward.out_noise = cfg["out_noise"]
    rc.forward.out_noise_per_channel = True
    rc.pre_post.input_range.init_value = 3.0
    rc.pre_post.input_range.decay = 0.01
    if cfg["w_noise"] > 0:
        rc.modifier.type = WeightModifierType.ADD_NORMAL_PER_CHANNEL
        rc.modifier.std_dev = cfg["w_noise"]
    torch.manual_seed(0)
    kw = dict(d_model=cfg["D"], n_experts=cfg["E"], expert_size=cfg["F"], k=cfg["k"], precision=precision,
              noise_seed=SEED)
    if ep_group is not None:
        from analog_moe.ep import ExpertParallelAnalogSigmaMoELayer
        layer = ExpertParallelAnalogSigmaMoELayer(rc, group=ep_group, **kw)
    else:
        layer = AnalogSigmaMoELayer(rc, **kw)
    layer = layer.to(device).to(dtype)
    if cfg.get("zipf"):
        # bias the router so that expert popularity follows Zipf(s): logit offset -s*ln(rank)*c
        with torch.no_grad():
            rank = torch.arange(1, cfg["E"] + 1, device=device, dtype=torch.float32)
            layer.router_bias = (-cfg["zipf"] * torch.log(rank) * 1.6).to(dtype)
    layer.train(cfg["bwd"])
    return layer


def step(layer, x, gy, bwd):
    if bwd:
        x.grad = None
        for p_ in layer.parameters():
            p_.grad = None
        y, _ = layer(x)
        y.backward(gy)
        return y
    with torch.no_grad():
        y, _ = layer(x)
    return y


def ep_parity_gate(cfg, rank, world, device, group):
    """Correctness evidence for a multi-GPU line: before anything is timed, a small noise-free expert-parallel step
    (DAC + ADC, input ranges that differ per expert, decay on, skewed routing) is compared with a single-GPU layer that
    holds all experts, on every rank: outputs and all gradients relative to their scale (max over ranks), and the number
    of the down-projection's ADC codes that differ."""
    import torch.distributed as dist
    from analog_moe import AnalogSigmaMoELayer, TorchInferenceRPUConfig
    from analog_moe.ep import ExpertParallelAnalogSigmaMoELayer
    dtype = torch.float32 if cfg["dtype"] == "fp32" else torch.bfloat16
    D, F, E, k, T = 256, 128, max(cfg["E"], world), cfg["k"], 384 + 32 * rank
    rc = TorchInferenceRPUConfig()
    rc.forward.inp_res, rc.forward.out_res, rc.forward.out_bound = 254.0, cfg.get("out_res", 254.0), OUT_BOUND
    rc.pre_post.input_range.decay = 0.01
    torch.manual_seed(0)
    dense = AnalogSigmaMoELayer(rc, d_model=D, n_experts=E, expert_size=F, k=k).to(device).to(dtype).train()
    with torch.no_grad():
        dense.input_range.copy_(torch.linspace(2.0, 3.5, 2 * E).view(2, E))
    ep = ExpertParallelAnalogSigmaMoELayer(rc, group=group, d_model=D, n_experts=E, expert_size=F, k=k)
    ep = ep.to(device).to(dtype).train()
    ep.load_global_weights(dense.keys.data, dense.values.data, dense.expert_sel.weight.data, dense.input_range.data)
    bias = (-1.2 * torch.log(torch.arange(1, E + 1, device=device, dtype=torch.float32)) * 1.6).to(dtype)
    dense.router_bias = ep.router_bias = bias              # some experts (hence ranks) get far more rows than others
    dense.keep_codes = ep.keep_codes = True
    g = torch.Generator().manual_seed(10 + rank)
    x1 = torch.randn(1, T, D, generator=g).to(device).to(dtype).requires_grad_()
    x2 = x1.detach().clone().requires_grad_()
    gy = torch.randn(1, T, D, generator=g).to(device).to(dtype)
    y1, _ = dense(x1)
    y1.backward(gy)
    y2, _ = ep(x2)
    y2.backward(gy)
    rel = lambda a, b: float((a.float() - b.float()).abs().max()) / max(1.0, float(b.float().abs().max()))
    errs = [rel(y2, y1), rel(x2.grad, x1.grad)]
    El = E // world
    sl = slice(rank * El, (rank + 1) * El)
    for name in ("keys", "values"):
        full = getattr(dense, name).grad.float().clone()
        dist.all_reduce(full, group=group)               # the owner's gradient = sum of the dense layers' over the ranks
        errs.append(rel(getattr(ep, name).grad, full[sl]))
    full = dense.input_range.grad.float().clone()
    dist.all_reduce(full, group=group)
    errs.append(rel(ep.input_range.grad, full[:, sl]))
    a, b = dense.expert_sel.weight.grad.float().clone(), ep.expert_sel.weight.grad.float().clone()
    dist.all_reduce(a, group=group)
    dist.all_reduce(b, group=group)
    errs.append(rel(b, a))
    mism = 0
    if dense.last_codes is not None and ep.last_codes is not None:
        mism = int((dense.last_codes != ep.last_codes).sum())
    t = torch.tensor([max(errs), float(mism)], device=device, dtype=torch.float64)
    dist.all_reduce(t[0:1], op=dist.ReduceOp.MAX, group=group)
    dist.all_reduce(t[1:2], op=dist.ReduceOp.SUM, group=group)
    if getattr(ep, "_xchg", None) is not None:
        ep._xchg.check("parity gate")
    return dict(max_rel=float(t[0]), code_mismatches=int(t[1]),
                what=f"noise-free expert-parallel step vs one layer holding all {E} experts, skewed routing, decay on: "
                     "y, dx, dkeys, dvalues, d_input_range, router gradient relative to their scale (max over ranks); "
                     "ADC codes of the down-projection that differ (sum over ranks)")


def single_gpu_parity_gate(cfg, device, precision):
    """Beside a single-GPU line: one projection of the benchmark's kind (DAC + ADC, per-expert input ranges, no noise) in
    the precision that is timed against the same calls on the CUDA-core fp32 kernels (the reference's own fp32
    arithmetic), call by call on the same inputs - forward, input gradient with clip mask and per-slot input-range
    gradient, weight gradient.  Reported: the ADC codes that differ (they may, by one code, where the pre-rounding
    value sits next to a rounding tie) and the largest error of each result relative to its scale; forward values are
    compared where the codes agree.  (Whole layers are not compared here: a hidden activation that crosses a DAC tie
    changes the second projection's input by a whole quantisation step, which says nothing about the kernels.)"""
    from analog_moe import ops, _cabi
    dtype = torch.float32 if cfg["dtype"] == "fp32" else torch.bfloat16
    T, k, D, F, E = 1024, cfg["k"], 512, cfg["F"], cfg["E"]
    P = T * k
    g = torch.Generator().manual_seed(3)
    mk = lambda *shape, scale=1.0: (torch.randn(*shape, generator=g) * scale).to(device).to(dtype)
    r = ops.select_sort(torch.randn(T, E, generator=g).to(device), k)
    x, W, gy = mk(T, D), mk(E, D, F, scale=D ** -0.5), mk(P, F)
    ir = torch.linspace(2.0, 3.5, E, device=device)
    out_res = cfg.get("out_res", 254.0)
    res = {}
    if precision is None:
        precision = ops.default_precision(dtype)
    for name, prec in (("timed", precision), ("fp32", _cabi.PREC_FP32_SIMT)):
        pw = ops.weight_prepass(W, prec)
        out, codes = ops.cvmm_fwd(x, r.token_index, r.slot_index, r.expert_offsets, pw, prec, P=P, dst_rows=P, ir=ir,
                                  ir_by_expert=True, inp_res=2.0 / 254.0, out_res=out_res, out_bound=OUT_BOUND,
                                  want_codes=True)
        dx, irg = ops.cvmm_dx(gy, r.slot_index, r.slot_index, r.expert_offsets, pw, prec, P=P, dst_rows=P, x_ref=x,
                              x_ref_row=r.token_index, ir=ir, ir_by_expert=True, want_ir_grad=True,
                              g_absmax=ops.grad_absmax(gy, prec))
        dw = ops.cvmm_dw(x, r.token_index, gy, r.slot_index, r.expert_offsets, E, prec, P=P, ir=ir, ir_by_expert=True,
                         g_absmax=ops.grad_absmax(gy, prec))
        res[name] = dict(out=out.float(), codes=codes.int(), dx=dx.float(), ir_grad=irg.float(), dw=dw.float())
    a, b = res["timed"], res["fp32"]
    dc = (a["codes"] - b["codes"]).abs()
    same = dc == 0
    rel = lambda u, v: float((u - v).abs().max()) / max(float(v.abs().max()), 1e-30)
    per = dict(forward=float(((a["out"] - b["out"]).abs() * same).max()) / float(b["out"].abs().max()),
               dx=rel(a["dx"], b["dx"]), ir_grad=rel(a["ir_grad"], b["ir_grad"]), dw=rel(a["dw"], b["dw"]))
    return dict(max_rel=max(per.values()), per_result=per, code_mismatches=int((dc > 0).sum()), codes=int(dc.numel()),
                max_code_distance=int(dc.max()),
                what="timed precision vs the CUDA-core fp32 kernels, call by call on the same inputs (noise off): errors "
                     "relative to each result's scale; ADC codes that differ")


def run_ours(args, cfg, rank, world, device):
    from analog_moe import ops, _cabi
    # parameters' AccumulateGrad nodes are created during warm-up on the default stream and used again under graph
    # capture on another stream: intended here
    if hasattr(torch.autograd.graph, "set_warn_on_accumulate_grad_stream_mismatch"):
        torch.autograd.graph.set_warn_on_accumulate_grad_stream_mismatch(False)
    dtype = torch.float32 if cfg["dtype"] == "fp32" else torch.bfloat16
    precision = _cabi.PRECISION_NAMES[args.precision] if args.precision else None
    group = None
    if world > 1:
        import torch.distributed as dist
        group = dist.group.WORLD
    parity = None
    if not args.steps_only and not args.timeline:
        parity = ep_parity_gate(cfg, rank, world, device, group) if world > 1 else \
            single_gpu_parity_gate(cfg, device, precision)
    layer = build_layer(cfg, device, dtype, precision, ep_group=group)
    if not cfg["bwd"]:
        layer.requires_grad_(False)        # forward-only configuration: an inference layer, its weights are frozen
    n_sets = 8
    xs_h, gys_h = make_inputs(cfg, 100 + rank, device, dtype, n_sets)
    xs_h = [t.pin_memory() for t in xs_h]
    gys_h = [t.pin_memory() for t in gys_h]
    xs = [t.to(device).requires_grad_(cfg["bwd"]) for t in xs_h]
    gys = [t.to(device) for t in gys_h]
    bwd = cfg["bwd"]

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    # ---------------- device-resident timing
    ops.TRACE = None
    for i in range(args.warmup):
        step(layer, xs[i % n_sets], gys[i % n_sets], bwd)
    barrier()
    if args.steps_only:
        # the command to put under a profiler: warm-up, then the steps themselves, eagerly, and nothing else
        for i in range(args.steps):
            step(layer, xs[i % n_sets], gys[i % n_sets], bwd)
        barrier()
        return None
    if args.kernel_times:
        from analog_moe.profiling import kernel_times
        kernel_times(args.kernel_times, lambda i: step(layer, xs[i % n_sets], gys[i % n_sets], bwd), rank, world)
        return None
    # One CUDA graph per input set (whole step: routing, both projections, backward).  The Philox
    # offsets come from a device counter that the graph itself advances, so replays draw new noise.
    # Expert-parallel runs are captured too when the exchange is device-driven (rows stored into peer memory, the plan
    # computed on the device); the NCCL all-to-all fallback needs one host read per step and stays eager.
    graphs, ys, launches_per_step = None, None, None
    if args.graph and (world == 1 or getattr(layer, "peer_exchange", False)):
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step(layer, xs[0], gys[0], bwd)
            torch.cuda.current_stream().wait_stream(side)
            pool = torch.cuda.graph_pool_handle()
            graphs, ys = [], []
            for i in range(n_sets):
                g = torch.cuda.CUDAGraph()
                ops.TRACE = ops.Trace(timed=False)
                with torch.cuda.graph(g, pool=pool):
                    ys.append(step(layer, xs[i], gys[i], bwd))
                launches_per_step = ops.TRACE.launches
                ops.TRACE = None
                graphs.append(g)
            for g in graphs[:3]:
                g.replay()
        except Exception as exc:          # capture not possible: measure eagerly and say so
            print(f"bench: CUDA graph capture failed ({exc!r}); running eagerly", file=sys.stderr)
            graphs = None
            ops.TRACE = None
            torch.cuda.synchronize()

    def run_step(i):
        if graphs is not None:
            graphs[i % n_sets].replay()
            return ys[i % n_sets]
        return step(layer, xs[i % n_sets], gys[i % n_sets], bwd)

    if args.timeline:
        from analog_moe.profiling import timeline
        barrier()
        timeline(args.timeline, run_step, rank)
        barrier()
        return None
    barrier()
    sampler = ClockSampler(device.index or 0)
    sampler.start()
    ops.TRACE = ops.Trace(timed=False)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        run_step(i)
    e1.record()
    barrier()
    sampler.stop_flag = True
    launches = ops.TRACE.launches if graphs is None else launches_per_step * args.steps
    ops.TRACE = None
    ms = e0.elapsed_time(e1)
    t_dev = torch.tensor([ms], device=device)

    # ---------------- end to end: pinned host inputs in, results out, every step
    # The caller-side loop is software-pipelined over three streams (copy-in, compute, copy-out) and three
    # buffer sets (a set is busy for copy-in + compute + copy-out, about 3 ms, so two sets cannot keep both PCIe
    # directions full), so that the PCIe copies of neighbouring steps overlap the kernels; every step still
    # moves its own inputs from pinned host memory and its own results (y, dx) back to pinned host memory.
    nbuf = 3
    if graphs is not None:
        bx, bg = [xs[b] for b in range(nbuf)], [gys[b] for b in range(nbuf)]    # static buffers of graphs 0..2
    else:
        bx = [torch.empty_like(xs[0]).requires_grad_(bwd) for _ in range(nbuf)]
        bg = [torch.empty_like(gys[0]) for _ in range(nbuf)]
    y_h = [torch.empty(xs_h[0].shape, dtype=dtype).pin_memory() for _ in range(nbuf)]
    dx_h = [torch.empty(xs_h[0].shape, dtype=dtype).pin_memory() for _ in range(nbuf)]
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    main = torch.cuda.current_stream()

    def e2e_run(n):
        ev_in = [None] * nbuf      # inputs of buffer b are on the device
        ev_done = [None] * nbuf    # compute on buffer b finished
        ev_out = [None] * nbuf     # results of buffer b are on the host
        for i in range(n):
            b = i % nbuf
            with torch.cuda.stream(s_in), torch.no_grad():
                if ev_done[b] is not None:
                    s_in.wait_event(ev_done[b])          # previous user of this buffer set has computed
                bx[b].copy_(xs_h[i % n_sets], non_blocking=True)
                if bwd:
                    bg[b].copy_(gys_h[i % n_sets], non_blocking=True)
                ev_in[b] = s_in.record_event()
            main.wait_event(ev_in[b])
            if ev_out[b] is not None:
                main.wait_event(ev_out[b])               # its previous results have left the device
            if graphs is not None:
                graphs[b].replay()
                y = ys[b]
            else:
                y = step(layer, bx[b], bg[b], bwd)
            ev_done[b] = main.record_event()
            with torch.cuda.stream(s_out), torch.no_grad():
                s_out.wait_event(ev_done[b])
                if ev_out[b] is not None:
                    ev_out[b].synchronize()              # the caller has consumed the host copy of step i-2
                y_h[b].copy_(y.detach(), non_blocking=True)
                if bwd:
                    dx_h[b].copy_(bx[b].grad, non_blocking=True)
                ev_out[b] = s_out.record_event()
        for b in range(nbuf):
            if ev_out[b] is not None:
                ev_out[b].synchronize()                  # all results are on the host

    e2e_run(4)
    barrier()
    k_e2e = max(4, min(args.steps, 50))
    e0.record()
    e2e_run(k_e2e)
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1)
    t_e2e = torch.tensor([ms_e2e], device=device)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(t_dev, op=dist.ReduceOp.MAX)
        dist.all_reduce(t_e2e, op=dist.ReduceOp.MAX)
    ms, ms_e2e = float(t_dev), float(t_e2e)
    elem = 4 if dtype == torch.float32 else 2
    h2d = cfg["T"] * cfg["D"] * elem * (2 if bwd else 1)
    d2h = cfg["T"] * cfg["D"] * elem * (2 if bwd else 1)

    # ---------------- per-kernel durations (separate pass, CUDA events around every library call)
    ops.TRACE = ops.Trace(timed=True)
    n_prof = max(3, min(args.steps, 20))
    for i in range(n_prof):
        step(layer, xs[i % n_sets], gys[i % n_sets], bwd)
    summ = ops.TRACE.summary()
    ops.TRACE = None
    # ---------------- the drop-in composition: the layer as the reference's layer files drive it, two CVMM.apply calls
    # with torch glue in between (eager, CUDA events)
    dropin_ms = dropin_graph_ms = None
    if world == 1 and hasattr(layer, "fused"):
        layer.fused = False
        for i in range(3):
            step(layer, xs[i % n_sets], gys[i % n_sets], bwd)
        torch.cuda.synchronize()
        n_d = max(3, min(args.steps, 20))
        e0.record()
        for i in range(n_d):
            step(layer, xs[i % n_sets], gys[i % n_sets], bwd)
        e1.record()
        torch.cuda.synchronize()
        dropin_ms = e0.elapsed_time(e1) / n_d
        # the same composition replayed from a CUDA graph (what is left when the host's share is taken out)
        dropin_graph_ms = None
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step(layer, xs[0], gys[0], bwd)
            torch.cuda.current_stream().wait_stream(side)
            dg = [torch.cuda.CUDAGraph() for _ in range(2)]
            for j, gph in enumerate(dg):
                with torch.cuda.graph(gph):
                    step(layer, xs[j], gys[j], bwd)
            for gph in dg:
                gph.replay()
            torch.cuda.synchronize()
            e0.record()
            for i in range(n_d):
                dg[i % 2].replay()
            e1.record()
            torch.cuda.synchronize()
            dropin_graph_ms = e0.elapsed_time(e1) / n_d
        except Exception as exc:
            print(f"bench: the drop-in composition was not captured ({exc!r})", file=sys.stderr)
            torch.cuda.synchronize()
        layer.fused = True
    return dict(ms=ms, ms_e2e=ms_e2e, k_e2e=k_e2e, launches=launches, h2d=h2d, d2h=d2h, kernels=summ,
                graph=graphs is not None, dropin_ms=dropin_ms, dropin_graph_ms=dropin_graph_ms if dropin_ms else None,
                parity=parity,
                clocks=sampler.result(), dtype=dtype, precision=layer._precision(xs[0]))


def run_reference_triton(cfg, device, steps, warmup):
    """GPU baseline: the reference's own Triton kernels on this GPU.  Its `CVMM.apply` (imported by path from the pip
    install under baseline/_ref, nothing of this repository on that path) runs the up-projection, a ReLU and the
    down-projection, forward + backward, on tensors of the benchmark's shapes, together with what its layer does in
    torch around the two calls: the per-slot input ranges, a noisy copy of both weight tensors and the materialised
    output noise (moe_layer_aihwkit_lightning.py:447-492).  The reference has no ADC and no router / top-k / sort of its
    own (those live in a third-party package), so neither is in this number; the sorted slot list is built once,
    outside the timed region.  Autotuning happens in the warm-up."""
    path = os.path.join(ROOT, "baseline", "_ref", "analog_moe", "triton_src", "cvmm.py")
    if not os.path.exists(path):
        return {"unavailable": "baseline/_ref is not installed"}
    import importlib.util
    spec = importlib.util.spec_from_file_location("_reference_triton_cvmm", path)
    ref = importlib.util.module_from_spec(spec)
    sys.modules["_reference_triton_cvmm"] = ref
    spec.loader.exec_module(ref)
    dtype = torch.float32 if cfg["dtype"] == "fp32" else torch.bfloat16
    T, D, F, E, k = cfg["T"], cfg["D"], cfg["F"], cfg["E"], cfg["k"]
    g = torch.Generator().manual_seed(7)
    mk = lambda *shape, scale=1.0: (torch.randn(*shape, generator=g) * scale).to(device=device, dtype=dtype)
    x = mk(1, T, D).requires_grad_(cfg["bwd"])
    gy = mk(1, T, D)
    keys = mk(E, D, F, scale=D ** -0.5).requires_grad_(cfg["bwd"])
    values = mk(E, F, D, scale=F ** -0.5).requires_grad_(cfg["bwd"])
    input_range = torch.full((2, E), 3.0, device=device, dtype=dtype, requires_grad=cfg["bwd"])
    logits = torch.randn(T, E, generator=g).to(device)
    gate, raw_sel = torch.sigmoid(logits).topk(k, dim=-1)
    ssel, perm = torch.sort(raw_sel.flatten(), stable=True)
    sel3, raw3 = ssel.view(1, T, k), raw_sel.view(1, T, k)
    gate = gate.view(1, T, k).to(dtype).requires_grad_(cfg["bwd"])
    tok = perm // k

    class IR:
        enable, decay, input_min_percentage = True, 0.01, 0.95

    class IO:
        pass

    inp_res = 2.0 / 254.0
    training = cfg["bwd"]

    def projection(inp, sel_index, w, ir_row, out_index, rw):
        bir = input_range[ir_row][sel3]
        wm = w
        if training and cfg["w_noise"] > 0:
            with torch.no_grad():
                noise_w = cfg["w_noise"] * w.abs().amax(1, keepdim=True) * torch.randn_like(w)
            wm = w + noise_w
        noise = None
        if training and cfg["out_noise"] > 0:
            noise = torch.randn(1, T, k, w.shape[-1], device=device) * cfg["out_noise"] * w.abs().amax(1)[raw3]
        return ref.CVMM.apply(inp, sel_index, sel3, wm, inp_res, bir, out_index, rw, noise, IR, IO())

    def one_step():
        for t in (x, keys, values, input_range, gate):
            t.grad = None
        h = torch.relu(projection(x, tok, keys, 0, perm, None))
        y = projection(h, perm, values, 1, None, gate)
        if training:
            y.backward(gy)
        return y

    ctx = torch.enable_grad() if training else torch.no_grad()
    with ctx:
        for _ in range(max(warmup, 2)):
            one_step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            one_step()
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    return dict(value=T / (ms * 1e-3), unit="tokens/s", ms_per_step=ms, steps=steps,
                what="reference Triton CVMM.apply x2 + ReLU, fwd" + ("+bwd" if training else "") +
                     ", with the noise tensors its layer materialises; no ADC, no router/top-k/sort (the reference has "
                     "none); eager launches as the reference makes them")


def run_cpu(cfg, steps, warmup, sample_tokens=None):
    """CPU restatement of the reference arithmetic (oracle), all host threads, bounded sample."""
    from oracle import cvmm_oracle as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    T = sample_tokens or cfg["T"]
    g = torch.Generator().manual_seed(7)
    D, F, E, k = cfg["D"], cfg["F"], cfg["E"], cfg["k"]
    x = torch.randn(T, D, generator=g)
    gy = torch.randn(T, D, generator=g)
    wg = torch.randn(E, D, generator=g) / D ** 0.5
    keys = torch.randn(E, D, F, generator=g) / D ** 0.5
    values = torch.randn(E, F, D, generator=g) / F ** 0.5
    ir = torch.full((2, E), 3.0)
    lc = O.LayerConfig(k=k, inp_res=2.0 / 254.0, use_ir=True, out_noise=cfg["out_noise"], w_noise=cfg["w_noise"],
                       out_res=cfg.get("out_res", 254.0) if cfg["adc"] else -1.0, out_bound=OUT_BOUND, seed=SEED,
                       ir_params=O.IRParams(decay=0.01))
    for _ in range(warmup):
        O.layer_forward_backward(x[:64], wg, keys, values, ir, lc, gy[:64] if cfg["bwd"] else None)
    t0 = time.perf_counter()
    for _ in range(steps):
        O.layer_forward_backward(x, wg, keys, values, ir, lc, gy if cfg["bwd"] else None)
    dt = time.perf_counter() - t0
    return dict(tokens_per_s=T * steps / dt, cores=cores, seconds=dt, tokens=T, steps=steps)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c2", choices=sorted(CONFIGS))
    ap.add_argument("--precision", default=None, help="f16 | split | bf16x1 | fp32 (default: f16 for fp32 data, bf16x1 for bf16 data)")
    ap.add_argument("--cpu-sample-tokens", type=int, default=None)
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline leg (profiling runs)")
    ap.add_argument("--no-gpu-baseline", action="store_true", help="skip the reference-Triton leg (profiling runs)")
    ap.add_argument("--steps-only", action="store_true",
                    help="run warm-up and the steps eagerly and exit (no parity gate, baselines or other legs): for profilers")
    ap.add_argument("--no-graph", dest="graph", action="store_false",
                    help="launch every step eagerly instead of replaying a CUDA graph of the step")
    ap.add_argument("--kernel-times", default=None, metavar="PATH",
                    help="instead of the timed run: write per-kernel device times of three eager steps to PATH")
    ap.add_argument("--timeline", default=None, metavar="PATH",
                    help="instead of the timed run: write rank 0's kernel timeline of one (graph-replayed) step to PATH")
    args = ap.parse_args()
    cfg = CONFIGS[args.config]
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    mode = "fwd+bwd" if cfg["bwd"] else "fwd"
    flops_per_token = (12 if cfg["bwd"] else 4) * cfg["k"] * cfg["D"] * cfg["F"]
    workload = (f"{args.config}: one AnalogSigmaMoELayer {mode}, d_model={cfg['D']} experts={cfg['E']} "
                f"expert_size={cfg['F']} top-k={cfg['k']} tokens/GPU={cfg['T']} {cfg['dtype']}, 8-bit DAC"
                f"{', ADC out_res=%g out_bound=%g' % (cfg.get('out_res', 254.0), OUT_BOUND) if cfg['adc'] else ''}"
                f", out_noise={cfg['out_noise']} weight_noise={cfg['w_noise']} (Philox seed {SEED})")
    base = dict(metric="analog_cvmm_%s_tokens_per_s" % mode.replace("+", "_"), unit="tokens/s", n_gpus=args.gpus,
                steps=args.steps, warmup=args.warmup, higher_is_better=True, scaling="weak", vs_baseline=None,
                data="synthetic", config={"workload": workload, "flops_per_token": flops_per_token})

    if args.impl == "reference":
        if rank != 0:
            return
        k = max(1, min(args.steps, 3))
        r = run_cpu(cfg, k, min(args.warmup, 1), args.cpu_sample_tokens)
        line = dict(base, impl="reference", value=r["tokens_per_s"], steps=k, ms_per_step=1e3 * r["seconds"] / k,
                    dtype="f32", n_gpus=args.gpus,
                    cpu_baseline=dict(value=r["tokens_per_s"], unit="tokens/s", cores=r["cores"], kind="port",
                                      sample=f"{k} full step(s) of {r['tokens']} tokens; CPU restatement of the "
                                             "reference arithmetic (the reference has no CPU path for this layer)"),
                    e2e=dict(value=r["tokens_per_s"], unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                    tflops=r["tokens_per_s"] * flops_per_token / 1e12)
        print(json.dumps(line), flush=True)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path (use --impl reference for the CPU arm)")
    local = int(os.environ.get("LOCAL_RANK", 0))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    r = run_ours(args, cfg, rank, world, device)
    if r is None:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    if rank == 0:
        pk = peaks()
        ms_step = r["ms"] / args.steps
        tokens = cfg["T"] * world
        value = tokens / (ms_step * 1e-3)
        e2e_val = tokens / (r["ms_e2e"] / r["k_e2e"] * 1e-3)
        # dominant kernel: the library call with the largest share of device time
        gemm_flops = 2.0 * cfg["T"] * cfg["k"] * cfg["D"] * cfg["F"]
        kern = r["kernels"]
        total_ms = sum(v["ms_total"] for v in kern.values())
        # (the small exchanges of an expert-parallel step are waits for the other ranks, not work: never "dominant")
        cand = [n for n in kern if not n.startswith("amoe_ep_share")] or list(kern)
        top = max(cand, key=lambda n: kern[n]["ms_total"])
        is_gemm = top.startswith(("amoe_cvmm_fwd", "amoe_cvmm_dx", "amoe_cvmm_dw"))
        if is_gemm:
            ach = gemm_flops / (kern[top]["ms_avg"] * 1e-3) / 1e12
            roof = dict(kernel=top, bound="tensor", achieved=ach, peak=pk["tf"], unit="TFLOP/s", frac=ach / pk["tf"],
                        traffic=ncu_traffic(args.config).get(top) if world == 1 else None,
                        peak_source=pk["src"], share_of_step=kern[top]["ms_total"] / total_ms)
        elif top.startswith("amoe_ep_put") and world > 1:
            # a row exchange: bytes that leave this GPU over NVLink (balanced routing: (G-1)/G of the rows) against the
            # 770 GB/s per direction a peer copy reaches on this pool
            esz = 4 if cfg["dtype"] == "fp32" else 2
            if top.startswith("amoe_ep_put_f16"):
                esz = 2
            elif top.startswith("amoe_ep_put_back") and top.endswith("[down]") and cfg["adc"]:
                esz = 1                                  # ADC codes
            nbytes = cfg["T"] * cfg["k"] * cfg["D"] * esz * (world - 1) / world
            ach = nbytes / (kern[top]["ms_avg"] * 1e-3) / 1e9
            roof = dict(kernel=top, bound="nvlink", achieved=ach, peak=770.0, unit="GB/s", frac=ach / 770.0, traffic=None,
                        peak_source="peer copy per direction measured on this pool", share_of_step=kern[top]["ms_total"] / total_ms)
        else:
            roof = dict(kernel=top, bound="hbm", achieved=None, peak=pk["hbm"], unit="GB/s", frac=None, traffic=None,
                        peak_source=pk["src"], share_of_step=kern[top]["ms_total"] / total_ms)
        # the arithmetic type of the contraction (not of the stored tensors): operand type x accumulator type
        # (f32 accumulation throughout; config.precision spells the mode out)
        arith = {0: "bf16", 1: "bf16x2", 2: "f32", 3: "f16"}[r["precision"]]
        line = dict(base, value=value, ms_per_step=ms_step, dtype=arith,
                    data_dtype="f32" if cfg["dtype"] == "fp32" else "bf16",
                    tflops=value * flops_per_token / 1e12, tflops_frac_of_peak=value * flops_per_token / 1e12 / pk["tf"] / world,
                    e2e=dict(value=e2e_val, unit="tokens/s", h2d_bytes_per_step=r["h2d"], d2h_bytes_per_step=r["d2h"]),
                    gpu_launches=r["launches"], roofline=roof, clocks=r["clocks"],
                    kernels={k_: round(v["ms_avg"] * 1e3, 1) for k_, v in sorted(kern.items())})
        line["config"]["l2"] = "inputs rotate over 8 buffer sets (> 126 MB L2) and one step touches > 400 MB"
        line["config"]["cuda_graph"] = r["graph"]
        line["config"]["precision"] = {0: "bf16x1", 1: "split (bf16 hi+lo, fp32 accumulate)", 2: "fp32 CUDA cores",
                                       3: "f16x1 (fp16 operands, fp32 accumulate; parity key: distance to the fp32 kernels)"}[r["precision"]]
        if r.get("parity") is not None:
            line["parity"] = r["parity"]
        if r.get("dropin_ms"):
            best = r.get("dropin_graph_ms") or r["dropin_ms"]
            line["dropin"] = dict(value=cfg["T"] / (best * 1e-3), unit="tokens/s", ms_per_step=best,
                                  eager_ms_per_step=r["dropin_ms"], cuda_graph=bool(r.get("dropin_graph_ms")),
                                  what="the same step as two CVMM.apply calls with torch glue (the path the reference's "
                                       "layer files take through triton_src); replayed from a CUDA graph where the "
                                       "composition could be captured, with the eager figure beside it")
        if world == 1 and not args.no_gpu_baseline:
            try:
                line["gpu_baseline"] = run_reference_triton(cfg, device, max(3, min(args.steps, 10)), 3)
            except Exception as exc:       # recorded, never retried: the reference's kernels are not ours to debug
                line["gpu_baseline"] = {"unavailable": f"reference Triton path failed: {exc!r}"[:300]}
        if world == 1 and not args.no_cpu_baseline:
            c = run_cpu(cfg, 1, 1, args.cpu_sample_tokens)
            line["cpu_baseline"] = dict(value=c["tokens_per_s"], unit="tokens/s", cores=c["cores"], kind="port",
                                        sample=f"1 full step of {c['tokens']} tokens ({c['seconds']:.1f} s)")
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
