#!/usr/bin/env python
"""Benchmark of the TRWP / ISGMR message-passing hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" = one forward + backward pass of the layer over one batch of synthetic input
(forward only for the inference workloads).  Default workload: the segmentation training step
(TRWP, 2 images of 512x512 per GPU, 21 labels, 4 directions, 5 iterations, gradients to unary,
label context and edge weights); the batch is sharded 2 images per GPU, so N GPUs process 2N
images (weak scaling) and only the 21x21 label-context gradient is all-reduced.

Prints ONE JSON line.  `value` is whole-job throughput in pixel*label*iter/s with inputs resident
in HBM; `e2e` is the same metric through the public operator API (MPModule) with host buffers,
host<->device copies inside the timed region; `roofline` describes the dominant kernel (backward
sweep for training workloads, forward sweep otherwise) from per-launch CUDA-event timings;
`cpu_baseline` is the CPU implementation timed on this host on a bounded sample.
"""
import argparse
import types
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (generator, kwargs, fwd+bwd?)
    "seg_trwp_train": ("config4_segmentation", {}, True),
    "stereo_trwp_infer": ("config2_stereo", {}, False),
    "denoise_isgmr_infer": ("config3_denoise", {}, False),
    "large_isgmr_train": ("config5_large", {}, True),
    "config1_trwp_train": ("config1", {"mode": "TRWP"}, True),
    "config1_isgmr_train": ("config1", {"mode": "ISGMR"}, True),
    # the segmentation inputs run through ISGMR instead of TRWP (21 labels: the per-direction launches of an
    # iteration run side by side)
    "seg_isgmr_train": ("config4_segmentation", {"mode": "ISGMR"}, True),
    # soft (expected-value) TRWP on the segmentation inputs: saves L*L edge values per pixel, direction and
    # iteration (18.5 GB per step at full size); the 256 x 256 copy is the one small enough to profile
    "seg_trwp_soft_train": ("config4_segmentation", {"soft": True}, True),
    "seg_trwp_soft_train_256": ("config4_segmentation", {"soft": True, "H": 256, "W": 256, "n_iter": 2}, True),
    # reduced copy of large_isgmr_train (same labels / directions) that is small enough to profile
    "large_isgmr_train_384": ("config5_large", {"H": 384, "W": 384, "n_iter": 4}, True),
}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="seg_trwp_train", choices=list(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--shard", default="batch", choices=["batch", "directions"],
                    help="batch (default): every rank owns its own images, weak scaling; directions: ISGMR "
                         "workloads only, ONE image set on all ranks with each iteration's directions spread "
                         "over them (strong scaling, one all-reduce per iteration)")
    return ap.parse_args()


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.idx), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "samples": len(sm),
                "reasons": sorted(reasons)}


def units_per_step(cfg, batch):
    _, _, L, H, W = cfg["unary"].shape
    return batch * H * W * L * cfg["n_iter"]


def algorithmic_bytes(cfg, batch, kind):
    """Bytes one sweep launch must move (fused model): forward 4L(D+2)+4 (+L+1 when indices are
    saved) per pixel and direction; backward 4L(2D+3)+L+9.  A TRWP launch covers one direction;
    an ISGMR launch (forward or backward) covers all D directions of an iteration."""
    _, _, L, H, W = cfg["unary"].shape
    D = cfg["n_dir"]
    n = batch * H * W
    if cfg.get("soft"):
        # soft TRWP additionally writes (forward, training) / reads (backward) the L*L edge values
        if kind == "fwd":
            return n * (4 * L * (D + 2) + 4 + (4 * L * L + 1 if cfg["training"] else 0))
        return n * (4 * L * (2 * D + 3) + 4 * L * L + 9)
    if kind == "fwd":
        per_dir = n * (4 * L * (D + 2) + 4 + ((L + 1) if cfg["training"] else 0))
        return per_dir * (D if cfg["mode"] == "ISGMR" else 1)
    return n * (4 * L * (2 * D + 3) + L + 9) * (D if cfg["mode"] == "ISGMR" else 1)


def dominant_kernel(cfg, kind):
    """Name of the sweep kernel the workload spends its time in (see mplayers_b200/csrc)."""
    L = cfg["unary"].shape[2]
    pair = 32 < L <= 64 and L % 4 == 0
    if cfg.get("soft"):
        return "bwd_soft_kernel" if kind == "bwd" else "fwd_warp_kernel<soft>"
    if kind == "bwd":
        if L <= 32:
            return "bwd_tma_kernel" if cfg["mode"] == "TRWP" else "bwd_warp_kernel"
        return "bwd_pair_kernel" if pair else "bwd_cta_kernel"
    if L <= 32:
        return "fwd_tma_kernel"
    if not cfg["training"] and cfg["label_context"].dim() == 1 and L % 4 == 0:
        return "fwd_wide_kernel"
    if pair:
        return "fwd_pair_smem_kernel"
    return "fwd_cta_tma_kernel" if L % 4 == 0 else "fwd_cta_kernel"


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from the ncu
# captures summarised under profiles/ (same workload, one GPU); None where no capture exists.
NCU_TRAFFIC = {
    ("seg_trwp_train", "bwd"): 149.3e6 + 80.9e6,
    ("seg_trwp_train", "fwd"): 222.4e6 + 33.9e6,
    ("stereo_trwp_infer", "fwd"): 1788.5e6 + 338.6e6,
    # captured on the 384 x 384 copy of the workload (a full-size launch is too large to replay under
    # the profiler); traffic is proportional to the pixel count, so the full-size figures are those
    # times (1024 / 384)^2
    ("large_isgmr_train_384", "fwd"): 748.7e6 + 354.4e6,
    ("large_isgmr_train_384", "bwd"): 426.3e6 + 299.6e6,
    ("large_isgmr_train", "fwd"): (748.7e6 + 354.4e6) * (1024 / 384) ** 2,
    ("large_isgmr_train", "bwd"): (426.3e6 + 299.6e6) * (1024 / 384) ** 2,
}


# ---------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------
def run_ours(a):
    import torch
    import torch.distributed as dist
    from mplayers_b200 import MPModule, _lib, synthetic

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != a.gpus:
        if world == 1 and a.gpus > 1:
            raise SystemExit("--gpus %d needs `python -m torch.distributed.run --nproc-per-node %d bench.py ...`"
                             % (a.gpus, a.gpus))
        a.gpus = world
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    gen_name, kw, train = WORKLOADS[a.workload]
    kw = dict(kw)
    soft = bool(kw.pop("soft", False))
    by_dir = a.shard == "directions"
    if gen_name in ("config4_segmentation", "config5_large", "config1") and not by_dir:
        kw["seed"] = rank  # every rank owns its own slice of the global batch
    cfg = getattr(synthetic, gen_name)(**kw)
    batch = cfg["unary"].shape[0]
    cfg["soft"] = soft
    args = synthetic.make_args(cfg)
    if soft:
        from mplayers_b200.MP_module_hard_soft import MPModule as SoftModule
        args.mpnet_enable_soft = True
        layer = SoftModule(args)
    else:
        layer = MPModule(args)
    if by_dir:
        if cfg["mode"] != "ISGMR":
            raise SystemExit("--shard directions needs an ISGMR workload (TRWP directions are sequential)")
        from mplayers_b200 import direction_sharding
        dcomm = direction_sharding.TorchDistComm() if world > 1 else types.SimpleNamespace(
            rank=0, world_size=1, all_reduce=lambda t: t)
        layer.shard_directions(comm=dcomm)
    ctx_param = torch.nn.Parameter(cfg["label_context"].to(dev), requires_grad=train)
    layer.set_label_context(ctx_param, None, None)
    layer.train(train)

    unary_host = cfg["unary"].pin_memory()
    ew_host = cfg["edge_weights"].pin_memory() if cfg["edge_weights"] is not None else None
    unary = unary_host.to(dev)
    ew = ew_host.to(dev) if ew_host is not None else None
    gen = torch.Generator(device="cpu")
    gen.manual_seed(1234 + rank)
    dcost = torch.rand(cfg["unary"].shape, generator=gen).to(dev)

    from mplayers_b200 import ISGMRFunction, TRWPFunction
    fn = TRWPFunction if cfg["mode"] == "TRWP" else ISGMRFunction
    if soft:
        from mplayers_b200.MP_module_hard_soft import TRWPSoftFunction
        fn = TRWPSoftFunction
    args.training = train
    args.enable_saving_label = False

    from mplayers_b200 import parallel

    def reduce_context_grad():
        if world > 1 and not by_dir:  # the only cross-GPU exchange of the batch-sharded layer
            parallel.allreduce_label_context_grad(ctx_param.grad)

    def step_layer(u_hwl, e_dhw, g_hwl):
        """The layer proper: extension-level layouts ([B,cv,H,W,L], [D,B,cv,H,W]), no permutes."""
        if train:
            u = u_hwl.detach().requires_grad_(True)
            e = e_dhw.detach().requires_grad_(True) if e_dhw is not None else None
            ctx_param.grad = None
            if by_dir:
                cost = direction_sharding.isgmr_direction_sharded(u, ctx_param, e, args, comm=dcomm)
            else:
                cost = fn.apply(u, ctx_param, e, args)[0]
            cost.backward(g_hwl)
            reduce_context_grad()
            return cost
        with torch.no_grad():
            if by_dir:
                return direction_sharding.isgmr_direction_sharded(u_hwl, ctx_param, e_dhw, args, comm=dcomm)
            return fn.apply(u_hwl, ctx_param, e_dhw, args)[0]

    def step(u, e):
        """The call a user makes: MPModule on [B,cv,L,H,W] / [B,D,H,W]; returns the loss tensor."""
        if train:
            u = u.detach().requires_grad_(True)
            if e is not None:
                e = e.detach().requires_grad_(True)
            ctx_param.grad = None
            cost = layer(u, e)[0]
            loss = (cost * dcost).sum()
            loss.backward()
            reduce_context_grad()
            return loss
        with torch.no_grad():
            cost = layer(u, e)[0]
        return cost.sum()

    u_hwl = unary.permute(0, 1, 3, 4, 2).contiguous()
    e_dhw = ew.unsqueeze(1).permute(2, 0, 1, 3, 4).contiguous() if ew is not None else None
    g_hwl = dcost.permute(0, 1, 3, 4, 2).contiguous()

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(max(a.warmup, 3)):
        step_layer(u_hwl, e_dhw, g_hwl)
        step(unary, ew)
    sync_all()

    # ---- device-resident timing -------------------------------------------------------------
    sampler = ClockSampler("GPU-" + str(torch.cuda.get_device_properties(local).uuid))
    if rank == 0:
        sampler.start()
    launches0 = _lib.kernel_launches()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    ev0.record()
    for _ in range(a.steps):
        step_layer(u_hwl, e_dhw, g_hwl)
    ev1.record()
    sync_all()
    ms = ev0.elapsed_time(ev1)
    launches = _lib.kernel_launches() - launches0
    clocks = sampler.stop() if rank == 0 else None

    # ---- end to end: host buffers in, loss (and the context gradient) out ---------------------
    # Every step copies its inputs from pinned host memory and reads its result back inside the
    # timed region; the copy of step i + 1 runs on a side stream while step i computes
    # (mplayers_b200.host_feed.HostFeeder), the read-back of step i is awaited one step later.
    from mplayers_b200.host_feed import HostFeeder
    feeder = HostFeeder([unary_host, ew_host], dev)
    host_in = [unary_host, ew_host]
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    d2h = 0
    outs = []
    feeder.prefetch(host_in)
    for i in range(a.steps):
        u, e = feeder.get()
        if i + 1 < a.steps:
            feeder.prefetch(host_in)
        loss = step(u, e)
        feeder.release()
        out = torch.empty(loss.shape, dtype=loss.dtype, pin_memory=True)
        out.copy_(loss.detach(), non_blocking=True)
        d2h = out.numel() * out.element_size()
        if train:
            gh = torch.empty(ctx_param.grad.shape, dtype=ctx_param.grad.dtype, pin_memory=True)
            gh.copy_(ctx_param.grad, non_blocking=True)
            d2h += gh.numel() * gh.element_size()
            outs.append((out, gh))
        else:
            outs.append((out,))
    e1.record()
    sync_all()
    ms_e2e = e0.elapsed_time(e1)
    h2d = unary_host.numel() * 4 + (ew_host.numel() * 4 if ew_host is not None else 0)

    # ---- per-launch timing of the sweep kernels (separate pass, events around every launch) ----
    L = _lib.lib()
    import ctypes
    L.mpl_profile_reset()
    L.mpl_profile_enable(1)
    for _ in range(min(a.steps, 5)):
        step_layer(u_hwl, e_dhw, g_hwl)
    torch.cuda.synchronize()
    L.mpl_profile_enable(0)
    prof = {}
    for kind, name in ((0, "fwd"), (1, "bwd"), (2, "elementwise")):
        t, n = ctypes.c_double(0), ctypes.c_int64(0)
        L.mpl_profile_read(kind, ctypes.byref(t), ctypes.byref(n))
        prof[name] = (t.value, n.value)

    # max over ranks
    if world > 1:
        t = torch.tensor([ms, ms_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])
        lt = torch.tensor([launches], device=dev, dtype=torch.int64)
        dist.all_reduce(lt)
        launches = int(lt[0])

    if rank == 0:
        units = units_per_step(cfg, batch) * (1 if by_dir else world)
        peak, peak_src = measured_peak()
        # the sweep kind the step spends most of its time in
        dom = "bwd" if (train and prof["bwd"][0] >= prof["fwd"][0]) else "fwd"
        t_dom, n_dom = prof[dom]
        roof = None
        if n_dom:
            per_launch_ms = t_dom / n_dom
            bytes_launch = algorithmic_bytes(cfg, batch, dom)
            achieved = bytes_launch / (per_launch_ms * 1e-3) / 1e9
            roof = {"bound": "hbm", "kernel": dominant_kernel(cfg, dom),
                    "achieved": round(achieved, 1), "peak": peak, "peak_source": peak_src, "unit": "GB/s",
                    "frac": round(achieved / peak, 4), "traffic": NCU_TRAFFIC.get((a.workload, dom)),
                    "avg_launch_ms": round(per_launch_ms, 5), "algorithmic_bytes_per_launch": bytes_launch}
        other = {}
        for k in ("fwd", "bwd", "elementwise"):
            if prof[k][1]:
                other[k] = {"launches": prof[k][1], "avg_ms": round(prof[k][0] / prof[k][1], 5)}
                if k in ("fwd", "bwd"):
                    other[k]["algorithmic_GBps"] = round(
                        algorithmic_bytes(cfg, batch, k) / (prof[k][0] / prof[k][1] * 1e-3) / 1e9, 1)
        _, _, Lb, H, W = cfg["unary"].shape
        line = {
            "metric": "TRWP/ISGMR fwd+bwd pixel*label*iter/s" if train else "TRWP/ISGMR fwd pixel*label*iter/s",
            "value": units * a.steps / (ms * 1e-3), "unit": "pixel*label*iter/s",
            "n_gpus": world, "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": ms / a.steps,
            "higher_is_better": True, "scaling": "strong" if by_dir else "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": a.workload, "mode": cfg["mode"], "shard": a.shard, "batch_per_gpu": batch,
                       "global_batch": batch * (1 if by_dir else world), "height": H, "width": W, "labels": Lb,
                       "directions": cfg["n_dir"], "iterations": cfg["n_iter"],
                       "pass": "fwd+bwd" if train else "fwd",
                       "l2": "working set per step (messages, indices, gradients) exceeds the 126 MB L2"},
            "e2e": {"value": units * a.steps / (ms_e2e * 1e-3), "unit": "pixel*label*iter/s",
                    "ms_per_step": ms_e2e / a.steps, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches, "clocks": clocks, "roofline": roof, "kernels": other,
        }
        if not a.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline(a.workload, target_s=12.0)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------
# CPU arms (the oracle / the reference's own CPU code are test infrastructure; this is the one
# place outside tests where they are executed, as the measured baseline)
# ---------------------------------------------------------------------------------------------
_CFG_CACHE = {}


def _cpu_sample(workload, edge):
    """Centred crop of the workload with `edge` x `edge` pixels (first image), numpy layouts."""
    import numpy as np
    from mplayers_b200 import synthetic
    gen_name, kw, train = WORKLOADS[workload]
    kw = dict(kw)
    soft = bool(kw.pop("soft", False))
    if workload not in _CFG_CACHE:
        _CFG_CACHE[workload] = getattr(synthetic, gen_name)(**kw)
        _CFG_CACHE[workload]["soft"] = soft
    cfg = _CFG_CACHE[workload]
    u = cfg["unary"][:1]
    _, _, L, H, W = u.shape
    eh, ew_ = min(edge, H), min(edge, W)
    h0, w0 = (H - eh) // 2, (W - ew_) // 2
    u = u[:, :, :, h0:h0 + eh, w0:w0 + ew_].permute(0, 1, 3, 4, 2).contiguous().numpy()
    e = cfg["edge_weights"]
    if e is not None:
        e = e[:1, :, h0:h0 + eh, w0:w0 + ew_].unsqueeze(1).permute(2, 0, 1, 3, 4).contiguous().numpy()
    return cfg, train, u, cfg["label_context"].numpy().astype(np.float32), e


def _time_cpu(workload, edge, use_reference=True):
    """One CPU pass over the sample.  Forward: the reference's own C++ CPU code when it was built
    (oracle/_ref), else the C port; backward (training workloads): the C port, because the
    reference has no CPU backward (MPLayers/TRWP/TRWP.cpp:316).  Returns (units, seconds, used_ref)."""
    import numpy as np
    from oracle import oracle, ref_cpu
    cfg, train, u, ctx, e = _cpu_sample(workload, edge)
    if cfg.get("soft"):  # the reference has no CPU implementation of the soft variant: C port
        t0 = time.perf_counter()
        fwd = oracle.forward_soft(u, ctx, e, cfg["n_dir"], cfg["n_iter"], training=train)
        g = np.random.default_rng(0).uniform(0, 1, size=u.shape).astype(np.float32)
        if train:
            oracle.backward_soft(ctx, e, g, fwd["edge_label"], fwd["norm_idx"])
        return u.shape[2] * u.shape[3] * u.shape[4] * cfg["n_iter"], time.perf_counter() - t0, False
    use_ref = use_reference and ref_cpu.available()
    fwd = None
    if use_ref:
        if train:  # indices for the backward leg come from the port; not part of the timed forward
            fwd = oracle.forward(cfg["mode"], u, ctx, e, cfg["n_dir"], cfg["n_iter"], training=True)
        t0 = time.perf_counter()
        ref_cpu.forward(cfg["mode"], u, ctx, cfg["n_dir"], cfg["n_iter"])
        t_f = time.perf_counter() - t0
    else:
        t0 = time.perf_counter()
        fwd = oracle.forward(cfg["mode"], u, ctx, e, cfg["n_dir"], cfg["n_iter"], training=train)
        t_f = time.perf_counter() - t0
    t_b = 0.0
    if train:
        g = np.random.default_rng(0).uniform(0, 1, size=u.shape).astype(np.float32)
        t1 = time.perf_counter()
        oracle.backward(cfg["mode"], ctx, e, g, fwd["min_idx"], fwd["norm_idx"])
        t_b = time.perf_counter() - t1
    units = u.shape[2] * u.shape[3] * u.shape[4] * cfg["n_iter"]
    return units, t_f + t_b, use_ref


def _pick_edge(workload, per_pass_s):
    """Largest power-of-two crop whose CPU pass stays near `per_pass_s` seconds."""
    edge = 32
    units, t, _ = _time_cpu(workload, edge)  # also warms up the libraries
    units, t, _ = _time_cpu(workload, edge)
    shape = _CFG_CACHE[workload]["unary"].shape
    while edge < max(shape[3], shape[4]):
        if t * 4 > per_pass_s:
            break
        edge *= 2
        units, t, _ = _time_cpu(workload, edge)
    return edge


def _describe(workload, edge, used_ref, units, t):
    from oracle import oracle
    train = WORKLOADS[workload][2]
    what = ("forward: the reference's ForwardCPU compiled from its sources (its fixed 16 OpenMP "
            "threads; edge weights ignored by that code)" if used_ref else "forward: C port")
    if train:
        what += "; backward: C port (the reference has no CPU backward), %d threads" % oracle.max_threads()
    return {"value": units / t, "unit": "pixel*label*iter/s", "cores": 16 if used_ref else oracle.max_threads(),
            "host_cpus": os.cpu_count(), "kind": "reference" if used_ref else "port",
            "seconds": round(t, 3),
            "sample": "centred %dx%d crop of one image of %s; %s"
                      % (min(edge, _CFG_CACHE[workload]["unary"].shape[3]),
                         min(edge, _CFG_CACHE[workload]["unary"].shape[4]), workload, what)}


def cpu_baseline(workload, target_s=12.0):
    edge = _pick_edge(workload, target_s / 3)
    best = None
    for _ in range(2):
        units, t, used_ref = _time_cpu(workload, edge)
        if best is None or t < best[1]:
            best = (units, t, used_ref)
    return _describe(workload, edge, best[2], best[0], best[1])


def run_reference(a):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    budget = 150.0 / max(a.steps + max(a.warmup, 1), 1)   # the whole run stays within a few minutes
    edge = _pick_edge(a.workload, min(budget, 8.0))
    for _ in range(max(a.warmup, 1)):
        _time_cpu(a.workload, edge)
    res = []
    t0 = time.perf_counter()
    for _ in range(a.steps):
        res.append(_time_cpu(a.workload, edge))
    wall = time.perf_counter() - t0
    res.sort(key=lambda r: r[1])
    units, t, used_ref = res[len(res) // 2]
    cb = _describe(a.workload, edge, used_ref, units, t)
    train = WORKLOADS[a.workload][2]
    line = {"impl": "reference",
            "metric": "TRWP/ISGMR fwd+bwd pixel*label*iter/s" if train else "TRWP/ISGMR fwd pixel*label*iter/s",
            "value": cb["value"], "unit": "pixel*label*iter/s", "n_gpus": a.gpus, "steps": a.steps,
            "warmup": max(a.warmup, 1), "ms_per_step": wall / a.steps * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": a.workload}, "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "pixel*label*iter/s", "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


if __name__ == "__main__":
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
