#!/usr/bin/env python
"""Benchmark of the TRWP / ISGMR message-passing hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" = one forward + backward pass of the layer over one batch of synthetic input
(forward only for the inference workloads).  Headline workload: the segmentation training step
(TRWP, 2 images of 512x512 per GPU, 21 labels, 4 directions, 5 iterations, gradients to unary,
label context and edge weights); the batch is sharded 2 images per GPU, so N GPUs process 2N
images (weak scaling) and only the 21x21 label-context gradient is all-reduced.

Prints ONE JSON line.  `value` is whole-job throughput in pixel*label*iter/s with inputs resident
in HBM; `e2e` is the same metric through the public operator API (MPModule) with host buffers,
host<->device copies inside the timed region; `roofline` describes the sweep kernels from
per-launch CUDA-event timings (`frac`: the dominant kernel; `fwd_frac`, `bwd_frac`: both sweep
kinds; `step_frac`: every algorithmic byte of the step over the whole step time);
`cpu_baseline` is the CPU implementation timed on this host on a bounded sample.  `workloads`
carries the other configurations (stereo and denoising inference, large ISGMR training) measured
the same way in the same run.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time
import types

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (generator, kwargs, fwd+bwd?)
    "seg_trwp_train": ("config4_segmentation", {}, True),
    "stereo_trwp_infer": ("config2_stereo", {}, False),
    # the same inputs as a training step (learning the truncated-linear function): indices saved, fwd+bwd
    "stereo_trwp_train": ("config2_stereo", {"training": True}, True),
    # reduced copy of it (same labels, directions and context) that is small enough to profile
    "stereo_trwp_train_188": ("config2_stereo", {"training": True, "H": 188, "W": 620}, True),
    "denoise_isgmr_infer": ("config3_denoise", {}, False),
    # the same inputs as a training step (learning the truncated-quadratic function), 10 iterations
    "denoise_isgmr_train": ("config3_denoise", {"training": True, "n_iter": 10}, True),
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
# the configurations carried in the `workloads` block next to the headline one
# (the stereo inputs also as a training step: the 192-label forward + backward)
EXTRA_WORKLOADS = ["stereo_trwp_infer", "stereo_trwp_train", "denoise_isgmr_infer", "large_isgmr_train"]
METRIC_UNIT = "pixel*label*iter/s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="seg_trwp_train", choices=list(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra-workloads", action="store_true",
                    help="measure the headline workload only (the `workloads` block is left out)")
    ap.add_argument("--min-timed-seconds", type=float, default=1.0,
                    help="the K timed steps are repeated until the device-timed region is at least this long")
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
    """Samples SM clocks and throttle reasons with nvidia-smi from before the warm-up to the end of
    the run; the summary uses the samples that fall inside the timed regions (marked by the caller)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_id):
        self.id = gpu_id
        self.proc = None
        self.samples = []   # (host time, fields)
        self.windows = []   # (t0, t1) of timed regions

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.id), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def wait_first_sample(self, timeout=10.0):
        t0 = time.time()
        while self.proc is not None and not self.samples and time.time() - t0 < timeout:
            time.sleep(0.05)

    def window(self, t0, t1):
        self.windows.append((t0, t1))

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

        def summarise(rows):
            sm, mx, reasons, power = [], None, set(), []
            for _, ln in rows:
                f = [x.strip() for x in ln.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx = float(f[2])
                    power.append(float(f[3]))
                except ValueError:
                    continue
                for name, v in zip(names, f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            sm.sort()
            return sm, mx, sorted(reasons), (max(power) if power else None)

        timed = [s for s in self.samples if any(a <= s[0] <= b for a, b in self.windows)]
        use = timed if timed else self.samples
        sm, mx, reasons, pw = summarise(use)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "samples": len(sm),
                "samples_total": len(self.samples), "power_w_max": pw, "reasons": reasons,
                "scope": "samples inside the timed regions" if timed else "whole run (no sample fell inside a timed region)"}


# ---------------------------------------------------------------------------------------------
# byte model (fused model: every sweep reads its inputs once and writes its outputs once)
# ---------------------------------------------------------------------------------------------
def units_per_step(cfg, batch):
    _, _, L, H, W = cfg["unary"].shape
    return batch * H * W * L * cfg["n_iter"]


def algorithmic_bytes(cfg, batch, kind):
    """Bytes one sweep launch must move: forward 4L(D+2)+4 (+L+1 when indices are saved) per pixel
    and direction; backward 4L(2D+3)+L+9.  A TRWP launch covers one direction; an ISGMR launch
    (forward or backward) covers all D directions of an iteration."""
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


def step_bytes(cfg, batch, train):
    """Algorithmic bytes of a whole step: every sweep of every iteration plus, once per pass, the
    cost aggregation / backward prologue (4L(D+2) per pixel).  Returns (forward, backward)."""
    _, _, L, H, W = cfg["unary"].shape
    D, I = cfg["n_dir"], cfg["n_iter"]
    n = batch * H * W
    launches = I if cfg["mode"] == "ISGMR" else I * D
    once = n * 4 * L * (D + 2)
    fwd = launches * algorithmic_bytes(cfg, batch, "fwd") + once
    bwd = (launches * algorithmic_bytes(cfg, batch, "bwd") + once) if train else 0
    return fwd, bwd


def dominant_kernel(cfg, kind):
    """Name of the sweep kernel the workload spends its time in (see mplayers_b200/csrc)."""
    L = cfg["unary"].shape[2]
    pair = 32 < L <= 64 and L % 4 == 0
    if cfg.get("soft"):
        return "bwd_soft_kernel" if kind == "bwd" else "fwd_warp_kernel<soft>"
    if kind == "bwd":
        if L <= 32:
            return "bwd_tma_kernel"
        if cfg["label_context"].dim() == 1 and 32 < L <= 256 and L % 4 == 0:
            return "bwd_wide_kernel"
        return "bwd_pair_kernel" if pair else "bwd_cta_kernel"
    if L <= 32:
        return "fwd_tma_kernel"
    if (not cfg["training"] or L > 64) and cfg["label_context"].dim() == 1 and L % 4 == 0:
        return "fwd_wide_kernel"
    if pair:
        return "fwd_pair_smem_kernel"
    return "fwd_cta_tma_kernel" if L % 4 == 0 else "fwd_cta_kernel"


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the sweep kernels, from the ncu
# captures summarised under profiles/ (same workload, one GPU); None where no capture exists.
NCU_TRAFFIC = {
    ("seg_trwp_train", "bwd"): 149.3e6 + 80.9e6,
    ("seg_trwp_train", "fwd"): 222.4e6 + 33.9e6,
    ("stereo_trwp_infer", "fwd"): 1788.5e6 + 338.6e6,
    ("stereo_trwp_train", "bwd"): 1163.8e6 + 1017.2e6,
    ("denoise_isgmr_infer", "fwd"): 728.4e6 + 245.6e6,
    # captured on the 384 x 384 copy of the workload (a full-size launch is too large to replay under
    # the profiler); traffic is proportional to the pixel count, so the full-size figures are those
    # times (1024 / 384)^2
    ("large_isgmr_train_384", "fwd"): 748.7e6 + 354.4e6,
    ("large_isgmr_train_384", "bwd"): 426.3e6 + 299.6e6,
    ("large_isgmr_train", "fwd"): (748.7e6 + 354.4e6) * (1024 / 384) ** 2,
    ("large_isgmr_train", "bwd"): (426.3e6 + 299.6e6) * (1024 / 384) ** 2,
}


def config_dict(workload, cfg_shape, mode, n_dir, n_iter, train, shard, batch, world):
    """The `config` object of the JSON line; identical for both arms of one invocation."""
    L, H, W = cfg_shape
    by_dir = shard == "directions"
    return {"workload": workload, "mode": mode, "shard": shard, "batch_per_gpu": batch,
            "global_batch": batch * (1 if by_dir else world), "height": H, "width": W, "labels": L,
            "directions": n_dir, "iterations": n_iter, "pass": "fwd+bwd" if train else "fwd",
            "l2": "working set per step (messages, indices, gradients) exceeds the 126 MB L2"}


# ---------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------
class Runner:
    """One workload on this rank's GPU: generated inputs, the layer, and the two kinds of step."""

    def __init__(self, workload, rank, world, local, shard):
        import torch
        from mplayers_b200 import MPModule, synthetic
        self.torch = torch
        self.workload, self.rank, self.world = workload, rank, world
        self.dev = torch.device("cuda", local)
        gen_name, kw, self.train = WORKLOADS[workload]
        kw = dict(kw)
        self.soft = bool(kw.pop("soft", False))
        self.by_dir = shard == "directions"
        if gen_name in ("config4_segmentation", "config5_large", "config1") and not self.by_dir:
            kw["seed"] = rank  # every rank owns its own slice of the global batch
        self.cfg = cfg = getattr(synthetic, gen_name)(**kw)
        self.batch = cfg["unary"].shape[0]
        cfg["soft"] = self.soft
        self.args = args = synthetic.make_args(cfg)
        if self.soft:
            from mplayers_b200.MP_module_hard_soft import MPModule as SoftModule
            args.mpnet_enable_soft = True
            self.layer = SoftModule(args)
        else:
            self.layer = MPModule(args)
        self.dcomm = None
        if self.by_dir:
            if cfg["mode"] != "ISGMR":
                raise SystemExit("--shard directions needs an ISGMR workload (TRWP directions are sequential)")
            from mplayers_b200 import direction_sharding
            self.dsh = direction_sharding
            self.dcomm = direction_sharding.TorchDistComm() if world > 1 else types.SimpleNamespace(
                rank=0, world_size=1, all_reduce=lambda t: t)
            self.layer.shard_directions(comm=self.dcomm)
        self.ctx_param = torch.nn.Parameter(cfg["label_context"].to(self.dev), requires_grad=self.train)
        self.layer.set_label_context(self.ctx_param, None, None)
        self.layer.train(self.train)

        self.unary_host = cfg["unary"].pin_memory()
        self.ew_host = cfg["edge_weights"].pin_memory() if cfg["edge_weights"] is not None else None
        self.unary = self.unary_host.to(self.dev)
        self.ew = self.ew_host.to(self.dev) if self.ew_host is not None else None
        gen = torch.Generator(device="cpu")
        gen.manual_seed(1234 + rank)
        self.dcost = torch.rand(cfg["unary"].shape, generator=gen).to(self.dev)

        from mplayers_b200 import ISGMRFunction, TRWPFunction
        self.fn = TRWPFunction if cfg["mode"] == "TRWP" else ISGMRFunction
        if self.soft:
            from mplayers_b200.MP_module_hard_soft import TRWPSoftFunction
            self.fn = TRWPSoftFunction
        args.training = self.train
        args.enable_saving_label = False
        # what MPModule.forward hands down for inference with a rank-1 context (no read-back per call)
        args.context_window = self.layer._context_window(self.ctx_param.detach(), self.ew) if not self.soft else 0
        self.u_hwl = self.unary.permute(0, 1, 3, 4, 2).contiguous()
        self.e_dhw = self.ew.unsqueeze(1).permute(2, 0, 1, 3, 4).contiguous() if self.ew is not None else None
        self.g_hwl = self.dcost.permute(0, 1, 3, 4, 2).contiguous()

    def reduce_context_grad(self):
        if self.world > 1 and not self.by_dir:  # the only cross-GPU exchange of the batch-sharded layer
            from mplayers_b200 import parallel
            parallel.allreduce_label_context_grad(self.ctx_param)

    def step_layer(self):
        """The layer proper: extension-level layouts ([B,cv,H,W,L], [D,B,cv,H,W]), no permutes."""
        torch = self.torch
        if self.train:
            u = self.u_hwl.detach().requires_grad_(True)
            e = self.e_dhw.detach().requires_grad_(True) if self.e_dhw is not None else None
            self.ctx_param.grad = None
            if self.by_dir:
                cost = self.dsh.isgmr_direction_sharded(u, self.ctx_param, e, self.args, comm=self.dcomm)
            else:
                cost = self.fn.apply(u, self.ctx_param, e, self.args)[0]
            cost.backward(self.g_hwl)
            self.reduce_context_grad()
            return cost
        with torch.no_grad():
            if self.by_dir:
                return self.dsh.isgmr_direction_sharded(self.u_hwl, self.ctx_param, self.e_dhw, self.args,
                                                        comm=self.dcomm)
            return self.fn.apply(self.u_hwl, self.ctx_param, self.e_dhw, self.args)[0]

    def step_module(self, u, e):
        """The call a user makes: MPModule on [B,cv,L,H,W] / [B,D,H,W]; returns the loss tensor."""
        torch = self.torch
        if self.train:
            u = u.detach().requires_grad_(True)
            if e is not None:
                e = e.detach().requires_grad_(True)
            self.ctx_param.grad = None
            cost = self.layer(u, e)[0]
            loss = (cost * self.dcost).sum()
            loss.backward()
            self.reduce_context_grad()
            return loss
        with torch.no_grad():
            cost = self.layer(u, e)[0]
        return cost.sum()

    def free(self):
        for k in ("unary", "ew", "dcost", "u_hwl", "e_dhw", "g_hwl", "unary_host", "ew_host", "layer", "cfg"):
            setattr(self, k, None)
        self.torch.cuda.empty_cache()


def measure(r, steps, warmup, min_seconds, sampler, sync_all, with_e2e=True):
    """Device-resident timing, end-to-end timing and per-launch sweep timing of one workload."""
    import ctypes
    torch = r.torch
    from mplayers_b200 import _lib
    for _ in range(max(warmup, 3)):
        r.step_layer()
        if with_e2e:
            r.step_module(r.unary, r.ew)
    sync_all()

    # ---- device-resident timing: K steps, repeated until the region is at least min_seconds long ----
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    r.step_layer()
    ev1.record()
    sync_all()
    est = max(ev0.elapsed_time(ev1), 1e-3)
    repeats = max(1, int(min_seconds * 1e3 / (est * steps) + 0.999))
    launches0 = _lib.kernel_launches()
    sync_all()
    t0 = time.time()
    ev0.record()
    for _ in range(repeats * steps):
        r.step_layer()
    ev1.record()
    sync_all()
    sampler.window(t0, time.time())
    ms = ev0.elapsed_time(ev1) / repeats          # per K steps
    launches = (_lib.kernel_launches() - launches0) // repeats

    # ---- end to end: host buffers in, loss (and the context gradient) out ---------------------
    # Every step copies its inputs from pinned host memory and reads its result back inside the
    # timed region; the copy of step i + 1 runs on a side stream while step i computes
    # (mplayers_b200.host_feed.HostFeeder), the read-back of step i is awaited one step later.
    ms_e2e = h2d = d2h = None
    if with_e2e:
        from mplayers_b200.host_feed import HostFeeder
        feeder = HostFeeder([r.unary_host, r.ew_host], r.dev)
        host_in = [r.unary_host, r.ew_host]
        n_e2e = steps * min(repeats, max(1, int(0.5 * repeats + 0.5)))
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time()
        e0.record()
        outs = []
        feeder.prefetch(host_in)
        for i in range(n_e2e):
            u, e = feeder.get()
            if i + 1 < n_e2e:
                feeder.prefetch(host_in)
            loss = r.step_module(u, e)
            feeder.release()
            out = torch.empty(loss.shape, dtype=loss.dtype, pin_memory=True)
            out.copy_(loss.detach(), non_blocking=True)
            d2h = out.numel() * out.element_size()
            if r.train:
                gh = torch.empty(r.ctx_param.grad.shape, dtype=r.ctx_param.grad.dtype, pin_memory=True)
                gh.copy_(r.ctx_param.grad, non_blocking=True)
                d2h += gh.numel() * gh.element_size()
                outs.append((out, gh))
            else:
                outs.append((out,))
            if len(outs) > 4:
                outs.pop(0)
        e1.record()
        sync_all()
        sampler.window(t0, time.time())
        ms_e2e = e0.elapsed_time(e1) * steps / n_e2e   # per K steps
        h2d = r.unary_host.numel() * 4 + (r.ew_host.numel() * 4 if r.ew_host is not None else 0)
        del feeder

    # ---- per-launch timing of the sweep kernels (separate pass, events around every launch) ----
    L = _lib.lib()
    L.mpl_profile_reset()
    L.mpl_profile_enable(1)
    t0 = time.time()
    for _ in range(min(steps, 5)):
        r.step_layer()
    torch.cuda.synchronize()
    sampler.window(t0, time.time())
    L.mpl_profile_enable(0)
    prof = {}
    for kind, name in ((0, "fwd"), (1, "bwd"), (2, "elementwise")):
        t, n = ctypes.c_double(0), ctypes.c_int64(0)
        L.mpl_profile_read(kind, ctypes.byref(t), ctypes.byref(n))
        prof[name] = (t.value, n.value)
    _lib.poll_status(wait=True)   # a staging wait that gave up anywhere above raises here
    return dict(ms=ms, ms_e2e=ms_e2e, h2d=h2d, d2h=d2h, launches=int(launches), prof=prof, repeats=repeats)


def roofline_of(r, workload, m, steps, peak, peak_src):
    """Per-kind launch times against the byte model, the dominant kernel, and the whole step."""
    cfg, batch, prof = r.cfg, r.batch, m["prof"]
    # direction sharding: a rank's sweep launch covers its own directions (or its part of a direction
    # pair's chains) only, and the step's bytes are spread over all ranks
    share = 1.0
    if r.by_dir and r.world > 1:
        _, count, _, parts = r.dsh.shard_plan(cfg["n_dir"], r.world)[r.rank]
        share = count / float(parts * cfg["n_dir"])
    kinds = {}
    for k in ("fwd", "bwd", "elementwise"):
        if prof[k][1]:
            kinds[k] = {"launches": prof[k][1], "avg_launch_ms": round(prof[k][0] / prof[k][1], 5)}
            if k in ("fwd", "bwd"):
                b = int(algorithmic_bytes(cfg, batch, k) * share)
                gbs = b / (prof[k][0] / prof[k][1] * 1e-3) / 1e9
                kinds[k].update({"kernel": dominant_kernel(cfg, k), "algorithmic_bytes_per_launch": b,
                                 "algorithmic_GBps": round(gbs, 1), "frac": round(gbs / peak, 4)})
                tr = NCU_TRAFFIC.get((workload, k))
                if tr is not None:
                    tr = tr * share
                    kinds[k]["dram_bytes_per_launch"] = tr
                    kinds[k]["dram_frac"] = round(tr / (prof[k][0] / prof[k][1] * 1e-3) / 1e9 / peak, 4)
    fb, bb = step_bytes(cfg, batch, r.train)
    ms_step = m["ms"] / steps
    step_frac = (fb + bb) / (ms_step * 1e-3) / 1e9 / peak / (r.world if r.by_dir else 1)
    dom = "bwd" if (r.train and prof["bwd"][0] >= prof["fwd"][0]) else "fwd"
    roof = None
    if dom in kinds:
        d = kinds[dom]
        roof = {"bound": "hbm", "kernel": d["kernel"], "achieved": d["algorithmic_GBps"], "peak": peak,
                "peak_source": peak_src, "unit": "GB/s", "frac": d["frac"],
                "traffic": d.get("dram_bytes_per_launch"), "avg_launch_ms": d["avg_launch_ms"],
                "algorithmic_bytes_per_launch": d["algorithmic_bytes_per_launch"],
                "fwd_frac": kinds.get("fwd", {}).get("frac"), "bwd_frac": kinds.get("bwd", {}).get("frac"),
                "step_frac": round(step_frac, 4), "step_algorithmic_bytes": fb + bb,
                "step_ms_at_peak": round((fb + bb) / peak / 1e6, 4)}
    return roof, kinds, round(step_frac, 4)


def run_ours(a):
    import torch
    import torch.distributed as dist
    from mplayers_b200 import _lib  # noqa: F401  (fails loudly here when the library is not built)

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
    sampler = ClockSampler("GPU-" + str(torch.cuda.get_device_properties(local).uuid))
    if rank == 0:
        sampler.start()           # before the warm-up: nvidia-smi needs a moment to deliver its first line
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(vals):
        if world == 1:
            return vals
        t = torch.tensor([v if v is not None else -1.0 for v in vals], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(x) if v is not None else None for x, v in zip(t, vals)]

    peak, peak_src = measured_peak()
    r = Runner(a.workload, rank, world, local, a.shard)
    if rank == 0:
        sampler.wait_first_sample()
    m = measure(r, a.steps, a.warmup, a.min_timed_seconds, sampler, sync_all)
    m["ms"], m["ms_e2e"] = max_over_ranks([m["ms"], m["ms_e2e"]])
    if world > 1:
        lt = torch.tensor([m["launches"]], device=dev, dtype=torch.int64)
        dist.all_reduce(lt)
        m["launches"] = int(lt[0])
    by_dir = a.shard == "directions"
    line = None
    if rank == 0:
        cfg, batch, train = r.cfg, r.batch, r.train
        units = units_per_step(cfg, batch) * (1 if by_dir else world)
        roof, kinds, _ = roofline_of(r, a.workload, m, a.steps, peak, peak_src)
        _, _, Lb, H, W = cfg["unary"].shape
        line = {
            "metric": "TRWP/ISGMR fwd+bwd pixel*label*iter/s" if train else "TRWP/ISGMR fwd pixel*label*iter/s",
            "value": units * a.steps / (m["ms"] * 1e-3), "unit": METRIC_UNIT,
            "n_gpus": world, "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": m["ms"] / a.steps,
            "timed_repeats": m["repeats"], "timed_seconds": round(m["ms"] * m["repeats"] * 1e-3, 3),
            "higher_is_better": True, "scaling": "strong" if by_dir else "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": config_dict(a.workload, (Lb, H, W), cfg["mode"], cfg["n_dir"], cfg["n_iter"], train, a.shard,
                                  batch, world),
            "e2e": {"value": units * a.steps / (m["ms_e2e"] * 1e-3), "unit": METRIC_UNIT,
                    "ms_per_step": m["ms_e2e"] / a.steps, "h2d_bytes_per_step": m["h2d"],
                    "d2h_bytes_per_step": m["d2h"]},
            "gpu_launches": m["launches"], "roofline": roof, "kernels": kinds,
        }
    r.free()
    del r

    # ---- the other configurations, measured the same way in the same run ----------------------
    extras = {}
    if not a.no_extra_workloads and not by_dir:
        for name in EXTRA_WORKLOADS:
            if name == a.workload:
                continue
            rr = Runner(name, rank, world, local, "batch")
            k = max(3, min(a.steps, 10))
            mm = measure(rr, k, 3, min(a.min_timed_seconds, 0.5), sampler, sync_all)
            mm["ms"], mm["ms_e2e"] = max_over_ranks([mm["ms"], mm["ms_e2e"]])
            if rank == 0:
                cfg = rr.cfg
                units = units_per_step(cfg, rr.batch) * world
                roof, kinds, step_frac = roofline_of(rr, name, mm, k, peak, peak_src)
                _, _, Lb, H, W = cfg["unary"].shape
                extras[name] = {
                    "metric": "TRWP/ISGMR fwd+bwd pixel*label*iter/s" if rr.train else "TRWP/ISGMR fwd pixel*label*iter/s",
                    "value": units * k / (mm["ms"] * 1e-3), "unit": METRIC_UNIT, "ms_per_step": mm["ms"] / k,
                    "steps": k, "timed_repeats": mm["repeats"],
                    "config": config_dict(name, (Lb, H, W), cfg["mode"], cfg["n_dir"], cfg["n_iter"], rr.train,
                                          "batch", rr.batch, world),
                    "e2e": {"value": units * k / (mm["ms_e2e"] * 1e-3), "unit": METRIC_UNIT,
                            "ms_per_step": mm["ms_e2e"] / k, "h2d_bytes_per_step": mm["h2d"],
                            "d2h_bytes_per_step": mm["d2h"]},
                    "gpu_launches": mm["launches"], "step_frac": step_frac,
                    "dram_frac": {kk: v.get("dram_frac") for kk, v in kinds.items() if kk in ("fwd", "bwd")},
                    "kernels": kinds, "roofline": roof}
            rr.free()
            del rr

    if rank == 0:
        line["clocks"] = sampler.stop()
        if extras:
            line["workloads"] = extras
        if not a.no_cpu_baseline and world == 1:
            # The reference's CUDA build is loaded BEFORE its CPU build: both extensions export the
            # same C symbols (MPLayers/TRWP/TRWP.h:23-25), and where the loader resolves them
            # process-wide the first one loaded serves both -- the CUDA build contains the CPU path
            # too, the CPU build has no device path.
            rc = reference_cuda(a.workload)
            if rc is not None:
                line["reference_cuda"] = rc
            line["cpu_baseline"] = cpu_baseline(a.workload, target_s=10.0)
            for name in extras:
                extras[name]["cpu_baseline"] = cpu_baseline(name, target_s=5.0)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------
# CPU arms (the oracle / the reference's own CPU code are test infrastructure; this is the one
# place outside tests where they are executed, as the measured baseline)
# ---------------------------------------------------------------------------------------------
_CFG_CACHE = {}


def _cpu_threads():
    """Threads of the C port, set explicitly so that a launcher's OMP_NUM_THREADS=1 does not decide it."""
    return max(1, min(os.cpu_count() or 1, 64))


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
    reference has no CPU backward (MPLayers/TRWP/TRWP.cpp:316).  Returns (units, seconds, used_ref);
    the seconds cover exactly the forward and backward passes (indices for the backward leg, when
    the reference's forward cannot provide them, are produced outside the timed spans)."""
    import numpy as np
    from oracle import oracle, ref_cpu
    nt = _cpu_threads()
    cfg, train, u, ctx, e = _cpu_sample(workload, edge)
    if cfg.get("soft"):  # the reference has no CPU implementation of the soft variant: C port
        t0 = time.perf_counter()
        fwd = oracle.forward_soft(u, ctx, e, cfg["n_dir"], cfg["n_iter"], training=train, n_threads=nt)
        g = np.random.default_rng(0).uniform(0, 1, size=u.shape).astype(np.float32)
        if train:
            oracle.backward_soft(ctx, e, g, fwd["edge_label"], fwd["norm_idx"], n_threads=nt)
        return u.shape[2] * u.shape[3] * u.shape[4] * cfg["n_iter"], time.perf_counter() - t0, False
    use_ref = use_reference and ref_cpu.available()
    fwd = None
    if use_ref:
        if train:  # indices for the backward leg come from the port; not part of the timed forward
            fwd = oracle.forward(cfg["mode"], u, ctx, e, cfg["n_dir"], cfg["n_iter"], training=True, n_threads=nt)
        t0 = time.perf_counter()
        ref_cpu.forward(cfg["mode"], u, ctx, cfg["n_dir"], cfg["n_iter"])
        t_f = time.perf_counter() - t0
    else:
        t0 = time.perf_counter()
        fwd = oracle.forward(cfg["mode"], u, ctx, e, cfg["n_dir"], cfg["n_iter"], training=train, n_threads=nt)
        t_f = time.perf_counter() - t0
    t_b = 0.0
    if train:
        g = np.random.default_rng(0).uniform(0, 1, size=u.shape).astype(np.float32)
        t1 = time.perf_counter()
        oracle.backward(cfg["mode"], ctx, e, g, fwd["min_idx"], fwd["norm_idx"], n_threads=nt)
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
    train = WORKLOADS[workload][2]
    nt = _cpu_threads()
    what = ("forward: the reference's ForwardCPU compiled from its sources (its fixed 16 OpenMP "
            "threads; edge weights ignored by that code)" if used_ref else "forward: C port, %d threads" % nt)
    if train:
        what += "; backward: C port (the reference has no CPU backward), %d threads" % nt
    return {"value": units / t, "unit": METRIC_UNIT, "cores": 16 if used_ref else nt,
            "port_threads": nt, "host_cpus": os.cpu_count(), "kind": "reference" if used_ref else "port",
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


def reference_cuda(workload):
    """Device time of one step of the reference's OWN CUDA kernels, recompiled unmodified for
    sm_100a (oracle/_ref/cuda, built by `python oracle/build.py --ref-cuda`), on the same inputs.
    Reported next to the CPU baseline when that build is present and the kernels can express the
    workload; None otherwise."""
    try:
        import torch
        from oracle import ref_cuda
        cfg = _cpu_sample(workload, 32)[0]   # the generated configuration (cached)
        if cfg.get("soft") or not ref_cuda.available(cfg["mode"]):
            return None
        u = cfg["unary"].permute(0, 1, 3, 4, 2).contiguous().cuda()
        b, cv, h, w, l = u.shape
        ctx = cfg["label_context"].cuda()
        if not ref_cuda.expressible(l, ctx.dim(), cfg["n_iter"], cfg["n_dir"], b * cv * h * w):
            return None
        e = cfg["edge_weights"]
        e = e.unsqueeze(1).permute(2, 0, 1, 3, 4).contiguous().cuda() if e is not None else None
        rho = 0.5 if cfg["mode"] == "TRWP" else 1.0
        train = WORKLOADS[workload][2]
        g = torch.rand(u.shape, device="cuda")

        def step():
            f = ref_cuda.forward(cfg["mode"], u, ctx, e, cfg["n_dir"], cfg["n_iter"], rho, training=train)
            if train:
                ref_cuda.backward(cfg["mode"], ctx, f["edge_weights"], g, f["min_idx"], f["norm_idx"], rho)

        step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 3
        return {"ms_per_step": round(ms, 3), "value": b * h * w * l * cfg["n_iter"] / (ms * 1e-3),
                "unit": METRIC_UNIT, "what": "the reference's CUDA extension recompiled for sm_100a, "
                "extension-level forward%s call on device-resident tensors" % (" + backward" if train else "")}
    except Exception as exc:  # a baseline must never take the bench line down
        return {"unavailable": str(exc)[:200]}


def run_reference(a):
    """The reference's CPU implementation of the same workload and config on this host's cores.
    Under a multi-process launcher rank 0 alone runs it (one host, however many GPUs the other arm
    uses); the thread count is set explicitly, so the value does not depend on the launcher."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", str(a.gpus)))
    budget = 150.0 / max(a.steps + max(a.warmup, 1), 1)   # the whole run stays within a few minutes
    edge = _pick_edge(a.workload, min(budget, 8.0))
    for _ in range(max(a.warmup, 1)):
        _time_cpu(a.workload, edge)
    res = []
    for _ in range(a.steps):
        res.append(_time_cpu(a.workload, edge))
    res.sort(key=lambda r: r[1])
    units, t, used_ref = res[len(res) // 2]
    cb = _describe(a.workload, edge, used_ref, units, t)
    cfg = _CFG_CACHE[a.workload]
    train = WORKLOADS[a.workload][2]
    batch = cfg["unary"].shape[0]
    _, _, L, H, W = cfg["unary"].shape
    line = {"impl": "reference",
            "metric": "TRWP/ISGMR fwd+bwd pixel*label*iter/s" if train else "TRWP/ISGMR fwd pixel*label*iter/s",
            "value": cb["value"], "unit": METRIC_UNIT, "n_gpus": a.gpus, "steps": a.steps,
            "warmup": max(a.warmup, 1), "ms_per_step": t * 1e3, "higher_is_better": True,
            "scaling": "strong" if a.shard == "directions" else "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": config_dict(a.workload, (L, H, W), cfg["mode"], cfg["n_dir"], cfg["n_iter"], train, a.shard,
                                  batch, world),
            "cpu_hosts": 1, "note": "one host's CPU cores time a bounded sample of the workload (ms_per_step is "
                                    "the median sample time); the value does not grow with n_gpus",
            "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": METRIC_UNIT, "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


if __name__ == "__main__":
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
