#!/usr/bin/env python
"""Benchmark of the cost-volume separation hot path: cells/s of forward + backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config 1..5] [--impl ours|reference|reference-cuda]

One "step" is one pass of the four ops over one batch of synthetic feature maps:
max/argmax/avg forward, compression forward, compression backward, max/avg backward (forward-only
configs run the first two).  A "cell" is one entry of the virtual volume S (B*H1*W1*H2*W2 per step).
Default workload: BASELINE config 5 (B=8, 135x240, C=256, Kc=4, fwd+bwd), the configuration the
throughput target is quoted on; it fits one GPU.  With N > 1 ranks (torchrun) the same job is split
by batch, then by image-1 rows (strong scaling); rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# (B, H, W, Kc, backward) of BASELINE.json's configs; C = 256 everywhere
CONFIGS = {
    1: dict(B=1, H=48, W=64, Kc=0, bwd=False, name="config1: B=1 48x64 C=256 fwd max/avg only"),
    2: dict(B=2, H=48, W=64, Kc=2, bwd=True, name="config2: B=2 48x64 C=256 Kc=2 fwd+bwd"),
    3: dict(B=4, H=55, W=128, Kc=4, bwd=False, name="config3: B=4 55x128 C=256 Kc=4 fwd"),
    4: dict(B=8, H=47, W=156, Kc=2, bwd=True, name="config4: B=8 47x156 C=256 Kc=2 fwd+bwd (fp32 operands)"),
    5: dict(B=8, H=135, W=240, Kc=4, bwd=True, name="config5: B=8 135x240 C=256 Kc=4 fwd+bwd"),
}
C_FEAT = 256
SEED = 1234  # the reference's default seed (train.py:52)

# DRAM bytes per cell (dram__bytes_read.sum + dram__bytes_write.sum of one launch / cells of that launch)
# from the ncu captures summarised under profiles/ (one table per operand width); traffic grows in proportion to
# the cells swept.
DRAM_BYTES_PER_CELL = {}
try:
    with open(os.path.join(ROOT, "profiles", "dram_bytes_per_cell.json")) as _f:
        DRAM_BYTES_PER_CELL = json.load(_f)
except OSError:
    pass


def flops_per_cell(cfg) -> int:
    """Algorithmic tensor work: 2*C per necessary contraction; forward 1 (no attention) or 2,
    backward 3 (S recompute for the attention gradients, gF1, gF2)."""
    n = 1 if cfg["Kc"] == 0 else 2
    if cfg["bwd"]:
        n += 3
    return n * 2 * C_FEAT


# --------------------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples the SM clock and the clock-event reasons of one GPU while a timed region runs.

    Reads NVML from a thread of this process every 10 ms (a timed region of a few tens of milliseconds still
    gets samples); when NVML cannot be loaded it falls back to an `nvidia-smi -lms 200` child process.
    Nothing is set: both only read."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, gpu_index: int):
        self.sm, self.smax, self.reasons = [], [], set()
        self.proc = self.out = self.thread = None
        self.source = None
        self._stop = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            handle = self._handle(pynvml, gpu_index)
            self.smax.append(float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM)))
            masks = ((pynvml.nvmlClocksEventReasonHwSlowdown, "hw_slowdown"),
                     (pynvml.nvmlClocksEventReasonHwThermalSlowdown, "hw_thermal_slowdown"),
                     (pynvml.nvmlClocksEventReasonSwThermalSlowdown, "sw_thermal_slowdown"),
                     (pynvml.nvmlClocksEventReasonSwPowerCap, "sw_power_cap"))

            def loop():
                while not self._stop.is_set():
                    try:
                        self.sm.append(float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)))
                        bits = pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle)
                        for mask, name in masks:
                            if bits & mask:
                                self.reasons.add(name)
                    except pynvml.NVMLError:
                        pass
                    self._stop.wait(0.010)

            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
            self.source = "nvml"
            return
        except Exception:
            self.thread = None
        try:
            self.out = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(gpu_index)], stdout=self.out, stderr=subprocess.DEVNULL)
            self.source = "nvidia-smi"
        except OSError:
            self.proc = None

    @staticmethod
    def _handle(pynvml, gpu_index):
        """NVML handle of CUDA device `gpu_index`, matched by PCI address so that a CUDA_VISIBLE_DEVICES
        remapping cannot pick another GPU's clocks."""
        try:
            p = torch.cuda.get_device_properties(gpu_index)
            bus = f"{p.pci_domain_id:08x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
            return pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
        except Exception:
            return pynvml.nvmlDeviceGetHandleByIndex(gpu_index)

    def stop(self):
        if self.thread is not None:
            self._stop.set()
            self.thread.join(2)
        elif self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.out.flush()
            self.out.seek(0)
            for line in self.out.read().splitlines():
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 7:
                    continue
                try:
                    self.sm.append(float(parts[0]))
                    self.smax.append(float(parts[1]))
                except ValueError:
                    continue
                for n, v in zip(self.NAMES, parts[3:7]):
                    if v.lower().startswith("active"):
                        self.reasons.add(n)
            self.out.close()
            os.unlink(self.out.name)
        else:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        return {"sm_mhz": statistics.median(self.sm) if self.sm else None,
                "sm_max_mhz": max(self.smax) if self.smax else None,
                "samples": len(self.sm), "source": self.source, "reasons": sorted(self.reasons)}


# --------------------------------------------------------------------------------------- workload
def attention_parameters(Kc, device=None):
    """Seeded N(0, 0.02) parameters of the two Conv3d(2, Kc, 3, padding=1) attention modules:
    [weight_u, bias_u, weight_v, bias_v]."""
    g = torch.Generator().manual_seed(SEED + 99)
    out = []
    for _ in range(2):
        out.append(torch.randn(Kc, 2, 3, 3, 3, generator=g) * 0.02)
        out.append(torch.randn(Kc, generator=g) * 0.02)
    return [t.to(device) for t in out] if device is not None else out


def make_job(cfg, shard, device, path="ops"):
    """Seeded N(0,1) features of this rank's shard (drawn for the whole job, then sliced, so every
    world size sees the same data) and N(0,1) upstream gradients; for the five reference ops also softmaxed
    random attention weights, for the level calls the attention parameters."""
    B, H, W, Kc = cfg["B"], cfg["H"], cfg["W"], cfg["Kc"]
    g = torch.Generator().manual_seed(SEED)
    f1 = torch.randn(B, C_FEAT, H, W, generator=g)
    f2 = torch.randn(B, C_FEAT, H, W, generator=g)
    from separableflowthesis_b200 import sharding as _sh
    e0, e1, _, _ = _sh.halo_range(shard, H)     # row shards: plus one halo row per side for the attention stencil
    f1_ext = f1[shard.b0:shard.b1, :, e0:e1].contiguous()
    f1 = f1[shard.b0:shard.b1, :, shard.r0:shard.r1].contiguous()
    f2 = f2[shard.b0:shard.b1].contiguous()
    job = {"f1_nchw": f1_ext, "f2_nchw": f2}
    if path == "level":
        f1 = f1_ext      # the level calls of a row shard run on the block plus its halo rows
    F1 = (f1.permute(0, 2, 3, 1).contiguous() / C_FEAT ** 0.5).to(device)
    F2 = f2.permute(0, 2, 3, 1).contiguous().to(device)
    b, h = F1.shape[0], F1.shape[1]
    gd = torch.Generator(device=device).manual_seed(SEED + 1 + shard.rank)
    job.update(F1=F1, F2=F2)
    job["cells"] = b * (shard.r1 - shard.r0) * W * H * W
    if path == "level":
        job["att"] = attention_parameters(Kc, device)
        if cfg["bwd"]:
            # drawn per sample for all image-1 rows, then sliced: every partition of the job sees the same gradients
            job["gSEP_u"] = torch.empty(b, 2 + Kc, W, h, W, device=device)
            job["gSEP_v"] = torch.empty(b, 2 + Kc, H, h, W, device=device)
            for i, bi in enumerate(range(shard.b0, shard.b1)):
                gs = torch.Generator(device=device).manual_seed(SEED + 1000 + bi)
                job["gSEP_u"][i] = torch.randn(2 + Kc, W, H, W, generator=gs, device=device)[:, :, e0:e1]
                job["gSEP_v"][i] = torch.randn(2 + Kc, H, H, W, generator=gs, device=device)[:, :, e0:e1]
            if shard.g_rows > 1:   # the outputs of halo rows are not used: no upstream gradient there
                _, _, i0, i1 = _sh.halo_range(shard, H)
                for t in (job["gSEP_u"], job["gSEP_v"]):
                    t[:, :, :, :i0] = 0
                    t[:, :, :, i1:] = 0
        job["shard"] = shard
        return job
    if Kc > 0:
        job["A_u"] = torch.randn(b, h, W, Kc, W, generator=gd, device=device).softmax(-1)
        job["A_v"] = torch.randn(b, h, W, Kc, H, generator=gd, device=device).softmax(-1)
    if cfg["bwd"]:
        job["gMA_u"] = torch.randn(b, h, W, 2, H, generator=gd, device=device)
        job["gMA_v"] = torch.randn(b, h, W, 2, W, generator=gd, device=device)
        if Kc > 0:
            job["gC_u"] = torch.randn(b, h, W, Kc, H, generator=gd, device=device)
            job["gC_v"] = torch.randn(b, h, W, Kc, W, generator=gd, device=device)
    return job


def run_level(ms, cfg, job, row_group=None):
    """The hot path on device-resident inputs as the call site runs it: one library call for the level's
    forward (max/avg sweep, attention weights, compression sweep) and one for its backward.  Row shards then sum
    gF2 over their group and hand the halo rows of gF1 to their neighbours."""
    F1, F2 = job["F1"], job["F2"]
    wu, bu, wv, bv = job["att"]
    out = ms.separation_level_forward(F1, F2, wu, bu, wv, bv, with_argmax=cfg["bwd"])
    if cfg["bwd"]:
        sep_u, sep_v, am_u, am_v, a_u, a_v = out
        grads = ms.separation_level_backward(F1, F2, wu, wv, sep_u, sep_v, am_u, am_v, a_u, a_v, job["gSEP_u"],
                                              job["gSEP_v"])
        shard = job["shard"]
        if shard.g_rows > 1:
            from separableflowthesis_b200 import sharding
            grads[0] = sharding.exchange_halo_grads(grads[0], shard, cfg["H"], row_group, dim=1)
            if grads[1].shape[0] % shard.g_rows == 0:   # each rank keeps the gradient of its slice of the samples
                grads[1] = sharding.reduce_scatter_batch(grads[1], row_group)
            else:
                grads[1] = sharding.reduce_row_partial(grads[1], row_group)
        out = out + grads
    return out


def run_ops(ms, cfg, job, fused=True, row_group=None):
    """The hot path on device-resident inputs through the five ops of the reference's module (random softmaxed
    attention weights stand in for the Conv3d modules the call site runs between them).  With `fused` the two
    backward ops run as the library's one-call backward (same outputs; feature gradients arrive summed)."""
    if "att" in job:
        return run_level(ms, cfg, job, row_group)
    F1, F2 = job["F1"], job["F2"]
    if cfg["bwd"]:
        MA_u, MA_v, AM_u, AM_v = ms.max_argmax_avg_forward(F1, F2)
    else:
        MA_u, MA_v = ms.max_avg_forward(F1, F2)
    out = [MA_u, MA_v]
    if cfg["Kc"] > 0:
        out += ms.compression_forward(F1, F2, job["A_u"], job["A_v"])
    if cfg["bwd"]:
        if cfg["Kc"] > 0 and fused:
            out += ms.separation_backward(F1, F2, AM_u, AM_v, job["gMA_u"], job["gMA_v"], job["A_u"], job["A_v"],
                                          job["gC_u"], job["gC_v"])
            return out
        if cfg["Kc"] > 0:
            out += ms.compression_backward(F1, F2, job["A_u"], job["A_v"], job["gC_u"], job["gC_v"])
        out += ms.max_argmax_avg_backward(F1, F2, AM_u, AM_v, job["gMA_u"], job["gMA_v"])
    return out


def launches_per_step(cfg, path="ops") -> int:
    """Kernels of this library launched by one step, from the op list (used only when the library's own count
    from the timing pass is not available)."""
    sweeps = (cfg["Kc"] + 3) // 4
    if path == "level":
        # forward: prepare 3, max/avg sweep, 2 attention modules x chunks, compression sweeps
        n = 3 + 1 + 2 * sweeps + sweeps
        if cfg["bwd"]:
            # prepare 2, attention-gradient sweeps, 2 x (logit chunks + input-grad chunks + weight grad + 2 reductions),
            # 4 interleave packs, 2 gradient GEMMs (+ 2 packs and 2 GEMMs per further chunk of 4 channels)
            n += 2 + sweeps + 2 * (2 * sweeps + 3) + 4 + 2 + 4 * (sweeps - 1)
        return n
    n = 3 + 1 + 2                               # max/avg forward: prepare(3) + sweep + unpack(2)
    if cfg["bwd"]:
        n += 2                                  # argmax unpack
    if cfg["Kc"] > 0:
        n += 2 + 2 + sweeps + 2                 # compression forward: prepare, pack, sweep(s), unpack
    if cfg["bwd"]:
        if cfg["Kc"] > 0:
            n += 2 + 2 + sweeps + 2 + 4 + 2     # one-call backward: prepare, pack, sweeps, unpack, interleave, 2 GEMMs
        else:
            n += 2 + 2 + 2                      # max/avg backward: prepare, interleave, 2 GEMMs
    return n


def run_lookup_bench(args, cfg, device, emit):
    """`--path lookup`: one refinement iteration of the reference's CorrBlock1D (core/corr.py:576-624) = the lookup of
    both aggregated volumes (dim 1, 4 levels, radius 4) at every image-1 pixel, forward and (training configs)
    backward, on device-resident volumes of the config's size.  HBM-bound: reported against the measured copy
    bandwidth."""
    import separableflowthesis_b200 as sfb
    from separableflowthesis_b200 import _lib
    B, H, W = cfg["B"], cfg["H"], cfg["W"]
    levels, radius, dim = 4, 4, 1
    gd = torch.Generator(device=device).manual_seed(SEED + 11)
    corr1 = torch.randn(B, dim, W, H, W, generator=gd, device=device, requires_grad=cfg["bwd"])
    corr2 = torch.randn(B, dim, H, H, W, generator=gd, device=device, requires_grad=cfg["bwd"])
    ys, xs = torch.meshgrid(torch.arange(H, device=device), torch.arange(W, device=device), indexing="ij")
    # a smooth displacement field (two low-frequency waves, amplitude ~8 pixels) plus sub-pixel noise, standing in
    # for the flow estimates of a refinement iteration, which are piecewise smooth
    yy, xx = ys.float() / H, xs.float() / W
    flow = torch.stack((8.0 * torch.sin(6.28 * (xx + 0.5 * yy)), 6.0 * torch.cos(6.28 * (yy - 0.3 * xx))))
    coords = (torch.stack((xs, ys)).float() + flow)[None].repeat(B, 1, 1, 1)
    coords = coords + 0.25 * torch.randn(B, 2, H, W, generator=gd, device=device)
    blk = sfb.CorrBlock1D(corr1, corr2, num_levels=levels, radius=radius)
    taps = 2 * radius + 1
    gout = torch.randn(B, levels * dim * taps, H, W, generator=gd, device=device)

    def step():
        o1, o2 = blk(coords)
        if cfg["bwd"]:
            corr1.grad = corr2.grad = None
            torch.autograd.backward([o1, o2], [gout, gout])

    for _ in range(max(args.warmup, 3)):
        step()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)   # > L2: the volumes alone may fit
    e0 = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    e1 = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    sampler = ClockSampler(device.index or 0)
    torch.cuda.synchronize()
    for i in range(args.steps):
        flush.zero_()
        e0[i].record()
        step()
        e1[i].record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = sum(a.elapsed_time(b) for a, b in zip(e0, e1)) / args.steps
    samples = 2.0 * B * H * W * levels * dim * taps
    # algorithmic bytes of one iteration: every output written once; per pixel, level and channel the 2r+2 volume
    # rows its taps touch; backward reads the output gradients and writes the volume gradients once
    out_bytes = samples * 4
    touched = 2.0 * B * H * W * levels * dim * (taps + 1) * 4
    vol = 4.0 * B * dim * H * W * (H + W)
    bytes_fwd = out_bytes + touched
    bytes_bwd = (out_bytes + vol) if cfg["bwd"] else 0.0
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    achieved = (bytes_fwd + bytes_bwd) / (ms * 1e-3) / 1e9
    emit({"metric": "3D cost-volume lookups/sec" + (" (fwd+bwd)" if cfg["bwd"] else " (fwd)"),
          "value": samples / (ms * 1e-3), "unit": "samples/s", "n_gpus": 1, "steps": args.steps,
          "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
          "vs_baseline": None, "dtype": "f32", "data": "synthetic",
          "config": {"workload": cfg["name"] + ": CorrBlock1D lookup, dim 1, 4 levels, radius 4, both volumes",
                     "path": "lookup", "l2": "L2 flushed between iterations"},
          "clocks": clocks, "gpu_launches": (2 + (2 if cfg["bwd"] else 0)) * args.steps,
          "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                       "traffic": None, "peak_source": "MEASURED_PEAKS.json hbm_gbs" if peaks else "fallback 6650"}})


def run_lookup4d_bench(args, cfg, device, emit):
    """`--path lookup4d`: one refinement iteration of the 4D lookup without the stored volume (the branch
    core/corr.py:491-510 leaves unimplemented; result of core/corr.py:192-247): 4 levels, radius 4, at every image-1
    pixel, forward and (training configs) backward, on the config's feature maps.  The stored volume would be
    B*N^2*4/3 floats (45 GB at config 5); here each value is recomputed from the feature rows."""
    import separableflowthesis_b200 as sfb
    B, H, W = cfg["B"], cfg["H"], cfg["W"]
    levels, radius = 4, 4
    gd = torch.Generator(device=device).manual_seed(SEED + 12)
    f1 = torch.randn(B, C_FEAT, H, W, generator=gd, device=device, requires_grad=cfg["bwd"])
    f2 = torch.randn(B, C_FEAT, H, W, generator=gd, device=device, requires_grad=cfg["bwd"])
    ys, xs = torch.meshgrid(torch.arange(H, device=device), torch.arange(W, device=device), indexing="ij")
    yy, xx = ys.float() / H, xs.float() / W
    # piecewise-smooth stand-in for a flow estimate: two low-frequency waves plus sub-pixel noise
    flow = torch.stack((8.0 * torch.sin(6.28 * (xx + 0.5 * yy)), 6.0 * torch.cos(6.28 * (yy - 0.3 * xx))))
    coords = (torch.stack((xs, ys)).float() + flow)[None].repeat(B, 1, 1, 1)
    coords = coords + 0.25 * torch.randn(B, 2, H, W, generator=gd, device=device)
    win = (2 * radius + 1) ** 2
    gout = torch.randn(B, levels * win, H, W, generator=gd, device=device)
    blk = sfb.AlternateCorrBlockSepflow(f1, f2, None, num_levels=levels, radius=radius, support_backward=cfg["bwd"])
    blk(coords)   # channels-last copies of the feature pyramid: once per pair of images, not per iteration

    def step():
        out = blk(coords)
        if cfg["bwd"]:
            f1.grad = f2.grad = None
            # the graph of the block's pooled, channels-last copies is shared by all iterations (in the model one
            # backward runs through all of them), so it must survive this iteration's backward
            out.backward(gout, retain_graph=True)

    for _ in range(max(args.warmup, 3)):
        step()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    e0 = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    e1 = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    sampler = ClockSampler(device.index or 0)
    torch.cuda.synchronize()
    for i in range(args.steps):
        flush.zero_()
        e0[i].record()
        step()
        e1[i].record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = sum(a.elapsed_time(b) for a, b in zip(e0, e1)) / args.steps
    samples = float(B) * H * W * levels * win
    # algorithmic HBM bytes of one iteration: features read once, outputs written once (backward: output gradients
    # read, feature gradients written); the gathers of image-2 rows are served by L1/L2
    feats = 4.0 * B * C_FEAT * H * W * (1 + sum(1.0 / 4 ** l for l in range(levels)))
    nbytes = (feats + samples * 4) * (2 if cfg["bwd"] else 1)
    flops = float(B) * H * W * levels * (2 * radius + 2) ** 2 * 2 * C_FEAT * (3 if cfg["bwd"] else 1)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    achieved = nbytes / (ms * 1e-3) / 1e9
    emit({"metric": "4D cost-volume lookups/sec without the stored volume" + (" (fwd+bwd)" if cfg["bwd"] else " (fwd)"),
          "value": samples / (ms * 1e-3), "unit": "samples/s", "n_gpus": 1, "steps": args.steps,
          "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
          "vs_baseline": None, "dtype": "f32", "data": "synthetic",
          "config": {"workload": cfg["name"] + ": 4D lookup, 4 levels, radius 4, C=256", "path": "lookup4d",
                     "l2": "L2 flushed between iterations", "fp32_tflops": flops / (ms * 1e-3) / 1e12},
          "clocks": clocks, "gpu_launches": (1 + (1 if cfg["bwd"] else 0)) * args.steps,
          "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                       "traffic": None, "peak_source": "MEASURED_PEAKS.json hbm_gbs" if peaks else "fallback 6650",
                       "note": "gather of image-2 feature rows through L1/L2; HBM traffic is not the limiter"}})


def run_reference_cuda(args, cfg, metric, unit, emit):
    """`--impl reference-cuda`: the five ops of the reference's own CUDA extension (oracle/_ref/MemorySaver.so, built
    unmodified from libs/MemorySaver/src) on one GPU, and this library's five ops on the same tensors, in the
    reference's layouts with random softmaxed attention weights (the op sequence the metric is defined on).  One
    line per implementation.  The reference needs seconds per step, so it runs `steps` capped at 3."""
    import importlib.util
    so = os.path.join(ROOT, "oracle", "_ref", "MemorySaver.so")
    if not os.path.exists(so):
        emit({"impl": "reference-cuda", "unavailable": "oracle/_ref/MemorySaver.so not built (oracle/build_ref_cuda.py)"})
        return
    if cfg["Kc"] != 2:
        emit({"impl": "reference-cuda",
              "unavailable": "the reference's forward kernel computes two attention channels only: use --config 2 or 4"})
        return
    from separableflowthesis_b200 import ops
    spec = importlib.util.spec_from_file_location("MemorySaver", so)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    device = torch.device("cuda", 0)
    B, H, W, Kc = cfg["B"], cfg["H"], cfg["W"], cfg["Kc"]
    g = torch.Generator().manual_seed(SEED)
    F1 = (torch.randn(B, H, W, C_FEAT, generator=g) / C_FEAT ** 0.5).to(device)
    F2 = torch.randn(B, H, W, C_FEAT, generator=g).to(device)
    A_u = torch.randn(B, H, W, Kc, W, generator=g).softmax(-1).to(device)
    A_v = torch.randn(B, H, W, Kc, H, generator=g).softmax(-1).to(device)
    gMu, gMv = torch.randn(B, H, W, 2, H, generator=g).to(device), torch.randn(B, H, W, 2, W, generator=g).to(device)
    gCu, gCv = torch.randn(B, H, W, Kc, H, generator=g).to(device), torch.randn(B, H, W, Kc, W, generator=g).to(device)
    cells = float(B) * (H * W) ** 2

    def step(mod):
        _, _, au, av = mod.max_argmax_avg_forward(F1, F2)
        mod.compression_forward(F1, F2, A_u, A_v)
        if cfg["bwd"]:
            mod.compression_backward(F1, F2, A_u, A_v, gCu, gCv)
            mod.max_argmax_avg_backward(F1, F2, au, av, gMu, gMv)

    for name, mod, steps, warm in (("reference-cuda", ref, min(args.steps, 3), 1), ("ours", ops, args.steps, max(args.warmup, 3))):
        for _ in range(warm):
            step(mod)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step(mod)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        emit({"impl": name, "metric": metric, "value": cells / (ms * 1e-3), "unit": unit, "n_gpus": 1, "steps": steps,
              "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
              "dtype": "f32" if name != "ours" else DTYPE_TEXT["fp16"], "data": "synthetic",
              "config": {"workload": cfg["name"], "path": "the five ops in the reference's layouts, device-resident"}})


class E2E:
    """The call a user of the reference makes: channels-first feature maps in host memory ->
    AlternateCorrBlockSepflow.separate (one level, Conv3d attention) -> backward with upstream
    gradients -> loss-sized results back on the host."""

    def __init__(self, cfg, job, device, chunks=1, levels=1, shard=None, row_group=None, prefetch=False,
                 f2_from_rank0=False):
        import separableflowthesis_b200 as sfb
        self.sfb, self.cfg, self.device = sfb, cfg, device
        self.prefetch, self.prefetched = prefetch, None
        self.chunks = chunks if shard is None or shard.g_rows == 1 else 1
        self.levels = levels
        self.shard, self.row_group = shard, row_group
        self.copy_stream = torch.cuda.Stream(device=device)
        self.h1 = job["f1_nchw"].pin_memory()
        # Row shards of one sample all need the whole of image 2.  `f2_from_rank0` (the name of the first variant; now
        # every rank holds a slice): each rank of the row group copies 1/G of the samples' image-2 features from the
        # host and an all-gather over NVLink completes them on every GPU, instead of G host copies of all of them.
        f2 = job["f2_nchw"]
        self.gather_f2 = bool(f2_from_rank0 and shard is not None and shard.g_rows > 1 and f2.shape[0] % shard.g_rows == 0)
        if self.gather_f2:
            per = f2.shape[0] // shard.g_rows
            ri = shard.rank % shard.g_rows
            f2 = f2[ri * per:(ri + 1) * per].contiguous()
        self.h2 = f2.pin_memory()
        self.att = None
        if cfg["Kc"] > 0:
            params = attention_parameters(cfg["Kc"])
            self.att = []
            for i in range(2):
                conv = torch.nn.Conv3d(2, cfg["Kc"], 3, padding=1)
                with torch.no_grad():
                    conv.weight.copy_(params[2 * i])
                    conv.bias.copy_(params[2 * i + 1])
                self.att.append(conv.to(device))
        self.up = None
        # two pinned result buffers: a step's result is read on the host while the next step is already queued
        self.host_out = [torch.empty(1024, dtype=torch.float32).pin_memory() for _ in range(2)]
        self.pending, self.last_value, self.nstep = None, None, 0
        self.h2d = self.h1.numel() * 4 + self.h2.numel() * 4
        self.d2h = 0

    def step(self):
        """One step: this step's features host -> device, separation forward + backward, results -> host.  The batch
        is processed as `self.chunks` micro-batches through the same public call; the copy of micro-batch i+1 runs on
        a second stream while micro-batch i computes (gradients of the shared attention parameters accumulate
        across micro-batches as autograd does for any repeated use).  With `prefetch` the copy of the NEXT step's
        first micro-batch is issued while this step's last one computes, as an input pipeline does; every step still
        copies all of its inputs from pinned host memory inside the timed region (the step after the last timed one
        gets its first micro-batch copied there too, unused).  The step's result travels to pinned host memory with an
        asynchronous copy and is read on the host once the NEXT step has been queued (drain() reads the last one), as a
        training loop that logs its loss one step late does: the GPU never waits for the host between steps."""
        cfg, dev = self.cfg, self.device
        n = self.h1.shape[0]
        chunks = max(1, min(self.chunks, n))
        bounds = [(i * n // chunks, (i + 1) * n // chunks) for i in range(chunks)]
        main = torch.cuda.current_stream()
        def stage(b0, b1):
            with torch.cuda.stream(self.copy_stream):
                f1 = self.h1[b0:b1].to(dev, non_blocking=True)
                if self.gather_f2:   # one micro-batch in this mode: this rank's slice, then the others' over NVLink
                    from separableflowthesis_b200 import sharding
                    f2 = sharding.allgather_batch(self.h2.to(dev, non_blocking=True), self.row_group)
                else:
                    f2 = self.h2[b0:b1].to(dev, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.copy_stream)
            return f1, f2, ev

        staged = []
        for i, (b0, b1) in enumerate(bounds):
            if i == 0 and self.prefetched is not None:
                staged.append(self.prefetched)
                self.prefetched = None
            else:
                staged.append(stage(b0, b1))
        params = [p for c in (self.att or []) for p in c.parameters()]
        for p in params:
            p.grad = None
        pieces, keep = [], []
        for (b0, b1), (f1, f2, ev) in zip(bounds, staged):
            main.wait_event(ev)
            f1.record_stream(main)   # allocated on the copy stream, used (and later freed) under the main stream
            f2.record_stream(main)
            if cfg["bwd"]:
                f1.requires_grad_(True)
                f2.requires_grad_(True)
            blk = self.sfb.AlternateCorrBlockSepflow(f1, f2, None, num_levels=self.levels, support_backward=cfg["bwd"])
            with torch.set_grad_enabled(cfg["bwd"]):
                sep_u, sep_v = blk(None, sep=True, attention_weights=tuple(self.att) if self.att else None)
            sharded_rows = self.shard is not None and self.shard.g_rows > 1
            if sharded_rows:   # computed on the block plus halo rows: keep this rank's own image-1 rows
                from separableflowthesis_b200 import sharding
                sep_u = sharding.interior(sep_u, self.shard, cfg["H"], 3)
                sep_v = sharding.interior(sep_v, self.shard, cfg["H"], 3)
            if cfg["bwd"]:
                if self.up is None:
                    gd = torch.Generator(device=dev).manual_seed(SEED + 7)
                    shape_u = (n,) + tuple(sep_u.shape[1:])
                    shape_v = (n,) + tuple(sep_v.shape[1:])
                    self.up = (torch.randn(shape_u, generator=gd, device=dev),
                               torch.randn(shape_v, generator=gd, device=dev))
                torch.autograd.backward([sep_u, sep_v], [self.up[0][b0:b1], self.up[1][b0:b1]])
                g1, g2 = f1.grad, f2.grad
                if sharded_rows:   # halo rows of gF1 go to the neighbouring shards, gF2 is summed over the row group
                    g1 = sharding.exchange_halo_grads(g1, self.shard, cfg["H"], self.row_group, dim=2)
                    g2 = (sharding.reduce_scatter_batch(g2, self.row_group) if self.gather_f2
                          else sharding.reduce_row_partial(g2, self.row_group))
                pieces += [g1.sum().reshape(1), g2.sum().reshape(1)]
            else:
                pieces += [sep_u.sum().reshape(1), sep_v.sum().reshape(1)]
            keep.append((f1, f2))
        if cfg["bwd"]:
            from separableflowthesis_b200 import sharding
            flat = sharding.reduce_parameter_grads(params)  # NCCL all-reduce when world_size > 1
            if flat is not None:
                pieces.append(flat[:1000])
        res = torch.cat(pieces)
        k = self.nstep & 1
        self.nstep += 1
        self.host_out[k][:res.numel()].copy_(res, non_blocking=True)
        done = torch.cuda.Event()
        done.record(main)
        self.d2h = res.numel() * 4
        if self.prefetch:
            self.prefetched = stage(*bounds[0])
        self.drain()                    # the PREVIOUS step's result (this step is queued behind it)
        self.pending = (done, k)
        return self.last_value

    def drain(self):
        """Waits for the result of the last step whose result has not been read yet and reads it."""
        if self.pending is not None:
            ev, k = self.pending
            ev.synchronize()
            self.last_value = float(self.host_out[k][0])
            self.pending = None
        return self.last_value


# --------------------------------------------------------------------------------------- CPU baseline
def cpu_sample(cfg, rows, threads):
    """One bounded sample of the workload through the oracle on the host cores: `rows` image-1 rows of
    one sample against the whole of image 2 (identical math, work is linear in image-1 rows)."""
    from oracle import separation_oracle as orc
    torch.set_num_threads(threads)
    H, W, Kc = cfg["H"], cfg["W"], cfg["Kc"]
    g = torch.Generator().manual_seed(SEED)
    F1 = torch.randn(1, rows, W, C_FEAT, generator=g) / C_FEAT ** 0.5
    F2 = torch.randn(1, H, W, C_FEAT, generator=g)
    A_u = torch.randn(1, rows, W, max(Kc, 1), W, generator=g).softmax(-1)
    A_v = torch.randn(1, rows, W, max(Kc, 1), H, generator=g).softmax(-1)
    gMA_u = torch.randn(1, rows, W, 2, H, generator=g)
    gMA_v = torch.randn(1, rows, W, 2, W, generator=g)
    gC_u = torch.randn(1, rows, W, max(Kc, 1), H, generator=g)
    gC_v = torch.randn(1, rows, W, max(Kc, 1), W, generator=g)

    att = attention_parameters(Kc) if Kc > 0 else None
    gS_u = torch.randn(1, 2 + Kc, W, rows, W, generator=g)
    gS_v = torch.randn(1, 2 + Kc, H, rows, W, generator=g)

    def run():
        if Kc > 0:   # the level as the reference's dense path chains it: ops + Conv3d attention + softmax
            fw = orc.separation_level_forward(F1, F2, *att)
            if cfg["bwd"]:
                orc.separation_level_backward(F1, F2, att[0], att[2], *fw, gS_u, gS_v)
            return
        fw = orc.max_argmax_avg_forward(F1, F2)
        if cfg["bwd"]:
            orc.max_argmax_avg_backward(F1, F2, fw[2], fw[3], gMA_u, gMA_v)
    return run, rows * W * H * W


def time_cpu(cfg, budget_s, steps=None, warmup=1):
    threads = os.cpu_count() or 1
    rows = 1
    run, cells = cpu_sample(cfg, rows, threads)
    t0 = time.perf_counter()
    run()
    t1 = time.perf_counter() - t0
    n_steps = steps if steps is not None else 3
    # grow the sample so that the whole measurement takes about budget_s
    rows = int(max(1, min(cfg["H"], budget_s / max(t1, 1e-3) / (n_steps + warmup))))
    run, cells = cpu_sample(cfg, rows, threads)
    for _ in range(warmup):
        run()
    t0 = time.perf_counter()
    for _ in range(n_steps):
        run()
    dt = (time.perf_counter() - t0) / n_steps
    return dict(value=cells / dt, unit="cells/s", cores=threads, kind="port",
                sample=f"{rows} of {cfg['H']} image-1 rows of one sample ({cells} cells) per step, {n_steps} steps, "
                       f"oracle (dense torch CPU fp32 matmul/einsum + max/mean + conv3d/softmax attention), "
                       f"{threads} threads"), dt, n_steps


# --------------------------------------------------------------------------------------- main
def resolve_path(args, cfg):
    if args.path == "auto":
        return "level" if cfg["Kc"] > 0 and not args.unfused else "ops"
    return args.path


def workload_config(args, cfg, world):
    """The `config` object of the JSON line.  Both arms print the same one for the same flags: it names the workload and
    how `--gpus N` partitions it, not which implementation ran (what a CPU arm actually timed is in its
    `cpu_baseline.sample`)."""
    import math
    g_batch = math.gcd(cfg["B"], world) if args.shard == "batch" else 1
    cells = float(cfg["B"]) * (cfg["H"] * cfg["W"]) ** 2
    return {"workload": cfg["name"], "path": resolve_path(args, cfg), "cells_per_step": cells,
            "flop_per_cell": flops_per_cell(cfg),
            "sharding": f"batch x rows = {g_batch} x {world // g_batch}",
            "l2": "inputs larger than L2" if args.config >= 3 else "inputs smaller than L2 (launch-bound case)"}


OPERAND_CODES = {"tf32": 0, "bf16": 1, "fp16": 2}
DTYPE_TEXT = {
    "fp16": "fp16 operands (10 mantissa bits like TF32; per-tensor power-of-two scaling; fp32 in HBM), fp32 accumulate",
    "tf32": "tf32 operands (fp32 in HBM), fp32 accumulate",
    "bf16": "bf16 operands in the sweeps and the gradient GEMMs (fp32 in HBM), fp32 accumulate",
}


def measure_tf32_peak(device, dtype=torch.float32):
    """cuBLAS GEMM 8192^3 through torch.matmul (TF32 for float32 inputs), best of 10 (burst) and back to back for ~1 s."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    n = 8192
    a = torch.randn(n, n, device=device).to(dtype)
    b = torch.randn(n, n, device=device).to(dtype)
    for _ in range(3):
        a @ b
    best = float("inf")
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); a @ b; e1.record(); e1.synchronize()
        best = min(best, e0.elapsed_time(e1))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = max(10, int(1000.0 / best))
    e0.record()
    for _ in range(reps):
        a @ b
    e1.record(); e1.synchronize()
    sustained = e0.elapsed_time(e1) / reps
    torch.backends.cuda.matmul.allow_tf32 = prev
    fl = 2.0 * n ** 3
    return fl / best / 1e9, fl / sustained / 1e9  # TFLOP/s


# --------------------------------------------------------------------------------------- sub-records
def extra_levels4(time_e2e, e2e_one_level):
    """The call site with the reference's four pyramid levels (core/corr.py:377-382,416: image 2 pooled three times,
    every op run per level), end to end like `e2e`.  The metric's cells are level-0 cells; levels 1-3 add 0.33x."""
    rec = time_e2e(4, 3, 2)
    out = {"ms_per_step": rec["ms_per_step"], "ms_per_step_min": rec["ms_per_step_min"],
           "level0_cells_per_s": rec["value"], "cells_incl_coarse_levels_per_s": rec["value"] * (1 + 1 / 4 + 1 / 16 + 1 / 64)}
    if e2e_one_level:
        out["ratio_to_one_level"] = rec["ms_per_step"] / e2e_one_level["ms_per_step"]
    return out


def extra_config4_bf16(ms, device, args):
    """BASELINE config 4 as it is stated (B=8, 47x156, Kc=2, BF16 operands, forward + backward) through the level
    calls, device-resident, with the largest deviation of the max/mean channels of a band of image-1 rows from an
    FP32 torch matmul on the same features (BF16 rounds the operands to 8 bits: ~1e-2 of the largest value)."""
    from separableflowthesis_b200 import _lib, sharding
    cfg = dict(CONFIGS[4])
    job = make_job(cfg, sharding.make_shard(cfg["B"], cfg["H"], 1, 0), device, "level")
    lib = _lib.load()
    prev = lib.sfb_set_sweep_operands(1)
    try:
        for _ in range(3):
            out = run_level(ms, cfg, job)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        steps = max(5, args.steps)
        e0.record()
        for _ in range(steps):
            out = run_level(ms, cfg, job)
        e1.record()
        torch.cuda.synchronize()
    finally:
        lib.sfb_set_sweep_operands(prev)
    t = e0.elapsed_time(e1) / steps
    sep_u, sep_v = out[0], out[1]
    r0, r1 = 20, 24
    prev_tf32 = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    F1, F2 = job["F1"][:1, r0:r1], job["F2"][:1]
    S = torch.matmul(F1.reshape(1, -1, C_FEAT), F2.reshape(1, -1, C_FEAT).transpose(1, 2))
    S = S.reshape(1, r1 - r0, cfg["W"], cfg["H"], cfg["W"])
    torch.backends.cuda.matmul.allow_tf32 = prev_tf32
    ref_v = torch.stack((S.max(4).values, S.mean(4)), 1).permute(0, 1, 4, 2, 3)   # (1, 2, H2, rows, W1): per-u channels
    ref_u = torch.stack((S.max(3).values, S.mean(3)), 1).permute(0, 1, 4, 2, 3)   # (1, 2, W2, rows, W1)
    err = max(((sep_v[:1, :2, :, r0:r1] - ref_v).abs().max() / ref_v.abs().max()).item(),
              ((sep_u[:1, :2, :, r0:r1] - ref_u).abs().max() / ref_u.abs().max()).item())
    return {"workload": cfg["name"].replace("(fp32 operands)", "(bf16 operands)"),
            "value": job["cells"] / (t * 1e-3), "unit": "cells/s", "ms_per_step": t, "steps": steps,
            "dtype": "bf16 operands in the sweeps and the gradient GEMMs, fp32 accumulate",
            "max_rel_err_max_mean_channels_vs_fp32": err, "band": f"sample 0, image-1 rows {r0}..{r1 - 1}"}


def extra_tf32_operands(ms, cfg, job, args):
    """The same job with TF32 operands (sfb_set_sweep_operands(TF32)): the operand type of the same precision at half
    the tensor-core rate, for comparison with the headline."""
    from separableflowthesis_b200 import _lib
    lib = _lib.load()
    prev = lib.sfb_set_sweep_operands(OPERAND_CODES["tf32"])
    try:
        for _ in range(3):
            run_level(ms, cfg, job)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        steps = max(5, args.steps)
        e0.record()
        for _ in range(steps):
            run_level(ms, cfg, job)
        e1.record()
        torch.cuda.synchronize()
    finally:
        lib.sfb_set_sweep_operands(prev)
    t = e0.elapsed_time(e1) / steps
    return {"dtype": DTYPE_TEXT["tf32"], "value": job["cells"] / (t * 1e-3), "unit": "cells/s", "ms_per_step": t,
            "steps": steps}


def extra_reference_cuda(args):
    """The reference's own CUDA extension (oracle/_ref/MemorySaver.so, built unmodified from libs/MemorySaver/src) on
    this GPU next to this library, on BASELINE config 2 (B=2, 48x64, Kc=2: the channel count its forward kernel
    computes), the five ops device-resident in the reference's layouts."""
    lines = []
    sub = argparse.Namespace(steps=max(2, min(args.steps, 3)), warmup=3)
    cfg = dict(CONFIGS[2])
    metric = "separated cost-volume cells/sec (fwd+bwd)"
    run_reference_cuda(sub, cfg, metric, "cells/s", lines.append)
    if len(lines) == 1:
        return lines[0]
    ref, ours = lines
    return {"workload": cfg["name"], "path": "the five ops in the reference's layouts, device-resident",
            "reference_cuda": {"value": ref["value"], "ms_per_step": ref["ms_per_step"], "steps": ref["steps"]},
            "this_library": {"value": ours["value"], "ms_per_step": ours["ms_per_step"], "steps": ours["steps"]},
            "ratio": ours["value"] / ref["value"], "unit": "cells/s"}


def extra_row_shard(args, cfg, world, rank, device, ms, time_e2e, barrier, max_over_ranks, sum_over_ranks, e0, e1,
                    batch_job):
    """The partition BASELINE config 5 names: every rank holds all samples and a block of image-1 rows (plus one halo
    row per side for the attention stencil).  Image 2's features are copied from the host once (each rank 1/N of the
    samples) and completed on every GPU by an all-gather over NVLink; the partial image-2 feature gradients are
    reduce-scattered back to those slices; halo rows of the image-1 gradient go to the neighbours.  Reports the
    device-resident and end-to-end throughput and how far the gradients are from the batch-sharded run's on the same
    seeded data."""
    from separableflowthesis_b200 import sharding
    shard = sharding.make_shard(cfg["B"], cfg["H"], world, rank, prefer="rows")
    group = sharding.new_row_groups(world, shard.g_rows)
    job = make_job(cfg, shard, device, "level")
    total_cells = sum_over_ranks(float(job["cells"]))

    def norms(j, grp):
        out = run_level(ms, cfg, j, grp)
        g1, g2, gw = out[6], out[7], torch.cat([out[8].reshape(-1), out[10].reshape(-1)]).double()
        torch.distributed.all_reduce(gw)   # the parameters are shared: their gradient is the sum over all ranks
        # every element of gF1 / gF2 is owned by exactly one rank in either partition
        return [sum_over_ranks(g1.double().abs().sum().item()), sum_over_ranks(g2.double().abs().sum().item()),
                gw.abs().sum().item()]

    n_batch = norms(batch_job, None)
    n_rows = norms(job, group)
    diff = [abs(a - b) / max(abs(a), 1e-30) for a, b in zip(n_batch, n_rows)]
    for _ in range(max(1, args.warmup - 1)):
        run_level(ms, cfg, job, group)
    barrier()
    e0.record()
    for _ in range(args.steps):
        run_level(ms, cfg, job, group)
    e1.record()
    barrier()
    t = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    e2e = time_e2e(1, args.steps, 2, sh=shard, grp=group, jb=job, f2_from_rank0=True)
    e2e_value = total_cells / (e2e["ms_per_step"] * 1e-3)
    f2_bytes = cfg["B"] * C_FEAT * cfg["H"] * cfg["W"] * 4
    return {"sharding": f"batch x rows = {shard.g_batch} x {shard.g_rows}", "value": total_cells / (t * 1e-3),
            "unit": "cells/s", "ms_per_step": t, "steps": args.steps,
            "e2e": {"value": e2e_value, "ms_per_step": e2e["ms_per_step"], "ms_per_step_min": e2e["ms_per_step_min"],
                    "h2d_bytes_per_step": e2e["h2d_bytes_per_step"], "d2h_bytes_per_step": e2e["d2h_bytes_per_step"]},
            "nvlink_bytes_per_rank_per_step": {
                "image2_features_all_gather": f2_bytes * (world - 1) // world,
                "image2_gradient_reduce_scatter": f2_bytes * (world - 1) // world,
                "image1_gradient_halo_rows": 2 * 2 * cfg["B"] * C_FEAT * cfg["W"] * 4},
            "rel_diff_vs_batch_sharded": {"sum_abs_gF1": diff[0], "sum_abs_gF2": diff[1], "sum_abs_gweights": diff[2]}}


def main():
    # Libraries (NCCL among them) print banners on stdout; keep stdout for the one JSON line by sending
    # everything else to stderr.
    json_fd = os.dup(1)
    os.dup2(2, 1)

    def emit(line: dict):
        os.write(json_fd, (json.dumps(line) + "\n").encode())

    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--config", type=int, default=5, choices=sorted(CONFIGS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-cuda"],
                    help="reference: the CPU port of the reference's dense path (the reference arm of the benchmark contract); "
                         "reference-cuda: the reference's own CUDA extension built by oracle/build_ref_cuda.py, timed on "
                         "the five ops next to this library's five ops (configs with Kc = 2 only: the reference's forward "
                         "kernel is compiled for two attention channels, MemorySaver_kernel_forward.cu:20)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-roofline", action="store_true", help="skip the per-kernel timing pass and the TF32 peak run")
    ap.add_argument("--unfused", action="store_true",
                    help="run the two backward ops as the reference's two separate calls instead of the one-call backward")
    ap.add_argument("--path", default="auto", choices=["auto", "level", "ops", "lookup", "lookup4d"],
                    help="level: one library call per pyramid-level forward / backward, as the call site runs it "
                         "(attention Conv3d + softmax included); ops: the five ops of the reference's module with "
                         "random attention weights; auto: level when the config has attention channels; lookup: "
                         "the CorrBlock1D lookup on the aggregated volumes instead of the separation; lookup4d: the 4D lookup "
                         "without the stored volume")
    ap.add_argument("--e2e-chunks", type=int, default=2,
                    help="micro-batches per end-to-end step (the host->device copy of one overlaps the compute of the "
                         "previous one); 1 = copy everything, then compute")
    ap.add_argument("--no-e2e-prefetch", action="store_true",
                    help="end to end: do not copy the next step's first micro-batch while this step computes")
    ap.add_argument("--shard", default="batch", choices=["batch", "rows"],
                    help="batch: samples first, image-1 rows for what is left (no data-path exchange when the batch "
                         "is a multiple of the GPUs); rows: every rank gets all samples and a block of image-1 rows "
                         "plus a halo row per side, gF2 is summed and halo-row gradients exchanged over NCCL")
    ap.add_argument("--operands", default="fp16", choices=["fp16", "tf32", "bf16"],
                    help="operand type of every contraction: fp16 (the library's default: TF32's 10 mantissa bits at "
                         "twice its tensor-core rate, per-tensor power-of-two scaling), tf32, or bf16 (BASELINE's bf16 "
                         "configuration; lower precision, so not the headline)")
    ap.add_argument("--levels", type=int, default=1,
                    help="pyramid levels of the end-to-end block (the metric counts level-0 cells; the reference's "
                         "model uses 4 levels = 1.33x the cells)")
    ap.add_argument("--batch", type=int, default=0, help="override the batch size (small ncu captures)")
    ap.add_argument("--repeats", type=int, default=5,
                    help="timed regions of --steps steps each; the first is the headline, all of them give the spread")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the sub-records (reference's CUDA kernels, config 4 in BF16, 4-level pyramid, row shards)")
    args = ap.parse_args()
    cfg = dict(CONFIGS[args.config])
    if args.batch > 0:
        cfg["B"] = args.batch
        cfg["name"] += f" [batch overridden to {args.batch}]"
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    unit = "cells/s"
    metric = "separated cost-volume cells/sec (fwd+bwd)" if cfg["bwd"] else "separated cost-volume cells/sec (fwd)"

    if args.impl == "reference":
        # The reference's own path cannot travel (Python + a CUDA extension that needs its checkout);
        # the timed CPU arm is the oracle port of its dense einsum path on all host cores, rank 0 only.
        if rank != 0:
            return
        base, dt, n_steps = time_cpu(cfg, budget_s=60.0, steps=args.steps, warmup=max(1, min(args.warmup, 2)))
        line = {"impl": "reference", "metric": metric, "value": base["value"], "unit": unit, "n_gpus": args.gpus,
                "steps": n_steps, "warmup": max(1, min(args.warmup, 2)), "ms_per_step": dt * 1e3,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": workload_config(args, cfg, max(world, args.gpus)),
                "cpu_baseline": base,
                "e2e": {"value": base["value"], "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        emit(line)
        return

    if args.impl == "reference-cuda":
        if rank == 0:
            run_reference_cuda(args, cfg, metric, unit, emit)
        return

    import torch.distributed as dist
    from separableflowthesis_b200 import _lib, ops as ms, sharding
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    shard = sharding.make_shard(cfg["B"], cfg["H"], world, rank, prefer=args.shard)
    row_group = sharding.new_row_groups(world, shard.g_rows) if world > 1 else None
    path = args.path
    if path in ("lookup", "lookup4d"):   # the lookups that follow the separation in the model, one GPU
        if rank == 0:
            (run_lookup_bench if path == "lookup" else run_lookup4d_bench)(args, cfg, device, emit)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    path = resolve_path(args, cfg)
    if path == "level" and cfg["Kc"] == 0:
        raise SystemExit("--path level needs attention channels")
    job = make_job(cfg, shard, device, path)
    _lib.load().sfb_set_sweep_operands(OPERAND_CODES[args.operands])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        t = torch.tensor([x], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    def sum_over_ranks(x):
        t = torch.tensor([x], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return t.item()

    total_cells = sum_over_ranks(float(job["cells"]))

    # ---- device-resident throughput ("value") ----
    for _ in range(args.warmup):
        run_ops(ms, cfg, job, not args.unfused, row_group)
    barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        run_ops(ms, cfg, job, not args.unfused, row_group)
    e1.record()
    barrier()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    clocks = sampler.stop() if sampler else None
    ms_per_step = ms_total / args.steps
    value = total_cells / (ms_per_step * 1e-3)
    # the same timed region again, for the spread (the headline stays the first region, timed as above)
    region_ms = [ms_per_step]
    for _ in range(max(0, args.repeats - 1)):
        barrier()
        e0.record()
        for _ in range(args.steps):
            run_ops(ms, cfg, job, not args.unfused, row_group)
        e1.record()
        barrier()
        region_ms.append(max_over_ranks(e0.elapsed_time(e1)) / args.steps)
    spread = {"regions": len(region_ms), "steps_per_region": args.steps, "ms_per_step_median": statistics.median(region_ms),
              "ms_per_step_min": min(region_ms), "ms_per_step_max": max(region_ms)}
    # host time of one step's launch path (Python + ctypes + tensor-map encodes + launches), device idle at the start
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(3):
        run_ops(ms, cfg, job, not args.unfused, row_group)
    host_ms_per_step = (time.perf_counter() - t0) / 3 * 1e3
    torch.cuda.synchronize()

    # ---- per-kernel device time of the same steps (separate pass: events around every launch) ----
    report = []
    if not args.no_roofline:
        _lib.kernel_timing(True)
        for _ in range(min(args.steps, 3)):
            run_ops(ms, cfg, job, not args.unfused, row_group)
        torch.cuda.synchronize()
        report = _lib.kernel_timing_report()
        _lib.kernel_timing(False)
    roofline, kernels = None, []
    # kernels of this library per step: counted by the library when the timing pass ran, else from the op list
    launches = (sum(r[2] for r in report) // min(args.steps, 3)) if report else launches_per_step(cfg, path)
    if rank == 0 and report:
        tot = sum(r[1] for r in report)
        kernels = [{"kernel": n, "launches": l, "ms_per_launch": t / l, "share": t / tot} for n, t, l in report]
        tf32_burst, tf32_sust = measure_tf32_peak(device)
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except OSError:
            pass
        # MEASURED_PEAKS.json has the dense BF16 rate (the kind::f16 pipe, which FP16 operands use as well); TF32 runs
        # at half of it.  The kernels are timed inside back-to-back steps under the power cap, so the sustained figure
        # is the denominator: the full one for 16-bit operands, half of it for TF32 operands.
        op16 = args.operands != "tf32"
        f16_sust = float(peaks["bf16_tflops_sustained"]) if "bf16_tflops_sustained" in peaks else None
        f16_burst = float(peaks["bf16_tflops"]) if "bf16_tflops" in peaks else None
        file_sust = (f16_sust if op16 else 0.5 * f16_sust) if f16_sust else None
        f16c_burst, f16c_sust = measure_tf32_peak(device, torch.float16) if op16 else (None, None)
        fl = 2.0 * C_FEAT * job["cells"]            # one contraction over this rank's cells per launch
        per_kernel = []
        for name, t, l in report:
            if not name.startswith(("sweep_kernel", "grad_gemm_kernel")):
                continue
            ach = fl / (t / l * 1e-3) / 1e12
            per_kernel.append({"kernel": name, "ms_per_launch": t / l, "share": t / tot, "achieved": ach,
                               "frac_of_pipe_sustained_file": ach / file_sust if file_sust else None,
                               "frac_of_half_bf16_sustained_file": ach / (0.5 * f16_sust) if f16_sust else None,
                               "frac_of_cublas_tf32_sustained": ach / tf32_sust,
                               "frac_of_cublas_fp16_sustained": ach / f16c_sust if f16c_sust else None})
        dominant = max(per_kernel, key=lambda k: k["share"])
        worst = min(per_kernel, key=lambda k: k["achieved"])
        peak = file_sust if file_sust else (f16c_sust if op16 else tf32_sust)
        bpc = DRAM_BYTES_PER_CELL.get("16bit_operands" if op16 else "tf32_operands", {}).get(dominant["kernel"])
        roofline = {"bound": "tensor", "kernel": dominant["kernel"], "achieved": dominant["achieved"], "peak": peak,
                    "unit": "TFLOP/s", "frac": dominant["achieved"] / peak,
                    "traffic": (bpc * job["cells"]) if bpc else None,
                    "peak_source": ((("bf16_tflops_sustained of MEASURED_PEAKS.json (of measured): the 16-bit tensor pipe "
                                      "these operands run on" if op16 else
                                      "0.5 x bf16_tflops_sustained of MEASURED_PEAKS.json (of measured; the file has no "
                                      "TF32 entry, TF32 runs at half the BF16 rate)")) if file_sust else
                                    "cuBLAS 8192^3 via torch.matmul measured in this run, sustained (of fallback: no "
                                    "MEASURED_PEAKS.json)"),
                    "peak_measured_file": {"bf16_sustained": f16_sust, "bf16_burst": f16_burst,
                                           "half_bf16_sustained": 0.5 * f16_sust if f16_sust else None,
                                           "half_bf16_burst": 0.5 * f16_burst if f16_burst else None},
                    "peak_cublas_tf32_this_run": {"sustained": tf32_sust, "burst": tf32_burst},
                    "peak_cublas_fp16_this_run": {"sustained": f16c_sust, "burst": f16c_burst},
                    "frac_of_half_bf16_sustained_file": dominant["achieved"] / (0.5 * f16_sust) if f16_sust else None,
                    "algorithmic_flop_per_launch": fl, "ms_per_launch": dominant["ms_per_launch"],
                    "worst_kernel": worst["kernel"], "worst_frac": worst["achieved"] / peak,
                    "whole_step_frac": value * flops_per_cell(cfg) / 1e12 / world / peak,
                    "whole_step_frac_of_half_bf16_sustained_file":
                        value * flops_per_cell(cfg) / 1e12 / world / (0.5 * f16_sust) if f16_sust else None,
                    "per_kernel": per_kernel}

    # ---- end to end through the public API with host buffers ----
    def time_e2e(levels, steps, regions, sh=shard, grp=row_group, jb=job, f2_from_rank0=False):
        """`regions` timed regions of `steps` steps each through AlternateCorrBlockSepflow from pinned host buffers; every
        region starts without anything copied ahead and ends without a prefetch for a step outside it."""
        runner = E2E(cfg, jb, device, chunks=args.e2e_chunks, levels=levels, shard=sh, row_group=grp,
                     prefetch=not args.no_e2e_prefetch, f2_from_rank0=f2_from_rank0)
        for _ in range(min(args.warmup, 3)):   # warm-up runs the same pipeline (allocator steady state)
            runner.step()
        runner.drain()
        per_step, host = [], []
        for _ in range(regions):
            barrier()
            runner.prefetched = None   # nothing copied before the timed region is used inside it
            t0 = time.perf_counter()
            e0.record()
            for i in range(steps):
                runner.prefetch = (not args.no_e2e_prefetch) and i < steps - 1   # the last step has no successor
                runner.step()
            runner.drain()   # the last step's result is read inside the timed region as well
            e1.record()
            host.append((time.perf_counter() - t0) / steps * 1e3)
            barrier()
            per_step.append(max_over_ranks(e0.elapsed_time(e1)) / steps)
        rec = {"value": total_cells / (per_step[0] * 1e-3), "unit": unit, "ms_per_step": per_step[0],
               "regions": regions, "steps_per_region": steps, "ms_per_step_median": statistics.median(per_step),
               "ms_per_step_min": min(per_step), "ms_per_step_max": max(per_step),
               "h2d_bytes_per_step": int(sum_over_ranks(float(runner.h2d))),
               "d2h_bytes_per_step": int(sum_over_ranks(float(runner.d2h))),
               "pyramid_levels": levels, "chunks": runner.chunks}
        del runner
        return rec

    e2e = None
    if not args.no_e2e:
        e2e = time_e2e(args.levels, args.steps, min(args.repeats, 3))
        e2e["path"] = (f"pinned host f1,f2 (B,C,H,W) -> AlternateCorrBlockSepflow(num_levels={args.levels}).separate with "
                       "Conv3d attention -> autograd backward -> all-reduce of attention-parameter grads -> host; "
                       f"{e2e['chunks']} micro-batch(es) per step, copy of one overlapping compute of the previous"
                       + ("" if args.no_e2e_prefetch else
                          "; the first micro-batch of the next timed step is copied while this step computes "
                          "(all copies of the timed steps run inside the timed region)")
                       + ".  What returns to the host every step: the two feature-gradient checksums of each micro-batch "
                         "and the summed attention-parameter gradients; the separated volumes and the feature gradients "
                         "stay on the device, where the model's next layers (cost aggregation, encoder backward) "
                         "consume them; the host reads a step's result (asynchronous copy to pinned memory) after it has "
                         "queued the next step, and the last one before the timed region ends")

    extras = {}
    if not args.no_extras and args.config == 5 and args.batch == 0 and path == "level":
        if world == 1:
            extras["levels4"] = extra_levels4(time_e2e, e2e)
            extras["config4_bf16"] = extra_config4_bf16(ms, device, args)
            if args.operands != "tf32":
                extras["tf32_operands"] = extra_tf32_operands(ms, cfg, job, args)
            extras["reference_cuda"] = extra_reference_cuda(args)
        else:
            extras["row_shard"] = extra_row_shard(args, cfg, world, rank, device, ms, time_e2e, barrier, max_over_ranks,
                                                  sum_over_ranks, e0, e1, job)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu, _, _ = time_cpu(cfg, budget_s=15.0)

    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    line = {
        "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": DTYPE_TEXT[args.operands],
        "data": "synthetic",
        "config": workload_config(args, cfg, world),
        "useful_tflops": value * flops_per_cell(cfg) / 1e12,
        "repeats": spread, "host_ms_per_step": host_ms_per_step,
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches * args.steps,
        "roofline": roofline, "kernels": kernels, "cpu_baseline": cpu,
    }
    line.update(extras)
    emit(line)


if __name__ == "__main__":
    main()
