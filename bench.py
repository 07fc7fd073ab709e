#!/usr/bin/env python
"""Benchmark of Flash Deformable 3D Attention on B200: forward + backward samples/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config 5] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

One "step" is one forward + backward pass of the operator over one synthetic batch of the chosen
benchmark configuration (default: self-attention on a 256x512x2048 tile at strides 8/16/32, B=2,
N=Lq=598016, G=8, D=32, K=8, bf16 value, fp32 offsets/logits).  A "sample" is one batch element.
Rank 0 prints ONE JSON line.

  value        B / (device time of one step), inputs resident in HBM, C-ABI calls, CUDA events,
               max over ranks.  With N > 1 GPUs the queries of every batch element are split over
               the ranks, value is replicated and the fp32 grad_value images are all-reduced
               (NCCL) before the cast -- total work is fixed, so scaling is "strong".
  e2e          same metric through the public autograd API with HOST (pinned) inputs: every step
               copies its inputs host->device and all results (out, grad_value, grad_packed)
               device->host inside the timed region.
  roofline     dominant kernel (backward scatter/gather): algorithmic bytes / CUDA-event time of
               that launch against the measured HBM copy bandwidth.
  cpu_baseline the CPU oracle (PyTorch restatement of the reference's CPU implementation) timed on
               this machine's host cores on a bounded sample of the same workload (N=1 only).

--impl reference times only that CPU implementation (rank 0; other ranks exit).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CONFIGS = {
    1: dict(name="cfg1 self-attn (4,8,8)+(2,4,4) fp32", shapes=[(4, 8, 8), (2, 4, 4)], B=1, Q=288, G=4, D=16, K=4,
            vdt="float32", coords="uniform"),
    2: dict(name="cfg2 self-attn 128x256x512 strides 16/32", shapes=[(8, 16, 32), (4, 8, 16)], B=2, Q=4608, G=8, D=32,
            K=4, vdt="bfloat16", coords="uniform"),
    3: dict(name="cfg3 cross-attn 200 queries, 128x256x512 strides 8/16/32",
            shapes=[(16, 32, 64), (8, 16, 32), (4, 8, 16)], B=4, Q=200, G=8, D=32, K=4, vdt="bfloat16", coords="clustered"),
    4: dict(name="cfg4 self-attn 256x512x2048 strides 16/32", shapes=[(16, 32, 128), (8, 16, 64)], B=1, Q=73728, G=8,
            D=32, K=4, vdt="bfloat16", coords="uniform"),
    5: dict(name="cfg5 self-attn 256x512x2048 strides 8/16/32", shapes=[(32, 64, 256), (16, 32, 128), (8, 16, 64)], B=2,
            Q=598016, G=8, D=32, K=8, vdt="bfloat16", coords="uniform"),
}
METRIC = "fwd+bwd samples/s (fwd samples/s and achieved GB/s vs HBM roofline beside it)"

# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per full-size launch of the backward kernels of
# config 5, from the ncu captures summarised under profiles/: measured on the reduced case
# (--batch 1 --queries 74752, 1/16 of the rows over the same per-batch-element volume) and scaled x16.
NCU_BACKWARD_TRAFFIC_BYTES = {5: 16 * (3.16e9 + 3.09e9)}


# ---------------------------------------------------------------------------------------------
# synthetic inputs
# ---------------------------------------------------------------------------------------------
def make_device_inputs(cfg, dev, q_begin, q_end, seed=0):
    """Seeded inputs of the configuration's shapes and distributions, generated on the device.
    Every rank generates the same full ``value`` (replicated) and its own query range."""
    vdt = getattr(torch, cfg["vdt"])
    shapes = torch.tensor(cfg["shapes"], dtype=torch.long, device=dev)
    sizes = shapes.prod(1)
    lsi = torch.cat((sizes.new_zeros(1), sizes.cumsum(0)[:-1]))
    N = int(sizes.sum())
    B, G, D, K, L = cfg["B"], cfg["G"], cfg["D"], cfg["K"], len(cfg["shapes"])
    Qr = q_end - q_begin
    gen = torch.Generator(device=dev).manual_seed(seed)
    value = torch.randn(B, N, G, D, generator=gen, device=dev, dtype=torch.float32).to(vdt)
    gen_q = torch.Generator(device=dev).manual_seed(seed * 1000 + 17 + q_begin)
    packed = torch.empty(B, Qr, G, L * K * 4, device=dev, dtype=torch.float32)
    loc = packed[..., : L * K * 3]
    if cfg["coords"] == "uniform":
        loc.copy_(torch.rand(B, Qr, G, L * K * 3, generator=gen_q, device=dev) * 1.1 - 0.05)
    else:
        centre = torch.rand(B, Qr, 1, 1, 3, generator=gen_q, device=dev)
        pts = centre + 0.05 * torch.randn(B, Qr, G, L * K, 3, generator=gen_q, device=dev)
        loc.copy_(pts.clamp_(-0.05, 1.05).reshape(B, Qr, G, L * K * 3))
    packed[..., L * K * 3:].copy_(torch.randn(B, Qr, G, L * K, generator=gen_q, device=dev))
    grad_out = torch.randn(B, Qr, G * D, generator=gen_q, device=dev, dtype=torch.float32).to(vdt)
    return value, shapes, lsi, packed, grad_out


def count_in_range_corners(cfg, packed):
    """Exact number of (point, corner) pairs that fall inside their level, from the coordinates
    themselves (same fp32 un-normalisation as the kernels)."""
    L, K = len(cfg["shapes"]), cfg["K"]
    B, Q, G, _ = packed.shape
    total = 0
    chunk = max(1, (1 << 24) // max(1, G * K * 3))
    for q0 in range(0, Q, chunk):
        loc = packed[:, q0:q0 + chunk, :, : L * K * 3].reshape(B, -1, G, L, K, 3)
        for lvl, (dz, hy, wx) in enumerate(cfg["shapes"]):
            n = None
            for axis, size in ((0, wx), (1, hy), (2, dz)):
                g = 2.0 * loc[:, :, :, lvl, :, axis] - 1.0
                c = ((g + 1.0) * float(size) - 1.0) * 0.5
                c0 = torch.floor(c)
                cnt = ((c0 >= 0) & (c0 < size)).to(torch.int32) + ((c0 + 1 >= 0) & (c0 + 1 < size)).to(torch.int32)
                n = cnt if n is None else n * cnt
            total += int(n.sum().item())
    return total


def byte_model(cfg, n_corners_in, B, Qr, N):
    """Algorithmic bytes of one launch of each kernel (gather model: rows gathered x row bytes)."""
    G, D, K, L = cfg["G"], cfg["D"], cfg["K"], len(cfg["shapes"])
    sv = 4 if cfg["vdt"] == "float32" else 2
    so = 4
    P = B * Qr * G * L * K
    rows = B * Qr * G * D
    fwd = n_corners_in * D * sv + P * 4 * so + rows * sv
    bwd_kernel = n_corners_in * D * sv + P * 4 * so + rows * sv + P * 4 * so + n_corners_in * D * 4
    cast = B * N * G * D * (4 + sv) if sv == 2 else 0
    return dict(points=P, corners_in=n_corners_in, fwd=fwd, bwd_kernel=bwd_kernel, cast=cast,
                fwd_bwd=fwd + bwd_kernel + cast)


# ---------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, dev_index):
        self.lines, self.proc = [], None
        try:
            ident = str(dev_index)
            try:
                ident = "GPU-" + str(torch.cuda.get_device_properties(dev_index).uuid)
            except Exception:
                pass
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", ident, f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def window(self, t0, t1):
        sm, mx, reasons = [], [], set()
        for t, line in self.lines:
            if t < t0 or t > t1 + 0.15:
                continue
            parts = [p.strip() for p in line.split(",")]
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except (ValueError, IndexError):
                continue
            for name, flag in zip(self.NAMES, parts[3:7]):
                if flag == "Active":
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()


# ---------------------------------------------------------------------------------------------
# CPU baseline / reference arm: the CPU oracle on host cores, bounded sample
# ---------------------------------------------------------------------------------------------
def cpu_reference_step_inputs(cfg, sample_q, seed=0):
    from oracle import fda_oracle

    value, sh, lsi, packed, grad_out = fda_oracle.make_inputs(
        cfg["shapes"], 1, sample_q, cfg["G"], cfg["D"], cfg["K"], seed=seed, coords=cfg["coords"])
    if cfg["vdt"] != "float32":
        value = value.to(getattr(torch, cfg["vdt"])).float()
        grad_out = grad_out.to(getattr(torch, cfg["vdt"])).float()
    return value, sh, packed, grad_out


def cpu_reference_time(cfg, sample_q, steps, warmup):
    """Seconds per pass (fwd, fwd+bwd) of the CPU oracle over ``sample_q`` queries of ONE batch element
    with the full-size value volume, all host threads."""
    from oracle import fda_oracle

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    value, sh, packed, grad_out = cpu_reference_step_inputs(cfg, sample_q)
    K = cfg["K"]
    t_f, t_fb = [], []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        fda_oracle.fused_forward(value, sh, packed, K, chunk=sample_q)
        t1 = time.perf_counter()
        fda_oracle.fused_forward_backward(value, sh, packed, grad_out, K, chunk=sample_q)
        t2 = time.perf_counter()
        if i >= warmup:
            t_f.append(t1 - t0)
            t_fb.append(t2 - t1)
    return min(t_f), min(t_fb), cores


def pick_cpu_sample(cfg, budget_s):
    """Largest power-of-two query count whose forward+backward is expected to fit ``budget_s``."""
    q = min(cfg["Q"], 1024)
    tf, tfb, _ = cpu_reference_time(cfg, q, 1, 0)
    while q * 2 <= cfg["Q"] and (tf + tfb) * 2.2 < budget_s and q < 65536:
        q *= 2
        tf, tfb, _ = cpu_reference_time(cfg, q, 1, 0)
    return q


def cpu_baseline_block(cfg, steps=1, warmup=0, budget_s=6.0):
    q = pick_cpu_sample(cfg, budget_s)
    tf, tfb, cores = cpu_reference_time(cfg, q, steps, warmup)
    scale = q / cfg["Q"]  # fraction of one sample (= one batch element) the pass covered
    return {
        "value": scale / tfb, "fwd_value": scale / tf, "unit": "samples/s", "cores": cores, "kind": "port",
        "sample": f"{q} of {cfg['Q']} queries of one batch element against the full-size value volume, fp32, "
                  f"torch {torch.__version__} CPU, linear extrapolation to a whole sample; fwd+bwd {tfb:.3f} s, fwd {tf:.3f} s",
    }


def run_reference_arm(args, cfg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    block = cpu_baseline_block(cfg, steps=max(1, args.steps), warmup=max(0, args.warmup), budget_s=8.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": block["value"], "fwd_value": block["fwd_value"],
        "unit": "samples/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": None, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": cfg["name"], "B": cfg["B"], "Lq": cfg["Q"], "G": cfg["G"], "D": cfg["D"], "K": cfg["K"],
                   "levels": cfg["shapes"]},
        "cpu_baseline": block,
        "e2e": {"value": block["value"], "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# optional: the reference's own CUDA kernels on this GPU (reported baseline; needs baseline/_ref/)
# ---------------------------------------------------------------------------------------------
def reference_cuda_block(cfg, value, shapes, lsi, packed, grad_out, steps=5, warmup=2):
    """Times the unmodified reference kernels (built by baseline/build_ref_cuda.sh) on the same inputs.
    They only take offsets/logits in the value dtype, so ``packed`` is cast to it first."""
    import importlib.util

    so = os.path.join(ROOT, "baseline", "_ref", "ops3d_ref_C.so")
    if not os.path.exists(so):
        return {"unavailable": "baseline/_ref/ops3d_ref_C.so not built (baseline/build_ref_cuda.sh <reference checkout>)"}
    spec = importlib.util.spec_from_file_location("ops3d_ref_C", so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    B, Q, G, D, K = cfg["B"], packed.shape[1], cfg["G"], cfg["D"], cfg["K"]
    pk = packed.to(value.dtype)
    # launch hints as the reference's findspec / findspec_bwd return them for G*D = 256
    from ops3d_b200.flash_deform_attn import findspec, findspec_bwd
    d_f, t_f = findspec(B, Q, G, D)
    d_b, t_b = findspec_bwd(B, Q, G, D)

    def fwd():
        return mod.flash_deform_attn_forward(value, shapes, lsi, pk, 64, K, d_f, t_f, True)

    def bwd():
        return mod.flash_deform_attn_backward(value, shapes, lsi, pk, grad_out, 64, K, d_b, t_b)

    for _ in range(warmup):
        fwd(); bwd()
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    tf = tb = 0.0
    for _ in range(steps):
        ev[0].record(); fwd(); ev[1].record(); bwd(); ev[2].record()
        torch.cuda.synchronize()
        tf += ev[0].elapsed_time(ev[1]); tb += ev[1].elapsed_time(ev[2])
    tf /= steps; tb /= steps
    return {"fwd_ms": tf, "bwd_ms": tb, "value": B / ((tf + tb) * 1e-3), "fwd_value": B / (tf * 1e-3), "unit": "samples/s",
            "note": "reference csrc/cuda kernels compiled unmodified for sm_100a; offsets/logits cast to the value dtype "
                    "(the only form they accept); includes their zero-fill and cast passes"}


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def run_ours(args, cfg):
    import torch.distributed as dist

    from ops3d_b200 import FlashDeformAttnFunction, capi
    from ops3d_b200.sharded import PeerReducer, query_range, sharded_flash_deform_attn

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run for N > 1")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operator has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    capi.load()

    B, Q, G, D, K = cfg["B"], cfg["Q"], cfg["G"], cfg["D"], cfg["K"]
    qb, qe = query_range(Q, rank, world)
    value, shapes, lsi, packed, grad_out = make_device_inputs(cfg, dev, qb, qe)
    N = value.shape[1]
    vdt = value.dtype
    out = torch.empty(B, qe - qb, G * D, dtype=vdt, device=dev)
    grad_value = torch.empty_like(value)
    grad_packed = torch.empty_like(packed)
    use_peer = world > 1 and args.reduce == "peer"
    reducer, peer_note = None, None
    if use_peer:
        # symmetric-memory set-up can be unavailable on a machine (no peer access): all ranks agree, then
        # either all use the fused exchange or all fall back to NCCL all-reduce + cast
        try:
            reducer = PeerReducer(value.shape, vdt, dev, spatial_shapes=shapes)
            ok = torch.ones(1, device=dev)
        except Exception as exc:  # noqa: BLE001
            peer_note = f"peer exchange unavailable ({type(exc).__name__}: {exc}); NCCL all-reduce used"
            ok = torch.zeros(1, device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if ok.item() == 0:
            reducer, use_peer = None, False
            os.environ["FDA_SHARDED_REDUCE"] = "nccl"  # the end-to-end leg follows suit
            peer_note = peer_note or "peer exchange unavailable on another rank; NCCL all-reduce used"
    reducer_passes = reducer.passes if use_peer else None
    L = len(cfg["shapes"])
    n_scratch = capi.scratch_bytes(value, packed, K)
    scratch = torch.empty(n_scratch, dtype=torch.uint8, device=dev) if (n_scratch and not use_peer) else None
    accum = None
    if not use_peer:
        accum = torch.empty(value.shape, dtype=torch.float32, device=dev) if vdt != torch.float32 else grad_value

    def step(ev=None):
        if ev: ev[0].record()
        capi.forward(value, shapes, lsi, packed, K, out=out)
        if ev: ev[1].record()
        if use_peer:
            # per batch element: scatter on this stream, fused NVLink reduce+cast overlapped on a side stream
            reducer.backward(value, shapes, lsi, packed, grad_out, K, grad_packed=grad_packed)
            if ev: ev[2].record(); ev[3].record()
            return
        capi.backward_accumulate_levels(value, shapes, lsi, packed, grad_out, K, accum, grad_packed, 0, L,
                                        capi.BWD_ZERO_IMAGE | capi.BWD_FINALIZE, scratch=scratch)
        if ev: ev[2].record()
        if world > 1:
            dist.all_reduce(accum)
        if vdt != torch.float32:
            capi.cast_grad_value(accum, grad_value)
        if ev: ev[3].record()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()

    events = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(args.steps)]
    launches0 = capi.KERNEL_LAUNCHES
    t_host0 = time.perf_counter()
    for ev in events:
        step(ev)
    torch.cuda.synchronize()
    t_host1 = time.perf_counter()
    gpu_launches = capi.KERNEL_LAUNCHES - launches0
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    total_ms = events[0][0].elapsed_time(events[-1][3])
    fwd_ms = sum(e[0].elapsed_time(e[1]) for e in events) / args.steps
    bwd_ms = sum(e[1].elapsed_time(e[2]) for e in events) / args.steps
    tail_ms = sum(e[2].elapsed_time(e[3]) for e in events) / args.steps
    clocks = sampler.window(t_host0, t_host1) if sampler else None

    times = torch.tensor([total_ms, fwd_ms, bwd_ms, tail_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    total_ms, fwd_ms, bwd_ms, tail_ms = times.tolist()
    ms_per_step = total_ms / args.steps

    ref_cuda = None
    if args.ref_cuda and world == 1:
        ref_cuda = reference_cuda_block(cfg, value, shapes, lsi, packed, grad_out)

    # ---- end to end through the public autograd API with host buffers --------------------------------
    e2e_ms, h2d, d2h, e2e_steps = None, 0, 0, 0
    if not args.no_e2e:
        e2e_steps = max(2, min(args.steps, 3))
        host_in = [t.cpu().pin_memory() for t in (value, packed, grad_out)]
        host_out = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in (out, grad_value, grad_packed)]
        h2d = sum(t.numel() * t.element_size() for t in host_in)
        d2h = sum(t.numel() * t.element_size() for t in host_out)
        del out, grad_value, grad_packed, accum, reducer, scratch
        torch.cuda.empty_cache()

        def e2e_step():
            v = host_in[0].to(dev, non_blocking=True).requires_grad_(True)
            pk = host_in[1].to(dev, non_blocking=True).requires_grad_(True)
            go = host_in[2].to(dev, non_blocking=True)
            if world > 1:
                o = sharded_flash_deform_attn(v, shapes, lsi, pk, 64, K)
            else:
                o = FlashDeformAttnFunction.apply(v, shapes, lsi, pk, 64, K, True)
            o.backward(go)
            host_out[0].copy_(o.detach(), non_blocking=True)
            host_out[1].copy_(v.grad, non_blocking=True)
            host_out[2].copy_(pk.grad, non_blocking=True)

        e2e_step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(e2e_steps):
            e2e_step()
        e1.record()
        torch.cuda.synchronize()
        e2e_ms = torch.tensor([e0.elapsed_time(e1) / e2e_steps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
        e2e_ms = e2e_ms.item()
        if sampler:
            sampler.stop()

    # ---- byte model and roofline (this rank's launches; all ranks do equal work) ----------------------
    corners = count_in_range_corners(cfg, packed)
    bm = byte_model(cfg, corners, B, qe - qb, N)
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    else:
        peak, peak_src = 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"
    achieved = bm["bwd_kernel"] / (bwd_ms * 1e-3) / 1e9
    roofline = {
        "bound": "hbm",
        "kernel": "backward pass = zero-fill + slab binning + fda_backward_binned_kernel + fda_backward_kernel (one C-ABI call)",
        "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
        "traffic": (NCU_BACKWARD_TRAFFIC_BYTES.get(args.config) if (world == 1 and not args.batch and not args.queries) else None),
        "traffic_source": "ncu capture of a 1/16-row case scaled x16 (profiles/), both backward kernels",
        "peak_source": peak_src, "algorithmic_bytes_per_launch": bm["bwd_kernel"], "ms_per_launch": bwd_ms,
        "fwd_kernel": {"achieved": bm["fwd"] / (fwd_ms * 1e-3) / 1e9, "frac": bm["fwd"] / (fwd_ms * 1e-3) / 1e9 / peak,
                       "algorithmic_bytes_per_launch": bm["fwd"], "ms_per_launch": fwd_ms},
        "whole_step": {"achieved": bm["fwd_bwd"] / (ms_per_step * 1e-3) / 1e9,
                       "frac": bm["fwd_bwd"] / (ms_per_step * 1e-3) / 1e9 / peak,
                       "frac_of_nominal_8TBs": bm["fwd_bwd"] / (ms_per_step * 1e-3) / 8e12},
        "points": bm["points"], "corners_in_range": bm["corners_in"],
    }

    if rank == 0:
        line = {
            "metric": METRIC, "value": B / (ms_per_step * 1e-3), "fwd_value": B / (fwd_ms * 1e-3), "unit": "samples/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "ms_fwd": fwd_ms, "ms_bwd_kernel": bwd_ms, "ms_reduce_and_cast": tail_ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16 value / f32 offsets, f32 accumulate" if cfg["vdt"] == "bfloat16" else "f32",
            "data": "synthetic",
            "config": {"workload": cfg["name"], "B": B, "Lq": Q, "N": N, "G": G, "D": D, "K": K, "levels": cfg["shapes"],
                       "sharding": (f"queries/{world}, value replicated, grad_value fp32 images summed by "
                                    + ("a fused peer-memory reduce+cast kernel overlapped per batch element" if use_peer
                                       else "NCCL all-reduce, then cast")) if world > 1 else "none",
                       "l2": "inputs larger than L2 (no flush needed)" if bm["fwd_bwd"] > 4e8 else "inputs smaller than L2",
                       **({"note": peer_note} if peer_note else {})},
            "roofline": roofline,
            "e2e": {"value": (B / (e2e_ms * 1e-3)) if e2e_ms else None, "unit": "samples/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms, "steps": e2e_steps},
            "gpu_launches": gpu_launches,
            "clocks": clocks,
        }
        if ref_cuda is not None:
            line["reference_cuda"] = ref_cuda
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_block(cfg)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", type=int, default=5, choices=sorted(CONFIGS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--reduce", default="peer", choices=["peer", "nccl"],
                    help="N > 1: how the fp32 grad_value images are summed (fused peer-memory kernel, or NCCL all-reduce + cast)")
    ap.add_argument("--batch", type=int, default=0, help="override B (smaller case for profiler captures)")
    ap.add_argument("--queries", type=int, default=0, help="override Lq (smaller case for profiler captures)")
    ap.add_argument("--ref-cuda", action="store_true",
                    help="also time the reference's own CUDA kernels (needs baseline/_ref/ops3d_ref_C.so; N=1)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (profiler captures)")
    args = ap.parse_args()
    cfg = dict(CONFIGS[args.config])
    if args.batch or args.queries:
        cfg["B"] = args.batch or cfg["B"]
        cfg["Q"] = args.queries or cfg["Q"]
        cfg["name"] += f" [reduced to B={cfg['B']}, Lq={cfg['Q']}]"
    if args.impl == "reference":
        run_reference_arm(args, cfg)
    else:
        args.warmup = max(args.warmup, 3)
        run_ours(args, cfg)


if __name__ == "__main__":
    main()
