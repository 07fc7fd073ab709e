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
               max over ranks.  With N > 1 GPUs the (batch, query) rows are split over the ranks in
               batch-aligned ranges, value is replicated and the partial fp32 grad_value images are
               summed over NVLink before the cast -- total work is fixed, so scaling is "strong".
  e2e          same metric with HOST (pinned) inputs and outputs through the package's host-buffer
               entry point (ops3d_b200.host_stream): every step copies its inputs host->device and
               all results (out, grad_value, grad_packed) device->host inside the timed region,
               query chunk by query chunk, overlapped with the kernels.
  roofline     dominant kernels (backward scatter/gather): algorithmic bytes (gather model: rows
               gathered or scattered x row bytes) / CUDA-event time against the measured HBM copy
               bandwidth; the DRAM bytes an ncu capture measured are reported beside it.
  cpu_baseline the CPU oracle (PyTorch restatement of the reference's CPU implementation) timed on
               this machine's host cores on a bounded sample of the same workload (N=1 only); the
               same pass is compared with the GPU results of those rows ("parity").
  parity       N=1: GPU vs CPU oracle on the sampled rows; N>1: sharded result vs an unsharded
               recomputation on one GPU (all ranks agree on the verdict).  Outside the timed region.

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

CPU_SAMPLE_QUERIES = 65536  # fixed sample of the CPU arm: queries of one batch element against the full-size volume


def kernel_fingerprint():
    """Hash of the kernel sources: ties the DRAM-traffic figures in profiles/traffic.json to the code they
    were captured from."""
    import hashlib

    h = hashlib.sha256()
    csrc = os.path.join(ROOT, "ops3d_b200", "csrc")
    for name in sorted(os.listdir(csrc)):
        if name.startswith(("fda_backward", "fda_device", "fda_forward")):
            h.update(open(os.path.join(csrc, name), "rb").read())
    return h.hexdigest()[:16]


def measured_traffic(config_id):
    """DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per full-size backward of the configuration,
    from the ncu capture recorded in profiles/traffic.json -- None when there is none or when the kernel
    sources changed since it was taken."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    if not os.path.exists(path):
        return None, "no capture recorded"
    rec = json.load(open(path))
    entry = rec.get("configs", {}).get(str(config_id))
    if entry is None:
        return None, "no capture for this configuration"
    if rec.get("kernel_fingerprint") != kernel_fingerprint():
        return None, "kernel sources changed since the capture in profiles/traffic.json"
    return float(entry["backward_dram_bytes_per_launch"]), entry.get("how", "")


# ---------------------------------------------------------------------------------------------
# synthetic inputs
# ---------------------------------------------------------------------------------------------
def make_device_inputs(cfg, dev, part, seed=0):
    """Seeded inputs of the configuration's shapes and distributions, generated on the device.
    Every rank generates the same full ``value`` (replicated) and the rows of its own partition
    ``[part.b_begin:part.b_end, part.q_begin:part.q_end]`` (of its own heads only under a head split)."""
    vdt = getattr(torch, cfg["vdt"])
    shapes = torch.tensor(cfg["shapes"], dtype=torch.long, device=dev)
    sizes = shapes.prod(1)
    lsi = torch.cat((sizes.new_zeros(1), sizes.cumsum(0)[:-1]))
    N = int(sizes.sum())
    B, G, D, K, L = cfg["B"], cfg["G"], cfg["D"], cfg["K"], len(cfg["shapes"])
    nb, Qr = part.b_end - part.b_begin, part.q_end - part.q_begin
    gen = torch.Generator(device=dev).manual_seed(seed)
    value = torch.randn(B, N, G, D, generator=gen, device=dev, dtype=torch.float32).to(vdt)
    gen_q = torch.Generator(device=dev).manual_seed(seed * 1000 + 17 + part.q_begin + 7919 * part.b_begin + 104729 * part.h_begin)
    if part.splits_heads:
        G = part.h_end - part.h_begin   # rows of this rank's heads
    packed = torch.empty(nb, Qr, G, L * K * 4, device=dev, dtype=torch.float32)
    loc = packed[..., : L * K * 3]
    if cfg["coords"] == "uniform":
        loc.copy_(torch.rand(nb, Qr, G, L * K * 3, generator=gen_q, device=dev) * 1.1 - 0.05)
    else:
        centre = torch.rand(nb, Qr, 1, 1, 3, generator=gen_q, device=dev)
        pts = centre + 0.05 * torch.randn(nb, Qr, G, L * K, 3, generator=gen_q, device=dev)
        loc.copy_(pts.clamp_(-0.05, 1.05).reshape(nb, Qr, G, L * K * 3))
    packed[..., L * K * 3:].copy_(torch.randn(nb, Qr, G, L * K, generator=gen_q, device=dev))
    grad_out = torch.randn(nb, Qr, G * D, generator=gen_q, device=dev, dtype=torch.float32).to(vdt)
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
# CPU baseline / reference arm: the CPU oracle on host cores, fixed bounded sample
# ---------------------------------------------------------------------------------------------
def config_block(cfg):
    """The workload description; identical in both arms."""
    N = sum(d * h * w for d, h, w in cfg["shapes"])
    return {"workload": cfg["name"], "B": cfg["B"], "Lq": cfg["Q"], "N": N, "G": cfg["G"], "D": cfg["D"], "K": cfg["K"],
            "levels": [list(s) for s in cfg["shapes"]],
            "value_dtype": cfg["vdt"], "offsets_dtype": "float32",
            "l2": "inputs larger than L2 (no flush between iterations)" if cfg["B"] * cfg["Q"] * cfg["G"] * len(cfg["shapes"]) * cfg["K"] * 16 > 2.6e8
                  else "inputs smaller than L2 (warm numbers; latency configuration)"}


def cpu_sample_inputs(cfg, sample_q, seed=0):
    """Inputs of the CPU arm when it runs alone: one batch element, ``sample_q`` queries, full-size volume."""
    from oracle import fda_oracle

    value, sh, lsi, packed, grad_out = fda_oracle.make_inputs(
        cfg["shapes"], 1, sample_q, cfg["G"], cfg["D"], cfg["K"], seed=seed, coords=cfg["coords"])
    if cfg["vdt"] != "float32":
        value = value.to(getattr(torch, cfg["vdt"])).float()
        grad_out = grad_out.to(getattr(torch, cfg["vdt"])).float()
    return value, sh, packed, grad_out


def cpu_reference_pass(value, sh, packed, grad_out, K, steps, warmup):
    """Best seconds per pass (fwd, fwd+bwd) of the CPU oracle on all host threads, after ``warmup`` untimed
    passes; also returns the results of the last fwd+bwd pass (used as the parity check's reference)."""
    from oracle import fda_oracle

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    t_f, t_fb, res = [], [], None
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        fda_oracle.fused_forward(value, sh, packed, K, chunk=packed.shape[1])
        t1 = time.perf_counter()
        res = fda_oracle.fused_forward_backward(value, sh, packed, grad_out, K, chunk=packed.shape[1])
        t2 = time.perf_counter()
        if i >= warmup:
            t_f.append(t1 - t0)
            t_fb.append(t2 - t1)
    return min(t_f), min(t_fb), cores, res


def cpu_block(cfg, sample_q, tf, tfb, cores):
    scale = sample_q / cfg["Q"]  # fraction of one sample (= one batch element) a pass covered
    return {
        "value": scale / tfb, "fwd_value": scale / tf, "unit": "samples/s", "cores": cores, "kind": "port",
        "sample": f"{sample_q} of {cfg['Q']} queries of one batch element against the full-size value volume, fp32, "
                  f"torch {torch.__version__} CPU, one untimed warm-up pass, linear extrapolation to a whole sample; "
                  f"fwd+bwd {tfb:.3f} s, fwd {tf:.3f} s",
    }


def run_reference_arm(args, cfg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample_q = min(cfg["Q"], CPU_SAMPLE_QUERIES)
    value, sh, packed, grad_out = cpu_sample_inputs(cfg, sample_q)
    tf, tfb, cores, _ = cpu_reference_pass(value, sh, packed, grad_out, cfg["K"], max(1, args.steps), max(1, args.warmup))
    block = cpu_block(cfg, sample_q, tf, tfb, cores)
    line = {
        "impl": "reference", "metric": METRIC, "value": block["value"], "fwd_value": block["fwd_value"],
        "unit": "samples/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": cfg["B"] / block["value"] * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": config_block(cfg),
        "cpu_baseline": block,
        "e2e": {"value": block["value"], "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# the reference's own CUDA kernels on this GPU (reported baseline; needs baseline/_ref/)
# ---------------------------------------------------------------------------------------------
def reference_cuda_block(cfg, value, shapes, lsi, packed, grad_out, steps=5, warmup=2):
    """Times the unmodified reference kernels (built by baseline/build_ref_cuda.sh) on the same inputs.
    They only take offsets/logits in the value dtype, so ``packed`` is cast to it first."""
    import importlib.util

    so = os.path.join(ROOT, "baseline", "_ref", "ops3d_ref_C.so")
    if not os.path.exists(so):
        return {"unavailable": "baseline/_ref/ops3d_ref_C.so not built (baseline/build_ref_cuda.sh <reference checkout>)"}
    try:
        spec = importlib.util.spec_from_file_location("ops3d_ref_C", so)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    except Exception as exc:  # noqa: BLE001  (built for another torch / python)
        return {"unavailable": f"baseline/_ref/ops3d_ref_C.so does not load: {type(exc).__name__}: {exc}"}
    B, Q, G, D, K = cfg["B"], packed.shape[1], cfg["G"], cfg["D"], cfg["K"]
    pk = packed.to(value.dtype)
    # launch hints as the reference's findspec / findspec_bwd return them
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
# parity checks (outside the timed region)
# ---------------------------------------------------------------------------------------------
def _max_err(got, ref):
    return (got.double().cpu() - ref.double().cpu()).abs().max().item()


def parity_vs_oracle(cfg, capi, value, shapes, lsi, packed, grad_out, out, grad_packed, sample_q):
    """N = 1: the CPU oracle on the first ``sample_q`` queries of batch element 0 against the full-size
    volume.  ``out`` / ``grad_packed`` rows are taken from the full-size launch (rows are independent);
    ``grad_value`` from a launch over exactly the sampled rows.  Returns (parity block, cpu_baseline block)."""
    K, LK = cfg["K"], len(cfg["shapes"]) * cfg["K"]
    v1, pk, go = value[:1], packed[:1, :sample_q].contiguous(), grad_out[:1, :sample_q].contiguous()
    gv_gpu, gp_sub = capi.backward(v1, shapes, lsi, pk, go, K)
    torch.cuda.synchronize()
    same_rows = bool(torch.equal(gp_sub, grad_packed[:1, :sample_q]))  # the rows do not depend on which launch held them
    tf, tfb, cores, (ref_out, ref_gv, ref_gp) = cpu_reference_pass(
        v1.float().cpu(), shapes.cpu(), pk.float().cpu(), go.float().cpu(), K, steps=1, warmup=1)
    tol = 1e-4 if cfg["vdt"] == "float32" else 2e-2
    checks = {
        "out": (_max_err(out[:1, :sample_q], ref_out), ref_out.abs().max().item()),
        "grad_value": (_max_err(gv_gpu, ref_gv), ref_gv.abs().max().item()),
        "grad_coords": (_max_err(grad_packed[:1, :sample_q, :, : 3 * LK], ref_gp[..., : 3 * LK]), ref_gp[..., : 3 * LK].abs().max().item()),
        "grad_logits": (_max_err(grad_packed[:1, :sample_q, :, 3 * LK:], ref_gp[..., 3 * LK:]), ref_gp[..., 3 * LK:].abs().max().item()),
    }
    ok = all(e <= tol * max(1.0 if cfg["vdt"] == "float32" else 1e-30, m) for e, m in checks.values())
    parity = {"ok": bool(ok), "against": "CPU oracle (PyTorch restatement of the reference's CPU implementation)",
              "rows": f"first {sample_q} queries of batch element 0, full-size volume; grad_value from a launch over those rows",
              "tolerance": f"{tol} x |ref|max" if cfg["vdt"] != "float32" else "1e-4 x max(1, |ref|max)",
              "max_abs": {k: e for k, (e, _) in checks.items()}, "ref_max": {k: m for k, (_, m) in checks.items()},
              "rows_identical_across_launches": same_rows}
    return parity, cpu_block(cfg, sample_q, tf, tfb, cores)


def parity_vs_unsharded(cfg, capi, dist, part, value, shapes, lsi, packed, grad_out, out, grad_value, grad_packed):
    """N > 1: every rank gathers all ranks' rows, recomputes the whole step unsharded on its own GPU and
    compares its out / grad_packed rows (exactly) and the reduced grad_value (2e-2 of the largest magnitude)."""
    K = cfg["K"]
    world = dist.get_world_size()
    B, Q, G, D = cfg["B"], cfg["Q"], cfg["G"], cfg["D"]
    nb, Qr = packed.shape[0], packed.shape[1]
    sizes = torch.tensor([nb, Qr], device=value.device)
    lo, hi = sizes.clone(), sizes.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN); dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    if not torch.equal(lo, hi):
        return {"ok": None, "skipped": "ranks hold different row counts; gather not implemented for ragged shards"}

    def gather_full(t):
        parts = torch.empty((world,) + tuple(t.shape), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(parts, t.contiguous())
        if part.kind == "queries":       # [R, B, Qr, ...] -> [B, R*Qr, ...]
            return parts.transpose(0, 1).reshape(B, world * Qr, *t.shape[2:]).contiguous()
        if part.kind == "batch-heads":   # [B * size, 1, Q, Gr(, ...)] -> [B, Q, size * Gr(, ...)]: rank order is head order
            size, gr = world // B, part.h_end - part.h_begin
            per_head = t.shape[2:] if t.dim() == 4 else (gr, t.shape[2] // gr)   # [.., Gr, X] or [.., Gr*D]
            full = parts.reshape(B, size, Q, *per_head).transpose(1, 2).reshape(B, Q, size * gr, *per_head[1:])
            return (full if t.dim() == 4 else full.reshape(B, Q, -1)).contiguous()
        return parts.reshape(B, Q, *t.shape[2:])  # batch / batch-groups: rank order is row order

    pk_full, go_full = gather_full(packed), gather_full(grad_out)
    out_ref = capi.forward(value, shapes, lsi, pk_full, K)
    gv_ref, gp_ref = capi.backward(value, shapes, lsi, pk_full, go_full, K)
    torch.cuda.synchronize()
    from ops3d_b200.sharded import shard_rows
    tol = 1e-4 if cfg["vdt"] == "float32" else 2e-2
    errs, scales = {}, {}
    for name, got, ref in (("out_rows", out, shard_rows(out_ref, part, G)), ("grad_packed_rows", grad_packed, shard_rows(gp_ref, part, G)),
                           ("grad_value", grad_value, gv_ref)):
        errs[name] = (got.float() - ref.float()).abs().max().item()
        scales[name] = ref.float().abs().max().item()
    ok = all(errs[k] <= tol * max(scales[k], 1e-30) for k in errs)
    keys = sorted(errs)
    stats = torch.tensor([0.0 if ok else 1.0] + [errs[k] for k in keys] + [scales[k] for k in keys],
                         device=value.device, dtype=torch.float64)
    dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    stats = stats.tolist()
    errs = dict(zip(keys, stats[1:1 + len(keys)]))
    scales = dict(zip(keys, stats[1 + len(keys):]))
    return {"ok": stats[0] == 0.0, "against": "unsharded recomputation of the whole step on each rank's own GPU",
            "max_abs": errs, "ref_max": scales, "rows_bit_equal": errs["out_rows"] == 0.0 and errs["grad_packed_rows"] == 0.0,
            "tolerance": f"{tol} x |ref|max per tensor (rows are expected to be bit-equal, grad_value to differ by summation order)",
            "ranks_checked": world}


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def run_ours(args, cfg):
    import torch.distributed as dist

    from ops3d_b200 import capi
    from ops3d_b200.host_stream import HostStreamedStep
    from ops3d_b200.sharded import PeerReducer, partition, shard_value

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
    part = partition(B, Q, rank, world, num_heads=G)
    nb, Qr = part.b_end - part.b_begin, part.q_end - part.q_begin
    Gr = (part.h_end - part.h_begin) if part.splits_heads else G   # heads of this rank's rows
    value, shapes, lsi, packed, grad_out = make_device_inputs(cfg, dev, part)
    value_local = shard_value(value, part)
    N = value.shape[1]
    vdt = value.dtype
    out = torch.empty(nb, Qr, Gr * D, dtype=vdt, device=dev)
    grad_packed = torch.empty_like(packed)
    use_peer = world > 1 and args.reduce == "peer"
    reducer, peer_note = None, None
    if use_peer:
        # symmetric-memory set-up can be unavailable on a machine (no peer access): all ranks agree, then
        # either all use the fused exchange or all fall back to NCCL all-reduce + cast
        try:
            reducer = PeerReducer(value.shape, vdt, dev, spatial_shapes=shapes, part=part)
            ok = torch.ones(1, device=dev)
        except Exception as exc:  # noqa: BLE001
            peer_note = f"peer exchange unavailable ({type(exc).__name__}: {exc}); NCCL all-reduce used"
            ok = torch.zeros(1, device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if ok.item() == 0:
            reducer, use_peer = None, False
            peer_note = peer_note or "peer exchange unavailable on another rank; NCCL all-reduce used"
    L = len(cfg["shapes"])
    # which backward the library takes for this rank's rows (it works batch element by batch element under the reducer)
    bwd_path = capi.backward_path(value_local[:1] if use_peer else value_local, packed[:1] if use_peer else packed, K)
    fwd_heads = capi.forward_head_group(value_local, packed, K)   # heads per group of the forward's row order
    # a step on one GPU follows fda_backward's own choice between the dense and the sparse handling of the fp32 image
    touched = world == 1 and vdt != torch.float32 and capi.backward_touched_rows(value_local, packed, K)
    grad_value = accum = scratch = accum_heads = None
    if not use_peer:
        n_scratch = capi.scratch_bytes(value_local, packed, K)
        scratch = torch.empty(n_scratch, dtype=torch.uint8, device=dev) if n_scratch else None
        grad_value = torch.empty_like(value)
        accum = torch.empty(value.shape, dtype=torch.float32, device=dev) if (vdt != torch.float32 or world > 1) else grad_value
        accum_heads = torch.empty(value_local.shape, dtype=torch.float32, device=dev) if part.splits_heads else None

    def phase_forward():
        # under a head split the compact copy of this rank's heads is part of the step (value changes every step)
        capi.forward(shard_value(value, part) if part.splits_heads else value_local, shapes, lsi, packed, K, out=out)

    def phase_backward():
        nonlocal grad_value
        if use_peer:
            # scatter on this stream, fused NVLink reduce+cast of finished pieces overlapped on a side stream
            grad_value, _ = reducer.backward(value, shapes, lsi, packed, grad_out, K, grad_packed=grad_packed)
            return
        if world > 1:
            accum.zero_()   # the batch elements other ranks work on contribute zeros to the sum
        if part.splits_heads:   # NCCL fallback under a head split: compact image, placed into the full one for the all-reduce
            capi.backward_accumulate_levels(shard_value(value, part), shapes, lsi, packed, grad_out, K, accum_heads, grad_packed,
                                            0, L, capi.BWD_ZERO_IMAGE | capi.BWD_FINALIZE, scratch=scratch)
            accum[part.b_begin:part.b_end, :, part.h_begin:part.h_end] = accum_heads
            return
        zero = 0 if world > 1 else (capi.BWD_ZERO_TOUCHED if touched else capi.BWD_ZERO_IMAGE)
        capi.backward_accumulate_levels(value_local, shapes, lsi, packed, grad_out, K, accum[part.b_begin:part.b_end],
                                        grad_packed, 0, L, zero | capi.BWD_FINALIZE, scratch=scratch)

    def phase_tail():
        if use_peer:
            return
        if world > 1:
            dist.all_reduce(accum)
        if touched:
            capi.cast_grad_value_touched(accum, grad_value, shapes, lsi, packed, K)
        elif accum is not grad_value:
            capi.cast_grad_value(accum, grad_value)

    phases = [phase_forward, phase_backward, phase_tail]

    def step(ev=None):
        for i, phase in enumerate(phases):
            if ev: ev[i].record()
            phase()
        if ev: ev[3].record()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()

    # Launch-bound configurations (a step of a few launches that each take microseconds) are replayed from CUDA
    # graphs, so that the device time is measured rather than the Python call overhead between launches.
    use_graph = world == 1 and (args.graph == "on" or (args.graph == "auto" and args.config in (1, 2, 3)))
    launches_per_step = None
    whole_graph = None
    if use_graph:
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            step()   # once more on the capture stream's side, so nothing is initialised during capture
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize()
        n0 = capi.KERNEL_LAUNCHES
        graphs = []
        for phase in phases:
            before = capi.KERNEL_LAUNCHES
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                phase()
            graphs.append(g if capi.KERNEL_LAUNCHES > before else None)  # a phase without launches (no cast for fp32)
        launches_per_step = capi.KERNEL_LAUNCHES - n0
        whole_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(whole_graph):
            for phase in (phase_forward, phase_backward, phase_tail):
                phase()
        phases = [(g.replay if g is not None else (lambda: None)) for g in graphs]
        for _ in range(3):
            step(); whole_graph.replay()
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
    total_ms = events[0][0].elapsed_time(events[-1][3])
    if whole_graph is not None:   # the step as ONE graph, replayed back to back: the step time proper
        w0, w1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0.record()
        for _ in range(args.steps):
            whole_graph.replay()
        w1.record()
        torch.cuda.synchronize()
        total_ms = w0.elapsed_time(w1)
    t_host1 = time.perf_counter()
    gpu_launches = capi.KERNEL_LAUNCHES - launches0 if launches_per_step is None else launches_per_step * args.steps
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    per_step = sorted(e[0].elapsed_time(e[3]) for e in events)   # each step on its own (launch gaps between steps excluded)
    step_median, step_min = statistics.median(per_step), per_step[0]
    fwd_ms = sum(e[0].elapsed_time(e[1]) for e in events) / args.steps
    bwd_ms = sum(e[1].elapsed_time(e[2]) for e in events) / args.steps
    tail_ms = sum(e[2].elapsed_time(e[3]) for e in events) / args.steps
    clocks = sampler.window(t_host0, t_host1) if sampler else None

    times = torch.tensor([total_ms, fwd_ms, bwd_ms, tail_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    total_ms, fwd_ms, bwd_ms, tail_ms = times.tolist()
    ms_per_step = total_ms / args.steps

    # ---- parity and baselines, outside the timed region ----------------------------------------------
    parity, cpu_baseline, ref_cuda = None, None, None
    if not args.no_parity:
        if world > 1:
            parity = parity_vs_unsharded(cfg, capi, dist, part, value, shapes, lsi, packed, grad_out, out, grad_value, grad_packed)
        elif not args.no_cpu_baseline:
            parity, cpu_baseline = parity_vs_oracle(cfg, capi, value, shapes, lsi, packed, grad_out, out, grad_packed,
                                                    min(Q, CPU_SAMPLE_QUERIES))
    if world == 1 and not args.no_ref_cuda:
        try:
            ref_cuda = reference_cuda_block(cfg, value, shapes, lsi, packed, grad_out)
        except Exception as exc:  # noqa: BLE001  (a reported baseline must not take the bench down)
            ref_cuda = {"unavailable": f"{type(exc).__name__}: {exc}"}

    # ---- byte model and roofline (this rank's launches; all ranks do equal work) ----------------------
    corners = count_in_range_corners(cfg, packed)
    bm = byte_model(dict(cfg, G=Gr), corners, nb, Qr, N)

    # ---- end to end: host buffers in, host buffers out, through the package's host-buffer entry point -
    e2e_ms, h2d, d2h, e2e_steps = None, 0, 0, 0
    if not args.no_e2e:
        e2e_steps = max(2, min(args.steps, 5))
        if part.splits_heads:
            # the host-buffer step streams query chunks: it runs on the query split of the batch groups, with rows and a
            # reducer of its own
            part_e = partition(B, Q, rank, world, mode="rows")
            del packed, grad_out, out, grad_packed
            _, _, _, packed, grad_out = make_device_inputs(cfg, dev, part_e)
            out = torch.empty(packed.shape[0], packed.shape[1], G * D, dtype=vdt, device=dev)
            grad_packed = None
            reducer = PeerReducer(value.shape, vdt, dev, spatial_shapes=shapes, part=part_e) if use_peer else None
        host_value = value.cpu().pin_memory()
        host_packed, host_go = packed.cpu().pin_memory(), grad_out.cpu().pin_memory()
        host_out = torch.empty(out.shape, dtype=out.dtype).pin_memory()
        host_gv = torch.empty(value.shape, dtype=vdt).pin_memory()
        host_gp = torch.empty(packed.shape, dtype=packed.dtype).pin_memory()
        del out, grad_value, grad_packed, accum, scratch, value, value_local, packed, grad_out, accum_heads
        torch.cuda.empty_cache()
        streamed = HostStreamedStep(host_value.shape, vdt, host_packed.shape, host_packed.dtype, K, shapes, lsi, dev,
                                    reducer=reducer)

        def e2e_step():
            streamed.run(host_value, host_packed, host_go, host_out, host_gv, host_gp)

        for _ in range(2):
            e2e_step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches_e2e0 = capi.KERNEL_LAUNCHES
        e0.record()
        for _ in range(e2e_steps):
            e2e_step()
        e1.record()
        torch.cuda.synchronize()
        e2e_launches = (capi.KERNEL_LAUNCHES - launches_e2e0) // e2e_steps
        h2d, d2h = streamed.h2d_bytes, streamed.d2h_bytes
        e2e_t = torch.tensor([e0.elapsed_time(e1) / e2e_steps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
        e2e_ms = e2e_t.item()
    if sampler:
        sampler.stop()

    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    else:
        peak, peak_src = 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"
    achieved = bm["bwd_kernel"] / (bwd_ms * 1e-3) / 1e9
    traffic, traffic_how = (measured_traffic(args.config) if (world == 1 and not args.batch and not args.queries and not args.half_volume)
                            else (None, "captured for the full single-GPU launch only"))
    roofline = {
        "bound": "hbm",
        "kernel": "backward pass (one C-ABI call) = " + ("fda_touch_rows_kernel (zeroes the image rows the points touch) + "
                                                         if touched else "zero-fill + ") + {
            2: "cell sort (fda_sort_pass_kernel count / fill, fda_scan_*) + fda_sorted_walk_kernel + fda_sort_finalize_kernel",
            1: "slab binning + fda_backward_binned_kernel + fda_backward_kernel",
            0: "fda_backward_kernel"}[bwd_path],
        "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
        "model": "gather model: every in-range corner row gathered (value dtype) and scattered (fp32) counts, plus the streamed "
                 "rows; part of it is served by L2 -- and the cell-sorted backward gathers and scatters once per run of points "
                 "in the same cell, not once per point -- so frac can exceed 1; dram_frac is the measured DRAM share",
        "traffic": traffic, "traffic_source": traffic_how,
        "dram_achieved": (traffic / (bwd_ms * 1e-3) / 1e9) if traffic else None,
        "dram_frac": (traffic / (bwd_ms * 1e-3) / 1e9 / peak) if traffic else None,
        "peak_source": peak_src, "algorithmic_bytes_per_launch": bm["bwd_kernel"], "ms_per_launch": bwd_ms,
        "fwd_kernel": {"achieved": bm["fwd"] / (fwd_ms * 1e-3) / 1e9, "frac": bm["fwd"] / (fwd_ms * 1e-3) / 1e9 / peak,
                       "algorithmic_bytes_per_launch": bm["fwd"], "ms_per_launch": fwd_ms,
                       "row_order": ("query by query" if fwd_heads >= Gr else f"head groups of {fwd_heads} (value rows of a group stay in L2)")},
        "whole_step": {"achieved": bm["fwd_bwd"] / (ms_per_step * 1e-3) / 1e9,
                       "frac": bm["fwd_bwd"] / (ms_per_step * 1e-3) / 1e9 / peak,
                       "frac_of_nominal_8TBs": bm["fwd_bwd"] / (ms_per_step * 1e-3) / 8e12},
        "points": bm["points"], "corners_in_range": bm["corners_in"],
    }

    if rank == 0:
        sharding = "none"
        if world > 1:
            how = {"batch": f"{nb} whole batch element(s) per rank (no cross-rank sum; finished images cast and broadcast)",
                   "batch-groups": f"{len(part.group)} ranks per batch element split its queries; partial fp32 images summed within the group",
                   "batch-heads": f"{len(part.group)} ranks per batch element split its heads ({Gr} each): no sum, every rank "
                                  "converts its finished slice of the image and stores it into every rank's grad_value",
                   "queries": f"queries of every batch element split over all {world} ranks"}[part.kind]
            sharding = (how + ", value replicated; exchange = " +
                        (("peer-memory cast+broadcast kernel" if part.splits_heads else "fused peer-memory reduce+cast kernel")
                         + " pipelined with the backward kernels" if use_peer else "NCCL all-reduce, then cast"))
        line = {
            "metric": METRIC, "value": B / (ms_per_step * 1e-3), "fwd_value": B / (fwd_ms * 1e-3), "unit": "samples/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "ms_per_step_median": step_median, "ms_per_step_min": step_min,   # rank 0's own steps
            "ms_fwd": fwd_ms, "ms_bwd_kernel": bwd_ms, "ms_reduce_and_cast": tail_ms,
            "grad_image": ("touched rows only (zeroed and converted from the point list)" if touched
                           else "none (fp32 value accumulates in grad_value)" if vdt == torch.float32 else "dense zero-fill and cast"),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16 value / f32 offsets, f32 accumulate" if cfg["vdt"] == "bfloat16" else "f32",
            "data": "synthetic", "config": config_block(cfg), "sharding": sharding,
            "roofline": roofline,
            "e2e": {"value": (B / (e2e_ms * 1e-3)) if e2e_ms else None, "unit": "samples/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": e2e_steps,
                    "how": "HostStreamedStep: query chunks double-buffered over upload / compute / download streams"
                           + ("; bytes are this rank's (each rank uploads its rows and its batch element(s) of value, "
                              "downloads its rows and 1/N of grad_value)" if world > 1 else "")},
            "gpu_launches": gpu_launches,
            "launch": ("CUDA graph replay (ms_per_step: the whole step as one graph; per-phase times: one graph per phase)"
                       if use_graph else "one C-ABI call per phase from Python"),
            "clocks": clocks,
        }
        if peer_note:
            line["note"] = peer_note
        if parity is not None:
            line["parity"] = parity
        if ref_cuda is not None:
            line["reference_cuda"] = ref_cuda
        if cpu_baseline is not None:
            line["cpu_baseline"] = cpu_baseline
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if parity is not None and parity.get("ok") is False:
        raise SystemExit("parity check failed: " + json.dumps(parity))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", type=int, default=5, choices=sorted(CONFIGS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU oracle pass (and with it the N=1 parity block)")
    ap.add_argument("--no-parity", action="store_true", help="skip the parity checks")
    ap.add_argument("--reduce", default="peer", choices=["peer", "nccl"],
                    help="N > 1: how the fp32 grad_value images are summed (fused peer-memory kernel, or NCCL all-reduce + cast)")
    ap.add_argument("--batch", type=int, default=0, help="override B (smaller case for profiler captures)")
    ap.add_argument("--queries", type=int, default=0, help="override Lq (smaller case for profiler captures)")
    ap.add_argument("--half-volume", action="store_true",
                    help="halve every level extent and scale Lq with the cells (1/8 of the volume and of the rows, the same "
                         "sampling points per cell): smaller case for profiler captures of the cell-sorted backward")
    ap.add_argument("--no-ref-cuda", action="store_true",
                    help="do not time the reference's own CUDA kernels (timed by default at N=1 when baseline/_ref/ops3d_ref_C.so exists)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (profiler captures)")
    ap.add_argument("--graph", default="auto", choices=["auto", "on", "off"],
                    help="replay the step from CUDA graphs (auto: the launch-bound configurations 1-3, one GPU)")
    args = ap.parse_args()
    cfg = dict(CONFIGS[args.config])
    if args.half_volume:
        cells = sum(d * h * w for d, h, w in cfg["shapes"])
        cfg["shapes"] = [tuple(max(1, v // 2) for v in shp) for shp in cfg["shapes"]]
        small = sum(d * h * w for d, h, w in cfg["shapes"])
        cfg["Q"] = max(1, cfg["Q"] * small // cells)
        cfg["name"] += f" [every level extent halved, Lq={cfg['Q']}]"
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
