"""Timings of the library's auxiliary kernels on their own (CUDA events, device-resident buffers):

    python -m ops3d_b200.microbench cast       fp32 accumulation image -> bf16 grad_value (fda_cast_kernel)
    python -m ops3d_b200.microbench pack       offsets + reference points + logits -> packed rows (fda_pack_kernel)
    python -m ops3d_b200.microbench prepass    slab sorting of the largest level (fda_bin_count / scan / fill kernels)
    python -m ops3d_b200.microbench project    the layer's query projections + packing: one GEMM that writes the packed
                                               tensor (project_and_pack) against two GEMMs + fda_pack_kernel
    python -m ops3d_b200.microbench dcnv4      DCNv4-3D forward + backward (3x3x3 stencil over a 32x64x64 volume, 8 groups x 32
                                               channels, fp16), and the reference's own kernels beside it when
                                               baseline/_ref/ops3d_ref_dcnv4.so has been built
    python -m ops3d_b200.microbench exchange   cross-GPU sum + cast (fda_peer_reduce_cast_kernel); a world of one
                                               on a single GPU, or under torch.distributed.run on several:
        python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
            --master-port P -m ops3d_b200.microbench exchange
    python -m ops3d_b200.microbench headpush   the head-sharded exchange (fda_head_slice_push_kernel): a compact fp32 image of
                                               2 of 8 heads converted and stored into the full gradient, a world of one

Sizes default to one rank's share of the largest benchmark configuration (256x512x2048 tile at strides
8/16/32, G=8, D=32, K=8); ``--mb`` sets the image size of ``cast`` / ``exchange`` / ``headpush``.  Each prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from . import capi

SHAPES5 = [(32, 64, 256), (16, 32, 128), (8, 16, 64)]


def _time(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def bench_cast(args, dev):
    n = int(args.mb * 1e6 / 4) // 8 * 8
    image = torch.randn(n, device=dev)
    out = torch.empty(n, dtype=torch.bfloat16, device=dev)
    ms = _time(lambda: capi.cast_grad_value(image, out), args.steps, args.warmup)
    return {"kernel": "fda_cast_kernel<bf16>", "elements": n, "ms": ms, "bytes": n * 6, "GBs": n * 6 / ms / 1e6}


def bench_pack(args, dev):
    B, Q, G, L, K = 1, args.queries, 8, 3, 8
    shapes = torch.tensor(SHAPES5, dtype=torch.long, device=dev)
    offsets = torch.randn(B, Q, G, L, K, 3, device=dev).bfloat16()
    ref = torch.rand(B, Q, L, 3, device=dev).bfloat16()
    logits = torch.randn(B, Q, G, L, K, device=dev).bfloat16()
    ms = _time(lambda: capi.pack_sampling(offsets, ref, logits, shapes), args.steps, args.warmup)
    nbytes = offsets.numel() * 2 + ref.numel() * 2 + logits.numel() * 2 + B * Q * G * L * K * 16
    return {"kernel": "fda_pack_kernel<bf16>", "rows": B * Q * G, "ms": ms, "bytes": nbytes, "GBs": nbytes / ms / 1e6}


def bench_prepass(args, dev):
    """The slab sorting of the largest level: slab group 0 of as many groups as there are slabs, i.e. the count,
    scan and fill kernels plus the binned kernel over a single slab."""
    B, Q, G, D, K, L = 1, args.queries, 8, 32, 8, 3
    shapes = torch.tensor(SHAPES5, dtype=torch.long, device=dev)
    sizes = shapes.prod(1)
    lsi = torch.cat((sizes.new_zeros(1), sizes.cumsum(0)[:-1]))
    N = int(sizes.sum())
    value = torch.randn(B, N, G, D, device=dev).bfloat16()
    packed = torch.empty(B, Q, G, L * K * 4, device=dev)
    packed[..., : L * K * 3] = torch.rand(B, Q, G, L * K * 3, device=dev) * 1.1 - 0.05
    packed[..., L * K * 3:] = torch.randn(B, Q, G, L * K, device=dev)
    grad_out = torch.randn(B, Q, G * D, device=dev).bfloat16()
    image = torch.zeros(B, N, G, D, device=dev)
    gp = torch.empty_like(packed)
    plan = capi.bin_plan(shapes.cpu(), value.shape, Q, K)
    if plan is None:
        return {"kernel": "fda_bin_*", "skipped": "binning does not apply to this problem"}
    scratch = torch.empty(capi.scratch_bytes(value, packed, K), dtype=torch.uint8, device=dev)
    slabs = plan[1]
    ms = _time(lambda: capi.backward_binned_part(value, shapes, lsi, packed, grad_out, K, image, gp, 0, slabs, 0, scratch),
               args.steps, args.warmup)
    return {"kernel": "fda_bin_count_kernel + fda_bin_scan_kernel + fda_bin_fill_kernel (+ 1 of %d slabs of the binned kernel)" % slabs,
            "rows": B * Q * G, "entries": B * Q * G * K, "ms": ms, "packed_bytes": packed.numel() * 4}


def bench_project(args, dev):
    """Forward of the part of ``MSDeformAttn3D`` that produces ``sampling_loc_attn`` from the queries, both ways."""
    from .msda3d import PackSamplingFunction, project_and_pack

    B, Q, C, G, L, K = 1, args.queries, 256, 8, 3, 8
    shapes = torch.tensor(SHAPES5, dtype=torch.long, device=dev)
    dt = torch.bfloat16
    query = torch.randn(B, Q, C, device=dev).to(dt)
    ref = torch.rand(B, Q, L, 3, device=dev)
    w_off = (torch.randn(G * L * K * 3, C, device=dev) * 0.05).to(dt)
    b_off = torch.randn(G * L * K * 3, device=dev).to(dt)
    w_log = (torch.randn(G * L * K, C, device=dev) * 0.05).to(dt)
    b_log = torch.randn(G * L * K, device=dev).to(dt)

    def fused():
        return project_and_pack(query, ref, w_off, b_off, w_log, b_log, shapes, G, K)

    def unfused():
        off = torch.nn.functional.linear(query, w_off, b_off).view(B, Q, G, L, K, 3)
        log = torch.nn.functional.linear(query, w_log, b_log).view(B, Q, G, L, K)
        return PackSamplingFunction.apply(off, ref, log, shapes)

    with torch.no_grad():
        a, b = fused(), unfused()
        err = (a - b).abs().max().item()   # the unfused path rounds offsets and logits to bf16 before packing
        ms_f = _time(fused, args.steps, args.warmup)
        ms_u = _time(unfused, args.steps, args.warmup)
    return {"what": "query projections + packing, bf16 in, fp32 packed out", "rows": B * Q * G, "packed_bytes": a.numel() * 4,
            "ms_fused_gemm": ms_f, "ms_two_gemms_plus_pack_kernel": ms_u, "speedup": ms_u / ms_f, "max_abs_difference": err}


def bench_dcnv4(args, dev):
    import importlib.util

    B, size_in, G, Dg, K = 2, (32, 64, 64), 8, 32, 27
    kernel, stride, pad, dilation = (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1)
    dt = torch.float16
    Q = size_in[0] * size_in[1] * size_in[2]
    padded = -(-(G * K * 4) // 8) * 8
    gen = torch.Generator(device=dev).manual_seed(0)
    value = torch.randn(B, *size_in, G * Dg, generator=gen, device=dev).to(dt)
    rows = torch.randn(B, *size_in, padded, generator=gen, device=dev).to(dt)
    grad_out = torch.randn(B, *size_in, G * Dg, generator=gen, device=dev).to(dt)
    cfg = (kernel, stride, pad, dilation, G, Dg, 1.0, 0, True)
    # The backward comparison runs with plain (not soft-maxed) masks: with soft-max and 32 % (Dg / d_stride) == 0 the
    # reference's backward_kernel_dcn_warp_primitive stores up to 2K floats past each group's mask slots
    # (csrc/cuda/dcnv4_col2im_cuda.cuh:520-533), past the end of grad_offset for the last cell -- it is not run here.
    cfg_b = cfg[:-1] + (False,)
    ms_f = _time(lambda: capi.dcnv4_forward(value, rows, *cfg), args.steps, args.warmup)
    ms_b = _time(lambda: capi.dcnv4_backward(value, rows, grad_out, *cfg_b), args.steps, args.warmup)
    ms_b_softmax = _time(lambda: capi.dcnv4_backward(value, rows, grad_out, *cfg), args.steps, args.warmup)
    points = B * Q * G * K
    gathered = points * 8 * Dg * 2           # upper bound: all 8 corners of every point in range
    res = {"kernel": "dcnv4_forward_kernel / dcnv4_backward_kernel<f16>", "points": points, "ms_forward": ms_f, "ms_backward": ms_b,
           "ms_backward_softmax": ms_b_softmax,
           "forward_gather_GBs": (gathered + rows.numel() * 2 + B * Q * G * Dg * 2) / ms_f / 1e6,
           "backward_gather_scatter_GBs": (gathered * 3 + 2 * rows.numel() * 2 + B * Q * G * Dg * 2) / ms_b / 1e6}
    lib = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref", "ops3d_ref_dcnv4.so")
    if os.path.exists(lib):
        try:
            spec = importlib.util.spec_from_file_location("ops3d_ref_dcnv4", lib)
            ref = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(ref)
            d_stride = 8
            block_thread = (Dg // d_stride) * G * 8   # 8 output cells per block (256 threads); Q is a multiple of 8
            rf = lambda: ref.dcnv4_forward(value, rows, *kernel, *stride, *pad, *dilation, G, Dg, 1.0, 64, 0, d_stride,  # noqa: E731
                                           block_thread, True)
            rb = lambda: ref.dcnv4_backward(value, rows, *kernel, *stride, *pad, *dilation, G, Dg, 1.0, 64, grad_out, 0,  # noqa: E731
                                            d_stride, block_thread, False)
            res["reference_ms_forward"] = _time(rf, args.steps, args.warmup)
            res["reference_ms_backward"] = _time(rb, args.steps, args.warmup)
            res["speedup_forward"] = res["reference_ms_forward"] / ms_f
            res["speedup_backward"] = res["reference_ms_backward"] / ms_b
        except Exception as exc:  # noqa: BLE001
            res["reference"] = f"unavailable: {type(exc).__name__}: {exc}"
    else:
        res["reference"] = "baseline/_ref/ops3d_ref_dcnv4.so not built (baseline/build_ref_cuda.sh <checkout> --dcnv4)"
    return res


def bench_exchange(args, dev, rank, world):
    import torch.distributed as dist

    n = int(args.mb * 1e6 / 4) // (8 * world) * (8 * world)
    if world == 1:
        image = torch.randn(n, device=dev)
        out = torch.empty(n, dtype=torch.bfloat16, device=dev)
        ms = _time(lambda: capi.peer_reduce_cast([image.data_ptr()], [out.data_ptr()], 0, n, torch.bfloat16, dev),
                   args.steps, args.warmup)
        return {"kernel": "fda_peer_reduce_cast_kernel<bf16, world 1>", "elements": n, "ms": ms, "bytes": n * 6,
                "GBs": n * 6 / ms / 1e6}
    import torch.distributed._symmetric_memory as symm_mem

    image = symm_mem.empty(n, dtype=torch.float32, device=dev)
    out = symm_mem.empty(n, dtype=torch.bfloat16, device=dev)
    h_image, h_out = symm_mem.rendezvous(image, dist.group.WORLD), symm_mem.rendezvous(out, dist.group.WORLD)
    image.normal_()
    img_ptrs, out_ptrs = [int(p) for p in h_image.buffer_ptrs], [int(p) for p in h_out.buffer_ptrs]

    def step():
        h_image.barrier(channel=0)
        capi.peer_reduce_cast(img_ptrs, out_ptrs, rank, n, torch.bfloat16, dev)
        h_out.barrier(channel=0)

    ms = torch.tensor([_time(step, args.steps, args.warmup)], device=dev, dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = ms.item()
    pulled = n * 4 * (world - 1) // world          # bytes this rank reads from its peers
    pushed = n * 2 * (world - 1) // world          # bytes this rank writes to its peers
    return {"kernel": f"barrier + fda_peer_reduce_cast_kernel<bf16, world {world}> + barrier", "elements": n, "ms": ms,
            "nvlink_in_bytes": pulled, "nvlink_out_bytes": pushed, "nvlink_in_GBs": pulled / ms / 1e6,
            "nvlink_out_GBs": pushed / ms / 1e6, "blocks": int(os.environ.get("FDA_PEER_REDUCE_BLOCKS", "32"))}


def bench_headpush(args, dev):
    """The head-sharded exchange in a world of one: a compact fp32 image of 2 of 8 heads, converted and stored into its
    place inside the full bf16 gradient (the kernel's stores are then all local)."""
    G, D, gr = 8, 32, 2
    cells = int(args.mb * 1e6 / 4) // (gr * D)
    image = torch.randn(cells, gr, D, device=dev)
    out = torch.zeros(cells, G, D, dtype=torch.bfloat16, device=dev)
    ms = _time(lambda: capi.head_slice_cast_push(image.data_ptr(), [out.data_ptr()], 0, 0, cells, gr * D, G * D, 3 * gr * D,
                                                 torch.bfloat16, dev), args.steps, args.warmup)
    n = image.numel()
    return {"kernel": "fda_head_slice_push_kernel<bf16, world 1>", "elements": n, "ms": ms, "bytes": n * 6, "GBs": n * 6 / ms / 1e6}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["cast", "pack", "prepass", "project", "dcnv4", "exchange", "headpush"])
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--mb", type=float, default=256.0, help="fp32 image size in MB (cast, exchange)")
    ap.add_argument("--queries", type=int, default=74752, help="queries of one batch element (pack, prepass)")
    args = ap.parse_args()
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    capi.load()
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    if args.what == "cast":
        res = bench_cast(args, dev)
    elif args.what == "pack":
        res = bench_pack(args, dev)
    elif args.what == "prepass":
        res = bench_prepass(args, dev)
    elif args.what == "project":
        res = bench_project(args, dev)
    elif args.what == "dcnv4":
        res = bench_dcnv4(args, dev)
    elif args.what == "headpush":
        res = bench_headpush(args, dev)
    else:
        res = bench_exchange(args, dev, rank, world)
    if rank == 0:
        print(json.dumps(res), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
