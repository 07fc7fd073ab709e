"""GPU checks of the multi-GPU pieces: the peer-memory reduce+cast kernel (degenerate world of one on a
single GPU) and, where two GPUs are visible, the query-sharded operator over NCCL / NVLink peer memory
against the unsharded operator."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import fda_oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_peer_reduce_cast_world_of_one_is_a_cast(dtype):
    from ops3d_b200 import capi

    image = torch.randn(3, 50, 4, 16, device="cuda")
    out = torch.empty(image.shape, dtype=dtype, device="cuda")
    capi.peer_reduce_cast([image.data_ptr()], [out.data_ptr()], 0, image.numel(), dtype, image.device)
    torch.cuda.synchronize()
    assert torch.equal(out, image.to(dtype))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_head_slice_cast_push_world_of_one_places_the_slice(dtype):
    """The head-sharded exchange on one GPU: a compact fp32 image of heads [2, 5) lands, converted, in its place
    inside the full gradient; cells outside the range and the other heads stay untouched."""
    from ops3d_b200 import capi

    cells, G, D, h0, h1 = 37, 8, 16, 2, 5
    image = torch.randn(cells, h1 - h0, D, device="cuda")
    out = torch.full((cells, G, D), 7.0, dtype=dtype, device="cuda")
    capi.head_slice_cast_push(image.data_ptr(), [out.data_ptr()], 0, 3, 30, (h1 - h0) * D, G * D, h0 * D, dtype, image.device)
    torch.cuda.synchronize()
    expect = torch.full((cells, G, D), 7.0, dtype=dtype, device="cuda")
    expect[3:33, h0:h1] = image[3:33].to(dtype)
    assert torch.equal(out, expect)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mode, batch, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      FDA_SHARDED_REDUCE="nccl" if mode in ("nccl", "heads-nccl") else "peer",
                      FDA_PEER_REDUCE_MODE=mode if mode in ("p2p", "push", "multimem") else "auto",
                      # the multicast and posted-store exchanges sum over all ranks: they need every rank on every image
                      FDA_PARTITION="queries" if mode in ("push", "multimem", "queries") else "auto")
    if mode in ("slab-pipeline", "heads-slabs"):  # force the slab-binned backward and its slab-group exchange on this small problem
        os.environ.update(FDA_L2_KEEP_FRACTION="0.00001", FDA_BIN_SLAB_MB="0.25", FDA_SLAB_PARTS="3")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from ops3d_b200 import FlashDeformAttnFunction, capi
        from ops3d_b200.sharded import partition, shard_rows, sharded_flash_deform_attn

        capi.reload_config()
        shapes = [(8, 16, 32), (4, 8, 16)]
        K = 4
        value, sh, lsi, packed, grad_out = fda_oracle.make_inputs(shapes, batch, 301, 8, 32, K, seed=31)
        G = 8
        part = partition(batch, 301, rank, world, num_heads=G if mode.startswith("heads") else None)
        sh, lsi = sh.to(dev), lsi.to(dev)
        ok = True
        for step in range(2):  # twice: buffers of the first backward are reused by the second
            v = value.to(dev, torch.bfloat16).requires_grad_(True)
            pk = shard_rows(packed, part).to(dev).requires_grad_(True)
            out = sharded_flash_deform_attn(v, sh, lsi, pk, 64, K, None, None, part)
            out.backward(shard_rows(grad_out, part, G).to(dev, torch.bfloat16))
            v1 = value.to(dev, torch.bfloat16).requires_grad_(True)
            pk1 = packed.to(dev).requires_grad_(True)
            out1 = FlashDeformAttnFunction.apply(v1, sh, lsi, pk1, 64, K, True)
            out1.backward(grad_out.to(dev, torch.bfloat16))
            torch.cuda.synchronize()
            scale = v1.grad.float().abs().max().item()
            ok &= torch.equal(out, shard_rows(out1, part, G))
            ok &= (v.grad.float() - v1.grad.float()).abs().max().item() <= 2e-2 * scale
            ok &= torch.equal(pk.grad, shard_rows(pk1.grad, part))
        # and against the CPU oracle, so the check does not rest on the single-GPU path alone
        _, ref_gv, _ = fda_oracle.fused_forward_backward(value.bfloat16(), sh.cpu(), packed, grad_out.bfloat16(), K)
        ok &= (v.grad.float().cpu() - ref_gv).abs().max().item() <= 2e-2 * ref_gv.abs().max().item()
        ret[rank] = (bool(ok), part.kind)
    finally:
        dist.destroy_process_group()


# mode, batch size -> partition kind with two ranks
CASES = [("p2p", 2, "batch"), ("p2p", 1, "batch-groups"), ("queries", 2, "queries"), ("push", 2, "queries"),
         ("multimem", 2, "queries"), ("nccl", 2, "batch"), ("nccl", 1, "batch-groups"), ("slab-pipeline", 2, "batch"),
         ("slab-pipeline", 1, "batch-groups"), ("heads", 1, "batch-heads"), ("heads-slabs", 1, "batch-heads"), ("heads-nccl", 1, "batch-heads")]


@pytest.mark.parametrize("mode,batch,kind", CASES)
def test_two_gpus_sharded_equals_unsharded(mode, batch, kind):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_worker, args=(2, _free_port(), mode, batch, ret), nprocs=2, join=True)
    assert dict(ret) == {0: (True, kind), 1: (True, kind)}


def _host_worker(rank, world, port, batch, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from ops3d_b200.host_stream import HostStreamedStep
        from ops3d_b200.sharded import PeerReducer, partition, shard_rows

        shapes = [(8, 16, 32), (4, 8, 16)]
        K, Q, G, D = 4, 301, 8, 32
        value, sh, lsi, packed, grad_out = fda_oracle.make_inputs(shapes, batch, Q, G, D, K, seed=33)
        part = partition(batch, Q, rank, world)
        value_h = value.bfloat16().pin_memory()
        packed_h = shard_rows(packed, part).pin_memory()
        go_h = shard_rows(grad_out, part).bfloat16().pin_memory()
        reducer = PeerReducer(value.shape, torch.bfloat16, dev, spatial_shapes=sh, part=part)
        step = HostStreamedStep(value.shape, torch.bfloat16, packed_h.shape, torch.float32, K, sh.to(dev), lsi.to(dev), dev,
                                chunk_queries=40, reducer=reducer)
        out_h = torch.empty(packed_h.shape[0], packed_h.shape[1], G * D, dtype=torch.bfloat16).pin_memory()
        gv_h = torch.zeros(value.shape, dtype=torch.bfloat16).pin_memory()
        gp_h = torch.empty(packed_h.shape).pin_memory()
        ref_out, ref_gv, ref_gp = fda_oracle.fused_forward_backward(value_h, sh, packed, grad_out.bfloat16(), K)
        ok = True
        for _ in range(2):  # twice: slots, events and the reducer's buffers are reused
            gv_h.zero_()
            f0, f1 = step.run(value_h, packed_h, go_h, out_h, gv_h, gp_h)
            torch.cuda.synchronize()
            ok &= (out_h.float() - shard_rows(ref_out, part)).abs().max().item() <= 2e-2 * ref_out.abs().max().item()
            ok &= (gp_h - shard_rows(ref_gp, part)).abs().max().item() <= 2e-2 * ref_gp.abs().max().item()
            # this rank downloaded its 1/world slice of the reduced grad_value; the device copy is complete on every rank
            ok &= (gv_h.view(-1)[f0:f1].float() - ref_gv.view(-1)[f0:f1]).abs().max().item() <= 2e-2 * ref_gv.abs().max().item()
            ok &= (reducer.out.float().cpu() - ref_gv).abs().max().item() <= 2e-2 * ref_gv.abs().max().item()
            ok &= (f1 - f0) >= ref_gv.numel() // world - 8
        ret[rank] = (bool(ok), part.kind)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("batch,kind", [(2, "batch"), (1, "batch-groups")])
def test_two_gpus_host_streamed_step(batch, kind):
    """Host buffers in, host buffers out, on two ranks: rows streamed in chunks, value slices all-gathered over
    NVLink when two ranks share a batch element, images exchanged once per batch element; against the CPU oracle."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_host_worker, args=(2, _free_port(), batch, ret), nprocs=2, join=True)
    assert dict(ret) == {0: (True, kind), 1: (True, kind)}
