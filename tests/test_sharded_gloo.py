"""World-size-2 check (gloo, CPU) of the row-partitioning logic and of the one exchange step of the
backward pass.  The per-rank operator is injected: here the CPU oracle stands in for the CUDA
kernels, so what is under test is the host logic -- ranges, the all-reduce, the cast, gradient
plumbing -- not the arithmetic."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import fda_oracle
from ops3d_b200.sharded import partition, query_range, shard_queries, shard_rows, sharded_flash_deform_attn


class OracleLocalOps:
    """Test double with the interface of ``CudaLocalOps``."""

    def forward(self, value, shapes, lsi, packed, K, im2col_step):
        return fda_oracle.fused_forward(value, shapes, packed, K)

    def backward_accumulate(self, value, shapes, lsi, packed, grad_out, K, im2col_step):
        _, gv, gp = fda_oracle.fused_forward_backward(value, shapes, packed, grad_out, K)
        return gv.float(), gp

    def cast(self, accum, dtype):
        return accum.to(dtype)


@pytest.mark.parametrize("Q,world", [(10, 2), (7, 3), (5, 8), (598016, 8), (0, 2)])
def test_query_ranges_tile_exactly(Q, world):
    ranges = [query_range(Q, r, world) for r in range(world)]
    assert ranges[0][0] == 0 and ranges[-1][1] == Q
    for (a, b), (c, d) in zip(ranges, ranges[1:]):
        assert b == c and a <= b and c <= d
    sizes = [b - a for a, b in ranges]
    assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        query_range(Q, world, world)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("B,Q,world,kind", [(2, 598016, 1, "queries"), (2, 598016, 2, "batch"), (2, 598016, 4, "batch-groups"),
                                             (2, 598016, 8, "batch-groups"), (4, 200, 2, "batch"), (1, 73728, 8, "batch-groups"),
                                             (3, 100, 2, "queries"), (2, 10, 3, "queries")])
def test_partition_tiles_the_rows_and_groups_share_one_batch_element(B, Q, world, kind):
    parts = [partition(B, Q, r, world, mode="auto") for r in range(world)]
    assert all(p.kind == kind for p in parts)
    covered = torch.zeros(B, Q, dtype=torch.int32)
    for r, p in enumerate(parts):
        covered[p.b_begin:p.b_end, p.q_begin:p.q_end] += 1
        assert p.group[p.group_rank] == r
        # the ranks of a group work on the same batch elements and no others do
        for other, q in enumerate(parts):
            shares = (q.b_begin, q.b_end) == (p.b_begin, p.b_end)
            assert shares == (other in p.group)
        assert p.b_end - p.b_begin == parts[0].b_end - parts[0].b_begin  # same image count on every rank
    assert bool((covered == 1).all())
    if kind != "queries":
        assert all(p.b_end - p.b_begin == max(1, B // world) for p in parts)
    forced = [partition(B, Q, r, world, mode="queries") for r in range(world)]
    assert all(p.kind == "queries" and (p.b_begin, p.b_end) == (0, B) for p in forced)
    with pytest.raises(ValueError):
        partition(B, Q, world, world)


@pytest.mark.parametrize("B,G,world,kind,heads", [(2, 8, 8, "batch-heads", 2), (2, 8, 4, "batch-heads", 4), (1, 8, 8, "batch-heads", 1),
                                                  (2, 8, 2, "batch", 0), (2, 6, 8, "batch-groups", 0), (1, 8, 16, "batch-groups", 0)])
def test_head_split_is_chosen_when_the_group_size_divides_the_heads(B, G, world, kind, heads):
    Q = 1000
    parts = [partition(B, Q, r, world, mode="auto", num_heads=G) for r in range(world)]
    assert all(p.kind == kind for p in parts)
    covered = torch.zeros(B, Q, G, dtype=torch.int32)
    for r, p in enumerate(parts):
        h0, h1 = (p.h_begin, p.h_end) if p.splits_heads else (0, G)
        assert (h1 - h0 == heads) if heads else not p.splits_heads
        covered[p.b_begin:p.b_end, p.q_begin:p.q_end, h0:h1] += 1
        assert p.group[p.group_rank] == r
    assert bool((covered == 1).all())
    # "rows" never splits heads; shard_rows cuts both row layouts to the rank's heads
    assert all(not partition(B, Q, r, world, mode="rows", num_heads=G).splits_heads for r in range(world))
    p = parts[-1]
    if p.splits_heads:
        t4, t3 = torch.arange(B * Q * G * 3.0).reshape(B, Q, G, 3), torch.arange(B * Q * G * 5.0).reshape(B, Q, G * 5)
        assert torch.equal(shard_rows(t4, p), t4[p.b_begin:p.b_end, :, p.h_begin:p.h_end])
        assert torch.equal(shard_rows(t3, p, G), t3.reshape(B, Q, G, 5)[p.b_begin:p.b_end, :, p.h_begin:p.h_end].reshape(-1, Q, heads * 5))
        with pytest.raises(ValueError):
            shard_rows(t3, p)


def _worker(rank, world, port, case, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        B, mode = case
        shapes = [(4, 6, 8), (2, 3, 4)]
        G = 2
        value, sh, lsi, packed, grad_out = fda_oracle.make_inputs(shapes, B, 13, G, 8, 4, seed=9)
        part = partition(B, 13, rank, world, mode="auto" if mode == "heads" else mode, num_heads=G if mode == "heads" else None)
        v = value.clone().requires_grad_(True)
        pk = shard_rows(packed, part).requires_grad_(True)
        out = sharded_flash_deform_attn(v, sh, lsi, pk, 64, 4, None, OracleLocalOps(), part)
        out.backward(shard_rows(grad_out, part, G))
        ref_out, ref_gv, ref_gp = fda_oracle.fused_forward_backward(value, sh, packed, grad_out, 4)
        ok = torch.allclose(out, shard_rows(ref_out, part, G), atol=1e-5)
        ok &= torch.allclose(v.grad, ref_gv, atol=1e-4)  # reduced over ranks: the full gradient on every rank
        ok &= torch.allclose(pk.grad, shard_rows(ref_gp, part), atol=1e-4)
        ret[rank] = (bool(ok), part.kind)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("case,kind", [((2, "auto"), "batch"), ((1, "auto"), "batch-groups"), ((2, "queries"), "queries"),
                                       ((3, "auto"), "queries"), ((1, "heads"), "batch-heads")])
def test_two_ranks_reproduce_the_unsharded_result(case, kind):
    world = 2
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), case, ret), nprocs=world, join=True)
    assert dict(ret) == {0: (True, kind), 1: (True, kind)}


def test_slab_plan_and_exchange_ranges_tile_the_image():
    """Host-side slab plan (the C function the kernels share) and the exchange ranges derived from it."""
    from ops3d_b200 import capi
    from ops3d_b200.sharded import slab_exchange_ranges

    shapes = torch.tensor([(32, 64, 256), (16, 32, 128), (8, 16, 64)])
    N, G, D = int(shapes.prod(1).sum()), 8, 32
    plan = capi.bin_plan(shapes, (1, N, G, D), 74752, 8)
    assert plan == (0, 32, 1)  # level 0 in 32 z-slabs of one plane (16.8 MB of image each; the kernels cut each once more along y)
    assert capi.bin_plan(torch.tensor([(4, 8, 8), (2, 4, 4)]), (1, 288, 4, 16), 288, 4) is None  # fits L2: no binning
    for level_first in (True, False):
        sh = shapes if level_first else shapes.flip(0)
        pl = capi.bin_plan(sh, (1, N, G, D), 1000, 8)
        for parts in (1, 3, 4, 32, 40):
            got = slab_exchange_ranges(sh, (1, N, G, D), pl, parts)
            assert got is not None
            n, part_ranges, rest_ranges = got
            assert n == min(parts, 32) and len(part_ranges) == n
            ranges = sorted(part_ranges + rest_ranges)
            assert ranges[0][0] == 0 and ranges[-1][1] == N * G * D
            for (a, b), (c, d) in zip(ranges, ranges[1:]):
                assert b == c and a < b  # contiguous, no gap, no overlap
            assert all(b > a for a, b in part_ranges)
