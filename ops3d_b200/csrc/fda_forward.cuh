// Forward kernel of Flash Deformable 3D Attention for sm_100a.
//
// Replaces forward_kernel_reg / forward_kernel of the reference
// (csrc/cuda/flash_deform_im2col_cuda.cuh:190-295 and :50-186) and its trilinear
// helper (csrc/cuda/common.h:52-138) with one kernel in two staging flavours:
//   kStage = false  every lane reads its row's logits and coordinates straight from
//                   global memory (lanes of a row read the same addresses, which the
//                   load unit merges); nothing is shared between threads.
//   kStage = true   each warp first copies the packed rows it owns (contiguous in
//                   global memory) into a private shared-memory tile with fully
//                   coalesced vector loads, converted to fp32.
// Per row: soft-max over the L*K logits, then for each point the 8-corner trilinear
// gather with one predicated 16-byte load per corner and lane, fp32 accumulation, and
// one 16-byte store of the finished channels.  No thread block barrier besides the one
// that publishes the level table; warps never wait on each other.
//
// Head groups (p.head_group = heads per group, a divisor of G): the grid walks the rows group by group -- all queries
// for heads [0, hg), then all queries for heads [hg, 2 hg), ... -- instead of query by query, so that at any time the
// gathers touch only hg / G of the value volume.  With a volume larger than L2 (config 5: 306 MB per batch element)
// and points spread all over it, a group of two heads (77 MB) stays L2-resident where the whole volume does not.
#pragma once

#include "fda_device.cuh"

#ifndef FDA_FWD_MIN_BLOCKS
#define FDA_FWD_MIN_BLOCKS 3
#endif

namespace fda {

template <typename VT, typename PT, bool kStage>
__global__ void __launch_bounds__(kThreads, FDA_FWD_MIN_BLOCKS) fda_forward_kernel(const Problem p) {
    constexpr int CPL = Vec16<VT>::kCPL;
    __shared__ LevelGeom geom[kMaxLevels];
    extern __shared__ __align__(16) float smem_tile[];

    const int tid = threadIdx.x;
    if (tid == 0) build_level_table(geom, p.shapes, p.lsi, p.L, p.GD, p.value_elem_bytes, false, p.l2_keep_bytes);
    const uint64_t pol_keep = l2_policy_evict_last(), pol_stream = l2_policy_evict_first();

    const int b = blockIdx.y;
    const int gs = 1 << p.gs_log2;
    const int lane_c = tid & (gs - 1);
    const int rows_per_block = (int)blockDim.x >> p.gs_log2;
    // position of the row in head-group order -> (query, head); with head_group == G this is the identity
    const int hg = p.head_group, rows_per_group = p.Q * hg;
    const int blocks_per_group = (rows_per_group + rows_per_block - 1) / rows_per_block;
    const int group = blockIdx.x / blocks_per_group;
    const int local0 = (blockIdx.x - group * blocks_per_group) * rows_per_block;
    auto row_at = [&](int local) -> int { const int q = local / hg; return q * p.G + group * hg + (local - q * hg); };
    const int local = local0 + (tid >> p.gs_log2);
    const bool row_ok = local < rows_per_group;
    const int row = row_ok ? row_at(local) : 0;  // q * G + g inside batch element b
    const bool active = row_ok && lane_c < p.lpg;
    const int LK = p.LK;

    const PT *packed_row = static_cast<const PT *>(p.packed) + ((size_t)b * p.rows_per_b + row) * (size_t)(4 * LK);
    const float *tile_row = nullptr;
    if (kStage) {
        const int warp = tid >> 5, lane = tid & 31;
        const int rows_per_warp = 32 >> p.gs_log2;
        const int first = local0 + warp * rows_per_warp;
        float *wtile = smem_tile + warp * rows_per_warp * p.row_stride;
        int nrows = rows_per_group - first;
        nrows = nrows < 0 ? 0 : (nrows > rows_per_warp ? rows_per_warp : nrows);
        const PT *packed_b = static_cast<const PT *>(p.packed) + (size_t)b * p.rows_per_b * (size_t)(4 * LK);
        if (hg == p.G) {  // the warp's rows are one contiguous span
            stage_rows<PT>(packed_b + (size_t)first * (size_t)(4 * LK), wtile, nrows, LK, p.row_stride, lane);
        } else {          // hg consecutive rows per query
            const int nvec = nrows * LK;
            const float inv_lk = 1.0f / (float)LK;
            for (int v = lane; v < nvec; v += 32) {
                const int r = row_of_vector(v, inv_lk);
                const int c = (v - r * LK) * 4;
                *reinterpret_cast<float4 *>(wtile + r * p.row_stride + c) =
                    load4_stream<PT>(packed_b + (size_t)row_at(first + r) * (size_t)(4 * LK) + c);
            }
        }
        tile_row = wtile + ((tid & 31) >> p.gs_log2) * p.row_stride;
    }
    __syncthreads();  // level table (and, when staging, this warp's tile) visible

    // Four consecutive row elements starting at element `e` (a multiple of 4), as fp32.
    auto get4 = [&](int e) -> float4 {
        if (!row_ok) return make_float4(0.f, 0.f, 0.f, 0.f);
        if (kStage) return *reinterpret_cast<const float4 *>(tile_row + e);
        return load4<PT>(packed_row + e);
    };

    // soft-max statistics over the L*K logits of this row
    const int nchunk = LK >> 2;
    float m = -INFINITY;
    for (int j = 0; j < nchunk; ++j) {
        const float4 lg = get4(3 * LK + 4 * j);
        m = fmaxf(m, fmaxf(fmaxf(lg.x, lg.y), fmaxf(lg.z, lg.w)));
    }
    float s = 0.f;
    for (int j = 0; j < nchunk; ++j) {
        const float4 lg = get4(3 * LK + 4 * j);
        s += __expf(lg.x - m) + __expf(lg.y - m) + __expf(lg.z - m) + __expf(lg.w - m);
    }
    const float inv = 1.0f / s;

    const int g = row % p.G;
    const VT *value_b = static_cast<const VT *>(p.value) + (size_t)b * p.N * p.GD + (size_t)g * p.D + (size_t)lane_c * CPL;

    float acc[CPL];
#pragma unroll
    for (int k = 0; k < CPL; ++k) acc[k] = 0.f;

    for (int j = 0; j < nchunk; ++j) {
        const float4 c0 = get4(12 * j), c1 = get4(12 * j + 4), c2 = get4(12 * j + 8);
        const float4 lg = get4(3 * LK + 4 * j);
        const float xs[4] = {c0.x, c0.w, c1.z, c2.y};
        const float ys[4] = {c0.y, c1.x, c1.w, c2.z};
        const float zs[4] = {c0.z, c1.y, c2.x, c2.w};
        const float ls[4] = {lg.x, lg.y, lg.z, lg.w};
        const LevelGeom lv = geom[j >> p.k_shift];
        const VT *lvl = value_b + (size_t)lv.start * p.GD;
        const uint64_t pol = (lv.keep & 1) ? pol_keep : pol_stream;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const float a = __expf(ls[t] - m) * inv;
            PointGeom pg;
            point_geometry(lv, p.GD, xs[t], ys[t], zs[t], pg);
            uint4 raw[8];
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                const bool in = active && pg.zin[n >> 2] && pg.yin[(n >> 1) & 1] && pg.xin[n & 1];
                raw[n] = in ? ldg16_hint(lvl + pg.off[n], pol) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                const float w = a * ((pg.wx[n & 1] * pg.wy[(n >> 1) & 1]) * pg.wz[n >> 2]);
                axpy16<VT>(raw[n], w, acc);
            }
        }
    }

    if (active) {
        VT *dst = static_cast<VT *>(p.out) + ((size_t)b * p.rows_per_b + row) * (size_t)p.D + (size_t)lane_c * CPL;
        stg16_hint(dst, Vec16<VT>::pack(acc), pol_stream);
    }
}

}  // namespace fda
