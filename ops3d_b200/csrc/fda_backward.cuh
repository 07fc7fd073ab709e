// Backward kernels of Flash Deformable 3D Attention for sm_100a.
//
// Replaces backward_kernel_warp_primitive / backward_kernel of the reference
// (csrc/cuda/flash_deform_col2im_cuda.cuh:248-429 and :50-244) and its trilinear
// helper (csrc/cuda/common.h:141-354):
//   * each warp stages the packed rows it owns into a private shared-memory tile
//     (coalesced), and at the end writes the finished gradient rows back from the
//     same tile (coalesced, already in the packed dtype) -- no fp32 copy of
//     grad_sampling_loc_attn, no later cast pass, no block barrier in the loop;
//   * per point: 8 predicated 16-byte corner loads, per-corner dot products with
//     grad_output, the four partial sums (d/dx, d/dy, d/dz, d/d alpha) reduced over
//     the lanes of the row with xor-shuffles;
//   * grad_value: fp32 scatter with red.global.add.v4.f32 (one 16-byte reduction per
//     lane and corner half), channels interleaved over the lanes of a row so that one
//     warp instruction covers whole 32-byte sectors of the accumulation image;
//   * soft-max backward in closed form, grad_logit_i = p_i * (dalpha_i - sum_j p_j dalpha_j),
//     instead of the reference's O((L*K)^2) Jacobian loop (:413-427).
//
// A launch may cover only some pyramid levels (level_mask).  A non-final launch leaves the raw
// dalpha of its points in an fp32 plane of the caller's scratch (or, without one, in the logit
// slots of grad_packed, which is exact for fp32 offsets only); the final launch (`resume`) picks up
// the finished coordinate slots of the other levels from grad_packed and their dalpha from the
// plane, adds its own and applies the soft-max backward over all points.  This lets a multi-GPU caller finish the largest level first and
// exchange its part of the gradient image while the remaining levels are still being computed,
// and lets the largest level be handled slab by slab (fda_backward_binned.cuh).
#pragma once

#include "fda_device.cuh"

#ifndef FDA_BWD_MIN_BLOCKS
#define FDA_BWD_MIN_BLOCKS 2
#endif

namespace fda {

// grad_output of one row as seen by one lane: its gather channels (for the dot products) and its
// scatter channels (4*lane_c + r*4*lpg, so that the lanes of a row cover contiguous bytes).
template <typename VT>
struct RowGrad {
    static constexpr int CPL = Vec16<VT>::kCPL;
    static constexpr int NRED = CPL / 4;
    float d[CPL];
    float s[NRED][4];
    __device__ __forceinline__ void load(const VT *go_row, int lane_c, int lpg, bool active, uint64_t pol) {
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        if (active) raw = ldg16_hint(go_row + (size_t)lane_c * CPL, pol);
        Vec16<VT>::unpack(raw, d);
#pragma unroll
        for (int r = 0; r < NRED; ++r) {
            float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
            if (active) f = load4<VT>(go_row + r * 4 * lpg + 4 * lane_c);
            s[r][0] = f.x; s[r][1] = f.y; s[r][2] = f.z; s[r][3] = f.w;
        }
    }
    // Two-step form of the loads above, so that a caller can issue the loads of its NEXT row early and convert
    // them when that row's turn comes: raw bits of the gather channels and of the scatter channels.
    struct Raw {
        uint4 d;
        uint4 s[NRED];
    };
    static __device__ __forceinline__ Raw issue(const VT *go_row, int lane_c, int lpg, bool active, uint64_t pol) {
        Raw r;
        r.d = make_uint4(0u, 0u, 0u, 0u);
        if (active) r.d = ldg16_hint(go_row + (size_t)lane_c * CPL, pol);
#pragma unroll
        for (int i = 0; i < NRED; ++i) {
            r.s[i] = make_uint4(0u, 0u, 0u, 0u);
            if (active) r.s[i] = load4_raw<VT>(go_row + i * 4 * lpg + 4 * lane_c);
        }
        return r;
    }
    static __device__ __forceinline__ Raw issue_paired(const VT *go_own, int lane_c, bool active, const VT *go_even,
                                                       const VT *go_odd, int tl, uint64_t pol) {
        Raw r;
        r.d = make_uint4(0u, 0u, 0u, 0u);
        if (active) r.d = ldg16_hint(go_own + (size_t)lane_c * CPL, pol);
#pragma unroll
        for (int i = 0; i < NRED; ++i) r.s[i] = make_uint4(0u, 0u, 0u, 0u);
        if (go_even) r.s[0] = load4_raw<VT>(go_even + 4 * tl);
        if (go_odd) r.s[NRED - 1] = load4_raw<VT>(go_odd + 4 * tl);
        return r;
    }
    __device__ __forceinline__ void take(const Raw &r) {
        Vec16<VT>::unpack(r.d, d);
#pragma unroll
        for (int i = 0; i < NRED; ++i) {
            const float4 f = cvt4<VT>(r.s[i]);
            s[i][0] = f.x; s[i][1] = f.y; s[i][2] = f.z; s[i][3] = f.w;
        }
    }
    // Paired layout (two rows of 4 lanes form a team of 8): s[0] = channels 4*tl.. of the EVEN row of the
    // team, s[1] = the same channels of the ODD row, tl = lane within the team.  `go_even` / `go_odd` may be
    // null when that row does not exist.
    __device__ __forceinline__ void load_paired(const VT *go_own, int lane_c, bool active, const VT *go_even,
                                                const VT *go_odd, int tl, uint64_t pol) {
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        if (active) raw = ldg16_hint(go_own + (size_t)lane_c * CPL, pol);
        Vec16<VT>::unpack(raw, d);
        float4 e = make_float4(0.f, 0.f, 0.f, 0.f), o = e;
        if (go_even) e = load4<VT>(go_even + 4 * tl);
        if (go_odd) o = load4<VT>(go_odd + 4 * tl);
        s[0][0] = e.x; s[0][1] = e.y; s[0][2] = e.z; s[0][3] = e.w;
        s[NRED - 1][0] = o.x; s[NRED - 1][1] = o.y; s[NRED - 1][2] = o.z; s[NRED - 1][3] = o.w;
    }
};

// Backward of one sampling point for the lanes of one row: gathers the 8 corners, scatters
// a*w*grad_out into the fp32 image, and returns (summed over the row's lanes) the gradients w.r.t.
// the normalised coordinates and dalpha = <sample, grad_out>.  Must be called by all 32 lanes.
//
// kPair (rows of exactly 4 lanes, 32 fp32 = 128 bytes of image per corner): two neighbouring rows
// form a team of 8 lanes and scatter together -- first the even row's corner, then the odd row's,
// each as 8 x 16 contiguous bytes, so that one reduction request to L2 covers a whole 128-byte line
// instead of two half-line requests.  acc_even / acc_odd are the two rows' image bases (head offset
// included, lane offset excluded); weight and offset of the partner row's corner come by shuffle.
// Core: geometry given (corner offsets, validity, weights).  gx/gy/gz_out are the derivatives of the sample
// dotted with grad_out w.r.t. the VOXEL coordinates (not yet multiplied by a or by d voxel / d input).
template <typename VT, bool kPair>
__device__ __forceinline__ void point_backward_geom(const PointGeom &pg, float a,
                                                    const VT *lvl, float *acc_lvl, const RowGrad<VT> &go, int red_stride,
                                                    bool active, int gs, uint64_t pol_v, uint64_t pol_g,
                                                    float &gx_out, float &gy_out, float &gz_out, float &da_out,
                                                    float *acc_even = nullptr, float *acc_odd = nullptr) {
    constexpr int CPL = Vec16<VT>::kCPL;
    constexpr int NRED = CPL / 4;
    uint4 raw[8];
    bool in[8];
#pragma unroll
    for (int n = 0; n < 8; ++n) {
        in[n] = active && pg.zin[n >> 2] && pg.yin[(n >> 1) & 1] && pg.xin[n & 1];
        raw[n] = in[n] ? ldg16_hint_ordered(lvl + pg.off[n], pol_v) : make_uint4(0u, 0u, 0u, 0u);
    }
    // Scatter first: the reductions depend on the weights and on grad_out only, so they are on their way to L2
    // while the eight gathers above are still in flight; the dot products below are the first use of the gathers.
#pragma unroll
    for (int n = 0; n < 8; ++n) {
        const float w = (pg.wx[n & 1] * pg.wy[(n >> 1) & 1]) * pg.wz[n >> 2];
        const float aw = a * w;
        if (kPair) {
            const unsigned lane = threadIdx.x & 31u;
            const bool odd = (lane >> 2) & 1u;
            const uint32_t code = in[n] ? pg.off[n] : 0x80000000u;  // offsets stay below 2^31
            const uint32_t code_p = __shfl_xor_sync(0xffffffffu, code, 4);
            const float aw_p = __shfl_xor_sync(0xffffffffu, aw, 4);
            const uint32_t code_e = odd ? code_p : code, code_o = odd ? code : code_p;
            const float aw_e = odd ? aw_p : aw, aw_o = odd ? aw : aw_p;
            const unsigned tl4 = (lane & 7u) * 4u;
            if (!(code_e >> 31))
                red_add_f32x4_hint(acc_even + code_e + tl4, aw_e * go.s[0][0], aw_e * go.s[0][1], aw_e * go.s[0][2], aw_e * go.s[0][3], pol_g);
            if (!(code_o >> 31))
                red_add_f32x4_hint(acc_odd + code_o + tl4, aw_o * go.s[NRED - 1][0], aw_o * go.s[NRED - 1][1], aw_o * go.s[NRED - 1][2],
                                   aw_o * go.s[NRED - 1][3], pol_g);
        } else if (in[n]) {
            float *dst = acc_lvl + pg.off[n];
#pragma unroll
            for (int r = 0; r < NRED; ++r)
                red_add_f32x4_hint(dst + r * red_stride, aw * go.s[r][0], aw * go.s[r][1], aw * go.s[r][2], aw * go.s[r][3], pol_g);
        }
    }
    float dot[8];
#pragma unroll
    for (int n = 0; n < 8; ++n) {
        float v[CPL];
        Vec16<VT>::unpack(raw[n], v);
#ifdef FDA_NO_FFMA2
        float d = 0.f;
#pragma unroll
        for (int k = 0; k < CPL; ++k) d = fmaf(v[k], go.d[k], d);
        dot[n] = d;  // 0 for corners outside the level
#else
        float d0 = 0.f, d1 = 0.f;  // even / odd channels, two per instruction
#pragma unroll
        for (int k = 0; k < CPL; k += 2) ffma2(d0, d1, v[k], v[k + 1], go.d[k], go.d[k + 1]);
        dot[n] = d0 + d1;  // 0 for corners outside the level
#endif
    }
    // d out / d x_im = sum_{z,y} wz*wy*(dot[z,y,1] - dot[z,y,0]), likewise y and z; dalpha = sum w*dot
    const float wzy[4] = {pg.wz[0] * pg.wy[0], pg.wz[0] * pg.wy[1], pg.wz[1] * pg.wy[0], pg.wz[1] * pg.wy[1]};
    const float wzx[4] = {pg.wz[0] * pg.wx[0], pg.wz[0] * pg.wx[1], pg.wz[1] * pg.wx[0], pg.wz[1] * pg.wx[1]};
    const float wyx[4] = {pg.wy[0] * pg.wx[0], pg.wy[0] * pg.wx[1], pg.wy[1] * pg.wx[0], pg.wy[1] * pg.wx[1]};
    float gx = wzy[0] * (dot[1] - dot[0]) + wzy[1] * (dot[3] - dot[2]) + wzy[2] * (dot[5] - dot[4]) + wzy[3] * (dot[7] - dot[6]);
    float gy = wzx[0] * (dot[2] - dot[0]) + wzx[1] * (dot[3] - dot[1]) + wzx[2] * (dot[6] - dot[4]) + wzx[3] * (dot[7] - dot[5]);
    float gz = wyx[0] * (dot[4] - dot[0]) + wyx[1] * (dot[5] - dot[1]) + wyx[2] * (dot[6] - dot[2]) + wyx[3] * (dot[7] - dot[3]);
    float da = 0.f;
#pragma unroll
    for (int n = 0; n < 8; ++n) da = fmaf((pg.wx[n & 1] * pg.wy[(n >> 1) & 1]) * pg.wz[n >> 2], dot[n], da);
    for (int mask = gs >> 1; mask > 0; mask >>= 1) {
        gx += __shfl_xor_sync(0xffffffffu, gx, mask);
        gy += __shfl_xor_sync(0xffffffffu, gy, mask);
        gz += __shfl_xor_sync(0xffffffffu, gz, mask);
        da += __shfl_xor_sync(0xffffffffu, da, mask);
    }
    gx_out = gx;
    gy_out = gy;
    gz_out = gz;
    da_out = da;
}

// Deformable-attention form: normalised coordinates, gradients w.r.t. them (voxel = coordinate * extent - 0.5).
template <typename VT, bool kPair>
__device__ __forceinline__ void point_backward(const LevelGeom &lv, int GD, float x, float y, float z, float a,
                                               const VT *lvl, float *acc_lvl, const RowGrad<VT> &go, int red_stride,
                                               bool active, int gs, uint64_t pol_v, uint64_t pol_g,
                                               float &gx_out, float &gy_out, float &gz_out, float &da_out,
                                               float *acc_even = nullptr, float *acc_odd = nullptr) {
    PointGeom pg;
    point_geometry(lv, GD, x, y, z, pg);
    float gx, gy, gz;
    point_backward_geom<VT, kPair>(pg, a, lvl, acc_lvl, go, red_stride, active, gs, pol_v, pol_g, gx, gy, gz, da_out,
                                   acc_even, acc_odd);
    gx_out = a * lv.fW * gx;
    gy_out = a * lv.fH * gy;
    gz_out = a * lv.fD * gz;
}

template <typename VT, typename PT, bool kPair>
__global__ void __launch_bounds__(kThreads, FDA_BWD_MIN_BLOCKS) fda_backward_kernel(const Problem p) {
    constexpr int CPL = Vec16<VT>::kCPL;
    __shared__ LevelGeom geom[kMaxLevels];
    __shared__ int s_mask, s_resume;
    extern __shared__ __align__(16) float smem_tile[];

    const int tid = threadIdx.x;
    if (tid == 0) {
        build_level_table(geom, p.shapes, p.lsi, p.L, p.GD, p.value_elem_bytes, true, p.l2_keep_bytes);
        // the slab-binned launches of this call (if any) own the largest level
        const BinPlan plan = make_bin_plan(p);
        s_mask = plan.enabled ? (p.level_mask & ~(1 << plan.level)) : p.level_mask;
        s_resume = p.resume | plan.enabled;
    }
    const uint64_t pol_keep = l2_policy_evict_last(), pol_stream = l2_policy_evict_first();

    const int b = blockIdx.y;
    const int gs = 1 << p.gs_log2;
    const int lane = tid & 31, warp = tid >> 5;
    const int lane_c = tid & (gs - 1);
    const int rows_per_block = (int)blockDim.x >> p.gs_log2;
    const int rows_per_warp = 32 >> p.gs_log2;
    const int row = blockIdx.x * rows_per_block + (tid >> p.gs_log2);  // q * G + g inside batch element b
    const bool row_ok = row < p.rows_per_b;
    const bool active = row_ok && lane_c < p.lpg;
    const int LK = p.LK;
    const float inv_lk = 1.0f / (float)LK;

    // Tile row layout (fp32): [0,3LK) coordinates -> coordinate gradients,
    // [3LK,4LK) logits -> dalpha -> logit gradients, [4LK,5LK) exp(logit - max).
    const int first = blockIdx.x * rows_per_block + warp * rows_per_warp;
    float *wtile = smem_tile + warp * rows_per_warp * p.row_stride;
    int nrows = p.rows_per_b - first;
    nrows = nrows < 0 ? 0 : (nrows > rows_per_warp ? rows_per_warp : nrows);
    const size_t warp_elem0 = ((size_t)b * p.rows_per_b + first) * (size_t)(4 * LK);
    stage_rows<PT>(static_cast<const PT *>(p.packed) + warp_elem0, wtile, nrows, LK, p.row_stride, lane);
    float *trow = wtile + (lane >> p.gs_log2) * p.row_stride;
    __syncthreads();  // level table and this warp's tile visible
    const int level_mask = s_mask;
    if (level_mask == 0 && !p.finalize) return;  // nothing left for this launch (uniform over the grid)

    const int nchunk = LK >> 2;
    float m = -INFINITY;
    for (int j = 0; j < nchunk; ++j) {
        const float4 lg = *reinterpret_cast<const float4 *>(trow + 3 * LK + 4 * j);
        m = fmaxf(m, fmaxf(fmaxf(lg.x, lg.y), fmaxf(lg.z, lg.w)));
    }
    float s = 0.f;
    for (int j = 0; j < nchunk; ++j) {
        const float4 lg = *reinterpret_cast<const float4 *>(trow + 3 * LK + 4 * j);
        const float4 e = make_float4(__expf(lg.x - m), __expf(lg.y - m), __expf(lg.z - m), __expf(lg.w - m));
        s += e.x + e.y + e.z + e.w;
        if (lane_c == 0) *reinterpret_cast<float4 *>(trow + 4 * LK + 4 * j) = e;
    }
    const float inv = 1.0f / s;
    __syncwarp();
    if (s_resume) {
        // slots of levels handled by an earlier launch: finished coordinate gradients and raw dalpha
        const PT *prev = static_cast<const PT *>(p.grad_packed) + warp_elem0;
        const float *prev_da = p.dalpha ? p.dalpha + ((size_t)b * p.rows_per_b + first) * (size_t)LK : nullptr;
        const int nvec = nrows * LK;
        for (int v = lane; v < nvec; v += 32) {
            const int r = row_of_vector(v, inv_lk);
            const int c = (v - r * LK) * 4;
            const int j = c < 3 * LK ? c / 12 : (c - 3 * LK) >> 2;
            if (!((level_mask >> (j >> p.k_shift)) & 1)) {
                float4 f;
                if (c >= 3 * LK && prev_da) f = __ldcs(reinterpret_cast<const float4 *>(prev_da + (size_t)r * LK + (c - 3 * LK)));
                else f = load4_stream<PT>(prev + (size_t)v * 4);
                *reinterpret_cast<float4 *>(wtile + r * p.row_stride + c) = f;
            }
        }
        __syncwarp();
    }

    const int g = row_ok ? row % p.G : 0;
    const size_t head_elem = (size_t)b * p.N * p.GD + (size_t)g * p.D;
    const VT *value_b = static_cast<const VT *>(p.value) + head_elem + (size_t)lane_c * CPL;
    float *accum_b = p.accum + head_elem + (size_t)lane_c * 4;

    RowGrad<VT> go;
    const VT *go_rows = static_cast<const VT *>(p.grad_out) + (size_t)b * p.rows_per_b * (size_t)p.D;
    float *acc_even = nullptr, *acc_odd = nullptr;  // kPair: image bases of the two rows of this lane's team
    if (kPair) {
        const int row_e = row & ~1, row_o = row | 1;  // rows of a team are neighbours; an odd last row has no partner
        go.load_paired(go_rows + (size_t)(row_ok ? row : 0) * p.D, lane_c, active,
                       row_e < p.rows_per_b ? go_rows + (size_t)row_e * p.D : nullptr,
                       row_o < p.rows_per_b ? go_rows + (size_t)row_o * p.D : nullptr, lane & 7, pol_stream);
        acc_even = p.accum + (size_t)b * p.N * p.GD + (size_t)(row_e % p.G) * p.D;
        acc_odd = p.accum + (size_t)b * p.N * p.GD + (size_t)(row_o % p.G) * p.D;
    } else {
        go.load(go_rows + (size_t)(row_ok ? row : 0) * p.D, lane_c, p.lpg, active, pol_stream);
    }
    const int red_stride = 4 * p.lpg;

    for (int j = 0; j < nchunk; ++j) {
        if (!((level_mask >> (j >> p.k_shift)) & 1)) continue;
        const float4 c0 = *reinterpret_cast<const float4 *>(trow + 12 * j);
        const float4 c1 = *reinterpret_cast<const float4 *>(trow + 12 * j + 4);
        const float4 c2 = *reinterpret_cast<const float4 *>(trow + 12 * j + 8);
        const float4 e4 = *reinterpret_cast<const float4 *>(trow + 4 * LK + 4 * j);
        const float xs[4] = {c0.x, c0.w, c1.z, c2.y};
        const float ys[4] = {c0.y, c1.x, c1.w, c2.z};
        const float zs[4] = {c0.z, c1.y, c2.x, c2.w};
        const float es[4] = {e4.x, e4.y, e4.z, e4.w};
        const LevelGeom lv = geom[j >> p.k_shift];
        const VT *lvl = value_b + (size_t)lv.start * p.GD;
        float *acc_lvl = accum_b + (size_t)lv.start * p.GD;
        const uint64_t pol_v = (lv.keep & 1) ? pol_keep : pol_stream;
        const uint64_t pol_g = (lv.keep & 2) ? pol_keep : pol_stream;
        float gxs[4], gys[4], gzs[4], das[4];
#pragma unroll
        for (int t = 0; t < 4; ++t)
            point_backward<VT, kPair>(lv, p.GD, xs[t], ys[t], zs[t], es[t] * inv, lvl, acc_lvl, go, red_stride, active, gs,
                                      pol_v, pol_g, gxs[t], gys[t], gzs[t], das[t],
                                      kPair ? acc_even + (size_t)lv.start * p.GD : nullptr,
                                      kPair ? acc_odd + (size_t)lv.start * p.GD : nullptr);
        __syncwarp();  // every lane of the row has read this chunk's coordinates
        if (lane_c == 0) {
            *reinterpret_cast<float4 *>(trow + 12 * j) = make_float4(gxs[0], gys[0], gzs[0], gxs[1]);
            *reinterpret_cast<float4 *>(trow + 12 * j + 4) = make_float4(gys[1], gzs[1], gxs[2], gys[2]);
            *reinterpret_cast<float4 *>(trow + 12 * j + 8) = make_float4(gzs[2], gxs[3], gys[3], gzs[3]);
            *reinterpret_cast<float4 *>(trow + 3 * LK + 4 * j) = make_float4(das[0], das[1], das[2], das[3]);
        }
    }
    __syncwarp();
    if (p.finalize) {
        float S = 0.f;  // sum_i p_i * dalpha_i over ALL points of the row
        for (int i = 0; i < LK; ++i) S = fmaf(trow[4 * LK + i] * inv, trow[3 * LK + i], S);
        __syncwarp();
        for (int i = lane_c; i < LK; i += gs) {
            const float a = trow[4 * LK + i] * inv;
            trow[3 * LK + i] = a * (trow[3 * LK + i] - S);
        }
        __syncwarp();
    }

    // coalesced write-back of the finished gradient rows of this warp
    PT *dst = static_cast<PT *>(p.grad_packed) + warp_elem0;
    const int nvec = nrows * LK;
    float *next_da = (!p.finalize && p.dalpha) ? p.dalpha + ((size_t)b * p.rows_per_b + first) * (size_t)LK : nullptr;
    for (int v = lane; v < nvec; v += 32) {
        const int r = row_of_vector(v, inv_lk);
        const int c = (v - r * LK) * 4;
        const float4 f = *reinterpret_cast<const float4 *>(wtile + r * p.row_stride + c);
        store4_stream<PT>(dst + (size_t)v * 4, f);
        // raw dalpha for the launch that finishes these rows, unrounded
        if (next_da && c >= 3 * LK) __stcs(reinterpret_cast<float4 *>(next_da + (size_t)r * LK + (c - 3 * LK)), f);
    }
}

// fp32 accumulation image -> grad_value in a 16-bit dtype; n4 = number of 4-element vectors.
template <typename VT>
__global__ void __launch_bounds__(256) fda_cast_kernel(const float *__restrict__ accum, VT *__restrict__ out, size_t n4) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const float4 f = __ldcs(reinterpret_cast<const float4 *>(accum) + i);
        store4<VT>(out + i * 4, f);
    }
}

}  // namespace fda
