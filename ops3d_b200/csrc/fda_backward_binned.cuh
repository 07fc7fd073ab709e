// Slab-binned backward for the largest pyramid level.
//
// Why: with sampling points spread over the whole volume, the scatter into the fp32 image of the
// largest level (537 MB per batch element at 32x64x256 cells, 8 heads x 32 channels) misses L2 on
// nearly every corner: a 128-byte read-modify-write through HBM per corner, which is what bounds
// the plain kernel.  Here the points of that level are first sorted into z-slabs whose share of the
// image (and of value) fits L2 comfortably; then the slabs are processed one after the other, so
// gathers and reductions of a slab hit L2 and every image line goes to HBM once.
//
//   fda_bin_count_kernel   one thread per row: which slab does each of the level's K points fall in;
//                          block histogram in shared memory, one global atomic per slab and block
//   fda_bin_scan_kernel    exclusive scan of the slab counts of every batch element
//   fda_bin_fill_kernel    one lane group per row (rows staged like in fda_backward_kernel): soft-max of
//                          the row, then appends {row*K+k, probability}
//                          to the point's slab list (block-local positions from shared-memory atomics,
//                          one global reservation per slab and block); points with no corner inside the
//                          level get their zero gradients written here
//   fda_backward_binned_kernel  grid (x, slab, batch): one lane group per list entry -- dense work,
//                          no divergence; same point_backward as the plain kernel; writes the point's
//                          coordinate gradients straight into grad_packed and its raw dalpha into the
//                          fp32 dalpha plane (into grad_packed's logit slot when there is no plane)
//
// The remaining levels, and the soft-max backward over all points, are done afterwards by
// fda_backward_kernel with `resume`.  Nothing here waits on another block.
#pragma once

#include "fda_backward.cuh"

namespace fda {

// brick (z-slab * ny + y-part) of a point from its normalised coordinates, or -1 when no corner lies inside the level
__device__ __forceinline__ int slab_of_point(const LevelGeom &lv, const BinPlan &plan, float x, float y, float z) {
    const float xf = floorf(unnormalize(x, lv.fW));
    const float yf = floorf(unnormalize(y, lv.fH));
    const float zf = floorf(unnormalize(z, lv.fD));
    // an axis has a corner in range iff floor in [-1, size-1]; written so that NaN fails
    const bool ok = (xf >= -1.f) && (xf <= (lv.fW - 1.0f)) && (yf >= -1.f) && (yf <= (lv.fH - 1.0f)) &&
                    (zf >= -1.f) && (zf <= (lv.fD - 1.0f));
    if (!ok) return -1;
    int z0 = (int)zf, y0 = (int)yf;
    z0 = z0 < 0 ? 0 : z0;
    y0 = y0 < 0 ? 0 : y0;
    return (z0 / plan.depth) * plan.ny + y0 / plan.ydepth;
}

__device__ __forceinline__ LevelGeom level_geom_of(const Problem &p, int l) {
    LevelGeom lv;
    lv.D = (int)p.shapes[3 * l];
    lv.H = (int)p.shapes[3 * l + 1];
    lv.W = (int)p.shapes[3 * l + 2];
    lv.start = (int)p.lsi[l];
    lv.keep = 0;
    lv.fD = (float)lv.D; lv.fH = (float)lv.H; lv.fW = (float)lv.W;
    return lv;
}

template <typename PT>
__global__ void __launch_bounds__(256) fda_bin_count_kernel(const Problem p) {
    __shared__ BinPlan plan;
    __shared__ LevelGeom lv;
    __shared__ unsigned int hist[kMaxSlabs];
    if (threadIdx.x == 0) {
        plan = make_bin_plan(p);
        lv = level_geom_of(p, plan.level);
    }
    for (int i = threadIdx.x; i < kMaxSlabs; i += blockDim.x) hist[i] = 0u;
    __syncthreads();
    if (!plan.enabled) return;
    const int b = blockIdx.y;
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row < p.rows_per_b) {
        const PT *pr = static_cast<const PT *>(p.packed) + ((size_t)b * p.rows_per_b + row) * (size_t)(4 * p.LK) + 3 * plan.level * p.K;
        for (int j = 0; j < (p.K >> 2); ++j) {  // 4 points = 12 coordinates = three 4-element vectors
            const float4 c0 = load4<PT>(pr + 12 * j), c1 = load4<PT>(pr + 12 * j + 4), c2 = load4<PT>(pr + 12 * j + 8);
            const int s0 = slab_of_point(lv, plan, c0.x, c0.y, c0.z), s1 = slab_of_point(lv, plan, c0.w, c1.x, c1.y);
            const int s2 = slab_of_point(lv, plan, c1.z, c1.w, c2.x), s3 = slab_of_point(lv, plan, c2.y, c2.z, c2.w);
            if (s0 >= 0) atomicAdd(&hist[s0], 1u);
            if (s1 >= 0) atomicAdd(&hist[s1], 1u);
            if (s2 >= 0) atomicAdd(&hist[s2], 1u);
            if (s3 >= 0) atomicAdd(&hist[s3], 1u);
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < plan.slabs * plan.ny; i += blockDim.x)
        if (hist[i]) atomicAdd(p.bin_counters + (size_t)b * kMaxSlabs + i, hist[i]);
}

// counters: [0] counts, [1] offsets (exclusive scan per batch element), [2] cursors (zeroed by the host)
__global__ void fda_bin_scan_kernel(const Problem p) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= p.B) return;
    const unsigned int *cnt = p.bin_counters + (size_t)b * kMaxSlabs;
    unsigned int *off = p.bin_counters + (size_t)(p.B + b) * kMaxSlabs;
    unsigned int run = 0;
    for (int s = 0; s < kMaxSlabs; ++s) {
        off[s] = run;
        run += cnt[s];
    }
}

// Same row -> lane-group mapping and warp-private staging as fda_backward_kernel, so the packed rows are
// read with coalesced vector loads; the K points of the level are spread over the lanes of the row.
template <typename PT>
__global__ void __launch_bounds__(kThreads) fda_bin_fill_kernel(const Problem p) {
    constexpr int kMaxK = 8;
    __shared__ BinPlan plan;
    __shared__ LevelGeom lv;
    __shared__ unsigned int hist[kMaxSlabs];
    __shared__ unsigned int base[kMaxSlabs];
    extern __shared__ __align__(16) float smem_tile[];
    const int tid = threadIdx.x;
    if (tid == 0) {
        plan = make_bin_plan(p);
        lv = level_geom_of(p, plan.level);
    }
    for (int i = tid; i < kMaxSlabs; i += blockDim.x) hist[i] = 0u;
    __syncthreads();
    if (!plan.enabled) return;
    const int b = blockIdx.y;
    const int gs = 1 << p.gs_log2;
    const int lane = tid & 31, warp = tid >> 5;
    const int lane_c = tid & (gs - 1);
    const int rows_per_block = (int)blockDim.x >> p.gs_log2;
    const int rows_per_warp = 32 >> p.gs_log2;
    const int row = blockIdx.x * rows_per_block + (tid >> p.gs_log2);
    const bool row_ok = row < p.rows_per_b;
    const int LK = p.LK, K = p.K;
    const int first = blockIdx.x * rows_per_block + warp * rows_per_warp;
    float *wtile = smem_tile + warp * rows_per_warp * p.row_stride;
    int nrows = p.rows_per_b - first;
    nrows = nrows < 0 ? 0 : (nrows > rows_per_warp ? rows_per_warp : nrows);
    stage_rows<PT>(static_cast<const PT *>(p.packed) + ((size_t)b * p.rows_per_b + first) * (size_t)(4 * LK), wtile, nrows,
                   LK, p.row_stride, lane);
    __syncwarp();
    const float *trow = wtile + (lane >> p.gs_log2) * p.row_stride;

    int slab[kMaxK];
    unsigned int pos[kMaxK];
    float prob[kMaxK];
#pragma unroll
    for (int j = 0; j < kMaxK; ++j) slab[j] = -2;  // -2: no point for this lane, -1: point without a corner in range
    if (row_ok) {
        float m = -INFINITY;
        for (int j = 0; j < (LK >> 2); ++j) {
            const float4 lg = *reinterpret_cast<const float4 *>(trow + 3 * LK + 4 * j);
            m = fmaxf(m, fmaxf(fmaxf(lg.x, lg.y), fmaxf(lg.z, lg.w)));
        }
        float s = 0.f;
        for (int j = 0; j < (LK >> 2); ++j) {
            const float4 lg = *reinterpret_cast<const float4 *>(trow + 3 * LK + 4 * j);
            s += __expf(lg.x - m) + __expf(lg.y - m) + __expf(lg.z - m) + __expf(lg.w - m);
        }
        const float inv = 1.0f / s;
        PT *gr = static_cast<PT *>(p.grad_packed) + ((size_t)b * p.rows_per_b + row) * (size_t)(4 * LK);
#pragma unroll
        for (int j = 0; j < kMaxK; ++j) {
            const int k = lane_c + j * gs;
            if (k < K) {
                const int i = plan.level * K + k;
                slab[j] = slab_of_point(lv, plan, trow[3 * i], trow[3 * i + 1], trow[3 * i + 2]);
                prob[j] = __expf(trow[3 * LK + i] - m) * inv;
                if (slab[j] >= 0) {
                    pos[j] = atomicAdd(&hist[slab[j]], 1u);
                } else {  // no corner inside the level: the point contributes nothing, its gradients are zero
                    store1<PT>(gr + 3 * i, 0.f); store1<PT>(gr + 3 * i + 1, 0.f); store1<PT>(gr + 3 * i + 2, 0.f);
                    if (p.dalpha) p.dalpha[((size_t)b * p.rows_per_b + row) * (size_t)LK + i] = 0.f;
                    else store1<PT>(gr + 3 * LK + i, 0.f);
                }
            }
        }
    }
    __syncthreads();
    for (int i = tid; i < plan.slabs * plan.ny; i += blockDim.x) {
        const unsigned int n = hist[i];
        base[i] = n ? atomicAdd(p.bin_counters + (size_t)(2 * p.B + b) * kMaxSlabs + i, n) : 0u;
    }
    __syncthreads();
    if (row_ok) {
        const unsigned int *off = p.bin_counters + (size_t)(p.B + b) * kMaxSlabs;
        uint2 *list = p.bin_entries + (size_t)b * p.bin_cap;
#pragma unroll
        for (int j = 0; j < kMaxK; ++j) {
            if (slab[j] >= 0) {
                const int k = lane_c + j * gs;
                const size_t at = (size_t)off[slab[j]] + base[slab[j]] + pos[j];
                list[at] = make_uint2((unsigned int)row * (unsigned int)K + (unsigned int)k, __float_as_uint(prob[j]));
            }
        }
    }
}

template <typename VT, typename PT, bool kPair>
__global__ void __launch_bounds__(kThreads, FDA_BWD_MIN_BLOCKS) fda_backward_binned_kernel(const Problem p) {
    constexpr int CPL = Vec16<VT>::kCPL;
    __shared__ BinPlan plan;
    __shared__ LevelGeom lv_s;
    if (threadIdx.x == 0) {
        plan = make_bin_plan(p);
        lv_s = level_geom_of(p, plan.level);
    }
    __syncthreads();
    const int b = blockIdx.z;
    if (!plan.enabled) return;
    // slab groups are cut between z-slabs; each z-slab has plan.ny bricks with a list of their own
    const int slab_first = (plan.slabs * p.slab_part / p.slab_parts) * plan.ny;
    const int slab_end = (plan.slabs * (p.slab_part + 1) / p.slab_parts) * plan.ny;
    const int slab = slab_first + (int)blockIdx.y;
    if (slab >= slab_end) return;
    const LevelGeom lv = lv_s;
    const unsigned int count = p.bin_counters[(size_t)b * kMaxSlabs + slab];
    const unsigned int offset = p.bin_counters[(size_t)(p.B + b) * kMaxSlabs + slab];
    const uint2 *list = p.bin_entries + (size_t)b * p.bin_cap + offset;

    const int tid = threadIdx.x;
    const int gs = 1 << p.gs_log2;
    const int lane_c = tid & (gs - 1);
    const int groups_per_block = (int)blockDim.x >> p.gs_log2;
    const int LK = p.LK, K = p.K;
#ifndef FDA_BIN_SLAB_POLICY
#define FDA_BIN_SLAB_POLICY 1
#endif
    const uint64_t pol_stream = l2_policy_evict_first();
    const uint64_t pol_keep = FDA_BIN_SLAB_POLICY == 1 ? l2_policy_evict_last() : l2_policy_evict_normal();
    const int red_stride = 4 * p.lpg;
    const int lvl_first = plan.level * K;  // index of the level's first point inside a row

    // Software pipeline over this group's entries: the entry is fetched two iterations ahead, its
    // coordinates and its grad_out rows one iteration ahead, so that the dependent chain entry ->
    // coordinates / grad_out -> corner gathers costs one memory latency per iteration instead of three,
    // and the reductions (which need grad_out but not the gathers) go out while the gathers are in flight.
    const unsigned int step = gridDim.x * groups_per_block;
    const unsigned int first = blockIdx.x * groups_per_block + (tid >> p.gs_log2);
    const PT *packed_b = static_cast<const PT *>(p.packed) + (size_t)b * p.rows_per_b * (size_t)(4 * LK) + 3 * lvl_first;
    auto fetch_entry = [&](unsigned int e) -> uint2 { return e < count ? __ldcs(list + e) : make_uint2(0u, 0u); };
    auto fetch_coords = [&](const uint2 &ent, bool have, float &x, float &y, float &z) {
        x = y = z = 0.f;
        if (have) {
            const unsigned int row = ent.x / (unsigned int)K, k = ent.x - row * (unsigned int)K;
            const PT *pc = packed_b + (size_t)row * (size_t)(4 * LK) + 3 * k;
            x = load1<PT>(pc); y = load1<PT>(pc + 1); z = load1<PT>(pc + 2);
        }
    };
    // grad_out rows of an entry (own row for the dot products; for the paired scatter the team's even and odd
    // rows, whose pointers the two halves of a team exchange by shuffle).  Must be called by all 32 lanes.
    const VT *go_base = static_cast<const VT *>(p.grad_out) + (size_t)b * p.rows_per_b * (size_t)p.D;
    auto issue_go = [&](const uint2 &ent, bool have) -> typename RowGrad<VT>::Raw {
        const unsigned int row = ent.x / (unsigned int)K;
        const VT *go_own = go_base + (size_t)row * (size_t)p.D;
        const bool act = have && lane_c < p.lpg;
        if (kPair) {
            const unsigned long long mine = have ? reinterpret_cast<unsigned long long>(go_own) : 0ull;
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, mine, 4);
            const bool odd = ((tid & 31) >> 2) & 1;
            return RowGrad<VT>::issue_paired(go_own, lane_c, act, reinterpret_cast<const VT *>(odd ? other : mine),
                                             reinterpret_cast<const VT *>(odd ? mine : other), tid & 7, pol_stream);
        }
        return RowGrad<VT>::issue(go_own, lane_c, p.lpg, act, pol_stream);
    };
    uint2 ent_cur = fetch_entry(first), ent_nxt = fetch_entry(first + step);
    float x, y, z;
    fetch_coords(ent_cur, first < count, x, y, z);
    typename RowGrad<VT>::Raw go_raw = issue_go(ent_cur, first < count);
    for (unsigned int e = first, base = blockIdx.x * groups_per_block; base < count; base += step, e += step) {
        // one iteration ahead: coordinates and grad_out rows of the next entry; two ahead: the entry itself
        const uint2 ent_nn = fetch_entry(e + 2 * step);
        float xn, yn, zn;
        fetch_coords(ent_nxt, e + step < count, xn, yn, zn);
        const typename RowGrad<VT>::Raw go_raw_nxt = issue_go(ent_nxt, e + step < count);
        const bool have = e < count;
        const int row = (int)(ent_cur.x / (unsigned int)K);
        const int k = (int)(ent_cur.x - (unsigned int)row * (unsigned int)K);
        const float a = __uint_as_float(ent_cur.y);
        const bool active = have && lane_c < p.lpg;
        const size_t grow = (size_t)b * p.rows_per_b + row;
        const int g = row % p.G;
        const size_t head_elem = (size_t)b * p.N * p.GD + (size_t)g * p.D + (size_t)lv.start * p.GD;
        const VT *lvl = static_cast<const VT *>(p.value) + head_elem + (size_t)lane_c * CPL;
        float *acc_lvl = p.accum + head_elem + (size_t)lane_c * 4;
        RowGrad<VT> go;
        go.take(go_raw);
        float *acc_even = nullptr, *acc_odd = nullptr;
        if (kPair) {
            // the partner entry of this lane's team is an arbitrary other row: exchange image bases by shuffle
            const unsigned long long mine_acc = reinterpret_cast<unsigned long long>(p.accum + head_elem);
            const unsigned long long other_acc = __shfl_xor_sync(0xffffffffu, mine_acc, 4);
            const bool odd = ((tid & 31) >> 2) & 1;
            acc_even = reinterpret_cast<float *>(odd ? other_acc : mine_acc);
            acc_odd = reinterpret_cast<float *>(odd ? mine_acc : other_acc);
        }
        float gx, gy, gz, da;
        point_backward<VT, kPair>(lv, p.GD, x, y, z, a, lvl, acc_lvl, go, red_stride, active, gs, pol_keep, pol_keep,
                                  gx, gy, gz, da, acc_even, acc_odd);
        if (have && lane_c == 0) {
            PT *gr = static_cast<PT *>(p.grad_packed) + grow * (size_t)(4 * LK);
            const int i = lvl_first + k;
            store1<PT>(gr + 3 * i, gx); store1<PT>(gr + 3 * i + 1, gy); store1<PT>(gr + 3 * i + 2, gz);
            if (p.dalpha) p.dalpha[grow * (size_t)LK + i] = da;  // unrounded, for the soft-max backward of the final launch
            else store1<PT>(gr + 3 * LK + i, da);
        }
        ent_cur = ent_nxt; ent_nxt = ent_nn;
        x = xn; y = yn; z = zn;
        go_raw = go_raw_nxt;
    }
}

}  // namespace fda
