// Cell-sorted backward for 16-bit values with 32 channels per head (rows of exactly four lanes).
//
// Every sampling point of a call is sorted by the cell of the pyramid it falls in (and its head); the sorted list is
// then walked so that consecutive points read the same eight value rows and add into the same eight rows of the fp32
// gradient image.  A lane group keeps both sets of rows in registers for as long as the cell does not change: eight
// gathers and eight reductions per RUN of equal cells instead of per POINT.
//
// Why: a (cell, head) row receives Q*K / cells contributions (9 / 73 / 584 on a 32x64x256 / 16x32x128 / 8x16x64
// pyramid with K = 8 points per level and one query per cell), and the plain and the slab-binned kernels are bound by
// exactly those gathers and reductions (the request path from the SMs to L2), not by HBM.
//
//   fda_sort_pass_kernel<count> rows staged like in fda_backward_kernel; one counter per (batch, cell, head)
//   fda_scan_*                exclusive scan of the counters (three small kernels, no waiting between blocks)
//   fda_sort_pass_kernel<fill> soft-max of the row; position = atomicAdd(counter of the point's bin); files the point
//                             there as one 32-byte record (one 256-bit store)
//   fda_sorted_walk_kernel    grid (x, batch): lane groups walk segments of the sorted list of the launch's levels.
//                             Everything a point needs from global memory (its grad_output row, and the eight value
//                             rows when it starts a run) is copied asynchronously into shared memory a few points
//                             ahead.  The eight dot products <value row, grad_output row> of a point are warp-level
//                             matrix instructions; the gradient image rows are accumulated in registers and sent with
//                             one reduction per corner when the run ends.  Writes {d/dx, d/dy, d/dz, dalpha} of the
//                             point into a row-ordered array (a scattered 16-byte store: the walk has DRAM bandwidth
//                             to spare, the pass that follows would pay 64 bytes per random 16-byte read).
//   fda_sort_finalize_kernel  per row: its points' results (contiguous), soft-max backward, finished row of
//                             grad_sampling_loc_attn, coalesced
//
// A launch over a level range that is not the first of a sequence (`resume`) re-uses the list made by the first.
// Nothing here waits on another block.  No counterpart in the reference (its backward is one thread group per query
// and head with atomicAdd per corner and channel, csrc/cuda/flash_deform_col2im_cuda.cuh:248-429).
#pragma once

#include "fda_backward.cuh"

namespace fda {

constexpr int kScanItems = 8;                         // counters per thread of a scan block
constexpr int kScanThreads = 1024;
constexpr int kScanTile = kScanItems * kScanThreads;  // counters per scan block
constexpr unsigned int kNoPosition = 0xffffffffu;     // a point without a corner inside its level
constexpr int kWalkSlot = 9;                          // 16-byte vectors per lane and point: grad_output row + eight value rows

// What the count and the fill pass agree on: bin and geometry tags of a point from its voxel coordinates.
struct SortTag {
    bool ok;             // some corner lies inside the level
    unsigned int bin;    // (first cell of the level + base cell clamped to the level) * G + head
    unsigned int in8;    // bit n: corner n = dz*4 + dy*2 + dx lies inside the level
    unsigned int off0;   // element offset of the (unclamped) base corner inside the level, modulo 2^32
};
__device__ __forceinline__ SortTag sort_tag_of(const LevelGeom &lv, int G, int GD, unsigned int g, float xv, float yv, float zv) {
    SortTag t;
    const float xf = floorf(xv), yf = floorf(yv), zf = floorf(zv);
    // an axis has a corner in range iff floor in [-1, size-1]; written so that NaN fails
    t.ok = (xf >= -1.f) && (xf <= lv.fW - 1.0f) && (yf >= -1.f) && (yf <= lv.fH - 1.0f) && (zf >= -1.f) && (zf <= lv.fD - 1.0f);
    t.bin = 0u; t.in8 = 0u; t.off0 = 0u;
    if (!t.ok) return t;
    const int x0 = (int)xf, y0 = (int)yf, z0 = (int)zf;  // in [-1, size-1]
    const unsigned int cx = x0 < 0 ? 0u : (unsigned int)x0, cy = y0 < 0 ? 0u : (unsigned int)y0, cz = z0 < 0 ? 0u : (unsigned int)z0;
    t.bin = ((unsigned int)lv.start + (cz * (unsigned int)lv.H + cy) * (unsigned int)lv.W + cx) * (unsigned int)G + g;
    const unsigned int mx = (unsigned int)(x0 >= 0) | (unsigned int)(x0 + 1 < lv.W) << 1;        // corners dx = 0, 1
    const unsigned int mxy = (y0 >= 0 ? mx : 0u) | (y0 + 1 < lv.H ? mx << 2 : 0u);              // dy*2 + dx
    t.in8 = (z0 >= 0 ? mxy : 0u) | (z0 + 1 < lv.D ? mxy << 4 : 0u);                             // dz*4 + dy*2 + dx
    const uint32_t sx = (uint32_t)GD, sy = (uint32_t)lv.W * sx, sz = (uint32_t)lv.H * sy;
    t.off0 = (uint32_t)z0 * sz + (uint32_t)y0 * sy + (uint32_t)x0 * sx;  // wraps for index -1; + stride wraps back
    return t;
}

// One 32-byte list record as ONE streaming store (sm_100: 256-bit vector store); `rec` is 32-byte aligned.
__device__ __forceinline__ void store_record(float4 *rec, const float4 &a, const float4 &b) {
    asm volatile("st.global.cs.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(rec), "f"(a.x), "f"(a.y), "f"(a.z), "f"(a.w),
                 "f"(b.x), "f"(b.y), "f"(b.z), "f"(b.w) : "memory");
}

// kFill = false: counts the points of every bin.  kFill = true: the counters hold the exclusive scan; files the points.
template <typename PT, bool kFill>
__global__ void __launch_bounds__(kThreads) fda_sort_pass_kernel(const Problem p) {
    __shared__ LevelGeom geom[kMaxLevels];
    extern __shared__ __align__(16) float smem_tile[];
    const int tid = threadIdx.x;
    if (tid == 0) build_level_table(geom, p.shapes, p.lsi, p.L, p.GD, p.value_elem_bytes, false, 0ull);
    const int b = blockIdx.y;
    const int gs = 1 << p.gs_log2;
    const int lane = tid & 31, warp = tid >> 5;
    const int lane_c = tid & (gs - 1);
    const int rows_per_block = (int)blockDim.x >> p.gs_log2;
    const int rows_per_warp = 32 >> p.gs_log2;
    const int row = blockIdx.x * rows_per_block + (tid >> p.gs_log2);
    const int LK = p.LK;
    const int first = blockIdx.x * rows_per_block + warp * rows_per_warp;
    float *wtile = smem_tile + warp * rows_per_warp * p.row_stride;
    int nrows = p.rows_per_b - first;
    nrows = nrows < 0 ? 0 : (nrows > rows_per_warp ? rows_per_warp : nrows);
    stage_rows<PT>(static_cast<const PT *>(p.packed) + ((size_t)b * p.rows_per_b + first) * (size_t)(4 * LK), wtile, nrows,
                   LK, p.row_stride, lane);
    __syncthreads();  // level table and this warp's tile visible
    if (row >= p.rows_per_b) return;
    const float *trow = wtile + (lane >> p.gs_log2) * p.row_stride;
    const unsigned int g = (unsigned int)(row % p.G);
    unsigned int *counters = p.sort_counters + (size_t)b * ((size_t)p.N * p.G);
    float m = 0.f, inv = 0.f;
    if (kFill) {
        m = -INFINITY;
        for (int j = 0; j < (LK >> 2); ++j) {
            const float4 lg = *reinterpret_cast<const float4 *>(trow + 3 * LK + 4 * j);
            m = fmaxf(m, fmaxf(fmaxf(lg.x, lg.y), fmaxf(lg.z, lg.w)));
        }
        float s = 0.f;
        for (int j = 0; j < (LK >> 2); ++j) {
            const float4 lg = *reinterpret_cast<const float4 *>(trow + 3 * LK + 4 * j);
            s += __expf(lg.x - m) + __expf(lg.y - m) + __expf(lg.z - m) + __expf(lg.w - m);
        }
        inv = 1.0f / s;
    }
    const size_t rowg = (size_t)b * p.rows_per_b + row;
    // Eight points at a time: all position requests go out before the first answer is needed.  Only the positions are
    // kept across the two loops; recomputing a point's coordinates and tags is cheaper than the registers that would
    // hold them (occupancy is what hides the latency of the requests).
    constexpr int kBatch = 8;
    for (int i0 = lane_c; i0 < LK; i0 += kBatch * gs) {
        unsigned int pos[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const int i = i0 + u * gs;
            pos[u] = kNoPosition;
            if (i < LK) {
                const LevelGeom lv = geom[(i >> 2) >> p.k_shift];
                const SortTag tag = sort_tag_of(lv, p.G, p.GD, g, unnormalize(trow[3 * i], lv.fW), unnormalize(trow[3 * i + 1], lv.fH),
                                                unnormalize(trow[3 * i + 2], lv.fD));
                if (tag.ok) {
                    if (kFill) pos[u] = atomicAdd(counters + tag.bin, 1u);
                    else atomicAdd(counters + tag.bin, 1u);
                }
            }
        }
        if (kFill) {
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const int i = i0 + u * gs;
                if (i < LK) {
                    if (pos[u] != kNoPosition) {
                        const int l = (i >> 2) >> p.k_shift;
                        const LevelGeom lv = geom[l];
                        const float xv = unnormalize(trow[3 * i], lv.fW), yv = unnormalize(trow[3 * i + 1], lv.fH),
                                    zv = unnormalize(trow[3 * i + 2], lv.fD);
                        const SortTag tag = sort_tag_of(lv, p.G, p.GD, g, xv, yv, zv);
                        // one 32-byte record = one whole sector (no read-modify-write behind the store)
                        const unsigned int meta = (unsigned int)l | (g << 4) | (tag.in8 << 20);
                        store_record(p.sort_entries + 2 * (size_t)pos[u], make_float4(xv, yv, zv, __expf(trow[3 * LK + i] - m) * inv),
                                     make_float4(__uint_as_float((unsigned int)rowg), __uint_as_float(meta), __uint_as_float(tag.off0),
                                                 __uint_as_float((unsigned int)i)));
                    }
                }
            }
        }
    }
}

// ---- exclusive scan of n counters, in place: tile sums -> scan of the sums (one block) -> scan of every tile ----
__device__ __forceinline__ unsigned int block_exclusive_scan(unsigned int v, unsigned int *warp_sums, unsigned int &total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned int inc = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const unsigned int t = __shfl_up_sync(0xffffffffu, inc, d);
        if (lane >= d) inc += t;
    }
    if (lane == 31) warp_sums[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        unsigned int w = lane < (int)(blockDim.x >> 5) ? warp_sums[lane] : 0u;
        unsigned int winc = w;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const unsigned int t = __shfl_up_sync(0xffffffffu, winc, d);
            if (lane >= d) winc += t;
        }
        warp_sums[lane] = winc - w;                 // exclusive offset of each warp
        if (lane == 31) warp_sums[32] = winc;       // block total
    }
    __syncthreads();
    total = warp_sums[32];
    const unsigned int r = warp_sums[warp] + inc - v;
    __syncthreads();  // warp_sums may be re-used by the caller's next round
    return r;
}

__global__ void __launch_bounds__(kScanThreads) fda_scan_tile_sums_kernel(const unsigned int *__restrict__ data, size_t n,
                                                                         unsigned int *__restrict__ tile_sums) {
    __shared__ unsigned int warp_sums[33];
    const size_t base = (size_t)blockIdx.x * kScanTile + (size_t)threadIdx.x * kScanItems;
    unsigned int s = 0;
#pragma unroll
    for (int k = 0; k < kScanItems; ++k) s += base + k < n ? data[base + k] : 0u;
    unsigned int total;
    (void)block_exclusive_scan(s, warp_sums, total);
    if (threadIdx.x == 0) tile_sums[blockIdx.x] = total;
}

__global__ void __launch_bounds__(kScanThreads) fda_scan_spine_kernel(unsigned int *tile_sums, unsigned int tiles) {
    __shared__ unsigned int warp_sums[33];
    unsigned int carry = 0;
    for (unsigned int base = 0; base < tiles; base += kScanThreads) {  // uniform trip count
        const unsigned int i = base + threadIdx.x;
        const unsigned int v = i < tiles ? tile_sums[i] : 0u;
        unsigned int total;
        const unsigned int ex = block_exclusive_scan(v, warp_sums, total);
        if (i < tiles) tile_sums[i] = carry + ex;
        carry += total;
    }
}

__global__ void __launch_bounds__(kScanThreads) fda_scan_apply_kernel(unsigned int *__restrict__ data, size_t n,
                                                                     const unsigned int *__restrict__ tile_offsets) {
    __shared__ unsigned int warp_sums[33];
    const size_t base = (size_t)blockIdx.x * kScanTile + (size_t)threadIdx.x * kScanItems;
    unsigned int v[kScanItems];
    unsigned int s = 0;
#pragma unroll
    for (int k = 0; k < kScanItems; ++k) {
        v[k] = base + k < n ? data[base + k] : 0u;
        s += v[k];
    }
    unsigned int total;
    unsigned int run = tile_offsets[blockIdx.x] + block_exclusive_scan(s, warp_sums, total);
#pragma unroll
    for (int k = 0; k < kScanItems; ++k) {
        if (base + k < n) data[base + k] = run;
        run += v[k];
    }
}

// ---- the walk over the sorted list ---------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(void *smem, const void *gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"((unsigned int)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
// the same through L2 only: for rows that are read once (they would only push re-used rows out of L1)
__device__ __forceinline__ void cp_async16_once(void *smem, const void *gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned int)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory");
}

// <value row, grad_output row> as warp-level matrix instructions: the four lanes of row group g hold row g of the A
// fragment (their 16-byte vectors of a value row ARE the fragment, no unpacking) and column g of the B fragment (their
// vectors of the grad_output row), so D[g][g] of an m16n8k16 product is the dot product over 16 channels, summed over
// the group's lanes.  Two corners ride in one instruction (fragment rows g and g + 8), two instructions cover the 32
// channels.  The other 7/8 of each product (row g against the grad_output of the other groups) is discarded.
// `first`: d = A * B (zero accumulator input); `mma`: c += A * B.
#define FDA_MMA_DOT(TYPES)                                                                                                             \
    static __device__ __forceinline__ void first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,      \
                                                 uint32_t b1) {                                                                         \
        asm("mma.sync.aligned.m16n8k16.row.col." TYPES " {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"           \
            : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));       \
    }                                                                                                                                   \
    static __device__ __forceinline__ void mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,        \
                                               uint32_t b1) {                                                                           \
        asm("mma.sync.aligned.m16n8k16.row.col." TYPES " {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"               \
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));                 \
    }
template <typename VT> struct MmaDot;
template <> struct MmaDot<__nv_bfloat16> { FDA_MMA_DOT("f32.bf16.bf16.f32") };
template <> struct MmaDot<__half> { FDA_MMA_DOT("f32.f16.f16.f32") };
#undef FDA_MMA_DOT

// Work unit: a segment of S consecutive list entries per lane group; the groups of a warp take consecutive segments, so a
// warp's share of one round is one contiguous span of the list, which it first copies to shared memory (coalesced).
// Shared memory: [warps][span] 32-byte records, then per lane a ring of kAhead slots of kWalkSlot 16-byte vectors.
// kAhead: points whose rows are in flight per lane.
template <typename VT, int kBlock, int kMinBlocks, int kAhead>
__global__ void __launch_bounds__(kBlock, kMinBlocks) fda_sorted_walk_kernel(const Problem p) {
    static_assert(Vec16<VT>::kCPL == 8, "16-bit value dtypes only");
    constexpr unsigned int kNoRun = 0xffffffffu;
    __shared__ LevelGeom geom[kMaxLevels];
    __shared__ unsigned int s_begin, s_end;
    extern __shared__ __align__(16) float smem_tile[];
    const int tid = threadIdx.x;
    const int b = blockIdx.y;
    if (tid == 0) {
        build_level_table(geom, p.shapes, p.lsi, p.L, p.GD, p.value_elem_bytes, true, p.l2_keep_bytes);
        // The launch's levels are a contiguous range, and the list is ordered (batch, level, cell, head): its entries
        // are one contiguous span per batch element.  After the fill pass a counter holds the END of its bin, i.e.
        // the start of the next one.
        const int lb = __ffs(p.level_mask) - 1, le = 32 - __clz(p.level_mask);
        const unsigned long long NG = (unsigned long long)p.N * p.G;
        const unsigned long long kf = (unsigned long long)b * NG + (unsigned long long)p.lsi[lb] * p.G;
        const unsigned long long ke = (unsigned long long)b * NG + (unsigned long long)(le < p.L ? p.lsi[le] : (long long)p.N) * p.G;
        s_begin = kf ? p.sort_counters[kf - 1] : 0u;
        s_end = ke ? p.sort_counters[ke - 1] : 0u;
    }
    __syncthreads();
    const unsigned int e_begin = s_begin, e_end = s_end;
    if (e_end <= e_begin) return;
    const int lane = tid & 31, warp = tid >> 5;
    const int tig = lane & 3, grp = lane >> 2;  // lane inside the row group, row group inside the warp
    const int owner = grp >> 1;                 // the lane of the group that ends up with D[g][g] (c[g & 1]) and D[g + 8][g] (c[2 + (g & 1)])
    const bool odd = grp & 1;
    const unsigned int warps_per_block = blockDim.x >> 5;
    const unsigned int S = (unsigned int)p.sort_seg;
    const unsigned int span = S * 8u;  // list entries a warp takes at a time
    const unsigned int nspan = (e_end - e_begin + span - 1) / span;
    const uint64_t pol_keep = l2_policy_evict_last(), pol_stream = l2_policy_evict_first();
    const VT *go_base = static_cast<const VT *>(p.grad_out) + (size_t)tig * 8;
    const VT *value_b = static_cast<const VT *>(p.value) + (size_t)b * p.N * p.GD + (size_t)tig * 8;
    float *image_b = p.accum + (size_t)b * p.N * p.GD + (size_t)tig * 8;
    // a group's segment starts (2 * S + 1) vectors after its neighbour's: the eight groups of a warp read their records
    // from eight different bank quads
    const unsigned int seg_stride = 2u * S + 1u;
    float4 *ent_s = reinterpret_cast<float4 *>(smem_tile) + (size_t)warp * 8u * seg_stride;
    uint4 *ring = reinterpret_cast<uint4 *>(smem_tile) + (size_t)warps_per_block * 8u * seg_stride + tid;  // vector v of slot k: ring[(k * kWalkSlot + v) * blockDim.x]

    float acc[8][8];
    uint4 va[8];                                   // the run's eight value rows (this lane's channels), zero where outside the level
    unsigned int run_off = 0u, run_meta = kNoRun;  // base offset of the run's cell; level | head << 4 | corner mask << 20

    // sends the run's eight image rows to memory and clears them
    auto flush = [&]() {
        if (run_meta != kNoRun) {
            const LevelGeom lv = geom[run_meta & 15u];
            const uint32_t sx = (uint32_t)p.GD, sy = (uint32_t)lv.W * sx, sz = (uint32_t)lv.H * sy;
            float *img = image_b + (size_t)lv.start * p.GD + (size_t)((run_meta >> 4) & 0xffffu) * p.D;
            const uint64_t pol = (lv.keep & 2) ? pol_keep : pol_stream;
            const unsigned int in8 = run_meta >> 20;
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                const bool in = (in8 >> n) & 1u;
                if (in) {
                    float *dst = img + (uint32_t)(run_off + ((n & 4) ? sz : 0u) + ((n & 2) ? sy : 0u) + ((n & 1) ? sx : 0u));
                    red_add_f32x4_hint(dst, acc[n][0], acc[n][1], acc[n][2], acc[n][3], pol);
                    red_add_f32x4_hint(dst + 4, acc[n][4], acc[n][5], acc[n][6], acc[n][7], pol);
                }
            }
        }
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int c = 0; c < 8; ++c) acc[n][c] = 0.f;
    };
    flush();  // clears the accumulators
#pragma unroll
    for (int n = 0; n < 8; ++n) va[n] = make_uint4(0u, 0u, 0u, 0u);

    for (unsigned int sp = blockIdx.x * warps_per_block + warp; sp < nspan; sp += gridDim.x * warps_per_block) {
        const unsigned int w0 = e_begin + sp * span;
        const unsigned int wn = (e_end - w0 < span) ? e_end - w0 : span;  // entries of this warp's span
        __syncwarp();  // the readers of the previous span are done with the records
        for (unsigned int v = lane; v < 2 * wn; v += 32) {
            const unsigned int sg = v / (2u * S);
            ent_s[sg * seg_stride + (v - sg * 2u * S)] = __ldcs(p.sort_entries + 2 * (size_t)w0 + v);
        }
        __syncwarp();
        const unsigned int t0 = (unsigned int)grp * S;  // this group's segment inside the span
        const unsigned int tn = t0 < wn ? (wn - t0 < S ? wn - t0 : S) : 0u;
        const float4 *ent_g = ent_s + (unsigned int)grp * seg_stride;

        // Asks for everything point t needs from global memory: its grad_output row, and -- when it starts a run, i.e.
        // its cell or head differs from the previous point's or it is the first of the segment -- the eight value rows.
        // Every lane commits one (possibly empty) copy group per point, so that "all but the newest kAhead - 1 groups
        // are complete" always means "the rows of the current point have arrived".
        auto request = [&](unsigned int t) {
            if (t < tn) {
                const float4 tag = ent_g[2 * t + 1];
                uint4 *slot = ring + (size_t)((t % (unsigned int)kAhead) * kWalkSlot) * blockDim.x;
                cp_async16_once(slot, go_base + (size_t)__float_as_uint(tag.x) * (size_t)p.D);
                const unsigned int meta = __float_as_uint(tag.y), off0 = __float_as_uint(tag.z);
                bool starts = t == 0;
                if (!starts) {
                    const float4 prev = ent_g[2 * t - 1];
                    starts = __float_as_uint(prev.y) != meta || __float_as_uint(prev.z) != off0;
                }
                if (starts) {
                    const LevelGeom lv = geom[meta & 15u];
                    const uint32_t sx = (uint32_t)p.GD, sy = (uint32_t)lv.W * sx, sz = (uint32_t)lv.H * sy;
                    const VT *lvl = value_b + (size_t)lv.start * p.GD + (size_t)((meta >> 4) & 0xffffu) * p.D;
                    const unsigned int in8 = meta >> 20;
#pragma unroll
                    for (int n = 0; n < 8; ++n) {
                        const bool in = (in8 >> n) & 1u;
                        if (in) cp_async16(slot + (size_t)(1 + n) * blockDim.x,
                                           lvl + (uint32_t)(off0 + ((n & 4) ? sz : 0u) + ((n & 2) ? sy : 0u) + ((n & 1) ? sx : 0u)));
                    }
                }
            }
            cp_async_commit();
        };
        for (unsigned int k = 0; k < (unsigned int)kAhead; ++k) request(k);
        for (unsigned int t = 0; t < S; ++t) {  // uniform trip count: the matrix instructions need the whole warp
            const bool have = t < tn;
            float4 ent = make_float4(0.f, 0.f, 0.f, 0.f), tag = ent;
            if (have) {
                ent = ent_g[2 * t];       // voxel x, y, z, probability
                tag = ent_g[2 * t + 1];   // row, level | head << 4 | corner mask << 20, base offset, point index inside the row
            }
            const unsigned int meta = __float_as_uint(tag.y), off0 = __float_as_uint(tag.z);
            cp_async_wait<kAhead - 1>();
            const uint4 *slot = ring + (size_t)((t % (unsigned int)kAhead) * kWalkSlot) * blockDim.x;
            if (have && (meta != run_meta || off0 != run_off)) {
                flush();
                run_meta = meta;
                run_off = off0;
                const unsigned int in8 = meta >> 20;
#pragma unroll
                for (int n = 0; n < 8; ++n) {
                    const bool in = (in8 >> n) & 1u;
                    va[n] = in ? slot[(size_t)(1 + n) * blockDim.x] : make_uint4(0u, 0u, 0u, 0u);
                }
            }
            uint4 gr = make_uint4(0u, 0u, 0u, 0u);
            if (have) gr = slot[0];
            // the weights of point_geometry_voxel
            const float xf = floorf(ent.x), yf = floorf(ent.y), zf = floorf(ent.z);
            const float wx[2] = {__fsub_rn(__fadd_rn(xf, 1.0f), ent.x), __fsub_rn(ent.x, xf)};
            const float wy[2] = {__fsub_rn(__fadd_rn(yf, 1.0f), ent.y), __fsub_rn(ent.y, yf)};
            const float wz[2] = {__fsub_rn(__fadd_rn(zf, 1.0f), ent.z), __fsub_rn(ent.z, zf)};
            const float a = have ? ent.w : 0.f;
            float dot[8];
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                float c[4];
                // a group without a point in this iteration multiplies stale rows with a zero grad_output row
                MmaDot<VT>::first(c, va[2 * h].x, va[2 * h + 1].x, va[2 * h].y, va[2 * h + 1].y, gr.x, gr.y);
                MmaDot<VT>::mma(c, va[2 * h].z, va[2 * h + 1].z, va[2 * h].w, va[2 * h + 1].w, gr.z, gr.w);
                dot[2 * h] = odd ? c[1] : c[0];  // meaningful in the owner lane only
                dot[2 * h + 1] = odd ? c[3] : c[2];
            }
            // Every lane does the owner's arithmetic (the warp pays for it either way): the corner weights are then
            // shared between the point's own gradients and its contribution to the image rows.
            const float wyx[4] = {wy[0] * wx[0], wy[0] * wx[1], wy[1] * wx[0], wy[1] * wx[1]};
            const float wzy[4] = {wz[0] * wy[0], wz[0] * wy[1], wz[1] * wy[0], wz[1] * wy[1]};
            const float wzx[4] = {wz[0] * wx[0], wz[0] * wx[1], wz[1] * wx[0], wz[1] * wx[1]};
            float w[8];  // corner n = dz*4 + dy*2 + dx
#pragma unroll
            for (int n = 0; n < 8; ++n) w[n] = wyx[n & 3] * wz[n >> 2];
            const float gx = wzy[0] * (dot[1] - dot[0]) + wzy[1] * (dot[3] - dot[2]) + wzy[2] * (dot[5] - dot[4]) + wzy[3] * (dot[7] - dot[6]);
            const float gy = wzx[0] * (dot[2] - dot[0]) + wzx[1] * (dot[3] - dot[1]) + wzx[2] * (dot[6] - dot[4]) + wzx[3] * (dot[7] - dot[5]);
            const float gz = wyx[0] * (dot[4] - dot[0]) + wyx[1] * (dot[5] - dot[1]) + wyx[2] * (dot[6] - dot[2]) + wyx[3] * (dot[7] - dot[3]);
            float da = 0.f;
#pragma unroll
            for (int n = 0; n < 8; ++n) da = fmaf(w[n], dot[n], da);
            if (have && tig == owner) {
                const LevelGeom lv = geom[meta & 15u];
                __stcs(p.sort_results + (size_t)__float_as_uint(tag.x) * (size_t)p.LK + __float_as_uint(tag.w),
                       make_float4(a * lv.fW * gx, a * lv.fH * gy, a * lv.fD * gz, da));
            }
            float god[8];
            Vec16<VT>::unpack(gr, god);
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                // corners outside the level collect finite garbage that flush() never sends (same run, same corners)
                const float aw = a * w[n];
#pragma unroll
                for (int c = 0; c < 8; c += 2) ffma2(acc[n][c], acc[n][c + 1], aw, aw, god[c], god[c + 1]);
            }
            request(t + kAhead);  // into the slot just read
        }
        cp_async_wait<0>();
        flush();
        run_meta = kNoRun;
    }
}

// Per row: the results of its points, soft-max backward, finished row of grad_sampling_loc_attn.  A point without a
// corner inside its level was never filed and has no result: its gradients are zero (the same test as in the fill pass).
template <typename PT>
__global__ void __launch_bounds__(kThreads) fda_sort_finalize_kernel(const Problem p) {
    __shared__ LevelGeom geom[kMaxLevels];
    extern __shared__ __align__(16) float smem_tile[];
    const int tid = threadIdx.x;
    if (tid == 0) build_level_table(geom, p.shapes, p.lsi, p.L, p.GD, p.value_elem_bytes, false, 0ull);
    const int b = blockIdx.y;
    const int gs = 1 << p.gs_log2;
    const int lane = tid & 31, warp = tid >> 5;
    const int lane_c = tid & (gs - 1);
    const int rows_per_block = (int)blockDim.x >> p.gs_log2;
    const int rows_per_warp = 32 >> p.gs_log2;
    const int row = blockIdx.x * rows_per_block + (tid >> p.gs_log2);
    const bool row_ok = row < p.rows_per_b;
    const int LK = p.LK;
    const int first = blockIdx.x * rows_per_block + warp * rows_per_warp;
    float *wtile = smem_tile + warp * rows_per_warp * p.row_stride;
    int nrows = p.rows_per_b - first;
    nrows = nrows < 0 ? 0 : (nrows > rows_per_warp ? rows_per_warp : nrows);
    const size_t warp_elem0 = ((size_t)b * p.rows_per_b + first) * (size_t)(4 * LK);
    stage_rows<PT>(static_cast<const PT *>(p.packed) + warp_elem0, wtile, nrows, LK, p.row_stride, lane);
    __syncthreads();  // level table and this warp's tile visible
    float *trow = wtile + (lane >> p.gs_log2) * p.row_stride;
    const size_t rowg = (size_t)b * p.rows_per_b + (row_ok ? row : 0);
    const unsigned int g = row_ok ? (unsigned int)(row % p.G) : 0u;
    const float4 *results = p.sort_results + rowg * (size_t)LK;
    const int rounds = (LK + gs - 1) >> p.gs_log2;  // uniform over the warp

    // Tile row layout: [0,3LK) coordinates -> coordinate gradients, [3LK,4LK) logits -> dalpha -> logit gradients,
    // [4LK,5LK) exp(logit - max).
    float m = -INFINITY;
    for (int j = 0; j < rounds; ++j) {
        const int i = lane_c + j * gs;
        if (row_ok && i < LK) m = fmaxf(m, trow[3 * LK + i]);
    }
    for (int mask = gs >> 1; mask > 0; mask >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, mask));
    float s = 0.f, S = 0.f;
    constexpr int kBatch = 8;  // the results of eight points are requested before the first one is used
    for (int j0 = 0; j0 < rounds; j0 += kBatch) {
        float4 r[kBatch];
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
            const int i = lane_c + (j0 + j) * gs;
            r[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (row_ok && i < LK) {
                const LevelGeom lv = geom[(i >> 2) >> p.k_shift];
                const SortTag tag = sort_tag_of(lv, p.G, p.GD, g, unnormalize(trow[3 * i], lv.fW), unnormalize(trow[3 * i + 1], lv.fH),
                                                unnormalize(trow[3 * i + 2], lv.fD));
                if (tag.ok) r[j] = __ldcs(results + i);
            }
        }
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
            const int i = lane_c + (j0 + j) * gs;
            if (row_ok && i < LK) {
                const float ex = __expf(trow[3 * LK + i] - m);
                trow[3 * i] = r[j].x; trow[3 * i + 1] = r[j].y; trow[3 * i + 2] = r[j].z;
                trow[3 * LK + i] = r[j].w;   // dalpha
                trow[4 * LK + i] = ex;
                s += ex;
                S = fmaf(ex, r[j].w, S);
            }
        }
    }
    for (int mask = gs >> 1; mask > 0; mask >>= 1) {
        s += __shfl_xor_sync(0xffffffffu, s, mask);
        S += __shfl_xor_sync(0xffffffffu, S, mask);
    }
    const float inv = row_ok ? 1.0f / s : 0.f;
    S *= inv;  // sum_i p_i * dalpha_i
    for (int j = 0; j < rounds; ++j) {
        const int i = lane_c + j * gs;
        if (row_ok && i < LK) trow[3 * LK + i] = trow[4 * LK + i] * inv * (trow[3 * LK + i] - S);
    }
    __syncwarp();
    PT *dst = static_cast<PT *>(p.grad_packed) + warp_elem0;
    const int nvec = nrows * LK;
    const float inv_lk = 1.0f / (float)LK;
    for (int v = lane; v < nvec; v += 32) {
        const int r = row_of_vector(v, inv_lk);
        const int c = (v - r * LK) * 4;
        store4_stream<PT>(dst + (size_t)v * 4, *reinterpret_cast<const float4 *>(wtile + r * p.row_stride + c));
    }
}

}  // namespace fda
