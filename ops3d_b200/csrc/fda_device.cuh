// Device-side building blocks shared by the forward and backward kernels of
// Flash Deformable 3D Attention for sm_100a.
//
// Thread mapping (both directions).  One "row" is one (query, head) pair of a
// batch element; its D channels are covered by `lpg` lanes that each own one
// 16-byte vector of the value dtype (8 channels for 16-bit types, 4 for fp32).
// Lanes of a row form a power-of-two group of `gs = 1 << gs_log2 >= lpg` lanes
// inside one warp (surplus lanes idle), so a warp-wide load instruction fetches
// 32/gs complete head rows (64 B each at D = 32, bf16): every 32-byte sector that
// crosses the memory system is fully used, which is what a random 8-corner
// gather can at best achieve.
//
// Coordinates follow torch.nn.functional.grid_sample(align_corners=False,
// padding_mode="zeros") bit for bit in fp32 -- un-normalisation
// ((g + 1) * size - 1) / 2 on g = 2*loc - 1, weights (x0 + 1) - x and x - x0 --
// because the parity target is the reference's PyTorch implementation
// (ops3d/flash_deform_attn.py:139-165).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fda {

constexpr int kMaxLevels = 5;
constexpr int kThreads = 256;

struct LevelGeom {
    int D, H, W;
    int start;  // first cell of the level inside one batch element
    int keep;   // bit 0: keep this level's value rows in L2, bit 1: keep its fp32 gradient image in L2
    float fD, fH, fW;  // the extents as floats (the kernels need them per point; the conversion is not free)
};

// Kernel parameter block (passed by value).
struct Problem {
    const void *value;
    const int64_t *shapes;
    const int64_t *lsi;
    const void *packed;
    void *out;              // forward only
    const void *grad_out;   // backward only
    float *accum;           // backward: fp32 image of grad_value
    void *grad_packed;      // backward
    int B, N, G, D, L, K, Q;
    int LK;          // L * K
    int k_shift;     // log2(K / 4): level of 4-point chunk j is j >> k_shift
    int gs_log2;     // log2 of lanes per row group
    int lpg;         // active lanes per row = D / channels-per-lane
    int rows_per_b;  // Q * G
    int GD;          // G * D
    int row_stride;  // floats per staged row in shared memory
    int head_group;  // forward: heads per group of the group-by-group row order (G: plain row order)
    unsigned long long l2_keep_bytes;  // how much per-batch-element data may be marked "evict last" in L2
    int value_elem_bytes;              // sizeof(value dtype)
    // backward only
    int level_mask;  // bit l set: the points of level l are processed by this launch
    int resume;      // slots of the other levels are taken from grad_packed (written by an earlier launch)
    int finalize;    // apply the soft-max backward to the logit slots (last launch over these rows)
    // backward, slab-binned handling of the largest level (see fda_backward_binned.cuh)
    int bin_allowed;                     // host says scratch is available and the image exceeds the L2 budget
    unsigned long long bin_slab_bytes;   // target bytes of one slab of the fp32 image
    unsigned int *bin_counters;          // [3][B][kMaxSlabs]: count, offset, cursor
    uint2 *bin_entries;                  // [B][bin_cap]: {row * K + k, soft-max probability}
    unsigned long long bin_cap;          // entries per batch element = rows_per_b * K
    int slab_part, slab_parts;           // the binned kernel of this launch covers slabs [S*part/parts, S*(part+1)/parts)
    int binned_elsewhere;                // the binned launches for this call were issued separately (plain kernel only)
    // fp32 plane [B][rows_per_b][LK] that carries raw dalpha from launch to launch (binned -> plain, level range ->
    // level range); null: the logit slots of grad_packed carry it (exact only when the packed dtype is fp32)
    float *dalpha;
    // backward, cell-sorted handling of all levels (see fda_backward_sorted.cuh); null: not used
    unsigned int *sort_counters;   // [B*N*G]: points per (batch, cell, head) -> exclusive scan -> end of each bin
    unsigned int *sort_tile_sums;  // scratch of the scan
    float4 *sort_entries;          // sorted list, 32 bytes per point: {voxel x, y, z inside the point's level, soft-max
                                   // probability} {row b*Q*G + q*G + g, level | head << 4 | corner mask << 20, element
                                   // offset of the base corner, index of the point inside its row}
    float4 *sort_results;          // [B*Q*G][L*K] in row order: {d/dx, d/dy, d/dz, dalpha} of every filed point
    int sort_seg;                  // list entries one lane group walks before it flushes its accumulators
};

constexpr int kMaxSlabs = 128;

// Which level (if any) is handled slab by slab, and how it is cut: along z into `slabs` slabs of `depth`
// planes, and -- when a single plane is still larger than the target -- each slab along y into `ny` bricks
// of `ydepth` rows.  Brick index = z-slab * ny + y-part; there are slabs * ny <= kMaxSlabs bricks.  A pure
// function of the shapes and launch parameters, so every kernel of one backward call -- and the host, when
// it has a host copy of the shapes -- derives the same plan.
struct BinPlan {
    int level, enabled, slabs, depth, ny, ydepth;
};
__host__ __device__ inline BinPlan bin_plan_from(const int64_t *shapes, int L, int GD, unsigned long long l2_keep_bytes,
                                                 unsigned long long slab_bytes, int level_mask, int allowed) {
    BinPlan plan;
    plan.level = 0; plan.enabled = 0; plan.slabs = 1; plan.depth = 1; plan.ny = 1; plan.ydepth = 1 << 30;
    if (!allowed) return plan;
    unsigned long long best = 0;
    for (int l = 0; l < L; ++l) {
        const unsigned long long c = (unsigned long long)shapes[3 * l] * shapes[3 * l + 1] * shapes[3 * l + 2];
        if (c > best) { best = c; plan.level = l; }
    }
    const unsigned long long image_bytes = best * (unsigned long long)GD * 4ull;
    const int Dz = (int)shapes[3 * plan.level], H = (int)shapes[3 * plan.level + 1];
    if (!((level_mask >> plan.level) & 1) || image_bytes <= l2_keep_bytes || Dz < 2) return plan;
    unsigned long long want = (image_bytes + slab_bytes - 1) / slab_bytes;
    if (want > (unsigned long long)kMaxSlabs) want = kMaxSlabs;
    if (want > (unsigned long long)Dz) want = Dz;
    if (want < 2) want = 2;
    plan.depth = (Dz + (int)want - 1) / (int)want;
    plan.slabs = (Dz + plan.depth - 1) / plan.depth;
    if (plan.depth == 1) {  // one plane per slab and possibly still too large: cut the planes along y
        const unsigned long long plane_bytes = image_bytes / (unsigned long long)Dz;
        unsigned long long ny = (plane_bytes + slab_bytes - 1) / slab_bytes;
        const unsigned long long room = (unsigned long long)(kMaxSlabs / plan.slabs);
        if (ny > room) ny = room;
        if (ny > (unsigned long long)H) ny = H;
        if (ny > 1) {
            plan.ydepth = (H + (int)ny - 1) / (int)ny;
            plan.ny = (H + plan.ydepth - 1) / plan.ydepth;
        }
    }
    plan.enabled = 1;
    return plan;
}
__device__ __forceinline__ BinPlan make_bin_plan(const Problem &p) {
    return bin_plan_from(p.shapes, p.L, p.GD, p.l2_keep_bytes, p.bin_slab_bytes, p.level_mask, p.bin_allowed);
}

// ---------------------------------------------------------------------------
// dtype traits: one 16-byte vector of the value dtype <-> fp32 registers
// ---------------------------------------------------------------------------
template <typename T> struct Vec16;

template <> struct Vec16<float> {
    static constexpr int kCPL = 4;
    static __device__ __forceinline__ void unpack(const uint4 &r, float (&v)[4]) {
        v[0] = __uint_as_float(r.x); v[1] = __uint_as_float(r.y);
        v[2] = __uint_as_float(r.z); v[3] = __uint_as_float(r.w);
    }
    static __device__ __forceinline__ uint4 pack(const float (&v)[4]) {
        return make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
    }
};

template <> struct Vec16<__nv_bfloat16> {
    static constexpr int kCPL = 8;
    static __device__ __forceinline__ void unpack(const uint4 &r, float (&v)[8]) {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {  // bf16 is the high half of an fp32
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ uint4 pack(const float (&v)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t *>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
};

template <> struct Vec16<__half> {
    static constexpr int kCPL = 8;
    static __device__ __forceinline__ void unpack(const uint4 &r, float (&v)[8]) {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ uint4 pack(const float (&v)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t *>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
};

// Packed fp32 x2 fused multiply-add (sm_100: one instruction for two lanes of fp32, same rounding as fmaf).
__device__ __forceinline__ void ffma2(float &d0, float &d1, float a0, float a1, float b0, float b1) {
    unsigned long long ra, rb, rd;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a0), "f"(a1));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b0), "f"(b1));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rd) : "f"(d0), "f"(d1));
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(rd) : "l"(ra), "l"(rb));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d0), "=f"(d1) : "l"(rd));
}

// acc[k] += w * v[k] for one 16-byte vector of the value dtype, two channels per instruction
template <typename VT>
__device__ __forceinline__ void axpy16(const uint4 &raw, float w, float (&acc)[Vec16<VT>::kCPL]) {
    float v[Vec16<VT>::kCPL];
    Vec16<VT>::unpack(raw, v);
#ifdef FDA_NO_FFMA2
#pragma unroll
    for (int k = 0; k < Vec16<VT>::kCPL; ++k) acc[k] = fmaf(w, v[k], acc[k]);
#else
#pragma unroll
    for (int k = 0; k < Vec16<VT>::kCPL; k += 2) ffma2(acc[k], acc[k + 1], w, w, v[k], v[k + 1]);
#endif
}

// Four consecutive elements (aligned to four elements) <-> float4.
template <typename T> __device__ __forceinline__ float4 load4(const T *p);
template <> __device__ __forceinline__ float4 load4<float>(const float *p) {
    return __ldg(reinterpret_cast<const float4 *>(p));
}
template <> __device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16 *p) {
    const uint2 r = __ldg(reinterpret_cast<const uint2 *>(p));
    return make_float4(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xffff0000u),
                       __uint_as_float(r.y << 16), __uint_as_float(r.y & 0xffff0000u));
}
template <> __device__ __forceinline__ float4 load4<__half>(const __half *p) {
    const uint2 r = __ldg(reinterpret_cast<const uint2 *>(p));
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&r.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&r.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

template <typename T> __device__ __forceinline__ void store4(T *p, const float4 &v);
template <> __device__ __forceinline__ void store4<float>(float *p, const float4 &v) {
    *reinterpret_cast<float4 *>(p) = v;
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16 *p, const float4 &v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2 *>(p) = make_uint2(*reinterpret_cast<uint32_t *>(&a), *reinterpret_cast<uint32_t *>(&b));
}
template <> __device__ __forceinline__ void store4<__half>(__half *p, const float4 &v) {
    __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
    *reinterpret_cast<uint2 *>(p) = make_uint2(*reinterpret_cast<uint32_t *>(&a), *reinterpret_cast<uint32_t *>(&b));
}

// Streaming (read-once / write-once, evict-first) variants for the per-query rows.
template <typename T> __device__ __forceinline__ float4 load4_stream(const T *p);
template <> __device__ __forceinline__ float4 load4_stream<float>(const float *p) {
    return __ldcs(reinterpret_cast<const float4 *>(p));
}
template <> __device__ __forceinline__ float4 load4_stream<__nv_bfloat16>(const __nv_bfloat16 *p) {
    const uint2 r = __ldcs(reinterpret_cast<const uint2 *>(p));
    return make_float4(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xffff0000u),
                       __uint_as_float(r.y << 16), __uint_as_float(r.y & 0xffff0000u));
}
template <> __device__ __forceinline__ float4 load4_stream<__half>(const __half *p) {
    const uint2 r = __ldcs(reinterpret_cast<const uint2 *>(p));
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&r.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&r.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
template <typename T> __device__ __forceinline__ void store4_stream(T *p, const float4 &v);
template <> __device__ __forceinline__ void store4_stream<float>(float *p, const float4 &v) {
    __stcs(reinterpret_cast<float4 *>(p), v);
}
template <> __device__ __forceinline__ void store4_stream<__nv_bfloat16>(__nv_bfloat16 *p, const float4 &v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    __stcs(reinterpret_cast<uint2 *>(p), make_uint2(*reinterpret_cast<uint32_t *>(&a), *reinterpret_cast<uint32_t *>(&b)));
}
template <> __device__ __forceinline__ void store4_stream<__half>(__half *p, const float4 &v) {
    __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
    __stcs(reinterpret_cast<uint2 *>(p), make_uint2(*reinterpret_cast<uint32_t *>(&a), *reinterpret_cast<uint32_t *>(&b)));
}

// One element <-> fp32.
template <typename PT> __device__ __forceinline__ float load1(const PT *p);
template <> __device__ __forceinline__ float load1<float>(const float *p) { return __ldg(p); }
template <> __device__ __forceinline__ float load1<__nv_bfloat16>(const __nv_bfloat16 *p) {
    return __uint_as_float((uint32_t)__ldg(reinterpret_cast<const unsigned short *>(p)) << 16);
}
template <> __device__ __forceinline__ float load1<__half>(const __half *p) {
    return __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short *>(p))));
}
template <typename PT> __device__ __forceinline__ void store1(PT *p, float v);
template <> __device__ __forceinline__ void store1<float>(float *p, float v) { *p = v; }
template <> __device__ __forceinline__ void store1<__nv_bfloat16>(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ void store1<__half>(__half *p, float v) { *p = __float2half_rn(v); }

// L2 eviction-priority policies.  The gather re-reads small pyramid levels hundreds of times while
// the largest level and the per-query rows stream through once; marking the former "evict last"
// and the latter "evict first" keeps the re-used levels resident in the 126 MB L2.
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ uint64_t l2_policy_evict_normal() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
// 16-byte read-only gather load with an L2 eviction policy.
__device__ __forceinline__ uint4 ldg16_hint(const void *p, uint64_t pol) {
    uint4 r;
    asm("ld.global.nc.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;"
        : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p), "l"(pol));
    return r;
}
// The same load, kept in program order relative to the reductions that follow it (see point_backward).
__device__ __forceinline__ uint4 ldg16_hint_ordered(const void *p, uint64_t pol) {
    uint4 r;
    asm volatile("ld.global.nc.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p), "l"(pol));
    return r;
}
// Four consecutive elements as raw bits (x, y used for 16-bit types), and their conversion to fp32.
template <typename T> __device__ __forceinline__ uint4 load4_raw(const T *p);
template <> __device__ __forceinline__ uint4 load4_raw<float>(const float *p) {
    return __ldg(reinterpret_cast<const uint4 *>(p));
}
template <> __device__ __forceinline__ uint4 load4_raw<__nv_bfloat16>(const __nv_bfloat16 *p) {
    const uint2 r = __ldg(reinterpret_cast<const uint2 *>(p));
    return make_uint4(r.x, r.y, 0u, 0u);
}
template <> __device__ __forceinline__ uint4 load4_raw<__half>(const __half *p) {
    const uint2 r = __ldg(reinterpret_cast<const uint2 *>(p));
    return make_uint4(r.x, r.y, 0u, 0u);
}
template <typename T> __device__ __forceinline__ float4 cvt4(const uint4 &r);
template <> __device__ __forceinline__ float4 cvt4<float>(const uint4 &r) {
    return make_float4(__uint_as_float(r.x), __uint_as_float(r.y), __uint_as_float(r.z), __uint_as_float(r.w));
}
template <> __device__ __forceinline__ float4 cvt4<__nv_bfloat16>(const uint4 &r) {
    return make_float4(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xffff0000u),
                       __uint_as_float(r.y << 16), __uint_as_float(r.y & 0xffff0000u));
}
template <> __device__ __forceinline__ float4 cvt4<__half>(const uint4 &r) {
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&r.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&r.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
// fp32 x4 reduction into global memory (one 16-byte L2 atomic operation, no return value).
__device__ __forceinline__ void red_add_f32x4_hint(float *p, float a, float b, float c, float d, uint64_t pol) {
    asm volatile("red.global.add.L2::cache_hint.v4.f32 [%0], {%1, %2, %3, %4}, %5;"
                 ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d), "l"(pol) : "memory");
}
__device__ __forceinline__ void stg16_hint(void *p, const uint4 &v, uint64_t pol) {
    asm volatile("st.global.L2::cache_hint.v4.u32 [%0], {%1, %2, %3, %4}, %5;"
                 ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w), "l"(pol) : "memory");
}

// Level table in shared memory, built by one thread.  Levels are taken smallest first; a level's
// fp32 gradient image (backward only; a miss there costs a 128-byte read AND write-back) and then
// its value rows are marked "keep" while they still fit in the budget.
__device__ __forceinline__ void build_level_table(LevelGeom *geom, const int64_t *shapes, const int64_t *lsi, int L,
                                                  int GD, int value_elem_bytes, bool with_grad_image,
                                                  unsigned long long budget) {
    unsigned long long cells[kMaxLevels];
    for (int l = 0; l < L; ++l) {
        geom[l].D = (int)shapes[3 * l];
        geom[l].H = (int)shapes[3 * l + 1];
        geom[l].W = (int)shapes[3 * l + 2];
        geom[l].start = (int)lsi[l];
        geom[l].keep = 0;
        geom[l].fD = (float)geom[l].D; geom[l].fH = (float)geom[l].H; geom[l].fW = (float)geom[l].W;
        cells[l] = (unsigned long long)shapes[3 * l] * shapes[3 * l + 1] * shapes[3 * l + 2];
    }
    unsigned done = 0;
    for (int it = 0; it < L; ++it) {
        int best = -1;
        for (int l = 0; l < L; ++l)
            if (!(done >> l & 1u) && (best < 0 || cells[l] < cells[best])) best = l;
        done |= 1u << best;
        const unsigned long long vbytes = cells[best] * (unsigned long long)GD * value_elem_bytes;
        const unsigned long long gbytes = cells[best] * (unsigned long long)GD * 4ull;
        if (with_grad_image && gbytes <= budget) { geom[best].keep |= 2; budget -= gbytes; }
        if (vbytes <= budget) { geom[best].keep |= 1; budget -= vbytes; }
    }
}

// ---------------------------------------------------------------------------
// Geometry of one sampling point: corner offsets, validity and weights
// ---------------------------------------------------------------------------
__device__ __forceinline__ float unnormalize(float loc, float size) {
    // grid = 2*loc - 1 (done by the PyTorch oracle before grid_sample), then
    // grid_sample's ((grid + 1) * size - 1) / 2; every step rounded on its own.
    const float g = __fadd_rn(__fmul_rn(2.0f, loc), -1.0f);
    return __fmul_rn(__fadd_rn(__fmul_rn(__fadd_rn(g, 1.0f), size), -1.0f), 0.5f);
}

struct PointGeom {
    float wx[2], wy[2], wz[2];   // weight of the low / high corner along each axis
    bool xin[2], yin[2], zin[2]; // corner index inside the level along each axis
    uint32_t off[8];             // element offset of corner (dz,dy,dx) -> index dz*4+dy*2+dx, modulo 2^32
};

// From voxel coordinates (xi, yi, zi) of the level (cell centres at integers).
__device__ __forceinline__ void point_geometry_voxel(const LevelGeom &lv, int GD, float xi, float yi, float zi, PointGeom &pg) {
    const float xf = floorf(xi), yf = floorf(yi), zf = floorf(zi);
    pg.wx[0] = __fsub_rn(__fadd_rn(xf, 1.0f), xi); pg.wx[1] = __fsub_rn(xi, xf);
    pg.wy[0] = __fsub_rn(__fadd_rn(yf, 1.0f), yi); pg.wy[1] = __fsub_rn(yi, yf);
    pg.wz[0] = __fsub_rn(__fadd_rn(zf, 1.0f), zi); pg.wz[1] = __fsub_rn(zi, zf);
    // float -> int conversion saturates; the unsigned compares below reject every index outside
    // [0, size), including saturated and wrapped ones, so no out-of-range address is ever formed.
    const uint32_t x0 = (uint32_t)(int)xf, y0 = (uint32_t)(int)yf, z0 = (uint32_t)(int)zf;
    const uint32_t W = (uint32_t)lv.W, H = (uint32_t)lv.H, Dz = (uint32_t)lv.D;
    pg.xin[0] = x0 < W; pg.xin[1] = (x0 + 1u) < W;
    pg.yin[0] = y0 < H; pg.yin[1] = (y0 + 1u) < H;
    pg.zin[0] = z0 < Dz; pg.zin[1] = (z0 + 1u) < Dz;
    const uint32_t sx = (uint32_t)GD, sy = W * sx, sz = H * sy;
    const uint32_t base = z0 * sz + y0 * sy + x0 * sx;  // wraps for index -1; base + stride wraps back
#pragma unroll
    for (int n = 0; n < 8; ++n)
        pg.off[n] = base + ((n & 4) ? sz : 0u) + ((n & 2) ? sy : 0u) + ((n & 1) ? sx : 0u);
}

// v / LK for the small vector indices of a warp's tile (v < 32 rows * 40 vectors) without an integer division:
// (v + 0.5) / LK lies at least 0.5 / LK away from the next integer, far more than the rounding error of the product.
__device__ __forceinline__ int row_of_vector(int v, float inv_lk) { return (int)(((float)v + 0.5f) * inv_lk); }

// From normalised coordinates in [0, 1] (the deformable-attention convention).
__device__ __forceinline__ void point_geometry(const LevelGeom &lv, int GD, float x, float y, float z, PointGeom &pg) {
    point_geometry_voxel(lv, GD, unnormalize(x, lv.fW), unnormalize(y, lv.fH), unnormalize(z, lv.fD), pg);
}

// Stage `nrows` consecutive packed rows (4*LK elements each, contiguous in global memory) into a
// warp-private shared-memory tile as fp32, `row_stride` floats apart.  Whole warp participates.
template <typename PT>
__device__ __forceinline__ void stage_rows(const PT *__restrict__ src, float *tile, int nrows, int LK, int row_stride, int lane) {
    const int nvec = nrows * LK;  // 4-element vectors
    const float inv_lk = 1.0f / (float)LK;
    for (int v = lane; v < nvec; v += 32) {
        const int r = row_of_vector(v, inv_lk);
        const int c = (v - r * LK) * 4;
        const float4 f = load4_stream<PT>(src + (size_t)v * 4);
        *reinterpret_cast<float4 *>(tile + r * row_stride + c) = f;
    }
}

}  // namespace fda
