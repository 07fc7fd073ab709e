// Cross-GPU sum + cast of the fp32 grad_value images over NVLink peer memory (two-shot all-reduce
// fused with the cast): rank r pulls slice r of every rank's image with plain peer loads, sums in
// fp32 in a fixed order, converts once to the value dtype
// and pushes the finished slice into every rank's grad_value with plain peer stores.
//
// Per rank 4*(R-1)/R bytes per element come in and sizeof(value)*(R-1)/R go out, against
// 2*4*(R-1)/R each way for an fp32 ring all-reduce followed by a separate cast pass.
//
// The kernel contains no waits.  The caller orders it between two cross-rank barriers: every
// rank's image complete before the first pull, every push landed before grad_value is read.
// Only plain ld/st touch peer memory -- no multicast, no TMA.
#include "../../include/fda_b200.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "fda_config.h"

namespace {

constexpr int kMaxPeers = 16;

struct PeerPtrs {
    const float *img[kMaxPeers];  // position p = rank (first + p) % world, the local rank first
    void *out[kMaxPeers];
};

template <typename VT> struct Out8;
template <> struct Out8<float> {
    static __device__ __forceinline__ void store(void *base, size_t unit, const float (&a)[8]) {
        float4 *p = reinterpret_cast<float4 *>(static_cast<float *>(base) + unit * 8);
        p[0] = make_float4(a[0], a[1], a[2], a[3]);
        p[1] = make_float4(a[4], a[5], a[6], a[7]);
    }
};
template <> struct Out8<__nv_bfloat16> {
    static __device__ __forceinline__ void store(void *base, size_t unit, const float (&a)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t *>(&h);
        }
        *reinterpret_cast<uint4 *>(static_cast<__nv_bfloat16 *>(base) + unit * 8) = make_uint4(w[0], w[1], w[2], w[3]);
    }
};
template <> struct Out8<__half> {
    static __device__ __forceinline__ void store(void *base, size_t unit, const float (&a)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2 h = __floats2half2_rn(a[2 * i], a[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t *>(&h);
        }
        *reinterpret_cast<uint4 *>(static_cast<__half *>(base) + unit * 8) = make_uint4(w[0], w[1], w[2], w[3]);
    }
};

// Each thread handles UNROLL 8-element units per iteration, units a whole grid-stride apart, and
// issues all of its peer loads (2 x 16 bytes per unit and rank) before the first use, so that few
// resident threads keep enough bytes in flight to cover NVLink latency while most SMs stay free
// for the scatter kernel running beside it.
// `world` images are summed (the ranks that hold partial sums of this range); the result goes to `n_out`
// outputs (every rank of the job).
template <typename VT, int WORLD, int UNROLL>
__global__ void __launch_bounds__(512) fda_peer_reduce_cast_kernel(const PeerPtrs pp, const int world_rt, const int n_out,
                                                                   size_t unit_begin, size_t unit_end) {
    constexpr int W = WORLD > 0 ? WORLD : kMaxPeers;
    const int world = WORLD > 0 ? WORLD : world_rt;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t u0 = unit_begin + (size_t)blockIdx.x * blockDim.x + threadIdx.x; u0 < unit_end; u0 += stride * UNROLL) {
        float4 lo[UNROLL][W], hi[UNROLL][W];
#pragma unroll
        for (int j = 0; j < UNROLL; ++j) {
            const size_t u = u0 + (size_t)j * stride;
#pragma unroll
            for (int p = 0; p < W; ++p) {
                if (p < world && u < unit_end) {
                    const float4 *src = reinterpret_cast<const float4 *>(pp.img[p] + u * 8);
                    lo[j][p] = __ldcg(src);      // L2 only: peer data must not be served from a stale L1 line
                    hi[j][p] = __ldcg(src + 1);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < UNROLL; ++j) {
            const size_t u = u0 + (size_t)j * stride;
            if (u < unit_end) {
                // Fixed summation order (local image first, then the ring); each element is summed by
                // exactly one rank and broadcast, so all ranks end up with identical bits.
                float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int p = 0; p < W; ++p) {
                    if (p < world) {
                        a[0] += lo[j][p].x; a[1] += lo[j][p].y; a[2] += lo[j][p].z; a[3] += lo[j][p].w;
                        a[4] += hi[j][p].x; a[5] += hi[j][p].y; a[6] += hi[j][p].z; a[7] += hi[j][p].w;
                    }
                }
                for (int p = 0; p < n_out; ++p) Out8<VT>::store(pp.out[p], u, a);
            }
        }
    }
}

// NVSwitch variant: the image and grad_value are bound to multicast objects.  One
// multimem.ld_reduce returns the fp32 sum over all ranks of 16 bytes (the switch reads every GPU's
// copy and adds in flight), one multimem.st writes the converted result into every GPU's copy.
// Per rank only 1/R of the image comes in and 1/R of grad_value goes out.
__device__ __forceinline__ float4 multimem_ld_reduce_add_f32x4(const float *mc) {
    float4 r;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "l"(mc) : "memory");
    return r;
}
__device__ __forceinline__ void multimem_st_16B(void *mc, const uint4 &v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                 ::"l"(mc), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
                 "f"(__uint_as_float(v.w)) : "memory");
}

template <typename VT> struct Pack8;  // 8 fp32 -> the bytes of 8 elements of VT
template <> struct Pack8<__nv_bfloat16> {
    static __device__ __forceinline__ void store(void *mc_base, size_t unit, const float4 &l, const float4 &h) {
        __nv_bfloat162 a = __floats2bfloat162_rn(l.x, l.y), b = __floats2bfloat162_rn(l.z, l.w);
        __nv_bfloat162 c = __floats2bfloat162_rn(h.x, h.y), d = __floats2bfloat162_rn(h.z, h.w);
        multimem_st_16B(static_cast<__nv_bfloat16 *>(mc_base) + unit * 8,
                        make_uint4(*reinterpret_cast<uint32_t *>(&a), *reinterpret_cast<uint32_t *>(&b),
                                   *reinterpret_cast<uint32_t *>(&c), *reinterpret_cast<uint32_t *>(&d)));
    }
};
template <> struct Pack8<__half> {
    static __device__ __forceinline__ void store(void *mc_base, size_t unit, const float4 &l, const float4 &h) {
        __half2 a = __floats2half2_rn(l.x, l.y), b = __floats2half2_rn(l.z, l.w);
        __half2 c = __floats2half2_rn(h.x, h.y), d = __floats2half2_rn(h.z, h.w);
        multimem_st_16B(static_cast<__half *>(mc_base) + unit * 8,
                        make_uint4(*reinterpret_cast<uint32_t *>(&a), *reinterpret_cast<uint32_t *>(&b),
                                   *reinterpret_cast<uint32_t *>(&c), *reinterpret_cast<uint32_t *>(&d)));
    }
};
template <> struct Pack8<float> {
    static __device__ __forceinline__ void store(void *mc_base, size_t unit, const float4 &l, const float4 &h) {
        float *p = static_cast<float *>(mc_base) + unit * 8;
        multimem_st_16B(p, make_uint4(__float_as_uint(l.x), __float_as_uint(l.y), __float_as_uint(l.z), __float_as_uint(l.w)));
        multimem_st_16B(p + 4, make_uint4(__float_as_uint(h.x), __float_as_uint(h.y), __float_as_uint(h.z), __float_as_uint(h.w)));
    }
};

template <typename VT, int UNROLL>
__global__ void __launch_bounds__(512) fda_multimem_reduce_cast_kernel(const float *mc_image, void *mc_out,
                                                                       size_t unit_begin, size_t unit_end) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t u0 = unit_begin + (size_t)blockIdx.x * blockDim.x + threadIdx.x; u0 < unit_end; u0 += stride * UNROLL) {
        float4 lo[UNROLL], hi[UNROLL];
#pragma unroll
        for (int j = 0; j < UNROLL; ++j) {
            const size_t u = u0 + (size_t)j * stride;
            if (u < unit_end) {
                lo[j] = multimem_ld_reduce_add_f32x4(mc_image + u * 8);
                hi[j] = multimem_ld_reduce_add_f32x4(mc_image + u * 8 + 4);
            }
        }
#pragma unroll
        for (int j = 0; j < UNROLL; ++j) {
            const size_t u = u0 + (size_t)j * stride;
            if (u < unit_end) Pack8<VT>::store(mc_out, u, lo[j], hi[j]);
        }
    }
}

// Push variant of the exchange (posted peer stores instead of peer loads): every rank first writes
// the slices it does NOT own into the owners' staging areas, then -- after a barrier -- each owner
// sums its own slice of its image with the world-1 staged partials, converts, and pushes the
// result to every rank.  NVLink carries writes at a higher rate than SM-issued reads.
struct PushPtrs {
    float *staging[kMaxPeers];  // position p = staging area of rank (rank + p) % world
    size_t slice_begin[kMaxPeers], slice_end[kMaxPeers];  // that rank's slice, in 8-element units
};

template <int UNROLL>
__global__ void __launch_bounds__(512) fda_peer_push_kernel(const float *__restrict__ image, const PushPtrs pp, const int world,
                                                            const size_t my_slot_offset /* floats */) {
    // blockIdx.y = peer position 1..world-1; x strides over that peer's slice
    const int p = blockIdx.y + 1;
    if (p >= world) return;
    const size_t ub = pp.slice_begin[p], ue = pp.slice_end[p];
    float *dst = pp.staging[p] + my_slot_offset;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t u0 = ub + (size_t)blockIdx.x * blockDim.x + threadIdx.x; u0 < ue; u0 += stride * UNROLL) {
        float4 lo[UNROLL], hi[UNROLL];
#pragma unroll
        for (int j = 0; j < UNROLL; ++j) {
            const size_t u = u0 + (size_t)j * stride;
            if (u < ue) {
                const float4 *src = reinterpret_cast<const float4 *>(image + u * 8);
                lo[j] = __ldcs(src);
                hi[j] = __ldcs(src + 1);
            }
        }
#pragma unroll
        for (int j = 0; j < UNROLL; ++j) {
            const size_t u = u0 + (size_t)j * stride;
            if (u < ue) {
                float4 *d = reinterpret_cast<float4 *>(dst + (u - ub) * 8);
                d[0] = lo[j];
                d[1] = hi[j];
            }
        }
    }
}

// Owner side: image slice + staged partials (fixed order: own image, then slots 0..world-1 skipping
// the own one) -> value dtype -> every rank's grad_value.
template <typename VT, int UNROLL>
__global__ void __launch_bounds__(512) fda_peer_reduce_staged_kernel(const float *__restrict__ image,
                                                                     const float *__restrict__ staging, size_t slot_stride,
                                                                     const PeerPtrs pp, const int world, const int rank,
                                                                     size_t unit_begin, size_t unit_end) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t u = unit_begin + (size_t)blockIdx.x * blockDim.x + threadIdx.x; u < unit_end; u += stride) {
        const float4 *src = reinterpret_cast<const float4 *>(image + u * 8);
        float4 l = __ldcs(src), h = __ldcs(src + 1);
        float a[8] = {l.x, l.y, l.z, l.w, h.x, h.y, h.z, h.w};
        for (int s = 0; s < world; ++s) {
            if (s == rank) continue;
            const float4 *q = reinterpret_cast<const float4 *>(staging + (size_t)s * slot_stride + (u - unit_begin) * 8);
            l = __ldcg(q); h = __ldcg(q + 1);  // written by a peer: read at L2
            a[0] += l.x; a[1] += l.y; a[2] += l.z; a[3] += l.w;
            a[4] += h.x; a[5] += h.y; a[6] += h.z; a[7] += h.w;
        }
        for (int p = 0; p < world; ++p) Out8<VT>::store(pp.out[p], u, a);
    }
}

inline int status_of(cudaError_t e) {
    if (e == cudaSuccess) return FDA_OK;
    fda::record_cuda_error((int)e);
    return FDA_ERR_CUDA;
}

template <typename VT>
cudaError_t launch(const PeerPtrs &pp, int n_in, int n_out, size_t ub, size_t ue, cudaStream_t st) {
    const size_t units = ue - ub;
    if (units == 0) return cudaSuccess;
    // Few, fat blocks: the kernel is bound by NVLink, not by SM throughput.  Measured with the exchange overlapped
    // with the scatter kernels: on 2 GPUs 16 to 1184 blocks take the same time; on 8 GPUs 8 / 16 / 32 blocks give
    // 13.7 / 9.1 / 8.6 ms per step (FDA_PEER_REDUCE_BLOCKS overrides).
    const int max_blocks = fda::config().peer_reduce_blocks;
    const int threads = 512;
    size_t blocks = (units + threads - 1) / threads;
    if (blocks > (size_t)max_blocks) blocks = (size_t)max_blocks;
    const unsigned g = (unsigned)blocks;
    switch (n_in) {  // images x units in flight per thread = 8
        case 1: fda_peer_reduce_cast_kernel<VT, 1, 8><<<g, threads, 0, st>>>(pp, n_in, n_out, ub, ue); break;
        case 2: fda_peer_reduce_cast_kernel<VT, 2, 4><<<g, threads, 0, st>>>(pp, n_in, n_out, ub, ue); break;
        case 4: fda_peer_reduce_cast_kernel<VT, 4, 2><<<g, threads, 0, st>>>(pp, n_in, n_out, ub, ue); break;
        case 8: fda_peer_reduce_cast_kernel<VT, 8, 1><<<g, threads, 0, st>>>(pp, n_in, n_out, ub, ue); break;
        default: fda_peer_reduce_cast_kernel<VT, 0, 1><<<g, threads, 0, st>>>(pp, n_in, n_out, ub, ue); break;
    }
    return cudaGetLastError();
}

template <typename VT>
cudaError_t launch_multimem(const float *mc_image, void *mc_out, size_t ub, size_t ue, cudaStream_t st) {
    const size_t units = ue - ub;
    if (units == 0) return cudaSuccess;
    const int max_blocks = fda::config().peer_reduce_blocks;
    const int threads = 512;
    size_t blocks = (units + threads - 1) / threads;
    if (blocks > (size_t)max_blocks) blocks = (size_t)max_blocks;
    fda_multimem_reduce_cast_kernel<VT, 4><<<(unsigned)blocks, threads, 0, st>>>(mc_image, mc_out, ub, ue);
    return cudaGetLastError();
}

}  // namespace

extern "C" int fda_multimem_reduce_cast(const float *mc_image, void *mc_output, int world, int rank,
                                        size_t num_elements, int value_dtype, void *stream) {
    if (!mc_image || !mc_output) return FDA_ERR_NULL_POINTER;
    if (world < 1 || rank < 0 || rank >= world) return FDA_ERR_BAD_SHAPE;
    if (value_dtype < 0 || value_dtype > 2) return FDA_ERR_BAD_DTYPE;
    if (num_elements % 8 != 0) return FDA_ERR_BAD_SHAPE;
    if ((reinterpret_cast<uintptr_t>(mc_image) & 15u) || (reinterpret_cast<uintptr_t>(mc_output) & 15u)) return FDA_ERR_MISALIGNED;
    const size_t units = num_elements / 8;
    const size_t ub = units * (size_t)rank / world, ue = units * (size_t)(rank + 1) / world;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    if (value_dtype == FDA_DTYPE_F32) e = launch_multimem<float>(mc_image, mc_output, ub, ue, st);
    else if (value_dtype == FDA_DTYPE_F16) e = launch_multimem<__half>(mc_image, mc_output, ub, ue, st);
    else e = launch_multimem<__nv_bfloat16>(mc_image, mc_output, ub, ue, st);
    return status_of(e);
}

extern "C" int fda_peer_push_partials(const float *image, float *const *peer_staging, size_t slot_stride_elements,
                                      int world, int rank, size_t num_elements, void *stream) {
    if (!image || !peer_staging) return FDA_ERR_NULL_POINTER;
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world) return FDA_ERR_BAD_SHAPE;
    if (num_elements % 8 != 0 || slot_stride_elements % 8 != 0) return FDA_ERR_BAD_SHAPE;
    if (world == 1) return FDA_OK;
    const size_t units = num_elements / 8;
    PushPtrs pp;
    size_t longest = 0;
    for (int p = 0; p < kMaxPeers; ++p) { pp.staging[p] = nullptr; pp.slice_begin[p] = pp.slice_end[p] = 0; }
    for (int p = 0; p < world; ++p) {
        const int r = (rank + p) % world;
        if (!peer_staging[r]) return FDA_ERR_NULL_POINTER;
        if (reinterpret_cast<uintptr_t>(peer_staging[r]) & 15u) return FDA_ERR_MISALIGNED;
        pp.staging[p] = peer_staging[r];
        pp.slice_begin[p] = units * (size_t)r / world;
        pp.slice_end[p] = units * (size_t)(r + 1) / world;
        const size_t len = pp.slice_end[p] - pp.slice_begin[p];
        if (len * 8 > slot_stride_elements) return FDA_ERR_BAD_SHAPE;
        if (len > longest) longest = len;
    }
    if (longest == 0) return FDA_OK;
    const int max_blocks = fda::config().peer_reduce_blocks;
    int bx = max_blocks / (world - 1);
    if (bx < 1) bx = 1;
    const size_t want = (longest + 511) / 512;
    if ((size_t)bx > want) bx = (int)want;
    const dim3 grid((unsigned)bx, (unsigned)(world - 1), 1);
    fda_peer_push_kernel<4><<<grid, 512, 0, static_cast<cudaStream_t>(stream)>>>(image, pp, world,
                                                                                (size_t)rank * slot_stride_elements);
    return status_of(cudaGetLastError());
}

extern "C" int fda_peer_reduce_staged_cast(const float *image, const float *staging, size_t slot_stride_elements,
                                           void *const *peer_outputs, int world, int rank, size_t num_elements,
                                           int value_dtype, void *stream) {
    if (!image || !staging || !peer_outputs) return FDA_ERR_NULL_POINTER;
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world) return FDA_ERR_BAD_SHAPE;
    if (value_dtype < 0 || value_dtype > 2) return FDA_ERR_BAD_DTYPE;
    if (num_elements % 8 != 0 || slot_stride_elements % 8 != 0) return FDA_ERR_BAD_SHAPE;
    PeerPtrs pp;
    for (int p = 0; p < kMaxPeers; ++p) { pp.img[p] = nullptr; pp.out[p] = nullptr; }
    for (int p = 0; p < world; ++p) {
        const int r = (rank + p) % world;
        if (!peer_outputs[r]) return FDA_ERR_NULL_POINTER;
        if (reinterpret_cast<uintptr_t>(peer_outputs[r]) & 15u) return FDA_ERR_MISALIGNED;
        pp.out[p] = peer_outputs[r];
    }
    const size_t units = num_elements / 8;
    const size_t ub = units * (size_t)rank / world, ue = units * (size_t)(rank + 1) / world;
    if (ue == ub) return FDA_OK;
    if ((ue - ub) * 8 > slot_stride_elements) return FDA_ERR_BAD_SHAPE;
    const int max_blocks = fda::config().peer_reduce_blocks;
    size_t blocks = (ue - ub + 511) / 512;
    if (blocks > (size_t)max_blocks) blocks = (size_t)max_blocks;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned g = (unsigned)blocks;
    if (value_dtype == FDA_DTYPE_F32)
        fda_peer_reduce_staged_kernel<float, 1><<<g, 512, 0, st>>>(image, staging, slot_stride_elements, pp, world, rank, ub, ue);
    else if (value_dtype == FDA_DTYPE_F16)
        fda_peer_reduce_staged_kernel<__half, 1><<<g, 512, 0, st>>>(image, staging, slot_stride_elements, pp, world, rank, ub, ue);
    else
        fda_peer_reduce_staged_kernel<__nv_bfloat16, 1><<<g, 512, 0, st>>>(image, staging, slot_stride_elements, pp, world, rank, ub, ue);
    return status_of(cudaGetLastError());
}

extern "C" int fda_group_reduce_cast(const float *const *group_images, int group_size, int group_rank,
                                     void *const *peer_outputs, int world, int rank,
                                     size_t num_elements, int value_dtype, void *stream) {
    if (!group_images || !peer_outputs) return FDA_ERR_NULL_POINTER;
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world) return FDA_ERR_BAD_SHAPE;
    if (group_size < 1 || group_size > world || group_rank < 0 || group_rank >= group_size) return FDA_ERR_BAD_SHAPE;
    if (value_dtype < 0 || value_dtype > 2) return FDA_ERR_BAD_DTYPE;
    if (num_elements % 8 != 0) return FDA_ERR_BAD_SHAPE;
    PeerPtrs pp;
    for (int p = 0; p < kMaxPeers; ++p) { pp.img[p] = nullptr; pp.out[p] = nullptr; }
    for (int p = 0; p < group_size; ++p) {
        const int r = (group_rank + p) % group_size;  // start with the local image, then walk the group's ring
        if (!group_images[r]) return FDA_ERR_NULL_POINTER;
        if (reinterpret_cast<uintptr_t>(group_images[r]) & 15u) return FDA_ERR_MISALIGNED;
        pp.img[p] = group_images[r];
    }
    for (int p = 0; p < world; ++p) {
        const int r = (rank + p) % world;  // local copy first
        if (!peer_outputs[r]) return FDA_ERR_NULL_POINTER;
        if (reinterpret_cast<uintptr_t>(peer_outputs[r]) & 15u) return FDA_ERR_MISALIGNED;
        pp.out[p] = peer_outputs[r];
    }
    const size_t units = num_elements / 8;
    const size_t ub = units * (size_t)group_rank / group_size, ue = units * (size_t)(group_rank + 1) / group_size;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    if (value_dtype == FDA_DTYPE_F32) e = launch<float>(pp, group_size, world, ub, ue, st);
    else if (value_dtype == FDA_DTYPE_F16) e = launch<__half>(pp, group_size, world, ub, ue, st);
    else e = launch<__nv_bfloat16>(pp, group_size, world, ub, ue, st);
    return status_of(e);
}

// Head-sharded backward: every rank owns a slice of the heads of a batch element, so its fp32 image
// [cells][slice] is already the final sum.  This kernel converts it to the value dtype and stores it into the slice's
// place inside every rank's full grad_value [cells][full]: position (cell, head_offset + e) for e < slice.  Plain
// peer stores, no waits; the caller runs one cross-rank barrier after it.
template <typename VT>
__global__ void __launch_bounds__(512) fda_head_slice_push_kernel(const float *__restrict__ image, const PeerPtrs pp, const int n_out,
                                                                  size_t unit_begin, size_t unit_end, unsigned int slice_units,
                                                                  unsigned int full_units, unsigned int head_units) {
    constexpr int kUnroll = 4;  // units per thread and iteration, a grid stride apart: all loads go out before the first store
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t u0 = unit_begin + (size_t)blockIdx.x * blockDim.x + threadIdx.x; u0 < unit_end; u0 += stride * kUnroll) {
        float4 lo[kUnroll], hi[kUnroll];
#pragma unroll
        for (int j = 0; j < kUnroll; ++j) {
            const size_t u = u0 + (size_t)j * stride;
            if (u < unit_end) {
                const float4 *src = reinterpret_cast<const float4 *>(image + u * 8);
                lo[j] = __ldcs(src);
                hi[j] = __ldcs(src + 1);
            }
        }
#pragma unroll
        for (int j = 0; j < kUnroll; ++j) {
            const size_t u = u0 + (size_t)j * stride;
            if (u < unit_end) {
                const float a[8] = {lo[j].x, lo[j].y, lo[j].z, lo[j].w, hi[j].x, hi[j].y, hi[j].z, hi[j].w};
                const size_t cell = u / slice_units;
                const size_t dst = cell * full_units + head_units + (u - cell * slice_units);  // 8-element unit inside the full tensor
                for (int p = 0; p < n_out; ++p) Out8<VT>::store(pp.out[p], dst, a);
            }
        }
    }
}

extern "C" int fda_head_slice_cast_push(const float *image_slice, void *const *peer_outputs, int world, int rank,
                                        size_t cell_begin, size_t cell_count, int slice_elements, int full_elements,
                                        int head_offset_elements, int value_dtype, void *stream) {
    if (!image_slice || !peer_outputs) return FDA_ERR_NULL_POINTER;
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world) return FDA_ERR_BAD_SHAPE;
    if (value_dtype < 0 || value_dtype > 2) return FDA_ERR_BAD_DTYPE;
    if (slice_elements <= 0 || full_elements < slice_elements || head_offset_elements < 0 ||
        head_offset_elements + slice_elements > full_elements)
        return FDA_ERR_BAD_SHAPE;
    if (slice_elements % 8 || full_elements % 8 || head_offset_elements % 8) return FDA_ERR_BAD_SHAPE;
    if (reinterpret_cast<uintptr_t>(image_slice) & 15u) return FDA_ERR_MISALIGNED;
    PeerPtrs pp;
    for (int p = 0; p < kMaxPeers; ++p) { pp.img[p] = nullptr; pp.out[p] = nullptr; }
    for (int p = 0; p < world; ++p) {
        const int r = (rank + p) % world;  // local copy first
        if (!peer_outputs[r]) return FDA_ERR_NULL_POINTER;
        if (reinterpret_cast<uintptr_t>(peer_outputs[r]) & 15u) return FDA_ERR_MISALIGNED;
        pp.out[p] = peer_outputs[r];
    }
    if (cell_count == 0) return FDA_OK;
    const unsigned int su = (unsigned int)slice_elements / 8u;
    const size_t ub = cell_begin * su, ue = (cell_begin + cell_count) * su;
    int blocks = fda::config().peer_reduce_blocks;
    const size_t need = (ue - ub + 511) / 512;
    if ((size_t)blocks > need) blocks = (int)need;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (value_dtype == FDA_DTYPE_F32)
        fda_head_slice_push_kernel<float><<<blocks, 512, 0, st>>>(image_slice, pp, world, ub, ue, su, (unsigned int)full_elements / 8u,
                                                                  (unsigned int)head_offset_elements / 8u);
    else if (value_dtype == FDA_DTYPE_F16)
        fda_head_slice_push_kernel<__half><<<blocks, 512, 0, st>>>(image_slice, pp, world, ub, ue, su, (unsigned int)full_elements / 8u,
                                                                   (unsigned int)head_offset_elements / 8u);
    else
        fda_head_slice_push_kernel<__nv_bfloat16><<<blocks, 512, 0, st>>>(image_slice, pp, world, ub, ue, su,
                                                                          (unsigned int)full_elements / 8u,
                                                                          (unsigned int)head_offset_elements / 8u);
    return status_of(cudaGetLastError());
}

extern "C" int fda_peer_reduce_cast(const float *const *peer_images, void *const *peer_outputs, int world, int rank,
                                    size_t num_elements, int value_dtype, void *stream) {
    // every rank holds a partial image: the group is the whole job
    return fda_group_reduce_cast(peer_images, world, rank, peer_outputs, world, rank, num_elements, value_dtype, stream);
}
