// Packing of sampling offsets, reference points and attention logits into the operator's planar
// input (the step a multi-scale deformable-attention layer performs between its linear projections
// and this operator):
//     loc[b,q,g,l,k,:] = reference_points[b,q,l,:] + offsets[b,q,g,l,k,:] / (W_l, H_l, D_l)
//     packed[b,q,g, 3*(l*K+k) + axis] = loc,   packed[b,q,g, 3*L*K + l*K + k] = logits[b,q,g,l,k]
// One pass over the data instead of a divide, a broadcast add and a concatenation.  The caller of
// the reference builds this tensor with torch.cat (tests/test_flash_deform_attn.py:31-37 there); the
// normalisation by the level extent is the multi-scale deformable attention convention.
#include "../../include/fda_b200.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace {

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

constexpr int kMaxLevels = 5;
constexpr int kPackThreads = 256;

// Block = (L*K lanes along x) x (rows along y): lane x of a row handles elements 4x .. 4x+3 of the row's 4*L*K
// packed floats, i.e. one 16-byte store (and one 8- or 16-byte load of offsets or logits); rows are walked with a
// grid stride.  No 64-bit division anywhere; the level extents sit in shared memory.
template <typename T>
__global__ void __launch_bounds__(kPackThreads) fda_pack_kernel(const T *__restrict__ offsets, const T *__restrict__ ref,
                                                                const T *__restrict__ logits, const int64_t *__restrict__ shapes,
                                                                float *__restrict__ packed, unsigned rows, int G, int L, int K) {
    __shared__ float extent[kMaxLevels * 3];  // [l][axis] = (W_l, H_l, D_l)
    if (threadIdx.y == 0 && threadIdx.x < L * 3) {
        const int l = threadIdx.x / 3, axis = threadIdx.x - 3 * l;
        extent[threadIdx.x] = (float)shapes[3 * l + (2 - axis)];
    }
    __syncthreads();
    const int LK = L * K;
    const int c = 4 * threadIdx.x;  // first of this lane's four elements within the row
    for (unsigned row = blockIdx.x * blockDim.y + threadIdx.y; row < rows; row += gridDim.x * blockDim.y) {
        float v[4];
        if (c < 3 * LK) {
            const unsigned bq = row / (unsigned)G;
            const T *src = offsets + (size_t)row * (size_t)(3 * LK) + c;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int e = c + j, i = e / 3, axis = e - 3 * i, l = i / K;
                // same arithmetic as the unfused composition: reference + offset / extent
                v[j] = to_f32(ref[((size_t)bq * L + l) * 3 + axis]) + to_f32(src[j]) / extent[3 * l + axis];
            }
        } else {
            const T *src = logits + (size_t)row * (size_t)LK + (c - 3 * LK);
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = to_f32(src[j]);
        }
        *reinterpret_cast<float4 *>(packed + (size_t)row * (size_t)(4 * LK) + c) = make_float4(v[0], v[1], v[2], v[3]);
    }
}

// Backward of the packing: grad_offsets = grad_loc / extent, grad_logits = grad of the logit slots (both cast to
// the layer's dtype), grad_reference_points[b,q,l,:] = sum over heads and points of grad_loc.  One block row (y)
// per query: its G heads are walked in turn, the per-(level, axis) sums collected in shared memory.
template <typename T>
__global__ void __launch_bounds__(kPackThreads) fda_pack_backward_kernel(const float *__restrict__ grad_packed,
                                                                         const int64_t *__restrict__ shapes,
                                                                         T *__restrict__ grad_offsets, T *__restrict__ grad_ref,
                                                                         T *__restrict__ grad_logits, unsigned queries, int G,
                                                                         int L, int K) {
    __shared__ float extent[kMaxLevels * 3];
    extern __shared__ float ref_sum[];  // [blockDim.y][L*3]
    if (threadIdx.y == 0 && threadIdx.x < L * 3) {
        const int l = threadIdx.x / 3, axis = threadIdx.x - 3 * l;
        extent[threadIdx.x] = (float)shapes[3 * l + (2 - axis)];
    }
    const int LK = L * K;
    const int c = 4 * threadIdx.x;
    float *my_sum = ref_sum + threadIdx.y * (L * 3);
    for (unsigned bq0 = blockIdx.x * blockDim.y; bq0 < queries; bq0 += gridDim.x * blockDim.y) {
        const unsigned bq = bq0 + threadIdx.y;
        if (threadIdx.x < L * 3) my_sum[threadIdx.x] = 0.f;
        __syncthreads();
        if (bq < queries) {
            for (int g = 0; g < G; ++g) {
                const size_t row = (size_t)bq * G + g;
                const float4 f = *reinterpret_cast<const float4 *>(grad_packed + row * (size_t)(4 * LK) + c);
                const float v[4] = {f.x, f.y, f.z, f.w};
                if (c < 3 * LK) {
                    T *dst = grad_offsets + row * (size_t)(3 * LK) + c;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int e = c + j, i = e / 3, axis = e - 3 * i, l = i / K;
                        dst[j] = from_f32<T>(v[j] / extent[3 * l + axis]);
                        atomicAdd(&my_sum[3 * l + axis], v[j]);
                    }
                } else {
                    T *dst = grad_logits + row * (size_t)LK + (c - 3 * LK);
#pragma unroll
                    for (int j = 0; j < 4; ++j) dst[j] = from_f32<T>(v[j]);
                }
            }
        }
        __syncthreads();
        if (bq < queries && threadIdx.x < L * 3) grad_ref[(size_t)bq * (L * 3) + threadIdx.x] = from_f32<T>(my_sum[threadIdx.x]);
        __syncthreads();
    }
}

inline dim3 pack_block(int LK) { return dim3((unsigned)LK, (unsigned)(kPackThreads / LK > 0 ? kPackThreads / LK : 1), 1); }

inline unsigned pack_grid(unsigned units, unsigned per_block) {
    unsigned blocks = (units + per_block - 1) / per_block;
    const unsigned cap = 148u * 16u;  // grid-stride beyond that
    return blocks > cap ? cap : (blocks ? blocks : 1u);
}

}  // namespace

extern "C" int fda_pack_sampling(const void *offsets, const void *reference_points, const void *logits,
                                 const int64_t *spatial_shapes, float *packed, int batch, int num_query, int num_heads,
                                 int num_levels, int num_points, int dtype, void *stream) {
    if (!offsets || !reference_points || !logits || !spatial_shapes || !packed) return FDA_ERR_NULL_POINTER;
    if (batch <= 0 || num_query <= 0 || num_heads <= 0) return FDA_ERR_BAD_SHAPE;
    if (num_points != 4 && num_points != 8) return FDA_ERR_BAD_POINTS;
    if (num_levels < 1 || num_levels > kMaxLevels) return FDA_ERR_BAD_LEVELS;
    if (dtype < 0 || dtype > 2) return FDA_ERR_BAD_DTYPE;
    const size_t rows64 = (size_t)batch * num_query * num_heads;
    if (rows64 >= ((size_t)1 << 31)) return FDA_ERR_BAD_SHAPE;
    const unsigned rows = (unsigned)rows64;
    const int LK = num_levels * num_points;
    const dim3 block = pack_block(LK);
    const unsigned g = pack_grid(rows, block.y);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == FDA_DTYPE_F32)
        fda_pack_kernel<float><<<g, block, 0, st>>>(static_cast<const float *>(offsets), static_cast<const float *>(reference_points),
                                                    static_cast<const float *>(logits), spatial_shapes, packed, rows, num_heads,
                                                    num_levels, num_points);
    else if (dtype == FDA_DTYPE_F16)
        fda_pack_kernel<__half><<<g, block, 0, st>>>(static_cast<const __half *>(offsets), static_cast<const __half *>(reference_points),
                                                     static_cast<const __half *>(logits), spatial_shapes, packed, rows, num_heads,
                                                     num_levels, num_points);
    else
        fda_pack_kernel<__nv_bfloat16><<<g, block, 0, st>>>(static_cast<const __nv_bfloat16 *>(offsets),
                                                            static_cast<const __nv_bfloat16 *>(reference_points),
                                                            static_cast<const __nv_bfloat16 *>(logits), spatial_shapes, packed, rows,
                                                            num_heads, num_levels, num_points);
    return cudaGetLastError() == cudaSuccess ? FDA_OK : FDA_ERR_CUDA;
}

extern "C" int fda_pack_sampling_backward(const float *grad_packed, const int64_t *spatial_shapes, void *grad_offsets,
                                          void *grad_reference_points, void *grad_logits, int batch, int num_query,
                                          int num_heads, int num_levels, int num_points, int dtype, void *stream) {
    if (!grad_packed || !spatial_shapes || !grad_offsets || !grad_reference_points || !grad_logits) return FDA_ERR_NULL_POINTER;
    if (batch <= 0 || num_query <= 0 || num_heads <= 0) return FDA_ERR_BAD_SHAPE;
    if (num_points != 4 && num_points != 8) return FDA_ERR_BAD_POINTS;
    if (num_levels < 1 || num_levels > kMaxLevels) return FDA_ERR_BAD_LEVELS;
    if (dtype < 0 || dtype > 2) return FDA_ERR_BAD_DTYPE;
    const size_t q64 = (size_t)batch * num_query;
    if (q64 * num_heads >= ((size_t)1 << 31)) return FDA_ERR_BAD_SHAPE;
    const unsigned queries = (unsigned)q64;
    const int LK = num_levels * num_points;
    const dim3 block = pack_block(LK);
    const unsigned g = pack_grid(queries, block.y);
    const size_t smem = (size_t)block.y * num_levels * 3 * sizeof(float);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == FDA_DTYPE_F32)
        fda_pack_backward_kernel<float><<<g, block, smem, st>>>(grad_packed, spatial_shapes, static_cast<float *>(grad_offsets),
                                                                static_cast<float *>(grad_reference_points),
                                                                static_cast<float *>(grad_logits), queries, num_heads, num_levels,
                                                                num_points);
    else if (dtype == FDA_DTYPE_F16)
        fda_pack_backward_kernel<__half><<<g, block, smem, st>>>(grad_packed, spatial_shapes, static_cast<__half *>(grad_offsets),
                                                                 static_cast<__half *>(grad_reference_points),
                                                                 static_cast<__half *>(grad_logits), queries, num_heads, num_levels,
                                                                 num_points);
    else
        fda_pack_backward_kernel<__nv_bfloat16><<<g, block, smem, st>>>(grad_packed, spatial_shapes,
                                                                        static_cast<__nv_bfloat16 *>(grad_offsets),
                                                                        static_cast<__nv_bfloat16 *>(grad_reference_points),
                                                                        static_cast<__nv_bfloat16 *>(grad_logits), queries, num_heads,
                                                                        num_levels, num_points);
    return cudaGetLastError() == cudaSuccess ? FDA_OK : FDA_ERR_CUDA;
}
