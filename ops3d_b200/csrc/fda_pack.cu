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

// One thread per packed element; rows of 4*L*K floats are contiguous in input and output.
template <typename T>
__global__ void __launch_bounds__(256) fda_pack_kernel(const T *__restrict__ offsets, const T *__restrict__ ref,
                                                       const T *__restrict__ logits, const int64_t *__restrict__ shapes,
                                                       float *__restrict__ packed, size_t rows, int G, int L, int K) {
    const int LK = L * K;
    const size_t total = rows * (size_t)(4 * LK);
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        const size_t row = e / (size_t)(4 * LK);  // (b*Q + q)*G + g
        const int c = (int)(e - row * (size_t)(4 * LK));
        float v;
        if (c < 3 * LK) {
            const int i = c / 3, axis = c - 3 * i, l = i / K;
            // axis 0,1,2 = x,y,z  <->  extents W,H,D = shapes[l][2], [1], [0]
            const float extent = (float)shapes[3 * l + (2 - axis)];
            const size_t bq = row / (size_t)G;
            v = to_f32(ref[(bq * L + l) * 3 + axis]) + to_f32(offsets[row * (size_t)(3 * LK) + c]) / extent;
        } else {
            v = to_f32(logits[row * (size_t)LK + (c - 3 * LK)]);
        }
        packed[e] = v;
    }
}

}  // namespace

extern "C" int fda_pack_sampling(const void *offsets, const void *reference_points, const void *logits,
                                 const int64_t *spatial_shapes, float *packed, int batch, int num_query, int num_heads,
                                 int num_levels, int num_points, int dtype, void *stream) {
    if (!offsets || !reference_points || !logits || !spatial_shapes || !packed) return FDA_ERR_NULL_POINTER;
    if (batch <= 0 || num_query <= 0 || num_heads <= 0 || num_points <= 0) return FDA_ERR_BAD_SHAPE;
    if (num_levels < 1 || num_levels > 5) return FDA_ERR_BAD_LEVELS;
    if (dtype < 0 || dtype > 2) return FDA_ERR_BAD_DTYPE;
    const size_t rows = (size_t)batch * num_query * num_heads;
    const size_t total = rows * 4 * (size_t)num_levels * num_points;
    size_t blocks = (total + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;  // grid-stride
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned g = (unsigned)blocks;
    if (dtype == FDA_DTYPE_F32)
        fda_pack_kernel<float><<<g, 256, 0, st>>>(static_cast<const float *>(offsets), static_cast<const float *>(reference_points),
                                                  static_cast<const float *>(logits), spatial_shapes, packed, rows, num_heads,
                                                  num_levels, num_points);
    else if (dtype == FDA_DTYPE_F16)
        fda_pack_kernel<__half><<<g, 256, 0, st>>>(static_cast<const __half *>(offsets), static_cast<const __half *>(reference_points),
                                                   static_cast<const __half *>(logits), spatial_shapes, packed, rows, num_heads,
                                                   num_levels, num_points);
    else
        fda_pack_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(offsets),
                                                          static_cast<const __nv_bfloat16 *>(reference_points),
                                                          static_cast<const __nv_bfloat16 *>(logits), spatial_shapes, packed, rows,
                                                          num_heads, num_levels, num_points);
    return cudaGetLastError() == cudaSuccess ? FDA_OK : FDA_ERR_CUDA;
}
