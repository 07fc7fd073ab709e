// ROI-Align 3D (forward, backward) and NMS 3D for sm_100a: the two small detection-head operators that sit
// beside deformable attention in the reference's extension.
//
// Replaces roi_align_3d_forward_cuda_kernel / roi_align_3d_backward_cuda_kernel
// (csrc/cuda/roi_align_3d_cuda_kernel.cuh:31,110) with their interpolation helpers
// (csrc/cuda/interpolation_helpers_3d.h), and nms_kernel_3d plus the host-side greedy sweep of nms_3d_cuda
// (csrc/cuda/nms_3d_cuda.cu:49-101,133-157).  Differences in structure, not in results:
//   * ROI-Align: one thread per output element as in the reference, but the ROI geometry is computed once per
//     thread in registers with the sample loops fully predicated; 16-bit features are read directly and
//     accumulated in fp32;
//   * NMS: the pairwise-IoU bit matrix is built 64 x 64 boxes per block as in the reference; the greedy sweep
//     runs on the DEVICE (one block: a 64-box chunk is resolved by one warp from the diagonal words, then all
//     threads OR the kept rows into the running removal mask), so the matrix never crosses PCIe and the host
//     only reads the number of kept boxes.
#include "../../include/fda_b200.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "fda_config.h"

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T *p);
template <> __device__ __forceinline__ float ldf<float>(const float *p) { return __ldg(p); }
template <> __device__ __forceinline__ float ldf<__half>(const __half *p) { return __half2float(__ldg(p)); }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16 *p) { return __bfloat162float(__ldg(p)); }
template <typename T> __device__ __forceinline__ T cvt_out(float v);
template <> __device__ __forceinline__ float cvt_out<float>(float v) { return v; }
template <> __device__ __forceinline__ __half cvt_out<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 cvt_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Corner indices and weights of one sample, the reference's rules (interpolation_helpers_3d.h): samples more than
// one voxel outside contribute nothing; coordinates are clamped to [0, size-1]; order 0 picks the nearest corner.
struct Sample {
    int z0, z1, y0, y1, x0, x1;
    float w[8];  // (z0y0x0, z0y0x1, z0y1x0, z0y1x1, z1y0x0, z1y0x1, z1y1x0, z1y1x1)
    bool valid;
};

__device__ __forceinline__ void axis_setup(float v, int size, int &i0, int &i1, float &l, float &h) {
    if (v <= 0.f) v = 0.f;
    i0 = (int)v;
    if (i0 >= size - 1) {
        i1 = i0 = size - 1;
        v = (float)i0;
    } else {
        i1 = i0 + 1;
    }
    l = v - (float)i0;
    h = 1.f - l;
}

__device__ __forceinline__ Sample make_sample(int depth, int height, int width, float z, float y, float x, int order) {
    Sample s;
    s.valid = !(y < -1.0f || y > (float)height || x < -1.0f || x > (float)width || z < -1.0f || z > (float)depth);
    if (!s.valid) {
        s.z0 = s.z1 = s.y0 = s.y1 = s.x0 = s.x1 = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) s.w[i] = 0.f;
        return s;
    }
    float lz, hz, ly, hy, lx, hx;
    axis_setup(z, depth, s.z0, s.z1, lz, hz);
    axis_setup(y, height, s.y0, s.y1, ly, hy);
    axis_setup(x, width, s.x0, s.x1, lx, hx);
    if (order == 0) {  // nearest: all weight on the closer corner along each axis (ties go to the lower one)
        lz = lz > 0.5f ? 1.f : 0.f; hz = 1.f - lz;
        ly = ly > 0.5f ? 1.f : 0.f; hy = 1.f - ly;
        lx = lx > 0.5f ? 1.f : 0.f; hx = 1.f - lx;
    }
    s.w[0] = hz * hy * hx; s.w[1] = hz * hy * lx; s.w[2] = hz * ly * hx; s.w[3] = hz * ly * lx;
    s.w[4] = lz * hy * hx; s.w[5] = lz * hy * lx; s.w[6] = lz * ly * hx; s.w[7] = lz * ly * lx;
    return s;
}

struct RoiGeom {
    int batch;
    float start_w, start_h, start_d, bin_w, bin_h, bin_d;
    int grid_w, grid_h, grid_d;
    float count;
};

template <typename RT>
__device__ __forceinline__ RoiGeom roi_geometry(const RT *roi, float spatial_scale, int sampling_ratio, int pd, int ph, int pw) {
    RoiGeom g;
    g.batch = (int)ldf<RT>(roi);
    g.start_w = ldf<RT>(roi + 1) * spatial_scale;
    g.start_h = ldf<RT>(roi + 2) * spatial_scale;
    g.start_d = ldf<RT>(roi + 3) * spatial_scale;
    const float rw = fmaxf(ldf<RT>(roi + 4) * spatial_scale - g.start_w, 1.f);
    const float rh = fmaxf(ldf<RT>(roi + 5) * spatial_scale - g.start_h, 1.f);
    const float rd = fmaxf(ldf<RT>(roi + 6) * spatial_scale - g.start_d, 1.f);
    g.bin_d = rd / (float)pd; g.bin_h = rh / (float)ph; g.bin_w = rw / (float)pw;
    g.grid_d = sampling_ratio > 0 ? sampling_ratio : (int)ceilf(rd / (float)pd);
    g.grid_h = sampling_ratio > 0 ? sampling_ratio : (int)ceilf(rh / (float)ph);
    g.grid_w = sampling_ratio > 0 ? sampling_ratio : (int)ceilf(rw / (float)pw);
    const int c = g.grid_d * g.grid_h * g.grid_w;
    g.count = (float)(c > 1 ? c : 1);
    return g;
}

template <typename T>
__global__ void __launch_bounds__(256) roi_align3d_forward_kernel(size_t total, const T *__restrict__ features,
                                                                  const T *__restrict__ rois, float spatial_scale,
                                                                  int sampling_ratio, int order, int channels, int depth,
                                                                  int height, int width, int pd, int ph, int pw,
                                                                  T *__restrict__ out) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t index = (size_t)blockIdx.x * blockDim.x + threadIdx.x; index < total; index += stride) {
        const int iw = (int)(index % pw);
        const int ih = (int)((index / pw) % ph);
        const int id = (int)((index / pw / ph) % pd);
        const int c = (int)((index / pw / ph / pd) % channels);
        const size_t n = index / pw / ph / pd / channels;
        const RoiGeom g = roi_geometry<T>(rois + n * 7, spatial_scale, sampling_ratio, pd, ph, pw);
        const T *vol = features + ((size_t)g.batch * channels + c) * (size_t)depth * height * width;
        const size_t hw = (size_t)height * width;
        float acc = 0.f;
        for (int iz = 0; iz < g.grid_d; ++iz) {
            const float z = g.start_d + id * g.bin_d + ((float)iz + .5f) * g.bin_d / (float)g.grid_d;
            for (int iy = 0; iy < g.grid_h; ++iy) {
                const float y = g.start_h + ih * g.bin_h + ((float)iy + .5f) * g.bin_h / (float)g.grid_h;
                for (int ix = 0; ix < g.grid_w; ++ix) {
                    const float x = g.start_w + iw * g.bin_w + ((float)ix + .5f) * g.bin_w / (float)g.grid_w;
                    const Sample s = make_sample(depth, height, width, z, y, x, order);
                    if (!s.valid) continue;
                    const T *p0 = vol + s.z0 * hw, *p1 = vol + s.z1 * hw;
                    acc += s.w[0] * ldf<T>(p0 + (size_t)s.y0 * width + s.x0) + s.w[1] * ldf<T>(p0 + (size_t)s.y0 * width + s.x1) +
                           s.w[2] * ldf<T>(p0 + (size_t)s.y1 * width + s.x0) + s.w[3] * ldf<T>(p0 + (size_t)s.y1 * width + s.x1) +
                           s.w[4] * ldf<T>(p1 + (size_t)s.y0 * width + s.x0) + s.w[5] * ldf<T>(p1 + (size_t)s.y0 * width + s.x1) +
                           s.w[6] * ldf<T>(p1 + (size_t)s.y1 * width + s.x0) + s.w[7] * ldf<T>(p1 + (size_t)s.y1 * width + s.x1);
                }
            }
        }
        out[index] = cvt_out<T>(acc / g.count);
    }
}

// grad_features (fp32, pre-zeroed by the caller as in the reference) += scatter of grad_output through the same weights.
template <typename T>
__global__ void __launch_bounds__(256) roi_align3d_backward_kernel(size_t total, const T *__restrict__ grad_out,
                                                                   const float *__restrict__ rois, float spatial_scale,
                                                                   int sampling_ratio, int order, int channels, int depth,
                                                                   int height, int width, int pd, int ph, int pw,
                                                                   float *__restrict__ grad_features) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t index = (size_t)blockIdx.x * blockDim.x + threadIdx.x; index < total; index += stride) {
        const int iw = (int)(index % pw);
        const int ih = (int)((index / pw) % ph);
        const int id = (int)((index / pw / ph) % pd);
        const int c = (int)((index / pw / ph / pd) % channels);
        const size_t n = index / pw / ph / pd / channels;
        const RoiGeom g = roi_geometry<float>(rois + n * 7, spatial_scale, sampling_ratio, pd, ph, pw);
        float *vol = grad_features + ((size_t)g.batch * channels + c) * (size_t)depth * height * width;
        const size_t hw = (size_t)height * width;
        const float go = ldf<T>(grad_out + index) / g.count;
        for (int iz = 0; iz < g.grid_d; ++iz) {
            const float z = g.start_d + id * g.bin_d + ((float)iz + .5f) * g.bin_d / (float)g.grid_d;
            for (int iy = 0; iy < g.grid_h; ++iy) {
                const float y = g.start_h + ih * g.bin_h + ((float)iy + .5f) * g.bin_h / (float)g.grid_h;
                for (int ix = 0; ix < g.grid_w; ++ix) {
                    const float x = g.start_w + iw * g.bin_w + ((float)ix + .5f) * g.bin_w / (float)g.grid_w;
                    const Sample s = make_sample(depth, height, width, z, y, x, order);
                    if (!s.valid) continue;
                    float *p0 = vol + s.z0 * hw, *p1 = vol + s.z1 * hw;
                    atomicAdd(p0 + (size_t)s.y0 * width + s.x0, go * s.w[0]);
                    atomicAdd(p0 + (size_t)s.y0 * width + s.x1, go * s.w[1]);
                    atomicAdd(p0 + (size_t)s.y1 * width + s.x0, go * s.w[2]);
                    atomicAdd(p0 + (size_t)s.y1 * width + s.x1, go * s.w[3]);
                    atomicAdd(p1 + (size_t)s.y0 * width + s.x0, go * s.w[4]);
                    atomicAdd(p1 + (size_t)s.y0 * width + s.x1, go * s.w[5]);
                    atomicAdd(p1 + (size_t)s.y1 * width + s.x0, go * s.w[6]);
                    atomicAdd(p1 + (size_t)s.y1 * width + s.x1, go * s.w[7]);
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// NMS 3D
// ---------------------------------------------------------------------------------------------------------
constexpr int kNmsBlock = 64;  // boxes per block = bits per mask word

__device__ __forceinline__ float iou3d(const float *a, const float *b) {
    const float left = fmaxf(a[0], b[0]), right = fminf(a[3], b[3]);
    const float top = fmaxf(a[1], b[1]), bottom = fminf(a[4], b[4]);
    const float front = fmaxf(a[2], b[2]), back = fminf(a[5], b[5]);
    const float w = fmaxf(right - left, 0.f), h = fmaxf(bottom - top, 0.f), d = fmaxf(back - front, 0.f);
    const float inter = w * h * d;
    const float sa = (a[3] - a[0]) * (a[4] - a[1]) * (a[5] - a[2]);
    const float sb = (b[3] - b[0]) * (b[4] - b[1]) * (b[5] - b[2]);
    return inter / (sa + sb - inter);
}

// mask[i * col_blocks + cb] bit j: box i (score order) suppresses box cb*64 + j (> i) -- boxes are [n][6], sorted by score.
__global__ void __launch_bounds__(kNmsBlock) nms3d_mask_kernel(int n, float threshold, const float *__restrict__ boxes,
                                                               unsigned long long *__restrict__ mask, int col_blocks) {
    const int row_start = blockIdx.y, col_start = blockIdx.x;
    if (col_start < row_start) return;  // the sweep only reads words at or right of the diagonal
    const int row_size = min(n - row_start * kNmsBlock, kNmsBlock), col_size = min(n - col_start * kNmsBlock, kNmsBlock);
    __shared__ float cols[kNmsBlock * 6];
    if ((int)threadIdx.x < col_size)
        for (int k = 0; k < 6; ++k) cols[threadIdx.x * 6 + k] = boxes[(size_t)(col_start * kNmsBlock + threadIdx.x) * 6 + k];
    __syncthreads();
    if ((int)threadIdx.x < row_size) {
        const int cur = row_start * kNmsBlock + threadIdx.x;
        float a[6];
        for (int k = 0; k < 6; ++k) a[k] = boxes[(size_t)cur * 6 + k];
        unsigned long long t = 0;
        const int start = row_start == col_start ? threadIdx.x + 1 : 0;
        for (int i = start; i < col_size; ++i)
            if (iou3d(a, cols + i * 6) > threshold) t |= 1ULL << i;
        mask[(size_t)cur * col_blocks + col_start] = t;
    }
}

// Greedy sweep in score order, one block.  keep[0 .. *num_keep) = positions (in score order) of the kept boxes.
__global__ void __launch_bounds__(256) nms3d_sweep_kernel(int n, int col_blocks, const unsigned long long *__restrict__ mask,
                                                          long long *__restrict__ keep, int *__restrict__ num_keep) {
    extern __shared__ unsigned long long removed[];  // [col_blocks]
    __shared__ unsigned long long kept_bits;         // boxes of the current chunk that survive
    __shared__ int kept_total;
    for (int j = threadIdx.x; j < col_blocks; j += blockDim.x) removed[j] = 0ull;
    if (threadIdx.x == 0) kept_total = 0;
    __syncthreads();
    for (int cb = 0; cb < col_blocks; ++cb) {
        const int size = min(n - cb * kNmsBlock, kNmsBlock);
        if (threadIdx.x == 0) {
            // inside the chunk the decision chain is sequential; it only needs the 64 diagonal words
            unsigned long long rem = removed[cb], kept = 0ull;
            for (int i = 0; i < size; ++i) {
                if (!((rem >> i) & 1ull)) {
                    kept |= 1ull << i;
                    rem |= mask[(size_t)(cb * kNmsBlock + i) * col_blocks + cb];
                    keep[kept_total++] = (long long)cb * kNmsBlock + i;
                }
            }
            kept_bits = kept;
        }
        __syncthreads();
        const unsigned long long kept = kept_bits;
        // every later column: OR the rows of the boxes kept in this chunk
        for (int j = cb + 1 + (int)threadIdx.x; j < col_blocks; j += blockDim.x) {
            unsigned long long acc = removed[j];
            for (int i = 0; i < size; ++i)
                if ((kept >> i) & 1ull) acc |= mask[(size_t)(cb * kNmsBlock + i) * col_blocks + j];
            removed[j] = acc;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) *num_keep = kept_total;
}

inline int status_of(cudaError_t e) {
    if (e == cudaSuccess) return FDA_OK;
    fda::record_cuda_error((int)e);
    return FDA_ERR_CUDA;
}

inline unsigned grid_for(size_t total) {
    size_t blocks = (total + 255) / 256;
    const size_t cap = 148 * 32;  // grid-stride beyond that
    return (unsigned)(blocks > cap ? cap : (blocks ? blocks : 1));
}

}  // namespace

extern "C" int fda_roi_align3d_forward(const void *features, const void *rois, void *output, int num_rois, int channels,
                                       int depth, int height, int width, int pooled_depth, int pooled_height,
                                       int pooled_width, float spatial_scale, int sampling_ratio, int order, int dtype,
                                       void *stream) {
    if (!features || !rois || !output) return FDA_ERR_NULL_POINTER;
    if (dtype < 0 || dtype > 2) return FDA_ERR_BAD_DTYPE;
    if (num_rois < 0 || channels <= 0 || depth <= 0 || height <= 0 || width <= 0 || pooled_depth <= 0 || pooled_height <= 0 ||
        pooled_width <= 0 || (order != 0 && order != 1))
        return FDA_ERR_BAD_SHAPE;
    const size_t total = (size_t)num_rois * channels * pooled_depth * pooled_height * pooled_width;
    if (total == 0) return FDA_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned g = grid_for(total);
#define FDA_ROI_FWD(T)                                                                                                     \
    roi_align3d_forward_kernel<T><<<g, 256, 0, st>>>(total, static_cast<const T *>(features), static_cast<const T *>(rois),    \
                                                     spatial_scale, sampling_ratio, order, channels, depth, height, width,   \
                                                     pooled_depth, pooled_height, pooled_width, static_cast<T *>(output))
    if (dtype == FDA_DTYPE_F32) FDA_ROI_FWD(float);
    else if (dtype == FDA_DTYPE_F16) FDA_ROI_FWD(__half);
    else FDA_ROI_FWD(__nv_bfloat16);
#undef FDA_ROI_FWD
    return status_of(cudaGetLastError());
}

extern "C" int fda_roi_align3d_backward(const void *grad_output, const float *rois, float *grad_features, int num_rois,
                                        int channels, int depth, int height, int width, int pooled_depth,
                                        int pooled_height, int pooled_width, float spatial_scale, int sampling_ratio,
                                        int order, int grad_output_dtype, void *stream) {
    if (!grad_output || !rois || !grad_features) return FDA_ERR_NULL_POINTER;
    if (grad_output_dtype < 0 || grad_output_dtype > 2) return FDA_ERR_BAD_DTYPE;
    if (num_rois < 0 || channels <= 0 || depth <= 0 || height <= 0 || width <= 0 || pooled_depth <= 0 || pooled_height <= 0 ||
        pooled_width <= 0 || (order != 0 && order != 1))
        return FDA_ERR_BAD_SHAPE;
    const size_t total = (size_t)num_rois * channels * pooled_depth * pooled_height * pooled_width;
    if (total == 0) return FDA_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned g = grid_for(total);
#define FDA_ROI_BWD(T)                                                                                                      \
    roi_align3d_backward_kernel<T><<<g, 256, 0, st>>>(total, static_cast<const T *>(grad_output), rois, spatial_scale,           \
                                                      sampling_ratio, order, channels, depth, height, width, pooled_depth,    \
                                                      pooled_height, pooled_width, grad_features)
    if (grad_output_dtype == FDA_DTYPE_F32) FDA_ROI_BWD(float);
    else if (grad_output_dtype == FDA_DTYPE_F16) FDA_ROI_BWD(__half);
    else FDA_ROI_BWD(__nv_bfloat16);
#undef FDA_ROI_BWD
    return status_of(cudaGetLastError());
}

extern "C" size_t fda_nms3d_workspace_bytes(int num_boxes) {
    if (num_boxes <= 0) return 0;
    const size_t col_blocks = ((size_t)num_boxes + kNmsBlock - 1) / kNmsBlock;
    return (size_t)num_boxes * col_blocks * sizeof(unsigned long long);
}

extern "C" int fda_nms3d(const float *boxes_sorted, int num_boxes, float iou_threshold, void *workspace,
                         size_t workspace_bytes, long long *keep, int *num_keep, void *stream) {
    if (!boxes_sorted || !keep || !num_keep) return FDA_ERR_NULL_POINTER;
    if (num_boxes < 0) return FDA_ERR_BAD_SHAPE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (num_boxes == 0) return status_of(cudaMemsetAsync(num_keep, 0, sizeof(int), st));
    const size_t need = fda_nms3d_workspace_bytes(num_boxes);
    if (!workspace || workspace_bytes < need) return FDA_ERR_WORKSPACE;
    const int col_blocks = (num_boxes + kNmsBlock - 1) / kNmsBlock;
    const size_t smem = (size_t)col_blocks * sizeof(unsigned long long);
    if (smem > 200 * 1024) return FDA_ERR_TOO_LARGE_STATIC;  // 1.6 M boxes
    auto *mask = static_cast<unsigned long long *>(workspace);
    nms3d_mask_kernel<<<dim3((unsigned)col_blocks, (unsigned)col_blocks), kNmsBlock, 0, st>>>(num_boxes, iou_threshold,
                                                                                              boxes_sorted, mask, col_blocks);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return status_of(e);
    if (smem > 48 * 1024) {
        e = cudaFuncSetAttribute(nms3d_sweep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return status_of(e);
    }
    nms3d_sweep_kernel<<<1, 256, smem, st>>>(num_boxes, col_blocks, mask, keep, num_keep);
    return status_of(cudaGetLastError());
}
