// DCNv4-3D (deformable convolution v4, volumetric) for sm_100a: forward and backward.
//
// Replaces forward_kernel_dcn / forward_kernel_dcn_reg (csrc/cuda/dcnv4_im2col_cuda.cuh:49,259),
// backward_kernel_dcn / backward_kernel_dcn_warp_primitive (csrc/cuda/dcnv4_col2im_cuda.cuh:48,319) and
// their host launchers (csrc/cuda/dcnv4_cuda.cu:19-189) of the reference.  Same gather / scatter skeleton
// as Flash Deformable Attention with one level and a fixed stencil:
//
//   out[b, q, g, :] = sum_k m_k * trilinear(value[b], p_k)[g, :]
//   p_k = p0(q) + (stencil_k * dilation + offset_k) * offset_scale          (voxel coordinates)
//
// q = (z, y, x) runs over the output volume, stencil_k over the kernel_w x kernel_h x kernel_d points
// (w outermost, d innermost; the centre point skipped when remove_center), m = mask (soft-maxed over
// the K points when `softmax`).  offset row of (b, q): `padded` elements, per group g a block of
// K*3 offsets (x, y, z per point) followed by K mask values at g*K*4 (csrc/cuda/dcnv4_im2col_cuda.cuh:118).
//
// Thread mapping as in fda_device.cuh: one row = (q, g), its channels over lanes that own one 16-byte
// vector each; the row's 4*K offset/mask values are staged in a warp-private shared-memory tile.
#include "../../include/fda_b200.h"

#include "fda_backward.cuh"
#include "fda_config.h"

namespace {

struct DcnProblem {
    const void *value;       // [B][Din*Hin*Win][G][D]
    const void *offset;      // [B][Q][padded]
    void *out;               // [B][Q][G*D]                      (forward)
    const void *grad_out;    // [B][Q][G*D]                      (backward)
    float *accum;            // fp32 image of grad_value         (backward)
    void *grad_offset;       // [B][Q][padded]                   (backward)
    int B, G, D, Q, K, padded;
    int Din, Hin, Win, Dout, Hout, Wout;
    int kd, kh, kw, sd, sh, sw, pd, ph, pw, dd, dh, dw;
    float offset_scale;
    int remove_center, softmax;
    int gs_log2, lpg, rows_per_b, GD, row_stride;
    unsigned long long l2_keep_bytes;
};

// Voxel position of stencil point (i, j, k) = (w, h, d index) for output cell (x, y, z), offsets (ox, oy, oz):
// the arithmetic of the reference (dcnv4_im2col_cuda.cuh:178-216), every step in fp32.
struct StencilBase {
    float w, h, d;
};
__device__ __forceinline__ StencilBase stencil_base(const DcnProblem &p, int q) {
    const int x = q % p.Wout, yz = q / p.Wout, y = yz % p.Hout, z = yz / p.Hout;
    const int p0w = ((p.dw * (p.kw - 1)) >> 1) - p.pw + x * p.sw;
    const int p0h = ((p.dh * (p.kh - 1)) >> 1) - p.ph + y * p.sh;
    const int p0d = ((p.dd * (p.kd - 1)) >> 1) - p.pd + z * p.sd;
    StencilBase s;
    s.w = (float)p0w - (float)((p.dw * (p.kw - 1)) >> 1) * p.offset_scale;
    s.h = (float)p0h - (float)((p.dh * (p.kh - 1)) >> 1) * p.offset_scale;
    s.d = (float)p0d - (float)((p.dd * (p.kd - 1)) >> 1) * p.offset_scale;
    return s;
}

// Walks the stencil in the reference's order (w outermost, d innermost), skipping the centre if asked.
struct StencilWalk {
    int i, j, k;
    __device__ __forceinline__ void start(const DcnProblem &p) { i = j = k = 0; skip_centre(p); }
    __device__ __forceinline__ void skip_centre(const DcnProblem &p) {
        if (p.remove_center && i == p.kw / 2 && j == p.kh / 2 && k == p.kd / 2) advance_raw(p);
    }
    __device__ __forceinline__ void advance_raw(const DcnProblem &p) {
        if (++k == p.kd) { k = 0; if (++j == p.kh) { j = 0; ++i; } }
    }
    __device__ __forceinline__ void next(const DcnProblem &p) { advance_raw(p); skip_centre(p); }
};

// Stage the 4*K values of every row of this warp (row = q*G + g -> offset + (b*Q + q)*padded + g*K*4) as fp32.
template <typename T>
__device__ __forceinline__ void stage_dcn_rows(const DcnProblem &p, int b, int first_row, int nrows, float *wtile, int lane) {
    const int per_row = 4 * p.K;
    const T *base = static_cast<const T *>(p.offset) + (size_t)b * p.Q * (size_t)p.padded;
    for (int r = 0; r < nrows; ++r) {
        const int row = first_row + r, q = row / p.G, g = row - q * p.G;
        const T *src = base + (size_t)q * p.padded + (size_t)g * per_row;
        for (int e = lane; e < per_row; e += 32) wtile[r * p.row_stride + e] = fda::load1<T>(src + e);
    }
}

template <typename T>
__global__ void __launch_bounds__(fda::kThreads, 3) dcnv4_forward_kernel(const DcnProblem p) {
    using namespace fda;
    constexpr int CPL = Vec16<T>::kCPL;
    extern __shared__ __align__(16) float smem_tile[];
    const int tid = threadIdx.x, b = blockIdx.y;
    const int gs = 1 << p.gs_log2, lane = tid & 31, warp = tid >> 5;
    const int lane_c = tid & (gs - 1);
    const int rows_per_block = (int)blockDim.x >> p.gs_log2, rows_per_warp = 32 >> p.gs_log2;
    const int row = blockIdx.x * rows_per_block + (tid >> p.gs_log2);
    const bool row_ok = row < p.rows_per_b, active = row_ok && lane_c < p.lpg;
    const int first = blockIdx.x * rows_per_block + warp * rows_per_warp;
    float *wtile = smem_tile + warp * rows_per_warp * p.row_stride;
    int nrows = p.rows_per_b - first;
    nrows = nrows < 0 ? 0 : (nrows > rows_per_warp ? rows_per_warp : nrows);
    stage_dcn_rows<T>(p, b, first, nrows, wtile, lane);
    __syncwarp();
    const float *trow = wtile + (lane >> p.gs_log2) * p.row_stride;
    const int K = p.K;

    float m = 0.f, inv = 1.f;
    if (p.softmax && row_ok) {
        m = -INFINITY;
        for (int k = 0; k < K; ++k) m = fmaxf(m, trow[3 * K + k]);
        float s = 0.f;
        for (int k = 0; k < K; ++k) s += __expf(trow[3 * K + k] - m);
        inv = 1.0f / s;
    }
    LevelGeom lv;
    lv.D = p.Din; lv.H = p.Hin; lv.W = p.Win; lv.start = 0; lv.keep = 0;
    lv.fD = (float)p.Din; lv.fH = (float)p.Hin; lv.fW = (float)p.Win;
    const bool keep = (unsigned long long)p.Din * p.Hin * p.Win * p.GD * sizeof(T) <= p.l2_keep_bytes;
    const uint64_t pol = keep ? l2_policy_evict_last() : l2_policy_evict_normal();
    const int q = row_ok ? row / p.G : 0, g = row_ok ? row - q * p.G : 0;
    const StencilBase sb = stencil_base(p, q);
    const T *value_b = static_cast<const T *>(p.value) + (size_t)b * p.Din * p.Hin * p.Win * (size_t)p.GD + (size_t)g * p.D +
                       (size_t)lane_c * CPL;
    float acc[CPL];
#pragma unroll
    for (int c = 0; c < CPL; ++c) acc[c] = 0.f;
    StencilWalk sw;
    sw.start(p);
    for (int k = 0; k < K; ++k, sw.next(p)) {
        const float ox = row_ok ? trow[3 * k] : 0.f, oy = row_ok ? trow[3 * k + 1] : 0.f, oz = row_ok ? trow[3 * k + 2] : 0.f;
        const float a = row_ok ? (p.softmax ? __expf(trow[3 * K + k] - m) * inv : trow[3 * K + k]) : 0.f;
        const float w_im = sb.w + ((float)(sw.i * p.dw) + ox) * p.offset_scale;
        const float h_im = sb.h + ((float)(sw.j * p.dh) + oy) * p.offset_scale;
        const float d_im = sb.d + ((float)(sw.k * p.dd) + oz) * p.offset_scale;
        PointGeom pg;
        point_geometry_voxel(lv, p.GD, w_im, h_im, d_im, pg);
        uint4 raw[8];
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            const bool in = active && pg.zin[n >> 2] && pg.yin[(n >> 1) & 1] && pg.xin[n & 1];
            raw[n] = in ? ldg16_hint(value_b + pg.off[n], pol) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int n = 0; n < 8; ++n) axpy16<T>(raw[n], a * ((pg.wx[n & 1] * pg.wy[(n >> 1) & 1]) * pg.wz[n >> 2]), acc);
    }
    if (active) {
        T *dst = static_cast<T *>(p.out) + ((size_t)b * p.rows_per_b + row) * (size_t)p.D + (size_t)lane_c * CPL;
        stg16_hint(dst, Vec16<T>::pack(acc), l2_policy_evict_first());
    }
}

// Tile row (fp32): [0,3K) offsets -> offset gradients, [3K,4K) masks -> raw dmask -> mask gradients, [4K,5K) soft-max probabilities.
template <typename T>
__global__ void __launch_bounds__(fda::kThreads, 2) dcnv4_backward_kernel(const DcnProblem p) {
    using namespace fda;
    constexpr int CPL = Vec16<T>::kCPL;
    extern __shared__ __align__(16) float smem_tile[];
    const int tid = threadIdx.x, b = blockIdx.y;
    const int gs = 1 << p.gs_log2, lane = tid & 31, warp = tid >> 5;
    const int lane_c = tid & (gs - 1);
    const int rows_per_block = (int)blockDim.x >> p.gs_log2, rows_per_warp = 32 >> p.gs_log2;
    const int row = blockIdx.x * rows_per_block + (tid >> p.gs_log2);
    const bool row_ok = row < p.rows_per_b, active = row_ok && lane_c < p.lpg;
    const int first = blockIdx.x * rows_per_block + warp * rows_per_warp;
    float *wtile = smem_tile + warp * rows_per_warp * p.row_stride;
    int nrows = p.rows_per_b - first;
    nrows = nrows < 0 ? 0 : (nrows > rows_per_warp ? rows_per_warp : nrows);
    stage_dcn_rows<T>(p, b, first, nrows, wtile, lane);
    __syncwarp();
    float *trow = wtile + (lane >> p.gs_log2) * p.row_stride;
    const int K = p.K;

    if (row_ok) {  // probabilities (or the masks themselves) into [4K, 5K): written by the row's first lane
        float m = -INFINITY, s = 0.f;
        if (p.softmax) {
            for (int k = 0; k < K; ++k) m = fmaxf(m, trow[3 * K + k]);
            for (int k = 0; k < K; ++k) s += __expf(trow[3 * K + k] - m);
        }
        const float inv = p.softmax ? 1.0f / s : 1.f;
        for (int k = lane_c; k < K; k += gs)
            trow[4 * K + k] = p.softmax ? __expf(trow[3 * K + k] - m) * inv : trow[3 * K + k];
    }
    __syncwarp();

    LevelGeom lv;
    lv.D = p.Din; lv.H = p.Hin; lv.W = p.Win; lv.start = 0; lv.keep = 0;
    lv.fD = (float)p.Din; lv.fH = (float)p.Hin; lv.fW = (float)p.Win;
    const size_t cells = (size_t)p.Din * p.Hin * p.Win;
    unsigned long long budget = p.l2_keep_bytes;
    const bool keep_image = cells * p.GD * 4ull <= budget;
    if (keep_image) budget -= cells * p.GD * 4ull;
    const bool keep_value = cells * p.GD * sizeof(T) <= budget;
    const uint64_t pol_keep = l2_policy_evict_last(), pol_stream = l2_policy_evict_first(), pol_norm = l2_policy_evict_normal();
    const uint64_t pol_v = keep_value ? pol_keep : pol_norm, pol_g = keep_image ? pol_keep : pol_norm;
    const int q = row_ok ? row / p.G : 0, g = row_ok ? row - q * p.G : 0;
    const StencilBase sb = stencil_base(p, q);
    const size_t head_elem = (size_t)b * cells * p.GD + (size_t)g * p.D;
    const T *value_b = static_cast<const T *>(p.value) + head_elem + (size_t)lane_c * CPL;
    float *accum_b = p.accum + head_elem + (size_t)lane_c * 4;
    RowGrad<T> go;
    go.load(static_cast<const T *>(p.grad_out) + ((size_t)b * p.rows_per_b + (row_ok ? row : 0)) * (size_t)p.D, lane_c, p.lpg,
            active, pol_stream);
    const int red_stride = 4 * p.lpg;

    StencilWalk sw;
    sw.start(p);
    for (int k = 0; k < K; ++k, sw.next(p)) {
        const float ox = row_ok ? trow[3 * k] : 0.f, oy = row_ok ? trow[3 * k + 1] : 0.f, oz = row_ok ? trow[3 * k + 2] : 0.f;
        const float a = row_ok ? trow[4 * K + k] : 0.f;
        const float w_im = sb.w + ((float)(sw.i * p.dw) + ox) * p.offset_scale;
        const float h_im = sb.h + ((float)(sw.j * p.dh) + oy) * p.offset_scale;
        const float d_im = sb.d + ((float)(sw.k * p.dd) + oz) * p.offset_scale;
        PointGeom pg;
        point_geometry_voxel(lv, p.GD, w_im, h_im, d_im, pg);
        float gx, gy, gz, da;
        point_backward_geom<T, false>(pg, a, value_b, accum_b, go, red_stride, active, gs, pol_v, pol_g, gx, gy, gz, da);
        __syncwarp();  // every lane of the row has read this point's offsets
        if (row_ok && lane_c == 0) {
            // d p / d offset = offset_scale along each axis (csrc/cuda/dcnv4_col2im_cuda.cuh:205)
            trow[3 * k] = a * p.offset_scale * gx;
            trow[3 * k + 1] = a * p.offset_scale * gy;
            trow[3 * k + 2] = a * p.offset_scale * gz;
            trow[3 * K + k] = da;
        }
    }
    __syncwarp();
    if (p.softmax) {  // uniform branch: the warp barrier inside is reached by every lane
        float S = 0.f;  // sum_j m_j * dmask_j
        if (row_ok)
            for (int k = 0; k < K; ++k) S = fmaf(trow[4 * K + k], trow[3 * K + k], S);
        __syncwarp();
        if (row_ok)
            for (int k = lane_c; k < K; k += gs) trow[3 * K + k] = trow[4 * K + k] * (trow[3 * K + k] - S);
    }
    __syncwarp();
    // write the finished gradient rows (the padding of the offset rows is cleared by the host's memset)
    const int per_row = 4 * K;
    T *gbase = static_cast<T *>(p.grad_offset) + (size_t)b * p.Q * (size_t)p.padded;
    for (int r = 0; r < nrows; ++r) {
        const int rr = first + r, qq = rr / p.G, gg = rr - qq * p.G;
        T *dst = gbase + (size_t)qq * p.padded + (size_t)gg * per_row;
        for (int e = lane; e < per_row; e += 32) fda::store1<T>(dst + e, wtile[r * p.row_stride + e]);
    }
}

inline int dtype_size(int dt) { return dt == FDA_DTYPE_F32 ? 4 : 2; }

int fill_problem(DcnProblem &p, int batch, int depth_in, int height_in, int width_in, int group, int group_channels,
                 const int *kernel, const int *stride, const int *pad, const int *dilation, float offset_scale,
                 int remove_center, int softmax, int padded_offset_dim, int dtype, int im2col_step) {
    if (dtype < 0 || dtype > 2) return FDA_ERR_BAD_DTYPE;
    if (batch <= 0 || depth_in <= 0 || height_in <= 0 || width_in <= 0 || group <= 0 || group_channels <= 0) return FDA_ERR_BAD_SHAPE;
    for (int a = 0; a < 3; ++a)
        if (kernel[a] <= 0 || stride[a] <= 0 || pad[a] < 0 || dilation[a] <= 0) return FDA_ERR_BAD_SHAPE;
    const int cpl = 16 / dtype_size(dtype);
    if (group_channels % cpl != 0 || group_channels / cpl > 32) return FDA_ERR_BAD_HEAD_DIM;
    const int step = batch < im2col_step ? batch : im2col_step;
    if (step <= 0 || batch % step != 0) return FDA_ERR_IM2COL_STEP;
    p.B = batch; p.G = group; p.D = group_channels;
    p.Din = depth_in; p.Hin = height_in; p.Win = width_in;
    p.kd = kernel[0]; p.kh = kernel[1]; p.kw = kernel[2];
    p.sd = stride[0]; p.sh = stride[1]; p.sw = stride[2];
    p.pd = pad[0]; p.ph = pad[1]; p.pw = pad[2];
    p.dd = dilation[0]; p.dh = dilation[1]; p.dw = dilation[2];
    p.Dout = (depth_in + 2 * p.pd - (p.dd * (p.kd - 1) + 1)) / p.sd + 1;
    p.Hout = (height_in + 2 * p.ph - (p.dh * (p.kh - 1) + 1)) / p.sh + 1;
    p.Wout = (width_in + 2 * p.pw - (p.dw * (p.kw - 1) + 1)) / p.sw + 1;
    if (p.Dout <= 0 || p.Hout <= 0 || p.Wout <= 0) return FDA_ERR_BAD_SHAPE;
    p.K = p.kd * p.kh * p.kw - (remove_center ? 1 : 0);
    if (p.K <= 0 || p.K > 343) return FDA_ERR_BAD_POINTS;
    if (padded_offset_dim < group * p.K * 4) return FDA_ERR_BAD_SHAPE;
    const long long Q = (long long)p.Dout * p.Hout * p.Wout;
    if (Q * group >= (1ll << 31) || (long long)depth_in * height_in * width_in * group * group_channels >= (1ll << 31)) return FDA_ERR_BAD_SHAPE;
    if (batch > 65535) return FDA_ERR_BAD_SHAPE;
    p.Q = (int)Q; p.padded = padded_offset_dim;
    p.offset_scale = offset_scale; p.remove_center = remove_center ? 1 : 0; p.softmax = softmax ? 1 : 0;
    p.lpg = group_channels / cpl;
    int lg = 0;
    while ((1 << lg) < p.lpg) ++lg;
    p.gs_log2 = lg;
    p.rows_per_b = p.Q * group;
    p.GD = group * group_channels;
    p.l2_keep_bytes = (unsigned long long)(fda::config().l2_keep_fraction * 126.0 * 1024 * 1024);
    return FDA_OK;
}

template <typename T>
int launch_dcn(const DcnProblem &p0, bool backward, cudaStream_t st) {
    DcnProblem p = p0;
    p.row_stride = (backward ? 5 : 4) * p.K + 1;  // odd: the rows of a warp start in different banks
    int threads = fda::kThreads;
    while (threads > 32 && (size_t)(threads >> p.gs_log2) * p.row_stride * sizeof(float) > 96 * 1024) threads >>= 1;
    const size_t smem = (size_t)(threads >> p.gs_log2) * p.row_stride * sizeof(float);
    if (smem > 200 * 1024) return FDA_ERR_TOO_LARGE_STATIC;
    const int rows_per_block = threads >> p.gs_log2;
    const dim3 grid((unsigned)((p.rows_per_b + rows_per_block - 1) / rows_per_block), (unsigned)p.B, 1);
    auto kern = backward ? dcnv4_backward_kernel<T> : dcnv4_forward_kernel<T>;
    if (smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) { fda::record_cuda_error((int)e); return FDA_ERR_CUDA; }
    }
    kern<<<grid, threads, smem, st>>>(p);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { fda::record_cuda_error((int)e); return FDA_ERR_CUDA; }
    return FDA_OK;
}

int dispatch_dcn(const DcnProblem &p, int dtype, bool backward, cudaStream_t st) {
    if (dtype == FDA_DTYPE_F32) return launch_dcn<float>(p, backward, st);
    if (dtype == FDA_DTYPE_F16) return launch_dcn<__half>(p, backward, st);
    return launch_dcn<__nv_bfloat16>(p, backward, st);
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

extern "C" int fda_dcnv4_output_size(int depth_in, int height_in, int width_in, const int *kernel, const int *stride,
                                     const int *pad, const int *dilation, int *depth_out, int *height_out, int *width_out) {
    if (!kernel || !stride || !pad || !dilation || !depth_out || !height_out || !width_out) return FDA_ERR_NULL_POINTER;
    for (int a = 0; a < 3; ++a)
        if (kernel[a] <= 0 || stride[a] <= 0 || pad[a] < 0 || dilation[a] <= 0) return FDA_ERR_BAD_SHAPE;
    *depth_out = (depth_in + 2 * pad[0] - (dilation[0] * (kernel[0] - 1) + 1)) / stride[0] + 1;
    *height_out = (height_in + 2 * pad[1] - (dilation[1] * (kernel[1] - 1) + 1)) / stride[1] + 1;
    *width_out = (width_in + 2 * pad[2] - (dilation[2] * (kernel[2] - 1) + 1)) / stride[2] + 1;
    return (*depth_out > 0 && *height_out > 0 && *width_out > 0) ? FDA_OK : FDA_ERR_BAD_SHAPE;
}

extern "C" int fda_dcnv4_forward(const void *value, const void *p_offset, void *output, int batch, int depth_in, int height_in,
                                 int width_in, int group, int group_channels, const int *kernel, const int *stride,
                                 const int *pad, const int *dilation, float offset_scale, int remove_center, int softmax,
                                 int padded_offset_dim, int dtype, int im2col_step, void *stream) {
    if (!value || !p_offset || !output || !kernel || !stride || !pad || !dilation) return FDA_ERR_NULL_POINTER;
    DcnProblem p{};
    if (int rc = fill_problem(p, batch, depth_in, height_in, width_in, group, group_channels, kernel, stride, pad, dilation,
                              offset_scale, remove_center, softmax, padded_offset_dim, dtype, im2col_step))
        return rc;
    if (!aligned16(value) || !aligned16(output)) return FDA_ERR_MISALIGNED;
    p.value = value; p.offset = p_offset; p.out = output;
    return dispatch_dcn(p, dtype, false, static_cast<cudaStream_t>(stream));
}

extern "C" size_t fda_dcnv4_backward_workspace_bytes(int batch, int depth_in, int height_in, int width_in, int group,
                                                     int group_channels, int dtype) {
    if (dtype == FDA_DTYPE_F32 || batch <= 0 || depth_in <= 0 || height_in <= 0 || width_in <= 0 || group <= 0 || group_channels <= 0)
        return 0;
    return (size_t)batch * depth_in * height_in * width_in * group * group_channels * sizeof(float);
}

extern "C" int fda_dcnv4_backward(const void *value, const void *p_offset, const void *grad_output, void *grad_value,
                                  void *grad_offset, void *workspace, size_t workspace_bytes, int batch, int depth_in,
                                  int height_in, int width_in, int group, int group_channels, const int *kernel,
                                  const int *stride, const int *pad, const int *dilation, float offset_scale,
                                  int remove_center, int softmax, int padded_offset_dim, int dtype, int im2col_step,
                                  void *stream) {
    if (!value || !p_offset || !grad_output || !grad_value || !grad_offset || !kernel || !stride || !pad || !dilation)
        return FDA_ERR_NULL_POINTER;
    DcnProblem p{};
    if (int rc = fill_problem(p, batch, depth_in, height_in, width_in, group, group_channels, kernel, stride, pad, dilation,
                              offset_scale, remove_center, softmax, padded_offset_dim, dtype, im2col_step))
        return rc;
    const size_t need = fda_dcnv4_backward_workspace_bytes(batch, depth_in, height_in, width_in, group, group_channels, dtype);
    if (need > 0 && (!workspace || workspace_bytes < need)) return FDA_ERR_WORKSPACE;
    if (!aligned16(value) || !aligned16(grad_output) || !aligned16(grad_value) || (need > 0 && !aligned16(workspace)))
        return FDA_ERR_MISALIGNED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t n = (size_t)batch * depth_in * height_in * width_in * group * group_channels;
    float *accum = need > 0 ? static_cast<float *>(workspace) : static_cast<float *>(grad_value);
    cudaError_t e = cudaMemsetAsync(accum, 0, n * sizeof(float), st);
    if (e == cudaSuccess)
        e = cudaMemsetAsync(grad_offset, 0, (size_t)batch * p.Q * (size_t)padded_offset_dim * dtype_size(dtype), st);
    if (e != cudaSuccess) { fda::record_cuda_error((int)e); return FDA_ERR_CUDA; }
    p.value = value; p.offset = p_offset; p.grad_out = grad_output; p.accum = accum; p.grad_offset = grad_offset;
    if (int rc = dispatch_dcn(p, dtype, true, st)) return rc;
    if (need == 0) return FDA_OK;
    return fda_cast_grad_value(accum, grad_value, n, dtype, stream);
}
