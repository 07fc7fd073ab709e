// Thin torch binding over the C ABI of include/fda_b200.h.
//
// Exposes, positional-only like the reference's module (csrc/vision.cpp:23-24):
//   flash_deform_attn_forward (value, spatial_shapes, level_start_index, sampling_loc_attn,
//                              im2col_step, K, d_stride, block_thread, use_reg) -> Tensor[B,Lq,G*D]
//   flash_deform_attn_backward(value, spatial_shapes, level_start_index, sampling_loc_attn,
//                              grad_output, im2col_step, K, d_stride, block_thread)
//                              -> [grad_value[B,N,G,D], grad_sampling_loc_attn[B,Lq,G,L*K*4]]
// with the argument meaning and error behaviour of csrc/flash_deform_attn.h:7-52 and
// csrc/cuda/flash_deform_attn_cuda.cu:20-179: RuntimeError for CPU / non-contiguous tensors and
// for batch % min(batch, im2col_step) != 0, ValueError for an unsupported level or point count.
// This file only checks tensors, allocates outputs from torch's allocator, and forwards raw
// pointers plus the current CUDA stream; all arithmetic lives behind the C ABI.
#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/fda_b200.h"

namespace {

int dtype_code(const at::Tensor &t, const char *name) {
    switch (t.scalar_type()) {
        case at::kFloat: return FDA_DTYPE_F32;
        case at::kHalf: return FDA_DTYPE_F16;
        case at::kBFloat16: return FDA_DTYPE_BF16;
        default: TORCH_CHECK(false, name, " must be float32, float16 or bfloat16, got ", t.scalar_type());
    }
    return -1;
}

void check_cuda_contiguous(const at::Tensor &t, const char *name) {
    TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor (this operator has no CPU implementation)");
    TORCH_CHECK(t.is_contiguous(), name, " tensor has to be contiguous");
}

void raise_status(int status, const char *what) {
    if (status == FDA_OK) return;
    std::string msg = std::string(what) + ": " + fda_status_string(status);
    if (status == FDA_ERR_CUDA) msg += std::string(" (") + cudaGetErrorString((cudaError_t)fda_last_cuda_error()) + ")";
    // the reference raises std::invalid_argument (-> ValueError) for level / point counts outside its ladders
    if (status == FDA_ERR_BAD_LEVELS || status == FDA_ERR_BAD_POINTS) throw std::invalid_argument(msg);
    TORCH_CHECK(false, msg);
}

struct Dims {
    int B, N, G, D, L, Q;
};

Dims check_common(const at::Tensor &value, const at::Tensor &spatial_shapes, const at::Tensor &level_start_index,
                  const at::Tensor &sampling_loc_attn, int K) {
    check_cuda_contiguous(value, "value");
    check_cuda_contiguous(spatial_shapes, "spatial_shapes");
    check_cuda_contiguous(level_start_index, "level_start_index");
    check_cuda_contiguous(sampling_loc_attn, "sampling_loc_attn");
    TORCH_CHECK(value.dim() == 4, "value must be [B, N, G, D]");
    TORCH_CHECK(sampling_loc_attn.dim() == 4, "sampling_loc_attn must be [B, Lq, G, L*K*4]");
    TORCH_CHECK(spatial_shapes.dim() == 2 && spatial_shapes.size(1) == 3, "spatial_shapes must be [L, 3]");
    TORCH_CHECK(spatial_shapes.scalar_type() == at::kLong && level_start_index.scalar_type() == at::kLong,
                "spatial_shapes and level_start_index must be int64");
    TORCH_CHECK(level_start_index.numel() == spatial_shapes.size(0), "level_start_index must have one entry per level");
    TORCH_CHECK(value.device() == sampling_loc_attn.device() && value.device() == spatial_shapes.device() &&
                    value.device() == level_start_index.device(),
                "all tensors must be on the same device");
    Dims d;
    d.B = (int)value.size(0); d.N = (int)value.size(1); d.G = (int)value.size(2); d.D = (int)value.size(3);
    d.L = (int)spatial_shapes.size(0);
    d.Q = (int)sampling_loc_attn.size(1);
    TORCH_CHECK(sampling_loc_attn.size(0) == d.B && sampling_loc_attn.size(2) == d.G,
                "sampling_loc_attn batch / head dimensions do not match value");
    TORCH_CHECK(sampling_loc_attn.size(3) == (int64_t)d.L * K * 4, "sampling_loc_attn last dimension (",
                sampling_loc_attn.size(3), ") does not match L*K*4 = ", (int64_t)d.L * K * 4);
    return d;
}

at::Tensor flash_deform_attn_forward(const at::Tensor &value, const at::Tensor &spatial_shapes,
                                     const at::Tensor &level_start_index, const at::Tensor &sampling_loc_attn,
                                     const int im2col_step, const int K, const int d_stride, const int block_thread,
                                     const bool use_reg) {
    const Dims d = check_common(value, spatial_shapes, level_start_index, sampling_loc_attn, K);
    const int vdt = dtype_code(value, "value"), pdt = dtype_code(sampling_loc_attn, "sampling_loc_attn");
    c10::cuda::CUDAGuard guard(value.device());
    if (d.Q == 0 || d.B == 0) return at::zeros({d.B, d.Q, d.G * d.D}, value.options());
    at::Tensor output = at::empty({d.B, d.Q, d.G * d.D}, value.options());
    const int rc = fda_forward(value.data_ptr(), spatial_shapes.data_ptr<int64_t>(), level_start_index.data_ptr<int64_t>(),
                               sampling_loc_attn.data_ptr(), output.data_ptr(), d.B, d.N, d.G, d.D, d.L, d.Q, K, vdt, pdt,
                               im2col_step, d_stride, block_thread, use_reg ? 1 : 0,
                               at::cuda::getCurrentCUDAStream().stream());
    raise_status(rc, "flash_deform_attn_forward");
    return output;
}

std::vector<at::Tensor> flash_deform_attn_backward(const at::Tensor &value, const at::Tensor &spatial_shapes,
                                                   const at::Tensor &level_start_index,
                                                   const at::Tensor &sampling_loc_attn, const at::Tensor &grad_output,
                                                   const int im2col_step, const int K, const int d_stride,
                                                   const int block_thread) {
    const Dims d = check_common(value, spatial_shapes, level_start_index, sampling_loc_attn, K);
    check_cuda_contiguous(grad_output, "grad_output");
    TORCH_CHECK(grad_output.scalar_type() == value.scalar_type(), "grad_output must have the dtype of value");
    TORCH_CHECK(grad_output.numel() == (int64_t)d.B * d.Q * d.G * d.D, "grad_output must be [B, Lq, G*D]");
    const int vdt = dtype_code(value, "value"), pdt = dtype_code(sampling_loc_attn, "sampling_loc_attn");
    c10::cuda::CUDAGuard guard(value.device());
    if (d.Q == 0 || d.B == 0) return {at::zeros_like(value), at::zeros_like(sampling_loc_attn)};
    at::Tensor grad_value = at::empty_like(value);
    at::Tensor grad_packed = at::empty_like(sampling_loc_attn);
    const size_t ws_bytes = fda_backward_workspace_bytes(d.B, d.N, d.G, d.D, d.L, d.Q, K, vdt, pdt);
    at::Tensor workspace;
    void *ws_ptr = nullptr;
    if (ws_bytes > 0) {
        workspace = at::empty({(int64_t)((ws_bytes + 3) / sizeof(float))}, value.options().dtype(at::kFloat));
        ws_ptr = workspace.data_ptr();
    }
    const int rc = fda_backward(value.data_ptr(), spatial_shapes.data_ptr<int64_t>(), level_start_index.data_ptr<int64_t>(),
                                sampling_loc_attn.data_ptr(), grad_output.data_ptr(), grad_value.data_ptr(),
                                grad_packed.data_ptr(), ws_ptr, ws_bytes, d.B, d.N, d.G, d.D, d.L, d.Q, K, vdt, pdt,
                                im2col_step, d_stride, block_thread, at::cuda::getCurrentCUDAStream().stream());
    raise_status(rc, "flash_deform_attn_backward");
    return {grad_value, grad_packed};
}

// DCNv4-3D with the positional signatures of the reference's binding (csrc/dcnv4.h:7-61, registered at
// csrc/vision.cpp:20-21).  d_stride and block_thread are the reference's launch hints: accepted, ignored.
struct DcnDims {
    int B, Din, Hin, Win, C, padded;
};

DcnDims check_dcn(const at::Tensor &value, const at::Tensor &p_offset, int group, int group_channels) {
    check_cuda_contiguous(value, "input");
    check_cuda_contiguous(p_offset, "offset");
    TORCH_CHECK(value.dim() == 5, "value must be [B, D, H, W, C]");
    TORCH_CHECK(p_offset.dim() == 5, "p_offset must be [B, D_out, H_out, W_out, padded_offset_dim]");
    TORCH_CHECK(p_offset.scalar_type() == value.scalar_type(), "p_offset must have the dtype of value");
    TORCH_CHECK(value.device() == p_offset.device(), "all tensors must be on the same device");
    DcnDims d;
    d.B = (int)value.size(0); d.Din = (int)value.size(1); d.Hin = (int)value.size(2); d.Win = (int)value.size(3);
    d.C = (int)value.size(4); d.padded = (int)p_offset.size(4);
    TORCH_CHECK(d.C == group * group_channels, "Input channels and group times group channels dont match: (", d.C, " vs ",
                group * group_channels, ").");
    return d;
}

at::Tensor dcnv4_forward(const at::Tensor &value, const at::Tensor &p_offset, const int kernel_d, const int kernel_h,
                         const int kernel_w, const int stride_d, const int stride_h, const int stride_w, const int pad_d,
                         const int pad_h, const int pad_w, const int dilation_d, const int dilation_h, const int dilation_w,
                         const int group, const int group_channels, const float offset_scale, const int im2col_step,
                         const int remove_center, const int d_stride, const int block_thread, const bool softmax) {
    (void)d_stride; (void)block_thread;
    const DcnDims d = check_dcn(value, p_offset, group, group_channels);
    const int kernel[3] = {kernel_d, kernel_h, kernel_w}, stride[3] = {stride_d, stride_h, stride_w};
    const int pad[3] = {pad_d, pad_h, pad_w}, dilation[3] = {dilation_d, dilation_h, dilation_w};
    int Do = 0, Ho = 0, Wo = 0;
    raise_status(fda_dcnv4_output_size(d.Din, d.Hin, d.Win, kernel, stride, pad, dilation, &Do, &Ho, &Wo), "dcnv4_forward");
    TORCH_CHECK(p_offset.size(0) == d.B && p_offset.size(1) == Do && p_offset.size(2) == Ho && p_offset.size(3) == Wo,
                "p_offset spatial shape does not match the output volume");
    c10::cuda::CUDAGuard guard(value.device());
    at::Tensor output = at::empty({d.B, Do, Ho, Wo, d.C}, value.options());
    raise_status(fda_dcnv4_forward(value.data_ptr(), p_offset.data_ptr(), output.data_ptr(), d.B, d.Din, d.Hin, d.Win, group,
                                   group_channels, kernel, stride, pad, dilation, offset_scale, remove_center, softmax ? 1 : 0,
                                   d.padded, dtype_code(value, "value"), im2col_step,
                                   at::cuda::getCurrentCUDAStream().stream()),
                 "dcnv4_forward");
    return output;
}

std::vector<at::Tensor> dcnv4_backward(const at::Tensor &value, const at::Tensor &p_offset, const int kernel_d,
                                       const int kernel_h, const int kernel_w, const int stride_d, const int stride_h,
                                       const int stride_w, const int pad_d, const int pad_h, const int pad_w,
                                       const int dilation_d, const int dilation_h, const int dilation_w, const int group,
                                       const int group_channels, const float offset_scale, const int im2col_step,
                                       const at::Tensor &grad_output, const int remove_center, const int d_stride,
                                       const int block_thread, const bool softmax) {
    (void)d_stride; (void)block_thread;
    const DcnDims d = check_dcn(value, p_offset, group, group_channels);
    check_cuda_contiguous(grad_output, "grad_output");
    TORCH_CHECK(grad_output.scalar_type() == value.scalar_type(), "grad_output must have the dtype of value");
    const int kernel[3] = {kernel_d, kernel_h, kernel_w}, stride[3] = {stride_d, stride_h, stride_w};
    const int pad[3] = {pad_d, pad_h, pad_w}, dilation[3] = {dilation_d, dilation_h, dilation_w};
    const int vdt = dtype_code(value, "value");
    c10::cuda::CUDAGuard guard(value.device());
    at::Tensor grad_value = at::empty_like(value);
    at::Tensor grad_offset = at::empty_like(p_offset);
    const size_t ws_bytes = fda_dcnv4_backward_workspace_bytes(d.B, d.Din, d.Hin, d.Win, group, group_channels, vdt);
    at::Tensor workspace;
    void *ws_ptr = nullptr;
    if (ws_bytes > 0) {
        workspace = at::empty({(int64_t)((ws_bytes + 3) / sizeof(float))}, value.options().dtype(at::kFloat));
        ws_ptr = workspace.data_ptr();
    }
    raise_status(fda_dcnv4_backward(value.data_ptr(), p_offset.data_ptr(), grad_output.data_ptr(), grad_value.data_ptr(),
                                    grad_offset.data_ptr(), ws_ptr, ws_bytes, d.B, d.Din, d.Hin, d.Win, group, group_channels,
                                    kernel, stride, pad, dilation, offset_scale, remove_center, softmax ? 1 : 0, d.padded, vdt,
                                    im2col_step, at::cuda::getCurrentCUDAStream().stream()),
                 "dcnv4_backward");
    return {grad_value, grad_offset};
}

// ROI-Align 3D and NMS 3D with the reference's binding signatures (csrc/roi_align_3d.h:96-136, csrc/nms_3d.h:28-44):
// the forward / backward write into tensors the caller allocated (and, for the backward, zero-filled).
void roi_align_3d_forward(at::Tensor input, at::Tensor rois, at::Tensor output, int aligned_depth, int aligned_height,
                          int aligned_width, float spatial_scale, int sampling_ratio, int order) {
    check_cuda_contiguous(input, "input");
    check_cuda_contiguous(rois, "rois");
    check_cuda_contiguous(output, "output");
    TORCH_CHECK(rois.dim() == 2 && rois.size(1) == 7, "wrong roi size! size_rois should be 7");
    TORCH_CHECK(input.dim() == 5, "input must be [N, C, D, H, W]");
    TORCH_CHECK(rois.scalar_type() == input.scalar_type() && output.scalar_type() == input.scalar_type(),
                "input, rois and output must share one dtype");
    TORCH_CHECK(output.numel() == rois.size(0) * input.size(1) * (int64_t)aligned_depth * aligned_height * aligned_width,
                "output must be [num_rois, C, aligned_depth, aligned_height, aligned_width]");
    c10::cuda::CUDAGuard guard(input.device());
    raise_status(fda_roi_align3d_forward(input.data_ptr(), rois.data_ptr(), output.data_ptr(), (int)rois.size(0), (int)input.size(1),
                                         (int)input.size(2), (int)input.size(3), (int)input.size(4), aligned_depth, aligned_height,
                                         aligned_width, spatial_scale, sampling_ratio, order, dtype_code(input, "input"),
                                         at::cuda::getCurrentCUDAStream().stream()),
                 "roi_align_3d_forward");
}

void roi_align_3d_backward(at::Tensor top_grad, at::Tensor rois, at::Tensor bottom_grad, int aligned_depth, int aligned_height,
                           int aligned_width, float spatial_scale, int sampling_ratio, int order) {
    check_cuda_contiguous(top_grad, "top_grad");
    check_cuda_contiguous(rois, "rois");
    check_cuda_contiguous(bottom_grad, "bottom_grad");
    TORCH_CHECK(rois.dim() == 2 && rois.size(1) == 7, "wrong roi size! size_rois should be 7");
    TORCH_CHECK(bottom_grad.dim() == 5, "bottom_grad must be [N, C, D, H, W]");
    TORCH_CHECK(rois.scalar_type() == at::kFloat && bottom_grad.scalar_type() == at::kFloat,
                "rois and bottom_grad must be float32 (gradients accumulate with fp32 atomics)");
    c10::cuda::CUDAGuard guard(top_grad.device());
    raise_status(fda_roi_align3d_backward(top_grad.data_ptr(), rois.data_ptr<float>(), bottom_grad.data_ptr<float>(), (int)rois.size(0),
                                          (int)bottom_grad.size(1), (int)bottom_grad.size(2), (int)bottom_grad.size(3),
                                          (int)bottom_grad.size(4), aligned_depth, aligned_height, aligned_width, spatial_scale,
                                          sampling_ratio, order, dtype_code(top_grad, "top_grad"),
                                          at::cuda::getCurrentCUDAStream().stream()),
                 "roi_align_3d_backward");
}

at::Tensor nms_3d(const at::Tensor &dets, const at::Tensor &scores, const float threshold) {
    TORCH_CHECK(dets.is_cuda() && scores.is_cuda(), "nms_3d: boxes and scores must be CUDA tensors (no CPU implementation)");
    c10::cuda::CUDAGuard guard(dets.device());
    if (dets.numel() == 0) return at::empty({0}, dets.options().dtype(at::kLong));
    TORCH_CHECK(dets.dim() == 2 && dets.size(1) == 6, "boxes must be [N, 6] = (x1, y1, z1, x2, y2, z2)");
    TORCH_CHECK(scores.numel() == dets.size(0), "one score per box");
    const int n = (int)dets.size(0);
    // score order; the stable sort makes ties deterministic (earlier box first)
    at::Tensor order = std::get<1>(scores.reshape({-1}).sort(/*stable=*/true, /*dim=*/0, /*descending=*/true));
    at::Tensor sorted = dets.index_select(0, order).to(at::kFloat).contiguous();
    const size_t ws_bytes = fda_nms3d_workspace_bytes(n);
    at::Tensor workspace = at::empty({(int64_t)(ws_bytes / 8 + 1)}, dets.options().dtype(at::kLong));
    at::Tensor keep = at::empty({n}, dets.options().dtype(at::kLong));
    at::Tensor num = at::zeros({1}, dets.options().dtype(at::kInt));
    raise_status(fda_nms3d(sorted.data_ptr<float>(), n, threshold, workspace.data_ptr(), ws_bytes,
                           reinterpret_cast<long long *>(keep.data_ptr<int64_t>()), num.data_ptr<int>(),
                           at::cuda::getCurrentCUDAStream().stream()),
                 "nms_3d");
    const int64_t kept = num.item<int>();  // the one host read: how many boxes survived
    return order.index_select(0, keep.narrow(0, 0, kept));
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "B200 Flash Deformable 3D Attention (torch binding over the fda_b200 C ABI)";
    m.def("flash_deform_attn_forward", &flash_deform_attn_forward, "Flash Deformable 3D Attention forward (sm_100a)");
    m.def("flash_deform_attn_backward", &flash_deform_attn_backward, "Flash Deformable 3D Attention backward (sm_100a)");
    m.def("nms_3d", &nms_3d, "non-maximum suppression for 3d boxes (sm_100a)");
    m.def("roi_align_3d_forward", &roi_align_3d_forward, "ROI-Align 3D forward (sm_100a)");
    m.def("roi_align_3d_backward", &roi_align_3d_backward, "ROI-Align 3D backward (sm_100a)");
    m.def("dcnv4_forward", &dcnv4_forward, "DCNv4-3D forward (sm_100a)");
    m.def("dcnv4_backward", &dcnv4_backward, "DCNv4-3D backward (sm_100a)");
}
