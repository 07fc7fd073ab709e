// Backward pass for callers that cannot provide (or allocate) a workspace.
//
// Who this is for: code that runs where device allocation is off the table -- an engine plug-in
// whose execute hook may not call cudaMalloc, a process whose memory pool has already claimed
// the whole GPU so that a fresh cudaMalloc fails, or a latency-critical loop that cannot afford
// the device-wide synchronisation an allocation implies.  Such callers still own their inputs
// and outputs, but have nowhere to put the fp32 accumulation image that the 16-bit backward
// needs.  Here that image lives in a fixed array inside the library.
//
// Cost and limits: the array occupies FDA_NOALLOC_MAX_ELEMENTS * 4 bytes (64 MiB) on every GPU
// that loads this library, until the process exits.  Problems whose grad_value has more elements
// than that are rejected.  All calls share the one array, so two calls that overlap in time on
// the same GPU (different streams, different threads) corrupt each other; issue them in order.
// The array keeps whatever the last call left in it; each call clears the part it uses first.
//
// First call on a device: it resolves the array's device address.  With the CUDA runtime's lazy
// module loading that lookup is also what loads this module onto the device and gives the array
// its 64 MiB, so a process whose pool is about to claim the whole GPU should make one (tiny) call
// at start-up, before the pool grows and before any stream capture; later calls only launch.
#include "../../include/fda_b200.h"

#include "fda_config.h"

#include <cuda_runtime.h>

#include <mutex>

namespace {

constexpr size_t kMaxElements = FDA_NOALLOC_MAX_ELEMENTS;
constexpr int kMaxDevices = 64;

// fp32 accumulation image.  Inside host code this NAME is only a handle for the runtime, not a
// device address: the address is looked up per device below and that pointer is what kernels get.
static __device__ __align__(256) float g_accum_image[kMaxElements];

std::mutex g_mu;
float *g_image_ptr[kMaxDevices] = {};

// Device address of the image on the current device; looked up on the first call per device.
int image_pointer(float **out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { fda::record_cuda_error((int)e); return FDA_ERR_CUDA; }
    if (dev < 0 || dev >= kMaxDevices) return FDA_ERR_TOO_LARGE_STATIC;
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_image_ptr[dev]) {
        float *ptr = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_accum_image);
        if (e != cudaSuccess || !ptr) {  // e.g. out of memory when the module cannot be loaded any more
            fda::record_cuda_error((int)(e != cudaSuccess ? e : cudaErrorInvalidSymbol));
            return FDA_ERR_CUDA;
        }
        g_image_ptr[dev] = ptr;
    }
    *out = g_image_ptr[dev];
    return FDA_OK;
}

}  // namespace

extern "C" int fda_backward_noalloc(const void *value, const int64_t *spatial_shapes, const int64_t *level_start_index,
                                    const void *sampling_loc_attn, const void *grad_output,
                                    void *grad_value, void *grad_sampling_loc_attn,
                                    int batch, int num_value, int num_heads, int head_dim, int num_levels,
                                    int num_query, int num_points, int value_dtype, int packed_dtype,
                                    int im2col_step, void *stream) {
    if (!grad_value) return FDA_ERR_NULL_POINTER;
    if (batch <= 0 || num_value <= 0 || num_heads <= 0 || head_dim <= 0) return FDA_ERR_BAD_SHAPE;
    const size_t n = (size_t)batch * num_value * num_heads * head_dim;
    if (value_dtype == FDA_DTYPE_F32) {
        // fp32 gradients accumulate straight into grad_value: no image needed, no size limit
        return fda_backward_accumulate(value, spatial_shapes, level_start_index, sampling_loc_attn, grad_output,
                                       static_cast<float *>(grad_value), grad_sampling_loc_attn, batch, num_value,
                                       num_heads, head_dim, num_levels, num_query, num_points, value_dtype,
                                       packed_dtype, im2col_step, stream);
    }
    if (n > kMaxElements) return FDA_ERR_TOO_LARGE_STATIC;
    float *image = nullptr;
    if (int rc = image_pointer(&image)) return rc;
    // zero-fills image[0, n) on `stream`, then scatters into it and writes grad_sampling_loc_attn
    int rc = fda_backward_accumulate(value, spatial_shapes, level_start_index, sampling_loc_attn, grad_output, image,
                                     grad_sampling_loc_attn, batch, num_value, num_heads, head_dim, num_levels,
                                     num_query, num_points, value_dtype, packed_dtype, im2col_step, stream);
    if (rc != FDA_OK) return rc;
    return fda_cast_grad_value(image, grad_value, n, value_dtype, stream);
}
