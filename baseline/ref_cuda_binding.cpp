// Binding TU used only to time the REFERENCE's own CUDA kernels as a reported baseline.
// It includes the reference's headers from the reference checkout (-I <checkout>/csrc at build
// time); no reference source is copied into this repository.  Built by baseline/build_ref_cuda.sh
// into baseline/_ref/ (git-ignored).
#include <torch/extension.h>
#define WITH_CUDA 1
#include "flash_deform_attn.h"

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("flash_deform_attn_forward", &flash_deform_attn_forward, "reference forward");
    m.def("flash_deform_attn_backward", &flash_deform_attn_backward, "reference backward");
}
