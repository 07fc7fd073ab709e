// Binding TU used only to run the REFERENCE's own DCNv4-3D CUDA kernels (golden vectors for the oracle).
// It includes the reference's headers from the reference checkout (-I <checkout>/csrc at build time); no
// reference source is copied into this repository.  Built by baseline/build_ref_cuda.sh --dcnv4 into
// baseline/_ref/ (git-ignored).
#include <torch/extension.h>
#define WITH_CUDA 1
#include "dcnv4.h"

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("dcnv4_forward", &dcnv4_forward, "reference DCNv4-3D forward");
    m.def("dcnv4_backward", &dcnv4_backward, "reference DCNv4-3D backward");
}
