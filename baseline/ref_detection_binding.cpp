// Binding TU used only to run the REFERENCE's own ROI-Align 3D and NMS 3D CUDA kernels (golden vectors for the
// oracles).  It includes the reference's headers from the reference checkout (-I <checkout>/csrc at build time); no
// reference source is copied into this repository.  Built by baseline/build_ref_cuda.sh --detection into
// baseline/_ref/ (git-ignored).
#include <torch/extension.h>
#define WITH_CUDA 1
#include "nms_3d.h"
#include "roi_align_3d.h"

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("nms_3d", &nms_3d, "reference NMS 3D");
    m.def("roi_align_3d_forward", &roi_align_3d_forward, "reference ROI-Align 3D forward");
    m.def("roi_align_3d_backward", &roi_align_3d_backward, "reference ROI-Align 3D backward");
}
