#!/usr/bin/env bash
# Builds the reference's Flash Deformable Attention CUDA kernels (unmodified, from the reference
# checkout given as $1) for sm_100a into baseline/_ref/ops3d_ref_C.so, as a baseline to time beside
# this repository's kernels.  Takes about ten minutes (the reference instantiates ~700 kernels).
#   build_ref_cuda.sh <checkout>            -> baseline/_ref/ops3d_ref_C.so       (deformable attention; timed by bench.py)
#   build_ref_cuda.sh <checkout> --dcnv4    -> baseline/_ref/ops3d_ref_dcnv4.so   (DCNv4-3D; golden vectors for the oracle)
#   build_ref_cuda.sh <checkout> --detection -> baseline/_ref/ops3d_ref_detection.so (ROI-Align 3D + NMS 3D; golden vectors)
set -euo pipefail
REF="${1:?path of the reference checkout}"
WHAT="${2:-}"
HERE="$(cd "$(dirname "$0")" && pwd)"
OUT="$HERE/_ref"
mkdir -p "$OUT"
PY=python
INC=$($PY - <<'PYEOF'
import sysconfig
from torch.utils import cpp_extension as ce
print(" ".join("-isystem " + p for p in ce.include_paths("cuda") + [sysconfig.get_paths()["include"]]))
PYEOF
)
TORCH_LIB=$($PY -c "import torch,os;print(os.path.join(os.path.dirname(torch.__file__),'lib'))")
ABI=$($PY -c "import torch;print(int(torch._C._GLIBCXX_USE_CXX11_ABI))")
if [ "$WHAT" = "--dcnv4" ]; then
  COMMON="-O3 -std=c++17 -DTORCH_EXTENSION_NAME=ops3d_ref_dcnv4 -DTORCH_API_INCLUDE_EXTENSION_H -D_GLIBCXX_USE_CXX11_ABI=$ABI $INC"
  nvcc -gencode arch=compute_100a,code=sm_100a $COMMON -DWITH_CUDA -DCUDA_HAS_FP16=1 \
       -D__CUDA_NO_HALF_OPERATORS__ -D__CUDA_NO_HALF_CONVERSIONS__ -D__CUDA_NO_HALF2_OPERATORS__ \
       -Xcompiler -fPIC -w -c "$REF/csrc/cuda/dcnv4_cuda.cu" -o "$OUT/dcnv4_cuda.o"
  g++ $COMMON -fPIC -w -I"$REF/csrc" -c "$HERE/ref_dcnv4_binding.cpp" -o "$OUT/ref_dcnv4_binding.o"
  g++ -shared "$OUT/dcnv4_cuda.o" "$OUT/ref_dcnv4_binding.o" -o "$OUT/ops3d_ref_dcnv4.so" \
      -L"$TORCH_LIB" -Wl,-rpath,"$TORCH_LIB" -L/usr/local/cuda/lib64 -lc10 -lc10_cuda -ltorch_cpu -ltorch_cuda -ltorch -ltorch_python -lcudart
  rm -f "$OUT"/*.o
  echo "built $OUT/ops3d_ref_dcnv4.so"
  exit 0
fi
if [ "$WHAT" = "--detection" ]; then
  COMMON="-O3 -std=c++17 -DTORCH_EXTENSION_NAME=ops3d_ref_detection -DTORCH_API_INCLUDE_EXTENSION_H -D_GLIBCXX_USE_CXX11_ABI=$ABI $INC"
  for tu in roi_align_3d_cuda nms_3d_cuda; do
    nvcc -gencode arch=compute_100a,code=sm_100a $COMMON -DWITH_CUDA -DCUDA_HAS_FP16=1 \
         -D__CUDA_NO_HALF_OPERATORS__ -D__CUDA_NO_HALF_CONVERSIONS__ -D__CUDA_NO_HALF2_OPERATORS__ \
         -Xcompiler -fPIC -w -c "$REF/csrc/cuda/$tu.cu" -o "$OUT/$tu.o"
  done
  g++ $COMMON -fPIC -w -I"$REF/csrc" -c "$HERE/ref_detection_binding.cpp" -o "$OUT/ref_detection_binding.o"
  g++ -shared "$OUT/roi_align_3d_cuda.o" "$OUT/nms_3d_cuda.o" "$OUT/ref_detection_binding.o" -o "$OUT/ops3d_ref_detection.so" \
      -L"$TORCH_LIB" -Wl,-rpath,"$TORCH_LIB" -L/usr/local/cuda/lib64 -lc10 -lc10_cuda -ltorch_cpu -ltorch_cuda -ltorch -ltorch_python -lcudart
  rm -f "$OUT"/*.o
  echo "built $OUT/ops3d_ref_detection.so"
  exit 0
fi
COMMON="-O3 -std=c++17 -DTORCH_EXTENSION_NAME=ops3d_ref_C -DTORCH_API_INCLUDE_EXTENSION_H -D_GLIBCXX_USE_CXX11_ABI=$ABI $INC"
nvcc -gencode arch=compute_100a,code=sm_100a $COMMON -DWITH_CUDA -DCUDA_HAS_FP16=1 \
     -D__CUDA_NO_HALF_OPERATORS__ -D__CUDA_NO_HALF_CONVERSIONS__ -D__CUDA_NO_HALF2_OPERATORS__ \
     -Xcompiler -fPIC -w -c "$REF/csrc/cuda/flash_deform_attn_cuda.cu" -o "$OUT/flash_deform_attn_cuda.o"
g++ $COMMON -fPIC -w -I"$REF/csrc" -c "$HERE/ref_cuda_binding.cpp" -o "$OUT/ref_cuda_binding.o"
g++ -shared "$OUT/flash_deform_attn_cuda.o" "$OUT/ref_cuda_binding.o" -o "$OUT/ops3d_ref_C.so" \
    -L"$TORCH_LIB" -Wl,-rpath,"$TORCH_LIB" -L/usr/local/cuda/lib64 -lc10 -lc10_cuda -ltorch_cpu -ltorch_cuda -ltorch -ltorch_python -lcudart
rm -f "$OUT"/*.o
echo "built $OUT/ops3d_ref_C.so"
