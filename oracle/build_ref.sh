#!/usr/bin/env bash
# TEST INFRASTRUCTURE ONLY.  Builds the UNMODIFIED reference SM100 ops (MXFP8 grouped quant and
# MXFP8 block-scaled grouped GEMM) from the sources where they lie, into oracle/_ref/ (git-ignored).
# The result is used only as an on-GPU checker / comparison baseline in single-GPU runs.
#
# usage: oracle/build_ref.sh <path-to-reference-checkout>
# Needs: nvcc 12.9, the CUTLASS 4.x header tree bundled with flashinfer, torch headers.
set -euo pipefail
REF=${1:?usage: oracle/build_ref.sh <path-to-reference-checkout>}
HERE=$(cd "$(dirname "$0")" && pwd)
OUT=$HERE/_ref
mkdir -p "$OUT"
PY=${PYTHON:-python}
SP=$($PY -c 'import sysconfig; print(sysconfig.get_paths()["purelib"])')
PYINC=$($PY -c 'import sysconfig; print(sysconfig.get_paths()["include"])')
CUT=$SP/flashinfer/data/cutlass
TI=$SP/torch/include
TL=$SP/torch/lib
INC="-I$CUT/include -I$CUT/tools/util/include -I$TI -I$TI/torch/csrc/api/include -I$PYINC -I/usr/include/python3.12 -I/usr/local/cuda/include"
NVFLAGS="-O3 -DNDEBUG -Xcompiler -fPIC -std=c++17 --generate-code=arch=compute_100a,code=[sm_100a] \
 -DCUTLASS_ENABLE_TENSOR_CORE_MMA=1 -DCUTLASS_ENABLE_GDC_FOR_SM100=1 -DCUTLASS_DEBUG_TRACE_LEVEL=0 \
 --expt-relaxed-constexpr --expt-extended-lambda -D_GLIBCXX_USE_CXX11_ABI=1 --threads 2"
SRC=$REF/expert_specialization/csrc
( nvcc -c $SRC/cuda/es_sm100_mxfp8_blockscaled_group_quant.cu -o $OUT/ref_quant.o $INC $NVFLAGS ) &
P1=$!
( nvcc -c $SRC/cuda/es_sm100_mxfp8_blockscaled.cu -o $OUT/ref_gemm.o $INC $NVFLAGS ) &
P2=$!
g++ -c $SRC/expert_specialization.cpp -o $OUT/ref_registry.o $INC -O2 -fPIC -std=c++17 -D_GLIBCXX_USE_CXX11_ABI=1
g++ -c $HERE/ref_sm90_stub.cpp -o $OUT/ref_sm90_stub.o $INC -O2 -fPIC -std=c++17 -D_GLIBCXX_USE_CXX11_ABI=1
wait $P1; wait $P2
g++ -shared -o $OUT/libes_reference.so $OUT/ref_quant.o $OUT/ref_gemm.o $OUT/ref_registry.o $OUT/ref_sm90_stub.o \
  -L$TL -L/usr/local/cuda/lib64 -Wl,-rpath,$TL -ltorch -ltorch_cpu -ltorch_cuda -lc10 -lc10_cuda -lcudart
rm -f $OUT/*.o
echo "built $OUT/libes_reference.so"
