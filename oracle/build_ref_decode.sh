#!/usr/bin/env bash
# Compiles the reference's CUDA decoder (kernel/decode_huffman.cu, unmodified) for sm_100a from the
# reference tree where it lies, plus the one-function binding in ref_recipe/, into
# oracle/_ref/mpserve_ref_decode.so.  Outputs go only to oracle/_ref/ (git-ignored).
# usage: oracle/build_ref_decode.sh [/path/to/reference]   (default: $MPSERVE_REFERENCE_ROOT, else ../reference
#        beside this repository)
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REF="${1:-${MPSERVE_REFERENCE_ROOT:-$HERE/../../reference}}"
OUT="$HERE/_ref"
[ -f "$REF/kernel/decode_huffman.cu" ] || { echo "reference sources not found under $REF" >&2; exit 3; }
mkdir -p "$OUT"
PY=python
NVCC="${NVCC:-$(command -v nvcc || echo /usr/local/cuda/bin/nvcc)}"
TORCH_INC=$($PY -c "import torch.utils.cpp_extension as c, sys; sys.stdout.write(' '.join('-I'+p for p in c.include_paths()))" 2>/dev/null)
TORCH_LIB=$($PY -c "import torch, os, sys; sys.stdout.write(os.path.join(os.path.dirname(torch.__file__), 'lib'))")
PY_INC=$($PY -c "import sysconfig, sys; sys.stdout.write(sysconfig.get_paths()['include'])")
EXT=$($PY -c "import sysconfig, sys; sys.stdout.write(sysconfig.get_config_var('EXT_SUFFIX'))")
unset CC CXX
"$NVCC" -O3 -std=c++17 -gencode arch=compute_100a,code=sm_100a -lineinfo -Xptxas -v \
    -Xcompiler -fPIC -w --expt-relaxed-constexpr \
    -DTORCH_EXTENSION_NAME=mpserve_ref_decode -DTORCH_API_INCLUDE_EXTENSION_H \
    $TORCH_INC -I"$PY_INC" \
    -c "$REF/kernel/decode_huffman.cu" -o "$OUT/ref_decode_huffman.o" 2> "$OUT/ref_decode_ptxas.log"
g++ -O2 -std=c++17 -fPIC -w \
    -DTORCH_EXTENSION_NAME=mpserve_ref_decode -DTORCH_API_INCLUDE_EXTENSION_H \
    $TORCH_INC -I"$PY_INC" -I/usr/local/cuda/include \
    -c "$HERE/ref_recipe/ref_decode_binding.cpp" -o "$OUT/ref_decode_binding.o"
g++ -shared "$OUT/ref_decode_huffman.o" "$OUT/ref_decode_binding.o" \
    -L"$TORCH_LIB" -Wl,-rpath,"$TORCH_LIB" -ltorch -ltorch_cpu -ltorch_cuda -lc10 -lc10_cuda -ltorch_python \
    -L/usr/local/cuda/lib64 -lcudart \
    -o "$OUT/mpserve_ref_decode$EXT"
rm -f "$OUT/ref_decode_huffman.o" "$OUT/ref_decode_binding.o"
echo "built $OUT/mpserve_ref_decode$EXT"
