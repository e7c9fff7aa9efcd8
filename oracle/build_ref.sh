#!/usr/bin/env bash
# Compiles the reference's CPU encoder (kernel/build_huffman.cu, host-only C++ despite its suffix)
# from the reference tree where it lies, plus the small binding in ref_recipe/, into
# oracle/_ref/mpserve_ref_build.so.  Outputs go only to oracle/_ref/ (git-ignored).
# usage: oracle/build_ref.sh [/path/to/reference]   (default: $MPSERVE_REFERENCE_ROOT, else ../reference
#        beside this repository)
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REF="${1:-${MPSERVE_REFERENCE_ROOT:-$HERE/../../reference}}"
OUT="$HERE/_ref"
[ -f "$REF/kernel/build_huffman.cu" ] || { echo "reference sources not found under $REF" >&2; exit 3; }
mkdir -p "$OUT"
PY=python
TORCH_INC=$($PY -c "import torch.utils.cpp_extension as c, sys; sys.stdout.write(' '.join('-I'+p for p in c.include_paths()))" 2>/dev/null)
TORCH_LIB=$($PY -c "import torch, os, sys; sys.stdout.write(os.path.join(os.path.dirname(torch.__file__), 'lib'))")
PY_INC=$($PY -c "import sysconfig, sys; sys.stdout.write(sysconfig.get_paths()['include'])")
EXT=$($PY -c "import sysconfig, sys; sys.stdout.write(sysconfig.get_config_var('EXT_SUFFIX'))")
g++ -O2 -std=c++17 -fPIC -shared -w \
    -DTORCH_EXTENSION_NAME=mpserve_ref_build -DTORCH_API_INCLUDE_EXTENSION_H \
    -include "$HERE/ref_recipe/gxx_shim.h" \
    $TORCH_INC -I"$PY_INC" -I/usr/local/cuda/include \
    -x c++ "$REF/kernel/build_huffman.cu" "$HERE/ref_recipe/ref_binding.cpp" \
    -L"$TORCH_LIB" -Wl,-rpath,"$TORCH_LIB" -ltorch -ltorch_cpu -lc10 -ltorch_python \
    -o "$OUT/mpserve_ref_build$EXT"
echo "built $OUT/mpserve_ref_build$EXT"
