#!/usr/bin/env bash
# Builds the reference-derived checkers into oracle/_ref/ (git-ignored).  TEST INFRASTRUCTURE ONLY.
#
#   libref_cpu.so        the reference's hysteresis and activation-quantisation kernel sources
#                        (kernels/int2/int2_hysteresis_v2.cu, int2_activation_quant.cu,
#                        int2_packed.cuh), compiled for the host with g++ against the stand-in
#                        headers in oracle/shim/.  The sources are streamed from where they lie,
#                        cut before their host-launch sections (which use <<< >>>), and followed by
#                        oracle/ref_cpu_driver.inc; nothing is copied into this repository.
#   int2_tc_ops_ref.so   (--cuda) the reference's nine extension sources compiled for sm_100a with
#                        its own flags (-O3 --use_fast_math), as a torch extension module that the
#                        GPU tests load to compare kernels on the same device.
#
# usage: oracle/build_ref.sh [--cuda] REFERENCE_ROOT      (or REFERENCE_ROOT in the environment)
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
WITH_CUDA=0
if [[ "${1:-}" == "--cuda" ]]; then WITH_CUDA=1; shift; fi
REF="${1:-${REFERENCE_ROOT:-}}"
[[ -n "$REF" ]] || { echo "usage: $0 [--cuda] REFERENCE_ROOT (the checkout of the reference project)" >&2; exit 2; }
SRC="$REF/kernels/int2"
OUT="$HERE/_ref"
[[ -d "$SRC" ]] || { echo "reference sources not found at $SRC" >&2; exit 3; }
mkdir -p "$OUT"

cut_before() { awk -v pat="$2" 'index($0, pat) { exit } { print }' "$1"; }

{
  cut_before "$SRC/int2_hysteresis_v2.cu" "// Host Interface"
  echo "#undef BLOCK_SIZE"
  cut_before "$SRC/int2_activation_quant.cu" "// C++ Interface Functions"
  echo "#define REF_WITH_QUANT 1"
  cat "$HERE/ref_cpu_driver.inc"
} | g++ -O2 -std=c++17 -fno-fast-math -ffp-contract=off -shared -fPIC -x c++ \
        -I "$HERE/shim" -I "$SRC" - -o "$OUT/libref_cpu.so"
echo "built $OUT/libref_cpu.so"

if [[ $WITH_CUDA == 1 ]]; then
  PY="${PYTHON:-python}"
  TORCH_INC=$($PY - <<'PYEOF'
import torch.utils.cpp_extension as c, sysconfig
print(" ".join("-I" + p for p in c.include_paths() + [sysconfig.get_paths()["include"]]))
PYEOF
)
  TORCH_LIB=$($PY -c "import torch, os; print(os.path.join(os.path.dirname(torch.__file__), 'lib'))")
  OBJ="$OUT/obj"; mkdir -p "$OBJ"
  COMMON="-O3 -std=c++17 -DTORCH_EXTENSION_NAME=int2_tc_ops_ref -DTORCH_API_INCLUDE_EXTENSION_H -D_GLIBCXX_USE_CXX11_ABI=1 $TORCH_INC"
  pids=()
  for f in int2_matmul_tc int2_matmul_int8_tc_v2 int2_backward_tc int2_backward_int8_tc_v2 \
           int2_hysteresis_tc int2_hysteresis_v2 int2_activation_quant int2_unpack; do
    nvcc $COMMON --use_fast_math -gencode arch=compute_100a,code=sm_100a -Xcompiler -fPIC \
         -c "$SRC/$f.cu" -o "$OBJ/$f.o" &
    pids+=($!)
  done
  g++ $COMMON -fPIC -I/usr/local/cuda/include -c "$SRC/int2_tc_ops.cpp" -o "$OBJ/int2_tc_ops.o" &
  pids+=($!)
  for p in "${pids[@]}"; do wait "$p"; done
  g++ -shared "$OBJ"/*.o -L"$TORCH_LIB" -L/usr/local/cuda/lib64 -lc10 -lc10_cuda -ltorch_cpu -ltorch_cuda \
      -ltorch -ltorch_python -lcudart -Wl,-rpath,"$TORCH_LIB" -o "$OUT/int2_tc_ops_ref.so"
  rm -rf "$OBJ"
  echo "built $OUT/int2_tc_ops_ref.so"
fi
