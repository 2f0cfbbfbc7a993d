#!/usr/bin/env bash
# Builds the reference's own CUDA extension (intra_attn_cuda) for sm_100 from the sources where
# they lie in the reference checkout, into oracle/_ref/ (git-ignored; nothing is copied into
# this repository).  It is the "existing Blackwell-loadable kernel" that bench_kernel.py's
# --ref-ext option times beside this library on the same GPU: a measured baseline, never part
# of the product path.
#
# The recipe restates the reference's setup.py (sources setup.py:38-47, flags setup.py:50-63,
# sm_100 gencode setup.py:31-32) as plain compiler calls; the reference's own build system is
# not run.  Its un-vendored CUTLASS submodule (csrc/cutlass, empty in the checkout) is replaced
# by the CUTLASS/CuTe header tree that ships inside the flashinfer wheel of this image.
#
# usage: oracle/build_ref_ext.sh [REFERENCE_DIR]      (default: where the build container keeps the reference checkout)
set -euo pipefail
REF="${1:-/root/reference}"
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
OUT="$HERE/_ref"
SRC="$REF/csrc/flash_attn/src"
[ -f "$REF/csrc/flash_attn/flash_api.cpp" ] || { echo "no reference checkout at $REF" >&2; exit 3; }
mkdir -p "$OUT/obj"

PY=python
SITE="$($PY -c 'import sysconfig; print(sysconfig.get_paths()["purelib"])')"
PYINC="$($PY -c 'import sysconfig; print(sysconfig.get_paths()["include"])')"
EXT_SUFFIX="$($PY -c 'import sysconfig; print(sysconfig.get_config_var("EXT_SUFFIX"))')"
CUTLASS="$SITE/flashinfer/data/cutlass/include"
[ -d "$CUTLASS/cute" ] || { echo "no CUTLASS headers at $CUTLASS" >&2; exit 4; }
TORCH="$SITE/torch"
CUDA="${CUDA_HOME:-/usr/local/cuda}"

INC=(-I"$REF/csrc/flash_attn" -I"$SRC" -I"$CUTLASS"
     -I"$TORCH/include" -I"$TORCH/include/torch/csrc/api/include" -I"$PYINC" -I"$CUDA/include")
DEFS=(-DTORCH_EXTENSION_NAME=intra_attn_cuda -DTORCH_API_INCLUDE_EXTENSION_H
      -D_GLIBCXX_USE_CXX11_ABI=1)
NVCC_FLAGS=(-O3 -std=c++17
    -U__CUDA_NO_HALF_OPERATORS__ -U__CUDA_NO_HALF_CONVERSIONS__
    -U__CUDA_NO_HALF2_OPERATORS__ -U__CUDA_NO_BFLOAT16_CONVERSIONS__
    --expt-relaxed-constexpr --expt-extended-lambda --use_fast_math
    -gencode arch=compute_100,code=sm_100
    -Xcompiler -fPIC -w)

KERNELS=(
    flash_fwd_hdim128_bf16_sm80_mask0_8group_text_front
    flash_fwd_hdim128_bf16_sm80_masksw_text_front
    flash_fwd_hdim128_bf16_sm80_mask0_16groups_llm_causal
    flash_fwd_hdim128_bf16_sm80_mask1_16groups_llm_causal
    flash_fwd_hdim128_bf16_sm80_masksw_llm_causal
)

pids=()
for k in "${KERNELS[@]}"; do
    "$CUDA/bin/nvcc" "${NVCC_FLAGS[@]}" "${DEFS[@]}" "${INC[@]}" \
        -c "$SRC/$k.cu" -o "$OUT/obj/$k.o" > "$OUT/obj/$k.log" 2>&1 &
    pids+=($!)
done
g++ -O3 -std=c++17 -fPIC -w "${DEFS[@]}" "${INC[@]}" \
    -c "$REF/csrc/flash_attn/flash_api.cpp" -o "$OUT/obj/flash_api.o" > "$OUT/obj/flash_api.log" 2>&1 &
pids+=($!)
fail=0
for p in "${pids[@]}"; do wait "$p" || fail=1; done
if [ "$fail" != 0 ]; then
    echo "reference extension: a translation unit failed to compile; logs in $OUT/obj/*.log" >&2
    tail -n 20 "$OUT"/obj/*.log >&2
    exit 5
fi

OBJS=("$OUT/obj/flash_api.o")
for k in "${KERNELS[@]}"; do OBJS+=("$OUT/obj/$k.o"); done
g++ -shared -o "$OUT/intra_attn_cuda$EXT_SUFFIX" "${OBJS[@]}" \
    -L"$TORCH/lib" -lc10 -ltorch -ltorch_cpu -ltorch_python -lc10_cuda -ltorch_cuda \
    -L"$CUDA/lib64" -lcudart -Wl,-rpath,"$TORCH/lib"
echo "built $OUT/intra_attn_cuda$EXT_SUFFIX"
