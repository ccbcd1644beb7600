#!/usr/bin/env bash
# Builds the parts of the reference that compile for sm_100a without modification, from the sources where they lie
# (the checkout named by $REF; a built-in default otherwise), into oracle/_ref/ (git-ignored):
#   libflagrot_w3ref.so    kernels/csrc/attn_cb_write3.cu + integrations/vllm_flagrot/csrc/flagrot_capi.cu
#                          (+ ref_link_stubs.cu for the symbols of the wgmma translation units)
#   libflagrot_kivi_ref.so integrations/vllm_flagrot/csrc/kivi.cu
#   pyref/*.bytecode       byte code of the reference's three ctypes front ends (kernels.py, kivi.py, prefill_mq.py),
#                          compiled by py_compile from the sources where they lie and loaded by oracle/pyref.py: the
#                          boundary test loads this repository's libraries through them, and bench.py --impl reference
#                          times their PyTorch page parser + fp32 attention on the host cores
# They are byte-for-byte GPU checkers for the writers / the KIVI library and the kernels to beat.  Test infrastructure:
# the shipped libraries never load them.  Skips quietly when the reference tree is absent (the GPU box uses the
# prebuilt files).
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REF="${REF:-${FLAGROT_REFERENCE:-$HERE/../../reference}}"      # default: a checkout named "reference" beside this repository
OUT="$HERE/_ref"
[ -d "$REF/kernels/csrc" ] || { echo "reference tree not found at $REF: keeping prebuilt oracle/_ref"; exit 0; }
mkdir -p "$OUT"
NVCC="${NVCC:-/usr/local/cuda/bin/nvcc}"
ARCH=(-gencode arch=compute_100a,code=sm_100a)
FLAGS=(-O3 -std=c++17 "${ARCH[@]}" --expt-relaxed-constexpr -lineinfo -Xcompiler -fPIC -I"$REF/kernels/csrc")
newer() { [ ! -e "$1" ] || [ -n "$(find "${@:2}" -newer "$1" -print -quit)" ]; }
if newer "$OUT/libflagrot_w3ref.so" "$REF/kernels/csrc" "$REF/integrations/vllm_flagrot/csrc/flagrot_capi.cu" "$HERE/ref_link_stubs.cu"; then
  TMP="$(mktemp -d)"
  "$NVCC" "${FLAGS[@]}" -c "$REF/kernels/csrc/attn_cb_write3.cu" -o "$TMP/w3.o" &
  "$NVCC" "${FLAGS[@]}" -c "$REF/integrations/vllm_flagrot/csrc/flagrot_capi.cu" -o "$TMP/capi.o" &
  "$NVCC" "${FLAGS[@]}" -c "$HERE/ref_link_stubs.cu" -o "$TMP/stubs.o" &
  wait
  "$NVCC" -shared "${ARCH[@]}" -cudart static -o "$OUT/libflagrot_w3ref.so" "$TMP/w3.o" "$TMP/capi.o" "$TMP/stubs.o"
  rm -rf "$TMP"
fi
if newer "$OUT/libflagrot_kivi_ref.so" "$REF/integrations/vllm_flagrot/csrc/kivi.cu"; then
  TMP="$(mktemp -d)"
  "$NVCC" "${FLAGS[@]}" -c "$REF/integrations/vllm_flagrot/csrc/kivi.cu" -o "$TMP/kivi.o"
  "$NVCC" -shared "${ARCH[@]}" -cudart static -o "$OUT/libflagrot_kivi_ref.so" "$TMP/kivi.o"
  rm -rf "$TMP"
fi
PYREF="$OUT/pyref"
PYSRC="$REF/integrations/vllm_flagrot/vllm_flagrot"
if newer "$PYREF/kernels.bytecode" "$PYSRC/kernels.py" "$PYSRC/kivi.py" "$PYSRC/prefill_mq.py"; then
  mkdir -p "$PYREF"
  for m in kernels kivi prefill_mq; do
    python -c "import py_compile, sys; py_compile.compile(sys.argv[1], cfile=sys.argv[2], dfile='vllm_flagrot/' + sys.argv[3] + '.py', doraise=True)" \
      "$PYSRC/$m.py" "$PYREF/$m.bytecode" "$m"
  done
fi
ls -la "$OUT" "$PYREF"
