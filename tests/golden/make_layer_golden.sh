#!/bin/sh
# Rebuilds tests/golden/reference_rope_scaling.json (the reference's llama3 frequency rescaling) and
# tests/golden/reference_layer.json (one whole tiny decoder composed of the reference's CPU kernels).
# Usage: tests/golden/make_layer_golden.sh /path/to/BlackwellLLM   (needs g++ and the CUDA headers)
set -e
REF="${1:?path of the fxslava/BlackwellLLM checkout}"
HERE="$(cd "$(dirname "$0")" && pwd)"
CUDA_INC="${CUDA_HOME:-/usr/local/cuda}/include"
TMP="${TMPDIR:-/tmp}"
g++ -std=c++17 -O1 -I"$REF/src/kernels" "$HERE/make_rope_scaling_golden.cpp" -o "$TMP/make_rope_scaling_golden"
"$TMP/make_rope_scaling_golden" "$HERE/reference_rope_scaling.json"
g++ -std=c++17 -O1 -I"$REF/tests/common" -I"$CUDA_INC" "$HERE/make_layer_golden.cpp" -o "$TMP/make_layer_golden"
"$TMP/make_layer_golden" "$HERE/reference_layer.json"
echo "wrote $HERE/reference_rope_scaling.json and $HERE/reference_layer.json"
