#!/bin/sh
# Rebuilds tests/golden/reference_cpu.json from the reference project's CPU kernels.
# Usage: tests/golden/make_golden.sh /path/to/BlackwellLLM   (needs g++ and the CUDA headers)
set -e
REF="${1:?path of the fxslava/BlackwellLLM checkout}"
HERE="$(cd "$(dirname "$0")" && pwd)"
CUDA_INC="${CUDA_HOME:-/usr/local/cuda}/include"
g++ -std=c++17 -O1 -I"$REF/tests/common" -I"$CUDA_INC" "$HERE/make_golden.cpp" -o "${TMPDIR:-/tmp}/make_golden"
"${TMPDIR:-/tmp}/make_golden" "$HERE/reference_cpu.json"
echo "wrote $HERE/reference_cpu.json"
