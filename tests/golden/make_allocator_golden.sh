#!/bin/sh
# Rebuilds tests/golden/reference_allocator.json: the reference project's own page allocator
# (src/core/paging/paged_kv_cache.h) under a seeded random sequence of operations.
# Usage: tests/golden/make_allocator_golden.sh /path/to/BlackwellLLM [/path/to/cuda/include]
set -e
REF="${1:?path of the fxslava/BlackwellLLM checkout}"
CUDA_INC="${2:-/usr/local/cuda/include}"
HERE="$(cd "$(dirname "$0")" && pwd)"
g++ -std=c++20 -O1 -I"$REF/src" -I"$REF/src/core" -I"$REF/include" -I"$CUDA_INC" "$HERE/make_allocator_golden.cpp" \
    -o "${TMPDIR:-/tmp}/make_allocator_golden"
"${TMPDIR:-/tmp}/make_allocator_golden" "$HERE/reference_allocator.json"
echo "wrote $HERE/reference_allocator.json"
