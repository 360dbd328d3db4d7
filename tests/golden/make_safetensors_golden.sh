#!/bin/sh
# Rebuilds tests/golden/reference_safetensors.json: checkpoints written by THIS package's writer
# (tests/golden/write_safetensors_cases.py: one file, and an index with two shards), read by the
# reference project's own loader (src/core/safetensors.cpp).
# Usage: tests/golden/make_safetensors_golden.sh /path/to/BlackwellLLM /include/dir/holding/nlohmann
set -e
REF="${1:?path of the fxslava/BlackwellLLM checkout}"
JSON_INC="${2:?include directory that holds nlohmann/json.hpp}"
HERE="$(cd "$(dirname "$0")" && pwd)"
TMP="${TMPDIR:-/tmp}/safetensors_golden"
rm -rf "$TMP"; mkdir -p "$TMP"
python "$HERE/write_safetensors_cases.py" "$TMP"
g++ -std=c++20 -O1 -I"$REF/src/core" -I"$REF/include" -I"$JSON_INC" "$HERE/make_safetensors_golden.cpp" \
    "$REF/src/core/safetensors.cpp" -o "$TMP/make_safetensors_golden"
"$TMP/make_safetensors_golden" "$HERE/reference_safetensors.json" "$TMP/single/model.safetensors" \
    "$TMP/sharded/model.safetensors.index.json"
echo "wrote $HERE/reference_safetensors.json"
