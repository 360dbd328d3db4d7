#!/bin/sh
# Rebuilds tests/golden/reference_config.json: the reference project's own config loader
# (src/core/config.cpp) run on tests/golden/config_cases.json.
# Usage: tests/golden/make_config_golden.sh /path/to/BlackwellLLM /path/to/dir/with/nlohmann/json.hpp's parent
set -e
REF="${1:?path of the fxslava/BlackwellLLM checkout}"
JSON_INC="${2:?include directory that holds nlohmann/json.hpp}"
HERE="$(cd "$(dirname "$0")" && pwd)"
g++ -std=c++20 -O1 -I"$REF/include" -I"$JSON_INC" "$HERE/make_config_golden.cpp" "$REF/src/core/config.cpp" \
    -o "${TMPDIR:-/tmp}/make_config_golden"
"${TMPDIR:-/tmp}/make_config_golden" "$HERE/config_cases.json" "$HERE/reference_config.json"
echo "wrote $HERE/reference_config.json"
