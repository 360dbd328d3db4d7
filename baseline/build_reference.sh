#!/bin/sh
# Builds the reference arm of bench.py: the UNMODIFIED sources of fxslava/BlackwellLLM's dense core
# (src/core, src/kernels; without its COM boundary engine_com.cpp and the DirectStorage loader, which are
# Windows-only and not on the generation path), compiled for sm_100a on Linux, plus the small driver
# baseline/ref_bench.cpp, which calls the reference's public C++ API (BlackwellEngine::prefill_status,
# fork, forward_batch).  Output: baseline/_ref/ref_bench (git-ignored).
#
#   baseline/build_reference.sh /path/to/BlackwellLLM
#
# Needs nvcc, g++ and a copy of nlohmann/json.hpp (the reference fetches it with CMake; here the copy that
# ships inside the installed cudnn_frontend Python package is used, or $NLOHMANN_INCLUDE).
set -e
REF="${1:?path of the fxslava/BlackwellLLM checkout}"
HERE="$(cd "$(dirname "$0")" && pwd)"
OUT="$HERE/_ref"
OBJ="$OUT/obj"
mkdir -p "$OBJ"
NVCC="${CUDA_HOME:-/usr/local/cuda}/bin/nvcc"
CUDA_INC="${CUDA_HOME:-/usr/local/cuda}/include"
JSON_INC="${NLOHMANN_INCLUDE:-$(python3 -c 'import glob, sysconfig; c = glob.glob(sysconfig.get_paths()["purelib"] + "/include/cudnn_frontend/thirdparty/nlohmann/json.hpp"); print(c[0].rsplit("/nlohmann/", 1)[0] if c else "")' 2>/dev/null || true)}"
[ -f "$JSON_INC/nlohmann/json.hpp" ] || { echo "nlohmann/json.hpp not found (set NLOHMANN_INCLUDE)"; exit 1; }
ARCH="-gencode arch=compute_100a,code=sm_100a"
for f in "$REF"/src/kernels/*.cu; do
    b="$(basename "$f" .cu)"
    # --use_fast_math: the reference's own flag for its CUDA files (its root CMakeLists.txt)
    "$NVCC" $ARCH -std=c++20 --use_fast_math -O3 -Xcompiler -fPIC -I"$REF/src" -c "$f" -o "$OBJ/k_$b.o" &
done
wait
CORE="engine.cpp engine_prefill_coordinator.cpp hybrid_snapshot_ring.cpp runtime_config.cpp ops_dispatcher.cpp
safetensors.cpp memory_pool.cpp kv_cache/continuous_kv_manager.cpp kv_cache/paged_kv_manager.cpp tokenizer/unicode.cpp
tokenizer/bpe_tokenizer.cpp tokenizer/tiktoken_tokenizer.cpp tokenizer/chat_template.cpp tokenizer/tokenizer_factory.cpp
weight_loader.cpp config.cpp"
for f in $CORE; do
    b="$(echo "$f" | tr '/' '_' | sed 's/\.cpp$//')"
    g++ -std=c++20 -O2 -fPIC -include "$HERE/linux_compat.h" -I"$REF/include" -I"$REF/src/core" -I"$REF/src" \
        -I"$JSON_INC" -I"$CUDA_INC" -c "$REF/src/core/$f" -o "$OBJ/c_$b.o" &
done
wait
g++ -std=c++20 -O2 -I"$REF/include" -I"$CUDA_INC" -c "$HERE/ref_bench.cpp" -o "$OBJ/ref_bench.o"
"$NVCC" $ARCH -o "$OUT/ref_bench" "$OBJ"/ref_bench.o "$OBJ"/c_*.o "$OBJ"/k_*.o -cudart static -lpthread -ldl
echo "built $OUT/ref_bench"
