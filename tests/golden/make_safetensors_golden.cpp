// Reads checkpoints with the reference project's own SafetensorsLoader (src/core/safetensors.cpp) and
// writes what it found (name, dtype, shape, byte size, absolute file offset, shard) to a JSON file:
// the anchor of tests/test_safetensors_vs_reference.py.  Built and run by make_safetensors_golden.sh.
#include "safetensors.h"
#include <nlohmann/json.hpp>
#include <algorithm>
#include <fstream>
#include <iostream>

int main(int argc, char** argv) {
    if (argc < 3) { std::cerr << "usage: make_safetensors_golden <out.json> <file-or-index>...\n"; return 2; }
    nlohmann::json out = nlohmann::json::object();
    for (int i = 2; i < argc; ++i) {
        const std::string path = argv[i];
        const std::string key = path.substr(path.find_last_of('/') + 1);
        SafetensorsLoader loader(path);
        std::vector<std::string> names = loader.list_tensors();
        std::sort(names.begin(), names.end());
        nlohmann::json arr = nlohmann::json::array();
        for (const auto& n : names) {
            const TensorEntry& e = loader.get_tensor(n);
            const std::string shard = e.file_path.substr(e.file_path.find_last_of("/\\") + 1);
            arr.push_back({{"name", e.name}, {"dtype", e.dtype}, {"shape", e.shape}, {"byte_size", e.byte_size},
                           {"file_offset", e.file_offset}, {"shard", shard}});
        }
        out[key] = arr;
    }
    std::ofstream f(argv[1]);
    f << out.dump(1) << "\n";
    return 0;
}
