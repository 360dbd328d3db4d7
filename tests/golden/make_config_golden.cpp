// Parses tiny config.json files with the reference project's own ConfigLoader (src/core/config.cpp)
// and writes what it read to a JSON file: the anchor of tests/test_config_vs_reference.py.
// Built and run by make_config_golden.sh; needs the reference checkout and nlohmann/json.hpp.
#include "blackwell/config.h"
#include <nlohmann/json.hpp>
#include <fstream>
#include <iostream>

int main(int argc, char** argv) {
    if (argc < 3) { std::cerr << "usage: make_config_golden <cases.json> <out.json>\n"; return 2; }
    std::ifstream in(argv[1]);
    nlohmann::json cases = nlohmann::json::parse(in), out = nlohmann::json::array();
    for (auto& c : cases) {
        const std::string path = "config_case.json";   // in the working directory: error texts quote it
        { std::ofstream f(path); f << c["config"].dump(); }
        nlohmann::json r;
        r["name"] = c["name"];
        r["config"] = c["config"];
        try {
            const ModelConfig m = ConfigLoader::load_from_json(path);
            r["parsed"] = {
                {"hidden_dim", m.hidden_dim}, {"intermediate_dim", m.intermediate_dim}, {"num_layers", m.num_layers},
                {"num_attention_heads", m.num_attention_heads}, {"num_key_value_heads", m.num_key_value_heads},
                {"vocab_size", m.vocab_size}, {"head_dim", m.head_dim}, {"rotary_dim", m.rotary_dim},
                {"max_position_embeddings", m.max_position_embeddings}, {"rope_theta", m.rope_theta},
                {"rms_norm_eps", m.rms_norm_eps}, {"rope_scaling_type", m.rope_scaling_type},
                {"rope_scaling_factor", m.rope_scaling_factor}, {"rope_low_freq_factor", m.rope_low_freq_factor},
                {"rope_high_freq_factor", m.rope_high_freq_factor}, {"rope_orig_max_pos", m.rope_orig_max_pos},
                {"has_qkv_bias", m.has_qkv_bias}, {"tie_word_embeddings", m.tie_word_embeddings}};
        } catch (const std::exception& e) {
            r["error"] = e.what();
        }
        out.push_back(r);
        std::remove(path.c_str());
    }
    std::ofstream f(argv[2]);
    f << out.dump(1) << "\n";
    return 0;
}
