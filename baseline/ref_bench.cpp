// Driver of bench.py's reference arm.  It contains no model code: it constructs the reference's
// BlackwellEngine from a checkpoint folder and times the reference's own public calls
// (include/blackwell/engine.h): prefill_status for the prompt, fork to make the batch's sequences, and
// forward_batch for the decode steps.  All numbers are host wall clock around calls that return only
// when their result is on the host (each call ends with a device-to-host read of its tokens).
//
//   ref_bench INDEX_OR_SAFETENSORS BATCH CONTEXT STEPS WARMUP PREFILL_TOKENS VOCAB [SHARED]
//
// SHARED: how many leading tokens the sequences of the batch have in common (their pages are shared
// copy-on-write by fork, the reference's way to make a batch); default 16, one page.
//
// Prints one line: prefill_ms=<..> decode_ms_per_step=<..> fill_s=<..> status=ok   (or status=<what failed>)
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "blackwell/engine.h"
#include "blackwell/runtime_config.h"

static double now_ms() {
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

int main(int argc, char** argv) {
    if (argc < 8) { std::fprintf(stderr, "usage: ref_bench PATH BATCH CONTEXT STEPS WARMUP PREFILL VOCAB\n"); return 2; }
    const std::string path = argv[1];
    const int B = std::atoi(argv[2]), C = std::atoi(argv[3]), steps = std::atoi(argv[4]), warm = std::atoi(argv[5]);
    const int P = std::atoi(argv[6]), V = std::atoi(argv[7]);
    // tokens that the forked sequences have in common (default: one page); the rest is each one's own
    const int shared = argc > 8 ? std::atoi(argv[8]) : 16;
    if (shared < 1 || shared > C - 1) { std::fprintf(stderr, "SHARED must be in [1, CONTEXT - 1]\n"); return 2; }
    try {
        blackwell::InferenceConfig req;
        req.max_context_length = (size_t)C + warm + steps + 64;
        req.max_batch_size = (size_t)B;
        req.require_branching = true;   // the paged cache; forward_batch needs it
        blackwell::RuntimeOverrides ov;
        ov.kv_mode = BlackwellEngine::KVCacheMode::Paged;
        const int blocks = (int)((req.max_context_length + 15) / 16);
        ov.kv_vram_cache_pages = B * (blocks + 2) + 64;   // every sequence's own pages stay on the device
        ov.kv_ram_slots = 0;                              // no host demotion tier
        BlackwellEngine eng(path, req, ov);

        unsigned long long s = 88172645463325252ull;
        auto rnd = [&]() { s ^= s << 13; s ^= s >> 7; s ^= s << 17; return (int)(s % (unsigned long long)V); };
        int next = 0;
        // ---- prefill of P tokens, one sequence (best of 2 after one untimed run)
        std::vector<int> prompt(P);
        for (auto& t : prompt) t = rnd();
        double prefill_ms = 1e30;
        for (int it = 0; it < 3; ++it) {
            eng.rewind(0, 0);
            cudaDeviceSynchronize();
            const double t0 = now_ms();
            if (eng.prefill_status(prompt.data(), P, 0, 0.0f, 1.0f, 0, &next) != blackwell::EngineStatus::Success) {
                std::printf("status=prefill_failed\n"); return 0; }
            cudaDeviceSynchronize();
            if (it > 0 && now_ms() - t0 < prefill_ms) prefill_ms = now_ms() - t0;
        }
        // ---- B sequences of C - 1 tokens: a shared first page, then each its own tokens
        const double f0 = now_ms();
        eng.rewind(0, 0);
        std::vector<int> common(shared);
        for (auto& t : common) t = rnd();
        if (eng.prefill_status(common.data(), shared, 0, 0.0f, 1.0f, 0, &next) != blackwell::EngineStatus::Success) {
            std::printf("status=fill_failed_shared\n"); return 0; }
        for (int b = 1; b < B; ++b) eng.fork(0, b);
        std::vector<int> own(C - 1 - shared);
        for (int b = 0; b < B && !own.empty(); ++b) {
            for (auto& t : own) t = rnd();
            std::fprintf(stderr, "[ref_bench] filling sequence %d of %d (%.1f s so far)\n", b + 1, B, (now_ms() - f0) / 1e3);
            if (eng.prefill_status(own.data(), (int)own.size(), shared, 0.0f, 1.0f, b, &next) != blackwell::EngineStatus::Success) {
                std::printf("status=fill_failed_seq_%d\n", b); return 0; }
        }
        const double fill_s = (now_ms() - f0) / 1e3;
        // ---- decode: one token each, greedy, the sampled token fed back
        std::vector<blackwell::DecodeRequest> reqs(B);
        for (int b = 0; b < B; ++b) reqs[b] = {b, rnd(), C - 1};
        auto step = [&]() {
            auto res = eng.forward_batch(reqs);
            for (int b = 0; b < B; ++b) { reqs[b].token_id = res[b].next_token_id; reqs[b].pos += 1; }
        };
        for (int i = 0; i < warm; ++i) step();
        cudaDeviceSynchronize();
        const double t0 = now_ms();
        for (int i = 0; i < steps; ++i) step();
        cudaDeviceSynchronize();
        const double ms = (now_ms() - t0) / steps;
        std::printf("prefill_ms=%.4f decode_ms_per_step=%.4f fill_s=%.2f status=ok\n", prefill_ms, ms, fill_s);
    } catch (const std::exception& e) {
        std::string w = e.what();
        for (auto& ch : w) if (ch == '\n' || ch == ' ') ch = '_';
        std::printf("status=exception:%s\n", w.c_str());
    }
    return 0;
}
