// Driver that composes ONE whole tiny decoder (embedding, one layer, final norm, tied head) ONLY of
// the reference project's own CPU kernels (its header tests/common/cpu_reference.h, taken from the
// reference checkout by include path at build time; nothing of it is copied here), in the order of
// its engine's layer loop (src/core/engine.cpp:946-1041): norm, q/k/v products, bias added before
// the rotation, rotation + cache append, attention with grouped heads, output product added to the
// residual stream, norm, gate and up products, SwiGLU, down product added to the residual stream;
// then the final norm and the head (the embedding table: tied).  The products are plain loops
// (y = W x with W [out, in], src/kernels/bf16_linear.cu:13-54).  Six positions, token by token, as
// the reference decodes.  Writes weights, tokens and logits as JSON;
// tests/test_plain_vs_reference_cpu.py feeds the same weights to the plain implementation.
// Build and run: see make_layer_golden.sh.
#include "cpu_reference.h"
#include <cstdio>
#include <vector>

static unsigned long long lcg_state = 2024;
static float rnd() {
    lcg_state = (lcg_state * 6364136223846793005ULL + 1442695040888963407ULL);
    return (float)((lcg_state >> 40) & 0xFFFFFF) / 8388608.0f - 1.0f;   // [-1, 1)
}
static float bf(float v) { return cpu_bf16_round(v); }   // weights live on the bfloat16 grid, as in a checkpoint
typedef std::vector<float> Vec;
static Vec make(size_t n, float scale) { Vec v(n); for (auto& x : v) x = bf(scale * rnd()); return v; }
static void dump(FILE* f, const char* name, const Vec& v, bool last = false) {
    fprintf(f, "  \"%s\": [", name);
    for (size_t i = 0; i < v.size(); ++i) fprintf(f, "%s%.9g", i ? ", " : "", v[i]);
    fprintf(f, "]%s\n", last ? "" : ",");
}
// y (=|+=) W x (+ b), W [out, in] row-major
static void linear(const Vec& W, const float* x, float* y, size_t out, size_t in, const Vec* b, bool accumulate) {
    for (size_t o = 0; o < out; ++o) {
        float dot = 0.f;
        for (size_t i = 0; i < in; ++i) dot += W[o * in + i] * x[i];
        if (b) dot += (*b)[o];
        y[o] = accumulate ? y[o] + dot : dot;
    }
}
static std::vector<__nv_bfloat16> as_bf16(const Vec& v) {
    std::vector<__nv_bfloat16> o(v.size());
    for (size_t i = 0; i < v.size(); ++i) o[i] = __float2bfloat16(v[i]);
    return o;
}

int main(int argc, char** argv) {
    FILE* f = fopen(argc > 1 ? argv[1] : "reference_layer.json", "w");
    if (!f) return 1;
    const size_t H = 24, nh = 4, nkv = 2, hd = 8, I = 40, V = 30, T = 6, max_seq = 8;
    const float theta = 10000.0f, eps = 1e-5f;
    const int tokens[T] = {3, 29, 0, 17, 3, 8};
    Vec E = make(V * H, 1.0f), n1 = make(H, 0.25f), n2 = make(H, 0.25f), nf = make(H, 0.25f);
    for (auto& x : n1) x = bf(1.0f + x);
    for (auto& x : n2) x = bf(1.0f + x);
    for (auto& x : nf) x = bf(1.0f + x);
    Vec Wq = make(nh * hd * H, 0.3f), Wk = make(nkv * hd * H, 0.3f), Wv = make(nkv * hd * H, 0.3f);
    Vec bq = make(nh * hd, 0.5f), bk = make(nkv * hd, 0.5f), bv = make(nkv * hd, 0.5f);
    Vec Wo = make(H * nh * hd, 0.3f), Wg = make(I * H, 0.3f), Wu = make(I * H, 0.3f), Wd = make(H * I, 0.3f);
    auto n1b = as_bf16(n1), n2b = as_bf16(n2), nfb = as_bf16(nf);

    Vec Kc(nkv * max_seq * hd, 0.f), Vc(nkv * max_seq * hd, 0.f), logits;
    for (size_t pos = 0; pos < T; ++pos) {
        Vec x(H), xn(H), q(nh * hd), k(nkv * hd), v(nkv * hd), o(nh * hd), g(I), u(I), a(I), lg(V);
        cpu_embedding_lookup(&tokens[pos], E.data(), x.data(), 1, H);
        cpu_rmsnorm_direct(x.data(), xn.data(), n1b.data(), 1, H, eps);
        linear(Wq, xn.data(), q.data(), nh * hd, H, &bq, false);      // bias before the rotation
        linear(Wk, xn.data(), k.data(), nkv * hd, H, &bk, false);
        linear(Wv, xn.data(), v.data(), nkv * hd, H, &bv, false);
        cpu_fused_rope_kv_append(q.data(), k.data(), v.data(), Kc.data(), Vc.data(), (int)pos, nh, nkv, hd, max_seq, theta);
        cpu_attention_decoding(q.data(), Kc.data(), Vc.data(), o.data(), (int)pos, nh, nkv, hd, max_seq);
        linear(Wo, o.data(), x.data(), H, nh * hd, nullptr, true);    // added to the residual stream
        cpu_rmsnorm_direct(x.data(), xn.data(), n2b.data(), 1, H, eps);
        linear(Wg, xn.data(), g.data(), I, H, nullptr, false);
        linear(Wu, xn.data(), u.data(), I, H, nullptr, false);
        cpu_fused_swiglu(g.data(), u.data(), a.data(), I);
        linear(Wd, a.data(), x.data(), H, I, nullptr, true);
        cpu_rmsnorm_direct(x.data(), xn.data(), nfb.data(), 1, H, eps);
        linear(E, xn.data(), lg.data(), V, H, nullptr, false);        // tied head
        logits.insert(logits.end(), lg.begin(), lg.end());
    }
    fprintf(f, "{\n  \"H\": %zu, \"nh\": %zu, \"nkv\": %zu, \"hd\": %zu, \"I\": %zu, \"V\": %zu, \"T\": %zu, \"theta\": %.1f, \"eps\": %.9g,\n",
            H, nh, nkv, hd, I, V, T, theta, eps);
    fprintf(f, "  \"tokens\": [");
    for (size_t i = 0; i < T; ++i) fprintf(f, "%s%d", i ? ", " : "", tokens[i]);
    fprintf(f, "],\n");
    dump(f, "embed", E); dump(f, "norm1", n1); dump(f, "norm2", n2); dump(f, "norm_f", nf);
    dump(f, "wq", Wq); dump(f, "wk", Wk); dump(f, "wv", Wv); dump(f, "bq", bq); dump(f, "bk", bk); dump(f, "bv", bv);
    dump(f, "wo", Wo); dump(f, "wg", Wg); dump(f, "wu", Wu); dump(f, "wd", Wd);
    dump(f, "logits", logits, true);
    fprintf(f, "}\n");
    fclose(f);
    return 0;
}
