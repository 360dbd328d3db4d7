// Driver that runs the reference project's own CPU kernels (its header
// tests/common/cpu_reference.h, taken from the reference checkout by include path at
// build time; nothing of it is copied here) on small seeded inputs and writes inputs
// and outputs as JSON.  tests/test_plain_vs_reference_cpu.py compares the plain
// implementation with these numbers.  Build and run: see make_golden.sh.
#include "cpu_reference.h"
#include <cstdio>
#include <vector>

static unsigned long long lcg_state = 12345;
static float rnd() {
    lcg_state = (lcg_state * 6364136223846793005ULL + 1442695040888963407ULL);
    return (float)((lcg_state >> 40) & 0xFFFFFF) / 8388608.0f - 1.0f;   // [-1, 1)
}
static void dump(FILE* f, const char* name, const std::vector<float>& v, bool last = false) {
    fprintf(f, "  \"%s\": [", name);
    for (size_t i = 0; i < v.size(); ++i) fprintf(f, "%s%.9g", i ? ", " : "", v[i]);
    fprintf(f, "]%s\n", last ? "" : ",");
}

int main(int argc, char** argv) {
    FILE* f = fopen(argc > 1 ? argv[1] : "reference_cpu.json", "w");
    if (!f) return 1;
    const size_t nh = 4, nkv = 2, hd = 8, T = 6, max_seq = 8;
    const float theta = 10000.0f;
    fprintf(f, "{\n  \"nh\": %zu, \"nkv\": %zu, \"hd\": %zu, \"T\": %zu, \"theta\": %.1f,\n", nh, nkv, hd, T, theta);

    // rope + cache append + single-query attention, position by position
    std::vector<float> Kc(nkv * max_seq * hd, 0.f), Vc(nkv * max_seq * hd, 0.f);
    std::vector<float> q_in, k_in, v_in, q_rot, k_rot, attn;
    for (size_t pos = 0; pos < T; ++pos) {
        std::vector<float> Q(nh * hd), K(nkv * hd), V(nkv * hd), O(nh * hd);
        for (auto& x : Q) x = rnd();
        for (auto& x : K) x = rnd();
        for (auto& x : V) x = rnd();
        q_in.insert(q_in.end(), Q.begin(), Q.end());
        k_in.insert(k_in.end(), K.begin(), K.end());
        v_in.insert(v_in.end(), V.begin(), V.end());
        cpu_fused_rope_kv_append(Q.data(), K.data(), V.data(), Kc.data(), Vc.data(), (int)pos, nh, nkv, hd, max_seq, theta);
        cpu_attention_decoding(Q.data(), Kc.data(), Vc.data(), O.data(), (int)pos, nh, nkv, hd, max_seq);
        q_rot.insert(q_rot.end(), Q.begin(), Q.end());
        k_rot.insert(k_rot.end(), K.begin(), K.end());
        attn.insert(attn.end(), O.begin(), O.end());
    }
    dump(f, "q_in", q_in); dump(f, "k_in", k_in); dump(f, "v_in", v_in);
    dump(f, "q_rot", q_rot); dump(f, "k_rot", k_rot); dump(f, "attn", attn);

    // RMSNorm (bf16-latched in the reference) and SwiGLU (likewise)
    const size_t H = 24, R = 3;
    std::vector<float> x(R * H), w(H), y(R * H);
    std::vector<__nv_bfloat16> wb(H);
    for (auto& v : x) v = 3.0f * rnd();
    for (size_t i = 0; i < H; ++i) { wb[i] = __float2bfloat16(1.0f + 0.25f * rnd()); w[i] = __bfloat162float(wb[i]); }
    cpu_rmsnorm_direct(x.data(), y.data(), wb.data(), R, H, 1e-5f);
    dump(f, "norm_x", x); dump(f, "norm_w", w); dump(f, "norm_y", y);
    std::vector<float> g(40), u(40), s(40);
    for (auto& v : g) v = 4.0f * rnd();
    for (auto& v : u) v = 2.0f * rnd();
    cpu_fused_swiglu(g.data(), u.data(), s.data(), g.size());
    dump(f, "swiglu_g", g); dump(f, "swiglu_u", u); dump(f, "swiglu_y", s);

    // embedding and argmax (ties: the reference keeps the first maximum)
    std::vector<float> table(5 * 4);
    for (auto& v : table) v = rnd();
    int toks[3] = {4, 0, 2};
    std::vector<float> emb(3 * 4);
    cpu_embedding_lookup(toks, table.data(), emb.data(), 3, 4);
    dump(f, "embed_table", table); dump(f, "embed_out", emb);
    std::vector<float> logits = {0.5f, 2.0f, -1.0f, 2.0f, 1.5f};
    int am = -1;
    cpu_argmax(logits.data(), &am, logits.size());
    dump(f, "argmax_logits", logits);
    fprintf(f, "  \"argmax\": %d\n}\n", am);
    fclose(f);
    return 0;
}
