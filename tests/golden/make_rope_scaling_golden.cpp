// Driver that runs the reference project's own llama3 wavelength-band rescaling
// (apply_rope_scaling in its src/kernels/rope.cuh, taken from the reference checkout by include
// path at build time; nothing of it is copied here) on the host and writes the rescaled
// frequencies as JSON.  The function is device code guarded by __CUDACC__; the shim below makes
// the host compiler accept it: the qualifiers become nothing and __fdividef a plain division
// (on the GPU it is an approximate division: within 2 ulp of this).
// tests/test_plain_vs_reference_cpu.py compares the plain implementation's and the product's
// frequency tables with these numbers.  Build and run: see make_layer_golden.sh.
#include <cmath>
#include <cstdio>
#define __CUDACC__
#define __device__
#define __forceinline__ inline
static inline float __fdividef(float a, float b) { return a / b; }
#include "rope.cuh"

int main(int argc, char** argv) {
    FILE* f = fopen(argc > 1 ? argv[1] : "reference_rope_scaling.json", "w");
    if (!f) return 1;
    struct Case { int hd; float theta, factor, low, high, orig; };
    // the first two have all three bands inside one head; the last is Llama-3.1's own setting
    const Case cases[] = {{32, 500000.0f, 8.0f, 1.0f, 4.0f, 32.0f},
                          {32, 10000.0f, 4.0f, 1.0f, 2.0f, 64.0f},
                          {128, 10000.0f, 8.0f, 1.0f, 4.0f, 2048.0f},
                          {128, 500000.0f, 8.0f, 1.0f, 4.0f, 8192.0f}};
    const int n = sizeof(cases) / sizeof(cases[0]);
    fprintf(f, "{\"cases\": [\n");
    for (int c = 0; c < n; ++c) {
        const Case& k = cases[c];
        RopeScaling s;
        s.enabled = 1; s.factor = k.factor; s.low_freq_factor = k.low; s.high_freq_factor = k.high; s.orig_ctx = k.orig;
        fprintf(f, " {\"head_dim\": %d, \"theta\": %.1f, \"factor\": %.1f, \"low\": %.1f, \"high\": %.1f, \"orig\": %.1f,\n"
                   "  \"plain\": [", k.hd, k.theta, k.factor, k.low, k.high, k.orig);
        // the frequency of pair j as the reference's kernels form it (src/kernels/rope.cu:21)
        for (int j = 0; j < k.hd / 2; ++j)
            fprintf(f, "%s%.9g", j ? ", " : "", 1.0f / powf(k.theta, (float)(2 * j) / (float)k.hd));
        fprintf(f, "],\n  \"scaled\": [");
        for (int j = 0; j < k.hd / 2; ++j)
            fprintf(f, "%s%.9g", j ? ", " : "", apply_rope_scaling(1.0f / powf(k.theta, (float)(2 * j) / (float)k.hd), s));
        fprintf(f, "],\n  \"band\": [");   // 0 unchanged, 1 divided by the factor, 2 in between
        for (int j = 0; j < k.hd / 2; ++j) {
            const float inv = 1.0f / powf(k.theta, (float)(2 * j) / (float)k.hd);
            const float wl = 6.28318530717958647692f / inv;
            fprintf(f, "%s%d", j ? ", " : "", wl < k.orig / k.high ? 0 : (wl > k.orig / k.low ? 1 : 2));
        }
        fprintf(f, "]}%s\n", c + 1 < n ? "," : "");
    }
    fprintf(f, "]}\n");
    fclose(f);
    return 0;
}
