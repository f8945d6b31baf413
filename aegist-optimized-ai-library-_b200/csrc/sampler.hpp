// The reference's sampler (aegist_rs/src/chat.rs:221-272), host side: top-k, then nucleus, then an
// inverse-CDF draw from a splitmix64 stream; temperature <= 0 is greedy and the first maximum wins.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <numeric>
#include <vector>

namespace b2 {
inline double splitmix_next_f64(uint64_t* s) {
    *s += 0x9E3779B97F4A7C15ull;
    uint64_t z = *s;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (double)(z >> 11) / (double)(1ull << 53);
}
}  // namespace b2

extern "C" uint32_t b2_sample(const float* logits, int vocab, float temperature, float top_p, int top_k, uint64_t* rng_state) {
    if (vocab <= 0) return 0;
    if (temperature <= 0.0f) {
        // first maximum wins. Two levels, so that the long pass is eight independent running maxima the compiler
        // turns into vector compares: the largest value of every block of 512, the first block that holds the
        // overall maximum, then the first position inside it. A NaN never wins a '>' and is never picked.
        constexpr int BL = 512;
        float gmax = -INFINITY;
        int gblock = -1;
        for (int b0 = 0; b0 < vocab; b0 += BL) {
            const int n = std::min(BL, vocab - b0);
            float m[8] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY, -INFINITY, -INFINITY, -INFINITY, -INFINITY};
            int i = 0;
            for (; i + 8 <= n; i += 8)
                for (int l = 0; l < 8; l++) m[l] = logits[b0 + i + l] > m[l] ? logits[b0 + i + l] : m[l];
            for (; i < n; i++) m[0] = logits[b0 + i] > m[0] ? logits[b0 + i] : m[0];
            float bm = m[0];
            for (int l = 1; l < 8; l++) bm = m[l] > bm ? m[l] : bm;
            if (bm > gmax) { gmax = bm; gblock = b0; }
        }
        if (gblock < 0) return 0;
        for (int i = gblock; i < std::min(gblock + BL, vocab); i++)
            if (logits[i] == gmax) return (uint32_t)i;
        return 0;
    }
    const int k = std::max(1, std::min(top_k, vocab));
    std::vector<uint32_t> idx(vocab);
    std::iota(idx.begin(), idx.end(), 0u);
    // descending by logit; equal logits keep the lower id first
    auto desc = [&](uint32_t a, uint32_t b) { return logits[a] > logits[b] || (logits[a] == logits[b] && a < b); };
    if (k < vocab) {
        std::partial_sort(idx.begin(), idx.begin() + k, idx.end(), desc);
        idx.resize(k);
    } else {
        std::sort(idx.begin(), idx.end(), desc);
    }
    const float top = logits[idx[0]];
    std::vector<double> p(k);
    double sum = 0;
    for (int j = 0; j < k; j++) { p[j] = std::exp((double)((logits[idx[j]] - top) / temperature)); sum += p[j]; }
    double cum = 0, total = 0;
    for (int j = 0; j < k; j++) {
        p[j] /= sum;
        const bool keep = cum < (double)top_p;   // the mass BEFORE this token
        cum += p[j];
        if (!keep) p[j] = 0;
        total += p[j];
    }
    double r = b2::splitmix_next_f64(rng_state) * total;
    for (int j = 0; j < k; j++) {
        r -= p[j];
        if (r < 0.0 && p[j] > 0.0) return idx[j];
    }
    return idx[0];
}
