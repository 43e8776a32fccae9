// attention_latent.cuh -- what is special about latent attention: every token leaves ONE low-rank latent c (RMS-normed) and ONE rotated
// key part in the cache, shared by all heads; a head's keys and values are W_uk c and W_uv c.  The engine never expands them: with
//     score = q_plain . (W_uk c) + q_rot . k_rot = (W_uk^T q_plain) . c + q_rot . k_rot
// a head's query becomes [W_uk^T q_plain | q_rot] against the cached row [c | k_rot], and its output W_uv (sum_j p_j c_j): ordinary
// attention of many query heads over a single key / value head whose values are the first `rank` columns of its keys.  The two
// per-head products are batched matrix products (gemm_any.cuh), the attention itself is the ragged kernel of attention_window.cuh.
//
//   latent_prep_kernel   per token: RMS norm of the latent (gain per channel) and rotary embedding of the shared key part into the page
//                        of the token's position; rotary embedding of every head's rotated query part into the absorbed-query buffer.
// Rotary: interleaved pairs (2i, 2i + 1) of the first 2 * n_freq coordinates turn by pos * freq[i]; cos and sin carry `mult` (YaRN's
// attention factor); further coordinates pass unchanged.  Angles are fp32 products, cos / sin the accurate functions.
#pragma once
#include <cmath>
#include <vector>

#include "attention_window.cuh"

namespace aha {

// Rotary frequencies with optional YaRN interpolation (host, double): dims rotated coordinates, base; factor > 0: frequencies whose
// wavelength exceeds the original context are divided by `factor`, short ones kept, a linear ramp between the coordinates whose
// wavelengths fit `fast` and `slow` times into `original`; cos / sin are multiplied by 0.1 ln(factor) + 1.
inline void yarn_frequencies(int dims, double base, double factor, double original, double fast, double slow, std::vector<float>& freq, float& mult) {
    const int n = dims / 2;
    freq.resize(n);
    mult = 1.f;
    const double pi = 3.14159265358979323846;
    auto dim_of = [&](double turns) { return dims * std::log(original / (2.0 * pi * turns)) / (2.0 * std::log(base)); };
    double lo = 0, hi = 0;
    if (factor > 0) {
        lo = std::max(std::floor(dim_of(fast)), 0.0);
        hi = std::min(std::ceil(dim_of(slow)), (double)(dims - 1));
        mult = (float)(0.1 * std::log(factor) + 1.0);
    }
    for (int i = 0; i < n; ++i) {
        const double f = std::pow(base, -2.0 * i / dims);
        if (factor > 0) {
            const double ramp = std::min(1.0, std::max(0.0, (i - lo) / std::max(hi - lo, 0.001)));
            freq[i] = (float)(f / factor * ramp + f * (1.0 - ramp));
        } else freq[i] = (float)f;
    }
}

struct LatentPrepArgs {
    float* proj; int ld;            // [T, ld] projected rows
    int q_off, dkv_off;             // first query column (heads x (dim + rot)), first latent column (rank + rot)
    int H, D, R, rank;
    const float* c_norm; float eps; // [rank]
    const float* freq; int n_freq; float mult;
    float* q_abs; int ld_q;         // [T, H * (rank + R)]: the rotated query part goes to columns h * (rank + R) + rank ...
    PagedKV kv;                     // G = 1, D = rank + R
    RaggedBatch rb;
};

static __global__ void latent_prep_kernel(LatentPrepArgs a) {
    __shared__ float red[32];
    const int t = blockIdx.x;
    const int e = a.rb.tok_entry[t], pos = a.rb.tok_pos[t], slot = a.rb.ent_slot[e];
    const float* row = a.proj + (size_t)t * a.ld;
    const int page = a.rb.page_tables[(size_t)slot * a.rb.max_pages + (pos >> kPageShift)];
    float* krow = a.kv.k_row(page, 0, pos & (kPage - 1));
    const float* d = row + a.dkv_off;
    float ss = 0.f;
    for (int i = threadIdx.x; i < a.rank; i += blockDim.x) ss = fmaf(d[i], d[i], ss);
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)a.rank + a.eps);
    for (int i = threadIdx.x; i < a.rank; i += blockDim.x) krow[i] = d[i] * inv * a.c_norm[i];
    // rotated parts: item (0, pair) is the shared key part, item (1 + h, pair) head h's query part; pairs beyond n_freq are single pass-through coordinates
    const int half = a.n_freq, rest = a.R - 2 * half, per = half + rest;
    const float fpos = (float)pos;
    for (int idx = threadIdx.x; idx < (1 + a.H) * per; idx += blockDim.x) {
        const int item = idx / per, j = idx % per;
        const float* src = item == 0 ? d + a.rank : row + a.q_off + (size_t)(item - 1) * (a.D + a.R) + a.D;
        float* dst = item == 0 ? krow + a.rank : a.q_abs + (size_t)t * a.ld_q + (size_t)(item - 1) * (a.rank + a.R) + a.rank;
        if (j < half) {
            float sn, cs;
            sincosf(fpos * a.freq[j], &sn, &cs);
            sn *= a.mult; cs *= a.mult;
            const float u = src[2 * j], v = src[2 * j + 1];
            dst[2 * j] = u * cs - v * sn;
            dst[2 * j + 1] = v * cs + u * sn;
        } else {
            const int c = 2 * half + (j - half);
            dst[c] = src[c];
        }
    }
}

}  // namespace aha
