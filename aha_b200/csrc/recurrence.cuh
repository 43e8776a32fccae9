// recurrence.cuh -- gated linear recurrences with a matrix state per head, kept in fp32 for every sequence slot.
//
// HGRN2 form (one forget gate per key channel that also weights what is written; no separate key):
//     f_t = lower + (1 - lower) * sigmoid(f_raw_t)            per (head, key channel i), lower in [0, 1]
//     q_t = silu(q_raw_t)
//     S_t[i][j] = f_t[i] S_{t-1}[i][j] + (1 - f_t[i]) v_t[j]
//     o_t[j]    = sum_i S_t[i][j] q_t[i]
//     out_t     = o_t / sqrt(mean_j o_t[j]^2 + eps) * norm_w[j]        (per head, gain shared by the heads)
// The step is ragged: block (entry, head) walks the entry's tokens in order, starting from the slot's state -- or from zero when the
// sequence starts in this step (position 0), so a slot that is used again needs no clearing -- and leaves the state in the slot.
// Gates, their sigmoid, the state and the output norm are fp32.
#pragma once
#include "common.cuh"
#include "ragged.cuh"

namespace aha {

struct Hgrn2Args {
    const float* qfv;      // [T, ld]: q_raw (H*D) | f_raw (H*D, bias already added) | v (H*Dv)
    int ld;
    const float* lower;    // [H*D]
    const float* norm_w;   // [Dv]
    float eps;
    float* state;          // [slots][H][D][Dv] of this layer
    size_t slot_stride;    // floats between slots
    float* out;            // [T, H*Dv]
    int H, D, Dv;
    RaggedBatch rb;
};

// Generic version: the head's state lives in shared memory ([D][Dv] floats), thread j owns column j (and j + blockDim, ...).
static __global__ void hgrn2_scan_kernel(Hgrn2Args a) {
    extern __shared__ float sm[];
    const int e = blockIdx.x, h = blockIdx.y;
    const int D = a.D, Dv = a.Dv;
    float* S = sm;                 // [D][Dv]
    float* fq = sm + (size_t)D * Dv;   // f[D] | q[D]
    float* red = fq + 2 * D;       // [32]
    const int t0 = a.rb.ent_start[e], t1 = a.rb.ent_start[e + 1];
    const int slot = a.rb.ent_slot[e];
    const bool fresh = a.rb.ent_pos0[e] == 0;
    float* st = a.state + (size_t)slot * a.slot_stride + (size_t)h * D * Dv;
    for (int i = threadIdx.x; i < D * Dv; i += blockDim.x) S[i] = fresh ? 0.f : st[i];
    __syncthreads();
    for (int t = t0; t < t1; ++t) {
        const float* row = a.qfv + (size_t)t * a.ld;
        for (int i = threadIdx.x; i < D; i += blockDim.x) {
            const float lo = a.lower[h * D + i];
            fq[i] = lo + (1.f - lo) * sigmoid_f(row[a.H * D + h * D + i]);
            fq[D + i] = silu_f(row[h * D + i]);
        }
        __syncthreads();
        float ss = 0.f;
        for (int j = threadIdx.x; j < Dv; j += blockDim.x) {
            const float v = row[2 * a.H * D + h * Dv + j];
            float o = 0.f;
            for (int i = 0; i < D; ++i) {
                const float f = fq[i];
                const float s = fmaf(f, S[i * Dv + j], (1.f - f) * v);
                S[i * Dv + j] = s;
                o = fmaf(s, fq[D + i], o);
            }
            ss = fmaf(o, o, ss);
            a.out[(size_t)t * a.H * Dv + h * Dv + j] = o;      // normalised below
        }
        ss = block_sum(ss, red);                                // (its barriers also order fq's reuse)
        const float inv = 1.0f / sqrtf(ss / (float)Dv + a.eps);
        for (int j = threadIdx.x; j < Dv; j += blockDim.x) {
            float* o = a.out + (size_t)t * a.H * Dv + h * Dv + j;
            *o = *o * inv * a.norm_w[j];
        }
        __syncthreads();
    }
    for (int i = threadIdx.x; i < D * Dv; i += blockDim.x) st[i] = S[i];
}

inline size_t hgrn2_scan_smem(int D, int Dv) { return ((size_t)D * Dv + 2 * D + 32) * sizeof(float); }

inline void hgrn2_scan(cudaStream_t st, const Hgrn2Args& a) {
    if (a.rb.E == 0) return;
    const int threads = std::min(1024, ((a.Dv + 31) / 32) * 32);
    hgrn2_scan_kernel<<<dim3(a.rb.E, a.H), threads, hgrn2_scan_smem(a.D, a.Dv), st>>>(a);
    AHA_CUDA_CHECK(cudaGetLastError());
}

}  // namespace aha
