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

// ---------------------------------------------------------------------------------------------------------------------------------
// The serving kernels.  The columns of a head's state are independent of one another (column j sees only v[j]), so the grid is
// (entry, head, 16-column slice) and the whole slice of the state lives in REGISTERS: thread (ig, jj) of 256 holds rows ig, ig + 16, ...
// of column jj.  Tokens are walked in order; a chunk of 32 tokens' gates, queries and values is staged into shared memory with
// cp.async while the previous chunk is computed (two buffers), so that the serial loop has no global load, no shuffle and no barrier
// in it: per token a thread does R fused multiply-adds on its state and R on its partial output; the partial outputs of a chunk are
// summed over the 16 row groups after its last token.
//   hgrn2_gates_kernel      q <- silu(q_raw), f <- lower + (1 - lower) sigmoid(f_raw), in place, once for all column slices
//   hgrn2_scan_reg_kernel   the recurrence; leaves o un-normalised in `out`
//   hgrn2_out_norm_kernel   per (token, head): o / sqrt(mean o^2 + eps) * norm_w
constexpr int kScanCols = 16, kScanChunk = 32, kScanThreads = 256;

static __global__ void hgrn2_gates_kernel(float* __restrict__ qfv, int ld, const float* __restrict__ lower, int HD, int T) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)T * HD) return;
    const int t = (int)(idx / HD), c = (int)(idx % HD);
    float* row = qfv + (size_t)t * ld;
    row[c] = silu_f(row[c]);
    const float lo = lower[c];
    row[HD + c] = lo + (1.f - lo) * sigmoid_f(row[HD + c]);
}

__device__ __forceinline__ void cp_async_f32(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_f32x4(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

template <int R>   // state rows per thread: D <= 16 R
static __global__ void __launch_bounds__(kScanThreads) hgrn2_scan_reg_kernel(Hgrn2Args a, int vec, int raw) {
    extern __shared__ __align__(16) float sm[];
    const int e = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * kScanCols;
    const int D = a.D, Dv = a.Dv, HD = a.H * a.D;
    const int tid = threadIdx.x, ig = tid & 15, jj = tid >> 4, j = j0 + jj;
    const int stage_floats = kScanChunk * (2 * D + kScanCols);
    float* pS = sm + 2 * stage_floats;               // [chunk][256]: every thread's partial output of a token (summed over its state rows)
    const int t0 = a.rb.ent_start[e], t1 = a.rb.ent_start[e + 1];
    const bool fresh = a.rb.ent_pos0[e] == 0;
    float* st = a.state + (size_t)a.rb.ent_slot[e] * a.slot_stride + (size_t)h * D * Dv;
    float s[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = ig + 16 * r;
        s[r] = (!fresh && i < D && j < Dv) ? st[(size_t)i * Dv + j] : 0.f;
    }
    const int nch = (t1 - t0 + kScanChunk - 1) / kScanChunk;
    auto stage = [&](int c) {
        float* qS = sm + (c & 1) * stage_floats;
        float* fS = qS + kScanChunk * D;
        float* vS = fS + kScanChunk * D;
        const int tt0 = t0 + c * kScanChunk, cnt = min(kScanChunk, t1 - tt0);
        if (raw) {      // decode-sized steps: the gates are formed here instead of by a launch of their own
            for (int idx = tid; idx < cnt * D; idx += kScanThreads) {
                const int tl = idx / D, i = idx % D;
                const float* row = a.qfv + (size_t)(tt0 + tl) * a.ld + h * D + i;
                const float lo = a.lower[h * D + i];
                qS[tl * D + i] = silu_f(row[0]);
                fS[tl * D + i] = lo + (1.f - lo) * sigmoid_f(row[HD]);
            }
        } else if (vec) {
            const int D4 = D >> 2;
            for (int idx = tid; idx < cnt * D4; idx += kScanThreads) {
                const int tl = idx / D4, i = (idx % D4) * 4;
                const float* row = a.qfv + (size_t)(tt0 + tl) * a.ld + h * D + i;
                cp_async_f32x4(qS + tl * D + i, row);
                cp_async_f32x4(fS + tl * D + i, row + HD);
            }
        } else {
            for (int idx = tid; idx < cnt * D; idx += kScanThreads) {
                const int tl = idx / D, i = idx % D;
                const float* row = a.qfv + (size_t)(tt0 + tl) * a.ld + h * D + i;
                cp_async_f32(qS + tl * D + i, row);
                cp_async_f32(fS + tl * D + i, row + HD);
            }
        }
        for (int idx = tid; idx < cnt * kScanCols; idx += kScanThreads) {
            const int tl = idx / kScanCols, c2 = idx % kScanCols;
            if (j0 + c2 < Dv) cp_async_f32(vS + idx, a.qfv + (size_t)(tt0 + tl) * a.ld + 2 * HD + h * Dv + j0 + c2);
            else vS[idx] = 0.f;
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (nch > 0) stage(0);
    for (int c = 0; c < nch; ++c) {
        if (c + 1 < nch) { stage(c + 1); asm volatile("cp.async.wait_group 1;" ::: "memory"); }
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        const float* qS = sm + (c & 1) * stage_floats;
        const float* fS = qS + kScanChunk * D;
        const float* vS = fS + kScanChunk * D;
        const int tt0 = t0 + c * kScanChunk, cnt = min(kScanChunk, t1 - tt0);
        // the serial part: nothing but shared-memory reads and fused multiply-adds; the sum over the 16 row groups waits for the chunk's end
#pragma unroll 4
        for (int tl = 0; tl < cnt; ++tl) {
            const float vj = vS[tl * kScanCols + jj];
            float o = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int i = ig + 16 * r;
                if (i < D) {
                    const float f = fS[tl * D + i];
                    s[r] = fmaf(f, s[r], (1.f - f) * vj);
                    o = fmaf(s[r], qS[tl * D + i], o);
                }
            }
            pS[tl * kScanThreads + tid] = o;
        }
        __syncthreads();
        for (int idx = tid; idx < cnt * kScanCols; idx += kScanThreads) {      // idx = token * 16 + column: its 16 partial sums are consecutive
            const float4* pp = reinterpret_cast<const float4*>(pS + (size_t)idx * 16);
            const float4 p0 = pp[0], p1 = pp[1], p2 = pp[2], p3 = pp[3];
            const float o = ((p0.x + p0.y) + (p0.z + p0.w)) + ((p1.x + p1.y) + (p1.z + p1.w)) + ((p2.x + p2.y) + (p2.z + p2.w)) + ((p3.x + p3.y) + (p3.z + p3.w));
            const int tl = idx / kScanCols, c2 = idx % kScanCols;
            if (j0 + c2 < Dv) a.out[(size_t)(tt0 + tl) * a.H * Dv + h * Dv + j0 + c2] = o;
        }
        __syncthreads();       // pS and the buffer of chunk c are free again
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = ig + 16 * r;
        if (i < D && j < Dv) st[(size_t)i * Dv + j] = s[r];
    }
}

// one warp per (token, head) row of `out`
static __global__ void __launch_bounds__(256) hgrn2_out_norm_kernel(float* __restrict__ out, const float* __restrict__ norm_w, float eps, int rows, int Dv) {
    const int row = (int)(((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    float* o = out + (size_t)row * Dv;
    float ss = 0.f;
    for (int j = lane; j < Dv; j += 32) ss = fmaf(o[j], o[j], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)Dv + eps);
    for (int j = lane; j < Dv; j += 32) o[j] = o[j] * inv * norm_w[j];
}

inline size_t hgrn2_scan_reg_smem(int D) { return ((size_t)2 * kScanChunk * (2 * D + kScanCols) + kScanChunk * kScanThreads) * sizeof(float); }

template <int R>
inline void hgrn2_scan_reg_launch(cudaStream_t st, const Hgrn2Args& a, int vec, int raw) {
    static bool attr = false;
    const size_t smem = hgrn2_scan_reg_smem(a.D);
    if (!attr) { AHA_CUDA_CHECK(cudaFuncSetAttribute(hgrn2_scan_reg_kernel<R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)hgrn2_scan_reg_smem(16 * R))); attr = true; }
    hgrn2_scan_reg_kernel<R><<<dim3(a.rb.E, a.H, (a.Dv + kScanCols - 1) / kScanCols), kScanThreads, smem, st>>>(a, vec, raw);
}

// impl 0: the register kernels (dim <= 256); 1: the plain shared-memory kernel above.  `qfv` is overwritten by the gates (impl 0).  Returns launches.
inline int hgrn2_scan(cudaStream_t st, const Hgrn2Args& a, int impl = 0) {
    if (a.rb.E == 0) return 0;
    if (impl == 1 || a.D > 256) {
        const int threads = std::min(1024, ((a.Dv + 31) / 32) * 32);
        hgrn2_scan_kernel<<<dim3(a.rb.E, a.H), threads, hgrn2_scan_smem(a.D, a.Dv), st>>>(a);
        AHA_CUDA_CHECK(cudaGetLastError());
        return 1;
    }
    const int HD = a.H * a.D, T = a.rb.T;
    const int raw = T <= 32 ? 1 : 0;     // few tokens: every column slice forms the gates itself (one launch less); else once, in place
    if (!raw) hgrn2_gates_kernel<<<(unsigned)(((size_t)T * HD + 255) / 256), 256, 0, st>>>(const_cast<float*>(a.qfv), a.ld, a.lower, HD, T);
    const int vec = (a.D % 4 == 0 && a.ld % 4 == 0 && (reinterpret_cast<uintptr_t>(a.qfv) & 15) == 0) ? 1 : 0;
    const int R = (a.D + 15) / 16;
    if (R <= 1) hgrn2_scan_reg_launch<1>(st, a, vec, raw);
    else if (R <= 2) hgrn2_scan_reg_launch<2>(st, a, vec, raw);
    else if (R <= 4) hgrn2_scan_reg_launch<4>(st, a, vec, raw);
    else if (R <= 8) hgrn2_scan_reg_launch<8>(st, a, vec, raw);
    else hgrn2_scan_reg_launch<16>(st, a, vec, raw);
    hgrn2_out_norm_kernel<<<(unsigned)(((size_t)T * a.H * 32 + 255) / 256), 256, 0, st>>>(a.out, a.norm_w, a.eps, T * a.H, a.Dv);
    AHA_CUDA_CHECK(cudaGetLastError());
    return raw ? 2 : 3;
}

}  // namespace aha
