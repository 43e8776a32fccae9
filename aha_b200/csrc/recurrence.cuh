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
//
// Keyed form (gated linear attention, selective state spaces): a separate key weights what is written,
//     S_t[i][j] = f_t[i] S_{t-1}[i][j] + k_t[i] v_t[j],      o_t[j] = sum_i S_t[i][j] q_t[i],
// with q, f, k already final in the row buffer (the caller's own gate kernel ran: gates_done) at the columns q_off / f_off / k_off and
// the values possibly in another buffer; the output norm is optional.  The same scan, segment and state machinery serves both forms.
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
    // long prompt portions cut into segments that are scanned side by side (see hgrn2_scan); all unset: every entry is walked whole
    float* seg_state = nullptr;   // [segments of the step][H][D][Dv]
    float* seg_decay = nullptr;   // [segments of the step][H*D]
    int seg_len = 0;              // tokens per segment
    int seg_max = 0;              // segments of the step's longest entry
    // where the operands are (hgrn2_scan fills the HGRN2 defaults in: f after q, v after f, all in qfv)
    int q_off = 0;                // column of the first query channel in a row of qfv
    int f_off = -1;               // ... of the first decay channel; -1: H*D
    int k_off = -1;               // ... of the first key channel; -1: no separate key, what is written is weighted by 1 - f
    const float* v = nullptr;     // [T, ld_v] values at column v_off; nullptr: in qfv at column 2*H*D
    int ld_v = 0, v_off = 0;
    int gates_done = 0;           // 1: q, f (and k) are final, no gate kernel and no in-kernel gate arithmetic
    const float* out_gate = nullptr; int out_gate_ld = 0;   // the output norm also multiplies by silu(out_gate[t][h*Dv + j])
};

// Segments of a step are numbered entry by entry; an entry has at least one.
__device__ __forceinline__ int hgrn2_seg_count(const RaggedBatch& rb, int e, int L) { return max(1, (rb.ent_start[e + 1] - rb.ent_start[e] + L - 1) / L); }
__device__ __forceinline__ int hgrn2_seg_base(const RaggedBatch& rb, int e, int L) {
    int b = 0;
    for (int i = 0; i < e; ++i) b += hgrn2_seg_count(rb, i, L);
    return b;
}

// Generic version: the head's state lives in shared memory ([D][Dv] floats), thread j owns column j (and j + blockDim, ...).
static __global__ void hgrn2_scan_kernel(Hgrn2Args a) {
    extern __shared__ float sm[];
    const int e = blockIdx.x, h = blockIdx.y;
    const int D = a.D, Dv = a.Dv;
    float* S = sm;                 // [D][Dv]
    float* fq = sm + (size_t)D * Dv;   // f[D] | q[D] | write weight[D]
    float* red = fq + 3 * D;       // [32]
    const int t0 = a.rb.ent_start[e], t1 = a.rb.ent_start[e + 1];
    const int slot = a.rb.ent_slot[e];
    const bool fresh = a.rb.ent_pos0[e] == 0;
    float* st = a.state + (size_t)slot * a.slot_stride + (size_t)h * D * Dv;
    for (int i = threadIdx.x; i < D * Dv; i += blockDim.x) S[i] = fresh ? 0.f : st[i];
    __syncthreads();
    for (int t = t0; t < t1; ++t) {
        const float* row = a.qfv + (size_t)t * a.ld;
        for (int i = threadIdx.x; i < D; i += blockDim.x) {
            if (a.gates_done) {
                fq[i] = row[a.f_off + h * D + i];
                fq[D + i] = row[a.q_off + h * D + i];
                fq[2 * D + i] = a.k_off >= 0 ? row[a.k_off + h * D + i] : 1.f - fq[i];
            } else {
                const float lo = a.lower[h * D + i];
                fq[i] = lo + (1.f - lo) * sigmoid_f(row[a.f_off + h * D + i]);
                fq[D + i] = silu_f(row[a.q_off + h * D + i]);
                fq[2 * D + i] = 1.f - fq[i];
            }
        }
        __syncthreads();
        float ss = 0.f;
        for (int j = threadIdx.x; j < Dv; j += blockDim.x) {
            const float v = a.v[(size_t)t * a.ld_v + a.v_off + h * Dv + j];
            float o = 0.f;
            for (int i = 0; i < D; ++i) {
                const float s = fmaf(fq[i], S[i * Dv + j], fq[2 * D + i] * v);
                S[i * Dv + j] = s;
                o = fmaf(s, fq[D + i], o);
            }
            ss = fmaf(o, o, ss);
            a.out[(size_t)t * a.H * Dv + h * Dv + j] = o;      // normalised below
        }
        ss = block_sum(ss, red);                                // (its barriers also order fq's reuse)
        if (a.norm_w) {
            const float inv = 1.0f / sqrtf(ss / (float)Dv + a.eps);
            for (int j = threadIdx.x; j < Dv; j += blockDim.x) {
                float* o = a.out + (size_t)t * a.H * Dv + h * Dv + j;
                float r = *o * inv * a.norm_w[j];
                if (a.out_gate) r *= silu_f(a.out_gate[(size_t)t * a.out_gate_ld + h * Dv + j]);
                *o = r;
            }
        }
        __syncthreads();
    }
    for (int i = threadIdx.x; i < D * Dv; i += blockDim.x) st[i] = S[i];
}

inline size_t hgrn2_scan_smem(int D, int Dv) { return ((size_t)D * Dv + 3 * D + 32) * sizeof(float); }

// ---------------------------------------------------------------------------------------------------------------------------------
// The serving kernels.  The columns of a head's state are independent of one another (column j sees only v[j]), so the grid is
// (entry, head, 32-column slice) and the whole slice of the state lives in REGISTERS: thread (ig, jj) of 256 holds, of the columns jj and
// jj + 16, the rows 4 ig .. 4 ig + 3 of every block of 64 rows.  A gate or query value read from shared memory (16 bytes = four rows a
// load) thus serves two columns, and the 16 threads of one column read 256 consecutive bytes.  Tokens are walked in order; a chunk of
// 16 tokens' gates, queries and values is staged into shared memory with cp.async while the previous chunk is computed (two buffers;
// rows are padded to 16 R with f = 1, q = 0), so that the serial loop has no global load, no shuffle, no barrier and no predicate in
// it: per token a thread does 2 R fused multiply-adds on its state and 2 R on its partial outputs; the partial outputs of a chunk are
// summed over the 16 row groups after its last token.
//   hgrn2_gates_kernel      q <- silu(q_raw), f <- lower + (1 - lower) sigmoid(f_raw), in place, once for all column slices
//   hgrn2_scan_reg_kernel   the recurrence; leaves o un-normalised in `out`
//   hgrn2_out_norm_kernel   per (token, head): o / sqrt(mean o^2 + eps) * norm_w
constexpr int kScanCols = 32, kScanChunk = 16, kScanThreads = 256;
constexpr int kScanPad = 20;     // floats between the partial-output groups of two columns: 16 + 4, so that the 16-byte reads of the sum spread over the banks

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

template <int R, bool KEYED>   // R: state rows per thread and column, a multiple of 4: D <= 16 R; KEYED: a separate key is staged beside the decay
static __global__ void __launch_bounds__(kScanThreads) hgrn2_scan_reg_kernel(Hgrn2Args a, int vec, int raw) {
    extern __shared__ __align__(16) float sm[];
    constexpr int Dp = 16 * R, R4 = R / 4, NA = KEYED ? 3 : 2;
    const int h = blockIdx.y, j0 = blockIdx.z * kScanCols;
    const int D = a.D, Dv = a.Dv, HD = a.H * a.D;
    const int tid = threadIdx.x, ig = tid & 15, jj = tid >> 4;
    constexpr int stage_floats = kScanChunk * (NA * Dp + kScanCols);
    float* pS = sm + 2 * stage_floats;               // [chunk][32 columns][kScanPad]: every thread's partial outputs of a token (summed over its state rows)
    int e = blockIdx.x, t0, t1;
    bool fresh;
    const float* st_in;
    float* st;
    if (a.seg_len > 0) {      // segment k of entry e: from the slot's state (k == 0) or from zero, to the segment's scratch
        e = blockIdx.x / a.seg_max;
        const int k = blockIdx.x % a.seg_max;
        if (k >= hgrn2_seg_count(a.rb, e, a.seg_len)) return;
        t0 = a.rb.ent_start[e] + k * a.seg_len;
        t1 = min(a.rb.ent_start[e + 1], t0 + a.seg_len);
        fresh = k > 0 || a.rb.ent_pos0[e] == 0;
        st_in = a.state + (size_t)a.rb.ent_slot[e] * a.slot_stride + (size_t)h * D * Dv;
        st = a.seg_state + ((size_t)(hgrn2_seg_base(a.rb, e, a.seg_len) + k) * a.H + h) * D * Dv;
    } else {
        t0 = a.rb.ent_start[e]; t1 = a.rb.ent_start[e + 1];
        fresh = a.rb.ent_pos0[e] == 0;
        st = a.state + (size_t)a.rb.ent_slot[e] * a.slot_stride + (size_t)h * D * Dv;
        st_in = st;
    }
    auto row_of = [&](int r) { return (r >> 2) * 64 + 4 * ig + (r & 3); };
    float s[R][2];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int i = row_of(r), j = j0 + 16 * c + jj;
            s[r][c] = (!fresh && i < D && j < Dv) ? st_in[(size_t)i * Dv + j] : 0.f;
        }
    // rows beyond `dim` of both buffers: f = 1, q = 0 (their state stays zero); no copy below touches them
    for (int idx = tid; idx < 2 * kScanChunk * (Dp - D); idx += kScanThreads) {
        const int b = idx / (kScanChunk * (Dp - D)), rem = idx % (kScanChunk * (Dp - D)), tl = rem / (Dp - D), i = D + rem % (Dp - D);
        float* qS = sm + b * stage_floats;
        qS[tl * Dp + i] = 0.f;
        qS[kScanChunk * Dp + tl * Dp + i] = 1.f;
        if (KEYED) qS[2 * kScanChunk * Dp + tl * Dp + i] = 0.f;
    }
    const int nch = (t1 - t0 + kScanChunk - 1) / kScanChunk;
    auto stage = [&](int c) {
        float* qS = sm + (c & 1) * stage_floats;
        float* fS = qS + kScanChunk * Dp;
        float* kS = fS + kScanChunk * Dp;       // KEYED only
        float* vS = qS + NA * kScanChunk * Dp;
        const int tt0 = t0 + c * kScanChunk, cnt = min(kScanChunk, t1 - tt0);
        if (raw) {      // decode-sized steps: the gates are formed here instead of by a launch of their own
            for (int idx = tid; idx < cnt * D; idx += kScanThreads) {
                const int tl = idx / D, i = idx % D;
                const float* row = a.qfv + (size_t)(tt0 + tl) * a.ld + h * D + i;
                const float lo = a.lower[h * D + i];
                qS[tl * Dp + i] = silu_f(row[a.q_off]);
                fS[tl * Dp + i] = lo + (1.f - lo) * sigmoid_f(row[a.f_off]);
            }
        } else if (vec) {
            const int D4 = D >> 2;
            for (int idx = tid; idx < cnt * D4; idx += kScanThreads) {
                const int tl = idx / D4, i = (idx % D4) * 4;
                const float* row = a.qfv + (size_t)(tt0 + tl) * a.ld + h * D + i;
                cp_async_f32x4(qS + tl * Dp + i, row + a.q_off);
                cp_async_f32x4(fS + tl * Dp + i, row + a.f_off);
                if (KEYED) cp_async_f32x4(kS + tl * Dp + i, row + a.k_off);
            }
        } else {
            for (int idx = tid; idx < cnt * D; idx += kScanThreads) {
                const int tl = idx / D, i = idx % D;
                const float* row = a.qfv + (size_t)(tt0 + tl) * a.ld + h * D + i;
                cp_async_f32(qS + tl * Dp + i, row + a.q_off);
                cp_async_f32(fS + tl * Dp + i, row + a.f_off);
                if (KEYED) cp_async_f32(kS + tl * Dp + i, row + a.k_off);
            }
        }
        for (int idx = tid; idx < cnt * kScanCols; idx += kScanThreads) {
            const int tl = idx / kScanCols, c2 = idx % kScanCols;
            if (j0 + c2 < Dv) cp_async_f32(vS + idx, a.v + (size_t)(tt0 + tl) * a.ld_v + a.v_off + h * Dv + j0 + c2);
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
        const float* fS = qS + kScanChunk * Dp;
        const float* kS = fS + kScanChunk * Dp;
        const float* vS = qS + NA * kScanChunk * Dp;
        const int tt0 = t0 + c * kScanChunk, cnt = min(kScanChunk, t1 - tt0);
        // the serial part: nothing but shared-memory reads and fused multiply-adds.  Tokens are taken G at a time with all loads of the
        // group ahead of its arithmetic (the stores of partial outputs would otherwise fence the next token's loads).  The sum over the
        // 16 row groups waits for the chunk's end.
        {
            constexpr int G = R >= 16 ? 1 : 2;
            const float4* fp = reinterpret_cast<const float4*>(fS) + ig;
            const float4* qp = reinterpret_cast<const float4*>(qS) + ig;
            const float4* kp = reinterpret_cast<const float4*>(kS) + ig;
            const float* vp = vS + jj;
            float* pp = pS + jj * kScanPad + ig;
            auto token = [&](const float4* fv, const float4* qv, const float4* kv, float v0, float v1, int tl) {
                float o0 = 0.f, o1 = 0.f;
#pragma unroll
                for (int r4 = 0; r4 < R4; ++r4) {
                    const float f[4] = {fv[r4].x, fv[r4].y, fv[r4].z, fv[r4].w}, q[4] = {qv[r4].x, qv[r4].y, qv[r4].z, qv[r4].w};
                    const float kk[4] = {kv[r4].x, kv[r4].y, kv[r4].z, kv[r4].w};
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const float g = KEYED ? kk[u] : 1.f - f[u];
                        float* sr = s[4 * r4 + u];
                        sr[0] = fmaf(f[u], sr[0], g * v0);
                        sr[1] = fmaf(f[u], sr[1], g * v1);
                        o0 = fmaf(sr[0], q[u], o0);
                        o1 = fmaf(sr[1], q[u], o1);
                    }
                }
                pp[tl * (kScanCols * kScanPad)] = o0;
                pp[tl * (kScanCols * kScanPad) + 16 * kScanPad] = o1;
            };
            int tl = 0;
            for (; tl + G <= cnt; tl += G) {
                float4 fv[G][R4], qv[G][R4], kv[G][KEYED ? R4 : 1];
                float v0[G], v1[G];
#pragma unroll
                for (int u = 0; u < G; ++u) {
                    v0[u] = vp[(tl + u) * kScanCols];
                    v1[u] = vp[(tl + u) * kScanCols + 16];
#pragma unroll
                    for (int r4 = 0; r4 < R4; ++r4) {
                        fv[u][r4] = fp[(tl + u) * (Dp / 4) + 16 * r4];
                        qv[u][r4] = qp[(tl + u) * (Dp / 4) + 16 * r4];
                        if (KEYED) kv[u][r4] = kp[(tl + u) * (Dp / 4) + 16 * r4];
                    }
                }
#pragma unroll
                for (int u = 0; u < G; ++u) token(fv[u], qv[u], KEYED ? kv[u] : fv[u], v0[u], v1[u], tl + u);
            }
            for (; tl < cnt; ++tl) {
                float4 fv[R4], qv[R4], kv[KEYED ? R4 : 1];
#pragma unroll
                for (int r4 = 0; r4 < R4; ++r4) {
                    fv[r4] = fp[tl * (Dp / 4) + 16 * r4];
                    qv[r4] = qp[tl * (Dp / 4) + 16 * r4];
                    if (KEYED) kv[r4] = kp[tl * (Dp / 4) + 16 * r4];
                }
                token(fv, qv, KEYED ? kv : fv, vp[tl * kScanCols], vp[tl * kScanCols + 16], tl);
            }
        }
        __syncthreads();
        for (int idx = tid; idx < cnt * kScanCols; idx += kScanThreads) {      // idx = token * 32 + column: its 16 partial sums are consecutive
            const float4* pq = reinterpret_cast<const float4*>(pS + (size_t)idx * kScanPad);
            const float4 p0 = pq[0], p1 = pq[1], p2 = pq[2], p3 = pq[3];
            const float o = ((p0.x + p0.y) + (p0.z + p0.w)) + ((p1.x + p1.y) + (p1.z + p1.w)) + ((p2.x + p2.y) + (p2.z + p2.w)) + ((p3.x + p3.y) + (p3.z + p3.w));
            const int tl = idx / kScanCols, c2 = idx % kScanCols;
            if (j0 + c2 < Dv) a.out[(size_t)(tt0 + tl) * a.H * Dv + h * Dv + j0 + c2] = o;
        }
        __syncthreads();       // pS and the buffer of chunk c are free again
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int i = row_of(r), j = j0 + 16 * c + jj;
            if (i < D && j < Dv) st[(size_t)i * Dv + j] = s[r][c];
        }
}

// one warp per (token, head) row of `out`
// (gate != nullptr: the row of head h of token t is also multiplied by silu(gate[t][h * Dv + j]); H heads per token)
static __global__ void __launch_bounds__(256) hgrn2_out_norm_kernel(float* __restrict__ out, const float* __restrict__ norm_w, float eps, int rows, int Dv,
                                                                    const float* __restrict__ gate = nullptr, int gate_ld = 0, int H = 1) {
    const int row = (int)(((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    float* o = out + (size_t)row * Dv;
    float ss = 0.f;
    for (int j = lane; j < Dv; j += 32) ss = fmaf(o[j], o[j], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)Dv + eps);
    if (gate) {
        const float* gr = gate + (size_t)(row / H) * gate_ld + (size_t)(row % H) * Dv;
        for (int j = lane; j < Dv; j += 32) o[j] = o[j] * inv * norm_w[j] * silu_f(gr[j]);
    } else {
        for (int j = lane; j < Dv; j += 32) o[j] = o[j] * inv * norm_w[j];
    }
}

// ---------------------------------------------------------------------------------------------------------------------------------
// Long prompt portions.  The recurrence is linear in the state with a diagonal decay, so an entry can be cut into segments that are
// scanned side by side, each from a zero state (the first from the slot's state).  With A_t[i] = f_{t0}[i] ... f_t[i], the product of
// the gates from the segment's first token t0 to t, and S0 the state before t0,
//     S_t = diag(A_t) S0 + S_t(from zero)      and so      o_t = o_t(from zero) + S0^T (A_t * q_t).
// Products of gates only shrink, so nothing is ever divided by a decay and nothing overflows; a product that underflows to zero is the
// right limit.  Four launches after the gates:
//   hgrn2_scan_reg_kernel       every segment from zero: local outputs, the segment's local end state into scratch
//   hgrn2_seg_decay_kernel      q_t <- A_t * q_t in place (segments after an entry's first), the segment's whole product into scratch
//   hgrn2_seg_combine_kernel    walks an entry's segments in order: scratch <- the state BEFORE the segment, slot <- the end state
//   hgrn2_seg_apply_kernel      out_t += S0^T (A_t * q_t), fp32 on the CUDA cores, a (64 tokens x 64 columns) tile per block
constexpr int kSegLen = 64;         // the shortest segment; segments are a power-of-two multiple of it (and so of kScanChunk)
constexpr int kSegLenMax = 256;
constexpr int kSegMinEntry = 256;   // a step whose longest entry has fewer tokens walks its entries whole

static __global__ void hgrn2_seg_decay_kernel(Hgrn2Args a) {
    const int e = blockIdx.x / a.seg_max, k = blockIdx.x % a.seg_max, h = blockIdx.y, i = threadIdx.x;
    if (k == 0 || k >= hgrn2_seg_count(a.rb, e, a.seg_len) || i >= a.D) return;
    const int HD = a.H * a.D;
    const int t0 = a.rb.ent_start[e] + k * a.seg_len, t1 = min(a.rb.ent_start[e + 1], t0 + a.seg_len);
    float* q = const_cast<float*>(a.qfv) + (size_t)t0 * a.ld + h * a.D + i;
    float prod = 1.f;
    for (int t = t0; t < t1; ++t, q += a.ld) {
        prod *= q[a.f_off];
        q[a.q_off] *= prod;
    }
    a.seg_decay[(size_t)(hgrn2_seg_base(a.rb, e, a.seg_len) + k) * HD + h * a.D + i] = prod;
}

static __global__ void hgrn2_seg_combine_kernel(Hgrn2Args a) {
    const int e = blockIdx.y;
    const size_t n = (size_t)a.H * a.D * a.Dv, idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const int nseg = hgrn2_seg_count(a.rb, e, a.seg_len), base = hgrn2_seg_base(a.rb, e, a.seg_len);
    const size_t row = idx / a.Dv;       // head * D + state row
    float* p = a.seg_state + (size_t)base * n + idx;
    const float* dec = a.seg_decay + (size_t)base * a.H * a.D + row;
    float S = p[0];
    for (int k = 1; k < nseg; k += 8) {      // eight segments' loads ahead of the chain of multiply-adds and the stores
        float loc[8], d[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (k + u < nseg) { loc[u] = p[(size_t)(k + u) * n]; d[u] = dec[(size_t)(k + u) * a.H * a.D]; }
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (k + u < nseg) { p[(size_t)(k + u) * n] = S; S = fmaf(d[u], S, loc[u]); }
    }
    a.state[(size_t)a.rb.ent_slot[e] * a.slot_stride + idx] = S;
}

static __global__ void __launch_bounds__(256) hgrn2_seg_apply_kernel(Hgrn2Args a) {
    __shared__ float Ss[64][64];
    __shared__ __align__(16) float Qs[64][64];
    const int e = blockIdx.x / a.seg_max, k = blockIdx.x % a.seg_max, h = blockIdx.y;
    if (k == 0 || k >= hgrn2_seg_count(a.rb, e, a.seg_len)) return;
    const int D = a.D, Dv = a.Dv, tid = threadIdx.x, tg = tid >> 5, jl = tid & 31, jb = blockIdx.z * 64;
    const int t0 = a.rb.ent_start[e] + k * a.seg_len, t1 = min(a.rb.ent_start[e + 1], t0 + a.seg_len);
    const float* S0 = a.seg_state + ((size_t)(hgrn2_seg_base(a.rb, e, a.seg_len) + k) * a.H + h) * D * Dv;
    for (int tt = t0; tt < t1; tt += 64) {
        float acc[8][2];       // tokens tg * 8 .. + 7, columns jl and jl + 32 of the block's 64
#pragma unroll
        for (int u = 0; u < 8; ++u) acc[u][0] = acc[u][1] = 0.f;
        for (int i0 = 0; i0 < D; i0 += 64) {
            for (int idx = tid; idx < 64 * 64; idx += 256) {
                const int ii = idx >> 6, jc = idx & 63;
                Ss[ii][jc] = (i0 + ii < D && jb + jc < Dv) ? S0[(size_t)(i0 + ii) * Dv + jb + jc] : 0.f;
                Qs[ii][jc] = (tt + ii < t1 && i0 + jc < D) ? a.qfv[(size_t)(tt + ii) * a.ld + a.q_off + h * D + i0 + jc] : 0.f;     // here ii is a token, jc a state row
            }
            __syncthreads();
#pragma unroll 2
            for (int ii = 0; ii < 64; ii += 4) {
                float s0[4], s1[4];
#pragma unroll
                for (int v = 0; v < 4; ++v) { s0[v] = Ss[ii + v][jl]; s1[v] = Ss[ii + v][jl + 32]; }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const float4 q = *reinterpret_cast<const float4*>(&Qs[tg * 8 + u][ii]);
                    acc[u][0] = fmaf(s0[3], q.w, fmaf(s0[2], q.z, fmaf(s0[1], q.y, fmaf(s0[0], q.x, acc[u][0]))));
                    acc[u][1] = fmaf(s1[3], q.w, fmaf(s1[2], q.z, fmaf(s1[1], q.y, fmaf(s1[0], q.x, acc[u][1]))));
                }
            }
            __syncthreads();
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int t = tt + tg * 8 + u;
            if (t < t1) {
                float* o = a.out + (size_t)t * a.H * Dv + h * Dv + jb + jl;
                if (jb + jl < Dv) o[0] += acc[u][0];
                if (jb + jl + 32 < Dv) o[32] += acc[u][1];
            }
        }
    }
}

inline size_t hgrn2_scan_reg_smem(int R, bool keyed) { return ((size_t)2 * kScanChunk * ((keyed ? 3 : 2) * 16 * R + kScanCols) + kScanChunk * kScanCols * kScanPad) * sizeof(float); }

template <int R, bool KEYED>
inline void hgrn2_scan_reg_launch(cudaStream_t st, const Hgrn2Args& a, int vec, int raw) {
    static bool attr = false;
    const size_t smem = hgrn2_scan_reg_smem(R, KEYED);
    if (!attr) { AHA_CUDA_CHECK(cudaFuncSetAttribute(hgrn2_scan_reg_kernel<R, KEYED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); attr = true; }
    hgrn2_scan_reg_kernel<R, KEYED><<<dim3(a.seg_len > 0 ? a.rb.E * a.seg_max : a.rb.E, a.H, (a.Dv + kScanCols - 1) / kScanCols), kScanThreads, smem, st>>>(a, vec, raw);
}

// impl 0: the register kernels (dim <= 256); 1: the plain shared-memory kernel above.  `qfv` is overwritten by the gates (impl 0).  Returns launches.
// With seg_len > 0 (the caller found an entry of at least kSegMinEntry tokens and gives scratch for the step's segments) entries are cut into segments.
inline int hgrn2_scan(cudaStream_t st, const Hgrn2Args& a_in, int impl = 0) {
    if (a_in.rb.E == 0) return 0;
    Hgrn2Args a = a_in;
    if (a.f_off < 0) a.f_off = a.H * a.D;
    if (!a.v) { a.v = a.qfv; a.ld_v = a.ld; a.v_off = 2 * a.H * a.D; }
    AHA_REQUIRE(a.k_off < 0 || a.gates_done, "recurrence: a separate key needs final gates");
    if (impl == 1 || a.D > 256) {
        const int threads = std::min(1024, ((a.Dv + 31) / 32) * 32);
        hgrn2_scan_kernel<<<dim3(a.rb.E, a.H), threads, hgrn2_scan_smem(a.D, a.Dv), st>>>(a);
        AHA_CUDA_CHECK(cudaGetLastError());
        return 1;
    }
    const int HD = a.H * a.D, T = a.rb.T;
    const bool seg = a.seg_len > 0;
    const int raw = (T <= 32 && !seg && !a.gates_done) ? 1 : 0;     // few tokens: every column slice forms the gates itself (one launch less); else once, in place
    if (!raw && !a.gates_done) hgrn2_gates_kernel<<<(unsigned)(((size_t)T * HD + 255) / 256), 256, 0, st>>>(const_cast<float*>(a.qfv), a.ld, a.lower, HD, T);
    const int vec = (a.D % 4 == 0 && a.ld % 4 == 0 && a.q_off % 4 == 0 && a.f_off % 4 == 0 && (a.k_off < 0 || a.k_off % 4 == 0) && (reinterpret_cast<uintptr_t>(a.qfv) & 15) == 0) ? 1 : 0;
    const int R = (a.D + 15) / 16;
    if (a.k_off >= 0) {
        if (R <= 4) hgrn2_scan_reg_launch<4, true>(st, a, vec, raw);
        else if (R <= 8) hgrn2_scan_reg_launch<8, true>(st, a, vec, raw);
        else hgrn2_scan_reg_launch<16, true>(st, a, vec, raw);
    } else {
        if (R <= 4) hgrn2_scan_reg_launch<4, false>(st, a, vec, raw);
        else if (R <= 8) hgrn2_scan_reg_launch<8, false>(st, a, vec, raw);
        else hgrn2_scan_reg_launch<16, false>(st, a, vec, raw);
    }
    if (seg) {
        const unsigned segs = (unsigned)(a.rb.E * a.seg_max);
        hgrn2_seg_decay_kernel<<<dim3(segs, a.H), ((a.D + 31) / 32) * 32, 0, st>>>(a);
        const size_t n = (size_t)a.H * a.D * a.Dv;
        hgrn2_seg_combine_kernel<<<dim3((unsigned)((n + 255) / 256), a.rb.E), 256, 0, st>>>(a);
        hgrn2_seg_apply_kernel<<<dim3(segs, a.H, (a.Dv + 63) / 64), 256, 0, st>>>(a);
    }
    if (a.norm_w) hgrn2_out_norm_kernel<<<(unsigned)(((size_t)T * a.H * 32 + 255) / 256), 256, 0, st>>>(a.out, a.norm_w, a.eps, T * a.H, a.Dv, a.out_gate, a.out_gate_ld, a.H);
    AHA_CUDA_CHECK(cudaGetLastError());
    return 1 + ((raw || a.gates_done) ? 0 : 1) + (a.norm_w ? 1 : 0) + (seg ? 3 : 0);
}

}  // namespace aha
