// ssm.cuh -- the gate arithmetic that turns projections into the operands of the keyed linear recurrence (recurrence.cuh), fp32:
//
//   gla_gates_kernel     gated linear attention: q <- q * qscale, decay <- sigmoid(z)^(1 / tau) = exp(-softplus(-z) / tau), in place
//   mamba2_gates_kernel  selective state space (Mamba-2): per token and head, dt = softplus(dt_raw + dt_bias) (no clamp),
//                        decay = exp(-exp(A_log) dt) for every state channel, key = dt * B, query = C, with B and C of the head's group
//                        (head h reads group h / (heads / groups)); written head by head so that the scan sees the usual layout
#pragma once
#include "common.cuh"

namespace aha {

__device__ __forceinline__ float softplus_f(float x) { return log1pf(expf(-fabsf(x))) + fmaxf(x, 0.f); }

static __global__ void gla_gates_kernel(float* __restrict__ rows, int ld, int q_off, int z_off, int HD, float qscale, float inv_tau, size_t total) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    float* row = rows + (idx / HD) * ld;
    const int c = (int)(idx % HD);
    row[q_off + c] *= qscale;
    row[z_off + c] = expf(-softplus_f(-row[z_off + c]) * inv_tau);
}

struct Mamba2GateArgs {
    const float* dt_raw; int ld_dt;          // [T, .] column h
    const float* bc; int ld_bc; int b_off, c_off;   // convolved, activated B and C: [T, .] columns b_off + g * N + i, c_off + g * N + i
    const float *dt_bias, *a_log;            // [H]
    float* out; int ld_out; int q_off, f_off, k_off;   // [T, .] head by head: q | decay | key, N channels a head
    int H, G, N, T;
};

static __global__ void mamba2_gates_kernel(Mamba2GateArgs a) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int HN = a.H * a.N;
    if (idx >= (size_t)a.T * HN) return;
    const size_t t = idx / HN;
    const int c = (int)(idx % HN), h = c / a.N, i = c % a.N, g = h / (a.H / a.G);
    const float dt = softplus_f(a.dt_raw[t * a.ld_dt + h] + a.dt_bias[h]);
    const float* bc = a.bc + t * a.ld_bc;
    float* o = a.out + t * a.ld_out;
    o[a.q_off + c] = bc[a.c_off + g * a.N + i];
    o[a.f_off + c] = expf(-expf(a.a_log[h]) * dt);
    o[a.k_off + c] = dt * bc[a.b_off + g * a.N + i];
}

}  // namespace aha
