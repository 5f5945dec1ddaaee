// hybrid_linear.cu — kernels around the linear-attention recurrences of the hybrid decoder family (API: hybrid_kernels.hpp): operands of
// gated linear attention (a decay per key channel), retention (a fixed decay per head, rotate-half rotary) and the xLSTM matrix memory (log
// gates, running maximum, normaliser); the norm after the sum that closes a sublayer of a post-norm design; the router that reads a token's
// experts from a table.  The recurrences themselves are hy_recurrence (hybrid_kernels.cu).  Everything here is fp32 arithmetic; TA is the
// element type of projection outputs and of the rows handed to the next matrix product.
#include "hybrid_common.cuh"
#include "hybrid_kernels.hpp"

namespace oa {

namespace {

using namespace hyk;

__device__ __forceinline__ float log_sigmoidf_(float z) { return z >= 0.f ? -log1pf(expf(-z)) : z - log1pf(expf(z)); }

// ---------------------------------------------------------------------------------------------------------------------------------
// norm after the sum
// ---------------------------------------------------------------------------------------------------------------------------------
template <typename TA>
__global__ void __launch_bounds__(256) hy_post_norm_kernel(float* __restrict__ x, float beta, const float* __restrict__ y1, const float* __restrict__ rw1,
                                                           const float* __restrict__ y2, const float* __restrict__ rw2, float branch_scale, const float* __restrict__ w,
                                                           TA* __restrict__ h, int ldh, int W, float eps) {
    HY_PDL();
    __shared__ float red[32];
    const long long t = blockIdx.x;
    float* xr = x + t * W; const float* a = y1 ? y1 + t * W : nullptr; const float* b = y2 ? y2 + t * W : nullptr;
    float r1 = 1.f, r2 = 1.f;
    if (rw1) {                                   // two sublayers side by side: each output RMS-normed over the width
        float s1 = 0.f, s2 = 0.f;
        for (int c = threadIdx.x; c < W; c += blockDim.x) { s1 = fmaf(a[c], a[c], s1); s2 = fmaf(b[c], b[c], s2); }
        r1 = 1.0f / sqrtf(block_sum(s1, red) / (float)W + eps); r2 = 1.0f / sqrtf(block_sum(s2, red) / (float)W + eps);
    }
    auto val = [&](int c) -> float {
        float v = beta * xr[c];
        if (rw1) v += branch_scale * (a[c] * r1 * rw1[c] + b[c] * r2 * rw2[c]);
        else if (a) v += a[c];
        return v;
    };
    float s = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) s += val(c);
    const float mean = block_sum(s, red) / (float)W;
    float q = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) { const float d = val(c) - mean; q = fmaf(d, d, q); }
    const float rstd = 1.0f / sqrtf(block_sum(q, red) / (float)W + eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x) {          // a thread rewrites only what it alone has read
        const float o = (val(c) - mean) * rstd * w[c];
        xr[c] = o;
        if (h) stf(h + t * ldh + c, o);
    }
}

// ---------------------------------------------------------------------------------------------------------------------------------
// operands of the recurrences
// ---------------------------------------------------------------------------------------------------------------------------------
template <typename TA>
__global__ void __launch_bounds__(128) hy_lin_prep_kernel(HyLinPrep p, const TA* __restrict__ q, const TA* __restrict__ k, const TA* __restrict__ v, int ld,
                                                          float* __restrict__ qq, float* __restrict__ kk, float* __restrict__ vv, float* __restrict__ dec_channel, float inv_tau,
                                                          const float* __restrict__ decay_head, float* __restrict__ dec_head, const float* __restrict__ rope_cos,
                                                          const float* __restrict__ rope_sin, HyRows r) {
    HY_PDL();
    const long long t = blockIdx.x;
    const int H = p.heads, D = p.dim, VD = p.vdim, half = p.rot_dims / 2, pos = r.positions[t];
    const float sc = rsqrtf((float)D), qs = p.q_scaled ? sc : 1.f, ks = p.k_scaled ? sc : 1.f;
    const TA* qr = q + t * ld; const TA* kr = k + t * ld;
    for (int i = threadIdx.x; i < H * D; i += blockDim.x) {
        const int d = i % D;
        float a = ldf(qr + i), b = ldf(kr + i);
        if (d < p.rot_dims) {                    // channel d pairs with d + half: (u, v) -> (u cos - v sin, v cos + u sin)
            const bool lo = d < half; const int j = lo ? d : d - half;
            const float c = rope_cos[(long long)pos * half + j], s = rope_sin[(long long)pos * half + j];
            const float ao = ldf(qr + (lo ? i + half : i - half)), bo = ldf(kr + (lo ? i + half : i - half));
            a = lo ? a * c - ao * s : a * c + ao * s;
            b = lo ? b * c - bo * s : b * c + bo * s;
        }
        qq[t * H * D + i] = a * qs; kk[t * H * D + i] = b * ks;
        if (dec_channel) dec_channel[t * H * D + i] = expf(log_sigmoidf_(dec_channel[t * H * D + i]) * inv_tau);
    }
    for (int i = threadIdx.x; i < H * VD; i += blockDim.x) vv[t * H * VD + i] = ldf(v + t * ld + i);
    if (dec_head) for (int i = threadIdx.x; i < H; i += blockDim.x) dec_head[t * H + i] = decay_head[i];
}

// Gates of the matrix memory, one CTA per (sequence, head).  Every thread owns a run of consecutive rows.  Pass 1: log gates
// i = cap tanh(z_i / cap), f = logsigmoid(cap tanh(z_f / cap)) and the run's effect on the running maximum as a pair (A, B): m_out =
// max(m_in + A, B) with A = sum of f and B = the maximum reached from minus infinity (the update m <- max(m + f, i) composes that way).
// One thread chains the runs' pairs from the carried maximum; pass 2 walks each run again from its incoming maximum and writes
// dec = exp(f + m_(t-1) - m_t), gin = exp(i - m_t), floor_ = exp(-m_t).  The last row of a run takes the chained value as its maximum, so
// that the next run starts from exactly the number this one ended with: the maximum is only a stabiliser (state, normaliser and floor
// all carry exp(-m_t)), what matters is that every row divides by the same number the next row multiplies with.
constexpr int MLSTM_SCAN_THREADS = 128;
__global__ void __launch_bounds__(MLSTM_SCAN_THREADS) hy_mlstm_gates_kernel(const float* __restrict__ gates, int ldg, int H, float cap, float* __restrict__ mstate,
                                                                            float* __restrict__ dec, float* __restrict__ gin, float* __restrict__ floor_, HyRows r) {
    HY_PDL();
    __shared__ float sA[MLSTM_SCAN_THREADS], sB[MLSTM_SCAN_THREADS], sM[MLSTM_SCAN_THREADS + 1];
    const int seq = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int row0 = r.seq_row0[seq], len = r.seq_row0[seq + 1] - row0, pos0 = r.seq_pos0[seq];
    const int per = (len + MLSTM_SCAN_THREADS - 1) / MLSTM_SCAN_THREADS, t0 = min(len, tid * per), t1 = min(len, t0 + per);
    const float inv_cap = 1.0f / cap;
    float A = 0.f, B = -INFINITY;
    for (int t = t0; t < t1; ++t) {
        const long long row = row0 + t;
        const float i = cap * tanhf(gates[row * ldg + h] * inv_cap), f = log_sigmoidf_(cap * tanhf(gates[row * ldg + H + h] * inv_cap));
        gin[row * H + h] = i; dec[row * H + h] = f;
        A += f; B = fmaxf(B + f, i);
    }
    sA[tid] = A; sB[tid] = B;
    __syncthreads();
    if (tid == 0) {
        float* ms = mstate + (long long)r.seq_state[seq] * H + h;
        float m = pos0 > 0 ? *ms : 0.f;                    // a sequence that starts in this step starts from 0
        for (int j = 0; j < MLSTM_SCAN_THREADS; ++j) { sM[j] = m; m = fmaxf(m + sA[j], sB[j]); }
        sM[MLSTM_SCAN_THREADS] = m; *ms = m;
    }
    __syncthreads();
    float m = sM[tid];
    for (int t = t0; t < t1; ++t) {
        const long long at = (long long)(row0 + t) * H + h;
        const float f = dec[at], i = gin[at];
        const float mn = t == t1 - 1 ? sM[tid + 1] : fmaxf(f + m, i);
        dec[at] = expf(f + m - mn); gin[at] = expf(i - mn); floor_[at] = expf(-mn);
        m = mn;
    }
}
template <typename TA>
__global__ void __launch_bounds__(128) hy_mlstm_prep_kernel(int H, int D, int VD, const TA* __restrict__ q, const TA* __restrict__ k, const TA* __restrict__ v, int ld,
                                                            const float* __restrict__ gin, float* __restrict__ qq, float* __restrict__ kk, float* __restrict__ vv) {
    HY_PDL();
    const long long t = blockIdx.x;
    const float sc = rsqrtf((float)D);
    for (int i = threadIdx.x; i < H * D; i += blockDim.x) { qq[t * H * D + i] = ldf(q + t * ld + i) * sc; kk[t * H * D + i] = ldf(k + t * ld + i) * gin[t * H + i / D]; }
    for (int i = threadIdx.x; i < H * VD; i += blockDim.x) vv[t * H * VD + i] = ldf(v + t * ld + i);
}

// ---------------------------------------------------------------------------------------------------------------------------------
// router by table: one warp per token
// ---------------------------------------------------------------------------------------------------------------------------------
template <typename TA>
__global__ void __launch_bounds__(128) hy_moe_router_table_kernel(const int32_t* __restrict__ tokens, const int32_t* __restrict__ table, int vocab, int top, int shared,
                                                                  const TA* __restrict__ h, int ldh, const TA* __restrict__ w_sg, int W, int32_t* __restrict__ idx,
                                                                  float* __restrict__ wgt, int T) {
    HY_PDL();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = blockIdx.x * 4 + warp;
    if (t >= T) return;
    const int n = top + (shared >= 0 ? 1 : 0);
    int id = tokens[t]; id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    if (lane < top) { idx[(long long)t * n + lane] = table[(long long)id * top + lane]; wgt[(long long)t * n + lane] = 1.0f / (float)top; }
    if (shared >= 0) {
        float d = 0.f;
        for (int c = lane; c < W; c += 32) d = fmaf(ldf(h + (long long)t * ldh + c), ldf(w_sg + c), d);
        d = warp_sum(d);
        if (lane == 0) { idx[(long long)t * n + top] = shared; wgt[(long long)t * n + top] = sigmoidf_(d); }
    }
}

}  // namespace

cudaError_t hy_post_norm(bool f32, float* x, float beta, const float* y1, const float* rw1, const float* y2, const float* rw2, float branch_scale, const float* w, void* h, int ldh,
                         int T, int W, float eps, cudaStream_t s) {
    if (T <= 0) return cudaSuccess;
    if (rw1 && (!y1 || !y2 || !rw2)) return cudaErrorInvalidValue;
    return f32 ? launch_plain(hy_post_norm_kernel<float>, dim3(T), dim3(256), 0, s, x, beta, y1, rw1, y2, rw2, branch_scale, w, (float*)h, ldh, W, eps)
               : launch_plain(hy_post_norm_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, s, x, beta, y1, rw1, y2, rw2, branch_scale, w, (__nv_bfloat16*)h, ldh, W, eps);
}

cudaError_t hy_lin_prep(bool f32, const HyLinPrep& p, const void* q, const void* k, const void* v, int ld, float* qq, float* kk, float* vv, float* dec_channel, float tau,
                        const float* decay_head, float* dec_head, const float* rope_cos, const float* rope_sin, const HyRows& r, cudaStream_t s) {
    if (r.T <= 0) return cudaSuccess;
    if (p.rot_dims > 0 && (!rope_cos || !rope_sin || (p.rot_dims & 1) || p.rot_dims > p.dim)) return cudaErrorInvalidValue;
    using bf = __nv_bfloat16;
    return f32 ? launch_plain(hy_lin_prep_kernel<float>, dim3(r.T), dim3(128), 0, s, p, (const float*)q, (const float*)k, (const float*)v, ld, qq, kk, vv, dec_channel, 1.0f / tau,
                              decay_head, dec_head, rope_cos, rope_sin, r)
               : launch_plain(hy_lin_prep_kernel<bf>, dim3(r.T), dim3(128), 0, s, p, (const bf*)q, (const bf*)k, (const bf*)v, ld, qq, kk, vv, dec_channel, 1.0f / tau, decay_head,
                              dec_head, rope_cos, rope_sin, r);
}

cudaError_t hy_mlstm_gates(const float* gates, int ldg, int heads, float cap, float* mstate, float* dec, float* gin, float* floor_, const HyRows& r, cudaStream_t s) {
    if (r.T <= 0) return cudaSuccess;
    return launch_plain(hy_mlstm_gates_kernel, dim3(r.S, heads), dim3(MLSTM_SCAN_THREADS), 0, s, gates, ldg, heads, cap, mstate, dec, gin, floor_, r);
}

cudaError_t hy_mlstm_prep(bool f32, int heads, int dim, int vdim, const void* q, const void* k, const void* v, int ld, const float* gin, float* qq, float* kk, float* vv, int T,
                          cudaStream_t s) {
    if (T <= 0) return cudaSuccess;
    using bf = __nv_bfloat16;
    return f32 ? launch_plain(hy_mlstm_prep_kernel<float>, dim3(T), dim3(128), 0, s, heads, dim, vdim, (const float*)q, (const float*)k, (const float*)v, ld, gin, qq, kk, vv)
               : launch_plain(hy_mlstm_prep_kernel<bf>, dim3(T), dim3(128), 0, s, heads, dim, vdim, (const bf*)q, (const bf*)k, (const bf*)v, ld, gin, qq, kk, vv);
}

cudaError_t hy_moe_router_table(bool f32, const int32_t* tokens, const int32_t* table, int vocab, int top, int shared, const void* h, int ldh, const void* w_sg, int W,
                                int32_t* idx, float* wgt, int T, cudaStream_t s) {
    if (T <= 0) return cudaSuccess;
    if (top < 1 || top + (shared >= 0 ? 1 : 0) > 32) return cudaErrorInvalidValue;
    using bf = __nv_bfloat16;
    return f32 ? launch_plain(hy_moe_router_table_kernel<float>, dim3((T + 3) / 4), dim3(128), 0, s, tokens, table, vocab, top, shared, (const float*)h, ldh, (const float*)w_sg, W, idx, wgt, T)
               : launch_plain(hy_moe_router_table_kernel<bf>, dim3((T + 3) / 4), dim3(128), 0, s, tokens, table, vocab, top, shared, (const bf*)h, ldh, (const bf*)w_sg, W, idx, wgt, T);
}

}  // namespace oa
