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

// The same with the row in registers (W a multiple of 4 up to 8192, 16-byte aligned rows): every input is read once, 16 bytes per access.
// The sums run per thread over its own float4s and then over the block, as in the form above with another assignment of channels to
// threads; a model takes one of the two forms for all of its steps.
__device__ __forceinline__ void st4a(float* p, const float4& v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4a(__nv_bfloat16* p, const float4& v) {
    *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
}
template <typename TA, int NV>      // NV float4 per thread: W <= 1024 NV
__global__ void __launch_bounds__(256) hy_post_norm_reg_kernel(float* __restrict__ x, float beta, const float* __restrict__ y1, const float* __restrict__ rw1,
                                                               const float* __restrict__ y2, const float* __restrict__ rw2, float branch_scale, const float* __restrict__ w,
                                                               TA* __restrict__ h, int ldh, int W, float eps) {
    HY_PDL();
    __shared__ float red[32];
    const long long t = blockIdx.x;
    const int n4 = W / 4;
    float4* xr = reinterpret_cast<float4*>(x + t * W);
    const float4* a = y1 ? reinterpret_cast<const float4*>(y1 + t * W) : nullptr; const float4* b = y2 ? reinterpret_cast<const float4*>(y2 + t * W) : nullptr;
    float4 v[NV];
    if (rw1) {
        float4 u[NV]; float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int i = threadIdx.x + k * 256;
            if (i < n4) { v[k] = a[i]; u[k] = b[i]; s1 += (v[k].x * v[k].x + v[k].y * v[k].y) + (v[k].z * v[k].z + v[k].w * v[k].w); s2 += (u[k].x * u[k].x + u[k].y * u[k].y) + (u[k].z * u[k].z + u[k].w * u[k].w); }
        }
        const float r1 = branch_scale / sqrtf(block_sum(s1, red) / (float)W + eps), r2 = branch_scale / sqrtf(block_sum(s2, red) / (float)W + eps);
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int i = threadIdx.x + k * 256;
            if (i < n4) {
                const float4 g1 = reinterpret_cast<const float4*>(rw1)[i], g2 = reinterpret_cast<const float4*>(rw2)[i], xv = xr[i];
                v[k].x = fmaf(beta, xv.x, v[k].x * r1 * g1.x + u[k].x * r2 * g2.x); v[k].y = fmaf(beta, xv.y, v[k].y * r1 * g1.y + u[k].y * r2 * g2.y);
                v[k].z = fmaf(beta, xv.z, v[k].z * r1 * g1.z + u[k].z * r2 * g2.z); v[k].w = fmaf(beta, xv.w, v[k].w * r1 * g1.w + u[k].w * r2 * g2.w);
            }
        }
    } else {
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int i = threadIdx.x + k * 256;
            if (i < n4) {
                const float4 xv = xr[i]; const float4 yv = a ? a[i] : make_float4(0.f, 0.f, 0.f, 0.f);
                v[k] = make_float4(fmaf(beta, xv.x, yv.x), fmaf(beta, xv.y, yv.y), fmaf(beta, xv.z, yv.z), fmaf(beta, xv.w, yv.w));
            }
        }
    }
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) if (threadIdx.x + k * 256 < n4) s += (v[k].x + v[k].y) + (v[k].z + v[k].w);
    const float mean = block_sum(s, red) / (float)W;
    float q = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) if (threadIdx.x + k * 256 < n4) { const float c0 = v[k].x - mean, c1 = v[k].y - mean, c2 = v[k].z - mean, c3 = v[k].w - mean; q += (c0 * c0 + c1 * c1) + (c2 * c2 + c3 * c3); }
    const float rstd = 1.0f / sqrtf(block_sum(q, red) / (float)W + eps);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = threadIdx.x + k * 256;
        if (i < n4) {
            const float4 g = reinterpret_cast<const float4*>(w)[i];
            const float4 o = make_float4((v[k].x - mean) * rstd * g.x, (v[k].y - mean) * rstd * g.y, (v[k].z - mean) * rstd * g.z, (v[k].w - mean) * rstd * g.w);
            xr[i] = o;
            if (h) st4a(h + t * ldh + 4 * i, o);
        }
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

// The same for bf16 rows whose heads come in aligned groups of 8 channels (dim, vdim, rot_dims / 2 multiples of 8): a thread owns 8 channels,
// every access is 16 bytes wide.  k_gate (matrix memory): k is multiplied by k_gate[t, head].  Per element the arithmetic is that of the
// kernels above and below: the same bits.
__device__ __forceinline__ void unpack8(const uint4& r, float* f) {
    f[0] = bf16lo(r.x); f[1] = bf16hi(r.x); f[2] = bf16lo(r.y); f[3] = bf16hi(r.y); f[4] = bf16lo(r.z); f[5] = bf16hi(r.z); f[6] = bf16lo(r.w); f[7] = bf16hi(r.w);
}
__device__ __forceinline__ void ld8f(const float* p, float* f) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ void st8f(float* p, const float* f) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]); *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
}
__global__ void __launch_bounds__(128) hy_lin_prep_vec8_kernel(HyLinPrep p, const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                                               int ld, float* __restrict__ qq, float* __restrict__ kk, float* __restrict__ vv, float* __restrict__ dec_channel,
                                                               float inv_tau, const float* __restrict__ decay_head, float* __restrict__ dec_head, const float* __restrict__ rope_cos,
                                                               const float* __restrict__ rope_sin, const float* __restrict__ k_gate, HyRows r) {
    HY_PDL();
    const long long t = blockIdx.x;
    const int H = p.heads, D = p.dim, VD = p.vdim, half = p.rot_dims / 2, pos = p.rot_dims > 0 ? r.positions[t] : 0;
    const float sc = rsqrtf((float)D), qs = p.q_scaled ? sc : 1.f, ks = p.k_scaled ? sc : 1.f;
    const __nv_bfloat16* qr = q + t * ld; const __nv_bfloat16* kr = k + t * ld;
    const int nqk = H * D / 8, nv = H * VD / 8;
    for (int it = threadIdx.x; it < nqk + nv; it += blockDim.x) {
        if (it >= nqk) {
            const int i = (it - nqk) * 8; float f[8];
            unpack8(*reinterpret_cast<const uint4*>(v + t * ld + i), f);
            st8f(vv + t * H * VD + i, f);
            continue;
        }
        const int i = it * 8, d = i % D;
        float a[8], b[8];
        unpack8(*reinterpret_cast<const uint4*>(qr + i), a); unpack8(*reinterpret_cast<const uint4*>(kr + i), b);
        if (d < p.rot_dims) {
            const bool lo = d < half; const int j = lo ? d : d - half, o = lo ? i + half : i - half;
            float ao[8], bo[8], c[8], sn[8];
            unpack8(*reinterpret_cast<const uint4*>(qr + o), ao); unpack8(*reinterpret_cast<const uint4*>(kr + o), bo);
            ld8f(rope_cos + (long long)pos * half + j, c); ld8f(rope_sin + (long long)pos * half + j, sn);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                a[e] = lo ? a[e] * c[e] - ao[e] * sn[e] : a[e] * c[e] + ao[e] * sn[e];
                b[e] = lo ? b[e] * c[e] - bo[e] * sn[e] : b[e] * c[e] + bo[e] * sn[e];
            }
        }
        const float kg = k_gate ? k_gate[t * H + i / D] : ks;
#pragma unroll
        for (int e = 0; e < 8; ++e) { a[e] *= qs; b[e] *= kg; }
        st8f(qq + t * H * D + i, a); st8f(kk + t * H * D + i, b);
        if (dec_channel) {
            float z[8]; ld8f(dec_channel + t * H * D + i, z);
#pragma unroll
            for (int e = 0; e < 8; ++e) z[e] = expf(log_sigmoidf_(z[e]) * inv_tau);
            st8f(dec_channel + t * H * D + i, z);
        }
    }
    if (dec_head) for (int i = threadIdx.x; i < H; i += blockDim.x) dec_head[t * H + i] = decay_head[i];
}
static bool lin_vec8_ok(bool f32, int dim, int vdim, int half, int ld, const void* q, const void* k, const void* v, const float* qq, const float* kk, const float* vv, const float* dec,
                        const float* rc, const float* rs) {
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    return !f32 && dim % 8 == 0 && vdim % 8 == 0 && half % 8 == 0 && ld % 8 == 0 && al(q) && al(k) && al(v) && al(qq) && al(kk) && al(vv) && al(dec) && al(rc) && al(rs);
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
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (W % 4 == 0 && W <= 8192 && ldh % 4 == 0 && al(x) && al(y1) && al(y2) && al(rw1) && al(rw2) && al(w) && al(h))      // by the model's sizes alone, never by the step
    {
#define HY_PN(NV) (f32 ? launch_plain(hy_post_norm_reg_kernel<float, NV>, dim3(T), dim3(256), 0, s, x, beta, y1, rw1, y2, rw2, branch_scale, w, (float*)h, ldh, W, eps) \
                       : launch_plain(hy_post_norm_reg_kernel<__nv_bfloat16, NV>, dim3(T), dim3(256), 0, s, x, beta, y1, rw1, y2, rw2, branch_scale, w, (__nv_bfloat16*)h, ldh, W, eps))
        return W <= 1024 ? HY_PN(1) : W <= 2048 ? HY_PN(2) : W <= 4096 ? HY_PN(4) : HY_PN(8);
#undef HY_PN
    }
    return f32 ? launch_plain(hy_post_norm_kernel<float>, dim3(T), dim3(256), 0, s, x, beta, y1, rw1, y2, rw2, branch_scale, w, (float*)h, ldh, W, eps)
               : launch_plain(hy_post_norm_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, s, x, beta, y1, rw1, y2, rw2, branch_scale, w, (__nv_bfloat16*)h, ldh, W, eps);
}

cudaError_t hy_lin_prep(bool f32, const HyLinPrep& p, const void* q, const void* k, const void* v, int ld, float* qq, float* kk, float* vv, float* dec_channel, float tau,
                        const float* decay_head, float* dec_head, const float* rope_cos, const float* rope_sin, const HyRows& r, cudaStream_t s) {
    if (r.T <= 0) return cudaSuccess;
    if (p.rot_dims > 0 && (!rope_cos || !rope_sin || (p.rot_dims & 1) || p.rot_dims > p.dim)) return cudaErrorInvalidValue;
    using bf = __nv_bfloat16;
    if (lin_vec8_ok(f32, p.dim, p.vdim, p.rot_dims / 2, ld, q, k, v, qq, kk, vv, dec_channel, rope_cos, rope_sin))      // by the model's sizes alone
        return launch_plain(hy_lin_prep_vec8_kernel, dim3(r.T), dim3(128), 0, s, p, (const bf*)q, (const bf*)k, (const bf*)v, ld, qq, kk, vv, dec_channel, 1.0f / tau, decay_head,
                            dec_head, rope_cos, rope_sin, (const float*)nullptr, r);
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
    if (lin_vec8_ok(f32, dim, vdim, 0, ld, q, k, v, qq, kk, vv, nullptr, nullptr, nullptr)) {
        HyRows r{}; r.T = T;                      // nothing is rotated: the kernel does not look at the rows' positions
        return launch_plain(hy_lin_prep_vec8_kernel, dim3(T), dim3(128), 0, s, HyLinPrep{heads, dim, vdim, true, false, 0}, (const bf*)q, (const bf*)k,
                            (const bf*)v, ld, qq, kk, vv, (float*)nullptr, 1.f, (const float*)nullptr, (float*)nullptr, (const float*)nullptr, (const float*)nullptr, gin, r);
    }
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
