// hybrid_streams.cu — the residual of designs whose sublayers run in sequence on several residual streams (API: hybrid_kernels.hpp).
//
// Hyper-connections: a row carries n streams x_1..x_n (fp32, [T, n, W]).  A sublayer reads u = sum_s in[s] x_s through its RMS norm and, when
// it has produced y, every stream becomes x_t <- sum_s mix[s, t] x_s + out[t] y — all from the old streams.  hy_stream_norm does the closing
// of one sublayer and the opening of the next in one pass over the row (the new streams never leave the registers between the two), so a
// layer costs two such passes.  n = 1 with in = mix = out = 1 is the plain pre-norm residual.
//
// Token shift: the mixer's normed input v_t is replaced by v_t + (v_(t-1) - v_t) * mu.  v_(t-1) is the unshifted row, so the norm kernel
// leaves v in fp32 and hy_token_shift reads rows t and t - 1; across steps the last v of a sequence lives in its state slot.  The exchange
// with the slot (old row out to `prev`, new row in) is done by the CTA of the sequence's last row, channel by channel by the same thread,
// so no other CTA reads the slot while it changes.
#include "hybrid_common.cuh"
#include "hybrid_kernels.hpp"

namespace oa {

namespace {

using namespace hyk;
using bf = __nv_bfloat16;
constexpr int HY_MAX_STREAMS = 8;

template <typename TA>
__global__ void hy_embed_streams_kernel(const int32_t* __restrict__ ids, const TA* __restrict__ table, float* __restrict__ xs, int W, int vocab, float scale, int n) {
    HY_PDL();
    const long long t = blockIdx.x; int id = ids[t]; id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = ldf(table + (long long)id * W + c) * scale;
        for (int s = 0; s < n; ++s) xs[(t * n + s) * W + c] = v;
    }
}

template <typename TA, int N>       // N: the number of streams (0: any, read at run time)
__global__ void __launch_bounds__(256) hy_stream_norm_kernel(HyStreams cf, float* __restrict__ xs, const float* __restrict__ y, const int32_t* __restrict__ rows,
                                                             const float* __restrict__ w, float eps, TA* __restrict__ h, int ldh, float* __restrict__ hn,
                                                             float* __restrict__ shift_state, float* __restrict__ prev, HyRows r, int W) {
    HY_PDL();
    extern __shared__ float u_s[];          // [W] the sublayer's input before the norm
    __shared__ float red[32];
    __shared__ float c_mix[HY_MAX_STREAMS * HY_MAX_STREAMS], c_out[HY_MAX_STREAMS], c_in[HY_MAX_STREAMS];
    const int n = N ? N : cf.n, t = blockIdx.x;
    if (threadIdx.x < n * n && y) c_mix[threadIdx.x] = cf.upd_mix[threadIdx.x];
    if (threadIdx.x < n) { if (y) c_out[threadIdx.x] = cf.upd_out[threadIdx.x]; c_in[threadIdx.x] = w ? cf.in[threadIdx.x] : 0.f; }
    __syncthreads();
    float* xr = xs + (long long)(rows ? rows[t] : t) * n * W;
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float x[N ? N : HY_MAX_STREAMS];
#pragma unroll
        for (int s = 0; s < (N ? N : HY_MAX_STREAMS); ++s) if (s < n) x[s] = xr[(long long)s * W + c];
        float u = 0.f;
        if (y) {
            const float yv = y[(long long)t * W + c];
#pragma unroll
            for (int to = 0; to < (N ? N : HY_MAX_STREAMS); ++to) {
                if (to >= n) break;
                float v = 0.f;
#pragma unroll
                for (int s = 0; s < (N ? N : HY_MAX_STREAMS); ++s) if (s < n) v = fmaf(c_mix[s * n + to], x[s], v);
                v = fmaf(c_out[to], yv, v);
                xr[(long long)to * W + c] = v;
                u = fmaf(c_in[to], v, u);
            }
        } else {
#pragma unroll
            for (int s = 0; s < (N ? N : HY_MAX_STREAMS); ++s) if (s < n) u = fmaf(c_in[s], x[s], u);
        }
        u_s[c] = u; ss = fmaf(u, u, ss);
    }
    if (!w) return;
    const float rr = 1.0f / sqrtf(block_sum(ss, red) / (float)W + eps);
    if (!shift_state) {
        for (int c = threadIdx.x; c < W; c += blockDim.x) stf(h + (long long)t * ldh + c, u_s[c] * rr * w[c]);
        return;
    }
    const int seq = r.row_seq[t]; const bool last = t + 1 == r.seq_row0[seq + 1];
    float* st = shift_state + (long long)r.seq_state[seq] * W;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = u_s[c] * rr * w[c];
        hn[(long long)t * W + c] = v;
        if (last) { prev[(long long)seq * W + c] = st[c]; st[c] = v; }
    }
}

template <typename TA>
__global__ void __launch_bounds__(256) hy_token_shift_kernel(const float* __restrict__ hn, const float* __restrict__ prev, const float* __restrict__ mu, TA* __restrict__ h, int ldh,
                                                             HyRows r, int W) {
    HY_PDL();
    const int t = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= W) return;
    const int seq = r.row_seq[t];
    const float v = hn[(long long)t * W + c];
    float p = 0.f;
    if (t > r.seq_row0[seq]) p = hn[(long long)(t - 1) * W + c];
    else if (r.seq_pos0[seq] > 0) p = prev[(long long)seq * W + c];
    stf(h + (long long)t * ldh + c, fmaf(p - v, mu[c], v));
}

template <typename TA>
__global__ void __launch_bounds__(128) hy_rmsnorm_act_kernel(const TA* __restrict__ in, int ld_in, int n, const float* __restrict__ w, TA* __restrict__ out, int ld_out, float eps) {
    HY_PDL();
    __shared__ float red[32];
    const long long t = blockIdx.x;
    float ss = 0.f;
    for (int c = threadIdx.x; c < n; c += blockDim.x) { const float v = ldf(in + t * ld_in + c); ss = fmaf(v, v, ss); }
    const float rr = 1.0f / sqrtf(block_sum(ss, red) / (float)n + eps);
    for (int c = threadIdx.x; c < n; c += blockDim.x) stf(out + t * ld_out + c, ldf(in + t * ld_in + c) * rr * w[c]);
}

template <typename TA>
__global__ void hy_sigmoid_gate_kernel(TA* __restrict__ x, int ldx, const TA* __restrict__ g, int ldg, int n) {
    HY_PDL();
    const long long t = blockIdx.y; const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c < n) stf(x + t * ldx + c, ldf(x + t * ldx + c) * sigmoidf_(ldf(g + t * ldg + c)));
}

template <typename TA>
cudaError_t stream_norm_t(const HyStreams& c, float* xs, const float* y, const int32_t* rows, const float* w, float eps, void* h, int ldh, float* hn, float* shift_state, float* prev,
                          const HyRows& r, int T, int W, cudaStream_t s) {
    const size_t smem = (size_t)W * 4;
    auto go = [&](auto kern) -> cudaError_t {
        if (smem > 48 * 1024) { cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); if (e != cudaSuccess) return e; }
        return launch_plain(kern, dim3(T), dim3(256), smem, s, c, xs, y, rows, w, eps, (TA*)h, ldh, hn, shift_state, prev, r, W);
    };
    switch (c.n) {
        case 1: return go(hy_stream_norm_kernel<TA, 1>);
        case 2: return go(hy_stream_norm_kernel<TA, 2>);
        case 4: return go(hy_stream_norm_kernel<TA, 4>);
        default: return go(hy_stream_norm_kernel<TA, 0>);
    }
}

}  // namespace

cudaError_t hy_embed_streams(bool f32, const int32_t* ids, const void* table, float* xs, int T, int W, int vocab, float scale, int n, cudaStream_t s) {
    return f32 ? launch_plain(hy_embed_streams_kernel<float>, dim3(T), dim3(256), 0, s, ids, (const float*)table, xs, W, vocab, scale, n)
               : launch_plain(hy_embed_streams_kernel<bf>, dim3(T), dim3(256), 0, s, ids, (const bf*)table, xs, W, vocab, scale, n);
}
cudaError_t hy_stream_norm(bool f32, const HyStreams& c, float* xs, const float* y, const int32_t* rows, const float* w, float eps, void* h, int ldh, float* hn, float* shift_state,
                           float* prev, const HyRows& r, int T, int W, cudaStream_t s) {
    if (c.n < 1 || c.n > HY_MAX_STREAMS || (size_t)W * 4 > 200 * 1024 || (rows && y) || T <= 0) return cudaErrorInvalidValue;
    return f32 ? stream_norm_t<float>(c, xs, y, rows, w, eps, h, ldh, hn, shift_state, prev, r, T, W, s) : stream_norm_t<bf>(c, xs, y, rows, w, eps, h, ldh, hn, shift_state, prev, r, T, W, s);
}
cudaError_t hy_token_shift(bool f32, const float* hn, const float* prev, const float* mu, void* h, int ldh, const HyRows& r, int W, cudaStream_t s) {
    const dim3 g((W + 255) / 256, r.T);
    return f32 ? launch_plain(hy_token_shift_kernel<float>, g, dim3(256), 0, s, hn, prev, mu, (float*)h, ldh, r, W)
               : launch_plain(hy_token_shift_kernel<bf>, g, dim3(256), 0, s, hn, prev, mu, (bf*)h, ldh, r, W);
}
cudaError_t hy_rmsnorm_act(bool f32, const void* in, int ld_in, int n, const float* w, void* out, int ld_out, float eps, int T, cudaStream_t s) {
    return f32 ? launch_plain(hy_rmsnorm_act_kernel<float>, dim3(T), dim3(128), 0, s, (const float*)in, ld_in, n, w, (float*)out, ld_out, eps)
               : launch_plain(hy_rmsnorm_act_kernel<bf>, dim3(T), dim3(128), 0, s, (const bf*)in, ld_in, n, w, (bf*)out, ld_out, eps);
}
cudaError_t hy_sigmoid_gate(bool f32, void* x, int ldx, const void* g, int ldg, int n, int T, cudaStream_t s) {
    const dim3 grid((n + 255) / 256, T);
    return f32 ? launch_plain(hy_sigmoid_gate_kernel<float>, grid, dim3(256), 0, s, (float*)x, ldx, (const float*)g, ldg, n)
               : launch_plain(hy_sigmoid_gate_kernel<bf>, grid, dim3(256), 0, s, (bf*)x, ldx, (const bf*)g, ldg, n);
}

}  // namespace oa
