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

// V channels per thread and access (4: 16-byte loads and stores of the fp32 streams; 1: any width)
template <int V> struct FVec;
template <> struct FVec<1> { float v[1]; __device__ __forceinline__ void load(const float* p) { v[0] = *p; } __device__ __forceinline__ void store(float* p) const { *p = v[0]; } };
template <> struct FVec<4> {
    float v[4];
    __device__ __forceinline__ void load(const float* p) { const float4 t = *reinterpret_cast<const float4*>(p); v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w; }
    __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <int V> __device__ __forceinline__ void store_act(float* p, const float* v) { FVec<V> t; for (int e = 0; e < V; ++e) t.v[e] = v[e]; t.store(p); }
template <int V> __device__ __forceinline__ void store_act(bf* p, const float* v) {
    if (V == 4) *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]));
    else p[0] = __float2bfloat16_rn(v[0]);
}

template <typename TA, int N, int V>       // N: the number of streams (0: any, read at run time)
__global__ void __launch_bounds__(256) hy_stream_norm_kernel(HyStreams cf, float* __restrict__ xs, const float* __restrict__ y, const int32_t* __restrict__ rows,
                                                             const float* __restrict__ w, float eps, TA* __restrict__ h, int ldh, float* __restrict__ hn,
                                                             float* __restrict__ shift_state, float* __restrict__ prev, HyRows r, int W) {
    HY_PDL();
    extern __shared__ __align__(16) float u_s[];          // [W] the sublayer's input before the norm
    __shared__ float red[32];
    __shared__ float c_mix[HY_MAX_STREAMS * HY_MAX_STREAMS], c_out[HY_MAX_STREAMS], c_in[HY_MAX_STREAMS];
    constexpr int NMAX = N ? N : HY_MAX_STREAMS;
    const int n = N ? N : cf.n, t = blockIdx.x;
    if (threadIdx.x < n * n && y) c_mix[threadIdx.x] = cf.upd_mix[threadIdx.x];
    if (threadIdx.x < n) { if (y) c_out[threadIdx.x] = cf.upd_out[threadIdx.x]; c_in[threadIdx.x] = w ? cf.in[threadIdx.x] : 0.f; }
    __syncthreads();
    const long long src = rows ? rows[t] : t;
    float* xr = xs + src * n * W;
    float ss = 0.f;
    for (int c = threadIdx.x * V; c < W; c += blockDim.x * V) {
        FVec<V> x[NMAX], u;
#pragma unroll
        for (int s = 0; s < NMAX; ++s) if (s < n) x[s].load(xr + (long long)s * W + c);
#pragma unroll
        for (int e = 0; e < V; ++e) u.v[e] = 0.f;
        if (y) {
            FVec<V> yv; yv.load(y + src * W + c);
#pragma unroll
            for (int to = 0; to < NMAX; ++to) {
                if (to >= n) break;
                FVec<V> nv;
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    float a = 0.f;
#pragma unroll
                    for (int s = 0; s < NMAX; ++s) if (s < n) a = fmaf(c_mix[s * n + to], x[s].v[e], a);
                    nv.v[e] = fmaf(c_out[to], yv.v[e], a);
                    u.v[e] = fmaf(c_in[to], nv.v[e], u.v[e]);
                }
                if (!rows) nv.store(xr + (long long)to * W + c);         // rows given: only the wanted rows' norm is asked for, the streams stay
            }
        } else {
#pragma unroll
            for (int s = 0; s < NMAX; ++s) if (s < n)
#pragma unroll
                for (int e = 0; e < V; ++e) u.v[e] = fmaf(c_in[s], x[s].v[e], u.v[e]);
        }
        u.store(u_s + c);
#pragma unroll
        for (int e = 0; e < V; ++e) ss = fmaf(u.v[e], u.v[e], ss);
    }
    if (!w) return;
    const float rr = 1.0f / sqrtf(block_sum(ss, red) / (float)W + eps);
    const int seq = shift_state ? r.row_seq[t] : 0; const bool last = shift_state && t + 1 == r.seq_row0[seq + 1];
    float* st = shift_state ? shift_state + (long long)r.seq_state[seq] * W : nullptr;
    for (int c = threadIdx.x * V; c < W; c += blockDim.x * V) {
        FVec<V> u, wv; u.load(u_s + c); wv.load(w + c);
        float v[V];
#pragma unroll
        for (int e = 0; e < V; ++e) v[e] = u.v[e] * rr * wv.v[e];
        if (!shift_state) { store_act<V>(h + (long long)t * ldh + c, v); continue; }
        store_act<V>(hn + (long long)t * W + c, v);
        if (last) { FVec<V> old; old.load(st + c); old.store(prev + (long long)seq * W + c); store_act<V>(st + c, v); }
    }
}

template <typename TA, int V>
__global__ void __launch_bounds__(256) hy_token_shift_kernel(const float* __restrict__ hn, const float* __restrict__ prev, const float* __restrict__ mu, TA* __restrict__ h, int ldh,
                                                             HyRows r, int W) {
    HY_PDL();
    const int t = blockIdx.y, c = (blockIdx.x * blockDim.x + threadIdx.x) * V;
    if (c >= W) return;
    const int seq = r.row_seq[t];
    FVec<V> v, p, m; v.load(hn + (long long)t * W + c); m.load(mu + c);
    if (t > r.seq_row0[seq]) p.load(hn + (long long)(t - 1) * W + c);
    else if (r.seq_pos0[seq] > 0) p.load(prev + (long long)seq * W + c);
    else for (int e = 0; e < V; ++e) p.v[e] = 0.f;
    float o[V];
#pragma unroll
    for (int e = 0; e < V; ++e) o[e] = fmaf(p.v[e] - v.v[e], m.v[e], v.v[e]);
    store_act<V>(h + (long long)t * ldh + c, o);
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
// bf16 rows in aligned groups of 8 channels: 16 bytes per access
__global__ void hy_sigmoid_gate_vec8_kernel(bf* __restrict__ x, int ldx, const bf* __restrict__ g, int ldg, int n) {
    HY_PDL();
    const long long t = blockIdx.y; const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= n) return;
    uint4 xv = *reinterpret_cast<const uint4*>(x + t * ldx + c); const uint4 gv = *reinterpret_cast<const uint4*>(g + t * ldg + c);
    auto two = [](uint32_t a, uint32_t b) { return pack_bf16x2(bf16lo(a) * sigmoidf_(bf16lo(b)), bf16hi(a) * sigmoidf_(bf16hi(b))); };
    xv.x = two(xv.x, gv.x); xv.y = two(xv.y, gv.y); xv.z = two(xv.z, gv.z); xv.w = two(xv.w, gv.w);
    *reinterpret_cast<uint4*>(x + t * ldx + c) = xv;
}

template <typename TA>
cudaError_t stream_norm_t(const HyStreams& c, float* xs, const float* y, const int32_t* rows, const float* w, float eps, void* h, int ldh, float* hn, float* shift_state, float* prev,
                          const HyRows& r, int T, int W, cudaStream_t s) {
    const size_t smem = (size_t)W * 4;
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const bool v4 = W % 4 == 0 && ldh % 4 == 0 && al16(xs) && al16(y) && al16(w) && al16(h) && al16(hn) && al16(shift_state) && al16(prev);
    auto go = [&](auto kern) -> cudaError_t {
        if (smem > 48 * 1024) { cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); if (e != cudaSuccess) return e; }
        return launch_plain(kern, dim3(T), dim3(256), smem, s, c, xs, y, rows, w, eps, (TA*)h, ldh, hn, shift_state, prev, r, W);
    };
    // the vector width follows from the model's sizes alone, so a row takes the same kernel in every step
    if (v4) switch (c.n) {
        case 1: return go(hy_stream_norm_kernel<TA, 1, 4>);
        case 2: return go(hy_stream_norm_kernel<TA, 2, 4>);
        case 4: return go(hy_stream_norm_kernel<TA, 4, 4>);
        default: return go(hy_stream_norm_kernel<TA, 0, 1>);
    }
    switch (c.n) {
        case 1: return go(hy_stream_norm_kernel<TA, 1, 1>);
        case 2: return go(hy_stream_norm_kernel<TA, 2, 1>);
        case 4: return go(hy_stream_norm_kernel<TA, 4, 1>);
        default: return go(hy_stream_norm_kernel<TA, 0, 1>);
    }
}

}  // namespace

cudaError_t hy_embed_streams(bool f32, const int32_t* ids, const void* table, float* xs, int T, int W, int vocab, float scale, int n, cudaStream_t s) {
    return f32 ? launch_plain(hy_embed_streams_kernel<float>, dim3(T), dim3(256), 0, s, ids, (const float*)table, xs, W, vocab, scale, n)
               : launch_plain(hy_embed_streams_kernel<bf>, dim3(T), dim3(256), 0, s, ids, (const bf*)table, xs, W, vocab, scale, n);
}
cudaError_t hy_stream_norm(bool f32, const HyStreams& c, float* xs, const float* y, const int32_t* rows, const float* w, float eps, void* h, int ldh, float* hn, float* shift_state,
                           float* prev, const HyRows& r, int T, int W, cudaStream_t s) {
    if (c.n < 1 || c.n > HY_MAX_STREAMS || (size_t)W * 4 > 200 * 1024 || (rows && shift_state) || T <= 0) return cudaErrorInvalidValue;
    return f32 ? stream_norm_t<float>(c, xs, y, rows, w, eps, h, ldh, hn, shift_state, prev, r, T, W, s) : stream_norm_t<bf>(c, xs, y, rows, w, eps, h, ldh, hn, shift_state, prev, r, T, W, s);
}
cudaError_t hy_token_shift(bool f32, const float* hn, const float* prev, const float* mu, void* h, int ldh, const HyRows& r, int W, cudaStream_t s) {
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (W % 4 == 0 && ldh % 4 == 0 && al16(hn) && al16(prev) && al16(mu) && al16(h)) {
        const dim3 g((W / 4 + 255) / 256, r.T);
        return f32 ? launch_plain(hy_token_shift_kernel<float, 4>, g, dim3(256), 0, s, hn, prev, mu, (float*)h, ldh, r, W)
                   : launch_plain(hy_token_shift_kernel<bf, 4>, g, dim3(256), 0, s, hn, prev, mu, (bf*)h, ldh, r, W);
    }
    const dim3 g((W + 255) / 256, r.T);
    return f32 ? launch_plain(hy_token_shift_kernel<float, 1>, g, dim3(256), 0, s, hn, prev, mu, (float*)h, ldh, r, W)
               : launch_plain(hy_token_shift_kernel<bf, 1>, g, dim3(256), 0, s, hn, prev, mu, (bf*)h, ldh, r, W);
}
cudaError_t hy_rmsnorm_act(bool f32, const void* in, int ld_in, int n, const float* w, void* out, int ld_out, float eps, int T, cudaStream_t s) {
    return f32 ? launch_plain(hy_rmsnorm_act_kernel<float>, dim3(T), dim3(128), 0, s, (const float*)in, ld_in, n, w, (float*)out, ld_out, eps)
               : launch_plain(hy_rmsnorm_act_kernel<bf>, dim3(T), dim3(128), 0, s, (const bf*)in, ld_in, n, w, (bf*)out, ld_out, eps);
}
cudaError_t hy_sigmoid_gate(bool f32, void* x, int ldx, const void* g, int ldg, int n, int T, cudaStream_t s) {
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (!f32 && n % 8 == 0 && ldx % 8 == 0 && ldg % 8 == 0 && al16(x) && al16(g))
        return launch_plain(hy_sigmoid_gate_vec8_kernel, dim3((n / 8 + 127) / 128, T), dim3(128), 0, s, (bf*)x, ldx, (const bf*)g, ldg, n);
    const dim3 grid((n + 255) / 256, T);
    return f32 ? launch_plain(hy_sigmoid_gate_kernel<float>, grid, dim3(256), 0, s, (float*)x, ldx, (const float*)g, ldg, n)
               : launch_plain(hy_sigmoid_gate_kernel<bf>, grid, dim3(256), 0, s, (bf*)x, ldx, (const bf*)g, ldg, n);
}

}  // namespace oa
