// hybrid_window.cu — windowed softmax attention over cached keys and values for the hybrid decoder family (API: hybrid_kernels.hpp), and the RMS
// norm pair that feeds a layer whose mixer and feed-forward read separate norms of the same residual.
//
// One mechanism with its constants as parameters (HyWinAttn): `heads` query heads on `kv_heads` key/value heads; `maps` score maps per head
// (2 = differential attention: the head's query and key rows hold [map 1 | map 2], both maps weigh the same values, and the head's output is
// (a1 - lambda a2) scaled to unit RMS times out_scale); a sliding window of `window` positions plus the first `keep_first` positions of the
// sequence; an optional RMS norm of every query / key map; an optional sink logit per head that only enlarges the softmax denominator; a
// sigmoid output gate per channel or per head; optional score modifiers — a soft cap (cap tanh(score / cap)) and a penalty per position of
// distance with a slope per head — and, in the preparation step, one RMS norm over the whole query / key projection and a query temperature
// that grows with the logarithm of the position.  Softmax, norms, score modifiers and gates are fp32 in both element types.
#include "hybrid_common.cuh"
#include "hybrid_kernels.hpp"

namespace oa {

namespace {

using namespace hyk;

// out1[t] = x[row] / sqrt(mean(x[row]^2) + eps) * w1 (and out2 with w2): one read of the residual row for both norms
template <typename TA>
__global__ void __launch_bounds__(256) hy_rmsnorm_pair_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows, const float* __restrict__ w1, TA* __restrict__ out1,
                                                              const float* __restrict__ w2, TA* __restrict__ out2, int ldo, int W, float eps) {
    HY_PDL();
    __shared__ float red[32];
    const int t = blockIdx.x; const float* xr = x + (long long)(rows ? rows[t] : t) * W;
    float s = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) { const float v = xr[c]; s = fmaf(v, v, s); }
    const float rr = 1.0f / sqrtf(block_sum(s, red) / (float)W + eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = xr[c] * rr;
        stf(out1 + (long long)t * ldo + c, v * w1[c]);
        if (out2) stf(out2 + (long long)t * ldo + c, v * w2[c]);
    }
}

// Per row: RMS norm of every query map in place (qk_norm), keys (normed alike) and values into the row's cache slot [kv_heads maps dim | kv_heads vdim].
// One warp per vector.
template <typename TA>
__global__ void __launch_bounds__(128) hy_win_prep_kernel(HyWinAttn a, TA* __restrict__ q, int ldq, const TA* __restrict__ k, const TA* __restrict__ v, int ldkv,
                                                          const float* __restrict__ qw, const float* __restrict__ kw, float eps, TA* __restrict__ cache, HyRows r) {
    HY_PDL();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, D = a.dim;
    const int nq = a.qk_norm ? a.heads * a.maps : 0, nk = k ? a.kv_heads * a.maps : 0, KW = a.kv_heads * a.maps * D, CW = KW + a.kv_heads * a.vdim;
    TA* crow = cache + (long long)r.slots[t] * CW;
    for (int u = warp; u < nq + nk; u += 4) {
        const bool is_q = u < nq; const int i = is_q ? u : u - nq;
        const TA* src = is_q ? q + (long long)t * ldq + (long long)i * D : k + (long long)t * ldkv + (long long)i * D;
        TA* dst = is_q ? q + (long long)t * ldq + (long long)i * D : crow + (long long)i * D;
        float rr = 1.f;
        if (a.qk_norm) {
            float ss = 0.f;
            for (int c = lane; c < D; c += 32) { const float x = ldf(src + c); ss = fmaf(x, x, ss); }
            rr = 1.0f / sqrtf(warp_sum(ss) / (float)D + eps);
        }
        const float* w = is_q ? qw : kw;
        for (int c = lane; c < D; c += 32) stf(dst + c, a.qk_norm ? ldf(src + c) * rr * w[c] : ldf(src + c));
    }
    if (v) for (int c = threadIdx.x; c < a.kv_heads * a.vdim; c += blockDim.x) crow[KW + c] = v[(long long)t * ldkv + c];
}

// The same for bf16 rows whose vectors come in aligned groups of 8 channels and whose dim / 8 is a power of two up to 32: a lane owns 16 bytes of a
// vector, the dim / 8 lanes of a vector meet by shuffles, every access is 16 bytes wide.  Sums run per lane and then over lanes, so the
// rounding of the norm differs from the kernel above in the last fp32 bit only; a model takes one of the two for all of its steps.
__global__ void __launch_bounds__(128) hy_win_prep_vec8_kernel(HyWinAttn a, __nv_bfloat16* __restrict__ q, int ldq, const __nv_bfloat16* __restrict__ k,
                                                               const __nv_bfloat16* __restrict__ v, int ldkv, const float* __restrict__ qw, const float* __restrict__ kw, float eps,
                                                               __nv_bfloat16* __restrict__ cache, HyRows r) {
    HY_PDL();
    const int t = blockIdx.x, tid = threadIdx.x, D = a.dim, GS = D / 8;
    const int nq = a.qk_norm ? a.heads * a.maps : 0, nk = k ? a.kv_heads * a.maps : 0, KW = a.kv_heads * a.maps * D, CW = KW + a.kv_heads * a.vdim;
    __nv_bfloat16* crow = cache + (long long)r.slots[t] * CW;
    const int per_pass = 128 / GS, part = tid % GS;
    for (int base = 0; base < nq + nk; base += per_pass) {
        const int u = base + tid / GS; const bool ok = u < nq + nk, is_q = u < nq; const int i = is_q ? u : u - nq;
        const __nv_bfloat16* src = is_q ? q + (long long)t * ldq + (long long)i * D + part * 8 : k + (long long)t * ldkv + (long long)i * D + part * 8;
        __nv_bfloat16* dst = is_q ? q + (long long)t * ldq + (long long)i * D + part * 8 : crow + (long long)i * D + part * 8;
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (ok) raw = *reinterpret_cast<const uint4*>(src);
        if (a.qk_norm) {
            const float x[8] = {bf16lo(raw.x), bf16hi(raw.x), bf16lo(raw.y), bf16hi(raw.y), bf16lo(raw.z), bf16hi(raw.z), bf16lo(raw.w), bf16hi(raw.w)};
            float ss = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) ss = fmaf(x[e], x[e], ss);
            for (int o = 1; o < GS; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float rr = 1.0f / sqrtf(ss / (float)D + eps);
            if (ok) {
                const float* w = (is_q ? qw : kw) + part * 8;
                const float4 w0 = *reinterpret_cast<const float4*>(w), w1 = *reinterpret_cast<const float4*>(w + 4);
                raw.x = pack_bf16x2(x[0] * rr * w0.x, x[1] * rr * w0.y); raw.y = pack_bf16x2(x[2] * rr * w0.z, x[3] * rr * w0.w);
                raw.z = pack_bf16x2(x[4] * rr * w1.x, x[5] * rr * w1.y); raw.w = pack_bf16x2(x[6] * rr * w1.z, x[7] * rr * w1.w);
            }
        }
        if (ok) *reinterpret_cast<uint4*>(dst) = raw;
    }
    if (v) for (int c = tid * 8; c < a.kv_heads * a.vdim; c += 128 * 8) *reinterpret_cast<uint4*>(crow + KW + c) = *reinterpret_cast<const uint4*>(v + (long long)t * ldkv + c);
}

// qk_norm = 2: one RMS norm over the whole q projection of the row (all heads and maps) and one over the whole k projection, weights of
// those sizes; then the query temperature.  Queries in place, keys and values into the row's cache slot.  One CTA per row.
__device__ __forceinline__ float win_q_temp(const HyWinAttn& a, int pos) {
    return a.q_temp_every > 0 ? 1.0f + a.q_temp_coef * logf((float)((pos + 1) / a.q_temp_every) + 1.0f) : 1.0f;
}
template <typename TA>
__global__ void __launch_bounds__(128) hy_win_prep_whole_kernel(HyWinAttn a, TA* __restrict__ q, int ldq, const TA* __restrict__ k, const TA* __restrict__ v, int ldkv,
                                                                const float* __restrict__ qw, const float* __restrict__ kw, float eps, TA* __restrict__ cache, HyRows r) {
    HY_PDL();
    __shared__ float red[32];
    const long long t = blockIdx.x;
    const int QW = a.heads * a.maps * a.dim, KW = a.kv_heads * a.maps * a.dim, CW = KW + a.kv_heads * a.vdim;
    TA* qr = q + t * ldq; TA* crow = cache + (long long)r.slots[t] * CW;
    float sq = 0.f, sk = 0.f;
    for (int c = threadIdx.x; c < QW; c += blockDim.x) { const float x = ldf(qr + c); sq = fmaf(x, x, sq); }
    if (k) for (int c = threadIdx.x; c < KW; c += blockDim.x) { const float x = ldf(k + t * ldkv + c); sk = fmaf(x, x, sk); }
    const float rq = 1.0f / sqrtf(block_sum(sq, red) / (float)QW + eps) * win_q_temp(a, r.positions[t]);
    const float rk = k ? 1.0f / sqrtf(block_sum(sk, red) / (float)KW + eps) : 0.f;
    for (int c = threadIdx.x; c < QW; c += blockDim.x) stf(qr + c, ldf(qr + c) * rq * qw[c]);
    if (k) for (int c = threadIdx.x; c < KW; c += blockDim.x) stf(crow + c, ldf(k + t * ldkv + c) * rk * kw[c]);
    if (v) for (int c = threadIdx.x; c < a.kv_heads * a.vdim; c += blockDim.x) crow[KW + c] = v[t * ldkv + c];
}

// The same for bf16 rows whose projections come in aligned groups of 8 channels: 16 bytes per access, the second pass re-reads what the first
// left in L1.  Sums run per thread over its own vectors and then over the block: the norm's rounding differs from the kernel above in the
// last fp32 bits only; a model takes one of the two for all of its steps.
__global__ void __launch_bounds__(128) hy_win_prep_whole_vec8_kernel(HyWinAttn a, __nv_bfloat16* __restrict__ q, int ldq, const __nv_bfloat16* __restrict__ k,
                                                                     const __nv_bfloat16* __restrict__ v, int ldkv, const float* __restrict__ qw, const float* __restrict__ kw, float eps,
                                                                     __nv_bfloat16* __restrict__ cache, HyRows r) {
    HY_PDL();
    __shared__ float red[32];
    const long long t = blockIdx.x;
    const int QW = a.heads * a.maps * a.dim, KW = a.kv_heads * a.maps * a.dim, VW = a.kv_heads * a.vdim, CW = KW + VW;
    __nv_bfloat16* qr = q + t * ldq; __nv_bfloat16* crow = cache + (long long)r.slots[t] * CW;
    auto sq8 = [](const uint4& u) {
        const float x[8] = {bf16lo(u.x), bf16hi(u.x), bf16lo(u.y), bf16hi(u.y), bf16lo(u.z), bf16hi(u.z), bf16lo(u.w), bf16hi(u.w)};
        float s = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) s = fmaf(x[e], x[e], s);
        return s;
    };
    auto scale8 = [](const uint4& u, float rr, const float* w) {
        const float4 w0 = *reinterpret_cast<const float4*>(w), w1 = *reinterpret_cast<const float4*>(w + 4);
        return make_uint4(pack_bf16x2(bf16lo(u.x) * rr * w0.x, bf16hi(u.x) * rr * w0.y), pack_bf16x2(bf16lo(u.y) * rr * w0.z, bf16hi(u.y) * rr * w0.w),
                          pack_bf16x2(bf16lo(u.z) * rr * w1.x, bf16hi(u.z) * rr * w1.y), pack_bf16x2(bf16lo(u.w) * rr * w1.z, bf16hi(u.w) * rr * w1.w));
    };
    float sq = 0.f, sk = 0.f;
    for (int c = threadIdx.x * 8; c < QW; c += blockDim.x * 8) sq += sq8(*reinterpret_cast<const uint4*>(qr + c));
    if (k) for (int c = threadIdx.x * 8; c < KW; c += blockDim.x * 8) sk += sq8(*reinterpret_cast<const uint4*>(k + t * ldkv + c));
    const float rq = 1.0f / sqrtf(block_sum(sq, red) / (float)QW + eps) * win_q_temp(a, r.positions[t]);
    const float rk = k ? 1.0f / sqrtf(block_sum(sk, red) / (float)KW + eps) : 0.f;
    for (int c = threadIdx.x * 8; c < QW; c += blockDim.x * 8) *reinterpret_cast<uint4*>(qr + c) = scale8(*reinterpret_cast<const uint4*>(qr + c), rq, qw + c);
    if (k) for (int c = threadIdx.x * 8; c < KW; c += blockDim.x * 8) *reinterpret_cast<uint4*>(crow + c) = scale8(*reinterpret_cast<const uint4*>(k + t * ldkv + c), rk, kw + c);
    if (v) for (int c = threadIdx.x * 8; c < VW; c += blockDim.x * 8) *reinterpret_cast<uint4*>(crow + KW + c) = *reinterpret_cast<const uint4*>(v + t * ldkv + c);
}

// score modifiers shared by every form: s is the scaled score of the query at position p (head h) with the key at position j
__device__ __forceinline__ float win_head_slope(const HyWinAttn& a, int h) { return a.slope_exp > 0.f ? exp2f(-a.slope_exp * (float)(h + 1) / (float)a.heads) : 0.f; }
__device__ __forceinline__ float win_tanh(float x) {          // 1 - 2 / (e^2x + 1): relative error of a few fp32 ulps from the SFU exponent and a full division
    const float e = ex2_approx(fminf(x * 2.8853900817779268f, 80.f));
    return 1.0f - 2.0f / (e + 1.0f);
}

// Rotary preparation: per row, the first rot.dims channels of every query head (in place) and key head turn by the row's position, every
// value head turns over all of its channels (v_cos given); keys and values go to the row's cache slot.  A thread owns a pair of channels.
template <typename TA>
__device__ __forceinline__ void rope_head(const TA* src, TA* dst, int n, int dims, int layout, const float* cs, const float* sn, int i) {
    // i < n / 2 + (n - dims) / 2 ... handled by the caller: i indexes pairs first (dims / 2 of them), then the unrotated rest one by one
    const int half = dims / 2;
    if (i < half) {
        const int a = layout ? i : 2 * i, b = layout ? i + half : 2 * i + 1;
        const float u = ldf(src + a), v = ldf(src + b);
        stf(dst + a, u * cs[i] - v * sn[i]); stf(dst + b, v * cs[i] + u * sn[i]);
    } else { const int c = dims + (i - half); if (src != dst) stf(dst + c, ldf(src + c)); }
}
template <typename TA>
__global__ void __launch_bounds__(128) hy_win_rope_prep_kernel(HyWinAttn a, HyRotary rot, TA* __restrict__ q, int ldq, const TA* __restrict__ k, const TA* __restrict__ v, int ldkv,
                                                               TA* __restrict__ cache, HyRows r) {
    HY_PDL();
    const long long t = blockIdx.x; const int D = a.dim, VD = a.vdim, pos = r.positions[t];
    const int KW = a.kv_heads * D, CW = KW + a.kv_heads * VD, half = rot.dims / 2, per = half + (D - rot.dims);      // work items per query / key head
    const float* cs = rot.cos + (long long)pos * half; const float* sn = rot.sin + (long long)pos * half;
    TA* crow = cache + (long long)r.slots[t] * CW;
    for (int i = threadIdx.x; i < a.heads * per; i += blockDim.x) { const int hd = i / per; TA* p = q + t * ldq + (long long)hd * D; rope_head(p, p, D, rot.dims, rot.layout, cs, sn, i - hd * per); }
    if (k) for (int i = threadIdx.x; i < a.kv_heads * per; i += blockDim.x) { const int hd = i / per; rope_head(k + t * ldkv + (long long)hd * D, crow + (long long)hd * D, D, rot.dims, rot.layout, cs, sn, i - hd * per); }
    if (v) {
        if (rot.v_cos) {
            const int vh = VD / 2; const float* vc = rot.v_cos + (long long)pos * vh; const float* vs = rot.v_sin + (long long)pos * vh;
            for (int i = threadIdx.x; i < a.kv_heads * vh; i += blockDim.x) { const int hd = i / vh; rope_head(v + t * ldkv + (long long)hd * VD, crow + KW + (long long)hd * VD, VD, VD, rot.layout, vc, vs, i - hd * vh); }
        } else for (int c = threadIdx.x; c < a.kv_heads * VD; c += blockDim.x) crow[KW + c] = v[t * ldkv + c];
    }
}

// Convolution, rotary and cache write in one pass (bf16; interleaved pairs; head sizes and segment offsets in aligned groups of 8 channels): a
// thread owns 8 channels of ROWS consecutive rows of the fused projection [q | k | v], keeps its taps' weights and the last inputs in
// registers (every input row is read once; the window is rebuilt from earlier rows, the carried tail or zeros wherever a sequence starts
// inside the block), and hands the fp32 convolution straight to the rotation: the 4 pairs of a thread's channels turn by the row's position
// (queries and keys on their first rot.dims channels, values on all), queries go to q_out, keys and values to the row's cache slot.
// ROWS = 16 for prefill-sized steps, 1 otherwise; a row's arithmetic is the same in both.
template <int TAPS, int ROWS>
__global__ void __launch_bounds__(128) hy_conv_rope_cache_kernel(HyWinAttn a, HyRotary rot, const __nv_bfloat16* __restrict__ in, int ld_in, int C, int off_q, int off_k, int off_v,
                                                                 const float* __restrict__ w, __nv_bfloat16* __restrict__ q_out, int ldq, __nv_bfloat16* __restrict__ cache,
                                                                 const __nv_bfloat16* __restrict__ tails, HyRows r) {
    HY_PDL();
    // the block's row metadata once, in shared memory: a thread's per-row chain is then one global load (its 16 bytes of input, requested a row ahead)
    __shared__ int s_row0[ROWS], s_pos0[ROWS], s_pos[ROWS], s_slot[ROWS], s_state[ROWS];
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8, t0 = blockIdx.y * ROWS;
    if (threadIdx.x < ROWS && t0 + threadIdx.x < r.T) {
        const int t = t0 + threadIdx.x, seq = r.row_seq[t];
        s_row0[threadIdx.x] = r.seq_row0[seq]; s_pos0[threadIdx.x] = r.seq_pos0[seq]; s_pos[threadIdx.x] = r.positions[t]; s_slot[threadIdx.x] = r.slots[t]; s_state[threadIdx.x] = r.seq_state[seq];
    }
    __syncthreads();
    const int D = a.dim, VD = a.vdim, KW = a.kv_heads * D, CW = KW + a.kv_heads * VD;
    int seg, local;                                      // 0: query, 1: key, 2: value; channel within the segment
    if (c >= off_q && c < off_q + a.heads * D) { seg = 0; local = c - off_q; }
    else if (c >= off_k && c < off_k + KW) { seg = 1; local = c - off_k; }
    else if (c >= off_v && c < off_v + a.kv_heads * VD) { seg = 2; local = c - off_v; }
    else return;
    const int d0 = seg == 2 ? local % VD : local % D;    // first of the thread's channels within its head
    const int n_rot = seg == 2 ? (rot.v_cos ? VD : 0) : rot.dims, half = n_rot / 2;
    const float* ct = seg == 2 ? rot.v_cos : rot.cos; const float* st = seg == 2 ? rot.v_sin : rot.sin;
    float wr[TAPS][8], win[TAPS][8];
#pragma unroll
    for (int e = 0; e < 8; ++e)
#pragma unroll
        for (int j = 0; j < TAPS; ++j) wr[j][e] = w[(c + e) * TAPS + j];
    auto unpack = [](const uint4& u, float* f) {
        const uint32_t x[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) { f[2 * i] = bf16lo(x[i]); f[2 * i + 1] = bf16hi(x[i]); }
    };
    constexpr int AHEAD = ROWS >= 4 ? 4 : 1;             // input rows requested ahead of the one being computed
    uint4 ring[AHEAD];
#pragma unroll
    for (int k = 0; k < AHEAD; ++k) if (t0 + k < r.T) ring[k] = *reinterpret_cast<const uint4*>(in + (long long)(t0 + k) * ld_in + c);
#pragma unroll
    for (int tt = 0; tt < ROWS; ++tt) {
        if (t0 + tt >= r.T) break;
        const int t = t0 + tt, row0 = s_row0[tt], i = t - row0;
        const uint4 cur = ring[tt % AHEAD];
        if (tt + AHEAD < ROWS && t + AHEAD < r.T) ring[tt % AHEAD] = *reinterpret_cast<const uint4*>(in + (long long)(t + AHEAD) * ld_in + c);
        if (tt == 0 || i == 0) {
            const int pos0 = s_pos0[tt];
            const __nv_bfloat16* tail = tails + (long long)s_state[tt] * (TAPS - 1) * C;
#pragma unroll
            for (int j = 0; j < TAPS - 1; ++j) {
                const int src = i - (TAPS - 1) + j;
                uint4 u = make_uint4(0u, 0u, 0u, 0u);
                if (src >= 0) u = *reinterpret_cast<const uint4*>(in + (long long)(row0 + src) * ld_in + c);
                else if (pos0 > 0) u = *reinterpret_cast<const uint4*>(tail + (long long)(TAPS - 1 + src) * C + c);
                unpack(u, win[j]);
            }
        }
        unpack(cur, win[TAPS - 1]);
        float y[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < TAPS; ++j) acc = fmaf(wr[j][e], win[j][e], acc);
            y[e] = acc;
        }
        const long long pos = s_pos[tt];
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const int d = d0 + 2 * p;
            if (d < n_rot) {
                const float cs = ct[pos * half + (d >> 1)], sn = st[pos * half + (d >> 1)], u = y[2 * p], v = y[2 * p + 1];
                y[2 * p] = u * cs - v * sn; y[2 * p + 1] = v * cs + u * sn;
            }
        }
        const uint4 o = make_uint4(pack_bf16x2(y[0], y[1]), pack_bf16x2(y[2], y[3]), pack_bf16x2(y[4], y[5]), pack_bf16x2(y[6], y[7]));
        __nv_bfloat16* dst = seg == 0 ? q_out + (long long)t * ldq + local : cache + (long long)s_slot[tt] * CW + (seg == 1 ? local : KW + local);
        *reinterpret_cast<uint4*>(dst) = o;
#pragma unroll
        for (int j = 0; j < TAPS - 1; ++j)
#pragma unroll
            for (int e = 0; e < 8; ++e) win[j][e] = win[j + 1][e];
    }
}

// The visible keys of a query at position p, in the order every kernel walks them: the kept first positions that the window no longer
// covers, then the window.  n = count; key(i) = i-th visible position.
struct WinKeys {
    int n_keep, lo, n;
    __device__ __forceinline__ WinKeys(int p, int window, int keep_first) { lo = max(0, p - window + 1); n_keep = min(keep_first, lo); n = n_keep + (p - lo + 1); }
    __device__ __forceinline__ int key(int i) const { return i < n_keep ? i : lo + (i - n_keep); }
};

constexpr int WIN_MAXV = 8;       // value channels per lane: vdim <= 32 * WIN_MAXV
// Plain form, any sizes, both element types: one CTA per (row, head); its four warps take the visible keys round-robin (a fixed order that
// depends on the row's position only), each with an online softmax per map; the CTA joins them, adds the sink to the denominator, and
// finishes the head: differential combination and unit RMS, gate, store.
template <typename TA>
__global__ void __launch_bounds__(128) hy_win_attention_kernel(HyWinAttn a, const TA* __restrict__ q, int ldq, const TA* __restrict__ cache, const float* __restrict__ sink,
                                                               const TA* __restrict__ gate, int ldg, TA* __restrict__ out, int ldo, float eps, HyRows r) {
    HY_PDL();
    extern __shared__ float sm[];
    __shared__ float red[32];
    const int t = blockIdx.x, h = blockIdx.y, D = a.dim, VD = a.vdim, NM = a.maps;
    const int KW = a.kv_heads * NM * D, CW = KW + a.kv_heads * VD, g = h / (a.heads / a.kv_heads);
    float* qs = sm;                              // [NM][D]
    float* part = qs + NM * D;                   // [4][NM][VD]
    float* mm = part + 4 * NM * VD;              // [4][NM]
    float* ll = mm + 4 * NM;                     // [4][NM]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < NM * D; i += blockDim.x) qs[i] = ldf(q + (long long)t * ldq + (long long)h * NM * D + i) * a.scale;
    __syncthreads();
    const int seq = r.row_seq[t], pos = r.positions[t];
    const int32_t* bt = r.block_tables + (long long)seq * r.max_pages_per_seq;
    const WinKeys wk(pos, a.window, a.keep_first);
    const float slope = win_head_slope(a, h);
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f}, acc[2][WIN_MAXV];
#pragma unroll
    for (int mp = 0; mp < 2; ++mp)
#pragma unroll
        for (int i = 0; i < WIN_MAXV; ++i) acc[mp][i] = 0.f;
    for (int i = warp; i < wk.n; i += 4) {
        const int j = wk.key(i);
        const TA* row = cache + ((long long)bt[j >> 6] * 64 + (j & 63)) * CW;
        const TA* kr = row + (long long)g * NM * D; const TA* vr = row + KW + (long long)g * VD;
        float vv[WIN_MAXV];
#pragma unroll
        for (int c = 0; c < WIN_MAXV; ++c) vv[c] = lane + 32 * c < VD ? ldf(vr + lane + 32 * c) : 0.f;
#pragma unroll
        for (int mp = 0; mp < 2; ++mp) {
            if (mp >= NM) break;
            float d = 0.f;
            for (int c = lane; c < D; c += 32) d = fmaf(qs[mp * D + c], ldf(kr + mp * D + c), d);
            d = warp_sum(d);
            if (a.softcap > 0.f) d = a.softcap * tanhf(d / a.softcap);
            d -= slope * (float)(pos - j);
            const float mn = fmaxf(m[mp], d), corr = expf(m[mp] - mn), p = expf(d - mn);
            l[mp] = l[mp] * corr + p; m[mp] = mn;
#pragma unroll
            for (int c = 0; c < WIN_MAXV; ++c) acc[mp][c] = fmaf(p, vv[c], acc[mp][c] * corr);
        }
    }
#pragma unroll
    for (int mp = 0; mp < 2; ++mp) {
        if (mp >= NM) break;
#pragma unroll
        for (int c = 0; c < WIN_MAXV; ++c) if (lane + 32 * c < VD) part[(warp * NM + mp) * VD + lane + 32 * c] = acc[mp][c];
        if (lane == 0) { mm[warp * NM + mp] = m[mp]; ll[warp * NM + mp] = l[mp]; }
    }
    __syncthreads();
    float f[2][4], inv[2];
    for (int mp = 0; mp < NM; ++mp) {
        float M = sink ? sink[h] : -INFINITY, L = 0.f;
        for (int w = 0; w < 4; ++w) M = fmaxf(M, mm[w * NM + mp]);
        for (int w = 0; w < 4; ++w) { f[mp][w] = mm[w * NM + mp] == -INFINITY ? 0.f : expf(mm[w * NM + mp] - M); L = fmaf(f[mp][w], ll[w * NM + mp], L); }
        if (sink) L += expf(sink[h] - M);
        inv[mp] = 1.0f / L;
    }
    float ss = 0.f;
    float o[WIN_MAXV];          // channel threadIdx.x + 128 * i of the head
#pragma unroll
    for (int i = 0; i < WIN_MAXV / 4; ++i) {
        const int c = threadIdx.x + 128 * i; o[i] = 0.f;
        if (c < VD) {
            float a1 = 0.f;
            for (int w = 0; w < 4; ++w) a1 = fmaf(f[0][w], part[(w * NM) * VD + c], a1);
            a1 *= inv[0];
            if (NM == 2) {
                float a2 = 0.f;
                for (int w = 0; w < 4; ++w) a2 = fmaf(f[1][w], part[(w * NM + 1) * VD + c], a2);
                a1 = a1 - a.lambda * (a2 * inv[1]);
            }
            o[i] = a1; ss = fmaf(a1, a1, ss);
        }
    }
    float post = 1.f;
    if (NM == 2) post = a.out_scale / sqrtf(block_sum(ss, red) / (float)VD + eps);
    if (a.out_rot) {                 // the head's output turned back by its own position: channels meet their partners through shared memory
        __syncthreads();
#pragma unroll
        for (int i = 0; i < WIN_MAXV / 4; ++i) { const int c = threadIdx.x + 128 * i; if (c < VD) part[c] = o[i] * post; }
        __syncthreads();
        const int vh = VD / 2; const float* cs = a.out_cos + (long long)pos * vh; const float* sn = a.out_sin + (long long)pos * vh;
#pragma unroll
        for (int i = 0; i < WIN_MAXV / 4; ++i) {
            const int c = threadIdx.x + 128 * i;
            if (c < VD) {
                const bool first = a.out_rot == 1 ? !(c & 1) : c < vh; const int pr = a.out_rot == 1 ? c >> 1 : (first ? c : c - vh);
                const int other = a.out_rot == 1 ? c ^ 1 : (first ? c + vh : c - vh);
                o[i] = first ? part[c] * cs[pr] + part[other] * sn[pr] : part[c] * cs[pr] - part[other] * sn[pr];       // (u, v) -> (u cos + v sin, v cos - u sin)
            }
        }
        post = 1.f;
    }
#pragma unroll
    for (int i = 0; i < WIN_MAXV / 4; ++i) {
        const int c = threadIdx.x + 128 * i;
        if (c < VD) {
            float y = o[i] * post;
            if (a.gate == 1) y *= sigmoidf_(ldf(gate + (long long)t * ldg + (long long)h * VD + c));
            else if (a.gate == 2) y *= sigmoidf_(ldf(gate + (long long)t * ldg + h));
            stf(out + (long long)t * ldo + (long long)h * VD + c, y);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------------------------
// Tensor-core form (bf16; dim a multiple of 16 up to 128, vdim 16 / 32 / 64 / 96 / 128): one CTA owns 64 query slots — consecutive
// (row, head) pairs of ONE sequence and ONE key/value head, so a prompt portion brings 64 / group rows per CTA and a decoding row its whole
// group — and streams that head's cached keys and values in 32-row tiles through a cp.async double buffer, straight from the pages.  Only
// tiles that hold a visible key are visited: the kept first positions below the window of the tile's first row, then the window.  Both
// score maps of a differential head are computed from the same key tile and weigh the same value tile; S = Q K^T and O += P V are
// mma.sync m16n8k16 products, the softmax is online in fp32 registers with the mask per query position.  The epilogue finishes the head in
// registers: sink into the denominator, a1 - lambda a2, unit RMS over the head's channels (a quad shuffle), gate, bf16 store into the
// output projection's input.
// ---------------------------------------------------------------------------------------------------------------------------------
constexpr int WIN_MQ = 64, WIN_KT = 32;
template <int MAPS, int NVB, bool MOD>      // MOD: soft cap and / or distance slope on the scores
__global__ void __launch_bounds__(128) hy_win_attention_mma_kernel(HyWinAttn a, const __nv_bfloat16* __restrict__ q, int ldq, const __nv_bfloat16* __restrict__ cache,
                                                                   const float* __restrict__ sink, const __nv_bfloat16* __restrict__ gate, int ldg,
                                                                   __nv_bfloat16* __restrict__ out, int ldo, float eps, HyRows r, const int32_t* __restrict__ tile_seq,
                                                                   const int32_t* __restrict__ tile_q0) {
    HY_PDL();
    extern __shared__ __align__(16) uint8_t win_smem[];
    constexpr int VD = NVB * 8, VP = VD + 8;
    const int D = a.dim, QD = MAPS * D, QP = QD + 8, HG = a.heads / a.kv_heads, g = blockIdx.y;
    const int KW = a.kv_heads * QD, CW = KW + a.kv_heads * VD;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(win_smem);      // [64][QP]
    __nv_bfloat16* Ks = Qs + WIN_MQ * QP;                                // [2][32][QP]
    __nv_bfloat16* Vs = Ks + 2 * WIN_KT * QP;                            // [2][32][VP]
    int* qpos = reinterpret_cast<int*>(Vs + 2 * WIN_KT * VP);            // [64]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int seq = tile_seq[blockIdx.x], q0 = tile_q0[blockIdx.x];
    const int row0 = r.seq_row0[seq], len = r.seq_row0[seq + 1] - row0;
    const int nq = min(WIN_MQ, len * HG - q0);
    for (int idx = tid; idx < WIN_MQ * (QD / 8); idx += 128) {
        const int qi = idx / (QD / 8), c = idx - qi * (QD / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (qi < nq) v = *reinterpret_cast<const uint4*>(q + (long long)(row0 + (q0 + qi) / HG) * ldq + (long long)(g * HG + (q0 + qi) % HG) * QD + c * 8);
        *reinterpret_cast<uint4*>(Qs + qi * QP + c * 8) = v;
    }
    for (int qi = tid; qi < WIN_MQ; qi += 128) qpos[qi] = qi < nq ? r.positions[row0 + (q0 + qi) / HG] : -1;
    auto qpos_of = [&](int qi) { return r.positions[row0 + (q0 + qi) / HG]; };
    const int pos_min = qpos_of(0), pos_max = qpos_of(nq - 1);
    const int lo_min = max(0, pos_min - a.window + 1);
    const int win_t0 = lo_min / WIN_KT, n_kt = pos_max / WIN_KT + 1;
    const int n_keep = min((min(a.keep_first, lo_min) + WIN_KT - 1) / WIN_KT, win_t0);      // tiles of kept first positions that lie wholly below the window's first tile
    const int n_it = n_keep + (n_kt - win_t0);
    const int32_t* bt = r.block_tables + (long long)seq * r.max_pages_per_seq;
    // a tile's 32 keys lie in one page (one block-table lookup per tile); a thread walks the tile's 16-byte chunks in steps of 128 with its
    // (row, chunk) pair advanced by additions
    const int kc = QD / 8, nc = kc + VD / 8, step_j = 128 / nc, step_c = 128 % nc, j0 = tid / nc, c0 = tid % nc;
    auto load_tile = [&](int it, int buf) {
        const int key0 = (it < n_keep ? it : win_t0 + (it - n_keep)) * WIN_KT;
        const __nv_bfloat16* page = cache + ((long long)bt[key0 >> 6] * 64 + (key0 & 63)) * CW;
        int j = j0, c = c0;
        while (j < WIN_KT) {
            __nv_bfloat16* dst = c < kc ? Ks + (buf * WIN_KT + j) * QP + c * 8 : Vs + (buf * WIN_KT + j) * VP + (c - kc) * 8;
            if (key0 + j <= pos_max) cp_async16(dst, page + (long long)j * CW + (c < kc ? g * QD + c * 8 : KW + g * VD + (c - kc) * 8));
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
            j += step_j; c += step_c;
            if (c >= nc) { c -= nc; ++j; }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float o[MAPS][NVB][4];
    float m_lo[MAPS], m_hi[MAPS], l_lo[MAPS], l_hi[MAPS];
#pragma unroll
    for (int mp = 0; mp < MAPS; ++mp) {
        m_lo[mp] = m_hi[mp] = -INFINITY; l_lo[mp] = l_hi[mp] = 0.f;
#pragma unroll
        for (int i = 0; i < NVB; ++i) { o[mp][i][0] = o[mp][i][1] = o[mp][i][2] = o[mp][i][3] = 0.f; }
    }
    // MOD: the scores are scaled, capped, given their distance penalty and brought to base-2 units right after the product
    const float qscale = MOD ? 1.0f : a.scale * 1.4426950408889634f;
    const float inv_cap = a.softcap > 0.f ? a.scale / a.softcap : 0.f;
    const float slope_lo = MOD ? win_head_slope(a, g * HG + (q0 + 16 * warp + (lane >> 2)) % HG) : 0.f, slope_hi = MOD ? win_head_slope(a, g * HG + (q0 + 16 * warp + (lane >> 2) + 8) % HG) : 0.f;
    const bool active = 16 * warp < nq;
    const int wp_min = active ? qpos_of(16 * warp) : 0, wp_max = active ? qpos_of(min(16 * warp + 15, nq - 1)) : 0;      // positions of the warp's first and last query slot
    load_tile(0, 0);
    for (int it = 0; it < n_it; ++it) {
        if (it + 1 < n_it) { load_tile(it + 1, (it + 1) & 1); asm volatile("cp.async.wait_group 1;" ::: "memory"); }
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        if (active) {
            const int kt = it < n_keep ? it : win_t0 + (it - n_keep);
            const __nv_bfloat16* Kb = Ks + (it & 1) * WIN_KT * QP; const __nv_bfloat16* Vb = Vs + (it & 1) * WIN_KT * VP;
            const int p_lo = qpos[16 * warp + (lane >> 2)], p_hi = qpos[16 * warp + (lane >> 2) + 8];
            // every key of the tile visible to every query slot of this warp (inside all of their windows, or all kept first positions): no mask
            const int k_first = kt * WIN_KT, k_last = k_first + WIN_KT - 1;
            const bool whole = k_last <= wp_min && (k_first > wp_max - a.window || k_last < a.keep_first);
            uint32_t pa[MAPS][2][4];        // P of this tile as A fragments, per map and 16-key half
#pragma unroll
            for (int mp = 0; mp < MAPS; ++mp) {
                float s[4][4];
#pragma unroll
                for (int i = 0; i < 4; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
                const uint32_t qa = smem_u32(Qs + (16 * warp + (lane & 15)) * QP + mp * D + (lane >> 4) * 8);
                const uint32_t ka = smem_u32(Kb + ((lane >> 4) * 8 + (lane & 7)) * QP + mp * D + ((lane >> 3) & 1) * 8);
                for (int ks = 0; ks < D / 16; ++ks) {
                    uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
                    ldmatrix_x4(qa + ks * 32, a0, a1, a2, a3);
                    ldmatrix_x4(ka + ks * 32, b0, b1, b2, b3);
                    mma_bf16_16816(s[0], a0, a1, a2, a3, b0, b1); mma_bf16_16816(s[1], a0, a1, a2, a3, b2, b3);
                    ldmatrix_x4(ka + 16 * QP * 2 + ks * 32, b0, b1, b2, b3);
                    mma_bf16_16816(s[2], a0, a1, a2, a3, b0, b1); mma_bf16_16816(s[3], a0, a1, a2, a3, b2, b3);
                }
                if (MOD) {
#pragma unroll
                    for (int nb = 0; nb < 4; ++nb)
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const int key = kt * WIN_KT + nb * 8 + (lane & 3) * 2 + (c & 1);
                            const float v = a.softcap > 0.f ? a.softcap * win_tanh(s[nb][c] * inv_cap) : s[nb][c] * a.scale;
                            s[nb][c] = (v - (c < 2 ? slope_lo * (float)(p_lo - key) : slope_hi * (float)(p_hi - key))) * 1.4426950408889634f;
                        }
                }
                float mx_lo = -INFINITY, mx_hi = -INFINITY;
                if (!whole) {                          // a tile on an edge of the mask: per query position
#pragma unroll
                    for (int nb = 0; nb < 4; ++nb)
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const int key = kt * WIN_KT + nb * 8 + (lane & 3) * 2 + (c & 1), p = c < 2 ? p_lo : p_hi;
                            if (!(key <= p && (p - key < a.window || key < a.keep_first))) s[nb][c] = -INFINITY;
                        }
                }
#pragma unroll
                for (int nb = 0; nb < 4; ++nb) { mx_lo = fmaxf(mx_lo, fmaxf(s[nb][0], s[nb][1])); mx_hi = fmaxf(mx_hi, fmaxf(s[nb][2], s[nb][3])); }
                mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1)); mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
                mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1)); mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
                // the running maximum is kept in scaled base-2 units; the raw scores are scaled inside the exponent's multiply-add.  A tile may
                // hold no visible key for some of its rows (their window starts later): their maximum then stays -inf
                const float n_lo = fmaxf(m_lo[mp], mx_lo * qscale), n_hi = fmaxf(m_hi[mp], mx_hi * qscale);
                const float b_lo = n_lo == -INFINITY ? 0.f : n_lo, b_hi = n_hi == -INFINITY ? 0.f : n_hi;
                const float c_lo = ex2_approx(m_lo[mp] - b_lo), c_hi = ex2_approx(m_hi[mp] - b_hi);
                m_lo[mp] = n_lo; m_hi[mp] = n_hi;
                float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
                for (int nb = 0; nb < 4; ++nb) {
                    s[nb][0] = ex2_approx(fmaf(s[nb][0], qscale, -b_lo)); s[nb][1] = ex2_approx(fmaf(s[nb][1], qscale, -b_lo));
                    s[nb][2] = ex2_approx(fmaf(s[nb][2], qscale, -b_hi)); s[nb][3] = ex2_approx(fmaf(s[nb][3], qscale, -b_hi));
                    sum_lo += s[nb][0] + s[nb][1]; sum_hi += s[nb][2] + s[nb][3];
                }
                l_lo[mp] = l_lo[mp] * c_lo + sum_lo; l_hi[mp] = l_hi[mp] * c_hi + sum_hi;
                if (__any_sync(0xffffffffu, c_lo != 1.f || c_hi != 1.f)) {      // no row's maximum rose: the sums keep their scale
#pragma unroll
                    for (int i = 0; i < NVB; ++i) { o[mp][i][0] *= c_lo; o[mp][i][1] *= c_lo; o[mp][i][2] *= c_hi; o[mp][i][3] *= c_hi; }
                }
#pragma unroll
                for (int kk = 0; kk < 2; ++kk) {
                    pa[mp][kk][0] = pack_bf16x2(s[2 * kk][0], s[2 * kk][1]); pa[mp][kk][1] = pack_bf16x2(s[2 * kk][2], s[2 * kk][3]);
                    pa[mp][kk][2] = pack_bf16x2(s[2 * kk + 1][0], s[2 * kk + 1][1]); pa[mp][kk][3] = pack_bf16x2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
                }
            }
            const uint32_t va = smem_u32(Vb + (((lane >> 3) & 1) * 8 + (lane & 7)) * VP + (lane >> 4) * 8);
#pragma unroll
            for (int kk = 0; kk < 2; ++kk)
#pragma unroll
                for (int np = 0; np < NVB / 2; ++np) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(va + kk * 16 * VP * 2 + np * 32, b0, b1, b2, b3);      // one value fragment serves both maps
#pragma unroll
                    for (int mp = 0; mp < MAPS; ++mp) {
                        mma_bf16_16816(o[mp][2 * np], pa[mp][kk][0], pa[mp][kk][1], pa[mp][kk][2], pa[mp][kk][3], b0, b1);
                        mma_bf16_16816(o[mp][2 * np + 1], pa[mp][kk][0], pa[mp][kk][1], pa[mp][kk][2], pa[mp][kk][3], b2, b3);
                    }
                }
        }
        __syncthreads();
    }
    if (!active) return;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int qi = 16 * warp + (lane >> 2) + half * 8;
        const bool ok = qi < nq;                       // every lane stays for the quad shuffles
        const int row = row0 + (q0 + (ok ? qi : 0)) / HG, head = g * HG + (q0 + (ok ? qi : 0)) % HG;
        float f[MAPS];
#pragma unroll
        for (int mp = 0; mp < MAPS; ++mp) {
            float l = half ? l_hi[mp] : l_lo[mp]; const float m = half ? m_hi[mp] : m_lo[mp];
            l += __shfl_xor_sync(0xffffffffu, l, 1); l += __shfl_xor_sync(0xffffffffu, l, 2);
            float up = 1.f;
            if (sink) {                                // the sink joins the denominator (scores are kept in base-2 units)
                const float s2 = sink[head] * 1.4426950408889634f, M = fmaxf(m, s2);
                up = m == -INFINITY ? 0.f : ex2_approx(m - M); l = l * up + ex2_approx(s2 - M);
            }
            f[mp] = l > 0.f ? up / l : 0.f;
        }
        float y[NVB][2], ss = 0.f;
#pragma unroll
        for (int nb = 0; nb < NVB; ++nb)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                float v = o[0][nb][half * 2 + e] * f[0];
                if (MAPS == 2) v -= a.lambda * (o[MAPS - 1][nb][half * 2 + e] * f[MAPS - 1]);
                y[nb][e] = v; ss = fmaf(v, v, ss);
            }
        float post = 1.f;
        if (MAPS == 2) {
            ss += __shfl_xor_sync(0xffffffffu, ss, 1); ss += __shfl_xor_sync(0xffffffffu, ss, 2);
            post = a.out_scale / sqrtf(ss / (float)VD + eps);
        }
        if (!ok) continue;
        if (a.out_rot) {               // the head's output turned back by the row's position; both channels of a pair sit in this thread
            const int vh = VD / 2, pos = r.positions[row]; const float* cs = a.out_cos + (long long)pos * vh; const float* sn = a.out_sin + (long long)pos * vh;
            if (a.out_rot == 1) {
#pragma unroll
                for (int nb = 0; nb < NVB; ++nb) { const int m = nb * 4 + (lane & 3); const float u = y[nb][0] * post, v = y[nb][1] * post; y[nb][0] = u * cs[m] + v * sn[m]; y[nb][1] = v * cs[m] - u * sn[m]; }
            } else {
#pragma unroll
                for (int nb = 0; nb < NVB / 2; ++nb)
#pragma unroll
                    for (int e = 0; e < 2; ++e) { const int m = nb * 8 + (lane & 3) * 2 + e; const float u = y[nb][e] * post, v = y[nb + NVB / 2][e] * post; y[nb][e] = u * cs[m] + v * sn[m]; y[nb + NVB / 2][e] = v * cs[m] - u * sn[m]; }
            }
            post = 1.f;
        }
        if (a.gate == 2) post *= sigmoidf_(__bfloat162float(gate[(long long)row * ldg + head]));
        __nv_bfloat16* dst = out + (long long)row * ldo + (long long)head * VD + (lane & 3) * 2;
        const __nv_bfloat16* gp = gate + (long long)row * ldg + (long long)head * VD + (lane & 3) * 2;
#pragma unroll
        for (int nb = 0; nb < NVB; ++nb) {
            float y0 = y[nb][0] * post, y1 = y[nb][1] * post;
            if (a.gate == 1) { const uint32_t gg = *reinterpret_cast<const uint32_t*>(gp + nb * 8); y0 *= sigmoidf_(bf16lo(gg)); y1 *= sigmoidf_(bf16hi(gg)); }
            *reinterpret_cast<uint32_t*>(dst + nb * 8) = pack_bf16x2(y0, y1);
        }
    }
}

// Decoding form of the same computation, for tiles of at most 16 query slots (a decoding row's group of heads, or a very short portion): the
// prefill form above would leave three of its four warps idle and walk the window tile by tile on one warp.  Here the CTA's eight warps
// deal the visible key tiles out among themselves (warp w takes tiles w, w + 8, ...), each with its own shared-memory tile and its own
// online softmax over the same 16 query slots; the partial sums, maxima and denominators then meet in shared memory and 16 threads per
// query slot join them in warp order and finish the head (sink, a1 - lambda a2, unit RMS, gate).  Which tiles a warp takes depends on the
// row's position only.
constexpr int WIN_DEC_WARPS = 8;
template <int MAPS, int NVB, bool MOD>
__global__ void __launch_bounds__(256) hy_win_decode_mma_kernel(HyWinAttn a, const __nv_bfloat16* __restrict__ q, int ldq, const __nv_bfloat16* __restrict__ cache,
                                                                const float* __restrict__ sink, const __nv_bfloat16* __restrict__ gate, int ldg,
                                                                __nv_bfloat16* __restrict__ out, int ldo, float eps, HyRows r, const int32_t* __restrict__ tile_seq,
                                                                const int32_t* __restrict__ tile_q0) {
    HY_PDL();
    extern __shared__ __align__(16) uint8_t win_smem[];
    __shared__ float pm[WIN_DEC_WARPS][MAPS][16], pl[WIN_DEC_WARPS][MAPS][16];
    __shared__ int qpos[16];
    constexpr int VD = NVB * 8, VP = VD + 8;
    const int D = a.dim, QD = MAPS * D, QP = QD + 8, HG = a.heads / a.kv_heads, g = blockIdx.y;
    const int KW = a.kv_heads * QD, CW = KW + a.kv_heads * VD;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(win_smem);      // [16][QP]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    __nv_bfloat16* Kw = Qs + 16 * QP + (size_t)warp * WIN_KT * (QP + VP);     // this warp's tile: [32][QP] keys, [32][VP] values
    __nv_bfloat16* Vw = Kw + WIN_KT * QP;
    float* po = reinterpret_cast<float*>(Qs + 16 * QP);                  // after the loop: [warps][MAPS][16][VD] partial sums over the tile buffers
    const int seq = tile_seq[blockIdx.x], q0 = tile_q0[blockIdx.x];
    const int row0 = r.seq_row0[seq], len = r.seq_row0[seq + 1] - row0;
    const int nq = min(16, len * HG - q0);
    for (int idx = tid; idx < 16 * (QD / 8); idx += 256) {
        const int qi = idx / (QD / 8), c = idx - qi * (QD / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (qi < nq) v = *reinterpret_cast<const uint4*>(q + (long long)(row0 + (q0 + qi) / HG) * ldq + (long long)(g * HG + (q0 + qi) % HG) * QD + c * 8);
        *reinterpret_cast<uint4*>(Qs + qi * QP + c * 8) = v;
    }
    if (tid < 16) qpos[tid] = tid < nq ? r.positions[row0 + (q0 + tid) / HG] : -1;
    __syncthreads();
    const int pos_min = r.positions[row0 + q0 / HG], pos_max = r.positions[row0 + (q0 + nq - 1) / HG];
    const int lo_min = max(0, pos_min - a.window + 1);
    const int win_t0 = lo_min / WIN_KT, n_kt = pos_max / WIN_KT + 1;
    const int n_keep = min((min(a.keep_first, lo_min) + WIN_KT - 1) / WIN_KT, win_t0);
    const int n_it = n_keep + (n_kt - win_t0);
    const int32_t* bt = r.block_tables + (long long)seq * r.max_pages_per_seq;
    float o[MAPS][NVB][4];
    float m_lo[MAPS], m_hi[MAPS], l_lo[MAPS], l_hi[MAPS];
#pragma unroll
    for (int mp = 0; mp < MAPS; ++mp) {
        m_lo[mp] = m_hi[mp] = -INFINITY; l_lo[mp] = l_hi[mp] = 0.f;
#pragma unroll
        for (int i = 0; i < NVB; ++i) { o[mp][i][0] = o[mp][i][1] = o[mp][i][2] = o[mp][i][3] = 0.f; }
    }
    const float qscale = a.scale * 1.4426950408889634f;
    const float inv_cap = a.softcap > 0.f ? a.scale / a.softcap : 0.f;
    const float slope_lo = MOD ? win_head_slope(a, g * HG + (q0 + (lane >> 2)) % HG) : 0.f, slope_hi = MOD ? win_head_slope(a, g * HG + (q0 + (lane >> 2) + 8) % HG) : 0.f;
    const int p_lo = qpos[lane >> 2], p_hi = qpos[(lane >> 2) + 8];
    const int kc = QD / 8, nc = kc + VD / 8, step_j = 32 / nc, step_c = 32 % nc, j0 = lane / nc, c0 = lane % nc;      // a lane walks its warp's tile chunks in steps of 32
    for (int it = warp; it < n_it; it += WIN_DEC_WARPS) {
        const int kt = it < n_keep ? it : win_t0 + (it - n_keep);
        __syncwarp();                                  // the previous tile has been read by every lane
        {
            const int key0 = kt * WIN_KT;              // the tile's 32 keys lie in one page
            const __nv_bfloat16* page = cache + ((long long)bt[key0 >> 6] * 64 + (key0 & 63)) * CW;
            int j = j0, c = c0;
            while (j < WIN_KT) {
                __nv_bfloat16* dst = c < kc ? Kw + j * QP + c * 8 : Vw + j * VP + (c - kc) * 8;
                if (key0 + j <= pos_max) cp_async16(dst, page + (long long)j * CW + (c < kc ? g * QD + c * 8 : KW + g * VD + (c - kc) * 8));
                else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
                j += step_j; c += step_c;
                if (c >= nc) { c -= nc; ++j; }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncwarp();
        uint32_t pa[MAPS][2][4];
#pragma unroll
        for (int mp = 0; mp < MAPS; ++mp) {
            float s[4][4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
            const uint32_t qa = smem_u32(Qs + (lane & 15) * QP + mp * D + (lane >> 4) * 8);
            const uint32_t ka = smem_u32(Kw + ((lane >> 4) * 8 + (lane & 7)) * QP + mp * D + ((lane >> 3) & 1) * 8);
            for (int ks = 0; ks < D / 16; ++ks) {
                uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
                ldmatrix_x4(qa + ks * 32, a0, a1, a2, a3);
                ldmatrix_x4(ka + ks * 32, b0, b1, b2, b3);
                mma_bf16_16816(s[0], a0, a1, a2, a3, b0, b1); mma_bf16_16816(s[1], a0, a1, a2, a3, b2, b3);
                ldmatrix_x4(ka + 16 * QP * 2 + ks * 32, b0, b1, b2, b3);
                mma_bf16_16816(s[2], a0, a1, a2, a3, b0, b1); mma_bf16_16816(s[3], a0, a1, a2, a3, b2, b3);
            }
            float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
            for (int nb = 0; nb < 4; ++nb)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int key = kt * WIN_KT + nb * 8 + (lane & 3) * 2 + (c & 1), p = c < 2 ? p_lo : p_hi;
                    const bool vis = key <= p && (p - key < a.window || key < a.keep_first);
                    if (MOD) {
                        const float v = a.softcap > 0.f ? a.softcap * win_tanh(s[nb][c] * inv_cap) : s[nb][c] * a.scale;
                        s[nb][c] = vis ? (v - (c < 2 ? slope_lo : slope_hi) * (float)(p - key)) * 1.4426950408889634f : -INFINITY;
                    } else
                    s[nb][c] = vis ? s[nb][c] * qscale : -INFINITY;
                    if (c < 2) mx_lo = fmaxf(mx_lo, s[nb][c]); else mx_hi = fmaxf(mx_hi, s[nb][c]);
                }
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1)); mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1)); mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
            const float n_lo = fmaxf(m_lo[mp], mx_lo), n_hi = fmaxf(m_hi[mp], mx_hi);
            const float b_lo = n_lo == -INFINITY ? 0.f : n_lo, b_hi = n_hi == -INFINITY ? 0.f : n_hi;
            const float c_lo = ex2_approx(m_lo[mp] - b_lo), c_hi = ex2_approx(m_hi[mp] - b_hi);
            m_lo[mp] = n_lo; m_hi[mp] = n_hi;
            float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
            for (int nb = 0; nb < 4; ++nb) {
                s[nb][0] = ex2_approx(s[nb][0] - b_lo); s[nb][1] = ex2_approx(s[nb][1] - b_lo); s[nb][2] = ex2_approx(s[nb][2] - b_hi); s[nb][3] = ex2_approx(s[nb][3] - b_hi);
                sum_lo += s[nb][0] + s[nb][1]; sum_hi += s[nb][2] + s[nb][3];
            }
            l_lo[mp] = l_lo[mp] * c_lo + sum_lo; l_hi[mp] = l_hi[mp] * c_hi + sum_hi;
#pragma unroll
            for (int i = 0; i < NVB; ++i) { o[mp][i][0] *= c_lo; o[mp][i][1] *= c_lo; o[mp][i][2] *= c_hi; o[mp][i][3] *= c_hi; }
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
                pa[mp][kk][0] = pack_bf16x2(s[2 * kk][0], s[2 * kk][1]); pa[mp][kk][1] = pack_bf16x2(s[2 * kk][2], s[2 * kk][3]);
                pa[mp][kk][2] = pack_bf16x2(s[2 * kk + 1][0], s[2 * kk + 1][1]); pa[mp][kk][3] = pack_bf16x2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
            }
        }
        const uint32_t va = smem_u32(Vw + (((lane >> 3) & 1) * 8 + (lane & 7)) * VP + (lane >> 4) * 8);
#pragma unroll
        for (int kk = 0; kk < 2; ++kk)
#pragma unroll
            for (int np = 0; np < NVB / 2; ++np) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(va + kk * 16 * VP * 2 + np * 32, b0, b1, b2, b3);
#pragma unroll
                for (int mp = 0; mp < MAPS; ++mp) {
                    mma_bf16_16816(o[mp][2 * np], pa[mp][kk][0], pa[mp][kk][1], pa[mp][kk][2], pa[mp][kk][3], b0, b1);
                    mma_bf16_16816(o[mp][2 * np + 1], pa[mp][kk][0], pa[mp][kk][1], pa[mp][kk][2], pa[mp][kk][3], b2, b3);
                }
            }
    }
    __syncthreads();                                   // every warp is done with its tile buffer: the partials go over them
#pragma unroll
    for (int mp = 0; mp < MAPS; ++mp) {
        float ll = l_lo[mp], lh = l_hi[mp];
        ll += __shfl_xor_sync(0xffffffffu, ll, 1); ll += __shfl_xor_sync(0xffffffffu, ll, 2);
        lh += __shfl_xor_sync(0xffffffffu, lh, 1); lh += __shfl_xor_sync(0xffffffffu, lh, 2);
        if ((lane & 3) == 0) { pm[warp][mp][lane >> 2] = m_lo[mp]; pm[warp][mp][(lane >> 2) + 8] = m_hi[mp]; pl[warp][mp][lane >> 2] = ll; pl[warp][mp][(lane >> 2) + 8] = lh; }
        float* dst = po + ((size_t)(warp * MAPS + mp) * 16 + (lane >> 2)) * VD + (lane & 3) * 2;
#pragma unroll
        for (int nb = 0; nb < NVB; ++nb) {
            *reinterpret_cast<float2*>(dst + nb * 8) = make_float2(o[mp][nb][0], o[mp][nb][1]);
            *reinterpret_cast<float2*>(dst + 8 * VD + nb * 8) = make_float2(o[mp][nb][2], o[mp][nb][3]);
        }
    }
    __syncthreads();
    // 16 threads per query slot: channels sub, sub + 16, ...
    const int qi = tid >> 4, sub = tid & 15;
    const bool ok = qi < nq;
    const int row = row0 + (q0 + (ok ? qi : 0)) / HG, head = g * HG + (q0 + (ok ? qi : 0)) % HG;
    float wgt[MAPS][WIN_DEC_WARPS], inv[MAPS];
#pragma unroll
    for (int mp = 0; mp < MAPS; ++mp) {
        float M = sink ? sink[head] * 1.4426950408889634f : -INFINITY, L = 0.f;
#pragma unroll
        for (int w = 0; w < WIN_DEC_WARPS; ++w) M = fmaxf(M, pm[w][mp][qi]);
#pragma unroll
        for (int w = 0; w < WIN_DEC_WARPS; ++w) { wgt[mp][w] = pm[w][mp][qi] == -INFINITY ? 0.f : ex2_approx(pm[w][mp][qi] - M); L = fmaf(wgt[mp][w], pl[w][mp][qi], L); }
        if (sink) L += ex2_approx(sink[head] * 1.4426950408889634f - M);
        inv[mp] = L > 0.f ? 1.0f / L : 0.f;
    }
    float y[NVB / 2], ss = 0.f;
#pragma unroll
    for (int i = 0; i < NVB / 2; ++i) {
        const int c = sub + 16 * i;
        float v[MAPS];
#pragma unroll
        for (int mp = 0; mp < MAPS; ++mp) {
            float acc = 0.f;
#pragma unroll
            for (int w = 0; w < WIN_DEC_WARPS; ++w) acc = fmaf(wgt[mp][w], po[((size_t)(w * MAPS + mp) * 16 + qi) * VD + c], acc);
            v[mp] = acc * inv[mp];
        }
        y[i] = MAPS == 2 ? v[0] - a.lambda * v[MAPS - 1] : v[0];
        ss = fmaf(y[i], y[i], ss);
    }
    float post = 1.f;
    if (MAPS == 2) {
#pragma unroll
        for (int sh = 1; sh < 16; sh <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, sh);
        post = a.out_scale / sqrtf(ss / (float)VD + eps);
    }
    if (a.out_rot == 1) {              // the head's output turned back by the row's position: channel c meets c ^ 1 in the neighbouring lane
        const int vh = VD / 2, pos = r.positions[row]; const float* cs = a.out_cos + (long long)pos * vh; const float* sn = a.out_sin + (long long)pos * vh;
#pragma unroll
        for (int i = 0; i < NVB / 2; ++i) {
            const int c = sub + 16 * i; const float mine = y[i] * post, other = __shfl_xor_sync(0xffffffffu, mine, 1);
            y[i] = (c & 1) ? mine * cs[c >> 1] - other * sn[c >> 1] : mine * cs[c >> 1] + other * sn[c >> 1];
        }
        post = 1.f;
    }
    if (!ok) return;
    if (a.gate == 2) post *= sigmoidf_(__bfloat162float(gate[(long long)row * ldg + head]));
#pragma unroll
    for (int i = 0; i < NVB / 2; ++i) {
        const int c = sub + 16 * i;
        float v = y[i] * post;
        if (a.gate == 1) v *= sigmoidf_(__bfloat162float(gate[(long long)row * ldg + (long long)head * VD + c]));
        out[(long long)row * ldo + (long long)head * VD + c] = __float2bfloat16_rn(v);
    }
}

}  // namespace

cudaError_t hy_rmsnorm_pair(bool f32, const float* x, const int32_t* rows, const float* w1, void* out1, const float* w2, void* out2, int ldo, int T, int W, float eps, cudaStream_t s) {
    if (T <= 0) return cudaSuccess;
    return f32 ? launch_plain(hy_rmsnorm_pair_kernel<float>, dim3(T), dim3(256), 0, s, x, rows, w1, (float*)out1, w2, (float*)out2, ldo, W, eps)
               : launch_plain(hy_rmsnorm_pair_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, s, x, rows, w1, (__nv_bfloat16*)out1, w2, (__nv_bfloat16*)out2, ldo, W, eps);
}

cudaError_t hy_win_prep(bool f32, const HyWinAttn& a, void* q, int ldq, const void* k, const void* v, int ldkv, const float* q_norm_w, const float* k_norm_w, float eps, void* cache,
                        const HyRows& r, cudaStream_t s) {
    if (r.T <= 0 || (!a.qk_norm && !k && a.q_temp_every <= 0)) return cudaSuccess;
    using bf = __nv_bfloat16;
    if (a.qk_norm == 2 && !f32 && (a.heads * a.maps * a.dim) % 8 == 0 && (a.kv_heads * a.maps * a.dim) % 8 == 0 && (a.kv_heads * a.vdim) % 8 == 0 && ldq % 8 == 0 && ldkv % 8 == 0 &&
        ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(cache) | reinterpret_cast<uintptr_t>(q_norm_w) |
          reinterpret_cast<uintptr_t>(k_norm_w)) & 15) == 0)
        return launch_plain(hy_win_prep_whole_vec8_kernel, dim3(r.T), dim3(128), 0, s, a, (bf*)q, ldq, (const bf*)k, (const bf*)v, ldkv, q_norm_w, k_norm_w, eps, (bf*)cache, r);
    if (a.qk_norm == 2)
        return f32 ? launch_plain(hy_win_prep_whole_kernel<float>, dim3(r.T), dim3(128), 0, s, a, (float*)q, ldq, (const float*)k, (const float*)v, ldkv, q_norm_w, k_norm_w, eps, (float*)cache, r)
                   : launch_plain(hy_win_prep_whole_kernel<bf>, dim3(r.T), dim3(128), 0, s, a, (bf*)q, ldq, (const bf*)k, (const bf*)v, ldkv, q_norm_w, k_norm_w, eps, (bf*)cache, r);
    if (a.q_temp_every > 0) return cudaErrorInvalidValue;      // the query temperature is applied by the whole-projection form only
    const int gs = a.dim / 8;
    const bool aligned = ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(cache) |
                           reinterpret_cast<uintptr_t>(q_norm_w) | reinterpret_cast<uintptr_t>(k_norm_w)) & 15) == 0;
    if (!f32 && a.dim % 8 == 0 && gs <= 32 && (gs & (gs - 1)) == 0 && a.vdim % 8 == 0 && ldq % 8 == 0 && ldkv % 8 == 0 && aligned)
        return launch_plain(hy_win_prep_vec8_kernel, dim3(r.T), dim3(128), 0, s, a, (bf*)q, ldq, (const bf*)k, (const bf*)v, ldkv, q_norm_w, k_norm_w, eps, (bf*)cache, r);
    return f32 ? launch_plain(hy_win_prep_kernel<float>, dim3(r.T), dim3(128), 0, s, a, (float*)q, ldq, (const float*)k, (const float*)v, ldkv, q_norm_w, k_norm_w, eps, (float*)cache, r)
               : launch_plain(hy_win_prep_kernel<bf>, dim3(r.T), dim3(128), 0, s, a, (bf*)q, ldq, (const bf*)k, (const bf*)v, ldkv, q_norm_w, k_norm_w, eps, (bf*)cache, r);
}

cudaError_t hy_win_rope_prep(bool f32, const HyWinAttn& a, const HyRotary& rot, void* q, int ldq, const void* k, const void* v, int ldkv, void* cache, const HyRows& r, cudaStream_t s) {
    if (a.maps != 1 || a.qk_norm || (rot.dims & 1) || rot.dims > a.dim || (rot.v_cos && (a.vdim & 1))) return cudaErrorInvalidValue;
    return f32 ? launch_plain(hy_win_rope_prep_kernel<float>, dim3(r.T), dim3(128), 0, s, a, rot, (float*)q, ldq, (const float*)k, (const float*)v, ldkv, (float*)cache, r)
               : launch_plain(hy_win_rope_prep_kernel<__nv_bfloat16>, dim3(r.T), dim3(128), 0, s, a, rot, (__nv_bfloat16*)q, ldq, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, ldkv, (__nv_bfloat16*)cache, r);
}
bool hy_conv_rope_cache_supported(const HyWinAttn& a, const HyRotary& rot, int taps) {
    return a.maps == 1 && !a.qk_norm && taps >= 2 && taps <= 4 && a.dim % 8 == 0 && a.vdim % 8 == 0 && rot.layout == 0 && rot.dims % 2 == 0 && rot.dims <= a.dim;
}
template <int TAPS>
static cudaError_t conv_rope_launch(const HyWinAttn& a, const HyRotary& rot, const void* in, int ld_in, int C, int off_q, int off_k, int off_v, const float* w, void* q_out, int ldq, void* cache,
                                    const void* tails, const HyRows& r, cudaStream_t s) {
    using bf = __nv_bfloat16;
    if (r.T >= 512) return launch_plain(hy_conv_rope_cache_kernel<TAPS, 16>, dim3((C / 8 + 127) / 128, (r.T + 15) / 16), dim3(128), 0, s, a, rot, (const bf*)in, ld_in, C, off_q, off_k, off_v, w,
                                        (bf*)q_out, ldq, (bf*)cache, (const bf*)tails, r);
    return launch_plain(hy_conv_rope_cache_kernel<TAPS, 1>, dim3((C / 8 + 127) / 128, r.T), dim3(128), 0, s, a, rot, (const bf*)in, ld_in, C, off_q, off_k, off_v, w, (bf*)q_out, ldq,
                        (bf*)cache, (const bf*)tails, r);
}
cudaError_t hy_conv_rope_cache(const HyWinAttn& a, const HyRotary& rot, const void* in, int ld_in, int C, int off_q, int off_k, int off_v, const float* w, int taps, void* q_out, int ldq,
                               void* cache, const void* tails, const HyRows& r, cudaStream_t s) {
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (!hy_conv_rope_cache_supported(a, rot, taps) || C % 8 || ld_in % 8 || ldq % 8 || off_q % 8 || off_k % 8 || off_v % 8 || !al16(in) || !al16(q_out) || !al16(cache) || !al16(tails))
        return cudaErrorInvalidValue;
    switch (taps) {
        case 2: return conv_rope_launch<2>(a, rot, in, ld_in, C, off_q, off_k, off_v, w, q_out, ldq, cache, tails, r, s);
        case 3: return conv_rope_launch<3>(a, rot, in, ld_in, C, off_q, off_k, off_v, w, q_out, ldq, cache, tails, r, s);
        default: return conv_rope_launch<4>(a, rot, in, ld_in, C, off_q, off_k, off_v, w, q_out, ldq, cache, tails, r, s);
    }
}
bool hy_win_supported(const HyWinAttn& a) {
    return a.maps >= 1 && a.maps <= 2 && a.vdim <= 32 * WIN_MAXV && a.dim >= 1 && a.heads % a.kv_heads == 0 &&
           (size_t)(a.maps * a.dim + 4 * a.maps * a.vdim + 8 * a.maps) * 4 <= 200 * 1024;
}

cudaError_t hy_win_attention(bool f32, const HyWinAttn& a, const void* q, int ldq, const void* cache, const float* sink, const void* gate, int ldg, void* out, int ldo, float eps,
                             const HyRows& r, cudaStream_t s) {
    if (r.T <= 0) return cudaSuccess;
    if (!hy_win_supported(a)) return cudaErrorInvalidValue;
    using bf = __nv_bfloat16;
    const size_t smem = (size_t)(a.maps * a.dim + 4 * a.maps * a.vdim + 8 * a.maps) * 4;
    if (smem > 48 * 1024) {
        cudaError_t e = f32 ? cudaFuncSetAttribute(hy_win_attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                            : cudaFuncSetAttribute(hy_win_attention_kernel<bf>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    return f32 ? launch_plain(hy_win_attention_kernel<float>, dim3(r.T, a.heads), dim3(128), smem, s, a, (const float*)q, ldq, (const float*)cache, sink, (const float*)gate, ldg,
                              (float*)out, ldo, eps, r)
               : launch_plain(hy_win_attention_kernel<bf>, dim3(r.T, a.heads), dim3(128), smem, s, a, (const bf*)q, ldq, (const bf*)cache, sink, (const bf*)gate, ldg, (bf*)out, ldo,
                              eps, r);
}

static bool win_modded(const HyWinAttn& a) { return a.softcap > 0.f || a.slope_exp > 0.f; }
bool hy_win_mma_supported(const HyWinAttn& a) {
    const bool vd_ok = a.vdim == 16 || a.vdim == 32 || a.vdim == 64 || a.vdim == 96 || a.vdim == 128;
    return hy_win_supported(a) && a.dim % 16 == 0 && a.dim <= 128 && vd_ok && !(win_modded(a) && a.maps != 1) && a.out_rot != 2;      // score modifiers on the tensor cores: one map; outputs turned back in pairs of neighbours only
}
template <int MAPS, int NVB, bool MOD>
static cudaError_t win_mma_launch(const HyWinAttn& a, const void* q, int ldq, const void* cache, const float* sink, const void* gate, int ldg, void* out, int ldo, float eps,
                                  const HyRows& r, const int32_t* tile_seq, const int32_t* tile_q0, int n_tiles, cudaStream_t s) {
    using bf = __nv_bfloat16;
    const int QP = MAPS * a.dim + 8, VP = NVB * 8 + 8;
    const size_t smem = (size_t)(WIN_MQ * QP + 2 * WIN_KT * QP + 2 * WIN_KT * VP) * 2 + WIN_MQ * 4;
    static size_t raised = 0;          // per instantiation
    if (smem > 48 * 1024 && smem > raised) {
        cudaError_t e = cudaFuncSetAttribute(hy_win_attention_mma_kernel<MAPS, NVB, MOD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        raised = smem;
    }
    return launch_plain(hy_win_attention_mma_kernel<MAPS, NVB, MOD>, dim3(n_tiles, a.kv_heads), dim3(128), smem, s, a, (const bf*)q, ldq, (const bf*)cache, sink, (const bf*)gate, ldg,
                        (bf*)out, ldo, eps, r, tile_seq, tile_q0);
}
template <int MAPS, int NVB, bool MOD>
static cudaError_t win_decode_launch(const HyWinAttn& a, const void* q, int ldq, const void* cache, const float* sink, const void* gate, int ldg, void* out, int ldo, float eps,
                                     const HyRows& r, const int32_t* tile_seq, const int32_t* tile_q0, int n_tiles, cudaStream_t s) {
    using bf = __nv_bfloat16;
    const int QP = MAPS * a.dim + 8, VP = NVB * 8 + 8;
    const size_t tiles = (size_t)WIN_DEC_WARPS * WIN_KT * (QP + VP) * 2, parts = (size_t)WIN_DEC_WARPS * MAPS * 16 * NVB * 8 * 4;
    const size_t smem = (size_t)16 * QP * 2 + (tiles > parts ? tiles : parts);
    static size_t raised = 0;
    if (smem > 48 * 1024 && smem > raised) {
        cudaError_t e = cudaFuncSetAttribute(hy_win_decode_mma_kernel<MAPS, NVB, MOD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        raised = smem;
    }
    return launch_plain(hy_win_decode_mma_kernel<MAPS, NVB, MOD>, dim3(n_tiles, a.kv_heads), dim3(256), smem, s, a, (const bf*)q, ldq, (const bf*)cache, sink, (const bf*)gate, ldg,
                        (bf*)out, ldo, eps, r, tile_seq, tile_q0);
}
cudaError_t hy_win_attention_mma(const HyWinAttn& a, const void* q, int ldq, const void* cache, const float* sink, const void* gate, int ldg, void* out, int ldo, float eps,
                                 const HyRows& r, const int32_t* tile_seq, const int32_t* tile_q0, int n_tiles, cudaStream_t s) {
    if (n_tiles <= 0) return cudaSuccess;
    if (!hy_win_mma_supported(a)) return cudaErrorInvalidValue;
#define WIN_CASE(M, N) if (a.maps == M && a.vdim == N * 8) return win_mma_launch<M, N, false>(a, q, ldq, cache, sink, gate, ldg, out, ldo, eps, r, tile_seq, tile_q0, n_tiles, s)
#define WIN_CASE_MOD(N) if (a.vdim == N * 8) return win_mma_launch<1, N, true>(a, q, ldq, cache, sink, gate, ldg, out, ldo, eps, r, tile_seq, tile_q0, n_tiles, s)
    if (win_modded(a)) { WIN_CASE_MOD(2); WIN_CASE_MOD(4); WIN_CASE_MOD(8); WIN_CASE_MOD(12); WIN_CASE_MOD(16); return cudaErrorInvalidValue; }
    WIN_CASE(1, 2); WIN_CASE(1, 4); WIN_CASE(1, 8); WIN_CASE(1, 12); WIN_CASE(1, 16);
    WIN_CASE(2, 2); WIN_CASE(2, 4); WIN_CASE(2, 8); WIN_CASE(2, 12); WIN_CASE(2, 16);
#undef WIN_CASE
#undef WIN_CASE_MOD
    return cudaErrorInvalidValue;
}
cudaError_t hy_win_decode_mma(const HyWinAttn& a, const void* q, int ldq, const void* cache, const float* sink, const void* gate, int ldg, void* out, int ldo, float eps,
                              const HyRows& r, const int32_t* tile_seq, const int32_t* tile_q0, int n_tiles, cudaStream_t s) {
    if (n_tiles <= 0) return cudaSuccess;
    if (!hy_win_mma_supported(a)) return cudaErrorInvalidValue;
#define WIN_CASE(M, N) if (a.maps == M && a.vdim == N * 8) return win_decode_launch<M, N, false>(a, q, ldq, cache, sink, gate, ldg, out, ldo, eps, r, tile_seq, tile_q0, n_tiles, s)
#define WIN_CASE_MOD(N) if (a.vdim == N * 8) return win_decode_launch<1, N, true>(a, q, ldq, cache, sink, gate, ldg, out, ldo, eps, r, tile_seq, tile_q0, n_tiles, s)
    if (win_modded(a)) { WIN_CASE_MOD(2); WIN_CASE_MOD(4); WIN_CASE_MOD(8); WIN_CASE_MOD(12); WIN_CASE_MOD(16); return cudaErrorInvalidValue; }
    WIN_CASE(1, 2); WIN_CASE(1, 4); WIN_CASE(1, 8); WIN_CASE(1, 12); WIN_CASE(1, 16);
    WIN_CASE(2, 2); WIN_CASE(2, 4); WIN_CASE(2, 8); WIN_CASE(2, 12); WIN_CASE(2, 16);
#undef WIN_CASE
#undef WIN_CASE_MOD
    return cudaErrorInvalidValue;
}

}  // namespace oa
