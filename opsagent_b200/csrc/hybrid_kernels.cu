// hybrid_kernels.cu — see hybrid_kernels.hpp.  Plain CUDA kernels, one per mechanism, written for any sizes a configuration may give.
// TA is the activation / matrix element type (__nv_bfloat16 or float); all arithmetic is fp32.
#include <cuda_bf16.h>
#include <math.h>

#include <utility>

#include "hybrid_kernels.hpp"
#include "hybrid_common.cuh"

namespace oa {

namespace {

using namespace hyk;

// ---------------------------------------------------------------------------------------------------------------------------------
// GEMM: 64 x 64 tile, 16-wide k slices, 256 threads x (4 x 4) outputs.  The k order of every output is fixed (0..K-1), so a row's result
// does not depend on which other rows share its launch.
// ---------------------------------------------------------------------------------------------------------------------------------
template <typename TA, int MODE>
__global__ void __launch_bounds__(256) hy_gemm_kernel(const TA* __restrict__ A, int lda, const TA* __restrict__ B, int ldb, void* Cv, int ldc, int M, int N, int K,
                                                      const float* __restrict__ bias, float alpha, long long sA, long long sB, long long sC, int act) {
    HY_PDL();
    __shared__ float As[16][64 + 4], Bs[16][64 + 4];
    A += (long long)blockIdx.z * sA; B += (long long)blockIdx.z * sB;
    const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64, tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += 16) {
        for (int i = tid; i < 64 * 16; i += 256) {
            const int r = i >> 4, k = i & 15;
            As[k][r] = (m0 + r < M && k0 + k < K) ? ldf(A + (long long)(m0 + r) * lda + k0 + k) : 0.f;
            Bs[k][r] = (n0 + r < N && k0 + k < K) ? ldf(B + (long long)(n0 + r) * ldb + k0 + k) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { a[i] = As[k][ty * 4 + i]; b[i] = Bs[k][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j] * alpha + (bias ? bias[n] : 0.f);
            if (act == 1) { v = fmaxf(v, 0.f); v *= v; }
            else if (act == 2) v = gelu_tanhf_(v);
            const long long at = (long long)blockIdx.z * sC + (long long)m * ldc + n;
            if (MODE == HY_STORE) stf(reinterpret_cast<TA*>(Cv) + at, v);
            else if (MODE == HY_STORE_F32) reinterpret_cast<float*>(Cv)[at] = v;
            else reinterpret_cast<float*>(Cv)[at] += v;
        }
    }
}

// The same product for a handful of rows (decoding steps), bf16 operands with K in aligned groups of 8: one warp per output column keeps
// its row of B in registers (K <= 1024: four 16-byte pieces per lane) and walks the M rows of A; a lane sums its pieces in order, then the
// warp joins by a butterfly, so a row's result does not depend on the other rows.  The tile kernel above leaves most of a 64-row tile empty
// at these sizes and runs K / 16 barrier-separated slices on a few CTAs.
template <int MODE>
__global__ void __launch_bounds__(256) hy_gemm_fewrows_kernel(const __nv_bfloat16* __restrict__ A, int lda, const __nv_bfloat16* __restrict__ B, int ldb, void* Cv, int ldc, int M, int N,
                                                              int K, const float* __restrict__ bias, float alpha, long long sA, long long sB, long long sC, int act) {
    HY_PDL();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n = blockIdx.x * 8 + warp;
    if (n >= N) return;
    A += (long long)blockIdx.y * sA; B += (long long)blockIdx.y * sB;
    uint4 b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) { const int k = (lane + 32 * i) * 8; b[i] = k < K ? *reinterpret_cast<const uint4*>(B + (long long)n * ldb + k) : make_uint4(0, 0, 0, 0); }
    for (int m = 0; m < M; ++m) {
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = (lane + 32 * i) * 8;
            if (k < K) {
                const uint4 a = *reinterpret_cast<const uint4*>(A + (long long)m * lda + k);
                acc = fmaf(bf16lo(a.x), bf16lo(b[i].x), acc); acc = fmaf(bf16hi(a.x), bf16hi(b[i].x), acc); acc = fmaf(bf16lo(a.y), bf16lo(b[i].y), acc); acc = fmaf(bf16hi(a.y), bf16hi(b[i].y), acc);
                acc = fmaf(bf16lo(a.z), bf16lo(b[i].z), acc); acc = fmaf(bf16hi(a.z), bf16hi(b[i].z), acc); acc = fmaf(bf16lo(a.w), bf16lo(b[i].w), acc); acc = fmaf(bf16hi(a.w), bf16hi(b[i].w), acc);
            }
        }
        acc = warp_sum(acc);
        if (lane == 0) {
            float v = acc * alpha + (bias ? bias[n] : 0.f);
            if (act == 1) { v = fmaxf(v, 0.f); v *= v; }
            else if (act == 2) v = gelu_tanhf_(v);
            const long long at = (long long)blockIdx.y * sC + (long long)m * ldc + n;
            if (MODE == HY_STORE) reinterpret_cast<__nv_bfloat16*>(Cv)[at] = __float2bfloat16_rn(v);
            else if (MODE == HY_STORE_F32) reinterpret_cast<float*>(Cv)[at] = v;
            else reinterpret_cast<float*>(Cv)[at] += v;
        }
    }
}

template <typename TA>
__global__ void hy_embed_kernel(const int32_t* ids, const TA* table, float* x, float* x0, int T, int W, int vocab, float scale, TA* h, int ldh) {
    HY_PDL();
    const int t = blockIdx.x; int id = ids[t]; id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = ldf(table + (long long)id * W + c) * scale; x[(long long)t * W + c] = v;
        if (x0) x0[(long long)t * W + c] = v;
        if (h) stf(h + (long long)t * ldh + c, v);
    }
}
template <typename TA>
__global__ void hy_concat_kernel(const float* x, const float* x0, TA* cat, int T, int W) {
    HY_PDL();
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < W; c += blockDim.x) { stf(cat + (long long)t * 2 * W + c, x[(long long)t * W + c]); stf(cat + (long long)t * 2 * W + W + c, x0[(long long)t * W + c]); }
}
// one read of the row: W <= 8192, a multiple of 4; each thread keeps up to 8 float4 of it
template <typename TA>
__global__ void __launch_bounds__(256) hy_layernorm_reg_kernel(const float* x, const int32_t* rows, const float* w, TA* out, int ldo, int W, float eps) {
    HY_PDL();
    __shared__ float red[32];
    const int t = blockIdx.x; const float4* xr = reinterpret_cast<const float4*>(x + (long long)(rows ? rows[t] : t) * W);
    const int n4 = W / 4;
    float4 v[8]; float s = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) { const int i = threadIdx.x + k * 256; if (i < n4) { v[k] = xr[i]; s += (v[k].x + v[k].y) + (v[k].z + v[k].w); } }
    const float mean = block_sum(s, red) / (float)W;
    float q = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) { const int i = threadIdx.x + k * 256; if (i < n4) { const float a = v[k].x - mean, b = v[k].y - mean, c = v[k].z - mean, d = v[k].w - mean; q += (a * a + b * b) + (c * c + d * d); } }
    const float rstd = 1.0f / sqrtf(block_sum(q, red) / (float)W + eps);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int i = threadIdx.x + k * 256;
        if (i < n4) {
            const float4 g = reinterpret_cast<const float4*>(w)[i]; TA* o = out + (long long)t * ldo + 4 * i;
            stf(o, (v[k].x - mean) * rstd * g.x); stf(o + 1, (v[k].y - mean) * rstd * g.y); stf(o + 2, (v[k].z - mean) * rstd * g.z); stf(o + 3, (v[k].w - mean) * rstd * g.w);
        }
    }
}
template <typename TA>
__global__ void __launch_bounds__(256) hy_layernorm_kernel(const float* x, const int32_t* rows, const float* w, TA* out, int ldo, int W, float eps) {
    HY_PDL();
    __shared__ float red[32];
    const int t = blockIdx.x; const float* xr = x + (long long)(rows ? rows[t] : t) * W;
    float s = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) s += xr[c];
    const float mean = block_sum(s, red) / (float)W;
    float v = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) { const float d = xr[c] - mean; v += d * d; }
    const float rstd = 1.0f / sqrtf(block_sum(v, red) / (float)W + eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x) stf(out + (long long)t * ldo + c, (xr[c] - mean) * rstd * w[c]);
}

// ---------------------------------------------------------------------------------------------------------------------------------
// latent attention
// ---------------------------------------------------------------------------------------------------------------------------------
template <typename TA>
__global__ void __launch_bounds__(128) hy_mla_prep_kernel(HyLatentAttn a, const TA* q, int ldq, const TA* ckv, int ldc, const float* norm_w, float eps,
                                                           const float* rope_cos, const float* rope_sin, TA* cache, float* q_abs, HyRows r) {
    HY_PDL();
    __shared__ float red[32];
    const int t = blockIdx.x, R = a.kv_rank, rot = a.rot_dim, half = a.rot_dims / 2, E = R + rot;
    const TA* c = ckv + (long long)t * ldc;
    float ss = 0.f;
    for (int i = threadIdx.x; i < R; i += blockDim.x) { const float v = ldf(c + i); ss += v * v; }
    const float rr = 1.0f / sqrtf(block_sum(ss, red) / (float)R + eps);
    TA* dst = cache + (long long)r.slots[t] * E;
    for (int i = threadIdx.x; i < R; i += blockDim.x) stf(dst + i, ldf(c + i) * rr * norm_w[i]);
    const int pos = r.positions[t];
    const float* cs = rope_cos + (long long)pos * half; const float* sn = rope_sin + (long long)pos * half;
    for (int i = threadIdx.x; i < rot; i += blockDim.x) {          // shared rotated key
        float v;
        if (i < 2 * half) {
            const bool second = a.rot_layout ? i >= half : (i & 1); const int p = a.rot_layout ? (second ? i - half : i) : i >> 1;
            const float u0 = ldf(c + R + (a.rot_layout ? p : 2 * p)), u1 = ldf(c + R + (a.rot_layout ? p + half : 2 * p + 1));
            v = second ? (u1 * cs[p] + u0 * sn[p]) : (u0 * cs[p] - u1 * sn[p]);
        } else v = ldf(c + R + i);
        stf(dst + R + i, v);
    }
    for (int i = threadIdx.x; i < a.heads * rot; i += blockDim.x) {   // rotated query parts
        const int h = i / rot, d = i - h * rot; const TA* qh = q + (long long)t * ldq + (long long)h * (a.dim + rot) + a.dim;
        float v;
        if (d < 2 * half) {
            const bool second = a.rot_layout ? d >= half : (d & 1); const int p = a.rot_layout ? (second ? d - half : d) : d >> 1;
            const float u0 = ldf(qh + (a.rot_layout ? p : 2 * p)), u1 = ldf(qh + (a.rot_layout ? p + half : 2 * p + 1));
            v = second ? (u1 * cs[p] + u0 * sn[p]) : (u0 * cs[p] - u1 * sn[p]);
        } else v = ldf(qh + d);
        q_abs[((long long)t * a.heads + h) * E + R + d] = v;
    }
}

constexpr int MLA_ACC = 32;     // latent channels per lane: kv_rank <= 32 * MLA_ACC
template <typename TA>
__global__ void __launch_bounds__(128) hy_mla_attention_kernel(HyLatentAttn a, const float* q_abs, const TA* cache, TA* lat_out, HyRows r) {
    HY_PDL();
    extern __shared__ float sm[];
    const int t = blockIdx.x, h = blockIdx.y, R = a.kv_rank, E = R + a.rot_dim;
    float* qs = sm;                      // [E]
    float* macc = sm + E;                // [4][R] partial outputs, then [4] m, [4] l
    float* mm = macc + 4 * R; float* ll = mm + 4;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float* qr = q_abs + ((long long)t * a.heads + h) * E;
    for (int i = threadIdx.x; i < E; i += blockDim.x) qs[i] = qr[i] * a.scale;
    __syncthreads();
    const int seq = r.row_seq[t], pos = r.positions[t];
    const int32_t* bt = r.block_tables + (long long)seq * r.max_pages_per_seq;
    float m = -INFINITY, l = 0.f, acc[MLA_ACC];
#pragma unroll
    for (int i = 0; i < MLA_ACC; ++i) acc[i] = 0.f;
    const int j_lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;         // a warp's keys depend on the row's position only
    for (int j = j_lo + warp; j <= pos; j += 4) {
        const TA* kr = cache + ((long long)bt[j >> 6] * 64 + (j & 63)) * E;
        float d = 0.f;
        for (int i = lane; i < E; i += 32) d = fmaf(qs[i], ldf(kr + i), d);
        d = warp_sum(d);
        const float mn = fmaxf(m, d), corr = expf(m - mn), p = expf(d - mn);
        l = l * corr + p; m = mn;
#pragma unroll
        for (int i = 0; i < MLA_ACC; ++i) { const int c = lane + 32 * i; if (c < R) acc[i] = acc[i] * corr + p * ldf(kr + c); }
    }
#pragma unroll
    for (int i = 0; i < MLA_ACC; ++i) { const int c = lane + 32 * i; if (c < R) macc[warp * R + c] = acc[i]; }
    if (lane == 0) { mm[warp] = m; ll[warp] = l; }
    __syncthreads();
    const float sk = a.sink ? a.sink[h] : -INFINITY;                        // the sink: one more term of the denominator, no value
    float M = fmaxf(fmaxf(fmaxf(mm[0], mm[1]), fmaxf(mm[2], mm[3])), sk), L = 0.f, f[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) { f[w] = mm[w] == -INFINITY ? 0.f : expf(mm[w] - M); L += f[w] * ll[w]; }
    if (a.sink) L += expf(sk - M);
    const float inv = 1.0f / L;
    for (int c = threadIdx.x; c < R; c += blockDim.x) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) v += f[w] * macc[w * R + c];
        stf(lat_out + ((long long)t * a.heads + h) * R + c, v * inv);
    }
}

// ---------------------------------------------------------------------------------------------------------------------------------
// latent attention on the tensor cores (bf16): one CTA owns 64 queries — consecutive (row, head) pairs of ONE sequence, so all of them read
// the same cached rows — and streams that sequence's cache in 32-row tiles through a double-buffered cp.async ring.  S = Q K^T and
// O += P V are mma.sync m16n8k16 products on the same shared-memory tile (the cached row is key AND value); softmax is online, in fp32
// registers, with the mask applied per query position.  A CTA accumulates NVB * 8 of the latent's channels (blockIdx.y picks which).
// ---------------------------------------------------------------------------------------------------------------------------------
constexpr int MLA_MQ = 64;
template <int NVB, int MLA_KT>      // MLA_KT = cache rows per tile: 32, or 16 where that lets two CTAs share an SM
__global__ void __launch_bounds__(128) hy_mla_attention_mma_kernel(HyLatentAttn a, const float* __restrict__ q_abs, const __nv_bfloat16* __restrict__ cache,
                                                                   __nv_bfloat16* __restrict__ lat_out, HyRows r, const int32_t* __restrict__ tile_seq,
                                                                   const int32_t* __restrict__ tile_q0, HyMlaSplit sp) {
    HY_PDL();
    extern __shared__ __align__(16) uint8_t mla_smem[];
    const int R = a.kv_rank, E = R + a.rot_dim, EP = E + 8, H = a.heads;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(mla_smem);      // [MLA_MQ][EP]
    __nv_bfloat16* Ks = Qs + MLA_MQ * EP;                                // [2][MLA_KT][EP]
    int* qpos = reinterpret_cast<int*>(Ks + 2 * MLA_KT * EP);            // [MLA_MQ]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int seq = tile_seq[blockIdx.x], q0 = tile_q0[blockIdx.x], vbase = blockIdx.y * NVB * 8;
    const int row0 = r.seq_row0[seq], len = r.seq_row0[seq + 1] - row0;
    const int nq = min(MLA_MQ, len * H - q0);
    const float qscale = a.scale * 1.4426950408889634f;
    for (int idx = tid; idx < MLA_MQ * (E / 2); idx += 128) {
        const int qi = idx / (E / 2), e = (idx - qi * (E / 2)) * 2;
        float2 v = make_float2(0.f, 0.f);
        if (qi < nq) { const int row = row0 + (q0 + qi) / H, h = (q0 + qi) % H; v = *reinterpret_cast<const float2*>(q_abs + ((long long)row * H + h) * E + e); }
        *reinterpret_cast<uint32_t*>(Qs + qi * EP + e) = pack_bf16x2(v.x * qscale, v.y * qscale);
    }
    for (int qi = tid; qi < MLA_MQ; qi += 128) qpos[qi] = qi < nq ? r.positions[row0 + (q0 + qi) / H] : 0;
    // a decoding row's keys may be cut into parts (one CTA each): this CTA walks cache rows [k0, k1) and leaves an unnormalised partial
    const int k0 = sp.tile_k0 ? sp.tile_k0[blockIdx.x] : 0, k1 = sp.tile_k0 ? sp.tile_k1[blockIdx.x] : 0, slot = sp.tile_k0 ? sp.tile_slot[blockIdx.x] : -1;
    int max_pos = r.positions[row0 + (q0 + nq - 1) / H];
    if (k1 > 0 && k1 - 1 < max_pos) max_pos = k1 - 1;
    const int win = a.window > 0 ? a.window : 0x40000000;
    const int first_vis = max(k0, r.positions[row0 + q0 / H] - win + 1);       // the first cache row any query of the tile sees
    const int kt0 = max(first_vis, 0) / MLA_KT, n_kt = max_pos / MLA_KT + 1;
    const int32_t* bt = r.block_tables + (long long)seq * r.max_pages_per_seq;
    auto load_tile = [&](int kt, int buf) {
        const int chunks = E / 8;
        for (int idx = tid; idx < MLA_KT * chunks; idx += 128) {
            const int j = idx / chunks, c = idx - j * chunks, key = kt * MLA_KT + j;
            __nv_bfloat16* dst = Ks + (buf * MLA_KT + j) * EP + c * 8;
            if (key <= max_pos) cp_async16(dst, cache + ((long long)bt[key >> 6] * 64 + (key & 63)) * E + c * 8);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float o[NVB][4];
#pragma unroll
    for (int i = 0; i < NVB; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
    const bool active = 16 * warp < nq;
    load_tile(kt0, 0);
    for (int kt = kt0; kt < n_kt; ++kt) {
        if (kt + 1 < n_kt) { load_tile(kt + 1, (kt + 1 - kt0) & 1); asm volatile("cp.async.wait_group 1;" ::: "memory"); }
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        if (active) {
            const __nv_bfloat16* Kb = Ks + ((kt - kt0) & 1) * MLA_KT * EP;
            constexpr int NB = MLA_KT / 8;
            float s[NB][4];
#pragma unroll
            for (int i = 0; i < NB; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
            const uint32_t qa = smem_u32(Qs + (16 * warp + (lane & 15)) * EP + (lane >> 4) * 8);
            const uint32_t ka = smem_u32(Kb + ((lane >> 4) * 8 + (lane & 7)) * EP + ((lane >> 3) & 1) * 8);
            for (int ks = 0; ks < E / 16; ++ks) {
                uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
                ldmatrix_x4(qa + ks * 32, a0, a1, a2, a3);
                ldmatrix_x4(ka + ks * 32, b0, b1, b2, b3);
                mma_bf16_16816(s[0], a0, a1, a2, a3, b0, b1); mma_bf16_16816(s[1], a0, a1, a2, a3, b2, b3);
                if (NB == 4) {
                    ldmatrix_x4(ka + 16 * EP * 2 + ks * 32, b0, b1, b2, b3);
                    mma_bf16_16816(s[NB - 2], a0, a1, a2, a3, b0, b1); mma_bf16_16816(s[NB - 1], a0, a1, a2, a3, b2, b3);
                }
            }
            const int p_lo = qpos[16 * warp + (lane >> 2)], p_hi = qpos[16 * warp + (lane >> 2) + 8];
            float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int key = kt * MLA_KT + nb * 8 + (lane & 3) * 2 + (c & 1), pq = c < 2 ? p_lo : p_hi;
                    if (key > pq || pq - key >= win) s[nb][c] = -INFINITY;
                    if (c < 2) mx_lo = fmaxf(mx_lo, s[nb][c]); else mx_hi = fmaxf(mx_hi, s[nb][c]);
                }
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1)); mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1)); mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
            const float t_lo = fmaxf(m_lo, mx_lo), t_hi = fmaxf(m_hi, mx_hi);
            const float n_lo = t_lo == -INFINITY ? 0.f : t_lo, n_hi = t_hi == -INFINITY ? 0.f : t_hi;       // a query whose window starts behind this tile has seen nothing yet
            const float c_lo = exp2f(m_lo - n_lo), c_hi = exp2f(m_hi - n_hi);
            m_lo = t_lo; m_hi = t_hi;
            float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                s[nb][0] = exp2f(s[nb][0] - n_lo); s[nb][1] = exp2f(s[nb][1] - n_lo); s[nb][2] = exp2f(s[nb][2] - n_hi); s[nb][3] = exp2f(s[nb][3] - n_hi);
                sum_lo += s[nb][0] + s[nb][1]; sum_hi += s[nb][2] + s[nb][3];
            }
            l_lo = l_lo * c_lo + sum_lo; l_hi = l_hi * c_hi + sum_hi;
#pragma unroll
            for (int i = 0; i < NVB; ++i) { o[i][0] *= c_lo; o[i][1] *= c_lo; o[i][2] *= c_hi; o[i][3] *= c_hi; }
            const uint32_t va = smem_u32(Kb + (((lane >> 3) & 1) * 8 + (lane & 7)) * EP + vbase + (lane >> 4) * 8);
#pragma unroll
            for (int kk = 0; kk < NB / 2; ++kk) {
                const uint32_t a0 = pack_bf16x2(s[2 * kk][0], s[2 * kk][1]), a1 = pack_bf16x2(s[2 * kk][2], s[2 * kk][3]);
                const uint32_t a2 = pack_bf16x2(s[2 * kk + 1][0], s[2 * kk + 1][1]), a3 = pack_bf16x2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int np = 0; np < NVB / 2; ++np) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(va + kk * 16 * EP * 2 + np * 32, b0, b1, b2, b3);
                    mma_bf16_16816(o[2 * np], a0, a1, a2, a3, b0, b1); mma_bf16_16816(o[2 * np + 1], a0, a1, a2, a3, b2, b3);
                }
            }
        }
        __syncthreads();
    }
    if (!active) return;
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1); l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1); l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    const int q_lo = 16 * warp + (lane >> 2), q_hi = q_lo + 8;
    if (slot >= 0) {                                  // partial: fp32 sums, running maximum (base-2 scores) and denominator per query
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int qi = half ? q_hi : q_lo;
            if (qi >= nq) continue;
            float* dst = sp.ws_o + ((long long)slot * H + qi) * R + vbase + (lane & 3) * 2;
#pragma unroll
            for (int nb = 0; nb < NVB; ++nb) *reinterpret_cast<float2*>(dst + nb * 8) = make_float2(o[nb][half * 2], o[nb][half * 2 + 1]);
            if (blockIdx.y == 0 && (lane & 3) == 0) { sp.ws_ml[((long long)slot * H + qi) * 2] = half ? m_hi : m_lo; sp.ws_ml[((long long)slot * H + qi) * 2 + 1] = half ? l_hi : l_lo; }
        }
        return;
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int qi = half ? q_hi : q_lo;
        if (qi >= nq) continue;
        const int row = row0 + (q0 + qi) / H, h = (q0 + qi) % H;
        float l = half ? l_hi : l_lo, up = 1.f;
        if (a.sink) {                 // the sink joins the denominator (scores are kept in base-2 units)
            const float m = half ? m_hi : m_lo, s2 = a.sink[h] * 1.4426950408889634f, M = fmaxf(m, s2);
            up = m == -INFINITY ? 0.f : exp2f(m - M); l = l * up + exp2f(s2 - M);
        }
        const float inv = l > 0.f ? up / l : 0.f;
        __nv_bfloat16* dst = lat_out + ((long long)row * H + h) * R + vbase + (lane & 3) * 2;
#pragma unroll
        for (int nb = 0; nb < NVB; ++nb) *reinterpret_cast<uint32_t*>(dst + nb * 8) = pack_bf16x2(o[nb][half * 2] * inv, o[nb][half * 2 + 1] * inv);
    }
}

// joins the parts of a decoding row: out = sum_p 2^(m_p - M) O_p / sum_p 2^(m_p - M) l_p, parts in order
__global__ void __launch_bounds__(128) hy_mla_merge_kernel(const int32_t* item_row, const int32_t* item_slot0, const int32_t* item_parts, const float* ws_o,
                                                           const float* ws_ml, __nv_bfloat16* lat_out, int H, int R, const float* sink) {
    HY_PDL();
    const int row = item_row[blockIdx.x], slot0 = item_slot0[blockIdx.x], P = item_parts[blockIdx.x], h = blockIdx.y;
    const float s2 = sink ? sink[h] * 1.4426950408889634f : -INFINITY;       // the sink, in the partials' base-2 units
    float M = s2;
    for (int p = 0; p < P; ++p) M = fmaxf(M, ws_ml[((long long)(slot0 + p) * H + h) * 2]);
    float L = sink ? exp2f(s2 - M) : 0.f;
    for (int p = 0; p < P; ++p) { const float* ml = ws_ml + ((long long)(slot0 + p) * H + h) * 2; L += exp2f(ml[0] - M) * ml[1]; }
    const float inv = 1.0f / L;
    for (int c = threadIdx.x; c < R; c += blockDim.x) {
        float acc = 0.f;
        for (int p = 0; p < P; ++p) acc += exp2f(ws_ml[((long long)(slot0 + p) * H + h) * 2] - M) * ws_o[((long long)(slot0 + p) * H + h) * R + c];
        lat_out[((long long)row * H + h) * R + c] = __float2bfloat16_rn(acc * inv);
    }
}

// ---------------------------------------------------------------------------------------------------------------------------------
// prefill form of latent attention: per-head keys [W_uk c | rotated shared part] and values W_uv c of a sequence's whole context are first
// materialised by one GEMM over its gathered cache rows (hy_gather_ctx + the tcgen05 GEMM); then this kernel runs ordinary causal
// multi-head attention on them — 64 query rows of one (sequence, head) per CTA, 32-row key / value tiles through a cp.async double buffer,
// S = Q K^T over dim + rot_dim and O += P V over vdim on mma.sync, online softmax in fp32 — and writes the heads' outputs straight into
// the output projection's input.  Per key it costs dim + rot_dim + vdim multiply-adds instead of the absorbed form's 2 kv_rank + rot_dim.
// ---------------------------------------------------------------------------------------------------------------------------------
template <int NVB>
__global__ void __launch_bounds__(128) hy_mha_prefill_mma_kernel(HyLatentAttn a, const __nv_bfloat16* __restrict__ q, int ldq, const float* __restrict__ q_abs,
                                                                 const __nv_bfloat16* __restrict__ kv_ctx, int ld_kv, const __nv_bfloat16* __restrict__ lat_ctx,
                                                                 __nv_bfloat16* __restrict__ mix, int ld_mix, HyRows r, const int32_t* __restrict__ tile_seq,
                                                                 const int32_t* __restrict__ tile_head, const int32_t* __restrict__ tile_row0,
                                                                 const int32_t* __restrict__ seq_base) {
    HY_PDL();
    extern __shared__ __align__(16) uint8_t mha_smem[];
    constexpr int KT = 32, VD = NVB * 8;
    const int R = a.kv_rank, E = R + a.rot_dim, H = a.heads, DN = a.dim, DQ = a.dim + a.rot_dim, QP = DQ + 8, VP = VD + 8;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(mha_smem);      // [64][QP]
    __nv_bfloat16* Ks = Qs + MLA_MQ * QP;                                // [2][KT][QP]
    __nv_bfloat16* Vs = Ks + 2 * KT * QP;                                // [2][KT][VP]
    int* qpos = reinterpret_cast<int*>(Vs + 2 * KT * VP);                // [64]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int seq = tile_seq[blockIdx.x], h = tile_head[blockIdx.x], qr0 = tile_row0[blockIdx.x];
    const int row0 = r.seq_row0[seq] + qr0, nq = min(MLA_MQ, r.seq_row0[seq + 1] - row0);
    const long long base = seq_base[seq];
    const float qscale = a.scale * 1.4426950408889634f;
    for (int idx = tid; idx < MLA_MQ * (DQ / 2); idx += 128) {
        const int qi = idx / (DQ / 2), e = (idx - qi * (DQ / 2)) * 2;
        uint32_t v = 0;
        if (qi < nq) {
            if (e < DN) v = *reinterpret_cast<const uint32_t*>(q + (long long)(row0 + qi) * ldq + h * DQ + e);
            else { const float2 f = *reinterpret_cast<const float2*>(q_abs + ((long long)(row0 + qi) * H + h) * E + R + (e - DN)); v = pack_bf16x2(f.x, f.y); }
        }
        *reinterpret_cast<uint32_t*>(Qs + qi * QP + e) = v;
    }
    for (int qi = tid; qi < MLA_MQ; qi += 128) qpos[qi] = qi < nq ? r.positions[row0 + qi] : 0;
    const int max_pos = r.positions[row0 + nq - 1];
    const int win = a.window > 0 ? a.window : 0x40000000;
    const int kt_first = max(0, r.positions[row0] - win + 1) / KT, n_kt = max_pos / KT + 1;      // tiles before the first query's window hold nothing visible
    auto load_tile = [&](int kt, int buf) {
        const int kc = DQ / 8, nc = DN / 8, vc = VD / 8;
        for (int idx = tid; idx < KT * (kc + vc); idx += 128) {
            const int j = idx / (kc + vc), c = idx - j * (kc + vc), key = kt * KT + j;
            __nv_bfloat16* dst = c < kc ? Ks + (buf * KT + j) * QP + c * 8 : Vs + (buf * KT + j) * VP + (c - kc) * 8;
            if (key <= max_pos) {
                const __nv_bfloat16* src = c < nc ? kv_ctx + (base + key) * ld_kv + h * DN + c * 8
                                         : c < kc ? lat_ctx + (base + key) * E + R + (c - nc) * 8
                                                  : kv_ctx + (base + key) * ld_kv + H * DN + h * VD + (c - kc) * 8;
                cp_async16(dst, src);
            } else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float o[NVB][4];
#pragma unroll
    for (int i = 0; i < NVB; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
    const bool active = 16 * warp < nq;
    load_tile(kt_first, kt_first & 1);
    for (int kt = kt_first; kt < n_kt; ++kt) {
        if (kt + 1 < n_kt) { load_tile(kt + 1, (kt + 1) & 1); asm volatile("cp.async.wait_group 1;" ::: "memory"); }
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        if (active) {
            const __nv_bfloat16* Kb = Ks + (kt & 1) * KT * QP; const __nv_bfloat16* Vb = Vs + (kt & 1) * KT * VP;
            float s[4][4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
            const uint32_t qa = smem_u32(Qs + (16 * warp + (lane & 15)) * QP + (lane >> 4) * 8);
            const uint32_t ka = smem_u32(Kb + ((lane >> 4) * 8 + (lane & 7)) * QP + ((lane >> 3) & 1) * 8);
            for (int ks = 0; ks < DQ / 16; ++ks) {
                uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
                ldmatrix_x4(qa + ks * 32, a0, a1, a2, a3);
                ldmatrix_x4(ka + ks * 32, b0, b1, b2, b3);
                mma_bf16_16816(s[0], a0, a1, a2, a3, b0, b1); mma_bf16_16816(s[1], a0, a1, a2, a3, b2, b3);
                ldmatrix_x4(ka + 16 * QP * 2 + ks * 32, b0, b1, b2, b3);
                mma_bf16_16816(s[2], a0, a1, a2, a3, b0, b1); mma_bf16_16816(s[3], a0, a1, a2, a3, b2, b3);
            }
            const int p_lo = qpos[16 * warp + (lane >> 2)], p_hi = qpos[16 * warp + (lane >> 2) + 8];
            float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
            for (int nb = 0; nb < 4; ++nb)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int key = kt * KT + nb * 8 + (lane & 3) * 2 + (c & 1), pq = c < 2 ? p_lo : p_hi;
                    s[nb][c] = (key > pq || pq - key >= win) ? -INFINITY : s[nb][c] * qscale;
                    if (c < 2) mx_lo = fmaxf(mx_lo, s[nb][c]); else mx_hi = fmaxf(mx_hi, s[nb][c]);
                }
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1)); mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1)); mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
            const float t_lo = fmaxf(m_lo, mx_lo), t_hi = fmaxf(m_hi, mx_hi);
            const float n_lo = t_lo == -INFINITY ? 0.f : t_lo, n_hi = t_hi == -INFINITY ? 0.f : t_hi;       // a query whose window starts behind this tile has seen nothing yet
            const float c_lo = exp2f(m_lo - n_lo), c_hi = exp2f(m_hi - n_hi);
            m_lo = t_lo; m_hi = t_hi;
            float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
            for (int nb = 0; nb < 4; ++nb) {
                s[nb][0] = exp2f(s[nb][0] - n_lo); s[nb][1] = exp2f(s[nb][1] - n_lo); s[nb][2] = exp2f(s[nb][2] - n_hi); s[nb][3] = exp2f(s[nb][3] - n_hi);
                sum_lo += s[nb][0] + s[nb][1]; sum_hi += s[nb][2] + s[nb][3];
            }
            l_lo = l_lo * c_lo + sum_lo; l_hi = l_hi * c_hi + sum_hi;
#pragma unroll
            for (int i = 0; i < NVB; ++i) { o[i][0] *= c_lo; o[i][1] *= c_lo; o[i][2] *= c_hi; o[i][3] *= c_hi; }
            const uint32_t va = smem_u32(Vb + (((lane >> 3) & 1) * 8 + (lane & 7)) * VP + (lane >> 4) * 8);
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
                const uint32_t a0 = pack_bf16x2(s[2 * kk][0], s[2 * kk][1]), a1 = pack_bf16x2(s[2 * kk][2], s[2 * kk][3]);
                const uint32_t a2 = pack_bf16x2(s[2 * kk + 1][0], s[2 * kk + 1][1]), a3 = pack_bf16x2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int np = 0; np < NVB / 2; ++np) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(va + kk * 16 * VP * 2 + np * 32, b0, b1, b2, b3);
                    mma_bf16_16816(o[2 * np], a0, a1, a2, a3, b0, b1); mma_bf16_16816(o[2 * np + 1], a0, a1, a2, a3, b2, b3);
                }
            }
        }
        __syncthreads();
    }
    if (!active) return;
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1); l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1); l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int qi = 16 * warp + (lane >> 2) + half * 8;
        if (qi >= nq) continue;
        float l = half ? l_hi : l_lo, up = 1.f;
        if (a.sink) {                 // the sink joins the denominator (scores are kept in base-2 units)
            const float m = half ? m_hi : m_lo, s2 = a.sink[h] * 1.4426950408889634f, M = fmaxf(m, s2);
            up = m == -INFINITY ? 0.f : exp2f(m - M); l = l * up + exp2f(s2 - M);
        }
        const float inv = l > 0.f ? up / l : 0.f;
        __nv_bfloat16* dst = mix + (long long)(row0 + qi) * ld_mix + h * VD + (lane & 3) * 2;
        const __nv_bfloat16* gp = a.gate ? reinterpret_cast<const __nv_bfloat16*>(a.gate) + (long long)(row0 + qi) * a.ldg + h * VD + (lane & 3) * 2 : nullptr;
#pragma unroll
        for (int nb = 0; nb < NVB; ++nb) {
            float y0 = o[nb][half * 2] * inv, y1 = o[nb][half * 2 + 1] * inv;
            if (gp) { const uint32_t gg = *reinterpret_cast<const uint32_t*>(gp + nb * 8); y0 *= sigmoidf_(bf16lo(gg)); y1 *= sigmoidf_(bf16hi(gg)); }
            *reinterpret_cast<uint32_t*>(dst + nb * 8) = pack_bf16x2(y0, y1);
        }
    }
}
// cache rows 0 .. ctx-1 of the listed sequences, contiguous: lat_ctx[seq_base[s] + j] = cache row j of sequence s (seq_base < 0: not listed)
__global__ void __launch_bounds__(128) hy_gather_ctx_kernel(const __nv_bfloat16* __restrict__ cache, int E, const int32_t* __restrict__ block_tables, int mpps,
                                                            const int32_t* __restrict__ seq_base, const int32_t* __restrict__ seq_row0, const int32_t* __restrict__ positions,
                                                            __nv_bfloat16* __restrict__ lat_ctx) {
    HY_PDL();
    const int seq = blockIdx.x; const long long base = seq_base[seq];
    if (base < 0) return;
    const int ctx = positions[seq_row0[seq + 1] - 1] + 1, chunks = E / 8;
    for (int idx = blockIdx.y * 16 * chunks + threadIdx.x; idx < min(ctx, (int)(blockIdx.y + 1) * 16) * chunks; idx += 128) {
        const int j = idx / chunks, c = idx - j * chunks;
        *reinterpret_cast<uint4*>(lat_ctx + (base + j) * E + c * 8) =
            *reinterpret_cast<const uint4*>(cache + ((long long)block_tables[(long long)seq * mpps + (j >> 6)] * 64 + (j & 63)) * E + c * 8);
    }
}

// ---------------------------------------------------------------------------------------------------------------------------------
// short causal convolution with carried tails
// ---------------------------------------------------------------------------------------------------------------------------------
template <typename TA>
__device__ __forceinline__ float conv_input(const TA* in, int ld_in, int C, const TA* tail, int taps, int row0, int pos0, int src, int c) {
    if (src >= 0) return ldf(in + (long long)(row0 + src) * ld_in + c);
    if (pos0 <= 0) return 0.f;
    return ldf(tail + (long long)(taps - 1 + src) * C + c);
}
template <typename TA>
__global__ void hy_conv_silu_kernel(const TA* in, int ld_in, int C, const float* w, const float* bias, int taps, TA* out, int ld_out, const TA* tails, HyRows r, int act) {
    HY_PDL();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, t = blockIdx.y;
    if (c >= C) return;
    const int seq = r.row_seq[t], row0 = r.seq_row0[seq], i = t - row0, pos0 = r.seq_pos0[seq];
    const TA* tail = tails + (long long)r.seq_state[seq] * (taps - 1) * C;
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < taps; ++j) acc = fmaf(w[c * taps + j], conv_input(in, ld_in, C, tail, taps, row0, pos0, i - (taps - 1) + j, c), acc);
    stf(out + (long long)t * ld_out + c, act ? siluf_(acc) : acc);
}
// bf16 rows of prefill-sized steps whose channels come in aligned groups of 8: a thread computes 8 channels of CONV_ROWS consecutive rows
// from 16-byte loads, with its taps' weights and the last inputs in registers, so that every input row is read once.  The sum runs over
// the taps in the same order as in the kernel above: both give the same bits.
constexpr int CONV_ROWS = 16;
__device__ __forceinline__ void bf8_to_f32(const uint4& u, float* f) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}
template <int TAPS>
__global__ void __launch_bounds__(128) hy_conv_silu_vec8_kernel(const __nv_bfloat16* __restrict__ in, int ld_in, int C, const float* __restrict__ w, const float* __restrict__ bias,
                                                                 __nv_bfloat16* __restrict__ out, int ld_out, const __nv_bfloat16* __restrict__ tails, HyRows r, int act) {
    HY_PDL();
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8, t0 = blockIdx.y * CONV_ROWS;
    if (c >= C) return;
    float wr[TAPS][8], win[TAPS][8], b8[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        b8[e] = bias ? bias[c + e] : 0.f;
#pragma unroll
        for (int j = 0; j < TAPS; ++j) wr[j][e] = w[(c + e) * TAPS + j];
    }
    for (int tt = 0; tt < CONV_ROWS && t0 + tt < r.T; ++tt) {
        const int t = t0 + tt, seq = r.row_seq[t], row0 = r.seq_row0[seq], i = t - row0;
        if (tt == 0 || i == 0) {                        // the inputs before this row: earlier rows of the step, the carried tail, or zeros
            const int pos0 = r.seq_pos0[seq];
            const __nv_bfloat16* tail = tails + (long long)r.seq_state[seq] * (TAPS - 1) * C;
#pragma unroll
            for (int j = 0; j < TAPS - 1; ++j) {
                const int src = i - (TAPS - 1) + j;
                uint4 u = make_uint4(0u, 0u, 0u, 0u);
                if (src >= 0) u = *reinterpret_cast<const uint4*>(in + (long long)(row0 + src) * ld_in + c);
                else if (pos0 > 0) u = *reinterpret_cast<const uint4*>(tail + (long long)(TAPS - 1 + src) * C + c);
                bf8_to_f32(u, win[j]);
            }
        }
        bf8_to_f32(*reinterpret_cast<const uint4*>(in + (long long)t * ld_in + c), win[TAPS - 1]);
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float a0 = b8[2 * e], a1 = b8[2 * e + 1];
#pragma unroll
            for (int j = 0; j < TAPS; ++j) { a0 = fmaf(wr[j][2 * e], win[j][2 * e], a0); a1 = fmaf(wr[j][2 * e + 1], win[j][2 * e + 1], a1); }
            const __nv_bfloat162 h = act ? __floats2bfloat162_rn(siluf_(a0), siluf_(a1)) : __floats2bfloat162_rn(a0, a1);
            o[e] = *reinterpret_cast<const uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(out + (long long)t * ld_out + c) = make_uint4(o[0], o[1], o[2], o[3]);
#pragma unroll
        for (int j = 0; j < TAPS - 1; ++j)
#pragma unroll
            for (int e = 0; e < 8; ++e) win[j][e] = win[j + 1][e];
    }
}
template <typename TA>
__global__ void hy_conv_tails_kernel(const TA* in, int ld_in, int C, int taps, TA* tails, HyRows r) {
    HY_PDL();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, seq = blockIdx.y;
    if (c >= C) return;
    const int row0 = r.seq_row0[seq], len = r.seq_row0[seq + 1] - row0, pos0 = r.seq_pos0[seq];
    TA* tail = tails + (long long)r.seq_state[seq] * (taps - 1) * C;
    float v[16];
    for (int j = 0; j < taps - 1; ++j) v[j] = conv_input(in, ld_in, C, tail, taps, row0, pos0, len - (taps - 1) + j, c);
    for (int j = 0; j < taps - 1; ++j) stf(tail + (long long)j * C + c, v[j]);
}

// ---------------------------------------------------------------------------------------------------------------------------------
// recurrences
// ---------------------------------------------------------------------------------------------------------------------------------
template <typename TA>
__global__ void __launch_bounds__(128) hy_delta_prep_kernel(HyDelta d, const TA* conv, int ld_conv, const TA* b, int ld_b, const TA* a, int ld_a, const float* A_log,
                                                             const float* dt_bias, float* qq, float* kk, float* vv, float* dec, float* beta) {
    HY_PDL();
    const int t = blockIdx.x, KH = d.kv_heads, H = d.heads, D = d.dim, VD = d.vdim;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const TA* cr = conv + (long long)t * ld_conv;
    for (int u = warp; u < 2 * KH; u += 4) {                    // unit vectors per q / k head
        const TA* src = cr + (long long)u * D;                   // q heads then k heads, contiguous
        float ss = 0.f;
        for (int i = lane; i < D; i += 32) { const float v = ldf(src + i); ss += v * v; }
        ss = warp_sum(ss);
        const float sc = (u < KH ? rsqrtf((float)D) : 1.0f) / sqrtf(ss + 1e-6f);
        float* dst = (u < KH ? qq + ((long long)t * KH + u) * D : kk + ((long long)t * KH + (u - KH)) * D);
        for (int i = lane; i < D; i += 32) dst[i] = ldf(src + i) * sc;
    }
    for (int i = threadIdx.x; i < H * VD; i += blockDim.x) vv[(long long)t * H * VD + i] = ldf(cr + 2 * KH * D + i);
    for (int i = threadIdx.x; i < H; i += blockDim.x) beta[(long long)t * H + i] = sigmoidf_(ldf(b + (long long)t * ld_b + i));
    for (int i = threadIdx.x; i < H * D; i += blockDim.x)
        dec[(long long)t * H * D + i] = expf(-expf(A_log[i / D]) * softplusf_(ldf(a + (long long)t * ld_a + i) + dt_bias[i]));
}
template <typename TA>
__global__ void __launch_bounds__(128) hy_mamba_prep_kernel(HyMamba m, const TA* conv, int ld_conv, const TA* dt, int ld_dt, const float* A_log, const float* dt_bias,
                                                             float* qq, float* kk, float* vv, float* dec) {
    HY_PDL();
    const int t = blockIdx.x, H = m.heads, VD = m.vdim, N = m.state, G = m.groups, inner = H * VD;
    const TA* cr = conv + (long long)t * ld_conv;
    for (int i = threadIdx.x; i < G * N; i += blockDim.x) { kk[(long long)t * G * N + i] = ldf(cr + inner + i); qq[(long long)t * G * N + i] = ldf(cr + inner + G * N + i); }
    for (int i = threadIdx.x; i < inner; i += blockDim.x) {
        const int h = i / VD; const float step = softplusf_(ldf(dt + (long long)t * ld_dt + h) + dt_bias[h]);
        vv[(long long)t * inner + i] = step * ldf(cr + i);
    }
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        const float step = softplusf_(ldf(dt + (long long)t * ld_dt + h) + dt_bias[h]);
        dec[(long long)t * H + h] = expf(-expf(A_log[h]) * step);
    }
}

constexpr int REC_COLS = 64;      // state columns (value channels) per CTA; a column evolves independently of the others
template <int MODE>
__global__ void __launch_bounds__(REC_COLS) hy_recurrence_kernel(const float* qq, const float* kk, const float* vv, const float* dec, const float* beta, float* out,
                                                                 float* state, int H, int QH, int D, int VD, HyRows r, float* norm_state, float* norm_out) {
    constexpr bool DELTA = MODE == HY_REC_DELTA, CH = MODE != HY_REC_SCALAR;
    HY_PDL();
    extern __shared__ float sm[];
    float* S = sm;                         // [D][REC_COLS]
    float* qs = S + D * REC_COLS; float* ks = qs + D; float* ds = ks + D;
    const int seq = blockIdx.x, h = blockIdx.y, col = blockIdx.z * REC_COLS + threadIdx.x, j = threadIdx.x;
    const bool is_norm = norm_state && col == VD, ok = col < VD || is_norm;      // the normaliser: one more value channel whose value is 1
    const int row0 = r.seq_row0[seq], len = r.seq_row0[seq + 1] - row0, pos0 = r.seq_pos0[seq], qh = h / (H / QH);
    float* st = is_norm ? norm_state + ((long long)r.seq_state[seq] * H + h) * D : state + ((long long)r.seq_state[seq] * H + h) * D * VD + col;
    const long long st_stride = is_norm ? 1 : VD;
    for (int d = 0; d < D; ++d) S[d * REC_COLS + j] = (ok && pos0 > 0) ? st[d * st_stride] : 0.f;
    for (int i = 0; i < len; ++i) {
        const long long t = row0 + i;
        __syncthreads();
        for (int d = j; d < D; d += REC_COLS) {
            qs[d] = qq[(t * QH + qh) * D + d]; ks[d] = kk[(t * QH + qh) * D + d];
            if (CH) ds[d] = dec[(t * H + h) * D + d];
        }
        __syncthreads();
        const float v = is_norm ? 1.f : ok ? vv[(t * H + h) * VD + col] : 0.f;
        float o = 0.f;
        if (DELTA) {
            float dot = 0.f;
            for (int d = 0; d < D; ++d) { const float s = S[d * REC_COLS + j] * ds[d]; S[d * REC_COLS + j] = s; dot = fmaf(s, ks[d], dot); }
            const float u = beta[t * H + h] * (v - dot);
            for (int d = 0; d < D; ++d) { const float s = fmaf(ks[d], u, S[d * REC_COLS + j]); S[d * REC_COLS + j] = s; o = fmaf(s, qs[d], o); }
        } else if (CH) {
            for (int d = 0; d < D; ++d) { const float s = fmaf(ks[d], v, S[d * REC_COLS + j] * ds[d]); S[d * REC_COLS + j] = s; o = fmaf(s, qs[d], o); }
        } else {
            const float a = dec[t * H + h];
            for (int d = 0; d < D; ++d) { const float s = fmaf(ks[d], v, S[d * REC_COLS + j] * a); S[d * REC_COLS + j] = s; o = fmaf(s, qs[d], o); }
        }
        if (is_norm) norm_out[t * H + h] = o;
        else if (ok) out[(t * H + h) * VD + col] = o;
    }
    if (ok) for (int d = 0; d < D; ++d) st[d * st_stride] = S[d * REC_COLS + j];
}

// Register-resident variant for dim <= DM (dim and vdim multiples of 4): a state column (value channel) lives in the registers of LANES
// threads (LANES = 1: one thread holds all DM rows, 128 columns per CTA, and a step needs no traffic between threads; LANES = 4: the CTA's
// four warps hold a quarter of the rows each for the same 32 columns — a lane is a column, so the operand reads stay warp-wide broadcasts —
// and a token's per-token chain is a quarter as long: the delta rule's dot product meets through shared memory and one more barrier per
// token, the read-out's four partial sums are joined one token later by one of the warps, off the chain).  The per-token operands (q, k, decay rows, 128 values, the scalar)
// arrive through an 8-deep cp.async ring in shared memory — every thread keeps its own source pointer and advances it by a constant per
// token — and are read from there as 16-byte broadcasts.  The dependent chains of a step are split over four accumulators.  128 / LANES
// columns per CTA.  The order of every sum is fixed for a given LANES, and LANES is chosen from the sizes alone, never from the step.
constexpr int REC_STAGES = 8, REC_CTA_COLS = 128;
template <int MODE, int DM, int LANES>
__global__ void __launch_bounds__(128) hy_recurrence_reg_kernel(const float* __restrict__ qq, const float* __restrict__ kk, const float* __restrict__ vv,
                                                                const float* __restrict__ dec, const float* __restrict__ beta, float* __restrict__ out,
                                                                float* __restrict__ state, int H, int QH, int D, int VD, HyRows r, float* __restrict__ norm_state,
                                                                float* __restrict__ norm_out) {
    constexpr bool DELTA = MODE == HY_REC_DELTA, CH = MODE != HY_REC_SCALAR;
    HY_PDL();
    extern __shared__ __align__(16) float rec_ring[];
    constexpr int stride = 3 * DM + REC_CTA_COLS + 4;     // floats per stage: q[DM] k[DM] g[DM] v[128] scalar (padded to 16 bytes); pad rows: q = k = 0, decay 1
    constexpr int DR = DM / LANES, COLS = REC_CTA_COLS / LANES;       // rows per thread, columns per CTA
    const int tid = threadIdx.x, part = tid / COLS, cl = tid % COLS, col = blockIdx.z * COLS + cl, r0 = part * DR;      // LANES = 4: part = warp
    __shared__ float rec_pd[LANES][COLS], rec_po[2][LANES][COLS];      // partial dot products of the current token; partial read-outs of this and the last token
    const int seq = blockIdx.x, h = blockIdx.y;
    const bool is_norm = norm_state && col == VD, ok = col < VD || is_norm;      // the normaliser: one more value channel whose value is 1
    const int row0 = r.seq_row0[seq], len = r.seq_row0[seq + 1] - row0, pos0 = r.seq_pos0[seq], qh = h / (H / QH);
    float* st = is_norm ? norm_state + ((long long)r.seq_state[seq] * H + h) * D : state + ((long long)r.seq_state[seq] * H + h) * D * VD + col;
    const long long st_stride = is_norm ? 1 : VD;
    float S[DR];
#pragma unroll
    for (int i = 0; i < DR; ++i) S[i] = (ok && pos0 > 0 && r0 + i < D) ? st[(r0 + i) * st_stride] : 0.f;
    for (int i = tid; i < REC_STAGES * stride; i += 128) { const int w = i % stride; rec_ring[i] = (w >= 2 * DM && w < 3 * DM) ? 1.f : 0.f; }
    __syncthreads();
    // this thread's copy roles: one 16-byte piece per token (threads 0..95: q / k / decay rows, 96..127: the values), thread 0 also the scalar
    const int dq = D / 4, n_vec = (CH ? 3 : 2) * dq;
    const float* src = nullptr; int dst = 0; long long step = 0;
    if (tid < n_vec) {
        const int which = tid / dq, c = tid - which * dq;
        src = (which == 0 ? qq + ((long long)row0 * QH + qh) * D : which == 1 ? kk + ((long long)row0 * QH + qh) * D : dec + ((long long)row0 * H + h) * D) + c * 4;
        step = which == 2 ? (long long)H * D : (long long)QH * D; dst = which * DM + c * 4;
    } else if (tid >= 96) {
        const int c = tid - 96;
        if (c * 4 < COLS && blockIdx.z * COLS + c * 4 < VD) { src = vv + ((long long)row0 * H + h) * VD + blockIdx.z * COLS + c * 4; step = (long long)H * VD; dst = 3 * DM + c * 4; }
    }
    const float* src_sc = (tid == 0 && MODE != HY_REC_CHANNEL) ? (DELTA ? beta : dec) + (long long)row0 * H + h : nullptr;
    int issued = 0;
    auto issue = [&]() {                             // next token of the sequence's rows -> ring slot issued % REC_STAGES
        if (issued < len) {
            float* slot = rec_ring + (issued % REC_STAGES) * stride;
            if (src) { cp_async16(slot + dst, src); src += step; }
            if (src_sc) { asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(slot + 3 * DM + REC_CTA_COLS)), "l"(src_sc) : "memory"); src_sc += H; }
        }
        ++issued;
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    for (int i = 0; i < REC_STAGES - 1; ++i) issue();
    float* op = is_norm ? norm_out + (long long)row0 * H + h : out + ((long long)row0 * H + h) * VD + col;
    const long long o_stride = is_norm ? H : (long long)H * VD;
    auto join = [&](int i) {                         // LANES = 4: token i's read-out, its four partial sums added in warp order by warp i % 4
        if (ok && part == (i & 3)) { const float* p = &rec_po[i & 1][0][cl]; op[i * o_stride] = (p[0] + p[COLS]) + (p[2 * COLS] + p[3 * COLS]); }
    };
    for (int i = 0; i < len; ++i) {
        asm volatile("cp.async.wait_group %0;" ::"n"(REC_STAGES - 2) : "memory");
        __syncthreads();                             // token i has landed for everybody; slot (i - 1) % STAGES is free again
        issue();
        if (LANES == 4 && i > 0) join(i - 1);        // its partials were written before this barrier; their buffer is written again at token i + 1, behind the next one
        const float* slot = rec_ring + (i % REC_STAGES) * stride;
        const float v = is_norm ? 1.f : slot[3 * DM + cl], sc = slot[3 * DM + REC_CTA_COLS];
        const float* sq = slot + r0; const float* sk = slot + DM + r0; const float* sg = slot + 2 * DM + r0;
        float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
        if (DELTA) {
            float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
            for (int j = 0; j < DR; j += 4) {
                const float4 g4 = *reinterpret_cast<const float4*>(sg + j), k4 = *reinterpret_cast<const float4*>(sk + j);
                S[j] *= g4.x; S[j + 1] *= g4.y; S[j + 2] *= g4.z; S[j + 3] *= g4.w;
                d0 = fmaf(S[j], k4.x, d0); d1 = fmaf(S[j + 1], k4.y, d1); d2 = fmaf(S[j + 2], k4.z, d2); d3 = fmaf(S[j + 3], k4.w, d3);
            }
            float dot = (d0 + d1) + (d2 + d3);
            if (LANES == 4) {                        // every thread reads the partials before it reaches the next token's first barrier, behind which they are written again
                rec_pd[part][cl] = dot;
                __syncthreads();
                dot = (rec_pd[0][cl] + rec_pd[1][cl]) + (rec_pd[2][cl] + rec_pd[3][cl]);
            }
            const float u = sc * (v - dot);
#pragma unroll
            for (int j = 0; j < DR; j += 4) {
                const float4 q4 = *reinterpret_cast<const float4*>(sq + j), k4 = *reinterpret_cast<const float4*>(sk + j);
                S[j] = fmaf(k4.x, u, S[j]); S[j + 1] = fmaf(k4.y, u, S[j + 1]); S[j + 2] = fmaf(k4.z, u, S[j + 2]); S[j + 3] = fmaf(k4.w, u, S[j + 3]);
                o0 = fmaf(S[j], q4.x, o0); o1 = fmaf(S[j + 1], q4.y, o1); o2 = fmaf(S[j + 2], q4.z, o2); o3 = fmaf(S[j + 3], q4.w, o3);
            }
        } else if (CH) {
#pragma unroll
            for (int j = 0; j < DR; j += 4) {
                const float4 q4 = *reinterpret_cast<const float4*>(sq + j), k4 = *reinterpret_cast<const float4*>(sk + j), g4 = *reinterpret_cast<const float4*>(sg + j);
                S[j] = fmaf(k4.x, v, S[j] * g4.x); S[j + 1] = fmaf(k4.y, v, S[j + 1] * g4.y); S[j + 2] = fmaf(k4.z, v, S[j + 2] * g4.z); S[j + 3] = fmaf(k4.w, v, S[j + 3] * g4.w);
                o0 = fmaf(S[j], q4.x, o0); o1 = fmaf(S[j + 1], q4.y, o1); o2 = fmaf(S[j + 2], q4.z, o2); o3 = fmaf(S[j + 3], q4.w, o3);
            }
        } else {
#pragma unroll
            for (int j = 0; j < DR; j += 4) {
                const float4 q4 = *reinterpret_cast<const float4*>(sq + j), k4 = *reinterpret_cast<const float4*>(sk + j);
                S[j] = fmaf(k4.x, v, S[j] * sc); S[j + 1] = fmaf(k4.y, v, S[j + 1] * sc); S[j + 2] = fmaf(k4.z, v, S[j + 2] * sc); S[j + 3] = fmaf(k4.w, v, S[j + 3] * sc);
                o0 = fmaf(S[j], q4.x, o0); o1 = fmaf(S[j + 1], q4.y, o1); o2 = fmaf(S[j + 2], q4.z, o2); o3 = fmaf(S[j + 3], q4.w, o3);
            }
        }
        float o = (o0 + o1) + (o2 + o3);
        if (LANES == 4) rec_po[i & 1][part][cl] = o;
        else if (ok) op[i * o_stride] = o;
    }
    if (LANES == 4 && len > 0) { __syncthreads(); join(len - 1); }
    if (ok)
#pragma unroll
        for (int i = 0; i < DR; ++i) if (r0 + i < D) st[(r0 + i) * st_stride] = S[i];
}

template <typename TA>
__global__ void __launch_bounds__(128) hy_gated_norm_kernel(const float* o, int C, int group, const float* w, int wlen, const TA* gate, int ld_gate, int gate_before, int act,
                                                             const float* skip, int skip_block, const TA* xs, int ld_xs, TA* out, int ld_out, float eps,
                                                             const float* den_dot, const float* den_floor) {
    HY_PDL();
    __shared__ float red[32];
    const int t = blockIdx.x, c0 = blockIdx.y * group;
    const float dv = den_dot ? 1.0f / (fmaxf(fabsf(den_dot[(long long)t * gridDim.y + blockIdx.y]), den_floor[(long long)t * gridDim.y + blockIdx.y]) + 1e-6f) : 1.f;
    float ss = 0.f;
    for (int i = threadIdx.x; i < group; i += blockDim.x) {
        const int c = c0 + i;
        float v = o[(long long)t * C + c] * dv;
        if (skip) v = fmaf(skip[c / skip_block], ldf(xs + (long long)t * ld_xs + c), v);
        if (gate_before) { const float g = ldf(gate + (long long)t * ld_gate + c); v *= act ? siluf_(g) : sigmoidf_(g); }
        ss += v * v;
    }
    const float rr = 1.0f / sqrtf(block_sum(ss, red) / (float)group + eps);
    for (int i = threadIdx.x; i < group; i += blockDim.x) {
        const int c = c0 + i;
        float v = o[(long long)t * C + c] * dv;
        if (skip) v = fmaf(skip[c / skip_block], ldf(xs + (long long)t * ld_xs + c), v);
        const float g = ldf(gate + (long long)t * ld_gate + c), ga = act ? siluf_(g) : sigmoidf_(g);
        if (gate_before) v *= ga;
        v = v * rr * (w ? w[c % wlen] : 1.f);
        if (!gate_before) v *= ga;
        stf(out + (long long)t * ld_out + c, v);
    }
}

// The same for groups that one warp handles well (prefill-sized steps): a warp per (row, group), four consecutive channels per lane and
// step, no block barrier.  The second pass re-reads what the first left in L1.
__device__ __forceinline__ void ld4(const float* p, float* f) { const float4 u = *reinterpret_cast<const float4*>(p); f[0] = u.x; f[1] = u.y; f[2] = u.z; f[3] = u.w; }
__device__ __forceinline__ void ld4(const __nv_bfloat16* p, float* f) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    f[0] = __uint_as_float(u.x << 16); f[1] = __uint_as_float(u.x & 0xffff0000u); f[2] = __uint_as_float(u.y << 16); f[3] = __uint_as_float(u.y & 0xffff0000u);
}
__device__ __forceinline__ void st4(float* p, const float* f) { *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]); }
__device__ __forceinline__ void st4(__nv_bfloat16* p, const float* f) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}
template <typename TA>
__global__ void __launch_bounds__(128) hy_gated_norm_warp_kernel(const float* __restrict__ o, int C, int group, const float* __restrict__ w, int wlen, const TA* __restrict__ gate,
                                                                  int ld_gate, int gate_before, int act, const float* __restrict__ skip, int skip_block, const TA* __restrict__ xs,
                                                                  int ld_xs, TA* __restrict__ out, int ld_out, float eps, long long n_items,
                                                                  const float* __restrict__ den_dot, const float* __restrict__ den_floor) {
    HY_PDL();
    const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (item >= n_items) return;
    const int lane = threadIdx.x & 31, G = C / group, t = (int)(item / G), c0 = (int)(item % G) * group;
    const float dv = den_dot ? 1.0f / (fmaxf(fabsf(den_dot[item]), den_floor[item]) + 1e-6f) : 1.f;
    float ss = 0.f, v[4], g[4], x4[4];
    for (int i = lane * 4; i < group; i += 128) {
        const int c = c0 + i;
        ld4(o + (long long)t * C + c, v);
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] *= dv;
        if (skip) { ld4(xs + (long long)t * ld_xs + c, x4);
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = fmaf(skip[(c + e) / skip_block], x4[e], v[e]); }
        if (gate_before) { ld4(gate + (long long)t * ld_gate + c, g);
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] *= act ? siluf_(g[e]) : sigmoidf_(g[e]); }
#pragma unroll
        for (int e = 0; e < 4; ++e) ss += v[e] * v[e];
    }
    const float rr = 1.0f / sqrtf(warp_sum(ss) / (float)group + eps);
    for (int i = lane * 4; i < group; i += 128) {
        const int c = c0 + i;
        ld4(o + (long long)t * C + c, v);
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] *= dv;
        if (skip) { ld4(xs + (long long)t * ld_xs + c, x4);
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = fmaf(skip[(c + e) / skip_block], x4[e], v[e]); }
        ld4(gate + (long long)t * ld_gate + c, g);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float ga = act ? siluf_(g[e]) : sigmoidf_(g[e]);
            if (gate_before) v[e] *= ga;
            v[e] = v[e] * rr * (w ? w[(c + e) % wlen] : 1.f);
            if (!gate_before) v[e] *= ga;
        }
        st4(out + (long long)t * ld_out + c, v);
    }
}

// ---------------------------------------------------------------------------------------------------------------------------------
// mixture of experts
// ---------------------------------------------------------------------------------------------------------------------------------
// arg-max over the warp: larger value wins, equal values -> lower index
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o); const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
}
// one warp per token: scores from the fp32 router logits, group-limited choice, weights
__global__ void __launch_bounds__(128) hy_moe_router_kernel(HyRouter m, const float* logits, int ldz, const float* correction, int32_t* idx, float* wgt, int T) {
    HY_PDL();
    extern __shared__ float sm[];
    const int E = m.experts, G = m.groups, per = E / G;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = blockIdx.x * 4 + warp;
    if (t >= T) return;
    float* sc = sm + warp * (2 * E + G);   // [E] sigmoid scores
    float* ch = sc + E;                    // [E] choice scores (masked: -inf)
    float* gs = ch + E;                    // [G] group scores
    for (int e = lane; e < E; e += 32) { const float sg = sigmoidf_(logits[(long long)t * ldz + e]); sc[e] = sg; ch[e] = sg + correction[e]; }
    __syncwarp();
    if (G > 1 && m.keep < G) {
        for (int g = lane; g < G; g += 32) {                     // a group's score: the sum of its two largest choice scores
            float a = -INFINITY, b = -INFINITY;
            for (int i = 0; i < per; ++i) { const float v = ch[g * per + i]; if (v > a) { b = a; a = v; } else if (v > b) b = v; }
            gs[g] = per >= 2 ? a + b : a;
        }
        __syncwarp();
        for (int k = 0; k < m.keep; ++k) {                        // keep the best groups: mark a kept group by +inf
            float bv = -INFINITY; int bi = 0x7fffffff;
            for (int g = lane; g < G; g += 32) { const float v = gs[g]; if (v != INFINITY && (v > bv || (v == bv && g < bi))) { bv = v; bi = g; } }
            warp_argmax(bv, bi);
            if (lane == 0 && bi < G) gs[bi] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32) if (gs[e / per] != INFINITY) ch[e] = -INFINITY;
        __syncwarp();
    }
    float mine = 0.f; int my_e = 0;      // lane k keeps choice k
    for (int k = 0; k < m.top; ++k) {
        float bv = -INFINITY; int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) { const float v = ch[e]; if (v > bv || (v == bv && e < bi && v != -INFINITY)) { bv = v; bi = e; } }
        warp_argmax(bv, bi);
        if (bi >= E) bi = 0;
        if (lane == k) { my_e = bi; mine = sc[bi]; }
        if (lane == 0) ch[bi] = -INFINITY;
        __syncwarp();
    }
    float sum = lane < m.top ? mine : 0.f;
    sum = warp_sum(sum);
    if (lane < m.top) { idx[(long long)t * m.top + lane] = my_e; wgt[(long long)t * m.top + lane] = mine / (sum + 1e-20f) * m.scale; }
}

// one warp per token: z = logits + bias, the `top` largest logits (ties -> lower index), weights = softmax over the chosen ones
__global__ void __launch_bounds__(128) hy_moe_router_softmax_kernel(HyRouter m, const float* logits, int ldz, const float* bias, int32_t* idx, float* wgt, int T) {
    HY_PDL();
    extern __shared__ float sm[];
    const int E = m.experts, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = blockIdx.x * 4 + warp;
    if (t >= T) return;
    float* ch = sm + warp * E;
    for (int e = lane; e < E; e += 32) ch[e] = logits[(long long)t * ldz + e] + (bias ? bias[e] : 0.f);
    __syncwarp();
    float mine = -INFINITY, first = 0.f; int my_e = 0;      // lane k keeps choice k; choice 0 is the largest logit
    for (int k = 0; k < m.top; ++k) {
        float bv = -INFINITY; int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) { const float v = ch[e]; if (v > bv || (v == bv && e < bi && v != -INFINITY)) { bv = v; bi = e; } }
        warp_argmax(bv, bi);
        if (bi >= E) bi = 0;
        if (k == 0) first = bv;
        if (lane == k) { my_e = bi; mine = bv; }
        if (lane == 0) ch[bi] = -INFINITY;
        __syncwarp();
    }
    const float p = lane < m.top ? expf(mine - first) : 0.f;
    const float sum = warp_sum(p);
    if (lane < m.top) { idx[(long long)t * m.top + lane] = my_e; wgt[(long long)t * m.top + lane] = p / sum; }
}

template <typename TA>
__global__ void __launch_bounds__(256) hy_moe_gate_up_kernel(const TA* h, int ldh, const TA* gu, int ldw, int W, int ff, int ffp, const int32_t* idx, int top, TA* act) {
    HY_PDL();
    const int row = blockIdx.x, t = row / top, e = idx[row], warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int f = blockIdx.y * 8 + warp;
    if (f >= ffp) return;
    float v = 0.f;
    if (f < ff) {
        const TA* wg = gu + ((long long)e * 2 * ffp + (f >> 4) * 32 + (f & 15)) * ldw; const TA* wu = wg + 16LL * ldw; const TA* hr = h + (long long)t * ldh;
        float g = 0.f, u = 0.f;
        for (int i = lane; i < W; i += 32) { const float x = ldf(hr + i); g = fmaf(x, ldf(wg + i), g); u = fmaf(x, ldf(wu + i), u); }
        g = warp_sum(g); u = warp_sum(u);
        v = siluf_(g) * u;
    }
    if (lane == 0) stf(act + (long long)row * ffp + f, v);
}
// experts without a gate: act = relu(up h)^2, up rows [E][ffp][ldw]
template <typename TA>
__global__ void __launch_bounds__(256) hy_moe_up_relu2_kernel(const TA* h, int ldh, const TA* up, int ldw, int W, int ff, int ffp, const int32_t* idx, int top, TA* act) {
    HY_PDL();
    const int row = blockIdx.x, t = row / top, e = idx[row], warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int f = blockIdx.y * 8 + warp;
    if (f >= ffp) return;
    float v = 0.f;
    if (f < ff) {
        const TA* wu = up + ((long long)e * ffp + f) * ldw; const TA* hr = h + (long long)t * ldh;
        float u = 0.f;
        for (int i = lane; i < W; i += 32) u = fmaf(ldf(hr + i), ldf(wu + i), u);
        u = fmaxf(warp_sum(u), 0.f);
        v = u * u;
    }
    if (lane == 0) stf(act + (long long)row * ffp + f, v);
}
template <typename TA>
__global__ void __launch_bounds__(256) hy_moe_down_kernel(const TA* act, const TA* down, int W, int ffp, const int32_t* idx, const float* wgt, int top, float* x, float beta) {
    HY_PDL();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n = blockIdx.y * 8 + warp;
    if (n >= W) return;
    float acc = 0.f;
    for (int c = 0; c < top; ++c) {
        const int e = idx[(long long)t * top + c];
        const TA* wd = down + ((long long)e * W + n) * ffp; const TA* ar = act + ((long long)t * top + c) * ffp;
        float d = 0.f;
        for (int i = lane; i < ffp; i += 32) d = fmaf(ldf(ar + i), ldf(wd + i), d);
        d = warp_sum(d);
        acc = fmaf(wgt[(long long)t * top + c], d, acc);
    }
    if (lane == 0) x[(long long)t * W + n] = fmaf(beta, x[(long long)t * W + n], acc);
}

// Expert plan in three small kernels: (1) pairs per expert, (2) one CTA lays the experts' 128-row tiles out one after the other, (3) every
// (token, choice) pair takes the next free row of its expert's tiles.  Which row of a tile a pair gets does not matter: the products treat
// rows independently and a token's choices are added in choice order afterwards, so the result is the same for any assignment.
__global__ void hy_moe_count_kernel(const int32_t* idx, int n, int32_t* cnt) {
    HY_PDL();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int e = i < n ? idx[i] : -1;
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    if (e >= 0 && (threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&cnt[e], __popc(peers));
}
__global__ void __launch_bounds__(1024) hy_moe_layout_kernel(int32_t* cnt, int E, int32_t* base, int32_t* tile_expert, int32_t* n_tiles_out, int max_tiles) {
    HY_PDL();
    if (threadIdx.x == 0) {
        int tiles = 0;
        for (int e = 0; e < E; ++e) {
            base[e] = tiles * 128;
            const int nt = (cnt[e] + 127) / 128;
            for (int k = 0; k < nt && tiles + k < max_tiles; ++k) tile_expert[tiles + k] = e;
            tiles += nt;
        }
        n_tiles_out[0] = tiles < max_tiles ? tiles : max_tiles;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;        // reused as the fill counters of step (3)
}
__global__ void hy_moe_assign_kernel(const int32_t* idx, int n, const int32_t* base, int32_t* fill, int32_t* row_src, int32_t* dst_of) {
    HY_PDL();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int e = i < n ? idx[i] : -1;
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    if (e < 0) return;
    const int lane = threadIdx.x & 31, leader = __ffs(peers) - 1;
    int first = 0;
    if (lane == leader) first = atomicAdd(&fill[e], __popc(peers));
    first = __shfl_sync(peers, first, leader);
    const int dst = base[e] + first + __popc(peers & ((1u << lane) - 1u));
    dst_of[i] = dst; row_src[dst] = i;
}
// the same plan in one CTA for decode-sized steps (n = T * top pairs): counters live in shared memory
__global__ void __launch_bounds__(1024) hy_moe_plan_small_kernel(const int32_t* idx, int n, int E, int32_t* tile_expert, int32_t* row_src, int32_t* n_tiles_out,
                                                                 int32_t* dst_of, int max_tiles) {
    HY_PDL();
    extern __shared__ int32_t plan_sm[];
    int32_t* cnt = plan_sm; int32_t* base = plan_sm + E; __shared__ int tiles_sh;
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) atomicAdd(&cnt[idx[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int tiles = 0;
        for (int e = 0; e < E; ++e) {
            base[e] = tiles * 128;
            const int nt = (cnt[e] + 127) / 128;
            for (int k = 0; k < nt && tiles + k < max_tiles; ++k) tile_expert[tiles + k] = e;
            tiles += nt;
        }
        tiles_sh = tiles < max_tiles ? tiles : max_tiles; n_tiles_out[0] = tiles_sh;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < tiles_sh * 128; i += blockDim.x) row_src[i] = -1;
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) { const int e = idx[i], dst = base[e] + atomicAdd(&cnt[e], 1); dst_of[i] = dst; row_src[dst] = i; }
}
__global__ void hy_moe_gather_kernel(const __nv_bfloat16* h, int ldh, int W, const int32_t* row_src, const int32_t* n_tiles, int top, __nv_bfloat16* out) {
    HY_PDL();
    const int row = blockIdx.x;
    if (row >= n_tiles[0] * 128) return;
    const int src = row_src[row];
    const uint4 z = make_uint4(0, 0, 0, 0);
    for (int c = threadIdx.x * 8; c < W; c += blockDim.x * 8)
        *reinterpret_cast<uint4*>(out + (long long)row * W + c) = src >= 0 ? *reinterpret_cast<const uint4*>(h + (long long)(src / top) * ldh + c) : z;
}
__global__ void hy_moe_combine_kernel(const float* y, int ldy, const int32_t* dst_of, const float* wgt, int top, float* x, int W, float beta) {
    HY_PDL();
    const int t = blockIdx.x;                       // W and ldy are multiples of 4 on this path
    for (int c = threadIdx.x * 4; c < W; c += blockDim.x * 4) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = 0; k < top; ++k) {
            const float w = wgt[(long long)t * top + k];
            const float4 v = *reinterpret_cast<const float4*>(y + (long long)dst_of[(long long)t * top + k] * ldy + c);
            acc.x = fmaf(w, v.x, acc.x); acc.y = fmaf(w, v.y, acc.y); acc.z = fmaf(w, v.z, acc.z); acc.w = fmaf(w, v.w, acc.w);
        }
        float4* xp = reinterpret_cast<float4*>(x + (long long)t * W + c);
        float4 xv = *xp; xv.x = fmaf(beta, xv.x, acc.x); xv.y = fmaf(beta, xv.y, acc.y); xv.z = fmaf(beta, xv.z, acc.z); xv.w = fmaf(beta, xv.w, acc.w); *xp = xv;
    }
}

__global__ void hy_gather_rows_f32_kernel(const float* x, const int32_t* rows, float* out, int W) {
    HY_PDL();
    const int i = blockIdx.x;
    for (int c = threadIdx.x; c < W; c += blockDim.x) out[(long long)i * W + c] = x[(long long)rows[i] * W + c];
}
__global__ void __launch_bounds__(256) hy_argmax_rows_kernel(float* logits, int V, float softcap, int32_t* out_ids) {
    HY_PDL();
    __shared__ float bv[8]; __shared__ int bi[8];
    float* lr = logits + (long long)blockIdx.x * V;
    float v = -INFINITY; int i = 0x7fffffff;
    for (int c = threadIdx.x; c < V; c += blockDim.x) {
        float f = lr[c];
        if (softcap > 0.f) { f = softcap * tanhf(f / softcap); lr[c] = f; }
        if (f > v || (f == v && c < i)) { v = f; i = c; }
    }
    warp_argmax(v, i);
    if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = v; bi[threadIdx.x >> 5] = i; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) if (bv[w] > v || (bv[w] == v && bi[w] < i)) { v = bv[w]; i = bi[w]; }
        out_ids[blockIdx.x] = i < V ? i : 0;
    }
}
__global__ void hy_add_rowvec_kernel(float* x, const float* v, int W) {
    HY_PDL();
    for (int c = threadIdx.x; c < W; c += blockDim.x) x[(long long)blockIdx.x * W + c] += v[c];
}

}  // namespace

#define HY_DISPATCH(f32, KERN, ...) ((f32) ? launch_plain(KERN<float>, __VA_ARGS__) : launch_plain(KERN<__nv_bfloat16>, __VA_ARGS__))
using bf = __nv_bfloat16;

template <typename TA>
static cudaError_t gemm_t(int mode, const void* A, int lda, const void* B, int ldb, void* C, int ldc, int M, int N, int K, const float* bias, float alpha, int batch,
                          long long sA, long long sB, long long sC, cudaStream_t s, int act) {
    dim3 grid((N + 63) / 64, (M + 63) / 64, batch);
    const TA* a = reinterpret_cast<const TA*>(A); const TA* b = reinterpret_cast<const TA*>(B);
    switch (mode) {
        case HY_STORE: return launch_plain(hy_gemm_kernel<TA, HY_STORE>, grid, dim3(256), 0, s, a, lda, b, ldb, C, ldc, M, N, K, bias, alpha, sA, sB, sC, act);
        case HY_STORE_F32: return launch_plain(hy_gemm_kernel<TA, HY_STORE_F32>, grid, dim3(256), 0, s, a, lda, b, ldb, C, ldc, M, N, K, bias, alpha, sA, sB, sC, act);
        case HY_ACC_F32: return launch_plain(hy_gemm_kernel<TA, HY_ACC_F32>, grid, dim3(256), 0, s, a, lda, b, ldb, C, ldc, M, N, K, bias, alpha, sA, sB, sC, act);
    }
    return cudaErrorInvalidValue;
}
cudaError_t hy_gemm(bool f32, int mode, const void* A, int lda, const void* B, int ldb, void* C, int ldc, int M, int N, int K, const float* bias, float alpha, int batch,
                    long long sA, long long sB, long long sC, cudaStream_t s, int act) {
    if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return cudaSuccess;
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (!f32 && M <= HY_GEMM_FEW_ROWS && K % 8 == 0 && K <= 1024 && lda % 8 == 0 && ldb % 8 == 0 && sA % 8 == 0 && sB % 8 == 0 && al16(A) && al16(B)) {
        const dim3 grid((N + 7) / 8, batch);
        switch (mode) {
            case HY_STORE: return launch_plain(hy_gemm_fewrows_kernel<HY_STORE>, grid, dim3(256), 0, s, (const bf*)A, lda, (const bf*)B, ldb, C, ldc, M, N, K, bias, alpha, sA, sB, sC, act);
            case HY_STORE_F32: return launch_plain(hy_gemm_fewrows_kernel<HY_STORE_F32>, grid, dim3(256), 0, s, (const bf*)A, lda, (const bf*)B, ldb, C, ldc, M, N, K, bias, alpha, sA, sB, sC, act);
            default: return launch_plain(hy_gemm_fewrows_kernel<HY_ACC_F32>, grid, dim3(256), 0, s, (const bf*)A, lda, (const bf*)B, ldb, C, ldc, M, N, K, bias, alpha, sA, sB, sC, act);
        }
    }
    return f32 ? gemm_t<float>(mode, A, lda, B, ldb, C, ldc, M, N, K, bias, alpha, batch, sA, sB, sC, s, act)
               : gemm_t<bf>(mode, A, lda, B, ldb, C, ldc, M, N, K, bias, alpha, batch, sA, sB, sC, s, act);
}
cudaError_t hy_embed(bool f32, const int32_t* ids, const void* table, float* x, float* x0, int T, int W, int vocab, float scale, cudaStream_t s, void* h, int ldh) {
    return f32 ? launch_plain(hy_embed_kernel<float>, dim3(T), dim3(128), 0, s, ids, (const float*)table, x, x0, T, W, vocab, scale, (float*)h, ldh)
               : launch_plain(hy_embed_kernel<bf>, dim3(T), dim3(128), 0, s, ids, (const bf*)table, x, x0, T, W, vocab, scale, (bf*)h, ldh);
}
cudaError_t hy_concat(bool f32, const float* x, const float* x0, void* cat, int T, int W, cudaStream_t s) {
    return f32 ? launch_plain(hy_concat_kernel<float>, dim3(T), dim3(128), 0, s, x, x0, (float*)cat, T, W)
               : launch_plain(hy_concat_kernel<bf>, dim3(T), dim3(128), 0, s, x, x0, (bf*)cat, T, W);
}
cudaError_t hy_layernorm(bool f32, const float* x, const int32_t* rows, const float* w, void* out, int ldo, int T, int W, float eps, cudaStream_t s) {
    if (T <= 0) return cudaSuccess;
    if (W % 4 == 0 && W <= 8192 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0)
        return f32 ? launch_plain(hy_layernorm_reg_kernel<float>, dim3(T), dim3(256), 0, s, x, rows, w, (float*)out, ldo, W, eps)
                   : launch_plain(hy_layernorm_reg_kernel<bf>, dim3(T), dim3(256), 0, s, x, rows, w, (bf*)out, ldo, W, eps);
    return f32 ? launch_plain(hy_layernorm_kernel<float>, dim3(T), dim3(256), 0, s, x, rows, w, (float*)out, ldo, W, eps)
               : launch_plain(hy_layernorm_kernel<bf>, dim3(T), dim3(256), 0, s, x, rows, w, (bf*)out, ldo, W, eps);
}
cudaError_t hy_mla_prep(bool f32, const HyLatentAttn& a, const void* q, int ldq, const void* ckv, int ldc, const float* norm_w, float eps, const float* rope_cos,
                        const float* rope_sin, void* cache, float* q_abs, const HyRows& r, cudaStream_t s) {
    return f32 ? launch_plain(hy_mla_prep_kernel<float>, dim3(r.T), dim3(128), 0, s, a, (const float*)q, ldq, (const float*)ckv, ldc, norm_w, eps, rope_cos, rope_sin, (float*)cache, q_abs, r)
               : launch_plain(hy_mla_prep_kernel<bf>, dim3(r.T), dim3(128), 0, s, a, (const bf*)q, ldq, (const bf*)ckv, ldc, norm_w, eps, rope_cos, rope_sin, (bf*)cache, q_abs, r);
}
cudaError_t hy_mla_attention(bool f32, const HyLatentAttn& a, const float* q_abs, const void* cache, void* lat_out, const HyRows& r, cudaStream_t s) {
    if (a.kv_rank > 32 * MLA_ACC) return cudaErrorInvalidValue;
    const size_t smem = (size_t)(a.kv_rank + a.rot_dim + 4 * a.kv_rank + 8) * 4;
    return f32 ? launch_plain(hy_mla_attention_kernel<float>, dim3(r.T, a.heads), dim3(128), smem, s, a, q_abs, (const float*)cache, (float*)lat_out, r)
               : launch_plain(hy_mla_attention_kernel<bf>, dim3(r.T, a.heads), dim3(128), smem, s, a, q_abs, (const bf*)cache, (bf*)lat_out, r);
}
static size_t mla_mma_smem(int E, int kt) { return (size_t)(MLA_MQ + 2 * kt) * (E + 8) * 2 + MLA_MQ * 4; }
static int mla_mma_nvb(const HyLatentAttn& a) {
    const int E = a.kv_rank + a.rot_dim;
    if (E % 16 != 0 || a.kv_rank % 64 != 0) return 0;
    const int nvb = a.kv_rank % 256 == 0 ? 32 : (a.kv_rank % 128 == 0 ? 16 : 8);
    return mla_mma_smem(E, 16) <= 200 * 1024 ? nvb : 0;
}
bool hy_mla_mma_supported(const HyLatentAttn& a) { return mla_mma_nvb(a) != 0; }
template <int NVB, int KT>
static cudaError_t mla_mma_launch(const HyLatentAttn& a, const float* q_abs, const void* cache, void* lat_out, const HyRows& r, const int32_t* tile_seq,
                                  const int32_t* tile_q0, int n_tiles, const HyMlaSplit& sp, cudaStream_t s) {
    static bool done[16] = {};
    cudaError_t e = ensure_dynamic_smem(hy_mla_attention_mma_kernel<NVB, KT>, 200 * 1024, done);      // set once per device: the most any size asks for
    if (e != cudaSuccess) return e;
    dim3 grid(n_tiles, a.kv_rank / (NVB * 8));
    return launch_plain(hy_mla_attention_mma_kernel<NVB, KT>, grid, dim3(128), mla_mma_smem(a.kv_rank + a.rot_dim, KT), s, a, q_abs, (const bf*)cache, (bf*)lat_out, r,
                        tile_seq, tile_q0, sp);
}
cudaError_t hy_mla_merge(const int32_t* item_row, const int32_t* item_slot0, const int32_t* item_parts, int n_items, const float* ws_o, const float* ws_ml, void* lat_out,
                         int heads, int kv_rank, cudaStream_t s, const float* sink) {
    if (n_items <= 0) return cudaSuccess;
    return launch_plain(hy_mla_merge_kernel, dim3(n_items, heads), dim3(128), 0, s, item_row, item_slot0, item_parts, ws_o, ws_ml, (bf*)lat_out, heads, kv_rank, sink);
}
cudaError_t hy_mla_attention_mma(const HyLatentAttn& a, const float* q_abs, const void* cache, void* lat_out, const HyRows& r, const int32_t* tile_seq,
                                 const int32_t* tile_q0, int n_tiles, const HyMlaSplit& sp, cudaStream_t s) {
    const int nvb = mla_mma_nvb(a), E = a.kv_rank + a.rot_dim;
    if (!nvb) return cudaErrorInvalidValue;
    // 32-row tiles when two CTAs (8 warps) still fit an SM's shared memory or nothing smaller would make them fit; else 16-row tiles
    // (a step with few tiles — decoding — is a latency chain per CTA: the larger tile halves its length)
    // — and never a tile that the 200 KB opt-in limit does not hold (wide latents: only the 16-row tile is left)
    const bool kt32 = mla_mma_smem(E, 32) <= 200 * 1024 &&
                      (mla_mma_smem(E, 32) <= 113 * 1024 || mla_mma_smem(E, 16) > 113 * 1024 || n_tiles * (a.kv_rank / (nvb * 8)) < 296);
#define HY_MLA(NVB) (kt32 ? mla_mma_launch<NVB, 32>(a, q_abs, cache, lat_out, r, tile_seq, tile_q0, n_tiles, sp, s) : mla_mma_launch<NVB, 16>(a, q_abs, cache, lat_out, r, tile_seq, tile_q0, n_tiles, sp, s))
    return nvb == 32 ? HY_MLA(32) : nvb == 16 ? HY_MLA(16) : HY_MLA(8);
#undef HY_MLA
}
static int mha_nvb(const HyLatentAttn& a) {
    if ((a.dim + a.rot_dim) % 16 != 0 || a.dim % 8 != 0 || a.rot_dim % 8 != 0 || a.kv_rank % 8 != 0) return 0;
    return a.vdim == 128 ? 16 : a.vdim == 64 ? 8 : a.vdim == 32 ? 4 : a.vdim == 16 ? 2 : 0;
}
bool hy_mha_prefill_supported(const HyLatentAttn& a) { return mha_nvb(a) != 0 && a.dim + a.rot_dim <= 512; }
cudaError_t hy_gather_ctx(const void* cache, int E, const HyRows& r, const int32_t* seq_base, int max_ctx, void* lat_ctx, cudaStream_t s) {
    return launch_plain(hy_gather_ctx_kernel, dim3(r.S, (max_ctx + 15) / 16), dim3(128), 0, s, (const bf*)cache, E, r.block_tables, r.max_pages_per_seq, seq_base, r.seq_row0,
                        r.positions, (bf*)lat_ctx);
}
template <int NVB>
static cudaError_t mha_launch(const HyLatentAttn& a, const void* q, int ldq, const float* q_abs, const void* kv_ctx, int ld_kv, const void* lat_ctx, void* mix, int ld_mix,
                              const HyRows& r, const int32_t* tile_seq, const int32_t* tile_head, const int32_t* tile_row0, const int32_t* seq_base, int n_tiles, cudaStream_t s) {
    static bool done[16] = {};
    cudaError_t e = ensure_dynamic_smem(hy_mha_prefill_mma_kernel<NVB>, 200 * 1024, done);
    if (e != cudaSuccess) return e;
    const size_t smem = (size_t)(MLA_MQ + 64) * (a.dim + a.rot_dim + 8) * 2 + (size_t)64 * (NVB * 8 + 8) * 2 + MLA_MQ * 4;
    return launch_plain(hy_mha_prefill_mma_kernel<NVB>, dim3(n_tiles), dim3(128), smem, s, a, (const bf*)q, ldq, q_abs, (const bf*)kv_ctx, ld_kv, (const bf*)lat_ctx, (bf*)mix,
                        ld_mix, r, tile_seq, tile_head, tile_row0, seq_base);
}
cudaError_t hy_mha_prefill(const HyLatentAttn& a, const void* q, int ldq, const float* q_abs, const void* kv_ctx, int ld_kv, const void* lat_ctx, void* mix, int ld_mix,
                           const HyRows& r, const int32_t* tile_seq, const int32_t* tile_head, const int32_t* tile_row0, const int32_t* seq_base, int n_tiles, cudaStream_t s) {
    if (n_tiles <= 0) return cudaSuccess;
    switch (mha_nvb(a)) {
        case 16: return mha_launch<16>(a, q, ldq, q_abs, kv_ctx, ld_kv, lat_ctx, mix, ld_mix, r, tile_seq, tile_head, tile_row0, seq_base, n_tiles, s);
        case 8: return mha_launch<8>(a, q, ldq, q_abs, kv_ctx, ld_kv, lat_ctx, mix, ld_mix, r, tile_seq, tile_head, tile_row0, seq_base, n_tiles, s);
        case 4: return mha_launch<4>(a, q, ldq, q_abs, kv_ctx, ld_kv, lat_ctx, mix, ld_mix, r, tile_seq, tile_head, tile_row0, seq_base, n_tiles, s);
        case 2: return mha_launch<2>(a, q, ldq, q_abs, kv_ctx, ld_kv, lat_ctx, mix, ld_mix, r, tile_seq, tile_head, tile_row0, seq_base, n_tiles, s);
    }
    return cudaErrorInvalidValue;
}
cudaError_t hy_conv_silu(bool f32, const void* in, int ld_in, int C, const float* w, const float* bias, int taps, void* out, int ld_out, const void* tails, const HyRows& r,
                         cudaStream_t s, int act) {
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (!f32 && r.T >= 512 && taps >= 2 && taps <= 4 && C % 8 == 0 && ld_in % 8 == 0 && ld_out % 8 == 0 && al16(in) && al16(out) && al16(tails)) {
        const dim3 g((C / 8 + 127) / 128, (r.T + CONV_ROWS - 1) / CONV_ROWS);
        switch (taps) {
            case 2: return launch_plain(hy_conv_silu_vec8_kernel<2>, g, dim3(128), 0, s, (const bf*)in, ld_in, C, w, bias, (bf*)out, ld_out, (const bf*)tails, r, act);
            case 3: return launch_plain(hy_conv_silu_vec8_kernel<3>, g, dim3(128), 0, s, (const bf*)in, ld_in, C, w, bias, (bf*)out, ld_out, (const bf*)tails, r, act);
            default: return launch_plain(hy_conv_silu_vec8_kernel<4>, g, dim3(128), 0, s, (const bf*)in, ld_in, C, w, bias, (bf*)out, ld_out, (const bf*)tails, r, act);
        }
    }
    dim3 grid((C + 127) / 128, r.T);
    return f32 ? launch_plain(hy_conv_silu_kernel<float>, grid, dim3(128), 0, s, (const float*)in, ld_in, C, w, bias, taps, (float*)out, ld_out, (const float*)tails, r, act)
               : launch_plain(hy_conv_silu_kernel<bf>, grid, dim3(128), 0, s, (const bf*)in, ld_in, C, w, bias, taps, (bf*)out, ld_out, (const bf*)tails, r, act);
}
cudaError_t hy_conv_tails(bool f32, const void* in, int ld_in, int C, int taps, void* tails, const HyRows& r, cudaStream_t s) {
    if (taps <= 1) return cudaSuccess;
    dim3 grid((C + 127) / 128, r.S);
    return f32 ? launch_plain(hy_conv_tails_kernel<float>, grid, dim3(128), 0, s, (const float*)in, ld_in, C, taps, (float*)tails, r)
               : launch_plain(hy_conv_tails_kernel<bf>, grid, dim3(128), 0, s, (const bf*)in, ld_in, C, taps, (bf*)tails, r);
}
cudaError_t hy_delta_prep(bool f32, const HyDelta& d, const void* conv, int ld_conv, const void* b, int ld_b, const void* a, int ld_a, const float* A_log,
                          const float* dt_bias, float* qq, float* kk, float* vv, float* dec, float* beta, int T, cudaStream_t s) {
    return f32 ? launch_plain(hy_delta_prep_kernel<float>, dim3(T), dim3(128), 0, s, d, (const float*)conv, ld_conv, (const float*)b, ld_b, (const float*)a, ld_a, A_log, dt_bias, qq, kk, vv, dec, beta)
               : launch_plain(hy_delta_prep_kernel<bf>, dim3(T), dim3(128), 0, s, d, (const bf*)conv, ld_conv, (const bf*)b, ld_b, (const bf*)a, ld_a, A_log, dt_bias, qq, kk, vv, dec, beta);
}
cudaError_t hy_mamba_prep(bool f32, const HyMamba& m, const void* conv, int ld_conv, const void* dt, int ld_dt, const float* A_log, const float* dt_bias, float* qq,
                          float* kk, float* vv, float* dec, int T, cudaStream_t s) {
    return f32 ? launch_plain(hy_mamba_prep_kernel<float>, dim3(T), dim3(128), 0, s, m, (const float*)conv, ld_conv, (const float*)dt, ld_dt, A_log, dt_bias, qq, kk, vv, dec)
               : launch_plain(hy_mamba_prep_kernel<bf>, dim3(T), dim3(128), 0, s, m, (const bf*)conv, ld_conv, (const bf*)dt, ld_dt, A_log, dt_bias, qq, kk, vv, dec);
}
cudaError_t hy_recurrence(int mode, const float* qq, const float* kk, const float* vv, const float* dec, const float* beta, float* out, float* state, int heads,
                          int qk_heads, int dim, int vdim, const HyRows& r, cudaStream_t s, float* norm_state, float* norm_out) {
    if (mode < 0 || mode > 2 || (norm_state && (mode == HY_REC_DELTA || !norm_out))) return cudaErrorInvalidValue;
    const int cols = vdim + (norm_state ? 1 : 0);
    if (dim <= 128 && dim % 4 == 0 && vdim % 4 == 0) {
        // one thread per column runs a chain of 4 dim dependent-ish operations per token with one or two warps per scheduler; beyond 32
        // rows the rows are split over the CTA's four warps (by the sizes alone: the order of a sum never depends on the step)
        const bool wide = dim > 32;
        dim3 grid(r.S, heads, (cols * (wide ? 4 : 1) + REC_CTA_COLS - 1) / REC_CTA_COLS);
        const int dm = dim <= 32 ? 32 : dim <= 64 ? 64 : 128;
        const size_t ring = (size_t)REC_STAGES * (3 * dm + REC_CTA_COLS + 4) * 4;
#define HY_REC(MD, DM, LN) launch_plain(hy_recurrence_reg_kernel<MD, DM, LN>, grid, dim3(128), ring, s, qq, kk, vv, dec, beta, out, state, heads, qk_heads, dim, vdim, r, norm_state, norm_out)
#define HY_REC_DM(MD, LN) (dm == 32 ? HY_REC(MD, 32, LN) : dm == 64 ? HY_REC(MD, 64, LN) : HY_REC(MD, 128, LN))
        if (mode == HY_REC_DELTA) return wide ? HY_REC_DM(HY_REC_DELTA, 4) : HY_REC_DM(HY_REC_DELTA, 1);
        if (mode == HY_REC_CHANNEL) return wide ? HY_REC_DM(HY_REC_CHANNEL, 4) : HY_REC_DM(HY_REC_CHANNEL, 1);
        return wide ? HY_REC_DM(HY_REC_SCALAR, 4) : HY_REC_DM(HY_REC_SCALAR, 1);
#undef HY_REC_DM
#undef HY_REC
    }
    const size_t smem = (size_t)(dim * REC_COLS + 3 * dim) * 4;
    dim3 grid(r.S, heads, (cols + REC_COLS - 1) / REC_COLS);
    static bool attr_done[3][16] = {};
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    if (smem > 48 * 1024) {      // the limit is set once per kernel and device: raise it to the most any size may ask for
        cudaError_t e = mode == HY_REC_DELTA ? ensure_dynamic_smem(hy_recurrence_kernel<HY_REC_DELTA>, 200 * 1024, attr_done[0])
                      : mode == HY_REC_CHANNEL ? ensure_dynamic_smem(hy_recurrence_kernel<HY_REC_CHANNEL>, 200 * 1024, attr_done[2])
                                               : ensure_dynamic_smem(hy_recurrence_kernel<HY_REC_SCALAR>, 200 * 1024, attr_done[1]);
        if (e != cudaSuccess) return e;
    }
#define HY_RECG(MD) launch_plain(hy_recurrence_kernel<MD>, grid, dim3(REC_COLS), smem, s, qq, kk, vv, dec, beta, out, state, heads, qk_heads, dim, vdim, r, norm_state, norm_out)
    return mode == HY_REC_DELTA ? HY_RECG(HY_REC_DELTA) : mode == HY_REC_CHANNEL ? HY_RECG(HY_REC_CHANNEL) : HY_RECG(HY_REC_SCALAR);
#undef HY_RECG
}
cudaError_t hy_gated_norm(bool f32, const float* o, int C, int group, const float* w, int wlen, const void* gate, int ld_gate, int gate_before, int act, const float* skip,
                          int skip_block, const void* xs, int ld_xs, void* out, int ld_out, float eps, int T, cudaStream_t s, const float* den_dot, const float* den_floor) {
    // The choice of kernel rests on the sizes of the model only, never on the step: a row's bits do not depend on its batch.
    const size_t ea = f32 ? 4 : 2;
    auto al = [](const void* p, size_t a) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; };
    if (group % 4 == 0 && group <= 512 && C % 4 == 0 && ld_gate % 4 == 0 && ld_out % 4 == 0 && (!skip || ld_xs % 4 == 0) && al(o, 16) && al(gate, 4 * ea) && al(out, 4 * ea) && al(xs, 4 * ea)) {
        const long long n = (long long)T * (C / group);
        const dim3 g((unsigned)((n + 3) / 4));
        return f32 ? launch_plain(hy_gated_norm_warp_kernel<float>, g, dim3(128), 0, s, o, C, group, w, wlen, (const float*)gate, ld_gate, gate_before, act, skip, skip_block, (const float*)xs, ld_xs, (float*)out, ld_out, eps, n, den_dot, den_floor)
                   : launch_plain(hy_gated_norm_warp_kernel<bf>, g, dim3(128), 0, s, o, C, group, w, wlen, (const bf*)gate, ld_gate, gate_before, act, skip, skip_block, (const bf*)xs, ld_xs, (bf*)out, ld_out, eps, n, den_dot, den_floor);
    }
    dim3 grid(T, C / group);
    return f32 ? launch_plain(hy_gated_norm_kernel<float>, grid, dim3(128), 0, s, o, C, group, w, wlen, (const float*)gate, ld_gate, gate_before, act, skip, skip_block, (const float*)xs, ld_xs, (float*)out, ld_out, eps, den_dot, den_floor)
               : launch_plain(hy_gated_norm_kernel<bf>, grid, dim3(128), 0, s, o, C, group, w, wlen, (const bf*)gate, ld_gate, gate_before, act, skip, skip_block, (const bf*)xs, ld_xs, (bf*)out, ld_out, eps, den_dot, den_floor);
}
cudaError_t hy_moe_router(const HyRouter& m, const float* logits, int ldz, const float* correction, int32_t* idx, float* wgt, int T, cudaStream_t s) {
    const size_t smem = (size_t)4 * (2 * m.experts + m.groups) * 4;
    return launch_plain(hy_moe_router_kernel, dim3((T + 3) / 4), dim3(128), smem, s, m, logits, ldz, correction, idx, wgt, T);
}
cudaError_t hy_moe_router_softmax(const HyRouter& m, const float* logits, int ldz, const float* bias, int32_t* idx, float* wgt, int T, cudaStream_t s) {
    if (m.top > 32) return cudaErrorInvalidValue;
    return launch_plain(hy_moe_router_softmax_kernel, dim3((T + 3) / 4), dim3(128), (size_t)4 * m.experts * 4, s, m, logits, ldz, bias, idx, wgt, T);
}
cudaError_t hy_moe_gate_up(bool f32, int relu2, const void* h, int ldh, const void* gu, int ldw, int W, int ff, int ffp, const int32_t* idx, int top, void* act, int T, cudaStream_t s) {
    dim3 grid(T * top, (ffp + 7) / 8);
    if (relu2)
        return f32 ? launch_plain(hy_moe_up_relu2_kernel<float>, grid, dim3(256), 0, s, (const float*)h, ldh, (const float*)gu, ldw, W, ff, ffp, idx, top, (float*)act)
                   : launch_plain(hy_moe_up_relu2_kernel<bf>, grid, dim3(256), 0, s, (const bf*)h, ldh, (const bf*)gu, ldw, W, ff, ffp, idx, top, (bf*)act);
    return f32 ? launch_plain(hy_moe_gate_up_kernel<float>, grid, dim3(256), 0, s, (const float*)h, ldh, (const float*)gu, ldw, W, ff, ffp, idx, top, (float*)act)
               : launch_plain(hy_moe_gate_up_kernel<bf>, grid, dim3(256), 0, s, (const bf*)h, ldh, (const bf*)gu, ldw, W, ff, ffp, idx, top, (bf*)act);
}
cudaError_t hy_moe_down(bool f32, const void* act, const void* down, int W, int ffp, const int32_t* idx, const float* wgt, int top, float* x, int T, cudaStream_t s, float beta) {
    dim3 grid(T, (W + 7) / 8);
    return f32 ? launch_plain(hy_moe_down_kernel<float>, grid, dim3(256), 0, s, (const float*)act, (const float*)down, W, ffp, idx, wgt, top, x, beta)
               : launch_plain(hy_moe_down_kernel<bf>, grid, dim3(256), 0, s, (const bf*)act, (const bf*)down, W, ffp, idx, wgt, top, x, beta);
}
cudaError_t hy_moe_plan(const int32_t* idx, int T, int top, int experts, int32_t* tile_expert, int32_t* row_src, int32_t* n_tiles_out, int32_t* dst_of, int max_tiles,
                        cudaStream_t s) {
    // scratch after n_tiles_out[0]: [4 ..] counters [experts], then bases [experts]
    int32_t* cnt = n_tiles_out + 4; int32_t* base = cnt + experts; const int n = T * top;
    if (n <= 4096) return launch_plain(hy_moe_plan_small_kernel, dim3(1), dim3(1024), (size_t)2 * experts * 4, s, idx, n, experts, tile_expert, row_src, n_tiles_out, dst_of, max_tiles);
    cudaError_t e = cudaMemsetAsync(cnt, 0, (size_t)experts * 4, s);
    if (e != cudaSuccess) return e;
    if ((e = cudaMemsetAsync(row_src, 0xFF, (size_t)max_tiles * 128 * 4, s)) != cudaSuccess) return e;
    if ((e = launch_plain(hy_moe_count_kernel, dim3((n + 255) / 256), dim3(256), 0, s, idx, n, cnt)) != cudaSuccess) return e;
    if ((e = launch_plain(hy_moe_layout_kernel, dim3(1), dim3(1024), 0, s, cnt, experts, base, tile_expert, n_tiles_out, max_tiles)) != cudaSuccess) return e;
    return launch_plain(hy_moe_assign_kernel, dim3((n + 255) / 256), dim3(256), 0, s, idx, n, base, cnt, row_src, dst_of);
}
cudaError_t hy_moe_gather(const void* h, int ldh, int W, const int32_t* row_src, const int32_t* n_tiles, int top, void* out, int max_tiles, cudaStream_t s) {
    return launch_plain(hy_moe_gather_kernel, dim3(max_tiles * 128), dim3(128), 0, s, (const bf*)h, ldh, W, row_src, n_tiles, top, (bf*)out);
}
cudaError_t hy_moe_combine(const float* y, int ldy, const int32_t* dst_of, const float* wgt, int top, float* x, int W, int T, cudaStream_t s, float beta) {
    return launch_plain(hy_moe_combine_kernel, dim3(T), dim3(256), 0, s, y, ldy, dst_of, wgt, top, x, W, beta);
}
cudaError_t hy_gather_rows_f32(const float* x, const int32_t* rows, float* out, int n, int W, cudaStream_t s) {
    if (n <= 0) return cudaSuccess;
    return launch_plain(hy_gather_rows_f32_kernel, dim3(n), dim3(128), 0, s, x, rows, out, W);
}
cudaError_t hy_argmax_rows(float* logits, int n, int V, float softcap, int32_t* out_ids, cudaStream_t s) {
    if (n <= 0) return cudaSuccess;
    return launch_plain(hy_argmax_rows_kernel, dim3(n), dim3(256), 0, s, logits, V, softcap, out_ids);
}
cudaError_t hy_add_rowvec(float* x, const float* v, int T, int W, cudaStream_t s) { return launch_plain(hy_add_rowvec_kernel, dim3(T), dim3(256), 0, s, x, v, W); }

}  // namespace oa
