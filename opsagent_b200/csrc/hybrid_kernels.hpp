// hybrid_kernels.hpp — launch API of the kernels behind the hybrid decoder family (hybrid_kernels.cu, hybrid_window.cu, hybrid_linear.cu, hybrid_streams.cu): layer norm and RMS
// norm, latent attention over a paged latent cache, windowed attention over paged keys and values (sliding window, kept first tokens,
// differential maps, sink, output gates, soft cap and distance slope on the scores, a norm over the whole projection, a query temperature),
// causal short convolutions with carried tails, the linear recurrences (gated delta rule with per-channel decay, Mamba-2, gated linear
// attention, retention, the xLSTM matrix memory with its normaliser and running maximum) and their operand kernels (hybrid_linear.cu), gated
// group norms, the norm after the sum of post-norm designs, the routers (group-limited sigmoid; softmax over the chosen logits; a table of
// token ids) and the routed experts (SwiGLU; squared ReLU); several residual streams joined by learned coefficients with the RMS norm that
// opens a sublayer, the token shift, rotary preparation of cached keys and values (also fused with short convolutions), rotated values and
// the counter-rotation of the heads' outputs, window / sink / gate on latent attention (hybrid_streams.cu, hybrid_window.cu, hybrid_kernels.cu).
// Each mechanism takes its sizes and constants as arguments.
//
// `f32` selects the activation / matrix element type: false = bf16 storage with fp32 accumulation, true = everything in fp32.  What must be
// fp32 in both modes (residual stream, norms, softmax, router, recurrent state, decays, gates of a recurrence) always is.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace oa {

// per-step row metadata (device pointers into the step's metadata arena).  Rows of one sequence are contiguous.
struct HyRows {
    const int32_t* positions;     // [T] position of each row in its sequence
    const int32_t* slots;         // [T] cache row of each token: page * 64 + offset
    const int32_t* row_seq;       // [T] sequence index of each row
    const int32_t* seq_row0;      // [S + 1] first row of each sequence
    const int32_t* seq_pos0;      // [S] position of a sequence's first row in this step (0: the sequence starts here, its state is taken as zero)
    const int32_t* seq_state;     // [S] recurrent-state slot
    const int32_t* block_tables;  // [S, max_pages_per_seq]
    int max_pages_per_seq, T, S;
};

enum HyGemmMode : int { HY_STORE = 0, HY_STORE_F32 = 1, HY_ACC_F32 = 2 };
// C[z][M,N] (op)= alpha * A[z][M,K] . B[z][N,K]^T (+ bias[N]), z < batch with element strides sA/sB/sC.  Plain tiled FMA GEMM in fp32
// accumulation for any sizes: the fp32 mode's matrix product, and the bf16 mode's fallback where a shape does not fit the tensor-core tiles.
// act = 1: the stored value is relu(.)^2, act = 2: the tanh form of GELU (HY_STORE / HY_STORE_F32)
// bf16 steps of at most HY_GEMM_FEW_ROWS rows with K <= 1024 in aligned groups of 8 take a one-warp-per-output-column kernel instead of the tile kernel
constexpr int HY_GEMM_FEW_ROWS = 32;
cudaError_t hy_gemm(bool f32, int mode, const void* A, int lda, const void* B, int ldb, void* C, int ldc, int M, int N, int K, const float* bias,
                    float alpha, int batch, long long sA, long long sB, long long sC, cudaStream_t s, int act = 0);

// x[t] = table[ids[t]] * scale (fp32); x0 (optional) keeps a copy for a looped block's re-injection
// h (optional, [T, ldh] in the activation type): the same rows as the input of sublayers that read the residual itself
cudaError_t hy_embed(bool f32, const int32_t* ids, const void* table, float* x, float* x0, int T, int W, int vocab, float scale, cudaStream_t s, void* h = nullptr, int ldh = 0);
// cat[t] = [x[t] ; x0[t]] in the activation type (input of the looped block's re-injection projection)
cudaError_t hy_concat(bool f32, const float* x, const float* x0, void* cat, int T, int W, cudaStream_t s);
// out[t] = (x[t] - mean) / sqrt(var + eps) * w   (optionally of the rows `rows[i]` only)
cudaError_t hy_layernorm(bool f32, const float* x, const int32_t* rows, const float* w, void* out, int ldo, int T, int W, float eps, cudaStream_t s);

// out1[t] = x[r] / sqrt(mean(x[r]^2) + eps) * w1, and out2 likewise with w2 when given (r = rows[t] or t): the two norms of a layer whose
// mixer and feed-forward read separate norms of the same residual, or a single RMS norm
cudaError_t hy_rmsnorm_pair(bool f32, const float* x, const int32_t* rows, const float* w1, void* out1, const float* w2, void* out2, int ldo, int T, int W, float eps, cudaStream_t s);

// Norm after the sum, in place on the fp32 residual: v = beta x[t] + branch, x[t] <- layer norm of v with weight w (mean taken off, eps inside
// the root), and h[t] (activation type) = the new x[t], the next sublayer's input.  branch: nothing (y1 == null: the sublayer has already added
// itself into x), y1[t], or — when rw1 is given — branch_scale * (rms_norm(y1[t]) * rw1 + rms_norm(y2[t]) * rw2), two sublayers side by side
// whose outputs are RMS-normed over the width before they meet.
cudaError_t hy_post_norm(bool f32, float* x, float beta, const float* y1, const float* rw1, const float* y2, const float* rw2, float branch_scale, const float* w, void* h, int ldh,
                         int T, int W, float eps, cudaStream_t s);

// Windowed attention over cached keys and values.  A cache row holds one token: [kv_heads x maps x dim keys | kv_heads x vdim values].
// Position i sees j <= i with i - j < window or j < keep_first.  maps = 2: differential attention, out = (a1 - lambda a2) / rms(.) * out_scale
// per head.  gate: 0 none, 1 sigmoid(gate[t, head * vdim + c]), 2 sigmoid(gate[t, head]).  sink (per head, or null) joins the denominator only.
// Score modifiers (all optional): softcap > 0: s <- softcap tanh(s / softcap) after the scale; slope_exp > 0: head h then loses
// 2^(-slope_exp (h + 1) / heads) * (i - j).  qk_norm = 2: one RMS norm over the whole q (k) projection of a row, weights [heads maps dim]
// ([kv_heads maps dim]); q_temp_every > 0: the query at position p is multiplied by 1 + q_temp_coef ln(floor((p + 1) / q_temp_every) + 1).
// out_rot (1: pairs 2m / 2m + 1, 2: pairs m / m + vdim / 2): every head's output at position i is turned by -i over all vdim channels with the
// angles of out_cos / out_sin ([position, vdim / 2]) before the gate: the counterpart of values that were cached turned by their own position.
struct HyWinAttn { int heads, kv_heads, dim, vdim, maps, window, keep_first, qk_norm, gate; float scale, lambda, out_scale; float softcap = 0.f, slope_exp = 0.f, q_temp_coef = 0.f; int q_temp_every = 0;
                   int out_rot = 0; const float* out_cos = nullptr; const float* out_sin = nullptr; };
// Rotary preparation of a cached-key/value attention layer (maps = 1, no query / key norm): the first rot_dims channels of every query head (in
// place) and key head turn by the row's position (layout 0: pairs 2i / 2i + 1, 1: pairs i / i + rot_dims / 2; tables [position, rot_dims / 2]);
// with v_cos / v_sin ([position, vdim / 2]) every value head turns over all of its channels in the same layout; keys and values go to cache row slots[t].
struct HyRotary { int dims, layout; const float* cos; const float* sin; const float* v_cos; const float* v_sin; };
cudaError_t hy_win_rope_prep(bool f32, const HyWinAttn& a, const HyRotary& rot, void* q, int ldq, const void* k, const void* v, int ldkv, void* cache, const HyRows& r, cudaStream_t s);
// The same preparation fused with the short convolutions in front of it (bf16; taps 2 .. 4; interleaved pairs; dim, vdim and the segment
// offsets multiples of 8): `in` [T, ld_in] is the fused projection with the segments q / k / v at columns off_q / off_k / off_v, w [C, taps]
// the taps of all of its C columns, tails the sequences' carried inputs as hy_conv_silu reads them (hy_conv_tails stores the new ones
// afterwards).  The fp32 convolution goes straight into the rotation; queries land in q_out [T, ldq] (head by head), keys and values in the cache.
bool hy_conv_rope_cache_supported(const HyWinAttn& a, const HyRotary& rot, int taps);
cudaError_t hy_conv_rope_cache(const HyWinAttn& a, const HyRotary& rot, const void* in, int ld_in, int C, int off_q, int off_k, int off_v, const float* w, int taps, void* q_out, int ldq,
                               void* cache, const void* tails, const HyRows& r, cudaStream_t s);
bool hy_win_supported(const HyWinAttn& a);
// q [T, ldq] (head by head, map by map): RMS-normed in place with q_norm_w when qk_norm; k / v [T, ldkv] (null: this layer reads a cache
// another layer fills): keys normed alike with k_norm_w, both stored at cache row slots[t].  qk_norm = 2: one norm over the row's whole q (k) projection,
// weights of that size, then the query temperature
cudaError_t hy_win_prep(bool f32, const HyWinAttn& a, void* q, int ldq, const void* k, const void* v, int ldkv, const float* q_norm_w, const float* k_norm_w, float eps, void* cache,
                        const HyRows& r, cudaStream_t s);
// plain form (any sizes, both element types; prefill rows and decoding rows alike): out[t, head * vdim ..] in the activation type
cudaError_t hy_win_attention(bool f32, const HyWinAttn& a, const void* q, int ldq, const void* cache, const float* sink, const void* gate, int ldg, void* out, int ldo, float eps,
                             const HyRows& r, cudaStream_t s);

// tensor-core form (bf16; dim a multiple of 16 up to 128, vdim 16 / 32 / 64 / 96 / 128), for prompt portions and decoding rows alike: a tile =
// 64 consecutive (row, head-of-the-group) pairs of one sequence starting at pair tile_q0 (pair p = row p / group, head p % group of the
// CTA's key/value head, group = heads / kv_heads); grid = tiles x kv_heads.  The host lists the tiles of a step.
constexpr int HY_WIN_TILE_QUERIES = 64;
bool hy_win_mma_supported(const HyWinAttn& a);
cudaError_t hy_win_attention_mma(const HyWinAttn& a, const void* q, int ldq, const void* cache, const float* sink, const void* gate, int ldg, void* out, int ldo, float eps,
                                 const HyRows& r, const int32_t* tile_seq, const int32_t* tile_q0, int n_tiles, cudaStream_t s);

// decoding form of the same: tiles of at most HY_WIN_DECODE_QUERIES pairs (a decoding row's group of heads, a very short portion); the CTA's
// warps deal the key tiles out among themselves and join their partial softmaxes in shared memory
constexpr int HY_WIN_DECODE_QUERIES = 16;
cudaError_t hy_win_decode_mma(const HyWinAttn& a, const void* q, int ldq, const void* cache, const float* sink, const void* gate, int ldg, void* out, int ldo, float eps,
                              const HyRows& r, const int32_t* tile_seq, const int32_t* tile_q0, int n_tiles, cudaStream_t s);

struct HyLatentAttn {             // sizes of one latent-attention layer
    int heads, dim, rot_dim, vdim, kv_rank, rot_dims; float scale;
    // optional parts: window > 0: position i sees j with 0 <= i - j < window (0: every j <= i); rot_layout 1: rotary pairs channel i with
    // i + rot_dims / 2 instead of 2i with 2i + 1; sink (device, one fp32 logit per head): joins the softmax denominator only, unscaled
    int window = 0, rot_layout = 0; const float* sink = nullptr;
    // prefill form only: out[t, c] *= sigmoid(gate[t, c]) over the concatenated heads (bf16, pitch ldg), in the attention kernel's epilogue
    const void* gate = nullptr; int ldg = 0;
};
// From the q projection (q: [T, ldq], head by head [dim | rot_dim]) and the down projection (ckv: [T, ldc] = [kv_rank | rot_dim]):
// latent = rmsnorm(ckv[:rank]) * norm_w and the rotated shared key go to cache row slots[t] ([rank + rot_dim] per row); the rotated query
// parts go to q_abs[t, h, rank:] (fp32, [T, heads, rank + rot_dim]).
cudaError_t hy_mla_prep(bool f32, const HyLatentAttn& a, const void* q, int ldq, const void* ckv, int ldc, const float* norm_w, float eps,
                        const float* rope_cos, const float* rope_sin, void* cache, float* q_abs, const HyRows& r, cudaStream_t s);
// causal softmax attention of every row over its sequence's cached rows 0..position, with absorbed queries q_abs = [W_uk^T q_unrotated | q_rotated]:
// lat_out[t, h, :rank] = sum_j softmax_j(scale * q_abs[t,h] . cache[j]) cache[j][:rank]
cudaError_t hy_mla_attention(bool f32, const HyLatentAttn& a, const float* q_abs, const void* cache, void* lat_out, const HyRows& r, cudaStream_t s);

// the same on the tensor cores (bf16 only; sizes: kv_rank a multiple of 64, kv_rank + rot_dim of 16).  A tile = 64 consecutive (row, head)
// pairs of one sequence starting at pair tile_q0 of sequence tile_seq; the host lists the tiles of a step.
// Decoding rows with long contexts: a tile may cover only the cache rows [tile_k0, tile_k1) (multiples of 32; k1 = 0: to the query's position)
// and then leaves its fp32 partial (sums, running maximum, denominator) in workspace slot tile_slot (-1: final result); hy_mla_merge joins the
// parts of a row in order.  How a row is cut depends on its own position only, never on the rest of the step.
constexpr int HY_MLA_TILE_QUERIES = 64;
struct HyMlaSplit { const int32_t* tile_k0; const int32_t* tile_k1; const int32_t* tile_slot; float* ws_o; float* ws_ml; };   // tile_k0 == null: no tile is cut
bool hy_mla_mma_supported(const HyLatentAttn& a);
cudaError_t hy_mla_attention_mma(const HyLatentAttn& a, const float* q_abs, const void* cache, void* lat_out, const HyRows& r, const int32_t* tile_seq,
                                 const int32_t* tile_q0, int n_tiles, const HyMlaSplit& sp, cudaStream_t s);
cudaError_t hy_mla_merge(const int32_t* item_row, const int32_t* item_slot0, const int32_t* item_parts, int n_items, const float* ws_o, const float* ws_ml, void* lat_out,
                         int heads, int kv_rank, cudaStream_t s, const float* sink = nullptr);

// Prefill form (bf16; dim and rot_dim multiples of 8, their sum of 16, vdim 16 / 32 / 64 / 128): hy_gather_ctx copies the cache rows 0..ctx-1 of
// the sequences with seq_base[s] >= 0 to lat_ctx[seq_base[s] + j]; a GEMM makes kv_ctx = lat_ctx[:, :rank] . [W_uk ; W_uv]^T ([rows, heads dim |
// heads vdim]); hy_mha_prefill then runs causal attention per (sequence, head) — a tile is 64 query rows starting at row tile_row0 of its
// sequence — and writes mix[row, head * vdim ..].  Queries: unrotated part from q ([T, ldq], head by head [dim | rot_dim]), rotated part
// from q_abs[.., rank:].
bool hy_mha_prefill_supported(const HyLatentAttn& a);
cudaError_t hy_gather_ctx(const void* cache, int E, const HyRows& r, const int32_t* seq_base, int max_ctx, void* lat_ctx, cudaStream_t s);
cudaError_t hy_mha_prefill(const HyLatentAttn& a, const void* q, int ldq, const float* q_abs, const void* kv_ctx, int ld_kv, const void* lat_ctx, void* mix, int ld_mix,
                           const HyRows& r, const int32_t* tile_seq, const int32_t* tile_head, const int32_t* tile_row0, const int32_t* seq_base, int n_tiles, cudaStream_t s);

// y = silu(causal conv over time of `in` per channel (+ bias)); inputs before a sequence's first row of this step come from its tail
// (the last taps-1 inputs of earlier steps; zeros at the start of a sequence).  hy_conv_tails then stores the new tails.
// act = 0: no activation (y is the convolution itself)
cudaError_t hy_conv_silu(bool f32, const void* in, int ld_in, int C, const float* w, const float* bias, int taps, void* out, int ld_out,
                         const void* tails, const HyRows& r, cudaStream_t s, int act = 1);
cudaError_t hy_conv_tails(bool f32, const void* in, int ld_in, int C, int taps, void* tails, const HyRows& r, cudaStream_t s);

struct HyDelta { int heads, kv_heads, dim, vdim; };
// unit-norm q (times dim^-1/2) and k, v, beta = sigmoid(b), per-channel decay exp(-exp(A_log_h) softplus(a + dt_bias)) — all fp32
cudaError_t hy_delta_prep(bool f32, const HyDelta& d, const void* qkv_conv, int ld_conv, const void* b, int ld_b, const void* a, int ld_a,
                          const float* A_log, const float* dt_bias, float* qq, float* kk, float* vv, float* dec, float* beta, int T, cudaStream_t s);
struct HyMamba { int heads, vdim, state, groups; };
// dt = softplus(dt + dt_bias); decay exp(-exp(A_log_h) dt); kk = B, qq = C, vv = dt * x — all fp32
cudaError_t hy_mamba_prep(bool f32, const HyMamba& m, const void* xbc_conv, int ld_conv, const void* dt, int ld_dt, const float* A_log,
                          const float* dt_bias, float* qq, float* kk, float* vv, float* dec, int T, cudaStream_t s);
// The linear recurrence both mixers share, per (sequence, head) on an fp32 state S[dim, vdim] carried in `state` (slot-major):
//   delta:  S <- diag(dec_t) S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t
//   plain:  S <- dec_t S + k_t v_t^T;                                            o_t = S^T q_t
// qq/kk: [T, qk_heads, dim]; vv/out: [T, heads, vdim]; dec: [T, heads, dim] (delta) or [T, heads]; head h reads q/k head h / (heads / qk_heads)
// mode HY_REC_CHANNEL: S <- diag(dec_t) S + k_t v_t^T with dec [T, heads, dim] (gated linear attention).
// norm_state != null (plain modes): one more value channel whose value is always 1 — the normaliser n_t = dec_t n_(t-1) + k_t, kept in
// norm_state [slots, heads, dim]; its read-out n_t . q_t goes to norm_out [T, heads].
enum HyRecMode : int { HY_REC_SCALAR = 0, HY_REC_DELTA = 1, HY_REC_CHANNEL = 2 };
cudaError_t hy_recurrence(int mode, const float* qq, const float* kk, const float* vv, const float* dec, const float* beta, float* out,
                          float* state, int heads, int qk_heads, int dim, int vdim, const HyRows& r, cudaStream_t s, float* norm_state = nullptr, float* norm_out = nullptr);

// Operands of the linear-attention recurrences, all fp32.  q / k / v: projection outputs [T, ld] (head by head).
struct HyLinPrep { int heads, dim, vdim; bool q_scaled, k_scaled; int rot_dims; };     // dim^-1/2 on q and / or on k (after the rotation); rotate-half rotary on the first rot_dims channels of every head of q and k (0: none): channel i pairs with i + rot_dims / 2, cos / sin tables [position, rot_dims / 2]
// channel decay (z != null): dec[t, h, d] = sigmoid(z[t, h, d])^(1 / tau) = exp(logsigmoid(z) / tau), in place on the fp32 z (= dec);  head decay: dec[t, h] = decay[h]
cudaError_t hy_lin_prep(bool f32, const HyLinPrep& p, const void* q, const void* k, const void* v, int ld, float* qq, float* kk, float* vv, float* dec_channel, float tau,
                        const float* decay_head, float* dec_head, const float* rope_cos, const float* rope_sin, const HyRows& r, cudaStream_t s);
// Matrix memory.  gates [T, ldg] fp32 = [W_i h + b_i | W_f h + b_f] (heads each).  hy_mlstm_gates: log gates i = cap tanh(. / cap),
// f = logsigmoid(cap tanh(. / cap)); the running maximum m_t = max(f_t + m_(t-1), i_t) per (sequence, head), carried in mstate [slots, heads]
// (a sequence whose step starts at position 0 starts from m = 0); out: dec[t, h] = exp(f + m_(t-1) - m_t), gin[t, h] = exp(i - m_t), floor_[t, h] = exp(-m_t)
cudaError_t hy_mlstm_gates(const float* gates, int ldg, int heads, float cap, float* mstate, float* dec, float* gin, float* floor_, const HyRows& r, cudaStream_t s);
// qq = q dim^-1/2, kk = gin * k, vv = v
cudaError_t hy_mlstm_prep(bool f32, int heads, int dim, int vdim, const void* q, const void* k, const void* v, int ld, const float* gin, float* qq, float* kk, float* vv, int T, cudaStream_t s);
// group-wise RMS norm with a gate: v = o (+ skip[c / skip_block] * xs[t, c]); gate_before ? v *= act(gate) : -; v /= rms over each group of
// `group` channels; v *= w[c % wlen]; !gate_before ? v *= act(gate) : -.  act: 0 = sigmoid, 1 = silu.
// w == null: no weight.  den_dot != null: every group's o is first divided by max(|den_dot[t, g]|, den_floor[t, g]) + 1e-6 (the matrix memory's normaliser)
cudaError_t hy_gated_norm(bool f32, const float* o, int C, int group, const float* w, int wlen, const void* gate, int ld_gate, int gate_before, int act,
                          const float* skip, int skip_block, const void* xs, int ld_xs, void* out, int ld_out, float eps, int T, cudaStream_t s,
                          const float* den_dot = nullptr, const float* den_floor = nullptr);

struct HyRouter { int experts, top, groups, keep; float scale; int kind; };     // kind 0: the sigmoid router below; 1: hy_moe_router_softmax
// sigmoid router over fp32 logits [T, ldz] with a selection-only correction and group-limited choice: a group's score is the sum of its two
// largest corrected scores, only the best `keep` groups compete; idx[t, top], wgt[t, top] = chosen uncorrected sigmoids / their sum * scale
cudaError_t hy_moe_router(const HyRouter& m, const float* logits, int ldz, const float* correction, int32_t* idx, float* wgt, int T, cudaStream_t s);
// router whose weights are the softmax over the chosen logits only: z = logits + bias (fp32), the `top` largest (ties -> lower index), wgt = softmax of those
cudaError_t hy_moe_router_softmax(const HyRouter& m, const float* logits, int ldz, const float* bias, int32_t* idx, float* wgt, int T, cudaStream_t s);
// router without scores: token id -> its `top` experts from table [vocab, top], weight 1 / top each.  shared >= 0: one more choice for every
// token, expert `shared` with weight sigmoid(w_sg . h[t]) (fp32 sum).  idx / wgt: [T, top (+ 1)]
cudaError_t hy_moe_router_table(bool f32, const int32_t* tokens, const int32_t* table, int vocab, int top, int shared, const void* h, int ldh, const void* w_sg, int W,
                                int32_t* idx, float* wgt, int T, cudaStream_t s);
// routed experts, one (token, choice) at a time (decode-sized batches and the fp32 mode).  relu2 == 0: SwiGLU, gu: [E][2 ffp][ldw] with gate / up
// rows interleaved in blocks of 16; relu2 == 1: act = relu(up h)^2, gu: [E][ffp][ldw] (up rows only).  down: [E][W][ffp]; act: [T * top, ffp]
cudaError_t hy_moe_gate_up(bool f32, int relu2, const void* h, int ldh, const void* gu, int ldw, int W, int ff, int ffp, const int32_t* idx, int top, void* act, int T, cudaStream_t s);
// x[t] = beta * x[t] + sum over choices
cudaError_t hy_moe_down(bool f32, const void* act, const void* down, int W, int ffp, const int32_t* idx, const float* wgt, int top, float* x, int T, cudaStream_t s, float beta = 1.f);

// grouped (tensor-core) expert path: rows sorted by expert into 128-row tiles
// counts -> tile table: tile_expert[n_tiles], row_src[max_tiles * 128] (token * top + choice, or -1), dst_of[T * top]; n_tiles_out holds the tile
// count at [0] and 2 * experts words of scratch from [4]
cudaError_t hy_moe_plan(const int32_t* idx, int T, int top, int experts, int32_t* tile_expert, int32_t* row_src, int32_t* n_tiles_out, int32_t* dst_of, int max_tiles, cudaStream_t s);
cudaError_t hy_moe_gather(const void* h, int ldh, int W, const int32_t* row_src, const int32_t* n_tiles, int top, void* out, int max_tiles, cudaStream_t s);
// x[t] = beta * x[t] + sum over choices (in order) wgt[t,c] * y[dst_of[t*top+c]]
cudaError_t hy_moe_combine(const float* y, int ldy, const int32_t* dst_of, const float* wgt, int top, float* x, int W, int T, cudaStream_t s, float beta = 1.f);

// ---- several residual streams joined by learned coefficients (hyper-connections), token shift (hybrid_streams.cu) ----
// xs [T, n, W] fp32 holds the n residual streams of every row (n = 1: a plain residual).
// x[t, s] = table[ids[t]] * scale for every stream s
cudaError_t hy_embed_streams(bool f32, const int32_t* ids, const void* table, float* xs, int T, int W, int vocab, float scale, int n, cudaStream_t s);
// One pass over the rows, each part optional:
//  (1) y != null: the sublayer that has just run closes, all streams at once from the old ones: x_t <- sum_s upd_mix[s * n + t] x_s + upd_out[t] y   (y [T, W] fp32)
//  (2) w != null: the next sublayer's input u = sum_s in[s] x_s, v = u / sqrt(mean(u^2) + eps) * w.  rows != null: row t of the output reads row
//      rows[t] of xs and of y (the rows whose logits are wanted); then (1) only enters u, the streams themselves stay, and no token shift follows.
//      shift_state == null: v goes to h[t] (activation type, pitch ldh).
//      shift_state != null (token shift follows): v goes to hn[t] (fp32 [T, W]); the CTA of a sequence's last row also moves the sequence's carried
//      row shift_state[slot] to prev[seq] and stores v in its place.  hy_token_shift then makes h[t] = v_t + (v_(t-1) - v_t) * mu, with v_(t-1) from
//      hn, from prev (first row of a step that continues a sequence) or zero (first token).
struct HyStreams { int n; const float* upd_mix; const float* upd_out; const float* in; };
cudaError_t hy_stream_norm(bool f32, const HyStreams& c, float* xs, const float* y, const int32_t* rows, const float* w, float eps, void* h, int ldh, float* hn, float* shift_state,
                           float* prev, const HyRows& r, int T, int W, cudaStream_t s);
cudaError_t hy_token_shift(bool f32, const float* hn, const float* prev, const float* mu, void* h, int ldh, const HyRows& r, int W, cudaStream_t s);
// out[t, :n] = in[t, :n] / sqrt(mean(in[t, :n]^2) + eps) * w — RMS norm of a projection's first n columns (fp32 arithmetic, activation type in and out)
cudaError_t hy_rmsnorm_act(bool f32, const void* in, int ld_in, int n, const float* w, void* out, int ld_out, float eps, int T, cudaStream_t s);
// x[t, c] *= sigmoid(g[t, c]) for c < n, in place (activation type)
cudaError_t hy_sigmoid_gate(bool f32, void* x, int ldx, const void* g, int ldg, int n, int T, cudaStream_t s);

cudaError_t hy_gather_rows_f32(const float* x, const int32_t* rows, float* out, int n, int W, cudaStream_t s);
// softcap > 0: logits <- softcap * tanh(logits / softcap), in place, before the arg-max (ties -> lowest id)
cudaError_t hy_argmax_rows(float* logits, int n, int V, float softcap, int32_t* out_ids, cudaStream_t s);
// x[t, :] += v[:]
cudaError_t hy_add_rowvec(float* x, const float* v, int T, int W, cudaStream_t s);

}  // namespace oa
