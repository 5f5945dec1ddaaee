// hybrid_model.hpp — device-resident model of the hybrid decoder family (configuration: hybrid_config.hpp, kernels: hybrid_kernels.hpp).
// It plugs into the same scheduler as the Llama-family DeviceModel: rows of a step arrive as a StepInput (prefill chunks and single decode
// tokens alike), attention layers keep their compressed keys (latent attention) or their keys and values (windowed attention) in the engine's
// 64-token pages, recurrent layers keep an fp32 state and their convolution tails (or, for a matrix memory, its normaliser and running
// maximum) in the sequence's state slot.  Designs whose norm follows the sum (x <- norm(alpha x + sublayer(x))) run mixer and feed-forward in
// sequence; pre-norm designs run them either side by side on norms of the same residual or in sequence, the latter optionally on several
// residual streams (hyper-connections) and with a token shift in front of the mixer whose carried row lives in the state slot too.
#pragma once
#include <functional>
#include <string>
#include <vector>

#include "hybrid_config.hpp"
#include "hybrid_kernels.hpp"
#include "model.hpp"

namespace oa {

class HybridModel : public ModelBase {
public:
    HybridModel(const ModelConfig& cfg, const EngineOptions& opt);
    ~HybridModel() override;
    void forward(const StepInput& in, float* logits_out) override;
    const char* kt_name(int id) const override;
    // debug: copy of the residual stream after every layer execution of the NEXT forward ([runs, T, width] fp32, host); empty = off
    std::vector<float>* capture_layers = nullptr;

private:
    struct Mat {                    // [N, ld] matrix in the activation type, ld = K rounded up to 8 (zero padded); B operand of C = A . B^T
        void* p = nullptr; int N = 0, K = 0, ld = 0;
        bool tc = false; CUtensorMap tm[4];           // tensor-core path (bf16): B-operand maps for BLOCK_N = 32, 64, 128, 256
    };
    struct HostMat { int N = 0, K = 0; std::vector<float> v; };
    struct LayerW {
        float *norm1 = nullptr, *norm2 = nullptr;      // norm2: the feed-forward's own norm (designs with two norms per layer)
        Mat in, a2, g2, o, router, kv_up;
        float* in_bias = nullptr; void* in_bias_act = nullptr;      // bias of the fused input projection (fp32, and in the activation type for the tensor-core epilogue)
        float *q_norm = nullptr, *k_norm = nullptr, *sink = nullptr, lambda = 0.f;     // windowed attention
        float* router_bias = nullptr;
        int off_a = 0, off_b = 0, off_c = 0, off_d = 0;   // column offsets of the fused input projection's segments (see hybrid_model.cpp)
        int a_rank = 0, g_rank = 0;
        void *uk_t = nullptr, *uv = nullptr; float* dkv_norm = nullptr; int rope = -1;      // latent attention
        std::vector<Mat> uk_heads, uv_heads;          // per-head views of uk_t / uv with tensor maps (prefill-sized steps run them on the tensor cores)
        float *A_log = nullptr, *dt_bias = nullptr, *norm_w = nullptr, *conv_w = nullptr, *conv_b = nullptr, *D = nullptr;
        int conv_ch = 0;
        float* correction = nullptr; void *gu = nullptr, *down = nullptr; int ffp = 0;       // experts: gu [E][2 ffp][ldw], down [E][W][ffp]
        CUtensorMap tm_gu[2], tm_down[2]; bool moe_tc = false;                               // grouped tensor-core path: BLOCK_N = 128, 256
        int n_exp = 0, n_top = 0, ff_max = 0;         // experts and choices per token as the kernels see them (a shared expert is one more expert that every token chooses)
        int32_t* table = nullptr; void* shared_gate = nullptr;                               // router by token id; gate row of the shared expert
        Mat up, dn;                                   // dense feed-forward
        // designs with sublayers in sequence: token shift weight, hyper-connection coefficients of the mixer (1) and the feed-forward (2), all fp32 on the device
        float *shift = nullptr, *hc_in[2] = {nullptr, nullptr}, *hc_mix[2] = {nullptr, nullptr}, *hc_out[2] = {nullptr, nullptr}, *o_bias = nullptr;
        Mat uq; float* dq_norm = nullptr; int rope_v = -1;      // latent attention with a low-rank query; rotary table of rotated values
        // linear attention and attention beside a matrix memory: segments of the fused input projection, second stage and biases
        int off_q = 0, off_k = 0, off_v = 0, off_g = 0, off_a1 = 0, off_lq = 0, off_lk = 0, off_lv = 0;
        float *a2_bias = nullptr, *decay = nullptr, *o2_bias = nullptr, *out_w1 = nullptr, *out_w2 = nullptr, *gates_bias = nullptr;
        Mat o2, gates;                                // output projection of the attention side; [W_i ; W_f] of the matrix memory (fp32 out)
    };
    struct RopeTable { float base; int dims; HyRotScaling sc; float *cos = nullptr, *sin = nullptr; };
    // per-step plan of one attention layer: offsets (in words) of its tile lists in the step's metadata arena
    struct TileList { bool mma = false, any_small = false; size_t o_seq = 0, o_q0 = 0, o_k0 = 0, o_k1 = 0, o_slot = 0, o_mrow = 0, o_mslot = 0, o_mparts = 0; int n = 0, n_merge = 0;
                      size_t o_pseq = 0, o_phead = 0, o_prow0 = 0, o_base = 0; int n_ptiles = 0, ctx_rows = 0, max_ctx = 0;
                      size_t o_wseq = 0, o_wq0 = 0, o_dseq = 0, o_dq0 = 0; int n_w = 0, n_d = 0; };

    void* dmalloc(size_t bytes);
    float* upload_f32(const std::vector<float>& v);
    void* upload_act(const std::vector<float>& v);                        // in the activation type
    Mat upload_mat(const HostMat& m);
    HostMat tensor(const std::string& name, int N, int K);                // checkpoint tensor (or seeded values) as fp32 [N, K]; K == 0: any width
    std::vector<float> vec(const std::string& name, int n, float init_mean, float init_spread);
    void gemm(int mode, const void* A, int lda, const Mat& B, void* C, int ldc, int M, const float* bias, float alpha, const void* bias_act = nullptr, int act = 0);
    // routed experts (and a dense feed-forward): x = beta x + sum of the chosen experts' outputs
    void moe(const LayerW& w, const HyLayer& l, const void* h, const HyRows& r, const std::function<void(int)>& mark, const int32_t* tokens = nullptr, float beta = 1.f);
    int rope_table(float base, int dims, const HyRotScaling* sc = nullptr);
    // latent attention of one layer execution: q [T, ldq] (head by head [dim | rot_dim]) and the down projection ckv [T, ldc] -> heads' outputs in mix_
    void latent_mixer(const HyRun& run, const HyLayer& l, const LayerW& w, const HyRows& r, const TileList& tl, const std::function<void(int)>& mark, void* q, int ldq, void* ckv, int ldc,
                      const void* gate = nullptr, int ldg = 0);          // gate: sigmoid output gate per channel of the concatenated heads
    // attention over cached keys and values: q / k / v [T, ld] -> heads' outputs in mix_ (gate: null or [T, ldg])
    void window_mixer(const HyRun& run, const HyLayer& l, const LayerW& w, const HyRows& r, const TileList& tl, const std::function<void(int)>& mark, void* q, void* k, void* v, int ld,
                      const void* gate, int ldg, bool prepared = false);      // prepared: queries are rotated and the cache row is written already
    void forward_sequential(const HyRows& r, const std::vector<TileList>& tile_lists, const int32_t* d_tokens, const std::function<void(int)>& mark);
    HyLatentAttn latent_params(const HyLayer& l, const LayerW& w) const;
    void linear_mixer(const HyRun& run, const HyLayer& l, const LayerW& w, const HyRows& r, const std::function<void(int)>& mark);
    bool has_tensor(const std::string& name) const;
    int cache_row_width(const HyLayer& l) const { return (l.type == HY_WINDOW_ATTENTION || l.type == HY_ATTENTION_BESIDE_MEMORY) ? l.kv_heads * (l.maps * l.dim + l.vdim) : l.kv_rank + l.rot_dim; }

    HybridConfig hc_; bool f32_ = false; size_t es_ = 2;
    struct SafeTensorsHolder; SafeTensorsHolder* st_ = nullptr;
    std::vector<void*> allocs_;
    std::vector<LayerW> lw_; std::vector<RopeTable> ropes_;
    void* embed_ = nullptr; Mat head_, loop_in_; float *loop_step_ = nullptr, *final_norm_ = nullptr;
    std::vector<void*> caches_;                    // per attention execution: [num_pages * 64][kv_rank + rot_dim] in the activation type
    std::vector<float*> states_; std::vector<void*> tails_;      // per recurrent execution: [slots][heads * dim * vdim] fp32, [slots][(taps - 1) * channels]
    std::vector<float*> shift_states_;             // per layer execution of a design with a token shift: [slots][width] fp32, the last normed row of the sequence
    const float *pend_mix_ = nullptr, *pend_out_ = nullptr; bool pending_ = false;      // the last sublayer's y_ is folded into the streams by whoever reads them next
    float *xs_ = nullptr, *hn_ = nullptr, *shift_prev_ = nullptr, *ones_ = nullptr; void* cq_ = nullptr; int ld_cq_ = 0, n_streams_ = 1;      // residual streams [T, n, W]; normed rows before the shift; carried rows of the step's sequences
    std::vector<float*> aux_;                      // per matrix-memory execution: [slots][heads * dim] normaliser, then [slots][heads] running maximum
    int MR_ = 0, MS_ = 0, Wld_ = 0;
    // activations
    float *x_ = nullptr, *x0_ = nullptr, *q_abs_ = nullptr, *qq_ = nullptr, *kk_ = nullptr, *vv_ = nullptr, *dec_ = nullptr, *beta_ = nullptr, *rec_ = nullptr, *wgt_ = nullptr,
          *logits_ = nullptr, *moe_y_ = nullptr, *rlog_ = nullptr;
    void *cat_ = nullptr, *h_ = nullptr, *h2_ = nullptr, *proj_ = nullptr, *p2_ = nullptr, *conv_ = nullptr, *lat_ = nullptr, *mix_ = nullptr, *act_ = nullptr, *hs_ = nullptr, *moe_a_ = nullptr;
    int ld_proj_ = 0, ld_p2_ = 0, ld_conv_ = 0, ld_mix_ = 0, ld_mix2_ = 0, ld_gates_ = 0;
    float *y_ = nullptr, *y2_ = nullptr, *gates_ = nullptr, *gin_ = nullptr, *floor_ = nullptr, *ndot_ = nullptr;     // post-norm designs: sublayer outputs; matrix memory: gates and normaliser terms
    void* mix2_ = nullptr;                         // attention side of a layer with two mixers
    int32_t *idx_ = nullptr, *d_out_ids_ = nullptr, *tile_expert_ = nullptr, *row_src_ = nullptr, *n_tiles_ = nullptr, *dst_of_ = nullptr; int max_tiles_ = 0;
    int32_t* h_meta_buf_[2] = {nullptr, nullptr}; cudaEvent_t meta_ev_[2] = {nullptr, nullptr}; int meta_idx_ = 0;
    int32_t* d_meta_ = nullptr; size_t meta_cap_words_ = 0;
    std::vector<int32_t> row_seq_, seq_pos0_, tile_seq_, tile_q0_, tile_k0_, tile_k1_, tile_slot_, merge_row_, merge_slot_, merge_parts_;
    std::vector<int32_t> ptile_seq_, ptile_head_, ptile_row0_, seq_base_;
    void *lat_ctx_ = nullptr, *kv_ctx_ = nullptr; int ld_kv_ = 0, ctx_cap_ = 0;    // prefill form of attention: gathered cache rows of whole contexts and their keys / values
    float *split_o_ = nullptr, *split_ml_ = nullptr; int split_slots_ = 0;       // partials of decoding rows whose cache rows are cut into parts
};

}  // namespace oa
