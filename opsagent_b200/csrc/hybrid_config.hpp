// hybrid_config.hpp — configuration of the hybrid decoder family: a stack of parallel-residual layers whose token mixer is one of latent
// attention (a compressed key/value cache), a gated delta rule with per-channel decay, a Mamba-2 state-space layer, or windowed attention
// over cached keys and values (sliding window with optional kept first tokens, one or two score maps per head, optional sink, output gate,
// optionally reading another layer's cache), each beside a routed mixture-of-experts feed-forward, with an optional looped block that
// re-injects the embedding.  Four designs are registered: "Ratasun" (one weight-only layer norm per layer, sigmoid group-limited router, SwiGLU
// experts), "Zurevik" (two RMS norms per layer, softmax over the chosen router logits, squared-ReLU experts, scaled embedding, soft-capped
// logits) and "Rofizen" (norm after the sum: x <- norm(alpha x + sublayer(x)), mixer and feed-forward in sequence; mixers: gated linear
// attention with a decay per key channel, retention with a fixed decay per head and rotate-half rotary, or causal soft-capped attention with
// a distance penalty beside an xLSTM matrix memory; feed-forward: dense squared-ReLU, or SwiGLU experts chosen by a table of token ids plus
// a gated shared expert).  "Gosavik": pre-norm sublayers in sequence (x += mixer(rms1(x)), x += ff(rms2(x))) over several residual streams
// joined by learned coefficients (hyper-connections), a token shift in front of every mixer, a looped block without re-injection; mixers:
// latent attention with a low-rank query, rotate-half rotary with YaRN-scaled frequencies, a sliding window, a sink and a per-channel output
// gate, or causal grouped-query attention with projection biases, short convolutions on q / k / v, interleaved rotary, rotated values
// and a sink; feed-forward: dense with the tanh form of GELU.
// Every size and constant is read from the checkpoint folder's config.json; nothing here is specific to one checkpoint.
#pragma once
#include <cstdio>
#include <fstream>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "json_dom.hpp"

namespace oa {

enum HyMixer : int { HY_LATENT_ATTENTION = 0, HY_CHANNEL_DELTA = 1, HY_MAMBA2 = 2, HY_WINDOW_ATTENTION = 3, HY_LINEAR_ATTENTION = 4, HY_ATTENTION_BESIDE_MEMORY = 5 };
enum HyNorm : int { HY_LAYER_NORM = 0, HY_RMS_NORM = 1 };
enum HyRouterKind : int { HY_ROUTER_SIGMOID_GROUPS = 0, HY_ROUTER_SOFTMAX_CHOSEN = 1, HY_ROUTER_TOKEN_TABLE = 2 };   // weights: sigmoid scores renormalised and scaled / softmax over the chosen logits / a table row per token id, 1 / top each
// linear-attention recurrences over an fp32 state S[dim, vdim] per head, o_t = S_t^T q_t:
//   channel decay: S_t = diag(a_t) S_(t-1) + k_t v_t^T, a_t = sigmoid(z_t)^(1 / tau) per key channel from a low-rank projection (gated linear attention)
//   head decay:    S_t = decay_h S_(t-1) + k_t v_t^T with a fixed decay per head, rotate-half rotary on q and k (retention)
//   matrix memory: S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k_t v_t^T with log gates i, f, a running maximum m and a normaliser n (xLSTM's mLSTM)
enum HyLinearKind : int { HY_LIN_CHANNEL_DECAY = 0, HY_LIN_HEAD_DECAY = 1, HY_LIN_MATRIX_MEMORY = 2 };
enum HyLinearNorm : int { HY_LIN_NORM_HEAD_WEIGHT = 0, HY_LIN_NORM_NONE = 1, HY_LIN_NORM_ALL_WEIGHT = 2 };   // weight of the per-head RMS norm: [vdim] shared by heads / none / [heads * vdim]

struct HyLinear {
    int kind = HY_LIN_CHANNEL_DECAY, heads = 0, dim = 0, vdim = 0;
    float tau = 1.f, gate_cap = 0.f, rot_base = 10000.f; int rot_dims = 0;
    std::vector<float> decay;             // head decay: one per head
    int norm = HY_LIN_NORM_HEAD_WEIGHT, gate_silu = 1;      // output gate: silu (1) or sigmoid (0) of a projection, per channel
    bool q_scaled = true, k_scaled = false;                  // dim^-1/2 on q, or on k (after the rotation)
};
enum HyExpertAct : int { HY_EXPERT_SWIGLU = 0, HY_EXPERT_RELU2 = 1, HY_EXPERT_GELU_TANH = 2 };     // down(silu(gate x) * up x) / down(relu(up x)^2) / down(gelu_tanh(up x))
enum HyRotLayout : int { HY_ROT_INTERLEAVED = 0, HY_ROT_HALVES = 1 };                         // channel 2i pairs with 2i + 1 / channel i with i + dims / 2
// YaRN: with where(t) = dims ln(original / (2 pi t)) / (2 ln base), lo = max(floor(where(fast)), 0), hi = min(ceil(where(slow)), dims - 1) and
// ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), frequency i is f_i / factor * ramp_i + f_i (1 - ramp_i); cos and sin carry the amplitude 0.1 ln(factor) + 1
struct HyRotScaling { bool on = false; float factor = 1.f, original = 0.f, fast = 0.f, slow = 0.f; };
enum HyGate : int { HY_GATE_NONE = 0, HY_GATE_CHANNEL = 1, HY_GATE_HEAD = 2 };

struct HyMoe {
    bool present = false;
    int experts = 0, top = 0, groups = 1, keep = 1, ff = 0;
    float scale = 1.f;
    int router = HY_ROUTER_SIGMOID_GROUPS, act = HY_EXPERT_SWIGLU;
    bool dense = false;                   // one feed-forward for every token (no router, no experts): down(act(up h)), width ff
    int shared_ff = 0;                    // > 0: a shared expert of this width runs for every token, times sigmoid(w_sg . h)
};

struct HyLayer {
    int type = HY_LATENT_ATTENTION;
    // latent attention: heads x (dim unrotated + rot_dim rotated) query/key, vdim values, kv_rank latent; rotary on the first rot_dims of the rotated part
    // channel delta:    heads value heads of vdim, kv_heads query/key heads of dim, conv taps
    // mamba2:           heads x vdim inner channels, state N, groups of B/C, norm_groups, conv taps
    int heads = 0, kv_heads = 0, dim = 0, rot_dim = 0, vdim = 0, kv_rank = 0, rot_dims = 0, conv = 0, state = 0, groups = 1, norm_groups = 1;
    float rot_base = 10000.f, scale = 1.f;
    // window attention: heads query heads on kv_heads key/value heads, `maps` score maps per head (2 = differential: q and k hold [map 1 | map 2] per
    // head, out = a1 - lambda a2, unit RMS per head, times 1 - diff); position i sees j <= i with i - j < window or j < keep_first; qk_norm: RMS
    // norm of every query / key map with a weight shared by heads and maps; bias: q/k/v projection biases; sink: a learned logit per head in
    // the softmax denominator only; gate: sigmoid output gate per channel or per head; kv_from >= 0: keys and values of that layer's cache
    // qk_norm = 2: one RMS norm over the whole q (and k) projection, before the split into heads, with a weight of that size.  softcap > 0:
    // score <- softcap tanh(score / softcap).  slope_exp > 0: head h's score loses 2^(-slope_exp (h + 1) / heads) per position of distance.
    // q_temp_every > 0: q at position p is multiplied by 1 + q_temp_coef ln(floor((p + 1) / q_temp_every) + 1).  out_bias: bias of the output projection
    int maps = 1, window = 0, keep_first = 0, qk_norm = 0, bias = 0, sink = 0, gate = HY_GATE_NONE, kv_from = -1;
    float diff = 0.f, softcap = 0.f, slope_exp = 0.f, q_temp_coef = 0.f; int q_temp_every = 0, out_bias = 0;
    // latent attention, optional parts: q_rank > 0: queries through a latent, q = W_uq rms_norm(W_dq h); rot_layout / rot_scaling: pairing and
    // YaRN scaling of the rotary; window > 0: position i sees j with 0 <= i - j < window; sink; gate = HY_GATE_CHANNEL: sigmoid(W_g h) per channel.
    // windowed attention, optional parts: conv > 0: a short causal convolution (no bias, no activation) on every channel of q, k and v, right
    // after the projection; rot_dims > 0: rotary on the first rot_dims channels of every query / key head; v_rot: the value of position j is
    // cached turned by j over all vdim channels (pair m by j rot_base^(-2m / vdim)), a head's output at position i is turned back by -i
    int q_rank = 0, rot_layout = HY_ROT_INTERLEAVED, v_rot = 0;
    HyRotScaling rot_scaling;
    HyLinear lin;                         // HY_LINEAR_ATTENTION, and the memory side of HY_ATTENTION_BESIDE_MEMORY (whose attention side uses the fields above)
    HyMoe moe;
};

struct HyRun { int layer = 0, pass = -1; bool first_of_pass = false; int cache_idx = -1, state_idx = -1; bool cache_owner = false; int index = 0; };   // one execution of a layer (a looped layer runs once per pass)

struct HybridConfig {
    std::string dir;                      // checkpoint folder (config.json [+ model.safetensors]; without the latter the weights are seeded)
    int width = 0, vocab = 0;
    float eps = 1e-6f, logit_scale = 1.f;
    std::string arch = "ratasun";        // registry key of the design
    int norm = HY_LAYER_NORM;             // the layers' (and the final) norm
    bool two_norms = false;               // mixer and feed-forward each read their own norm of the same residual
    float embed_scale = 1.f, logit_softcap = 0.f;      // x = embed[token] * scale; logits <- cap * tanh(logits / cap) (0: none)
    bool post_norm = false; float post_alpha = 1.f;    // norm after the sum: x <- norm1(alpha x + mixer(x)), x <- norm2(alpha x + ff(x)); the sublayers read x itself
    // sublayers in sequence, each on its own norm of the residual it finds: x <- x + mixer(norm1(x)), then x <- x + ff(norm2(x)).
    // streams > 0 (hyper-connections): the residual is `streams` copies x_1..x_s of the embedding; sublayer q reads u = sum_s in_q[s] x_s and
    // every stream becomes x_t <- sum_s mix_q[s, t] x_s + out_q[t] sublayer(norm(u)); after the last layer x = sum_s x_s.
    // token_shift: the mixer's input h_t (after the norm) is replaced by h_t + (h_(t-1) - h_t) * shift, h_(t-1) as it was before its own
    // replacement (zeros before the first token); every layer execution carries the last h of a sequence in its state slot.
    bool sequential = false, token_shift = false; int streams = 0;
    bool loop_reinject = true;                          // a looped block re-injects the embedding before every pass (x <- W_in [x ; x0] + step[pass])
    std::vector<HyLayer> layers;
    int loop_start = 0, loop_stop = 0, loop_times = 0;    // times == 0: no looped block
    std::vector<HyRun> runs;
    int n_caches = 0, n_states = 0;

    static double num(const Json& o, const char* k, const char* where) {
        const Json* j = o.get(k);
        if (!j || j->t != Json::Num) throw std::runtime_error(std::string("config.json: ") + where + " needs a number '" + k + "'");
        return j->n;
    }
    static int integer(const Json& o, const char* k, const char* where) { return (int)std::llround(num(o, k, where)); }
    static const Json& obj(const Json& o, const char* k, const char* where) {
        const Json* j = o.get(k);
        if (!j || j->t != Json::Obj) throw std::runtime_error(std::string("config.json: ") + where + " needs an object '" + k + "'");
        return *j;
    }

    static std::string read_file(const std::string& path) {
        std::ifstream f(path, std::ios::binary);
        if (!f) throw std::runtime_error("cannot read " + path);
        std::stringstream ss; ss << f.rdbuf(); return ss.str();
    }
    // the "architecture" key of <dir>/config.json (empty if there is none): the model registry dispatches on it
    static std::string architecture_of(const std::string& dir) {
        Json j; std::string err;
        if (!parse_json(read_file(dir + "/config.json"), j, err)) throw std::runtime_error("config.json: " + err);
        return j.str("architecture");
    }

    // the model registry of this family: config.json's "architecture" -> registry key ("" = not one of ours)
    static std::string registry_key(const std::string& architecture) {
        if (architecture == "Ratasun") return "ratasun";
        if (architecture == "Zurevik") return "zurevik";
        if (architecture == "Rofizen") return "rofizen";
        if (architecture == "Gosavik") return "gosavik";
        return "";
    }

    static HybridConfig load(const std::string& dir) {
        Json j; std::string err;
        if (!parse_json(read_file(dir + "/config.json"), j, err)) throw std::runtime_error("config.json: " + err);
        HybridConfig c; c.dir = dir;
        c.arch = registry_key(j.str("architecture"));
        if (c.arch.empty()) throw std::runtime_error("config.json: unknown architecture '" + j.str("architecture") + "'");
        const bool zu = c.arch == "zurevik", ro = c.arch == "rofizen", go = c.arch == "gosavik";
        if (go) {
            c.norm = HY_RMS_NORM; c.sequential = true; c.token_shift = true; c.loop_reinject = false;
            if (j.get("streams") && j.get("streams")->t == Json::Num) { c.streams = integer(j, "streams", "the model"); if (c.streams < 1 || c.streams > 8) throw std::runtime_error("config.json: streams must be 1 .. 8"); }
        }
        if (zu) { c.norm = HY_RMS_NORM; c.two_norms = true; }
        if (ro) { c.post_norm = true; c.post_alpha = (float)num(j, "postln_alpha", "the model"); }
        if (const Json* e = j.get("embedding")) if (e->t == Json::Obj && e->get("scale")) c.embed_scale = (float)num(*e, "scale", "embedding");
        if (j.get("logit_softcap") && j.get("logit_softcap")->t == Json::Num) c.logit_softcap = (float)num(j, "logit_softcap", "the model");
        c.width = integer(j, "width", "the model"); c.vocab = integer(j, "vocab", "the model");
        c.eps = (float)num(obj(j, "norm", "the model"), "eps", "norm");
        c.logit_scale = j.get("logit_scale") ? (float)num(j, "logit_scale", "the model") : 1.f;
        const Json* ls = j.get("layers");
        if (!ls || ls->t != Json::Arr || ls->a.empty()) throw std::runtime_error("config.json: 'layers' must be a non-empty list");
        for (const Json& lj : ls->a) {
            HyLayer l; const std::string type = lj.str("type");
            const Json& m = obj(lj, "mixer", "a layer");
            if (type == "latent_attention") {
                l.type = HY_LATENT_ATTENTION;
                l.heads = integer(m, "heads", type.c_str()); l.dim = integer(m, "dim", type.c_str()); l.rot_dim = integer(m, "rot_dim", type.c_str());
                l.vdim = integer(m, "vdim", type.c_str()); l.kv_rank = integer(m, "kv_rank", type.c_str()); l.scale = (float)num(m, "scale", type.c_str());
                const Json& r = obj(m, "rot", type.c_str());
                l.rot_base = (float)num(r, "base", "rot"); l.rot_dims = integer(r, "dims", "rot");
                if (l.rot_dims > l.rot_dim || (l.rot_dims & 1)) throw std::runtime_error("config.json: rot.dims must be even and <= rot_dim");
                if (go) {
                    l.q_rank = integer(m, "q_rank", type.c_str()); l.rot_layout = HY_ROT_HALVES; l.sink = 1; l.gate = HY_GATE_CHANNEL;
                    if (const Json* mk = m.get("mask")) if (mk->t == Json::Obj) { l.window = integer(*mk, "size", "mask"); if (l.window < 1) throw std::runtime_error("config.json: mask.size must be at least 1"); }
                    if (const Json* sc = r.get("scaling")) if (sc->t == Json::Obj) {
                        l.rot_scaling.on = true; l.rot_scaling.factor = (float)num(*sc, "factor", "scaling"); l.rot_scaling.original = (float)num(*sc, "original", "scaling");
                        l.rot_scaling.fast = (float)num(*sc, "fast", "scaling"); l.rot_scaling.slow = (float)num(*sc, "slow", "scaling");
                        if (!(l.rot_scaling.factor > 0.f) || !(l.rot_scaling.original > 0.f) || !(l.rot_scaling.fast > 0.f) || !(l.rot_scaling.slow > 0.f) || !(l.rot_base > 1.f))
                            throw std::runtime_error("config.json: bad rotary scaling");
                    }
                    if (l.q_rank <= 0 || l.dim < 0 || l.rot_dim < 0 || l.dim + l.rot_dim <= 0 || l.kv_rank <= 0 || l.kv_rank > 1024) throw std::runtime_error("config.json: bad latent attention sizes");
                }
            } else if (type == "channel_delta") {
                l.type = HY_CHANNEL_DELTA;
                l.heads = integer(m, "heads", type.c_str()); l.kv_heads = integer(m, "kv_heads", type.c_str()); l.dim = integer(m, "dim", type.c_str());
                l.vdim = integer(m, "vdim", type.c_str()); l.conv = integer(m, "conv", type.c_str());
                if (l.kv_heads <= 0 || l.heads % l.kv_heads) throw std::runtime_error("config.json: kv_heads must divide heads");
            } else if (type == "mamba2") {
                l.type = HY_MAMBA2;
                l.heads = integer(m, "heads", type.c_str()); l.vdim = integer(m, "vdim", type.c_str()); l.state = integer(m, "state", type.c_str());
                l.groups = integer(m, "groups", type.c_str()); l.norm_groups = integer(m, "norm_groups", type.c_str()); l.conv = integer(m, "conv", type.c_str());
                if (l.groups <= 0 || l.heads % l.groups || l.norm_groups <= 0 || (l.heads * l.vdim) % l.norm_groups) throw std::runtime_error("config.json: groups must divide heads, norm_groups the inner size");
            } else if (go && type == "attention") {
                // causal grouped-query attention: projection biases, short convolutions, interleaved rotary on queries and keys, rotated values, a sink per head
                l.type = HY_WINDOW_ATTENTION;
                l.heads = integer(m, "heads", type.c_str()); l.kv_heads = integer(m, "kv_heads", type.c_str()); l.dim = integer(m, "dim", type.c_str());
                l.vdim = integer(m, "vdim", type.c_str()); l.scale = (float)num(m, "scale", type.c_str()); l.conv = integer(m, "conv", type.c_str());
                const Json& r = obj(m, "rot", type.c_str());
                l.rot_base = (float)num(r, "base", "rot"); l.rot_dims = integer(r, "dims", "rot"); l.rot_layout = HY_ROT_INTERLEAVED;
                l.window = 1 << 30; l.bias = 1; l.out_bias = 1; l.sink = 1; l.v_rot = 1;
                if (const Json* mk = m.get("mask")) if (mk->t == Json::Obj) { l.window = integer(*mk, "size", "mask"); if (l.window < 1) throw std::runtime_error("config.json: mask.size must be at least 1"); }
                if (l.kv_heads <= 0 || l.heads % l.kv_heads || l.dim <= 0 || l.vdim > 256 || (l.vdim & 1) || l.dim > 1024 || l.rot_dims < 0 || l.rot_dims > l.dim || (l.rot_dims & 1) || l.conv < 1 || l.conv > 16 || !(l.rot_base > 0.f))
                    throw std::runtime_error("config.json: bad attention sizes");
            } else if (type == "attention" || type == "attention_2") {
                // "attention": differential (two score maps), query/key norm, kept first tokens, gate per channel;
                // "attention_2": one map, projection biases, a sink per head, gate per head, optionally another layer's keys and values
                const bool diff = type == "attention";
                l.type = HY_WINDOW_ATTENTION;
                l.heads = integer(m, "heads", type.c_str()); l.kv_heads = integer(m, "kv_heads", type.c_str()); l.dim = integer(m, "dim", type.c_str());
                l.vdim = integer(m, "vdim", type.c_str()); l.scale = (float)num(m, "scale", type.c_str());
                const Json& mk = obj(m, "mask", type.c_str());
                l.window = integer(mk, "size", "mask");
                if (mk.get("keep_first") && mk.get("keep_first")->t == Json::Num) l.keep_first = integer(mk, "keep_first", "mask");
                l.maps = diff ? 2 : 1; l.qk_norm = diff; l.bias = !diff; l.sink = !diff; l.gate = diff ? HY_GATE_CHANNEL : HY_GATE_HEAD;
                if (diff) l.diff = (float)num(m, "diff", type.c_str());
                if (!diff && m.get("kv_from") && m.get("kv_from")->t == Json::Num) {
                    l.kv_from = integer(m, "kv_from", type.c_str());
                    if (l.kv_from < 0 || l.kv_from >= (int)c.layers.size()) throw std::runtime_error("config.json: kv_from must name an earlier layer");
                    const HyLayer& src = c.layers[l.kv_from];
                    if (src.type != HY_WINDOW_ATTENTION || src.kv_from >= 0 || src.maps != l.maps || src.kv_heads != l.kv_heads || src.dim != l.dim || src.vdim != l.vdim)
                        throw std::runtime_error("config.json: kv_from must name a layer with keys and values of its own and of this layer's sizes");
                }
                if (l.kv_heads <= 0 || l.heads % l.kv_heads || l.dim <= 0 || l.window < 1 || l.keep_first < 0 || l.vdim > 256 || l.dim > 1024) throw std::runtime_error("config.json: bad attention sizes");
            } else if (ro && (type == "gla" || type == "retention")) {
                l.type = HY_LINEAR_ATTENTION; HyLinear& n = l.lin;
                n.heads = l.heads = integer(m, "heads", type.c_str()); n.dim = l.dim = integer(m, "dim", type.c_str()); n.vdim = l.vdim = integer(m, "vdim", type.c_str());
                if (type == "gla") { n.kind = HY_LIN_CHANNEL_DECAY; n.tau = (float)num(m, "tau", "gla"); n.norm = HY_LIN_NORM_HEAD_WEIGHT; if (!(n.tau > 0.f)) throw std::runtime_error("config.json: gla needs tau > 0"); }
                else {
                    n.kind = HY_LIN_HEAD_DECAY; n.norm = HY_LIN_NORM_NONE; n.q_scaled = false; n.k_scaled = true;
                    const Json* d = m.get("decay");
                    if (!d || d->t != Json::Arr || (int)d->a.size() != n.heads) throw std::runtime_error("config.json: retention needs a list 'decay' with one number per head");
                    for (const Json& x : d->a) { if (x.t != Json::Num) throw std::runtime_error("config.json: 'decay' holds numbers"); n.decay.push_back((float)x.n); }
                    const Json& r = obj(m, "rot", "retention");
                    n.rot_base = (float)num(r, "base", "rot"); n.rot_dims = integer(r, "dims", "rot");
                    if (n.rot_dims < 0 || n.rot_dims > n.dim || (n.rot_dims & 1)) throw std::runtime_error("config.json: rot.dims must be even and <= dim");
                }
                if (n.dim <= 0 || n.dim > 1024) throw std::runtime_error("config.json: bad linear-attention sizes");
            } else if (ro && type == "parallel") {
                // causal attention (left) beside a matrix memory (right), both reading the layer's input; the halves of their RMS-normed outputs are added
                l.type = HY_ATTENTION_BESIDE_MEMORY;
                const Json& a = obj(m, "left", "parallel"); const Json& b = obj(m, "right", "parallel");
                l.heads = integer(a, "heads", "left"); l.kv_heads = integer(a, "kv_heads", "left"); l.dim = integer(a, "dim", "left"); l.vdim = integer(a, "vdim", "left");
                l.scale = (float)num(a, "scale", "left"); l.slope_exp = 8.f;
                if (a.get("softcap") && a.get("softcap")->t == Json::Num) l.softcap = (float)num(a, "softcap", "left");          // absent or 0: scores are not capped
                if (const Json* qt = a.get("q_temp")) if (qt->t == Json::Obj) { l.q_temp_coef = (float)num(*qt, "coef", "q_temp"); l.q_temp_every = integer(*qt, "every", "q_temp"); if (l.q_temp_every < 1) throw std::runtime_error("config.json: q_temp.every must be at least 1"); }
                l.window = 1 << 30; l.qk_norm = 2; l.bias = 1; l.out_bias = 1;
                if (l.kv_heads <= 0 || l.heads % l.kv_heads || l.dim <= 0 || l.vdim > 256 || l.dim > 1024 || l.softcap < 0.f) throw std::runtime_error("config.json: bad attention sizes");
                HyLinear& n = l.lin;
                n.kind = HY_LIN_MATRIX_MEMORY; n.heads = integer(b, "heads", "right"); n.dim = integer(b, "dim", "right"); n.vdim = integer(b, "vdim", "right");
                n.gate_cap = (float)num(b, "gate_cap", "right"); n.norm = HY_LIN_NORM_ALL_WEIGHT; n.gate_silu = 0;
                if (n.heads <= 0 || n.dim <= 0 || n.dim > 1024 || n.vdim <= 0 || !(n.gate_cap > 0.f)) throw std::runtime_error("config.json: bad matrix-memory sizes");
            } else throw std::runtime_error("config.json: unknown layer type '" + type + "'");
            const bool recurrent = l.type == HY_CHANNEL_DELTA || l.type == HY_MAMBA2;
            if (l.heads <= 0 || l.vdim <= 0 || (recurrent && (l.conv < 1 || l.conv > 16))) throw std::runtime_error("config.json: bad mixer sizes");
            const Json* mj = lj.get("mlp");
            if (mj && mj->t == Json::Obj && (ro || go) && mj->str("kind") == "dense") {
                l.moe.present = true; l.moe.dense = true; l.moe.act = go ? HY_EXPERT_GELU_TANH : HY_EXPERT_RELU2; l.moe.experts = 1; l.moe.top = 1;
                l.moe.ff = integer(*mj, "ff", "mlp");
                if (l.moe.ff <= 0) throw std::runtime_error("config.json: bad feed-forward width");
            } else if (mj && mj->t == Json::Obj) {
                if (go || mj->str("kind") != "moe") throw std::runtime_error("config.json: unknown mlp kind '" + mj->str("kind") + "'");
                const Json& r = obj(*mj, "router", "mlp");
                l.moe.present = true; l.moe.ff = integer(obj(*mj, "expert", "mlp"), "ff", "expert");
                l.moe.experts = integer(r, "experts", "router"); l.moe.top = integer(r, "top", "router");
                if (zu) { l.moe.router = HY_ROUTER_SOFTMAX_CHOSEN; l.moe.act = HY_EXPERT_RELU2; }
                else if (ro) {
                    l.moe.router = HY_ROUTER_TOKEN_TABLE;
                    if (const Json* sh = mj->get("shared")) if (sh->t == Json::Obj) { l.moe.shared_ff = integer(*sh, "ff", "shared"); if (l.moe.shared_ff <= 0) throw std::runtime_error("config.json: bad shared expert width"); }
                    if (l.moe.ff <= 0) throw std::runtime_error("config.json: bad expert width");
                }
                else l.moe.scale = (float)num(r, "scale", "router");
                if (const Json* g = r.get("groups")) if (g->t == Json::Obj) { l.moe.groups = integer(*g, "count", "groups"); l.moe.keep = integer(*g, "keep", "groups"); }
                if (l.moe.groups <= 0 || l.moe.experts % l.moe.groups || l.moe.keep <= 0 || l.moe.keep > l.moe.groups || l.moe.top <= 0 ||
                    l.moe.top > l.moe.keep * (l.moe.experts / l.moe.groups) || l.moe.top > 31 + (l.moe.shared_ff ? 0 : 1) || l.moe.experts > 1024)
                    throw std::runtime_error("config.json: bad router sizes");
            }
            c.layers.push_back(l);
        }
        const Json* lp = j.get("loop");
        if (lp && lp->t == Json::Obj) {
            c.loop_start = integer(*lp, "start", "loop"); c.loop_stop = integer(*lp, "stop", "loop"); c.loop_times = integer(*lp, "times", "loop");
            if (c.loop_start < 0 || c.loop_stop <= c.loop_start || c.loop_stop > (int)c.layers.size() || c.loop_times < 1) throw std::runtime_error("config.json: bad loop");
        }
        // expand the schedule of layer executions: each execution owns its cache (attention) or state (recurrent mixers)
        auto add = [&](int layer, int pass, bool first) {
            HyRun r; r.layer = layer; r.pass = pass; r.first_of_pass = first;
            const HyLayer& l = c.layers[layer];
            if (l.type == HY_WINDOW_ATTENTION && l.kv_from >= 0) {          // the cache of the (only) execution of the layer it reads
                for (const HyRun& o : c.runs) if (o.layer == l.kv_from) r.cache_idx = o.cache_idx;
                if (r.cache_idx < 0 || (c.loop_times > 0 && layer >= c.loop_start && layer < c.loop_stop) || (c.loop_times > 0 && l.kv_from >= c.loop_start && l.kv_from < c.loop_stop))
                    throw std::runtime_error("config.json: a layer that reads another layer's cache cannot be part of a looped block");
            } else if (l.type == HY_LATENT_ATTENTION || l.type == HY_WINDOW_ATTENTION) {
                r.cache_idx = c.n_caches++; r.cache_owner = true;
                if (l.type == HY_WINDOW_ATTENTION && l.conv > 1) r.state_idx = c.n_states++;        // the convolutions' tails
            }
            else if (l.type == HY_ATTENTION_BESIDE_MEMORY) { r.cache_idx = c.n_caches++; r.cache_owner = true; r.state_idx = c.n_states++; }     // a cache for the attention side, a state for the memory side
            else r.state_idx = c.n_states++;
            r.index = (int)c.runs.size();
            c.runs.push_back(r);
        };
        for (int i = 0; i < (int)c.layers.size();) {
            if (c.loop_times > 0 && i == c.loop_start) {
                for (int t = 0; t < c.loop_times; ++t) for (int k = c.loop_start; k < c.loop_stop; ++k) add(k, t, k == c.loop_start);
                i = c.loop_stop;
            } else { add(i, -1, false); ++i; }
        }
        if (c.width <= 0 || c.vocab <= 0) throw std::runtime_error("config.json: bad width / vocab");
        return c;
    }
};

}  // namespace oa
