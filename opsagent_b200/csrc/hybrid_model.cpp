// hybrid_model.cpp — see hybrid_model.hpp.
#include "hybrid_model.hpp"

#include <sys/stat.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <stdexcept>

#include "common.cuh"
#include "safetensors.hpp"

namespace oa {

struct HybridModel::SafeTensorsHolder { SafeTensors st; explicit SafeTensorsHolder(const std::string& p) : st(p) {} };

static int up8(int n) { return (n + 7) & ~7; }
static int up16(int n) { return (n + 15) & ~15; }

struct HyDeviceGuard {
    int prev = -1;
    explicit HyDeviceGuard(int dev) { cudaGetDevice(&prev); cudaSetDevice(dev); }
    ~HyDeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

void* HybridModel::dmalloc(size_t bytes) {
    void* p = nullptr;
    cuda_check(cudaMalloc(&p, bytes ? bytes : 16), "cudaMalloc");
    cuda_check(cudaMemset(p, 0, bytes ? bytes : 16), "cudaMemset");
    allocs_.push_back(p);
    return p;
}
float* HybridModel::upload_f32(const std::vector<float>& v) {
    float* d = reinterpret_cast<float*>(dmalloc(v.size() * 4));
    cuda_check(cudaMemcpy(d, v.data(), v.size() * 4, cudaMemcpyHostToDevice), "H2D");
    return d;
}
void* HybridModel::upload_act(const std::vector<float>& v) {
    weight_bytes += v.size() * es_;
    if (f32_) return upload_f32(v);
    std::vector<uint16_t> b(v.size());
    for (size_t i = 0; i < v.size(); ++i) b[i] = f32_to_bf16_bits(v[i]);
    void* d = dmalloc(b.size() * 2);
    cuda_check(cudaMemcpy(d, b.data(), b.size() * 2, cudaMemcpyHostToDevice), "H2D");
    return d;
}
HybridModel::Mat HybridModel::upload_mat(const HostMat& m) {
    Mat d; d.N = m.N; d.K = m.K; d.ld = up8(m.K);
    std::vector<float> padded((size_t)up8(m.N) * d.ld, 0.f);          // rows padded too: a tensor-core tile may read past N
    for (int r = 0; r < m.N; ++r) std::memcpy(&padded[(size_t)r * d.ld], &m.v[(size_t)r * m.K], (size_t)m.K * 4);
    d.p = upload_act(padded);
    if (!f32_ && opt.hy_tensor_core) {
        const int bns[4] = {32, 64, 128, 256}; d.tc = true;
        for (int i = 0; i < 4; ++i)
            if (make_tmap_bf16_2d(&d.tm[i], d.p, (uint64_t)up8(m.N), (uint64_t)d.ld, (uint64_t)d.ld, (uint32_t)bns[i], 64) != 0) d.tc = false;
    }
    return d;
}

static uint64_t name_hash(const std::string& s, uint64_t seed) {
    uint64_t h = 0xcbf29ce484222325ull ^ seed;
    for (unsigned char c : s) { h ^= c; h *= 0x100000001b3ull; }
    return h;
}
static float unit_rand(uint64_t& st) {        // uniform in [-1, 1)
    st += 0x9E3779B97F4A7C15ull; uint64_t z = st; z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull; z = (z ^ (z >> 27)) * 0x94D049BB133111EBull; z ^= z >> 31;
    return (float)((double)(z >> 11) * (1.0 / 9007199254740992.0) * 2.0 - 1.0);
}
static float bf16_round(float f) { const uint32_t u = (uint32_t)f32_to_bf16_bits(f) << 16; float o; std::memcpy(&o, &u, 4); return o; }

static void st_to_f32(const StTensor& t, std::vector<float>& out) {
    size_t n = 1; for (int64_t d : t.shape) n *= (size_t)d;
    out.resize(n);
    if (t.dtype == "BF16") { const uint16_t* s = reinterpret_cast<const uint16_t*>(t.data); for (size_t i = 0; i < n; ++i) { const uint32_t u = (uint32_t)s[i] << 16; std::memcpy(&out[i], &u, 4); } }
    else if (t.dtype == "F32") std::memcpy(out.data(), t.data, n * 4);
    else throw std::runtime_error("checkpoint dtype " + t.dtype + " is not supported for this model family (BF16 or F32)");
}

HybridModel::HostMat HybridModel::tensor(const std::string& name, int N, int K) {
    HostMat m; m.N = N; m.K = K;
    if (st_) {
        const StTensor& t = st_->st.get(name);
        const bool ok = t.shape.size() == 2 && t.shape[0] == N && (K == 0 || t.shape[1] == K);
        if (!ok) throw std::runtime_error("checkpoint tensor " + name + " does not have the shape the configuration implies");
        m.K = (int)t.shape[1];
        st_to_f32(t, m.v);
    } else {
        if (K == 0) m.K = K = std::max(8, hc_.width / 16);     // low-rank width of a seeded model
        uint64_t s = name_hash(name, cfg.seed);
        const float a = std::sqrt(3.0f / (float)K);
        m.v.resize((size_t)N * K);
        for (auto& x : m.v) x = bf16_round(a * unit_rand(s));
    }
    return m;
}
std::vector<float> HybridModel::vec(const std::string& name, int n, float init_mean, float init_spread) {
    std::vector<float> v;
    if (st_) {
        const StTensor& t = st_->st.get(name);
        size_t have = 1; for (int64_t d : t.shape) have *= (size_t)d;
        if ((int)have != n) throw std::runtime_error("checkpoint tensor " + name + " does not have the size the configuration implies");
        st_to_f32(t, v);
    } else {
        uint64_t s = name_hash(name, cfg.seed); v.resize(n);
        for (auto& x : v) x = bf16_round(init_mean + init_spread * unit_rand(s));
    }
    return v;
}
bool HybridModel::has_tensor(const std::string& name) const { return st_ && st_->st.has(name); }
// cos / sin of position * f_i, f_i = base^(-2 i / dims), angles in double, [max_seq_len, dims / 2].  With YaRN scaling (sc) the frequency is a
// blend of f_i and f_i / factor along a ramp over i, and both tables carry the amplitude 0.1 ln(factor) + 1.
int HybridModel::rope_table(float base, int dims, const HyRotScaling* sc) {
    const HyRotScaling none; const HyRotScaling& k = sc ? *sc : none;
    for (size_t i = 0; i < ropes_.size(); ++i) {
        const RopeTable& t = ropes_[i];
        if (t.base == base && t.dims == dims && t.sc.on == k.on && (!k.on || (t.sc.factor == k.factor && t.sc.original == k.original && t.sc.fast == k.fast && t.sc.slow == k.slow))) return (int)i;
    }
    RopeTable rt; rt.base = base; rt.dims = dims; rt.sc = k; const int half = dims / 2;
    std::vector<float> cs((size_t)opt.max_seq_len * std::max(1, half)), sn(cs.size());
    double amp = 1.0, lo = 0.0, hi = 0.0;
    if (k.on) {
        const double pi = 3.14159265358979323846;
        auto where = [&](double turns) { return dims * std::log((double)k.original / (2.0 * pi * turns)) / (2.0 * std::log((double)base)); };
        lo = std::max(std::floor(where(k.fast)), 0.0); hi = std::min(std::ceil(where(k.slow)), (double)(dims - 1));
        amp = 0.1 * std::log((double)k.factor) + 1.0;
    }
    for (int i = 0; i < half; ++i) {
        double f = std::pow((double)base, -2.0 * i / (double)dims);
        if (k.on) { const double ramp = std::min(1.0, std::max(0.0, (i - lo) / std::max(hi - lo, 0.001))); f = f / k.factor * ramp + f * (1.0 - ramp); }
        for (int ps = 0; ps < opt.max_seq_len; ++ps) { cs[(size_t)ps * half + i] = (float)(std::cos(ps * f) * amp); sn[(size_t)ps * half + i] = (float)(std::sin(ps * f) * amp); }
    }
    rt.cos = upload_f32(cs); rt.sin = upload_f32(sn); ropes_.push_back(rt);
    return (int)ropes_.size() - 1;
}
static void append_rows(std::vector<float>& dst, int& rows, int K, const std::vector<float>& src, int src_rows, int align) {
    while (rows % align) { dst.resize(dst.size() + K, 0.f); ++rows; }
    dst.insert(dst.end(), src.begin(), src.end()); rows += src_rows;
}

HybridModel::HybridModel(const ModelConfig& c, const EngineOptions& o) : ModelBase(c, o), hc_(*c.hybrid) {
    HyDeviceGuard guard(opt.device);
    cuda_check(cudaSetDevice(opt.device), "cudaSetDevice");
    cudaDeviceProp prop;
    cuda_check(cudaGetDeviceProperties(&prop, opt.device), "cudaGetDeviceProperties");
    if (prop.major != 10) throw std::runtime_error("opsagent_b200 requires an sm_100 (Blackwell B200) device");
    if (opt.tp != 1) throw std::runtime_error("the hybrid model family runs on one GPU per engine (tp = 1)");
    sm_count = prop.multiProcessorCount;
    cuda_check(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking), "cudaStreamCreate");
    f32_ = opt.f32 != 0; es_ = f32_ ? 4 : 2;
    const int W = hc_.width, V = hc_.vocab; Wld_ = up8(W);
    {
        struct stat sb; const std::string f = hc_.dir + "/model.safetensors";
        if (stat(f.c_str(), &sb) == 0) st_ = new SafeTensorsHolder(f);
    }
    // ---- weights ----
    embed_ = upload_act(tensor("embed", V, W).v);
    head_ = upload_mat(tensor("head", V, W));
    final_norm_ = upload_f32(vec("final.norm", W, 1.f, 0.1f));
    if (hc_.loop_times > 0 && hc_.loop_reinject) { loop_in_ = upload_mat(tensor("loop.in", W, 2 * W)); loop_step_ = upload_f32(vec("loop.step", hc_.loop_times * W, 0.f, 0.1f)); }
    lw_.resize(hc_.layers.size());
    int max_in = 8, max_p2 = 8, max_conv = 8, max_mix = 8, max_qabs = 8, max_lat = 8, max_qk = 8, max_v = 8, max_dec = 8, max_h = 8, max_act = 8, max_top = 1, max_E = 1, max_ffp = 16, max_lat_heads = 1, max_kv = 0, max_Eattn = 8, max_mix2 = 0, max_gates = 0, max_cq = 0;
    for (size_t li = 0; li < hc_.layers.size(); ++li) {
        const HyLayer& l = hc_.layers[li]; LayerW& w = lw_[li];
        const std::string p = "l" + std::to_string(li) + ".", mx = p + "mix.";
        w.norm1 = upload_f32(vec(p + "norm1", W, 1.f, 0.1f));
        if ((hc_.two_norms || hc_.post_norm || hc_.sequential) && (l.moe.present || (hc_.post_norm && has_tensor(p + "norm2")))) w.norm2 = upload_f32(vec(p + "norm2", W, 1.f, 0.1f));
        if (hc_.token_shift && (!st_ || has_tensor(p + "shift"))) w.shift = upload_f32(vec(p + "shift", W, 0.5f, 0.5f));
        if (hc_.sequential && hc_.streams > 0) {
            const int n = hc_.streams;
            for (int q = 0; q < (l.moe.present ? 2 : 1); ++q) {
                const std::string hp = p + (q ? "hc2." : "hc1.");
                std::vector<float> mixv = vec(hp + "mix", n * n, 0.f, 0.1f);
                if (!st_) for (int i = 0; i < n; ++i) mixv[(size_t)i * n + i] += 1.f;          // seeded: near the identity
                w.hc_in[q] = upload_f32(vec(hp + "in", n, 1.f / (float)n, 0.1f / (float)n)); w.hc_mix[q] = upload_f32(mixv); w.hc_out[q] = upload_f32(vec(hp + "out", n, 1.f, 0.1f));
            }
        }
        HostMat in; in.K = W; int rows = 0;
        if (l.type == HY_WINDOW_ATTENTION) {
            // fused input projection [q | k | v | gate] (k, v only where the layer fills a cache of its own), each segment on a multiple of 8 rows
            const int qd = l.heads * l.maps * l.dim, kd = l.kv_heads * l.maps * l.dim, vd = l.kv_heads * l.vdim;
            const int gd = l.gate == HY_GATE_CHANNEL ? l.heads * l.vdim : l.gate == HY_GATE_HEAD ? l.heads : 0;
            if (!hy_win_supported(HyWinAttn{l.heads, l.kv_heads, l.dim, l.vdim, l.maps, l.window, l.keep_first, l.qk_norm, l.gate, l.scale, 0.f, 1.f}))
                throw std::runtime_error("config.json: attention sizes beyond what the kernels hold (vdim <= 256)");
            std::vector<float> bias;
            auto seg = [&](const char* nm, int n, bool biased) -> int {
                while (rows % 8) { in.v.resize(in.v.size() + W, 0.f); ++rows; }
                const int off = rows;
                append_rows(in.v, rows, W, tensor(mx + nm, n, W).v, n, 1);
                if (l.bias) { bias.resize(off, 0.f); std::vector<float> b = biased ? vec(mx + nm + ".b", n, 0.f, 0.2f) : std::vector<float>(n, 0.f); bias.insert(bias.end(), b.begin(), b.end()); }
                return off;
            };
            w.off_a = seg("q", qd, true);
            if (l.kv_from < 0) { w.off_b = seg("k", kd, true); w.off_c = seg("v", vd, true); }
            if (gd) w.off_d = seg("g", gd, false);
            if (l.bias) { bias.resize(up8(rows), 0.f); w.in_bias = upload_f32(bias); w.in_bias_act = upload_act(bias); }
            if (l.qk_norm) { w.q_norm = upload_f32(vec(mx + "q.norm", l.dim, 1.f, 0.1f)); w.k_norm = upload_f32(vec(mx + "k.norm", l.dim, 1.f, 0.1f)); }
            if (l.sink) w.sink = upload_f32(vec(mx + "sink", l.heads, 0.f, 1.f));
            if (l.out_bias) w.o_bias = upload_f32(vec(mx + "o.b", W, 0.f, 0.1f));
            if (l.conv > 0) {          // short convolutions on q | k | v: one weight table over the fused projection's columns (padding columns: zero taps)
                w.conv_ch = up8(rows);
                std::vector<float> cw((size_t)w.conv_ch * l.conv, 0.f);
                auto put_conv = [&](const char* nm, int n, int off) { std::vector<float> c = vec(mx + nm + ".conv", n * l.conv, 0.f, 0.5f); std::memcpy(&cw[(size_t)off * l.conv], c.data(), c.size() * 4); };
                put_conv("q", qd, w.off_a); put_conv("k", kd, w.off_b); put_conv("v", vd, w.off_c);
                w.conv_w = upload_f32(cw); max_conv = std::max(max_conv, w.conv_ch);
            }
            if (l.rot_dims > 0) w.rope = rope_table(l.rot_base, l.rot_dims);
            if (l.v_rot) w.rope_v = rope_table(l.rot_base, l.vdim);
            if (l.maps == 2) {        // lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff: one number per layer, fp32
                const float sp = 1.0f / std::sqrt((float)l.dim);
                std::vector<float> q1 = vec(mx + "lq1", l.dim, 0.f, sp), k1 = vec(mx + "lk1", l.dim, 0.f, sp), q2 = vec(mx + "lq2", l.dim, 0.f, sp), k2 = vec(mx + "lk2", l.dim, 0.f, sp);
                float d1 = 0.f, d2 = 0.f;
                for (int i = 0; i < l.dim; ++i) { d1 += q1[i] * k1[i]; d2 += q2[i] * k2[i]; }
                w.lambda = std::exp(d1) - std::exp(d2) + l.diff;
            }
            w.o = upload_mat(tensor(mx + "o", W, l.heads * l.vdim));
            max_mix = std::max(max_mix, l.heads * l.vdim);
        } else if (l.type == HY_LINEAR_ATTENTION || l.type == HY_ATTENTION_BESIDE_MEMORY) {
            // fused input projection, every segment on a multiple of 8 rows: [q | k | v | gate (| a1)] of the linear-attention side, and for a
            // layer with attention beside it [q | k | v] of that side (with their biases) in front
            const HyLinear& n = l.lin; const bool two = l.type == HY_ATTENTION_BESIDE_MEMORY;
            const std::string lx = two ? mx + "right." : mx;
            const int qk = n.heads * n.dim, vd = n.heads * n.vdim;
            std::vector<float> bias;
            auto seg = [&](const std::string& nm, int nrows, bool biased) -> int {
                while (rows % 8) { in.v.resize(in.v.size() + W, 0.f); ++rows; }
                const int off = rows;
                append_rows(in.v, rows, W, tensor(nm, nrows, W).v, nrows, 1);
                if (two) { bias.resize(off, 0.f); std::vector<float> b = biased ? vec(nm + ".b", nrows, 0.f, 0.2f) : std::vector<float>(nrows, 0.f); bias.insert(bias.end(), b.begin(), b.end()); }
                return off;
            };
            if (two) {
                if (!hy_win_supported(HyWinAttn{l.heads, l.kv_heads, l.dim, l.vdim, l.maps, l.window, l.keep_first, l.qk_norm, l.gate, l.scale, 0.f, 1.f}))
                    throw std::runtime_error("config.json: attention sizes beyond what the kernels hold (vdim <= 256)");
                w.off_lq = seg(mx + "left.q", l.heads * l.dim, true); w.off_lk = seg(mx + "left.k", l.kv_heads * l.dim, true); w.off_lv = seg(mx + "left.v", l.kv_heads * l.vdim, true);
                w.q_norm = upload_f32(vec(mx + "left.q.norm", l.heads * l.dim, 1.f, 0.1f)); w.k_norm = upload_f32(vec(mx + "left.k.norm", l.kv_heads * l.dim, 1.f, 0.1f));
                w.o2 = upload_mat(tensor(mx + "left.o", W, l.heads * l.vdim)); w.o2_bias = upload_f32(vec(mx + "left.o.b", W, 0.f, 0.1f));
                w.out_w1 = upload_f32(vec(mx + "left.out", W, 1.f, 0.1f)); w.out_w2 = upload_f32(vec(mx + "right.out", W, 1.f, 0.1f));
                max_mix2 = std::max(max_mix2, l.heads * l.vdim);
            }
            w.off_q = seg(lx + "q", qk, false); w.off_k = seg(lx + "k", qk, false); w.off_v = seg(lx + "v", vd, false); w.off_g = seg(lx + "g", vd, false);
            if (n.kind == HY_LIN_CHANNEL_DECAY) {
                HostMat a1 = tensor(lx + "a1", st_ ? (int)st_->st.get(lx + "a1").shape[0] : std::max(8, W / 16), W);
                while (rows % 8) { in.v.resize(in.v.size() + W, 0.f); ++rows; }
                w.off_a1 = rows; w.a_rank = a1.N; append_rows(in.v, rows, W, a1.v, a1.N, 1);
                w.a2 = upload_mat(tensor(lx + "a2", qk, w.a_rank)); w.a2_bias = upload_f32(vec(lx + "a2.b", qk, 1.f, 1.f));
            }
            if (n.kind == HY_LIN_HEAD_DECAY) {
                w.decay = upload_f32(n.decay);
                if (n.rot_dims > 0) w.rope = rope_table(n.rot_base, n.rot_dims);
            }
            if (n.kind == HY_LIN_MATRIX_MEMORY) {       // log gates: their own small product with an fp32 result, [W_i ; W_f] and [b_i | b_f]
                HostMat g; g.K = W; int gr = 0;
                append_rows(g.v, gr, W, tensor(lx + "i", n.heads, W).v, n.heads, 1); append_rows(g.v, gr, W, tensor(lx + "f", n.heads, W).v, n.heads, 1);
                while (gr % 8) { g.v.resize(g.v.size() + W, 0.f); ++gr; }
                g.N = gr; w.gates = upload_mat(g);
                std::vector<float> gb = vec(lx + "i.b", n.heads, 0.f, 0.5f), fb = vec(lx + "f.b", n.heads, 2.f, 1.f);
                gb.insert(gb.end(), fb.begin(), fb.end()); gb.resize(gr, 0.f);
                w.gates_bias = upload_f32(gb); max_gates = std::max(max_gates, gr);
            }
            if (n.norm == HY_LIN_NORM_HEAD_WEIGHT) w.norm_w = upload_f32(vec(lx + "norm", n.vdim, 1.f, 0.1f));
            else if (n.norm == HY_LIN_NORM_ALL_WEIGHT) w.norm_w = upload_f32(vec(lx + "norm", vd, 1.f, 0.1f));
            if (two) { bias.resize(up8(rows), 0.f); w.in_bias = upload_f32(bias); w.in_bias_act = upload_act(bias); }
            w.o = upload_mat(tensor(lx + "o", W, vd));
            max_mix = std::max(max_mix, vd); max_qk = std::max(max_qk, qk); max_v = std::max(max_v, vd);
            max_dec = std::max(max_dec, n.kind == HY_LIN_CHANNEL_DECAY ? qk : n.heads); max_h = std::max(max_h, n.heads);
        } else if (l.type == HY_LATENT_ATTENTION) {
            const int qd = l.heads * (l.dim + l.rot_dim), E = l.kv_rank + l.rot_dim;
            if (l.q_rank > 0) {        // queries through a latent: [dq | dkv (| g)] in the fused projection, W_uq as a second stage after the latent's norm
                append_rows(in.v, rows, W, tensor(mx + "dq", l.q_rank, W).v, l.q_rank, 1); w.off_a = 0;
                w.dq_norm = upload_f32(vec(mx + "dq.norm", l.q_rank, 1.f, 0.1f)); w.uq = upload_mat(tensor(mx + "uq", qd, l.q_rank));
                max_cq = std::max(max_cq, up8(l.q_rank)); max_p2 = std::max(max_p2, up8(qd));
            } else { append_rows(in.v, rows, W, tensor(mx + "q", qd, W).v, qd, 1); w.off_a = 0; }
            while (rows % 8) { in.v.resize(in.v.size() + W, 0.f); ++rows; }
            w.off_b = rows; append_rows(in.v, rows, W, tensor(mx + "dkv", E, W).v, E, 1);
            if (l.gate == HY_GATE_CHANNEL) {
                while (rows % 8) { in.v.resize(in.v.size() + W, 0.f); ++rows; }
                w.off_d = rows; append_rows(in.v, rows, W, tensor(mx + "g", l.heads * l.vdim, W).v, l.heads * l.vdim, 1);
            }
            if (l.sink) w.sink = upload_f32(vec(mx + "sink", l.heads, 0.f, 1.f));
            w.dkv_norm = upload_f32(vec(mx + "dkv.norm", l.kv_rank, 1.f, 0.1f));
            // W_uk per head transposed to [rank, dim]: the absorbed query W_uk^T q is then an ordinary A . B^T product
            HostMat uk = tensor(mx + "uk", l.heads * l.dim, l.kv_rank);
            std::vector<float> ukt((size_t)l.heads * l.kv_rank * l.dim);
            for (int h = 0; h < l.heads; ++h) for (int d = 0; d < l.dim; ++d) for (int r = 0; r < l.kv_rank; ++r)
                ukt[((size_t)h * l.kv_rank + r) * l.dim + d] = uk.v[((size_t)h * l.dim + d) * l.kv_rank + r];
            w.uk_t = upload_act(ukt);
            HostMat uvm = tensor(mx + "uv", l.heads * l.vdim, l.kv_rank);
            w.uv = upload_act(uvm.v);
            if (!f32_ && opt.hy_tensor_core && opt.hy_unabsorbed_rows > 0 && hy_mha_prefill_supported(latent_params(l, w))) {
                HostMat kvu; kvu.N = l.heads * (l.dim + l.vdim); kvu.K = l.kv_rank; kvu.v = uk.v; kvu.v.insert(kvu.v.end(), uvm.v.begin(), uvm.v.end());
                w.kv_up = upload_mat(kvu);       // [W_uk ; W_uv]: keys and values of a whole context in one product (prefill form)
                max_kv = std::max(max_kv, up8(kvu.N));
            }
            w.o = upload_mat(tensor(mx + "o", W, l.heads * l.vdim));
            if (!f32_ && opt.hy_tensor_core && l.dim % 8 == 0 && l.rot_dim % 8 == 0 && l.kv_rank % 8 == 0 && l.vdim % 8 == 0) {
                const int bns[4] = {32, 64, 128, 256}; bool all = true;
                for (int h = 0; h < l.heads && all; ++h) {
                    Mat a; a.p = reinterpret_cast<char*>(w.uk_t) + (size_t)h * l.kv_rank * l.dim * 2; a.N = l.kv_rank; a.K = a.ld = l.dim; a.tc = true;
                    Mat b; b.p = reinterpret_cast<char*>(w.uv) + (size_t)h * l.vdim * l.kv_rank * 2; b.N = l.vdim; b.K = b.ld = l.kv_rank; b.tc = true;
                    for (int i = 0; i < 4; ++i)
                        all = all && make_tmap_bf16_2d(&a.tm[i], a.p, (uint64_t)a.N, (uint64_t)a.ld, (uint64_t)a.ld, (uint32_t)bns[i], 64) == 0 &&
                              make_tmap_bf16_2d(&b.tm[i], b.p, (uint64_t)b.N, (uint64_t)b.ld, (uint64_t)b.ld, (uint32_t)bns[i], 64) == 0;
                    w.uk_heads.push_back(a); w.uv_heads.push_back(b);
                }
                if (!all) { w.uk_heads.clear(); w.uv_heads.clear(); }
            }
            w.rope = rope_table(l.rot_base, l.rot_dims, l.rot_scaling.on ? &l.rot_scaling : nullptr);
            max_Eattn = std::max(max_Eattn, E); max_lat_heads = std::max(max_lat_heads, l.heads); max_qabs = std::max(max_qabs, l.heads * E); max_lat = std::max(max_lat, l.heads * l.kv_rank); max_mix = std::max(max_mix, l.heads * l.vdim);
        } else if (l.type == HY_CHANNEL_DELTA) {
            const int qk = l.kv_heads * l.dim, vd = l.heads * l.vdim;
            append_rows(in.v, rows, W, tensor(mx + "q", qk, W).v, qk, 1); append_rows(in.v, rows, W, tensor(mx + "k", qk, W).v, qk, 1);
            append_rows(in.v, rows, W, tensor(mx + "v", vd, W).v, vd, 1);
            w.off_a = 0; w.conv_ch = 2 * qk + vd;
            while (rows % 8) { in.v.resize(in.v.size() + W, 0.f); ++rows; }
            w.off_b = rows; append_rows(in.v, rows, W, tensor(mx + "b", l.heads, W).v, l.heads, 1);
            while (rows % 8) { in.v.resize(in.v.size() + W, 0.f); ++rows; }
            HostMat a1 = tensor(mx + "a1", st_ ? (int)st_->st.get(mx + "a1").shape[0] : std::max(8, W / 16), W);
            w.off_c = rows; w.a_rank = a1.N; append_rows(in.v, rows, W, a1.v, a1.N, 1);
            while (rows % 8) { in.v.resize(in.v.size() + W, 0.f); ++rows; }
            HostMat g1 = tensor(mx + "g1", st_ ? (int)st_->st.get(mx + "g1").shape[0] : std::max(8, W / 16), W);
            w.off_d = rows; w.g_rank = g1.N; append_rows(in.v, rows, W, g1.v, g1.N, 1);
            w.a2 = upload_mat(tensor(mx + "a2", l.heads * l.dim, w.a_rank)); w.g2 = upload_mat(tensor(mx + "g2", vd, w.g_rank));
            w.A_log = upload_f32(vec(mx + "A_log", l.heads, 0.f, 0.5f)); w.dt_bias = upload_f32(vec(mx + "dt_bias", l.heads * l.dim, 0.f, 0.5f));
            w.norm_w = upload_f32(vec(mx + "norm", l.vdim, 1.f, 0.1f));
            std::vector<float> cw = vec(mx + "q.conv", qk * l.conv, 0.f, 0.5f), ck = vec(mx + "k.conv", qk * l.conv, 0.f, 0.5f), cv = vec(mx + "v.conv", vd * l.conv, 0.f, 0.5f);
            cw.insert(cw.end(), ck.begin(), ck.end()); cw.insert(cw.end(), cv.begin(), cv.end());
            w.conv_w = upload_f32(cw);
            w.o = upload_mat(tensor(mx + "o", W, vd));
            max_p2 = std::max(max_p2, up8(l.heads * l.dim) + vd); max_conv = std::max(max_conv, w.conv_ch); max_mix = std::max(max_mix, vd);
            max_qk = std::max(max_qk, qk); max_v = std::max(max_v, vd); max_dec = std::max(max_dec, l.heads * l.dim); max_h = std::max(max_h, l.heads);
        } else {
            const int inner = l.heads * l.vdim, gn = l.groups * l.state, n_in = 2 * inner + 2 * gn + l.heads;
            append_rows(in.v, rows, W, tensor(mx + "in", n_in, W).v, n_in, 1);
            w.off_a = 0; w.off_b = inner; w.off_c = 2 * inner + 2 * gn; w.conv_ch = inner + 2 * gn;
            w.conv_w = upload_f32(vec(mx + "conv", w.conv_ch * l.conv, 0.f, 0.5f)); w.conv_b = upload_f32(vec(mx + "conv.b", w.conv_ch, 0.f, 0.1f));
            w.dt_bias = upload_f32(vec(mx + "dt_bias", l.heads, 0.f, 0.5f)); w.A_log = upload_f32(vec(mx + "A_log", l.heads, 0.f, 0.5f));
            w.D = upload_f32(vec(mx + "D", l.heads, 1.f, 0.2f)); w.norm_w = upload_f32(vec(mx + "norm", inner, 1.f, 0.1f));
            w.o = upload_mat(tensor(mx + "o", W, inner));
            max_conv = std::max(max_conv, w.conv_ch); max_mix = std::max(max_mix, inner); max_qk = std::max(max_qk, gn); max_v = std::max(max_v, inner);
            max_dec = std::max(max_dec, l.heads); max_h = std::max(max_h, l.heads);
        }
        in.N = rows; w.in = upload_mat(in);
        max_in = std::max(max_in, up8(rows));
        if (l.moe.present && l.moe.dense) {
            const std::string mp = p + "mlp.";
            w.up = upload_mat(tensor(mp + "up", l.moe.ff, W)); w.dn = upload_mat(tensor(mp + "down", W, l.moe.ff));
            max_act = std::max(max_act, up8(l.moe.ff));
        } else if (l.moe.present) {
            const HyMoe& m = l.moe; const std::string mp = p + "mlp.";
            w.n_exp = m.experts + (m.shared_ff > 0 ? 1 : 0); w.n_top = m.top + (m.shared_ff > 0 ? 1 : 0); w.ff_max = std::max(m.ff, m.shared_ff);
            if (m.router == HY_ROUTER_TOKEN_TABLE) {
                std::vector<int32_t> tb((size_t)V * m.top);
                if (st_) {
                    const StTensor& t = st_->st.get(mp + "table");
                    if (t.dtype != "I32" || t.shape.size() != 2 || t.shape[0] != V || t.shape[1] != m.top) throw std::runtime_error("checkpoint tensor " + mp + "table does not have the shape the configuration implies");
                    std::memcpy(tb.data(), t.data, tb.size() * 4);
                } else {
                    uint64_t sd = name_hash(mp + "table", cfg.seed);
                    for (int v = 0; v < V; ++v) {       // `top` different experts per token id: consecutive ones from a random first
                        const int first = std::min(m.experts - 1, (int)((unit_rand(sd) * 0.5f + 0.5f) * (float)m.experts));
                        for (int c = 0; c < m.top; ++c) tb[(size_t)v * m.top + c] = (first + c) % m.experts;
                    }
                }
                for (int32_t e : tb) if (e < 0 || e >= m.experts) throw std::runtime_error("checkpoint tensor " + mp + "table names an expert that does not exist");
                w.table = (int32_t*)dmalloc(tb.size() * 4);
                cuda_check(cudaMemcpy(w.table, tb.data(), tb.size() * 4, cudaMemcpyHostToDevice), "H2D");
                if (m.shared_ff > 0) { std::vector<float> sg = tensor(mp + "shared.sg", 1, W).v; sg.resize(Wld_, 0.f); w.shared_gate = upload_act(sg); }
            } else {
            w.router = upload_mat(tensor(mp + "router", m.experts, W));
            if (m.router == HY_ROUTER_SOFTMAX_CHOSEN) w.router_bias = upload_f32(vec(mp + "router.b", m.experts, 0.f, 0.05f));
            else w.correction = upload_f32(vec(mp + "correction", m.experts, 0.f, 0.05f));
            }
            w.ffp = up16(w.ff_max);
            // first-stage rows per expert: SwiGLU experts hold gate and up rows interleaved in blocks of 16, gate-less experts their up rows
            const int rows1 = m.act == HY_EXPERT_RELU2 ? w.ffp : 2 * w.ffp;
            std::vector<float> gu((size_t)w.n_exp * rows1 * Wld_, 0.f), dn((size_t)w.n_exp * W * w.ffp, 0.f);
            for (int e = 0; e < w.n_exp; ++e) {
                const bool shared = e == m.experts; const int eff = shared ? m.shared_ff : m.ff;       // the shared expert is stored behind the routed ones, rows beyond its width stay zero
                const std::string ep = shared ? mp + "shared." : mp + "e" + std::to_string(e) + ".";
                HostMat u = tensor(ep + "up", eff, W), d = tensor(ep + "down", W, eff);
                if (m.act == HY_EXPERT_RELU2) {
                    for (int f = 0; f < eff; ++f) std::memcpy(&gu[((size_t)e * w.ffp + f) * Wld_], &u.v[(size_t)f * W], (size_t)W * 4);
                } else {
                    HostMat g = tensor(ep + "gate", eff, W);
                    for (int f = 0; f < eff; ++f) {
                        const size_t pg = ((size_t)e * 2 * w.ffp + (size_t)(f >> 4) * 32 + (f & 15)) * Wld_;
                        std::memcpy(&gu[pg], &g.v[(size_t)f * W], (size_t)W * 4); std::memcpy(&gu[pg + (size_t)16 * Wld_], &u.v[(size_t)f * W], (size_t)W * 4);
                    }
                }
                for (int n = 0; n < W; ++n) std::memcpy(&dn[((size_t)e * W + n) * w.ffp], &d.v[(size_t)n * eff], (size_t)eff * 4);
            }
            w.gu = upload_act(gu); w.down = upload_act(dn);
            if (!f32_ && opt.hy_tensor_core && W % 8 == 0) {
                w.moe_tc = true;
                for (int i = 0; i < 2; ++i) {
                    const uint32_t bn = i ? 256 : 128;
                    if (make_tmap_bf16_2d(&w.tm_gu[i], w.gu, (uint64_t)w.n_exp * rows1, (uint64_t)Wld_, (uint64_t)Wld_, bn, 64) != 0 ||
                        make_tmap_bf16_2d(&w.tm_down[i], w.down, (uint64_t)w.n_exp * W, (uint64_t)w.ffp, (uint64_t)w.ffp, bn, 64) != 0) w.moe_tc = false;
                }
            }
            max_ffp = std::max(max_ffp, w.ffp);
            max_act = std::max(max_act, w.n_top * w.ffp); max_top = std::max(max_top, w.n_top); max_E = std::max(max_E, w.n_exp);
        }
    }
    delete st_; st_ = nullptr;

    // ---- activations ----
    MR_ = std::max(opt.max_step_tokens, opt.max_batch); MS_ = MR_;      // every row of a step may be asked for (the caller then brings the logits buffer)
    const size_t MR = (size_t)MR_;
    x_ = (float*)dmalloc(MR * W * 4); x0_ = (float*)dmalloc(MR * W * 4);
    cat_ = dmalloc(MR * 2 * Wld_ * es_); h_ = dmalloc(MR * Wld_ * es_);
    if (hc_.two_norms) h2_ = dmalloc(MR * Wld_ * es_);
    ld_proj_ = max_in; ld_p2_ = up8(max_p2); ld_conv_ = up8(max_conv); ld_mix_ = up8(max_mix);
    proj_ = dmalloc(MR * ld_proj_ * es_); p2_ = dmalloc(MR * ld_p2_ * es_); conv_ = dmalloc(MR * ld_conv_ * es_); mix_ = dmalloc(MR * ld_mix_ * es_);
    q_abs_ = (float*)dmalloc(MR * max_qabs * 4); lat_ = dmalloc(MR * up8(max_lat) * es_);
    qq_ = (float*)dmalloc(MR * max_qk * 4); kk_ = (float*)dmalloc(MR * max_qk * 4); vv_ = (float*)dmalloc(MR * max_v * 4); rec_ = (float*)dmalloc(MR * max_v * 4);
    dec_ = (float*)dmalloc(MR * max_dec * 4); beta_ = (float*)dmalloc(MR * max_h * 4);
    idx_ = (int32_t*)dmalloc(MR * max_top * 4); wgt_ = (float*)dmalloc(MR * max_top * 4);
    max_tiles_ = (int)((MR * max_top + 127) / 128) + max_E;
    rlog_ = (float*)dmalloc(MR * max_E * 4);
    bool any_moe_tc = false; for (const LayerW& w : lw_) any_moe_tc |= w.moe_tc;
    act_ = dmalloc(std::max(MR * max_act, any_moe_tc ? (size_t)max_tiles_ * 128 * max_ffp : 0) * es_);
    if (any_moe_tc) {
        moe_a_ = dmalloc((size_t)max_tiles_ * 128 * Wld_ * 2); moe_y_ = (float*)dmalloc((size_t)max_tiles_ * 128 * W * 4);
        tile_expert_ = (int32_t*)dmalloc((size_t)max_tiles_ * 4); row_src_ = (int32_t*)dmalloc((size_t)max_tiles_ * 128 * 4);
        n_tiles_ = (int32_t*)dmalloc((size_t)(4 + 2 * max_E) * 4); dst_of_ = (int32_t*)dmalloc(MR * max_top * 4);
    }
    if (hc_.post_norm) { y_ = (float*)dmalloc(MR * W * 4); y2_ = (float*)dmalloc(MR * W * 4); }
    if (hc_.sequential) {
        n_streams_ = std::max(1, hc_.streams);
        y_ = (float*)dmalloc(MR * W * 4); xs_ = (float*)dmalloc(MR * n_streams_ * W * 4);
        ones_ = upload_f32(std::vector<float>(64, 1.f));
        if (hc_.token_shift) { hn_ = (float*)dmalloc(MR * W * 4); shift_prev_ = (float*)dmalloc((size_t)opt.max_batch * W * 4); }
        if (max_cq > 0) { ld_cq_ = max_cq; cq_ = dmalloc(MR * ld_cq_ * es_); }
    }
    if (max_mix2 > 0) { ld_mix2_ = up8(max_mix2); mix2_ = dmalloc(MR * ld_mix2_ * es_); }
    if (max_gates > 0) {
        ld_gates_ = max_gates; gates_ = (float*)dmalloc(MR * ld_gates_ * 4);
        gin_ = (float*)dmalloc(MR * max_h * 4); floor_ = (float*)dmalloc(MR * max_h * 4); ndot_ = (float*)dmalloc(MR * max_h * 4);
    }
    hs_ = dmalloc((size_t)MS_ * Wld_ * es_); d_out_ids_ = (int32_t*)dmalloc((size_t)MS_ * 4);
    logits_ = (float*)dmalloc((size_t)opt.max_batch * V * 4);      // own logits: sampling steps only (one row per sequence)
    cuda_check(cudaMallocHost(&h_out_ids, (size_t)MS_ * 4), "cudaMallocHost");
    mask_words = (V + 31) / 32; mask_slots = 0; max_mask_updates = 0;       // grammar-constrained sampling is not wired to this family's head

    // ---- paged latent cache + state slots ----
    size_t page_bytes = 0;
    for (const HyRun& r : hc_.runs) if (r.cache_owner) page_bytes += (size_t)64 * cache_row_width(hc_.layers[r.layer]) * es_;
    if (opt.num_pages > 0) num_pages = opt.num_pages;
    else {
        size_t free_b = 0, total_b = 0;
        cuda_check(cudaMemGetInfo(&free_b, &total_b), "cudaMemGetInfo");
        double budget = opt.kv_gb > 0 ? opt.kv_gb * 1e9 : (double)free_b - 6e9;
        budget = std::min(budget, (double)free_b - 2e9);
        num_pages = (int)std::max(0.0, std::min(budget / (double)std::max<size_t>(page_bytes, 1), 4.0e6));
    }
    max_pages_per_seq = opt.max_seq_len / 64;
    if (num_pages < 1) throw std::runtime_error("cache pool too small");
    caches_.resize(hc_.n_caches); states_.resize(hc_.n_states); tails_.resize(hc_.n_states); aux_.resize(hc_.n_states);
    state_slots = (hc_.n_states > 0 || hc_.token_shift) ? opt.max_batch : 0;
    if (hc_.token_shift) { shift_states_.resize(hc_.runs.size()); for (size_t i = 0; i < hc_.runs.size(); ++i) shift_states_[i] = (float*)dmalloc((size_t)state_slots * W * 4); }
    for (const HyRun& r : hc_.runs) {
        const HyLayer& l = hc_.layers[r.layer];
        if (r.cache_owner) { const size_t b = (size_t)num_pages * 64 * cache_row_width(l) * es_; caches_[r.cache_idx] = dmalloc(b); kv_pool_bytes += b; }
        if (r.state_idx >= 0 && (l.type == HY_LINEAR_ATTENTION || l.type == HY_ATTENTION_BESIDE_MEMORY)) {
            const HyLinear& n = l.lin;
            states_[r.state_idx] = (float*)dmalloc((size_t)state_slots * n.heads * n.dim * n.vdim * 4);
            if (n.kind == HY_LIN_MATRIX_MEMORY) aux_[r.state_idx] = (float*)dmalloc((size_t)state_slots * n.heads * (n.dim + 1) * 4);
        } else if (r.state_idx >= 0 && l.type == HY_WINDOW_ATTENTION) {
            tails_[r.state_idx] = dmalloc((size_t)state_slots * std::max(1, l.conv - 1) * lw_[r.layer].conv_ch * es_);          // the convolutions' last inputs
        } else if (r.state_idx >= 0) {
            const int sd = l.type == HY_CHANNEL_DELTA ? l.dim : l.state;
            states_[r.state_idx] = (float*)dmalloc((size_t)state_slots * l.heads * sd * l.vdim * 4);
            tails_[r.state_idx] = dmalloc((size_t)state_slots * std::max(1, l.conv - 1) * lw_[r.layer].conv_ch * es_);
        }
    }
    meta_cap_words_ = 4 * MR + (size_t)MS_ + (size_t)opt.max_batch * (max_pages_per_seq + 8) + 64;
    ctx_cap_ = 2 * MR_;
    if (max_kv > 0) { ld_kv_ = max_kv; lat_ctx_ = dmalloc((size_t)ctx_cap_ * max_Eattn * 2); kv_ctx_ = dmalloc((size_t)ctx_cap_ * ld_kv_ * 2); }
    for (const HyLayer& l : hc_.layers) if (l.type == HY_LATENT_ATTENTION) meta_cap_words_ += 3 * ((MR / 64 + (size_t)opt.max_batch) * l.heads + 8) + (size_t)opt.max_batch + 8;
    split_slots_ = std::min(16 * opt.max_batch, 4096);
    for (const HyLayer& l : hc_.layers) if (l.type == HY_LATENT_ATTENTION) meta_cap_words_ += 5 * (MR * l.heads / HY_MLA_TILE_QUERIES + (size_t)opt.max_batch + (size_t)split_slots_ + 8) + 3 * ((size_t)opt.max_batch + 4);
    for (const HyLayer& l : hc_.layers) if (l.type == HY_WINDOW_ATTENTION || l.type == HY_ATTENTION_BESIDE_MEMORY) meta_cap_words_ += 2 * (MR * (size_t)(l.heads / l.kv_heads) / HY_WIN_TILE_QUERIES + 2 * (size_t)opt.max_batch + 16);
    if (hc_.n_caches > 0 && !f32_) { split_o_ = (float*)dmalloc((size_t)split_slots_ * max_lat * 4); split_ml_ = (float*)dmalloc((size_t)split_slots_ * max_lat_heads * 2 * 4); }
    for (int i = 0; i < 2; ++i) {
        cuda_check(cudaMallocHost(&h_meta_buf_[i], meta_cap_words_ * 4), "cudaMallocHost meta");
        cuda_check(cudaEventCreateWithFlags(&meta_ev_[i], cudaEventDisableTiming), "cudaEventCreate meta");
    }
    d_meta_ = (int32_t*)dmalloc(meta_cap_words_ * 4);
    cuda_check(cudaStreamSynchronize(stream), "init sync");
}

HybridModel::~HybridModel() {
    HyDeviceGuard guard(opt.device);
    if (stream) cudaStreamSynchronize(stream);
    for (void* p : allocs_) cudaFree(p);
    if (h_out_ids) cudaFreeHost(h_out_ids);
    for (int i = 0; i < 2; ++i) { if (h_meta_buf_[i]) cudaFreeHost(h_meta_buf_[i]); if (meta_ev_[i]) cudaEventDestroy(meta_ev_[i]); }
    if (stream) cudaStreamDestroy(stream);
    delete st_;
}

// N-tile of the tensor-core GEMM: the widest tile that still gives about one CTA per SM (half of them for one or two row tiles)
static int pick_tile_n(int M, int N, int sms) {
    const int m_tiles = (M + 127) / 128;
    const long long want = m_tiles <= 2 ? sms / 2 : sms;
    for (int bn : {256, 128, 64, 32}) if ((long long)((N + bn - 1) / bn) * m_tiles >= want) return bn;
    return 32;
}
static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

void HybridModel::gemm(int mode, const void* A, int lda, const Mat& B, void* C, int ldc, int M, const float* bias, float alpha, const void* bias_act, int act) {
    // bf16: the framework's tcgen05 tile GEMM (TMA operands, fp32 accumulator in TMEM) wherever pitches and pointers fit its 16-byte rules;
    // a bf16 store may write the columns up to N rounded up to 8 (every such output has that room), an fp32 output needs N itself to fit
    bool tc = B.tc && !f32_ && lda % 8 == 0 && aligned16(A) && lda >= B.ld;
    if (mode == HY_STORE) tc = tc && ldc % 8 == 0 && aligned16(C) && (!bias || (bias_act && aligned16(bias_act))) && alpha == 1.f;     // a bias in the activation type, padded to N rounded up to 8
    else tc = tc && B.N % 8 == 0 && ldc % 4 == 0 && aligned16(C) && (!bias || aligned16(bias)) && act == 0;
    CUtensorMap tmA;
    if (tc && make_tmap_bf16_2d(&tmA, A, (uint64_t)M, (uint64_t)B.ld, (uint64_t)lda, 128, 64) != 0) tc = false;
    if (!tc) { cuda_check(hy_gemm(f32_, mode, A, lda, B.p, B.ld, C, ldc, M, B.N, B.K, bias, alpha, 1, 0, 0, 0, stream, act), "gemm"); return; }
    GemmParams g{}; g.M = M; g.N = up8(B.N); g.K = B.ld;
    const int bn = pick_tile_n(M, g.N, sm_count);
    if (mode == HY_STORE) { g.out = C; g.ldo = ldc; g.bias = bias ? bias_act : nullptr; g.store_act = act; cuda_check(launch_gemm(&tmA, &B.tm[bn == 32 ? 0 : bn == 64 ? 1 : bn == 128 ? 2 : 3], g, EPI_STORE, bn, stream), "gemm (tcgen05)"); return; }
    g.f32_out = reinterpret_cast<float*>(C); g.ldf = ldc; g.f32_accumulate = mode == HY_ACC_F32; g.alpha = alpha; g.bias_f32 = bias;
    cuda_check(launch_gemm(&tmA, &B.tm[bn == 32 ? 0 : bn == 64 ? 1 : bn == 128 ? 2 : 3], g, EPI_F32, bn, stream), "gemm (tcgen05, fp32 out)");
}

void HybridModel::moe(const LayerW& w, const HyLayer& l, const void* h_in, const HyRows& r, const std::function<void(int)>& MARK, const int32_t* tokens, float beta) {
    const HyMoe& m = l.moe; const int W = hc_.width, T = r.T;
    const bool relu2 = m.act == HY_EXPERT_RELU2; const int rows1 = relu2 ? w.ffp : 2 * w.ffp;
    if (m.dense) {        // one feed-forward for every row: up product with the activation in its epilogue, down product into the sublayer's fp32 output
        gemm(HY_STORE, h_in, Wld_, w.up, act_, up8(m.ff), T, nullptr, 1.f, nullptr, relu2 ? 1 : m.act == HY_EXPERT_GELU_TANH ? 2 : 0); MARK(25);
        gemm(HY_STORE_F32, act_, up8(m.ff), w.dn, y_, W, T, nullptr, 1.f); MARK(26);
        return;
    }
    HyRouter hr{m.experts, m.top, m.groups, m.keep, m.scale, m.router};
    if (m.router == HY_ROUTER_TOKEN_TABLE) {
        cuda_check(hy_moe_router_table(f32_, tokens, w.table, hc_.vocab, m.top, m.shared_ff > 0 ? m.experts : -1, h_in, Wld_, w.shared_gate, W, idx_, wgt_, T, stream), "router (table)");
    } else {
        // router logits: bf16 (or fp32) inputs, exact products, fp32 accumulation and output
        gemm(HY_STORE_F32, h_in, Wld_, w.router, rlog_, m.experts, T, nullptr, 1.f);
        if (m.router == HY_ROUTER_SOFTMAX_CHOSEN) cuda_check(hy_moe_router_softmax(hr, rlog_, m.experts, w.router_bias, idx_, wgt_, T, stream), "router");
        else cuda_check(hy_moe_router(hr, rlog_, m.experts, w.correction, idx_, wgt_, T, stream), "router");
    }
    MARK(12);
    if (w.moe_tc && T >= opt.hy_moe_grouped_rows) {
        // prefill-sized batches: rows sorted by expert into 128-row tiles, two grouped tcgen05 GEMMs (SwiGLU in the first one's epilogue),
        // then each token adds its choices' rows in choice order
        const int bound = std::min(max_tiles_, (T * w.n_top + 127) / 128 + std::min(w.n_exp, T * w.n_top));
        cuda_check(hy_moe_plan(idx_, T, w.n_top, w.n_exp, tile_expert_, row_src_, n_tiles_, dst_of_, bound, stream), "expert plan");
        cuda_check(hy_moe_gather(h_in, Wld_, Wld_, row_src_, n_tiles_, w.n_top, moe_a_, bound, stream), "expert gather"); MARK(16);
        CUtensorMap tmA, tmB;
        if (make_tmap_bf16_2d(&tmA, moe_a_, (uint64_t)bound * 128, (uint64_t)Wld_, (uint64_t)Wld_, 128, 64) != 0 ||
            make_tmap_bf16_2d(&tmB, act_, (uint64_t)bound * 128, (uint64_t)w.ffp, (uint64_t)w.ffp, 128, 64) != 0) throw std::runtime_error("tensor map for the expert activations failed");
        GemmParams g{}; g.M = bound * 128; g.N = rows1; g.K = Wld_; g.out = act_; g.ldo = w.ffp; g.store_act = relu2 ? 1 : 0;
        g.m_tile_group = tile_expert_; g.n_m_tiles = n_tiles_; g.group_rows = rows1;
        const int bn1 = rows1 >= 256 ? 256 : 128;
        cuda_check(launch_gemm(&tmA, &w.tm_gu[bn1 == 256], g, relu2 ? EPI_STORE : EPI_SWIGLU, bn1, stream), "experts first stage (grouped tcgen05)"); MARK(17);
        GemmParams d{}; d.M = bound * 128; d.N = W; d.K = w.ffp; d.f32_out = moe_y_; d.ldf = W; d.alpha = 1.f;
        d.m_tile_group = tile_expert_; d.n_m_tiles = n_tiles_; d.group_rows = W;
        const int bn2 = W >= 256 ? 256 : 128;
        cuda_check(launch_gemm(&tmB, &w.tm_down[bn2 == 256], d, EPI_F32, bn2, stream), "experts down (grouped tcgen05)"); MARK(18);
        cuda_check(hy_moe_combine(moe_y_, W, dst_of_, wgt_, w.n_top, x_, W, T, stream, beta), "expert combine"); MARK(19);
        return;
    }
    cuda_check(hy_moe_gate_up(f32_, relu2, h_in, Wld_, w.gu, Wld_, W, w.ff_max, w.ffp, idx_, w.n_top, act_, T, stream), "experts first stage");
    cuda_check(hy_moe_down(f32_, act_, w.down, W, w.ffp, idx_, wgt_, w.n_top, x_, T, stream, beta), "experts down"); MARK(13);
}

const char* HybridModel::kt_name(int id) const {
    static const char* n[32] = {"h2d+embed", "layer_norm", "in_proj_gemm", "latent_absorb+up_gemm", "latent_cache_write", "latent_attention", "conv", "recurrence_prep",
                                "recurrence", "gated_norm", "low_rank_gemm", "out_proj_gemm", "router", "experts_per_token", "loop_in", "head+argmax",
                                "expert_plan+gather", "expert_gate_up_gemm", "expert_down_gemm", "expert_combine", "context_gather+kv_up_gemm", "attention_prefill_form", "rms_norm", "window_qk_norm+cache_write",
                                "window_attention", "dense_ff_up_gemm", "dense_ff_down_gemm", "post_norm", "linear_attention_prep", "memory_gates", "", ""};
    return n[id & 31];
}

static HyWinAttn win_params(const HyLayer& l, float lambda) {
    HyWinAttn a{l.heads, l.kv_heads, l.dim, l.vdim, l.maps, l.window, l.keep_first, l.qk_norm, l.gate, l.scale, lambda, 1.f - l.diff};
    a.softcap = l.softcap; a.slope_exp = l.slope_exp; a.q_temp_coef = l.q_temp_coef; a.q_temp_every = l.q_temp_every;
    a.out_rot = l.v_rot ? (l.rot_layout == HY_ROT_HALVES ? 2 : 1) : 0;
    return a;
}

// The linear-attention side of a layer: operands from the fused input projection (proj_), the recurrence on the sequence's state slot, the
// per-head norm and output gate; leaves the output projection's input in mix_.
void HybridModel::linear_mixer(const HyRun& run, const HyLayer& l, const LayerW& w, const HyRows& r, const std::function<void(int)>& MARK) {
    const HyLinear& n = l.lin; const int H = n.heads, D = n.dim, VD = n.vdim, T = r.T;
    auto at = [&](void* base, size_t elems) -> void* { return reinterpret_cast<char*>(base) + elems * es_; };
    const void *q = at(proj_, w.off_q), *k = at(proj_, w.off_k), *v = at(proj_, w.off_v), *g = at(proj_, w.off_g);
    float* st = states_[run.state_idx];
    if (n.kind == HY_LIN_CHANNEL_DECAY) {
        gemm(HY_STORE_F32, at(proj_, w.off_a1), ld_proj_, w.a2, dec_, H * D, T, w.a2_bias, 1.f); MARK(10);       // the decay's pre-activation in fp32
        cuda_check(hy_lin_prep(f32_, HyLinPrep{H, D, VD, n.q_scaled, n.k_scaled, 0}, q, k, v, ld_proj_, qq_, kk_, vv_, dec_, n.tau, nullptr, nullptr, nullptr, nullptr, r, stream), "linear attention operands"); MARK(28);
        cuda_check(hy_recurrence(HY_REC_CHANNEL, qq_, kk_, vv_, dec_, nullptr, rec_, st, H, H, D, VD, r, stream), "gated linear attention"); MARK(8);
        cuda_check(hy_gated_norm(f32_, rec_, H * VD, VD, w.norm_w, VD, g, ld_proj_, 0, n.gate_silu, nullptr, 1, nullptr, 0, mix_, ld_mix_, hc_.eps, T, stream), "gated norm"); MARK(9);
    } else if (n.kind == HY_LIN_HEAD_DECAY) {
        const float* rc = w.rope >= 0 ? ropes_[w.rope].cos : nullptr; const float* rs = w.rope >= 0 ? ropes_[w.rope].sin : nullptr;
        cuda_check(hy_lin_prep(f32_, HyLinPrep{H, D, VD, n.q_scaled, n.k_scaled, n.rot_dims}, q, k, v, ld_proj_, qq_, kk_, vv_, nullptr, 1.f, w.decay, dec_, rc, rs, r, stream), "retention operands"); MARK(28);
        cuda_check(hy_recurrence(HY_REC_SCALAR, qq_, kk_, vv_, dec_, nullptr, rec_, st, H, H, D, VD, r, stream), "retention"); MARK(8);
        cuda_check(hy_gated_norm(f32_, rec_, H * VD, VD, nullptr, 1, g, ld_proj_, 0, n.gate_silu, nullptr, 1, nullptr, 0, mix_, ld_mix_, hc_.eps, T, stream), "gated norm"); MARK(9);
    } else {
        float* aux = aux_[run.state_idx];
        gemm(HY_STORE_F32, h_, Wld_, w.gates, gates_, ld_gates_, T, w.gates_bias, 1.f);
        cuda_check(hy_mlstm_gates(gates_, ld_gates_, H, n.gate_cap, aux + (size_t)state_slots * H * D, dec_, gin_, floor_, r, stream), "matrix memory gates"); MARK(29);
        cuda_check(hy_mlstm_prep(f32_, H, D, VD, q, k, v, ld_proj_, gin_, qq_, kk_, vv_, T, stream), "matrix memory operands"); MARK(28);
        cuda_check(hy_recurrence(HY_REC_SCALAR, qq_, kk_, vv_, dec_, nullptr, rec_, st, H, H, D, VD, r, stream, aux, ndot_), "matrix memory"); MARK(8);
        cuda_check(hy_gated_norm(f32_, rec_, H * VD, VD, w.norm_w, H * VD, g, ld_proj_, 0, n.gate_silu, nullptr, 1, nullptr, 0, mix_, ld_mix_, hc_.eps, T, stream, ndot_, floor_), "gated norm"); MARK(9);
    }
}


HyLatentAttn HybridModel::latent_params(const HyLayer& l, const LayerW& w) const {
    HyLatentAttn a{l.heads, l.dim, l.rot_dim, l.vdim, l.kv_rank, l.rot_dims, l.scale};
    a.window = l.type == HY_LATENT_ATTENTION ? l.window : 0; a.rot_layout = l.rot_layout; a.sink = w.sink;
    return a;
}

void HybridModel::window_mixer(const HyRun& run, const HyLayer& l, const LayerW& w, const HyRows& r, const TileList& tl, const std::function<void(int)>& MARK, void* q, void* k, void* v, int ld,
                               const void* gate, int ldg, bool prepared) {
    HyWinAttn a{l.heads, l.kv_heads, l.dim, l.vdim, l.maps, l.window, l.keep_first, l.qk_norm, l.gate, l.scale, w.lambda, 1.f - l.diff};
    if (l.v_rot) { a.out_rot = l.rot_layout == HY_ROT_HALVES ? 2 : 1; a.out_cos = ropes_[w.rope_v].cos; a.out_sin = ropes_[w.rope_v].sin; }
    if (!prepared && (l.rot_dims > 0 || l.v_rot)) {
        const HyRotary rot{l.rot_dims, l.rot_layout, l.rot_dims > 0 ? ropes_[w.rope].cos : nullptr, l.rot_dims > 0 ? ropes_[w.rope].sin : nullptr,
                           l.v_rot ? ropes_[w.rope_v].cos : nullptr, l.v_rot ? ropes_[w.rope_v].sin : nullptr};
        cuda_check(hy_win_rope_prep(f32_, a, rot, q, ld, k, v, ld, caches_[run.cache_idx], r, stream), "rotary + cache write");
    } else if (!prepared) cuda_check(hy_win_prep(f32_, a, q, ld, k, v, ld, w.q_norm, w.k_norm, hc_.eps, caches_[run.cache_idx], r, stream), "query / key norm + cache write");
    if (!prepared) MARK(23);
    if (tl.mma) {
        cuda_check(hy_win_attention_mma(a, q, ld, caches_[run.cache_idx], w.sink, gate, ldg, mix_, ld_mix_, hc_.eps, r, d_meta_ + tl.o_wseq, d_meta_ + tl.o_wq0, tl.n_w, stream), "windowed attention (mma)");
        cuda_check(hy_win_decode_mma(a, q, ld, caches_[run.cache_idx], w.sink, gate, ldg, mix_, ld_mix_, hc_.eps, r, d_meta_ + tl.o_dseq, d_meta_ + tl.o_dq0, tl.n_d, stream), "windowed attention (mma, decoding rows)");
    } else cuda_check(hy_win_attention(f32_, a, q, ld, caches_[run.cache_idx], w.sink, gate, ldg, mix_, ld_mix_, hc_.eps, r, stream), "windowed attention");
    MARK(24);
}

void HybridModel::latent_mixer(const HyRun& run, const HyLayer& l, const LayerW& w, const HyRows& r, const TileList& tl, const std::function<void(int)>& MARK, void* q, int ldq, void* ckv, int ldc,
                               const void* gate, int ldg) {
    auto at = [&](void* base, size_t elems) -> void* { return reinterpret_cast<char*>(base) + elems * es_; };
    const int T = r.T;
    const HyLatentAttn a = latent_params(l, w);
    const int E = l.kv_rank + l.rot_dim;
    cuda_check(hy_mla_prep(f32_, a, q, ldq, ckv, ldc, w.dkv_norm, hc_.eps, ropes_[w.rope].cos, ropes_[w.rope].sin, caches_[run.cache_idx], q_abs_, r, stream), "latent cache write"); MARK(4);
    if (tl.any_small) {
        // absorbed queries: q_abs[t, h, :rank] = W_uk[h]^T q_unrotated[t, h]
        const bool head_tc = !w.uk_heads.empty() && T >= 256 && ldq % 8 == 0;      // prefill-sized steps: one tcgen05 GEMM per head; smaller ones: one batched launch
        if (head_tc) for (int hd = 0; hd < l.heads; ++hd) gemm(HY_STORE_F32, at(q, (size_t)hd * (l.dim + l.rot_dim)), ldq, w.uk_heads[hd], q_abs_ + (size_t)hd * E, l.heads * E, T, nullptr, 1.f);
        else cuda_check(hy_gemm(f32_, HY_STORE_F32, q, ldq, w.uk_t, l.dim, q_abs_, l.heads * E, T, l.kv_rank, l.dim, nullptr, 1.f, l.heads,
                                l.dim + l.rot_dim, (long long)l.kv_rank * l.dim, E, stream), "query absorption");
        MARK(3);
        if (tl.mma) {
            HyMlaSplit sp{nullptr, nullptr, nullptr, split_o_, split_ml_};
            if (tl.n_merge > 0) { sp.tile_k0 = d_meta_ + tl.o_k0; sp.tile_k1 = d_meta_ + tl.o_k1; sp.tile_slot = d_meta_ + tl.o_slot; }
            cuda_check(hy_mla_attention_mma(a, q_abs_, caches_[run.cache_idx], lat_, r, d_meta_ + tl.o_seq, d_meta_ + tl.o_q0, tl.n, sp, stream), "latent attention (mma)");
            cuda_check(hy_mla_merge(d_meta_ + tl.o_mrow, d_meta_ + tl.o_mslot, d_meta_ + tl.o_mparts, tl.n_merge, split_o_, split_ml_, lat_, l.heads, l.kv_rank, stream, a.sink), "latent attention (join)");
        } else cuda_check(hy_mla_attention(f32_, a, q_abs_, caches_[run.cache_idx], lat_, r, stream), "latent attention");
        MARK(5);
        if (head_tc) for (int hd = 0; hd < l.heads; ++hd) gemm(HY_STORE, at(lat_, (size_t)hd * l.kv_rank), l.heads * l.kv_rank, w.uv_heads[hd], at(mix_, (size_t)hd * l.vdim), ld_mix_, T, nullptr, 1.f);
        else cuda_check(hy_gemm(f32_, HY_STORE, lat_, l.heads * l.kv_rank, w.uv, l.kv_rank, mix_, ld_mix_, T, l.vdim, l.kv_rank, nullptr, 1.f, l.heads, l.kv_rank,
                                (long long)l.vdim * l.kv_rank, l.vdim, stream), "value up-projection");
        MARK(3);
        if (gate) { cuda_check(hy_sigmoid_gate(f32_, mix_, ld_mix_, gate, ldg, l.heads * l.vdim, T, stream), "output gate"); MARK(9); }
    }
    if (tl.n_ptiles > 0) {      // prefill form for the sequences that bring many rows (after the absorbed path, whose up-projection wrote every row of mix_)
        cuda_check(hy_gather_ctx(caches_[run.cache_idx], E, r, d_meta_ + tl.o_base, tl.max_ctx, lat_ctx_, stream), "context gather");
        gemm(HY_STORE, lat_ctx_, E, w.kv_up, kv_ctx_, ld_kv_, tl.ctx_rows, nullptr, 1.f); MARK(20);
        HyLatentAttn ag = a; ag.gate = gate; ag.ldg = ldg;          // the gate rides in the attention kernel's epilogue
        cuda_check(hy_mha_prefill(ag, q, ldq, q_abs_, kv_ctx_, ld_kv_, lat_ctx_, mix_, ld_mix_, r, d_meta_ + tl.o_pseq, d_meta_ + tl.o_phead,
                                  d_meta_ + tl.o_prow0, d_meta_ + tl.o_base, tl.n_ptiles, stream), "attention (prefill form)"); MARK(21);
    }
}

// Designs whose sublayers run in sequence on pre-norms of the residual they find: per layer execution
//   [close the previous sublayer + open the mixer: streams' update, u = in . x, RMS norm] -> token shift -> input projection -> mixer -> output
//   projection (fp32 y) -> [close the mixer + open the feed-forward] -> up product with the activation -> down product (fp32 y).
// A sublayer's y is folded into the streams by the kernel that opens the next sublayer, so a layer costs two passes over the residual.
void HybridModel::forward_sequential(const HyRows& r, const std::vector<TileList>& tile_lists, const int32_t* d_tokens, const std::function<void(int)>& MARK) {
    auto at = [&](void* base, size_t elems) -> void* { return reinterpret_cast<char*>(base) + elems * es_; };
    const int T = r.T, W = hc_.width, n = n_streams_;
    const bool hyper = hc_.streams > 0;
    const float *pend_mix = nullptr, *pend_out = nullptr;      // coefficients of the sublayer whose y_ has not been folded into the streams yet
    bool pending = false;
    auto open = [&](const float* in, const float* norm_w, float* shift_state, const char* what) {
        const HyStreams c{n, pend_mix, pend_out, in};
        cuda_check(hy_stream_norm(f32_, c, xs_, pending ? y_ : nullptr, nullptr, norm_w, hc_.eps, h_, Wld_, hn_, shift_state, shift_prev_, r, T, W, stream), what);
        pending = false;
    };
    for (const HyRun& run : hc_.runs) {
        const HyLayer& l = hc_.layers[run.layer]; const LayerW& w = lw_[run.layer];
        float* sstate = w.shift ? shift_states_[run.index] : nullptr;
        open(hyper ? w.hc_in[0] : ones_, w.norm1, sstate, "streams + norm (mixer)");
        if (sstate) cuda_check(hy_token_shift(f32_, hn_, shift_prev_, w.shift, h_, Wld_, r, W, stream), "token shift");
        MARK(22);
        gemm(HY_STORE, h_, Wld_, w.in, proj_, ld_proj_, T, w.in_bias, 1.f, w.in_bias_act); MARK(2);
        if (l.type == HY_LATENT_ATTENTION) {
            void* q = at(proj_, w.off_a); int ldq = ld_proj_;
            if (l.q_rank > 0) {
                cuda_check(hy_rmsnorm_act(f32_, at(proj_, w.off_a), ld_proj_, l.q_rank, w.dq_norm, cq_, ld_cq_, hc_.eps, T, stream), "query latent norm");
                gemm(HY_STORE, cq_, ld_cq_, w.uq, p2_, ld_p2_, T, nullptr, 1.f); MARK(10);
                q = p2_; ldq = ld_p2_;
            }
            latent_mixer(run, l, w, r, tile_lists[run.layer], MARK, q, ldq, at(proj_, w.off_b), ld_proj_, l.gate == HY_GATE_CHANNEL ? at(proj_, w.off_d) : nullptr, ld_proj_);
        } else if (l.type == HY_WINDOW_ATTENTION) {
            void* src = proj_; int ld = ld_proj_;
            const HyWinAttn wa = win_params(l, 0.f);
            const HyRotary rot{l.rot_dims, l.rot_layout, l.rot_dims > 0 ? ropes_[w.rope].cos : nullptr, l.rot_dims > 0 ? ropes_[w.rope].sin : nullptr,
                               l.v_rot ? ropes_[w.rope_v].cos : nullptr, l.v_rot ? ropes_[w.rope_v].sin : nullptr};
            if (!f32_ && l.conv > 1 && run.cache_owner && hy_conv_rope_cache_supported(wa, rot, l.conv)) {
                // convolution, rotation and cache write in one kernel; the fp32 convolution is rounded once, after the rotation
                cuda_check(hy_conv_rope_cache(wa, rot, proj_, ld_proj_, w.conv_ch, w.off_a, w.off_b, w.off_c, w.conv_w, l.conv, at(conv_, w.off_a), ld_conv_, caches_[run.cache_idx],
                                              tails_[run.state_idx], r, stream), "conv + rotary + cache write");
                cuda_check(hy_conv_tails(f32_, proj_, ld_proj_, w.conv_ch, l.conv, tails_[run.state_idx], r, stream), "conv tails"); MARK(6);
                window_mixer(run, l, w, r, tile_lists[run.layer], MARK, at(conv_, w.off_a), nullptr, nullptr, ld_conv_, l.gate ? at(proj_, w.off_d) : nullptr, ld_proj_, true);
            } else {
            if (l.conv > 0) {
                cuda_check(hy_conv_silu(f32_, proj_, ld_proj_, w.conv_ch, w.conv_w, nullptr, l.conv, conv_, ld_conv_, run.state_idx >= 0 ? tails_[run.state_idx] : nullptr, r, stream, 0), "conv");
                if (l.conv > 1) cuda_check(hy_conv_tails(f32_, proj_, ld_proj_, w.conv_ch, l.conv, tails_[run.state_idx], r, stream), "conv tails");
                MARK(6); src = conv_; ld = ld_conv_;
            }
            window_mixer(run, l, w, r, tile_lists[run.layer], MARK, at(src, w.off_a), at(src, w.off_b), at(src, w.off_c), ld, l.gate ? at(proj_, w.off_d) : nullptr, ld_proj_);
            }
        } else throw std::runtime_error("forward: this design has no such mixer");
        gemm(HY_STORE_F32, mix_, ld_mix_, w.o, y_, W, T, w.o_bias, 1.f); MARK(11);
        pending = true; pend_mix = hyper ? w.hc_mix[0] : ones_; pend_out = hyper ? w.hc_out[0] : ones_;
        if (l.moe.present) {
            open(hyper ? w.hc_in[1] : ones_, w.norm2, nullptr, "streams + norm (feed-forward)"); MARK(22);
            moe(w, l, h_, r, MARK, d_tokens);
            pending = true; pend_mix = hyper ? w.hc_mix[1] : ones_; pend_out = hyper ? w.hc_out[1] : ones_;
        }
        if (capture_layers) {          // debug: the residual (sum of the streams) after this execution
            open(nullptr, nullptr, nullptr, "streams (capture)");
            cuda_check(cudaStreamSynchronize(stream), "capture sync");
            std::vector<float> tmp((size_t)T * n * W);
            cuda_check(cudaMemcpy(tmp.data(), xs_, tmp.size() * 4, cudaMemcpyDeviceToHost), "capture D2H");
            const size_t n0 = capture_layers->size(); capture_layers->resize(n0 + (size_t)T * W, 0.f);
            for (int t = 0; t < T; ++t) for (int sidx = 0; sidx < n; ++sidx) for (int c = 0; c < W; ++c) (*capture_layers)[n0 + (size_t)t * W + c] += tmp[((size_t)t * n + sidx) * W + c];
        }
    }
    pending_ = pending; pend_mix_ = pend_mix; pend_out_ = pend_out;      // the final norm folds the last y_ into the rows it reads; the streams themselves are not needed again
}

void HybridModel::forward(const StepInput& in, float* logits_out) {
    const int T = (int)in.tokens.size(), S = in.n_seqs, NS = (int)in.sample_rows.size(), W = hc_.width, V = hc_.vocab;
    if (T <= 0 || T > MR_ || NS > MS_ || S <= 0 || S > opt.max_batch) throw std::runtime_error("forward: bad batch size");
    if ((int)in.seq_row0.size() != S + 1 || (int)in.state_slots.size() != S || in.seq_row0[S] != T) throw std::runtime_error("forward: this model needs the rows of every sequence (seq_row0) and its state slot");
    row_seq_.resize(T); seq_pos0_.resize(S);
    for (int s = 0; s < S; ++s) {
        if (in.seq_row0[s + 1] <= in.seq_row0[s]) throw std::runtime_error("forward: empty sequence in a step");
        if (state_slots > 0 && (in.state_slots[s] < 0 || in.state_slots[s] >= state_slots)) throw std::runtime_error("forward: state slot out of range");
        seq_pos0_[s] = in.positions[in.seq_row0[s]];
        for (int t = in.seq_row0[s]; t < in.seq_row0[s + 1]; ++t) { row_seq_[t] = s; if (in.positions[t] != seq_pos0_[s] + (t - in.seq_row0[s])) throw std::runtime_error("forward: rows of a sequence must be consecutive positions"); }
        if (in.positions[in.seq_row0[s + 1] - 1] >= opt.max_seq_len) throw std::runtime_error("forward: position beyond max_seq_len");
    }
    meta_idx_ ^= 1; int32_t* hm = h_meta_buf_[meta_idx_];
    cuda_check(cudaEventSynchronize(meta_ev_[meta_idx_]), "meta staging fence");
    size_t wd = 0;
    auto put = [&](const void* src, size_t words) -> size_t {
        size_t at = wd; if (at + words > meta_cap_words_) throw std::runtime_error("forward: metadata arena overflow");
        if (words) std::memcpy(hm + at, src, words * 4);
        wd = (at + words + 3) & ~size_t(3); return at;
    };
    const size_t o_tok = put(in.tokens.data(), T), o_pos = put(in.positions.data(), T), o_slot = put(in.slots.data(), T), o_samp = put(in.sample_rows.data(), NS);
    const size_t o_bt = put(in.block_tables.data(), in.block_tables.size()), o_rs = put(row_seq_.data(), T), o_r0 = put(in.seq_row0.data(), S + 1);
    const size_t o_p0 = put(seq_pos0_.data(), S), o_st = put(in.state_slots.data(), S);
    // attention plans, one per attention layer.  Sequences that bring at least hy_unabsorbed_rows rows take the prefill form (keys / values of
    // their context up-projected by a GEMM, ordinary multi-head attention); the others — decoding rows, short portions — the absorbed form:
    // tiles of 64 consecutive (row, head) pairs of one sequence, a decoding row with a long context cut into parts.
    std::vector<TileList> tile_lists(hc_.layers.size());
    for (size_t li = 0; li < hc_.layers.size(); ++li) {
        const HyLayer& l = hc_.layers[li]; TileList& tl = tile_lists[li];
        if (l.type == HY_WINDOW_ATTENTION || l.type == HY_ATTENTION_BESIDE_MEMORY) {
            // windowed attention on the tensor cores: tiles of 64 consecutive (row, head-of-the-group) pairs of one sequence; a decoding row is one tile per key/value head
            tl.mma = !f32_ && opt.hy_tensor_core && ld_proj_ % 8 == 0 && (l.type == HY_WINDOW_ATTENTION ? ld_mix_ : ld_mix2_) % 8 == 0 && hy_win_mma_supported(win_params(l, 0.f));
            if (!tl.mma) continue;
            tile_seq_.clear(); tile_q0_.clear(); ptile_seq_.clear(); ptile_row0_.clear();
            const int group = l.heads / l.kv_heads;
            for (int sq = 0; sq < S; ++sq) {
                const int nq = (in.seq_row0[sq + 1] - in.seq_row0[sq]) * group;
                if (nq <= HY_WIN_DECODE_QUERIES) { ptile_seq_.push_back(sq); ptile_row0_.push_back(0); continue; }       // decoding rows: the form whose warps split the keys
                for (int q0 = 0; q0 < nq; q0 += HY_WIN_TILE_QUERIES) { tile_seq_.push_back(sq); tile_q0_.push_back(q0); }
            }
            tl.n_w = (int)tile_seq_.size(); tl.o_wseq = put(tile_seq_.data(), tile_seq_.size()); tl.o_wq0 = put(tile_q0_.data(), tile_q0_.size());
            tl.n_d = (int)ptile_seq_.size(); tl.o_dseq = put(ptile_seq_.data(), ptile_seq_.size()); tl.o_dq0 = put(ptile_row0_.data(), ptile_row0_.size());
            continue;
        }
        if (l.type != HY_LATENT_ATTENTION) continue;
        const bool prefill_form = lw_[li].kv_up.tc && kv_ctx_;
        tl.mma = !f32_ && opt.hy_tensor_core && hy_mla_mma_supported(latent_params(l, lw_[li]));
        tile_seq_.clear(); tile_q0_.clear(); tile_k0_.clear(); tile_k1_.clear(); tile_slot_.clear(); merge_row_.clear(); merge_slot_.clear(); merge_parts_.clear();
        ptile_seq_.clear(); ptile_head_.clear(); ptile_row0_.clear(); seq_base_.assign(S, -1);
        int next_slot = 0;
        for (int sq = 0; sq < S; ++sq) {
            const int len = in.seq_row0[sq + 1] - in.seq_row0[sq], nq = len * l.heads, ctx_end = seq_pos0_[sq] + len;
            // many rows, or a short portion that is a good part of its own context (the start of a prompt cut by the step's token budget)
            if (prefill_form && (len >= opt.hy_unabsorbed_rows || (len >= 2 && ctx_end <= 8 * len)) && tl.ctx_rows + ctx_end <= ctx_cap_) {
                seq_base_[sq] = tl.ctx_rows; tl.ctx_rows += ctx_end; tl.max_ctx = std::max(tl.max_ctx, ctx_end);
                for (int hd = 0; hd < l.heads; ++hd) for (int q0 = 0; q0 < len; q0 += 64) { ptile_seq_.push_back(sq); ptile_head_.push_back(hd); ptile_row0_.push_back(q0); }
                continue;
            }
            tl.any_small = true;
            if (!tl.mma) continue;
            const int ctx = seq_pos0_[sq] + 1, vis0 = l.window > 0 ? std::max(0, ctx - l.window) / 32 * 32 : 0;       // first visible cache row of a decoding row, on a tile border
            // a decoding row with a long context: its visible cache rows in 2..16 parts, one CTA each, joined afterwards — up to four parts of
            // >= 128 rows, beyond that parts of >= 256 rows.  The cut depends on the row's position only.
            const int vis = ctx - vis0;
            int parts = (len == 1 && nq <= HY_MLA_TILE_QUERIES) ? std::min(16, std::max(vis / 256, std::min(4, vis / 128))) : 1;
            if (parts > 1 && next_slot + parts > split_slots_) parts = 1;
            if (parts > 1) {
                const int per = ((ctx - vis0 + parts - 1) / parts + 31) / 32 * 32; parts = (ctx - vis0 + per - 1) / per;
                merge_row_.push_back(in.seq_row0[sq]); merge_slot_.push_back(next_slot); merge_parts_.push_back(parts);
                for (int pz = 0; pz < parts; ++pz) {
                    tile_seq_.push_back(sq); tile_q0_.push_back(0); tile_k0_.push_back(vis0 + pz * per); tile_k1_.push_back(std::min(ctx, vis0 + (pz + 1) * per)); tile_slot_.push_back(next_slot++);
                }
                continue;
            }
            for (int q0 = 0; q0 < nq; q0 += HY_MLA_TILE_QUERIES) { tile_seq_.push_back(sq); tile_q0_.push_back(q0); tile_k0_.push_back(0); tile_k1_.push_back(0); tile_slot_.push_back(-1); }
        }
        tl.n = (int)tile_seq_.size(); tl.n_merge = (int)merge_row_.size(); tl.n_ptiles = (int)ptile_seq_.size();
        tl.o_seq = put(tile_seq_.data(), tile_seq_.size()); tl.o_q0 = put(tile_q0_.data(), tile_q0_.size());
        tl.o_k0 = put(tile_k0_.data(), tile_k0_.size()); tl.o_k1 = put(tile_k1_.data(), tile_k1_.size()); tl.o_slot = put(tile_slot_.data(), tile_slot_.size());
        tl.o_mrow = put(merge_row_.data(), merge_row_.size()); tl.o_mslot = put(merge_slot_.data(), merge_slot_.size()); tl.o_mparts = put(merge_parts_.data(), merge_parts_.size());
        tl.o_pseq = put(ptile_seq_.data(), ptile_seq_.size()); tl.o_phead = put(ptile_head_.data(), ptile_head_.size()); tl.o_prow0 = put(ptile_row0_.data(), ptile_row0_.size());
        tl.o_base = put(seq_base_.data(), seq_base_.size());
    }
    cuda_check(cudaMemcpyAsync(d_meta_, hm, wd * 4, cudaMemcpyHostToDevice, stream), "meta H2D");
    cuda_check(cudaEventRecord(meta_ev_[meta_idx_], stream), "meta event");
    h2d_bytes += wd * 4;
    HyRows r{d_meta_ + o_pos, d_meta_ + o_slot, d_meta_ + o_rs, d_meta_ + o_r0, d_meta_ + o_p0, d_meta_ + o_st, d_meta_ + o_bt, max_pages_per_seq, T, S};
    static const char* dbg_layers = std::getenv("OA_DEBUG_LAYERS");      // debug: file that receives the residual stream after every layer execution of each forward
    std::vector<float> dbg_buf;
    if (dbg_layers && !capture_layers) capture_layers = &dbg_buf;
    if (capture_layers) capture_layers->clear();

    size_t ek = 0;
    if (profile_all) {
        const size_t need = hc_.runs.size() * 32 + 16;
        if (ev_all.size() < need) { size_t o = ev_all.size(); ev_all.resize(need); for (size_t i = o; i < need; ++i) cudaEventCreate(&ev_all[i]); }
        ev_ids.assign(ev_all.size(), 0);
        cudaEventRecord(ev_all[ek++], stream);
    }
    const std::function<void(int)> MARK = [&](int id) { if (profile_all && ek < ev_all.size()) { ev_ids[ek] = id; cudaEventRecord(ev_all[ek++], stream); } };
    if (hc_.sequential) { cuda_check(hy_embed_streams(f32_, d_meta_ + o_tok, embed_, xs_, T, W, V, hc_.embed_scale, n_streams_, stream), "embed"); MARK(0); forward_sequential(r, tile_lists, d_meta_ + o_tok, MARK); }
    else { cuda_check(hy_embed(f32_, d_meta_ + o_tok, embed_, x_, hc_.loop_times > 0 ? x0_ : nullptr, T, W, V, hc_.embed_scale, stream, hc_.post_norm ? h_ : nullptr, Wld_), "embed"); MARK(0); }
    auto at = [&](void* base, size_t elems) -> void* { return reinterpret_cast<char*>(base) + elems * es_; };
    for (const HyRun& run : hc_.runs) {
        if (hc_.sequential) break;          // forward_sequential() has run every layer execution
        const HyLayer& l = hc_.layers[run.layer]; const LayerW& w = lw_[run.layer];
        if (run.first_of_pass && hc_.loop_reinject) {         // re-injection: x <- W_in [x ; x0] + step[pass]
            cuda_check(hy_concat(f32_, x_, x0_, cat_, T, W, stream), "concat");
            gemm(HY_STORE_F32, cat_, 2 * W, loop_in_, x_, W, T, loop_step_ + (size_t)run.pass * W, 1.f); MARK(14);
        }
        if (hc_.post_norm) {
            // norm after the sum: the sublayers read the residual itself (h_ holds it in the activation type), their outputs come back in fp32
            // (y_, y2_) and hy_post_norm closes each half: x <- norm(alpha x + sublayer(x))
            gemm(HY_STORE, h_, Wld_, w.in, proj_, ld_proj_, T, w.in_bias, 1.f, w.in_bias_act); MARK(2);
            const bool two = l.type == HY_ATTENTION_BESIDE_MEMORY;
            if (two) {
                const HyWinAttn a = win_params(l, 0.f);
                cuda_check(hy_win_prep(f32_, a, at(proj_, w.off_lq), ld_proj_, at(proj_, w.off_lk), at(proj_, w.off_lv), ld_proj_, w.q_norm, w.k_norm, hc_.eps, caches_[run.cache_idx], r, stream),
                           "query / key norm + cache write"); MARK(23);
                const TileList& tl = tile_lists[run.layer];
                if (tl.mma) {
                    cuda_check(hy_win_attention_mma(a, at(proj_, w.off_lq), ld_proj_, caches_[run.cache_idx], nullptr, nullptr, 0, mix2_, ld_mix2_, hc_.eps, r, d_meta_ + tl.o_wseq, d_meta_ + tl.o_wq0,
                                                    tl.n_w, stream), "attention (mma)");
                    cuda_check(hy_win_decode_mma(a, at(proj_, w.off_lq), ld_proj_, caches_[run.cache_idx], nullptr, nullptr, 0, mix2_, ld_mix2_, hc_.eps, r, d_meta_ + tl.o_dseq, d_meta_ + tl.o_dq0,
                                                 tl.n_d, stream), "attention (mma, decoding rows)");
                } else cuda_check(hy_win_attention(f32_, a, at(proj_, w.off_lq), ld_proj_, caches_[run.cache_idx], nullptr, nullptr, 0, mix2_, ld_mix2_, hc_.eps, r, stream), "attention");
                MARK(24);
                gemm(HY_STORE_F32, mix2_, ld_mix2_, w.o2, y2_, W, T, w.o2_bias, 1.f); MARK(11);
            }
            linear_mixer(run, l, w, r, MARK);
            gemm(HY_STORE_F32, mix_, ld_mix_, w.o, y_, W, T, nullptr, 1.f); MARK(11);
            if (two) cuda_check(hy_post_norm(f32_, x_, hc_.post_alpha, y2_, w.out_w1, y_, w.out_w2, 0.5f, w.norm1, h_, Wld_, T, W, hc_.eps, stream), "norm after the mixers");
            else cuda_check(hy_post_norm(f32_, x_, hc_.post_alpha, y_, nullptr, nullptr, nullptr, 1.f, w.norm1, h_, Wld_, T, W, hc_.eps, stream), "norm after the mixer");
            MARK(27);
            if (l.moe.present && l.moe.dense) {
                moe(w, l, h_, r, MARK);
                cuda_check(hy_post_norm(f32_, x_, hc_.post_alpha, y_, nullptr, nullptr, nullptr, 1.f, w.norm2, h_, Wld_, T, W, hc_.eps, stream), "norm after the feed-forward"); MARK(27);
            } else if (l.moe.present) {
                moe(w, l, h_, r, MARK, d_meta_ + o_tok, hc_.post_alpha);      // x <- alpha x + experts, choice by choice
                cuda_check(hy_post_norm(f32_, x_, 1.f, nullptr, nullptr, nullptr, nullptr, 1.f, w.norm2, h_, Wld_, T, W, hc_.eps, stream), "norm after the experts"); MARK(27);
            } else if (w.norm2) { cuda_check(hy_post_norm(f32_, x_, hc_.post_alpha, nullptr, nullptr, nullptr, nullptr, 1.f, w.norm2, h_, Wld_, T, W, hc_.eps, stream), "second norm"); MARK(27); }
            if (capture_layers) {
                cuda_check(cudaStreamSynchronize(stream), "capture sync");
                const size_t n0 = capture_layers->size(); capture_layers->resize(n0 + (size_t)T * W);
                cuda_check(cudaMemcpy(capture_layers->data() + n0, x_, (size_t)T * W * 4, cudaMemcpyDeviceToHost), "capture D2H");
            }
            continue;
        }
        if (hc_.norm == HY_RMS_NORM) { cuda_check(hy_rmsnorm_pair(f32_, x_, nullptr, w.norm1, h_, w.norm2, w.norm2 ? h2_ : nullptr, Wld_, T, W, hc_.eps, stream), "rms norm"); MARK(22); }
        else { cuda_check(hy_layernorm(f32_, x_, nullptr, w.norm1, h_, Wld_, T, W, hc_.eps, stream), "layer norm"); MARK(1); }
        gemm(HY_STORE, h_, Wld_, w.in, proj_, ld_proj_, T, w.in_bias, 1.f, w.in_bias_act); MARK(2);
        if (l.type == HY_WINDOW_ATTENTION) {
            const bool own = run.cache_owner;
            window_mixer(run, l, w, r, tile_lists[run.layer], MARK, at(proj_, w.off_a), own ? at(proj_, w.off_b) : nullptr, own ? at(proj_, w.off_c) : nullptr, ld_proj_, l.gate ? at(proj_, w.off_d) : nullptr, ld_proj_);
        } else if (l.type == HY_LATENT_ATTENTION) {
            latent_mixer(run, l, w, r, tile_lists[run.layer], MARK, at(proj_, w.off_a), ld_proj_, at(proj_, w.off_b), ld_proj_);
        } else if (l.type == HY_CHANNEL_DELTA) {
            const HyDelta d{l.heads, l.kv_heads, l.dim, l.vdim};
            cuda_check(hy_conv_silu(f32_, at(proj_, w.off_a), ld_proj_, w.conv_ch, w.conv_w, nullptr, l.conv, conv_, ld_conv_, tails_[run.state_idx], r, stream), "conv");
            cuda_check(hy_conv_tails(f32_, at(proj_, w.off_a), ld_proj_, w.conv_ch, l.conv, tails_[run.state_idx], r, stream), "conv tails"); MARK(6);
            const int off_g = up8(l.heads * l.dim);
            gemm(HY_STORE, at(proj_, w.off_c), ld_proj_, w.a2, p2_, ld_p2_, T, nullptr, 1.f);
            gemm(HY_STORE, at(proj_, w.off_d), ld_proj_, w.g2, at(p2_, off_g), ld_p2_, T, nullptr, 1.f); MARK(10);
            cuda_check(hy_delta_prep(f32_, d, conv_, ld_conv_, at(proj_, w.off_b), ld_proj_, p2_, ld_p2_, w.A_log, w.dt_bias, qq_, kk_, vv_, dec_, beta_, T, stream), "delta prep"); MARK(7);
            cuda_check(hy_recurrence(HY_REC_DELTA, qq_, kk_, vv_, dec_, beta_, rec_, states_[run.state_idx], l.heads, l.kv_heads, l.dim, l.vdim, r, stream), "delta rule"); MARK(8);
            cuda_check(hy_gated_norm(f32_, rec_, l.heads * l.vdim, l.vdim, w.norm_w, l.vdim, at(p2_, off_g), ld_p2_, 0, 0, nullptr, 1, nullptr, 0, mix_, ld_mix_, hc_.eps, T, stream), "gated norm"); MARK(9);
        } else {
            const HyMamba m{l.heads, l.vdim, l.state, l.groups};
            const int inner = l.heads * l.vdim;
            cuda_check(hy_conv_silu(f32_, at(proj_, w.off_b), ld_proj_, w.conv_ch, w.conv_w, w.conv_b, l.conv, conv_, ld_conv_, tails_[run.state_idx], r, stream), "conv");
            cuda_check(hy_conv_tails(f32_, at(proj_, w.off_b), ld_proj_, w.conv_ch, l.conv, tails_[run.state_idx], r, stream), "conv tails"); MARK(6);
            cuda_check(hy_mamba_prep(f32_, m, conv_, ld_conv_, at(proj_, w.off_c), ld_proj_, w.A_log, w.dt_bias, qq_, kk_, vv_, dec_, T, stream), "mamba prep"); MARK(7);
            cuda_check(hy_recurrence(HY_REC_SCALAR, qq_, kk_, vv_, dec_, nullptr, rec_, states_[run.state_idx], l.heads, l.groups, l.state, l.vdim, r, stream), "state-space recurrence"); MARK(8);
            cuda_check(hy_gated_norm(f32_, rec_, inner, inner / l.norm_groups, w.norm_w, inner, at(proj_, w.off_a), ld_proj_, 1, 1, w.D, l.vdim, conv_, ld_conv_, mix_, ld_mix_,
                                     hc_.eps, T, stream), "gated norm"); MARK(9);
        }
        gemm(HY_ACC_F32, mix_, ld_mix_, w.o, x_, W, T, nullptr, 1.f); MARK(11);
        if (l.moe.present) moe(w, l, w.norm2 ? h2_ : h_, r, MARK);
        if (capture_layers) {
            cuda_check(cudaStreamSynchronize(stream), "capture sync");
            const size_t n0 = capture_layers->size(); capture_layers->resize(n0 + (size_t)T * W);
            cuda_check(cudaMemcpy(capture_layers->data() + n0, x_, (size_t)T * W * 4, cudaMemcpyDeviceToHost), "capture D2H");
        }
    }
    if (capture_layers == &dbg_buf) {
        if (FILE* f = std::fopen(dbg_layers, "wb")) { std::fwrite(dbg_buf.data(), 4, dbg_buf.size(), f); std::fclose(f); }
        capture_layers = nullptr;
    }
    if (NS > 0) {
        if (hc_.sequential) {      // x = the sum of the streams, of the wanted rows only
            const HyStreams fin{n_streams_, pend_mix_, pend_out_, ones_};
            cuda_check(hy_stream_norm(f32_, fin, xs_, pending_ ? y_ : nullptr, d_meta_ + o_samp, final_norm_, hc_.eps, hs_, Wld_, nullptr, nullptr, nullptr, r, NS, W, stream), "final norm");
        } else if (hc_.norm == HY_RMS_NORM) cuda_check(hy_rmsnorm_pair(f32_, x_, d_meta_ + o_samp, final_norm_, hs_, nullptr, nullptr, Wld_, NS, W, hc_.eps, stream), "final norm");
        else cuda_check(hy_layernorm(f32_, x_, d_meta_ + o_samp, final_norm_, hs_, Wld_, NS, W, hc_.eps, stream), "final norm");
        if (!logits_out && NS > opt.max_batch) throw std::runtime_error("forward: more sampled rows than sequences need a caller's logits buffer");
        float* lg = logits_out ? logits_out : logits_;
        gemm(HY_STORE_F32, hs_, Wld_, head_, lg, V, NS, nullptr, hc_.logit_scale);
        cuda_check(hy_argmax_rows(lg, NS, V, hc_.logit_softcap, d_out_ids_, stream), "soft cap + argmax");
        cuda_check(cudaMemcpyAsync(h_out_ids, d_out_ids_, (size_t)NS * 4, cudaMemcpyDeviceToHost, stream), "ids D2H");
        d2h_bytes += (size_t)NS * 4; MARK(15);
    }
    if (profile_all) {
        cuda_check(cudaStreamSynchronize(stream), "profile sync");
        for (size_t i = 1; i < ek; ++i) { float ms = 0; cudaEventElapsedTime(&ms, ev_all[i - 1], ev_all[i]); kt_ms[ev_ids[i] & 31] += ms; kt_n[ev_ids[i] & 31]++; }
    }
}

std::unique_ptr<ModelBase> make_model(const ModelConfig& cfg, const EngineOptions& opt) {
    if (cfg.hybrid) return std::unique_ptr<ModelBase>(new HybridModel(cfg, opt));        // every design of the hybrid family: one class, configured by the design's traits
    if (opt.f32) throw std::runtime_error("the Llama-family models run in bf16 only; float32 is available for the hybrid family");
    return std::unique_ptr<ModelBase>(new DeviceModel(cfg, opt));
}

}  // namespace oa
