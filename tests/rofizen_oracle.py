"""Plain float64 restatement of the Rofizen design, one function per mechanism, no cache and no batching: every function takes the whole
sequence [T, ...] and walks it position by position where the mechanism is a recurrence.  It shares nothing with the engine; the GPU tests
compare the engine's logits (whole prompts, portions, decoding, mixed batches) with `forward()` of this file.

Notation: h is a sublayer's input [T, W]; weights are stored [out, in] and applied as h @ W.T; `w` is a dict name -> ndarray (float64, the
expert tables int)."""
import math

import numpy as np


def layer_norm(x, weight, eps):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * weight


def rms_unit(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


def rotate_half(x, positions, base, dims):
    """x [T, heads, dim]: the first `dims` channels of every head are rotated, channel i paired with i + dims/2"""
    out = x.copy()
    half = dims // 2
    f = base ** (-2.0 * np.arange(half) / dims)
    ang = positions[:, None] * f[None, :]                      # [T, half]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


# ---- token mixers ------------------------------------------------------------------------------------------------------------------

def softmax_branch(h, w, p, m, eps):
    """causal soft-capped attention with a distance penalty, grouped key/value heads, a norm over the whole q / k projection and a query
    temperature that grows with the position"""
    T = h.shape[0]
    H, G, D, VD = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ w[p + "q"].T + w[p + "q.b"]
    k = h @ w[p + "k"].T + w[p + "k.b"]
    v = h @ w[p + "v"].T + w[p + "v.b"]
    q = rms_unit(q, eps) * w[p + "q.norm"]
    k = rms_unit(k, eps) * w[p + "k.norm"]
    pos = np.arange(T)
    temp = 1.0 + m["q_temp"]["coef"] * np.log(np.floor((pos + 1) / m["q_temp"]["every"]) + 1.0)
    q = (q * temp[:, None]).reshape(T, H, D)
    k = k.reshape(T, G, D)
    v = v.reshape(T, G, VD)
    out = np.zeros((T, H, VD))
    cap = m["softcap"]
    for hd in range(H):
        g = hd // (H // G)
        slope = 2.0 ** (-8.0 * (hd + 1) / H)
        for i in range(T):
            s = (k[: i + 1, g] @ q[i, hd]) * m["scale"]
            s = cap * np.tanh(s / cap)
            s = s - slope * (i - np.arange(i + 1))
            e = np.exp(s - s.max())
            out[i, hd] = (e / e.sum()) @ v[: i + 1, g]
    return out.reshape(T, H * VD) @ w[p + "o"].T + w[p + "o.b"]


def matrix_memory_branch(h, w, p, m, eps):
    """matrix memory with exponential input gate and a running maximum that starts at zero"""
    T = h.shape[0]
    H, D, VD, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ w[p + "q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ w[p + "k"].T).reshape(T, H, D)
    v = (h @ w[p + "v"].T).reshape(T, H, VD)
    ig = cap * np.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)                   # [T, H], log input gate
    fg = log_sigmoid(cap * np.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))      # log forget gate
    S = np.zeros((H, D, VD))
    n = np.zeros((H, D))
    mx = np.zeros(H)
    o = np.zeros((T, H, VD))
    for t in range(T):
        m_new = np.maximum(fg[t] + mx, ig[t])
        a = np.exp(fg[t] + mx - m_new)
        b = np.exp(ig[t] - m_new)
        S = a[:, None, None] * S + b[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = a[:, None] * n + b[:, None] * k[t]
        mx = m_new
        num = np.einsum("hdv,hd->hv", S, q[t])
        den = np.maximum(np.abs((n * q[t]).sum(-1)), np.exp(-mx)) + 1e-6
        o[t] = num / den[:, None]
    o = rms_unit(o, eps).reshape(T, H * VD) * w[p + "norm"]
    return (o * sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps):
    left = softmax_branch(h, w, p + "left.", m["left"], eps)
    right = matrix_memory_branch(h, w, p + "right.", m["right"], eps)
    return 0.5 * (rms_unit(left, eps) * w[p + "left.out"] + rms_unit(right, eps) * w[p + "right.out"])


def gla_mixer(h, w, p, m, eps):
    """gated linear attention: a decay per key channel from a low-rank projection"""
    T = h.shape[0]
    H, D, VD = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ w[p + "k"].T).reshape(T, H, D)
    v = (h @ w[p + "v"].T).reshape(T, H, VD)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = np.exp(log_sigmoid(z) / m["tau"]).reshape(T, H, D)
    S = np.zeros((H, D, VD))
    o = np.zeros((T, H, VD))
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hdv,hd->hv", S, q[t])
    o = (rms_unit(o, eps) * w[p + "norm"]).reshape(T, H * VD)
    return (o * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def retention_mixer(h, w, p, m, eps):
    """linear attention with one fixed decay per head and rotary positions on q and k"""
    T = h.shape[0]
    H, D, VD = m["heads"], m["dim"], m["vdim"]
    pos = np.arange(T, dtype=np.float64)
    q = rotate_half((h @ w[p + "q"].T).reshape(T, H, D), pos, m["rot"]["base"], m["rot"]["dims"])
    k = rotate_half((h @ w[p + "k"].T).reshape(T, H, D), pos, m["rot"]["base"], m["rot"]["dims"]) * D ** -0.5
    v = (h @ w[p + "v"].T).reshape(T, H, VD)
    decay = np.asarray(m["decay"], dtype=np.float64)
    S = np.zeros((H, D, VD))
    o = np.zeros((T, H, VD))
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hdv,hd->hv", S, q[t])
    o = rms_unit(o, eps).reshape(T, H * VD)
    return (o * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


MIXERS = {"parallel": parallel_mixer, "gla": gla_mixer, "retention": retention_mixer}


# ---- feed-forward --------------------------------------------------------------------------------------------------------------------

def dense_ff(h, w, p):
    return np.maximum(h @ w[p + "up"].T, 0.0) ** 2 @ w[p + "down"].T


def gated_expert(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def table_moe(h, tokens, w, p, mlp):
    """every token id owns `top` experts (a table row), each weighted 1 / top; a shared expert, gated by one sigmoid per token, is added"""
    top = mlp["router"]["top"]
    table = w[p + "table"]
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(top):
            out[t] += gated_expert(h[t:t + 1], w, p + "e%d." % int(table[tokens[t], c]))[0] / top
    if mlp.get("shared"):
        out = out + gated_expert(h, w, p + "shared.") * sigmoid(h @ w[p + "shared.sg"].T)
    return out


# ---- the model -----------------------------------------------------------------------------------------------------------------------

def forward(cfg, w, tokens, layers_out=None):
    """logits [T, vocab] of one sequence; layers_out (a list) receives the residual stream after every layer"""
    tokens = np.asarray(tokens)
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = w["embed"][tokens] * cfg["embedding"]["scale"]
    for i, layer in enumerate(cfg["layers"]):
        p = "l%d." % i
        x = layer_norm(alpha * x + MIXERS[layer["type"]](x, w, p + "mix.", layer["mixer"], eps), w[p + "norm1"], eps)
        mlp = layer.get("mlp")
        if mlp:
            y = dense_ff(x, w, p + "mlp.") if mlp["kind"] == "dense" else table_moe(x, tokens, w, p + "mlp.", mlp)
            x = layer_norm(alpha * x + y, w[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    return layer_norm(x, w["final.norm"], eps) @ w["head"].T


# ---- random models for the tests -------------------------------------------------------------------------------------------------------

def tensor_shapes(cfg):
    """name -> shape of every tensor a configuration implies"""
    W, V = cfg["width"], cfg["vocab"]
    s = {"embed": (V, W), "head": (V, W), "final.norm": (W,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = "l%d." % i, layer["mixer"]
        s[p + "norm1"] = (W,)
        x = p + "mix."
        if layer["type"] == "parallel":
            a, b = m["left"], m["right"]
            s.update({x + "left.q": (a["heads"] * a["dim"], W), x + "left.q.b": (a["heads"] * a["dim"],), x + "left.k": (a["kv_heads"] * a["dim"], W),
                      x + "left.k.b": (a["kv_heads"] * a["dim"],), x + "left.v": (a["kv_heads"] * a["vdim"], W), x + "left.v.b": (a["kv_heads"] * a["vdim"],),
                      x + "left.q.norm": (a["heads"] * a["dim"],), x + "left.k.norm": (a["kv_heads"] * a["dim"],), x + "left.o": (W, a["heads"] * a["vdim"]),
                      x + "left.o.b": (W,), x + "left.out": (W,), x + "right.out": (W,),
                      x + "right.q": (b["heads"] * b["dim"], W), x + "right.k": (b["heads"] * b["dim"], W), x + "right.v": (b["heads"] * b["vdim"], W),
                      x + "right.g": (b["heads"] * b["vdim"], W), x + "right.o": (W, b["heads"] * b["vdim"]), x + "right.norm": (b["heads"] * b["vdim"],),
                      x + "right.i": (b["heads"], W), x + "right.i.b": (b["heads"],), x + "right.f": (b["heads"], W), x + "right.f.b": (b["heads"],)})
        else:
            qk, vd = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            s.update({x + "q": (qk, W), x + "k": (qk, W), x + "v": (vd, W), x + "g": (vd, W), x + "o": (W, vd)})
            if layer["type"] == "gla":
                r = m.get("_rank", 8)
                s.update({x + "norm": (m["vdim"],), x + "a1": (r, W), x + "a2": (qk, r), x + "a2.b": (qk,)})
        mlp = layer.get("mlp")
        if mlp:
            s[p + "norm2"] = (W,)
            y = p + "mlp."
            if mlp["kind"] == "dense":
                s.update({y + "up": (mlp["ff"], W), y + "down": (W, mlp["ff"])})
            else:
                ff = mlp["expert"]["ff"]
                for e in range(mlp["router"]["experts"]):
                    s.update({y + "e%d.gate" % e: (ff, W), y + "e%d.up" % e: (ff, W), y + "e%d.down" % e: (W, ff)})
                s[y + "table"] = (V, mlp["router"]["top"])
                if mlp.get("shared"):
                    sf = mlp["shared"]["ff"]
                    s.update({y + "shared.gate": (sf, W), y + "shared.up": (sf, W), y + "shared.down": (W, sf), y + "shared.sg": (1, W)})
    return s


def bf16_round(a):
    """round float64 values to the nearest bfloat16 (ties to even), returned as float64"""
    u = np.asarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32).astype(np.float64)


def random_weights(cfg, seed, spread=1.0):
    """bf16-representable random weights: matrices ~ U(-a, a) with a = spread * sqrt(3 / fan_in), norm weights near 1, biases small; the
    expert table holds `top` different experts per token id"""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith(".table"):
            E = cfg["layers"][int(name[1:name.index(".")])]["mlp"]["router"]["experts"]
            w[name] = np.stack([rng.permutation(E)[: shape[1]] for _ in range(shape[0])]).astype(np.int32)
        elif len(shape) == 1:
            is_norm = name.endswith("norm") or name.endswith("norm1") or name.endswith("norm2") or name.endswith(".out")
            w[name] = bf16_round((1.0 if is_norm else 0.0) + 0.25 * rng.uniform(-1, 1, shape))
        else:
            a = spread * math.sqrt(3.0 / shape[1])
            w[name] = bf16_round(rng.uniform(-a, a, shape))
    return w


def write_checkpoint(folder, cfg, w):
    """config.json + model.safetensors (bf16 matrices and vectors, int32 tables) in `folder`"""
    import json
    import os
    import struct
    os.makedirs(folder, exist_ok=True)
    clean = json.loads(json.dumps(cfg))
    for l in clean["layers"]:
        l["mixer"].pop("_rank", None)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(clean, f)
    header, blobs, at = {}, [], 0
    for name, a in w.items():
        if a.dtype == np.int32:
            b, dt = a.astype("<i4").tobytes(), "I32"
        else:
            b, dt = (np.asarray(a, dtype=np.float32).view(np.uint32) >> 16).astype("<u2").tobytes(), "BF16"
        header[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [at, at + len(b)]}
        blobs.append(b)
        at += len(b)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))


# ---- configurations for the tests ---------------------------------------------------------------------------------------------------------

def rel_err(got, want):
    """per row: RMS over the vocabulary of the difference (its mean taken off), relative to the spread of the expected logits"""
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    return np.sqrt((d * d).mean(-1)) / want.std()


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=24, shared_ff=40):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared_ff:
        m["shared"] = {"ff": shared_ff}
    return m


def gla_layer(heads=3, dim=8, vdim=12, tau=4.0, rank=5, mlp=None):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "_rank": rank}, "mlp": mlp}


def retention_layer(heads=3, dim=12, vdim=8, decay=None, rot_dims=8, rot_base=500.0, mlp=None):
    decay = decay or [1.0 - 2.0 ** (-3 - i) for i in range(heads)]
    return {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay, "rot": {"base": rot_base, "dims": rot_dims}}, "mlp": mlp}


def parallel_layer(heads=4, kv_heads=2, dim=8, vdim=12, scale=0.4, softcap=6.0, coef=0.5, every=5, r_heads=3, r_dim=12, r_vdim=8, gate_cap=7.0, mlp=None):
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap, "q_temp": {"coef": coef, "every": every}},
                      "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "gate_cap": gate_cap}}}


def make_config(layers, width=40, vocab=77, embed_scale=3.0, alpha=1.7, eps=1e-5):
    return {"architecture": "Rofizen", "embedding": {"scale": embed_scale}, "layers": layers, "norm": {"eps": eps}, "postln_alpha": alpha, "vocab": vocab, "width": width}


def sharpen(w, factor):
    """queries that single out keys: the attention side's query norm weights and the matrix memory's input-gate rows grow by `factor`"""
    for name in w:
        if name.endswith("left.q.norm") or name.endswith("right.i"):
            w[name] = bf16_round(w[name] * factor)
    return w
