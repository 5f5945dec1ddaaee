"""Plain float64 restatement of the Gosavik design, one function per mechanism, no cache and no batching: every function takes the whole
sequence [T, ...] and loops over positions where a mechanism looks back.  It shares nothing with the engine; the GPU tests compare the
engine's logits (whole prompts, portions, decoding, mixed batches) with `forward()` of this file.

Notation: h is a sublayer's input [T, W]; weights are stored [out, in] and applied as h @ W.T; `w` is a dict name -> float64 ndarray."""
import json
import math
import os
import struct

import numpy as np


def rms_norm(x, weight, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * weight


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def token_shift(h, mu):
    """h_t <- h_t + (h_(t-1) - h_t) * mu, with the previous row as it was before the replacement and zeros before the first"""
    prev = np.concatenate([np.zeros_like(h[:1]), h[:-1]], 0)
    return h + (prev - h) * mu


def frequencies(base, dims, scaling=None):
    """-> (f [dims / 2], amplitude): plain rotary frequencies, or the YaRN blend of f and f / factor with its amplitude 0.1 ln(factor) + 1"""
    i = np.arange(dims // 2)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    fac, orig = scaling["factor"], scaling["original"]
    where = lambda turns: dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(where(scaling["fast"])), 0)
    hi = min(math.ceil(where(scaling["slow"])), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / fac * ramp + f * (1.0 - ramp), 0.1 * math.log(fac) + 1.0


def rotate(x, pos, f, amp, halves, sign=1.0):
    """x [T, heads, n]: the first 2 len(f) channels of every head turn by sign * pos * f; pairs (i, i + len f) or (2i, 2i + 1)"""
    n = 2 * len(f)
    ang = sign * pos[:, None] * f[None, :]
    c, s = (np.cos(ang) * amp)[:, None, :], (np.sin(ang) * amp)[:, None, :]
    out = x.copy()
    if halves:
        u, v = x[..., : n // 2], x[..., n // 2: n]
        out[..., : n // 2] = u * c - v * s
        out[..., n // 2: n] = v * c + u * s
    else:
        u, v = x[..., 0:n:2], x[..., 1:n:2]
        out[..., 0:n:2] = u * c - v * s
        out[..., 1:n:2] = v * c + u * s
    return out


def sink_softmax_rows(q, k, v, scale, sink, window):
    """q [T, D], k [T, D], v [T, VD] of one head: position i sees j <= i with i - j < window (None: all); exp(sink) joins the denominator"""
    T = q.shape[0]
    out = np.zeros((T, v.shape[1]))
    for i in range(T):
        j0 = 0 if window is None else max(0, i - window + 1)
        s = (k[j0: i + 1] @ q[i]) * scale
        m = max(s.max(), sink)
        e = np.exp(s - m)
        out[i] = (e @ v[j0: i + 1]) / (e.sum() + math.exp(sink - m))
    return out


def latent_attention(h, w, p, m, eps):
    T = h.shape[0]
    H, D, R, VD, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(T, dtype=np.float64)
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).reshape(T, H, D + R)
    ckv = h @ w[p + "dkv"].T
    c = rms_norm(ckv[:, :C], w[p + "dkv.norm"], eps)
    f, amp = frequencies(m["rot"]["base"], m["rot"]["dims"], m["rot"].get("scaling"))
    k_rot = rotate(ckv[:, None, C:], pos, f, amp, True)[:, 0]
    q_rot = rotate(q[..., D:], pos, f, amp, True)
    ku = (c @ w[p + "uk"].T).reshape(T, H, D)
    vu = (c @ w[p + "uv"].T).reshape(T, H, VD)
    window = m["mask"]["size"] if m.get("mask") else None
    out = np.zeros((T, H, VD))
    for hd in range(H):
        qh = np.concatenate([q[:, hd, :D], q_rot[:, hd]], 1)
        kh = np.concatenate([ku[:, hd], k_rot], 1)
        out[:, hd] = sink_softmax_rows(qh, kh, vu[:, hd], m["scale"], w[p + "sink"][hd], window)
    gate = sigmoid(h @ w[p + "g"].T)
    return (out.reshape(T, H * VD) * gate) @ w[p + "o"].T


def short_conv(u, cw):
    """u [T, C], cw [C, taps]: y_t = sum_j cw[:, j] u_(t - taps + 1 + j), zeros before the start"""
    T, taps = u.shape[0], cw.shape[1]
    pad = np.concatenate([np.zeros((taps - 1, u.shape[1])), u], 0)
    y = np.zeros_like(u)
    for j in range(taps):
        y += pad[j: j + T] * cw[:, j]
    return y


def attention(h, w, p, m, eps):
    T = h.shape[0]
    H, G, D, VD = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(T, dtype=np.float64)
    q = short_conv(h @ w[p + "q"].T + w[p + "q.b"], w[p + "q.conv"]).reshape(T, H, D)
    k = short_conv(h @ w[p + "k"].T + w[p + "k.b"], w[p + "k.conv"]).reshape(T, G, D)
    v = short_conv(h @ w[p + "v"].T + w[p + "v.b"], w[p + "v.conv"]).reshape(T, G, VD)
    f, amp = frequencies(m["rot"]["base"], m["rot"]["dims"])
    q, k = rotate(q, pos, f, amp, False), rotate(k, pos, f, amp, False)
    fv, _ = frequencies(m["rot"]["base"], VD)
    v = rotate(v, pos, fv, 1.0, False)
    out = np.zeros((T, H, VD))
    for hd in range(H):
        g = hd // (H // G)
        out[:, hd] = sink_softmax_rows(q[:, hd], k[:, g], v[:, g], m["scale"], w[p + "sink"][hd], None)
    out = rotate(out, pos, fv, 1.0, False, sign=-1.0)
    return out.reshape(T, H * VD) @ w[p + "o"].T + w[p + "o.b"]


def feed_forward(h, w, p):
    return gelu_tanh(h @ w[p + "up"].T) @ w[p + "down"].T


def hyper_step(xs, w, p, sub):
    """xs [streams, T, W]: u = sum_s in[s] x_s; y = sub(u); x_t <- sum_s mix[s, t] x_s + out[t] y"""
    u = np.tensordot(w[p + "in"], xs, 1)
    y = sub(u)
    return np.tensordot(w[p + "mix"].T, xs, 1) + w[p + "out"][:, None, None] * y[None]


def schedule(cfg):
    """layer indices in the order they run (a looped block repeats with the same weights)"""
    n, lp = len(cfg["layers"]), cfg.get("loop")
    if not lp:
        return list(range(n))
    return list(range(lp["start"])) + list(range(lp["start"], lp["stop"])) * lp["times"] + list(range(lp["stop"], n))


def forward(cfg, w, tokens, layers_out=None):
    eps = cfg["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)]
    S = cfg.get("streams", 0)
    xs = np.stack([x] * S) if S else None
    for li in schedule(cfg):
        l, p = cfg["layers"][li], "l%d." % li
        mixer = latent_attention if l["type"] == "latent_attention" else attention

        def mix_sub(u, l=l, p=p, mixer=mixer):
            h = rms_norm(u, w[p + "norm1"], eps)
            if p + "shift" in w:
                h = token_shift(h, w[p + "shift"])
            return mixer(h, w, p + "mix.", l["mixer"], eps)

        def ff_sub(u, p=p):
            return feed_forward(rms_norm(u, w[p + "norm2"], eps), w, p + "mlp.")

        if S:
            xs = hyper_step(xs, w, p + "hc1.", mix_sub)
            if l.get("mlp"):
                xs = hyper_step(xs, w, p + "hc2.", ff_sub)
            x = xs.sum(0)
        else:
            x = x + mix_sub(x)
            if l.get("mlp"):
                x = x + ff_sub(x)
        if layers_out is not None:
            layers_out.append(x.copy())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T


# ---- small random checkpoints for the tests ----------------------------------------------------------------------------------------

def latent_layer(heads=3, dim=8, rot_dim=8, vdim=8, kv_rank=16, q_rank=12, window=9, base=100.0, scaling=True, scale=None, mlp=48):
    rot = {"base": base, "dims": rot_dim}
    if scaling:
        rot["scaling"] = {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0} if scaling is True else scaling
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "rot": rot,
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    if window:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m, "mlp": {"kind": "dense", "ff": mlp} if mlp else None}


def attention_layer(heads=4, kv_heads=2, dim=8, vdim=8, conv=3, rot_dims=None, base=1000.0, scale=None, mlp=48):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "rot": {"base": base, "dims": dim if rot_dims is None else rot_dims},
         "scale": scale if scale is not None else dim ** -0.5}
    return {"type": "attention", "mixer": m, "mlp": {"kind": "dense", "ff": mlp} if mlp else None}


def make_config(layers, width=40, vocab=61, streams=2, loop=None, eps=1e-5):
    cfg = {"architecture": "Gosavik", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers}
    if streams:
        cfg["streams"] = streams
    if loop:
        cfg["loop"] = loop
    return cfg


def tensor_shapes(cfg):
    W, S = cfg["width"], cfg.get("streams", 0)
    sh = {"embed": (cfg["vocab"], W), "head": (cfg["vocab"], W), "final.norm": (W,)}
    for i, l in enumerate(cfg["layers"]):
        p, m = "l%d." % i, l["mixer"]
        sh[p + "norm1"] = (W,)
        sh[p + "shift"] = (W,)
        if l["type"] == "latent_attention":
            H, D, R, VD, C, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            sh.update({p + "mix.dq": (Q, W), p + "mix.dq.norm": (Q,), p + "mix.uq": (H * (D + R), Q), p + "mix.dkv": (C + R, W), p + "mix.dkv.norm": (C,),
                       p + "mix.uk": (H * D, C), p + "mix.uv": (H * VD, C), p + "mix.sink": (H,), p + "mix.g": (H * VD, W), p + "mix.o": (W, H * VD)})
        else:
            H, G, D, VD, K = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            for nm, n in (("q", H * D), ("k", G * D), ("v", G * VD)):
                sh.update({p + "mix." + nm: (n, W), p + "mix." + nm + ".b": (n,), p + "mix." + nm + ".conv": (n, K)})
            sh.update({p + "mix.sink": (H,), p + "mix.o": (W, H * VD), p + "mix.o.b": (W,)})
        if l.get("mlp"):
            sh.update({p + "norm2": (W,), p + "mlp.up": (l["mlp"]["ff"], W), p + "mlp.down": (W, l["mlp"]["ff"])})
        for q in ("hc1.", "hc2.") if S else ():
            if q == "hc2." and not l.get("mlp"):
                continue
            sh.update({p + q + "in": (S,), p + q + "out": (S,), p + q + "mix": (S, S)})
    return sh


def bf16(a):
    """round to the nearest bfloat16 (ties to even), as float64"""
    b = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    b = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16 << 16).astype(np.uint32)
    return b.view(np.float32).astype(np.float64)


def random_weights(cfg, seed=0, spread=1.0):
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith("norm") or name.endswith("norm1") or name.endswith("norm2"):
            v = 1.0 + 0.2 * rng.standard_normal(shape)
        elif name.endswith("shift"):
            v = rng.uniform(0.0, 1.0, shape)
        elif name.endswith("sink"):
            v = rng.standard_normal(shape)
        elif name.endswith(".b"):
            v = 0.3 * rng.standard_normal(shape)
        elif name.endswith(".conv"):
            v = rng.standard_normal(shape) / math.sqrt(shape[1]) + np.eye(1, shape[1], shape[1] - 1) * 0.7
        elif ".hc" in name:
            S = shape[0]
            v = {"in": np.full(shape, 1.0 / S), "out": np.ones(shape), "mix": np.eye(S)}[name.rsplit(".", 1)[1]] + 0.25 * rng.standard_normal(shape)
        elif name == "embed":
            v = rng.standard_normal(shape)
        else:
            v = spread * rng.standard_normal(shape) / math.sqrt(shape[-1])
        w[name] = bf16(v)
    return w


def write_checkpoint(folder, cfg, w):
    """config.json + model.safetensors (bfloat16): 8-byte header length, JSON header, data"""
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, at = {}, [], 0
    for name, a in w.items():
        raw = (np.ascontiguousarray(a, dtype=np.float32).view(np.uint32) >> 16).astype("<u2").tobytes()
        header[name] = {"dtype": "BF16", "shape": list(a.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))


def rel_err(got, want):
    """per row: rms of the difference (means taken off) over the rms spread of the wanted logits"""
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    return np.sqrt((d * d).mean(-1)) / np.sqrt(((want - want.mean(-1, keepdims=True)) ** 2).mean())
