"""Host side of the Gosavik design (no GPU): the configuration reader accepts what the design allows and refuses the rest with a client
error, the registry keys on config.json's "architecture", and the float64 oracle the GPU tests lean on has the properties its mechanisms
are named for."""
import ctypes as C
import json
import os

import numpy as np
import pytest

import gosavik_oracle as G
from opsagent_b200 import _lib


def model_info(folder, **extra):
    L = _lib.load()
    buf = C.create_string_buffer(4096)
    rc = L.oa_host_model_info(json.dumps(dict({"model_dir": str(folder)}, **extra)).encode(), buf, 4096)
    return rc, (json.loads(buf.value.decode()) if rc == 0 else None)


def write_cfg(folder, cfg):
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)


def good_cfg():
    return G.make_config([G.latent_layer(), G.attention_layer(), G.attention_layer(mlp=None)], width=40, vocab=77, streams=3, loop={"start": 1, "stop": 3, "times": 2})


def test_config_reader_accepts_the_design(tmp_path):
    write_cfg(tmp_path, good_cfg())
    rc, info = model_info(tmp_path)
    assert rc == 0 and info["hidden"] == 40 and info["vocab"] == 77 and info["n_layers"] == 5     # 1 + 2 x 2 executions
    assert model_info(tmp_path, dtype="float32")[0] == 0
    cfg = good_cfg()
    del cfg["streams"], cfg["loop"], cfg["layers"][0]["mixer"]["mask"], cfg["layers"][0]["mixer"]["rot"]["scaling"]        # plain residual, no loop, causal, plain rotary
    write_cfg(tmp_path, cfg)
    rc, info = model_info(tmp_path)
    assert rc == 0 and info["n_layers"] == 3


def mutate(path, value):
    def f(cfg):
        node = cfg
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
    return f


@pytest.mark.parametrize("change", [
    mutate(["layers", 0, "type"], "sliding_attention"),
    mutate(["layers", 0, "mixer", "rot", "dims"], 10),                 # more rotated channels than rot_dim
    mutate(["layers", 0, "mixer", "q_rank"], 0),
    mutate(["layers", 0, "mixer", "mask", "size"], 0),
    mutate(["layers", 0, "mixer", "rot", "scaling", "factor"], 0.0),
    mutate(["layers", 1, "mixer", "kv_heads"], 3),                     # does not divide heads
    mutate(["layers", 1, "mixer", "vdim"], 7),                         # values turn in pairs
    mutate(["layers", 1, "mixer", "rot", "dims"], 5),                  # odd
    mutate(["layers", 1, "mixer", "rot", "dims"], 12),                 # more than the head holds
    mutate(["layers", 1, "mixer", "conv"], 0),
    mutate(["layers", 1, "mlp", "kind"], "moe"),
    mutate(["layers", 1, "mlp", "ff"], 0),
    mutate(["streams"], 9),
    mutate(["loop", "stop"], 7),
    mutate(["vocab"], 0),
], ids=lambda f: "")
def test_config_reader_refuses(tmp_path, change):
    cfg = good_cfg()
    change(cfg)
    write_cfg(tmp_path, cfg)
    assert model_info(tmp_path)[0] == 400


def test_oracle_mechanisms():
    cfg = good_cfg()
    W = G.random_weights(cfg, 1)
    toks = np.random.default_rng(0).integers(0, cfg["vocab"], 60).tolist()
    full = G.forward(cfg, W, toks)
    assert np.abs(G.forward(cfg, W, toks[:17]) - full[:17]).max() < 1e-9          # causal: a prefix sees nothing of what follows
    # rotation: both layouts are pure rotations of the first dims channels, position 0 unchanged, and sign = -1 undoes sign = +1
    x = np.random.default_rng(2).standard_normal((5, 2, 12))
    f, amp = G.frequencies(100.0, 8)
    pos = np.arange(5.0)
    for halves in (True, False):
        y = G.rotate(x, pos, f, amp, halves)
        assert np.allclose(y[0], x[0]) and np.allclose(y[..., 8:], x[..., 8:]) and np.allclose((y ** 2).sum(-1), (x ** 2).sum(-1))
        assert np.allclose(G.rotate(y, pos, f, amp, halves, sign=-1.0), x)
    a = 3.0 * 100.0 ** (-2.0 * 1 / 8)
    y = G.rotate(x, pos, f, amp, True)
    assert np.allclose(y[3, 0, 1], x[3, 0, 1] * np.cos(a) - x[3, 0, 5] * np.sin(a)) and np.allclose(y[3, 0, 5], x[3, 0, 5] * np.cos(a) + x[3, 0, 1] * np.sin(a))
    y = G.rotate(x, pos, f, amp, False)
    assert np.allclose(y[3, 0, 2], x[3, 0, 2] * np.cos(a) - x[3, 0, 3] * np.sin(a)) and np.allclose(y[3, 0, 3], x[3, 0, 3] * np.cos(a) + x[3, 0, 2] * np.sin(a))
    # scaled frequencies: the fastest pairs keep their frequency, the slowest are divided by the factor, the amplitude grows with ln(factor)
    sc = {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}
    f0, _ = G.frequencies(100.0, 16)
    f1, amp1 = G.frequencies(100.0, 16, sc)
    assert np.isclose(f1[0], f0[0]) and np.isclose(f1[-1], f0[-1] / 4.0) and np.all(f1 <= f0 + 1e-15) and np.isclose(amp1, 0.1 * np.log(4.0) + 1.0)
    # the sink only enlarges the denominator: a very low sink is plain softmax, a very high one silences the head
    q, k, v = (np.random.default_rng(s).standard_normal((6, 4)) for s in (3, 4, 5))
    plain = G.sink_softmax_rows(q, k, v, 0.5, -1e9, None)
    assert np.allclose(plain[0], v[0]) and np.abs(G.sink_softmax_rows(q, k, v, 0.5, 50.0, None)).max() < 1e-12
    assert np.allclose(G.sink_softmax_rows(q, k, v, 0.5, -1e9, 1), v)              # a window of one sees itself only
    assert np.allclose(G.sink_softmax_rows(q, k, v, 0.5, -1e9, 3)[:3], plain[:3]) and not np.allclose(G.sink_softmax_rows(q, k, v, 0.5, -1e9, 3)[3:], plain[3:])
    # token shift: weight 0 keeps the row, weight 1 takes the previous row, zeros before the first
    h = np.random.default_rng(6).standard_normal((4, 3))
    assert np.allclose(G.token_shift(h, 0.0), h) and np.allclose(G.token_shift(h, 1.0)[1:], h[:-1]) and np.allclose(G.token_shift(h, 1.0)[0], 0.0)
    # convolution: the last tap weighs the current input
    u = np.random.default_rng(7).standard_normal((5, 2))
    assert np.allclose(G.short_conv(u, np.array([[0.0, 0.0, 1.0], [0.0, 1.0, 0.0]])), np.stack([u[:, 0], np.concatenate([[0.0], u[:-1, 1]])], 1))
    # several streams with in = 1 / n, mix = identity, out = 1 are the plain residual, summed n-fold... the sum of the streams grows by n y
    xs = np.stack([h, h])
    w = {"p.in": np.array([0.5, 0.5]), "p.mix": np.eye(2), "p.out": np.ones(2)}
    assert np.allclose(G.hyper_step(xs, w, "p.", lambda u: 2.0 * u).sum(0), 2 * h + 2 * 2.0 * h)
    assert abs(G.gelu_tanh(np.array([1.0]))[0] - 0.8411919906) < 1e-9
