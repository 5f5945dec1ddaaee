"""Host side of the Rofizen design (no GPU): the configuration reader accepts what the design allows and refuses the rest with a client
error, and the float64 oracle the GPU tests lean on behaves as its mechanisms claim."""
import ctypes as C
import json
import os

import numpy as np
import pytest

import rofizen_oracle as R
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
    return R.make_config([R.parallel_layer(mlp=R.moe()), R.gla_layer(mlp=R.dense()), R.retention_layer(mlp=R.moe(experts=4, top=4, shared_ff=0)), R.gla_layer(mlp=None)], width=40, vocab=77)


def test_config_reader_accepts_the_design(tmp_path):
    write_cfg(tmp_path, good_cfg())
    rc, info = model_info(tmp_path)
    assert rc == 0 and info["hidden"] == 40 and info["vocab"] == 77 and info["n_layers"] == 4
    assert model_info(tmp_path, dtype="float32")[0] == 0
    cfg = good_cfg()                                       # nothing rotated; one head everywhere
    cfg["layers"][2]["mixer"]["rot"]["dims"] = 0
    cfg["layers"][1]["mixer"].update(heads=1)
    write_cfg(tmp_path / "b", cfg)
    assert model_info(tmp_path / "b")[0] == 0


def mutate(path, value):
    def f(cfg):
        node = cfg
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
    return f


def drop(path):
    def f(cfg):
        node = cfg
        for k in path[:-1]:
            node = node[k]
        del node[path[-1]]
    return f


@pytest.mark.parametrize("change", [
    mutate(["layers", 0, "type"], "serial"),
    mutate(["layers", 0, "mixer", "left", "kv_heads"], 3),             # does not divide heads
    mutate(["layers", 0, "mixer", "left", "vdim"], 300),               # beyond what the kernels hold
    mutate(["layers", 0, "mixer", "left", "softcap"], -2.0),
    mutate(["layers", 0, "mixer", "left", "q_temp", "every"], 0),
    mutate(["layers", 0, "mixer", "right", "gate_cap"], -1.0),
    mutate(["layers", 1, "mixer", "tau"], 0.0),
    mutate(["layers", 2, "mixer", "decay"], [0.5]),                    # one number per head
    mutate(["layers", 2, "mixer", "rot", "dims"], 7),                  # odd
    mutate(["layers", 2, "mixer", "rot", "dims"], 14),                 # more than the head holds
    mutate(["layers", 2, "mlp", "router", "top"], 5),                  # more choices than experts
    mutate(["layers", 0, "mlp", "shared", "ff"], 0),
    mutate(["layers", 1, "mlp", "ff"], 0),
    mutate(["layers", 1, "mlp", "kind"], "sparse"),
    drop(["postln_alpha"]),
    mutate(["vocab"], 0),
], ids=lambda f: "")
def test_config_reader_refuses(tmp_path, change):
    cfg = good_cfg()
    change(cfg)
    write_cfg(tmp_path, cfg)
    assert model_info(tmp_path)[0] == 400


def test_oracle_mechanisms():
    cfg = good_cfg()
    W = R.random_weights(cfg, 1)
    toks = np.random.default_rng(0).integers(0, cfg["vocab"], 60).tolist()
    full = R.forward(cfg, W, toks)
    assert np.abs(R.forward(cfg, W, toks[:17]) - full[:17]).max() < 1e-9          # causal: a prefix sees nothing of what follows
    assert all(len(set(r)) == len(r) for r in W["l0.mlp.table"].tolist())          # the entries of a table row differ
    # rotation: pairs (i, i + dims / 2), untouched beyond dims, a pure rotation (norms kept), position 0 unchanged
    x = np.random.default_rng(2).standard_normal((5, 2, 12))
    y = R.rotate_half(x, np.arange(5.0), 100.0, 8)
    assert np.allclose(y[0], x[0]) and np.allclose(y[..., 8:], x[..., 8:]) and np.allclose((y ** 2).sum(-1), (x ** 2).sum(-1))
    a = 3.0 * 100.0 ** (-2.0 * 1 / 8)
    assert np.allclose(y[3, 0, 1], x[3, 0, 1] * np.cos(a) - x[3, 0, 5] * np.sin(a)) and np.allclose(y[3, 0, 5], x[3, 0, 5] * np.cos(a) + x[3, 0, 1] * np.sin(a))
    # the matrix memory does not depend on the stabiliser where the floor of the denominator is out of reach: shifting both log gates' maxima by
    # starting the running maximum elsewhere would only rescale numerator and denominator alike; and the layer norm takes its mean off
    assert abs(R.layer_norm(np.arange(6.0)[None], np.ones(6), 1e-5).mean()) < 1e-12
    h = np.random.default_rng(3).standard_normal((9, 40))
    left = R.softmax_branch(h, W, "l0.mix.left.", cfg["layers"][0]["mixer"]["left"], 1e-5)
    assert left.shape == (9, 40) and np.isfinite(left).all()
