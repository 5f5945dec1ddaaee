"""Throughput of the hybrid family beside the closest existing models (`bench.py --arch ratasun | zurevik | rofizen | gosavik`): Ratasun beside the
Llama-family model of equal width, depth and active feed-forward size; Zurevik and Rofizen beside the Ratasun model of equal width, depth and
experts (the closest design: routed experts in every layer; recurrent mixers with an fp32 state like Rofizen's) and beside that Llama-family model;
Gosavik (dense feed-forward, attention mixers only) beside the Llama-family model of equal width, depth and feed-forward size — the closest model as a whole —
and beside Ratasun, whose latent attention is the closest kernel to its own.  Random weights (seeded on load), synthetic token ids; prefill = real chunked prefill of batch x (ctx-1) tokens,
decode = steps of the whole batch, both timed with CUDA events inside the engine (oa_bench_decode).  With --breakdown the per-kernel-class
device times come from the engine's in-situ event timing (OA_PROFILE_ALL), one pass for prefill and one for decode."""
from __future__ import annotations

import json
import os
import tempfile


def sizes(name: str) -> dict:
    if name == "small":
        att = {"heads": 16, "dim": 64, "rot_dim": 32, "vdim": 64, "kv_rank": 256, "scale": 96 ** -0.5, "rot": {"base": 10000.0, "dims": 32}}
        dl = {"heads": 8, "kv_heads": 4, "dim": 64, "vdim": 128, "conv": 4}
        mb = {"heads": 16, "vdim": 64, "state": 64, "groups": 2, "norm_groups": 1, "conv": 4}
        moe = {"kind": "moe", "expert": {"ff": 512}, "router": {"experts": 16, "top": 4, "scale": 2.0, "groups": {"count": 4, "keep": 2}}}
        width, vocab = 1024, 32000
    else:
        att = {"heads": 16, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "scale": 192 ** -0.5, "rot": {"base": 10000.0, "dims": 64}}
        dl = {"heads": 16, "kv_heads": 8, "dim": 128, "vdim": 128, "conv": 4}
        mb = {"heads": 32, "vdim": 64, "state": 128, "groups": 4, "norm_groups": 1, "conv": 4}
        moe = {"kind": "moe", "expert": {"ff": 1024}, "router": {"experts": 32, "top": 4, "scale": 2.0, "groups": {"count": 4, "keep": 2}}}
        width, vocab = 2048, 32000
    layers = [{"type": t, "mixer": m, "mlp": moe} for t, m in (("latent_attention", att), ("channel_delta", dl), ("mamba2", mb), ("latent_attention", att))]
    cfg = {"architecture": "Ratasun", "width": width, "vocab": vocab, "norm": {"eps": 1e-6}, "logit_scale": 1.0, "layers": layers,
           "loop": {"start": 1, "stop": 3, "times": 2}}
    runs = 6
    ff_active = moe["router"]["top"] * moe["expert"]["ff"]
    hd = 64 if width == 1024 else 128
    llama = {"model": "custom", "hidden": width, "n_layers": runs, "n_heads": width // hd, "n_kv_heads": max(1, width // hd // 4), "head_dim": hd, "ffn": ff_active, "vocab": vocab}
    return {"hybrid": cfg, "llama": llama, "runs": runs}


def zurevik_sizes(name: str) -> dict:
    """Zurevik at the width, depth (6 layers), expert count and expert size of sizes(name): four differential layers (sliding window of 512 that keeps
    the first 8 tokens) and two sink layers (window 1024), the second reading the first one's keys and values."""
    if name == "small":
        diff = {"heads": 16, "kv_heads": 4, "dim": 32, "vdim": 64, "diff": 0.4, "scale": 32 ** -0.5, "mask": {"size": 512, "keep_first": 8}}
        sink = {"heads": 16, "kv_heads": 4, "dim": 64, "vdim": 64, "scale": 64 ** -0.5, "mask": {"size": 1024}}
        moe, width = {"kind": "moe", "expert": {"ff": 512}, "router": {"experts": 16, "top": 4}}, 1024
    else:
        diff = {"heads": 16, "kv_heads": 4, "dim": 64, "vdim": 128, "diff": 0.4, "scale": 64 ** -0.5, "mask": {"size": 512, "keep_first": 8}}
        sink = {"heads": 16, "kv_heads": 4, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "mask": {"size": 1024}}
        moe, width = {"kind": "moe", "expert": {"ff": 1024}, "router": {"experts": 32, "top": 4}}, 2048
    order = [("attention", diff), ("attention", diff), ("attention_2", sink), ("attention", diff), ("attention", diff), ("attention_2", dict(sink, kv_from=2))]
    return {"architecture": "Zurevik", "width": width, "vocab": 32000, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0}, "logit_softcap": 50.0,
            "layers": [{"type": t, "mixer": m, "mlp": moe} for t, m in order]}


def rofizen_sizes(name: str) -> dict:
    """Rofizen at the width, depth (6 layers) and active feed-forward size of sizes(name): gated linear attention, retention, attention beside a
    matrix memory, twice; the first layer's feed-forward is dense, the others choose 3 experts by table and add a gated shared expert."""
    if name == "small":
        heads, dim, vdim, width, ff, experts = 8, 64, 128, 1024, 512, 16
        left = {"heads": 16, "kv_heads": 4, "dim": 64, "vdim": 64, "scale": 64 ** -0.5}
    else:
        heads, dim, vdim, width, ff, experts = 16, 128, 128, 2048, 1024, 32
        left = {"heads": 16, "kv_heads": 4, "dim": 128, "vdim": 128, "scale": 128 ** -0.5}
    left.update(softcap=30.0, q_temp={"coef": 0.1, "every": 256})
    gla = {"heads": heads, "dim": dim, "vdim": vdim, "tau": 16.0}
    ret = {"heads": heads, "dim": dim, "vdim": vdim, "decay": [1.0 - 2.0 ** (-5 - 5 * h / heads) for h in range(heads)], "rot": {"base": 10000.0, "dims": dim}}
    par = {"left": left, "right": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": 15.0}}
    moe = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": 3}, "shared": {"ff": ff}}
    order = [("gla", gla, {"kind": "dense", "ff": 4 * ff}), ("retention", ret, moe), ("parallel", par, moe), ("gla", gla, moe), ("retention", ret, moe), ("parallel", par, moe)]
    return {"architecture": "Rofizen", "width": width, "vocab": 32000, "norm": {"eps": 1e-5}, "embedding": {"scale": width ** 0.5}, "postln_alpha": 2.0,
            "layers": [{"type": t, "mixer": m, "mlp": f} for t, m, f in order]}


def gosavik_sizes(name: str) -> dict:
    """Gosavik at the width and depth (6 layer executions: latent attention, then [attention, latent attention] twice with the same weights, then
    attention) of sizes(name), with a dense feed-forward of the Llama case's size, four residual streams, windows of 512 and YaRN-scaled rotary."""
    if name == "small":
        lat = {"heads": 16, "dim": 64, "rot_dim": 32, "vdim": 64, "kv_rank": 256, "q_rank": 384, "scale": 96 ** -0.5}
        att = {"heads": 16, "kv_heads": 4, "dim": 64, "vdim": 64, "conv": 4, "scale": 64 ** -0.5, "rot": {"base": 1000000.0, "dims": 64}}
        width, ff = 1024, 2048
    else:
        lat = {"heads": 16, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "q_rank": 768, "scale": 192 ** -0.5}
        att = {"heads": 16, "kv_heads": 4, "dim": 128, "vdim": 128, "conv": 4, "scale": 128 ** -0.5, "rot": {"base": 1000000.0, "dims": 128}}
        width, ff = 2048, 4096
    lat.update(mask={"size": 512}, rot={"base": 10000.0, "dims": lat["rot_dim"], "scaling": {"factor": 4.0, "original": 2048, "fast": 24.0, "slow": 2.0}})
    mlp = {"kind": "dense", "ff": ff}
    order = [("latent_attention", lat), ("attention", att), ("latent_attention", lat), ("attention", att)]
    return {"architecture": "Gosavik", "width": width, "vocab": 32000, "norm": {"eps": 1e-5}, "streams": 4, "loop": {"start": 1, "stop": 3, "times": 2},
            "layers": [{"type": t, "mixer": m, "mlp": mlp} for t, m in order]}


def one(engine_cfg: dict, batch: int, ctx: int, steps: int, warmup: int, breakdown: bool) -> dict:
    from .engine import Engine
    out = {}
    with Engine(engine_cfg) as eng:
        eng.bench_decode(min(batch, 4), min(ctx, 512), 2, 1)      # untimed: first launches load every kernel (lazy module loading) and raise shared-memory limits
        r = eng.bench_decode(batch, ctx, steps, warmup)
        out["prefill_tok_s"] = batch * (ctx - 1) / (r["prefill_ms"] / 1e3)
        out["prefill_ms"] = r["prefill_ms"]
        out["decode_tok_s"] = batch / (r["ms_per_step"] / 1e3)
        out["decode_ms_per_step"] = r["ms_per_step"]
        out["launches_per_step"] = r["launches_per_step"]
        out["weight_bytes"] = eng.stats()["weight_bytes"]
        if breakdown:
            os.environ["OA_PROFILE_ALL"] = "1"
            eng.kernel_times(reset=True)
            eng.bench_decode(batch, ctx, 4, 1)
            out["decode_kernel_ms"] = {k: round(v[0] / 4, 4) for k, v in eng.kernel_times(reset=True).items() if v[1]}
            os.environ["OA_PROFILE_PREFILL"] = "1"
            eng.bench_decode(batch, ctx, 1, 0)
            out["prefill_kernel_ms"] = {k: round(v[0], 3) for k, v in eng.kernel_times(reset=True).items() if v[1]}
            del os.environ["OA_PROFILE_PREFILL"], os.environ["OA_PROFILE_ALL"]
    return out


def run(args) -> None:
    zu = args.arch in ("zurevik", "rofizen", "gosavik")
    res = {"metric": args.arch + "_vs_ratasun_and_llama_throughput" if zu else "hybrid_vs_llama_throughput", "unit": "tokens/s", "data": "synthetic", "dtype": "bf16", "cases": []}
    for name in args.arch_sizes.split(","):
        sz = sizes(name)
        batch, ctx = args.arch_batch, args.arch_ctx
        pages = batch * ((ctx + args.steps + args.warmup + 64) // 64 + 1)
        common = {"num_pages": pages, "max_batch": batch, "max_seq_len": (ctx + args.steps + args.warmup + 127) // 64 * 64, "max_step_tokens": 8192, "prefix_cache": 0}

        def folder_model(cfg):
            with tempfile.TemporaryDirectory() as d:
                with open(os.path.join(d, "config.json"), "w") as f:
                    json.dump(cfg, f)
                return one(dict(common, model_dir=d, **json.loads(args.engine_extra)), batch, ctx, args.steps, args.warmup, args.breakdown)
        case = {"size": name, "batch": batch, "ctx": ctx, "layer_runs": sz["runs"]}
        if zu:
            case[args.arch] = folder_model({"zurevik": zurevik_sizes, "rofizen": rofizen_sizes, "gosavik": gosavik_sizes}[args.arch](name))
        case["ratasun"] = hy = folder_model(sz["hybrid"])
        case["llama_equal_size"] = ll = one(dict(common, **sz["llama"]), batch, ctx, args.steps, args.warmup, args.breakdown)
        new = case[args.arch] if zu else hy
        case["prefill_ratio"], case["decode_ratio"] = new["prefill_tok_s"] / ll["prefill_tok_s"], new["decode_tok_s"] / ll["decode_tok_s"]
        if zu:
            case["prefill_ratio_to_ratasun"], case["decode_ratio_to_ratasun"] = new["prefill_tok_s"] / hy["prefill_tok_s"], new["decode_tok_s"] / hy["decode_tok_s"]
        res["cases"].append(case)
    print(json.dumps(res))
