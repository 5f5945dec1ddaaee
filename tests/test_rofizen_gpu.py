"""The Rofizen design of the hybrid family on the GPU against the slow float64 oracle (tests/rofizen_oracle.py): each mechanism alone, and —
through Engine.trace_step, which drives the scheduler's own batch builder, pages and state slots — prompts cut into portions, token-by-token
decoding, mixed batches, pages and slots that are used again, far tokens that decide, the first tokens of a sequence, the steps of the query
temperature, and greedy generation through the scheduler.  Small random checkpoints are written per test."""
import numpy as np
import pytest

import rofizen_oracle as R

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4          # fp32 engine against the float64 oracle (relative to the logits' spread)
BF16_TOL = 0.12         # bf16 matrices / activations: 90 % of the rows; the median is held to a quarter of it
SAME_TOL = 2e-5         # fp32 engine, two schedules of the same tokens


def engine(folder, dtype="float32", pages=8, slots=4, **kw):
    from opsagent_b200 import Engine
    return Engine(dict({"model_dir": str(folder), "dtype": dtype, "num_pages": pages, "max_seq_len": 64 * pages, "max_step_tokens": 64 * pages,
                        "max_batch": slots, "prefix_cache": 0}, **kw))


def checkpoint(tmp_path, cfg, seed=0, sharp=0.0, spread=1.0):
    W = R.random_weights(cfg, seed, spread)
    if sharp:
        R.sharpen(W, sharp)
    R.write_checkpoint(str(tmp_path), cfg, W)
    return W


def tokens_of(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


def replay(eng, rid, toks, cuts):
    """feed toks to request rid in portions of the given sizes (the rest one by one), wanting every position; -> logits [len(toks), vocab]"""
    out, at = [], 0
    sizes = list(cuts)
    while at < len(toks):
        n = min(sizes.pop(0) if sizes else 1, len(toks) - at)
        out.append(eng.trace_step([(rid, toks[at:at + n], list(range(n)))], [rid] if at + n == len(toks) else []))
        at += n
    return np.concatenate(out)


def check(got, want, dtype):
    e = R.rel_err(got.astype(np.float64), want)
    if dtype == "float32":
        assert e.max() < F32_TOL, f"worst row {e.argmax()} differs by {e.max():.3e}"
    else:
        assert np.quantile(e, 0.9) < BF16_TOL and np.median(e) < BF16_TOL / 4, f"bf16 rows differ: median {np.median(e):.3e}, 90% {np.quantile(e, 0.9):.3e}"


SINGLE = {
    "gla": [R.gla_layer()],
    "gla_one_head_tau_one_rank_one": [R.gla_layer(heads=1, dim=20, vdim=4, tau=1.0, rank=1)],
    "gla_rows_split_over_warps": [R.gla_layer(heads=2, dim=64, vdim=36, tau=9.0, rank=8)],
    "gla_sizes_off_every_vector": [R.gla_layer(heads=3, dim=6, vdim=7, tau=2.5, rank=3)],
    "retention": [R.retention_layer()],
    "retention_whole_head_rotated": [R.retention_layer(heads=2, dim=16, vdim=16, rot_dims=16, rot_base=77.0)],
    "retention_nothing_rotated_odd_sizes": [R.retention_layer(heads=5, dim=7, vdim=5, rot_dims=0)],
    "retention_wide_state": [R.retention_layer(heads=2, dim=128, vdim=40, rot_dims=32, decay=[0.9, 0.999])],
    "attention_beside_memory": [R.parallel_layer()],
    "attention_beside_memory_equal_heads": [R.parallel_layer(heads=3, kv_heads=3, dim=16, vdim=16, every=1, coef=0.2, softcap=30.0, r_heads=2, r_dim=16, r_vdim=32, gate_cap=3.0)],
    "attention_beside_memory_one_kv_head": [R.parallel_layer(heads=6, kv_heads=1, dim=5, vdim=9, every=64, scale=1.1, r_heads=1, r_dim=6, r_vdim=7, gate_cap=20.0)],
    "memory_rows_split_over_warps": [R.parallel_layer(heads=2, kv_heads=2, dim=32, vdim=64, r_heads=2, r_dim=48, r_vdim=64)],
    "dense": [R.gla_layer(mlp=R.dense(52))],
    "experts_and_shared": [R.retention_layer(mlp=R.moe())],
    "experts_top1_no_shared": [R.gla_layer(mlp=R.moe(experts=3, top=1, ff=10, shared_ff=0))],
    "experts_all_chosen_small_shared": [R.gla_layer(mlp=R.moe(experts=4, top=4, ff=40, shared_ff=9))],
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_each_mechanism_alone(tmp_path, name, dtype):
    cfg = R.make_config(SINGLE[name], width=38 if "off_every" in name else 36 if "odd" in name else 40)
    W = checkpoint(tmp_path, cfg, seed=len(name))
    toks = tokens_of(cfg, 70, 1)                       # crosses a page border
    want = R.forward(cfg, W, toks)
    with engine(tmp_path, dtype) as eng:
        check(replay(eng, 1, toks, [70]), want, dtype)           # whole prompt
        check(replay(eng, 2, toks, [1, 1, 2, 3, 57, 2]), want, dtype)   # the first tokens alone, short portions, then token by token


def stack_cfg(**kw):
    layers = [R.parallel_layer(mlp=R.moe()), R.gla_layer(mlp=R.dense()), R.retention_layer(mlp=R.moe(experts=5, top=3, ff=20, shared_ff=0)), R.gla_layer(heads=2, dim=16, vdim=16, mlp=None),
              R.parallel_layer(heads=2, kv_heads=1, dim=16, vdim=8, every=64, r_heads=4, r_dim=4, r_vdim=12, mlp=R.dense(24)), R.retention_layer(heads=2, dim=8, vdim=24, rot_dims=4, mlp=R.moe(top=1))]
    return R.make_config(layers, **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_and_decoding_match_the_whole_prompt(tmp_path, dtype):
    cfg = stack_cfg()
    W = checkpoint(tmp_path, cfg, seed=3)
    toks = tokens_of(cfg, 140, 2)
    want = R.forward(cfg, W, toks)
    with engine(tmp_path, dtype) as eng:
        outs = [replay(eng, 7, toks, cuts) for cuts in ([140], [2, 62, 1, 2, 61, 12], [63, 2, 64], [5], [127, 1, 1, 11], [64, 64, 2, 2, 2, 2, 2, 2])]
    for got in outs:
        check(got, want, dtype)
        if dtype == "float32":
            assert R.rel_err(got.astype(np.float64), outs[0].astype(np.float64)).max() < SAME_TOL


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_requests_in_one_batch_and_reused_pages_and_slots(tmp_path, dtype):
    """Requests at different stages share every step (a prompt portion beside single tokens); later requests take over the pages and the state
    slots of finished ones: a stale cache row, a state that was not started from zero or a wrong block table would show."""
    cfg = stack_cfg()
    W = checkpoint(tmp_path, cfg, seed=5)
    lens = {1: 100, 2: 37, 3: 66, 4: 90, 5: 20}
    toks = {r: tokens_of(cfg, n, 20 + r) for r, n in lens.items()}
    want = {r: R.forward(cfg, W, toks[r]) for r in lens}
    got = {r: [] for r in lens}
    at = {r: 0 for r in lens}
    with engine(tmp_path, dtype, pages=4, slots=2) as eng:
        def step(parts):
            entries, end = [], []
            for r, n in parts:
                n = min(n, lens[r] - at[r])
                entries.append((r, toks[r][at[r]:at[r] + n], list(range(n))))
                at[r] += n
                if at[r] == lens[r]:
                    end.append(r)
            out = eng.trace_step(entries, end)
            k = 0
            for r, t, w in entries:
                got[r].append(out[k:k + len(w)])
                k += len(w)
        step([(1, 60)])
        step([(1, 1), (2, 30)])                       # 1 decodes beside a portion of 2
        step([(1, 3), (2, 7)])                        # 2 ends: its page and slot are free
        step([(1, 36), (5, 2)])                       # 1 ends, 5 starts on 2's page and slot
        step([(5, 18), (3, 64)])                      # 5 ends; 3 fills exactly one page, in 1's slot
        step([(3, 2), (4, 2)])                        # 3 ends on a page's second token; 4 starts
        while at[4] < lens[4]:
            step([(4, 29)])
        assert eng.stats()["pages_free"] == 4
        for r in lens:                                # each alone, whole, in the same engine
            alone = replay(eng, 10 + r, toks[r], [lens[r]])
            assert R.rel_err(np.concatenate(got[r]).astype(np.float64), alone.astype(np.float64)).max() < (SAME_TOL if dtype == "float32" else 3e-2)
    for r in lens:
        check(np.concatenate(got[r]), want[r], dtype)


def far_cfg(every=50):
    # slow decays, a query temperature that steps inside a page, a memory whose input gate singles tokens out
    layers = [R.parallel_layer(heads=2, kv_heads=1, dim=16, vdim=16, scale=0.5, softcap=40.0, coef=0.8, every=every, r_heads=2, r_dim=16, r_vdim=16, gate_cap=12.0),
              R.retention_layer(heads=2, dim=16, vdim=16, rot_dims=8, decay=[0.998, 0.9995]), R.gla_layer(heads=2, dim=16, vdim=16, tau=64.0, rank=4, mlp=R.moe())]
    return R.make_config(layers, width=48, vocab=64)


def test_far_tokens_decide_through_pages_state_and_decoding(tmp_path):
    """Sharp queries and slow decays: what the first page held decides the last rows (the oracle without it answers differently there) — through
    the attention side's cache on other pages, and through the states.  The query temperature steps every 50 positions: a step one position
    early or late shows in the oracle.  The engine agrees with the oracle whole, in portions cut around page borders and temperature steps, and
    decoding over them."""
    cfg = far_cfg()
    W = checkpoint(tmp_path, cfg, seed=9, sharp=5.0)
    toks = tokens_of(cfg, 460, 5)
    want = R.forward(cfg, W, toks)
    assert R.rel_err(R.forward(cfg, W, toks[64:])[-40:], want[-40:]).max() > 50 * F32_TOL
    for every in (49, 51):
        assert (R.rel_err(R.forward(far_cfg(every), W, toks), want) > 20 * F32_TOL).sum() > 10, "the temperature's step does not show in the oracle"
    with engine(tmp_path, pages=8) as eng:
        check(replay(eng, 1, toks, [460]), want, "float32")
        check(replay(eng, 2, toks, [48, 2, 13, 1, 63, 2, 20, 1, 99, 2, 132]), want, "float32")      # portions that start and end around 49 / 50, 64, 128, 149 / 150, 249 / 250; then decoding over 384, 399 / 400, 448, 449 / 450
    with engine(tmp_path, "bfloat16", pages=8) as eng:
        for cuts in ([460], [48, 2, 13, 1, 63, 2, 20, 1, 99, 2, 132]):
            e = R.rel_err(replay(eng, 1, toks, cuts).astype(np.float64), want)
            assert np.quantile(e, 0.95) < 0.15 and e.max() < 0.5, f"bf16, cuts {cuts}: 95% {np.quantile(e, 0.95):.3e}, worst {e.max():.3e}"


def test_first_tokens_and_running_maximum_start(tmp_path):
    """The matrix memory's running maximum starts at 0, not at the first input gate: with strongly negative input gates the first rows differ
    between the two readings (exp(-m) floors the denominator), and a slot that another request used before must start from 0 again."""
    cfg = R.make_config([R.parallel_layer(r_heads=2, r_dim=8, r_vdim=8, gate_cap=14.0)], width=40, vocab=50)
    W = R.random_weights(cfg, 4)
    W["l0.mix.right.i.b"] = R.bf16_round(np.full(2, -9.0))
    R.write_checkpoint(str(tmp_path), cfg, W)
    A, B = tokens_of(cfg, 30, 1), tokens_of(cfg, 9, 2)
    with engine(tmp_path, slots=1) as eng:
        check(replay(eng, 1, A, [30]), R.forward(cfg, W, A), "float32")
        check(replay(eng, 2, B, [1, 1, 2]), R.forward(cfg, W, B), "float32")          # the same slot, first tokens one by one
        check(replay(eng, 3, A, [2, 2]), R.forward(cfg, W, A), "float32")


def test_long_decoding(tmp_path):
    cfg = stack_cfg()
    W = checkpoint(tmp_path, cfg, seed=11)
    toks = tokens_of(cfg, 200, 7)
    with engine(tmp_path) as eng:
        check(replay(eng, 1, toks, [3]), R.forward(cfg, W, toks), "float32")     # 197 single-token steps over three page borders


TC_STACKS = {
    # head sizes that take the tensor-core attention kernels (dim a multiple of 16, vdim 16 / 32 / 64 / 96 / 128) and the register-resident recurrences
    "groups_of_two_and_96_value_channels": [R.parallel_layer(heads=4, kv_heads=2, dim=32, vdim=96, every=100, r_heads=2, r_dim=32, r_vdim=64, mlp=R.moe(experts=8, top=2, ff=64, shared_ff=32)),
                                            R.gla_layer(heads=2, dim=64, vdim=64, tau=16.0, rank=8, mlp=R.dense(128)),
                                            R.retention_layer(heads=4, dim=32, vdim=32, rot_dims=32, mlp=R.moe(experts=4, top=1, ff=48, shared_ff=80))],
    "large_group_and_wide_heads": [R.parallel_layer(heads=8, kv_heads=1, dim=128, vdim=64, scale=0.1, every=33, r_heads=2, r_dim=128, r_vdim=32),
                                   R.parallel_layer(heads=40, kv_heads=2, dim=16, vdim=16, every=7, r_heads=4, r_dim=16, r_vdim=16, mlp=R.dense(64))],
}


@pytest.mark.parametrize("name", sorted(TC_STACKS))
def test_bf16_tensor_core_path_and_plain_path_agree_with_the_oracle(tmp_path, name):
    """Prompts long enough for several query and key tiles and for the grouped expert products, whole, in portions that straddle tiles, and
    decoding, on the tensor-core kernels and on the plain kernels (hy_tensor_core = 0)."""
    cfg = R.make_config(TC_STACKS[name], width=64, vocab=96)
    W = checkpoint(tmp_path, cfg, seed=13, sharp=2.0)
    toks = tokens_of(cfg, 330, 8)
    want = R.forward(cfg, W, toks)
    for tc in (1, 0):
        with engine(tmp_path, "bfloat16", pages=6, hy_tensor_core=tc) as eng:
            for cuts in ([330], [17, 33, 63, 130, 41, 30], [300]):
                e = R.rel_err(replay(eng, 1, toks, cuts).astype(np.float64), want)
                assert np.quantile(e, 0.95) < 0.1 and e.max() < 0.3, f"tensor cores {tc}, cuts {cuts}: 95% {np.quantile(e, 0.95):.3e}, worst {e.max():.3e}"


def test_table_and_shared_gate_decide(tmp_path):
    """The experts come from the table row of the token id (another table answers differently), each weighs 1 / top, and the shared expert is
    scaled by its sigmoid gate (a gate row of zeros, i.e. one half for every token, answers differently)."""
    mlp = R.moe(experts=8, top=3, ff=16, shared_ff=24)
    cfg = R.make_config([R.gla_layer(mlp=mlp), R.retention_layer(mlp=mlp)], width=40, vocab=60)
    W = checkpoint(tmp_path, cfg, seed=23)
    toks = tokens_of(cfg, 70, 3)
    want = R.forward(cfg, W, toks)
    other = dict(W)
    other["l0.mlp.table"] = (W["l0.mlp.table"] + 1) % 8
    assert R.rel_err(R.forward(cfg, other, toks), want).max() > 0.02
    flat = dict(W)
    flat["l1.mlp.shared.sg"] = np.zeros_like(W["l1.mlp.shared.sg"])
    assert R.rel_err(R.forward(cfg, flat, toks), want).max() > 0.01
    for dtype in ("float32", "bfloat16"):
        with engine(tmp_path, dtype) as eng:
            check(replay(eng, 1, toks, [70]), want, dtype)
            check(replay(eng, 2, toks, [33, 2, 30]), want, dtype)


def test_greedy_generation_through_the_scheduler(tmp_path):
    """oa_tokens_submit -> continuous batching -> greedy sampling: three requests on two sequence slots (one waits), each compared with the
    oracle's greedy continuation wherever the oracle's top-1 margin is not a near tie."""
    cfg = stack_cfg()
    W = checkpoint(tmp_path, cfg, seed=12)
    prompts = [tokens_of(cfg, n, 30 + n) for n in (9, 70, 33)]
    n_new = 12
    with engine(tmp_path, pages=6, slots=2) as eng:
        tickets = [eng.tokens_submit(p, n_new, flags=1) for p in prompts]
        outs = [eng.wait(t).token_ids for t in tickets]
        assert eng.stats()["pages_free"] == 6
    for p, out in zip(prompts, outs):
        seq = list(p)
        assert len(out) == n_new
        for tok in out:
            lg = R.forward(cfg, W, seq)[-1]
            top2 = np.sort(lg)[-2:]
            if int(np.argmax(lg)) != tok:
                assert top2[1] - top2[0] < 1e-3, "greedy token differs from the oracle's outside a near tie"
                break
            seq.append(tok)
