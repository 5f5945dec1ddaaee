"""The Gosavik design of the hybrid family on the GPU against the slow float64 oracle (tests/gosavik_oracle.py): each mechanism alone, and —
through Engine.trace_step, which drives the scheduler's own batch builder, pages and state slots — prompts cut into portions, token-by-token
decoding, mixed batches, pages and slots that are used again, window edges, far keys, the sink, the first tokens of a sequence, long
decoding, the tensor-core kernels against the plain ones, and greedy generation through the scheduler.  Small random checkpoints are
written per test."""
import numpy as np
import pytest

import gosavik_oracle as G

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4          # fp32 engine against the float64 oracle (relative to the logits' spread)
BF16_TOL = 0.12         # bf16 matrices / activations: 90 % of the rows; the median is held to a quarter of it
SAME_TOL = 2e-5         # fp32 engine, two schedules of the same tokens


def engine(folder, dtype="float32", pages=8, slots=4, **kw):
    from opsagent_b200 import Engine
    return Engine(dict({"model_dir": str(folder), "dtype": dtype, "num_pages": pages, "max_seq_len": 64 * pages, "max_step_tokens": 64 * pages,
                        "max_batch": slots, "prefix_cache": 0}, **kw))


def checkpoint(tmp_path, cfg, seed=0, sharp=0.0):
    W = G.random_weights(cfg, seed)
    if sharp:
        sharpen(W, sharp)
    G.write_checkpoint(str(tmp_path), cfg, W)
    return W


def sharpen(w, factor):
    """queries that single out keys: the query projections (and their biases) grow by `factor`"""
    for name in w:
        if name.endswith("mix.uq") or name.endswith("mix.q") or name.endswith("mix.q.b"):
            w[name] = G.bf16(w[name] * factor)
    return w


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
    e = G.rel_err(got.astype(np.float64), want)
    if dtype == "float32":
        assert e.max() < F32_TOL, f"worst row {e.argmax()} differs by {e.max():.3e}"
    else:
        assert np.quantile(e, 0.9) < BF16_TOL and np.median(e) < BF16_TOL / 4, f"bf16 rows differ: median {np.median(e):.3e}, 90% {np.quantile(e, 0.9):.3e}"


SINGLE = {
    # (layers, streams)
    "latent": ([G.latent_layer()], 2),
    "latent_window_of_one": ([G.latent_layer(window=1)], 2),
    "latent_window_beyond_the_prompt_no_scaling": ([G.latent_layer(window=500, scaling=False)], 3),
    "latent_no_mask_one_head_odd_sizes": ([G.latent_layer(heads=1, dim=6, rot_dim=10, vdim=5, kv_rank=9, q_rank=7, window=None, scale=0.7)], 1),
    "latent_wide_rotated_part_ramp_inside": ([G.latent_layer(heads=2, dim=4, rot_dim=32, vdim=12, kv_rank=24, q_rank=40, window=33, base=10000.0,
                                                            scaling={"factor": 16.0, "original": 64, "fast": 16.0, "slow": 2.0})], 4),
    "attention": ([G.attention_layer()], 2),
    "attention_equal_heads_two_taps_part_rotated": ([G.attention_layer(heads=3, kv_heads=3, dim=12, vdim=6, conv=2, rot_dims=4, scale=0.4)], 0),
    "attention_one_kv_head_one_tap_nothing_rotated": ([G.attention_layer(heads=6, kv_heads=1, dim=5, vdim=10, conv=1, rot_dims=0)], 1),
    "attention_five_taps_wide_values": ([G.attention_layer(heads=2, kv_heads=2, dim=16, vdim=40, conv=5, base=50.0)], 3),
    "no_feed_forward": ([G.latent_layer(mlp=None), G.attention_layer(mlp=None)], 2),
    "plain_residual": ([G.latent_layer(), G.attention_layer()], 0),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_each_mechanism_alone(tmp_path, name, dtype):
    layers, streams = SINGLE[name]
    cfg = G.make_config(layers, width=38 if "odd" in name else 40, streams=streams, eps=1e-6 if "odd" in name else 1e-5)
    W = checkpoint(tmp_path, cfg, seed=len(name))
    toks = tokens_of(cfg, 70, 1)                       # crosses a page border
    want = G.forward(cfg, W, toks)
    with engine(tmp_path, dtype) as eng:
        check(replay(eng, 1, toks, [70]), want, dtype)           # whole prompt
        check(replay(eng, 2, toks, [1, 1, 2, 3, 57, 2]), want, dtype)   # the first tokens alone, short portions, then token by token


def stack_cfg(**kw):
    layers = [G.latent_layer(window=11), G.attention_layer(), G.attention_layer(heads=2, kv_heads=1, dim=16, vdim=8, conv=4, rot_dims=8, mlp=None),
              G.latent_layer(heads=2, dim=16, rot_dim=4, vdim=12, kv_rank=20, q_rank=9, window=70, scaling=False, mlp=24), G.attention_layer(heads=6, kv_heads=3, dim=4, vdim=6, conv=2)]
    return G.make_config(layers, **dict({"streams": 3, "loop": {"start": 1, "stop": 4, "times": 3}}, **kw))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_and_decoding_match_the_whole_prompt(tmp_path, dtype):
    cfg = stack_cfg()
    W = checkpoint(tmp_path, cfg, seed=3)
    toks = tokens_of(cfg, 140, 2)
    want = G.forward(cfg, W, toks)
    with engine(tmp_path, dtype) as eng:
        outs = [replay(eng, 7, toks, cuts) for cuts in ([140], [2, 62, 1, 2, 61, 12], [63, 2, 64], [5], [127, 1, 1, 11], [64, 64, 2, 2, 2, 2, 2, 2])]
    for got in outs:
        check(got, want, dtype)
        if dtype == "float32":
            assert G.rel_err(got.astype(np.float64), outs[0].astype(np.float64)).max() < SAME_TOL


def test_loop_runs_its_layers_with_a_state_per_pass(tmp_path):
    """the looped block repeats with the same weights; every pass has its own cache, convolution tails and shifted row: decoding through a
    model whose passes shared any of them would differ from the oracle"""
    cfg = stack_cfg(loop={"start": 0, "stop": 2, "times": 2}, streams=2)
    W = checkpoint(tmp_path, cfg, seed=4)
    toks = tokens_of(cfg, 40, 3)
    assert G.schedule(cfg) == [0, 1, 0, 1, 2, 3, 4]
    with engine(tmp_path) as eng:
        check(replay(eng, 1, toks, [7, 2]), G.forward(cfg, W, toks), "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_requests_in_one_batch_and_reused_pages_and_slots(tmp_path, dtype):
    """Requests at different stages share every step (a prompt portion beside single tokens); later requests take over the pages and the state
    slots of finished ones: a stale cache row, a shifted row or a convolution tail that was not started from zero, or a wrong block table would show."""
    cfg = stack_cfg()
    W = checkpoint(tmp_path, cfg, seed=5)
    lens = {1: 100, 2: 37, 3: 66, 4: 90, 5: 20}
    toks = {r: tokens_of(cfg, n, 20 + r) for r, n in lens.items()}
    want = {r: G.forward(cfg, W, toks[r]) for r in lens}
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
            assert G.rel_err(np.concatenate(got[r]).astype(np.float64), alone.astype(np.float64)).max() < (SAME_TOL if dtype == "float32" else 3e-2)
    for r in lens:
        check(np.concatenate(got[r]), want[r], dtype)


def edge_cfg(window=70, conv=3, streams=2):
    layers = [G.latent_layer(heads=2, dim=8, rot_dim=8, vdim=8, kv_rank=16, q_rank=12, window=window, scale=1.0),
              G.attention_layer(heads=2, kv_heads=1, dim=16, vdim=16, conv=conv, scale=0.8)]
    return G.make_config(layers, width=48, vocab=64, streams=streams)


def test_window_edges_and_far_keys_decide(tmp_path):
    """Sharp queries: single keys carry the rows.  The oracle itself shows what each mechanism is worth — a window one token longer or shorter,
    a prompt without its first page (the causal layer reads hundreds of tokens back) — and
    the engine agrees with the right reading whole, in portions cut around the window's edge and page borders, and decoding over them."""
    cfg = edge_cfg()
    W = checkpoint(tmp_path, cfg, seed=9, sharp=6.0)
    toks = tokens_of(cfg, 300, 5)
    want = G.forward(cfg, W, toks)
    for w in (69, 71):
        assert (G.rel_err(G.forward(edge_cfg(window=w), W, toks), want)[70:] > 20 * F32_TOL).sum() > 20, "the window's edge does not show in the oracle"
    assert G.rel_err(G.forward(cfg, W, toks[64:])[-40:], want[-40:]).max() > 50 * F32_TOL, "far keys do not show in the oracle"
    cuts = [68, 2, 1, 1, 56, 2, 61, 2, 63, 40]           # portions that start and end around 69 / 70 / 71, 128, 192, 256; then decoding
    with engine(tmp_path, pages=6) as eng:
        check(replay(eng, 1, toks, [300]), want, "float32")
        check(replay(eng, 2, toks, cuts), want, "float32")
        check(replay(eng, 3, toks, [60]), want, "float32")            # decoding from 60 on: the window's edge passes over decoded tokens
    with engine(tmp_path, "bfloat16", pages=6) as eng:
        for c in ([300], cuts, [60]):
            e = G.rel_err(replay(eng, 1, toks, c).astype(np.float64), want)
            assert np.quantile(e, 0.95) < 0.15 and e.max() < 0.5, f"bf16, cuts {c}: 95% {np.quantile(e, 0.95):.3e}, worst {e.max():.3e}"


def test_one_key_just_inside_and_just_outside_the_window(tmp_path):
    """One latent-attention layer, no feed-forward, no token shift, no rotated key part: a row's scores depend on the keys' tokens only.  The
    prompt repeats one token except for a single other token early on, chosen so that its key outscores the rest: while it is inside the
    window it owns the softmax, one position later it is gone.  The oracle with a window one shorter differs at exactly that row by more
    than the logits' spread; the engine agrees with the right window in a prompt, in portions that start and end on the edge, and decoded."""
    window, p0, n = 37, 9, 90

    def cfg_of(w):
        return G.make_config([G.latent_layer(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=8, q_rank=8, window=w, scale=1.0, mlp=None)], width=32, vocab=40, streams=2)
    cfg = cfg_of(window)
    W = G.random_weights(cfg, 21)
    W["l0.mix.dkv"][8:] = 0.0
    W["l0.shift"][:] = 0.0
    W["l0.mix.uq"] = G.bf16(W["l0.mix.uq"] * 4.0)
    G.write_checkpoint(str(tmp_path), cfg, W)
    edge = p0 + window - 1                              # the last row that still sees position p0
    best = None
    rng = np.random.default_rng(0)
    for _ in range(40):
        a, b = (int(v) for v in rng.integers(0, 40, 2))
        toks = [a] * n
        toks[p0] = b
        want = G.forward(cfg, W, toks)
        e = G.rel_err(G.forward(cfg_of(window - 1), W, toks), want)[edge]
        if a != b and (best is None or e > best[0]):
            best = (e, toks, want)
    assert best[0] > 0.5, "the window's edge does not show in the oracle"
    _, toks, want = best
    assert G.rel_err(want[edge + 1:edge + 2], want[edge:edge + 1])[0] > 0.5              # the row after the edge answers differently
    for dtype in ("float32", "bfloat16"):
        with engine(tmp_path, dtype) as eng:
            for cuts in ([n], [edge, 1, 1, 2], [edge - 1, 2, 2], [edge + 1, 2], [p0 + 2]):
                got = replay(eng, 1, toks, cuts)
                check(got, want, dtype)
                assert G.rel_err(got[edge - 1:edge + 2].astype(np.float64), want[edge - 1:edge + 2]).max() < (F32_TOL if dtype == "float32" else 0.1)


def test_the_sink_counts_once_and_unscaled(tmp_path):
    """Sinks between 1 and 3 beside moderate scores: leaving the sink out, multiplying it by the layer's scale or counting it twice each
    moves the oracle's rows by tens of the fp32 tolerance; the engine agrees with the right reading."""
    layers = [G.latent_layer(heads=2, dim=8, rot_dim=8, vdim=8, kv_rank=16, q_rank=12, window=70, scale=0.5), G.attention_layer(heads=2, kv_heads=1, dim=16, vdim=16, conv=3, scale=0.3)]
    cfg = G.make_config(layers, width=48, vocab=64, streams=2)
    W = G.random_weights(cfg, 17)
    rng = np.random.default_rng(1)
    sinks = [k for k in W if k.endswith("sink")]
    for k in sinks:
        W[k] = G.bf16(rng.uniform(1.0, 3.0, W[k].shape))
    G.write_checkpoint(str(tmp_path), cfg, W)
    toks = tokens_of(cfg, 80, 1)
    want = G.forward(cfg, W, toks)
    for wrong in (lambda s, sc: np.full_like(s, -60.0), lambda s, sc: s * sc, lambda s, sc: s + np.log(2.0)):
        V = dict(W)
        for i, k in enumerate(sinks):
            V[k] = wrong(W[k], cfg["layers"][i]["mixer"]["scale"])
        assert np.median(G.rel_err(G.forward(cfg, V, toks), want)) > 50 * F32_TOL
    for dtype in ("float32", "bfloat16"):
        with engine(tmp_path, dtype) as eng:
            check(replay(eng, 1, toks, [80]), want, dtype)
            check(replay(eng, 2, toks, [30, 2]), want, dtype)


def test_first_tokens_start_from_zero_on_a_reused_slot(tmp_path):
    """The token shift reads zeros before the first token and the convolutions zeros before the sequence: with shift weights near one the first
    rows depend on exactly that, and a slot that another request used before must start from zero again."""
    cfg = edge_cfg(window=5, conv=4, streams=1)
    W = G.random_weights(cfg, 4)
    for k in W:
        if k.endswith("shift"):
            W[k] = G.bf16(np.full_like(W[k], 0.9))
    G.write_checkpoint(str(tmp_path), cfg, W)
    A, B = tokens_of(cfg, 30, 1), tokens_of(cfg, 9, 2)
    with engine(tmp_path, slots=1) as eng:
        check(replay(eng, 1, A, [30]), G.forward(cfg, W, A), "float32")
        check(replay(eng, 2, B, [1, 1, 2]), G.forward(cfg, W, B), "float32")          # the same slot, first tokens one by one
        check(replay(eng, 3, A, [2, 2]), G.forward(cfg, W, A), "float32")


def test_long_decoding(tmp_path):
    cfg = stack_cfg()
    W = checkpoint(tmp_path, cfg, seed=11)
    toks = tokens_of(cfg, 200, 7)
    with engine(tmp_path) as eng:
        check(replay(eng, 1, toks, [3]), G.forward(cfg, W, toks), "float32")     # 197 single-token steps over three page borders


TC_STACKS = {
    # sizes that take the tensor-core attention kernels: latent rank a multiple of 64 with head sizes of the prefill form; key / value heads of 16 .. 128 channels
    "window_inside_a_tile_and_beyond": [G.latent_layer(heads=4, dim=32, rot_dim=16, vdim=32, kv_rank=64, q_rank=48, window=45, base=10000.0, mlp=96),
                                        G.attention_layer(heads=4, kv_heads=2, dim=32, vdim=32, conv=4, mlp=96),
                                        G.latent_layer(heads=2, dim=64, rot_dim=32, vdim=64, kv_rank=128, q_rank=32, window=600, scaling=False, mlp=None)],
    "large_group_and_wide_heads": [G.attention_layer(heads=8, kv_heads=1, dim=64, vdim=128, conv=3, rot_dims=32, scale=0.2, mlp=None),
                                   G.latent_layer(heads=8, dim=16, rot_dim=16, vdim=16, kv_rank=64, q_rank=24, window=130, mlp=64),
                                   G.attention_layer(heads=20, kv_heads=2, dim=16, vdim=16, conv=2)],
}


@pytest.mark.parametrize("name", sorted(TC_STACKS))
def test_bf16_tensor_core_path_and_plain_path_agree_with_the_oracle(tmp_path, name):
    """Prompts long enough for several query and key tiles, whole, in portions that straddle tiles and windows, and decoding (rows whose
    cache is read in parts included), on the tensor-core kernels and on the plain kernels (hy_tensor_core = 0)."""
    cfg = G.make_config(TC_STACKS[name], width=64, vocab=96, streams=2)
    W = checkpoint(tmp_path, cfg, seed=13, sharp=2.0)
    toks = tokens_of(cfg, 700, 8)
    want = G.forward(cfg, W, toks)
    for tc in (1, 0):
        with engine(tmp_path, "bfloat16", pages=12, hy_tensor_core=tc) as eng:
            for cuts in ([700], [17, 33, 63, 130, 41, 300, 100], [690]):
                e = G.rel_err(replay(eng, 1, toks, cuts).astype(np.float64), want)
                assert np.quantile(e, 0.95) < 0.1 and e.max() < 0.3, f"tensor cores {tc}, cuts {cuts}: 95% {np.quantile(e, 0.95):.3e}, worst {e.max():.3e}"


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
            lg = G.forward(cfg, W, seq)[-1]
            top2 = np.sort(lg)[-2:]
            if int(np.argmax(lg)) != tok:
                assert top2[1] - top2[0] < 1e-3, "greedy token differs from the oracle's outside a near tie"
                break
            seq.append(tok)
