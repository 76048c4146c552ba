"""Sebavik on the GPU against the plain fp64 restatement (oracle/sebavik_plain.py): each mechanism alone, constants that
must matter (cap, distance bias, sink, blend factor, clamp, convolution, pair table, token input, depth weights), prefill
against token-by-token decoding, portions, unequal batches, reuse of pages and slots, a marked key far back, at page
borders and just inside / just outside the window and the kept first tokens (in prompts, in decoding, in portions, on the
SIMT and the tensor-core attention), the first tokens of a sequence, long decoding, other sizes, and greedy generation
through LLM.generate, the generate command line and the trace replay."""
import copy

import numpy as np
import pytest
import torch

from oracle import sebavik_plain as plain
from tests.sebavik_helpers import (SMALL, TOL, Harness, attn, close, dense, model_config, moe, near_ties, needle_model,
                                   needle_tokens, oracle_logits, rand_tokens, rel_err, row_errs, run)

pytestmark = pytest.mark.gpu


# ---- each mechanism alone ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["attention", "dense", "experts", "bare", "blend"])
def test_mechanism_alone(which, dtype):
    tiny = dict(heads=1, kv_heads=1, dim=8, vdim=8, size=4, keep=0, v_mix=False)
    if which == "bare":          # no convolution, no pair table, no token input, no cap, no mask: the block's skeleton
        cfg = model_config([attn(size=None, cap=None, v_mix=False, mlp=None)], taps=0, side=0, buckets=0, mult=1.0)
    else:
        layers = {"attention": [attn(mlp=None)], "dense": [attn(mlp=dense(), **tiny)], "experts": [attn(mlp=moe(), **tiny)],
                  "blend": [attn(mlp=None, v_mix=False), attn(mlp=None), attn(mlp=None, v_mix=False), attn(mlp=None)]}[which]
        cfg = model_config(layers)
    toks = rand_tokens(45, cfg["vocab"], 3)
    got, want = run(cfg, toks, dtype)
    assert close(got, want, dtype)


@pytest.mark.parametrize("kw", [dict(experts=8, top=3), dict(experts=1, top=1), dict(experts=5, top=5, ff=8),
                                dict(experts=40, top=2, ff=9), dict(experts=12, top=3, ff=48)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_router_shapes(kw, dtype):
    """One expert, every expert chosen, more experts than a warp, expert sizes that the tensor-core product does not take
    and ones it takes; many tokens so that the expert-sorted path runs, few so that the per-pair one does.  The router's
    weights are made three times larger so that near ties between the last chosen and the first rejected expert are rare."""
    cfg = model_config([attn(heads=1, kv_heads=1, dim=8, vdim=8, mlp=moe(**kw)), attn(heads=2, kv_heads=1, dim=8, vdim=8, mlp=moe(**kw))])
    w = plain.random_weights(cfg, 0)
    for i in range(2):
        w[f"l{i}.mlp.router"] = (w[f"l{i}.mlp.router"].float() * 3.0).to(torch.bfloat16)
    toks = rand_tokens(80, cfg["vocab"], 4)
    got, want = run(cfg, toks, dtype, cuts=[60, 1, 7, 1], weights=w)
    assert close(got, want, dtype, near_ties(cfg, w, toks) if dtype == "bfloat16" else ())


def _edit(cfg, w, what):
    cfg, w = copy.deepcopy(cfg), dict(w)
    m0 = cfg["layers"][0]["mixer"]
    if what == "cap":
        m0["softcap"] = 60.0
    elif what == "bias strength":
        w["l0.mix.r1"] = w["l0.mix.r1"].float() * 0.0
    elif what == "bias reach":
        w["l0.mix.r2"] = w["l0.mix.r2"].float() * 3.0
    elif what == "sink":
        w["l0.mix.sink"] = w["l0.mix.sink"].float() - 30.0
    elif what == "blend":
        w["l1.mix.vmix"] = torch.tensor(0.0)
    elif what == "clamp":
        cfg["layers"][0]["mlp"]["limit"] = 30.0
    elif what == "convolution":
        w["l0.canon2"] = w["l0.canon2"].float() * 0.0
    elif what == "pair table":
        cfg["embedding"]["bigram"]["mul_prev"] += 1
    elif what == "token input":
        w["side.embed"] = w["side.embed"].float().roll(1, 1)
    elif what == "depth weights":
        w["l1.dwa"] = w["l1.dwa"].float().flip(0)
    elif what == "residual factor":
        cfg["residual_mult"] = 1.0
    elif what == "window":
        m0["mask"]["size"] += 1
    elif what == "kept tokens":
        m0["mask"]["keep_first"] -= 1
    elif what == "query bias":
        w["l0.mix.q.b"] = w["l0.mix.q.b"].float() * 0.0
    return cfg, w


@pytest.mark.parametrize("what", ["cap", "bias strength", "bias reach", "sink", "blend", "clamp", "convolution", "pair table",
                                  "token input", "depth weights", "residual factor", "window", "kept tokens", "query bias"])
def test_constant_matters_and_is_honoured(what):
    """Changing the constant changes the oracle's answer clearly, and the engine agrees with the unchanged oracle."""
    cfg = model_config([attn(scale=1.5, cap=4.0, size=9, keep=2, mlp=dense(48, 0.4)), attn(scale=1.5, cap=4.0, mlp=None)])
    w = plain.random_weights(cfg, 9)
    w["l0.mix.sink"] = torch.full((4,), 3.0)
    w["l0.mix.q.b"] = w["l0.mix.q.b"].float() * 4.0
    toks = rand_tokens(48, cfg["vocab"], 10)
    want = oracle_logits(cfg, w, toks)
    cfg2, w2 = _edit(cfg, w, what)
    assert rel_err(oracle_logits(cfg2, w2, toks)[20:], want[20:]) > 3e-3, "the oracle does not depend on it"
    got, _ = run(cfg, toks, "float32", cuts=[31, 2, 1], weights=w)
    assert rel_err(got, want) < TOL["float32"]


# ---- prefill == decode, portions -------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_equals_token_by_token(dtype):
    toks = rand_tokens(70, SMALL["vocab"], 5)
    whole, want = run(SMALL, toks, dtype)
    single, _ = run(SMALL, toks, dtype, cuts=[1])
    skip = near_ties(SMALL, plain.random_weights(SMALL, 0), toks) if dtype == "bfloat16" else ()
    assert close(whole, want, dtype, skip)
    assert close(single, want, dtype, skip)
    if dtype == "float32":
        assert close(single, whole)


@pytest.mark.parametrize("cuts", [[2], [3, 2, 7, 1, 16, 5], [17, 2, 2, 31], [33, 1]])
def test_portions(cuts):
    toks = rand_tokens(90, SMALL["vocab"], 7)
    got, want = run(SMALL, toks, "float32", cuts=cuts)
    assert close(got, want)


def test_step_larger_than_the_runner_capacity_is_cut():
    toks = rand_tokens(100, SMALL["vocab"], 8)
    got, want = run(SMALL, toks, "float32", max_step_tokens=32)
    assert close(got, want)


# ---- batches of unequal requests, reuse of pages and slots ------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_and_reuse(dtype):
    w = plain.random_weights(SMALL, 11)
    V = SMALL["vocab"]
    reqs = {"a": rand_tokens(50, V, 1), "b": rand_tokens(7, V, 2), "c": rand_tokens(33, V, 3), "d": rand_tokens(1, V, 4),
            "e": rand_tokens(41, V, 5), "f": rand_tokens(20, V, 6)}
    ref = {k: oracle_logits(SMALL, w, v) for k, v in reqs.items()}
    hz = Harness(SMALL, w, dtype=dtype, page_size=16, num_pages=9, slots=3)          # a, c, e cannot be live together
    got = {k: [] for k in reqs}
    at = {k: 0 for k in reqs}

    def step(parts):
        ent = []
        for k, n in parts:
            n = min(n, len(reqs[k]) - at[k])
            ent.append((k, reqs[k][at[k]:at[k] + n], range(n)))
        out = hz.step(ent)
        o = 0
        for k, t, _ in ent:
            got[k].append(out[o:o + len(t)])
            o += len(t)
            at[k] += len(t)
            if at[k] == len(reqs[k]):
                hz.end(k)
    try:
        step([("a", 20), ("b", 3), ("d", 1)])           # d ends: its slot and page are free again
        step([("a", 1), ("b", 2), ("c", 9)])
        step([("c", 24), ("a", 1), ("b", 2)])           # c and b end
        step([("a", 12), ("e", 2)])
        step([("e", 17), ("a", 1), ("f", 5)])
        while at["a"] < 50 or at["e"] < 41 or at["f"] < 20:
            step([(k, 1 if k != "f" else 4) for k in ("a", "e", "f") if at[k] < len(reqs[k])])
        assert len(hz.sched.block_manager.free_block_ids) == 9 and len(hz.sched.state_manager.free_slots) == 3
    finally:
        hz.close()
    for k in reqs:
        skip = near_ties(SMALL, w, reqs[k]) if dtype == "bfloat16" else ()
        assert close(np.concatenate(got[k], 0), ref[k], dtype, skip), k


def test_slot_and_pages_used_again_start_from_the_empty_state():
    """The slot's convolution tails and its previous token belong to the request before: a new request must not see them."""
    w = plain.random_weights(SMALL, 12)
    V = SMALL["vocab"]
    hz = Harness(SMALL, w, "float32", page_size=16, num_pages=4, slots=1)
    try:
        for i in range(3):
            toks = rand_tokens(40 + i, V, 20 + i)
            got = hz.feed("x", toks, cuts=[13, 1])
            hz.end("x")
            assert close(got, oracle_logits(SMALL, w, toks))
    finally:
        hz.close()


# ---- a key that must be found, or must not be: window, kept first tokens, page borders --------------------------------------------
N, SIZE, KEEP = 150, 24, 5
# asked from position 149: the window holds 126 .. 149, the first five tokens are kept, everything between is hidden
NEEDLES = [0, 1, 4, 5, 6, 15, 16, 31, 32, 63, 64, 124, 125, 126, 127, 148]


@pytest.mark.parametrize("needle_at", NEEDLES)
@pytest.mark.parametrize("how", ["prompt", "decode", "portions"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_marked_key_is_seen_exactly_where_the_mask_says(needle_at, how, dtype):
    cfg, w = needle_model(size=SIZE, keep=KEEP)
    toks, without = needle_tokens(N, needle_at)
    want = oracle_logits(cfg, w, toks)
    changed = rel_err(oracle_logits(cfg, w, without)[-1], want[-1])
    assert (changed > 0.3) if plain.sees(N - 1, needle_at, SIZE, KEEP) else (changed < 1e-9)     # it decides, or it is hidden
    cuts = {"prompt": [N], "decode": [N - 30, 1], "portions": [5, 2, 3, 17, 2, 6]}[how]
    hz = Harness(cfg, w, dtype, page_size=16, num_pages=12, slots=1)
    try:
        got = hz.feed("n", toks, cuts=cuts)
    finally:
        hz.close()
    tol = TOL["float32"] if dtype == "float32" else 4e-2
    assert rel_err(got[-1], want[-1]) < tol
    assert rel_err(got, want) < tol


@pytest.mark.parametrize("size,keep", [(1, 0), (1, 3), (5, 0), (16, 16), (17, 40), (64, 1), (40, 70), (None, 0)])
def test_windows_and_kept_tokens_of_other_shapes(size, keep):
    """A window of one token, no kept tokens, both equal to the page, more kept tokens than the window holds, a window of one
    key tile, kept tokens beyond one key tile, no mask at all; asked in decoding after a long portion and a short one."""
    cfg, w = needle_model(size=size, keep=keep, dim=16, heads=2, kv_heads=2, scale=2.0)
    n = 140
    far = n - 1 - (size or 0)
    for needle_at in (0, max(keep - 1, 0), keep, max(far, 0), min(max(far + 1, 0), n - 2), n - 2):
        toks, _ = needle_tokens(n, needle_at)
        want = oracle_logits(cfg, w, toks)
        for dtype in ("float32", "bfloat16"):
            hz = Harness(cfg, w, dtype, page_size=16, num_pages=10, slots=1)
            try:
                got = hz.feed("n", toks, cuts=[n - 21, 2, 1])
            finally:
                hz.close()
            assert rel_err(got, want) < (TOL["float32"] if dtype == "float32" else 4e-2), (needle_at, dtype)


@pytest.mark.parametrize("needle_at", [0, 63, 64, 69, 70, 200, 329, 330, 398])
def test_far_key_among_hundreds_on_the_tensor_core_attention(needle_at):
    """400 tokens, a window of 70 and 70 kept first tokens (more than one key tile of each): the marked key sits among the
    kept tokens, at tile borders, in the hidden stretch and at the window's edge; a long prompt portion, then decoding."""
    n, size, keep = 400, 70, 70
    cfg, w = needle_model(size=size, keep=keep, dim=24, vdim=40, heads=4, kv_heads=2, scale=1.5)
    toks, without = needle_tokens(n, needle_at)
    want = oracle_logits(cfg, w, toks)
    changed = rel_err(oracle_logits(cfg, w, without)[-1], want[-1])
    assert (changed > 0.3) if plain.sees(n - 1, needle_at, size, keep) else (changed < 1e-9)
    for cuts in ([n], [n - 3, 1]):
        hz = Harness(cfg, w, "bfloat16", page_size=32, num_pages=13, slots=1)
        try:
            got = hz.feed("n", toks, cuts=cuts)
        finally:
            hz.close()
        assert rel_err(got[-1], want[-1]) < 4e-2
        assert rel_err(got[300:], want[300:]) < 4e-2


def test_scores_beyond_the_cap():
    """Queries and keys so large that most scores sit on the cap: the cap decides the weights, in both builds."""
    cfg = model_config([attn(scale=4.0, cap=3.0, mlp=None), attn(scale=4.0, cap=3.0, heads=2, kv_heads=2, dim=32, vdim=12, mlp=None)])
    w = plain.random_weights(cfg, 14)
    toks = rand_tokens(60, cfg["vocab"], 15)
    want = oracle_logits(cfg, w, toks)
    loose = copy.deepcopy(cfg)
    for lc in loose["layers"]:
        lc["mixer"]["softcap"] = 100.0
    assert rel_err(oracle_logits(loose, w, toks), want) > 0.05
    got, _ = run(cfg, toks, "float32", cuts=[40, 1], weights=w)
    assert rel_err(got, want) < TOL["float32"]
    got16, _ = run(cfg, toks, "bfloat16", cuts=[40, 1], weights=w)
    assert close(got16, want, "bfloat16")


# ---- the first tokens, long decoding, other sizes --------------------------------------------------------------------------------
@pytest.mark.parametrize("n", [1, 2, 3, 5])
def test_first_tokens(n):
    toks = rand_tokens(n, SMALL["vocab"], 40 + n)
    got, want = run(SMALL, toks, "float32")
    assert close(got, want)
    single, _ = run(SMALL, toks, "float32", cuts=[1])
    assert close(single, want)


def test_long_decoding():
    toks = rand_tokens(260, SMALL["vocab"], 50)
    got, want = run(SMALL, toks, "float32", cuts=[4, 1], num_pages=20)
    assert close(got, want)
    got16, _ = run(SMALL, toks, "bfloat16", cuts=[4, 1], num_pages=20)
    assert close(got16, want, "bfloat16", near_ties(SMALL, plain.random_weights(SMALL, 0), toks))


OTHER = [
    # everything equal to one where it can be: one head, key size one, a window of one, one tap, a token input of one, one
    # expert, one bucket, a residual factor of one
    model_config([attn(heads=1, kv_heads=1, dim=1, vdim=1, size=1, keep=0, mlp=moe(experts=1, top=1, ff=8)),
                  attn(heads=3, kv_heads=1, dim=6, vdim=1, size=2, keep=1, mlp=dense(8, 1.0))], width=24, vocab=50, taps=1, side=1,
                 buckets=1, mult=1.0),
    # key heads == query heads, head sizes the tensor-core attention takes with its wider tile, many experts of a size the
    # tensor-core product takes, three taps, the first layer does not blend
    model_config([attn(heads=4, kv_heads=4, dim=24, vdim=40, size=13, keep=2, v_mix=False, mlp=moe(experts=16, top=4, ff=32)),
                  attn(heads=4, kv_heads=2, dim=72, vdim=104, size=30, keep=0, mlp=dense(64, 2.0)),
                  attn(heads=2, kv_heads=2, dim=128, vdim=104, size=50, keep=7, mlp=None)], width=72, vocab=130, taps=3, side=12,
                 buckets=509, eps=1e-6, mult=0.25),
    # sizes that are not multiples of 8 anywhere, head sizes beyond a warp, two taps, no pair table, no token input
    model_config([attn(heads=6, kv_heads=2, dim=20, vdim=70, size=9, keep=4, mlp=moe(experts=3, top=2, ff=13)),
                  attn(heads=1, kv_heads=1, dim=144, vdim=33, size=100, keep=0, cap=None, v_mix=False, mlp=dense(27, 0.5)),
                  attn(heads=2, kv_heads=2, dim=9, vdim=70, size=None, mlp=None)], width=44, vocab=61, taps=2, side=0, buckets=0),
]


@pytest.mark.parametrize("idx", range(len(OTHER)))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_sizes(idx, dtype):
    cfg = OTHER[idx]
    toks = rand_tokens(60, cfg["vocab"], 60 + idx)
    got, want = run(cfg, toks, dtype, cuts=[21, 3, 1], page_size=32, num_pages=4)
    assert close(got, want, dtype, near_ties(cfg, plain.random_weights(cfg, 0), toks) if dtype == "bfloat16" else ())


# layer-sized models (the tensor-core products, attention tiles and sorted experts take over in the bf16 build): layers of
# unlike head shapes, windows over several 64-token pages, more kept tokens than a key tile, a layer without feed-forward
LAYER_SIZED = [
    model_config([attn(heads=8, kv_heads=2, dim=32, vdim=48, size=100, keep=4, scale=0.18, cap=30.0, mlp=moe(8, 2, 96)),
                  attn(heads=8, kv_heads=2, dim=32, vdim=48, size=100, keep=4, scale=0.18, cap=30.0, mlp=dense(384, 2.0)),
                  attn(heads=4, kv_heads=4, dim=128, vdim=48, size=190, keep=70, scale=0.09, cap=15.0, v_mix=False, mlp=None),
                  attn(heads=8, kv_heads=2, dim=32, vdim=48, size=33, keep=2, scale=0.18, cap=30.0, mlp=moe(40, 5, 32))],
                 width=256, vocab=300, emb_scale=2.0, mult=0.7, taps=4, side=8, buckets=509),
    model_config([attn(heads=3, kv_heads=1, dim=80, vdim=40, size=150, keep=70, scale=0.11, cap=25.0, mlp=moe(7, 3, 50)),
                  attn(heads=3, kv_heads=3, dim=80, vdim=40, size=150, keep=0, scale=0.11, cap=25.0, v_mix=False, mlp=dense(200, 1.5)),
                  attn(heads=6, kv_heads=1, dim=40, vdim=40, size=257, keep=5, scale=0.16, cap=10.0, mlp=moe(7, 3, 50))],
                 width=192, vocab=333, emb_scale=3.0, mult=0.5, taps=3, side=12, buckets=251),
]


@pytest.mark.parametrize("idx", range(len(LAYER_SIZED)))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_sized_models_through_a_randomly_cut_mixed_schedule(idx, dtype):
    """Six requests, four slots, pages for the four longest only: portions of changing size beside single tokens, a
    request now and then left out of a step, the last 30 tokens of each one by one.  bf16 rows are judged as a whole: a
    router's near tie that rounding flips changes that token and those that see it."""
    import random
    cfg = LAYER_SIZED[idx]
    w = plain.random_weights(cfg, 90 + idx)
    for name in [n for n in w if n.endswith("mlp.router")]:        # larger router weights: fewer near ties for bf16 to flip
        w[name] = (w[name].float() * 4.0).to(torch.bfloat16)
    V = cfg["vocab"]
    lens = [400, 230, 64, 5, 310, 129]
    reqs = {f"r{i}": rand_tokens(n, V, 91 + i) for i, n in enumerate(lens)}
    ref = {k: oracle_logits(cfg, w, v) for k, v in reqs.items()}
    pages = sum(-(-n // 64) for n in sorted(lens)[-4:])
    hz = Harness(cfg, w, dtype=dtype, page_size=64, num_pages=pages, slots=4, max_step_tokens=2048)
    rng = random.Random(7 + idx)
    got, at, live, waiting = {k: [] for k in reqs}, {k: 0 for k in reqs}, [], list(reqs)
    try:
        while live or waiting:
            while waiting and len(live) < 4:
                live.append(waiting.pop(0))
            ent = []
            for k in live:
                if len(live) > 1 and rng.random() < 0.15:
                    continue
                left = len(reqs[k]) - at[k]
                n = min(rng.choice([2, 3, 17, 64, 65, 100, 129]), left - 30) if left > 30 else 1
                ent.append((k, reqs[k][at[k]:at[k] + n], range(n)))
            if not ent:
                continue
            out = hz.step(ent)
            o = 0
            for k, t, _ in ent:
                got[k].append(out[o:o + len(t)])
                o += len(t)
                at[k] += len(t)
                if at[k] == len(reqs[k]):
                    hz.end(k)
                    live.remove(k)
        assert len(hz.sched.block_manager.free_block_ids) == pages and len(hz.sched.state_manager.free_slots) == 4
    finally:
        hz.close()
    errs = {k: row_errs(np.concatenate(got[k], 0), ref[k]) for k in reqs}
    e = np.concatenate(list(errs.values()))
    if dtype == "float32":              # but for rows behind a tie that even 32-bit rounding may flip
        for k in reqs:
            errs[k][near_ties(cfg, w, reqs[k], margin=1e-4)] = 0.0
        worst = max(v.max() for v in errs.values())
        assert worst < 1e-4, worst
    else:
        assert np.median(e) < 1.5e-2 and np.mean(e < TOL[dtype]) > 0.9, (np.median(e), e.max())


# ---- greedy generation through the engine's own entry points ------------------------------------------------------------------------
def _greedy_ok(cfg, w, prompt, ids):
    seq = list(prompt)
    for tok in ids:
        lg = oracle_logits(cfg, w, seq)[-1]
        assert tok == int(np.argmax(lg)) or lg.max() - lg[tok] < 1e-3 * (lg.max() - lg.min()), "not the oracle's greedy token"
        seq.append(tok)


def test_greedy_generation_through_llm_generate():
    from jacobiforcing_b200 import LLM, SamplingParams
    from jacobiforcing_b200.hybrid_config import HybridConfig
    w = plain.random_weights(SMALL, 70)
    hc = HybridConfig.from_dict(SMALL)
    llm = LLM(None, hf_config=hc, state_dict=w, dtype="float32", kvcache_block_size=16, num_kvcache_blocks=16, max_num_seqs=2,
              max_model_len=128, max_num_batched_tokens=24)
    V = SMALL["vocab"]
    prompts = [rand_tokens(30, V, 71), rand_tokens(5, V, 72), rand_tokens(17, V, 73)]      # three requests, two slots,
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True), use_tqdm=False)
    llm.exit()                                                                               # prompts cut at 24 tokens
    for prompt, out in zip(prompts, outs):
        assert len(out["token_ids"]) == 8
        _greedy_ok(SMALL, w, prompt, out["token_ids"])


def test_generate_command_line_and_trace_replay_on_a_checkpoint_directory(tmp_path):
    import json
    import os
    import subprocess
    import sys
    from tests.test_hybrid_host import _write_checkpoint
    w = plain.random_weights(SMALL, 75)
    _write_checkpoint(tmp_path, SMALL, w)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    prompt = rand_tokens(21, SMALL["vocab"], 76)
    out = subprocess.run([sys.executable, "-m", "jacobiforcing_b200.generate", "--model", str(tmp_path), "--prompt-ids",
                          ",".join(map(str, prompt)), "--max-tokens", "6", "--dtype", "float32", "--page-size", "16",
                          "--max-model-len", "64", "--max-num-batched-tokens", "64"], cwd=root, capture_output=True, text=True)
    assert out.returncode == 0, out.stderr[-2000:]
    _greedy_ok(SMALL, w, prompt, json.loads(out.stdout.strip().splitlines()[-1])["token_ids"])
    # trace replay: two requests, portions beside single tokens, one ends and its slot and pages are used again
    a, b = rand_tokens(30, SMALL["vocab"], 77), rand_tokens(9, SMALL["vocab"], 78)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:17], "want": [0, 16]}, {"id": "b", "tokens": b[:2], "want": [1]}], "end": []},
             {"step": 1, "entries": [{"id": "b", "tokens": b[2:], "want": [6]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[17:18], "want": [0]}, {"id": "c", "tokens": b, "want": [8]}], "end": ["c"]},
             {"step": 3, "entries": [{"id": "a", "tokens": a[18:], "want": []}], "end": ["a"]}]
    outdir = tmp_path / "out"
    r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", str(tmp_path), "--dtype", "float32", "--out",
                        str(outdir), "--max-tokens", "128", "--page-size", "16"], input="\n".join(json.dumps(x) for x in steps) + "\n",
                       cwd=root, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
    la, lb = oracle_logits(SMALL, w, a), oracle_logits(SMALL, w, b)
    V = SMALL["vocab"]
    g0 = np.fromfile(outdir / "0.f32", dtype="<f4").reshape(-1, V)
    g1 = np.fromfile(outdir / "1.f32", dtype="<f4").reshape(-1, V)
    g2 = np.fromfile(outdir / "2.f32", dtype="<f4").reshape(-1, V)
    assert not (outdir / "3.f32").exists()
    assert rel_err(g0, np.stack([la[0], la[16], lb[1]])) < TOL["float32"]
    assert rel_err(g1, lb[8:9]) < TOL["float32"]
    assert rel_err(g2, np.stack([la[17], lb[8]])) < TOL["float32"]
