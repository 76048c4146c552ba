"""Vosolorn on the GPU against the plain fp64 restatement (oracle/vosolorn_plain.py): each mechanism alone, prefill against
token-by-token decoding, portions, unequal batches, reuse of pages and slots, a marked key far back, at page borders and
just inside / just outside the window and the pooled blocks (in prompts, in decoding, with blocks completed across steps),
the values' rotation far from the start, capped gates and the running maximum's start, the first tokens of a sequence,
long decoding, other sizes, and greedy generation through LLM.generate, the generate command line and the trace replay."""
import copy

import numpy as np
import pytest
import torch

from oracle import vosolorn_plain as plain
from tests.vosolorn_helpers import (SMALL, TOL, Harness, attn, close, dense, mlstm, model_config, moe, needle_model, needle_tokens,
                                    oracle_logits, rand_tokens, rel_err, run)

pytestmark = pytest.mark.gpu


# ---- each mechanism alone ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["attention", "mlstm", "dense", "experts"])
def test_mechanism_alone(which, dtype):
    layers = {"attention": [attn(mlp=None)], "mlstm": [mlstm(mlp=None)], "dense": [mlstm(heads=1, dim=4, vdim=4, mlp=dense())],
              "experts": [mlstm(heads=1, dim=4, vdim=4, mlp=moe())]}[which]
    cfg = model_config(layers)
    toks = rand_tokens(45, cfg["vocab"], 3)
    got, want = run(cfg, toks, dtype)
    assert close(got, want, dtype)


@pytest.mark.parametrize("kw", [dict(experts=8, top=3), dict(experts=1, top=1, shared=0), dict(experts=5, top=5, ff=8, shared=16),
                                dict(experts=40, top=2, ff=9, shared=7), dict(experts=6, top=2, shared=0)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_router_shapes(kw, dtype):
    """One expert, every expert chosen, more experts than a warp, expert sizes that the tensor-core product does not take,
    with and without the shared expert; many tokens so that the expert-sorted path runs, few so that the per-pair one does."""
    cfg = model_config([mlstm(heads=1, dim=4, vdim=4, mlp=moe(**kw)), attn(heads=1, kv_heads=1, dim=4, vdim=4, dims=2, mlp=moe(**kw))])
    toks = rand_tokens(80, cfg["vocab"], 4)
    got, want = run(cfg, toks, dtype, cuts=[60, 1, 7, 1])
    assert close(got, want, dtype)


def test_router_bias_decides():
    """A bias far above the logits forces the choice; without it the answer changes."""
    cfg = model_config([mlstm(heads=1, dim=4, vdim=4, mlp=moe(experts=6, top=2, shared=0))])
    w = plain.random_weights(cfg, 5)
    w["l0.mlp.router.b"] = torch.tensor([0.0, 9.0, 0.0, 0.0, 7.0, 0.0])
    toks = rand_tokens(30, cfg["vocab"], 6)
    want = oracle_logits(cfg, w, toks)
    w0 = dict(w)
    w0["l0.mlp.router.b"] = torch.zeros(6)
    assert rel_err(oracle_logits(cfg, w0, toks), want) > 0.05
    for dtype in ("float32", "bfloat16"):
        got, _ = run(cfg, toks, dtype, weights=w, cuts=[20, 1])
        assert rel_err(got, want) < TOL[dtype]


# ---- prefill == decode, portions -------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_equals_token_by_token(dtype):
    toks = rand_tokens(70, SMALL["vocab"], 5)
    whole, want = run(SMALL, toks, dtype)
    single, _ = run(SMALL, toks, dtype, cuts=[1])
    assert close(whole, want, dtype)
    assert close(single, want, dtype)
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
        assert close(np.concatenate(got[k], 0), ref[k], dtype), k


def test_slot_and_pages_used_again_start_from_the_empty_state():
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


# ---- a key that must be found, or must not be: window, pooled blocks, page borders ----------------------------------------------
N, SIZE, POOL = 150, 24, 4
# asked from position 149: the window holds 126 .. 149, the blocks up to position 123 are complete behind it, 124 and 125
# have left the window while their block is not yet seen
NEEDLES = [0, 1, 3, 4, 15, 16, 31, 32, 63, 64, 119, 120, 123, 124, 125, 126, 127, 148]


def _seen(j):
    toks, blocks = plain.visible(N - 1, SIZE, POOL)
    return j in toks or j // POOL in blocks


@pytest.mark.parametrize("needle_at", NEEDLES)
@pytest.mark.parametrize("how", ["prompt", "decode", "portions"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_marked_key_is_seen_exactly_where_the_mask_says(needle_at, how, dtype):
    cfg, w = needle_model(size=SIZE, pool=POOL)
    toks, without = needle_tokens(N, needle_at)
    want = oracle_logits(cfg, w, toks)
    changed = rel_err(oracle_logits(cfg, w, without)[-1], want[-1])
    assert (changed > 0.3) if _seen(needle_at) else (changed < 1e-9)        # the marked key decides the answer, or is hidden
    cuts = {"prompt": [N], "decode": [N - 30, 1], "portions": [5, 2, 3, 17, 2, 6]}[how]     # blocks complete across steps
    hz = Harness(cfg, w, dtype, page_size=16, num_pages=12, slots=1)
    try:
        got = hz.feed("n", toks, cuts=cuts)
    finally:
        hz.close()
    tol = TOL["float32"] if dtype == "float32" else 4e-2
    assert rel_err(got[-1], want[-1]) < tol
    assert rel_err(got, want) < tol


@pytest.mark.parametrize("size,pool", [(1, 1), (5, 1), (3, 7), (16, 16), (17, 5), (40, 3), (5, 20)])
def test_windows_and_pools_of_other_shapes(size, pool):
    """A window of one token, a pool of one (every token behind the window is its own block: full attention), a pool longer
    than the window, both equal to the page, pools that do not divide the page (blocks straddle pages), a pool longer than
    the page."""
    cfg, w = needle_model(size=size, pool=pool, dim=16, heads=2, kv_heads=2, scale=2.0 * pool ** 0.5)
    n = 75
    for needle_at in (0, n - 1 - size, max(0, n - size - pool), n - 2):
        toks, _ = needle_tokens(n, needle_at)
        want = oracle_logits(cfg, w, toks)
        hz = Harness(cfg, w, "float32", page_size=16, num_pages=6, slots=1)
        try:
            got = hz.feed("n", toks, cuts=[n - 21, 2, 1])
        finally:
            hz.close()
        assert rel_err(got, want) < TOL["float32"], needle_at


def test_value_rotation_decides_far_from_the_start():
    """Values are turned by their own position and the output back by the query's; positions run to 400, in a prompt and in
    decoding.  A base one percent off shows in the oracle, so a wrong angle would show here."""
    cfg = model_config([attn(heads=2, kv_heads=1, dim=16, vdim=24, size=30, pool=5, base=50.0, dims=16, scale=0.3, mlp=None)])
    w = plain.random_weights(cfg, 21)
    toks = rand_tokens(400, cfg["vocab"], 22)
    want = oracle_logits(cfg, w, toks)
    off = copy.deepcopy(cfg)
    off["layers"][0]["mixer"]["rot"]["base"] = 50.5
    assert rel_err(oracle_logits(off, w, toks)[300:], want[300:]) > 0.02
    got, _ = run(cfg, toks, "float32", cuts=[370, 1], weights=w, page_size=32, num_pages=13)
    assert rel_err(got, want) < TOL["float32"]


# ---- matrix memory: the gates' cap, the running maximum's start -------------------------------------------------------------------
@pytest.mark.parametrize("i_bias,f_bias", [(-8.0, 3.0), (30.0, -30.0), (0.0, 40.0), (12.0, 0.5)])
def test_gate_cap_and_the_maximum_that_starts_at_zero(i_bias, f_bias):
    """An input gate far below zero: the maximum stays at its start of zero for the first tokens, so the denominator's
    floor is one.  Pre-activations beyond the cap: the cap decides the gate."""
    cfg = model_config([mlstm(heads=2, dim=6, vdim=10, cap=5.0, mlp=None)])
    w = plain.random_weights(cfg, 23)
    w["l0.mix.i.b"] = torch.full((2,), i_bias)
    w["l0.mix.f.b"] = torch.full((2,), f_bias)
    toks = rand_tokens(50, cfg["vocab"], 24)
    want = oracle_logits(cfg, w, toks)
    uncapped = copy.deepcopy(cfg)
    uncapped["layers"][0]["mixer"]["gate_cap"] = 50.0
    if abs(i_bias) > 20 or abs(f_bias) > 20:
        assert rel_err(oracle_logits(uncapped, w, toks), want) > 1e-3
    got, _ = run(cfg, toks, "float32", cuts=[1, 2, 30, 1], weights=w)
    assert rel_err(got, want) < TOL["float32"]


@pytest.mark.parametrize("dim,vdim", [(16, 24), (64, 128), (128, 64), (48, 250)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_matrix_memory_long_portions(dim, vdim, dtype):
    """Head sizes whose rows start on 16-byte boundaries and portions of several staged batches: the raw rows of the next
    batch travel while the current one runs; a last batch that is not full; a portion that ends inside a batch."""
    cfg = model_config([mlstm(heads=2, dim=dim, vdim=vdim, cap=8.0, mlp=None)], width=64)
    toks = rand_tokens(150, cfg["vocab"], 33)
    got, want = run(cfg, toks, dtype, cuts=[70, 45, 33, 1], num_pages=12)
    assert close(got, want, dtype)
    if dtype == "float32":
        whole, _ = run(cfg, toks, dtype, num_pages=12)
        assert close(whole, want)


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
    assert close(got16, want, "bfloat16")


OTHER = [
    # everything equal to one where it can be: one head, one key head, key size two, window and pool of one, one expert
    model_config([mlstm(heads=1, dim=1, vdim=1, cap=1.0, mlp=moe(experts=1, top=1, ff=8, shared=0)),
                  attn(heads=1, kv_heads=1, dim=2, vdim=2, size=1, pool=1, dims=2, mlp=None),
                  attn(heads=3, kv_heads=1, dim=6, vdim=4, size=2, pool=9, dims=0, mlp=dense(8))], width=24, vocab=50),
    # key heads == query heads, all dimensions rotated, a value size above a warp, a key size above a warp on the matrix
    # memory, many experts of a size the tensor-core product takes
    model_config([attn(heads=4, kv_heads=4, dim=24, vdim=40, size=13, pool=2, dims=24, mlp=moe(experts=16, top=4, ff=32, shared=64)),
                  mlstm(heads=2, dim=40, vdim=70, cap=10.0, mlp=dense(64)),
                  mlstm(heads=4, dim=64, vdim=31, cap=0.5, mlp=None)], width=72, vocab=130, logit_scale=0.5, eps=1e-6),
    # head sizes beyond what a thread keeps in registers (the state lives in shared memory), width not a multiple of 8,
    # value rows wider than the key rows, feed-forward sizes that are not multiples of 8
    model_config([mlstm(heads=2, dim=136, vdim=24, mlp=dense(27)), attn(heads=6, kv_heads=2, dim=20, vdim=70, size=9, pool=6, dims=10,
                                                                         mlp=moe(experts=3, top=2, ff=13, shared=5)),
                  mlstm(heads=1, dim=16, vdim=300, mlp=None)], width=44, vocab=61),
]


@pytest.mark.parametrize("idx", range(len(OTHER)))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_sizes(idx, dtype):
    cfg = OTHER[idx]
    toks = rand_tokens(60, cfg["vocab"], 60 + idx)
    got, want = run(cfg, toks, dtype, cuts=[21, 3, 1], page_size=32, num_pages=4)
    assert close(got, want, dtype)


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
