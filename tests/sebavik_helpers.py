"""Shared pieces of the Sebavik tests: small configurations (sizes chosen unequal on purpose: key and value sizes differ,
fewer key heads than query heads, windows that are no multiple of the page, kept first tokens), random bf16 weights from
the plain oracle, a one-layer model in which one marked token decides the answer, and the error measures.  The engine is
driven through tests.hybrid_helpers.Harness (scheduler + runner)."""
from __future__ import annotations

import copy

import numpy as np
import torch

from oracle import sebavik_plain as plain
from tests.hybrid_helpers import Harness, rand_tokens, rel_err  # noqa: F401  (re-exported)


def dense(ff=56, limit=0.8):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts=6, top=2, ff=24):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def attn(heads=4, kv_heads=2, dim=16, vdim=12, size=11, keep=3, scale=0.35, cap=6.0, v_mix=True, mlp="default"):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "v_mix": v_mix}
    if size is not None:
        m["mask"] = {"size": size, "keep_first": keep}
    if cap is not None:
        m["softcap"] = cap
    return {"type": "attention", "mixer": m, "mlp": dense() if mlp == "default" else mlp}


def model_config(layers, width=40, vocab=70, emb_scale=2.0, mult=0.6, taps=4, side=5, buckets=37, eps=2e-5):
    cfg = {"architecture": "Sebavik", "embedding": {"scale": emb_scale}, "layers": copy.deepcopy(layers), "norm": {"eps": eps},
           "residual_mult": mult, "vocab": vocab, "width": width}
    if taps:
        cfg["canon"] = {"taps": taps}
    if side:
        cfg["token_side"] = {"dim": side}
    if buckets:
        cfg["embedding"]["bigram"] = {"buckets": buckets, "mul_prev": 13, "mul_cur": 7}
    return cfg


# both feed-forwards, a layer without one, a layer that does not blend its values between two that do, other head shapes
SMALL = model_config([attn(), attn(mlp=moe()), attn(heads=2, kv_heads=2, dim=8, vdim=20, size=7, keep=0, v_mix=False, mlp=None),
                      attn(heads=6, kv_heads=2, dim=24, vdim=12, size=19, keep=9, cap=2.5, mlp=moe(4, 1, 16)),
                      attn(heads=2, kv_heads=1, dim=16, vdim=24, size=5, keep=1, v_mix=False, mlp=dense(32, 0.3))])


def oracle_logits(config, weights, tokens, dtype=torch.float64):
    return plain.forward(config, weights, list(tokens), dtype=dtype).numpy()


def row_errs(got: np.ndarray, want: np.ndarray) -> np.ndarray:
    """Per row: root mean square of the centred difference over the centred reference."""
    got, want = np.atleast_2d(got).astype(np.float64), np.atleast_2d(want).astype(np.float64)
    d = got - want
    d = d - d.mean(1, keepdims=True)
    w = want - want.mean(1, keepdims=True)
    return np.sqrt((d ** 2).mean(1)) / np.sqrt((w ** 2).mean(1) + 1e-30)


TOL = {"float32": 3e-4, "bfloat16": 6e-2}


def close(got, want, dtype="float32", skip=()) -> bool:
    """float32: every row within the tolerance.  bfloat16: the rows in `skip` are not judged (see near_ties); of the others a
    fifth may lie outside (typical rows are ten times below the tolerance)."""
    e = row_errs(got, want)
    if dtype == "float32":
        return bool(e.max() < TOL[dtype])
    keep = np.ones(len(e), dtype=bool)
    keep[[i for i in skip if i < len(e)]] = False
    if not keep.any():
        return True
    e = e[keep]
    return bool(np.mean(e < TOL[dtype]) >= 0.8 and np.median(e) < TOL[dtype] / 3)


def near_ties(config, weights, tokens, margin=0.015):
    """Rows that a bf16 run may legitimately answer differently: a token whose last chosen and first rejected expert lie
    closer than `margin` in the oracle may choose the other one after rounding, and the tokens that follow within the
    longest window (and convolution) see that token's keys and values."""
    found = []
    inner = plain.route

    def watching(h, router, top):
        z = torch.sort(h @ router.T, 1, descending=True).values
        if top < z.shape[1]:
            found.extend(torch.nonzero(z[:, top - 1] - z[:, top] < margin).flatten().tolist())
        return inner(h, router, top)
    plain.route = watching
    try:
        plain.forward(config, weights, list(tokens))
    finally:
        plain.route = inner
    reach = max((lc["mixer"].get("mask") or {}).get("size") or len(tokens) for lc in config["layers"]) + 4
    return sorted({r for t in found for r in range(t, min(t + reach, len(tokens)))})


def run(config, tokens, dtype="float32", cuts=None, seed=0, weights=None, **kw):
    w = weights if weights is not None else plain.random_weights(config, seed)
    hz = Harness(config, w, dtype=dtype, **kw)
    try:
        got = hz.feed("a", tokens, cuts)
    finally:
        hz.close()
    return got, oracle_logits(config, w, tokens)


def needle_model(size=24, keep=5, dim=32, vdim=16, heads=2, kv_heads=1, width=64, scale=1.0, cap=30.0, taps=4):
    """One attention layer in which token 61 asks for token 60.  The stream's first quarter is a token's key address, the
    second quarter its query address, the second half its content.  Only token 60 has a key address, so every other key
    is zero and scores zero (less its distance bias); token 61's query address is token 60's key address, so that key
    scores far above zero and takes nearly all the weight wherever the mask lets it be seen, and its content decides the
    answer.  Values read the content half.  The input convolution, the pair table, the projections' biases and the sink are
    out of the way (zero); the distance bias is small."""
    cfg = model_config([attn(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, size=size, keep=keep, scale=scale, cap=cap,
                             v_mix=False, mlp=None)], width=width, vocab=64, taps=taps, side=0, buckets=11, mult=1.0)
    w = plain.random_weights(cfg, 31)
    g = torch.Generator().manual_seed(32)
    half, q4 = width // 2, width // 4
    m = torch.randn(kv_heads * dim, q4, generator=g)
    wk = torch.zeros(kv_heads * dim, width)
    wk[:, :q4] = m
    wq = torch.zeros(heads * dim, width)
    for h in range(heads):
        gq = h // (heads // kv_heads)
        wq[h * dim:(h + 1) * dim, q4:half] = m[gq * dim:(gq + 1) * dim]
    wv = torch.zeros(kv_heads * vdim, width)
    wv[:, half:] = torch.randn(kv_heads * vdim, half, generator=g) / half ** 0.5
    e = w["embed"].float()
    e[:, :half] = 0.0
    e[60, :q4] = torch.randn(q4, generator=g)
    e[61, q4:half] = e[60, :q4]
    e[60, half:] *= 3.0
    zero = {"q.b": heads * dim, "k.b": kv_heads * dim, "v.b": kv_heads * vdim, "sink": heads}
    for k, v in {"q": wq, "k": wk, "v": wv, "r1": torch.full((heads,), 0.05), "r2": torch.full((heads,), 0.5)}.items():
        w["l0.mix." + k] = v.to(torch.bfloat16).float()
    for k, n in zero.items():
        w["l0.mix." + k] = torch.zeros(n)
    w["embed"] = e.to(torch.bfloat16).float()
    w["bigram"] = torch.zeros_like(w["bigram"].float())
    w["l0.norm1"] = torch.ones(width)
    if taps:
        w["l0.canon1"] = torch.zeros(width, taps)
    return cfg, w


def needle_tokens(n, needle_at):
    """(tokens with the marked token and the asking token last, the same without the marked token)."""
    toks = [2 + (i % 50) for i in range(n)]
    without = list(toks)
    toks[needle_at] = 60
    toks[-1] = without[-1] = 61
    return toks, without
