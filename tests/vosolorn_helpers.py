"""Shared pieces of the Vosolorn tests: small configurations (sizes chosen unequal on purpose: key and value sizes differ,
fewer key heads than query heads, a pool that does not divide the page, a window that is no multiple of the pool), random
bf16 weights from the plain oracle, a one-layer model in which one marked token decides the answer, and the error
measures.  The engine is driven through tests.hybrid_helpers.Harness (scheduler + runner)."""
from __future__ import annotations

import copy

import numpy as np
import torch

from oracle import vosolorn_plain as plain
from tests.hybrid_helpers import Harness, rand_tokens, rel_err  # noqa: F401  (re-exported)


def dense(ff=56):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=24, shared=40):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def attn(heads=4, kv_heads=2, dim=16, vdim=12, size=11, pool=3, base=500.0, dims=8, scale=0.4, mlp="default"):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": size, "pool": pool},
                      "rot": {"base": base, "dims": dims}, "scale": scale},
            "mlp": dense() if mlp == "default" else mlp}


def mlstm(heads=3, dim=10, vdim=14, cap=6.0, mlp="default"):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap},
            "mlp": moe() if mlp == "default" else mlp}


def model_config(layers, width=40, vocab=70, logit_scale=1.7, eps=1e-5):
    return {"architecture": "Vosolorn", "layers": copy.deepcopy(layers), "logit_scale": logit_scale, "norm": {"eps": eps},
            "vocab": vocab, "width": width}


# both mixers with both feed-forwards, a layer without feed-forward, a second attention layer with other sizes
SMALL = model_config([mlstm(), attn(), mlstm(heads=2, dim=8, vdim=20, mlp=dense(32)), attn(heads=2, kv_heads=2, dim=8, vdim=20, size=7,
                                                                                            pool=4, dims=8, mlp=moe(4, 1, 16, 0)),
                      mlstm(heads=1, dim=12, vdim=6, mlp=None)])


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


def close(got, want, dtype="float32") -> bool:
    """float32: every row within the tolerance.  bfloat16: a token whose best experts are nearly tied may choose another
    one after rounding, and the recurrent layers carry that token's different result into the next few tokens; so a fifth
    of the rows may lie outside (typical rows are ten times below the tolerance)."""
    e = row_errs(got, want)
    if dtype == "float32":
        return bool(e.max() < TOL[dtype])
    return bool(np.mean(e < TOL[dtype]) >= 0.8 and np.median(e) < TOL[dtype] / 3)


def run(config, tokens, dtype="float32", cuts=None, seed=0, weights=None, **kw):
    w = weights if weights is not None else plain.random_weights(config, seed)
    hz = Harness(config, w, dtype=dtype, **kw)
    try:
        got = hz.feed("a", tokens, cuts)
    finally:
        hz.close()
    return got, oracle_logits(config, w, tokens)


def needle_model(size=24, pool=4, dim=32, vdim=16, heads=2, kv_heads=1, width=64, scale=1.0, dims=8):
    """One attention layer in which token 61 asks for token 60.  The stream's first quarter is a token's key address, the
    second quarter its query address, the second half its content.  Only token 60 has a key address, so every other key
    is zero and scores zero; token 61's query address is token 60's key address, so that key (or the pooled key of its
    block, which is a `pool`-th of it) scores far above zero and takes nearly all the weight wherever the mask lets it be
    seen, and its content decides the answer.  Values read the content half."""
    cfg = model_config([attn(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, size=size, pool=pool, dims=dims, scale=scale,
                             base=100.0, mlp=None)], width=width, vocab=64)
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
    for k, v in {"q": wq, "k": wk, "v": wv, "q.norm": torch.ones(dim), "k.norm": torch.ones(dim)}.items():
        w["l0.mix." + k] = v.to(torch.bfloat16).float()
    w["embed"] = e.to(torch.bfloat16).float()
    w["embed.norm"] = torch.ones(width)
    return cfg, w


def needle_tokens(n, needle_at):
    """(tokens with the marked token and the asking token last, the same without the marked token)."""
    toks = [2 + (i % 50) for i in range(n)]
    without = list(toks)
    toks[needle_at] = 60
    toks[-1] = without[-1] = 61
    return toks, without
