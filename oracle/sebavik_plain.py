"""Plain, slow restatement of the Sebavik design: a pre-norm decoder over one residual stream,
x <- x + m * ls1 * mixer(c1(n1(x))),  x <- x + m * ls2 * ff(c2(n2(x))),  then a per-layer token input and an average over
the depth.  n = RMS norm with a plain weight; c(h) = h + a short causal convolution of h over time per channel; m one
number of the model; ls a per-channel layer scale.  Mixer: softmax attention without rotation whose scores are scaled,
capped by a tanh and lowered by a logarithmic distance bias, over a sliding window plus the first tokens of the sequence,
with a per-head sink in the denominator, biased projections, fewer key / value heads than query heads and values that are
blended with the values of the first such layer.  Feed-forwards: a clamped gated dense layer and a mixture of gated silu
experts chosen by the largest router logits (softmax over the chosen).  The embedding is scaled and a hashed embedding of
the (previous, current) token pair is added; the output head is the embedding table.

One function per mechanism, whole sequences only, plain torch on the CPU: every token of a sequence from position 0, no
cache, no state hand-over, no batching.  It shares no code with the product path.

Notation: T tokens, W width, weights are [out, in] and applied as x @ w.T; `p` maps a sublayer's tensor leaf name ("q",
"q.b", "sink", ...) to its tensor, `c` is the sublayer's block of the configuration.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

DT = torch.float64


# ---- elementary pieces -------------------------------------------------------------------------------------------
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def time_conv(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """h [T, W], w [W, taps]: out_t = sum_j w[:, j] * h_(t - taps + 1 + j), zeros before the first token."""
    T, taps = h.shape[0], w.shape[1]
    out = torch.zeros_like(h)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    return out


def sublayer_input(x: torch.Tensor, norm_w: torch.Tensor, conv_w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    h = unit_rms(x, eps) * norm_w
    return h if conv_w is None else h + time_conv(h, conv_w)


# ---- embedding ---------------------------------------------------------------------------------------------------
def pair_rows(tokens: List[int], c: dict) -> List[int]:
    """Row of the hashed pair table for every token; the first token of a sequence uses the table's last row."""
    n = int(c["buckets"])
    return [n if t == 0 else (tokens[t - 1] * int(c["mul_prev"]) + tokens[t] * int(c["mul_cur"])) % n for t in range(len(tokens))]


def embed(tokens: List[int], weights: Dict[str, torch.Tensor], cfg: dict, dtype=DT) -> torch.Tensor:
    e = cfg["embedding"]
    x = weights["embed"].to(dtype)[tokens] * float(e["scale"])
    if e.get("bigram"):
        x = x + weights["bigram"].to(dtype)[pair_rows(tokens, e["bigram"])]
    return x


# ---- attention -----------------------------------------------------------------------------------------------------
def sees(i: int, j: int, size: Optional[int], keep_first: int) -> bool:
    return j <= i and (size is None or i - j < size or j < keep_first)


def attention_values(h: torch.Tensor, p: Dict[str, torch.Tensor], c: dict) -> torch.Tensor:
    """The layer's own values [T, G, Dv] before any blending."""
    return (h @ p["v"].T + p["v.b"]).reshape(h.shape[0], c["kv_heads"], c["vdim"])


def attention(h: torch.Tensor, p: Dict[str, torch.Tensor], c: dict, v: torch.Tensor) -> torch.Tensor:
    """v: the values this layer attends over (already blended where the design says so)."""
    T = h.shape[0]
    H, G, D, Dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    mask = c.get("mask") or {}
    size, keep = mask.get("size"), int(mask.get("keep_first", 0))
    cap = c.get("softcap")
    q = (h @ p["q"].T + p["q.b"]).reshape(T, H, D)
    k = (h @ p["k"].T + p["k.b"]).reshape(T, G, D)
    out = torch.zeros(T, H, Dv, dtype=h.dtype)
    for i in range(T):
        js = [j for j in range(i + 1) if sees(i, j, size, keep)]
        dist = torch.tensor([i - j for j in js], dtype=h.dtype)
        for hh in range(H):
            g = hh // (H // G)
            s = (k[js, g] @ q[i, hh]) * float(c["scale"])
            if cap:
                s = float(cap) * torch.tanh(s / float(cap))
            s = s - p["r1"][hh] * torch.log1p(p["r2"][hh] * dist)
            top = torch.maximum(s.max(), p["sink"][hh])
            w = torch.exp(s - top)
            w = w / (w.sum() + torch.exp(p["sink"][hh] - top))             # the sink: one more term below, nothing above
            out[i, hh] = w @ v[js, g]
    return out.reshape(T, H * Dv) @ p["o"].T


# ---- feed-forwards ---------------------------------------------------------------------------------------------------
def clamped_gated(h: torch.Tensor, p: Dict[str, torch.Tensor], c: dict) -> torch.Tensor:
    lim = float(c["limit"])
    g = torch.clamp(h @ p["gate"].T, max=lim)
    u = torch.clamp(h @ p["up"].T, min=-lim, max=lim)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ p["down"].T


def route(h: torch.Tensor, router: torch.Tensor, top: int):
    """Per token: the experts with the largest logits (ties to the lower index) and a softmax over their logits alone."""
    z = h @ router.T
    ids, wts = [], []
    for t in range(h.shape[0]):
        order = sorted(range(z.shape[1]), key=lambda e: (-float(z[t, e]), e))[:top]
        zz = torch.stack([z[t, e] for e in order])
        ids.append(order)
        wts.append(torch.softmax(zz, 0))
    return ids, wts


def experts(h: torch.Tensor, p: Dict[str, torch.Tensor], c: dict) -> torch.Tensor:
    ids, wts = route(h, p["router"], int(c["router"]["top"]))
    out = torch.zeros(h.shape[0], p["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, w in zip(ids[t], wts[t]):
            a = h[t] @ p[f"e{e}.gate"].T
            out[t] += w * ((a * torch.sigmoid(a) * (h[t] @ p[f"e{e}.up"].T)) @ p[f"e{e}.down"].T)
    return out


# ---- per-layer token input --------------------------------------------------------------------------------------------------
def token_input(x: torch.Tensor, tokens: List[int], table: torch.Tensor, layer: int, dim: int, p: Dict[str, torch.Tensor],
                eps: float) -> torch.Tensor:
    e = table[tokens][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ p["gate"].T) * e) @ p["proj"].T
    return unit_rms(y, eps) * p["norm"]


# ---- the model -----------------------------------------------------------------------------------------------------------------
def sub(weights: Dict[str, torch.Tensor], prefix: str, dtype) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v.to(dtype) for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=DT, layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence from position 0.  layers_out: receives the stream after every layer."""
    eps, m = float(cfg["norm"]["eps"]), float(cfg["residual_mult"])
    taps = int((cfg.get("canon") or {}).get("taps", 0))
    side_dim = int((cfg.get("token_side") or {}).get("dim", 0))
    x = embed(tokens, weights, cfg, dtype)
    kept = [x]                                   # X_0 .. : the embedding output and every layer's own result
    v_first = None
    for i, lc in enumerate(cfg["layers"]):
        w = sub(weights, f"l{i}.", dtype)
        c = lc["mixer"]
        h = sublayer_input(x, w["norm1"], w["canon1"] if taps else None, eps)
        pm = sub(w, "mix.", dtype)
        v = attention_values(h, pm, c)
        if c.get("v_mix"):
            if v_first is None:
                v_first = v
            else:
                v = (1.0 - pm["vmix"]) * v + pm["vmix"] * v_first
        x = x + m * w["ls1"] * attention(h, pm, c, v)
        mlp = lc.get("mlp")
        if mlp is not None:
            h = sublayer_input(x, w["norm2"], w["canon2"] if taps else None, eps)
            y = clamped_gated(h, sub(w, "mlp.", dtype), mlp) if mlp["kind"] == "dense" else experts(h, sub(w, "mlp.", dtype), mlp)
            x = x + m * w["ls2"] * y
        if side_dim:
            x = x + m * token_input(x, tokens, weights["side.embed"].to(dtype), i, side_dim, sub(w, "side.", dtype), eps)
        kept.append(x)
        x = sum(w["dwa"][j] * kept[j] for j in range(i + 2))
        if layers_out is not None:
            layers_out.append(x.clone())
    return (unit_rms(x, eps) * weights["final.norm"].to(dtype)) @ weights["embed"].to(dtype).T


# ---- tensors of a configuration, random weights -----------------------------------------------------------------------------------
def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    W, V, L = int(cfg["width"]), int(cfg["vocab"]), len(cfg["layers"])
    taps = int((cfg.get("canon") or {}).get("taps", 0))
    side = int((cfg.get("token_side") or {}).get("dim", 0))
    out = {"embed": (V, W), "final.norm": (W,)}
    pair = cfg["embedding"].get("bigram")
    if pair:
        out["bigram"] = (int(pair["buckets"]) + 1, W)
    if side:
        out["side.embed"] = (V, side * L)
    for i, lc in enumerate(cfg["layers"]):
        p, c = f"l{i}.", lc["mixer"]
        H, G, D, Dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
        out.update({p + "norm1": (W,), p + "ls1": (W,), p + "dwa": (i + 2,),
                    p + "mix.q": (H * D, W), p + "mix.q.b": (H * D,), p + "mix.k": (G * D, W), p + "mix.k.b": (G * D,),
                    p + "mix.v": (G * Dv, W), p + "mix.v.b": (G * Dv,), p + "mix.vmix": (), p + "mix.r1": (H,), p + "mix.r2": (H,),
                    p + "mix.sink": (H,), p + "mix.o": (W, H * Dv)})
        if taps:
            out[p + "canon1"] = (W, taps)
        if side:
            out.update({p + "side.gate": (side, W), p + "side.proj": (W, side), p + "side.norm": (W,)})
        mlp = lc.get("mlp")
        if mlp is None:
            continue
        out.update({p + "norm2": (W,), p + "ls2": (W,)})
        if taps:
            out[p + "canon2"] = (W, taps)
        if mlp["kind"] == "dense":
            out.update({p + "mlp.gate": (mlp["ff"], W), p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
        else:
            ff = mlp["expert"]["ff"]
            out[p + "mlp.router"] = (mlp["router"]["experts"], W)
            for e in range(mlp["router"]["experts"]):
                out.update({p + f"mlp.e{e}.gate": (ff, W), p + f"mlp.e{e}.up": (ff, W), p + f"mlp.e{e}.down": (W, ff)})
    return out


def random_weights(cfg: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random bf16 weights: matrices ~ N(0, 1 / in) (queries and keys twice that, so that the cap, the bias and the mask
    matter), norm weights and layer scales near one, distance-bias numbers and blend factors inside (0, 1), depth weights
    that favour the layer's own result."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".", 1)[1] if name.startswith("l") and name[1].isdigit() else name
        if leaf in ("embed", "side.embed"):
            t = torch.randn(shape, generator=g)
        elif leaf == "bigram":
            t = torch.randn(shape, generator=g) * 0.5
        elif leaf in ("canon1", "canon2"):
            t = torch.randn(shape, generator=g) * 0.3
        elif len(shape) == 2:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
            if leaf in ("mix.q", "mix.k"):
                t = t * 2.0
        elif leaf in ("mix.q.b", "mix.k.b", "mix.v.b"):
            t = torch.randn(shape, generator=g) * 0.3
        elif leaf == "mix.r1":
            t = 0.2 + 0.8 * torch.rand(shape, generator=g)
        elif leaf == "mix.r2":
            t = 0.05 + 0.45 * torch.rand(shape, generator=g)
        elif leaf == "mix.sink":
            t = torch.randn(shape, generator=g)
        elif leaf == "mix.vmix":
            t = 0.2 + 0.6 * torch.rand(shape, generator=g)
        elif leaf == "dwa":
            t = torch.randn(shape, generator=g) * 0.25
            t[-1] += 1.0
        elif leaf in ("ls1", "ls2"):
            t = 0.5 + torch.rand(shape, generator=g)
        else:
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        out[name] = t.to(torch.bfloat16)
    return out
