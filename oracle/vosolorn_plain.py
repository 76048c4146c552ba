"""Plain, slow restatement of the Vosolorn design: a decoder over one residual stream whose sublayers read the stream
itself and are normed on the way back,  x <- x + ls1 * rms(mixer(x)) * w1,  x <- x + ls2 * rms(ff(x)) * w2.  Two mixers
(softmax attention over a sliding window plus one pooled key / value per block of tokens that has left the window, with
per-head query / key norms, interleaved rotary pairs and values that are rotated by their own position and turned back by
the query's; the matrix memory of xLSTM with capped gates and a running maximum that starts at zero) and two feed-forwards
(a gated dense layer with the tanh form of gelu; a mixture of un-gated erf-gelu experts chosen by the largest router
logits, weighted by a softmax over the chosen logits, beside a shared expert).  The embedding is normed, the output head is
the embedding table.

One function per mechanism, whole sequences only, plain torch on the CPU: every token of a sequence from position 0, no
cache, no state hand-over, no batching.  It shares no code with the product path.

Notation: T tokens, W width, weights are [out, in] and applied as x @ w.T; `p` maps a sublayer's tensor leaf name ("q",
"k.norm", "router.b", ...) to its tensor, `c` is the sublayer's block of the configuration.
"""
from __future__ import annotations

import math
from typing import Dict, List

import torch

DT = torch.float64


# ---- elementary pieces -------------------------------------------------------------------------------------------
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def turn_pairs(v: torch.Tensor, positions: torch.Tensor, dims: int, base: float, sign: float = 1.0) -> torch.Tensor:
    """Rotate the first `dims` entries of the last axis, entry 2i with entry 2i + 1, by sign * position * base^(-2i/dims).
    v [T, ..., D], positions [T]."""
    out = v.clone()
    if dims <= 0:
        return out
    i = torch.arange(dims // 2, dtype=DT)
    ang = sign * positions.to(DT)[:, None] * base ** (-2.0 * i / dims)            # [T, dims / 2]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [dims // 2]
    cos, sin = torch.cos(ang).reshape(shape).to(v.dtype), torch.sin(ang).reshape(shape).to(v.dtype)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * cos - b * sin
    out[..., 1:dims:2] = b * cos + a * sin
    return out


# ---- attention over a window and pooled blocks ------------------------------------------------------------------------
def visible(i: int, size: int, pool: int):
    """What position i sees: the token positions of its window and the blocks whose last token is already behind the window."""
    toks = [j for j in range(max(0, i - size + 1), i + 1)]
    blocks = [b for b in range((i + 1) // pool + 1) if b * pool + pool - 1 <= i - size]
    return toks, blocks


def window_pool_attention(h: torch.Tensor, p: Dict[str, torch.Tensor], c: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, D, Dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    size, pool = c["mask"]["size"], c["mask"]["pool"]
    base, dims = float(c["rot"]["base"]), int(c["rot"]["dims"])
    pos = torch.arange(T)
    q = unit_rms((h @ p["q"].T).reshape(T, H, D), eps) * p["q.norm"]
    k = unit_rms((h @ p["k"].T).reshape(T, G, D), eps) * p["k.norm"]
    v = (h @ p["v"].T).reshape(T, G, Dv)
    q, k = turn_pairs(q, pos, dims, base), turn_pairs(k, pos, dims, base)
    v = turn_pairs(v, pos, Dv, base)                          # a value carries its own position
    out = torch.zeros(T, H, Dv, dtype=h.dtype)
    for i in range(T):
        toks, blocks = visible(i, size, pool)
        keys = [k[j] for j in toks] + [k[b * pool:(b + 1) * pool].mean(0) for b in blocks]
        vals = [v[j] for j in toks] + [v[b * pool:(b + 1) * pool].mean(0) for b in blocks]
        K, V = torch.stack(keys), torch.stack(vals)           # [n, G, .]
        for hh in range(H):
            g = hh // (H // G)
            w = torch.softmax((K[:, g] @ q[i, hh]) * c["scale"], 0)
            out[i, hh] = w @ V[:, g]
    out = turn_pairs(out, pos, Dv, base, sign=-1.0)           # turned back by the query's position
    return out.reshape(T, H * Dv) @ p["o"].T


# ---- matrix memory with capped gates --------------------------------------------------------------------------------
def mlstm_mixer(h: torch.Tensor, p: Dict[str, torch.Tensor], c: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, Dv, cap = c["heads"], c["dim"], c["vdim"], float(c["gate_cap"])
    q = (h @ p["q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ p["k"].T).reshape(T, H, D)
    v = (h @ p["v"].T).reshape(T, H, Dv)
    li = cap * torch.tanh((h @ p["i"].T + p["i.b"]) / cap)                                         # log input gate [T, H]
    lf = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ p["f"].T + p["f.b"]) / cap))         # log forget gate
    S = torch.zeros(H, D, Dv, dtype=h.dtype)
    n = torch.zeros(H, D, dtype=h.dtype)
    m = torch.zeros(H, dtype=h.dtype)                         # the running maximum starts at 0
    o = torch.zeros(T, H, Dv, dtype=h.dtype)
    for t in range(T):
        m_new = torch.maximum(lf[t] + m, li[t])
        a, b = torch.exp(lf[t] + m - m_new), torch.exp(li[t] - m_new)
        S = a[:, None, None] * S + b[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = a[:, None] * n + b[:, None] * k[t]
        m = m_new
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        o[t] = torch.einsum("hdv,hd->hv", S, q[t]) / den[:, None]
    o = unit_rms(o, eps).reshape(T, H * Dv) * p["norm"]
    return (o * torch.sigmoid(h @ p["g"].T)) @ p["o"].T


# ---- feed-forwards -----------------------------------------------------------------------------------------------------
def gated_ff(h: torch.Tensor, p: Dict[str, torch.Tensor]) -> torch.Tensor:
    return (gelu_tanh(h @ p["gate"].T) * (h @ p["up"].T)) @ p["down"].T


def plain_expert(h: torch.Tensor, p: Dict[str, torch.Tensor], name: str) -> torch.Tensor:
    return gelu_erf(h @ p[name + ".up"].T) @ p[name + ".down"].T


def route(h: torch.Tensor, p: Dict[str, torch.Tensor], top: int):
    """ids [T, top] of the largest router logits (ties to the lower index) and the softmax over those logits alone."""
    z = (h @ p["router"].T + p["router.b"]).to(torch.float64)
    ids = torch.zeros(h.shape[0], top, dtype=torch.long)
    for t in range(h.shape[0]):
        row = z[t].clone()
        for j in range(top):
            ids[t, j] = int(torch.argmax(row))
            row[ids[t, j]] = -math.inf
    return ids, torch.softmax(torch.gather(z, 1, ids), -1)


def expert_mixture(h: torch.Tensor, p: Dict[str, torch.Tensor], c: dict) -> torch.Tensor:
    ids, wts = route(h, p, int(c["router"]["top"]))
    y = torch.zeros(h.shape[0], p["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(ids.shape[1]):
            y[t] += wts[t, j].to(h.dtype) * plain_expert(h[t:t + 1], p, f"e{int(ids[t, j])}")[0]
    if c.get("shared"):
        y = y + plain_expert(h, p, "shared")
    return y


# ---- the model -------------------------------------------------------------------------------------------------------------
def _sub(w, prefix):
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=DT, want_layers: bool = False):
    """Logits [T, vocab] of one whole sequence (and the residual stream after every layer [L, T, W])."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    eps = float(config["norm"]["eps"])
    x = unit_rms(w["embed"][torch.tensor(tokens)], eps) * w["embed.norm"]
    streams = []
    for i, lc in enumerate(config["layers"]):
        pre = f"l{i}."
        mix = _sub(w, pre + "mix.")
        if lc["type"] == "attention":
            y = window_pool_attention(x, mix, lc["mixer"], eps)
        elif lc["type"] == "mlstm":
            y = mlstm_mixer(x, mix, lc["mixer"], eps)
        else:
            raise NotImplementedError(lc["type"])
        x = x + w[pre + "ls1"] * (unit_rms(y, eps) * w[pre + "norm1"])
        mlp = lc.get("mlp")
        if mlp is not None:
            ff = _sub(w, pre + "mlp.")
            y = gated_ff(x, ff) if mlp["kind"] == "dense" else expert_mixture(x, ff, mlp)
            x = x + w[pre + "ls2"] * (unit_rms(y, eps) * w[pre + "norm2"])
        streams.append(x.clone())
    logits = (unit_rms(x, eps) * w["final.norm"]) @ w["embed"].T * float(config["logit_scale"])
    if want_layers:
        return logits, torch.stack(streams)
    return logits


# ---- shapes and random weights -------------------------------------------------------------------------------------------
def tensor_shapes(config: dict) -> Dict[str, tuple]:
    W, V = config["width"], config["vocab"]
    s = {"embed": (V, W), "embed.norm": (W,), "final.norm": (W,)}
    for i, lc in enumerate(config["layers"]):
        p, m = f"l{i}.", lc["mixer"]
        s[p + "norm1"] = s[p + "ls1"] = (W,)
        if lc["type"] == "attention":
            H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            s.update({p + "mix.q": (H * D, W), p + "mix.k": (G * D, W), p + "mix.v": (G * Dv, W), p + "mix.q.norm": (D,),
                      p + "mix.k.norm": (D,), p + "mix.o": (W, H * Dv)})
        else:
            H, D, Dv = m["heads"], m["dim"], m["vdim"]
            s.update({p + "mix.q": (H * D, W), p + "mix.k": (H * D, W), p + "mix.v": (H * Dv, W), p + "mix.g": (H * Dv, W),
                      p + "mix.o": (W, H * Dv), p + "mix.norm": (H * Dv,), p + "mix.i": (H, W), p + "mix.i.b": (H,),
                      p + "mix.f": (H, W), p + "mix.f.b": (H,)})
        mlp = lc.get("mlp")
        if mlp is None:
            continue
        s[p + "norm2"] = s[p + "ls2"] = (W,)
        if mlp["kind"] == "dense":
            s.update({p + "mlp.gate": (mlp["ff"], W), p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
        else:
            E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            for e in range(E):
                s[p + f"mlp.e{e}.up"], s[p + f"mlp.e{e}.down"] = (ff, W), (W, ff)
            s[p + "mlp.router"], s[p + "mlp.router.b"] = (E, W), (E,)
            if mlp.get("shared"):
                s[p + "mlp.shared.up"], s[p + "mlp.shared.down"] = (mlp["shared"]["ff"], W), (W, mlp["shared"]["ff"])
    return s


def random_weights(config: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random bf16 weights: matrices ~ N(0, 1/in), norm weights and layer scales near
    one, gate biases that keep the forget gate open, router biases of the size of the logits."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.split(".", 1)[1] if name.startswith("l") and name[1].isdigit() else name
        if len(shape) == 2 and name != "embed":
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
            if leaf in ("mix.q", "mix.k"):
                t = t * 2.0
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        elif leaf == "mix.f.b":
            t = 2.0 + torch.rand(shape, generator=g) * 2.0
        elif leaf in ("mix.i.b", "mlp.router.b"):
            t = torch.randn(shape, generator=g) * 0.5
        elif leaf in ("ls1", "ls2"):
            t = 0.5 + torch.rand(shape, generator=g)
        else:
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        out[name] = t.to(torch.bfloat16)
    return out
