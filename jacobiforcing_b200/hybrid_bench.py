"""Throughput of the layered hybrid decoders beside the closest existing model at equal size: prefill tokens/s, decode
tokens/s, device time per kernel group with its distance from the roofline (tensor peak for prefill products, HBM
bandwidth for decode).  Random weights, synthetic tokens.  `bench.py --compare-hybrid`: Kinetar beside the Qwen2 engine at
equal width / depth / feed-forward size.  `bench.py --compare-famepel`: Famepel beside Kinetar at equal width / depth and
equal ACTIVE feed-forward size per token (top x expert size = the dense size).  `bench.py --compare-vosolorn`: Vosolorn
beside Famepel at equal width / depth (both are normed-sublayer designs with layer scales, a matrix-state recurrence,
attention and routed experts).  `bench.py --compare-sebavik`: Sebavik beside Vosolorn with attention in every layer (both: windowed
attention over paged keys and values, a gated dense feed-forward alternating with routed experts, RMS norms)."""
from __future__ import annotations

import time
from typing import Dict, List

import numpy as np

SIZES = {
    "w1024": dict(width=1024, layers=4, ff=4096, heads=8, kv_heads=2, dim=128, vocab=32000),
    "w2048": dict(width=2048, layers=4, ff=8192, heads=16, kv_heads=4, dim=128, vocab=32000),
    "w4096": dict(width=4096, layers=2, ff=14336, heads=32, kv_heads=8, dim=128, vocab=32000),
}


def hybrid_description(sz: dict) -> dict:
    W = sz["width"]
    par = {"type": "parallel",
           "mixer": {"left": {"conv": 4, "dim": sz["dim"], "heads": sz["heads"], "kv_heads": sz["kv_heads"],
                              "q_temp": {"coef": 0.5, "every": 1024}, "scale": sz["dim"] ** -0.5, "vdim": sz["dim"]},
                     "left_scale": 0.7,
                     "right": {"conv": 4, "dt_rank": W // 16, "inner": 2 * W, "state": 16}, "right_scale": 0.7},
           "mlp": {"ff": sz["ff"], "kind": "dense"}}
    dl = {"type": "channel_delta",
          "mixer": {"conv": 4, "dim": 128, "heads": W // 128, "kv_heads": max(1, W // 256), "vdim": 128},
          "mlp": {"ff": sz["ff"], "kind": "dense"}}
    layers = [par if i % 2 == 0 else dl for i in range(sz["layers"])]
    return {"architecture": "Kinetar", "embedding": {"scale": 1.0}, "layers": layers, "logit_scale": 1.0,
            "norm": {"eps": 1e-6}, "vocab": sz["vocab"], "width": W}


def hybrid_weights(desc: dict, seed: int, low: int = 64) -> Dict[str, np.ndarray]:
    rng = np.random.default_rng(seed)
    W, V = desc["width"], desc["vocab"]

    def lin(n, k):
        return (rng.standard_normal((n, k), dtype=np.float32) / np.sqrt(k)).astype(np.float32)

    def vec(n, s=0.1, b=0.0):
        return (rng.standard_normal(n, dtype=np.float32) * s + b).astype(np.float32)
    w = {"embed": lin(V, W) * 4.0, "final.norm": vec(W), "head": lin(V, W)}
    for i, lc in enumerate(desc["layers"]):
        p, m = f"l{i}.", lc["mixer"]
        w[p + "norm1"] = vec(W)
        if lc["type"] == "parallel":
            a, s = m["left"], m["right"]
            nq, nk, I, N, R = a["heads"] * a["dim"], a["kv_heads"] * a["dim"], s["inner"], s["state"], s["dt_rank"]
            L, Rt = p + "mix.left.", p + "mix.right."
            w.update({L + "q": lin(nq, W), L + "k": lin(nk, W), L + "q.conv": vec((nq, a["conv"]), 0.5),
                      L + "k.conv": vec((nk, a["conv"]), 0.5), L + "sink": vec(a["heads"], 1.0), L + "g": lin(nq, W),
                      L + "o": lin(W, nq), Rt + "in": lin(2 * I, W), Rt + "conv": vec((I, s["conv"]), 0.5),
                      Rt + "conv.b": vec(I), Rt + "x": lin(R + 2 * N, I), Rt + "dt": lin(I, R), Rt + "dt.b": vec(I, 0.5, -1.0),
                      Rt + "A_log": np.log(rng.uniform(0.2, 3.0, (I, N))).astype(np.float32), Rt + "D": vec(I, 0.3, 1.0),
                      Rt + "o": lin(W, I)})
        else:
            nq, nv = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"]
            M = p + "mix."
            w.update({M + "q": lin(nq, W), M + "k": lin(nq, W), M + "v": lin(nv, W), M + "q.conv": vec((nq, m["conv"]), 0.5),
                      M + "k.conv": vec((nq, m["conv"]), 0.5), M + "v.conv": vec((nv, m["conv"]), 0.5),
                      M + "b": lin(m["heads"], W), M + "A_log": np.log(rng.uniform(0.1, 1.5, m["heads"])).astype(np.float32),
                      M + "norm": vec(m["vdim"], 0.2, 1.0), M + "a1": lin(low, W), M + "a2": lin(m["heads"] * m["dim"], low),
                      M + "dt_bias": vec(m["heads"] * m["dim"], 0.5, -1.0), M + "g1": lin(low, W), M + "g2": lin(nv, low),
                      M + "o": lin(W, nv)})
        w[p + "mlp.up"] = lin(lc["mlp"]["ff"], W)
        w[p + "mlp.down"] = lin(W, lc["mlp"]["ff"])
    return w


def famepel_description(sz: dict) -> dict:
    """Layers in the order recurrence, gated recurrence, recurrence, latent attention (the last attention layer borrows the
    first one's cache when there are two), sizes in the proportions of published models of each kind: recurrence inner =
    2 width in heads of 64 with a state of 128; latent attention with a key/value rank of 512 + 64 rotated, query rank
    3 width / 4, heads of 128; routed experts of ff / top each, `top` of 8 x top experts per token."""
    W, top = sz["width"], sz.get("top", 4)
    ff = sz["ff"] // top
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": 8 * top, "top": top, "scale": 2.5,
                                                             "groups": {"count": 4, "keep": 2}}}
    ssd = {"type": "mamba2", "mixer": {"heads": 2 * W // 64, "vdim": 64, "state": 128, "groups": 8, "conv": 4, "norm_groups": 8},
           "mlp": mlp}
    glr = {"type": "hgrn2", "mixer": {"heads": W // 128, "dim": 128, "vdim": 128}, "mlp": mlp}

    def lat(kv_from=None):
        m = {"heads": sz["heads"], "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": sz.get("kv_rank", 512), "q_rank": 3 * W // 4,
             "scale": 192 ** -0.5, "rot": {"base": 10000.0, "dims": 64,
                                           "scaling": {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
        if kv_from is not None:
            m["kv_from"] = kv_from
        return {"type": "latent_attention", "mixer": m, "mlp": mlp}
    order = ["ssd", "glr", "ssd", "lat"]
    layers, first_lat = [], None
    for i in range(sz["layers"]):
        k = order[i % 4]
        if k == "lat":
            layers.append(lat(first_lat))
            first_lat = i if first_lat is None else first_lat
        else:
            layers.append(ssd if k == "ssd" else glr)
    return {"architecture": "Famepel", "embedding": {"scale": 1.0}, "layers": layers, "norm": {"eps": 1e-6},
            "vocab": sz["vocab"], "width": W}


def famepel_weights(desc: dict, seed: int) -> Dict[str, np.ndarray]:
    rng = np.random.default_rng(seed)
    W, V = desc["width"], desc["vocab"]

    def lin(n, k):
        return (rng.standard_normal((n, k), dtype=np.float32) / np.sqrt(k)).astype(np.float32)

    def vec(n, s=0.1, b=0.0):
        return (rng.standard_normal(n, dtype=np.float32) * s + b).astype(np.float32)
    w = {"embed": lin(V, W) * 4.0, "head": lin(V, W)}

    def norm(name):
        w[name], w[name + ".b"], w[name + ".alpha"] = vec(W, 0.1, 1.0), vec(W), np.float32(0.7).reshape(())
    norm("final.norm")
    for i, lc in enumerate(desc["layers"]):
        p, m, M = f"l{i}.", lc["mixer"], f"l{i}.mix."
        for n in ("norm1", "norm1b", "norm2", "norm2b"):
            norm(p + n)
        w[p + "ls1"], w[p + "ls2"] = vec(W, 0.1, 0.7), vec(W, 0.1, 0.7)
        if lc["type"] == "mamba2":
            H, inner, gn = m["heads"], m["heads"] * m["vdim"], m["groups"] * m["state"]
            w.update({M + "in": lin(2 * inner + 2 * gn + H, W), M + "conv": vec((inner + 2 * gn, m["conv"]), 0.5),
                      M + "conv.b": vec(inner + 2 * gn), M + "dt_bias": vec(H, 0.5, -1.0),
                      M + "A_log": np.log(rng.uniform(0.2, 2.0, H)).astype(np.float32), M + "D": vec(H, 0.3, 1.0),
                      M + "norm": vec(inner, 0.1, 1.0), M + "o": lin(W, inner)})
        elif lc["type"] == "latent_attention":
            H, R = m["heads"], m["kv_rank"]
            w.update({M + "dq": lin(m["q_rank"], W), M + "dq.norm": vec(m["q_rank"], 0.1, 1.0),
                      M + "uq": lin(H * (m["dim"] + m["rot_dim"]), m["q_rank"]), M + "uk": lin(H * m["dim"], R),
                      M + "uv": lin(H * m["vdim"], R), M + "sink": vec(H, 1.0), M + "o": lin(W, H * m["vdim"])})
            if m.get("kv_from") is None:
                w.update({M + "dkv": lin(R + m["rot_dim"], W), M + "dkv.norm": vec(R, 0.1, 1.0)})
        else:
            nq, nv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            w.update({M + "q": lin(nq, W), M + "f": lin(nq, W), M + "f.b": vec(nq, 0.5), M + "lower": rng.uniform(0, 0.9, nq).astype(np.float32),
                      M + "v": lin(nv, W), M + "norm": vec(m["vdim"], 0.1, 1.0), M + "o": lin(W, nv)})
        ff, E = lc["mlp"]["expert"]["ff"], lc["mlp"]["router"]["experts"]
        w[p + "mlp.router"] = lin(E, W) * 2.0
        for e in range(E):
            w[f"{p}mlp.e{e}.gate"], w[f"{p}mlp.e{e}.up"], w[f"{p}mlp.e{e}.down"] = lin(ff, W), lin(ff, W), lin(W, ff)
    return w


def vosolorn_description(sz: dict) -> dict:
    """Layers in the order matrix memory, matrix memory, window attention, matrix memory; feed-forwards alternate between
    the gated dense layer and the expert mixture.  Matrix memory in heads of 64 keys x 128 values (values = width), attention
    in heads of 128 over a window of 1024 tokens and pooled blocks of 16, half of each head rotated; experts of ff / top
    each (8 x top of them, `top` per token) beside a shared expert of the same size."""
    W, top = sz["width"], sz.get("top", 4)
    ffe = sz["ff"] // top
    moe = {"kind": "moe", "expert": {"ff": ffe}, "router": {"experts": 8 * top, "top": top}, "shared": {"ff": ffe}}
    dense = {"kind": "dense", "ff": sz["ff"]}
    mem = {"heads": W // 128, "dim": 64, "vdim": 128, "gate_cap": 12.0}
    att = {"heads": sz["heads"], "kv_heads": sz["kv_heads"], "dim": 128, "vdim": 128, "mask": {"size": 1024, "pool": 16},
           "rot": {"base": 1e6, "dims": 64}, "scale": 128 ** -0.5}
    layers = []
    for i in range(sz["layers"]):
        kind = "attention" if i % 4 == 2 or sz.get("all_attention") else "mlstm"
        layers.append({"type": kind, "mixer": att if kind == "attention" else mem, "mlp": moe if i % 2 else dense})
    return {"architecture": "Vosolorn", "layers": layers, "logit_scale": 1.0, "norm": {"eps": 1e-6}, "vocab": sz["vocab"], "width": W}


def vosolorn_weights(desc: dict, seed: int) -> Dict[str, np.ndarray]:
    rng = np.random.default_rng(seed)
    W, V = desc["width"], desc["vocab"]

    def lin(n, k):
        return (rng.standard_normal((n, k), dtype=np.float32) / np.sqrt(k)).astype(np.float32)

    def vec(n, s=0.1, b=0.0):
        return (rng.standard_normal(n, dtype=np.float32) * s + b).astype(np.float32)
    w = {"embed": lin(V, W) * 4.0, "embed.norm": vec(W, 0.1, 1.0), "final.norm": vec(W, 0.1, 1.0)}
    for i, lc in enumerate(desc["layers"]):
        p, m, M = f"l{i}.", lc["mixer"], f"l{i}.mix."
        w[p + "norm1"], w[p + "ls1"] = vec(W, 0.1, 1.0), vec(W, 0.1, 0.7)
        if lc["type"] == "attention":
            H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w.update({M + "q": lin(H * D, W), M + "k": lin(G * D, W), M + "v": lin(G * Dv, W), M + "q.norm": vec(D, 0.1, 1.0),
                      M + "k.norm": vec(D, 0.1, 1.0), M + "o": lin(W, H * Dv)})
        else:
            H, nq, nv = m["heads"], m["heads"] * m["dim"], m["heads"] * m["vdim"]
            w.update({M + "q": lin(nq, W), M + "k": lin(nq, W), M + "v": lin(nv, W), M + "g": lin(nv, W), M + "o": lin(W, nv),
                      M + "norm": vec(nv, 0.1, 1.0), M + "i": lin(H, W), M + "i.b": vec(H, 0.5), M + "f": lin(H, W),
                      M + "f.b": vec(H, 0.5, 3.0)})
        mlp = lc["mlp"]
        w[p + "norm2"], w[p + "ls2"] = vec(W, 0.1, 1.0), vec(W, 0.1, 0.7)
        if mlp["kind"] == "dense":
            w.update({p + "mlp.gate": lin(mlp["ff"], W), p + "mlp.up": lin(mlp["ff"], W), p + "mlp.down": lin(W, mlp["ff"])})
        else:
            ff, E = mlp["expert"]["ff"], mlp["router"]["experts"]
            w[p + "mlp.router"], w[p + "mlp.router.b"] = lin(E, W) * 2.0, vec(E, 0.3)
            for e in range(E):
                w[f"{p}mlp.e{e}.up"], w[f"{p}mlp.e{e}.down"] = lin(ff, W), lin(W, ff)
            w[p + "mlp.shared.up"], w[p + "mlp.shared.down"] = lin(mlp["shared"]["ff"], W), lin(W, mlp["shared"]["ff"])
    return w


def sebavik_description(sz: dict) -> dict:
    """Every layer: biased attention in heads of 128 over a window of 1024 tokens plus 64 kept first tokens, scores capped at
    30, values blended with the first layer's; feed-forwards alternate between the clamped gated dense layer and gated
    experts of ff / top each (8 x top of them, `top` per token); input convolutions of 4 taps, a token input of 32, a pair
    table of 65521 buckets, depth average."""
    W, top = sz["width"], sz.get("top", 4)
    moe = {"kind": "moe", "expert": {"ff": sz["ff"] // top}, "router": {"experts": 8 * top, "top": top}}
    dense = {"kind": "dense", "ff": sz["ff"], "limit": 7.0}
    att = {"heads": sz["heads"], "kv_heads": sz["kv_heads"], "dim": 128, "vdim": 128, "mask": {"size": 1024, "keep_first": 64},
           "scale": 128 ** -0.5, "softcap": 30.0, "v_mix": True}
    layers = [{"type": "attention", "mixer": att, "mlp": moe if i % 2 else dense} for i in range(sz["layers"])]
    return {"architecture": "Sebavik", "canon": {"taps": 4}, "embedding": {"scale": 1.0, "bigram": {"buckets": 65521, "mul_prev": 53, "mul_cur": 29}},
            "layers": layers, "norm": {"eps": 1e-6}, "residual_mult": 0.7, "token_side": {"dim": 32}, "vocab": sz["vocab"], "width": W}


def sebavik_weights(desc: dict, seed: int) -> Dict[str, np.ndarray]:
    rng = np.random.default_rng(seed)
    W, V, L = desc["width"], desc["vocab"], len(desc["layers"])
    taps, side = desc["canon"]["taps"], desc["token_side"]["dim"]

    def lin(n, k):
        return (rng.standard_normal((n, k), dtype=np.float32) / np.sqrt(k)).astype(np.float32)

    def vec(n, s=0.1, b=0.0):
        return (rng.standard_normal(n, dtype=np.float32) * s + b).astype(np.float32)
    w = {"embed": lin(V, W) * 4.0, "bigram": lin(desc["embedding"]["bigram"]["buckets"] + 1, W), "side.embed": lin(V, side * L) * 4.0,
         "final.norm": vec(W, 0.1, 1.0)}
    for i, lc in enumerate(desc["layers"]):
        p, m, M = f"l{i}.", lc["mixer"], f"l{i}.mix."
        H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        w.update({p + "norm1": vec(W, 0.1, 1.0), p + "ls1": vec(W, 0.1, 0.7), p + "canon1": vec((W, taps), 0.3),
                  p + "dwa": np.concatenate([vec(i + 1, 0.1), np.ones(1, np.float32)]),
                  M + "q": lin(H * D, W), M + "q.b": vec(H * D), M + "k": lin(G * D, W), M + "k.b": vec(G * D), M + "v": lin(G * Dv, W),
                  M + "v.b": vec(G * Dv), M + "vmix": np.float32(0.3).reshape(()), M + "r1": vec(H, 0.1, 0.5), M + "r2": vec(H, 0.01, 0.1),
                  M + "sink": vec(H, 1.0), M + "o": lin(W, H * Dv),
                  p + "side.gate": lin(side, W), p + "side.proj": lin(W, side), p + "side.norm": vec(W, 0.1, 1.0)})
        mlp = lc["mlp"]
        w.update({p + "norm2": vec(W, 0.1, 1.0), p + "ls2": vec(W, 0.1, 0.7), p + "canon2": vec((W, taps), 0.3)})
        if mlp["kind"] == "dense":
            w.update({p + "mlp.gate": lin(mlp["ff"], W), p + "mlp.up": lin(mlp["ff"], W), p + "mlp.down": lin(W, mlp["ff"])})
        else:
            ff, E = mlp["expert"]["ff"], mlp["router"]["experts"]
            w[p + "mlp.router"] = lin(E, W) * 2.0
            for e in range(E):
                w[f"{p}mlp.e{e}.gate"], w[f"{p}mlp.e{e}.up"], w[f"{p}mlp.e{e}.down"] = lin(ff, W), lin(ff, W), lin(W, ff)
    return w


def _sebavik_costs(desc: dict, hc, prompt: int) -> dict:
    """Multiply-adds per token per kernel group (the dense feed-forward counts under gemm_in / gemm_out, where its products
    run); for attention the multiply-adds of one whole prompt over the keys a position really sees."""
    W = desc["width"]
    per = {"gemm_in": 0, "gemm_out": 0, "small_gemm": 0, "experts": 0, "expert_weights": 0, "delta": 0, "attention_prompt": 0}
    for s in hc.layers:
        per["gemm_in"] += (s.b_heads * s.b_dim + s.b_kv_heads * (s.b_dim + s.b_vdim)) * W
        per["gemm_out"] += s.b_heads * s.b_vdim * W
        win = s.b_window if s.b_window > 0 else prompt
        seen = sum(min(i + 1, win) + min(s.b_keep_first, max(0, i + 1 - win)) for i in range(prompt))
        per["attention_prompt"] += seen * s.b_heads * (s.b_dim + s.b_vdim)
        if s.ff_kind == 3:
            per["gemm_in"] += 2 * s.ff * W
            per["gemm_out"] += s.ff * W
        elif s.ff_kind == 2:
            per["experts"] += s.x_top * 3 * s.ff * W
            per["expert_weights"] += s.x_experts * 3 * s.ff * W
    per["head"] = desc["vocab"] * W
    return per


def _vosolorn_costs(desc: dict, hc, prompt: int) -> dict:
    """Multiply-adds per token per kernel group (the dense feed-forward counts under gemm_in / gemm_out, where its products
    run); for attention the multiply-adds of one whole prompt, for the recurrence those of one token."""
    W = desc["width"]
    per = {"gemm_in": 0, "gemm_out": 0, "small_gemm": 0, "experts": 0, "expert_weights": 0, "delta": 0, "attention_prompt": 0}
    for s in hc.layers:
        if s.mixer == 5:
            per["gemm_in"] += (s.w_heads * s.w_dim + s.w_kv_heads * (s.w_dim + s.w_vdim)) * W
            per["gemm_out"] += s.w_heads * s.w_vdim * W
            seen = sum(min(i + 1, s.w_window) + max(0, (i - s.w_window + 1) // s.w_pool) for i in range(prompt))
            per["attention_prompt"] += seen * s.w_heads * (s.w_dim + s.w_vdim)
        else:
            per["gemm_in"] += (2 * s.t_heads * s.t_dim + 2 * s.t_heads * s.t_vdim + 2 * s.t_heads) * W
            per["gemm_out"] += s.t_heads * s.t_vdim * W
            per["delta"] += 2 * s.t_heads * s.t_dim * (s.t_vdim + 1)
        if s.ff_kind == 3:
            per["gemm_in"] += 2 * s.ff * W
            per["gemm_out"] += s.ff * W
        elif s.ff_kind == 2:
            per["experts"] += (s.x_top * s.ff + s.x_shared_ff) * 2 * W
            per["expert_weights"] += (s.x_experts * s.ff + s.x_shared_ff) * 2 * W
    per["head"] = desc["vocab"] * W
    return per


def _famepel_costs(desc: dict, hc, prompt: int = 0) -> dict:
    """Multiply-adds per token per kernel group; for the experts both the work of a token (its `top` experts) and the
    weights of ALL experts (what a long prefill streams once per step)."""
    W = desc["width"]
    per = {"gemm_in": 0, "gemm_out": 0, "small_gemm": 0, "experts": 0, "expert_weights": 0, "delta": 0, "attention_prompt": 0}
    for s in hc.layers:
        if s.mixer == 2:
            inner = s.m_heads * s.m_vdim
            per["gemm_in"] += (2 * inner + 2 * s.m_groups * s.m_state + s.m_heads) * W
            per["gemm_out"] += inner * W
        elif s.mixer == 3:
            own = s.l_kv_from < 0
            per["gemm_in"] += (s.l_q_rank + (s.l_kv_rank + s.l_rot_dim if own else 0)) * W
            per["gemm_out"] += s.l_heads * s.l_vdim * W
            per["small_gemm"] += s.l_heads * ((s.l_dim + s.l_rot_dim) * s.l_q_rank + s.l_dim * s.l_kv_rank + s.l_vdim * s.l_kv_rank)
            per["attention_prompt"] += prompt * (prompt + 1) // 2 * s.l_heads * (2 * s.l_kv_rank + s.l_rot_dim)
        else:
            per["gemm_in"] += (2 * s.g_heads * s.g_dim + s.g_heads * s.g_vdim) * W
            per["gemm_out"] += s.g_heads * s.g_vdim * W
            per["delta"] += 2 * s.g_heads * s.g_dim * s.g_vdim
        if s.ff_kind == 2:
            per["experts"] += s.x_top * 3 * s.ff * W
            per["expert_weights"] += s.x_experts * 3 * s.ff * W
    per["head"] = desc["vocab"] * W
    return per


def _hybrid_costs(desc: dict, hc, prompt: int = 0) -> dict:
    """Multiply-add FLOPs per token and weight bytes per kernel group (bf16 weights)."""
    if desc["architecture"] == "Famepel":
        return _famepel_costs(desc, hc, prompt)
    if desc["architecture"] == "Vosolorn":
        return _vosolorn_costs(desc, hc, prompt)
    if desc["architecture"] == "Sebavik":
        return _sebavik_costs(desc, hc, prompt)
    W = desc["width"]
    per = {"gemm_in": 0, "gemm_out": 0, "small_gemm": 0}
    for s in hc.layers:
        if s.mixer == 0:
            n_in = s.a_heads * s.a_dim + s.a_kv_heads * s.a_dim + s.a_heads * s.a_vdim + 2 * s.s_inner + s.ff
            k_out = s.a_heads * s.a_vdim + s.s_inner + s.ff
            small = (s.s_dt_rank + 2 * s.s_state) * s.s_inner + s.s_inner * s.s_dt_rank
        else:
            nq, nv = s.d_kv_heads * s.d_dim, s.d_heads * s.d_vdim
            n_in = 2 * nq + nv + s.d_heads + s.d_low_a + s.d_low_g + s.ff
            k_out = nv + s.ff
            small = s.d_heads * s.d_dim * s.d_low_a + nv * s.d_low_g
        per["gemm_in"] += n_in * W
        per["gemm_out"] += k_out * W
        per["small_gemm"] += small
    per["head"] = desc["vocab"] * W
    return per


def run_hybrid(size: str, prompt: int, decode_steps: int, batches: List[int], peaks: dict, seed: int = 0,
               design: str = "Kinetar") -> dict:
    from .hybrid_config import HybridConfig
    from .hybrid_runtime import HybridRuntime
    sz = SIZES[size]
    if design == "Famepel":
        desc = famepel_description(sz)
        w = famepel_weights(desc, seed)
    elif design in ("Vosolorn", "VosolornAttention"):
        desc = vosolorn_description(dict(sz, all_attention=design == "VosolornAttention"))
        w = vosolorn_weights(desc, seed)
    elif design == "Sebavik":
        desc = sebavik_description(sz)
        w = sebavik_weights(desc, seed)
    else:
        desc = hybrid_description(sz)
        w = hybrid_weights(desc, seed)
    hc = HybridConfig.from_dict(desc, {k: v.shape for k, v in w.items()})
    page = 256
    maxb = max(batches)
    pages_per = -(-(prompt + decode_steps + 1) // page)
    rt = HybridRuntime(hc, dtype="bfloat16", max_step_tokens=2048, max_step_entries=maxb, page_size=page,
                       num_pages=pages_per * maxb, max_pages_per_seq=pages_per, num_slots=maxb, max_want=maxb)
    rt.load_state_dict(w)
    del w
    rng = np.random.default_rng(seed + 1)
    # every request decodes its own token stream (routed layers would otherwise send all of a batch to the same experts)
    toks_all = [rng.integers(0, sz["vocab"], prompt + decode_steps + 1).tolist() for _ in range(maxb)]
    costs = _hybrid_costs(desc, hc, prompt)
    out = {"size": size, "description": {k: sz[k] for k in sz}, "memory": rt.memory_info()}

    def prefill(slot):
        ms, at = 0.0, 0
        toks = toks_all[slot]
        pages = list(range(slot * pages_per, (slot + 1) * pages_per))
        while at < prompt:
            n = min(2048, prompt - at)
            rt.step([(toks[at:at + n], at, slot, pages)], [n - 1] if at + n == prompt else [], want_logits=False, sample=True)
            ms += float(rt.lib.hy_last_step_ms(rt.h))
            at += n
        return ms
    for _ in range(3):
        prefill(0)
    rt.profile(True)
    t0 = time.perf_counter()
    runs = [prefill(0) for _ in range(3)]
    wall = (time.perf_counter() - t0) / 3
    prof = rt.profile_read()
    rt.profile(False)
    ms = float(np.median(runs))
    out["prefill"] = {"tokens": prompt, "device_ms": ms, "tokens_per_s": prompt / ms * 1e3, "e2e_tokens_per_s": prompt / wall,
                      "ms_by_group": {k: v / 3 for k, v in prof.items()}}
    tf = {}
    for g in ("gemm_in", "gemm_out") + (("experts",) if costs.get("experts") else ()):
        t = prof[g] / 3 * 1e-3
        tf[g] = {"tflops": 2.0 * costs[g] * prompt / t / 1e12, "of_measured_bf16_peak": 2.0 * costs[g] * prompt / t / 1e12 / peaks["bf16_tflops"]}
    # the mixers' own kernels: achieved multiply-add rate (a recurrence runs on the fp32 pipes, attention here too or on
    # mma.sync); the two designs' figures stand side by side in the comparison
    if costs.get("delta") and prof.get("delta"):
        tf["recurrence"] = {"tflops": 2.0 * costs["delta"] * prompt / (prof["delta"] / 3 * 1e-3) / 1e12}
    if costs.get("attention_prompt") and prof.get("attention"):
        tf["attention"] = {"tflops": 2.0 * costs["attention_prompt"] / (prof["attention"] / 3 * 1e-3) / 1e12}
    out["prefill"]["roofline"] = tf
    out["decode"] = {}
    for B in batches:
        for s in range(B):
            prefill(s)
        entries = lambda step: [([toks_all[s][prompt + step]], prompt + step, s, list(range(s * pages_per, (s + 1) * pages_per)))
                                for s in range(B)]
        for step in range(3):
            rt.step(entries(step), list(range(B)), want_logits=False, sample=True)
        rt.profile(True)
        ms = 0.0
        t0 = time.perf_counter()
        for step in range(3, decode_steps):
            rt.step(entries(step), list(range(B)), want_logits=False, sample=True)
            ms += float(rt.lib.hy_last_step_ms(rt.h))
        wall = time.perf_counter() - t0
        n = decode_steps - 3
        prof = rt.profile_read()
        rt.profile(False)
        roof = {}
        for g in ("gemm_in", "gemm_out", "head"):
            t = prof[g] / n * 1e-3
            roof[g] = {"gb_per_s": 2.0 * costs[g] / t / 1e9, "of_measured_hbm": 2.0 * costs[g] / t / 1e9 / peaks["hbm_gbs"]}
        if costs.get("experts"):
            # a decoded token reads its `top` experts; B tokens at most B times that (they may share experts)
            t = prof["experts"] / n * 1e-3
            roof["experts"] = {"gb_per_s_if_no_expert_is_shared": 2.0 * costs["experts"] * B / t / 1e9,
                               "of_measured_hbm": min(2.0 * costs["experts"] * B, 2.0 * costs["expert_weights"]) / t / 1e9 / peaks["hbm_gbs"]}
        wbytes = 2.0 * sum(v for k, v in costs.items() if k not in ("expert_weights", "delta", "attention_prompt"))
        out["decode"][f"batch{B}"] = {"ms_per_step": ms / n, "tokens_per_s": B * n / ms * 1e3, "e2e_tokens_per_s": B * n / wall,
                                      "ms_by_group": {k: v / n for k, v in prof.items()}, "roofline": roof,
                                      "weights_over_time_of_measured_hbm": wbytes / (ms / n * 1e-3) / 1e9 / peaks["hbm_gbs"]}
    out["launches"] = rt.launches
    rt.close()
    return out


def run_qwen2(size: str, prompt: int, decode_steps: int, batches: List[int], peaks: dict, seed: int = 0) -> dict:
    """The closest existing model: Qwen2 of the same width / depth / feed-forward / heads through JacobiRuntime (prefill in
    chunks of 2048 rows; decoding = one row per request per forward)."""
    import torch
    from .runtime import JacobiRuntime, PAGE
    sz = SIZES[size]
    cfg = dict(hidden_size=sz["width"], num_hidden_layers=sz["layers"], num_attention_heads=sz["heads"],
               num_key_value_heads=sz["kv_heads"], head_dim=sz["dim"], intermediate_size=sz["ff"], vocab_size=sz["vocab"],
               tie_word_embeddings=False, rope_theta=1e6, max_position_embeddings=32768, rms_norm_eps=1e-6)
    maxb = max(batches)
    pages_per = -(-(prompt + decode_steps + 64) // PAGE)
    rt = JacobiRuntime(cfg, max_rows=2048, max_seqs=maxb, num_kv_pages=pages_per * maxb + 1, max_pages_per_seq=pages_per)
    import bench as _bench
    _bench.load_random_weights(rt, cfg, seed, "cuda")
    hd = cfg["head_dim"]
    inv = 1.0 / (cfg["rope_theta"] ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))
    ang = torch.arange(prompt + decode_steps + 64, dtype=torch.float32)[:, None] * inv[None, :]
    emb = torch.cat([ang, ang], -1)
    rt.set_rope_tables(emb.cos().numpy(), emb.sin().numpy())
    rng = np.random.default_rng(seed + 1)
    toks = rng.integers(0, sz["vocab"], prompt + decode_steps + 1).tolist()
    out = {"size": size}

    def prefill():
        s = rt.new_sequence()
        _, _, ms = rt.prefill(s, toks[:prompt], [])
        return s, ms
    for _ in range(3):
        s, _ = prefill()
        rt.release(s)
    runs = []
    t0 = time.perf_counter()
    for _ in range(3):
        s, ms = prefill()
        rt.release(s)
        runs.append(ms)
    wall = (time.perf_counter() - t0) / 3
    ms = float(np.median(runs))
    W, I, L = sz["width"], sz["ff"], sz["layers"]
    qkv = (sz["heads"] + 2 * sz["kv_heads"]) * sz["dim"]
    wparams = L * (qkv * W + sz["heads"] * sz["dim"] * W + 3 * W * I)
    out["prefill"] = {"tokens": prompt, "device_ms": ms, "tokens_per_s": prompt / ms * 1e3, "e2e_tokens_per_s": prompt / wall,
                      "layer_gemm_tflops_if_all_time_were_gemm": 2.0 * wparams * prompt / (ms * 1e-3) / 1e12}
    out["decode"] = {}
    for B in batches:
        seqs = [prefill()[0] for _ in range(B)]
        ms, n = 0.0, 0
        t0 = None
        for step in range(decode_steps):
            if step == 3:
                t0 = time.perf_counter()
            groups = [(k, 1, k, prompt + step) for k in range(B)]
            commits = [(k, k, prompt + step) for k in range(B)]
            for s in seqs:
                rt.ensure_capacity(s, prompt + step + 1)
            r = rt.forward([toks[prompt + step]] * B, groups, seqs, 0, B, commits)
            if step >= 3:
                ms += r["ms"]
                n += 1
        wall = time.perf_counter() - t0
        wbytes = 2.0 * (wparams + sz["vocab"] * W)
        out["decode"][f"batch{B}"] = {"ms_per_step": ms / n, "tokens_per_s": B * n / ms * 1e3, "e2e_tokens_per_s": B * n / wall,
                                      "weights_over_time_of_measured_hbm": wbytes / (ms / n * 1e-3) / 1e9 / peaks["hbm_gbs"]}
        for s in seqs:
            rt.release(s)
    out["launches"] = int(rt.launches)
    rt.close()
    return out
