"""Configuration of layered hybrid decoders: a list of layers over one residual stream.

Architecture "Kinetar": each layer is a mixer beside a feed-forward that share one RMS norm.  Mixers: "parallel" (softmax
attention with a sink whose values are its keys, beside a selective scan) and "channel_delta" (gated delta rule with a
decay per key channel); squared-ReLU feed-forward; sinusoidal positions.

Architecture "Famepel": each layer is norm - mixer - norm, then norm - feed-forward - norm, with element-wise tanh norms
and a per-channel layer scale on each sublayer.  Mixers: "mamba2" (state-space recurrence with one decay per head),
"latent_attention" (attention over a shared low-rank latent with a rotated key part and a sink; a layer may use an earlier
layer's cached latent), "hgrn2" (gated linear recurrence); routed gated experts; positions only through the rotation.

Architecture "Vosolorn": the sublayers read the residual stream itself and an RMS norm with a layer scale sits on each
sublayer's output; the embedding is normed and serves as the output head.  Mixers: "attention" (softmax attention over a
sliding window plus one pooled key / value per block of tokens whose last token is already behind the window, per-head query / key
norms, interleaved rotary pairs, values rotated by their own position) and "mlstm" (matrix memory with capped
exponential gates under a running maximum); feed-forward "dense" (gated, tanh-gelu) or "moe" (plain erf-gelu experts
chosen by the largest router logits plus a bias, softmax over the chosen, beside a shared expert).

Architecture "Sebavik": pre-norm blocks whose sublayers read the RMS-normed stream through a short causal convolution over
time (h + conv(h)) and whose results are scaled per channel and by one factor of the model; a per-layer token input (a
slice of a second embedding table, gated by the stream) and a weighted average over the depth close every layer.  Mixer
"attention": no rotation; scores scaled, capped by a tanh and lowered by a logarithmic distance bias; a sliding window
plus the sequence's first tokens; a per-head sink in the softmax's denominator; biased projections; values blended with
those of the first such layer.  Feed-forward "dense" (clamped gated pair) or "moe" (gated silu experts chosen by the
largest router logits, softmax over the chosen).  The scaled embedding gets a hashed embedding of the (previous, current)
token pair added and serves as the output head.

Every size and every constant that can differ between models is read from config.json; sizes that only the tensors know
(the inner sizes of the two-step decay and gate projections) are read from the checkpoint's tensor shapes."""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import numpy as np

MIX_ATTN_SCAN, MIX_DELTA, MIX_SSD, MIX_LATENT, MIX_GLR, MIX_WINDOW, MIX_MLSTM, MIX_BIASED = 0, 1, 2, 3, 4, 5, 6, 7
FF_NONE, FF_RELU2, FF_ROUTED, FF_GATED = 0, 1, 2, 3
ACT_SILU, ACT_GELU_TANH, ACT_GELU_ERF, ACT_CLAMPED = 0, 1, 2, 3
ROUTE_SIGMOID_GROUPS, ROUTE_TOP_SOFTMAX = 0, 1
NORM_RMS_OFFSET, NORM_TANH, NORM_RMS = 0, 1, 2
BLOCK_PARALLEL, BLOCK_SANDWICH, BLOCK_POSTNORM, BLOCK_PRENORM = 0, 1, 2, 3
POS_SINUSOID, POS_NONE = 0, 1
_ST_DTYPES = {"BF16": (0, 2), "F32": (1, 4), "F16": (2, 2), "I32": (3, 4)}


@dataclass
class LayerSpec:
    mixer: int
    # attention beside scan
    a_heads: int = 0
    a_kv_heads: int = 0
    a_dim: int = 0
    a_vdim: int = 0
    a_conv: int = 1
    a_qt_every: int = 1
    a_scale: float = 1.0
    a_qt_coef: float = 0.0
    s_inner: int = 0
    s_state: int = 0
    s_dt_rank: int = 0
    s_conv: int = 1
    left_scale: float = 1.0
    right_scale: float = 1.0
    # gated delta rule
    d_heads: int = 0
    d_kv_heads: int = 0
    d_dim: int = 0
    d_vdim: int = 0
    d_conv: int = 1
    d_low_a: int = 0
    d_low_g: int = 0
    ff_kind: int = FF_NONE
    ff: int = 0
    # state-space recurrence with one decay per head
    m_heads: int = 0
    m_vdim: int = 0
    m_state: int = 0
    m_groups: int = 1
    m_conv: int = 1
    m_norm_groups: int = 1
    # attention over a shared latent
    l_heads: int = 0
    l_dim: int = 0
    l_rot_dim: int = 0
    l_vdim: int = 0
    l_kv_rank: int = 0
    l_q_rank: int = 0
    l_kv_from: int = -1
    l_scale: float = 1.0
    r_dims: int = 0
    r_base: float = 10000.0
    r_factor: float = 0.0
    r_original: float = 0.0
    r_fast: float = 0.0
    r_slow: float = 0.0
    # gated linear recurrence
    g_heads: int = 0
    g_dim: int = 0
    g_vdim: int = 0
    # routed experts
    x_experts: int = 0
    x_top: int = 0
    x_groups: int = 1
    x_keep: int = 1
    x_scale: float = 1.0
    x_route: int = ROUTE_SIGMOID_GROUPS
    x_plain: int = 0
    x_act: int = ACT_SILU
    x_shared_ff: int = 0
    ff_act: int = ACT_SILU
    # attention over a window and pooled blocks
    w_heads: int = 0
    w_kv_heads: int = 0
    w_dim: int = 0
    w_vdim: int = 0
    w_window: int = 1
    w_pool: int = 1
    w_rot_dims: int = 0
    w_rot_values: int = 0
    w_qk_norm: int = 0
    w_rot_base: float = 10000.0
    w_scale: float = 1.0
    # matrix memory
    t_heads: int = 0
    t_dim: int = 0
    t_vdim: int = 0
    t_gate_cap: float = 0.0
    # attention with capped scores, a distance bias, a window plus kept first tokens and a sink
    b_heads: int = 0
    b_kv_heads: int = 0
    b_dim: int = 0
    b_vdim: int = 0
    b_window: int = 0
    b_keep_first: int = 0
    b_v_mix: int = 0
    b_scale: float = 1.0
    b_softcap: float = 0.0
    ff_limit: float = 0.0

    def cache_elems_per_token(self) -> int:
        """Elements this layer keeps in the paged cache for every token of a request."""
        if self.mixer == MIX_ATTN_SCAN:
            return self.a_kv_heads * self.a_dim
        if self.mixer == MIX_LATENT and self.l_kv_from < 0:
            return self.l_kv_rank + self.l_rot_dim
        if self.mixer == MIX_WINDOW:                  # keys and values, and their pooled blocks
            return -(-self.w_kv_heads * (self.w_dim + self.w_vdim) * (self.w_pool + 1) // self.w_pool)
        if self.mixer == MIX_BIASED:
            return self.b_kv_heads * (self.b_dim + self.b_vdim)
        return 0


def _ssd_spec(m: dict) -> LayerSpec:
    heads, groups = int(m["heads"]), int(m["groups"])
    if groups <= 0 or heads % groups:
        raise ValueError("mamba2: heads must be a multiple of groups")
    if (heads * int(m["vdim"])) % int(m["norm_groups"]):
        raise ValueError("mamba2: heads * vdim must be a multiple of norm_groups")
    return LayerSpec(MIX_SSD, m_heads=heads, m_vdim=int(m["vdim"]), m_state=int(m["state"]), m_groups=groups,
                     m_conv=int(m["conv"]), m_norm_groups=int(m["norm_groups"]))


def _latent_spec(m: dict, i: int, done: List[LayerSpec]) -> LayerSpec:
    rot = m["rot"]
    sc = rot.get("scaling") or None
    spec = LayerSpec(MIX_LATENT, l_heads=int(m["heads"]), l_dim=int(m["dim"]), l_rot_dim=int(m["rot_dim"]),
                     l_vdim=int(m["vdim"]), l_kv_rank=int(m["kv_rank"]), l_q_rank=int(m["q_rank"]),
                     l_kv_from=-1 if m.get("kv_from") is None else int(m["kv_from"]), l_scale=float(m["scale"]),
                     r_dims=int(rot["dims"]), r_base=float(rot["base"]))
    if sc:
        spec.r_factor, spec.r_original = float(sc["factor"]), float(sc["original"])
        spec.r_fast, spec.r_slow = float(sc["fast"]), float(sc["slow"])
    if spec.r_dims % 2 or spec.r_dims > spec.l_rot_dim:
        raise ValueError("latent_attention: rot.dims must be even and at most rot_dim")
    j = spec.l_kv_from
    if j >= 0:
        if j >= i or done[j].mixer != MIX_LATENT or done[j].l_kv_from >= 0:
            raise ValueError(f"layer {i}: kv_from must name an earlier latent_attention layer with a down-projection of its own")
        if (done[j].l_kv_rank, done[j].l_rot_dim) != (spec.l_kv_rank, spec.l_rot_dim):
            raise ValueError(f"layer {i}: kv_rank and rot_dim must equal those of layer {j}")
    return spec


def _routed_ff(spec: LayerSpec, mlp: dict) -> None:
    r = mlp["router"]
    spec.ff_kind, spec.ff = FF_ROUTED, int(mlp["expert"]["ff"])
    spec.x_experts, spec.x_top, spec.x_scale = int(r["experts"]), int(r["top"]), float(r["scale"])
    g = r.get("groups") or {"count": 1, "keep": 1}
    spec.x_groups, spec.x_keep = int(g["count"]), int(g["keep"])
    if spec.x_groups <= 0 or spec.x_experts % spec.x_groups or not 1 <= spec.x_keep <= spec.x_groups:
        raise ValueError("routed feed-forward: experts must split into groups.count equal groups, 1 <= keep <= count")
    if not 1 <= spec.x_top <= spec.x_keep * (spec.x_experts // spec.x_groups):
        raise ValueError("routed feed-forward: top exceeds the experts a token may choose from")


def _window_spec(m: dict) -> LayerSpec:
    rot, mask = m.get("rot") or {}, m["mask"]
    spec = LayerSpec(MIX_WINDOW, w_heads=int(m["heads"]), w_kv_heads=int(m["kv_heads"]), w_dim=int(m["dim"]),
                     w_vdim=int(m["vdim"]), w_window=int(mask["size"]), w_pool=int(mask["pool"]),
                     w_rot_dims=int(rot.get("dims", 0)), w_rot_values=1 if rot else 0, w_qk_norm=1,
                     w_rot_base=float(rot.get("base", 10000.0)), w_scale=float(m["scale"]))
    if spec.w_kv_heads <= 0 or spec.w_heads % spec.w_kv_heads:
        raise ValueError("attention: heads must be a multiple of kv_heads")
    if spec.w_rot_dims % 2 or spec.w_rot_dims > spec.w_dim:
        raise ValueError("attention: rot.dims must be even and at most dim")
    if spec.w_rot_values and spec.w_vdim % 2:
        raise ValueError("attention: rotated values need an even vdim")
    if spec.w_window < 1 or spec.w_pool < 1:
        raise ValueError("attention: mask.size and mask.pool must be at least 1")
    return spec


def _plain_experts_ff(spec: LayerSpec, mlp: dict) -> None:
    r = mlp["router"]
    spec.ff_kind, spec.ff = FF_ROUTED, int(mlp["expert"]["ff"])
    spec.x_experts, spec.x_top = int(r["experts"]), int(r["top"])
    spec.x_route, spec.x_plain, spec.x_act = ROUTE_TOP_SOFTMAX, 1, ACT_GELU_ERF
    spec.x_shared_ff = int(mlp["shared"]["ff"]) if mlp.get("shared") else 0
    if not 1 <= spec.x_top <= spec.x_experts:
        raise ValueError("mixture of experts: top must lie in 1..experts")


def _biased_spec(m: dict) -> LayerSpec:
    mask = m.get("mask") or {}
    spec = LayerSpec(MIX_BIASED, b_heads=int(m["heads"]), b_kv_heads=int(m["kv_heads"]), b_dim=int(m["dim"]),
                     b_vdim=int(m["vdim"]), b_window=int(mask.get("size") or 0), b_keep_first=int(mask.get("keep_first") or 0),
                     b_v_mix=1 if m.get("v_mix") else 0, b_scale=float(m["scale"]), b_softcap=float(m.get("softcap") or 0.0))
    if spec.b_heads <= 0 or spec.b_kv_heads <= 0 or spec.b_heads % spec.b_kv_heads:
        raise ValueError("attention: heads must be a positive multiple of kv_heads")
    if spec.b_dim <= 0 or spec.b_vdim <= 0:
        raise ValueError("attention: dim and vdim must be positive")
    if spec.b_window < 0 or spec.b_keep_first < 0:
        raise ValueError("attention: mask.size and mask.keep_first must not be negative")
    return spec


def _gated_experts_ff(spec: LayerSpec, mlp: dict) -> None:
    r = mlp["router"]
    spec.ff_kind, spec.ff = FF_ROUTED, int(mlp["expert"]["ff"])
    spec.x_experts, spec.x_top = int(r["experts"]), int(r["top"])
    spec.x_route, spec.x_plain, spec.x_act = ROUTE_TOP_SOFTMAX, 0, ACT_SILU
    if not 1 <= spec.x_top <= spec.x_experts:
        raise ValueError("mixture of experts: top must lie in 1..experts")


@dataclass
class HybridConfig:
    architecture: str
    width: int
    vocab: int
    emb_scale: float
    logit_scale: float
    norm_eps: float
    layers: List[LayerSpec] = field(default_factory=list)
    norm_kind: int = NORM_RMS_OFFSET
    block_kind: int = BLOCK_PARALLEL
    pos_kind: int = POS_SINUSOID
    embed_norm: bool = False
    tied_head: bool = False
    resid_mult: float = 1.0
    canon_taps: int = 0
    side_dim: int = 0
    depth_avg: int = 0
    pair_buckets: int = 0
    pair_mul_prev: int = 0
    pair_mul_cur: int = 0
    # what the engine's configuration reads from a model description
    max_position_embeddings: int = 1 << 30          # positions enter through a sinusoid or a rotation: no table to run out of
    is_hybrid: bool = True

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, cfg: dict, shapes: Optional[Dict[str, Tuple[int, ...]]] = None) -> "HybridConfig":
        """cfg: the parsed config.json; shapes: tensor name -> shape (needed by channel_delta layers)."""
        if cfg.get("architecture") == "Famepel":
            return cls._famepel(cfg)
        if cfg.get("architecture") == "Vosolorn":
            return cls._vosolorn(cfg)
        if cfg.get("architecture") == "Sebavik":
            return cls._sebavik(cfg)
        layers = []
        for i, lc in enumerate(cfg["layers"]):
            m = lc["mixer"]
            kind = lc["type"]
            if kind == "parallel":
                a, s = m["left"], m["right"]
                qt = a.get("q_temp") or {"coef": 0.0, "every": 1}
                spec = LayerSpec(MIX_ATTN_SCAN, a_heads=int(a["heads"]), a_kv_heads=int(a["kv_heads"]), a_dim=int(a["dim"]),
                                 a_vdim=int(a["vdim"]), a_conv=int(a["conv"]), a_qt_every=int(qt["every"]),
                                 a_scale=float(a["scale"]), a_qt_coef=float(qt["coef"]), s_inner=int(s["inner"]),
                                 s_state=int(s["state"]), s_dt_rank=int(s["dt_rank"]), s_conv=int(s["conv"]),
                                 left_scale=float(m["left_scale"]), right_scale=float(m["right_scale"]))
            elif kind == "channel_delta":
                if shapes is None:
                    raise ValueError("channel_delta layers need the checkpoint's tensor shapes")
                spec = LayerSpec(MIX_DELTA, d_heads=int(m["heads"]), d_kv_heads=int(m["kv_heads"]), d_dim=int(m["dim"]),
                                 d_vdim=int(m["vdim"]), d_conv=int(m["conv"]),
                                 d_low_a=int(shapes[f"l{i}.mix.a1"][0]), d_low_g=int(shapes[f"l{i}.mix.g1"][0]))
            else:
                raise NotImplementedError(f"layer type {kind!r}")
            mlp = lc.get("mlp")
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise NotImplementedError(f"feed-forward kind {mlp.get('kind')!r}")
                spec.ff_kind, spec.ff = FF_RELU2, int(mlp["ff"])
            layers.append(spec)
        return cls(architecture=cfg["architecture"], width=int(cfg["width"]), vocab=int(cfg["vocab"]),
                   emb_scale=float(cfg["embedding"]["scale"]), logit_scale=float(cfg["logit_scale"]),
                   norm_eps=float(cfg["norm"]["eps"]), layers=layers)

    @classmethod
    def _famepel(cls, cfg: dict) -> "HybridConfig":
        layers: List[LayerSpec] = []
        for i, lc in enumerate(cfg["layers"]):
            kind, m = lc["type"], lc["mixer"]
            if kind == "mamba2":
                spec = _ssd_spec(m)
            elif kind == "latent_attention":
                spec = _latent_spec(m, i, layers)
            elif kind == "hgrn2":
                spec = LayerSpec(MIX_GLR, g_heads=int(m["heads"]), g_dim=int(m["dim"]), g_vdim=int(m["vdim"]))
            else:
                raise NotImplementedError(f"layer type {kind!r}")
            mlp = lc.get("mlp")
            if mlp is not None:
                if mlp.get("kind") != "moe":
                    raise NotImplementedError(f"feed-forward kind {mlp.get('kind')!r}")
                _routed_ff(spec, mlp)
            layers.append(spec)
        return cls(architecture="Famepel", width=int(cfg["width"]), vocab=int(cfg["vocab"]),
                   emb_scale=float(cfg["embedding"]["scale"]), logit_scale=1.0, norm_eps=float(cfg["norm"]["eps"]),
                   layers=layers, norm_kind=NORM_TANH, block_kind=BLOCK_SANDWICH, pos_kind=POS_NONE)

    @classmethod
    def _vosolorn(cls, cfg: dict) -> "HybridConfig":
        layers: List[LayerSpec] = []
        for lc in cfg["layers"]:
            kind, m = lc["type"], lc["mixer"]
            if kind == "attention":
                spec = _window_spec(m)
            elif kind == "mlstm":
                spec = LayerSpec(MIX_MLSTM, t_heads=int(m["heads"]), t_dim=int(m["dim"]), t_vdim=int(m["vdim"]),
                                 t_gate_cap=float(m["gate_cap"]))
            else:
                raise NotImplementedError(f"layer type {kind!r}")
            mlp = lc.get("mlp")
            if mlp is not None:
                if mlp.get("kind") == "dense":
                    spec.ff_kind, spec.ff, spec.ff_act = FF_GATED, int(mlp["ff"]), ACT_GELU_TANH
                elif mlp.get("kind") == "moe":
                    _plain_experts_ff(spec, mlp)
                else:
                    raise NotImplementedError(f"feed-forward kind {mlp.get('kind')!r}")
            layers.append(spec)
        return cls(architecture="Vosolorn", width=int(cfg["width"]), vocab=int(cfg["vocab"]), emb_scale=1.0,
                   logit_scale=float(cfg.get("logit_scale", 1.0)), norm_eps=float(cfg["norm"]["eps"]), layers=layers,
                   norm_kind=NORM_RMS, block_kind=BLOCK_POSTNORM, pos_kind=POS_NONE, embed_norm=True, tied_head=True)

    @classmethod
    def _sebavik(cls, cfg: dict) -> "HybridConfig":
        layers: List[LayerSpec] = []
        mixes = []
        for i, lc in enumerate(cfg["layers"]):
            if lc["type"] != "attention":
                raise NotImplementedError(f"layer type {lc['type']!r}")
            spec = _biased_spec(lc["mixer"])
            if spec.b_v_mix:
                mixes.append(spec)
                if (spec.b_kv_heads, spec.b_vdim) != (mixes[0].b_kv_heads, mixes[0].b_vdim):
                    raise ValueError(f"layer {i}: blended values need the kv_heads and vdim of the first blending layer")
            mlp = lc.get("mlp")
            if mlp is not None:
                if mlp.get("kind") == "dense":
                    spec.ff_kind, spec.ff, spec.ff_act, spec.ff_limit = FF_GATED, int(mlp["ff"]), ACT_CLAMPED, float(mlp["limit"])
                elif mlp.get("kind") == "moe":
                    _gated_experts_ff(spec, mlp)
                else:
                    raise NotImplementedError(f"feed-forward kind {mlp.get('kind')!r}")
            layers.append(spec)
        emb = cfg["embedding"]
        pair = emb.get("bigram") or {}
        taps = int((cfg.get("canon") or {}).get("taps", 0))
        if not 0 <= taps <= 16:
            raise ValueError("canon.taps must lie in 0..16")
        return cls(architecture="Sebavik", width=int(cfg["width"]), vocab=int(cfg["vocab"]), emb_scale=float(emb.get("scale", 1.0)),
                   logit_scale=1.0, norm_eps=float(cfg["norm"]["eps"]), layers=layers, norm_kind=NORM_RMS,
                   block_kind=BLOCK_PRENORM, pos_kind=POS_NONE, tied_head=True, resid_mult=float(cfg.get("residual_mult", 1.0)),
                   canon_taps=taps, side_dim=int((cfg.get("token_side") or {}).get("dim", 0)), depth_avg=1,
                   pair_buckets=int(pair.get("buckets", 0)), pair_mul_prev=int(pair.get("mul_prev", 0)),
                   pair_mul_cur=int(pair.get("mul_cur", 0)))

    @classmethod
    def from_dir(cls, path: str) -> "HybridConfig":
        with open(os.path.join(path, "config.json")) as f:
            cfg = json.load(f)
        shapes = {}
        for name in sorted(os.listdir(path)):
            if name.endswith(".safetensors"):
                shapes.update({k: tuple(v[1]) for k, v in read_safetensors_header(os.path.join(path, name))[0].items()})
        return cls.from_dict(cfg, shapes)


def read_safetensors_header(path: str):
    """({name: (dtype, shape, begin, end)}, offset of the data section).  The file is an 8-byte little-endian length, that
    many bytes of JSON, then the data."""
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        hdr = json.loads(f.read(n))
    out = {k: (v["dtype"], v["shape"], v["data_offsets"][0], v["data_offsets"][1]) for k, v in hdr.items() if k != "__metadata__"}
    return out, 8 + n


def iter_safetensors(path: str):
    """(name, dtype code of the C ABI, shape, contiguous numpy byte view) for every tensor of one file."""
    hdr, base = read_safetensors_header(path)
    data = np.memmap(path, dtype=np.uint8, mode="r")
    for name, (dt, shape, b, e) in hdr.items():
        if dt not in _ST_DTYPES:
            raise ValueError(f"tensor {name}: dtype {dt} is not supported")
        yield name, _ST_DTYPES[dt][0], list(shape), np.ascontiguousarray(data[base + b:base + e])
