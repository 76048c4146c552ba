"""Host-side pieces of the Vosolorn design (no GPU): configuration reader and registry, the binding's structures against the
header, and closed forms of the plain oracle's mechanisms (the oracle is the yardstick of the GPU tests, so it is checked
against hand-derived values here)."""
import math
import os
import re

import pytest
import torch

from oracle import vosolorn_plain as plain
from tests.test_hybrid_host import _write_checkpoint
from tests.vosolorn_helpers import SMALL, attn, dense, mlstm, model_config, moe, needle_model, needle_tokens, oracle_logits, rel_err


def test_config_reader_and_registry(tmp_path):
    from jacobiforcing_b200.hybrid_config import (ACT_GELU_ERF, ACT_GELU_TANH, BLOCK_POSTNORM, FF_GATED, FF_NONE, FF_ROUTED, MIX_MLSTM,
                                                  MIX_WINDOW, NORM_RMS, POS_NONE, ROUTE_TOP_SOFTMAX, HybridConfig)
    from jacobiforcing_b200.registry import architecture_of, resolve
    w = plain.random_weights(SMALL, 0)
    _write_checkpoint(tmp_path, SMALL, w)
    assert architecture_of(str(tmp_path)) == "Vosolorn"
    fam = resolve(str(tmp_path))
    assert fam.name == "hybrid" and fam.native_config
    hc = fam.load_config(str(tmp_path))
    assert isinstance(hc, HybridConfig) and hc.is_hybrid and hc.embed_norm and hc.tied_head
    assert (hc.norm_kind, hc.block_kind, hc.pos_kind) == (NORM_RMS, BLOCK_POSTNORM, POS_NONE) and abs(hc.logit_scale - 1.7) < 1e-7
    assert [s.mixer for s in hc.layers] == [MIX_MLSTM, MIX_WINDOW, MIX_MLSTM, MIX_WINDOW, MIX_MLSTM]
    a, b = hc.layers[1], hc.layers[3]
    assert (a.w_heads, a.w_kv_heads, a.w_dim, a.w_vdim, a.w_window, a.w_pool, a.w_rot_dims, a.w_rot_values, a.w_qk_norm) == \
        (4, 2, 16, 12, 11, 3, 8, 1, 1)
    assert a.w_rot_base == 500.0 and abs(a.w_scale - 0.4) < 1e-7
    assert (a.ff_kind, a.ff, a.ff_act) == (FF_GATED, 56, ACT_GELU_TANH)
    assert (b.ff_kind, b.ff, b.x_experts, b.x_top, b.x_route, b.x_plain, b.x_act, b.x_shared_ff) == \
        (FF_ROUTED, 16, 4, 1, ROUTE_TOP_SOFTMAX, 1, ACT_GELU_ERF, 0)
    m = hc.layers[0]
    assert (m.t_heads, m.t_dim, m.t_vdim, m.t_gate_cap, m.x_shared_ff) == (3, 10, 14, 6.0, 40)
    assert hc.layers[4].ff_kind == FF_NONE
    # keys and values of a token plus its share of the pooled block
    assert a.cache_elems_per_token() == -(-2 * 28 * 4 // 3) and m.cache_elems_per_token() == 0
    from jacobiforcing_b200.config import Config
    c = Config(str(tmp_path), kvcache_block_size=64, num_kvcache_blocks=8, max_num_batched_tokens=128)
    assert c.hf_config.architecture == "Vosolorn"


@pytest.mark.parametrize("bad", ["type", "kv_heads", "dims_odd", "dims_large", "vdim_odd", "top", "ff_kind", "pool"])
def test_config_reader_refuses(bad):
    from jacobiforcing_b200.hybrid_config import HybridConfig
    cfg = model_config([attn(), mlstm()])
    if bad == "type":
        cfg["layers"][0]["type"] = "mystery"
    elif bad == "kv_heads":
        cfg["layers"][0]["mixer"]["kv_heads"] = 3
    elif bad == "dims_odd":
        cfg["layers"][0]["mixer"]["rot"]["dims"] = 7
    elif bad == "dims_large":
        cfg["layers"][0]["mixer"]["rot"]["dims"] = 18
    elif bad == "vdim_odd":
        cfg["layers"][0]["mixer"]["vdim"] = 11
    elif bad == "top":
        cfg["layers"][1]["mlp"]["router"]["top"] = 7
    elif bad == "ff_kind":
        cfg["layers"][1]["mlp"]["kind"] = "mystery"
    elif bad == "pool":
        cfg["layers"][0]["mixer"]["mask"]["pool"] = 0
    with pytest.raises((ValueError, NotImplementedError)):
        HybridConfig.from_dict(cfg)


def test_binding_structures_follow_the_header():
    """Field names and order of the ctypes structures equal those of the C structures (both sides changed together)."""
    from jacobiforcing_b200 import _hybrid_cabi as cabi
    from jacobiforcing_b200.hybrid_config import LayerSpec
    src = open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "jacobi_hybrid.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    for cname, struct in (("hy_layer_cfg", cabi.LayerCfg), ("hy_model_cfg", cabi.ModelCfg), ("hy_runtime_cfg", cabi.RuntimeCfg)):
        body = re.search(r"typedef struct \{([^{}]*)\}\s*" + cname + ";", src).group(1)
        fields = []
        for decl in body.split(";"):
            decl = decl.strip()
            if decl:
                kind, names = decl.split(None, 1)
                fields += [(n.strip(), kind) for n in names.split(",")]
        got = [(n, "float" if t.__name__ == "c_float" else "int32_t") for n, t in struct._fields_]
        assert got == fields, cname
    spec = LayerSpec(0)
    assert all(hasattr(spec, n) for n, _ in cabi.LayerCfg._fields_)


def test_mask_by_hand():
    # window of 4, blocks of 3: position 9 sees tokens 6..9 and the blocks that end at or before position 5: {0, 1}
    assert plain.visible(9, 4, 3) == ([6, 7, 8, 9], [0, 1])
    # position 8 sees tokens 5..8; block 1 = 3..5 ends at 5 > 8 - 4, so only block 0; tokens 3 and 4 are not seen at all
    assert plain.visible(8, 4, 3) == ([5, 6, 7, 8], [0])
    assert plain.visible(2, 4, 3) == ([0, 1, 2], [])
    assert plain.visible(5, 1, 1) == ([5], [0, 1, 2, 3, 4])                 # pool of one: everything is seen


def test_rotation_and_attention_closed_forms():
    v = torch.tensor([[[1.0, 0.0, 2.0, 0.0, 5.0, 6.0]]], dtype=torch.float64).repeat(3, 1, 1)
    r = plain.turn_pairs(v, torch.arange(3), 4, 100.0)
    assert torch.allclose(r[0], v[0]) and torch.allclose(r[:, :, 4:], v[:, :, 4:])          # position 0, unrotated rest
    assert torch.allclose(r[2, 0, :2], torch.tensor([math.cos(2.0), math.sin(2.0)], dtype=torch.float64))
    assert torch.allclose(r[2, 0, 2:4], 2 * torch.tensor([math.cos(0.2), math.sin(0.2)], dtype=torch.float64))
    back = plain.turn_pairs(r, torch.arange(3), 4, 100.0, sign=-1.0)
    assert torch.allclose(back, v)
    # one head, keys all zero: uniform weights over what is visible; values unrotated in effect when they are constant
    # pairs (c, 0) turned by j and the mean turned back by i
    c = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "mask": {"size": 2, "pool": 2}, "rot": {"base": 10.0, "dims": 2}, "scale": 1.0}
    p = {"q": torch.zeros(2, 2), "k": torch.zeros(2, 2), "v": torch.tensor([[1.0, 0.0], [0.0, 0.0]]), "q.norm": torch.ones(2),
         "k.norm": torch.ones(2), "o": torch.eye(2)}
    p = {k: t.double() for k, t in p.items()}
    h = torch.tensor([[1.0, 0.0]] * 5, dtype=torch.float64)
    y = plain.window_pool_attention(h, p, c, 1e-6)
    # position 4 sees tokens 3, 4 and block 0 (positions 0, 1; block 1 ends at 3 > 4 - 2): three rows of weight 1/3
    rot = lambda a: torch.tensor([math.cos(a), math.sin(a)], dtype=torch.float64)
    mean = (rot(3) + rot(4) + (rot(0) + rot(1)) / 2) / 3
    want = torch.stack([mean[0] * math.cos(4) + mean[1] * math.sin(4), mean[1] * math.cos(4) - mean[0] * math.sin(4)])
    assert torch.allclose(y[4], want)


def test_matrix_memory_first_steps_by_hand():
    c = {"heads": 1, "dim": 1, "vdim": 2, "gate_cap": 2.0}
    z = torch.zeros
    p = {"q": torch.tensor([[2.0]]), "k": torch.tensor([[3.0]]), "v": torch.tensor([[1.0], [-1.0]]), "g": z(2, 1),
         "i": z(1, 1), "f": z(1, 1), "i.b": torch.tensor([-9.0]), "f.b": torch.tensor([9.0]), "norm": torch.ones(2),
         "o": torch.eye(2)}
    p = {k: t.double() for k, t in p.items()}
    h = torch.ones(2, 1, dtype=torch.float64)
    y = plain.mlstm_mixer(h, p, c, 0.0)
    li = 2.0 * math.tanh(-4.5)
    lf = -math.log1p(math.exp(-2.0 * math.tanh(4.5)))
    m1 = max(lf + 0.0, li)                                  # the maximum starts at 0: the forget gate wins
    assert m1 == lf
    b1 = math.exp(li - m1)
    n1 = b1 * 3.0
    den = max(abs(n1 * 2.0), math.exp(-m1)) + 1e-6
    o = torch.tensor([b1 * 3.0 * 2.0 / den, -b1 * 3.0 * 2.0 / den], dtype=torch.float64)
    want = o / torch.sqrt((o * o).mean()) * 0.5             # unit rms, gate sigmoid(0)
    assert torch.allclose(y[0], want)
    assert torch.allclose(y[1] / y[1].abs(), torch.tensor([1.0, -1.0], dtype=torch.float64))


def test_route_and_mixture_by_hand():
    p = {"router": torch.tensor([[1.0], [3.0], [2.0], [3.0]]), "router.b": torch.tensor([0.0, 0.0, 1.5, 0.0])}
    p = {k: t.double() for k, t in p.items()}
    ids, wts = plain.route(torch.ones(1, 1, dtype=torch.float64), p, 2)
    assert ids.tolist() == [[2, 1]]                          # 3.5 first, then the lower index of the tie at 3
    e = math.exp(-0.5)
    assert torch.allclose(wts, torch.tensor([[1 / (1 + e), e / (1 + e)]], dtype=torch.float64))
    assert abs(float(plain.gelu_erf(torch.tensor(1.0, dtype=torch.float64))) - 0.8413447460685429) < 1e-12
    assert abs(float(plain.gelu_tanh(torch.tensor(1.0, dtype=torch.float64))) - 0.8411919906082768) < 1e-12


def test_marked_key_model_shows_the_mask():
    """The GPU tests' one-layer model: the marked key changes the answer where the mask shows it and nowhere else."""
    cfg, w = needle_model(size=6, pool=4)
    n = 30                                                   # asked from 29: window 24..29, blocks up to position 23
    for j, seen in ((0, True), (19, True), (23, True), (24, True), (28, True)):
        toks, without = needle_tokens(n, j)
        d = rel_err(oracle_logits(cfg, w, without)[-1], oracle_logits(cfg, w, toks)[-1])
        assert (d > 0.3) == seen, j
    cfg, w = needle_model(size=5, pool=4)                    # window 25..29, blocks up to position 23: 24 is hidden
    toks, without = needle_tokens(n, 24)
    assert rel_err(oracle_logits(cfg, w, without)[-1], oracle_logits(cfg, w, toks)[-1]) < 1e-9
