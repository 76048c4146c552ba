"""Sebavik without a GPU: the configuration reader and its refusals, the registry, and closed forms of the plain oracle
(mask, pair rows, convolution over time, clamped pair, routing with a tie, sink and distance bias by hand, depth average)."""
import copy
import json
import math

import pytest
import torch

from jacobiforcing_b200 import hybrid_config as hcfg
from jacobiforcing_b200.hybrid_config import HybridConfig
from jacobiforcing_b200.registry import FAMILIES, family_of_config, resolve
from oracle import sebavik_plain as plain
from tests.sebavik_helpers import SMALL, attn, dense, model_config, moe


def test_config_reader_reads_every_size_and_constant():
    hc = HybridConfig.from_dict(SMALL)
    assert (hc.architecture, hc.width, hc.vocab, len(hc.layers)) == ("Sebavik", 40, 70, 5)
    assert (hc.block_kind, hc.norm_kind, hc.pos_kind, hc.tied_head) == (hcfg.BLOCK_PRENORM, hcfg.NORM_RMS, hcfg.POS_NONE, True)
    assert (hc.resid_mult, hc.canon_taps, hc.side_dim, hc.depth_avg) == (0.6, 4, 5, 1)
    assert (hc.pair_buckets, hc.pair_mul_prev, hc.pair_mul_cur, hc.emb_scale) == (37, 13, 7, 2.0)
    a = hc.layers[3]
    assert (a.mixer, a.b_heads, a.b_kv_heads, a.b_dim, a.b_vdim, a.b_window, a.b_keep_first, a.b_v_mix) == (hcfg.MIX_BIASED, 6, 2, 24, 12, 19, 9, 1)
    assert (a.b_softcap, a.b_scale) == (2.5, 0.35)
    assert (a.ff_kind, a.x_experts, a.x_top, a.ff, a.x_route, a.x_plain, a.x_act) == (hcfg.FF_ROUTED, 4, 1, 16, hcfg.ROUTE_TOP_SOFTMAX, 0, hcfg.ACT_SILU)
    d = hc.layers[4]
    assert (d.ff_kind, d.ff, d.ff_act, d.ff_limit, d.b_v_mix) == (hcfg.FF_GATED, 32, hcfg.ACT_CLAMPED, 0.3, 0)
    assert hc.layers[2].ff_kind == hcfg.FF_NONE and hc.layers[2].b_keep_first == 0
    assert a.cache_elems_per_token() == 2 * (24 + 12)


def test_what_the_configuration_leaves_out_does_not_exist():
    cfg = model_config([attn(size=None, cap=None, v_mix=False, mlp=None)], taps=0, side=0, buckets=0)
    hc = HybridConfig.from_dict(cfg)
    assert (hc.canon_taps, hc.side_dim, hc.pair_buckets) == (0, 0, 0)
    assert (hc.layers[0].b_window, hc.layers[0].b_softcap, hc.layers[0].b_v_mix) == (0, 0.0, 0)
    assert set(plain.tensor_shapes(cfg)) & {"bigram", "side.embed", "l0.canon1", "l0.norm2"} == set()


def test_config_reader_refuses_what_a_kernel_would_index_with():
    bad = copy.deepcopy(SMALL)
    bad["layers"][0]["mixer"]["kv_heads"] = 3
    with pytest.raises(ValueError):
        HybridConfig.from_dict(bad)
    bad = copy.deepcopy(SMALL)
    bad["layers"][1]["mixer"]["vdim"] = 16                    # blends with layer 0, whose values are 12 wide
    with pytest.raises(ValueError):
        HybridConfig.from_dict(bad)
    bad = copy.deepcopy(SMALL)
    bad["layers"][1]["mlp"]["router"]["top"] = 7
    with pytest.raises(ValueError):
        HybridConfig.from_dict(bad)
    bad = copy.deepcopy(SMALL)
    bad["layers"][0]["type"] = "mamba2"
    with pytest.raises(NotImplementedError):
        HybridConfig.from_dict(bad)
    bad = copy.deepcopy(SMALL)
    bad["layers"][0]["mlp"]["kind"] = "other"
    with pytest.raises(NotImplementedError):
        HybridConfig.from_dict(bad)


def test_registry_serves_it_through_the_hybrid_family(tmp_path):
    assert FAMILIES["Sebavik"].name == "hybrid"
    (tmp_path / "config.json").write_text(json.dumps(SMALL))
    assert resolve(str(tmp_path)).name == "hybrid"
    assert family_of_config(HybridConfig.from_dict(SMALL)) is FAMILIES["Sebavik"]


# ---- closed forms of the oracle --------------------------------------------------------------------------------------------------
def test_mask_by_hand():
    seen = [j for j in range(12) if plain.sees(11, j, 4, 2)]
    assert seen == [0, 1, 8, 9, 10, 11]
    assert [j for j in range(6) if plain.sees(3, j, 2, 3)] == [0, 1, 2, 3]          # kept tokens and the window overlap; nothing later
    assert all(plain.sees(9, j, None, 0) for j in range(10))


def test_pair_rows_by_hand():
    c = {"buckets": 10, "mul_prev": 3, "mul_cur": 7}
    assert plain.pair_rows([4, 9, 9, 0], c) == [10, (12 + 63) % 10, (27 + 63) % 10, 27 % 10]


def test_time_conv_by_hand():
    h = torch.tensor([[1.0, 10.0], [2.0, 20.0], [3.0, 30.0], [4.0, 40.0]], dtype=torch.float64)
    w = torch.tensor([[0.5, 0.0, 2.0], [0.0, 1.0, 0.0]], dtype=torch.float64)   # channel 0: half of t - 2 and twice t; channel 1: t - 1
    out = plain.time_conv(h, w)
    assert out[:, 0].tolist() == [2.0, 4.0, 6.5, 9.0]
    assert out[:, 1].tolist() == [0.0, 10.0, 20.0, 30.0]
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    got = plain.sublayer_input(x, torch.ones(2, dtype=torch.float64), None, 0.0)
    assert torch.allclose(got, x / math.sqrt(12.5))


def test_clamped_pair_by_hand():
    p = {"gate": torch.tensor([[1.0], [1.0]], dtype=torch.float64), "up": torch.tensor([[1.0], [-1.0]], dtype=torch.float64),
         "down": torch.eye(2, dtype=torch.float64)}
    y = plain.clamped_gated(torch.tensor([[5.0]], dtype=torch.float64), p, {"limit": 2.0})      # gate 5 -> 2, up 5 -> 2 and -5 -> -2
    s = 2.0 / (1.0 + math.exp(-1.702 * 2.0))
    assert torch.allclose(y, torch.tensor([[s * 3.0, s * -1.0]], dtype=torch.float64))
    y = plain.clamped_gated(torch.tensor([[-5.0]], dtype=torch.float64), p, {"limit": 2.0})     # the gate has no lower clamp
    s = -5.0 / (1.0 + math.exp(1.702 * 5.0))
    assert torch.allclose(y, torch.tensor([[s * -1.0, s * 3.0]], dtype=torch.float64))


def test_routing_with_a_tie_and_softmax_over_the_chosen():
    router = torch.tensor([[1.0], [2.0], [2.0], [-1.0]], dtype=torch.float64)
    ids, wts = plain.route(torch.tensor([[1.0]], dtype=torch.float64), router, 3)
    assert ids == [[1, 2, 0]]
    e = [math.exp(2.0), math.exp(2.0), math.exp(1.0)]
    assert torch.allclose(wts[0], torch.tensor(e, dtype=torch.float64) / sum(e))


def test_sink_and_distance_bias_by_hand():
    """Zero queries: every score is minus the bias.  r1 = 1, r2 = 1: weights 1 / (1 + distance); the sink adds exp(sink) below."""
    c = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 1, "scale": 1.0, "softcap": 5.0, "mask": {"size": 2, "keep_first": 1}}
    z = torch.zeros
    p = {"q": z(2, 1, dtype=torch.float64), "q.b": z(2, dtype=torch.float64), "k": z(2, 1, dtype=torch.float64), "k.b": z(2, dtype=torch.float64),
         "r1": torch.ones(1, dtype=torch.float64), "r2": torch.ones(1, dtype=torch.float64),
         "sink": torch.tensor([math.log(0.5)], dtype=torch.float64), "o": torch.ones(1, 1, dtype=torch.float64)}
    v = torch.tensor([[[1.0]], [[10.0]], [[100.0]], [[1000.0]]], dtype=torch.float64)
    out = plain.attention(z(4, 1, dtype=torch.float64), p, c, v)
    # position 3 sees 0 (kept, distance 3), 2 and 3: weights 1/4, 1/2, 1 over 1/4 + 1/2 + 1 + 1/2
    assert math.isclose(float(out[3, 0]), (0.25 * 1.0 + 0.5 * 100.0 + 1000.0) / 2.25, rel_tol=1e-12)
    assert math.isclose(float(out[0, 0]), 1.0 / 1.5, rel_tol=1e-12)


def test_depth_average_and_blend_in_the_forward_pass():
    """A model whose sublayers add nothing (layer scales of zero): the stream after layer i is the depth weights' sum times
    the embedding output, layer after layer."""
    cfg = model_config([attn(mlp=None), attn(mlp=None)], side=0)
    w = {k: v.float() for k, v in plain.random_weights(cfg, 3).items()}
    w["l0.ls1"] = torch.zeros(40)
    w["l1.ls1"] = torch.zeros(40)
    w["l0.dwa"] = torch.tensor([0.25, 0.5])
    w["l1.dwa"] = torch.tensor([1.0, 2.0, -1.0])
    lo = []
    plain.forward(cfg, w, [3, 5, 8], layers_out=lo)
    x0 = plain.embed([3, 5, 8], w, cfg)
    assert torch.allclose(lo[0], 0.75 * x0)
    assert torch.allclose(lo[1], (1.0 + 2.0 - 0.75) * x0)
