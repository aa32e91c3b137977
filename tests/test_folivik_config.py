"""The Folivik design's configuration, tensor names, cache and state needs, and the plain
implementation's own mechanisms worked out by hand (no GPU)."""
import copy
import math

import pytest
import torch

import helpers as H
import folivik_plain as P
from binfer_b200.cache.manager import CacheManager, KVNeed
from binfer_b200.config import (ConfigError, ConvWindowAttentionSpec, FolivikConfig,
                                LatentAttentionSpec, Mamba2Spec, MoESpec, parse_config)
from binfer_b200.parts.base import BuildEnv
from binfer_b200.parts.model import DecoderModel, param_specs_for

CPU = BuildEnv(torch.float32, torch.device("cpu"))
F64 = torch.float64


def test_the_registry_picks_the_family_by_its_one_name():
    cfg = parse_config(H.FOL_A)
    assert isinstance(cfg, FolivikConfig)
    assert cfg.to_dict() == H.FOL_A and cfg.to_dict() is not H.FOL_A


def test_layers_become_specs_with_their_own_sizes():
    spec = FolivikConfig.from_dict(H.FOL_A).to_spec()
    assert spec.hidden_size == 64 and spec.vocab_size == 300 and not spec.tie_word_embeddings
    assert spec.final_norm.kind == "rmsnorm" and spec.final_norm.scalar_weight
    assert spec.final_norm.eps == 1e-5 and spec.embedding_scale == 1.0
    assert all(l.block == "prenorm" and l.norm.scalar_weight for l in spec.layers)
    assert [e.layer for e in spec.schedule] == [0, 1, 2]
    m, a, la = [l.mixer for l in spec.layers]
    assert isinstance(m, Mamba2Spec)
    assert (m.num_heads, m.groups, m.state_dim, m.head_dim, m.conv_taps, m.norm_groups) == (
        4, 2, 16, 24, 3, 2) and m.conv_bias and m.norm_eps == 1e-5
    assert isinstance(a, ConvWindowAttentionSpec)
    assert (a.num_heads, a.num_kv_heads, a.head_dim, a.value_dim, a.window) == (4, 2, 32, 16, 24)
    assert (a.conv_taps, a.position, a.unit_norm, a.proj_norm, a.sinks, a.keep_first) == (
        0, None, True, False, False, 0)
    assert a.head_norm_weight and a.head_temperature and a.log_distance_bias and a.scale == 0.3
    assert isinstance(la, LatentAttentionSpec)
    assert (la.num_heads, la.head_dim, la.rot_dim, la.value_dim, la.kv_rank, la.q_rank) == (
        3, 24, 8, 20, 40, 24)
    assert la.position.layout == "interleaved" and la.position.rotary_dim == 8 and la.head_gate
    f = spec.layers[0].ffn
    assert isinstance(f, MoESpec) and f.scoring == "softmax_all" and f.correction
    assert (f.num_experts, f.identity, f.top, f.groups, f.groups_keep) == (8, 1, 2, 3, 2)
    assert (f.expert_size, f.shared_size, f.route_scale, f.weight_eps) == (32, 48, 1.5, 1e-20)
    assert spec.layers[2].ffn is None
    g = FolivikConfig.from_dict(H.FOL_B).to_spec().layers[0].ffn      # no groups, nothing shared
    assert (g.groups, g.groups_keep, g.identity, g.shared_size, g.route_scale) == (1, 1, 0, 0, 1.0)
    c = FolivikConfig.from_dict(H.FOL_C).to_spec().layers[2].mixer
    assert c.position.rotary_dim == 4 and c.rot_dim == 6


def test_tensor_names_and_shapes():
    shapes = {s.name: s.shape for s in param_specs_for(FolivikConfig.from_dict(H.FOL_A).to_spec())}
    assert shapes["embed"] == (300, 64) and shapes["head"] == (300, 64)
    assert shapes["final.norm"] == () and shapes["l0.norm1"] == () and shapes["l1.norm2"] == ()
    inner, chan = 4 * 24, 4 * 24 + 2 * 2 * 16
    assert shapes["l0.mix.in"] == (2 * inner + 2 * 2 * 16 + 4, 64)
    assert shapes["l0.mix.conv"] == (chan, 3) and shapes["l0.mix.conv.b"] == (chan,)
    assert shapes["l0.mix.dt_bias"] == shapes["l0.mix.A_log"] == shapes["l0.mix.D"] == (4,)
    assert shapes["l0.mix.norm"] == (inner,) and shapes["l0.mix.o"] == (64, inner)
    assert shapes["l0.mlp.router"] == (9, 64) and shapes["l0.mlp.correction"] == (9,)
    assert shapes["l0.mlp.e7.gate"] == (32, 64) and shapes["l0.mlp.e7.down"] == (64, 32)
    assert "l0.mlp.e8.gate" not in shapes                    # the ninth output has no tensors
    assert shapes["l0.mlp.shared.up"] == (48, 64) and shapes["l0.mlp.shared.down"] == (64, 48)
    assert shapes["l1.mix.q"] == (128, 64) and shapes["l1.mix.k"] == (64, 64)
    assert shapes["l1.mix.v"] == (32, 64) and shapes["l1.mix.o"] == (64, 64)
    assert shapes["l1.mix.q.norm"] == shapes["l1.mix.k.norm"] == (32,)
    assert shapes["l1.mix.temp"] == shapes["l1.mix.r1"] == shapes["l1.mix.r2"] == (4,)
    assert shapes["l2.mix.dq"] == (24, 64) and shapes["l2.mix.dq.norm"] == (24,)
    assert shapes["l2.mix.uq"] == (96, 24) and shapes["l2.mix.dkv"] == (48, 64)
    assert shapes["l2.mix.dkv.norm"] == (40,) and shapes["l2.mix.uk"] == (72, 40)
    assert shapes["l2.mix.uv"] == (60, 40) and shapes["l2.mix.g"] == (3, 64)
    assert shapes["l2.mix.o"] == (64, 60) and "l2.mix.q" not in shapes
    assert "l2.norm2" not in shapes and not any(n.startswith("l2.mlp.") for n in shapes)
    shapes = {s.name: s.shape for s in param_specs_for(FolivikConfig.from_dict(H.FOL_B).to_spec())}
    assert "l0.mlp.shared.gate" not in shapes and shapes["l0.mlp.router"] == (5, 48)
    assert shapes["l2.mlp.router"] == (6, 48) and "l2.mlp.e4.gate" not in shapes
    assert "l1.norm2" not in shapes
    # a convolution of one tap still has its tensor and its bias
    shapes = {s.name: s.shape for s in param_specs_for(FolivikConfig.from_dict(H.FOL_C).to_spec())}
    assert shapes["l1.mix.conv"] == (2 * 10 + 2 * 6, 1) and shapes["l1.mix.conv.b"] == (32,)


def test_cache_and_state_needs_per_layer():
    model = DecoderModel(FolivikConfig.from_dict(H.FOL_A).to_spec(), CPU)
    kv, st = model.kv_needs(), model.state_needs()
    assert kv[0] is None and kv[1] == KVNeed(2, 32, 24, 16)
    assert kv[2] == KVNeed(1, 48, None, 0)                 # the latent and the shared key part
    chan = 4 * 24 + 2 * 2 * 16
    assert st[0].shape == (4 * 16 * 24 + 2 * chan,) and st[1] is None and st[2] is None
    cm = CacheManager(kv, st, page_size=8, num_pages=6, max_requests=2)
    assert len(cm.groups) == 2
    # a convolution of one tap keeps no rows
    model = DecoderModel(FolivikConfig.from_dict(H.FOL_C).to_spec(), CPU)
    assert model.state_needs()[1].shape == (2 * 6 * 10,)


@pytest.mark.parametrize("bad,msg", [
    (lambda r: r["layers"][0].update(type="delta"), "type"),
    (lambda r: r["layers"][0]["mixer"].update(groups=3), "multiple"),
    (lambda r: r["layers"][0]["mixer"].update(norm_groups=5), "norm_groups"),
    (lambda r: r["layers"][0]["mixer"].pop("state"), "state"),
    (lambda r: r["layers"][1]["mixer"].update(kv_heads=3), "multiple"),
    (lambda r: r["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda r: r["layers"][2]["mixer"].pop("q_rank"), "q_rank"),
    (lambda r: r["layers"][2]["mixer"]["rot"].update(dims=10), "dims"),
    (lambda r: r["layers"][0]["mlp"].update(kind="dense"), "kind"),
    (lambda r: r["layers"][0]["mlp"]["router"].update(top=10), "top"),
    (lambda r: r["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda r: r["layers"][0]["mlp"]["router"]["groups"].update(keep=4), "groups"),
    (lambda r: r["layers"][1]["mlp"]["router"].update(top=4, groups={"count": 2, "keep": 1}), "top"),
    (lambda r: r["layers"][0]["mlp"].pop("expert"), "expert"),
    (lambda r: r.pop("width"), "width"),
    (lambda r: r["norm"].update(eps=0.0), "eps"),
])
def test_a_bad_configuration_is_refused(bad, msg):
    raw = copy.deepcopy(H.FOL_A)
    bad(raw)
    with pytest.raises(ConfigError, match=msg):
        FolivikConfig.from_dict(raw)


def test_a_norm_with_one_number_is_loaded_as_a_vector_of_it():
    from binfer_b200.config.specs import NormSpec
    from binfer_b200.parts.norms import RMSNorm
    n = RMSNorm(NormSpec(eps=1e-6, scalar_weight=True), 5, "n", CPU)
    assert n.param_specs()[0].shape == ()
    n.load(lambda spec: torch.tensor(1.25))
    assert n.weight.tolist() == [1.25] * 5 and n.weight.is_contiguous()


# ------------------------------------------------- the plain implementation, by hand
def test_plain_rotation_in_neighbouring_pairs():
    x = torch.arange(2 * 1 * 6, dtype=F64).view(2, 1, 6) + 1.0
    y = P.rotate_pairs(x, 100.0, 4)
    assert torch.equal(y[0], x[0]) and torch.equal(y[..., 4:], x[..., 4:])
    c, s = math.cos(1.0), math.sin(1.0)                       # pair 0 at position 1: (7, 8)
    assert abs(float(y[1, 0, 0]) - (7 * c - 8 * s)) < 1e-12
    assert abs(float(y[1, 0, 1]) - (8 * c + 7 * s)) < 1e-12
    c, s = math.cos(0.1), math.sin(0.1)                       # pair 1: 100^(-2/4)
    assert abs(float(y[1, 0, 2]) - (9 * c - 10 * s)) < 1e-12


def test_plain_convolution_has_its_bias_and_its_last_tap_now():
    u = torch.tensor([[1.0], [2.0], [4.0]], dtype=F64)
    y = P.causal_conv(u, torch.tensor([[100.0, 10.0, 1.0]], dtype=F64), torch.tensor([0.5], dtype=F64))
    assert y.view(-1).tolist() == [1.5, 12.5, 124.5]


def test_plain_window_and_distance_bias():
    """Two positions inside a window of two see each other, the third token back is out; the
    bias b1 ln(1 + b2 d) is taken off, nothing at distance 0."""
    T = 4
    q = torch.ones(T, 1, 2, dtype=F64)
    k = torch.zeros(T, 1, 2, dtype=F64)
    v = torch.eye(T, dtype=F64).view(T, 1, T)
    o = P.softmax_attention(q, k, v, 1.0, 2, bias=lambda h, d: 0.7 * torch.log1p(3.0 * d))
    assert o[0, 0].tolist() == [1.0, 0.0, 0.0, 0.0]
    near = 1.0 / (1.0 + math.exp(-0.7 * math.log(4.0)))      # own weight beside one neighbour
    assert abs(float(o[2, 0, 2]) - near) < 1e-12 and abs(float(o[2, 0, 1]) - (1 - near)) < 1e-12
    assert float(o[2, 0, 0]) == 0.0 and float(o[3, 0, 1]) == 0.0


def test_plain_state_space_step_by_hand():
    """One head, state of one, value of one, identity projections: two tokens."""
    mx = {"heads": 1, "vdim": 1, "state": 1, "groups": 1, "conv": 1, "norm_groups": 1}
    w = {"m.in": torch.eye(5), "m.conv": torch.ones(3, 1), "m.conv.b": torch.zeros(3),
         "m.dt_bias": torch.tensor([0.0]), "m.A_log": torch.tensor([0.0]),
         "m.D": torch.tensor([2.0]), "m.norm": torch.ones(1), "m.o": torch.eye(1)}
    w = {n: t.double() for n, t in w.items()}
    # rows: z, x, B, C, dt
    h = torch.tensor([[1.0, 1.0, 2.0, 3.0, 0.0], [1.0, -1.0, 1.0, 1.0, 1.0]], dtype=F64)
    x, B, C = P.silu(h[:, 1]), P.silu(h[:, 2]), P.silu(h[:, 3])
    dt = torch.log1p(torch.exp(h[:, 4]))
    s0 = dt[0] * B[0] * x[0]
    s1 = math.exp(-float(dt[1])) * s0 + dt[1] * B[1] * x[1]
    y = torch.stack([s0 * C[0] + 2.0 * x[0], s1 * C[1] + 2.0 * x[1]]) * P.silu(h[:, 0])
    want = y / torch.sqrt(y * y + 1e-6)
    out = P.mamba2(h, w, "m.", mx, 1e-6)
    assert torch.allclose(out.view(-1), want, atol=1e-12)


def test_plain_router_groups_corrections_and_identity_experts():
    """Six outputs in three groups of two, the best two groups kept, two chosen.  Scores rise
    with the index; corrections lift output 0 for the choice only.  Groups count by their best
    choice score: (0, 1) through the lifted 0, (4, 5) through 5; (2, 3) is out, although 3
    scores higher than 0 and 1.  Chosen: 0 (lifted) and 5; their weights are their scores
    without the correction, over their sum, times the factor."""
    z = torch.tensor([[0.0, 0.1, 0.2, 0.3, 0.4, 0.5]], dtype=F64)
    w = {"r.router": torch.eye(6, dtype=F64), "r.correction": torch.tensor(
        [1.0, 0.0, 0.0, 0.0, 0.0, 0.0], dtype=F64)}
    router = {"experts": 4, "identity": 2, "top": 2, "scale": 3.0, "groups": {"count": 3, "keep": 2}}
    ids, wts = P.route(z, w, "r.", router)
    s = torch.softmax(z, -1)[0]
    assert sorted(ids[0].tolist()) == [0, 5]
    got = dict(zip(ids[0].tolist(), wts[0].tolist()))
    assert abs(got[0] - 3.0 * float(s[0] / (s[0] + s[5]))) < 1e-12
    assert abs(got[5] - 3.0 * float(s[5] / (s[0] + s[5]))) < 1e-12
    # corrections far below zero: an output outside the kept groups still cannot be chosen
    w["r.correction"] = torch.tensor([-5.0, -5.0, -1.0, -1.0, -5.0, -4.0], dtype=F64)
    router["groups"] = {"count": 3, "keep": 1}
    ids, _ = P.route(z, w, "r.", router)
    assert sorted(ids[0].tolist()) == [2, 3]
    # output 5 is an identity expert: the mixture returns the input times its weight
    mlp = {"router": {"experts": 4, "identity": 2, "top": 1, "scale": 2.0}, "shared": None}
    w = {"r.router": torch.eye(6, dtype=F64), "r.correction": torch.zeros(6, dtype=F64)}
    out = P.mixture_of_experts(z, w, "r.", mlp)
    assert torch.allclose(out, 2.0 * z, atol=1e-12)
