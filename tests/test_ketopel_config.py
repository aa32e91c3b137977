"""The looped design's configuration, tensor names, schedule, cache and state needs, and the
plain implementation's own mechanisms (no GPU)."""
import copy
import math

import pytest
import torch

import helpers as H
import ketopel_plain as P
from binfer_b200.cache.manager import CacheManager, KVNeed
from binfer_b200.config import (ConfigError, ConvWindowAttentionSpec, GatedDeltaRuleSpec,
                                GatedMLPSpec, KetopelConfig, LatentAttentionSpec,
                                ParallelMixersSpec, PassStart, RampScaling, RetentionSpec,
                                RopeSpec, parse_config)
from binfer_b200.parts.base import BuildEnv
from binfer_b200.parts.model import DecoderModel, param_specs_for
from binfer_b200.parts.rope import RotaryEncoding

CPU = BuildEnv(torch.float32, torch.device("cpu"))


def test_the_registry_picks_the_family_by_its_one_name():
    cfg = parse_config(H.KET_A)
    assert isinstance(cfg, KetopelConfig)
    assert cfg.to_dict() == H.KET_A and cfg.to_dict() is not H.KET_A


def test_layers_become_specs_with_their_own_sizes():
    spec = KetopelConfig.from_dict(H.KET_A).to_spec()
    assert spec.hidden_size == 64 and spec.vocab_size == 300 and not spec.tie_word_embeddings
    assert spec.embedding_scale == 2.0 and spec.final_norm.kind == "rmsnorm"
    assert spec.final_norm.eps == 1e-5 and spec.final_norm.offset == 0.0
    assert all(l.block == "prenorm" for l in spec.layers)
    d, p, la = [l.mixer for l in spec.layers]
    assert isinstance(d, GatedDeltaRuleSpec)
    assert (d.num_heads, d.num_qk_heads, d.qk_dim, d.v_dim, d.conv_taps) == (4, 2, 16, 24, 3)
    assert d.unit_eps == 1e-6 and d.norm_eps == 1e-5
    assert isinstance(p, ParallelMixersSpec) and [b.prefix for b in p.branches] == ["left.", "right."]
    assert [b.scale for b in p.branches] == [0.7, 1.2]
    a, r = p.branches[0].spec, p.branches[1].spec
    assert isinstance(a, ConvWindowAttentionSpec) and isinstance(r, RetentionSpec)
    assert (a.num_heads, a.num_kv_heads, a.head_dim, a.value_dim) == (4, 2, 32, 16)
    assert (a.conv_taps, a.window, a.sinks, a.unit_norm, a.proj_norm) == (0, None, False, False, True)
    assert a.scale == 0.2 and a.softcap == 20.0 and a.position.rotary_dim == 16
    assert a.position.ramp_scaling == RampScaling(8.0, 64.0, 4.0, 1.0) and a.position.layout == "half"
    assert (r.num_heads, r.qk_dim, r.v_dim, r.decays) == (2, 16, 32, (0.9, 0.99))
    assert (r.activation, r.k_scale, r.norm_over, r.norm_weight, r.gate) == (
        "silu", 1.0, "all", True, "sigmoid") and r.position is None
    assert isinstance(la, LatentAttentionSpec)
    assert (la.num_heads, la.head_dim, la.rot_dim, la.value_dim, la.kv_rank) == (3, 24, 8, 20, 40)
    assert la.position.layout == "interleaved" and la.position.rotary_dim == 8 and la.head_gate
    f = spec.layers[0].ffn
    assert isinstance(f, GatedMLPSpec) and f.activation == "gelu_tanh" and f.intermediate_size == 96
    assert spec.layers[2].ffn is None
    b = KetopelConfig.from_dict(H.KET_B).to_spec().layers[1].mixer.branches[0].spec
    assert b.softcap == 0.0 and b.position.ramp_scaling is None and b.position.rotary_dim == 24


def test_the_schedule_walks_the_looped_layers_again():
    spec = KetopelConfig.from_dict(H.KET_A).to_spec()
    assert [(e.layer, e.before) for e in spec.schedule] == [
        (0, PassStart(False, 0)), (1, None), (0, PassStart(True, 1)), (1, None), (2, None)]
    assert spec.pass_table == ("loop.step", 2)
    spec = KetopelConfig.from_dict(H.KET_B).to_spec()
    assert [e.layer for e in spec.schedule] == [0] + [1, 2, 3] * 3
    assert [e.before for e in spec.schedule][1::3] == [PassStart(False, 0), PassStart(True, 1),
                                                      PassStart(True, 2)]
    spec = KetopelConfig.from_dict(H.KET_C).to_spec()          # one pass: the vector alone
    assert [(e.layer, e.before) for e in spec.schedule] == [(0, None), (1, None),
                                                            (2, PassStart(False, 0))]
    raw = copy.deepcopy(H.KET_C)
    del raw["loop"]
    spec = KetopelConfig.from_dict(raw).to_spec()
    assert all(e.before is None for e in spec.schedule) and spec.pass_table is None
    assert "loop.step" not in {s.name for s in param_specs_for(spec)}
    assert all(e.cache_from is None for e in KetopelConfig.from_dict(H.KET_B).to_spec().schedule)


def test_tensor_names_and_shapes():
    shapes = {s.name: s.shape for s in param_specs_for(KetopelConfig.from_dict(H.KET_A).to_spec())}
    assert shapes["embed"] == (300, 64) and shapes["head"] == (300, 64)
    assert shapes["final.norm"] == (64,) and shapes["loop.step"] == (2, 64)
    assert shapes["l0.norm1"] == (64,) and shapes["l0.norm2"] == (64,)
    assert shapes["l0.mix.q"] == (32, 64) and shapes["l0.mix.k"] == (32, 64)
    assert shapes["l0.mix.v"] == (96, 64) and shapes["l0.mix.g"] == (96, 64)
    assert shapes["l0.mix.q.conv"] == (32, 3) and shapes["l0.mix.v.conv"] == (96, 3)
    assert shapes["l0.mix.b"] == (4, 64) and shapes["l0.mix.a"] == (4, 64)
    assert shapes["l0.mix.A_log"] == (4,) and shapes["l0.mix.dt_bias"] == (4,)
    assert shapes["l0.mix.norm"] == (24,) and shapes["l0.mix.o"] == (64, 96)
    assert shapes["l0.mlp.gate"] == (96, 64) and shapes["l0.mlp.down"] == (64, 96)
    assert shapes["l1.mix.left.q"] == (128, 64) and shapes["l1.mix.left.k"] == (64, 64)
    assert shapes["l1.mix.left.v"] == (32, 64) and shapes["l1.mix.left.o"] == (64, 64)
    assert shapes["l1.mix.left.q.norm"] == (128,) and shapes["l1.mix.left.k.norm"] == (64,)
    assert shapes["l1.mix.right.q"] == (32, 64) and shapes["l1.mix.right.v"] == (64, 64)
    assert shapes["l1.mix.right.g"] == (64, 64) and shapes["l1.mix.right.norm"] == (64,)
    assert shapes["l1.mix.right.o"] == (64, 64)
    assert shapes["l2.mix.q"] == (96, 64) and shapes["l2.mix.dkv"] == (48, 64)
    assert shapes["l2.mix.dkv.norm"] == (40,) and shapes["l2.mix.uk"] == (72, 40)
    assert shapes["l2.mix.uv"] == (60, 40) and shapes["l2.mix.g"] == (3, 64)
    assert shapes["l2.mix.o"] == (64, 60)
    assert "l2.norm2" not in shapes and "l2.mlp.gate" not in shapes
    assert not any(n.endswith(".sink") or ".conv" in n for n in shapes if n.startswith("l1."))
    # a convolution of one tap still has its tensor
    shapes = {s.name: s.shape for s in param_specs_for(KetopelConfig.from_dict(H.KET_B).to_spec())}
    assert shapes["l3.mix.q.conv"] == (40, 1) and "l1.norm2" not in shapes


def test_cache_and_state_needs_per_layer_run():
    model = DecoderModel(KetopelConfig.from_dict(H.KET_A).to_spec(), CPU)
    kv, st = model.kv_needs(), model.state_needs()
    assert len(kv) == len(st) == 5
    assert kv[0] is None and kv[2] is None
    assert kv[1] == kv[3] == KVNeed(2, 32, None, 16)
    assert kv[4] == KVNeed(1, 48, None, 0)                 # the latent and the shared key part
    delta = 4 * 16 * 24 + 2 * (2 * 2 * 16 + 4 * 24)        # the memory and two convolution rows
    assert st[0].shape == st[2].shape == (delta,)
    assert st[1].shape == st[3].shape == (2 * 16 * 32,) and st[4] is None
    cm = CacheManager(kv, st, page_size=8, num_pages=6, max_requests=2)
    assert len(cm.groups) == 2 and [len(g.entries) for g in cm.groups] == [2, 1]
    # a convolution of one tap keeps no rows; every pass has a state of its own
    model = DecoderModel(KetopelConfig.from_dict(H.KET_B).to_spec(), CPU)
    st = model.state_needs()
    assert st[3].shape == (2 * 40 * 12,) and st[2].shape == (3 * 8 * 8 + 3 * (3 * 8 * 3),)
    assert len(st) == 10 and st[0] is None and st[1].shape == (3 * 8 * 8,)


@pytest.mark.parametrize("bad,msg", [
    (lambda r: r["layers"][0].update(type="window"), "type"),
    (lambda r: r["layers"][0]["mixer"].update(heads=3), "multiple"),
    (lambda r: r["layers"][1]["mixer"]["right"].update(decay=[0.9]), "decay"),
    (lambda r: r["layers"][1]["mixer"]["left"].pop("scale"), "scale"),
    (lambda r: r["layers"][1]["mixer"]["left"]["rot"].update(dims=40), "dims"),
    (lambda r: r["layers"][2]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda r: r["layers"][0]["mlp"].update(kind="moe"), "kind"),
    (lambda r: r["loop"].update(stop=4), "loop"),
    (lambda r: r["loop"].update(times=0), "times"),
    (lambda r: r.pop("width"), "width"),
])
def test_a_bad_configuration_is_refused(bad, msg):
    raw = copy.deepcopy(H.KET_A)
    bad(raw)
    with pytest.raises(ConfigError, match=msg):
        KetopelConfig.from_dict(raw)


def test_frequencies_stretched_by_pair_index():
    """The part's table against the plain implementation's, and against values worked out by
    hand: 8 pairs, base 10000, 64 positions, factor 8, ramp between 4 turns and 1 turn."""
    rot = {"base": 10000.0, "dims": 16, "scaling": {"factor": 8.0, "original": 64, "fast": 4.0,
                                                   "slow": 1.0}}
    f, mag = P.rotary_table(rot)
    enc = RotaryEncoding(RopeSpec(theta=10000.0, rotary_dim=16,
                                  ramp_scaling=RampScaling(8.0, 64.0, 4.0, 1.0)), 32, CPU)
    assert torch.allclose(enc.inv_freq.double(), f, rtol=1e-6)
    assert abs(enc.magnitude - mag) < 1e-12 and abs(mag - (0.1 * math.log(8.0) + 1.0)) < 1e-12
    n = lambda t: 16 * math.log(64 / (2 * math.pi * t)) / (2 * math.log(10000.0))   # noqa: E731
    lo, hi = max(math.floor(n(4.0)), 0), min(math.ceil(n(1.0)), 15)
    assert (lo, hi) == (0, 3)                                        # n(1) = 2.016
    plain = [10000.0 ** (-2 * i / 16) for i in range(8)]
    assert abs(float(f[0]) - plain[0]) < 1e-15                       # the fastest wave stays
    assert abs(float(f[1]) - (2 / 3 * plain[1] + 1 / 3 * plain[1] / 8)) < 1e-15
    assert abs(float(f[2]) - (1 / 3 * plain[2] + 2 / 3 * plain[2] / 8)) < 1e-15
    assert all(abs(float(f[i]) - plain[i] / 8) < 1e-15 for i in range(3, 8))
    # without scaling nothing is stretched and nothing grows
    f0, m0 = P.rotary_table({"base": 500.0, "dims": 6})
    e0 = RotaryEncoding(RopeSpec(theta=500.0, rotary_dim=6), 10, CPU)
    assert m0 == 1.0 and e0.magnitude == 1.0 and torch.allclose(e0.inv_freq.double(), f0, rtol=1e-6)


def test_plain_rotation_layouts_and_convolution():
    x = torch.arange(2 * 1 * 8, dtype=torch.float64).view(2, 1, 8) + 1.0
    rot = {"base": 100.0, "dims": 4}
    half, inter = P.rotate(x, rot, False), P.rotate(x, rot, True)
    assert torch.equal(half[0], x[0]) and torch.equal(inter[0], x[0])       # position 0
    assert torch.equal(half[..., 4:], x[..., 4:]) and torch.equal(inter[..., 4:], x[..., 4:])
    c, s = math.cos(1.0), math.sin(1.0)                                    # pair 0 at position 1
    assert abs(float(half[1, 0, 0]) - (9 * c - 11 * s)) < 1e-12            # pairs (0, 2)
    assert abs(float(half[1, 0, 2]) - (11 * c + 9 * s)) < 1e-12
    assert abs(float(inter[1, 0, 0]) - (9 * c - 10 * s)) < 1e-12           # pairs (0, 1)
    assert abs(float(inter[1, 0, 1]) - (10 * c + 9 * s)) < 1e-12
    u = torch.tensor([[1.0], [2.0], [4.0]], dtype=torch.float64)
    y = P.causal_conv(u, torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64))
    assert y.view(-1).tolist() == [1.0, 12.0, 124.0]                       # the last tap is now


def test_plain_delta_rule_writes_and_reads_in_order():
    """One head, keys that are unit vectors already: after writing v at key k with beta = 1
    the read-out at k returns v at once (the read sees the current token's write)."""
    w = {"m.q": torch.eye(4), "m.k": torch.eye(4), "m.v": torch.eye(4), "m.g": torch.eye(4),
         "m.o": torch.eye(4), "m.b": torch.full((1, 4), 50.0), "m.a": torch.zeros(1, 4),
         "m.A_log": torch.tensor([-40.0]), "m.dt_bias": torch.zeros(1), "m.norm": torch.ones(4),
         "m.q.conv": torch.ones(4, 1), "m.k.conv": torch.ones(4, 1), "m.v.conv": torch.ones(4, 1)}
    w = {n: t.double() for n, t in w.items()}
    h = torch.tensor([[9.0, 0.0, 0.0, 0.0]], dtype=torch.float64)
    out = P.gated_delta_rule(h, w, "m.", {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 4, "conv": 1},
                             1e-6)
    v = P.silu(h)
    o = v * 0.5                                    # q = k / sqrt(4), |k| = 1, beta = 1, g = 1
    want = P.rms_norm(o, torch.ones(4, dtype=torch.float64), 1e-6) * P.silu(h)
    assert torch.allclose(out, want, atol=1e-6)
