"""Typed configuration of the Folivik decoder, read from its config.json keys.

A Folivik layer is a pre-norm block, ``x += mixer(norm1(x)); x += ff(norm2(x))``, whose RMS
norms have a weight of one number (the model's last norm too).  ``layers`` lists the layers
in order; each names one of three mixers and its feed-forward (``mlp: null``: none):

* ``latent_attention``: softmax attention whose keys and values are expanded from one cached
  latent per token, with queries that go through a latent of their own (``q_rank``), one
  rotated key part that all heads share (interleaved pairs) and a sigmoid gate per head.
* ``attention``: grouped softmax attention inside a sliding window, with an RMS norm with a
  weight on each q and k head, no rotation, a factor per head on the scores and a bias that
  grows with the logarithm of the distance.
* ``mamba2``: a selective state space layer with a scalar decay per head and token, a short
  causal convolution with a bias on x, B and C, a gate before a grouped RMS norm.

The feed-forward is a mixture of gated experts (``silu``): the scores are the softmax over all
router outputs; a correction per output is added for the choice only; the outputs form groups
of which only the best can be chosen from; the last ``identity`` outputs stand for experts
that return their input; a shared expert runs for every token.

Keys: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``layers``; of a layer ``type``,
``mixer``, ``mlp.{kind, expert.ff, router.{experts, top, identity, scale, groups.{count,
keep}}, shared.ff}``; of latent attention ``heads, dim, rot_dim, vdim, kv_rank, q_rank, scale,
rot.{base, dims}``; of attention ``heads, kv_heads, dim, vdim, scale, mask.size``; of mamba2
``heads, vdim, state, groups, conv, norm_groups``.  Tensors: ``embed``, ``head``,
``final.norm`` and ``l<i>.{norm1, norm2, mix.*, mlp.{e<j>.{gate, up, down}, shared.{gate, up,
down}, router, correction}}``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .specs import (ConfigError, ConvWindowAttentionSpec, LatentAttentionSpec, LayerSpec,
                    Mamba2Spec, ModelSpec, MoESpec, NameLayout, NormSpec, RopeSpec, ScheduleEntry)


def _need(d: Dict[str, Any], key: str, where: str) -> Any:
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"Missing required config key: {where}{key}")
    return d[key]


def _positive(v: Any, what: str) -> int:
    if isinstance(v, bool) or int(v) != v or int(v) <= 0:
        raise ConfigError(f"{what} must be a positive integer, got {v!r}")
    return int(v)


def _count(v: Any, what: str) -> int:
    if v is None:
        return 0
    if isinstance(v, bool) or int(v) != v or int(v) < 0:
        raise ConfigError(f"{what} must be a whole number that is not negative, got {v!r}")
    return int(v)


@dataclass(frozen=True)
class FolivikConfig:
    raw: Dict[str, Any]
    vocab_size: int
    hidden_size: int
    norm_eps: float
    layers: Tuple[LayerSpec, ...]
    architectures: Tuple[str, ...] = ("Folivik",)

    # ------------------------------------------------------------------ parse
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "FolivikConfig":
        width = _positive(_need(raw, "width", ""), "width")
        vocab = _positive(_need(raw, "vocab", ""), "vocab")
        eps = float(_need(_need(raw, "norm", ""), "eps", "norm."))
        if not eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {eps}")
        entries = _need(raw, "layers", "")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("layers must be a non-empty list")
        norm = NormSpec(kind="rmsnorm", eps=eps, scalar_weight=True)
        parsers = {"latent_attention": cls._latent, "attention": cls._attention,
                   "mamba2": cls._mamba2}
        layers: List[LayerSpec] = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]."
            kind = _need(entry, "type", where)
            if kind not in parsers:
                raise ConfigError(f"{where}type {kind!r} is not supported (supported: "
                                  f"{sorted(parsers)})")
            mixer = parsers[kind](_need(entry, "mixer", where), eps, where + "mixer.")
            layers.append(LayerSpec(mixer=mixer, ffn=cls._mlp(entry.get("mlp"), where + "mlp."),
                                    norm=norm, block="prenorm"))
        return cls(raw=copy.deepcopy(raw), vocab_size=vocab, hidden_size=width, norm_eps=eps,
                   layers=tuple(layers),
                   architectures=(str(raw.get("architecture", "Folivik")),))

    @staticmethod
    def _latent(mx: Dict[str, Any], eps: float, where: str) -> LatentAttentionSpec:
        rot_dim = _positive(_need(mx, "rot_dim", where), where + "rot_dim")
        rot = _need(mx, "rot", where)
        base = float(_need(rot, "base", where + "rot."))
        dims = _positive(rot.get("dims") or rot_dim, where + "rot.dims")
        if dims % 2 or dims > rot_dim:
            raise ConfigError(f"{where}rot.dims must be even and at most {rot_dim}, got {dims}")
        if not base > 1.0:
            raise ConfigError(f"{where}rot.base must exceed 1, got {base}")
        return LatentAttentionSpec(
            num_heads=_positive(_need(mx, "heads", where), where + "heads"),
            head_dim=_positive(_need(mx, "dim", where), where + "dim"), rot_dim=rot_dim,
            value_dim=_positive(_need(mx, "vdim", where), where + "vdim"),
            kv_rank=_positive(_need(mx, "kv_rank", where), where + "kv_rank"),
            q_rank=_positive(_need(mx, "q_rank", where), where + "q_rank"),
            scale=float(_need(mx, "scale", where)), norm_eps=eps,
            position=RopeSpec(theta=base, rotary_dim=dims, layout="interleaved"),
            head_gate=True)

    @staticmethod
    def _attention(mx: Dict[str, Any], eps: float, where: str) -> ConvWindowAttentionSpec:
        heads = _positive(_need(mx, "heads", where), where + "heads")
        kv_heads = _positive(mx.get("kv_heads") or heads, where + "kv_heads")
        if heads % kv_heads:
            raise ConfigError(f"{where}heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
        dim = _positive(_need(mx, "dim", where), where + "dim")
        mask = mx.get("mask") or {}
        window = mask.get("size")
        return ConvWindowAttentionSpec(
            num_heads=heads, num_kv_heads=kv_heads, head_dim=dim,
            value_dim=_positive(mx.get("vdim") or dim, where + "vdim"), conv_taps=0,
            position=None, unit_norm=True, norm_eps=eps, scale=float(_need(mx, "scale", where)),
            window=None if window is None else _positive(window, where + "mask.size"),
            keep_first=0, sinks=False, proj_norm=False, softcap=0.0, head_norm_weight=True,
            head_temperature=True, log_distance_bias=True)

    @staticmethod
    def _mamba2(mx: Dict[str, Any], eps: float, where: str) -> Mamba2Spec:
        heads = _positive(_need(mx, "heads", where), where + "heads")
        groups = _positive(mx.get("groups") or 1, where + "groups")
        if heads % groups:
            raise ConfigError(f"{where}heads ({heads}) must be a multiple of groups ({groups})")
        vdim = _positive(_need(mx, "vdim", where), where + "vdim")
        parts = _positive(mx.get("norm_groups") or 1, where + "norm_groups")
        if (heads * vdim) % parts:
            raise ConfigError(f"{where}norm_groups ({parts}) must divide heads * vdim "
                              f"({heads * vdim})")
        return Mamba2Spec(
            num_heads=heads, head_dim=vdim,
            state_dim=_positive(_need(mx, "state", where), where + "state"), groups=groups,
            conv_taps=_positive(_need(mx, "conv", where), where + "conv"), conv_bias=True,
            norm_groups=parts, norm_eps=eps)

    @staticmethod
    def _mlp(mlp: Optional[Dict[str, Any]], where: str) -> Optional[MoESpec]:
        if mlp is None:
            return None
        kind = mlp.get("kind", "moe")
        if kind != "moe":
            raise ConfigError(f"{where}kind {kind!r} is not supported (supported: 'moe')")
        router = _need(mlp, "router", where)
        w = where + "router."
        experts = _positive(_need(router, "experts", w), w + "experts")
        identity = _count(router.get("identity"), w + "identity")
        top = _positive(_need(router, "top", w), w + "top")
        if top > experts + identity:
            raise ConfigError(f"{w}top ({top}) exceeds the router's outputs ({experts + identity})")
        groups = router.get("groups") or {}
        count = _positive(groups.get("count") or 1, w + "groups.count")
        keep = _positive(groups.get("keep") or count, w + "groups.keep")
        if (experts + identity) % count or keep > count:
            raise ConfigError(f"{w}groups: {count} groups must divide the router's "
                              f"{experts + identity} outputs, and keep ({keep}) not exceed them")
        if top > keep * ((experts + identity) // count):
            raise ConfigError(f"{w}top ({top}) exceeds what {keep} groups hold")
        shared = mlp.get("shared") or {}
        return MoESpec(
            num_experts=experts, top=top,
            expert_size=_positive(_need(_need(mlp, "expert", where), "ff", where + "expert."),
                                  where + "expert.ff"),
            shared_size=_count(shared.get("ff"), where + "shared.ff"), shared_gate=False,
            activation="silu", scoring="softmax_all",
            route_scale=float(router.get("scale", 1.0)), weight_eps=1e-20, correction=True,
            groups=count, groups_keep=keep, identity=identity)

    # ------------------------------------------------------------- derivation
    def to_spec(self) -> ModelSpec:
        norm = NormSpec(kind="rmsnorm", eps=self.norm_eps, scalar_weight=True)
        names = NameLayout(embed="embed", layer_prefix="l{i}.", input_norm="norm1",
                           post_mixer_norm="norm2", mixer="mix", ffn="mlp",
                           final_norm="final.norm", lm_head="head", norm_suffix="")
        return ModelSpec(
            architecture=self.architectures[0], hidden_size=self.hidden_size,
            vocab_size=self.vocab_size, layers=self.layers,
            schedule=tuple(ScheduleEntry(i) for i in range(len(self.layers))),
            final_norm=norm, tie_word_embeddings=False, max_position_embeddings=1 << 30,
            eos_token_ids=(), bos_token_id=None, pad_token_id=None, names=names)

    def to_dict(self) -> Dict[str, Any]:
        """The config.json that :meth:`from_dict` reads back to this object."""
        return copy.deepcopy(self.raw)

    # ---------------------------------------------------------------- memory
    def num_parameters(self) -> int:
        from ..parts.model import param_specs_for
        total = 0
        for s in param_specs_for(self.to_spec()):
            n = 1
            for d in s.shape:
                n *= d
            total += n
        return total
