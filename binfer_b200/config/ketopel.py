"""Typed configuration of the Ketopel decoder, read from its config.json keys.

A Ketopel layer is a pre-norm block, ``x += mixer(norm1(x)); x += ff(norm2(x))``, with RMS
norms (weights that multiply directly) and a dense gated feed-forward whose activation is
the tanh form of gelu, or none (``mlp: null``).  Each layer names one of three mixers:

* ``parallel``: two mixers side by side on the same input, ``left_scale * left + right_scale
  * right``.  Left: grouped softmax attention whose q and k projections are RMS-normed over
  all heads at once, with partial rotary positions in halves (optionally stretched by pair
  index, ``rot.scaling``), a score scale from the config and a soft cap.  Right: lightning
  attention, a linear attention with a fixed decay per head, ``silu`` on q, k and v, one RMS
  norm with a weight over the concatenated heads and a sigmoid gate.
* ``latent_attention``: softmax attention whose keys and values are expanded from one cached
  latent vector per token, with one rotated key part that all heads share (interleaved
  pairs) and a sigmoid gate per head.
* ``delta``: the gated delta rule, with a short causal convolution and ``silu`` on q, k and
  v, unit-vector q and k, and a norm weight that the heads share.

``loop`` walks the layers ``start .. stop - 1`` ``times`` times in a row with the same
weights; every pass keeps a cache and state of its own.  Before each pass but the first the
embedding output is added to the stream again, and before every pass row t of the tensor
``loop.step`` (t the pass's number).  The embedding output is ``embed[token] *
embedding.scale``; the model ends in its norm (``final.norm``) and an output head.

Keys: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``layers``,
``loop.{start, stop, times}``; of a layer ``type``, ``mixer``, ``mlp.{kind, ff}``; of the
parallel mixer ``left.{heads, kv_heads, dim, vdim, scale, softcap, rot.{base, dims,
scaling.{factor, original, fast, slow}}}``, ``right.{heads, dim, vdim, decay}``,
``left_scale``, ``right_scale``; of latent attention ``heads, dim, rot_dim, vdim, kv_rank,
scale, rot.{base, dims}``; of the delta rule ``heads, kv_heads, dim, vdim, conv``.  Tensors:
``embed``, ``head``, ``final.norm``, ``loop.step`` and ``l<i>.{norm1, norm2, mix.*, mlp.{gate,
up, down}}``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .specs import (ConfigError, ConvWindowAttentionSpec, GatedDeltaRuleSpec, GatedMLPSpec,
                    LatentAttentionSpec, LayerSpec, MixerBranch, ModelSpec, NameLayout, NormSpec,
                    ParallelMixersSpec, PassStart, RampScaling, RetentionSpec, RopeSpec,
                    ScheduleEntry)

PASS_TABLE_NAME = "loop.step"
_MLP_NAMES = ("gate", "up", "down")


def _need(d: Dict[str, Any], key: str, where: str) -> Any:
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"Missing required config key: {where}{key}")
    return d[key]


def _positive(v: Any, what: str) -> int:
    if isinstance(v, bool) or int(v) != v or int(v) <= 0:
        raise ConfigError(f"{what} must be a positive integer, got {v!r}")
    return int(v)


def _rope(rot: Optional[Dict[str, Any]], dim: int, where: str, layout: str = "half",
          default_dims: Optional[int] = None) -> Optional[RopeSpec]:
    if not rot:
        return None
    base = float(_need(rot, "base", where))
    dims = _positive(rot.get("dims") or default_dims or dim, where + "dims")
    if dims % 2 or dims > dim:
        raise ConfigError(f"{where}dims must be even and at most {dim}, got {dims}")
    if not base > 1.0:
        raise ConfigError(f"{where}base must exceed 1, got {base}")
    sc = rot.get("scaling")
    ramp = None
    if sc:
        w = where + "scaling."
        ramp = RampScaling(factor=float(_need(sc, "factor", w)),
                           original=float(_need(sc, "original", w)),
                           fast=float(_need(sc, "fast", w)), slow=float(_need(sc, "slow", w)))
        if ramp.factor <= 0 or ramp.original <= 0 or ramp.fast <= 0 or ramp.slow <= 0:
            raise ConfigError(f"{w}factor, original, fast and slow must be positive")
    return RopeSpec(theta=base, rotary_dim=dims, ramp_scaling=ramp, layout=layout)


@dataclass(frozen=True)
class KetopelConfig:
    raw: Dict[str, Any]
    vocab_size: int
    hidden_size: int
    norm_eps: float
    embedding_scale: float
    layers: Tuple[LayerSpec, ...]
    loop: Optional[Tuple[int, int, int]]        # (start, stop, times)
    architectures: Tuple[str, ...] = ("Ketopel",)

    # ------------------------------------------------------------------ parse
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "KetopelConfig":
        width = _positive(_need(raw, "width", ""), "width")
        vocab = _positive(_need(raw, "vocab", ""), "vocab")
        eps = float(_need(_need(raw, "norm", ""), "eps", "norm."))
        if not eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {eps}")
        scale = float((raw.get("embedding") or {}).get("scale", 1.0))
        entries = _need(raw, "layers", "")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("layers must be a non-empty list")
        norm = NormSpec(kind="rmsnorm", eps=eps)
        parsers = {"parallel": cls._parallel, "latent_attention": cls._latent,
                   "delta": cls._delta}
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
        loop = None
        lp = raw.get("loop")
        if lp:
            start, stop = int(_need(lp, "start", "loop.")), int(_need(lp, "stop", "loop."))
            times = _positive(_need(lp, "times", "loop."), "loop.times")
            if not 0 <= start < stop <= len(layers):
                raise ConfigError(f"loop: start {start} and stop {stop} must name a run of the "
                                  f"{len(layers)} layers")
            loop = (start, stop, times)
        return cls(raw=copy.deepcopy(raw), vocab_size=vocab, hidden_size=width, norm_eps=eps,
                   embedding_scale=scale, layers=tuple(layers), loop=loop,
                   architectures=(str(raw.get("architecture", "Ketopel")),))

    @staticmethod
    def _parallel(mx: Dict[str, Any], eps: float, where: str) -> ParallelMixersSpec:
        left = _need(mx, "left", where)
        w = where + "left."
        heads = _positive(_need(left, "heads", w), w + "heads")
        kv_heads = _positive(left.get("kv_heads") or heads, w + "kv_heads")
        if heads % kv_heads:
            raise ConfigError(f"{w}heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
        dim = _positive(_need(left, "dim", w), w + "dim")
        softcap = float(left.get("softcap") or 0.0)
        if softcap < 0:
            raise ConfigError(f"{w}softcap must not be negative")
        attention = ConvWindowAttentionSpec(
            num_heads=heads, num_kv_heads=kv_heads, head_dim=dim,
            value_dim=_positive(left.get("vdim") or dim, w + "vdim"), conv_taps=0,
            position=_rope(left.get("rot"), dim, w + "rot."), unit_norm=False, norm_eps=eps,
            scale=float(_need(left, "scale", w)), window=None, keep_first=0, sinks=False,
            proj_norm=True, softcap=softcap)
        right = _need(mx, "right", where)
        w = where + "right."
        r_heads = _positive(_need(right, "heads", w), w + "heads")
        r_dim = _positive(_need(right, "dim", w), w + "dim")
        decay = _need(right, "decay", w)
        if not isinstance(decay, list) or len(decay) != r_heads:
            raise ConfigError(f"{w}decay must list one number per head ({r_heads})")
        lightning = RetentionSpec(
            num_heads=r_heads, qk_dim=r_dim, v_dim=_positive(right.get("vdim") or r_dim, w + "vdim"),
            decays=tuple(float(d) for d in decay), position=None, norm_eps=eps, k_scale=1.0,
            activation="silu", norm_over="all", norm_weight=True, gate="sigmoid")
        return ParallelMixersSpec(branches=(
            MixerBranch(attention, "left.", float(mx.get("left_scale", 1.0))),
            MixerBranch(lightning, "right.", float(mx.get("right_scale", 1.0)))))

    @staticmethod
    def _latent(mx: Dict[str, Any], eps: float, where: str) -> LatentAttentionSpec:
        rot_dim = _positive(_need(mx, "rot_dim", where), where + "rot_dim")
        return LatentAttentionSpec(
            num_heads=_positive(_need(mx, "heads", where), where + "heads"),
            head_dim=_positive(_need(mx, "dim", where), where + "dim"), rot_dim=rot_dim,
            value_dim=_positive(_need(mx, "vdim", where), where + "vdim"),
            kv_rank=_positive(_need(mx, "kv_rank", where), where + "kv_rank"),
            scale=float(_need(mx, "scale", where)), norm_eps=eps,
            position=_rope(_need(mx, "rot", where), rot_dim, where + "rot.", "interleaved",
                           rot_dim),
            head_gate=True)

    @staticmethod
    def _delta(mx: Dict[str, Any], eps: float, where: str) -> GatedDeltaRuleSpec:
        heads = _positive(_need(mx, "heads", where), where + "heads")
        qk_heads = _positive(mx.get("kv_heads") or heads, where + "kv_heads")
        if heads % qk_heads:
            raise ConfigError(f"{where}heads ({heads}) must be a multiple of kv_heads ({qk_heads})")
        taps = int(mx.get("conv") or 0)
        if taps < 0:
            raise ConfigError(f"{where}conv must not be negative")
        return GatedDeltaRuleSpec(
            num_heads=heads, num_qk_heads=qk_heads,
            qk_dim=_positive(_need(mx, "dim", where), where + "dim"),
            v_dim=_positive(_need(mx, "vdim", where), where + "vdim"), conv_taps=taps,
            unit_eps=1e-6, norm_eps=eps)

    @staticmethod
    def _mlp(mlp: Optional[Dict[str, Any]], where: str) -> Optional[GatedMLPSpec]:
        if mlp is None:
            return None
        kind = mlp.get("kind", "dense")
        if kind != "dense":
            raise ConfigError(f"{where}kind {kind!r} is not supported (supported: 'dense')")
        return GatedMLPSpec(intermediate_size=_positive(_need(mlp, "ff", where), where + "ff"),
                            activation="gelu_tanh", names=_MLP_NAMES)

    # ------------------------------------------------------------- derivation
    def schedule(self) -> Tuple[ScheduleEntry, ...]:
        """One entry per layer run; a looped run of layers repeats, and the first entry of
        every pass says what the stream takes before it."""
        n = len(self.layers)
        if self.loop is None:
            return tuple(ScheduleEntry(i) for i in range(n))
        start, stop, times = self.loop
        out = [ScheduleEntry(i) for i in range(start)]
        for t in range(times):
            for i in range(start, stop):
                before = PassStart(embedding=t > 0, row=t) if i == start else None
                out.append(ScheduleEntry(i, None, before))
        return tuple(out + [ScheduleEntry(i) for i in range(stop, n)])

    def to_spec(self) -> ModelSpec:
        norm = NormSpec(kind="rmsnorm", eps=self.norm_eps)
        names = NameLayout(embed="embed", layer_prefix="l{i}.", input_norm="norm1",
                           post_mixer_norm="norm2", mixer="mix", ffn="mlp",
                           final_norm="final.norm", lm_head="head", norm_suffix="")
        return ModelSpec(
            architecture=self.architectures[0], hidden_size=self.hidden_size,
            vocab_size=self.vocab_size, layers=self.layers, schedule=self.schedule(),
            final_norm=norm, tie_word_embeddings=False, max_position_embeddings=1 << 30,
            eos_token_ids=(), bos_token_id=None, pad_token_id=None,
            embedding_scale=self.embedding_scale, names=names,
            pass_table=(PASS_TABLE_NAME, self.loop[2]) if self.loop is not None else None)

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
