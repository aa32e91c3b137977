"""Architecture-neutral descriptions of a decoder: what each layer is made of.

A model family (for instance ``config/qwen3.py``) turns its own ``config.json``
keys into a :class:`ModelSpec`.  Everything downstream (weights, parts, cache
manager, step function) reads only these specs, never a family's config, so a
new architecture is a new config class plus, where needed, new parts.

The reference keeps every size in one flat ``LlamaConfig`` and branches on it
inside the engine (src/model/config.ts:5-60, src/engine/batched_engine.ts:834,
1186); here each part gets exactly the sizes and constants it needs.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class RopeSpec:
    """Rotate-half rotary position encoding over the first ``rotary_dim`` of a head."""

    kind: str = "rope"
    theta: float = 10000.0
    rotary_dim: int = 0          # 0 means the whole head
    # linear position scaling (angle = position / factor * inv_freq); 1.0 = none
    factor: float = 1.0
    # scaling by wavelength: see WavelengthScaling; None = none
    wavelength_scaling: Optional["WavelengthScaling"] = None
    # scaling by pair index with a ramp between two indices: see RampScaling; None = none
    ramp_scaling: Optional["RampScaling"] = None
    # "half": the pair (i, i + rot/2); "interleaved": the pair (2i, 2i + 1)
    layout: str = "half"
    # where in a head the rotated sizes start (0: the head's first ``rotary_dim`` sizes)
    offset: int = 0


@dataclass(frozen=True)
class WavelengthScaling:
    """Frequencies stretched by their wavelength ``l = 2 pi / f`` against a context length
    ``original``: short waves (``l < original / high``) stay, long ones (``l > original /
    low``) become ``f / factor``, and between the two, with ``s = (original / l - low) /
    (high - low)``, ``(1 - s) f / factor + s f``."""

    factor: float = 1.0
    low: float = 1.0
    high: float = 4.0
    original: float = 8192.0


@dataclass(frozen=True)
class RampScaling:
    """Frequencies stretched for contexts beyond ``original`` positions, by pair index.  A
    wave that makes t turns over ``original`` positions has the (real-valued) index
    ``n(t) = rot ln(original / (2 pi t)) / (2 ln theta)``.  With ``lo = max(floor(n(fast)),
    0)``, ``hi = min(ceil(n(slow)), rot - 1)`` and ``r_i = clamp((i - lo) / max(hi - lo,
    0.001), 0, 1)`` the frequency of pair i is ``(1 - r_i) f_i + r_i f_i / factor``: fast
    waves stay, slow ones are divided by ``factor``.  Cosines and sines are multiplied by
    ``magnitude`` (None: ``0.1 ln(factor) + 1``), which scales q and k alike."""

    factor: float = 1.0
    original: float = 4096.0
    fast: float = 32.0
    slow: float = 1.0
    magnitude: Optional[float] = None


@dataclass(frozen=True)
class NormSpec:
    """``offset``: what is added to the stored weight to get the one that multiplies (1.0 for
    a family whose norm weights hold the deviation from one)."""

    kind: str = "rmsnorm"      # or "layernorm": mean taken off, weight and bias
    eps: float = 1e-6
    offset: float = 0.0
    # layernorm: what follows the weight tensor's name to give the bias tensor's (None: no bias)
    bias_suffix: Optional[str] = None
    # rmsnorm: the weight tensor is a single number that multiplies every coordinate
    scalar_weight: bool = False


@dataclass(frozen=True)
class ScoreSpec:
    """What is done to an attention score ``s = (q . k) * scale`` of query position p and key
    position j before the softmax.  None of it is Qwen3's; a family whose attention has it
    names it here, and the mixer takes the kernel that applies it.

    ``softcap`` c > 0: ``s <- c * tanh(s / c)``.  ``slopes`` (one number per query head):
    ``s <- s + slope_h * (j - p)``, a bias per distance.  ``sinks``: a learned logit per query
    head (tensor ``sinks [heads]`` of the mixer) that joins the softmax's denominator and
    takes no value: ``P_j = exp(s_j) / (exp(sink_h) + sum_j exp(s_j))``."""

    softcap: float = 0.0
    slopes: Optional[Tuple[float, ...]] = None
    sinks: bool = False


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query causal attention over a paged key/value cache."""

    kind: str = "attention"
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    qk_norm: bool = False        # per-head RMSNorm on q and k before the rotation
    qk_norm_eps: float = 1e-6
    bias: bool = False           # q/k/v/o projection biases
    window: Optional[int] = None  # keys j with p - window < j <= p; None = all keys
    scale: Optional[float] = None  # None = 1/sqrt(head_dim)
    position: Optional[object] = None   # RopeSpec, or any spec whose kind is registered
    score: Optional[ScoreSpec] = None   # changes to the scores before the softmax; None: none

    @property
    def group_size(self) -> int:
        return self.num_heads // self.num_kv_heads

    @property
    def softmax_scale(self) -> float:
        return self.scale if self.scale is not None else self.head_dim ** -0.5


@dataclass(frozen=True)
class GatedMLPSpec:
    """Dense gated feed-forward: down(act(gate(x)) * up(x))."""

    kind: str = "gated_mlp"
    intermediate_size: int = 0
    activation: str = "silu"     # or "gelu_tanh": 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
    bias: bool = False
    # the tensors' names inside the feed-forward's prefix: gate, up, down
    names: Tuple[str, str, str] = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")


@dataclass(frozen=True)
class PooledWindowAttentionSpec:
    """Grouped-query attention over a window of tokens and, behind the window, one mean key
    and value per block of ``pool`` tokens (a block is seen once all of it lies before the
    window); keys of size ``head_dim``, values of size ``value_dim``.

    ``value_rotation`` (a :class:`RopeSpec` over the whole value head): values are cached
    turned by their own position and a head's output is turned back by the query's.
    ``sink``: a constant logit that joins the softmax's denominator and has no value (0.0
    adds one to the denominator); None: no sink.  ``head_gate``: each head's output is
    multiplied by the sigmoid of a projection of the mixer's input, one number per head.
    ``own_cache`` False: the layer reads another layer's keys and values and has no key or
    value tensors of its own.  ``names``: the tensors inside the mixer's prefix."""

    kind: str = "pooled_window_attention"
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    value_dim: int = 0
    qk_norm: bool = True
    qk_norm_eps: float = 1e-6
    window: Optional[int] = None     # tokens j with p - window < j <= p; None: every token
    pool: int = 0                    # 0: nothing behind the window is seen
    scale: Optional[float] = None    # None = 1/sqrt(head_dim)
    position: Optional[RopeSpec] = None
    value_rotation: Optional[RopeSpec] = None
    interleaved: bool = False        # pairs (2m, 2m+1) instead of (m, m + half), q, k and v alike
    sink: Optional[float] = None
    head_gate: bool = False
    own_cache: bool = True
    names: Tuple[Tuple[str, str], ...] = (
        ("q", "q_proj.weight"), ("k", "k_proj.weight"), ("v", "v_proj.weight"),
        ("o", "o_proj.weight"), ("g", "g_proj.weight"), ("q_norm", "q_norm.weight"),
        ("k_norm", "k_norm.weight"))

    @property
    def softmax_scale(self) -> float:
        return self.scale if self.scale is not None else self.head_dim ** -0.5


@dataclass(frozen=True)
class MLSTMSpec:
    """A matrix memory with exponential input and forget gates per head (mLSTM), its state
    ``S [qk_dim, v_dim]``, ``n [qk_dim]`` and a running maximum carried per request.
    ``gate_cap`` c > 0: a gate's pre-activation z becomes ``c tanh(z / c)``.  ``norm_eps``:
    of the per-head root mean square that divides the memory's output.  ``names``: the
    tensors inside the mixer's prefix."""

    kind: str = "mlstm"
    num_heads: int = 0
    qk_dim: int = 0
    v_dim: int = 0
    gate_cap: float = 0.0
    norm_eps: float = 1e-6
    names: Tuple[Tuple[str, str], ...] = (
        ("q", "q.weight"), ("k", "k.weight"), ("v", "v.weight"), ("g", "g.weight"),
        ("o", "o.weight"), ("norm", "norm.weight"), ("i", "i.weight"), ("i_bias", "i.bias"),
        ("f", "f.weight"), ("f_bias", "f.bias"))


@dataclass(frozen=True)
class ConvWindowAttentionSpec:
    """Grouped-query softmax attention whose q, k and v projections pass a short causal
    convolution over time, with a sliding window that keeps the request's first tokens.

    Order: projection, convolution per channel (``conv_taps`` taps, 0 or 1: none), an RMS norm
    with weights over the whole q projection and over the whole k projection, all heads at
    once (``proj_norm``; tensors ``q_norm``, ``k_norm`` of the projections' sizes; without a
    convolution only), rotation of q and k (``position``), each q and k head divided by its
    root mean square (``unit_norm``, no weight, ``norm_eps``), scores ``(q . k) * scale``, a
    soft cap ``s <- c tanh(s / c)`` (``softcap`` c > 0), the mask (position i
    sees j <= i with ``i - j < window`` or ``j < keep_first``; ``window`` None: every j <= i),
    softmax whose denominator also holds ``exp(sink_h)`` when ``sinks``, values of size
    ``value_dim``, output projection.  ``names``: the tensors inside the mixer's prefix;
    a convolution's tensor is the projection's name with ``conv_suffix``.

    ``head_norm_weight``: the norm of each q and k head (``unit_norm``) is followed by a weight
    of ``head_dim`` numbers that the heads share (tensors ``q_head_norm``, ``k_head_norm``).
    ``head_temperature``: head h's scores are multiplied by the number ``temp[h]`` (a tensor of
    the mixer).  ``log_distance_bias``: ``b1_h ln(1 + b2_h (i - j))`` is taken off the score of
    query i and key j (tensors ``bias_slope`` b1 and ``bias_rate`` b2, one number per head)."""

    kind: str = "conv_window_attention"
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    value_dim: int = 0
    conv_taps: int = 0
    position: Optional[RopeSpec] = None
    unit_norm: bool = True
    norm_eps: float = 1e-6
    scale: Optional[float] = None
    window: Optional[int] = None
    keep_first: int = 0
    sinks: bool = False
    proj_norm: bool = False
    softcap: float = 0.0
    head_norm_weight: bool = False
    head_temperature: bool = False
    log_distance_bias: bool = False
    names: Tuple[Tuple[str, str], ...] = (("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"),
                                          ("sink", "sink"), ("q_norm", "q.norm"),
                                          ("k_norm", "k.norm"), ("q_head_norm", "q.norm"),
                                          ("k_head_norm", "k.norm"), ("temp", "temp"),
                                          ("bias_slope", "r1"), ("bias_rate", "r2"))
    conv_suffix: str = ".conv"

    @property
    def softmax_scale(self) -> float:
        return self.scale if self.scale is not None else self.head_dim ** -0.5


@dataclass(frozen=True)
class RetentionSpec:
    """Linear attention with a fixed decay per head: ``S <- decay_h S + k v^T``, ``o = S^T q``
    (no softmax, no denominator).  q and k are turned by ``position`` and k multiplied by
    ``k_scale`` (None: ``qk_dim ** -0.5``); each head's output is divided by its root mean
    square (``norm_eps``, no weight), multiplied by ``silu`` of a gate projection and projected.

    ``activation`` ("silu"): applied to the q, k and v projections first (lightning
    attention).  ``norm_over`` "all": one root mean square over the concatenated heads
    instead of one per head.  ``norm_weight``: the normed output is multiplied by a tensor
    ``norm`` of ``heads * v_dim`` numbers.  ``gate``: "silu" or "sigmoid"."""

    kind: str = "retention"
    num_heads: int = 0
    qk_dim: int = 0
    v_dim: int = 0
    decays: Tuple[float, ...] = ()
    position: Optional[RopeSpec] = None
    norm_eps: float = 1e-6
    k_scale: Optional[float] = None
    activation: Optional[str] = None
    norm_over: str = "head"
    norm_weight: bool = False
    gate: str = "silu"
    names: Tuple[Tuple[str, str], ...] = (("q", "q"), ("k", "k"), ("v", "v"), ("g", "g"),
                                          ("o", "o"), ("norm", "norm"))


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Causal softmax attention whose keys and values are expanded from one cached latent
    vector per token.  A down projection yields ``kv_rank + rot_dim`` numbers: the first
    ``kv_rank``, RMS-normed with a weight, are the latent c; the last ``rot_dim``, rotated,
    are a key part that all heads share.  Head h has the key ``[W_uk,h c | shared part]``
    against a query ``[head_dim plain | rot_dim rotated]`` and the value ``W_uv,h c`` of
    ``value_dim`` numbers.  Only c and the shared part are cached.  ``head_gate``: head h's
    output is multiplied by the sigmoid of a projection of the mixer's input to one number
    per head.  ``position``: the rotation of the ``rot_dim`` parts (layout and offset are
    set by the mixer).  ``q_rank`` > 0: the queries go through a latent too, ``q = W_uq
    rmsnorm(W_dq h)`` with a weight of ``q_rank`` numbers (tensors ``dq``, ``dq_norm``, ``uq``
    in place of ``q``).  ``names``: the tensors inside the mixer's prefix."""

    kind: str = "latent_attention"
    num_heads: int = 0
    head_dim: int = 0            # plain (unrotated) sizes of a query/key head
    rot_dim: int = 0
    value_dim: int = 0
    kv_rank: int = 0
    scale: Optional[float] = None    # None = 1/sqrt(head_dim + rot_dim)
    norm_eps: float = 1e-6
    position: Optional[RopeSpec] = None
    head_gate: bool = True
    q_rank: int = 0
    names: Tuple[Tuple[str, str], ...] = (("q", "q"), ("dkv", "dkv"), ("dkv_norm", "dkv.norm"),
                                          ("uk", "uk"), ("uv", "uv"), ("g", "g"), ("o", "o"),
                                          ("dq", "dq"), ("dq_norm", "dq.norm"), ("uq", "uq"))

    @property
    def softmax_scale(self) -> float:
        return self.scale if self.scale is not None else (self.head_dim + self.rot_dim) ** -0.5


@dataclass(frozen=True)
class GatedDeltaRuleSpec:
    """A matrix memory written by the delta rule with a decay per token and head.  Per value
    head, with a state ``S [qk_dim, v_dim]`` that starts at zero::

        S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

    q and k have ``num_qk_heads`` heads (value head h reads head ``h // (num_heads /
    num_qk_heads)``); q, k and v pass a causal convolution of ``conv_taps`` taps per channel
    and ``silu``; q and k are then made unit vectors per head (``x / sqrt(sum x^2 +
    unit_eps)``) and q multiplied by ``qk_dim ** -0.5``.  ``beta = sigmoid(W_b h)`` and
    ``g = exp(-exp(A_log) softplus(W_a h + dt_bias))``, one each per value head.  Each head's
    output is divided by its root mean square (``norm_eps``), multiplied by a weight of
    ``v_dim`` numbers that the heads share and by ``silu`` of a gate projection."""

    kind: str = "gated_delta_rule"
    num_heads: int = 0
    num_qk_heads: int = 0
    qk_dim: int = 0
    v_dim: int = 0
    conv_taps: int = 0
    unit_eps: float = 1e-6
    norm_eps: float = 1e-6
    names: Tuple[Tuple[str, str], ...] = (
        ("q", "q"), ("k", "k"), ("v", "v"), ("b", "b"), ("a", "a"), ("g", "g"), ("o", "o"),
        ("A_log", "A_log"), ("dt_bias", "dt_bias"), ("norm", "norm"))
    conv_suffix: str = ".conv"


@dataclass(frozen=True)
class Mamba2Spec:
    """A selective state space layer in its scalar-decay form (Mamba-2).  One input projection
    yields ``[z | x | B | C | dt]``: ``inner = num_heads * head_dim`` numbers each for the gate
    z and the input x, ``groups * state_dim`` each for B and C, one step size per head.  x, B
    and C pass a causal convolution of ``conv_taps`` taps per channel (with a bias when
    ``conv_bias``) and ``silu``.  Per head h, which reads group ``h // (num_heads / groups)``,
    with a state ``S [state_dim, head_dim]`` that starts at zero::

        dt = softplus(dt + dt_bias_h);   S <- exp(-exp(A_log_h) dt) S + dt B x^T
        y = S^T C + D_h x

    The concatenated heads are multiplied by ``silu(z)``, then RMS-normed in ``norm_groups``
    equal parts (each by its own root mean square, ``norm_eps``), times a weight of ``inner``
    numbers, and projected.  ``names``: the tensors inside the mixer's prefix."""

    kind: str = "mamba2"
    num_heads: int = 0
    head_dim: int = 0
    state_dim: int = 0
    groups: int = 1
    conv_taps: int = 0
    conv_bias: bool = True
    norm_groups: int = 1
    norm_eps: float = 1e-6
    names: Tuple[Tuple[str, str], ...] = (
        ("in", "in"), ("conv", "conv"), ("conv_bias", "conv.b"), ("dt_bias", "dt_bias"),
        ("A_log", "A_log"), ("D", "D"), ("norm", "norm"), ("o", "o"))


@dataclass(frozen=True)
class MixerBranch:
    """One of the mixers that run side by side: its spec, the name that follows the
    combined mixer's prefix (``left.``), and the factor of its output in the sum."""

    spec: object = None
    prefix: str = ""
    scale: float = 1.0


@dataclass(frozen=True)
class ParallelMixersSpec:
    """Several mixers that read the same input; the result is ``sum_i scale_i mixer_i(h)``."""

    kind: str = "parallel_mixers"
    branches: Tuple[MixerBranch, ...] = ()


@dataclass(frozen=True)
class MoESpec:
    """Mixture of gated feed-forward experts: each token runs the ``top`` experts with the
    largest router logits, weighted by the softmax over those logits alone.  A shared expert
    (``shared_size`` > 0) runs for every token, multiplied by the sigmoid of a projection of
    its own to one number when ``shared_gate``.  Names inside the feed-forward's prefix:
    ``expert_prefix.format(e=...)`` and ``shared_prefix`` before ``names`` (gate, up, down);
    ``router_name``; ``shared_gate_name`` inside the shared expert's prefix.

    ``scoring`` "softmax_all": the scores are the softmax over every router output instead, and
    the chosen experts' weights are their scores divided by their sum (plus ``weight_eps``),
    times ``route_scale``.  ``correction``: a tensor (``correction_name``, one number per
    router output) is added to the scores for the choice only.  ``groups`` > 1: the router's
    outputs form that many equal groups of neighbours, a group counts by its largest choice
    score, and only the outputs of the best ``groups_keep`` groups can be chosen.
    ``identity`` > 0: the router has that many outputs behind the experts' that stand for
    experts whose output is their input (no tensors)."""

    kind: str = "moe"
    num_experts: int = 0
    top: int = 0
    expert_size: int = 0
    shared_size: int = 0
    shared_gate: bool = False
    activation: str = "silu"
    names: Tuple[str, str, str] = ("gate", "up", "down")
    expert_prefix: str = "e{e}."
    shared_prefix: str = "shared."
    router_name: str = "router"
    shared_gate_name: str = "sg"
    scoring: str = "softmax_top"
    route_scale: float = 1.0
    weight_eps: float = 0.0
    correction: bool = False
    correction_name: str = "correction"
    groups: int = 1
    groups_keep: int = 1
    identity: int = 0


@dataclass(frozen=True)
class LayerSpec:
    """One decoder layer: which mixer, which feed-forward, which norm, how arranged."""

    mixer: object = None         # a mixer spec with a ``kind`` attribute
    ffn: object = None           # a feed-forward spec with a ``kind`` attribute (None: the
                                 # arrangement has no second sublayer in this layer)
    norm: NormSpec = NormSpec()
    block: str = "prenorm"       # arrangement of the parts inside the layer: "prenorm",
                                 # "sublayer_norm", or "parallel" (one norm, both sublayers
                                 # read it, their sum is added)


@dataclass(frozen=True)
class PassStart:
    """What is added to the residual stream right before a schedule entry that opens a pass
    over a run of layers that is walked several times: the embedding output once more
    (``embedding``), then row ``row`` of the model's table of pass vectors
    (:attr:`ModelSpec.pass_table`; None: nothing)."""

    embedding: bool = False
    row: Optional[int] = None


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.

    ``layer`` indexes :attr:`ModelSpec.layers`.  ``cache_from`` is ``None`` when
    this execution keeps a cache of its own, else the index of the schedule
    entry whose cache it reads (it then writes none).  ``before``: see
    :class:`PassStart`.
    """

    layer: int
    cache_from: Optional[int] = None
    before: Optional[PassStart] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: NormSpec
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 4096
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    pad_token_id: Optional[int] = None
    # multiplies the embedding output / the logits; 1.0 = none
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    # tensor-name layout of the family (prefixes for embed, layers, norm, head)
    names: "NameLayout" = None
    # (tensor name, rows) of a table ``[rows, hidden_size]`` whose rows schedule entries add
    # to the stream (ScheduleEntry.before); None: the model has none
    pass_table: Optional[Tuple[str, int]] = None


@dataclass(frozen=True)
class NameLayout:
    """Where a family keeps its tensors in a checkpoint (Hugging Face names).

    The reference builds these strings inline at each use
    (src/engine/batched_engine.ts:773,802,811-813,1717,1737,1753-1755).
    """

    embed: str = "model.embed_tokens.weight"
    layer_prefix: str = "model.layers.{i}."
    input_norm: str = "input_layernorm"
    post_mixer_norm: str = "post_attention_layernorm"
    mixer: str = "self_attn"
    ffn: str = "mlp"
    final_norm: str = "model.norm.weight"
    lm_head: str = "lm_head.weight"
    # what follows a layer norm's name to give its tensor's name
    norm_suffix: str = ".weight"
    # further norms of a layer, for arrangements that have more than the two above:
    # (role, name inside the layer) pairs
    more_norms: Tuple[Tuple[str, str], ...] = ()

    def norm(self, role: str) -> str:
        """The name, inside a layer, of the norm that plays ``role``: ``input``,
        ``post_mixer`` or one of ``more_norms``."""
        table = {"input": self.input_norm, "post_mixer": self.post_mixer_norm,
                 **dict(self.more_norms)}
        if role not in table:
            raise KeyError(f"no norm with the role {role!r} in this family's names "
                           f"(known: {sorted(table)})")
        return table[role]


class ConfigError(ValueError):
    """A config.json that is missing a key or asks for something unsupported."""
