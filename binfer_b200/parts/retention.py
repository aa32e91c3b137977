"""Retention (linear attention with a fixed decay per head) as a mixer part with
per-request state.

Per head, with a state ``S [dk, dv]`` that starts at zero for a new request::

    q = rot(W_q h)      k = rot(W_k h) / sqrt(dk)      v = W_v h
    S <- decay_h S + k v^T          o = S^T q

and the mixer returns ``W_o (o / rms_head(o) * silu(W_g h))``.  There is no softmax and no
denominator.  The spec's options give lightning attention: ``silu`` on the q, k and v
projections, no factor on k, one root mean square over all heads of a token with a weight,
and a sigmoid gate.  The q, k, v and gate projections are one product against the stacked weight;
rotation, recurrence and the head norm are float whatever the engine's precision; the state
lives in the cache manager's slots and is carried from step to step, so a prompt can be cut
anywhere and a request can share a step with others.  ``w_in`` / ``w_out`` /
``run(proj, ctx, view, out, out_scale)`` let ``ParallelMixers`` run it as a branch.
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch

from ..cache.manager import StateNeed
from ..config.specs import RetentionSpec
from ..csrc import ops
from ..weights.loader import ParamSpec
from .base import BuildEnv, EntryView, Mixer, StepContext, build_position, register_mixer
from .linear import linear


class RetentionMixer(Mixer):
    def __init__(self, spec: RetentionSpec, hidden_size: int, prefix: str, env: BuildEnv):
        if spec.qk_dim > ops.RETENTION_MAX_QK_DIM:
            raise ValueError(f"retention: a key size of {spec.qk_dim} is not supported "
                             f"(at most {ops.RETENTION_MAX_QK_DIM})")
        if len(spec.decays) != spec.num_heads:
            raise ValueError("retention: one decay per head is needed")
        self.spec, self.hidden, self.prefix, self.env = spec, hidden_size, prefix, env
        self.heads, self.dk, self.dv = spec.num_heads, spec.qk_dim, spec.v_dim
        self.qk_size, self.v_size = self.heads * self.dk, self.heads * self.dv
        self.position = (build_position(spec.position, self.dk, env)
                         if spec.position is not None else None)
        if self.position is not None and (self.position.inv_freq is None
                                          or getattr(self.position, "interleaved", False)
                                          or getattr(self.position, "offset", 0)
                                          or getattr(self.position, "magnitude", 1.0) != 1.0):
            raise ValueError("retention takes plain rotary encodings in halves only")
        if spec.activation not in (None, "silu"):
            raise ValueError(f"retention: activation {spec.activation!r} is not supported")
        if spec.norm_over not in ("head", "all") or spec.gate not in ("silu", "sigmoid"):
            raise ValueError("retention: norm_over is 'head' or 'all', gate 'silu' or 'sigmoid'")
        self.k_scale = self.dk ** -0.5 if spec.k_scale is None else float(spec.k_scale)
        self.plain_out = (spec.norm_over == "head" and not spec.norm_weight
                          and spec.gate == "silu")
        self.norm_w = None
        self.decays = torch.tensor(spec.decays, dtype=torch.float64).to(torch.float32).to(env.device)
        self.names = dict(spec.names)
        self.in_rows, self.out_cols = 2 * self.qk_size + 2 * self.v_size, self.v_size
        self.w_in = self.w_out = None

    # ----------------------------------------------------------------- weights
    def _spec(self, role: str) -> ParamSpec:
        shape = {"q": (self.qk_size, self.hidden), "k": (self.qk_size, self.hidden),
                 "v": (self.v_size, self.hidden), "g": (self.v_size, self.hidden),
                 "o": (self.hidden, self.v_size), "norm": (self.v_size,)}[role]
        if role == "norm":
            return ParamSpec(self.prefix + self.names[role], shape, init="norm", role="vector")
        return ParamSpec(self.prefix + self.names[role], shape)

    def param_specs(self) -> List[ParamSpec]:
        roles = ("q", "k", "v", "g", "o") + (("norm",) if self.spec.norm_weight else ())
        return [self._spec(r) for r in roles]

    def load(self, get: Callable[[ParamSpec], torch.Tensor]) -> None:
        g = lambda role: get(self._spec(role))          # noqa: E731
        self.w_in = torch.cat([g("q"), g("k"), g("v"), g("g")], dim=0).contiguous()
        self.w_out = g("o")
        if self.spec.norm_weight:
            self.norm_w = g("norm")

    # ------------------------------------------------------------------- state
    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.heads * self.dk * self.dv,), "float32")

    # ----------------------------------------------------------------- forward
    def forward(self, x: torch.Tensor, ctx: StepContext, view: EntryView) -> torch.Tensor:
        out = torch.empty((x.shape[0], self.out_cols), dtype=x.dtype, device=x.device)
        self.run(linear(x, self.w_in), ctx, view, out, 1.0)
        return linear(out, self.w_out)

    def run(self, proj: torch.Tensor, ctx: StepContext, view: EntryView, out: torch.Tensor,
            out_scale: float) -> None:
        T = proj.shape[0]
        o_raw = torch.empty((T, self.v_size), dtype=torch.float32, device=proj.device)
        inv = self.position.inv_freq if self.position is not None else None
        ops.retention_scan(proj, 0, self.qk_size, 2 * self.qk_size, self.decays, inv,
                           ctx.positions, view.state, ctx.q_start, ctx.state_slots, o_raw, ctx.B,
                           self.heads, self.dk, self.dv, self.k_scale, ctx.err,
                           max_q=1 if ctx.decode_only else ctx.max_q_len,
                           silu=self.spec.activation == "silu")
        g_off = 2 * self.qk_size + self.v_size
        if self.plain_out:
            ops.retention_out(o_raw, proj, g_off, out, self.heads, self.dv, self.spec.norm_eps,
                              out_scale)
        else:
            ops.gated_norm_out(o_raw, proj, g_off, self.norm_w, out, self.heads, self.dv,
                               self.spec.norm_eps, over_all=self.spec.norm_over == "all",
                               gate=self.spec.gate, out_scale=out_scale)


register_mixer("retention", RetentionMixer)
