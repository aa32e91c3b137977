"""The gated delta rule (a matrix memory with a decay per token and head, written by the
delta rule) as a mixer part with per-request state.

Per value head, with a state ``S [dk, dv]`` that starts at zero for a new request::

    q, k, v = silu(conv(W_q h)), silu(conv(W_k h)), silu(conv(W_v h))
    q = q / |q| / sqrt(dk)      k = k / |k|          (per head; |x| = sqrt(sum x^2 + 1e-6))
    beta = sigmoid(W_b h)       g = exp(-exp(A_log) softplus(W_a h + dt_bias))
    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

and the mixer returns ``W_o (o / rms_head(o) * w_norm * silu(W_g h))``.  q and k have fewer
heads than v where the spec says so.  All projections are one product against the stacked
weight; the convolution's reach behind a step's first token (the projected values of the
request's last ``taps - 1`` tokens) and ``S`` are per-request state, float whatever the
engine's precision, in the cache manager's slots: ``[S | convolution rows]``.  So a prompt
can be cut anywhere and a request can share a step with others.
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch

from ..cache.manager import StateNeed
from ..config.specs import GatedDeltaRuleSpec
from ..csrc import ops
from ..weights.loader import ParamSpec
from .base import BuildEnv, EntryView, Mixer, StepContext, register_mixer
from .linear import linear


class GatedDeltaRule(Mixer):
    def __init__(self, spec: GatedDeltaRuleSpec, hidden_size: int, prefix: str, env: BuildEnv):
        s = spec
        if min(s.num_heads, s.num_qk_heads, s.qk_dim, s.v_dim) <= 0 or s.num_heads % s.num_qk_heads:
            raise ValueError("delta rule: num_heads must be a positive multiple of num_qk_heads")
        if s.qk_dim > ops.DELTA_MAX_QK_DIM:
            raise ValueError(f"delta rule: a key size of {s.qk_dim} is not supported "
                             f"(at most {ops.DELTA_MAX_QK_DIM})")
        if s.conv_taps > ops.CONV_MAX_TAPS:
            raise ValueError(f"delta rule: a convolution of {s.conv_taps} taps is not supported "
                             f"(at most {ops.CONV_MAX_TAPS})")
        self.spec, self.hidden, self.prefix, self.env = spec, hidden_size, prefix, env
        self.H, self.G, self.dk, self.dv = s.num_heads, s.num_qk_heads, s.qk_dim, s.v_dim
        self.qk_size, self.v_size = self.G * self.dk, self.H * self.dv
        self.channels = 2 * self.qk_size + self.v_size
        self.taps = max(0, int(s.conv_taps))
        self.names = dict(s.names)
        # rows of the stacked projection: q, k, v | output gate | beta's logits | the decay's
        self.g_off = self.channels
        self.b_off = self.g_off + self.v_size
        self.a_off = self.b_off + self.H
        self.memory = self.H * self.dk * self.dv
        self.w_in = self.w_o = self.conv_w = self.A_log = self.dt_bias = self.norm_w = None

    # ----------------------------------------------------------------- weights
    def _spec(self, role: str) -> ParamSpec:
        mats = {"q": (self.qk_size, self.hidden), "k": (self.qk_size, self.hidden),
                "v": (self.v_size, self.hidden), "g": (self.v_size, self.hidden),
                "b": (self.H, self.hidden), "a": (self.H, self.hidden),
                "o": (self.hidden, self.v_size)}
        if role in mats:
            return ParamSpec(self.prefix + self.names[role], mats[role])
        if role in ("A_log", "dt_bias"):
            return ParamSpec(self.prefix + self.names[role], (self.H,), init="around_zero",
                             role="vector")
        if role == "norm":
            return ParamSpec(self.prefix + self.names[role], (self.dv,), init="norm",
                             role="vector")
        src = role[:-5]                          # "q.conv" -> q
        return ParamSpec(self.prefix + self.names[src] + self.spec.conv_suffix,
                         (mats[src][0], self.taps), init="conv", role="vector")

    def _roles(self) -> List[str]:
        roles = ["q", "k", "v", "b", "a", "g", "o", "A_log", "dt_bias", "norm"]
        if self.taps:
            roles += ["q.conv", "k.conv", "v.conv"]
        return roles

    def param_specs(self) -> List[ParamSpec]:
        return [self._spec(r) for r in self._roles()]

    def load(self, get: Callable[[ParamSpec], torch.Tensor]) -> None:
        g = lambda role: get(self._spec(role))          # noqa: E731
        self.w_in = torch.cat([g("q"), g("k"), g("v"), g("g"), g("b"), g("a")], dim=0).contiguous()
        self.w_o = g("o")
        self.A_log, self.dt_bias, self.norm_w = g("A_log"), g("dt_bias"), g("norm")
        if self.taps:
            self.conv_w = torch.cat([g("q.conv"), g("k.conv"), g("v.conv")], dim=0).contiguous()

    # ------------------------------------------------------------------- state
    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.memory + max(0, self.taps - 1) * self.channels,), "float32")

    # ----------------------------------------------------------------- forward
    def forward(self, x: torch.Tensor, ctx: StepContext, view: EntryView) -> torch.Tensor:
        s, T = self.spec, x.shape[0]
        proj = linear(x, self.w_in)
        memory = view.state[:, :self.memory]
        conv_state = view.state[:, self.memory:] if self.taps > 1 else None
        qkv = torch.empty((T, self.channels), dtype=torch.float32, device=x.device)
        gates = torch.empty((T, 2, self.H), dtype=torch.float32, device=x.device)
        ops.delta_encode(proj, self.conv_w, self.taps, conv_state, ctx.state_slots,
                         ctx.seq_of_token, ctx.q_start, self.b_off, self.a_off, self.A_log,
                         self.dt_bias, qkv, gates, self.H, self.G, self.dk, self.dv, s.unit_eps,
                         self.dk ** -0.5, ctx.err)
        if self.taps > 1:
            ops.conv_state_shift(proj[:, :self.channels], conv_state, ctx.state_slots,
                                 ctx.q_start, ctx.B, self.taps)
        o_raw = torch.empty((T, self.v_size), dtype=torch.float32, device=x.device)
        ops.delta_scan(qkv, gates, memory, ctx.q_start, ctx.state_slots, o_raw, ctx.B, self.H,
                       self.G, self.dk, self.dv, ctx.err,
                       max_q=1 if ctx.decode_only else ctx.max_q_len)
        out = torch.empty((T, self.v_size), dtype=x.dtype, device=x.device)
        ops.gated_norm_out(o_raw, proj, self.g_off, self.norm_w, out, self.H, self.dv,
                           s.norm_eps, over_all=False, gate="silu")
        return linear(out, self.w_o)


register_mixer("gated_delta_rule", GatedDeltaRule)
