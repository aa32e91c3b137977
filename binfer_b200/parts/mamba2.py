"""A selective state space layer with a scalar decay per head and token (Mamba-2, in the
form its authors call state space duality) as a mixer part with per-request state.

One product gives ``[z | x | B | C | dt]``.  x, B and C pass a causal convolution per channel
(with a bias) and ``silu``; per head h, which reads B and C of group ``h // (heads / groups)``,
with a state ``S [N, P]`` that starts at zero for a new request::

    dt = softplus(dt + dt_bias_h)
    S <- exp(-exp(A_log_h) dt) S + dt B x^T        y = S^T C + D_h x

and the mixer returns ``W_o (norm_parts(y * silu(z)) * w_norm)``: the gate first, then an RMS
norm over each of ``norm_groups`` equal parts of the concatenated heads.

The recurrence is the engine's linear scan (the one retention runs) with ``q = C``, ``k = B``,
``v = dt x`` and a decay per token and head; what enters it is float whatever the engine's
precision.  ``S`` and the convolution's reach behind a step's first token (the projected
values of the request's last ``taps - 1`` tokens) are per-request state, float, in the cache
manager's slots: ``[S | convolution rows]``.  So a prompt can be cut anywhere and a request
can share a step with others.
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch

from ..cache.manager import StateNeed
from ..config.specs import Mamba2Spec
from ..csrc import ops
from ..weights.loader import ParamSpec
from .base import BuildEnv, EntryView, Mixer, StepContext, register_mixer
from .linear import linear


class Mamba2(Mixer):
    def __init__(self, spec: Mamba2Spec, hidden_size: int, prefix: str, env: BuildEnv):
        s = spec
        if min(s.num_heads, s.head_dim, s.state_dim, s.groups, s.norm_groups) <= 0 \
                or s.num_heads % s.groups:
            raise ValueError("mamba2: sizes must be positive, heads a multiple of groups")
        if (s.num_heads * s.head_dim) % s.norm_groups:
            raise ValueError("mamba2: norm_groups must divide heads * head_dim")
        if s.state_dim > ops.RETENTION_MAX_QK_DIM:
            raise ValueError(f"mamba2: a state of {s.state_dim} is not supported (at most "
                             f"{ops.RETENTION_MAX_QK_DIM})")
        if s.conv_taps > ops.CONV_MAX_TAPS:
            raise ValueError(f"mamba2: a convolution of {s.conv_taps} taps is not supported "
                             f"(at most {ops.CONV_MAX_TAPS})")
        self.spec, self.hidden, self.prefix, self.env = spec, hidden_size, prefix, env
        self.H, self.P, self.N, self.G = s.num_heads, s.head_dim, s.state_dim, s.groups
        self.inner = self.H * self.P
        self.channels = self.inner + 2 * self.G * self.N
        self.taps = max(0, int(s.conv_taps))
        self.names = dict(s.names)
        # rows of the input projection: z | x, B, C (the convolved channels) | dt
        self.xbc_off = self.inner
        self.dt_off = self.inner + self.channels
        self.in_rows = self.dt_off + self.H
        self.memory = self.H * self.N * self.P
        self.w_in = self.w_o = self.conv_w = self.conv_b = None
        self.A_log = self.dt_bias = self.D = self.norm_w = None

    # ----------------------------------------------------------------- weights
    def _spec(self, role: str) -> ParamSpec:
        n = self.prefix + self.names[role]
        if role == "in":
            return ParamSpec(n, (self.in_rows, self.hidden))
        if role == "o":
            return ParamSpec(n, (self.hidden, self.inner))
        if role == "conv":
            return ParamSpec(n, (self.channels, self.taps), init="conv", role="vector")
        if role == "conv_bias":
            return ParamSpec(n, (self.channels,), init="around_zero", role="vector")
        if role == "norm":
            return ParamSpec(n, (self.inner,), init="norm", role="vector")
        if role == "A_log":
            return ParamSpec(n, (self.H,), init="log_rate", role="vector")
        if role == "D":
            return ParamSpec(n, (self.H,), init="norm", role="vector")
        return ParamSpec(n, (self.H,), init="around_zero", role="vector")      # dt_bias

    def _roles(self) -> List[str]:
        roles = ["in"]
        if self.taps:
            roles.append("conv")
            if self.spec.conv_bias:
                roles.append("conv_bias")
        return roles + ["dt_bias", "A_log", "D", "norm", "o"]

    def param_specs(self) -> List[ParamSpec]:
        return [self._spec(r) for r in self._roles()]

    def load(self, get: Callable[[ParamSpec], torch.Tensor]) -> None:
        g = lambda role: get(self._spec(role))          # noqa: E731
        self.w_in, self.w_o = g("in"), g("o")
        self.A_log, self.dt_bias, self.D, self.norm_w = g("A_log"), g("dt_bias"), g("D"), g("norm")
        if self.taps:
            self.conv_w = g("conv")
            if self.spec.conv_bias:
                self.conv_b = g("conv_bias")

    # ------------------------------------------------------------------- state
    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.memory + max(0, self.taps - 1) * self.channels,), "float32")

    # ----------------------------------------------------------------- forward
    def forward(self, x: torch.Tensor, ctx: StepContext, view: EntryView) -> torch.Tensor:
        s, T, dev = self.spec, x.shape[0], x.device
        proj = linear(x, self.w_in)
        memory = view.state[:, :self.memory]
        conv_state = view.state[:, self.memory:] if self.taps > 1 else None
        qk = torch.empty((T, 2, self.G, self.N), dtype=torch.float32, device=dev)
        vf = torch.empty((T, self.H, self.P), dtype=torch.float32, device=dev)
        skip = torch.empty((T, self.inner), dtype=torch.float32, device=dev)
        decay = torch.empty((T, self.H), dtype=torch.float32, device=dev)
        ops.mamba2_encode(proj, self.xbc_off, self.dt_off, self.conv_w, self.conv_b, self.taps,
                          conv_state, ctx.state_slots, ctx.seq_of_token, ctx.q_start, self.A_log,
                          self.dt_bias, self.D, qk, vf, skip, decay, self.H, self.G, self.N,
                          self.P, ctx.err)
        if self.taps > 1:
            ops.conv_state_shift(proj[:, self.xbc_off:self.dt_off], conv_state, ctx.state_slots,
                                 ctx.q_start, ctx.B, self.taps)
        o_raw = torch.empty((T, self.inner), dtype=torch.float32, device=dev)
        ops.linear_scan(qk, vf, decay, memory, ctx.q_start, ctx.state_slots, o_raw, ctx.B, self.H,
                        self.G, self.N, self.P, ctx.err,
                        max_q=1 if ctx.decode_only else ctx.max_q_len)
        out = torch.empty((T, self.inner), dtype=x.dtype, device=dev)
        ops.gate_norm_out(o_raw, skip, proj, 0, self.norm_w, out, s.norm_groups, s.norm_eps)
        return linear(out, self.w_o)


register_mixer("mamba2", Mamba2)
