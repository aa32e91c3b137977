"""Mixture of gated feed-forward experts, with an optional shared expert.

A token's router logits ``z = W_router h`` are taken in float; the ``top`` experts with the
largest logits run, weighted by the softmax over those logits alone; the shared expert runs
for every token, times ``sigmoid(w_sg . h)`` when it has a gate.  Expert: ``W_down
(silu(W_gate h) * (W_up h))``.

How it runs here: the gate and up projections of all experts (and the shared one) are one
stacked weight, so one product gives every expert's pre-activations; a kernel applies the
activation and multiplies each expert's block by the token's weight for it (zero when not
chosen); one product with the down projections laid side by side then sums the weighted
experts in its own accumulation.  Unchosen experts cost arithmetic but no extra pass over
memory, no token is moved, and a token's result does not depend on what else is in the
batch.

The router has a second way of scoring (``MoESpec.scoring`` "softmax_all"): scores are the
softmax over all of the router's outputs; a correction per output (a tensor) is added for the
choice only; the outputs may form groups of which only the best can be chosen from; the
chosen scores are divided by their sum and multiplied by a factor.  The router's last
``identity`` outputs stand for experts that return their input: they have no tensors, the
router adds their weights up in one column, and a small kernel adds input times that column
to the result.

A step of very few tokens in bfloat16 (a request that decodes alone) would read every expert
for nothing; there the chosen experts' rows alone are read, a warp per output row
(``ops.moe_sparse``).  The float32 engine keeps the one path, so that its sums have one order.
"""
from __future__ import annotations

import os
from typing import Callable, List

import torch

from ..config.specs import MoESpec
from ..csrc import ops
from ..weights.loader import ParamSpec
from .base import BuildEnv, FeedForward, StepContext, register_ffn
from .linear import linear


# BINFER_B200_MOE_SPARSE=0: every step computes every expert
SPARSE = os.environ.get("BINFER_B200_MOE_SPARSE", "1") != "0"


class MoEFeedForward(FeedForward):
    def __init__(self, spec: MoESpec, hidden_size: int, prefix: str, env: BuildEnv):
        if spec.activation != "silu":
            raise ValueError(f"activation {spec.activation!r} is not supported (supported: 'silu')")
        self.identity = int(getattr(spec, "identity", 0) or 0)
        if not 1 <= spec.top <= spec.num_experts + self.identity:
            raise ValueError("moe: top must be between 1 and the number of router outputs")
        if spec.scoring not in ("softmax_top", "softmax_all"):
            raise ValueError(f"moe: unknown scoring {spec.scoring!r}")
        if spec.scoring == "softmax_top" and (self.identity or spec.groups > 1
                                              or spec.correction):
            raise ValueError("moe: corrections, groups and identity outputs go with the "
                             "softmax over all outputs")
        n = spec.num_experts + self.identity
        if (spec.groups < 1 or n % spec.groups or not 1 <= spec.groups_keep <= spec.groups
                or spec.top > spec.groups_keep * (n // spec.groups)):
            raise ValueError("moe: the groups must divide the router's outputs and the kept "
                             "ones hold the choices")
        self.spec, self.hidden, self.prefix, self.env = spec, hidden_size, prefix, env
        self.E, self.top, self.ff, self.ff_sh = (spec.num_experts, spec.top, spec.expert_size,
                                                 spec.shared_size)
        self.F = self.E * self.ff + self.ff_sh
        self.gated_shared = bool(spec.shared_gate and self.ff_sh)
        # columns of a token's row of weights: the experts, the shared expert's gate, the sum
        # of the chosen identity outputs
        self.cols = self.E + (1 if self.gated_shared else 0) + (1 if self.identity else 0)
        self.id_col = self.cols - 1 if self.identity else -1
        self.w_gate_up = self.w_down = self.w_router = self.correction = None

    def _expert_specs(self, p: str, ff: int) -> List[ParamSpec]:
        gate, up, down = self.spec.names
        return [ParamSpec(p + gate, (ff, self.hidden)), ParamSpec(p + up, (ff, self.hidden)),
                ParamSpec(p + down, (self.hidden, ff))]

    def _groups(self) -> List[List[ParamSpec]]:
        s = self.spec
        groups = [self._expert_specs(self.prefix + s.expert_prefix.format(e=e), self.ff)
                  for e in range(self.E)]
        if self.ff_sh:
            groups.append(self._expert_specs(self.prefix + s.shared_prefix, self.ff_sh))
        return groups

    def _router_specs(self) -> List[ParamSpec]:
        s = self.spec
        specs = [ParamSpec(self.prefix + s.router_name, (self.E + self.identity, self.hidden),
                           init="router", role="vector")]
        if self.gated_shared:
            specs.append(ParamSpec(self.prefix + s.shared_prefix + s.shared_gate_name,
                                   (1, self.hidden), role="vector"))
        return specs

    def _correction_spec(self) -> ParamSpec:
        return ParamSpec(self.prefix + self.spec.correction_name, (self.E + self.identity,),
                         init="around_zero", role="vector")

    def param_specs(self) -> List[ParamSpec]:
        return ([x for g in self._groups() for x in g] + self._router_specs()
                + ([self._correction_spec()] if self.spec.correction else []))

    def load(self, get: Callable[[ParamSpec], torch.Tensor]) -> None:
        groups = self._groups()
        self.w_gate_up = torch.cat([get(g[0]) for g in groups] + [get(g[1]) for g in groups],
                                   dim=0).contiguous()
        self.w_down = torch.cat([get(g[2]) for g in groups], dim=1).contiguous()
        # the router (and the shared expert's gate as one more row) in float
        self.w_router = torch.cat([get(s) for s in self._router_specs()], dim=0).contiguous()
        if self.spec.correction:
            self.correction = get(self._correction_spec())

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        T, s = x.shape[0], self.spec
        route_w = torch.empty((T, self.cols), dtype=torch.float32, device=x.device)
        top_ids = torch.empty((T, self.top), dtype=torch.int32, device=x.device)
        top_w = torch.empty((T, self.top), dtype=torch.float32, device=x.device)
        ops.moe_route(x, self.w_router, self.E, self.top, self.gated_shared, route_w, top_ids,
                      top_w, scoring=s.scoring, correction=self.correction, groups=s.groups,
                      groups_keep=s.groups_keep, identity=self.identity,
                      route_scale=s.route_scale, weight_eps=s.weight_eps)
        if (SPARSE and x.dtype == torch.bfloat16 and 2 * T * self.top <= self.E
                and ops.moe_sparse_takes(self.hidden, self.ff, self.ff_sh, self.top)):
            # so few tokens that most experts are chosen by none: read the chosen ones alone
            out = torch.empty((T, self.hidden), dtype=x.dtype, device=x.device)
            ops.moe_sparse(x, self.w_gate_up, self.w_down, top_ids, top_w, route_w, out, self.E,
                           self.ff, self.ff_sh, self.top, shared_gate=self.gated_shared,
                           identity_col=self.id_col)
            return out
        gu = linear(x, self.w_gate_up)
        act = torch.empty((T, self.F), dtype=x.dtype, device=x.device)
        ops.moe_act(gu, route_w, act, self.E, self.ff, shared_gate=self.gated_shared)
        out = linear(act, self.w_down)
        if self.identity:
            ops.moe_identity_add(out, x, route_w, self.id_col)
        return out


register_ffn("moe", MoEFeedForward)
