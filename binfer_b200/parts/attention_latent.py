"""Attention over a cached latent vector per token, as a mixer part.

A down projection of the mixer's input yields ``rank + dr`` numbers per token: the first
``rank``, RMS-normed with a weight, are the latent ``c``; the last ``dr``, rotated by the
token's position, are a key part that all heads share.  Head h's key is ``[W_uk,h c | shared
part]``, its value ``W_uv,h c``, its query ``[d plain | dr rotated]``; scores are scaled,
masked causally and pass an ordinary softmax; each head's output may be multiplied by the
sigmoid of one projected number per head; the output projection follows.

Only ``c`` and the shared key part are cached: one cache "head" of ``rank + dr`` numbers per
token and no values.  Keys and values are never expanded.  Because ``q_h . (W_uk,h c) =
(W_uk,h^T q_h) . c``, each query head's plain part is first carried into latent coordinates
(a product per head against ``W_uk,h^T``), the attention then runs with one shared key head
of ``rank + dr`` numbers whose first ``rank`` are also the value, and each head's result, a
mixture of latents, is expanded by ``W_uv,h`` afterwards.  That is one path for prompt
portions and single tokens alike, so the logits cannot depend on how a prompt was cut.

With ``q_rank`` the queries go through a latent of their own: the stacked product yields
``W_dq h`` in place of the queries, an RMS norm with a weight follows (float arithmetic), and
a second product ``W_uq`` gives the query heads.
"""
from __future__ import annotations

import dataclasses
import os
from typing import Callable, List, Optional

import torch

from ..cache.manager import KVNeed
from ..config.specs import LatentAttentionSpec
from ..csrc import ops
from ..weights.loader import ParamSpec
from .base import BuildEnv, EntryView, Mixer, StepContext, build_position, register_mixer
from .linear import linear, linear_heads

# BINFER_B200_LATENT_TENSOR_CORES=0: the one-warp-per-row kernel also in bfloat16 (the float32
# path), to tell the two apart when something differs
TENSOR_CORES = os.environ.get("BINFER_B200_LATENT_TENSOR_CORES", "1") != "0"


class LatentAttention(Mixer):
    def __init__(self, spec: LatentAttentionSpec, hidden_size: int, prefix: str, env: BuildEnv):
        s = spec
        if min(s.num_heads, s.head_dim, s.value_dim, s.kv_rank) <= 0 or s.rot_dim < 0:
            raise ValueError("latent attention: heads and sizes must be positive")
        if s.kv_rank + s.rot_dim > ops.GENERIC_MAX_HEAD_DIM or s.kv_rank > ops.GENERIC_MAX_VALUE_DIM:
            raise ValueError(f"latent attention: a latent of {s.kv_rank} with a rotated part of "
                             f"{s.rot_dim} is not supported (latent at most "
                             f"{ops.GENERIC_MAX_VALUE_DIM}, together at most "
                             f"{ops.GENERIC_MAX_HEAD_DIM})")
        self.spec, self.hidden, self.prefix, self.env = spec, hidden_size, prefix, env
        self.H, self.d, self.dr, self.dv, self.rank = (s.num_heads, s.head_dim, s.rot_dim,
                                                       s.value_dim, s.kv_rank)
        self.q_size = self.H * (self.d + self.dr)
        self.kv_size = self.rank + self.dr
        self.q_rank = int(getattr(s, "q_rank", 0) or 0)
        # rows of the stacked product in front: the queries, or their latent
        self.q_rows = self.q_rank if self.q_rank else self.q_size
        self.position = None
        if s.position is not None and self.dr:
            # the rotated sizes are a vector of their own: dr numbers, rotated from its start
            self.position = build_position(dataclasses.replace(s.position, offset=0), self.dr, env)
            if self.position.inv_freq is None:
                raise ValueError("latent attention takes rotary encodings only")
        self.names = dict(s.names)
        self.gate_off = self.q_rows + self.kv_size
        self.w_proj = self.w_ukT = self.w_uv = self.w_o = self.norm_w = None
        self.w_uq = self.q_norm_w = None

    # ----------------------------------------------------------------- weights
    def _spec(self, role: str) -> ParamSpec:
        n = self.prefix + self.names[role]
        shape = {"q": (self.q_size, self.hidden), "dkv": (self.kv_size, self.hidden),
                 "dkv_norm": (self.rank,), "uk": (self.H * self.d, self.rank),
                 "uv": (self.H * self.dv, self.rank), "g": (self.H, self.hidden),
                 "o": (self.hidden, self.H * self.dv), "dq": (self.q_rank, self.hidden),
                 "dq_norm": (self.q_rank,), "uq": (self.q_size, self.q_rank)}[role]
        if role in ("dkv_norm", "dq_norm"):
            return ParamSpec(n, shape, init="norm", role="vector")
        return ParamSpec(n, shape)

    def _roles(self) -> List[str]:
        q = ["dq", "dq_norm", "uq"] if self.q_rank else ["q"]
        return q + ["dkv", "dkv_norm", "uk", "uv"] + (["g"] if self.spec.head_gate else []) + ["o"]

    def param_specs(self) -> List[ParamSpec]:
        return [self._spec(r) for r in self._roles()]

    def load(self, get: Callable[[ParamSpec], torch.Tensor]) -> None:
        g = lambda role: get(self._spec(role))          # noqa: E731
        rows = [g("dq") if self.q_rank else g("q"), g("dkv")] + (
            [g("g")] if self.spec.head_gate else [])
        self.w_proj = torch.cat(rows, dim=0).contiguous()
        if self.q_rank:
            self.w_uq, self.q_norm_w = g("uq"), g("dq_norm")
        self.norm_w = g("dkv_norm")
        # per head: W_uk,h^T [rank, d] carries a query into latent coordinates; W_uv,h
        # [dv, rank] expands a mixture of latents into the head's value
        self.w_ukT = g("uk").view(self.H, self.d, self.rank).transpose(1, 2).contiguous()
        self.w_uv = g("uv").view(self.H, self.dv, self.rank).contiguous()
        self.w_o = g("o")

    # ------------------------------------------------------------------- cache
    def kv_need(self) -> Optional[KVNeed]:
        return KVNeed(1, self.kv_size, None, 0)      # one head per token, no values

    # ----------------------------------------------------------------- forward
    def forward(self, x: torch.Tensor, ctx: StepContext, view: EntryView) -> torch.Tensor:
        s, T, H = self.spec, x.shape[0], self.H
        if not view.writes_cache:
            raise ValueError("latent attention keeps a cache of its own")
        g = view.group
        proj = linear(x, self.w_proj)
        q_abs = torch.empty((T, H, self.kv_size), dtype=x.dtype, device=x.device)
        pos = self.position
        if self.q_rank:
            c_q = torch.empty((T, self.q_rank), dtype=x.dtype, device=x.device)
            ops.section_norm(proj, 0, self.q_rank, self.q_norm_w, s.norm_eps, c_q)
            q = linear(c_q, self.w_uq)
        else:
            q = proj[:, :self.q_size]
        ops.latent_encode(proj, 0, self.q_rows, self.norm_w, s.norm_eps,
                          pos.inv_freq if pos is not None else None,
                          bool(pos is not None and pos.interleaved),
                          pos.magnitude if pos is not None else 1.0, ctx.positions, ctx.slots[g],
                          q_abs, view.k_cache, H, self.d, self.dr, self.rank, ctx.err, q=q)
        q_heads = q.view(T, H, self.d + self.dr)
        linear_heads(q_heads[:, :, :self.d], self.w_ukT, q_abs[:, :, :self.rank])
        o_lat = torch.empty((T, H, self.rank), dtype=x.dtype, device=x.device)
        if (TENSOR_CORES and s.softmax_scale > 0
                and ops.latent_attention_takes(x.dtype, self.rank, self.dr)):
            # bfloat16: tiles of (token, head) rows against tiles of cache rows, each fetched
            # once as keys and values, on the tensor cores
            ops.latent_attention(q_abs, view.k_cache, ctx.q_start, ctx.positions,
                                 ctx.block_tables[g], o_lat, ctx.B,
                                 1 if ctx.decode_only else ctx.max_q_len, H, self.rank,
                                 s.softmax_scale, ctx.err, max_ctx=ctx.max_ctx_len)
        else:
            ops.paged_attention_generic(
                q_abs.view(T, H * self.kv_size), view.k_cache, view.k_cache, ctx.seq_of_token,
                ctx.positions, ctx.block_tables[g], o_lat.view(T, H * self.rank), H, 1,
                self.kv_size, None, s.softmax_scale, ctx.err, value_dim=self.rank,
                v_stride=self.kv_size)
        out = torch.empty((T, H, self.dv), dtype=x.dtype, device=x.device)
        linear_heads(o_lat, self.w_uv, out)
        out = out.view(T, H * self.dv)
        if s.head_gate:
            ops.head_gate_mul(out, proj[:, self.gate_off:self.gate_off + H], H, self.dv)
        return linear(out, self.w_o)


register_mixer("latent_attention", LatentAttention)
