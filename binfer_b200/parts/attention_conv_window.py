"""Softmax attention whose projections pass a short convolution, with a window that keeps
the request's first tokens, as a mixer part.

Order of operations: one product for q, k and v; a causal convolution over time on every
channel of the three (the projected values of a request's last ``taps - 1`` tokens are
per-request state, so a prompt can be cut anywhere); optionally an RMS norm with weights over
the whole q projection and the whole k projection, all heads at once; rotation of q and k;
optionally each q and k head divided by its root mean square, after the rotation; k and v
into the pages; scores with an optional soft cap; attention in
which position i sees j <= i with ``i - j < window`` or ``j < keep_first`` (kept tokens stay
at their true positions) and whose softmax has a learned logit per head in its denominator;
the output projection.  Every key, also those of the step's own tokens, is read from the
pages, so portions can share a step with decoded tokens.

Three more things a spec may ask for: a weight behind the heads' norm (``dim`` numbers for q
and for k that the heads share: an RMS norm with a weight per head); a learned factor per
head on the scores, which is carried by the queries (the kernel that norms the heads
multiplies head h's query by it, in float); and a bias per head that grows with the logarithm
of the distance, ``b1_h ln(1 + b2_h (i - j))``, taken off the scaled score inside the attention
kernels.

The mixer can run alone (``forward``) or as a branch of ``ParallelMixers``, which stacks the
branches' input and output projections into one product each: ``w_in`` / ``w_out`` and
``run(proj, ctx, view, out, out_scale)`` are that interface.
"""
from __future__ import annotations

import os
from typing import Callable, List, Optional

import torch

from ..cache.manager import KVNeed, StateNeed
from ..config.specs import ConvWindowAttentionSpec
from ..csrc import ops
from ..weights.loader import ParamSpec
from .base import BuildEnv, EntryView, Mixer, StepContext, build_position, register_mixer
from .linear import linear

# BINFER_B200_CWA_TENSOR_CORES=0: the one-warp-per-row kernel also in bfloat16 (the float32
# engine always runs it: its sums have one fixed order per position)
TENSOR_CORES = os.environ.get("BINFER_B200_CWA_TENSOR_CORES", "1") != "0"
# BINFER_B200_CWA_DECODE_KERNEL=0: steps of single tokens, and steps of long prompt portions
# alone, on the tiled kernel too
DECODE_KERNEL = os.environ.get("BINFER_B200_CWA_DECODE_KERNEL", "1") != "0"
# the longest portion of a step from which the engine's prefill kernel (blocks of 256 rows a
# head) is taken instead of the tiled kernel
PREFILL_KERNEL_ROWS = 256


class ConvWindowAttention(Mixer):
    def __init__(self, spec: ConvWindowAttentionSpec, hidden_size: int, prefix: str,
                 env: BuildEnv):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if spec.head_dim > 256 or spec.value_dim > 256:
            raise ValueError(f"head sizes {spec.head_dim}, {spec.value_dim} are not supported "
                             f"(at most 256)")
        if spec.conv_taps > ops.CONV_MAX_TAPS:
            raise ValueError(f"a convolution of {spec.conv_taps} taps is not supported "
                             f"(at most {ops.CONV_MAX_TAPS})")
        self.spec, self.hidden, self.prefix, self.env = spec, hidden_size, prefix, env
        self.H, self.G, self.dk, self.dv = (spec.num_heads, spec.num_kv_heads, spec.head_dim,
                                            spec.value_dim)
        self.q_size, self.k_size, self.v_size = self.H * self.dk, self.G * self.dk, self.G * self.dv
        self.channels = self.q_size + self.k_size + self.v_size
        self.taps = max(0, int(spec.conv_taps))     # one tap: a factor per channel, no state
        self.position = (build_position(spec.position, self.dk, env)
                         if spec.position is not None else None)
        if self.position is not None and (self.position.inv_freq is None
                                          or getattr(self.position, "interleaved", False)
                                          or getattr(self.position, "offset", 0)):
            raise ValueError("this attention takes rotary encodings over the first sizes of a "
                             "head, in halves, only")
        if spec.proj_norm and self.taps:
            raise ValueError("a norm over the whole projection goes without a convolution")
        if spec.head_norm_weight and not spec.unit_norm:
            raise ValueError("a weight behind the heads' norm needs that norm (unit_norm)")
        if spec.head_norm_weight and spec.proj_norm:
            raise ValueError("the norm over the whole projection and the weighted norm of the "
                             "heads share their tensors' names: one of them only")
        self.names = dict(spec.names)
        self.in_rows, self.out_cols = self.channels, self.H * self.dv
        self.w_in = self.w_out = self.conv_w = self.sinks = self.proj_norm_w = None
        self.head_w = self.temp = self.bias_slope = self.bias_rate = None

    # ----------------------------------------------------------------- weights
    def _spec(self, role: str) -> ParamSpec:
        base = {"q": (self.q_size, self.hidden), "k": (self.k_size, self.hidden),
                "v": (self.v_size, self.hidden), "o": (self.hidden, self.H * self.dv)}
        if role in base:
            return ParamSpec(self.prefix + self.names[role], base[role])
        if role == "sink":
            return ParamSpec(self.prefix + self.names["sink"], (self.H,), init="around_zero",
                             role="vector")
        if role in ("q_head_norm", "k_head_norm"):
            return ParamSpec(self.prefix + self.names[role], (self.dk,), init="norm",
                             role="vector")
        if role == "temp":
            return ParamSpec(self.prefix + self.names[role], (self.H,), init="norm", role="vector")
        if role in ("bias_slope", "bias_rate"):
            return ParamSpec(self.prefix + self.names[role], (self.H,), init="rate", role="vector")
        if role in ("q_norm", "k_norm"):
            return ParamSpec(self.prefix + self.names[role],
                             (self.q_size if role == "q_norm" else self.k_size,), init="norm",
                             role="vector")
        src = role[:-5]                          # "q.conv" -> q
        return ParamSpec(self.prefix + self.names[src] + self.spec.conv_suffix,
                         (base[src][0], self.taps), init="conv", role="vector")

    def _roles(self) -> List[str]:
        roles = ["q", "k", "v", "o"]
        if self.taps:
            roles += ["q.conv", "k.conv", "v.conv"]
        if self.spec.sinks:
            roles.append("sink")
        if self.spec.proj_norm:
            roles += ["q_norm", "k_norm"]
        if self.spec.head_norm_weight:
            roles += ["q_head_norm", "k_head_norm"]
        if self.spec.head_temperature:
            roles.append("temp")
        if self.spec.log_distance_bias:
            roles += ["bias_slope", "bias_rate"]
        return roles

    def param_specs(self) -> List[ParamSpec]:
        return [self._spec(r) for r in self._roles()]

    def load(self, get: Callable[[ParamSpec], torch.Tensor]) -> None:
        g = lambda role: get(self._spec(role))          # noqa: E731
        self.w_in = torch.cat([g("q"), g("k"), g("v")], dim=0).contiguous()
        self.w_out = g("o")
        if self.taps:
            self.conv_w = torch.cat([g("q.conv"), g("k.conv"), g("v.conv")], dim=0).contiguous()
        if self.spec.sinks:
            self.sinks = g("sink")
        if self.spec.proj_norm:
            self.proj_norm_w = torch.cat([g("q_norm"), g("k_norm")]).contiguous()
        if self.spec.head_norm_weight:
            self.head_w = torch.stack([g("q_head_norm"), g("k_head_norm")]).contiguous()
        if self.spec.head_temperature:
            self.temp = g("temp")
        if self.spec.log_distance_bias:
            self.bias_slope, self.bias_rate = g("bias_slope"), g("bias_rate")

    # ------------------------------------------------------------ cache, state
    def kv_need(self) -> Optional[KVNeed]:
        s = self.spec
        return KVNeed(self.G, self.dk, s.window, None if self.dv == self.dk else self.dv,
                      keep_first=s.keep_first if s.window is not None else 0)

    def state_need(self) -> Optional[StateNeed]:
        if self.taps <= 1:
            return None
        return StateNeed(((self.taps - 1) * self.channels,), "float32")

    # ----------------------------------------------------------------- forward
    def forward(self, x: torch.Tensor, ctx: StepContext, view: EntryView) -> torch.Tensor:
        out = torch.empty((x.shape[0], self.out_cols), dtype=x.dtype, device=x.device)
        self.run(linear(x, self.w_in), ctx, view, out, 1.0)
        return linear(out, self.w_out)

    def run(self, proj: torch.Tensor, ctx: StepContext, view: EntryView, out: torch.Tensor,
            out_scale: float) -> None:
        """From the projections ``proj [T, channels]`` to the heads' outputs times
        ``out_scale`` in ``out [T, heads * value_dim]`` (both may be column blocks)."""
        s, T, g = self.spec, proj.shape[0], view.group
        if not view.writes_cache:
            raise ValueError("this attention keeps a cache of its own")
        q = torch.empty((T, self.q_size), dtype=proj.dtype, device=proj.device)
        inv = self.position.inv_freq if self.position is not None else None
        state = view.state if self.taps > 1 else None
        factors = None
        if s.proj_norm:
            factors = torch.empty((T, 2), dtype=torch.float32, device=proj.device)
            ops.section_rms(proj, 0, self.q_size, self.q_size, self.k_size, s.norm_eps, factors)
        ops.conv_encode(proj, self.conv_w, self.taps, state, ctx.state_slots, ctx.seq_of_token,
                        ctx.q_start, inv, ctx.positions, ctx.slots[g], q, view.k_cache,
                        view.v_cache, self.H, self.G, self.dk, self.dv, s.unit_norm, s.norm_eps,
                        ctx.err, pre_factor=factors, pre_weight=self.proj_norm_w,
                        rot_magnitude=getattr(self.position, "magnitude", 1.0),
                        head_weight=self.head_w, q_head_scale=self.temp)
        if self.taps > 1:
            ops.conv_state_shift(proj, state, ctx.state_slots, ctx.q_start, ctx.B, self.taps)
        keep = s.keep_first if s.window is not None else 0
        biased = self.bias_slope is not None      # (the engine's decode and prefill kernels take none)
        if (DECODE_KERNEL and not biased and ctx.decode_only and s.window is None and self.sinks is None
                and s.softmax_scale > 0 and out.stride(0) % 4 == 0 and out.data_ptr() % 8 == 0
                and ops.decode_attention_takes_capped(q, view.k_cache, self.H, self.G, self.dk,
                                                      self.dv, T)):
            # bfloat16 steps of single tokens, no window and no sinks: the engine's decode
            # kernel (resident CTAs, tiles by TMA), which takes the soft cap and writes the
            # scaled result into the branch's columns
            ops.decode_attention(q, view.k_cache, view.v_cache, None, T, ctx.seq_of_token,
                                 ctx.positions, ctx.block_tables[g], out, self.H, self.G,
                                 self.dk, None, s.softmax_scale, ctx.max_ctx_len, ctx.err,
                                 variant="persistent", softcap=s.softcap, out_scale=out_scale)
            return
        if (DECODE_KERNEL and not biased and not ctx.decode_only and ctx.n_decode == 0 and ctx.n_prefill
                and ctx.max_prefill_rows >= PREFILL_KERNEL_ROWS and s.window is None
                and self.sinks is None and s.softmax_scale > 0 and out.stride(0) % 8 == 0
                and out.data_ptr() % 16 == 0
                and ops.prefill_attention_takes_capped(q, view.k_cache, self.dk, self.dv)):
            # bfloat16 steps of prompt portions alone, heads of 128: the engine's tcgen05
            # prefill kernel, which takes the soft cap and writes into the branch's columns
            ops.prefill_attention(q, view.k_cache, view.v_cache, ctx.prefill_items,
                                  ctx.n_prefill, ctx.max_prefill_rows, ctx.block_tables[g], out,
                                  self.H, self.G, self.dk, None, s.softmax_scale, ctx.err,
                                  variant="umma2", max_ctx=ctx.max_ctx_len, softcap=s.softcap,
                                  out_scale=out_scale)
            return
        if (TENSOR_CORES and s.softmax_scale > 0
                and ops.pwm_attention_takes(proj.dtype, self.H, self.G, self.dk, self.dv)):
            # bfloat16: tiles of (token, head of a group) rows on the tensor cores, prompt
            # portions and single tokens alike (the windowed kernel, without pooled blocks)
            ops.pwm_attention(q, view.k_cache, view.v_cache, None, None, ctx.q_start,
                              ctx.positions, ctx.block_tables[g], None, None, None, False, out,
                              ctx.B, 1 if ctx.decode_only else ctx.max_q_len, self.H, self.G,
                              self.dk, self.dv, s.window, 0, s.softmax_scale, None, ctx.err,
                              max_ctx=ctx.max_ctx_len, sinks=self.sinks, keep_first=keep,
                              out_scale=out_scale, softcap=s.softcap, log_slope=self.bias_slope,
                              log_rate=self.bias_rate)
            return
        ops.paged_attention_generic(
            q, view.k_cache, view.v_cache, ctx.seq_of_token, ctx.positions, ctx.block_tables[g],
            out, self.H, self.G, self.dk, s.window, s.softmax_scale, ctx.err, sinks=self.sinks,
            value_dim=self.dv, keep_first=keep, out_scale=out_scale, softcap=s.softcap,
            log_slope=self.bias_slope, log_rate=self.bias_rate)


register_mixer("conv_window_attention", ConvWindowAttention)
