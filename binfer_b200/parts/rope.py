"""Rotary position encoding (rotate-half layout) as a part of the attention mixer.

``f_i = theta^(-2i/rot) / factor`` for ``i < rot/2``; a token at absolute
position ``p`` rotates the pair ``(i, i + rot/2)`` of each q and k head by the
angle ``p * f_i`` (src/engine/tp_context.ts:181-221;
cuda/kernels/bf16_kernels.cu:133-185).  The reference builds a cos/sin table for
4096 positions on the host and truncates it to bfloat16
(src/tensor/tensor.ts:136-145); here only the ``rot/2`` frequencies are kept, in
float32, and the kernel forms the angle and its sine and cosine in float32, so
no position limit and no table precision enter.  ``RopeSpec.wavelength_scaling``
stretches the long waves (``config.specs.WavelengthScaling``); ``RopeSpec.ramp_scaling``
stretches them by pair index and makes cosines and sines larger by ``magnitude``
(``config.specs.RampScaling``).  ``layout`` and ``offset`` say which sizes of a head make a
pair and where the rotated sizes start; the kernels that take them read them here.
"""
from __future__ import annotations

import math

import torch

from ..config.specs import RopeSpec
from .base import BuildEnv, PositionEncoding, register_position


class RotaryEncoding(PositionEncoding):
    """Holds ``inv_freq`` (float32 ``[rot/2]``) for the qkv post-processing kernel."""

    def __init__(self, spec: RopeSpec, head_dim: int, env: BuildEnv):
        rot = spec.rotary_dim or head_dim
        if rot % 2 or rot > head_dim:
            raise ValueError(f"rotary_dim {rot} must be even and at most head_dim {head_dim}")
        if spec.layout not in ("half", "interleaved"):
            raise ValueError(f"unknown rotary layout {spec.layout!r}")
        if spec.offset < 0 or spec.offset + rot > head_dim:
            raise ValueError("the rotated sizes must lie inside the head")
        self.rotary_dim = rot
        self.interleaved = spec.layout == "interleaved"
        self.offset = int(spec.offset)
        self.magnitude = 1.0
        i = torch.arange(rot // 2, dtype=torch.float64)
        inv = (float(spec.theta) ** (-2.0 * i / rot)) / float(spec.factor)
        ws = getattr(spec, "wavelength_scaling", None)
        if ws is not None:
            # by wavelength l = 2 pi / f: short waves stay, long ones are divided by the
            # factor, those between are mixed
            wave = 2.0 * math.pi / inv
            s = (float(ws.original) / wave - float(ws.low)) / (float(ws.high) - float(ws.low))
            mixed = (1.0 - s) * inv / float(ws.factor) + s * inv
            inv = torch.where(wave < float(ws.original) / float(ws.high), inv,
                              torch.where(wave > float(ws.original) / float(ws.low),
                                          inv / float(ws.factor), mixed))
        rs = getattr(spec, "ramp_scaling", None)
        if rs is not None:
            def index_of(turns: float) -> float:
                return rot * math.log(float(rs.original) / (2.0 * math.pi * turns)) / (
                    2.0 * math.log(float(spec.theta)))
            lo = max(math.floor(index_of(float(rs.fast))), 0)
            hi = min(math.ceil(index_of(float(rs.slow))), rot - 1)
            ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            inv = inv / float(rs.factor) * ramp + inv * (1.0 - ramp)
            self.magnitude = float(0.1 * math.log(float(rs.factor)) + 1.0
                                   if rs.magnitude is None else rs.magnitude)
        self.inv_freq = inv.to(torch.float32).to(env.device)


register_position("rope", RotaryEncoding)
