"""RMSNorm over the residual stream, fused with the stream's pending add.

``y = x * rsqrt(mean(x^2) + eps) * w`` with the weight multiplying directly
(cuda/kernels/bf16_kernels.cu:40-84).  The reference runs the residual add and
the norm as two kernels (src/engine/batched_engine.ts:1164-1178); here the add
rides on the norm.
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch

from ..config.specs import NormSpec
from ..csrc import ops
from ..weights.loader import ParamSpec
from .base import BuildEnv, Norm, ResidualStream, register_norm


class RMSNorm(Norm):
    def __init__(self, spec: NormSpec, size: int, name: str, env: BuildEnv):
        self.eps = float(spec.eps)
        self.offset = float(getattr(spec, "offset", 0.0))
        self.size = size
        self.name = name
        self.env = env
        # a weight of one number for all coordinates: held as a vector of that number, so
        # that every kernel that takes a norm's weight takes this one too
        self.scalar = bool(getattr(spec, "scalar_weight", False))
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> List[ParamSpec]:
        init = "around_zero" if self.offset else "norm"
        return [ParamSpec(self.name, () if self.scalar else (self.size,), init=init,
                          role="vector")]

    def load(self, get: Callable[[ParamSpec], torch.Tensor]) -> None:
        self.weight = get(self.param_specs()[0])
        if self.scalar:
            self.weight = self.weight.reshape(1).expand(self.size).contiguous()
        if self.offset:
            # the weight that multiplies is offset + what the checkpoint holds, in float
            self.weight = (self.weight.float() + self.offset).contiguous()

    def forward(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None,
                n_rows: int = 0) -> torch.Tensor:
        """Normed activations of every row, or of ``rows`` only (the stream is then
        left as it is: nothing reads it afterwards).  May return ``ScaledRows`` when the
        stream holds this norm's output already (``ResidualStream.add_linear``)."""
        if rows is None and stream.ready_for is self:
            out, stream.ready, stream.ready_for = stream.ready, None, None
            return out           # ScaledRows: the product before already prepared this norm
        if stream.pending2 is not None:
            stream.flush()       # a pair of adds: this norm's kernel folds one only
        stream.ready = stream.ready_for = None
        n = n_rows if rows is not None else stream.x.shape[0]
        out = torch.empty((n, self.size), dtype=self.env.dtype, device=self.env.device)
        ops.add_rmsnorm(stream.x, stream.pending, self.weight, out, self.eps, rows=rows,
                        write_back=rows is None)
        if rows is None:
            stream.pending = None
        return out


    def add_normed(self, stream: ResidualStream, y: torch.Tensor) -> None:
        """``stream.x += y * rsqrt(mean(y^2) + eps) * w`` in one kernel, which also leaves the
        new stream in the activation type for the next sublayer's products."""
        stream.flush()
        stream.ready = stream.ready_for = None
        if y.dtype != self.env.dtype or y.shape != stream.x.shape:
            raise ValueError("add_normed: the sublayer's output must have the stream's shape "
                             "and the engine's activation type")
        reading = None
        if self.env.dtype != torch.float32:
            reading = torch.empty(stream.x.shape, dtype=self.env.dtype, device=self.env.device)
        ops.rmsnorm_add(stream.x, y, self.weight, reading, self.eps)
        stream.reading = reading

    def fused_scale(self):
        """(weight, eps): what a product needs to prepare this norm in its epilogue."""
        return self.weight, self.eps


register_norm("rmsnorm", RMSNorm)


class LayerNorm(Norm):
    takes_second_delta = True      # forward(..., also=): see ResidualStream.add_pair

    """``y = (x - mean) / sqrt(var + eps) * w + b`` with the variance the mean of the squared
    deviations; the bias tensor is the weight's name with ``NormSpec.bias_suffix`` (None: no
    bias).  Folds the stream's pending add, and a second one (``also``), into the same pass."""

    def __init__(self, spec: NormSpec, size: int, name: str, env: BuildEnv):
        self.eps = float(spec.eps)
        self.size, self.name, self.env = size, name, env
        self.bias_name = None if spec.bias_suffix is None else name + spec.bias_suffix
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def param_specs(self) -> List[ParamSpec]:
        specs = [ParamSpec(self.name, (self.size,), init="norm", role="vector")]
        if self.bias_name is not None:
            specs.append(ParamSpec(self.bias_name, (self.size,), init="around_zero",
                                   role="vector"))
        return specs

    def load(self, get: Callable[[ParamSpec], torch.Tensor]) -> None:
        specs = self.param_specs()
        self.weight = get(specs[0])
        self.bias = get(specs[1]) if len(specs) > 1 else None

    def forward(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None,
                n_rows: int = 0, also: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Normed activations of every row, or of ``rows`` only (the stream is then left as it
        is).  ``also``: one more sublayer output to add beside the pending one."""
        stream.ready = stream.ready_for = None
        n = n_rows if rows is not None else stream.x.shape[0]
        out = torch.empty((n, self.size), dtype=self.env.dtype, device=self.env.device)
        ops.add_layernorm(stream.x, stream.pending, also, self.weight, self.bias, out, self.eps,
                          rows=rows, write_back=rows is None)
        if rows is None:
            stream.pending = None
            stream.reading = None
        return out


register_norm("layernorm", LayerNorm)
