"""RMS norm: ``y = weight * x / sqrt(mean(x^2) + eps)`` with the statistics in float32
(tokasaurus/model/llama.py:44-51).  The kernel also folds in the residual add that precedes the
norm (llama.py:284 and :336 add, the next block's :230 / :325 normalises)."""

from __future__ import annotations

import torch

from tokasaurus_b200.kernels import ops
from tokasaurus_b200.parts.base import Norm, ResidualStream, WeightSpec


class RMSNorm(Norm):
    def __init__(self, width: int, eps: float, weight_name: str):
        self.width = width
        self.eps = float(eps)
        self.weight_name = weight_name
        self.weight: torch.Tensor | None = None
        self.out_dtype: torch.dtype | None = None

    def weight_specs(self):
        return (WeightSpec(self.weight_name, (self.width,), role="vector"),)

    def bind(self, weights, rt) -> None:
        self.weight = weights[self.weight_name]
        self.out_dtype = rt.dtype

    def _run(self, x: torch.Tensor, delta=None) -> torch.Tensor:
        out = torch.empty(x.shape, dtype=self.out_dtype, device=x.device)
        ops.add_rmsnorm(x, delta, self.weight, self.eps, out)
        return out

    def forward(self, ctx, stream: ResidualStream):
        out = self._run(stream.x, stream.delta)
        stream.delta = None
        return out


class GroupRMSNorm(Norm):
    """RMS norm in equal consecutive parts of a row: every part is divided by its own ``sqrt(mean(part^2) + eps)``, then
    the whole row is multiplied by one weight vector.  ``groups`` = 1 is the plain RMS norm.  Blocks that norm AFTER the
    residual sum (``parts.block.PostNormBlock``) hand their sum to the same kernel; ``forward`` serves an output head."""

    def __init__(self, width: int, eps: float, weight_name: str, groups: int = 1, optional: bool = False):
        """``optional``: checkpoints may lack the weight; ``weight`` is then None after ``bind`` and the norm's owner
        leaves the norm out."""
        self.optional = bool(optional)
        if groups <= 0 or width % groups:
            raise ValueError(f"a row of {width} values does not divide into {groups} equal parts")
        self.width, self.eps, self.weight_name, self.groups = width, float(eps), weight_name, int(groups)
        self.weight: torch.Tensor | None = None
        self.out_dtype: torch.dtype | None = None

    def weight_specs(self):
        return (WeightSpec(self.weight_name, (self.width,), role="vector", optional=self.optional),)

    def kernel_modules(self, dtype):
        return (("post_norm.cu", None),)

    def bind(self, weights, rt) -> None:
        self.weight = weights.get(self.weight_name) if self.optional else weights[self.weight_name]
        self.out_dtype = rt.dtype

    def apply_sum(self, x: torch.Tensor, y, alpha: float) -> torch.Tensor | None:
        """x = weight * N(alpha * x + y) in place on the float32 rows ``x``; returns the new rows in the activation type
        (None in a float32 engine: they are ``x`` itself)."""
        h = None if self.out_dtype == torch.float32 else torch.empty(x.shape, dtype=self.out_dtype, device=x.device)
        ops.sum_group_norm(x, y, alpha, self.weight, self.eps, self.groups, h)
        return h

    def forward(self, ctx, stream: ResidualStream):
        # (the stream ends here: norming it in place costs no copy)
        h = self.apply_sum(stream.x, stream.delta, 1.0)
        stream.delta = None
        return stream.x if h is None else h


class LayerNorm(Norm):
    """``y = (x - mean) / sqrt(var + eps) * weight + bias`` with ``var = mean((x - mean)^2)``, statistics in float32;
    the kernel folds the residual add in like ``RMSNorm``'s."""

    def __init__(self, width: int, eps: float, weight_name: str, bias_name: str):
        self.width = width
        self.eps = float(eps)
        self.weight_name = weight_name
        self.bias_name = bias_name
        self.weight: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None
        self.out_dtype: torch.dtype | None = None

    def weight_specs(self):
        return (WeightSpec(self.weight_name, (self.width,), role="vector"),
                WeightSpec(self.bias_name, (self.width,), role="vector"))

    def kernel_modules(self, dtype):
        return (("norm_conv.cu", None),)

    def bind(self, weights, rt) -> None:
        self.weight = weights[self.weight_name]
        self.bias = weights[self.bias_name]
        self.out_dtype = rt.dtype

    def forward(self, ctx, stream: ResidualStream):
        out = torch.empty(stream.x.shape, dtype=self.out_dtype, device=stream.x.device)
        ops.add_layernorm(stream.x, stream.delta, self.weight, self.bias, self.eps, out)
        stream.delta = None
        return out
