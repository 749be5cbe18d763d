"""Differential attention: two softmax attention maps a head over the same values, one subtracted from the other.

q and k hold two vectors a head ([map 0 | map 1]); each map is an attention of its own (``parts.sink_attention``: biases,
q and k norms with weights, a rotation on part of a vector, grouped key/value heads, a window that keeps a request's
first positions in sight).  With a_0 and a_1 the maps' outputs of a head,

    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff          (one number a layer; four learned vectors of ``dim`` values)
    o = a_0 - lambda a_1,    o <- o / sqrt(mean(o^2) + eps) * (1 - diff)     (over the head's vdim values, no weight)

and, optionally, head h's o is multiplied by sigmoid(W_g x)_h, a gate read from the mixer's own input, before the output
projection.  The maps' outputs reach the combining kernel in float32; lambda, the norm and the gate are float32.  The
gate's matrix rides in the q|k|v product.
"""

from __future__ import annotations

import torch

from tokasaurus_b200.kernels import ops
from tokasaurus_b200.parts.base import WeightSpec
from tokasaurus_b200.parts.sink_attention import SinkAttention


class DifferentialAttention(SinkAttention):
    def __init__(self, width: int, n_heads: int, n_kv_heads: int, dim: int, vdim: int, scale: float, diff: float,
                 window: int | None, keep_first: int, norm_eps: float, q_name: str, k_name: str, v_name: str, o_name: str,
                 lambda_names: tuple[str, str, str, str], gate_name: str | None = None,
                 bias_names: tuple[str, str, str] | None = None, qk_norm_names: tuple[str, str] | None = None,
                 rotary=None, rotary_pairs: bool = False):
        """``lambda_names``: the tensors lq1, lk1, lq2, lk2 ([dim] each).  ``gate_name``: the output gate's matrix
        [heads, width] or None."""
        super().__init__(width, n_heads, n_kv_heads, dim, vdim, scale, None, window, norm_eps, q_name, k_name, v_name,
                         o_name, None, bias_names=bias_names, unit_norm=qk_norm_names is not None,
                         qk_norm_names=qk_norm_names, rotary=rotary, rotary_pairs=rotary_pairs,
                         keep_first=keep_first if window else 0, maps=2,
                         extra_names=((gate_name, n_heads),) if gate_name is not None else ())
        self.diff = float(diff)
        self.lambda_names = tuple(lambda_names)
        self.gated = gate_name is not None
        self.lam: torch.Tensor | None = None

    def weight_specs(self):
        return tuple(super().weight_specs()) + tuple(WeightSpec(n, (self.dim,), role="vector") for n in self.lambda_names)

    def bind(self, weights, rt) -> None:
        super().bind(weights, rt)
        lq1, lk1, lq2, lk2 = (weights[n].float() for n in self.lambda_names)
        self.lam = (torch.exp((lq1 * lk1).sum()) - torch.exp((lq2 * lk2).sum()) + self.diff).reshape(1).contiguous()

    def _combine(self, ctx, attn, qkv, out_rows):
        out = torch.empty((attn.shape[0], self.n_heads * self.vdim), dtype=self.w_o.dtype, device=attn.device)
        ops.diff_combine(attn, self.lam, self.norm_eps, 1.0 - self.diff, qkv if self.gated else None, self.extra_off,
                         out_rows, out, self.n_heads, self.dim, self.vdim)
        return out
