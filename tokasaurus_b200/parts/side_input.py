"""A per-layer input that depends on the token alone, added to the residual stream:

    e = table[token][offset : offset + dim],   g = gelu_tanh(W_gate x) * e,   y = W_proj g,
    x <- x + y / sqrt(mean(y^2) + eps) * w

``table`` is a second embedding table that holds every layer's ``dim`` values of a token side by side (one tensor for
the model; each layer's part reads its own slice).  The two products are the engine's matrix products; the gate, the
table lookup and the product of the two are one kernel, the norm and the sum another (statistics and sum float32).  A
token's id is found as the embedding finds it (a decoding request's last sampled token never leaves the device).
"""

from __future__ import annotations

import torch

from tokasaurus_b200.kernels import ops
from tokasaurus_b200.parts.base import Part, ResidualStream, WeightSpec


class TokenSideInput(Part):
    def __init__(self, width: int, dim: int, vocab: int, table_name: str, table_width: int, offset: int, gate_name: str,
                 proj_name: str, norm_name: str, eps: float):
        if not 0 <= offset <= table_width - dim:
            raise ValueError(f"columns {offset} .. {offset + dim} lie outside a table of {table_width} columns")
        self.width, self.dim, self.vocab, self.table_width, self.offset = width, dim, vocab, table_width, offset
        self.names = dict(table=table_name, gate=gate_name, proj=proj_name, norm=norm_name)
        self.eps = float(eps)

    def weight_specs(self):
        n = self.names
        return (WeightSpec(n["table"], (self.vocab, self.table_width)), WeightSpec(n["gate"], (self.dim, self.width)),
                WeightSpec(n["proj"], (self.width, self.dim)), WeightSpec(n["norm"], (self.width,), role="vector"))

    def kernel_modules(self, dtype):
        return (("post_norm.cu", None),)

    def bind(self, weights, rt) -> None:
        n = self.names
        self.table = weights[n["table"]]
        self.w_gate = weights[n["gate"]].contiguous()
        self.w_proj = weights[n["proj"]].contiguous()
        self.norm_w = weights[n["norm"]].contiguous()
        self.dtype = rt.dtype

    def forward(self, ctx, stream: ResidualStream, h: torch.Tensor, rows=None) -> None:
        """``h``: the stream's rows in the activation type; ``rows``: the tokens these rows belong to (None: all, in
        order).  Adds to ``stream.x`` in place and leaves the new rows in ``stream.h``."""
        z = ops.linear(h, self.w_gate, out_dtype=torch.float32)
        g = torch.empty(z.shape, dtype=h.dtype, device=h.device)
        ops.gelu_gate_rows(z, self.table, self.offset, ctx.token_ids, ctx.token_seq, ctx.seq_slot, ctx.last_token, rows,
                           g, ctx.status)
        y = ops.linear(g, self.w_proj, out_dtype=torch.float32)
        h_new = None if self.dtype == torch.float32 else torch.empty(stream.x.shape, dtype=self.dtype, device=h.device)
        ops.scaled_norm_add(stream.x, y, self.norm_w, None, 1.0, self.eps, h_new)
        stream.h = h_new
