"""Grouped-query attention over a sliding window with a cap on the scores and a sink in the softmax.

q = W_q h + b_q, k = W_k h + b_k (``dim`` values a head), v = W_v h + b_v (``vdim`` values a head; the two sizes may
differ); optionally every q head and every k head is divided by its root mean square (an RMS norm without a weight);
no rotation.  With c the cap,

    s_ij = c * tanh(scale * q_i . k_j / c),      o_i = sum_j exp(s_ij) v_j / (exp(sink_h) + sum_j exp(s_ij))

over the last ``window`` positions (the query's own included; None: all).  The sink is a learned number per head that
takes part in the denominator only.  The output projection may carry a bias (``out_bias``), which the block adds.

A token's key and value of one key/value head are cached side by side as one row [k | v] (one plane): rows
``[page, kv head, slot, dim + vdim]``.  The projections are one product with a float32 result; biases, the unit norms,
scores, weights and sums are float32.  In float32, and for head sizes that are no multiples of 16, one FP32-pipe kernel
serves every token; in bfloat16 otherwise the tensor-core kernels of csrc/attention_sink.cu do (weights rounded to
bfloat16 for their product with the values, as in the framework's other attention kernels).

Options that other designs bring: a weight vector on the q and k norms (``qk_norm_names``); a rotation of q and k by
position on the first ``rotary.rotary_dim`` channels of a head, in neighbouring pairs or in halves (``rotary``,
``rotary_pairs``; after the norm); values that ARE the keys as projected, before norm and rotation
(``values_are_keys``: no W_v, vdim = dim); a learned factor on every head's scale and a learned number added to its
scores (``head_scale_name``, ``head_bias_name``); and ``weights="sigmoid"``: no softmax, the weight of a visible key
is sigmoid(score), not normalised over the keys (then there is no sink).

``keep_first``: with a window, a request's first so many positions stay visible to every later query (position i sees
j if j <= i and (i - j < window or j < keep_first)); their pages stay in the cache.  ``maps`` > 1: so many attention
maps a head, each with query and key vectors of its own (q and k hold them head by head, [map 0 | map 1 | ...]) and a
softmax of its own over the same values; the cached row is [k of map 0 | k of map 1 | ... | v].  What becomes of the
maps' outputs is a subclass's business (``_combine``; ``parts.diff_attention.DifferentialAttention``).  ``extra_names``:
further matrices over the mixer's input whose rows ride in the same product as q, k and v (an output gate's, say);
their float32 results are the trailing columns of the product that ``_combine`` is handed.
"""

from __future__ import annotations

import torch

from tokasaurus_b200.kernels import ops
from tokasaurus_b200.parts.base import Mixer, PagedCacheNeed, WeightSpec


class SinkAttention(Mixer):
    graph_safe = True

    def __init__(self, width: int, n_heads: int, n_kv_heads: int, dim: int, vdim: int, scale: float,
                 softcap: float | None, window: int | None, norm_eps: float, q_name: str, k_name: str, v_name: str,
                 o_name: str, sink_name: str | None, bias_names: tuple[str, str, str] | None = None,
                 out_bias_name: str | None = None, unit_norm: bool = True, qk_norm_names: tuple[str, str] | None = None,
                 rotary=None, rotary_pairs: bool = True, values_are_keys: bool = False,
                 head_scale_name: str | None = None, head_bias_name: str | None = None, weights: str = "softmax",
                 keep_first: int = 0, maps: int = 1, extra_names: tuple[tuple[str, int], ...] = ()):
        """``extra_names``: (tensor name, rows) of matrices [rows, width] appended to the q|k|v product."""
        if n_heads % n_kv_heads:
            raise ValueError(f"n_heads={n_heads} is not a multiple of n_kv_heads={n_kv_heads}")
        if weights not in ("softmax", "sigmoid"):
            raise ValueError(f"attention weights are 'softmax' or 'sigmoid', not {weights!r}")
        if weights == "sigmoid" and sink_name is not None:
            raise ValueError("sigmoid weights are not normalised: there is no sink")
        if values_are_keys and vdim != dim:
            raise ValueError(f"values that are the keys have the keys' size {dim}, not {vdim}")
        if qk_norm_names is not None and not unit_norm:
            raise ValueError("norm weights need the norm")
        if maps < 1 or (maps > 1 and (values_are_keys or type(self) is SinkAttention)):
            raise ValueError("several attention maps a head need a part that combines them, and values of their own")
        if keep_first < 0 or (keep_first and not window):
            raise ValueError("positions kept in sight need a window to be kept from")
        self.maps, self.keep_first, self.extra_names = int(maps), int(keep_first), tuple(extra_names)
        if rotary is not None and rotary.rotary_dim > dim:
            raise ValueError(f"{rotary.rotary_dim} rotated channels in heads of {dim}")
        self.sigmoid = weights == "sigmoid"
        self.qk_norm_names, self.rotary, self.rotary_pairs = qk_norm_names, rotary, bool(rotary_pairs)
        self.values_are_keys = bool(values_are_keys)
        self.head_scale_name, self.head_bias_name = head_scale_name, head_bias_name
        self.qk_norm_w = self.rot_freq = self.head_scale = self.head_bias = None
        self.width, self.n_heads, self.n_kv_heads, self.dim, self.vdim = width, n_heads, n_kv_heads, dim, vdim
        self.scale = float(scale)
        self.softcap = float(softcap) if softcap else None
        self.window = int(window) if window else None
        self.norm_eps, self.unit_norm = float(norm_eps), bool(unit_norm)
        self.names = (q_name, k_name, v_name, o_name)
        self.sink_name, self.bias_names, self.out_bias_name = sink_name, bias_names, out_bias_name
        self.defines = ops.sink_attention_defines(dim, vdim, self.sigmoid, self.maps)
        self.sinks = self.qkv_bias = self.out_bias = None

    def weight_specs(self):
        q, k, v, o = self.names
        H, G, d, e = self.n_heads, self.n_kv_heads, self.dim, self.vdim
        M = self.maps
        specs = [WeightSpec(q, (H * M * d, self.width)), WeightSpec(k, (G * M * d, self.width)), WeightSpec(o, (self.width, H * e))]
        specs += [WeightSpec(n, (rows, self.width)) for n, rows in self.extra_names]
        if not self.values_are_keys:
            specs.append(WeightSpec(v, (G * e, self.width)))
        if self.qk_norm_names is not None:
            specs += [WeightSpec(n, (d,), role="vector") for n in self.qk_norm_names]
        specs += [WeightSpec(n, (H * M,), role="vector") for n in (self.head_scale_name, self.head_bias_name) if n is not None]
        if self.bias_names is not None:
            specs += [WeightSpec(n, (rows,), role="vector")
                      for n, rows in zip(self.bias_names, (H * d, G * d) if self.values_are_keys else (H * M * d, G * M * d, G * e))]
        if self.out_bias_name is not None:
            specs.append(WeightSpec(self.out_bias_name, (self.width,), role="vector"))
        if self.sink_name is not None:
            specs.append(WeightSpec(self.sink_name, (H * M,), role="vector"))
        return tuple(specs)

    def kernel_modules(self, dtype):
        return (("attention_sink.cu", self.defines),)

    def cache_need(self):
        return PagedCacheNeed(self.n_kv_heads, self.maps * self.dim + self.vdim, self.window, planes=1,
                              keep_first=self.keep_first)

    def bind(self, weights, rt) -> None:
        q, k, v, o = self.names
        self.w_qkv = torch.cat([weights[q], weights[k]] + ([] if self.values_are_keys else [weights[v]])
                               + [weights[n] for n, _ in self.extra_names], dim=0).contiguous()
        # where the extra matrices' results start in a row of the product
        self.extra_off = self.w_qkv.shape[0] - sum(rows for _, rows in self.extra_names)
        self.w_o = weights[o].contiguous()
        if self.bias_names is not None:
            names = self.bias_names[:2] if self.values_are_keys else self.bias_names
            self.qkv_bias = torch.cat([weights[n].float() for n in names]).contiguous()
        if self.qk_norm_names is not None:
            self.qk_norm_w = torch.stack([weights[n].float() for n in self.qk_norm_names]).contiguous()
        if self.rotary is not None and self.rotary.rotary_dim > 0:
            self.rot_freq = self.rotary.inv_freq64().to(rt.device)
        if self.head_scale_name is not None:
            self.head_scale = weights[self.head_scale_name].contiguous()
        if self.head_bias_name is not None:
            self.head_bias = weights[self.head_bias_name].contiguous()
        if self.out_bias_name is not None:
            self.out_bias = weights[self.out_bias_name].contiguous()
        if self.sink_name is not None:
            self.sinks = weights[self.sink_name].contiguous()

    def _combine(self, ctx, attn, qkv, out_rows):
        """What goes into the output projection, from the attention's result ``attn`` ([rows, heads * maps * vdim]; with
        several maps float32) and the float32 product ``qkv`` of all tokens; ``out_rows`` names the tokens of attn's
        rows (None: all)."""
        return attn

    def forward(self, ctx, h, cache, out_rows=None):
        H, G, d, e, M = self.n_heads, self.n_kv_heads, self.dim, self.vdim, self.maps
        T = h.shape[0]
        tables = ctx.tables[cache.group]
        qkv = ops.linear(h, self.w_qkv, out_dtype=torch.float32)
        q = torch.empty((T, H * M * d), dtype=h.dtype, device=h.device)
        ops.sink_attn_prep(qkv, self.qkv_bias, self.unit_norm, self.norm_eps, q, cache.k, ctx.positions, ctx.token_seq,
                           tables.indptr, tables.page_ids, H, G, d, e, cache.page_size, cache.writable, ctx.status,
                           norm_w=self.qk_norm_w, rot_freq=self.rot_freq,
                           rot_dims=self.rotary.rotary_dim if self.rot_freq is not None else 0,
                           rot_pairs=self.rotary_pairs, values_are_keys=self.values_are_keys, sigmoid=self.sigmoid, maps=M)
        out_dtype = h.dtype if M == 1 else torch.float32  # several maps' outputs stay unrounded for what combines them
        if ops.can_use_attn_sink_tc(h.dtype, d, e, M):
            # bfloat16: every token on the tensor cores (single tokens and portions by a kernel each); wanted rows are
            # cut out afterwards
            attn = torch.empty((T, H * M * e), dtype=out_dtype, device=h.device)
            ops.attn_sink_tc(q, attn, cache.k, ctx.seq_q_start, ctx.seq_q_len, ctx.seq_kv_len, tables.indptr,
                             tables.page_ids, ctx.n_seqs, self.sinks, H, G, d, e, cache.page_size, self.scale, self.softcap,
                             self.window, ctx.status, portions=not ctx.single_token_step, head_scale=self.head_scale,
                             head_bias=self.head_bias, sigmoid=self.sigmoid, maps=M, keep_first=self.keep_first)
            if out_rows is not None:
                cut = torch.empty((out_rows.numel(), H * M * e), dtype=out_dtype, device=h.device)
                ops.gather_rows(attn, out_rows, cut)
                attn = cut
            return ops.linear_out_f32(self._combine(ctx, attn, qkv, out_rows), self.w_o, ctx.status)
        n_rows = T if out_rows is None else out_rows.numel()
        attn = torch.empty((n_rows, H * M * e), dtype=out_dtype, device=h.device)
        ops.attn_sink(q, attn, cache.k, ctx.token_seq, ctx.positions, tables.indptr, tables.page_ids, out_rows, n_rows,
                      self.sinks, H, G, d, e, cache.page_size, self.scale, self.softcap, self.window, ctx.status,
                      head_scale=self.head_scale, head_bias=self.head_bias, sigmoid=self.sigmoid, maps=M,
                      keep_first=self.keep_first)
        return ops.linear_out_f32(self._combine(ctx, attn, qkv, out_rows), self.w_o, ctx.status)
