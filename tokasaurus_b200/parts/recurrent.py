"""A mixer that carries a matrix state per head instead of keys and values: a gated linear recurrence in the HGRN2
form, where the forget gate also decides what is written,

    S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T,        o_t = S_t^T q_t,
    q = silu(W_q h),   v = W_v h,   f = low + (1 - low) * sigmoid(W_f h + b_f),

followed by an RMS norm of every head's o_t over its ``vdim`` values (one weight vector shared by the heads) and
the output projection.  The state is float32, starts at zero and lives in the request's slot; gates, sums and the
norm are float32 whatever the engine's precision.  The three projections are one matrix product with a float32 result.
"""

from __future__ import annotations

import torch

from tokasaurus_b200.kernels import ops
from tokasaurus_b200.parts.base import Mixer, StateNeed, WeightSpec


class GatedLinearRecurrence(Mixer):
    graph_safe = True

    def __init__(self, width: int, n_heads: int, dim: int, vdim: int, norm_eps: float, q_name: str, f_name: str,
                 f_bias_name: str, lower_name: str, v_name: str, norm_name: str, o_name: str):
        self.width, self.n_heads, self.dim, self.vdim = width, n_heads, dim, vdim
        self.norm_eps = float(norm_eps)
        self.names = dict(q=q_name, f=f_name, f_bias=f_bias_name, lower=lower_name, v=v_name, norm=norm_name, o=o_name)
        ops.recurrence_defines(dim, vdim)  # refuses sizes the kernel does not take
        self.w_qfv: torch.Tensor | None = None
        self.w_o: torch.Tensor | None = None

    def weight_specs(self):
        n, H, d, v = self.names, self.n_heads, self.dim, self.vdim
        return (
            WeightSpec(n["q"], (H * d, self.width)), WeightSpec(n["f"], (H * d, self.width)),
            WeightSpec(n["v"], (H * v, self.width)), WeightSpec(n["o"], (self.width, H * v)),
            WeightSpec(n["f_bias"], (H * d,), role="vector"), WeightSpec(n["lower"], (H * d,), role="vector"),
            WeightSpec(n["norm"], (v,), role="vector"),
        )

    def kernel_modules(self, dtype):
        return (("recurrence.cu", ops.recurrence_defines(self.dim, self.vdim)),)

    def cache_need(self):
        return StateNeed((self.n_heads, self.vdim, self.dim), "float32")  # S transposed: [head][value][key channel]

    def bind(self, weights, rt) -> None:
        n = self.names
        self.w_qfv = torch.cat([weights[n["q"]], weights[n["f"]], weights[n["v"]]], dim=0).contiguous()
        self.w_o = weights[n["o"]].contiguous()
        self.f_bias = weights[n["f_bias"]].contiguous()
        self.lower = weights[n["lower"]].contiguous()
        self.norm_w = weights[n["norm"]].contiguous()

    def forward(self, ctx, h, cache, out_rows=None):
        qfv = ops.linear(h, self.w_qfv, out_dtype=torch.float32)
        o = torch.empty((h.shape[0], self.n_heads * self.vdim), dtype=h.dtype, device=h.device)
        ops.gated_recurrence(qfv, cache.state, self.f_bias, self.lower, self.norm_w, o, ctx.seq_slot, ctx.seq_q_start,
                             ctx.seq_q_len, ctx.n_seqs, self.n_heads, self.dim, self.vdim, self.norm_eps, cache.writable)
        if out_rows is not None:
            cut = torch.empty((out_rows.numel(), o.shape[1]), dtype=o.dtype, device=o.device)
            ops.gather_rows(o, out_rows, cut)
            o = cut
        return ops.linear(o, self.w_o)


class DecayedLinearAttention(Mixer):
    """Linear attention with one fixed decay a head:

        S_t = lambda_h S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t,   q, k, v = silu(W_q h), silu(W_k h), silu(W_v h),

    then an RMS norm over all heads' o_t together (one weight vector), a gate sigmoid(W_g h), and the output projection.
    The state (float32, S^T per head, zero at admission) lives in the request's slot; the four projections are one
    matrix product with a float32 result, the recurrence, the norm and the gate are float32.  The walk over the
    tokens is the kernel that the selective state space uses too (csrc/decay_recurrence.cu)."""

    graph_safe = True

    def __init__(self, width: int, n_heads: int, dim: int, vdim: int, decay, norm_eps: float, q_name: str, k_name: str,
                 v_name: str, g_name: str, norm_name: str, o_name: str):
        if len(decay) != n_heads:
            raise ValueError(f"{len(decay)} decays for {n_heads} heads")
        self.width, self.n_heads, self.dim, self.vdim = width, n_heads, dim, vdim
        self.decay = tuple(float(d) for d in decay)
        self.norm_eps = float(norm_eps)
        self.names = dict(q=q_name, k=k_name, v=v_name, g=g_name, norm=norm_name, o=o_name)
        self.defines = ops.decay_recurrence_defines(dim, vdim)  # refuses sizes the kernel does not take
        self.walk_builds = ops.decay_walk_modules(dim, vdim)

    def weight_specs(self):
        n, H, d, e = self.names, self.n_heads, self.dim, self.vdim
        return (WeightSpec(n["q"], (H * d, self.width)), WeightSpec(n["k"], (H * d, self.width)),
                WeightSpec(n["v"], (H * e, self.width)), WeightSpec(n["g"], (H * e, self.width)),
                WeightSpec(n["o"], (self.width, H * e)), WeightSpec(n["norm"], (H * e,), role="vector"))

    def kernel_modules(self, dtype):
        return tuple(("decay_recurrence.cu", d) for d in self.walk_builds) + (("post_norm.cu", None),)

    def cache_need(self):
        return StateNeed((self.n_heads * self.vdim * self.dim,), "float32")  # S^T: [head][value][key channel]

    def bind(self, weights, rt) -> None:
        n = self.names
        self.w_qkvg = torch.cat([weights[n["q"]], weights[n["k"]], weights[n["v"]], weights[n["g"]]], dim=0).contiguous()
        self.w_o = weights[n["o"]].contiguous()
        self.norm_w = weights[n["norm"]].contiguous()
        self.decay_t = torch.tensor(self.decay, dtype=torch.float64).to(torch.float32).to(rt.device)

    def forward(self, ctx, h, cache, out_rows=None):
        H, d, e = self.n_heads, self.dim, self.vdim
        T = h.shape[0]
        proj = ops.linear(h, self.w_qkvg, out_dtype=torch.float32)
        q, k = proj[:, :H * d], proj[:, H * d:2 * H * d]
        v, g = proj[:, 2 * H * d:2 * H * d + H * e], proj[:, 2 * H * d + H * e:]
        ops.silu_cols(proj, 2 * H * d + H * e, self.defines)  # q, k and v, in place
        raw = torch.empty((T, H * e), dtype=torch.float32, device=h.device)
        ops.decay_walk(q, k, v, 1, None, self.decay_t, None, cache.state, raw, ctx.seq_slot, ctx.seq_q_start,
                       ctx.seq_q_len, ctx.n_seqs, H, d, e, cache.writable)
        if out_rows is not None:
            raw, g = _rows(raw, out_rows), _rows(g.contiguous(), out_rows)
        o = torch.empty(raw.shape, dtype=h.dtype, device=h.device)
        ops.gated_group_norm(raw, g, self.norm_w, o, 1, self.norm_eps, gate_first=False)
        return ops.linear_out_f32(o, self.w_o, ctx.status)


class GatedLinearAttention(Mixer):
    """Linear attention whose state decays by a different, input-dependent factor in every key channel:

        S_t = diag(f_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T (q_t * q_scale),   f_t = sigmoid(A2 (A1 h_t) + b)^(1 / tau),

    with q, k = W_q h, W_k h (``dim`` a head), v = W_v h (``vdim`` a head) and the decays made by a low-rank product (the
    rank is A1's row count).  Every head's o_t is RMS-normed over its ``vdim`` values with one weight vector that the
    heads share, multiplied by silu(W_g h) and projected.  The state (float32, S^T per head, zero at admission) lives in
    the request's slot; the five projections are one matrix product with a float32 result; the second low-rank factor,
    the decays, the recurrence, the norm and the gate are float32.  The walk over the tokens is the kernel that decayed
    linear attention and the selective state space use (csrc/decay_recurrence.cu), in its build with a decay vector."""

    graph_safe = True

    def __init__(self, width: int, n_heads: int, dim: int, vdim: int, tau: float, norm_eps: float, q_name: str, k_name: str,
                 v_name: str, g_name: str, a1_name: str, a2_name: str, a2_bias_name: str, norm_name: str, o_name: str,
                 rank: int | None = None, q_scale: float | None = None):
        """``rank`` None: read from the shape of the tensor ``a1_name``.  ``q_scale`` None: dim^(-1/2)."""
        if not tau > 0:
            raise ValueError(f"tau must be positive, got {tau}")
        self.width, self.n_heads, self.dim, self.vdim = width, n_heads, dim, vdim
        self.tau, self.norm_eps, self.rank = float(tau), float(norm_eps), rank
        self.q_scale = float(dim) ** -0.5 if q_scale is None else float(q_scale)
        self.names = dict(q=q_name, k=k_name, v=v_name, g=g_name, a1=a1_name, a2=a2_name, a2_bias=a2_bias_name,
                          norm=norm_name, o=o_name)
        self.defines = ops.decay_recurrence_defines(dim, vdim)  # refuses sizes the kernel does not take
        self.walk_builds = ops.decay_walk_modules(dim, vdim)

    def weight_specs(self):
        n, H, d, e, r = self.names, self.n_heads, self.dim, self.vdim, self.rank if self.rank is not None else -1
        return (WeightSpec(n["q"], (H * d, self.width)), WeightSpec(n["k"], (H * d, self.width)),
                WeightSpec(n["v"], (H * e, self.width)), WeightSpec(n["g"], (H * e, self.width)),
                WeightSpec(n["a1"], (r, self.width)), WeightSpec(n["a2"], (H * d, r)),
                WeightSpec(n["a2_bias"], (H * d,), role="vector"), WeightSpec(n["norm"], (e,), role="vector"),
                WeightSpec(n["o"], (self.width, H * e)))

    def kernel_modules(self, dtype):
        return tuple(("decay_recurrence.cu", d) for d in self.walk_builds) + (("post_norm.cu", None),)

    def cache_need(self):
        return StateNeed((self.n_heads * self.vdim * self.dim,), "float32")  # S^T: [head][value][key channel]

    def bind(self, weights, rt) -> None:
        n = self.names
        a1, a2 = weights[n["a1"]], weights[n["a2"]]
        if a1.shape[0] != a2.shape[1]:
            raise ValueError(f"{n['a1']} has {a1.shape[0]} rows but {n['a2']} has {a2.shape[1]} columns")
        self.rank = int(a1.shape[0])
        self.w_in = torch.cat([weights[n["q"]], weights[n["k"]], weights[n["v"]], weights[n["g"]], a1], dim=0).contiguous()
        self.a2t = a2.float().t().contiguous()  # [rank, heads * dim]: the second factor is applied in float32
        self.a2_bias = weights[n["a2_bias"]].contiguous()
        self.w_o = weights[n["o"]].contiguous()
        self.norm_w = weights[n["norm"]].contiguous()

    def forward(self, ctx, h, cache, out_rows=None):
        H, d, e = self.n_heads, self.dim, self.vdim
        T = h.shape[0]
        proj = ops.linear(h, self.w_in, out_dtype=torch.float32)
        q, k = proj[:, :H * d], proj[:, H * d:2 * H * d]
        v, g = proj[:, 2 * H * d:2 * H * d + H * e], proj[:, 2 * H * d + H * e:2 * H * (d + e)]
        f = torch.empty((T, H * d), dtype=torch.float32, device=h.device)
        ops.gla_gates(proj, 2 * H * (d + e), self.rank, self.a2t, self.a2_bias, self.tau, f, 0, H * d, self.q_scale,
                      self.defines)
        raw = torch.empty((T, H * e), dtype=torch.float32, device=h.device)
        ops.decay_walk(q, k, v, 1, None, None, None, cache.state, raw, ctx.seq_slot, ctx.seq_q_start, ctx.seq_q_len,
                       ctx.n_seqs, H, d, e, cache.writable, decay_vec=f)
        if out_rows is not None:
            raw, g = _rows(raw, out_rows), _rows(g.contiguous(), out_rows)
        o = torch.empty(raw.shape, dtype=h.dtype, device=h.device)
        ops.gated_group_norm(raw, g, self.norm_w, o, H, self.norm_eps, gate_first=False, silu_gate=True)
        return ops.linear_out_f32(o, self.w_o, ctx.status)


class Retention(Mixer):
    """Linear attention with one fixed decay a head, rotated queries and keys, no softmax and no denominator:

        S_t = lambda_h S_(t-1) + (k_t * k_scale) v_t^T,   o_t = S_t^T q_t,

    q, k = W_q h, W_k h rotated by position on the first ``rotary.rotary_dim`` channels of a head (channel i paired with
    channel i + rotary_dim / 2; angles float64), k scaled AFTER the rotation; v = W_v h.  Every head's o_t is divided by
    its root mean square (no weight), multiplied by silu(W_g h) and projected.  State, products and float32 parts as
    in ``DecayedLinearAttention``, whose walk kernel this is."""

    graph_safe = True

    def __init__(self, width: int, n_heads: int, dim: int, vdim: int, decay, rotary, norm_eps: float, q_name: str,
                 k_name: str, v_name: str, g_name: str, o_name: str, k_scale: float | None = None,
                 rotary_pairs: bool = False):
        """``rotary``: a ``parts.rope.RotaryEncoding`` or None.  ``k_scale`` None: dim^(-1/2)."""
        if len(decay) != n_heads:
            raise ValueError(f"{len(decay)} decays for {n_heads} heads")
        if rotary is not None and rotary.rotary_dim > dim:
            raise ValueError(f"{rotary.rotary_dim} rotated channels in heads of {dim}")
        self.width, self.n_heads, self.dim, self.vdim = width, n_heads, dim, vdim
        self.decay = tuple(float(x) for x in decay)
        self.rotary, self.rotary_pairs = rotary, bool(rotary_pairs)
        self.norm_eps = float(norm_eps)
        self.k_scale = float(dim) ** -0.5 if k_scale is None else float(k_scale)
        self.names = dict(q=q_name, k=k_name, v=v_name, g=g_name, o=o_name)
        self.defines = ops.decay_recurrence_defines(dim, vdim)
        self.walk_builds = ops.decay_walk_modules(dim, vdim)

    def weight_specs(self):
        n, H, d, e = self.names, self.n_heads, self.dim, self.vdim
        return (WeightSpec(n["q"], (H * d, self.width)), WeightSpec(n["k"], (H * d, self.width)),
                WeightSpec(n["v"], (H * e, self.width)), WeightSpec(n["g"], (H * e, self.width)),
                WeightSpec(n["o"], (self.width, H * e)))

    def kernel_modules(self, dtype):
        return tuple(("decay_recurrence.cu", d) for d in self.walk_builds) + (("post_norm.cu", None),)

    def cache_need(self):
        return StateNeed((self.n_heads * self.vdim * self.dim,), "float32")  # S^T: [head][value][key channel]

    def bind(self, weights, rt) -> None:
        n = self.names
        self.w_qkvg = torch.cat([weights[n["q"]], weights[n["k"]], weights[n["v"]], weights[n["g"]]], dim=0).contiguous()
        self.w_o = weights[n["o"]].contiguous()
        self.decay_t = torch.tensor(self.decay, dtype=torch.float64).to(torch.float32).to(rt.device)
        rot = self.rotary.rotary_dim if self.rotary is not None else 0
        self.freq = (self.rotary.inv_freq64() if rot else torch.zeros(0, dtype=torch.float64)).to(rt.device)

    def forward(self, ctx, h, cache, out_rows=None):
        H, d, e = self.n_heads, self.dim, self.vdim
        T = h.shape[0]
        proj = ops.linear(h, self.w_qkvg, out_dtype=torch.float32)
        q, k = proj[:, :H * d], proj[:, H * d:2 * H * d]
        v, g = proj[:, 2 * H * d:2 * H * d + H * e], proj[:, 2 * H * d + H * e:]
        ops.rotate_scale(proj, 0, H * d, H, d, self.freq.numel() * 2, self.rotary_pairs, self.freq, ctx.positions,
                         ctx.token_seq, 1.0, self.k_scale, self.defines)
        raw = torch.empty((T, H * e), dtype=torch.float32, device=h.device)
        ops.decay_walk(q, k, v, 1, None, self.decay_t, None, cache.state, raw, ctx.seq_slot, ctx.seq_q_start,
                       ctx.seq_q_len, ctx.n_seqs, H, d, e, cache.writable)
        if out_rows is not None:
            raw, g = _rows(raw, out_rows), _rows(g.contiguous(), out_rows)
        o = torch.empty(raw.shape, dtype=h.dtype, device=h.device)
        ops.gated_group_norm(raw, g, None, o, H, self.norm_eps, gate_first=False, silu_gate=True)
        return ops.linear_out_f32(o, self.w_o, ctx.status)


def _rows(t: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    cut = torch.empty((rows.numel(), t.shape[1]), dtype=t.dtype, device=t.device)
    ops.gather_rows(t, rows, cut)
    return cut
