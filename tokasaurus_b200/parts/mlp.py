"""SiLU-gated feed-forward: ``down(silu(gate(h)) * up(h))`` without biases
(tokasaurus/model/llama.py:319-339; :329-332 are the three products and the activation).  The
gate and up matrices are stacked so that one matrix product makes gate|up."""

from __future__ import annotations

import torch

from tokasaurus_b200.kernels import ops
from tokasaurus_b200.parts.base import FeedForward, WeightSpec


class GatedMLP(FeedForward):
    """``activation`` "gelu_tanh": the gate goes through the tanh form of GELU instead of the SiLU (the products whose
    epilogue is the SiLU gate are then not used).  ``out_f32``: the update leaves as float32 rows or as the float32
    slices of a K-split product, for the residual sum."""

    def __init__(self, width: int, inner: int, gate_name: str, up_name: str, down_name: str, activation: str = "silu",
                 out_f32: bool = False):
        if activation not in ("silu", "gelu_tanh"):
            raise ValueError(f"the gate's activation is 'silu' or 'gelu_tanh', not {activation!r}")
        self.activation, self.out_f32 = activation, bool(out_f32)
        self.width = width
        self.inner = inner
        self.names = (gate_name, up_name, down_name)
        self.interleave = 0
        self.w_gate_up: torch.Tensor | None = None
        self.w_down: torch.Tensor | None = None

    def weight_specs(self):
        g, u, d = self.names
        return (
            WeightSpec(g, (self.inner, self.width)),
            WeightSpec(u, (self.inner, self.width)),
            WeightSpec(d, (self.width, self.inner)),
        )

    def bind(self, weights, rt) -> None:
        g, u, d = self.names
        # bfloat16: gate and up rows interleaved in groups of 8, the layout whose product the small-batch
        # kernel can turn into silu(gate) * up in its epilogue
        self.interleave = 8 if (rt.dtype == torch.bfloat16 and self.inner % 8 == 0) else 0
        if self.interleave:
            self.w_gate_up = ops.interleave_gate_up(weights[g], weights[u])
        else:
            self.w_gate_up = torch.cat([weights[g], weights[u]], dim=0).contiguous()
        self.w_down = weights[d].contiguous()

    def forward(self, ctx, h):
        """Returns the update [rows, width] in h's dtype, or as float32 slices [slices, rows, width]
        that the next norm adds (few rows, bfloat16)."""
        status = ctx.status if ctx is not None else None
        if self.activation != "silu":
            gu = ops.linear(h, self.w_gate_up)
            act = torch.empty((h.shape[0], self.inner), dtype=h.dtype, device=h.device)
            ops.silu_mul(gu, act, self.interleave, act=self.activation)
            return ops.linear_out_f32(act, self.w_down, status) if self.out_f32 else ops.linear(act, self.w_down)
        if self.interleave and ops.can_use_few_rows(h, self.w_gate_up) and self.w_gate_up.shape[0] % 16 == 0:
            act = ops.linear_few_rows_gated(h, self.w_gate_up, status)
            return ops.linear_few_rows(act, self.w_down, status)
        if self.interleave and h.shape[0] >= ops.TCGEN05_M_MIN and ops.can_use_tcgen05(h, self.w_gate_up):
            # many rows: the tcgen05 product with the SiLU gate in its epilogue (no activation pass over memory)
            act = ops.gemm_tcgen05(h, self.w_gate_up,
                                   status if status is not None else torch.zeros(1, dtype=torch.int32, device=h.device),
                                   gated=True)
        else:
            gu = ops.linear(h, self.w_gate_up)
            act = torch.empty((h.shape[0], self.inner), dtype=h.dtype, device=h.device)
            ops.silu_mul(gu, act, self.interleave)
        if ops.can_use_few_rows(act, self.w_down):
            return ops.linear_few_rows(act, self.w_down, status)
        return ops.linear(act, self.w_down)


class ClampedGLU(FeedForward):
    """``down(g * sigmoid(alpha * g) * (u + 1))`` with ``g = min(gate(h), limit)`` and ``u = clamp(up(h), -limit,
    limit)``; no biases.  The gate and up matrices are stacked into one product (in bfloat16 with their rows
    interleaved in groups of 8, the layout whose tcgen05 product applies the unit in its epilogue: steps of many rows
    have no activation pass over memory); the update leaves as float32 (a norm reads it)."""

    def __init__(self, width: int, inner: int, limit: float, gate_name: str, up_name: str, down_name: str,
                 alpha: float = 1.702):
        self.width, self.inner, self.limit, self.alpha = width, inner, float(limit), float(alpha)
        self.names = (gate_name, up_name, down_name)

    def weight_specs(self):
        g, u, d = self.names
        return (WeightSpec(g, (self.inner, self.width)), WeightSpec(u, (self.inner, self.width)),
                WeightSpec(d, (self.width, self.inner)))

    def kernel_modules(self, dtype):
        return (("post_norm.cu", None),) + ((("gemm_tcgen05.cu", None),) if dtype == "bfloat16" else ())

    def bind(self, weights, rt) -> None:
        g, u, d = self.names
        self.interleave = 8 if (rt.dtype == torch.bfloat16 and self.inner % 8 == 0) else 0
        if self.interleave:
            self.w_gate_up = ops.interleave_gate_up(weights[g], weights[u])
        else:
            self.w_gate_up = torch.cat([weights[g], weights[u]], dim=0).contiguous()
        self.w_down = weights[d].contiguous()

    def forward(self, ctx, h):
        if self.interleave and h.shape[0] >= ops.TCGEN05_M_MIN and ops.can_use_tcgen05(h, self.w_gate_up):
            status = ctx.status if ctx is not None else torch.zeros(1, dtype=torch.int32, device=h.device)
            act = ops.gemm_tcgen05_clamped(h, self.w_gate_up, status, self.limit, self.alpha)
        else:
            gu = ops.linear(h, self.w_gate_up)
            act = torch.empty((h.shape[0], self.inner), dtype=h.dtype, device=h.device)
            ops.clamped_glu(gu, act, self.limit, self.alpha, self.interleave)
        return ops.linear_out_f32(act, self.w_down, ctx.status if ctx is not None else None)


class PolyNormMLP(FeedForward):
    """``down(act(up(h)))`` with the PolyNorm activation ``act(z) = a N(z) + b N(z^2) + c N(z^3) + e``, where powers
    are taken element by element and N divides a token's vector of inner values by its root mean square
    (``x / sqrt(mean(x^2) + eps)``).  The four numbers are a tensor of the model.  The norms are float32: the up
    product's float32 result goes straight into the activation kernel."""

    def __init__(self, width: int, inner: int, eps: float, up_name: str, down_name: str, coef_name: str):
        self.width, self.inner, self.eps = width, inner, float(eps)
        self.names = (up_name, down_name, coef_name)

    def weight_specs(self):
        u, d, c = self.names
        return (WeightSpec(u, (self.inner, self.width)), WeightSpec(d, (self.width, self.inner)),
                WeightSpec(c, (4,), role="vector"))

    def kernel_modules(self, dtype):
        return (("norm_conv.cu", None),)

    def bind(self, weights, rt) -> None:
        u, d, c = self.names
        self.w_up = weights[u].contiguous()
        self.w_down = weights[d].contiguous()
        self.coef = weights[c].contiguous()

    def forward(self, ctx, h):
        z = ops.linear(h, self.w_up, out_dtype=torch.float32)
        act = torch.empty(z.shape, dtype=h.dtype, device=h.device)
        ops.polynorm(z, self.coef, self.eps, act)
        return ops.linear(act, self.w_down)


class RoutedExperts(FeedForward):
    """A mixture of small SiLU-gated feed-forwards: a router (logits in float32, with a bias) picks each token's
    ``top`` experts by the largest logits and weighs them by the softmax over the chosen logits; the output is the
    weighted sum of their outputs, plus a shared expert (any ``FeedForward``) that every token runs through.

    A step's (token, choice) pairs are ordered by expert on the device, and the experts' products run over that
    ordering with each block looking its expert up; nothing about the routing is read back to the host.

    ``scored`` = dict(correction=<tensor name or None>, groups, keep, scale): the other way of choosing.  Scores
    s = sigmoid(logits); the choice goes by s + correction (a learned vector that takes no part in the weights), among
    the experts of the best ``keep`` of ``groups`` equal groups of neighbours only (a group scores the sum of its two
    largest choice scores); the weights are the chosen experts' s over their sum, times ``scale``.
    ``expert="gelu"``: an expert is ``down(gelu(up h))`` with the exact GELU and no gate; ``expert_names(e)`` then gives
    (up, down).  ``out_dtype`` float32: the weighted sum leaves as float32 rows (for a norm that reads it).

    ``over_all`` = dict(scale): a third way of weighing: the choice is the plain one (largest logits), the weights are
    the chosen experts' shares of the softmax over ALL experts, times ``scale``, not renormalised.
    ``expert="clamped"`` with ``clamp`` = (limit, alpha): an expert is ``down(g * sigmoid(alpha g) * (u + 1))`` with
    g = min(gate(h), limit), u = clamp(up(h), -limit, limit).  ``shared_gate_name``: a vector [1, width]; the shared
    expert's output counts sigmoid(that vector . h) times, one number a token (float32)."""

    # (token, choice) pairs from which the gathered tcgen05 products are used (bfloat16).  Below, the few-rows kernel
    # fetches every chosen expert's weights once as well, but spends one multiply-add a row on every weight it
    # fetches.  Measured on B200, the whole part replayed from a graph, 16 experts of 1,024 x 2,048, two chosen:
    # 2 pairs 36 against 44 us, 8 pairs 62 against 64, 16 pairs 83 against 70, 48 pairs 117 against 80 (32 experts of
    # 1,024 x 4,096, four chosen: 8 pairs 117 against 118, 16 pairs 179 against 132, 96 pairs 366 against 219).
    TENSOR_CORE_PAIRS_MIN = 12

    def __init__(self, width: int, inner: int, n_experts: int, top: int, router_name: str, router_bias_name: str | None,
                 expert_names, shared: FeedForward | None = None, scored: dict | None = None, expert: str = "silu_gated",
                 out_dtype: torch.dtype | None = None, over_all: dict | None = None, clamp: tuple[float, float] | None = None,
                 shared_gate_name: str | None = None):
        """``expert_names(e)`` -> (gate, up, down) tensor names of expert e."""
        if not 0 < top <= n_experts:
            raise ValueError(f"top={top} of {n_experts} experts")
        if expert not in ("silu_gated", "gelu", "clamped"):
            raise ValueError(f"an expert is 'silu_gated', 'gelu' or 'clamped', not {expert!r}")
        if (expert == "clamped") != (clamp is not None) or (clamp is not None and not clamp[0] > 0):
            raise ValueError("a clamped expert has a positive limit and a factor, other experts neither")
        if over_all is not None and scored is not None:
            raise ValueError("the weights come from the softmax over all experts or from sigmoid scores, not both")
        if shared_gate_name is not None and shared is None:
            raise ValueError("a gate on the shared expert needs a shared expert")
        self.over_all = over_all
        self.clamp = (float(clamp[0]), float(clamp[1])) if clamp is not None else None
        self.shared_gate_name = shared_gate_name
        if scored is not None:
            g, keep = int(scored.get("groups", 1)), int(scored.get("keep", 1))
            if g <= 0 or n_experts % g or not 0 < keep <= g or top > keep * (n_experts // g):
                raise ValueError(f"{n_experts} experts in {g} groups of which {keep} are kept, {top} chosen")
        self.scored, self.gelu, self.out_dtype = scored, expert == "gelu", out_dtype
        self.width, self.inner, self.n_experts, self.top = width, inner, n_experts, top
        self.router_name, self.router_bias_name = router_name, router_bias_name
        self.expert_names = [tuple(expert_names(e)) for e in range(n_experts)]
        self.shared = shared

    def weight_specs(self):
        specs = [WeightSpec(self.router_name, (self.n_experts, self.width), role="vector")]
        if self.router_bias_name is not None:
            specs.append(WeightSpec(self.router_bias_name, (self.n_experts,), role="vector"))
        if self.scored is not None and self.scored.get("correction") is not None:
            specs.append(WeightSpec(self.scored["correction"], (self.n_experts,), role="vector"))
        for names in self.expert_names:
            specs += [WeightSpec(n, (self.inner, self.width)) for n in names[:-1]] + [WeightSpec(names[-1], (self.width, self.inner))]
        if self.shared is not None:
            specs += list(self.shared.weight_specs())
        if self.shared_gate_name is not None:
            specs.append(WeightSpec(self.shared_gate_name, (1, self.width), role="vector"))
        return tuple(specs)

    def kernel_modules(self, dtype):
        tc = (("gemm_tcgen05.cu", None),) if dtype == "bfloat16" else ()
        return (("moe.cu", None),) + tc + (tuple(self.shared.kernel_modules(dtype)) if self.shared is not None else ())

    def bind(self, weights, rt) -> None:
        self.router_w = weights[self.router_name].contiguous()
        # the shared expert's gate: a one-row product in float32, like the router's own
        self.shared_gate_w = (weights[self.shared_gate_name].float().view(1, self.width).contiguous()
                              if self.shared_gate_name is not None else None)
        self.router_b = weights[self.router_bias_name].contiguous() if self.router_bias_name is not None else None
        self.route_args = None
        if self.scored is not None:
            c = self.scored.get("correction")
            self.route_args = dict(correction=weights[c].contiguous() if c is not None else None,
                                   groups=int(self.scored.get("groups", 1)), keep=int(self.scored.get("keep", 1)),
                                   scale=float(self.scored.get("scale", 1.0)))
        # [E, 2 * inner, width]: each expert's gate rows, then its up rows ([E, inner, width]: the up rows of an
        # ungated expert);  [E, width, inner]
        self.w_gate_up = torch.stack([torch.cat([weights[n] for n in names[:-1]], dim=0) for names in self.expert_names]).contiguous()
        self.w_down = torch.stack([weights[names[-1]] for names in self.expert_names]).contiguous()
        # for steps of many rows in bfloat16: the same weights with every expert's gate and up rows interleaved in
        # groups of 8, the layout whose product the tcgen05 kernel turns into silu(gate) * up in its epilogue
        self.w_gate_up_tc = None
        # (sizes below one tile of the kernel's TMA boxes stay with the other kernels)
        if rt.dtype == torch.bfloat16 and self.inner % 8 == 0 and self.width % 8 == 0 and self.inner >= 64 and self.width >= 128:
            self.w_gate_up_tc = self.w_gate_up if self.gelu else torch.stack(
                [ops.interleave_gate_up(weights[g], weights[u]) for g, u, _ in self.expert_names]).contiguous()
        if self.shared is not None:
            self.shared.bind(weights, rt)

    def forward(self, ctx, h):
        T, dev = h.shape[0], h.device
        top, E = self.top, self.n_experts
        top_idx = torch.empty((T, top), dtype=torch.int32, device=dev)
        top_w = torch.empty((T, top), dtype=torch.float32, device=dev)
        # rows of padding tokens (a step graph's) choose nothing; a cut-down set of rows has none
        token_seq = ctx.token_seq if (ctx is not None and T == ctx.n_tokens) else None
        ops.moe_route(h, self.router_w, self.router_b, token_seq, top, top_idx, top_w, self.route_args,
                      over_all=self.over_all is not None, scale=float((self.over_all or {}).get("scale", 1.0)))
        shared_gate = None
        if self.shared_gate_name is not None:
            shared_gate = torch.empty((T,), dtype=torch.float32, device=dev)
            ops.moe_logits(h, self.shared_gate_w, shared_gate.view(T, 1))
        offsets = torch.empty((E + 1,), dtype=torch.int32, device=dev)
        place_of = torch.empty((T * top,), dtype=torch.int32, device=dev)
        shared = self.shared.forward(ctx, h) if self.shared is not None else None
        out = torch.empty((T, self.width), dtype=self.out_dtype or h.dtype, device=dev)
        if self.w_gate_up_tc is not None and T * top >= self.TENSOR_CORE_PAIRS_MIN:
            # many rows: the rows gathered expert by expert, every span on a 128-row tile boundary, and the two
            # products on the tcgen05 tensor cores, each row tile with its own expert's weights
            tile = 128
            n_tiles = (T * top) // tile + E
            order = torch.empty((n_tiles * tile,), dtype=torch.int32, device=dev)
            src_token = torch.empty((n_tiles * tile,), dtype=torch.int32, device=dev)
            tile_group = torch.empty((n_tiles,), dtype=torch.int32, device=dev)
            ops.moe_order(top_idx, E, offsets, order, place_of, pad=tile, tile_group=tile_group, src_token=src_token)
            rows = torch.empty((n_tiles * tile, self.width), dtype=h.dtype, device=dev)
            ops.moe_gather(h, src_token, rows)
            status = ctx.status if ctx is not None else torch.zeros(1, dtype=torch.int32, device=dev)
            act = ops.gemm_tcgen05_grouped(rows, self.w_gate_up_tc, tile_group, status, gated=not self.gelu, gelu=self.gelu,
                                           clamp=self.clamp)
            y = ops.gemm_tcgen05_grouped(act, self.w_down, tile_group, status)
            ops.moe_combine(y, place_of, top_w, shared, out, shared_gate)
            return out
        order = torch.empty((T * top,), dtype=torch.int32, device=dev)
        ops.moe_order(top_idx, E, offsets, order, place_of)
        act = torch.empty((T * top, self.inner), dtype=h.dtype, device=dev)
        ops.moe_gemm(h, self.w_gate_up, act, offsets, order, top, gated=not self.gelu, gelu=self.gelu, clamp=self.clamp)
        y = torch.empty((T * top, self.width), dtype=torch.float32, device=dev)
        ops.moe_gemm(act, self.w_down, y, offsets, None, top, gated=False)
        ops.moe_combine(y, place_of, top_w, shared, out, shared_gate)
        return out
