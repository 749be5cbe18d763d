"""Attention whose keys and values are made from a small per-token latent ("latent attention").

Per token the mixer makes  c = rmsnorm(W_dkv h)[:rank] * w  and one rotated key part  k_rot = rotate(W_dkv h)[rank:]
shared by all heads; only this row [c | k_rot] is cached (one plane, one "head" of rank + rot values a token).
A head's key is [W_uk c | k_rot], its value W_uv c; queries come through a latent of their own,
q = W_uq rmsnorm(W_dq h), laid out head by head as [dim plain | rot rotated].  The score is
(q_plain . k_plain + q_rot . k_rot) * scale over the last ``window`` positions (all if None), softmax, W_o.

The engine never expands keys or values: with  q_abs = W_uk^T q_plain  the score is  q_abs . c + q_rot . k_rot  and
the weighted sum of values is  W_uv (sum_j p_j c_j), so the attention kernel reads the cached rows as they are, the
same rows for every head.  The rotation pairs dimension 2i with 2i + 1 (interleaved) on the first ``rot_dims``
values of the rotated part.  A mixer with ``own_kv=False`` has no W_dkv and reads the rows another layer call wrote
(the model's run order gives it that call's cache entry).

Options that other designs bring: queries projected straight from the mixer's input (``q_rank=None``: q = W_q h, tensor
``names["q"]``, no query latent and no norm of one); a rotation given as a ``parts.rope.RotaryEncoding`` (``rotary``: its
frequencies, plain or yarn-blended, in float64 with angles, sines and cosines made in float64, its factor on sine and
cosine, its size the rotated share) in halves (``rotary_pairs=False``: channel i with channel i + dims / 2) or pairs; an
output gate (``names["g"]``: head h's output times sigmoid(W_g h)_h, the gate's matrix riding in the down-projection's
product); ``out_f32``: the output projection leaves float32 rows (or the float32 slices of a K-split product) for the
residual sum.
"""

from __future__ import annotations

import torch

from tokasaurus_b200.kernels import ops
from tokasaurus_b200.parts.attention import QUERY_TILE, AttentionPlanning, decode_block_slots
from tokasaurus_b200.parts.base import Mixer, PagedCacheNeed, WeightSpec

TENSOR_CORE_ROW_MAX = 256  # the widest cached row the mma.sync attention kernels are built for


class LatentAttention(AttentionPlanning, Mixer):
    """In bfloat16, when the cached row (rank + rot values) is a multiple of 16 values and at most 256, the attention
    runs on the framework's tensor-core kernels for grouped queries: the rows are at once the keys (all rank + rot
    values) and the values (the kernel's output beyond the first rank values is not used) of ONE key/value head that
    every query head reads, single tokens through the split-key kernel and portions through the tiled one, planned
    on the host like ``PagedAttention``'s.  Otherwise (float32, other sizes, only some rows wanted) the FP32-pipe
    kernel of csrc/latent_attention.cu serves every token."""

    graph_safe = True

    def __init__(self, width: int, n_heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, q_rank: int,
                 scale: float, rot_base: float, rot_dims: int, norm_eps: float, window: int | None, names: dict,
                 own_kv: bool = True, cache_window: int | None | str = "same", rotary=None, rotary_pairs: bool = True,
                 out_f32: bool = False):
        """``names``: tensors dq, dq_norm, uq, dkv, dkv_norm (both unused without ``own_kv``), uk, uv, o.
        ``cache_window``: how many of the latest rows the cache entry must keep (None: all); by default this mixer's
        own ``window``.  Mixers that read one entry with different windows all name the widest one here, so that the
        entry has one need and no page comes back while a reader can still see it."""
        if rotary is not None:
            rot_base, rot_dims = rotary.theta, rotary.rotary_dim
        if rot_dims > rot_dim or rot_dims % 2:
            raise ValueError(f"rot_dims={rot_dims} must be even and at most rot_dim={rot_dim}")
        self.rotary, self.halves, self.out_f32 = rotary, not rotary_pairs, bool(out_f32)
        self.gated = "g" in names and names["g"] is not None
        if q_rank is None and not own_kv:
            raise ValueError("a mixer without a query latent makes its own cached rows")
        self.freq64, self.mag = None, 1.0
        self.width, self.n_heads, self.dim, self.rot_dim, self.vdim = width, n_heads, dim, rot_dim, vdim
        self.kv_rank, self.q_rank = kv_rank, q_rank
        self.scale, self.rot_base, self.rot_dims = float(scale), float(rot_base), int(rot_dims)
        self.norm_eps = float(norm_eps)
        self.window = window
        self.cache_window = window if cache_window == "same" else cache_window
        if self.cache_window is not None and (window is None or window > self.cache_window):
            raise ValueError(f"a window of {window} rows cannot be read from a cache entry that keeps {self.cache_window}")
        self.names = dict(names)
        self.own_kv = own_kv
        # what the planning of the tensor-core kernels reads
        self.n_kv_heads = 1
        self.head_dim = kv_rank + rot_dim
        self.block_slots = decode_block_slots(self.head_dim) if self._rows_fit_tensor_cores() else 0
        self.sm_count = 0
        self.dtype = None

    def _rows_fit_tensor_cores(self) -> bool:
        return self.head_dim % 16 == 0 and self.head_dim <= TENSOR_CORE_ROW_MAX

    def _query_tile(self) -> int:
        return QUERY_TILE

    def plan_key(self):
        if self.dtype != torch.bfloat16 or not self._rows_fit_tensor_cores():
            return None
        return super().plan_key()

    def weight_specs(self):
        n, H = self.names, self.n_heads
        specs = [
            WeightSpec(n["uk"], (H * self.dim, self.kv_rank)), WeightSpec(n["uv"], (H * self.vdim, self.kv_rank)),
            WeightSpec(n["o"], (self.width, H * self.vdim)),
        ]
        if self.q_rank is None:
            specs.append(WeightSpec(n["q"], (H * (self.dim + self.rot_dim), self.width)))
        else:
            specs += [WeightSpec(n["dq"], (self.q_rank, self.width)), WeightSpec(n["dq_norm"], (self.q_rank,), role="vector"),
                      WeightSpec(n["uq"], (H * (self.dim + self.rot_dim), self.q_rank))]
        if self.gated:
            specs.append(WeightSpec(n["g"], (H, self.width)))
        if self.own_kv:
            specs += [WeightSpec(n["dkv"], (self.kv_rank + self.rot_dim, self.width)),
                      WeightSpec(n["dkv_norm"], (self.kv_rank,), role="vector")]
        return tuple(specs)

    def kernel_modules(self, dtype):
        mods = [("latent_attention.cu", {"TKB_LAT_RANK": self.kv_rank})]
        if dtype == "bfloat16" and self._rows_fit_tensor_cores():
            mods.append(("attention_mma.cu", {"TKB_HD": self.head_dim}))
        return tuple(mods)

    def cache_need(self):
        return PagedCacheNeed(1, self.kv_rank + self.rot_dim, self.cache_window, planes=1)

    def bind(self, weights, rt) -> None:
        n, H = self.names, self.n_heads
        down = ([weights[n["dq"]]] if self.q_rank is not None else []) + ([weights[n["dkv"]]] if self.own_kv else [])
        self.kv_off = self.q_rank or 0
        self.gate_off = sum(w.shape[0] for w in down)  # the gate's logits follow the latents in the product's rows
        if self.gated:
            down.append(weights[n["g"]])
        self.w_down = torch.cat(down, dim=0).contiguous()
        self.dq_norm = weights[n["dq_norm"]].contiguous() if self.q_rank is not None else None
        self.dkv_norm = weights[n["dkv_norm"]].contiguous() if self.own_kv else None
        self.w_uq = weights[n["uq" if self.q_rank is not None else "q"]].contiguous()
        if self.rotary is not None:
            self.freq64 = self.rotary.inv_freq64().to(rt.device)
            self.mag = float(self.rotary.magnitude())
        # per head: W_uk[h] is [dim, rank], so q_plain[h] @ W_uk[h] folds the key up-projection into the query;
        # the FP32 product wants its second operand as [N, K] = [rank, dim]
        self.w_uk = weights[n["uk"]].view(H, self.dim, self.kv_rank).contiguous()
        self.w_uk_t = self.w_uk.transpose(1, 2).contiguous() if rt.dtype == torch.float32 else None
        self.w_uv = weights[n["uv"]].view(H, self.vdim, self.kv_rank).contiguous()
        self.w_o = weights[n["o"]].contiguous()
        i = torch.arange(self.rot_dims // 2, dtype=torch.float64)
        self.inv_freq = (self.rot_base ** (-2.0 * i / max(self.rot_dims, 1))).to(torch.float32).to(rt.device)
        self.dtype = rt.dtype
        limits = getattr(rt, "limits", None)
        if self._rows_fit_tensor_cores():
            self.block_slots = decode_block_slots(self.head_dim, limits)
        from tokasaurus_b200.kernels.device import NO_DEVICE

        self.sm_count = (limits or NO_DEVICE).sm_count

    def forward(self, ctx, h, cache, out_rows=None):
        T, H, R, rd, dim = h.shape[0], self.n_heads, self.kv_rank, self.rot_dim, self.dim
        tables = ctx.tables[cache.group]
        proj = ops.linear(h, self.w_down, out_dtype=torch.float32)  # [T, (q_rank) (+ rank + rot) (+ heads)]
        q_rank = self.q_rank or 0
        cq = torch.empty((T, q_rank), dtype=h.dtype, device=h.device) if q_rank else None
        write = self.own_kv and cache.writable
        rot_args = dict(freq64=self.freq64, halves=self.halves, mag=self.mag)
        ops.latent_prep(proj, 0, q_rank, self.dq_norm, cq, self.kv_off if write else -1, R, rd, self.rot_dims,
                        self.dkv_norm, self.inv_freq, cache.k if write else None, ctx.positions, ctx.token_seq,
                        tables.indptr, tables.page_ids, cache.page_size, self.norm_eps, ctx.status, h.dtype, **rot_args)
        q = ops.linear(cq if q_rank else h, self.w_uq)  # [T, H * (dim + rot)]
        q3 = q.view(T, H, dim + rd)
        plan = ctx.plans.get(self.plan_key()) if (out_rows is None and self.plan_key() is not None) else None
        if plan is not None:
            return self._forward_tensor_cores(ctx, q, q3, cache, tables, plan, proj)
        if self.rot_dims:
            ops.rotate_pairs(q, H, dim + rd, dim, rd, self.rot_dims, self.inv_freq, ctx.positions, ctx.token_seq, R,
                             **rot_args)
        q_abs = torch.empty((T, H, R), dtype=h.dtype, device=h.device)
        if h.dtype == torch.float32:
            for hh in range(H):
                ops.sgemm_tn(q3[:, hh, :dim], self.w_uk_t[hh], q_abs[:, hh, :])
        else:
            torch.bmm(q3[:, :, :dim].transpose(0, 1), self.w_uk, out=q_abs.transpose(0, 1))
        n_rows = T if out_rows is None else out_rows.numel()
        o_lat = torch.empty((n_rows, H, R), dtype=h.dtype, device=h.device)
        ops.latent_attn(q_abs, q3[:, :, dim:], o_lat, cache.k, ctx.token_seq, ctx.positions, tables.indptr,
                        tables.page_ids, out_rows, n_rows, cache.page_size, self.scale, self.window, ctx.status)
        return self._values_out(ctx, o_lat, n_rows, proj, out_rows)

    def _values_out(self, ctx, o_lat, n_rows, proj, out_rows):
        """o_lat [rows, H, rank] (any strides with a unit last one) through W_uv, head by head, the output gate (its
        logits are columns of ``proj``, the tokens of o_lat's rows named by ``out_rows``) and W_o."""
        H = self.n_heads
        val = torch.empty((n_rows, H, self.vdim), dtype=o_lat.dtype, device=o_lat.device)
        if o_lat.dtype == torch.float32:
            for hh in range(H):
                ops.sgemm_tn(o_lat[:, hh, :], self.w_uv[hh], val[:, hh, :])
        else:
            torch.bmm(o_lat.transpose(0, 1), self.w_uv.transpose(1, 2), out=val.transpose(0, 1))
        val = val.view(n_rows, H * self.vdim)
        if self.gated:
            ops.head_sigmoid_gate(val, proj, self.gate_off, out_rows, H, self.vdim, self.kv_rank)
        if self.out_f32:
            return ops.linear_out_f32(val, self.w_o, ctx.status)
        return ops.linear(val, self.w_o)

    def _forward_tensor_cores(self, ctx, q, q3, cache, tables, plan, proj):
        T, H, R, rd, dim = q.shape[0], self.n_heads, self.kv_rank, self.rot_dim, self.dim
        Dk = R + rd
        # queries as the kernels read them: head by head [q_abs (rank) | rotated q_rot (rot)]
        q_lat = torch.empty((T, H, Dk), dtype=q.dtype, device=q.device)
        torch.bmm(q3[:, :, :dim].transpose(0, 1), self.w_uk, out=q_lat[:, :, :R].transpose(0, 1))
        ops.rotate_pairs(q, H, dim + rd, dim, rd, self.rot_dims, self.inv_freq, ctx.positions, ctx.token_seq, R,
                         out=q_lat.view(T, H * Dk), out_head_stride=Dk, out_off=R, freq64=self.freq64, halves=self.halves,
                         mag=self.mag)
        q2 = q_lat.view(T, H * Dk)
        attn = torch.empty((T, H * Dk), dtype=q.dtype, device=q.device)
        caps = ctx.plan_caps.get(self.plan_key()) if ctx.plan_caps else None
        counts = ctx.host_plans[self.plan_key()]["counts"]
        items_cap = caps["items"] if caps else int(counts[0])
        dec_cap = caps["dec"] if caps else int(counts[1])
        tiles_cap = caps["tiles"] if caps else int(counts[2])
        c = plan["counts"]
        rows = cache.k  # keys and values at once
        if dec_cap:
            ops.attn_decode_mma(q2, rows, rows, ctx.seq_q_start, ctx.seq_kv_len, tables.indptr, tables.page_ids,
                                plan["items"], c[0:1], items_cap, plan["dec_seqs"], plan["dec_item_start"], c[1:2],
                                dec_cap, attn, H, 1, Dk, cache.page_size, self.scale, self.window,
                                item_entry=plan["item_entry"], tma=bool(counts[5]), status=ctx.status)
        if tiles_cap:
            ops.attn_prefill_mma(q2, attn, rows, rows, ctx.seq_q_start, ctx.seq_q_len, ctx.seq_kv_len, tables.indptr,
                                 tables.page_ids, plan["tiles"], c[2:3], tiles_cap, H, 1, Dk, cache.page_size, self.scale,
                                 self.window, ctx.status)
        return self._values_out(ctx, attn.view(T, H, Dk)[:, :, :R], T, proj, None)
