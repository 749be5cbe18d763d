"""The Verozen decoder put together from parts, and its registry entry.

A decoder that norms AFTER each residual sum (``parts.block.PostNormBlock``: ``x = norm(alpha * x + sublayer(x))``, RMS
norms in equal parts of a row), and adds a per-token side input after every layer's feed-forward
(``parts.side_input.TokenSideInput``: a slice of a second embedding table, gated by the stream).  config.json lists the
layers one by one; a layer's mixer is gated linear attention with a decay for every key channel
(``parts.recurrent.GatedLinearAttention``), retention with a fixed decay a head and rotated q and k
(``parts.recurrent.Retention``), or grouped-query attention whose weights are sigmoids, not a softmax, whose values are
the keys as projected, with normed and partly rotated q and k (``parts.sink_attention.SinkAttention`` with
``weights="sigmoid"``); its feed-forward is a mixture of ungated GELU experts chosen by sigmoid scores within the best
groups (``parts.mlp.RoutedExperts`` with ``scored=`` and ``expert="gelu"``) or absent.

Tensor names: ``embed``, ``side.embed``; per layer i ``l<i>.norm1`` / ``.norm2``, the mixer's ``l<i>.mix.*``, the
feed-forward's ``l<i>.mlp.router`` / ``.correction`` / ``.e<j>.up`` / ``.e<j>.down``, the side input's
``l<i>.side.gate`` / ``.proj`` / ``.norm``; ``final.norm``; ``head``.
"""

from __future__ import annotations

import torch

from tokasaurus_b200.config.registry import register_architecture
from tokasaurus_b200.config.verozen_config import GatedLinearAttentionConfig, RetentionConfig, VerozenConfig
from tokasaurus_b200.parts import (
    DecoderModel,
    GatedLinearAttention,
    GroupRMSNorm,
    OutputHead,
    PostNormBlock,
    Retention,
    RotaryEncoding,
    RoutedExperts,
    SinkAttention,
    TokenEmbedding,
    TokenSideInput,
)


def build_verozen(cfg: VerozenConfig) -> DecoderModel:
    W, eps, groups = cfg.width, cfg.norm_eps, cfg.norm_groups
    n_layers = len(cfg.layers)
    blocks = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}", layer.mixer
        rot = getattr(m, "rot", None)
        rotary = RotaryEncoding(rot.dims, rot.base) if rot is not None else None
        if isinstance(m, GatedLinearAttentionConfig):
            mixer = GatedLinearAttention(W, m.heads, m.dim, m.vdim, m.tau, eps, q_name=f"{p}.mix.q", k_name=f"{p}.mix.k",
                                         v_name=f"{p}.mix.v", g_name=f"{p}.mix.g", a1_name=f"{p}.mix.a1",
                                         a2_name=f"{p}.mix.a2", a2_bias_name=f"{p}.mix.a2.b", norm_name=f"{p}.mix.norm",
                                         o_name=f"{p}.mix.o", rank=m.rank)
        elif isinstance(m, RetentionConfig):
            mixer = Retention(W, m.heads, m.dim, m.vdim, m.decay, rotary, eps, q_name=f"{p}.mix.q", k_name=f"{p}.mix.k",
                              v_name=f"{p}.mix.v", g_name=f"{p}.mix.g", o_name=f"{p}.mix.o", rotary_pairs=False)
        else:
            mixer = SinkAttention(W, m.heads, m.kv_heads, m.dim, m.vdim, m.scale, None, None, eps, q_name=f"{p}.mix.q",
                                  k_name=f"{p}.mix.k", v_name=None, o_name=f"{p}.mix.o", sink_name=None, unit_norm=True,
                                  qk_norm_names=(f"{p}.mix.q.norm", f"{p}.mix.k.norm"), rotary=rotary, rotary_pairs=True,
                                  values_are_keys=True, head_scale_name=f"{p}.mix.temp", head_bias_name=f"{p}.mix.pb",
                                  weights="sigmoid")
        ff = layer.mlp
        ffn = None
        if ff is not None:
            ffn = RoutedExperts(W, ff.ff, ff.experts, ff.top, f"{p}.mlp.router", None,
                                lambda e, p=p: (f"{p}.mlp.e{e}.up", f"{p}.mlp.e{e}.down"),
                                scored=dict(correction=f"{p}.mlp.correction", groups=ff.groups, keep=ff.keep, scale=ff.scale),
                                expert="gelu", out_dtype=torch.float32)
        side = None
        if cfg.side_dim is not None:
            side = TokenSideInput(W, cfg.side_dim, cfg.vocab, "side.embed", n_layers * cfg.side_dim, i * cfg.side_dim,
                                  f"{p}.side.gate", f"{p}.side.proj", f"{p}.side.norm", eps)
        blocks.append(PostNormBlock(mixer, GroupRMSNorm(W, eps, f"{p}.norm1", groups), ffn,
                                    GroupRMSNorm(W, eps, f"{p}.norm2", groups, optional=ffn is None),
                                    alpha=cfg.alpha, side=side))
    return DecoderModel(embedding=TokenEmbedding(cfg.vocab, W, "embed"), blocks=blocks,
                        head=OutputHead(cfg.vocab, W, GroupRMSNorm(W, eps, "final.norm", groups), "head"))


register_architecture("Verozen", VerozenConfig.from_dict, build_verozen, model_types=("verozen",), replace=True)
