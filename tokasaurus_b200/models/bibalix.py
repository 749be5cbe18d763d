"""The Bibalix decoder put together from parts, and its registry entry.

A pre-norm decoder (``parts.block.PreNormBlock`` over layer norms with weight and bias) whose layers config.json lists
one by one.  A layer's mixer is differential attention (``parts.diff_attention.DifferentialAttention``: two softmax
maps a head over the same values, grouped key/value heads, biases, q and k norms with weights, a rotation in halves on
part of a vector, a window that keeps a request's first positions in sight, an output gate a head) or latent attention
(``parts.latent_attention.LatentAttention`` with queries projected straight from the input, a yarn-blended rotation in
halves of the rotated share, a window, an output gate a head).  Its feed-forward is dense with a tanh-GELU gate
(``parts.mlp.GatedMLP``), a mixture of clamped gated units weighed by their shares of the softmax over all experts, with
a gated shared expert (``parts.mlp.RoutedExperts``, ``parts.mlp.ClampedGLU``), or absent.  The head is a layer norm and
the embedding table itself.

Tensor names: ``embed``; per layer i ``l<i>.norm1`` / ``.norm2`` (biases ``.b``), the mixer's ``l<i>.mix.*``, the
feed-forward's ``l<i>.mlp.gate`` / ``.up`` / ``.down`` (dense) or ``.router``, ``.e<j>.gate`` / ``.up`` / ``.down``,
``.shared.gate`` / ``.up`` / ``.down`` / ``.sg`` (mixture); ``final.norm`` (bias ``.b``).
"""

from __future__ import annotations

from tokasaurus_b200.config.bibalix_config import BibalixConfig, DifferentialAttentionConfig
from tokasaurus_b200.config.registry import register_architecture
from tokasaurus_b200.parts import (
    ClampedGLU,
    DecoderModel,
    DifferentialAttention,
    GatedMLP,
    LatentAttention,
    LayerNorm,
    OutputHead,
    PreNormBlock,
    RotaryEncoding,
    RoutedExperts,
    TokenEmbedding,
)

CLAMPED_UNIT_ALPHA = 1.702  # the factor inside the clamped unit's sigmoid


def _rotary(rot):
    if rot is None:
        return None
    if rot.scaling is None:
        return RotaryEncoding(rot.dims, rot.base)
    s = rot.scaling
    return RotaryEncoding(rot.dims, rot.base, "yarn", factor=s.factor, original_max_position_embeddings=s.original,
                          yarn_fast=s.fast, yarn_slow=s.slow)


def build_bibalix(cfg: BibalixConfig) -> DecoderModel:
    W, eps = cfg.width, cfg.norm_eps
    blocks = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}", layer.mixer
        if isinstance(m, DifferentialAttentionConfig):
            mixer = DifferentialAttention(
                W, m.heads, m.kv_heads, m.dim, m.vdim, m.scale, m.diff, m.window, m.keep_first, eps, q_name=f"{p}.mix.q",
                k_name=f"{p}.mix.k", v_name=f"{p}.mix.v", o_name=f"{p}.mix.o",
                lambda_names=(f"{p}.mix.lq1", f"{p}.mix.lk1", f"{p}.mix.lq2", f"{p}.mix.lk2"), gate_name=f"{p}.mix.g",
                bias_names=(f"{p}.mix.q.b", f"{p}.mix.k.b", f"{p}.mix.v.b"),
                qk_norm_names=(f"{p}.mix.q.norm", f"{p}.mix.k.norm"), rotary=_rotary(m.rot), rotary_pairs=False)
        else:
            mixer = LatentAttention(
                W, m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, None, m.scale, 10000.0, 0, eps, m.window,
                names=dict(q=f"{p}.mix.q", dkv=f"{p}.mix.dkv", dkv_norm=f"{p}.mix.dkv.norm", uk=f"{p}.mix.uk",
                           uv=f"{p}.mix.uv", o=f"{p}.mix.o", g=f"{p}.mix.g"),
                rotary=_rotary(m.rot), rotary_pairs=False, out_f32=True)
        ff = layer.mlp
        if ff is None:
            ffn = None
        elif ff.kind == "dense":
            ffn = GatedMLP(W, ff.ff, f"{p}.mlp.gate", f"{p}.mlp.up", f"{p}.mlp.down", activation="gelu_tanh", out_f32=True)
        else:
            shared = None
            if ff.shared_ff is not None:
                shared = ClampedGLU(W, ff.shared_ff, ff.shared_limit, f"{p}.mlp.shared.gate", f"{p}.mlp.shared.up",
                                    f"{p}.mlp.shared.down", alpha=CLAMPED_UNIT_ALPHA)
            ffn = RoutedExperts(W, ff.ff, ff.experts, ff.top, f"{p}.mlp.router", None,
                                lambda e, p=p: (f"{p}.mlp.e{e}.gate", f"{p}.mlp.e{e}.up", f"{p}.mlp.e{e}.down"), shared,
                                expert="clamped", clamp=(ff.limit, CLAMPED_UNIT_ALPHA),
                                over_all=dict(scale=ff.router_scale),
                                shared_gate_name=f"{p}.mlp.shared.sg" if shared is not None else None)
        blocks.append(PreNormBlock(
            mixer_norm=LayerNorm(W, eps, f"{p}.norm1", f"{p}.norm1.b"), mixer=mixer,
            ffn_norm=LayerNorm(W, eps, f"{p}.norm2", f"{p}.norm2.b") if ffn is not None else None, ffn=ffn))
    return DecoderModel(embedding=TokenEmbedding(cfg.vocab, W, "embed"), blocks=blocks,
                        head=OutputHead(cfg.vocab, W, LayerNorm(W, eps, "final.norm", "final.norm.b"), "embed"))


register_architecture("Bibalix", BibalixConfig.from_dict, build_bibalix, model_types=("bibalix",), replace=True)
