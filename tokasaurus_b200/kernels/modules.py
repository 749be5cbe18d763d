"""The list of kernel modules (source file, compile-time constants) that exist, and which of them a model of given
head sizes and precision needs: what is compiled at a first call is what that model runs."""

from __future__ import annotations

# every precision: embedding, norms, rotary + cache write, activation, row gather; sampling
SHARED = [("elementwise.cu", None), ("sampling.cu", None)]
# float32: the FP32-FMA product; attention on the FP32 pipes (per head size, below)
FLOAT32 = [("sgemm.cu", None)]
# bfloat16: small-batch products (mma.sync and tcgen05), the tcgen05 product for many rows
BFLOAT16 = [("linear_smallm.cu", None), ("gemm_tcgen05.cu", None), ("gemm_tcgen05_decode.cu", None)]
# tested alternatives that no model needs: built by the build check, loaded by whoever calls them
EXTRA = [("linear_decode.cu", None)]


def head_dim_modules(head_dim: int, dtype: str | None = None) -> list[tuple[str, dict | None]]:
    mods = [("attention_simt.cu", {"TKB_HD": head_dim})]  # float32; in bfloat16 steps whose planner declines
    if dtype in (None, "bfloat16"):
        mods.append(("attention_mma.cu", {"TKB_HD": head_dim}))
        if head_dim == 64:
            mods.append(("attention_tc.cu", None))  # tcgen05 kernel for prompt portions
        if head_dim == 128:
            mods.append(("attention_tc_acc.cu", {"TKB_HD": 128}))  # the same with the output in tensor memory
    return mods


def family_modules() -> list[tuple[str, dict | None]]:
    """Kernel modules of parts that only some model families use (layer norm and short convolution, the gated linear
    recurrence, attention over cached latents, routed experts; norms on sublayer outputs, the recurrence with one decay a
    head and token, attention with capped scores and a sink or with sigmoid weights, with two maps a head), at one or two sets of compile-time sizes each: the build
    check compiles these; a model compiles the sizes it needs (``Part.kernel_modules``)."""
    return [("post_norm.cu", None), ("decay_recurrence.cu", {"TKB_DR_LANES": 32, "TKB_DR_DPT": 4}),
            ("decay_recurrence.cu", {"TKB_DR_LANES": 16, "TKB_DR_DPT": 8}), ("decay_recurrence.cu", {"TKB_DR_LANES": 8, "TKB_DR_DPT": 16}), ("attention_sink.cu", {"TKB_QK": 128, "TKB_VD": 64}),
            ("attention_sink.cu", {"TKB_QK": 24, "TKB_VD": 40}), ("attention_sink.cu", {"TKB_QK": 64, "TKB_VD": 64, "TKB_SIGMOID": 1}),
            ("norm_conv.cu", None), ("moe.cu", None), ("recurrence.cu", {"TKB_REC_DPT": 16, "TKB_REC_CPT": 1}),
            ("recurrence.cu", {"TKB_REC_DPT": 3, "TKB_REC_CPT": 2}), ("latent_attention.cu", {"TKB_LAT_RANK": 192}),
            ("attention_mma.cu", {"TKB_HD": 256}), ("attention_sink.cu", {"TKB_QK": 64, "TKB_VD": 128, "TKB_MAPS": 2}),
            ("attention_sink.cu", {"TKB_QK": 24, "TKB_VD": 40, "TKB_MAPS": 2})]


def optional_modules(head_dim: int) -> list[tuple[str, dict | None]]:
    """Built by the build check, loaded only by callers that ask for them."""
    return EXTRA + [("attention_decode_static.cu", {"TKB_HD": head_dim})]


def all_modules(head_dims, dtype: str | None = None) -> list[tuple[str, dict | None]]:
    """``dtype`` "float32" or "bfloat16": what an engine of that precision needs; None: everything."""
    mods = list(SHARED)
    if dtype in (None, "float32"):
        mods += FLOAT32
    if dtype in (None, "bfloat16"):
        mods += BFLOAT16
    for hd in head_dims:
        mods += head_dim_modules(hd, dtype)
    return mods
