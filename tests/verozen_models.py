"""Small Verozen models for the tests: configurations whose sizes differ wherever they could be confused, weights with
signs and sizes of their own, and the plain implementation's logits.

Every model exists twice.  ``dyn``: routers whose choice moves from token to token, with margins (asserted here, on the
plain implementation) wide enough that float32 arithmetic cannot turn a choice.  ``tier``: the same model with
corrections that fix the choice (one expert a tier, tiers further apart than a sigmoid's range), for bfloat16, whose
rounding of a router's input would turn close choices and, through states and cached keys, everything after them;
there the weights of the chosen experts still move with the token."""

from __future__ import annotations

import copy

import numpy as np
import torch

import cuttings
import plain_verozen as plain

F64 = torch.float64


def gla(heads, dim, vdim, tau, rank=None):
    m = dict(heads=heads, dim=dim, vdim=vdim, tau=tau)
    if rank is not None:
        m["rank"] = rank
    return dict(type="gla", mixer=m)


def ret(heads, dim, vdim, decay, rot_dims, base=10000.0):
    return dict(type="retention", mixer=dict(heads=heads, dim=dim, vdim=vdim, decay=decay, rot=dict(dims=rot_dims, base=base)))


def att(heads, kv_heads, dim, scale, rot_dims, base=10000.0):
    return dict(type="attention", mixer=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=scale,
                                             rot=dict(dims=rot_dims, base=base)))


def moe(ff, experts, top, count, keep, scale):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top, scale=scale, groups=dict(count=count, keep=keep)))


MODELS = {
    # all three mixers; norms in three parts; a rank that the configuration gives; attention whose heads are rotated on
    # half their channels; groups of two experts of which half are kept
    "a": dict(page=8, lengths=[100, 37, 64, 5, 81, 1, 50], seed=104,
              config=dict(architecture="Verozen", vocab=131, width=96, norm=dict(eps=1e-5, groups=3), postln_alpha=1.7,
                          token_side=dict(dim=8),
                          layers=[dict(gla(3, 16, 24, 8.0, rank=5), mlp=moe(40, 8, 2, 4, 2, 1.5)),
                                  dict(att(4, 2, 32, 0.2, 16), mlp=moe(56, 8, 2, 4, 2, 1.5)),
                                  dict(ret(2, 24, 40, [0.9, 0.99], 24), mlp=None),
                                  dict(gla(2, 24, 8, 2.0), mlp=moe(40, 6, 1, 1, 1, 1.0))])),
    # retention first, rotated on a quarter of its channels; a layer without a feed-forward; no side input; norms in one
    # part; alpha 1; one chosen expert; as many key/value heads as heads; head sizes that are no multiples of 16
    "b": dict(page=16, lengths=[130, 70, 33, 16, 97],
              config=dict(architecture="Verozen", vocab=97, width=64, norm=dict(eps=1e-6, groups=1), postln_alpha=1.0,
                          layers=[dict(ret(3, 16, 12, [0.5, 0.97, 0.999], 4, 500.0), mlp=moe(24, 4, 1, 2, 1, 2.0)),
                                  dict(gla(4, 8, 20, 16.0), mlp=None),
                                  dict(att(3, 3, 24, 0.3, 24, 1e6), mlp=moe(32, 5, 3, 5, 4, 0.7))])),
    # sizes that the tensor-core kernels take (heads of 16 and 64 on one key/value head, experts of 64 on a width of
    # 128); groups of one expert; every group kept; three chosen; a long request
    "c": dict(page=16, lengths=[300, 150, 40, 210, 33, 64], seed=106,
              config=dict(architecture="Verozen", vocab=113, width=128, norm=dict(eps=1e-6, groups=4), postln_alpha=3.0,
                          token_side=dict(dim=24),
                          layers=[dict(att(8, 1, 16, 0.25, 16), mlp=moe(64, 6, 3, 6, 6, 1.0)),
                                  dict(gla(2, 64, 32, 32.0, rank=16), mlp=moe(64, 6, 3, 3, 2, 2.5)),
                                  dict(ret(4, 32, 16, [0.8, 0.95, 0.99, 0.999], 32, 1e6), mlp=moe(72, 4, 2, 2, 2, 1.0)),
                                  dict(att(2, 2, 64, 0.125, 32), mlp=moe(64, 6, 2, 2, 1, 1.0))])),
    # attention only, of two shapes: two cache groups, no state
    "d": dict(page=8, lengths=[120, 33, 75, 9, 50],
              config=dict(architecture="Verozen", vocab=101, width=64, norm=dict(eps=1e-5, groups=2), postln_alpha=2.0,
                          token_side=dict(dim=4),
                          layers=[dict(att(4, 2, 16, 0.3, 8), mlp=moe(48, 4, 2, 2, 2, 1.0)),
                                  dict(att(2, 1, 40, 0.2, 40, 300.0), mlp=None)])),
    # no attention at all: no pages, only slots
    "e": dict(page=16, lengths=[90, 20, 47, 3, 61],
              config=dict(architecture="Verozen", vocab=89, width=80, norm=dict(eps=1e-6, groups=5), postln_alpha=2.5,
                          token_side=dict(dim=16),
                          layers=[dict(gla(5, 8, 16, 4.0, rank=3), mlp=moe(32, 6, 2, 3, 2, 1.5)),
                                  dict(ret(2, 40, 24, [0.97, 0.9], 20), mlp=moe(32, 6, 2, 3, 2, 1.5))])),
}

MIN_MARGIN = 2e-4  # of a sigmoid score: hundreds of times what float32 sums of a router's width can move one
TIER_MARGIN = 0.2  # between tiers: far more than bfloat16 rounding of a router's input moves a score


def adjust(name: str, t: torch.Tensor, g: torch.Generator, tiered: bool) -> torch.Tensor:
    """Vectors that are no norm weights get signs and sizes of their own; routers get rows long enough to move scores."""
    tail = name.split(".", 1)[1] if "." in name else name
    if tail == "mix.a2.b":
        return torch.randn(t.shape, generator=g) * 1.5 + 2.0          # decays from a few tokens to hundreds
    if tail == "mix.a2":
        return torch.randn(t.shape, generator=g) * 0.4
    if tail == "mix.temp":
        return torch.rand(t.shape, generator=g) * 0.6 + 0.7
    if tail == "mix.pb":
        return torch.randn(t.shape, generator=g) * 0.7 - 3.0
    if tail == "mlp.router":
        return torch.randn(t.shape, generator=g) * 0.25
    if tail == "mlp.correction":
        if tiered:
            return -1.5 * torch.randperm(t.numel(), generator=g).to(torch.float32)
        return torch.randn(t.shape, generator=g) * 0.3 - 0.5              # choice scores of both signs
    if tail == "side.norm":
        return torch.rand(t.shape, generator=g) * 0.5 + 0.1
    if name == "side.embed":
        return torch.randn(t.shape, generator=g)
    return t


def make_models(root, names=None):
    from safetensors import safe_open
    from safetensors.torch import save_file
    from tokasaurus_b200.weights import write_model_folder

    out = {}
    for index, (name, spec) in enumerate(MODELS.items()):
        if names is not None and name not in names:
            continue
        V = spec["config"]["vocab"]
        reqs = {f"{name}{i}": cuttings.random_tokens(n, V, 40 + i) for i, n in enumerate(spec["lengths"])}
        for kind in ("dyn", "tier"):
            folder = write_model_folder(root / f"{name}_{kind}", spec["config"], seed=31 + index, std=0.12, norm_init="uniform")
            w = {}
            with safe_open(str(folder / "model.safetensors"), framework="pt") as f:
                for k in f.keys():
                    w[k] = f.get_tensor(k)
            g = torch.Generator().manual_seed(spec.get("seed", 7 + index))
            for k in sorted(w):
                w[k] = adjust(k, w[k], g, kind == "tier").to(w[k].dtype)
            save_file(w, str(folder / "model.safetensors"))
            w64 = {k: v.to(F64) for k, v in w.items()}
            want, noise, margin = {}, {}, float("inf")
            for rid, t in reqs.items():
                ms = []
                want[rid] = plain.forward(spec["config"], w64, t, margins=ms).numpy()
                noise[rid] = rounding_noise(spec["config"], w64, t, want[rid], variant_dtype(kind))
                margin = min([margin] + [float(m.min()) for m in ms])
            assert margin > (MIN_MARGIN if kind == "dyn" else TIER_MARGIN), \
                f"model {name} ({kind}): a router's choice rests on a margin of {margin:.2g}"
            out[(name, kind)] = dict(folder=folder, config=spec["config"], weights=w64, reqs=reqs, want=want,
                                     noise=noise, page=spec["page"], margin=margin)
    return out


def variant(dtype: str) -> str:
    return "dyn" if dtype == "float32" else "tier"


def variant_dtype(kind: str) -> str:
    return "float32" if kind == "dyn" else "bfloat16"


def row_error(d):
    """Per position: the root mean square over the vocabulary of a difference of logits, its mean taken off."""
    return np.sqrt(((d - d.mean(axis=1, keepdims=True)) ** 2).mean(axis=1))


def rounding_noise(config, w64, tokens, want, dtype):
    """How far rounding alone moves the logits at every position: the plain implementation once more, in float32
    arithmetic (``float32``) or in float64 with the rows that enter every matrix product rounded to bfloat16
    (``bfloat16``), against its float64 logits.  Some positions are many times more sensitive than most (a score near a
    sigmoid's steep part early in a sequence, a part of a row with a small mean square before a norm), so the
    comparisons measure each position against its own noise, not against one number for all."""
    if dtype == "float32":
        got = plain.forward(config, {k: v.to(torch.float32) for k, v in w64.items()}, tokens).numpy().astype(np.float64)
    else:
        with plain.rounded(plain.to_bfloat16_and_back):
            got = plain.forward(config, w64, tokens).numpy()
    return row_error(got - want)


def check_logits(got, m, dtype, what):
    """A position's limit is 3 times what rounding alone does there (``rounding_noise``; at least the request's median,
    since one draw of the rounding can come out small).  No position is over 1.5 times its limit, and at most one in
    fifty (or one) over the limit itself."""
    for rid, ref in m["want"].items():
        noise = m["noise"][rid]
        limit = 3.0 * np.maximum(noise, np.median(noise))
        err = row_error(got[rid] - ref)
        over = np.nonzero(err > limit)[0]
        far = np.nonzero(err > 1.5 * limit)[0]
        assert far.size == 0, (f"{dtype} {what}: request {rid}: first wrong token at position {far[0]} "
                               f"(error {err[far[0]]:.3g}, limit {limit[far[0]]:.3g}); {far.size} of {len(err)} far over")
        assert over.size <= max(1, len(err) // 50), (f"{dtype} {what}: request {rid}: {over.size} of {len(err)} positions "
                                                    f"over their limits, the first at {over[0]}")


def changed(config, path, value):
    """A copy of ``config`` with the mixers' (or feed-forwards') entry ``path`` replaced wherever it exists."""
    cfg = copy.deepcopy(config)
    for l in cfg["layers"]:
        for part in ("mixer", "mlp"):
            d = l.get(part)
            keys = path.split(".")
            while d is not None and len(keys) > 1:
                d = d.get(keys[0])
                keys = keys[1:]
            if d is not None and keys[0] in d:
                d[keys[0]] = value(d[keys[0]]) if callable(value) else value
    return cfg
