"""Small Bibalix models for the tests: configurations whose sizes differ wherever they could be confused, weights with
signs and sizes of their own, and the plain implementation's logits.

Every model exists twice.  ``dyn``: routers whose choice moves from token to token, with margins (asserted here, on the
plain implementation) wide enough that float32 arithmetic cannot turn a choice.  ``tier``: the same model with routers
whose first channel holds one expert a tier while the norm before them makes that channel 1 for every token (weight 0,
bias 1), so that the choice is the same for every token while the chosen experts' weights still move with it: for
bfloat16, whose rounding of a router's input would turn close choices and, through cached keys, everything after
them."""

from __future__ import annotations

import copy

import numpy as np
import torch

import cuttings
import plain_bibalix as plain

F64 = torch.float64


def lat(heads, dim, rot_dim, vdim, rank, scale, window=None, rot=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=rank, scale=scale)
    if window is not None:
        m["mask"] = dict(size=window)
    if rot is not None:
        m["rot"] = rot
    return dict(type="latent_attention", mixer=m)


def att(heads, kv_heads, dim, vdim, scale, diff, window=None, keep=None, rot=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, diff=diff)
    if window is not None:
        m["mask"] = dict(size=window) if keep is None else dict(size=window, keep_first=keep)
    if rot is not None:
        m["rot"] = rot
    return dict(type="attention", mixer=m)


def yarn(dims, base, factor, original, fast=32.0, slow=1.0):
    return dict(dims=dims, base=base, scaling=dict(factor=factor, original=original, fast=fast, slow=slow))


def moe(ff, limit, experts, top, scale, shared=None):
    d = dict(kind="moe", expert=dict(ff=ff, limit=limit), router=dict(experts=experts, top=top, scale=scale))
    if shared is not None:
        d["shared"] = dict(ff=shared[0], limit=shared[1])
    return d


def dense(ff):
    return dict(kind="dense", ff=ff)


MODELS = {
    # both mixers in both kernel families: cached rows of 32 and 64 values (tensor cores in bfloat16) and of 26 and
    # 2 * 24 + 40 (FP32 pipes); rotation on part of the rotated share, blended and plain; a latent layer without a
    # window and without a feed-forward; windows that are no multiples of the page size; kept first positions that end
    # inside a page and beyond one; one, two and all experts chosen
    "a": dict(page=8, lengths=[100, 37, 64, 5, 81, 1, 50], seed=11,
              config=dict(architecture="Bibalix", vocab=131, width=96, norm=dict(eps=1e-5),
                          layers=[dict(lat(3, 16, 8, 24, 24, 0.2, 21, yarn(8, 100.0, 2.0, 16, 4.0, 1.0)), mlp=moe(40, 3.0, 6, 2, 1.5, (24, 1.5))),
                                  dict(att(4, 2, 16, 32, 0.25, 0.4, 37, 3, dict(dims=8, base=500.0)), mlp=dense(72)),
                                  dict(att(2, 2, 24, 40, 0.2, 0.2, 50, 9, dict(dims=24, base=10000.0)), mlp=None),
                                  dict(lat(2, 12, 6, 10, 20, 0.3, None, dict(dims=4, base=50.0)), mlp=moe(32, 0.8, 4, 1, 1.0))])),
    # sizes that the tensor-core kernels take everywhere, expert products on the grouped tensor-core path (64 x 128);
    # more kept first positions than one 64-key tile holds, and than the window; a window of exactly one page with one
    # kept position; eight query heads on one key/value head; all experts chosen; long requests
    "b": dict(page=16, lengths=[300, 150, 40, 210, 33, 64], seed=12,
              config=dict(architecture="Bibalix", vocab=113, width=128, norm=dict(eps=1e-6),
                          layers=[dict(att(8, 1, 32, 64, 0.18, 0.3, 45, 70, dict(dims=32, base=10000.0)), mlp=moe(64, 2.0, 8, 4, 2.0, (64, 1.0))),
                                  dict(lat(4, 32, 16, 32, 48, 0.15, 33, yarn(16, 30000.0, 3.0, 64)), mlp=dense(96)),
                                  dict(att(2, 2, 64, 16, 0.125, 0.6, 16, 1, dict(dims=32, base=1e6)), mlp=moe(72, 1.2, 3, 3, 0.7, (40, 2.5)))])),
    # attention only: no window at all, a window that keeps nothing, no rotation, one head, three key/value heads of
    # six; dense feed-forwards and none
    "c": dict(page=8, lengths=[120, 33, 75, 9, 50], seed=13,
              config=dict(architecture="Bibalix", vocab=101, width=64, norm=dict(eps=1e-5),
                          layers=[dict(att(1, 1, 16, 16, 0.3, 0.5), mlp=dense(40)),
                                  dict(att(6, 3, 8, 24, 0.35, 0.1, 25, None), mlp=None),
                                  dict(att(3, 1, 20, 12, 0.25, 0.7, 11, 11, dict(dims=10, base=300.0)), mlp=dense(56))])),
    # latent attention only, one cache group shared by two layers and a second one: a rotated share that is all of a
    # head's query (dim 8 beside rot 24), a rank that is no multiple of 8, windows of one and two pages
    "d": dict(page=16, lengths=[90, 20, 47, 3, 61], seed=14,
              config=dict(architecture="Bibalix", vocab=89, width=80, norm=dict(eps=1e-6),
                          layers=[dict(lat(5, 8, 24, 16, 40, 0.2, 16, yarn(24, 1000.0, 8.0, 32, 8.0, 2.0)), mlp=moe(32, 2.0, 5, 2, 1.0)),
                                  dict(lat(5, 8, 24, 16, 40, 0.2, 16, yarn(24, 1000.0, 8.0, 32, 8.0, 2.0)), mlp=dense(48)),
                                  dict(lat(2, 20, 10, 28, 21, 0.25, 32, dict(dims=10, base=10000.0)), mlp=moe(24, 1.0, 6, 3, 2.5, (16, 0.5)))])),
    # sizes that fit no vector load: a width that is no multiple of four, an odd vocabulary, heads of 10 and 6 channels,
    # a rank of 18, inner sizes of 26 and 22; two experts of which one is chosen
    "e": dict(page=8, lengths=[70, 21, 44, 2, 33], seed=15,
              config=dict(architecture="Bibalix", vocab=77, width=70, norm=dict(eps=1e-5),
                          layers=[dict(att(3, 1, 10, 14, 0.3, 0.35, 19, 2, dict(dims=6, base=200.0)), mlp=moe(22, 1.5, 2, 1, 1.3, (26, 1.0))),
                                  dict(lat(3, 6, 10, 14, 18, 0.3, 13, yarn(10, 300.0, 2.0, 8, 4.0, 0.5)), mlp=dense(26))])),
}

MIN_MARGIN = 5e-5  # of a router's logit: far more than float32 sums of a router's width can move one
TIER_MARGIN = 0.3  # between tiers: far more than bfloat16 rounding of a router's input moves a logit


def adjust(name: str, t: torch.Tensor, g: torch.Generator, tiered: bool) -> torch.Tensor:
    """Vectors that are no norm weights get signs and sizes of their own."""
    tail = name.split(".", 1)[1] if "." in name else name
    if tiered and tail in ("norm2", "norm2.b"):
        t = torch.randn(t.shape, generator=g) * 0.2 if tail == "norm2.b" else t.clone().float()
        t[0] = 1.0 if tail == "norm2.b" else 0.0                          # the feed-forward's input has a channel that is 1
        return t
    if tail.endswith(".b") and tail.startswith("mix."):
        return torch.randn(t.shape, generator=g) * 0.3                    # projection biases
    if tail.endswith(".b"):
        return torch.randn(t.shape, generator=g) * 0.2                    # layer-norm biases
    if tail in ("mix.lq1", "mix.lk1", "mix.lq2", "mix.lk2"):
        return torch.randn(t.shape, generator=g) * (0.9 / t.numel() ** 0.25)  # lambda of both signs, of order 1
    if tail == "mix.g":
        return torch.randn(t.shape, generator=g) * 0.3                    # gates well away from 1/2
    if tail == "mlp.shared.sg":
        return torch.randn(t.shape, generator=g) * 0.3
    if tail == "mlp.router":
        r = torch.randn(t.shape, generator=g) * 0.25
        if tiered:
            r = r * 0.08
            r[:, 0] = 2.0 * torch.randperm(t.shape[0], generator=g).to(torch.float32)  # times the channel that is 1
        return r
    return t


def router_margins(config, w64, tokens):
    """The smallest gap between the last chosen expert's logit and the first one's that is not, over tokens and layers."""
    gaps, layers = [], []
    logits = plain.forward(config, w64, tokens, layers_out=layers)
    x = [w64["embed"][torch.as_tensor(tokens)]] + layers
    eps = float(config["norm"]["eps"])
    for i, layer in enumerate(config["layers"]):
        mlp = layer.get("mlp")
        if not mlp or mlp["kind"] != "moe" or mlp["router"]["top"] >= mlp["router"]["experts"]:
            continue
        # the stream after the mixer: the layer's output minus its feed-forward's share is not kept, so run the mixer again
        p = f"l{i}."
        h = plain.layer_norm(x[i], w64[p + "norm1"], w64[p + "norm1.b"], eps)
        mixer = {"attention": plain.differential_attention, "latent_attention": plain.latent_attention}[layer["type"]]
        mid = x[i] + mixer(h, w64, p + "mix.", layer["mixer"], eps)
        z = plain.layer_norm(mid, w64[p + "norm2"], w64[p + "norm2.b"], eps) @ w64[p + "mlp.router"].T
        s = torch.sort(z, dim=-1, descending=True).values
        top = mlp["router"]["top"]
        gaps.append(float((s[:, top - 1] - s[:, top]).min()))
    return (min(gaps) if gaps else float("inf")), logits


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
            g = torch.Generator().manual_seed(spec["seed"])
            for k in sorted(w):
                w[k] = adjust(k, w[k], g, kind == "tier").to(w[k].dtype)
            save_file(w, str(folder / "model.safetensors"))
            w64 = {k: v.to(F64) for k, v in w.items()}
            want, noise, margin = {}, {}, float("inf")
            for rid, t in reqs.items():
                mg, logits = router_margins(spec["config"], w64, t)
                want[rid] = logits.numpy()
                noise[rid] = rounding_noise(spec["config"], w64, t, want[rid], variant_dtype(kind))
                margin = min(margin, mg)
            assert margin > (MIN_MARGIN if kind == "dyn" else TIER_MARGIN), \
                f"model {name} ({kind}): a router's choice rests on a margin of {margin:.2g}"
            out[(name, kind)] = dict(folder=folder, config=spec["config"], weights=w64, reqs=reqs, want=want,
                                     noise=noise, page=spec["page"], margin=margin)
    return out


def variant(dtype: str) -> str:
    return "dyn" if dtype == "float32" else "tier"


def variant_dtype(kind: str) -> str:
    return "float32" if kind == "dyn" else "bfloat16"


def to_bfloat16_and_back(x):
    return x.to(torch.bfloat16).to(x.dtype)


def row_error(d):
    """Per position: the root mean square over the vocabulary of a difference of logits, its mean taken off."""
    return np.sqrt(((d - d.mean(axis=1, keepdims=True)) ** 2).mean(axis=1))


def rounding_noise(config, w64, tokens, want, dtype):
    """How far rounding alone moves the logits at every position: the plain implementation once more, in float32
    arithmetic (``float32``) or in float64 with the operands of every matrix product rounded to bfloat16
    (``bfloat16``), against its float64 logits."""
    if dtype == "float32":
        got = plain.forward(config, w64, tokens, dtype=torch.float32).numpy().astype(np.float64)
    else:
        got = plain.forward(config, w64, tokens, round_fn=to_bfloat16_and_back).numpy()
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
