"""The Bibalix decoder stated plainly: whole sequences, no cache, one function a mechanism, float64 by default.

It shares no code with the engine.  ``forward(cfg, weights, tokens)`` takes the config.json dictionary, a dict of
tensors by name and one sequence's token ids, and returns the logits at every position (and, if asked, the residual
stream after every layer).  ``round_fn`` (identity by default) is applied to the inputs of every matrix product: with a
bfloat16 rounding it shows what rounding alone does to the logits.
"""

from __future__ import annotations

import math

import torch


def _ident(x):
    return x


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotary_frequencies(rot: dict, dims: int, dtype=torch.float64):
    """(frequencies [dims / 2], factor on cos and sin) of a rotation; with ``scaling`` the ramp between scaled and
    unscaled frequencies."""
    base = float(rot["base"])
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def turn(t):
        return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turn(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn(float(sc["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_halves(x, positions, freq, mag, dims):
    """x [T, ..., D]: the first ``dims`` channels turned, channel i with channel i + dims / 2."""
    if dims == 0:
        return x
    ang = positions.to(freq.dtype)[:, None] * freq[None, :]  # [T, dims / 2]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = (torch.cos(ang) * mag).view(shape), (torch.sin(ang) * mag).view(shape)
    u, v = x[..., : dims // 2], x[..., dims // 2: dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def visible(T: int, size: int | None, keep_first: int = 0):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if size is not None:
        ok = ok & ((i - j < size) | (j < keep_first))
    return ok


def softmax_attention(q, k, v, scale, mask):
    """q [T, H, d], k [T, H, d], v [T, H, e] -> [T, H, e]."""
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    s = s.masked_fill(~mask[None], float("-inf"))
    return torch.einsum("hij,jhe->ihe", torch.softmax(s, dim=-1), v)


def differential_attention(h, w, p, m, eps, rnd=_ident):
    """The mixer 'attention': two softmax maps a head over the same values, o = a1 - lambda a2."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"]
    diff = float(m["diff"])
    pos = torch.arange(T)
    hr = rnd(h)
    q = (hr @ rnd(w[p + "q"]).T + w[p + "q.b"]).view(T, H, 2, d)
    k = (hr @ rnd(w[p + "k"]).T + w[p + "k.b"]).view(T, G, 2, d)
    v = (hr @ rnd(w[p + "v"]).T + w[p + "v.b"]).view(T, G, e)
    q = rms(q, eps) * w[p + "q.norm"]
    k = rms(k, eps) * w[p + "k.norm"]
    rot = m.get("rot")
    if rot:
        dims = int(rot.get("dims", d))
        f, mag = rotary_frequencies(rot, dims, h.dtype)
        q, k = rotate_halves(q, pos, f, mag, dims), rotate_halves(k, pos, f, mag, dims)
    mask = visible(T, m.get("mask", {}).get("size"), m.get("mask", {}).get("keep_first", 0))
    rep = H // G
    kx = k.repeat_interleave(rep, dim=1)  # query head h reads key/value head h // rep
    vx = v.repeat_interleave(rep, dim=1)
    q, kx, vx = rnd(q), rnd(kx), rnd(vx)
    a1 = softmax_attention(q[:, :, 0], kx[:, :, 0], vx, float(m["scale"]), mask)
    a2 = softmax_attention(q[:, :, 1], kx[:, :, 1], vx, float(m["scale"]), mask)
    lam = torch.exp((w[p + "lq1"] * w[p + "lk1"]).sum()) - torch.exp((w[p + "lq2"] * w[p + "lk2"]).sum()) + diff
    o = rms(a1 - lam * a2, eps) * (1.0 - diff)
    gate = torch.sigmoid(hr @ rnd(w[p + "g"]).T)  # [T, H]
    o = o * gate[:, :, None]
    return rnd(o.reshape(T, H * e)) @ rnd(w[p + "o"]).T


def latent_attention(h, w, p, m, eps, rnd=_ident):
    """The mixer 'latent_attention': keys and values made from one normed latent a token, one shared rotated key part."""
    T = h.shape[0]
    H, d, r, e, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    hr = rnd(h)
    q = (hr @ rnd(w[p + "q"]).T).view(T, H, d + r)
    ckr = hr @ rnd(w[p + "dkv"]).T
    c = rms(ckr[:, :R], eps) * w[p + "dkv.norm"]
    kr = ckr[:, R:]
    rot = m.get("rot")
    if rot:
        dims = int(rot.get("dims", r))
        f, mag = rotary_frequencies(rot, dims, h.dtype)
        qr = rotate_halves(q[:, :, d:], pos, f, mag, dims)
        kr = rotate_halves(kr, pos, f, mag, dims)
    else:
        qr = q[:, :, d:]
    cr = rnd(c)
    kp = (cr @ rnd(w[p + "uk"]).T).view(T, H, d)
    v = (cr @ rnd(w[p + "uv"]).T).view(T, H, e)
    qq = torch.cat([q[:, :, :d], qr], dim=-1)
    kk = torch.cat([kp, kr[:, None, :].expand(T, H, r)], dim=-1)
    mask = visible(T, m.get("mask", {}).get("size"))
    o = softmax_attention(rnd(qq), rnd(kk), rnd(v), float(m["scale"]), mask)
    gate = torch.sigmoid(hr @ rnd(w[p + "g"]).T)
    o = o * gate[:, :, None]
    return rnd(o.reshape(T, H * e)) @ rnd(w[p + "o"]).T


def dense_ff(h, w, p, rnd=_ident):
    hr = rnd(h)
    return rnd(gelu_tanh(hr @ rnd(w[p + "gate"]).T) * (hr @ rnd(w[p + "up"]).T)) @ rnd(w[p + "down"]).T


def clamped_expert(h, w, p, limit, rnd=_ident):
    hr = rnd(h)
    g = (hr @ rnd(w[p + "gate"]).T).clamp(max=limit)
    u = (hr @ rnd(w[p + "up"]).T).clamp(-limit, limit)
    return rnd(g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ rnd(w[p + "down"]).T


def route(h, w_router, top: int, scale: float, rnd=_ident):
    """(chosen experts [T, top], their weights [T, top], all scores [T, E])."""
    s = torch.softmax(rnd(h) @ w_router.T, dim=-1)
    order = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :top]
    return order, torch.gather(s, 1, order) * scale, s


def moe_ff(h, w, p, mlp, rnd=_ident):
    r = mlp["router"]
    idx, wt, _ = route(h, w[p + "router"], int(r["top"]), float(r.get("scale", 1.0)), rnd)
    out = torch.zeros_like(h)
    limit = float(mlp["expert"]["limit"])
    for e in range(int(r["experts"])):
        rows, slot = (idx == e).nonzero(as_tuple=True)
        if rows.numel():
            out[rows] += wt[rows, slot][:, None] * clamped_expert(h[rows], w, f"{p}e{e}.", limit, rnd)
    sh = mlp.get("shared")
    if sh:
        gate = torch.sigmoid(rnd(h) @ rnd(w[p + "shared.sg"]).T)  # [T, 1]
        out = out + gate * clamped_expert(h, w, p + "shared.", float(sh["limit"]), rnd)
    return out


def forward(cfg: dict, w: dict, tokens, dtype=torch.float64, round_fn=None, layers_out: list | None = None):
    rnd = round_fn or _ident
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
        mixer = {"attention": differential_attention, "latent_attention": latent_attention}[layer["type"]]
        x = x + mixer(h, w, p + "mix.", layer["mixer"], eps, rnd)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps)
            x = x + (dense_ff(h, w, p + "mlp.", rnd) if mlp["kind"] == "dense" else moe_ff(h, w, p + "mlp.", mlp, rnd))
        if layers_out is not None:
            layers_out.append(x.clone())
    h = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    return rnd(h) @ rnd(w["embed"]).T
