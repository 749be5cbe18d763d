"""A plain, slow statement of the Verozen decoder: whole sequences, no cache, float64, one function a
mechanism.  It shares no code with the engine; the tests compare the engine with it.

Notation: T tokens, W the model width, rows are tokens, positions p = 0, 1, ...  Linear weights are [out, in].

* group norm:        N_g(x): x cut into g equal consecutive parts, each part / sqrt(mean(part^2) + eps), all * w
* a layer:           x = N_g(a x + mixer(x)),  x = N_g(a x + ff(x)),  x = x + N_1(P (gelu_tanh(G x) * e_token)) * w_s
                     (norms after the sums; e_token is the layer's slice of a second embedding table)
* gated linear attention:  S_t = diag(f_t) S_(t-1) + k_t v_t^T,  o_t = S_t^T (q_t / sqrt(d)),
                     f = sigmoid(A2 (A1 h) + b)^(1/tau) per key channel; each head's o RMS-normed with one shared
                     weight; gate silu(W_g h)
* retention:         S_t = lambda_h S_(t-1) + (k_t / sqrt(d)) v_t^T,  o_t = S_t^T q_t,  q and k rotated in halves
                     (channel i with i + dims/2); each head's o divided by its root mean square; gate silu(W_g h)
* sigmoid attention: q and k RMS-normed per head with a weight, rotated in neighbouring pairs (2i, 2i + 1) on the
                     first dims channels, the values are the keys as projected; weight of key j <= i is
                     sigmoid(q_i . k_j * scale * temp_h + bias_h), not normalised over the keys
* routed experts:    s = sigmoid(R h); choice scores c = s + correction; experts in equal groups of neighbours, a group
                     scores the sum of its two largest c, only the best `keep` groups may be chosen from; the `top`
                     largest c are chosen; weights s / (sum of the chosen s + 1e-20) * scale; expert = D gelu_erf(U h)
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64

# When set (``rounded``), every matrix product's left operand is passed through it first: rounding the rows to 16 bits
# and back shows how far a 16-bit engine's rounding alone moves the logits at each position.
_ROUND = None


class rounded:
    """``with rounded(fn): forward(...)``: the inputs of all matrix products go through ``fn``."""

    def __init__(self, fn):
        self.fn = fn

    def __enter__(self):
        global _ROUND
        self.before, _ROUND = _ROUND, self.fn

    def __exit__(self, *exc):
        global _ROUND
        _ROUND = self.before


def to_bfloat16_and_back(x):
    return x.to(torch.bfloat16).to(x.dtype)


def lin(x, w):
    """W x for every row of x; W is [out, in]."""
    return (x if _ROUND is None else _ROUND(x)) @ w.T


def group_norm(x, w, eps, groups=1):
    T, n = x.shape[0], x.shape[-1]
    parts = x.reshape(T, groups, n // groups)
    y = (parts / torch.sqrt((parts * parts).mean(-1, keepdim=True) + eps)).reshape(x.shape)
    return y if w is None else y * w


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z):
    return 0.5 * z * (1 + torch.erf(z / math.sqrt(2)))


def angles(T, dims, base, start=0):
    p = torch.arange(start, start + T, dtype=F64)[:, None]
    i = torch.arange(dims // 2, dtype=F64)[None, :]
    return p * base ** (-2 * i / dims)


def rotate_halves(x, dims, base, start=0):
    """x [T, H, d]: channel i pairs with channel i + dims/2, for i < dims/2; channels from dims on pass."""
    a = angles(x.shape[0], dims, base, start)[:, None, :]
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    out = x.clone()
    out[..., :dims // 2] = u * torch.cos(a) - v * torch.sin(a)
    out[..., dims // 2:dims] = v * torch.cos(a) + u * torch.sin(a)
    return out


def rotate_pairs(x, dims, base, start=0):
    """x [T, H, d]: channel 2i pairs with channel 2i + 1, for 2i < dims; channels from dims on pass."""
    a = angles(x.shape[0], dims, base, start)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * torch.cos(a) - v * torch.sin(a)
    out[..., 1:dims:2] = v * torch.cos(a) + u * torch.sin(a)
    return out


def linear_recurrence(q, k, v, decay):
    """q, k [T, H, d], v [T, H, e], decay [T, H, d] (a factor for every key channel).  o_t = S_t^T q_t."""
    T, H, d = q.shape
    S = torch.zeros(H, d, v.shape[-1], dtype=q.dtype)
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for t in range(T):
        S = decay[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hde,hd->he", S, q[t])
    return out, S


def gla_mixer(h, p, heads, dim, vdim, tau, eps):
    """p: q, k, v, g, o, norm, a1, a2, a2.b."""
    T = h.shape[0]
    q = lin(h, p["q"]).reshape(T, heads, dim) * dim ** -0.5
    k = lin(h, p["k"]).reshape(T, heads, dim)
    v = lin(h, p["v"]).reshape(T, heads, vdim)
    z = lin(h, p["a1"]) @ p["a2"].T + p["a2.b"]  # the second factor takes unrounded rows
    f = torch.sigmoid(z).pow(1.0 / tau).reshape(T, heads, dim)
    o, _ = linear_recurrence(q, k, v, f)
    o = group_norm(o.reshape(T * heads, vdim), p["norm"], eps).reshape(T, heads * vdim)
    return lin(o * silu(lin(h, p["g"])), p["o"])


def retention_mixer(h, p, heads, dim, vdim, decay, rot_dims, rot_base, eps, start=0):
    """p: q, k, v, g, o."""
    T = h.shape[0]
    q = rotate_halves(lin(h, p["q"]).reshape(T, heads, dim), rot_dims, rot_base, start)
    k = rotate_halves(lin(h, p["k"]).reshape(T, heads, dim), rot_dims, rot_base, start) * dim ** -0.5
    v = lin(h, p["v"]).reshape(T, heads, vdim)
    lam = torch.as_tensor(decay, dtype=h.dtype)[None, :, None].expand(T, heads, dim)
    o, _ = linear_recurrence(q, k, v, lam)
    o = group_norm(o.reshape(T * heads, vdim), None, eps).reshape(T, heads * vdim)
    return lin(o * silu(lin(h, p["g"])), p["o"])


def sigmoid_attention(q, k, v, scale, temp, bias):
    """q [T, H, d], k [T, G, d], v [T, G, e], temp and bias [H]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    seen = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
    for h in range(H):
        g = h // (H // G)
        s = lin(q[:, h], k[:, g]) * scale * temp[h] + bias[h]
        out[:, h] = lin(torch.sigmoid(s) * seen, v[:, g].T)
    return out


def attention_mixer(h, p, heads, kv_heads, dim, scale, rot_dims, rot_base, eps, start=0):
    """p: q, k, q.norm, k.norm, temp, pb, o."""
    T = h.shape[0]
    q = lin(h, p["q"]).reshape(T, heads, dim)
    k = lin(h, p["k"]).reshape(T, kv_heads, dim)
    v = k
    q = group_norm(q.reshape(T * heads, dim), p["q.norm"], eps).reshape(T, heads, dim)
    k = group_norm(k.reshape(T * kv_heads, dim), p["k.norm"], eps).reshape(T, kv_heads, dim)
    q, k = rotate_pairs(q, rot_dims, rot_base, start), rotate_pairs(k, rot_dims, rot_base, start)
    o = sigmoid_attention(q, k, v, scale, p["temp"], p["pb"])
    return lin(o.reshape(T, heads * dim), p["o"])


def route(h, router, correction, top, n_groups, keep, scale):
    """Returns the chosen experts [T, top] and their weights [T, top]."""
    s = torch.sigmoid(lin(h, router))
    c = s + correction
    T, E = c.shape
    per = E // n_groups
    grouped = c.reshape(T, n_groups, per)
    gscore = grouped.topk(min(2, per), dim=-1).values.sum(-1)
    best = gscore.topk(keep, dim=-1).indices
    allowed = torch.zeros(T, n_groups, dtype=torch.bool)
    allowed.scatter_(1, best, True)
    c = c.masked_fill(~allowed.repeat_interleave(per, dim=1), -math.inf)
    idx = c.topk(top, dim=-1).indices
    w = s.gather(1, idx)
    return idx, w / (w.sum(-1, keepdim=True) + 1e-20) * scale


def route_margins(h, router, correction, top, n_groups, keep):
    """Per token, how far the choice is from going another way: the smaller of (the last kept group's score minus the
    first dropped group's) and (the last chosen expert's choice score minus the first unchosen allowed one's)."""
    c = torch.sigmoid(lin(h, router)) + correction
    T, E = c.shape
    per = E // n_groups
    out = torch.full((T,), math.inf, dtype=h.dtype)
    gscore = c.reshape(T, n_groups, per).topk(min(2, per), dim=-1).values.sum(-1)
    order = gscore.sort(dim=-1, descending=True)
    if keep < n_groups:
        out = torch.minimum(out, order.values[:, keep - 1] - order.values[:, keep])
    allowed = torch.zeros(T, n_groups, dtype=torch.bool)
    allowed.scatter_(1, order.indices[:, :keep], True)
    c = c.masked_fill(~allowed.repeat_interleave(per, dim=1), -math.inf).sort(dim=-1, descending=True).values
    if top < keep * per:
        out = torch.minimum(out, c[:, top - 1] - c[:, top])
    return out


def routed_experts(h, p, n_experts, top, n_groups, keep, scale, margins=None):
    """p: router, correction, e<j>.up, e<j>.down."""
    idx, w = route(h, p["router"], p["correction"], top, n_groups, keep, scale)
    if margins is not None:
        margins.append(route_margins(h, p["router"], p["correction"], top, n_groups, keep))
    out = torch.zeros(h.shape[0], p["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            out[t] += w[t, j] * lin(gelu_erf(lin(h[t], p[f"e{e}.up"])), p[f"e{e}.down"])
    return out


def side_input(x, tokens, table, layer, dim, p, eps):
    """p: gate, proj, norm.  ``table`` holds every layer's ``dim`` values of a token side by side."""
    e = table[torch.as_tensor(tokens)][:, layer * dim:(layer + 1) * dim]
    y = lin(gelu_tanh(lin(x, p["gate"])) * e, p["proj"])
    return x + group_norm(y, p["norm"], eps)


def sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def run_mixer(layer, h, p, eps, start=0):
    m = layer["mixer"]
    if layer["type"] == "gla":
        return gla_mixer(h, p, m["heads"], m["dim"], m["vdim"], m["tau"], eps)
    if layer["type"] == "retention":
        return retention_mixer(h, p, m["heads"], m["dim"], m["vdim"], m["decay"], m["rot"]["dims"], m["rot"]["base"],
                               eps, start)
    if layer["type"] == "attention":
        return attention_mixer(h, p, m["heads"], m["kv_heads"], m["dim"], m["scale"], m["rot"]["dims"],
                               m["rot"]["base"], eps, start)
    raise ValueError(layer["type"])


def forward(config, weights, tokens, layers_out=None, margins=None):
    """Logits [T, vocab] of one sequence; ``weights`` {name: float64 tensor}.  ``layers_out`` (a list) receives the
    stream after every layer, ``margins`` (a list) every router's per-token margins."""
    eps, groups, a = config["norm"]["eps"], config["norm"]["groups"], config["postln_alpha"]
    x = weights["embed"][torch.as_tensor(tokens)]
    for i, layer in enumerate(config["layers"]):
        pre = f"l{i}."
        x = group_norm(a * x + run_mixer(layer, x, sub(weights, pre + "mix."), eps), weights[pre + "norm1"], eps, groups)
        ff = layer.get("mlp")
        if ff is not None:
            r = ff["router"]
            y = routed_experts(x, sub(weights, pre + "mlp."), r["experts"], r["top"], r["groups"]["count"],
                               r["groups"]["keep"], r["scale"], margins)
            x = group_norm(a * x + y, weights[pre + "norm2"], eps, groups)
        if config.get("token_side") is not None:
            x = side_input(x, tokens, weights["side.embed"], i, config["token_side"]["dim"], sub(weights, pre + "side."), eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return lin(group_norm(x, weights["final.norm"], eps, groups), weights["head"])
