"""The Bibalix decoder on the GPU against the plain implementation in ``plain_bibalix`` (float64, whole sequences, no
cache): every mechanism's kernels alone, then small random models of several shapes (``bibalix_models``) through trace
replay in four cuttings and both precisions with pools that hold exactly what a trace needs, the stream layer by
layer, long decoding, and greedy generation through the engine's entry point and scheduler."""

import numpy as np
import pytest
import torch

import bibalix_models as bm
import cuttings
import plain_bibalix as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
F64 = torch.float64


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def rel_err(got, want):
    want = np.asarray(want, dtype=np.float64)
    return float(np.abs(np.asarray(got, dtype=np.float64) - want).max() / max(np.abs(want).max(), 1e-30))


def row_err(got, want):
    """The largest error of a row relative to that row's largest value."""
    want = np.asarray(want, dtype=np.float64)
    d = np.abs(np.asarray(got, dtype=np.float64) - want).max(axis=1)
    return float((d / np.maximum(np.abs(want).max(axis=1), 1e-30)).max())


@pytest.fixture(scope="module")
def ops():
    from tokasaurus_b200.kernels import ops as o
    return o


def paged(n_tokens, page, seed):
    """A block table of scattered pages for one request."""
    n_pages = -(-n_tokens // page)
    perm = np.random.default_rng(seed).permutation(n_pages + 5)[:n_pages]
    return [int(p) for p in perm], n_pages + 5


# ------------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,dim,rot,dims,scaling", [(3, 16, 8, 8, (2.0, 16, 4.0, 1.0)), (2, 12, 6, 4, None),
                                                        (5, 8, 24, 24, (8.0, 32, 8.0, 2.0)), (1, 32, 64, 32, (3.0, 256, 16.0, 1.0))])
def test_rotation_in_halves_with_blended_frequencies(ops, dtype, heads, dim, rot, dims, scaling):
    """The rotated share of every query head, at positions into the thousands: channel i with channel i + dims / 2,
    frequencies blended between scaled and unscaled, sine and cosine times the scheme's factor."""
    from tokasaurus_b200.parts import RotaryEncoding

    rd = dict(dims=dims, base=700.0)
    enc = RotaryEncoding(dims, 700.0)
    if scaling is not None:
        rd["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
        enc = RotaryEncoding(dims, 700.0, "yarn", factor=scaling[0], original_max_position_embeddings=scaling[1],
                             yarn_fast=scaling[2], yarn_slow=scaling[3])
    f, mag = plain.rotary_frequencies(rd, dims)
    assert float((enc.inv_freq64() - f).abs().max()) == 0.0 and abs(enc.magnitude() - mag) < 1e-15
    pos = [0, 1, 2, 77, 500, 4097, 30011]
    g = torch.Generator().manual_seed(dims)
    x = torch.randn(len(pos), heads, dim + rot, generator=g).to(DT[dtype])
    want = torch.cat([x.double()[:, :, :dim], plain.rotate_halves(x.double()[:, :, dim:], torch.tensor(pos), f, mag, dims)], -1)
    xd = x.to(DEV).view(len(pos), heads * (dim + rot)).clone()
    ops.rotate_pairs(xd, heads, dim + rot, dim, rot, dims, None, i32(pos), i32([0] * len(pos)), 24,
                     freq64=enc.inv_freq64().to(DEV), halves=True, mag=enc.magnitude())
    assert rel_err(xd.float().cpu().view(want.shape), want) < (2e-6 if dtype == "float32" else 8e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_latent_rows_normed_rotated_and_cached(ops, dtype):
    """The cached row of a token: the normed latent and the shared key part rotated in halves on part of its channels,
    at scattered pages; the gate's logits ride in the same rows of the product and are left alone."""
    from tokasaurus_b200.parts import RotaryEncoding

    rank, rot, dims, page, n, eps = 20, 10, 6, 8, 45, 1e-5
    enc = RotaryEncoding(dims, 50.0, "yarn", factor=3.0, original_max_position_embeddings=8, yarn_fast=2.0, yarn_slow=0.5)
    g = torch.Generator().manual_seed(3)
    proj = torch.randn(n, rank + rot + 4, generator=g)
    w = torch.rand(rank, generator=g) + 0.5
    table, n_pages = paged(n, page, 1)
    cache = torch.full((n_pages, 1, page, rank + rot), float("nan"), dtype=DT[dtype], device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.latent_prep(proj.to(DEV), 0, 0, None, None, 0, rank, rot, dims, w.to(DEV), None, cache, i32(list(range(n))),
                    i32([0] * n), i32([0, len(table)]), i32(table), page, eps, status, DT[dtype],
                    freq64=enc.inv_freq64().to(DEV), halves=True, mag=enc.magnitude())
    assert int(status.item()) == 0
    c = plain.rms(proj[:, :rank].double(), eps) * w.double()
    kr = plain.rotate_halves(proj[:, rank:rank + rot].double(), torch.arange(n), enc.inv_freq64(), enc.magnitude(), dims)
    rows = torch.stack([cache[table[t // page], 0, t % page] for t in range(n)]).float().cpu()
    assert rel_err(rows, torch.cat([c, kr], -1)) < (2e-6 if dtype == "float32" else 8e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_output_gate_a_head(ops, dtype):
    heads, vdim, T = 5, 12, 9
    g = torch.Generator().manual_seed(5)
    val = torch.randn(4, heads * vdim, generator=g).to(DT[dtype])
    gate = torch.randn(T, 7 + heads, generator=g) * 2
    rows = [8, 0, 3, 3]
    want = val.double().view(4, heads, vdim) * torch.sigmoid(gate[rows, 7:].double())[:, :, None]
    vd = val.to(DEV).clone()
    ops.head_sigmoid_gate(vd, gate.to(DEV), 7, i32(rows), heads, vdim, 24)
    assert rel_err(vd.float().cpu().view(want.shape), want) < (1e-6 if dtype == "float32" else 8e-3)
    vd = val.to(DEV).clone()
    ops.head_sigmoid_gate(vd, gate.to(DEV)[:4], 7, None, heads, vdim, 24)
    want = val.double().view(4, heads, vdim) * torch.sigmoid(gate[:4, 7:].double())[:, :, None]
    assert rel_err(vd.float().cpu().view(want.shape), want) < (1e-6 if dtype == "float32" else 8e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("inner,interleave", [(24, 0), (40, 8), (7, 0)])
def test_gate_through_the_tanh_form_of_gelu(ops, dtype, inner, interleave):
    g = torch.Generator().manual_seed(inner)
    gate, up = (torch.randn(13, inner, generator=g) * 3).to(DT[dtype]), torch.randn(13, inner, generator=g).to(DT[dtype])
    gu = ops.interleave_gate_up(gate.t().contiguous(), up.t().contiguous()).t().contiguous() if interleave else torch.cat([gate, up], 1)
    out = torch.empty(13, inner, dtype=DT[dtype], device=DEV)
    ops.silu_mul(gu.to(DEV).contiguous(), out, interleave, act="gelu_tanh")
    want = plain.gelu_tanh(gate.double()) * up.double()
    assert rel_err(out.float().cpu(), want) < (1e-6 if dtype == "float32" else 8e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,E,top,H,inner,shared", [(3, 4, 2, 64, 40, 24), (5, 6, 1, 96, 32, None), (70, 8, 4, 128, 64, 64),
                                                    (400, 5, 5, 96, 72, 40), (150, 3, 2, 128, 64, None)])
def test_clamped_experts_weighed_by_the_softmax_over_all(ops, dtype, T, E, top, H, inner, shared):
    """The routed feed-forward as a part: the chosen experts' shares of the softmax over ALL experts times a number,
    clamped gated units (few rows, tiled, and in bfloat16 the grouped tensor-core products), and a shared expert that
    counts sigmoid(sg . h) times."""
    from tokasaurus_b200.engine.runtime import Runtime
    from tokasaurus_b200.parts import ClampedGLU, RoutedExperts

    g = torch.Generator().manual_seed(T + E)
    limit, slimit, scale = 0.9, 0.6, 1.7
    w = {"r": torch.randn(E, H, generator=g) * 0.3, "sg": torch.randn(1, H, generator=g) * 0.3}
    for e in range(E):
        w[f"e{e}.gate"], w[f"e{e}.up"] = torch.randn(inner, H, generator=g) * 0.15, torch.randn(inner, H, generator=g) * 0.15
        w[f"e{e}.down"] = torch.randn(H, inner, generator=g) * 0.15
    mlp = dict(kind="moe", expert=dict(ff=inner, limit=limit), router=dict(experts=E, top=top, scale=scale))
    sh = None
    if shared is not None:
        w["shared.gate"], w["shared.up"] = torch.randn(shared, H, generator=g) * 0.2, torch.randn(shared, H, generator=g) * 0.2
        w["shared.down"] = torch.randn(H, shared, generator=g) * 0.2
        w["shared.sg"] = w["sg"]
        mlp["shared"] = dict(ff=shared, limit=slimit)
        sh = ClampedGLU(H, shared, slimit, "shared.gate", "shared.up", "shared.down")
    w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    w["router"] = w["r"]
    h = torch.randn(T, H, generator=g).to(DT[dtype])
    part = RoutedExperts(H, inner, E, top, "router", None, lambda e: (f"e{e}.gate", f"e{e}.up", f"e{e}.down"), sh,
                         expert="clamped", clamp=(limit, 1.702), over_all=dict(scale=scale),
                         shared_gate_name="shared.sg" if sh is not None else None)
    rt = Runtime.make(DEV, dtype)
    dev = {k: (v.to(DEV) if k in ("router", "shared.sg") else v.to(DEV, DT[dtype])) for k, v in w.items()}
    part.bind(dev, rt)
    got = part.forward(None, h.to(DEV)).float().cpu()
    w64 = {k: v.double() for k, v in w.items()}
    idx, wt, s = plain.route(h.double(), w64["router"], top, scale)
    srt = torch.sort(h.double() @ w64["router"].T, dim=-1, descending=True).values
    assert top == E or float((srt[:, top - 1] - srt[:, top]).min()) > 2e-5  # no choice rests on a close call
    assert float(wt.sum(-1).max()) <= scale + 1e-9 and (top == E or float(wt.sum(-1).min()) < 0.99 * scale)  # not renormalised
    want = plain.moe_ff(h.double(), w64, "", mlp)
    assert rel_err(got, want) < (3e-5 if dtype == "float32" else 3e-2)


def two_map_attention(raw, bias, nw, heads, kv, dim, vdim, scale, window, keep, rot, base, lam, eps, mult, gate):
    """The differential form from raw projections [n, q | k | v], with plain's building blocks."""
    n = raw.shape[0]
    x = raw.double() + bias.double()
    q = (plain.rms(x[:, :heads * 2 * dim].reshape(n, heads, 2, dim), eps) * nw[0].double())
    k = (plain.rms(x[:, heads * 2 * dim:(heads + kv) * 2 * dim].reshape(n, kv, 2, dim), eps) * nw[1].double())
    v = x[:, (heads + kv) * 2 * dim:].reshape(n, kv, vdim)
    if rot:
        f, mag = plain.rotary_frequencies(dict(base=base, dims=rot), rot)
        q, k = plain.rotate_halves(q, torch.arange(n), f, mag, rot), plain.rotate_halves(k, torch.arange(n), f, mag, rot)
    rep = heads // kv
    kx, vx = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    mask = plain.visible(n, window, keep)
    a0 = plain.softmax_attention(q[:, :, 0], kx[:, :, 0], vx, scale, mask)
    a1 = plain.softmax_attention(q[:, :, 1], kx[:, :, 1], vx, scale, mask)
    o = plain.rms(a0 - lam * a1, eps) * mult * torch.sigmoid(gate.double())[:, :, None]
    return o.reshape(n, heads * vdim)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim,vdim,rot,page,heads,kv,window,keep", [
    (16, 32, 8, 16, 4, 2, 37, 3), (32, 64, 32, 16, 8, 1, 45, 70), (24, 40, 24, 8, 2, 2, 50, 9), (64, 16, 32, 16, 2, 2, 16, 1),
    (48, 80, 48, 16, 20, 1, 130, 5), (16, 16, 0, 8, 3, 3, 64, 64), (32, 32, 16, 16, 2, 1, None, 0)])
def test_differential_attention_at_the_window_and_at_the_kept_positions(ops, dtype, dim, vdim, rot, page, heads, kv, window, keep):
    """Two maps a head over the same values, a window that keeps the first positions in sight.  Made-up keys that
    made-up queries score far above all others stand (a) a window back from two neighbouring queries, of which one
    sees it and one does not, at a page's first and last slot, and (b) at the last kept position and at the first one
    that is not kept, asked for from far away.  In one piece, in portions and token by token, on the FP32 pipes and (in
    bfloat16, for sizes they take) on the tensor cores beside a second request of one token."""
    n, eps, lam, mult, base = 330, 1e-6, 0.7, 0.6, 1000.0
    scale = 24.0 / dim  # scores of aligned pairs stand out: q and k are normed to a mean square of 1
    g = torch.Generator().manual_seed(dim + page + heads)
    nw = torch.rand(2, dim, generator=g) * 0.4 + 0.8
    bias = torch.randn((heads + kv) * 2 * dim + kv * vdim, generator=g) * 0.1
    C = bias.numel()
    freq = None
    if rot:
        from tokasaurus_b200.parts import RotaryEncoding
        freq = RotaryEncoding(rot, base).inv_freq64().to(DEV)
    for far_at in (page * 2, page * 3 - 1):
        raw = torch.randn(n, C + heads, generator=g)  # the gate's logits ride behind q | k | v
        raw[:, C:] *= 2
        u = torch.randn(dim, generator=g).sign() * 5
        u[:rot] = 0 if rot < dim else u[:rot]  # aligned on the channels that are not rotated, where there are some

        def put(qs, key, m):
            for r in qs:
                raw[r, :heads * 2 * dim].view(heads, 2, dim)[:, m] = u - bias[:heads * 2 * dim].view(heads, 2, dim)[:, m]
            raw[key, heads * 2 * dim:(heads + kv) * 2 * dim].view(kv, 2, dim)[:, m] = \
                u - bias[heads * 2 * dim:(heads + kv) * 2 * dim].view(kv, 2, dim)[:, m]

        if window is not None:
            put([far_at + window - 1, far_at + window], far_at, 0)       # the first sees it, the second does not
            if keep and keep < far_at:
                put([n - 1, n - 7], keep - 1, 1)                             # the last kept position, in the other map
                raw[keep, heads * 2 * dim:(heads + kv) * 2 * dim].view(kv, 2, dim)[:, 1] = \
                    raw[keep - 1, heads * 2 * dim:(heads + kv) * 2 * dim].view(kv, 2, dim)[:, 1]  # and the first that is not
        else:
            put([n - 1, n - 2], far_at, 0)
        args = (bias, nw, heads, kv, dim, vdim, scale, window, keep, rot, base, lam, eps, mult, raw[:, C:])
        want = two_map_attention(raw[:, :C], *args)
        if window is not None and rot < dim and far_at >= keep:
            # what the comparison below would miss if the kernels were off by one: the plain result moves a lot
            for w2, k2, rows in [(window + 1, keep, [far_at + window])] + ([(window, keep - 1, [n - 1])] if keep else []):
                other = two_map_attention(raw[:, :C], bias, nw, heads, kv, dim, vdim, scale, w2, k2, rot, base, lam, eps, mult, raw[:, C:])
                assert float((other[rows] - want[rows]).abs().max()) > 0.2 * float(want[rows].abs().max()), (w2, k2)
        table, n_pages = paged(n, page, far_at + 1)
        lam_d = torch.tensor([lam], dtype=torch.float32, device=DEV)
        cuts = ([n], [n - 5, 3, 1, 1], [far_at + 1, (window or 40) - 2, 2, 1, n - far_at - (window or 40) - 2])
        for cut in cuts:
            cache = torch.full((n_pages, kv, page, 2 * dim + vdim), float("nan"), dtype=DT[dtype], device=DEV)
            status = torch.zeros(1, dtype=torch.int32, device=DEV)
            got, at = [], 0
            for m in cut:
                pos = list(range(at, at + m))
                rd = raw[at:at + m].to(DEV)
                qd = torch.empty(m, heads * 2 * dim, dtype=DT[dtype], device=DEV)
                need = -(-(at + m) // page)
                ops.sink_attn_prep(rd, bias.to(DEV), True, eps, qd, cache, i32(pos), i32([0] * m), i32([0, need]),
                                   i32(table[:need]), heads, kv, dim, vdim, page, True, status, norm_w=nw.to(DEV),
                                   rot_freq=freq, rot_dims=rot, rot_pairs=False, maps=2)
                a = torch.empty(m, heads * 2 * vdim, dtype=torch.float32, device=DEV)
                ops.attn_sink(qd, a, cache, i32([0] * m), i32(pos), i32([0, need]), i32(table[:need]), None, m, None, heads,
                              kv, dim, vdim, page, scale, None, window, status, maps=2, keep_first=keep)
                out = torch.empty(m, heads * vdim, dtype=DT[dtype], device=DEV)
                ops.diff_combine(a, lam_d, eps, mult, rd, C, None, out, heads, dim, vdim)
                got.append(out.float().cpu())
                if ops.can_use_attn_sink_tc(DT[dtype], dim, vdim):
                    if at == 0:
                        q_first, gate_first = qd[:1].clone(), rd[:1].clone()
                    a2 = torch.full((m + 1, heads * 2 * vdim), float("nan"), dtype=torch.float32, device=DEV)
                    ops.attn_sink_tc(torch.cat([qd, q_first]), a2, cache, i32([0, m]), i32([m, 1]), i32([at + m, 1]),
                                     i32([0, need, need + 1]), i32(table[:need] + table[:1]), 2, None, heads, kv, dim, vdim, page,
                                     scale, None, window, status, portions=m > 1, maps=2, keep_first=keep)
                    out2 = torch.empty(m + 1, heads * vdim, dtype=DT[dtype], device=DEV)
                    ops.diff_combine(a2, lam_d, eps, mult, torch.cat([rd, gate_first]), C, None, out2, heads, dim, vdim)
                    assert row_err(out2[:m].float().cpu(), want[at:at + m]) < 6e-2, ("tensor cores", far_at, cut[:2], at)
                    assert row_err(out2[m:].float().cpu(), want[:1]) < 6e-2
                at += m
            assert at == n and int(status.item()) == 0
            assert row_err(torch.cat(got), want) < (1e-4 if dtype == "float32" else 6e-2), (far_at, cut[:2])


def test_single_tokens_over_several_blocks_with_kept_positions(ops):
    """Three requests that bring one token each at contexts of 300, 70 and 1: a request's kept positions and its window
    are tiles that several blocks share out, whose softmax shares are merged afterwards."""
    dim, vdim, heads, kv, page, window, keep, scale, eps = 32, 48, 6, 2, 16, 150, 20, 0.3, 1e-6
    g = torch.Generator().manual_seed(9)
    lens = [300, 70, 1]
    n_pages = sum(-(-n // page) for n in lens)
    C = (heads + kv) * 2 * dim + kv * vdim
    cache = torch.full((n_pages, kv, page, 2 * dim + vdim), float("nan"), dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    perm = [int(x) for x in np.random.default_rng(3).permutation(n_pages)]
    nw = torch.ones(2, dim)
    tables, want, last_q, last_raw = [], [], [], []
    for n in lens:
        raw = torch.randn(n, C + heads, generator=g)
        table, perm = perm[:-(-n // page)], perm[-(-n // page):]
        tables.append(table)
        qd = torch.empty(n, heads * 2 * dim, dtype=torch.bfloat16, device=DEV)
        ops.sink_attn_prep(raw.to(DEV), None, True, eps, qd, cache, i32(list(range(n))), i32([0] * n), i32([0, len(table)]),
                           i32(table), heads, kv, dim, vdim, page, True, status, maps=2)
        last_q.append(qd[-1:])
        last_raw.append(raw[-1:])
        want.append(two_map_attention(raw[:, :C], torch.zeros(C), nw, heads, kv, dim, vdim, scale, window, keep, 0, 1.0, 0.4,
                                      eps, 0.5, raw[:, C:])[-1])
    indptr = [0] + [int(x) for x in np.cumsum([len(t) for t in tables])]
    a = torch.full((3, heads * 2 * vdim), float("nan"), dtype=torch.float32, device=DEV)
    ops.attn_sink_tc(torch.cat(last_q), a, cache, i32([0, 1, 2]), i32([1, 1, 1]), i32(lens), i32(indptr), i32(sum(tables, [])),
                     3, None, heads, kv, dim, vdim, page, scale, None, window, status, portions=False, maps=2, keep_first=keep)
    out = torch.empty(3, heads * vdim, dtype=torch.bfloat16, device=DEV)
    ops.diff_combine(a, torch.tensor([0.4], device=DEV), eps, 0.5, torch.cat(last_raw).to(DEV), C, None, out, heads, dim, vdim)
    assert int(status.item()) == 0
    assert row_err(out.float().cpu(), torch.stack(want)) < 5e-2


# ------------------------------------------------------------------------------------------------ whole models
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    return bm.make_models(tmp_path_factory.mktemp("bibalix_models"))


CUTS = dict(whole=cuttings.whole, prefix_then_single=cuttings.prefix_then_single,
            changing_portions=cuttings.changing_portions, mixed=cuttings.mixed)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cut", list(CUTS))
@pytest.mark.parametrize("which", list(bm.MODELS))
def test_cuttings_match_plain(models, which, cut, dtype):
    """Whole prompts, prompts then single tokens, portions of changing size down to one and two tokens, and up to four
    requests side by side in four slots, in a pool that holds exactly what the trace needs: pages are used again (those
    behind a window within a request's own life, too, while the pages of kept first positions stay), and a later
    request must see nothing of an earlier one's keys."""
    from tokasaurus_b200.engine.trace import TraceReplayer

    m = models[(which, bm.variant(dtype))]
    steps = CUTS[cut](m["reqs"])
    rp = TraceReplayer(str(m["folder"]), dtype, cuttings.max_live_tokens(steps, m["page"]), page_size=m["page"], max_requests=4)
    cache = rp.runner.cache
    owners, outs = {}, []
    for st in steps:
        outs.append(rp.run_step(st))
        cache.check()
        for rid, rc in cache.requests.items():
            for gi in range(len(cache.groups)):
                for p in rc.live_pages(gi):
                    owners.setdefault((gi, p), set()).add(rid)
                kept = cache.kept_pages(gi)
                assert all(p >= 0 for p in rc.tables[gi][:kept]), "a page of kept first positions was given back"
    assert not cache.requests and cache.num_free_pages() == [g.allocator.num_pages for g in cache.groups]
    bm.check_logits(cuttings.collect(steps, outs), m, dtype, cut)
    if cut == "mixed":
        assert any(len(v) > 1 for v in owners.values()), "no page was used by two requests"


def test_layer_by_layer(models):
    """The residual stream after every layer, float32, one prompt in one step and in two."""
    from tokasaurus_b200.engine.batch import StepEntry
    from tokasaurus_b200.engine.trace import TraceReplayer

    for which in bm.MODELS:
        m = models[(which, "dyn")]
        rid, toks = next(iter(m["reqs"].items()))
        want = []
        plain.forward(m["config"], m["weights"], toks, layers_out=want)
        for cut in ([len(toks)], [len(toks) - 7, 7]):
            rp = TraceReplayer(str(m["folder"]), "float32", 512, page_size=m["page"], max_requests=2)
            rp.runner.cache.admit(rid)
            got, at = [], 0
            for n in cut:
                rp.runner.cache.ensure_capacity(rid, at + n)
                part = []
                rp.runner.step([StepEntry(rid, toks[at:at + n], at, list(range(n)))], layer_outputs=part)
                got.append(part)
                at += n
            assert len(got[0]) == len(want)
            for i, b in enumerate(want):
                a = torch.cat([part[i].cpu() for part in got])
                assert rel_err(a, b) < 1e-4, (which, i, cut)


def test_every_constant_shows_in_the_logits(models):
    """The comparisons above would not notice a lost constant if it carried no weight: on the plain implementation,
    changing each moves the logits by many times the tolerance of the float32 comparisons."""
    for which, paths in (("a", ["scale", "diff", "mask.size", "mask.keep_first", "rot.dims", "rot.base", "rot.scaling.factor",
                                "rot.scaling.original", "router.scale", "router.top", "expert.limit", "shared.limit"]),
                         ("b", ["mask.size", "mask.keep_first"]), ("d", ["mask.size", "rot.scaling.fast", "rot.scaling.slow"])):
        m = models[(which, "dyn")]
        rid, toks = max(m["reqs"].items(), key=lambda kv: len(kv[1]))
        ref = m["want"][rid]
        tol = 3 * float(m["noise"][rid].max())

        def moved(config, weights=None):
            return float(bm.row_error(plain.forward(config, weights or m["weights"], toks).numpy() - ref).max())

        step = {"scale": lambda s: s * 1.1, "diff": lambda d: d + 0.05, "mask.size": lambda s: s + 1,
                "mask.keep_first": lambda k: k - 1, "rot.dims": lambda d: d - 2, "rot.base": lambda b: b * 2,
                "rot.scaling.factor": lambda f: f * 1.5, "rot.scaling.original": lambda o: o * 2,
                "rot.scaling.fast": lambda f: f / 4, "rot.scaling.slow": lambda s: s * 4, "router.scale": lambda s: s * 1.1,
                "router.top": lambda t: t + 1, "expert.limit": lambda l: l * 0.5, "shared.limit": lambda l: l * 0.5}
        for path in paths:
            assert moved(bm.changed(m["config"], path, step[path])) > 30 * tol, (which, path)
        assert moved(dict(m["config"], norm=dict(eps=1e-2))) > 30 * tol
        if which == "a":
            for name, f in (("l1.mix.lq1", lambda t: t * 1.3), ("l1.mix.lk2", lambda t: t * 1.3), ("l1.mix.g", lambda t: t * 0),
                            ("l0.mix.g", lambda t: t * 0), ("l1.mix.q.norm", lambda t: t * 0 + 1), ("l1.mix.k.b", lambda t: t * 0),
                            ("l0.mix.dkv.norm", lambda t: t * 0 + 1), ("l0.mlp.shared.sg", lambda t: t * 0), ("l1.norm1.b", lambda t: t * 0),
                            ("final.norm.b", lambda t: t * 0)):
                w = dict(m["weights"])
                w[name] = f(w[name].clone())
                assert moved(m["config"], w) > 30 * tol, name


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(models, dtype):
    """A short prompt, then 150 tokens one by one: decoded keys fill page after page, windows pass over decoded tokens
    and pages behind them come back while the kept first ones stay."""
    from tokasaurus_b200.engine.trace import TraceReplayer

    for which in bm.MODELS:
        m = models[(which, bm.variant(dtype))]
        toks = cuttings.random_tokens(160, m["config"]["vocab"], 7)
        mg, want = bm.router_margins(m["config"], m["weights"], toks)
        assert mg > (bm.MIN_MARGIN if dtype == "float32" else bm.TIER_MARGIN)
        want = want.numpy()
        steps = cuttings.prefix_then_single({"long": toks}, tail=150)
        rp = TraceReplayer(str(m["folder"]), dtype, cuttings.max_live_tokens(steps, m["page"]), page_size=m["page"], max_requests=4)
        got = cuttings.collect(steps, [rp.run_step(st) for st in steps])
        noise = bm.rounding_noise(m["config"], m["weights"], toks, want, dtype)
        bm.check_logits(got, dict(want={"long": want}, noise={"long": noise}), dtype, "long decoding")


def plain_greedy(m, prompt, n):
    ids, out = list(prompt), []
    for _ in range(n):
        out.append(int(plain.forward(m["config"], m["weights"], ids)[-1].argmax()))
        ids.append(out[-1])
    return out


@pytest.mark.parametrize("which", ["a", "c", "d"])
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_entry_point(models, graphs, which):
    """Greedy generation in float32 through ``Engine.generate``: the scheduler admits, cuts prompts into portions,
    decodes (from CUDA graphs or kernel by kernel) and frees; five requests in three slots, so slots and pages are
    handed on; prompts longer than the windows, so pages come back while a request runs."""
    from tokasaurus_b200.engine.engine import Engine

    m = models[(which, "tier")]
    V = m["config"]["vocab"]
    prompts = [cuttings.random_tokens(n, V, 300 + n) for n in (30, 3, 61, 17, 9)]
    n_new = 10
    want = [plain_greedy(m, p, n_new) for p in prompts]
    eng = Engine(model=str(m["folder"]), dtype="float32", page_size=m["page"], kv_cache_num_tokens=512,
                 max_tokens_per_forward=24, max_seqs_per_forward=3, allocator_sanity_checks=True, use_cudagraphs=graphs)
    outs = eng.generate(prompts, max_num_tokens=n_new, ignore_eos=True)
    assert [o.completion_ids for o in outs] == want
    cache = eng.runner.cache
    assert not cache.requests and cache.num_free_pages() == [g.allocator.num_pages for g in cache.groups]


@pytest.mark.parametrize("which", ["a", "b"])
def test_bfloat16_generation_from_graphs_equals_kernel_by_kernel(models, which):
    """The serving precision: decode steps replayed from CUDA graphs choose the tokens that the same steps choose kernel by
    kernel (the same kernels on the same data), and every chosen token is near the plain statement's best at its place."""
    from tokasaurus_b200.engine.engine import Engine

    m = models[(which, "tier")]
    V = m["config"]["vocab"]
    prompts = [cuttings.random_tokens(n, V, 500 + n) for n in (70, 5, 33, 120)]
    got = []
    for graphs in (False, True):
        eng = Engine(model=str(m["folder"]), dtype="bfloat16", page_size=m["page"], kv_cache_num_tokens=1024,
                     max_tokens_per_forward=64, max_seqs_per_forward=4, allocator_sanity_checks=True, use_cudagraphs=graphs)
        got.append([o.completion_ids for o in eng.generate(prompts, max_num_tokens=12, ignore_eos=True)])
        del eng
    assert got[0] == got[1]
    for p, ids in zip(prompts, got[0]):
        logits = plain.forward(m["config"], m["weights"], p + ids[:-1])[len(p) - 1:]
        top = float(logits.abs().max())
        for i, t in enumerate(ids):
            assert float(logits[i, t]) >= float(logits[i].max()) - 0.05 * top, (which, i)


def test_command_line_generates(models, tmp_path):
    """``toka model=<folder>`` picks the model class from config.json and generates."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    m = models[("b", "tier")]
    prompt = cuttings.random_tokens(12, m["config"]["vocab"], 1)
    toka = Path(__file__).resolve().parent.parent / "bin" / "toka"
    r = subprocess.run([sys.executable, str(toka), f"model={m['folder']}", "dtype=float32", "page_size=16",
                        "kv_cache_num_tokens=256", "max_num_tokens=6", "ignore_eos=T", f"prompt_ids={json.dumps(prompt)}"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    want = plain_greedy(m, prompt, 6)
    assert json.loads(r.stdout.strip().splitlines()[-1])["completion_ids"] == want
