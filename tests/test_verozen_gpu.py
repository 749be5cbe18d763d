"""The Verozen decoder on the GPU against the plain implementation in ``plain_verozen`` (float64, whole sequences, no
cache): every mechanism's kernels alone, then small random models of several shapes (``verozen_models``) through trace
replay in four cuttings and both precisions with pools that hold exactly what a trace needs, the stream layer by
layer, long decoding, and greedy generation through the engine's entry point and scheduler."""

import numpy as np
import pytest
import torch

import cuttings
import plain_verozen as plain
import verozen_models as vm

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-5, "bfloat16": 2.5e-2}
F64 = torch.float64


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def rel_err(got, want):
    want = np.asarray(want, dtype=np.float64)
    return float(np.abs(np.asarray(got, dtype=np.float64) - want).max() / max(np.abs(want).max(), 1e-30))


def row_err(got, want):
    """The largest error of a row relative to that row's largest value (rows of very different sizes)."""
    want = np.asarray(want, dtype=np.float64)
    d = np.abs(np.asarray(got, dtype=np.float64) - want).max(axis=1)
    return float((d / np.maximum(np.abs(want).max(axis=1), 1e-30)).max())


@pytest.fixture(scope="module")
def ops():
    from tokasaurus_b200.kernels import ops as o
    return o


def walk_defines(ops, dim, vdim):
    return ops.decay_recurrence_defines(dim, vdim)


# ------------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,groups", [(24, 1), (96, 3), (200, 5), (1056, 2)])
def test_norm_after_the_sum_in_parts(ops, dtype, H, groups):
    """x = w * N_g(a x + y) for y as float32 rows, as slices of a split product, in the activation type, and absent."""
    g = torch.Generator().manual_seed(H)
    x, w = torch.randn(5, H, generator=g) * 3, torch.rand(H, generator=g) + 0.5
    x[:, :H // groups] *= 7  # the parts' sizes differ: one norm over the whole row would show
    sl = torch.randn(3, 5, H, generator=g)
    for a, y in ((2.5, sl[0]), (1.0, sl), (0.7, sl[1].to(DT[dtype])), (1.3, None)):
        ysum = 0 if y is None else (y.double().sum(0) if y.dim() == 3 else y.double())
        want = plain.group_norm(a * x.double() + ysum, w.double(), 1e-6, groups)
        xd = x.to(DEV)
        h = torch.empty(5, H, dtype=DT[dtype], device=DEV) if dtype == "bfloat16" else None
        ops.sum_group_norm(xd, None if y is None else y.to(DEV), a, w.to(DEV), 1e-6, groups, h)
        assert rel_err(xd.cpu(), want) < 2e-6
        if h is not None:
            assert rel_err(h.float().cpu(), want) < TOL[dtype]
    if groups > 1:
        assert rel_err(plain.group_norm(x.double(), w.double(), 1e-6, 1), plain.group_norm(x.double(), w.double(), 1e-6, groups)) > 0.1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gate_times_a_slice_of_the_side_table(ops, dtype):
    """gelu_tanh(z) * table[token][off : off + dim] for tokens given by id, by the request's last sampled token (id < 0),
    and for a cut-down set of rows."""
    g = torch.Generator().manual_seed(2)
    V, dim, layers = 37, 12, 3
    table = torch.randn(V, layers * dim, generator=g).to(DT[dtype])
    ids = [5, 36, -1, 0, 17, -1]
    token_seq, seq_slot, last = [0, 0, 1, 2, 2, 3], [2, 0, 3, 1], [11, 22, 33, 7]
    real = [5, 36, last[seq_slot[1]], 0, 17, last[seq_slot[3]]]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for off_layer in (0, 2):
        for rows in (None, [4, 2, 5]):
            n = 6 if rows is None else len(rows)
            z = torch.randn(n, dim, generator=g) * 2
            out = torch.empty(n, dim, dtype=DT[dtype], device=DEV)
            ops.gelu_gate_rows(z.to(DEV), table.to(DEV), off_layer * dim, i32(ids), i32(token_seq), i32(seq_slot), i32(last),
                               None if rows is None else i32(rows), out, status)
            toks = real if rows is None else [real[r] for r in rows]
            want = plain.gelu_tanh(z.double()) * table.double()[toks][:, off_layer * dim:(off_layer + 1) * dim]
            assert rel_err(out.float().cpu(), want) < TOL[dtype]
    assert int(status.item()) == 0
    out = torch.empty(1, dim, dtype=DT[dtype], device=DEV)
    ops.gelu_gate_rows(torch.ones(1, dim, device=DEV), table.to(DEV), 0, i32([V]), i32([0]), i32([0]), i32([0]), None, out, status)
    assert int(status.item()) == 1 and float(out.float().abs().max()) == 0.0  # an id outside the table: flagged, zeros


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,vdim", [(3, 24), (1, 130), (6, 64)])
def test_head_norm_with_shared_weight_and_silu_gate(ops, dtype, heads, vdim):
    g = torch.Generator().manual_seed(heads + vdim)
    wide = torch.randn(7, 2 * heads * vdim + 5, generator=g)
    y, gate = wide[:, 2:2 + heads * vdim], wide[:, heads * vdim + 5:]
    y[:, :vdim] *= 9  # one head much larger: a norm over all heads together would show
    w = torch.rand(vdim, generator=g) + 0.5
    for weight in (w, None):
        n = plain.group_norm(y.double().reshape(7 * heads, vdim), None if weight is None else weight.double(), 1e-5)
        want = n.reshape(7, heads * vdim) * plain.silu(gate.double())
        out = torch.empty(7, heads * vdim, dtype=DT[dtype], device=DEV)
        wd = wide.to(DEV)
        ops.gated_group_norm(wd[:, 2:2 + heads * vdim], wd[:, heads * vdim + 5:], None if weight is None else weight.to(DEV),
                             out, heads, 1e-5, gate_first=False, silu_gate=True)
        assert rel_err(out.float().cpu(), want) < TOL[dtype]


@pytest.mark.parametrize("T", [21, 531])  # no multiples of the tokens a block takes
@pytest.mark.parametrize("C,rank,tau", [(48, 5, 8.0), (192, 16, 16.0), (72, 40, 1.0), (8, 1, 3.0), (300, 19, 4.0)])
def test_decays_of_gated_linear_attention(ops, C, rank, tau, T):
    """f = sigmoid(low A2^T + b)^(1 / tau) from the low-rank columns of the projections, also where the sigmoid is
    within rounding of 0 or 1; q scaled in place; the other columns untouched.  A token's decays do not depend on how
    many tokens the step brings."""
    g = torch.Generator().manual_seed(C)
    proj = torch.randn(T, C + 7 + rank, generator=g)
    proj[0, C + 7:] *= 40
    proj[1, C + 7:] *= -40
    a2, b = torch.randn(C, rank, generator=g), torch.randn(C, generator=g) * 2
    z = proj[:, C + 7:].double() @ a2.double().T + b.double()
    want = torch.exp(torch.nn.functional.logsigmoid(z) / tau)
    pd = proj.to(DEV)
    f = torch.empty(T, C, device=DEV)
    ops.gla_gates(pd, C + 7, rank, a2.t().contiguous().to(DEV), b.to(DEV), tau, f, 0, C, 0.37, walk_defines(ops, 16, 16))
    assert float(z.abs().max()) > 30
    # a float32 sum of terms whose sizes add up to S is off by a few units of 6e-8 S; f moves by df/dz times that
    spread = proj[:, C + 7:].double().abs() @ a2.double().abs().T + b.double().abs()
    slope = want * torch.sigmoid(-z) / tau
    assert bool(((f.cpu().double() - want).abs() <= 1e-6 + 2.5e-7 * spread * slope).all())
    assert rel_err(pd[:, :C].cpu(), proj[:, :C].double() * 0.37) < 1e-6
    assert float((pd[:, C:] - proj[:, C:].to(DEV)).abs().max()) == 0.0
    if T > 500:
        few = torch.empty(40, C, device=DEV)
        part = proj[T - 40:].to(DEV).contiguous()
        ops.gla_gates(part, C + 7, rank, a2.t().contiguous().to(DEV), b.to(DEV), tau, few, 0, C, 0.37, walk_defines(ops, 16, 16))
        assert torch.equal(few, f[T - 40:])


@pytest.mark.parametrize("heads,dim,rot,pairs", [(3, 16, 16, False), (2, 24, 8, False), (4, 32, 16, True), (1, 10, 10, True), (2, 12, 0, False)])
def test_rotation_in_halves_and_in_pairs(ops, heads, dim, rot, pairs):
    from tokasaurus_b200.parts import RotaryEncoding

    g = torch.Generator().manual_seed(dim + rot)
    pos = [0, 1, 2, 17, 500, 4095, 3, 100000]
    T, base = len(pos), 5000.0
    proj = torch.randn(T, 3 + 2 * heads * dim + 4, generator=g)
    q_off, k_off = 3, 3 + heads * dim
    freq = RotaryEncoding(rot, base).inv_freq64() if rot else torch.zeros(0, dtype=F64)
    pd = proj.to(DEV)
    ops.rotate_scale(pd, q_off, k_off, heads, dim, rot, pairs, freq.to(DEV), i32(pos), i32([0] * T), 1.0, 0.25,
                     walk_defines(ops, dim, dim))
    fn = plain.rotate_pairs if pairs else plain.rotate_halves
    for off, scale in ((q_off, 1.0), (k_off, 0.25)):
        x = proj[:, off:off + heads * dim].double().reshape(T, heads, dim)
        want = torch.stack([fn(x[t:t + 1], rot, base, start=p)[0] if rot else x[t] for t, p in enumerate(pos)]) * scale
        assert float((pd[:, off:off + heads * dim].cpu().double() - want.reshape(T, -1)).abs().max()) < 2e-6
    assert float((pd[:, :3] - proj[:, :3].to(DEV)).abs().max()) == 0.0 and float((pd[:, -4:] - proj[:, -4:].to(DEV)).abs().max()) == 0.0


@pytest.mark.parametrize("heads,dim,vdim", [(4, 24, 40), (2, 64, 16), (1, 7, 130), (6, 32, 64), (2, 200, 36)])
def test_walk_with_a_decay_for_every_key_channel(ops, heads, dim, vdim):
    """S_t = diag(f_t) S_(t-1) + k_t v_t^T over two requests in portions down to one token, beside each other, with
    every build of the walk the head size allows, against the whole sequences; the state that is left behind."""
    import itertools

    chosen = itertools.cycle(ops.decay_walk_modules(dim, vdim))
    monkey = pytest.MonkeyPatch()
    monkey.setattr(ops, "_walk_defines", lambda *a: next(chosen))
    g = torch.Generator().manual_seed(heads * 1000 + dim)
    lens = {0: 70, 1: 19}
    portions = {0: [2, 33, 1, 1, 17, 16], 1: [1, 2, 16]}
    n_state = heads * dim * vdim
    q = {s: torch.randn(n, heads * dim, generator=g) for s, n in lens.items()}
    k = {s: torch.randn(n, heads * dim, generator=g) * 0.5 for s, n in lens.items()}
    v = {s: torch.randn(n, heads * vdim, generator=g) for s, n in lens.items()}
    f = {s: torch.rand(n, heads * dim, generator=g) ** 0.2 for s, n in lens.items()}  # most near 1, some small
    state = torch.zeros(4, n_state + 13, device=DEV)
    state[:, n_state:] = 5.0
    slots = {0: 3, 1: 1}
    got, at = {s: [] for s in lens}, {s: 0 for s in lens}
    for step in range(6):
        live = [s for s in lens if step < len(portions[s])]
        ql = [portions[s][step] for s in live]
        qs = [int(x) for x in np.concatenate([[0], np.cumsum(ql)[:-1]])]
        cat = lambda d: torch.cat([d[s][at[s]:at[s] + n] for s, n in zip(live, ql)]).to(DEV)  # noqa: E731
        T = sum(ql)
        out = torch.empty(T, heads * vdim, device=DEV)
        wide = torch.cat([cat(q), cat(k), cat(v), torch.full((T, 4), 9.0, device=DEV)], dim=1)  # column slices of one tensor
        ops.decay_walk(wide[:, :heads * dim], wide[:, heads * dim:2 * heads * dim], wide[:, 2 * heads * dim:-4], 1, None, None,
                       None, state, out, i32([slots[s] for s in live]), i32(qs), i32(ql), len(live), heads, dim, vdim,
                       decay_vec=cat(f))
        for s, a, n in zip(live, qs, ql):
            got[s].append(out[a:a + n].cpu())
            at[s] += n
    for s, n in lens.items():
        want, S = plain.linear_recurrence(q[s].double().reshape(n, heads, dim), k[s].double().reshape(n, heads, dim),
                                          v[s].double().reshape(n, heads, vdim), f[s].double().reshape(n, heads, dim))
        assert rel_err(torch.cat(got[s]), want.reshape(n, -1)) < 2e-5, s
        left = state[slots[s], :n_state].cpu().reshape(heads, vdim, dim)
        assert rel_err(left, S.transpose(1, 2)) < 2e-5
    assert float((state[:, n_state:] - 5.0).abs().max()) == 0.0
    monkey.undo()


def paged(n_tokens, page, seed):
    """A block table of scattered pages for one request."""
    n_pages = -(-n_tokens // page)
    perm = np.random.default_rng(seed).permutation(n_pages + 5)[:n_pages]
    return [int(p) for p in perm], n_pages + 5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim,rot,page,heads,kv", [(64, 32, 16, 6, 2), (24, 24, 8, 3, 3), (20, 6, 16, 4, 1), (128, 64, 16, 2, 1), (32, 16, 16, 20, 1)])
def test_sigmoid_attention_sees_a_far_key(ops, dtype, dim, rot, page, heads, kv):
    """Weights sigmoid(score * temp + bias) with a bias that leaves ordinary keys almost nothing, and one made-up key,
    hundreds of positions back at a page's first or last slot, that the last queries score far above: its value (its
    own key as projected, before norm and rotation) must arrive in their outputs whole, from a portion and from single
    tokens, on the FP32 pipes and on the tensor cores, in one block or shared out among several."""
    from tokasaurus_b200.parts import RotaryEncoding

    n, scale, eps = 330, 0.5 / dim ** 0.5, 1e-6
    g = torch.Generator().manual_seed(dim + page)
    temp, pb = torch.rand(heads, generator=g) * 0.5 + 0.75, torch.randn(heads, generator=g) * 0.3 - 6.0
    nw = torch.rand(2, dim, generator=g) + 0.5
    freq = RotaryEncoding(rot, 10000.0).inv_freq64()
    for far_at in (page * 2, page * 3 - 1, 0):
        raw = torch.randn(n, (heads + kv) * dim, generator=g)
        probe = torch.zeros(dim)
        probe[rot:] = torch.randn(dim - rot, generator=g).sign() * 6 if dim > rot else 0.0  # channels that are not rotated
        if dim == rot:
            probe = torch.randn(dim, generator=g)
        seen_from = [n - 1, n - 2]
        for r in seen_from:
            raw[r, :heads * dim] = probe.repeat(heads) * 3
        raw[far_at, heads * dim:] = probe.repeat(kv) * 40
        x = raw.double()
        q = plain.group_norm(x[:, :heads * dim].reshape(n * heads, dim), nw[0].double(), eps).reshape(n, heads, dim)
        kk = plain.group_norm(x[:, heads * dim:].reshape(n * kv, dim), nw[1].double(), eps).reshape(n, kv, dim)
        q, kr = plain.rotate_pairs(q, rot, 10000.0), plain.rotate_pairs(kk, rot, 10000.0)
        v = x[:, heads * dim:].reshape(n, kv, dim)
        want = plain.sigmoid_attention(q, kr, v, scale, temp.double(), pb.double()).reshape(n, heads * dim)
        if dim > rot:  # the far key carries the last rows' outputs
            v0 = v.clone()
            v0[far_at] = 0
            without = plain.sigmoid_attention(q, kr, v0, scale, temp.double(), pb.double()).reshape(n, heads * dim)
            assert float(want[n - 1].abs().max()) > 5 * float(without[n - 1].abs().max())
        table, n_pages = paged(n, page, far_at + 1)
        for cut in ([n], [n - 5, 3, 1, 1], [far_at + 1, n - far_at - 3, 1, 1]):
            cache = torch.full((n_pages, kv, page, 2 * dim), float("nan"), dtype=DT[dtype], device=DEV)
            status = torch.zeros(1, dtype=torch.int32, device=DEV)
            got, at = [], 0
            for m in cut:
                pos = list(range(at, at + m))
                qd = torch.empty(m, heads * dim, dtype=DT[dtype], device=DEV)
                need = -(-(at + m) // page)
                ops.sink_attn_prep(raw[at:at + m].to(DEV), None, True, eps, qd, cache, i32(pos), i32([0] * m), i32([0, need]),
                                   i32(table[:need]), heads, kv, dim, dim, page, True, status, norm_w=nw.to(DEV),
                                   rot_freq=freq.to(DEV), rot_dims=rot, rot_pairs=True, values_are_keys=True, sigmoid=True)
                out = torch.empty(m, heads * dim, dtype=DT[dtype], device=DEV)
                ops.attn_sink(qd, out, cache, i32([0] * m), i32(pos), i32([0, need]), i32(table[:need]), None, m, None, heads,
                              kv, dim, dim, page, scale, None, None, status, head_scale=temp.to(DEV), head_bias=pb.to(DEV),
                              sigmoid=True)
                got.append(out.float().cpu())
                if ops.can_use_attn_sink_tc(DT[dtype], dim, dim):
                    # the same on the tensor cores, beside a second request of one token (this request's first token)
                    out2 = torch.full((m + 1, heads * dim), float("nan"), dtype=DT[dtype], device=DEV)
                    if at == 0:
                        q_first = qd[:1].clone()
                    ops.attn_sink_tc(torch.cat([qd, q_first]), out2, cache, i32([0, m]), i32([m, 1]), i32([at + m, 1]),
                                     i32([0, need, need + 1]), i32(table[:need] + table[:1]), 2, None, heads, kv, dim, dim, page,
                                     scale, None, None, status, portions=m > 1, head_scale=temp.to(DEV), head_bias=pb.to(DEV),
                                     sigmoid=True)
                    assert row_err(out2[:m].float().cpu(), want[at:at + m]) < 4e-2, ("tensor cores", far_at, cut[:2], at)
                    assert row_err(out2[m:].float().cpu(), want[:1]) < 4e-2
                at += m
            assert int(status.item()) == 0
            assert row_err(torch.cat(got), want) < (5e-5 if dtype == "float32" else 4e-2), (far_at, cut[:2])


def test_sigmoid_attention_single_tokens_over_several_blocks(ops):
    """Three requests that bring one token each at contexts of 300, 70 and 1: a request's keys are shared out among
    several blocks whose sums are added afterwards (no softmax: nothing to rescale, nothing counted twice)."""
    dim, heads, kv, page = 32, 6, 2, 16
    g = torch.Generator().manual_seed(9)
    temp, pb = torch.rand(heads, generator=g) + 0.5, torch.randn(heads, generator=g) - 2
    lens = [300, 70, 1]
    n_pages = sum(-(-n // page) for n in lens)
    cache = torch.full((n_pages, kv, page, 2 * dim), float("nan"), dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    perm = [int(x) for x in np.random.default_rng(3).permutation(n_pages)]
    tables, want, last_q = [], [], []
    for n in lens:
        raw = torch.randn(n, (heads + kv) * dim, generator=g)
        table, perm = perm[:-(-n // page)], perm[-(-n // page):]
        tables.append(table)
        qd = torch.empty(n, heads * dim, dtype=torch.bfloat16, device=DEV)
        ops.sink_attn_prep(raw.to(DEV), None, True, 1e-6, qd, cache, i32(list(range(n))), i32([0] * n), i32([0, len(table)]),
                           i32(table), heads, kv, dim, dim, page, True, status, values_are_keys=True, sigmoid=True)
        last_q.append(qd[-1:])
        x = raw.double()
        q = plain.group_norm(x[:, :heads * dim].reshape(n * heads, dim), None, 1e-6).reshape(n, heads, dim)
        k = plain.group_norm(x[:, heads * dim:].reshape(n * kv, dim), None, 1e-6).reshape(n, kv, dim)
        want.append(plain.sigmoid_attention(q, k, x[:, heads * dim:].reshape(n, kv, dim), 0.2, temp.double(), pb.double()).reshape(n, -1)[-1])
    indptr = [0] + [int(x) for x in np.cumsum([len(t) for t in tables])]
    out = torch.full((3, heads * dim), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.attn_sink_tc(torch.cat(last_q), out, cache, i32([0, 1, 2]), i32([1, 1, 1]), i32(lens), i32(indptr), i32(sum(tables, [])),
                     3, None, heads, kv, dim, dim, page, 0.2, None, None, status, portions=False, head_scale=temp.to(DEV),
                     head_bias=pb.to(DEV), sigmoid=True)
    assert int(status.item()) == 0
    assert rel_err(out.float().cpu(), torch.stack(want)) < 3e-2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,groups,keep,top", [(12, 4, 3, 2), (8, 8, 3, 1), (6, 1, 1, 3), (16, 2, 1, 4), (10, 5, 5, 10), (36, 3, 2, 5)])
def test_choice_by_scores_within_the_best_groups(ops, dtype, E, groups, keep, top):
    """Choice by sigmoid score + correction among the best groups, weights from the scores alone; corrections that make
    every choice score negative (an expert outside the kept groups counts as minus infinity, not as 0)."""
    g = torch.Generator().manual_seed(E + top)
    T, H = 200, 48
    h = torch.randn(T, H, generator=g).to(DT[dtype])
    router = torch.randn(E, H, generator=g) * 0.3
    for shift in (0.0, -3.0):
        corr = torch.randn(E, generator=g) * 0.4 + shift
        idx_w, w_w = plain.route(h.double(), router.double(), corr.double(), top, groups, keep, 1.7)
        margin = plain.route_margins(h.double(), router.double(), corr.double(), top, groups, keep)
        token_seq = [0] * (T - 1) + [-1]  # the last row is padding: it chooses nothing
        idx = torch.empty(T, top, dtype=torch.int32, device=DEV)
        w = torch.empty(T, top, dtype=torch.float32, device=DEV)
        ops.moe_route(h.to(DEV), router.to(DEV), None, i32(token_seq), top, idx, w,
                      dict(correction=corr.to(DEV), groups=groups, keep=keep, scale=1.7))
        idx, w = idx.cpu(), w.cpu()
        assert idx[-1].tolist() == [-1] * top
        sure = (margin > 1e-4).nonzero().flatten().tolist()
        assert len(sure) > T * 0.9
        for t in sure[:-1] if sure[-1] == T - 1 else sure:
            assert idx[t].tolist() == idx_w[t].tolist(), (t, shift)
            assert float((w[t].double() - w_w[t]).abs().max()) < 1e-5
        if shift < 0:
            assert float((torch.sigmoid(h.double() @ router.double().T) + corr.double()).max()) < 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,E,top,H,inner", [(3, 4, 2, 64, 40), (70, 6, 3, 128, 64), (400, 5, 2, 96, 72)])
def test_gelu_experts(ops, dtype, T, E, top, H, inner):
    """down(gelu(up h)) over (token, choice) pairs ordered by expert: the few-rows kernel, the tiled kernel, and in
    bfloat16 the tensor-core products with the GELU in their epilogue, through the part itself."""
    from tokasaurus_b200.engine.runtime import Runtime
    from tokasaurus_b200.parts import RoutedExperts

    g = torch.Generator().manual_seed(T)
    part = RoutedExperts(H, inner, E, top, "r", None, lambda e: (f"e{e}.up", f"e{e}.down"),
                         scored=dict(correction="c", groups=1, keep=1, scale=1.3), expert="gelu", out_dtype=torch.float32)
    w = {s.name: torch.randn(s.shape, generator=g) * (0.3 if s.name == "r" else 0.15) for s in part.weight_specs()}
    w["c"] = -1.5 * torch.randperm(E, generator=g).float()  # the choice is fixed: what is compared are the products
    w = {k: (v if k in ("r", "c") else v.to(DT[dtype])) for k, v in w.items()}
    rt = Runtime.make(DEV, dtype)
    part.bind({k: v.to(DEV) for k, v in w.items()}, rt)
    h = torch.randn(T, H, generator=g).to(DT[dtype])
    got = part.forward(None, h.to(DEV))
    assert got.dtype == torch.float32
    p = {k.replace("r", "router") if k == "r" else ("correction" if k == "c" else k): v.double() for k, v in w.items()}
    want = plain.routed_experts(h.double(), p, E, top, 1, 1, 1.3)
    assert rel_err(got.cpu(), want) < (2e-5 if dtype == "float32" else 3e-2)


# ------------------------------------------------------------------------------------------------ whole models
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    return vm.make_models(tmp_path_factory.mktemp("verozen_models"))


CUTS = dict(whole=cuttings.whole, prefix_then_single=cuttings.prefix_then_single,
            changing_portions=cuttings.changing_portions, mixed=cuttings.mixed)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cut", list(CUTS))
@pytest.mark.parametrize("which", list(vm.MODELS))
def test_cuttings_match_plain(models, which, cut, dtype):
    """Whole prompts, prompts then single tokens, portions of changing size down to one and two tokens, and up to four
    requests side by side in four slots, in a pool that holds exactly what the trace needs: pages and slots are used
    again, and a later request must see nothing of an earlier one's keys or state."""
    from tokasaurus_b200.engine.trace import TraceReplayer

    m = models[(which, vm.variant(dtype))]
    steps = CUTS[cut](m["reqs"])
    rp = TraceReplayer(str(m["folder"]), dtype, cuttings.max_live_tokens(steps, m["page"]), page_size=m["page"], max_requests=4)
    cache = rp.runner.cache
    owners, slots, outs = {}, {}, []
    for st in steps:
        outs.append(rp.run_step(st))
        cache.check()
        for rid, rc in cache.requests.items():
            slots.setdefault(rc.slot, set()).add(rid)
            for gi in range(len(cache.groups)):
                for p in rc.live_pages(gi):
                    owners.setdefault((gi, p), set()).add(rid)
    assert not cache.requests and cache.num_free_pages() == [g.allocator.num_pages for g in cache.groups]
    vm.check_logits(cuttings.collect(steps, outs), m, dtype, cut)
    if cut == "mixed":
        assert not cache.groups or any(len(v) > 1 for v in owners.values()), "no page was used by two requests"
        assert any(len(v) > 1 for v in slots.values()), "no slot was used by two requests"


def test_layer_by_layer(models):
    """The residual stream after every layer, float32, one prompt in one step and in two."""
    from tokasaurus_b200.engine.batch import StepEntry
    from tokasaurus_b200.engine.trace import TraceReplayer

    for which in vm.MODELS:
        m = models[(which, "dyn")]
        rid, toks = next(iter(m["reqs"].items()))
        want = []
        plain.forward(m["config"], m["weights"], toks, want)
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
    m = models[("a", "dyn")]
    rid, toks = max(m["reqs"].items(), key=lambda kv: len(kv[1]))
    ref = m["want"][rid]
    tol = 3 * float(m["noise"][rid].max())  # the widest limit of the float32 comparisons on this request

    def moved(config, weights=None):
        return float(vm.row_error(plain.forward(config, weights or m["weights"], toks).numpy() - ref).max())

    for path, value in (("tau", lambda t: t * 1.1), ("decay", lambda d: [x * 0.98 for x in d]), ("scale", lambda s: s * 1.1),
                        ("rot.dims", lambda d: d - 2), ("rot.base", lambda b: b * 2), ("router.scale", lambda s: s * 1.1),
                        ("router.groups", lambda g: dict(count=g["count"], keep=min(g["count"], g["keep"] + 1))),
                        ("router.top", lambda t: t + 1)):
        assert moved(vm.changed(m["config"], path, value)) > 30 * tol, path
    for key, value in (("postln_alpha", 1.0), ("norm", dict(eps=1e-5, groups=1)), ("token_side", None)):
        assert moved(dict(m["config"], **{key: value})) > 30 * tol, key
    for name, f in (("l1.mix.pb", lambda t: t - 1.0), ("l1.mix.temp", lambda t: t * 1.2), ("l1.mix.q.norm", lambda t: t * 0 + 1),
                    ("l0.mix.a2.b", lambda t: t + 0.5), ("l0.mix.norm", lambda t: t * 0 + 1), ("l0.mlp.correction", lambda t: t * 0),
                    ("l2.side.norm", lambda t: t * 1.2), ("side.embed", lambda t: t.roll(8, 1))):
        w = dict(m["weights"])
        w[name] = f(w[name].clone())
        assert moved(m["config"], w) > 30 * tol, name


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(models, dtype):
    """A short prompt, then 150 tokens one by one: states are carried 150 steps, decoded keys fill page after page."""
    from tokasaurus_b200.engine.trace import TraceReplayer

    for which in ("a", "c", "d", "e"):
        m = models[(which, vm.variant(dtype))]
        toks = cuttings.random_tokens(160, m["config"]["vocab"], 7)
        ms = []
        want = plain.forward(m["config"], m["weights"], toks, margins=ms).numpy()
        if dtype == "float32":
            assert min(float(x.min()) for x in ms) > 2e-5
        steps = cuttings.prefix_then_single({"long": toks}, tail=150)
        rp = TraceReplayer(str(m["folder"]), dtype, cuttings.max_live_tokens(steps, m["page"]), page_size=m["page"], max_requests=4)
        got = cuttings.collect(steps, [rp.run_step(st) for st in steps])
        noise = vm.rounding_noise(m["config"], m["weights"], toks, want, dtype)
        vm.check_logits(got, dict(want={"long": want}, noise={"long": noise}), dtype, "long decoding")


def plain_greedy(m, prompt, n):
    ids, out = list(prompt), []
    for _ in range(n):
        out.append(int(plain.forward(m["config"], m["weights"], ids)[-1].argmax()))
        ids.append(out[-1])
    return out


@pytest.mark.parametrize("which", ["a", "d", "e"])
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_entry_point(models, graphs, which):
    """Greedy generation in float32 through ``Engine.generate``: the scheduler admits, cuts prompts into portions,
    decodes (from CUDA graphs or kernel by kernel; a decoded token's side input is looked up from the id that never
    left the device) and frees; five requests in three slots, so slots are handed on.  Also for a model without any
    pages and for one without any state."""
    from tokasaurus_b200.engine.engine import Engine

    m = models[(which, "tier")]
    V = m["config"]["vocab"]
    prompts = [cuttings.random_tokens(n, V, 300 + n) for n in (30, 3, 41, 17, 9)]
    n_new = 10
    want = [plain_greedy(m, p, n_new) for p in prompts]
    eng = Engine(model=str(m["folder"]), dtype="float32", page_size=m["page"], kv_cache_num_tokens=512,
                 max_tokens_per_forward=24, max_seqs_per_forward=3, allocator_sanity_checks=True, use_cudagraphs=graphs)
    outs = eng.generate(prompts, max_num_tokens=n_new, ignore_eos=True)
    assert [o.completion_ids for o in outs] == want
    cache = eng.runner.cache
    assert not cache.requests and cache.num_free_pages() == [g.allocator.num_pages for g in cache.groups]


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
