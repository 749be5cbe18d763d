"""The Verozen configuration reader and the model description built from it (no GPU): every size and constant comes
from config.json, each layer's mixer gets the cache or state entry of its kind, the tensor names and shapes follow the
layers, and a configuration that cannot describe a model is refused with the key that is wrong.  Also the plain
implementation's own mechanisms against hand-made cases, since every GPU comparison rests on it."""

import math

import pytest
import torch

import plain_verozen as plain
from tokasaurus_b200.config import lookup_architecture
from tokasaurus_b200.config.model_config import ConfigError
from tokasaurus_b200.parts.base import PagedCacheNeed, StateNeed


def base_config():
    router = dict(experts=6, top=2, scale=1.5, groups=dict(count=3, keep=2))
    return dict(architecture="Verozen", vocab=97, width=48, norm=dict(eps=1e-5, groups=3), postln_alpha=1.7,
                token_side=dict(dim=4),
                layers=[dict(type="gla", mixer=dict(heads=3, dim=8, vdim=20, tau=8.0), mlp=dict(kind="moe", expert=dict(ff=24), router=router)),
                        dict(type="attention", mixer=dict(heads=4, kv_heads=2, dim=12, vdim=12, scale=0.2, rot=dict(dims=6, base=500.0)), mlp=None),
                        dict(type="retention", mixer=dict(heads=2, dim=16, vdim=10, decay=[0.9, 0.99], rot=dict(dims=8, base=1e6)),
                             mlp=dict(kind="moe", expert=dict(ff=40), router=dict(experts=5, top=1, scale=1.0)))])


def test_description_follows_the_configuration():
    d = base_config()
    arch = lookup_architecture(d)
    assert arch.name == "Verozen"
    cfg = arch.parse_config(d)
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.norm_groups, cfg.alpha, cfg.side_dim) == (97, 48, 1e-5, 3, 1.7, 4)
    assert (cfg.layers[0].mlp.groups, cfg.layers[0].mlp.keep) == (3, 2)
    assert (cfg.layers[2].mlp.groups, cfg.layers[2].mlp.keep) == (1, 1)  # no groups given: one group, kept
    model = arch.build_model(cfg)
    needs = model.cache_entries()
    assert needs[0] == StateNeed((3 * 8 * 20,), "float32")
    assert needs[1] == PagedCacheNeed(2, 24, None, planes=1)  # a row holds the rotated key and the key as projected
    assert needs[2] == StateNeed((2 * 16 * 10,), "float32")
    names = {s.name: s for s in model.weight_specs()}
    assert names["side.embed"].shape == (97, 3 * 4)
    assert names["l0.mix.a2"].shape[0] == 24 and names["l0.mix.a2.b"].shape == (24,) and names["l0.mix.norm"].shape == (20,)
    assert names["l0.mix.a1"].shape[0] < 0  # the rank is the weight file's
    assert names["l1.mix.q"].shape == (48, 48) and names["l1.mix.k"].shape == (24, 48) and "l1.mix.v" not in names
    assert names["l1.mix.q.norm"].shape == (12,) and names["l1.mix.temp"].shape == (4,) and names["l1.mix.pb"].shape == (4,)
    assert names["l1.norm2"].optional and not names["l0.norm2"].optional and "l1.mlp.router" not in names
    assert names["l2.mix.g"].shape == (20, 48) and names["l2.mix.o"].shape == (48, 20) and "l2.mix.norm" not in names
    assert names["l2.mlp.e4.up"].shape == (40, 48) and names["l2.mlp.e4.down"].shape == (48, 40) and "l2.mlp.e5.up" not in names
    assert names["l0.mlp.router"].role == "vector" and names["l0.mlp.correction"].shape == (6,)  # routers work in 32-bit
    assert names["l2.side.gate"].shape == (4, 48) and names["l2.side.proj"].shape == (48, 4)
    assert [b.alpha for b in model.blocks] == [1.7] * 3
    assert model.blocks[2].mixer.decay == (0.9, 0.99) and model.blocks[2].mixer.k_scale == 16 ** -0.5
    assert model.blocks[0].mixer.q_scale == 8 ** -0.5 and model.blocks[0].mixer.tau == 8.0
    d["token_side"] = None
    bare = arch.build_model(arch.parse_config(d))
    assert all(b.side is None for b in bare.blocks) and "side.embed" not in {s.name for s in bare.weight_specs()}


@pytest.mark.parametrize("change,word", [
    (lambda d: d["layers"][0].update(type="mamba"), "type"),
    (lambda d: d["layers"][0]["mixer"].update(tau=0.0), "tau"),
    (lambda d: d["layers"][0]["mixer"].pop("heads"), "heads"),
    (lambda d: d["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda d: d["layers"][1]["mixer"].update(vdim=16), "vdim"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=14), "rot.dims"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=5), "rot.dims"),
    (lambda d: d["layers"][2]["mixer"].update(decay=[0.9]), "decay"),
    (lambda d: d["layers"][0]["mlp"].update(kind="dense"), "kind"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=5), "top"),
    (lambda d: d["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda d: d["norm"].update(groups=5), "groups"),
    (lambda d: d.pop("width"), "width"),
    (lambda d: d.update(layers=[]), "layers"),
])
def test_bad_configurations_are_refused(change, word):
    d = base_config()
    change(d)
    arch = lookup_architecture(d)
    with pytest.raises(ConfigError) as e:
        arch.parse_config(d)
    assert word in str(e.value)


def test_random_model_folder_round_trips(tmp_path):
    """A folder written for a configuration holds exactly the tensors that the description names (an optional norm is
    left out), and reading it back gives the description's shapes, the low-rank factor's rows included."""
    from safetensors import safe_open
    from tokasaurus_b200.weights import write_model_folder

    d = base_config()
    d["layers"][0]["mixer"]["rank"] = 5
    folder = write_model_folder(tmp_path / "m", d, seed=3)
    arch = lookup_architecture(d)
    specs = {s.name: s for s in arch.build_model(arch.parse_config(d)).weight_specs()}
    with safe_open(str(folder / "model.safetensors"), framework="pt") as f:
        shapes = {k: tuple(f.get_tensor(k).shape) for k in f.keys()}
    assert set(shapes) == {n for n, s in specs.items() if not s.optional}
    assert shapes["l0.mix.a1"] == (5, 48) and shapes["l0.mix.a2"] == (24, 5)


# ------------------------------------------------------------------------------------ the plain implementation itself
def test_plain_norm_in_parts():
    x = torch.tensor([[3.0, 4.0, 0.0, 0.5]], dtype=torch.float64)
    w = torch.tensor([1.0, 2.0, 1.0, 4.0], dtype=torch.float64)
    got = plain.group_norm(x, w, 0.0, groups=2)
    r0, r1 = math.sqrt(12.5), math.sqrt(0.125)
    assert torch.allclose(got, torch.tensor([[3 / r0, 8 / r0, 0.0, 2 / r1]], dtype=torch.float64))
    one = plain.group_norm(x, w, 0.0, groups=1)
    assert not torch.allclose(got, one)


def test_plain_rotations_pair_the_right_channels():
    x = torch.zeros(1, 1, 8, dtype=torch.float64)
    x[0, 0, 0] = 1.0  # channel 0: paired with channel 1 (pairs) or with channel 2 (halves of the first 4)
    p = plain.rotate_pairs(x, 4, 100.0, start=3)
    h = plain.rotate_halves(x, 4, 100.0, start=3)
    a = 3.0  # f_0 = 1
    assert math.isclose(float(p[0, 0, 0]), math.cos(a)) and math.isclose(float(p[0, 0, 1]), math.sin(a))
    assert math.isclose(float(h[0, 0, 0]), math.cos(a)) and math.isclose(float(h[0, 0, 2]), math.sin(a))
    assert float(p[0, 0, 2:].abs().sum()) == 0.0 and float(h[0, 0, 1].abs()) == 0.0 and float(h[0, 0, 3:].abs().sum()) == 0.0
    y = torch.zeros(1, 1, 8, dtype=torch.float64)
    y[0, 0, 2] = 1.0  # pair 1 turns by f_1 = 100^(-2/4) = 0.1 a position; channels past the first 4 do not turn
    y[0, 0, 6] = 5.0
    p = plain.rotate_pairs(y, 4, 100.0, start=7)
    assert math.isclose(float(p[0, 0, 2]), math.cos(0.7)) and math.isclose(float(p[0, 0, 3]), math.sin(0.7))
    assert float(p[0, 0, 6]) == 5.0


def test_plain_recurrence_by_hand():
    """Two tokens, one head, two key channels, one value: S_1 = k_1 v_1; S_2 = f_2 * S_1 + k_2 v_2, row by row."""
    q = torch.tensor([[[1.0, 1.0]], [[1.0, 2.0]]], dtype=torch.float64)
    k = torch.tensor([[[2.0, 3.0]], [[1.0, 1.0]]], dtype=torch.float64)
    v = torch.tensor([[[5.0]], [[7.0]]], dtype=torch.float64)
    f = torch.tensor([[[0.0, 0.0]], [[0.5, 0.1]]], dtype=torch.float64)
    o, S = plain.linear_recurrence(q, k, v, f)
    assert math.isclose(float(o[0, 0, 0]), 25.0)
    assert torch.allclose(S[0, :, 0], torch.tensor([0.5 * 10 + 7, 0.1 * 15 + 7], dtype=torch.float64))
    assert math.isclose(float(o[1, 0, 0]), 12.0 + 2 * 8.5)


def test_plain_choice_within_the_best_groups():
    """Six experts in three pairs, two pairs kept, two experts chosen.  Sigmoid scores all 0.5 (a zero router), so the
    corrections alone decide: a group's score is the sum of its two choice scores; the best single expert sits in the
    dropped group and must not be chosen; the weights are the scores without corrections, so both are scale / 2."""
    h = torch.ones(1, 4, dtype=torch.float64)
    router = torch.zeros(6, 4, dtype=torch.float64)
    corr = torch.tensor([0.9, -2.0, 0.3, 0.2, 0.1, 0.35], dtype=torch.float64)  # group sums -1.1+1, 0.5+1, 0.45+1
    idx, w = plain.route(h, router, corr, 2, 3, 2, 3.0)
    assert sorted(idx[0].tolist()) == [2, 5]
    assert torch.allclose(w, torch.full((1, 2), 1.5, dtype=torch.float64))
    # every choice score negative: an expert outside the kept groups still loses to one inside
    idx, _ = plain.route(h, router, corr - 5.0, 2, 3, 2, 3.0)
    assert sorted(idx[0].tolist()) == [2, 5]
    # one group: plain top-k over the choice scores
    idx, _ = plain.route(h, router, corr, 2, 1, 1, 1.0)
    assert sorted(idx[0].tolist()) == [0, 5]


def test_plain_sigmoid_attention_is_causal_and_not_normalised():
    """One head, one channel, equal keys: every visible key weighs sigmoid(score * temp + bias), so the output grows
    with the number of keys seen (a softmax would hold it constant), and nothing of a later key arrives."""
    T = 5
    q = torch.ones(T, 1, 1, dtype=torch.float64)
    k = torch.full((T, 1, 1), 2.0, dtype=torch.float64)
    v = torch.arange(1.0, T + 1, dtype=torch.float64).reshape(T, 1, 1)
    temp, bias = torch.tensor([0.5], dtype=torch.float64), torch.tensor([-1.0], dtype=torch.float64)
    o = plain.sigmoid_attention(q, k, v, 3.0, temp, bias)
    wgt = 1.0 / (1.0 + math.exp(-(2.0 * 3.0 * 0.5 - 1.0)))
    for t in range(T):
        assert math.isclose(float(o[t, 0, 0]), wgt * sum(range(1, t + 2)))
