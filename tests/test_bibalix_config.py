"""The Bibalix configuration reader and the model description built from it (no GPU): every size and constant comes
from config.json, each layer's mixer gets a cache entry of its kind, the tensor names and shapes follow the layers, and
a configuration that cannot describe a model is refused with the key that is wrong.  The cache manager's books for a
window that keeps a request's first positions.  Also the plain implementation's own mechanisms against hand-made
cases, since every GPU comparison rests on it."""

import math

import pytest
import torch

import plain_bibalix as plain
from tokasaurus_b200.cache.manager import CacheManager
from tokasaurus_b200.config import lookup_architecture
from tokasaurus_b200.config.model_config import ConfigError
from tokasaurus_b200.parts.base import PagedCacheNeed


def base_config():
    return dict(architecture="Bibalix", vocab=97, width=48, norm=dict(eps=1e-5),
                layers=[dict(type="latent_attention",
                             mixer=dict(heads=3, dim=8, rot_dim=6, vdim=10, kv_rank=20, scale=0.2, mask=dict(size=21),
                                        rot=dict(dims=4, base=100.0, scaling=dict(factor=2.0, original=16, fast=4.0, slow=1.0))),
                             mlp=dict(kind="moe", expert=dict(ff=24, limit=3.0), router=dict(experts=6, top=2, scale=1.5),
                                      shared=dict(ff=16, limit=1.5))),
                        dict(type="attention",
                             mixer=dict(heads=4, kv_heads=2, dim=12, vdim=20, scale=0.25, diff=0.4, mask=dict(size=37, keep_first=3),
                                        rot=dict(dims=6, base=500.0)),
                             mlp=dict(kind="dense", ff=40)),
                        dict(type="attention", mixer=dict(heads=2, dim=8, vdim=8, scale=0.3, diff=0.1), mlp=None)])


def test_description_follows_the_configuration():
    d = base_config()
    arch = lookup_architecture(d)
    assert arch.name == "Bibalix"
    cfg = arch.parse_config(d)
    assert (cfg.vocab, cfg.width, cfg.norm_eps, len(cfg.layers)) == (97, 48, 1e-5, 3)
    assert cfg.layers[0].mixer.rot.scaling.original == 16 and cfg.layers[1].mixer.rot.scaling is None
    assert (cfg.layers[1].mixer.window, cfg.layers[1].mixer.keep_first) == (37, 3)
    assert (cfg.layers[2].mixer.window, cfg.layers[2].mixer.keep_first, cfg.layers[2].mixer.kv_heads) == (None, 0, 2)
    model = arch.build_model(cfg)
    needs = model.cache_entries()
    assert needs[0] == PagedCacheNeed(1, 26, 21, planes=1)                    # one row a token: latent and rotated key part
    assert needs[1] == PagedCacheNeed(2, 2 * 12 + 20, 37, planes=1, keep_first=3)  # both maps' keys and the value
    assert needs[2] == PagedCacheNeed(2, 2 * 8 + 8, None, planes=1)
    names = {s.name: s for s in model.weight_specs()}
    assert names["l0.mix.q"].shape == (3 * 14, 48) and names["l0.mix.dkv"].shape == (26, 48) and names["l0.mix.dkv.norm"].shape == (20,)
    assert names["l0.mix.uk"].shape == (24, 20) and names["l0.mix.uv"].shape == (30, 20) and names["l0.mix.g"].shape == (3, 48)
    assert names["l0.mix.o"].shape == (48, 30) and "l0.mix.dq" not in names
    assert names["l1.mix.q"].shape == (4 * 2 * 12, 48) and names["l1.mix.k"].shape == (2 * 2 * 12, 48) and names["l1.mix.v"].shape == (40, 48)
    assert names["l1.mix.q.b"].shape == (96,) and names["l1.mix.v.b"].shape == (40,) and names["l1.mix.q.norm"].shape == (12,)
    assert all(names[f"l1.mix.{n}"].shape == (12,) for n in ("lq1", "lk1", "lq2", "lk2")) and names["l1.mix.g"].shape == (4, 48)
    assert names["l0.mlp.router"].role == "vector" and names["l0.mlp.shared.sg"].shape == (1, 48)  # routers work in 32-bit
    assert names["l0.mlp.e5.gate"].shape == (24, 48) and names["l0.mlp.shared.down"].shape == (48, 16) and "l0.mlp.e6.up" not in names
    assert names["l1.mlp.gate"].shape == (40, 48) and "l2.norm2" not in names and names["final.norm.b"].shape == (48,)
    assert "head" not in names and model.head.weight_name == "embed"        # the head is the embedding table
    lat, diff = model.blocks[0].mixer, model.blocks[1].mixer
    assert (lat.window, lat.halves, lat.rot_dims, lat.q_rank, lat.gated) == (21, True, 4, None, True)
    assert lat.rotary.scaling_type == "yarn" and abs(lat.rotary.magnitude() - (0.1 * math.log(2.0) + 1)) < 1e-15
    assert (diff.maps, diff.keep_first, diff.window, diff.diff, diff.rotary.rotary_dim, diff.rotary_pairs) == (2, 3, 37, 0.4, 6, False)
    ffn = model.blocks[0].ffn
    assert ffn.clamp == (3.0, 1.702) and ffn.over_all == dict(scale=1.5) and ffn.shared.limit == 1.5
    assert model.blocks[1].ffn.activation == "gelu_tanh" and model.blocks[2].ffn is None
    mods = dict((s, d) for s, d in model.kernel_modules("float32"))
    assert mods["latent_attention.cu"] == {"TKB_LAT_RANK": 20} and "attention_sink.cu" in mods and "moe.cu" in mods


@pytest.mark.parametrize("change,word", [
    (lambda d: d["layers"][0].update(type="mamba"), "type"),
    (lambda d: d["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=14), "dims"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(scaling=dict(factor=2.0, original=8)), "scaling"),
    (lambda d: d["layers"][0]["mixer"]["mask"].update(keep_first=2), "keep_first"),
    (lambda d: d["layers"][1]["mixer"].pop("diff"), "diff"),
    (lambda d: d["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=7), "top"),
    (lambda d: d["layers"][0]["mlp"]["expert"].update(limit=0), "limit"),
    (lambda d: d["layers"][1]["mlp"].update(kind="glu"), "kind"),
    (lambda d: d.pop("vocab"), "vocab"),
])
def test_configurations_that_describe_no_model_are_refused(change, word):
    d = base_config()
    change(d)
    with pytest.raises(ConfigError) as e:
        lookup_architecture(d).parse_config(d)
    assert word in str(e.value)


def test_pages_of_kept_first_positions_stay():
    """A windowed group whose mixers keep a request's first positions in sight gives back the pages behind the window,
    not those of the kept positions; the pages come back in order and once; the books stay whole."""
    page = 8
    needs = {0: PagedCacheNeed(1, 16, 20, planes=1, keep_first=11), 1: PagedCacheNeed(1, 16, 20, planes=1), 2: PagedCacheNeed(1, 8, None)}
    cm = CacheManager(needs, page, 40, max_requests=2, device=None)
    assert [cm.kept_pages(g) for g in range(3)] == [2, 0, 0]
    cm.admit("r")
    seen = []
    for n in (5, 13, 30, 31, 64, 65, 200):
        cm.ensure_capacity("r", n)
        cm.release_behind_window("r", n)
        cm.check()
        rc = cm.requests["r"]
        first_visible = max(0, n - 20 + 1)
        for g, kept in ((0, 2), (1, 0)):
            t = rc.tables[g]
            gone = [i for i, p in enumerate(t) if p < 0]
            assert gone == list(range(kept, max(kept, first_visible // page))), (n, g, gone)
            assert rc.released[g] == len(gone)
        assert all(p >= 0 for p in rc.tables[2])
        seen.append(cm.num_free_pages())
    assert seen[-1][0] == 40 - (2 + (25 - 22)) and seen[-1][1] == 40 - 3 and seen[-1][2] == 40 - 25
    cm.free("r")
    assert cm.num_free_pages() == [40, 40, 40]


def test_plain_mechanisms_on_hand_made_cases():
    # who sees whom: a window of 3 that keeps the first 2 positions
    vis = plain.visible(7, 3, 2)
    assert vis[6].tolist() == [True, True, False, False, True, True, True] and vis[2].tolist() == [True, True, True] + [False] * 4
    assert plain.visible(4, None).tolist() == torch.tril(torch.ones(4, 4)).bool().tolist()
    # rotation in halves: channel 0 turns with channel 2 of four rotated ones; the fifth passes
    x = torch.tensor([[[1.0, 0.0, 0.0, 0.0, 7.0]]], dtype=torch.float64)
    f = torch.tensor([math.pi / 2, 0.0], dtype=torch.float64)
    y = plain.rotate_halves(x, torch.tensor([1]), f, 2.0, 4)[0, 0]
    assert torch.allclose(y, torch.tensor([0.0, 0.0, 2.0, 0.0, 7.0], dtype=torch.float64), atol=1e-12)
    # blended frequencies: fast pairs keep theirs, slow pairs are divided by the factor, sine and cosine grow
    fr, mag = plain.rotary_frequencies(dict(base=10000.0, scaling=dict(factor=4.0, original=64, fast=32.0, slow=1.0)), 32)
    plain_f = 10000.0 ** (-torch.arange(16, dtype=torch.float64) / 16)
    assert fr[0] == plain_f[0] and abs(float(fr[-1] / plain_f[-1]) - 0.25) < 1e-12 and abs(mag - (0.1 * math.log(4) + 1)) < 1e-15
    assert all(plain_f[i] / 4 - 1e-15 <= fr[i] <= plain_f[i] + 1e-15 for i in range(16))
    # the clamped unit: gate above the limit counts as the limit, up is clamped on both sides
    w = {"gate": torch.tensor([[1.0]]), "up": torch.tensor([[1.0]]), "down": torch.tensor([[1.0]])}
    out = plain.clamped_expert(torch.tensor([[5.0], [-5.0]], dtype=torch.float64), {k: v.double() for k, v in w.items()}, "", 2.0)
    assert abs(float(out[0]) - 2.0 / (1 + math.exp(-1.702 * 2.0)) * 3.0) < 1e-12
    assert abs(float(out[1]) - (-5.0) / (1 + math.exp(1.702 * 5.0)) * (-1.0)) < 1e-12
    # shares of the softmax over all experts, not renormalised
    idx, wt, s = plain.route(torch.tensor([[1.0]], dtype=torch.float64), torch.tensor([[0.0], [1.0], [3.0]], dtype=torch.float64), 2, 2.0)
    assert idx.tolist() == [[2, 1]] and abs(float(wt.sum()) - 2.0 * (math.e ** 3 + math.e) / (1 + math.e + math.e ** 3)) < 1e-12
    # gelu in its tanh form
    assert abs(float(plain.gelu_tanh(torch.tensor(1.0, dtype=torch.float64))) - 0.8411919906082768) < 1e-12
