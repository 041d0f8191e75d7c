"""Configuration of the Gozatar decoder, its weight list, and what it brought to the shared parts: sizes that the
checkpoint chooses, a mixer made of mixers with a bundle of caches inside a bundle, several residual streams."""
import copy

import pytest
import torch

from plain import gozatar_plain as G
from spissa_b200.cache import CacheManager
from spissa_b200.config import ConfigError, GozatarConfig, config_from_dict
from spissa_b200.engine.model import Model
from spissa_b200.parts import CacheBundle, KVCacheRequest, StateRequest
from spissa_b200.weights import load_tensors, write_random_model, write_safetensors
from spissa_b200.weights.loader import WeightError


def left(heads, kv, dim, vdim, conv=None, rot=None, base=10000.0, window=None, scale=0.3):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale)
    if conv:
        m["conv"] = conv
    if rot:
        m["rot"] = dict(dims=rot, base=base)
    if window:
        m["mask"] = dict(size=window)
    return m


CFG = dict(
    architecture="Gozatar", vocab=90, width=40, streams=3, norm=dict(eps=1e-4),
    layers=[
        dict(type="parallel", mixer=dict(left=left(4, 2, 6, 10, conv=4, rot=4, base=1000.0, window=70), left_scale=0.7,
                                         right=dict(heads=2, dim=8, vdim=12, tau=4.0), right_scale=0.4),
             mlp=dict(kind="dense", ff=56)),
        dict(type="parallel", mixer=dict(left=left(3, 3, 8, 8), left_scale=1.0,
                                         right=dict(heads=1, dim=4, vdim=20, tau=9.0, rank=5), right_scale=1.0), mlp=None),
        dict(type="parallel", mixer=dict(left=left(2, 1, 12, 4, conv=2, window=9), left_scale=0.5,
                                         right=dict(heads=3, dim=8, vdim=8, tau=1.0), right_scale=2.0),
             mlp=dict(kind="moe", expert=dict(ff=16, limit=1.5), shared=dict(ff=24, limit=3.0),
                      router=dict(experts=6, top=2, groups=dict(count=3, keep=2)))),
    ])


def test_registry_finds_the_architecture_and_the_configuration_round_trips():
    cfg = config_from_dict(CFG)
    assert isinstance(cfg, GozatarConfig)
    assert cfg.to_dict() == CFG
    again = config_from_dict(GozatarConfig(**{**cfg.__dict__, "raw": None}).to_dict())
    assert again.layers == cfg.layers and again.streams == 3


def test_weight_list():
    model = Model(config_from_dict(CFG).to_spec())
    shapes = {s.name: tuple(s.shape) for s in model.weight_specs()}
    assert shapes["embed"] == (90, 40) and shapes["head"] == (90, 40) and shapes["final.norm"] == (40,)
    assert shapes["l0.mix.left.q"] == (24, 40) and shapes["l0.mix.left.k"] == (12, 40) and shapes["l0.mix.left.v"] == (20, 40)
    assert shapes["l0.mix.left.o"] == (40, 40) and shapes["l0.mix.left.v.conv"] == (20, 4)
    assert "l1.mix.left.q.conv" not in shapes and "l1.mlp.up" not in shapes and "l1.norm2" not in shapes
    assert "l1.hc2.in" not in shapes and shapes["l1.hc1.mix"] == (3, 3) and shapes["l2.hc2.out"] == (3,)
    assert shapes["l0.mix.right.a1"] == (-16, 40) and shapes["l0.mix.right.a2"] == (16, -16)     # the checkpoint chooses
    assert shapes["l1.mix.right.a1"] == (5, 40) and shapes["l1.mix.right.a2"] == (4, 5) and shapes["l1.mix.right.norm"] == (20,)
    assert shapes["l2.mlp.router"] == (6, 40) and shapes["l2.mlp.correction"] == (6,)
    assert shapes["l2.mlp.e5.down"] == (40, 16) and shapes["l2.mlp.shared.gate"] == (24, 40)
    plain = Model(config_from_dict({k: v for k, v in CFG.items() if k != "streams"}).to_spec())
    assert not any(".hc" in s.name for s in plain.weight_specs()) and plain.spec.streams == 1


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="serial"), "known mixers"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=8), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(tau=0.0), "tau"),
    (lambda c: c["layers"][0]["mixer"].pop("left_scale"), "left_scale"),
    (lambda c: c["layers"][0]["mlp"].update(kind="experts"), "kind"),
    (lambda c: c["layers"][2]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["layers"][2]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["layers"][2]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c.update(streams=0), "streams"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_bad_configurations_are_refused_with_the_field_named(change, word):
    bad = copy.deepcopy(CFG)
    change(bad)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(bad)


def test_a_size_that_the_checkpoint_chooses(tmp_path):
    cfg = config_from_dict(CFG)
    write_random_model(cfg, tmp_path, seed=1)
    _, w = G_read(tmp_path)
    assert w["l0.mix.right.a1"].shape == (16, 40) and w["l1.mix.right.a1"].shape == (5, 40)
    # another rank in the file is taken as it comes ...
    w["l0.mix.right.a1"] = torch.randn(7, 40).to(torch.bfloat16)
    w["l0.mix.right.a2"] = torch.randn(16, 7).to(torch.bfloat16)
    write_safetensors(tmp_path / "model.safetensors", w)
    specs = Model(cfg.to_spec()).weight_specs()
    assert load_tensors(tmp_path, specs, "cpu", False)["l0.mix.right.a1"].shape == (7, 40)
    # ... a size the configuration fixes is not
    w["l1.mix.right.a1"] = torch.randn(6, 40).to(torch.bfloat16)
    write_safetensors(tmp_path / "model.safetensors", w)
    with pytest.raises(WeightError, match="l1.mix.right.a1"):
        load_tensors(tmp_path, specs, "cpu", False)


def G_read(folder):
    from plain.llama_plain import read_model_folder
    return read_model_folder(folder)


def test_a_mixer_of_mixers_gets_a_bundle_of_caches_inside_a_bundle():
    model = Model(config_from_dict(CFG).to_spec())
    reqs = model.cache_requests()
    assert reqs[0] == CacheBundle((
        ("left", CacheBundle((("kv", KVCacheRequest(2, 6, 70, v_head_dim=10)), ("conv", StateRequest((3, 56), torch.float32))))),
        ("right", StateRequest((2, 8, 12), torch.float32))))
    assert reqs[1].parts[0][1] == CacheBundle((("kv", KVCacheRequest(3, 8, None)),))          # no convolution: no state
    cache = CacheManager(reqs, max_tokens=64 * 4, max_seqs=2, page_size=64, dtype=torch.float32, device="cpu")
    assert len(cache.kv_groups) == 3 and len(cache.state_groups) == 5
    step = type("S", (), dict(page_tables={g: None for g in cache.kv_groups}, token_seq=None, positions=None, seq_row=None))
    view = cache.view(0, step, True)
    assert tuple(view["left"]["kv"].v_pool.shape) == (4, 2, 64, 10)
    assert tuple(view["left"]["conv"].state.shape) == (2, 3, 56) and tuple(view["right"].state.shape) == (2, 2, 8, 12)
    assert view["left"].get("nothing") is None and cache.view(1, step, True)["left"].get("conv") is None
    slot = cache.acquire()
    for n in (100, 1):
        cache.commit(cache.reserve([(slot, n)]))
    held = {g.request.window: [p is not None for p in cache.seqs[slot].pages[g.name]] for g in cache.kv_groups.values()}
    assert held == {70: [True, True], None: [True, True], 9: [False, True]}
    cache.check()
    cache.release(slot)


def test_the_plain_router_keeps_to_the_best_groups_and_weighs_without_the_correction():
    w = {"router": torch.zeros(6, 4, dtype=torch.float64), "correction": torch.tensor([0.0, 0.0, 5.0, -9.0, 0.1, 0.2]).double()}
    w["router"][:, 0] = torch.tensor([2.0, 1.0, -3.0, 3.0, 0.5, 0.4]).double()
    a = torch.tensor([[1.0, 0, 0, 0]]).double()
    # groups (0,1) (2,3) (4,5): scores 1.61, 0.05 + 5 − 8.05, 1.52: groups 0 and 2 stay; expert 2's large choice is out
    idx, wt = G.route(a, w, "", dict(experts=6, top=3, groups=dict(count=3, keep=2)))
    assert sorted(idx[0].tolist()) == [0, 1, 5]
    s = torch.sigmoid(torch.tensor([2.0, 1.0, 0.4]).double())
    assert torch.allclose(wt[0].sort().values, (s / s.sum()).sort().values)
    idx, _ = G.route(a, w, "", dict(experts=6, top=2))
    assert sorted(idx[0].tolist()) == [0, 2]
