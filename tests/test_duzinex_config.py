"""Configuration of the Duzinex decoder, its schedule and weight list, and the cache features it brought: several
caches for one run of a layer, values of another size than keys, a window that keeps the first tokens' pages."""
import pytest
import torch

from spissa_b200.cache import CacheManager
from spissa_b200.config import ConfigError, DuzinexConfig, config_from_dict
from spissa_b200.engine.model import Model
from spissa_b200.parts import CacheBundle, KVCacheRequest, StateRequest

CFG = dict(
    architecture="Duzinex", vocab=90, width=40, embedding=dict(scale=2.5), norm=dict(eps=1e-4),
    layers=[
        dict(type="mingru", mixer=dict(width=24), mlp=dict(kind="dense", ff=56)),
        dict(type="attention", mixer=dict(heads=4, kv_heads=2, dim=6, vdim=10, diff=0.25, scale=0.4, softcap=9.0,
                                          mask=dict(size=70, keep_first=65), rot=dict(dims=4, base=1000.0)), mlp=None),
        dict(type="retention", mixer=dict(heads=2, dim=8, vdim=12, decay=[0.9, 0.99]), mlp=dict(kind="dense", ff=16)),
    ],
    loop=dict(start=1, stop=3, times=3))


def test_registry_finds_the_architecture_by_its_singular_key():
    cfg = config_from_dict(CFG)
    assert isinstance(cfg, DuzinexConfig)
    assert cfg.to_dict() == CFG
    assert config_from_dict(DuzinexConfig(**{**cfg.__dict__, "raw": None}).to_dict()).layers == cfg.layers


def test_schedule_runs_the_loop_with_caches_of_its_own_and_takes_the_embedding_in_again():
    spec = config_from_dict(CFG).to_spec()
    assert [(e.layer, e.adds_embedding) for e in spec.schedule] == \
        [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False)]
    assert len({e.cache for e in spec.schedule}) == 7 and all(e.writes_cache for e in spec.schedule)
    one = config_from_dict({**CFG, "loop": None}).to_spec()
    assert [(e.layer, e.adds_embedding) for e in one.schedule] == [(0, False), (1, False), (2, False)]
    everything = config_from_dict({**CFG, "loop": dict(start=0, stop=3, times=2)}).to_spec()
    assert [(e.layer, e.adds_embedding) for e in everything.schedule] == \
        [(0, False), (1, False), (2, False), (0, True), (1, False), (2, False)]


def test_weight_list():
    model = Model(config_from_dict(CFG).to_spec())
    shapes = {s.name: tuple(s.shape) for s in model.weight_specs()}
    assert shapes["embed"] == (90, 40) and shapes["final.norm.alpha"] == () and shapes["final.norm.b"] == (40,)
    assert shapes["l0.shift"] == (40,) and shapes["l0.mix.z.b"] == (24,) and shapes["l0.mlp.act"] == (4,)
    assert shapes["l1.mix.q"] == (48, 40) and shapes["l1.mix.k"] == (24, 40) and shapes["l1.mix.v"] == (20, 40)
    assert shapes["l1.mix.o"] == (40, 40) and shapes["l1.mix.o.b"] == (40,) and shapes["l1.mix.lk2"] == (6,)
    assert "l1.mlp.up" not in shapes and "l1.norm2" not in shapes
    assert shapes["l2.mix.g"] == (24, 40) and shapes["l2.mix.o"] == (40, 24)
    assert "lm_head.weight" not in shapes


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="lstm"), "known mixers"),
    (lambda c: c["layers"][2]["mixer"].update(decay=[0.9]), "decay"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=8), "rot.dims"),
    (lambda c: c["layers"][0]["mlp"].update(kind="experts"), "kind"),
    (lambda c: c["loop"].update(stop=4), "loop"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_bad_configurations_are_refused_with_the_field_named(change, word):
    import copy
    bad = copy.deepcopy(CFG)
    change(bad)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(bad)


def test_a_run_with_several_caches_and_a_window_that_keeps_its_first_pages():
    model = Model(config_from_dict(CFG).to_spec())
    reqs = model.cache_requests()
    assert reqs[1] == CacheBundle((("mixer", KVCacheRequest(2, 12, 70, v_head_dim=10, keep_first=65)),
                                   ("shift", StateRequest((40,), torch.float32))))
    cache = CacheManager(reqs, max_tokens=64 * 8, max_seqs=2, page_size=64, dtype=torch.float32, device="cpu")
    (kv,) = cache.kv_groups.values()
    assert kv.k.shape == (3, 8, 2, 64, 12) and kv.v.shape == (3, 8, 2, 64, 10)          # three passes, caches of their own
    assert sorted(tuple(g.state.shape) for g in cache.state_groups.values()) == [(1, 2, 24), (3, 2, 2, 8, 12), (7, 2, 40)]
    slot = cache.acquire()
    for n in (300, 1, 1):
        res = cache.reserve([(slot, n)])
        cache.commit(res)
    held = [p is not None for p in cache.seqs[slot].pages[kv.name]]
    # 302 tokens: the next query at 302 sees keys from 233 on (page 3) and the first 65 (pages 0 and 1)
    assert held == [True, True, False, True, True]
    cache.check()
    cache.release(slot)
    assert kv.pages.free_count == 8
