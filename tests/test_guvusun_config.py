"""The Guvusun configuration on the CPU: what is read, what is refused, the layout as parts, the tensor names, the cache."""
import copy

import pytest
import torch

import guvusun_cases as gc
from coheryn_ai_studio_b200.config import ConfigError, architecture_for
from coheryn_ai_studio_b200.config.guvusun import GuvusunConfig, guvusun_model_spec
from coheryn_ai_studio_b200.parts.base import FixedState, PagedKV, Runtime
from coheryn_ai_studio_b200.parts.model import DecoderModel


def model_of(cfg):
    return DecoderModel(guvusun_model_spec(GuvusunConfig.from_dict(cfg)), Runtime(torch.float32, torch.device("cpu")))


def test_round_trip_and_registry():
    for cfg, _ in gc.CASES.values():
        c = GuvusunConfig.from_dict(cfg)
        assert GuvusunConfig.from_dict(c.to_dict()) == c
        assert architecture_for(cfg).name == "Guvusun"


def test_layout_and_tensor_names():
    m = model_of(gc.G1)
    names = set(m.tensor_specs())
    assert {"embed", "bigram", "embed.norm", "side.embed", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.dkv",
            "l0.mix.dkv.norm", "l0.mix.uk", "l0.mix.uv", "l0.mix.sink", "l0.mix.g", "l0.mix.o", "l0.mlp.router", "l0.mlp.correction",
            "l0.mlp.e5.down", "l0.side.gate", "l0.side.proj", "l0.side.norm", "l2.mlp.e3.gate"} <= names
    assert "l1.mix.dkv" not in names and "l1.norm2" not in names and "l1.mlp.router" not in names and "l0.mlp.e6.gate" not in names
    specs = m.tensor_specs()
    assert specs["bigram"].shape == (258, 64) and specs["side.embed"].shape == (300, 24) and specs["l0.mlp.router"].shape == (8, 64)
    assert specs["l1.mix.uv"].shape == (2 * 48, 32) and specs["l2.mix.q"].shape == (4 * (24 + 32), 64)
    assert [e.cache_from for e in m.spec.schedule] == [None, 0, None]
    needs = m.cache_requirements()
    assert needs == [PagedKV(1, 48, None, 0), None, PagedKV(1, 96, None, 0), FixedState((1,), torch.int32)]
    assert model_of(gc.G2).cache_requirements() == [PagedKV(1, 26, None, 0), PagedKV(1, 16, None, 0), None, None]   # no pair row: no state
    assert [e.cache_from for e in model_of(gc.G2).spec.schedule] == [None, None, 0, 1]


def test_cache_manager_takes_the_models_own_state():
    from coheryn_ai_studio_b200.cache import CacheManager
    m = model_of(gc.G1)
    cm = CacheManager(m.cache_requirements(), [e.cache_from for e in m.spec.schedule], torch.float32, torch.device("cpu"),
                      page_size=8, num_pages=6, max_requests=2)
    caches = cm.layer_caches()
    assert len(caches) == 4 and caches[3].kind == "state" and caches[3].state.shape == (2, 1) and caches[3].state.dtype == torch.int32
    assert caches[0].v is None and caches[1].k is caches[0].k and not caches[1].writes
    assert cm.bytes_per_token() == (48 + 96) * 4 and not cm.prefix_reuse


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="attention"), "not a mixer"),
    (lambda c: c["layers"][1]["mixer"].update(kv_from=1), "earlier layer"),
    (lambda c: c["layers"][1]["mixer"].update(kv_from=0, kv_rank=16), "other sizes"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "no key projection"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "do not fit"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=3), "equal groups"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "not implemented"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "dims"),
    (lambda c: c.update(vocab=0), "vocab"),
])
def test_refusals(change, message):
    cfg = copy.deepcopy(gc.G1)
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        GuvusunConfig.from_dict(cfg)
