"""The Zegelix configuration on the CPU: what is read, what is refused, the layout as parts, the tensor names, the cache,
and the plain implementation's own pieces against hand-made cases."""
import copy

import numpy as np
import pytest
import torch

import plain_zegelix as plain
import zegelix_cases as zc
from coheryn_ai_studio_b200.config import ConfigError, architecture_for
from coheryn_ai_studio_b200.config.zegelix import ZegelixConfig, zegelix_model_spec, zegelix_schedule
from coheryn_ai_studio_b200.parts.base import FixedState, PagedKV, Runtime
from coheryn_ai_studio_b200.parts.model import DecoderModel


def model_of(cfg):
    return DecoderModel(zegelix_model_spec(ZegelixConfig.from_dict(cfg)), Runtime(torch.float32, torch.device("cpu")))


def test_round_trip_and_registry():
    for cfg, _ in zc.CASES.values():
        c = ZegelixConfig.from_dict(cfg)
        assert ZegelixConfig.from_dict(c.to_dict()) == c
        assert architecture_for(cfg).name == "Zegelix"


def test_layout_tensor_names_and_cache():
    m = model_of(zc.Z1)
    specs = m.tensor_specs()
    assert {"embed", "loop.in", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.q.b", "l0.mix.k.b", "l0.mix.v.b",
            "l0.mix.temp", "l0.mix.sink", "l0.mix.g", "l0.mix.o", "l0.mlp.router", "l0.mlp.router.b", "l0.mlp.e5.down",
            "l0.mlp.shared.gate", "l0.mlp.shared.sg", "l1.mix.y", "l1.mix.y.b", "l1.mix.x", "l1.mix.conv", "l1.mix.conv.b",
            "l1.mix.ra", "l1.mix.ri.b", "l1.mix.lam", "l1.mix.o", "l3.mlp.e2.up"} <= set(specs)
    assert "head" not in specs and "l2.norm2" not in specs and "l2.mlp.router" not in specs and "l1.mlp.shared.gate" not in specs
    assert specs["loop.in"].shape == (64, 128) and specs["l1.mix.ra"].shape == (4, 16, 16) and specs["l1.mix.conv"].shape == (64, 4)
    assert specs["l0.mix.g"].shape == (4 * 16, 64) and specs["l0.mix.v"].shape == (2 * 16, 64) and specs["l0.mlp.shared.sg"].shape == (1, 64)
    assert [(e.layer, e.inject.mix if e.inject else None) for e in m.spec.schedule] == [
        (0, None), (1, "loop.in"), (2, None), (1, "loop.in"), (2, None), (3, None)]
    needs = m.cache_requirements()
    assert needs[0] == (PagedKV(2, 32, None, 16), PagedKV(2, 32, None, 16, stride=8))
    assert needs[1] == FixedState((64 * 4,), torch.float32) and needs[3] == needs[1]       # every pass its own state
    assert needs[2] == (PagedKV(2, 16, None, 32), PagedKV(2, 16, None, 32, stride=4)) and needs[5] == FixedState((32 * 2,), torch.float32)
    assert "loop.in" not in model_of(zc.Z2).tensor_specs()
    assert [e.layer for e in model_of(zc.Z3).spec.schedule] == [0, 1, 0, 1, 0, 1]
    assert zegelix_schedule(3, None) == zegelix_schedule(3, None) and len(zegelix_schedule(5, (2, 4, 3))) == 2 + 6 + 1


@pytest.mark.parametrize("path,value", [
    (("layers", 0, "type"), "conv"), (("layers", 1, "mixer", "blocks"), 3), (("layers", 0, "mixer", "kv_heads"), 3),
    (("layers", 0, "mixer", "rot", "dims"), 34), (("layers", 0, "mixer", "rot", "dims"), 7), (("layers", 0, "mixer", "vdim"), 15),
    (("layers", 0, "mixer", "mask", "pool"), 0), (("layers", 0, "mlp", "kind"), "dense"), (("layers", 0, "mlp", "router", "top"), 7),
    (("loop", "stop"), 1), (("loop", "times"), 0), (("layers", 1, "mixer", "conv"), 17), (("norm", "eps"), -1.0),
])
def test_refusals(path, value):
    cfg = copy.deepcopy(zc.Z1)
    o = cfg
    for key in path[:-1]:
        o = o[key]
    o[path[-1]] = value
    with pytest.raises(ConfigError):
        ZegelixConfig.from_dict(cfg)


def test_rows_per_page_of_a_block_cache():
    assert PagedKV(1, 8, stride=3).rows_per_page(16) == 6 and PagedKV(1, 8, stride=16).rows_per_page(16) == 1
    assert PagedKV(1, 8, stride=40).rows_per_page(16) == 1 and PagedKV(1, 8).rows_per_page(16) == 16
    # every block's row, found from its last position's page, is inside the page and no two blocks share one
    for page, pool in ((16, 3), (8, 3), (16, 16), (16, 40), (8, 1), (64, 5)):
        rows = PagedKV(1, 8, stride=pool).rows_per_page(page)
        seen = set()
        for b in range(200):
            last = b * pool + pool - 1
            lp = last // page
            row = b - (lp * page) // pool
            assert 0 <= row < rows and (lp, row) not in seen
            seen.add((lp, row))


def test_plain_window_and_blocks_on_a_hand_made_case():
    """One head, one channel of keys: scores are known, so are the sets of seen positions and blocks."""
    T, size, pool = 12, 3, 4
    q = np.ones((T, 1, 1)); k = np.zeros((T, 1, 1)); v = np.eye(T).reshape(T, 1, T)
    out = plain.attend_window_and_blocks(q, k, v, size, pool, 1.0, None)[:, 0]       # equal scores: the mean of what is seen
    for i in range(T):
        blocks = [b for b in range(T // pool) if b * pool + pool - 1 <= i - size]
        tokens = [j for j in range(T) if 0 <= i - j < size]
        want = np.zeros(T)
        for b in blocks:
            want[b * pool:(b + 1) * pool] += 1.0 / pool
        want[tokens] += 1.0
        assert np.allclose(out[i], want / (len(blocks) + len(tokens))), i
    assert plain.visible_blocks(5, 3, 4) == 0 and plain.visible_blocks(6, 3, 4) == 1 and plain.visible_blocks(10, 3, 4) == 2
    # the sink takes weight and brings no value
    out_sink = plain.attend_window_and_blocks(q, k, v, size, pool, 1.0, None, sink=np.array([0.0]))[:, 0]
    assert np.allclose(out_sink[0].sum(), 0.5) and np.allclose(out_sink[11].sum(), 5.0 / 6.0)


def test_plain_recurrence_on_a_hand_made_case():
    """With the gates' matrices zero, r = i = 1/2 everywhere: a is one number per channel and the scan a geometric sum."""
    C, T = 4, 9
    W = {"m.y": np.zeros((C, 3)), "m.y.b": np.full(C, 10.0), "m.x": np.zeros((C, 3)), "m.x.b": np.arange(1.0, C + 1),
         "m.conv": np.array([[0.0, 1.0]] * C), "m.conv.b": np.zeros(C), "m.ra": np.zeros((2, 2, 2)), "m.ra.b": np.zeros((2, 2)),
         "m.ri": np.zeros((2, 2, 2)), "m.ri.b": np.zeros((2, 2)), "m.lam": np.array([-3.0, 0.0, 1.0, 5.0]), "m.o": np.eye(C)}
    out = plain.gated_linear_recurrence(np.zeros((T, 3)), W, "m.", {})
    a = np.exp(-8.0 * 0.5 * np.log1p(np.exp(W["m.lam"])))
    for t in range(T):
        want = np.sqrt(1 - a * a) * 0.5 * W["m.x.b"] * (1 - a ** (t + 1)) / (1 - a) * plain.gelu_tanh(10.0)
        assert np.allclose(out[t], want), t
