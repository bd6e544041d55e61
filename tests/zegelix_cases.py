"""Small Zegelix configurations of the tests (they differ from each other in every size and option), folders of seeded
random weights for them, and the comparison of engine rows with the plain implementation."""
from __future__ import annotations

import json
from typing import Dict, List

import numpy as np

import plain_zegelix as plain
from plain_qwen2 import read_safetensors

LOUD = dict(matrix_std=0.12, bias_std=0.4, norm_jitter=0.1, conv_std=0.5)


def _moe(ff, limit, experts, top, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


def _attention(heads, kv_heads, dim, vdim, rot_dims, base, size, pool, scale, softcap, mlp=None):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": {"dims": rot_dims, "base": base},
                      "mask": {"size": size, "pool": pool}, "scale": scale, "softcap": softcap}}


def _rglru(width, blocks, conv, mlp=None):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv}, "mlp": mlp}


# Z1: sizes that vector widths and tensor-core tiles divide.  The repeated span is the middle of the stack (a layer before
# it, one behind it), two attention layers with different windows and blocks, a layer without feed-forward, heads of
# 32 key and 16 value channels of which 16 turn.
Z1 = {
    "architecture": "Zegelix", "vocab": 300, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0}, "logit_scale": 0.5,
    "loop": {"start": 1, "stop": 3, "times": 2},
    "layers": [
        _attention(4, 2, 32, 16, 16, 1000.0, 24, 8, 0.21, 12.0, mlp=_moe(32, 0.7, 6, 2, shared=(48, 2.5))),
        _rglru(64, 4, 4, mlp=_moe(32, 1.5, 4, 1)),
        _attention(2, 2, 16, 32, 16, 50.0, 9, 4, 0.3, 30.0, mlp=None),
        _rglru(32, 1, 2, mlp=_moe(16, 1.0, 3, 3, shared=(16, 1.0))),
    ]}

# Z2: sizes that no vector width and no tile divides (a width of 100, heads of 20 and 14 channels of which 12 turn, blocks
# of 3 positions under pages of 16 and of 8, a window of 7, recurrences of 36 channels in 3 blocks, 101 ids); blocks longer
# than the window in the second attention layer; no repeated span; a router that chooses all of its experts.
Z2 = {
    "architecture": "Zegelix", "vocab": 101, "width": 100, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0}, "logit_scale": 1.0,
    "layers": [
        _rglru(36, 3, 2, mlp=_moe(50, 2.0, 5, 5)),
        _attention(3, 3, 20, 14, 12, 77.0, 7, 3, 0.3, 8.0, mlp=_moe(30, 0.5, 4, 2, shared=(10, 3.0))),
        _attention(6, 2, 10, 6, 2, 9.0, 5, 9, 0.4, 50.0, mlp=None),
    ]}

# Z3: the whole stack repeated three times; one key head under six query heads; blocks of ONE position (every position
# behind the window is seen, as its own mean) and a window of one; a convolution of one tap (no inputs kept); one block.
Z3 = {
    "architecture": "Zegelix", "vocab": 515, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 11.0}, "logit_scale": 2.5,
    "loop": {"start": 0, "stop": 2, "times": 3},
    "layers": [
        _rglru(96, 1, 1, mlp=_moe(64, 1.0, 8, 4, shared=(32, 0.25))),
        _attention(6, 1, 16, 48, 8, 10000.0, 1, 1, 0.25, 5.0, mlp=_moe(32, 4.0, 2, 1)),
    ]}

CASES = {"Z1": (Z1, 41), "Z2": (Z2, 42), "Z3": (Z3, 43)}


def make_folder(tmp_path, name: str, config=None, seed=None) -> str:
    from coheryn_ai_studio_b200.config.zegelix import ZegelixConfig
    from coheryn_ai_studio_b200.engine import write_random_model
    from coheryn_ai_studio_b200.weights import InitPolicy
    cfg, s = CASES[name] if config is None else (config, seed)
    d = str(tmp_path / f"zegelix_{name}")
    write_random_model(d, ZegelixConfig.from_dict(cfg), s, InitPolicy(**LOUD))
    return d


def read_model(folder: str):
    with open(f"{folder}/config.json") as f:
        config = json.load(f)
    return config, {k: np.asarray(v, dtype=np.float64) for k, v in read_safetensors(f"{folder}/model.safetensors").items()}


_rows: Dict[tuple, np.ndarray] = {}


def plain_rows(folder: str, tokens: List[int], rounded: bool = False) -> np.ndarray:
    key = (folder, tuple(tokens), rounded)
    if key not in _rows:
        config, w = read_model(folder)
        _rows[key] = plain.forward(tokens, w, config, rounded=rounded)
    return _rows[key]


# float32: only the order of sums differs.  bfloat16: the weights are the same bits, activations are rounded to eight bits
# of mantissa between the kernels; what that costs a row by itself is measured on the plain model's rounded twin, and an
# engine row may be a small factor further from the unrounded row than the twin is (``replay.bf16_excess``).  A router's
# choice between two experts whose logits nearly tie can fall the other way after rounding, in the twin and in the engine
# at different rows; such a row is far from the unrounded one.  So over the rows of a test: the median within the bound,
# at most one row in ten (or two) beyond one and a half bounds.
TOL_F32 = 2e-4
WORST = {"float32": 0.0, "bfloat16": 0.0}


def check_rows(rows: Dict[tuple, np.ndarray], folder: str, sequences: Dict[str, List[int]], dtype: str, label: str = ""):
    from replay import bf16_excess
    assert rows, "nothing was compared"
    excesses = []
    for (rid, pos), row in sorted(rows.items()):
        ref = plain_rows(folder, sequences[rid])[pos]
        if dtype == "float32":
            d = np.abs(row.astype(np.float64) - ref).max()
            WORST[dtype] = max(WORST[dtype], float(d))
            assert d <= TOL_F32 * max(1.0, float(np.std(ref))), f"{label} {rid}@{pos}: |d| = {d:.3e}"
        else:
            twin = plain_rows(folder, sequences[rid], rounded=True)[pos]
            excesses.append((bf16_excess(row, ref.astype(np.float32), twin.astype(np.float32)), rid, pos))
    if excesses:
        values = np.array([e[0] for e in excesses])
        WORST[dtype] = max(WORST[dtype], float(np.median(values)))
        far = int((values > 1.5).sum())
        assert np.median(values) <= 1.0, f"{label}: median {np.median(values):.2f} of the bfloat16 bound"
        assert far <= max(2, len(values) // 10), f"{label}: {far} of {len(values)} rows beyond 1.5 bounds (worst {max(excesses)})"


def noisy_replay(folder: str, dtype: str, max_tokens: int, model, max_requests: int = 4, page_size: int = 16, **kw):
    """The replay harness with the state slots full of noise as well as the pages."""
    from replay import Replay
    r = Replay(folder, dtype, max_tokens=max_tokens, model=model, max_requests=max_requests, page_size=page_size, **kw)
    for t in r.cache.state_tensors():
        t.normal_(0.0, 4.0)
    return r


def prompt(seed: int, n: int, vocab: int) -> List[int]:
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()
