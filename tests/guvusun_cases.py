"""Small Guvusun configurations of the tests (they differ from each other in every size and option), folders of seeded
random weights for them, and the comparison of engine rows with the plain implementation."""
from __future__ import annotations

import json
from typing import Dict, List

import numpy as np

import plain_guvusun as plain
from plain_qwen2 import read_safetensors

LOUD = dict(matrix_std=0.12, bias_std=0.4, norm_jitter=0.1, conv_std=0.5)


def _rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def _moe(ff, experts, top, identity=0, groups=None, scale=1.0):
    r = {"experts": experts, "top": top, "identity": identity, "scale": scale}
    if groups is not None:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r}


def _layer(heads, dim, rot_dim, vdim, kv_rank, scale, rot, kv_from=None, mlp=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "rot": rot}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


# G1: sizes the tensor-core kernels take (cached rows of 48 and 96 channels).  A pair row in the embedding, a token input
# per layer, a layer that reads the first one's rows with other head counts and sizes, a layer without feed-forward,
# identity experts, groups of which half are kept, one choice among four experts without groups.
_R1 = _rot(16, 1000.0, (4.0, 64, 8.0, 1.0))
G1 = {
    "architecture": "Guvusun", "vocab": 300, "width": 64, "norm": {"eps": 1e-5}, "postln_alpha": 1.7,
    "embedding": {"bigram": {"buckets": 257, "mul_prev": 31, "mul_cur": 5}}, "token_side": {"dim": 8},
    "layers": [
        _layer(4, 16, 16, 16, 32, 0.21, _R1, mlp=_moe(32, 6, 3, identity=2, groups=(4, 2), scale=1.5)),
        _layer(2, 32, 16, 48, 32, 0.17, _R1, kv_from=0, mlp=None),
        _layer(4, 24, 32, 16, 64, 0.13, _rot(32, 50.0), mlp=_moe(48, 4, 1)),
    ]}

# G2: sizes that no vector width and no tensor-core tile divides (a width of 100, latent rows of 20 and 12 channels, rotated
# parts of 6 and 4, values of 10, 30 and 9, 50 expert channels, 101 ids); no pair row and no token input; the stream's factor
# is 1; a router whose choices are all of its experts; two layers that read earlier layers' rows, one of them the last.
_R2 = _rot(6, 77.0, (2.0, 16, 4.0, 0.5))
G2 = {
    "architecture": "Guvusun", "vocab": 101, "width": 100, "norm": {"eps": 1e-6}, "postln_alpha": 1.0,
    "layers": [
        _layer(3, 12, 6, 10, 20, 0.3, _R2, mlp=_moe(50, 5, 2, identity=1, groups=(3, 2), scale=2.5)),
        _layer(1, 20, 4, 30, 12, 0.25, _rot(4, 9.0), mlp=None),
        _layer(5, 7, 6, 9, 20, 0.35, _R2, kv_from=0, mlp=_moe(50, 3, 3)),
        _layer(2, 11, 4, 13, 12, 0.2, _rot(4, 9.0), kv_from=1, mlp=_moe(30, 2, 1, identity=2, groups=(2, 1), scale=0.7)),
    ]}

# G3: twenty heads over the one cached row (more than a decode CTA's row tile holds), multipliers beyond the buckets, a rotated
# part of which only half turns, rows of 64 channels, eight experts in two groups of which one is kept.
G3 = {
    "architecture": "Guvusun", "vocab": 515, "width": 128, "norm": {"eps": 1e-6}, "postln_alpha": 3.0,
    "embedding": {"bigram": {"buckets": 97, "mul_prev": 1000003, "mul_cur": 389}}, "token_side": {"dim": 16},
    "layers": [
        _layer(20, 16, 16, 16, 48, 0.2, _rot(8, 10000.0), mlp=_moe(64, 8, 4, groups=(2, 1), scale=2.0)),
        _layer(20, 8, 16, 8, 48, 0.25, _rot(8, 10000.0), kv_from=0, mlp=_moe(32, 8, 2, identity=4, groups=(3, 2), scale=1.0)),
    ]}

CASES = {"G1": (G1, 31), "G2": (G2, 32), "G3": (G3, 33)}


def make_folder(tmp_path, name: str, config=None, seed=None) -> str:
    from coheryn_ai_studio_b200.config.guvusun import GuvusunConfig
    from coheryn_ai_studio_b200.engine import write_random_model
    from coheryn_ai_studio_b200.weights import InitPolicy
    cfg, s = CASES[name] if config is None else (config, seed)
    d = str(tmp_path / f"guvusun_{name}")
    write_random_model(d, GuvusunConfig.from_dict(cfg), s, InitPolicy(**LOUD))
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
# choice between two experts whose scores nearly tie can fall the other way after rounding, in the twin and in the engine
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
        if t.dtype.is_floating_point:
            t.normal_(0.0, 4.0)
        else:
            t.random_(0, 90)
    return r


def prompt(seed: int, n: int, vocab: int) -> List[int]:
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()
