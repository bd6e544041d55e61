"""Typed configuration of the Guvusun decoder and its layout as parts.

The design: an embedding that adds a row chosen by a hash of (previous token, token) and is normalised
(``parts/embedding.py``: ``PairHashEmbedding``); layers that normalise AFTER the sum, x <- norm1(alpha x + mixer(x)),
x <- norm2(alpha x + ff(x)), followed by a per-layer token input x <- x + side_norm(proj(gelu(gate x) * table[token]))
(arrangement ``postnorm_residual``; ``parts/routed.py``: ``TokenTableGate``); one kind of mixer, ``latent_attention``
(``parts/attention.py``: ``LatentAttention``: queries with a plain and a rotated part per head, keys and values as two
products of one cached latent row per position plus a rotated key part shared by the heads, YaRN-scaled rotation
(``parts/position.py``: ``ComputedRope``), a sink with a learned score per head, a sigmoid gate per head; a layer with
``kv_from: j`` has no key projection and reads the rows layer j cached); a feed-forward of routed experts per layer
(``parts/routed.py``: ``RoutedExperts``: softmax router, correction added for the choice only, groups of neighbouring
experts of which the best are kept, identity experts) or none; a final norm and a head.

``config.json`` (key ``architecture``) gives every size and every constant that differs between models of the design.
Tensor names follow the checkpoint: ``embed``, ``bigram``, ``embed.norm``, ``side.embed``, ``head``, ``final.norm`` and
``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.side.*``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .kapudra import DEFAULT_MAX_POSITIONS, _int, _num, _obj
from .qwen2 import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .tutunex import _check_rot


@dataclass(frozen=True)
class GuvusunConfig:
    """The parsed ``config.json``; ``layers`` keeps each layer's object as read (validated)."""

    vocab: int
    width: int
    norm_eps: float
    alpha: float
    layers: Tuple[Dict[str, Any], ...]
    bigram: Optional[Tuple[int, int, int]] = None        # (buckets, mul_prev, mul_cur)
    side_dim: Optional[int] = None
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: tuple = ()

    architecture = "Guvusun"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "GuvusunConfig":
        if d.get("architecture", d.get("architectures", ["Guvusun"])) not in ("Guvusun", ["Guvusun"]):
            raise ConfigError("not a Guvusun configuration")
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("layers must be a non-empty list")
        for i, L in enumerate(layers):
            _check_layer(_obj(L, f"layers[{i}]"), f"layers[{i}]", i, layers)
        bigram = None
        emb = d.get("embedding")
        if emb is not None and _obj(emb, "embedding").get("bigram") is not None:
            b = _obj(emb["bigram"], "embedding.bigram")
            bigram = (_int(b, "buckets", "embedding.bigram", 1, 1 << 30), _int(b, "mul_prev", "embedding.bigram", 0, 1 << 30),
                      _int(b, "mul_cur", "embedding.bigram", 0, 1 << 30))
        side = d.get("token_side")
        return cls(
            vocab=_int(d, "vocab", "config"), width=_int(d, "width", "config"),
            norm_eps=_num(_obj(d.get("norm"), "norm"), "eps", "norm"),
            alpha=_num(d, "postln_alpha", "config", positive=False) if "postln_alpha" in d else 1.0, layers=tuple(layers),
            bigram=bigram, side_dim=_int(_obj(side, "token_side"), "dim", "token_side") if side is not None else None,
            max_positions=_int(d, "max_positions", "config") if "max_positions" in d else DEFAULT_MAX_POSITIONS)

    def to_dict(self) -> Dict[str, Any]:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "postln_alpha": self.alpha, "layers": list(self.layers)}
        if self.bigram is not None:
            out["embedding"] = {"bigram": {"buckets": self.bigram[0], "mul_prev": self.bigram[1], "mul_cur": self.bigram[2]}}
        if self.side_dim is not None:
            out["token_side"] = {"dim": self.side_dim}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out


_SHARED_KEYS = ("kv_rank", "rot_dim", "rot")


def _check_layer(L: Dict[str, Any], what: str, index: int, layers: List[Any]) -> None:
    kind = L.get("type")
    if kind != "latent_attention":
        raise ConfigError(f"{what}.type {kind!r} is not a mixer of this design (latent_attention)")
    m = _obj(L.get("mixer"), what + ".mixer")
    for key in ("heads", "dim", "vdim", "kv_rank"):
        _int(m, key, what + ".mixer")
    rot_dim = _int(m, "rot_dim", what + ".mixer", 0)
    _num(m, "scale", what + ".mixer")
    if m.get("rot") is not None:
        rot = _obj(m["rot"], what + ".mixer.rot")
        _check_rot(rot, max(rot_dim, 2), what + ".mixer.rot")
        if rot["dims"] > rot_dim:
            raise ConfigError(f"{what}.mixer.rot.dims {rot['dims']} exceeds the rotated part of {rot_dim} channels")
    src = m.get("kv_from")
    if src is not None:
        if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < index:
            raise ConfigError(f"{what}.mixer.kv_from {src!r} must name an earlier layer")
        other = layers[src] if isinstance(layers[src], dict) else {}
        om = other.get("mixer") if isinstance(other.get("mixer"), dict) else {}
        if om.get("kv_from") is not None:
            raise ConfigError(f"{what}.mixer.kv_from: layer {src} has no key projection of its own to share")
        if any(om.get(key) != m.get(key) for key in _SHARED_KEYS):
            raise ConfigError(f"{what}.mixer.kv_from: layer {src}'s cached rows have other sizes or another rotation")
    mlp = L.get("mlp")
    if mlp is not None:
        if _obj(mlp, what + ".mlp").get("kind") != "moe":
            raise ConfigError(f"{what}.mlp.kind {mlp.get('kind')!r} is not implemented (moe, or null for none)")
        _int(_obj(mlp.get("expert"), what + ".mlp.expert"), "ff", what + ".mlp.expert")
        r = _obj(mlp.get("router"), what + ".mlp.router")
        experts, top = _int(r, "experts", what + ".mlp.router"), _int(r, "top", what + ".mlp.router")
        identity = _int(r, "identity", what + ".mlp.router", 0) if r.get("identity") is not None else 0
        if r.get("scale") is not None:
            _num(r, "scale", what + ".mlp.router")
        count, keep = 1, 1
        if r.get("groups") is not None:
            g = _obj(r["groups"], what + ".mlp.router.groups")
            count = _int(g, "count", what + ".mlp.router.groups")
            keep = _int(g, "keep", what + ".mlp.router.groups", 1, count)
        if (experts + identity) % count:
            raise ConfigError(f"{what}.mlp.router: {experts + identity} outputs do not form {count} equal groups")
        if top > keep * ((experts + identity) // count):
            raise ConfigError(f"{what}.mlp.router: {top} choices do not fit {keep} groups of {(experts + identity) // count}")


def _mixer_spec(m: Dict[str, Any], width: int, eps: float) -> Tuple[PartSpec, Optional[PartSpec]]:
    """(mixer, position encoding of the layer)."""
    rot = m.get("rot")
    position = None
    if rot is not None and m["rot_dim"] > 0:
        position = PartSpec("rope_computed", dict(rotary_dim=rot["dims"], theta=float(rot["base"]),
                                                  scaling=dict(rot["scaling"]) if rot.get("scaling") is not None else None))
    return PartSpec("latent_attention", dict(
        hidden_size=width, num_heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"], v_head_dim=m["vdim"],
        kv_rank=m["kv_rank"], scale=float(m["scale"]), eps=eps, sink=True, gate=True, own_kv=m.get("kv_from") is None)), position


def _experts_spec(mlp: Dict[str, Any], width: int) -> PartSpec:
    r = mlp["router"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    return PartSpec("routed_experts", dict(
        hidden_size=width, expert_size=mlp["expert"]["ff"], experts=r["experts"], top=r["top"],
        identity=r.get("identity") or 0, groups=groups["count"], keep=groups["keep"],
        scale=float(r["scale"]) if r.get("scale") is not None else 1.0, correction=True, activation="silu"))


def guvusun_schedule(layers) -> List[ScheduleEntry]:
    """Every layer once, in order; a layer with ``kv_from: j`` reads the cache that layer j's entry wrote."""
    return [ScheduleEntry(i, cache_from=L["mixer"].get("kv_from")) for i, L in enumerate(layers)]


def guvusun_model_spec(c: GuvusunConfig) -> ModelSpec:
    norm = lambda: PartSpec("rmsnorm", dict(size=c.width, eps=c.norm_eps, tensor=""))
    layers = []
    for i, L in enumerate(c.layers):
        mixer, position = _mixer_spec(L["mixer"], c.width, c.norm_eps)
        parts = {"mixer": mixer, "mixer_norm": norm()}
        if L.get("mlp") is not None:
            parts.update({"feed_forward": _experts_spec(L["mlp"], c.width), "feed_forward_norm": norm()})
        if c.side_dim is not None:
            parts.update({"side": PartSpec("token_table_gate", dict(
                hidden_size=c.width, dim=c.side_dim, table="side.embed", first_column=i * c.side_dim, vocab_size=c.vocab)),
                "side_norm": norm()})
        layers.append(LayerSpec(f"l{i}", "postnorm_residual", parts, position,
                                names={"mixer": "mix", "mixer_norm": "norm1", "feed_forward": "mlp", "feed_forward_norm": "norm2",
                                       "side": "side", "side_norm": "side.norm"},
                                arrangement_params={"alpha": c.alpha}))
    extra = {}
    if c.side_dim is not None:
        extra["side.embed"] = ((c.vocab, len(c.layers) * c.side_dim), "matrix", "normal")
    b = c.bigram
    embedder = PartSpec("pair_hash_embedding", dict(
        vocab_size=c.vocab, hidden_size=c.width, table="embed", pair="bigram" if b is not None else None,
        buckets=b[0] if b is not None else 0, mul_prev=b[1] if b is not None else 0, mul_cur=b[2] if b is not None else 0,
        norm="embed.norm", eps=c.norm_eps))
    return ModelSpec(
        architecture=c.architecture, hidden_size=c.width, vocab_size=c.vocab, max_positions=c.max_positions,
        embedding_name="embed", layers=layers, schedule=guvusun_schedule(c.layers), final_norm=norm(),
        final_norm_name="final.norm", head_name="head", bare_tensor_names=True, extra_tensors=extra, embedder=embedder)
