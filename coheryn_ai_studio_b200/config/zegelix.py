"""Typed configuration of the Zegelix decoder and its layout as parts.

The design: an embedding multiplied by a constant; pre-norm layers x <- x + mixer(norm(x)), x <- x + ff(norm(x))
(arrangement ``prenorm_residual``; the feed-forward may be absent) with two kinds of mixer, chosen per layer by ``type``:

* ``rglru``      a gated linear recurrence per channel behind a short convolution, beside a GELU branch
                 (``parts/recurrent.py``: ``GatedLinearRecurrence``);
* ``attention``  grouped-query attention over a sliding window whose older keys are seen as means of blocks
                 (``parts/attention.py``: ``PooledWindowAttention``): biases on q, k and v, a rotation of the first
                 ``rot.dims`` channels of queries and keys, values rotated over all their channels and the output turned
                 back, a learned factor per head on the scores, a cap on them, a learned sink per head, an output gate;

a feed-forward of routed experts (``parts/routed.py``: ``RoutedExperts`` with ``top_softmax`` selection, a bias on the
router and a gated shared expert); a span of the layers may run several times in a row with the same weights, each pass
with caches of its own and, right before its first layer, the stream replaced by M [x ; embedding output]
(``StreamInject.mix``); a final norm; the logits from the embedding table itself, times a constant.

``config.json`` (key ``architecture``) gives every size and every constant that differs between models of the design.
Tensor names follow the checkpoint: ``embed``, ``loop.in``, ``final.norm`` and ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mix.*``, ``l<i>.mlp.*``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .kapudra import DEFAULT_MAX_POSITIONS, _int, _num, _obj
from .qwen2 import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, StreamInject

RECURRENCE_RATE = 8.0         # log a = -8 r softplus(lam): fixed by the design
EXPERT_ACTIVATION = "swish_clamped"


@dataclass(frozen=True)
class ZegelixConfig:
    """The parsed ``config.json``; ``layers`` keeps each layer's object as read (validated)."""

    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    logit_scale: float
    layers: Tuple[Dict[str, Any], ...]
    loop: Optional[Tuple[int, int, int]] = None      # (start, stop, times)
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: tuple = ()

    architecture = "Zegelix"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ZegelixConfig":
        if d.get("architecture", d.get("architectures", ["Zegelix"])) not in ("Zegelix", ["Zegelix"]):
            raise ConfigError("not a Zegelix configuration")
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("layers must be a non-empty list")
        for i, L in enumerate(layers):
            _check_layer(_obj(L, f"layers[{i}]"), f"layers[{i}]")
        loop = None
        if d.get("loop") is not None:
            lo = _obj(d["loop"], "loop")
            start, stop = _int(lo, "start", "loop", 0, len(layers)), _int(lo, "stop", "loop", 0, len(layers))
            if not start < stop:
                raise ConfigError(f"loop: layers {start}..{stop} are no span")
            loop = (start, stop, _int(lo, "times", "loop", 1, 1 << 10))
        return cls(
            vocab=_int(d, "vocab", "config"), width=_int(d, "width", "config"),
            embedding_scale=_num(_obj(d.get("embedding"), "embedding"), "scale", "embedding"),
            norm_eps=_num(_obj(d.get("norm"), "norm"), "eps", "norm"),
            logit_scale=_num(d, "logit_scale", "config") if d.get("logit_scale") is not None else 1.0,
            layers=tuple(layers), loop=loop,
            max_positions=_int(d, "max_positions", "config") if "max_positions" in d else DEFAULT_MAX_POSITIONS)

    def to_dict(self) -> Dict[str, Any]:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
               "logit_scale": self.logit_scale, "layers": list(self.layers)}
        if self.loop is not None:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out


def _check_expert(o: Dict[str, Any], what: str) -> None:
    _int(o, "ff", what)
    _num(o, "limit", what)


def _check_layer(L: Dict[str, Any], what: str) -> None:
    kind = L.get("type")
    m = _obj(L.get("mixer"), what + ".mixer")
    if kind == "rglru":
        width, blocks = _int(m, "width", what + ".mixer"), _int(m, "blocks", what + ".mixer")
        if width % blocks:
            raise ConfigError(f"{what}.mixer: {width} channels do not form {blocks} equal blocks")
        _int(m, "conv", what + ".mixer", 1, 16)
    elif kind == "attention":
        for key in ("heads", "kv_heads", "dim", "vdim"):
            _int(m, key, what + ".mixer")
        if m["heads"] % m["kv_heads"]:
            raise ConfigError(f"{what}.mixer: {m['heads']} heads do not divide into {m['kv_heads']} kv_heads")
        if m["vdim"] % 2:
            raise ConfigError(f"{what}.mixer.vdim {m['vdim']}: rotated values need an even number of channels")
        _num(m, "scale", what + ".mixer")
        _num(m, "softcap", what + ".mixer")
        rot = _obj(m.get("rot"), what + ".mixer.rot")
        dims = _int(rot, "dims", what + ".mixer.rot", 2)
        if dims % 2 or dims > m["dim"]:
            raise ConfigError(f"{what}.mixer.rot.dims {dims} must be even and at most the head's {m['dim']} channels")
        if not _num(rot, "base", what + ".mixer.rot") > 1:
            raise ConfigError(f"{what}.mixer.rot.base must exceed 1")
        mask = _obj(m.get("mask"), what + ".mixer.mask")
        _int(mask, "size", what + ".mixer.mask")
        _int(mask, "pool", what + ".mixer.mask")
    else:
        raise ConfigError(f"{what}.type {kind!r} is not a mixer of this design (rglru, attention)")
    mlp = L.get("mlp")
    if mlp is not None:
        if _obj(mlp, what + ".mlp").get("kind") != "moe":
            raise ConfigError(f"{what}.mlp.kind {mlp.get('kind')!r} is not implemented (moe, or null for none)")
        _check_expert(_obj(mlp.get("expert"), what + ".mlp.expert"), what + ".mlp.expert")
        router = _obj(mlp.get("router"), what + ".mlp.router")
        experts, top = _int(router, "experts", what + ".mlp.router"), _int(router, "top", what + ".mlp.router")
        if top > experts:
            raise ConfigError(f"{what}.mlp.router: {top} choices among {experts} experts")
        if mlp.get("shared") is not None:
            _check_expert(_obj(mlp["shared"], what + ".mlp.shared"), what + ".mlp.shared")


def _mixer_spec(L: Dict[str, Any], width: int) -> Tuple[PartSpec, Optional[PartSpec]]:
    """(mixer, position encoding of the layer)."""
    m = L["mixer"]
    if L["type"] == "rglru":
        return PartSpec("gated_linear_recurrence", dict(hidden_size=width, width=m["width"], blocks=m["blocks"],
                                                        conv_taps=m["conv"], rate=RECURRENCE_RATE)), None
    rot, mask = m["rot"], m["mask"]
    position = PartSpec("rope_computed", dict(rotary_dim=rot["dims"], theta=float(rot["base"])))
    return PartSpec("pooled_window_attention", dict(
        hidden_size=width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], v_head_dim=m["vdim"],
        scale=float(m["scale"]), window=mask["size"], pool=mask["pool"], qkv_bias=True, rotate_values=True,
        value_base=float(rot["base"]), head_temps=True, softcap=float(m["softcap"]), sink=True, gate=True)), position


def _feed_forward_spec(mlp: Dict[str, Any], width: int) -> PartSpec:
    shared = mlp.get("shared")
    return PartSpec("routed_experts", dict(
        hidden_size=width, expert_size=mlp["expert"]["ff"], experts=mlp["router"]["experts"], top=mlp["router"]["top"],
        activation=EXPERT_ACTIVATION, activation_constant=float(mlp["expert"]["limit"]), selection="top_softmax",
        router_bias=True,
        shared=dict(size=shared["ff"], activation_constant=float(shared["limit"]), gate=True) if shared is not None else None))


def zegelix_schedule(n_layers: int, loop: Optional[Tuple[int, int, int]], mix: str = "loop.in") -> List[ScheduleEntry]:
    """The layers in order, the span [start, stop) ``times`` times in a row; the first layer of every pass has the
    stream mixed with the embedding output in front of it."""
    if loop is None:
        return [ScheduleEntry(i) for i in range(n_layers)]
    start, stop, times = loop
    order = [ScheduleEntry(i) for i in range(start)]
    for _ in range(times):
        order += [ScheduleEntry(i, inject=StreamInject(mix=mix) if i == start else None) for i in range(start, stop)]
    return order + [ScheduleEntry(i) for i in range(stop, n_layers)]


def zegelix_model_spec(c: ZegelixConfig) -> ModelSpec:
    norm = lambda: PartSpec("rmsnorm", dict(size=c.width, eps=c.norm_eps, tensor=""))
    layers = []
    for i, L in enumerate(c.layers):
        mixer, position = _mixer_spec(L, c.width)
        parts = {"mixer_norm": norm(), "mixer": mixer}
        if L.get("mlp") is not None:
            parts.update({"feed_forward_norm": norm(), "feed_forward": _feed_forward_spec(L["mlp"], c.width)})
        layers.append(LayerSpec(f"l{i}", "prenorm_residual", parts, position,
                                names={"mixer_norm": "norm1", "mixer": "mix", "feed_forward_norm": "norm2",
                                       "feed_forward": "mlp"}))
    extra = {"loop.in": ((c.width, 2 * c.width), "matrix", "normal")} if c.loop is not None else {}
    return ModelSpec(
        architecture=c.architecture, hidden_size=c.width, vocab_size=c.vocab, max_positions=c.max_positions,
        embedding_name="embed", layers=layers, schedule=zegelix_schedule(len(c.layers), c.loop), final_norm=norm(),
        final_norm_name="final.norm", head_name=None, embedding_scale=c.embedding_scale, logit_scale=c.logit_scale,
        bare_tensor_names=True, extra_tensors=extra)
