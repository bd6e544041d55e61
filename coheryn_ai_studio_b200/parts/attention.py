"""Grouped-query causal attention over cache pages.

Formulas as the reference runs them (crates/coheryn-engine/src/inference.rs:450-508,
crates/coheryn-engine/src/cpu.rs:133-210): q, k, v = W x + b; rotate q and k by
position; append k, v to the cache; for head h of group g = h // (heads // kv_heads),
s_t = (q_h . K[t, g]) * scale over the cached positions t <= p, softmax in float32,
o_h = sum_t P_t V[t, g]; y = W_o o (+ b_o).  A ``window`` keeps only the last
``window`` positions (t > p - window).
"""
from __future__ import annotations

import types
from typing import Dict, Optional

import torch

from .. import ops
from ..config.spec import PartSpec
from ..weights.spec import TensorSpec
from .base import LayerCache, Mixer, PagedKV, Position, Runtime, StepContext, register_mixer


class Attention(Mixer):
    def __init__(self, runtime: Runtime, hidden_size: int, num_heads: int, num_kv_heads: int,
                 head_dim: int, qkv_bias: bool, o_bias: bool, window: Optional[int], scale: float,
                 position: Optional[Position] = None):
        super().__init__(runtime)
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads do not divide into {num_kv_heads} kv heads")
        if window is not None and window < 1:
            raise ValueError("an attention window must hold at least one position")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.head_dim, self.qkv_bias, self.o_bias = head_dim, bool(qkv_bias), bool(o_bias)
        self.window, self.scale, self.position = window, float(scale), position
        self.q_size = num_heads * head_dim
        self.kv_size = num_kv_heads * head_dim
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = None

    def cache_requirement(self):
        return PagedKV(self.num_kv_heads, self.head_dim, self.window)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        H = self.hidden_size
        specs = {
            "q_proj.weight": TensorSpec((self.q_size, H)),
            "k_proj.weight": TensorSpec((self.kv_size, H)),
            "v_proj.weight": TensorSpec((self.kv_size, H)),
            "o_proj.weight": TensorSpec((H, self.q_size)),
        }
        if self.qkv_bias:
            specs["q_proj.bias"] = TensorSpec((self.q_size,), role="vector", init="bias")
            specs["k_proj.bias"] = TensorSpec((self.kv_size,), role="vector", init="bias")
            specs["v_proj.bias"] = TensorSpec((self.kv_size,), role="vector", init="bias")
        if self.o_bias:
            specs["o_proj.bias"] = TensorSpec((H,), role="vector", init="bias")
        return specs

    def bind(self, tensors):
        # One matrix product for q, k and v: rows of the three matrices stacked.
        self.w_qkv = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"],
                                tensors["v_proj.weight"]], dim=0).contiguous()
        if self.qkv_bias:
            biases = [tensors["q_proj.bias"], tensors["k_proj.bias"], tensors["v_proj.bias"]]
            dt = torch.float32 if any(b.dtype == torch.float32 for b in biases) else biases[0].dtype
            self.b_qkv = torch.cat([b.to(dt) for b in biases]).contiguous()
        self.w_o = tensors["o_proj.weight"]
        self.b_o = tensors.get("o_proj.bias")

    def _rotated_queries(self, x: torch.Tensor, step: StepContext, cache: LayerCache) -> torch.Tensor:
        """q, k, v of every row; k and v (rotated k) written to the cache; returns the rotated q
        [T, heads * head size] (possibly a column slice of a wider buffer).  Three ways to the same
        values: few rows (decoding) rotate and write in the product's own epilogue; a product whose K
        the many-rows kernel splits leaves the addition of its slices to the rotation kernel; otherwise
        the product, then the rotation kernel."""
        rot = self.position.rotary_dim if self.position is not None else 0
        cos_sin = self.position.cos_sin() if self.position is not None else None
        slots = step.slots[cache.group]
        if self.position is not None and ops.qkv_rope_ok(x, self.w_qkv, cache.k, rot, self.head_dim):
            return ops.qkv_rope_small(x, self.w_qkv, self.b_qkv, step.positions, cos_sin, slots, cache.k, cache.v,
                                      self.num_heads, self.num_kv_heads, self.head_dim, cache.page_size)
        count = ops.qkv_parts_count(x, self.w_qkv, cache.k, rot, self.head_dim) if self.position is not None else 0
        if count > 1:
            return ops.qkv_rope_parts(x, self.w_qkv, self.b_qkv, step.positions, cos_sin, slots, cache.k, cache.v,
                                      self.num_heads, self.num_kv_heads, self.head_dim, cache.page_size, count)
        qkv = ops.linear(x, self.w_qkv, self.b_qkv)
        ops.rope_kv_write(qkv, step.positions, cos_sin, slots, cache.k, cache.v, self.num_heads, self.num_kv_heads,
                          self.head_dim, rot, cache.page_size)
        return qkv[:, :self.q_size]

    def _queries_only(self, x: torch.Tensor, positions: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        """For an execution that reads keys and values another one wrote: only q is made and rotated."""
        b = self.b_qkv[:self.q_size] if self.b_qkv is not None else None
        q = ops.linear(x, self.w_qkv[:self.q_size], b)
        rot = self.position.rotary_dim if self.position is not None else 0
        cos_sin = self.position.cos_sin() if self.position is not None else None
        ops.rope_kv_write(q, positions, cos_sin, None, None, None, self.num_heads, 0, self.head_dim, rot, cache.page_size)
        return q

    def forward(self, x: torch.Tensor, step: StepContext, cache: LayerCache) -> torch.Tensor:
        self._check(cache)
        q = self._rotated_queries(x, step, cache) if cache.writes else self._queries_only(x, step.positions, cache)
        return self._attend_q(q, step, cache)

    supports_tail = True

    def forward_tail(self, x: torch.Tensor, step: StepContext, cache: LayerCache) -> Optional[torch.Tensor]:
        """Keys and values of every row go to the cache; only the wanted rows attend."""
        self._check(cache)
        rows, tail = step.tail_rows, step.tail
        if not cache.writes:   # nothing to write: the wanted rows alone make their queries
            if not tail.num_tokens:
                return None
            return self._attend_q(self._queries_only(ops.gather_rows(x, rows), tail.positions, cache), tail, cache)
        q = self._rotated_queries(x, step, cache)
        if not tail.num_tokens:
            return None
        return self._attend_q(ops.gather_rows(q, rows), tail, cache)

    @staticmethod
    def _check(cache) -> None:
        if cache is None or cache.kind != "paged":
            raise ValueError("attention needs a paged key/value cache")

    def _attend_q(self, q: torch.Tensor, step: StepContext, cache: LayerCache) -> torch.Tensor:
        """Attention of rotated queries over the cache, then the output projection."""
        if self.partial_output and ops.attention_oproj_ok(q, self.w_o, step, self.num_heads, self.num_kv_heads, self.head_dim):
            # a small decode batch: the splits of the attention are merged inside the projection's kernel,
            # and the heads' contributions go to the next norm as partial sums
            return ops.attention_oproj(q, cache.k, cache.v, step, cache.group, self.num_heads, self.num_kv_heads,
                                       self.head_dim, cache.page_size, self.window, self.scale, self.w_o, self.b_o)
        o = torch.empty((q.shape[0], self.q_size), dtype=q.dtype, device=q.device)
        ops.attention(q, o, cache.k, cache.v, step, cache.group, self.num_heads, self.num_kv_heads, self.head_dim,
                      cache.page_size, self.window, self.scale)
        return ops.linear(o, self.w_o, self.b_o, partial_ok=self.partial_output)


class DistanceBiasAttention(Mixer):
    """Grouped-query causal attention without rotation: the score of key j for query i is
    (q . k) * scale - slope_h * (i - j), slope_h = 2^(-slope_exponent (h + 1) / heads) for head h (None: no bias);
    a ``window`` keeps the keys with i - j < window; ordinary softmax.  ``qk_norm = "projection"`` divides the
    WHOLE query projection (all heads at once), and the whole key projection, by its root mean square and
    multiplies by a weight (``q.norm``, ``k.norm``) before the heads are split.  Values may have another head
    size than keys.  The output is multiplied by ``out_scale`` before the output projection."""

    output_parts = 1

    def __init__(self, runtime: Runtime, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 window: Optional[int], scale: float, v_head_dim: Optional[int] = None,
                 slope_exponent: Optional[float] = 8.0, qk_norm: Optional[str] = None, eps: float = 1e-6,
                 out_scale: float = 1.0):
        super().__init__(runtime)
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads do not divide into {num_kv_heads} kv heads")
        if window is not None and window < 1:
            raise ValueError("an attention window must hold at least one position")
        if qk_norm not in (None, "projection"):
            raise ValueError(f"qk_norm {qk_norm!r} is not built (None, 'projection')")
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.dk, self.dv = int(head_dim), int(v_head_dim if v_head_dim is not None else head_dim)
        self.window, self.scale, self.eps, self.out_scale = window, float(scale), float(eps), float(out_scale)
        self.slope_exponent, self.qk_norm = slope_exponent, qk_norm
        self.slopes = self.slopes_log2 = self.w_qkv = self.w_o = self.q_norm = self.k_norm = None

    def cache_requirement(self):
        return PagedKV(self.num_kv_heads, self.dk, self.window, None if self.dv == self.dk else self.dv)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        W, H, G, dk, dv = self.hidden_size, self.num_heads, self.num_kv_heads, self.dk, self.dv
        specs = {"q": TensorSpec((H * dk, W)), "k": TensorSpec((G * dk, W)), "v": TensorSpec((G * dv, W)),
                 "o": TensorSpec((W, H * dv))}
        if self.qk_norm is not None:
            specs["q.norm"] = TensorSpec((H * dk,), role="vector", init="norm")
            specs["k.norm"] = TensorSpec((G * dk,), role="vector", init="norm")
        return specs

    def bind(self, tensors):
        self.w_qkv = torch.cat([tensors["q"], tensors["k"], tensors["v"]], dim=0).contiguous()
        self.w_o = tensors["o"]
        if self.qk_norm is not None:
            qn, kn = tensors["q.norm"], tensors["k.norm"]
            dt = torch.float32 if torch.float32 in (qn.dtype, kn.dtype) else qn.dtype
            self.q_norm, self.k_norm = qn.to(dt).contiguous(), kn.to(dt).contiguous()
        if self.slope_exponent is not None:
            H = self.num_heads
            slopes = torch.tensor([2.0 ** (-float(self.slope_exponent) * (h + 1) / H) for h in range(H)], dtype=torch.float64)
            self.slopes = slopes.to(torch.float32).to(self.w_o.device)
            self.slopes_log2 = (slopes * ops.LOG2_E).to(torch.float32).to(self.w_o.device)

    def output_weights(self):
        return [self.w_o]

    def forward_into(self, x: torch.Tensor, step: StepContext, cache: LayerCache, out: torch.Tensor) -> None:
        o = torch.empty((x.shape[0], self.num_heads * self.dv), dtype=self.runtime.dtype, device=x.device)
        self.forward_open(x, step, cache, [o])
        ops.linear(o, self.w_o, out=out[0])

    def forward_open(self, x: torch.Tensor, step: StepContext, cache: LayerCache, outs) -> None:
        """The attention's output in front of the output product into ``outs[0]`` ([T, heads * dv], rows may be strided)."""
        Attention._check(cache)
        H, G, dk, dv = self.num_heads, self.num_kv_heads, self.dk, self.dv
        nq, nk = H * dk, G * dk
        if cache.writes:
            proj = ops.linear(x, self.w_qkv, out_dtype=torch.float32)
            slots = step.slots[cache.group]
        else:       # keys and values another execution wrote: only the queries are made
            if self.out_scale != 1.0:
                raise ValueError("an attention that multiplies its output keeps the constant on the values it writes; "
                                 "it cannot read another execution's cache")
            proj = torch.empty((x.shape[0], self.w_qkv.shape[0]), dtype=torch.float32, device=x.device)
            ops.linear(x, self.w_qkv[:nq], out=proj[:, :nq])
            slots = None
        q = ops.qk_norm_kv_write(proj[:, :nq], proj[:, nq:nq + nk], proj[:, nq + nk:], self.q_norm, self.k_norm, self.eps,
                                 slots, cache.k, cache.v, H, G, dk, dv, cache.page_size, self.runtime.dtype,
                                 v_scale=self.out_scale)      # the output's constant rides on the values
        ops.attention_biased(q, outs[0], cache.k, cache.v, step, cache.group, H, G, dk, dv, cache.page_size, self.window,
                             self.scale, self.slopes, self.slopes_log2)

    def forward(self, x: torch.Tensor, step: StepContext, cache: LayerCache) -> torch.Tensor:
        out = torch.empty((1, x.shape[0], self.hidden_size), dtype=torch.float32, device=x.device)
        self.forward_into(x, step, cache, out)
        return out if self.partial_output else out[0]


class MapsAttention(Mixer):
    """Grouped-query causal attention with ``maps`` score maps per head (1: ordinary; 2: differential attention).

    A query head carries ``maps`` queries of ``head_dim`` channels and a key/value head ``maps`` keys, laid out head by
    head as [map 0, map 1]; all maps of a head attend over the SAME values.  With a_0, a_1 the maps' outputs the head
    gives a_0 - lambda a_1, lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + ``lambda_init`` (one number for the layer, from
    four vectors of ``head_dim`` entries), divided by its root mean square over the value channels (no weight) and
    multiplied by 1 - ``lambda_init``.  Options, all independent of the number of maps:

    * ``qk_norm = "head"``: every query and key map is divided by its root mean square over ``head_dim`` and multiplied
      by a weight (``q.norm``, ``k.norm``: [head_dim], shared by the heads);
    * ``position``: a rotation of the first ``rotary_dim`` channels of every map of q and k (none: positions do not
      enter the scores);
    * mask: ``chunk`` (i sees j <= i with i // chunk == j // chunk, counted from position 0 of the sequence), else
      ``window`` (i - j < window), else every j <= i;
    * ``sink``: the softmax's denominator has one more term exp(0), which carries no value;
    * ``head_norm``: the division by the root mean square for a single map too; ``out_factor`` multiplies the output.

    A layer may read the keys (as the cache holds them, rotated) and values that an earlier one wrote; it then has no
    key and value projections.  The output product is float32 when ``float32_output`` (a block that normalises it)."""

    output_parts = 1

    def __init__(self, runtime: Runtime, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 v_head_dim: Optional[int], scale: float, maps: int = 1, lambda_init: Optional[float] = None,
                 chunk: Optional[int] = None, window: Optional[int] = None, sink: bool = False, qk_norm: Optional[str] = None,
                 head_norm: Optional[bool] = None, out_factor: float = 1.0, eps: float = 1e-6, own_kv: bool = True,
                 float32_output: bool = False, out_scale: float = 1.0, position: Optional[Position] = None):
        super().__init__(runtime)
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads do not divide into {num_kv_heads} kv heads")
        if maps not in (1, 2):
            raise ValueError("an attention head has one score map or two")
        if maps == 2 and lambda_init is None:
            raise ValueError("two score maps need the constant of their difference (lambda_init)")
        if qk_norm not in (None, "head"):
            raise ValueError(f"qk_norm {qk_norm!r} is not built here (None, 'head')")
        for name, v in (("chunk", chunk), ("window", window)):
            if v is not None and v < 1:
                raise ValueError(f"an attention {name} must hold at least one position")
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.dk, self.dv = int(head_dim), int(v_head_dim if v_head_dim is not None else head_dim)
        self.maps, self.scale, self.eps = int(maps), float(scale), float(eps)
        self.lambda_init = float(lambda_init) if lambda_init is not None else 0.0
        self.chunk, self.window, self.sink, self.qk_norm = chunk, window, bool(sink), qk_norm
        self.head_norm = bool(head_norm) if head_norm is not None else self.maps == 2
        self.out_factor = float(out_factor) * float(out_scale) * ((1.0 - self.lambda_init) if self.maps == 2 else 1.0)
        self.own_kv, self.position = bool(own_kv), position
        if position is not None and position.rotary_dim > self.dk:
            raise ValueError(f"{position.rotary_dim} rotated channels do not fit a map of {self.dk}")
        self.out_dtype = torch.float32 if float32_output else None
        self.lam = 0.0
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = None

    def cache_requirement(self):
        # a page keeps every position: a chunk's keys are needed until the chunk ends, a window's while it passes
        return PagedKV(self.num_kv_heads, self.maps * self.dk, self.window if self.chunk is None else None, self.dv)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        W, H, G, dk, dv, M = self.hidden_size, self.num_heads, self.num_kv_heads, self.dk, self.dv, self.maps
        specs = {"q": TensorSpec((H * M * dk, W)), "o": TensorSpec((W, H * dv))}
        if self.own_kv:
            specs["k"] = TensorSpec((G * M * dk, W))
            specs["v"] = TensorSpec((G * dv, W))
        if self.qk_norm is not None:
            specs["q.norm"] = TensorSpec((dk,), role="vector", init="norm")
            specs["k.norm"] = TensorSpec((dk,), role="vector", init="norm")
        if M == 2:
            for name in ("lq1", "lk1", "lq2", "lk2"):
                specs[name] = TensorSpec((dk,), role="vector", init="bias")
        return specs

    def bind(self, tensors):
        mats = [tensors["q"]] + ([tensors["k"], tensors["v"]] if self.own_kv else [])
        self.w_qkv = torch.cat(mats, dim=0).contiguous() if len(mats) > 1 else mats[0]
        self.w_o = tensors["o"]
        if self.qk_norm is not None:
            qn, kn = tensors["q.norm"], tensors["k.norm"]
            dt = torch.float32 if torch.float32 in (qn.dtype, kn.dtype) else qn.dtype
            self.q_norm, self.k_norm = qn.to(dt).contiguous(), kn.to(dt).contiguous()
        if self.maps == 2:
            import math
            d = lambda a, b: float((tensors[a].double() * tensors[b].double()).sum().item())
            self.lam = math.exp(d("lq1", "lk1")) - math.exp(d("lq2", "lk2")) + self.lambda_init

    def output_weights(self):
        return [self.w_o]

    def _queries(self, x: torch.Tensor, step: StepContext, cache: LayerCache) -> torch.Tensor:
        """The projections of ``x``; queries (and, with projections of its own, keys) normalised and rotated; keys and
        values of every row written to the cache.  Returns q [T, heads * maps * dk] in the compute dtype."""
        Attention._check(cache)
        if cache.writes != self.own_kv:
            raise ValueError("an attention with key and value projections writes its cache; one without reads another's")
        H, G, dk, dv, M = self.num_heads, self.num_kv_heads, self.dk, self.dv, self.maps
        nq, nk = H * M * dk, G * M * dk
        proj = ops.linear(x, self.w_qkv, out_dtype=torch.float32)
        pos = self.position
        rot = pos.rotary_dim if pos is not None else 0
        return ops.unit_norm_rope_kv_write(
            proj[:, :nq], proj[:, nq:nq + nk] if self.own_kv else None, proj[:, nq + nk:] if self.own_kv else None,
            self.q_norm, self.k_norm, self.eps, step.positions, pos.frequency_pairs() if pos is not None else None, rot,
            pos.amplitude if pos is not None else 1.0, step.slots[cache.group] if self.own_kv else None, cache.k, cache.v,
            H * M, G * M, G, dk, dv, cache.page_size, self.runtime.dtype)

    def _attend(self, q: torch.Tensor, out: torch.Tensor, step: StepContext, cache: LayerCache) -> None:
        ops.attention_maps(q, out, cache.k, cache.v, step, cache.group, self.num_heads, self.num_kv_heads, self.dk, self.dv,
                           self.maps, cache.page_size, self.window, self.chunk, self.sink, self.scale, self.lam, self.head_norm,
                           self.eps, self.out_factor)

    def forward_open(self, x: torch.Tensor, step: StepContext, cache: LayerCache, outs) -> None:
        """The heads' outputs in front of the output product into ``outs[0]`` ([T, heads * dv], rows may be strided)."""
        self._attend(self._queries(x, step, cache), outs[0], step, cache)

    def forward_into(self, x: torch.Tensor, step: StepContext, cache: LayerCache, out: torch.Tensor) -> None:
        o = torch.empty((x.shape[0], self.num_heads * self.dv), dtype=self.runtime.dtype, device=x.device)
        self.forward_open(x, step, cache, [o])
        ops.linear(o, self.w_o, out=out[0])

    def forward(self, x: torch.Tensor, step: StepContext, cache: LayerCache) -> torch.Tensor:
        o = torch.empty((x.shape[0], self.num_heads * self.dv), dtype=self.runtime.dtype, device=x.device)
        self.forward_open(x, step, cache, [o])
        return ops.linear(o, self.w_o, out_dtype=self.out_dtype, partial_ok=self.partial_output)

    supports_tail = True

    def forward_tail(self, x: torch.Tensor, step: StepContext, cache: LayerCache) -> Optional[torch.Tensor]:
        """Keys and values of every row go to the cache; only the wanted rows attend (each as a one-token request of
        ``step.tail``).  An attention that reads another's cache makes the wanted rows' queries only."""
        rows, tail = step.tail_rows, step.tail
        if self.own_kv:
            q = self._queries(x, step, cache)
            if not tail.num_tokens:
                return None
            q = ops.gather_rows(q, rows)
        else:
            if not tail.num_tokens:
                return None
            q = self._queries(ops.gather_rows(x, rows), tail, cache)
        o = torch.empty((q.shape[0], self.num_heads * self.dv), dtype=self.runtime.dtype, device=x.device)
        self._attend(q, o, tail, cache)
        return ops.linear(o, self.w_o, out_dtype=self.out_dtype, partial_ok=self.partial_output)


class LatentAttention(Mixer):
    """Causal attention whose keys and values are two products of ONE latent row per position.

    Per token the layer makes queries of ``heads`` x [``head_dim`` plain | ``rot_dim`` rotated] channels and, when it
    owns its keys (``own_kv``), ``kv_rank`` latent channels (divided by their root mean square and multiplied by
    ``dkv.norm``) followed by ``rot_dim`` key channels shared by all heads.  Head h's key at position j is
    [uk_h c_j | rotated key_j], its value uv_h c_j; the score is (q_plain . uk_h c_j + q_rot . key_j) * ``scale``.
    The cache holds [c_j | rotated key_j] only, as ONE key head of ``kv_rank + rot_dim`` channels without value rows,
    and the products with uk and uv move to the query side:

        q_lat_h = uk_h^T q_plain_h,   score = ([q_lat_h | q_rot_h] . [c_j | key_j]) * scale,
        o_lat_h = sum_j w_j c_j,      head output = uv_h o_lat_h,

    so the attention itself is a multi-query attention over the cached rows whose values are the first ``kv_rank``
    channels of its keys.  The rotated parts turn over their first ``position.rotary_dim`` channels (the encoding's
    amplitude multiplies cos and sin; ``scale`` is taken as given).  Options: ``sink`` (one more term exp(sink_h) in the
    softmax's denominator with a learned score per head, tensor ``sink``, that carries no value) and ``gate`` (head h's
    output is multiplied by sigmoid(g x)_h, tensor ``g`` [heads, width], the same input as the projections).  A layer
    without keys of its own reads the rows (latent and rotated key) that an earlier one wrote, with its own uk and uv.

    Whole prompts (``_expands``) are attended in the EXPANDED form instead: the step's cached rows become keys
    [uk_h c | rotated key] and values uv_h c per head, which costs ``dim + rd`` and ``dv`` channels per score instead of
    ``rank + rd`` and ``rank``; the cache and everything that reads it later are the same either way."""

    output_parts = 1

    def __init__(self, runtime: Runtime, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int, v_head_dim: int,
                 kv_rank: int, scale: float, eps: float, sink: bool = False, gate: bool = False, own_kv: bool = True,
                 float32_output: bool = True, position: Optional[Position] = None):
        super().__init__(runtime)
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.dim, self.rd, self.dv, self.rank = int(head_dim), int(rot_dim), int(v_head_dim), int(kv_rank)
        if min(self.num_heads, self.dim, self.dv, self.rank) < 1 or self.rd < 0:
            raise ValueError("a latent attention needs positive head counts and sizes")
        self.scale, self.eps = float(scale), float(eps)
        self.sink, self.gate, self.own_kv, self.position = bool(sink), bool(gate), bool(own_kv), position
        if position is not None and position.rotary_dim > self.rd:
            raise ValueError(f"{position.rotary_dim} rotated channels do not fit a rotated part of {self.rd}")
        self.out_dtype = torch.float32 if float32_output else None
        self.w_in = self.w_uk = self.w_uv = self.w_o = self.w_norm = self.sink_scores = None

    @property
    def row(self) -> int:
        """Channels of a cached row."""
        return self.rank + self.rd

    def cache_requirement(self):
        return PagedKV(1, self.row, None, 0)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        W, H = self.hidden_size, self.num_heads
        specs = {"q": TensorSpec((H * (self.dim + self.rd), W)), "uk": TensorSpec((H * self.dim, self.rank)),
                 "uv": TensorSpec((H * self.dv, self.rank)), "o": TensorSpec((W, H * self.dv))}
        if self.own_kv:
            specs["dkv"] = TensorSpec((self.row, W))
            specs["dkv.norm"] = TensorSpec((self.rank,), role="vector", init="norm")
        if self.sink:
            specs["sink"] = TensorSpec((H,), role="vector", init="bias")
        if self.gate:
            specs["g"] = TensorSpec((H, W))
        return specs

    def bind(self, tensors):
        H = self.num_heads
        # one product for everything that reads the layer's input: queries, latent + key, gate logits
        mats = [tensors["q"]] + ([tensors["dkv"]] if self.own_kv else []) + ([tensors["g"]] if self.gate else [])
        self.w_in = torch.cat(mats, dim=0).contiguous() if len(mats) > 1 else mats[0]
        self.kv_col = H * (self.dim + self.rd) if self.own_kv else None
        self.gate_col = H * (self.dim + self.rd) + (self.row if self.own_kv else 0)
        self.w_norm = tensors["dkv.norm"] if self.own_kv else None
        # uk [heads * dim, rank] applied as uk_h^T: per head a matrix [rank, dim]; uv per head [dv, rank]
        self.w_uk = tensors["uk"].view(H, self.dim, self.rank).transpose(1, 2).contiguous()
        self.w_uv = tensors["uv"].view(H, self.dv, self.rank).contiguous()
        self.w_uk_rows = tensors["uk"].view(H, self.dim, self.rank).contiguous()      # uk_h itself: keys per head from latent rows
        self.w_o = tensors["o"]
        self.sink_scores = tensors["sink"].to(torch.float32).contiguous() if self.sink else None

    def output_weights(self):
        return [self.w_o]

    def _expands(self, step: StepContext) -> bool:
        """Whether this step's attention runs over keys and values EXPANDED per head instead of in the latent space.
        The latent form reads one row per position for all heads, which is what decoding wants, but multiplies
        ``rank + rd`` and ``rank`` channels per score where expanded keys and values take ``dim + rd`` and ``dv``.  For
        whole prompts (every request of the step starts at position 0, so the step's own rows are all the keys there
        are) of enough tokens, in bfloat16, the rows are expanded through uk and uv and attended with ``heads`` key
        heads by the same kernel."""
        dk = self.dim + self.rd
        q, kv = getattr(step, "q_lens", None), getattr(step, "kv_lens_host", None)
        if (self.runtime.dtype != torch.bfloat16 or not ops.MAPS_TC or not q or not kv or len(q) != len(kv)
                or any(a != b or a < 2 for a, b in zip(q, kv))):
            return False
        if dk % 16 or self.dv % 16 or self.rank % 8 or self.row % 8 or not 16 <= dk <= 256 or not 16 <= self.dv <= 256:
            return False
        latent = self.row + self.rank * (2 if self.rank > 256 else 1)
        return step.num_tokens >= ops.LATENT_EXPAND_MIN_TOKENS and latent >= ops.LATENT_EXPAND_RATIO * (dk + self.dv)

    def _queries(self, x: torch.Tensor, step: StepContext, cache: LayerCache, expand: bool = False):
        """(queries in the latent space [T, heads * (rank + rd)], gate logits float32 [T, heads] or None); the rows of
        the step written to the cache when the layer owns its keys.  ``expand``: the queries as the projection made
        them, [T, heads * (dim + rd)] with the rotated parts turned, for keys expanded per head."""
        Attention._check(cache)
        if cache.writes != self.own_kv:
            raise ValueError("a latent attention with a key projection writes its cache; one without reads another's")
        H = self.num_heads
        proj = ops.linear(x, self.w_in, out_dtype=torch.float32)
        pos = self.position
        q_plain, q_wide = ops.latent_prepare(
            proj, H, self.dim, self.rd, self.rank, self.kv_col, self.w_norm, self.eps, step.positions,
            pos.frequency_pairs() if pos is not None else None, pos.rotary_dim if pos is not None else 0,
            pos.amplitude if pos is not None else 1.0, step.slots[cache.group] if self.own_kv else None, cache.k,
            cache.page_size, self.runtime.dtype)
        gates = proj[:, self.gate_col:self.gate_col + H] if self.gate else None
        if expand:
            dk = self.dim + self.rd
            q_full = torch.empty((x.shape[0], H * dk), dtype=self.runtime.dtype, device=x.device)
            ops.copy_head_columns(q_plain, self.dim, 0, q_full, dk, 0, self.dim, H)
            if self.rd:
                ops.copy_head_columns(q_wide, self.row, self.rank, q_full, dk, self.dim, self.rd, H)
            return q_full, gates
        ops.grouped_linear(q_plain, self.w_uk, q_wide, a_col=self.dim, c_col=self.row)
        return q_wide, gates

    def _attend(self, q_wide, gates, out, step: StepContext, cache: LayerCache) -> None:
        H = self.num_heads
        o_lat = torch.empty((q_wide.shape[0], H * self.rank), dtype=self.runtime.dtype, device=q_wide.device)
        ops.attention_maps(q_wide, o_lat, cache.k, None, step, cache.group, H, 1, self.row, self.rank, 1, cache.page_size,
                           None, None, self.sink, self.scale, 0.0, False, self.eps, 1.0, sink_scores=self.sink_scores,
                           values_in_keys=True)
        ops.grouped_linear(o_lat, self.w_uv, out, a_col=self.rank, c_col=self.dv, factor=gates, factor_sigmoid=True)

    def _attend_expanded(self, q_full, gates, out, step: StepContext, cache: LayerCache) -> None:
        """Whole prompts: the step's cached rows (as the cache holds them) become keys [uk_h c | rotated key] and values
        uv_h c per head, in the layout of pages of ONE position, and the attention with score maps runs over them with
        ``heads`` key heads, which applies the gates to its float32 results."""
        H, dk, T = self.num_heads, self.dim + self.rd, q_full.shape[0]
        rows = ops.gather_rows(cache.k.view(-1, self.row), step.slots[cache.group])          # [T, rank + rd]
        keys = torch.empty((T, H * dk), dtype=rows.dtype, device=rows.device)
        values = torch.empty((T, H * self.dv), dtype=rows.dtype, device=rows.device)
        ops.grouped_linear(rows, self.w_uk_rows, keys, a_col=0, c_col=dk)
        if self.rd:
            ops.copy_head_columns(rows, 0, self.rank, keys, dk, self.dim, self.rd, H)
        ops.grouped_linear(rows, self.w_uv, values, a_col=0, c_col=self.dv)
        dense = getattr(step, "_dense_tables", None)
        if dense is None:            # "pages" of one position: request r's position j is row cu_q[r] + j of the step
            ar = torch.arange(step.max_q_len, dtype=torch.int32, device=rows.device)
            dense = (step.cu_q[:-1].to(torch.int32).unsqueeze(1) + ar.unsqueeze(0)).contiguous()
            try:
                step._dense_tables = dense
            except AttributeError:
                pass
        view = types.SimpleNamespace(block_tables=[dense], token_req=step.token_req, positions=step.positions, cu_q=step.cu_q,
                                     kv_lens=step.kv_lens, q_lens=step.q_lens, max_kv_len=step.max_kv_len)
        ops.attention_maps(q_full, out, keys.view(T, H, 1, dk), values.view(T, H, 1, self.dv), view, 0, H, H, dk, self.dv, 1, 1,
                           None, None, self.sink, self.scale, 0.0, False, self.eps, 1.0, sink_scores=self.sink_scores,
                           head_gates=gates)

    def forward_open(self, x: torch.Tensor, step: StepContext, cache: LayerCache, outs) -> None:
        """The gated heads' outputs in front of the output product into ``outs[0]`` ([T, heads * dv])."""
        if self._expands(step):
            q_full, gates = self._queries(x, step, cache, expand=True)
            self._attend_expanded(q_full, gates, outs[0], step, cache)
            return
        q_wide, gates = self._queries(x, step, cache)
        self._attend(q_wide, gates, outs[0], step, cache)

    def forward_into(self, x: torch.Tensor, step: StepContext, cache: LayerCache, out: torch.Tensor) -> None:
        o = torch.empty((x.shape[0], self.num_heads * self.dv), dtype=self.runtime.dtype, device=x.device)
        self.forward_open(x, step, cache, [o])
        ops.linear(o, self.w_o, out=out[0])

    def forward(self, x: torch.Tensor, step: StepContext, cache: LayerCache) -> torch.Tensor:
        o = torch.empty((x.shape[0], self.num_heads * self.dv), dtype=self.runtime.dtype, device=x.device)
        self.forward_open(x, step, cache, [o])
        return ops.linear(o, self.w_o, out_dtype=self.out_dtype, partial_ok=self.partial_output)

    supports_tail = True

    def forward_tail(self, x: torch.Tensor, step: StepContext, cache: LayerCache) -> Optional[torch.Tensor]:
        """The rows of every token go to the cache; only the wanted rows attend (each as a one-token request of
        ``step.tail``).  A layer that reads another's cache makes the wanted rows' queries only."""
        rows, tail = step.tail_rows, step.tail
        if self.own_kv:
            q_wide, gates = self._queries(x, step, cache)
            if not tail.num_tokens:
                return None
            q_wide = ops.gather_rows(q_wide, rows)
            gates = ops.gather_rows(gates, rows) if gates is not None else None
        else:
            if not tail.num_tokens:
                return None
            q_wide, gates = self._queries(ops.gather_rows(x, rows), tail, cache)
        o = torch.empty((q_wide.shape[0], self.num_heads * self.dv), dtype=self.runtime.dtype, device=x.device)
        self._attend(q_wide, gates, o, tail, cache)
        return ops.linear(o, self.w_o, out_dtype=self.out_dtype, partial_ok=self.partial_output)


class PooledWindowAttention(Mixer):
    """Grouped-query attention over a sliding window whose older keys are seen as block means.

    Position i sees the positions j with 0 <= i - j < ``window`` and, beside them, ONE key and value for each block of
    ``pool`` consecutive positions that lies wholly before the window: block b (positions b pool .. b pool + pool - 1)
    is seen when b pool + pool - 1 <= i - window; its key is the mean of the block's keys as the cache holds them
    (rotated), its value the mean of the values.  Positions that have left the window and whose block is not complete
    behind it are not seen.  Positions and blocks share one softmax.  ``pool`` None: a plain window; ``window`` None:
    every earlier position.  Options, each independent of the others:

    * ``qkv_bias``: biases on the three projections (tensors ``q.b``, ``k.b``, ``v.b``);
    * ``position``: the first ``rotary_dim`` channels of every query and key head turn by the position (pairs
      (i, i + rotary_dim / 2), angles computed from the frequencies);
    * ``rotate_values``: the value of position j turns by j over ALL its channels (pairs (m, m + vdim / 2), pair m by
      j base^(-2m / vdim), ``value_base`` being the base) and is cached so; a head's output at position i is turned
      back by -i, so a value enters with the angle of its distance;
    * ``head_temps``: the score (q . k) ``scale`` is multiplied by a learned number per head (tensor ``temp``);
    * ``softcap``: score <- cap tanh(score / cap);
    * ``sink``: the softmax's denominator has one more term exp(sink_h), a learned number per head (tensor ``sink``)
      without key or value, neither scaled nor capped;
    * ``gate``: the concatenated heads are multiplied by sigmoid(W_g x) (tensor ``g``), x being the mixer's input.

    The cache is two sets of pages: keys and values of every position, and one row per block (``PagedKV.stride``) that
    the step which completes a block fills from the cached rows."""

    output_parts = 1

    def __init__(self, runtime: Runtime, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 v_head_dim: Optional[int], scale: float, window: Optional[int] = None, pool: Optional[int] = None,
                 qkv_bias: bool = False, rotate_values: bool = False, value_base: Optional[float] = None,
                 head_temps: bool = False, softcap: Optional[float] = None, sink: bool = False, gate: bool = False,
                 float32_output: bool = True, position: Optional[Position] = None):
        super().__init__(runtime)
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads do not divide into {num_kv_heads} kv heads")
        for name, v in (("window", window), ("pool", pool)):
            if v is not None and v < 1:
                raise ValueError(f"an attention {name} must hold at least one position")
        if pool is not None and window is None:
            raise ValueError("block means stand for the positions before a window; without a window there are none")
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.dk, self.dv = int(head_dim), int(v_head_dim if v_head_dim is not None else head_dim)
        self.scale, self.window, self.pool = float(scale), window, pool
        self.qkv_bias, self.head_temps, self.sink, self.gate = bool(qkv_bias), bool(head_temps), bool(sink), bool(gate)
        self.softcap = float(softcap) if softcap else None
        self.position = position
        if position is not None and position.rotary_dim > self.dk:
            raise ValueError(f"{position.rotary_dim} rotated channels do not fit a head of {self.dk}")
        self.value_position = None
        if rotate_values:
            if self.dv % 2:
                raise ValueError("rotated values need an even number of channels")
            base = value_base if value_base is not None else getattr(position, "theta", None)
            if base is None:
                raise ValueError("rotated values need the base of their frequencies")
            from .base import POSITIONS, build_part
            self.value_position = build_part(POSITIONS, "position", PartSpec("rope_computed", dict(rotary_dim=self.dv, theta=float(base))), runtime)
        self.out_dtype = torch.float32 if float32_output else None
        self.w_in = self.b_in = self.w_o = self.temps = self.sinks = None

    def cache_requirement(self):
        kv = PagedKV(self.num_kv_heads, self.dk, None, None if self.dv == self.dk else self.dv)
        if self.pool is None:
            return kv
        return (kv, PagedKV(self.num_kv_heads, self.dk, None, None if self.dv == self.dk else self.dv, stride=self.pool))

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        W, H, G, dk, dv = self.hidden_size, self.num_heads, self.num_kv_heads, self.dk, self.dv
        specs = {"q": TensorSpec((H * dk, W)), "k": TensorSpec((G * dk, W)), "v": TensorSpec((G * dv, W)),
                 "o": TensorSpec((W, H * dv))}
        if self.qkv_bias:
            specs.update({"q.b": TensorSpec((H * dk,), role="vector", init="bias"),
                          "k.b": TensorSpec((G * dk,), role="vector", init="bias"),
                          "v.b": TensorSpec((G * dv,), role="vector", init="bias")})
        if self.head_temps:
            specs["temp"] = TensorSpec((H,), role="vector", init="norm")
        if self.sink:
            specs["sink"] = TensorSpec((H,), role="vector", init="bias")
        if self.gate:
            specs["g"] = TensorSpec((H * dv, W))
        return specs

    def bind(self, tensors):
        mats = [tensors["q"], tensors["k"], tensors["v"]] + ([tensors["g"]] if self.gate else [])
        self.w_in = torch.cat(mats, dim=0).contiguous()        # one product for everything that reads the input
        if self.qkv_bias:
            biases = [tensors[n].to(torch.float32) for n in ("q.b", "k.b", "v.b")]
            if self.gate:
                biases.append(torch.zeros(tensors["g"].shape[0], dtype=torch.float32, device=biases[0].device))
            self.b_in = torch.cat(biases).contiguous()
        self.w_o = tensors["o"]
        self.temps = tensors["temp"].to(torch.float32).contiguous() if self.head_temps else None
        self.sinks = tensors["sink"].to(torch.float32).contiguous() if self.sink else None

    def output_weights(self):
        return [self.w_o]

    def _caches(self, cache: LayerCache):
        if self.pool is None:
            Attention._check(cache)
            return cache, None
        if cache is None or cache.kind != "several" or len(cache.parts) != 2:
            raise ValueError("a window attention with block means needs pages for the positions and pages for the blocks")
        return cache.parts[0], cache.parts[1]

    def _write(self, x: torch.Tensor, step: StepContext, cache: LayerCache):
        """Projections of every row; keys and values rotated and cached, the blocks that the step completed averaged.
        Returns (rotated queries [T, heads * dk], the projections [T, ..] whose last columns are the gate's)."""
        kv, blocks = self._caches(cache)
        if not kv.writes:
            raise ValueError("this attention keeps its own keys and values")
        H, G, dk, dv = self.num_heads, self.num_kv_heads, self.dk, self.dv
        proj = ops.linear(x, self.w_in, self.b_in, out_dtype=torch.float32)
        pos = self.position
        freq_v = self.value_position.frequency_pairs() if self.value_position is not None else None
        q = ops.pooled_prepare(proj, step.positions, pos.frequency_pairs() if pos is not None else None,
                               pos.rotary_dim if pos is not None else 0, freq_v, step.slots[kv.group], kv.k, kv.v, H, G, dk, dv,
                               kv.page_size, self.runtime.dtype)
        if blocks is not None:
            ops.pooled_means(kv.k, kv.v, blocks.k, blocks.v, step, kv.group, blocks.group, G, dk, dv, kv.page_size, self.pool)
        return q, proj

    def _attend(self, q: torch.Tensor, proj: torch.Tensor, out: torch.Tensor, step: StepContext, cache: LayerCache) -> None:
        kv, blocks = self._caches(cache)
        H, G, dk, dv = self.num_heads, self.num_kv_heads, self.dk, self.dv
        freq_v = self.value_position.frequency_pairs() if self.value_position is not None else None
        gates = proj[:, H * dk + G * (dk + dv):] if self.gate else None
        ops.pooled_attention(q, out, kv.k, kv.v, blocks.k if blocks is not None else None,
                             blocks.v if blocks is not None else None, step, kv.group,
                             blocks.group if blocks is not None else None, H, G, dk, dv, kv.page_size, self.window, self.pool,
                             self.scale, self.softcap, self.temps, self.sinks, gates, freq_v)

    def forward_open(self, x: torch.Tensor, step: StepContext, cache: LayerCache, outs) -> None:
        """The gated heads in front of the output product into ``outs[0]`` [T, heads * vdim]."""
        q, proj = self._write(x, step, cache)
        self._attend(q, proj, outs[0], step, cache)

    def forward_into(self, x: torch.Tensor, step: StepContext, cache: LayerCache, out: torch.Tensor) -> None:
        o = torch.empty((x.shape[0], self.num_heads * self.dv), dtype=self.runtime.dtype, device=x.device)
        self.forward_open(x, step, cache, [o])
        ops.linear(o, self.w_o, out=out[0])

    def forward(self, x: torch.Tensor, step: StepContext, cache: LayerCache) -> torch.Tensor:
        o = torch.empty((x.shape[0], self.num_heads * self.dv), dtype=self.runtime.dtype, device=x.device)
        self.forward_open(x, step, cache, [o])
        return ops.linear(o, self.w_o, out_dtype=self.out_dtype, partial_ok=self.partial_output)

    supports_tail = True

    def forward_tail(self, x: torch.Tensor, step: StepContext, cache: LayerCache) -> Optional[torch.Tensor]:
        """Keys, values and block means of every row go to the cache; only the wanted rows attend, each as a one-token
        request of ``step.tail`` (the keys they look back on were written by this same step)."""
        q, proj = self._write(x, step, cache)
        rows, tail = step.tail_rows, step.tail
        if not tail.num_tokens:
            return None
        o = torch.empty((tail.num_tokens, self.num_heads * self.dv), dtype=self.runtime.dtype, device=x.device)
        self._attend(ops.gather_rows(q, rows), ops.gather_rows(proj, rows), o, tail, cache)
        return ops.linear(o, self.w_o, out_dtype=self.out_dtype, partial_ok=self.partial_output)


register_mixer("pooled_window_attention", PooledWindowAttention)
register_mixer("latent_attention", LatentAttention)
register_mixer("attention_maps", MapsAttention)
register_mixer("attention", Attention)
register_mixer("attention_distance_bias", DistanceBiasAttention)
