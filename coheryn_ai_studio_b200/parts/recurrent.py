"""Mixers that keep a state of fixed size per request instead of keys and values per position, and the mixer
that runs several mixers side by side.

* ``MatrixMemory`` (kind ``matrix_memory``): the stabilised matrix memory of xLSTM (mLSTM).  Per head, with
  q = W_q h / sqrt(d), k = W_k h, v = W_v h and the capped log gates i = c tanh((W_i h + b_i) / c),
  f = log sigmoid(c tanh((W_f h + b_f) / c)):  m' = max(f + m, i);  S' = e^(f + m - m') S + e^(i - m') k v^T;
  n' likewise with k alone;  o = S'^T q / (max(|n' . q|, e^(-m')) + 1e-6).  m starts at 0.  Each head's o is
  divided by its root mean square, the heads are multiplied by a weight and by sigmoid(W_g h), then W_o.
* ``GatedDeltaRule`` (kind ``gated_delta_rule``): q, k (kv heads) and v (heads) pass a short causal convolution
  per channel and SiLU; q and k become unit vectors per head (q also / sqrt(d)); beta = sigmoid(W_b h); one decay
  per head and key channel g = exp(-exp(A_log) softplus(W_a2 W_a1 h + dt_bias));  S <- diag(g) S;
  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.  Each head's o is divided by its root mean square,
  multiplied by a weight shared by the heads and by sigmoid(W_g2 W_g1 h), then W_o.  The last taps-1 inputs
  of the convolutions are part of the state.
* ``GatedLinearRecurrence`` (kind ``gated_linear_recurrence``): the recurrent block of Griffin (De et al., "Griffin:
  Mixing Gated Linear Recurrences with Local Attention for Efficient Language Models") with its real-gated linear
  recurrent unit.  Two branches of ``width`` channels: y = gelu_tanh(W_y h + b_y) and u = conv(W_x h + b_x), a short
  causal convolution per channel with a bias and no activation.  u is cut into ``blocks`` equal parts; in part b
  r = sigmoid(A_b u_b + a_b), i = sigmoid(B_b u_b + c_b) with square matrices.  log a = -``rate`` r softplus(lam);
  S_t = a S_(t-1) + sqrt(1 - a^2) i u, from S = 0 (no special case for the first token); the output is W_o (S * y).
  State: S (one float32 per channel) and the convolution's last taps-1 inputs.
* ``SideBySide`` (kind ``side_by_side``): mixers that read the same input; the result is the weighted sum of
  theirs.  Each child multiplies its own output by its weight before its output projection, and the
  children's outputs go to the next norm as separate summands.

Everything that enters a recurrence is float32: the projections are computed by the matrix products of the
compute dtype with float32 accumulation and handed on as float32; gates, decays, unit norms, the state and the
norm of the output are computed in float32 inside the scan kernels (``csrc/recurrent.cu``).  All projections
that read the mixer's input are one matrix product over the stacked weights.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence, Tuple

import torch

from .. import ops
from ..config.spec import PartSpec
from ..weights.spec import TensorSpec
from .base import MIXERS, FixedState, LayerCache, Mixer, NormedSum, Runtime, StepContext, build_part, register_mixer


class _StackedInput:
    """Rows of several weight matrices stacked so that one product makes all projections of an input;
    ``cut`` hands back the column range of each."""

    def __init__(self, named: Sequence[Tuple[str, torch.Tensor]]):
        self.weight = torch.cat([w for _, w in named], dim=0).contiguous()
        self.ranges, at = {}, 0
        for name, w in named:
            self.ranges[name] = (at, at + w.shape[0])
            at += w.shape[0]

    def project(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, self.weight, out_dtype=torch.float32)

    def cut(self, proj: torch.Tensor, first: str, last: Optional[str] = None) -> torch.Tensor:
        return proj[:, self.ranges[first][0]:self.ranges[last or first][1]]


class _StateMixer(Mixer):
    output_parts = 1

    def forward(self, x: torch.Tensor, step: StepContext, cache: Optional[LayerCache]) -> torch.Tensor:
        out = torch.empty((1, x.shape[0], self.hidden_size), dtype=torch.float32, device=x.device)
        self.forward_into(x, step, cache, out)
        return out if self.partial_output else out[0]

    @staticmethod
    def _state_of(cache: Optional[LayerCache]) -> torch.Tensor:
        if cache is None or cache.kind != "state":
            raise ValueError("this mixer needs a state slot per request")
        if not cache.writes:
            raise ValueError("a recurrent state cannot be shared between two executions of a layer")
        return cache.state


class MatrixMemory(_StateMixer):
    def __init__(self, runtime: Runtime, hidden_size: int, num_heads: int, head_dim: int, v_head_dim: int,
                 gate_cap: float, eps: float, out_scale: float = 1.0):
        super().__init__(runtime)
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.dk, self.dv, self.cap, self.eps, self.out_scale = int(head_dim), int(v_head_dim), float(gate_cap), float(eps), float(out_scale)
        if not self.cap > 0:
            raise ValueError("the gate cap must be positive")
        self.stacked = self.w_o = self.norm_w = self.b_i = self.b_f = None

    def cache_requirement(self):
        H, dk, dv = self.num_heads, self.dk, self.dv
        return FixedState((H * (dk * dv + dk + 1),), torch.float32)     # S, n, m of every head

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        W, H, dk, dv = self.hidden_size, self.num_heads, self.dk, self.dv
        return {"q": TensorSpec((H * dk, W)), "k": TensorSpec((H * dk, W)), "v": TensorSpec((H * dv, W)),
                "g": TensorSpec((H * dv, W)), "o": TensorSpec((W, H * dv)),
                "norm": TensorSpec((H * dv,), role="vector", init="norm"),
                "i": TensorSpec((H, W)), "i.b": TensorSpec((H,), role="vector", init="bias"),
                "f": TensorSpec((H, W)), "f.b": TensorSpec((H,), role="vector", init="bias")}

    def bind(self, tensors):
        self.stacked = _StackedInput([(n, tensors[n]) for n in ("q", "k", "v", "g", "i", "f")])
        self.w_o, self.norm_w = tensors["o"], tensors["norm"]
        dt = torch.float32 if torch.float32 in (tensors["i.b"].dtype, tensors["f.b"].dtype) else tensors["i.b"].dtype
        self.b_i, self.b_f = tensors["i.b"].to(dt).contiguous(), tensors["f.b"].to(dt).contiguous()

    def output_weights(self):
        return [self.w_o]

    def forward_into(self, x: torch.Tensor, step: StepContext, cache: Optional[LayerCache], out: torch.Tensor) -> None:
        o = torch.empty((x.shape[0], self.num_heads * self.dv), dtype=self.runtime.dtype, device=x.device)
        self.forward_open(x, step, cache, [o])
        ops.linear(o, self.w_o, out=out[0])

    def forward_open(self, x: torch.Tensor, step: StepContext, cache: Optional[LayerCache], outs) -> None:
        """The activations in front of the output product (normalised, gated, weighted) into ``outs[0]``."""
        state = self._state_of(cache)
        st, proj = self.stacked, self.stacked.project(x)
        o = outs[0]
        ops.matrix_memory_scan(st.cut(proj, "q"), st.cut(proj, "k"), st.cut(proj, "v"), st.cut(proj, "i"), st.cut(proj, "f"),
                               self.b_i, self.b_f, self.cap, state, step, self.num_heads, self.dk, self.dv, o, self.norm_w,
                               st.cut(proj, "g"), self.eps, self.out_scale)


class GatedDeltaRule(_StateMixer):
    def __init__(self, runtime: Runtime, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 v_head_dim: int, conv_taps: int, eps: float, decay_rank: Optional[int] = None,
                 gate_rank: Optional[int] = None, out_scale: float = 1.0, decay: str = "channel", low_rank: bool = True,
                 gate_activation: str = "sigmoid"):
        """``decay_rank`` / ``gate_rank``: the inner sizes of the two-step projections of the decay and of the output
        gate; None takes them from the checkpoint's tensors.  ``decay``: "channel" (a decay per head and key channel) or
        "head" (one per head: ``dt_bias`` then has one entry per head).  ``low_rank`` False: the decay's and the gate's
        pre-activations are single projections ``a`` and ``g`` of the input instead of two-step ones.
        ``gate_activation``: what the output gate's pre-activation passes, "sigmoid" or "silu"."""
        super().__init__(runtime)
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads do not divide into {num_kv_heads} query/key heads")
        if not 1 <= conv_taps <= 16:
            raise ValueError("the short convolution takes 1 to 16 taps")
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.dk, self.dv, self.taps, self.eps, self.out_scale = int(head_dim), int(v_head_dim), int(conv_taps), float(eps), float(out_scale)
        self.decay_rank, self.gate_rank = decay_rank, gate_rank
        if decay not in ("channel", "head") or gate_activation not in ("sigmoid", "silu"):
            raise ValueError("gated_delta_rule: decay is 'channel' or 'head', gate_activation 'sigmoid' or 'silu'")
        self.decay, self.low_rank, self.gate_activation = decay, bool(low_rank), gate_activation
        self.decay_size = self.num_heads * (self.dk if decay == "channel" else 1)
        self.channels = 2 * self.num_kv_heads * self.dk + self.num_heads * self.dv
        self.memory = self.num_heads * self.dk * self.dv

    def cache_requirement(self):
        return FixedState((self.memory + (self.taps - 1) * self.channels,), torch.float32)   # S of every head, then the convolutions' inputs

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        W, H, G, dk, dv, n = self.hidden_size, self.num_heads, self.num_kv_heads, self.dk, self.dv, self.taps
        ra, rg = self.decay_rank or -1, self.gate_rank or -1      # -1: any size, as the checkpoint has it
        specs = {"q": TensorSpec((G * dk, W)), "q.conv": TensorSpec((G * dk, n), role="vector", init="conv"),
                 "k": TensorSpec((G * dk, W)), "k.conv": TensorSpec((G * dk, n), role="vector", init="conv"),
                 "v": TensorSpec((H * dv, W)), "v.conv": TensorSpec((H * dv, n), role="vector", init="conv"),
                 "b": TensorSpec((H, W)), "A_log": TensorSpec((H,), role="vector", init="bias"),
                 "norm": TensorSpec((dv,), role="vector", init="norm"),
                 "dt_bias": TensorSpec((self.decay_size,), role="vector", init="bias"), "o": TensorSpec((W, H * dv))}
        if self.low_rank:
            specs.update({"a1": TensorSpec((ra, W)), "a2": TensorSpec((self.decay_size, ra)),
                          "g1": TensorSpec((rg, W)), "g2": TensorSpec((H * dv, rg))})
        else:
            specs.update({"a": TensorSpec((self.decay_size, W)), "g": TensorSpec((H * dv, W))})
        return specs

    def bind(self, tensors):
        convs = [tensors["q.conv"], tensors["k.conv"], tensors["v.conv"]]
        dt = torch.float32 if any(c.dtype == torch.float32 for c in convs) else convs[0].dtype
        self.conv_w = torch.cat([c.to(dt) for c in convs], dim=0).contiguous()
        self.w_o = tensors["o"]
        self.rate_log, self.dt_bias, self.norm_w = tensors["A_log"], tensors["dt_bias"], tensors["norm"]
        if not self.low_rank:
            self.stacked = _StackedInput([(n, tensors[n]) for n in ("q", "k", "v", "b", "a", "g")])
            self.w_second = None
            return
        if tensors["a1"].shape[0] != tensors["a2"].shape[1] or tensors["g1"].shape[0] != tensors["g2"].shape[1]:
            raise ValueError("the two steps of a low-rank projection do not fit each other")
        self.stacked = _StackedInput([(n, tensors[n]) for n in ("q", "k", "v", "b", "a1", "g1")])
        # The second steps of the two low-rank projections as ONE product: [a1 h | g1 h] (neighbours in the stacked
        # output) times the block-diagonal matrix of a2 and g2 (exact zeros elsewhere) gives [step | gate].
        a2, g2 = tensors["a2"], tensors["g2"]
        both = torch.zeros((a2.shape[0] + g2.shape[0], a2.shape[1] + g2.shape[1]), dtype=a2.dtype, device=a2.device)
        both[:a2.shape[0], :a2.shape[1]] = a2
        both[a2.shape[0]:, a2.shape[1]:] = g2
        self.w_second = both.contiguous()

    def output_weights(self):
        return [self.w_o]

    def forward_into(self, x: torch.Tensor, step: StepContext, cache: Optional[LayerCache], out: torch.Tensor) -> None:
        o = torch.empty((x.shape[0], self.num_heads * self.dv), dtype=self.runtime.dtype, device=x.device)
        self.forward_open(x, step, cache, [o])
        ops.linear(o, self.w_o, out=out[0])

    def forward_open(self, x: torch.Tensor, step: StepContext, cache: Optional[LayerCache], outs) -> None:
        state = self._state_of(cache)
        st, proj = self.stacked, self.stacked.project(x)
        G, H, dk, dv = self.num_kv_heads, self.num_heads, self.dk, self.dv
        qkv = ops.short_conv_silu(st.cut(proj, "q", "v"), self.conv_w, state[:, self.memory:], step)
        if self.low_rank:
            second = ops.linear(st.cut(proj, "a1", "g1"), self.w_second, out_dtype=torch.float32)
            step_pre, gate = second[:, :self.decay_size], second[:, self.decay_size:]
        else:
            step_pre, gate = st.cut(proj, "a"), st.cut(proj, "g")
        o = outs[0]
        ops.gated_delta_scan(qkv[:, :G * dk], qkv[:, G * dk:2 * G * dk], qkv[:, 2 * G * dk:], st.cut(proj, "b"), step_pre,
                             self.dt_bias, self.rate_log, state[:, :self.memory], step, H, G, dk, dv, o, self.norm_w, gate,
                             self.eps, self.out_scale, decay_per_channel=self.decay == "channel",
                             gate_activation=self.gate_activation)


class GatedLinearRecurrence(_StateMixer):
    def __init__(self, runtime: Runtime, hidden_size: int, width: int, blocks: int, conv_taps: int, rate: float = 8.0,
                 float32_output: bool = True):
        super().__init__(runtime)
        self.hidden_size, self.width, self.blocks, self.taps = int(hidden_size), int(width), int(blocks), int(conv_taps)
        if self.blocks < 1 or self.width % self.blocks:
            raise ValueError(f"{self.width} channels do not form {self.blocks} equal blocks")
        if not 1 <= self.taps <= 16:
            raise ValueError("the short convolution takes 1 to 16 taps")
        self.block, self.rate = self.width // self.blocks, float(rate)
        self.out_dtype = torch.float32 if float32_output else None
        self.w_in = self.b_in = self.conv_w = self.conv_b = self.w_gates = self.b_r = self.b_i = self.lam = self.w_o = None

    def cache_requirement(self):
        return FixedState((self.width * self.taps,), torch.float32)      # S, then the convolution's last taps-1 inputs

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        W, C, nb, bs = self.hidden_size, self.width, self.blocks, self.block
        return {"y": TensorSpec((C, W)), "y.b": TensorSpec((C,), role="vector", init="bias"),
                "x": TensorSpec((C, W)), "x.b": TensorSpec((C,), role="vector", init="bias"),
                "conv": TensorSpec((C, self.taps), role="vector", init="conv"),
                "conv.b": TensorSpec((C,), role="vector", init="bias"),
                "ra": TensorSpec((nb, bs, bs)), "ra.b": TensorSpec((nb, bs), role="vector", init="bias"),
                "ri": TensorSpec((nb, bs, bs)), "ri.b": TensorSpec((nb, bs), role="vector", init="bias"),
                "lam": TensorSpec((C,), role="vector", init="bias"), "o": TensorSpec((W, C))}

    def bind(self, tensors):
        f32 = lambda t: t.to(torch.float32).contiguous()
        self.w_in = torch.cat([tensors["y"], tensors["x"]], dim=0).contiguous()       # one product for both branches
        self.b_in = torch.cat([f32(tensors["y.b"]), f32(tensors["x.b"])]).contiguous()
        self.conv_w, self.conv_b = f32(tensors["conv"]), f32(tensors["conv.b"])
        # the gates of a recurrence are float32 arithmetic: per block the rows of both matrices, [r rows | i rows]
        self.w_gates = torch.cat([f32(tensors["ra"]), f32(tensors["ri"])], dim=1).contiguous()     # [blocks, 2 bs, bs]
        self.b_r, self.b_i = f32(tensors["ra.b"]).reshape(-1), f32(tensors["ri.b"]).reshape(-1)
        self.lam, self.w_o = f32(tensors["lam"]), tensors["o"]

    def output_weights(self):
        return [self.w_o]

    def forward(self, x: torch.Tensor, step: StepContext, cache: Optional[LayerCache]) -> torch.Tensor:
        o = torch.empty((x.shape[0], self.width), dtype=self.runtime.dtype, device=x.device)
        self.forward_open(x, step, cache, [o])
        return ops.linear(o, self.w_o, out_dtype=self.out_dtype, partial_ok=self.partial_output)

    def forward_into(self, x: torch.Tensor, step: StepContext, cache: Optional[LayerCache], out: torch.Tensor) -> None:
        o = torch.empty((x.shape[0], self.width), dtype=self.runtime.dtype, device=x.device)
        self.forward_open(x, step, cache, [o])
        ops.linear(o, self.w_o, out=out[0])

    supports_tail = True

    def forward_tail(self, x: torch.Tensor, step: StepContext, cache: Optional[LayerCache]) -> Optional[torch.Tensor]:
        """The state passes every row; the output product runs for the wanted rows only."""
        o = torch.empty((x.shape[0], self.width), dtype=self.runtime.dtype, device=x.device)
        self.forward_open(x, step, cache, [o])
        if not step.tail.num_tokens:
            return None
        return ops.linear(ops.gather_rows(o, step.tail_rows), self.w_o, out_dtype=self.out_dtype, partial_ok=self.partial_output)

    def forward_open(self, x: torch.Tensor, step: StepContext, cache: Optional[LayerCache], outs) -> None:
        """S * y, the activations in front of the output product, into ``outs[0]`` [T, width]."""
        state = self._state_of(cache)
        C, bs = self.width, self.block
        proj = ops.linear(x, self.w_in, self.b_in, out_dtype=torch.float32)
        u = ops.conv_bias(proj[:, C:], self.conv_w, self.conv_b, state[:, C:], step)
        gates = torch.empty((x.shape[0], 2 * C), dtype=torch.float32, device=x.device)
        ops.grouped_linear(u, self.w_gates, gates, a_col=bs, c_col=2 * bs)
        ops.gated_scan(gates, self.b_r, self.b_i, u, proj[:, :C], self.lam, self.rate, bs, state[:, :C], step, outs[0])


class SideBySide(Mixer):
    def __init__(self, runtime: Runtime, hidden_size: int, mixers: Sequence[Tuple[str, PartSpec, float]], position=None,
                 combine: str = "sum", eps: float = 1e-6):
        """``mixers``: (name under which the child's tensors stand, the child's PartSpec, the weight of its output).
        ``combine``: "sum" (the weighted sum of the children's outputs) or "normed_mean": every child's output is
        divided by its root mean square over the model width (``eps`` inside the root) and multiplied by a weight
        ``<name>.out`` [width]; the result is the mean of those (the children's weights must be 1)."""
        super().__init__(runtime)
        self.hidden_size = int(hidden_size)
        if not mixers:
            raise ValueError("side_by_side needs at least one mixer")
        if combine not in ("sum", "normed_mean"):
            raise ValueError(f"side_by_side: combine {combine!r} is not built (sum, normed_mean)")
        if combine == "normed_mean" and any(float(w) != 1.0 for _, _, w in mixers):
            raise ValueError("side_by_side: normalised outputs take no weights besides their norms'")
        self.combine, self.eps = combine, float(eps)
        self.out_weights = None
        self.children = []
        for name, spec, weight in mixers:
            extra = {"position": position} if position is not None else {}
            child = build_part(MIXERS, "mixer", spec, runtime, out_scale=float(weight), **extra)
            if not hasattr(child, "forward_into"):
                raise ValueError(f"side_by_side: {type(child).__name__} cannot write its output into a stack of summands")
            self.children.append((str(name), child))
        self.output_parts = sum(c.output_parts for _, c in self.children)
        self.capturable = all(c.capturable for _, c in self.children)

    def cache_requirement(self):
        return tuple(c.cache_requirement() for _, c in self.children)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = {f"{name}.{local}": ts for name, c in self.children for local, ts in c.tensor_specs().items()}
        if self.combine == "normed_mean":
            for name, _ in self.children:
                specs[f"{name}.out"] = TensorSpec((self.hidden_size,), role="vector", init="norm")
        return specs

    def bind(self, tensors):
        for name, c in self.children:
            c.bind({local: tensors[f"{name}.{local}"] for local in c.tensor_specs() if f"{name}.{local}" in tensors})
        if self.combine == "normed_mean":
            ws = [tensors[f"{name}.out"] for name, _ in self.children]
            dt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
            self.out_weights = torch.stack([w.to(dt) for w in ws], dim=0).contiguous()

    def forward_into(self, x: torch.Tensor, step: StepContext, cache: Optional[LayerCache], out: torch.Tensor) -> None:
        if self.combine != "sum":
            raise ValueError("side_by_side: normalised outputs are not summands of a block's sum; use forward")
        self._children_into(x, step, cache, out)

    def _children_into(self, x: torch.Tensor, step: StepContext, cache: Optional[LayerCache], out: torch.Tensor) -> None:
        if cache is None or cache.kind != "several" or len(cache.parts) != len(self.children):
            raise ValueError("side_by_side needs one cache per child")
        at = 0
        for (_, c), sub in zip(self.children, cache.parts):
            c.forward_into(x, step, sub, out[at:at + c.output_parts])
            at += c.output_parts

    def output_weights(self):
        if self.combine != "sum" or not all(hasattr(c, "output_weights") for _, c in self.children):
            return None      # normalised outputs cannot be joined into one product
        return [w for _, c in self.children for w in c.output_weights()]

    def forward_open(self, x: torch.Tensor, step: StepContext, cache: Optional[LayerCache], outs) -> None:
        if cache is None or cache.kind != "several" or len(cache.parts) != len(self.children):
            raise ValueError("side_by_side needs one cache per child")
        at = 0
        for (_, c), sub in zip(self.children, cache.parts):
            n = len(c.output_weights())
            c.forward_open(x, step, sub, outs[at:at + n])
            at += n

    def forward(self, x: torch.Tensor, step: StepContext, cache: Optional[LayerCache]) -> torch.Tensor:
        out = torch.empty((self.output_parts, x.shape[0], self.hidden_size), dtype=torch.float32, device=x.device)
        self._children_into(x, step, cache, out)
        if self.combine == "normed_mean":
            if self.output_parts != len(self.children):
                raise ValueError("side_by_side: a child with several summands cannot be normalised as one")
            return NormedSum(out, self.out_weights, 1.0 / len(self.children), self.eps)
        if self.partial_output:
            return out
        raise ValueError("side_by_side hands its children's outputs on as summands and needs norms that add them")


register_mixer("matrix_memory", MatrixMemory)
register_mixer("gated_delta_rule", GatedDeltaRule)
register_mixer("gated_linear_recurrence", GatedLinearRecurrence)
register_mixer("side_by_side", SideBySide)
