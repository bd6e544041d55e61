"""Feed-forwards that treat tokens differently: experts chosen by a router, and a gate that multiplies by a table row
of the token's id.

``routed_experts``: ``experts`` gated feed-forwards W_down (act(W_gate x) * (W_up x)) without biases, of which each
token uses ``top``.  The router has ``experts + identity`` outputs; the last ``identity`` of them stand for experts
without tensors whose output is the input itself.  With z = W_router x in float32 and s = softmax(z) over all outputs,
the choice scores are s + ``correction``; the outputs form ``groups`` equal groups of neighbours, a group's score is its
largest choice score, and only outputs of the ``keep`` best groups can be chosen (the others count as minus infinity);
the ``top`` largest choice scores are chosen, ties to the lower index.  The weights are the chosen outputs' s divided by
their sum (+ 1e-20) times ``scale``; the result is the weighted sum of the chosen experts' outputs.

``selection = "top_softmax"`` is the other common router: the choice scores are the logits themselves (plus a bias
``router.b`` when ``router_bias``), the ``top`` largest are chosen and the weights are the softmax over the chosen logits
alone (times ``scale``); groups and identity outputs work as above, ``correction`` does not apply.  ``shared``: one more
expert of the same form (tensors ``shared.gate``, ``shared.up``, ``shared.down``; its own size and activation constant)
that every token uses; with ``gate`` its output is multiplied by sigmoid(w . x), one number per token (tensor
``shared.sg`` [1, width]), before it is added.

The pairs (token, choice) that name a real expert are ordered by expert on the device, each expert's rows meet its
matrices in one grouped product (gate and up interleaved, the activation in the epilogue; then down; with many rows per
expert the products are the TMA + tcgen05 kernel of the dense layers over row tiles of 128, with fewer the kernel of
``csrc/routed.cu`` over tiles of 64, which reads the tokens' rows through the index), and a last kernel
adds a token's weighted rows in the order of its choices, so a token's result does not depend on the other tokens of the
step.  Nothing is read back to the host: the part can be captured in a CUDA graph.

``token_table_gate``: y = W_proj (gelu_tanh(W_gate x) * table[token id, columns of this layer]); the table belongs to the
model and is shared by the layers, each reading ``dim`` columns of its own.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..weights.spec import TensorSpec
from .base import FeedForward, Runtime, StepContext, register_feed_forward


class RoutedExperts(FeedForward):
    output_parts = 1

    def __init__(self, runtime: Runtime, hidden_size: int, expert_size: int, experts: int, top: int, identity: int = 0,
                 groups: int = 1, keep: Optional[int] = None, scale: float = 1.0, correction: bool = True,
                 activation: str = "silu", expert_prefix: str = "e", tensors=("gate", "up", "down"),
                 activation_constant: Optional[float] = None, selection: str = "softmax_top", router_bias: bool = False,
                 shared: Optional[dict] = None):
        """``shared``: None or {"size": .., "activation_constant": .. (None: the experts'), "gate": bool}."""
        super().__init__(runtime)
        if selection not in ("softmax_top", "top_softmax"):
            raise ValueError(f"router selection {selection!r} is not built (softmax_top, top_softmax)")
        self.selection, self.router_bias = selection, bool(router_bias)
        if selection == "top_softmax":
            correction = False
        elif router_bias:
            raise ValueError("a bias on the router's logits goes with selection 'top_softmax'")
        self.shared = None
        if shared is not None:
            const = shared.get("activation_constant", activation_constant)
            self.shared = dict(size=int(shared["size"]), constant=const, gate=bool(shared.get("gate", False)))
            ops.gated_epilogue_word(activation, const)
        self.hidden_size, self.expert_size = int(hidden_size), int(expert_size)
        self.experts, self.identity, self.top = int(experts), int(identity), int(top)
        self.outputs = self.experts + self.identity
        self.groups = int(groups) if groups else 1
        self.keep = int(keep) if keep is not None else self.groups
        self.scale, self.correction = float(scale), bool(correction)
        if self.experts < 1 or self.identity < 0:
            raise ValueError("a router needs at least one expert with tensors")
        if self.outputs % self.groups:
            raise ValueError(f"{self.outputs} router outputs do not form {self.groups} equal groups")
        if not 1 <= self.keep <= self.groups:
            raise ValueError(f"{self.keep} of {self.groups} groups cannot be kept")
        if not 1 <= self.top <= self.keep * (self.outputs // self.groups):
            raise ValueError(f"{self.top} choices do not fit {self.keep} groups of {self.outputs // self.groups}")
        self.epilogue = ops.gated_epilogue_word(activation, activation_constant)
        self.activation, self.prefix, self.names = activation, str(expert_prefix), tuple(tensors)
        self.w_router = self.w_correction = self.w_gate_up = self.w_down = self.w_shared_gate_up = self.w_shared_down = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        W, F = self.hidden_size, self.expert_size
        g, u, d = self.names
        specs = {"router": TensorSpec((self.outputs, W))}
        if self.correction:
            specs["correction"] = TensorSpec((self.outputs,), role="vector", init="normal")
        if self.router_bias:
            specs["router.b"] = TensorSpec((self.outputs,), role="vector", init="bias")
        if self.shared is not None:
            S = self.shared["size"]
            specs.update({f"shared.{g}": TensorSpec((S, W)), f"shared.{u}": TensorSpec((S, W)), f"shared.{d}": TensorSpec((W, S))})
            if self.shared["gate"]:
                specs["shared.sg"] = TensorSpec((1, W))
        for e in range(self.experts):
            p = f"{self.prefix}{e}."
            specs[p + g], specs[p + u], specs[p + d] = TensorSpec((F, W)), TensorSpec((F, W)), TensorSpec((W, F))
        return specs

    def bind(self, tensors):
        g, u, d = self.names
        self.w_router = tensors["router"]
        self.w_correction = tensors["correction"].to(torch.float32).contiguous() if self.correction else None
        if self.router_bias:
            self.w_correction = tensors["router.b"].to(torch.float32).contiguous()      # added to the logits: see ``choose``
        if self.shared is not None:
            sg_, su_ = tensors[f"shared.{g}"], tensors[f"shared.{u}"]
            self.w_shared_gate_up = torch.stack([sg_, su_], dim=1).reshape(2 * sg_.shape[0], sg_.shape[1]).contiguous()
            self.w_shared_down = tensors[f"shared.{d}"]
            if self.shared["gate"]:      # the gate's row rides under the router's: one product for both
                self.w_router = torch.cat([self.w_router, tensors["shared.sg"].reshape(1, -1)], dim=0).contiguous()
        # per expert gate and up rows interleaved (2j = gate_j, 2j+1 = up_j): a pair meets in one thread of the epilogue
        gu = [torch.stack([tensors[f"{self.prefix}{e}.{g}"], tensors[f"{self.prefix}{e}.{u}"]], dim=1)
              .reshape(2 * self.expert_size, self.hidden_size) for e in range(self.experts)]
        self.w_gate_up = torch.stack(gu, dim=0).contiguous()
        self.w_down = torch.stack([tensors[f"{self.prefix}{e}.{d}"] for e in range(self.experts)], dim=0).contiguous()

    def choose(self, x: torch.Tensor):
        """(chosen outputs int32 [T, top], their weights float32 [T, top])."""
        return self._choose(x)[:2]

    def _choose(self, x: torch.Tensor):
        """(ids, weights, pre-activation of the shared expert's gate [T] or None)."""
        logits = ops.linear(x, self.w_router, out_dtype=torch.float32)
        ids, weights = ops.route_select(logits[:, :self.outputs], self.w_correction, self.groups, self.keep, self.top, self.scale,
                                        chosen_softmax=self.selection == "top_softmax")
        return ids, weights, logits[:, self.outputs] if logits.shape[1] > self.outputs else None

    def forward(self, x: torch.Tensor, step: StepContext) -> torch.Tensor:
        T = x.shape[0]
        out = torch.empty((T, self.hidden_size), dtype=torch.float32, device=x.device)
        if T == 0:
            return out
        ids, weights, shared_gate = self._choose(x)
        shared = None
        if self.shared is not None:
            act = ops.gated_linear(x, self.w_shared_gate_up, self.activation, param=self.shared["constant"])
            shared = ops.linear(act, self.w_shared_down, out_dtype=torch.float32)
        wide = ops.grouped_tc_suits(x, T * self.top, self.experts, self.w_gate_up, self.w_down)
        rows = ops.route_sort(ids, self.experts, wide_tiles=wide)
        n = rows.n
        y = torch.empty((n, self.hidden_size), dtype=torch.float32, device=x.device)
        act = torch.empty((n, self.expert_size), dtype=x.dtype, device=x.device)
        if wide:       # many rows per expert: the inputs in sorted order, then both products by TMA + tcgen05
            ops.gemm_bf16_tc_grouped(ops.gather_rows(x, rows.token_of), self.w_gate_up, act, rows, self.epilogue)
            ops.gemm_bf16_tc_grouped(act, self.w_down, y, rows)
        else:
            ops.grouped_linear(x, self.w_gate_up, act, rows=rows, gather=True, epilogue=self.epilogue)
            ops.grouped_linear(act, self.w_down, y, rows=rows)
        ops.route_combine(y, x, ids, weights, rows, out, extra=shared, extra_gate=shared_gate)
        return out


class TokenTableGate(FeedForward):
    output_parts = 1

    def __init__(self, runtime: Runtime, hidden_size: int, dim: int, table: str, first_column: int, vocab_size: int,
                 tensors=("gate", "proj")):
        """``table``: the full name of the model's tensor [vocab, columns]; this part reads columns
        ``first_column .. first_column + dim``."""
        super().__init__(runtime)
        self.hidden_size, self.dim, self.vocab_size = int(hidden_size), int(dim), int(vocab_size)
        self.table_name, self.first_column, self.names = str(table), int(first_column), tuple(tensors)
        self.w_gate = self.w_proj = self.table = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        g, p = self.names
        return {g: TensorSpec((self.dim, self.hidden_size)), p: TensorSpec((self.hidden_size, self.dim))}

    def bind(self, tensors):
        self.w_gate, self.w_proj = tensors[self.names[0]], tensors[self.names[1]]

    def shared_tensors(self):
        return (self.table_name,)

    def bind_shared(self, tensors):
        self.table = tensors[self.table_name]
        if self.table.dim() != 2 or self.first_column + self.dim > self.table.shape[1]:
            raise ValueError(f"{self.table_name} has no columns {self.first_column}..{self.first_column + self.dim}")

    def forward(self, x: torch.Tensor, step: StepContext) -> torch.Tensor:
        z = ops.linear(x, self.w_gate, out_dtype=torch.float32)
        g = torch.empty((x.shape[0], self.dim), dtype=self.table.dtype, device=x.device)
        ops.gated_table_mul(z, self.table, self.first_column, step.token_ids, g)
        return ops.linear(g, self.w_proj, out_dtype=torch.float32)


register_feed_forward("routed_experts", RoutedExperts)
register_feed_forward("token_table_gate", TokenTableGate)
