"""Embedders: what turns token ids into the stream when a table row is not all of it.

``pair_hash_embedding``: x_t = table[id_t] (* scale) + pair[(id_{t-1} * mul_prev + id_t * mul_cur) mod buckets], with
row ``buckets`` of ``pair`` (its last) for the first token of a sequence, then optionally x / rms(x) * norm.  The token
before the first one of a step's portion is the last token of the request's previous step: one int32 word of fixed state
per request, written by the same step after it was read.  One kernel makes the float32 stream and its copy in the
compute dtype.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..weights.spec import TensorSpec
from .base import Embedder, FixedState, LayerCache, Runtime, StepContext, register_embedder


class PairHashEmbedding(Embedder):
    def __init__(self, runtime: Runtime, vocab_size: int, hidden_size: int, table: str, pair: Optional[str] = None,
                 buckets: int = 0, mul_prev: int = 0, mul_cur: int = 0, norm: Optional[str] = None, eps: float = 1e-6,
                 scale: Optional[float] = None):
        """``table``, ``pair``, ``norm``: full tensor names ([vocab, width], [buckets + 1, width], [width]); ``pair`` None:
        no pair rows; ``norm`` None: no norm."""
        super().__init__(runtime)
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.table_name, self.pair_name, self.norm_name = str(table), pair, norm
        self.buckets, self.mul_prev, self.mul_cur = int(buckets), int(mul_prev), int(mul_cur)
        if pair is not None and (self.buckets < 1 or self.mul_prev < 0 or self.mul_cur < 0):
            raise ValueError("pair rows need a positive number of buckets and non-negative multipliers")
        self.eps, self.scale = float(eps), scale
        self.table = self.pair = self.norm = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = {self.table_name: TensorSpec((self.vocab_size, self.hidden_size))}
        if self.pair_name is not None:
            specs[self.pair_name] = TensorSpec((self.buckets + 1, self.hidden_size))
        if self.norm_name is not None:
            specs[self.norm_name] = TensorSpec((self.hidden_size,), role="vector", init="norm")
        return specs

    def bind(self, tensors):
        self.table = tensors[self.table_name]
        self.pair = tensors[self.pair_name] if self.pair_name is not None else None
        self.norm = tensors[self.norm_name] if self.norm_name is not None else None

    def state_requirement(self):
        return FixedState((1,), torch.int32) if self.pair_name is not None else None

    def forward(self, step: StepContext, state: Optional[LayerCache], out: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
        cast = out if self.runtime.dtype == torch.float32 else torch.empty(out.shape, dtype=self.runtime.dtype, device=out.device)
        last = state.state if state is not None else None
        ops.embed_pair(self.table, self.pair, step, last, self.mul_prev, self.mul_cur, self.buckets, self.scale, self.norm,
                       self.eps, out, None if cast is out else cast, status)
        if last is not None:
            ops.store_last_ids(step, last)
        return cast


register_embedder("pair_hash_embedding", PairHashEmbedding)
