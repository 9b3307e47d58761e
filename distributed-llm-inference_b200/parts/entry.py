"""Parts that act on the residual stream between layers."""

from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import Part, ResidualStream, register_part


@register_part("stream_entry", "reinject")
class Reinject(Part):
    """What a looped span of layers adds to the stream before one of its passes: the embedding of the step's
    tokens once more (if ``table`` names the embedding tensor) and row ``row`` of a learned table of vectors
    [rows, size] (if ``vector`` names it).  One kernel: h += table[token_ids] + vector[row].
    params: size, vocab_size, table, vector, row, rows."""

    graph_capturable = True

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        p = spec.params
        self.size, self.vocab = int(p["size"]), int(p["vocab_size"])
        self.table_name, self.vector_name = p.get("table"), p.get("vector")
        self.row, self.rows = int(p.get("row", 0)), int(p.get("rows", 1))
        self.table: torch.Tensor | None = None
        self.vector: torch.Tensor | None = None

    def declare(self):
        out = {}
        if self.table_name:
            out[self.table_name] = TensorDecl((self.vocab, self.size))
        if self.vector_name:
            out[self.vector_name] = TensorDecl((self.rows, self.size), "vector32")
        return out

    def load(self, tensors):
        if self.table_name:
            self.table = tensors[self.table_name]
        if self.vector_name:
            self.vector = tensors[self.vector_name][self.row].contiguous()

    def apply(self, stream: ResidualStream, batch) -> None:
        h = stream.settle()
        if self.table is not None or self.vector is not None:
            ops.stream_reinject(h, self.table, batch.token_ids if self.table is not None else None, self.vector)
