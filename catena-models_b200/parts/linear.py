"""Projection y = x W^T with W stored [out, in], as every matrix of the reference is
(src/spec.rs:378-426).  Several tensors with the same input width can be packed row-wise
into one matrix at bind time, so that one matrix product serves them all (the reference
concatenates q, k, v and gate by column range inside its GEMM, src/lfm3.rs:1181-1196).
Which kernel runs (tensor-core GEMM, weight-streaming GEMV, 32-bit FMA) is the runtime's
decision from dtype and row count; this part only owns the weight.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import Part


class Linear(Part):
    prompt_capturable = True
    fused_decode_ok = True
    supports_append = True

    def __init__(self, names, rows, in_features, role="matrix", head_rows=None, head_cols=None):
        """head_rows: per tensor None or (heads, size, padded size): the tensor's rows are `heads` blocks of
        `size`, and each block is followed by padded - size rows of zeros in the bound matrix (outputs that
        are zero: a kernel with a fixed head size can then run heads of another size).  head_cols: the same
        for the columns of a single tensor (zero columns meet the padding of its input)."""
        self.names = [names] if isinstance(names, str) else list(names)
        self.rows = [rows] if isinstance(rows, int) else list(rows)
        self.in_features = in_features
        self.role = role
        self.weight = None
        self.head_rows = list(head_rows) if head_rows else [None] * len(self.names)
        self.head_cols = head_cols
        self.bound_rows = [r if p is None else p[0] * p[2] for r, p in zip(self.rows, self.head_rows)]
        self.out_features = sum(self.bound_rows)

    def tensor_specs(self):
        return [TensorSpec(n, (r, self.in_features), self.role) for n, r in zip(self.names, self.rows)]

    def bind(self, tensors, rt):
        parts = [self._padded(tensors[n], p) for n, p in zip(self.names, self.head_rows)]
        if len(parts) == 1:
            self.weight = parts[0]
        else:
            if len({p.dtype for p in parts}) > 1:
                parts = [p.to(torch.float32) for p in parts]
            self.weight = torch.cat(parts, dim=0).contiguous()
        self._bound = [self.weight]

    def _padded(self, w, rows):
        if rows is not None and rows[1] != rows[2]:
            heads, size, padded = rows
            out = torch.zeros((heads, padded, w.shape[1]), dtype=w.dtype, device=w.device)
            out[:, :size] = w.view(heads, size, w.shape[1])
            w = out.view(heads * padded, -1)
        if self.head_cols is not None and self.head_cols[1] != self.head_cols[2]:
            heads, size, padded = self.head_cols
            out = torch.zeros((w.shape[0], heads, padded), dtype=w.dtype, device=w.device)
            out[:, :, :size] = w.view(w.shape[0], heads, size)
            w = out.view(w.shape[0], heads * padded)
        return w.contiguous()

    def use_weight(self, weight):
        """Share another part's matrix (a tied output head uses the embedding table)."""
        self.weight = weight
        self._bound = []

    def apply(self, rt, x, out_dtype=None, partial_ok=False):
        """x @ weight^T.  `partial_ok`: the result goes straight into a residual sum that can add
        partial sums (StepBatch.partial_sums_ok says so), so the runtime may leave it as such."""
        return rt.linear(x, self.weight, out_dtype, partial_ok)
