"""Attention whose output is the difference of two softmax maps over the same values, behind short causal
taps on its projections.

Per token: q (heads x 2 x dim), k (kv_heads x 2 x dim) and v (kv_heads x value_dim) come from one product over
the packed rows [W_q; W_k; W_v; W_g] and get their biases; every channel of q, k and v then passes a causal
filter of `taps` taps over time (the last taps - 1 projected rows of a sequence are part of its state); the
leading channels of every q and k vector are turned by the position encoding; keys and values go to the
cache.  Each query head holds two query vectors (map 1, map 2) and meets the two key vectors of its
key/value head; each map is a softmax of (q . k) * scale over the keys j <= i with i - j < window or
j < keep_first (kept first tokens stay where they are: their positions are their own), and both maps weigh the
same values.  With lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff, one number per layer,

    o = a1 - lambda * a2,   o <- o / sqrt(mean(o^2) + eps) * (1 - diff)   per head,

then times sigmoid of the head's gate logit (a row of W_g per head, read from the mixer's input), then the
output projection.  Scores, softmax, the difference and the unit norm are float32.

A layer with `shares_kv` has no key and value tensors: it attends over the cache of the layer whose state
unit the plan lends it (`PlanEntry.reads`), with queries, taps, mask and lambda of its own.

State: the pages of keys and values (every position is kept, since kept first tokens rule out a ring), and
the last `taps` projected rows (float32; the row of position s lies in row s % taps).  Every kind of step runs the same two kernels, which read all keys
from the cache, so whole prompts, portions and single tokens agree.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.spec import CompositeStateSpec, FixedStateSpec, KVStateSpec
from ..weights.loader import TensorSpec
from .base import Mixer, register_part
from .linear import Linear


class DiffAttention(Mixer):
    prompt_capturable = True
    supports_append = True

    def __init__(self, prefix, hidden, heads, kv_heads, dim, value_dim, taps, window, keep_first, position, scale,
                 diff, eps, shares_kv=False, out_dtype=None):
        self.prefix, self.hidden = prefix, hidden
        self.heads, self.kv_heads, self.dim, self.value_dim = heads, kv_heads, dim, value_dim
        self.taps, self.window, self.keep_first = int(taps), int(window or 0), int(keep_first or 0)
        self.position, self.scale, self.diff, self.eps = position, float(scale), float(diff), float(eps)
        self.shares_kv = bool(shares_kv)
        self.out_dtype = {None: None, "float32": torch.float32}[out_dtype]
        self.q_size = heads * 2 * dim
        self.k_size, self.v_size = (0, 0) if self.shares_kv else (kv_heads * 2 * dim, kv_heads * value_dim)
        self.channels = self.q_size + self.k_size + self.v_size          # what the taps run over
        self.cache_head = -(-max(2 * dim, value_dim) // 8) * 8             # one entry size for a key row and a value row
        self.filtered = ["q"] if self.shares_kv else ["q", "k", "v"]
        rows = {"q": self.q_size, "k": self.k_size, "v": self.v_size}
        self.rows = [rows[n] for n in self.filtered]
        self.qkvg = Linear([prefix + n for n in self.filtered] + [prefix + "g"], self.rows + [heads], hidden)
        self.out = Linear(prefix + "o", hidden, heads * value_dim)
        self.bias = self.tap_w = None
        self.lam = 0.0

    def children(self):
        return [self.qkvg, self.out, self.position]

    def tensor_specs(self):
        p = self.prefix
        specs = []
        for n, r in zip(self.filtered, self.rows):
            specs += [TensorSpec(f"{p}{n}.b", (r,), "vector"), TensorSpec(f"{p}{n}.conv", (r, self.taps), "conv")]
        return specs + [TensorSpec(p + n, (self.dim,), "vector") for n in ("lq1", "lk1", "lq2", "lk2")]

    def bind(self, tensors, rt):
        p = self.prefix
        f32 = lambda n: tensors[p + n].to(torch.float32)
        self.bias = torch.cat([f32(n + ".b") for n in self.filtered]).contiguous()
        self.tap_w = torch.cat([f32(n + ".conv") for n in self.filtered]).contiguous()
        lam = torch.exp((f32("lq1") * f32("lk1")).sum()) - torch.exp((f32("lq2") * f32("lk2")).sum())
        self.lam = float(lam) + self.diff
        self._bound = [self.bias, self.tap_w]

    def state_spec(self):
        own = FixedStateSpec((max(1, self.taps * self.channels if self.taps > 1 else 1),), "float32")   # a ring of `taps` rows
        if self.shares_kv:
            return own
        return CompositeStateSpec((KVStateSpec(self.kv_heads, self.cache_head, 0), own))

    def forward(self, rt, batch, x, state):
        H, G, D, DV = self.heads, self.kv_heads, self.dim, self.value_dim
        if self.shares_kv:
            if not state.borrowed:
                raise ValueError("a layer that shares keys and values must be lent another layer's state unit by the plan")
            kv, own = state.borrowed[0].views[0], state
        else:
            kv, own = state.views
        proj = self.qkvg.apply(rt, x)                    # [T, channels + heads]
        q = torch.empty((batch.T, self.q_size), dtype=x.dtype, device=x.device)
        one_each = batch.kind == "decode"
        kernels.tap_rotate_store(proj, self.bias, self.tap_w, own.tensor, q, batch, self.q_size, D,
                                 self.position.rate_table(), getattr(self.position, "magnitude", 1.0),
                                 kv=None if self.shares_kv else (kv.pool, kv.pages, kv.ptab, G, 2 * D, DV),
                                 one_token_each=one_each)
        ctx = torch.empty((batch.T, H * DV), dtype=x.dtype, device=x.device)
        parts, splits = None, 1
        if one_each:
            # sized by the longest sequence that the step's class of lengths allows, so that a recording serves the class
            reach = kv.spec.entries(kv.spec.length_class(batch.max_end))
            keys = min(reach, self.window + self.keep_first) if self.window > 0 else reach
            splits = kernels.diff_attn_splits(batch.T, H, G, keys)
            if splits > 1:
                parts = rt.scratch("diff_attn_parts", batch.T * H * splits * (4 + 2 * DV))
        kernels.diff_attn(ctx, q, proj[:, self.channels:], kv.pool, kv.pages, kv.ptab, batch, H, G, D, DV, self.window,
                          self.keep_first, self.scale, self.lam, 1.0 - self.diff, self.eps, rows_form=one_each,
                          parts=parts, splits=splits,
                          tensor_cores=(not one_each and x.dtype == torch.bfloat16 and rt.tensor_core_prompts
                                        and kernels.diff_attn_mma_fits(D, DV, H, self.q_size, self.cache_head)))
        return self.out.apply(rt, ctx, out_dtype=self.out_dtype)


register_part("mixer", "diff_attention", DiffAttention)
