"""Arrangements for models whose residual stream is float32 whatever the activation dtype.

`SideBySide`: two mixers that read the same input; the result is a_scale * a + b_scale * b.  Each keeps
its own state (the layer's state spec is the pair of theirs).

`ParallelBlock`: one norm, and both sublayers read its output: with n = norm(h), h <- h + (mixer(n) +
feed_forward(n)); the feed-forward may be absent.  The sum of all terms, the float32 residual sum and the
norm of whatever runs next are one kernel (`residual_add_norm`), as the sandwich block's `add_norm` is.

`PreNormBlock`: the sequential arrangement on the same stream: a norm and a mixer, then a norm and a
feed-forward, each sum with a constant factor.

`LoopEntry`: the step between two passes of a looped stack: h <- W [h; h0] + step, h0 being the embedding
rows of the batch (the definition keeps them: `keep_embedding`) and `step` a learned row of the pass.  It
has no norm of its own and no state; the product's float32 result becomes the new residual stream, and the
row is added in the kernel that forms the next block's norm.

Sublayers hand their result over as a tensor or as `kernels.Terms` (pieces with a factor each), and a final
projection may leave its result in float32 (`out_dtype`): nothing is rounded between a projection and
the residual sum.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.spec import CompositeStateSpec
from ..weights.loader import TensorSpec
from .base import Block, Mixer, register_part
from .linear import Linear


def _terms(y):
    return y if isinstance(y, kernels.Terms) else kernels.Terms([(y, 1.0, 1)])


class SideBySide(Mixer):
    prompt_capturable = True
    supports_append = True

    def __init__(self, a, b, a_scale=1.0, b_scale=1.0):
        self.a, self.b, self.a_scale, self.b_scale = a, b, float(a_scale), float(b_scale)

    def children(self):
        return [self.a, self.b]

    def state_spec(self):
        return CompositeStateSpec((self.a.state_spec(), self.b.state_spec()))

    def forward(self, rt, batch, x, state):
        out = kernels.Terms()
        for i, (mixer, scale) in enumerate(((self.a, self.a_scale), (self.b, self.b_scale))):
            view = state.views[i]
            view.owned, view.unit = state.owned, (state.unit, i)
            out += [(e[0], e[1] * scale, *e[2:]) for e in _terms(mixer.forward(rt, batch, x, view))]
        return out


class ParallelBlock(Block):
    prompt_capturable = True
    supports_append = True

    def __init__(self, mixer, feed_forward, input_norm):
        self.mixer, self.feed_forward, self.input_norm = mixer, feed_forward, input_norm

    def children(self):
        return [p for p in (self.input_norm, self.mixer, self.feed_forward) if p is not None]

    def state_spec(self):
        return self.mixer.state_spec()

    def forward(self, rt, batch, h, n, state, next_norm):
        if h.dtype != torch.float32:
            raise ValueError("ParallelBlock works on a float32 residual stream (ModelDefinition.residual_float32)")
        batch.partial_sums_ok = False
        terms = _terms(self.mixer.forward(rt, batch, n, state))
        if self.feed_forward is not None:
            terms = kernels.Terms(terms + _terms(self.feed_forward.forward(rt, batch, n)))
        return _sum_and_norm(rt, h, terms, None, next_norm)


def _sum_and_norm(rt, h, terms, bias, next_norm):
    """h += terms (+ bias); the next norm in the same kernel when it is an RMS norm or a dynamic tanh."""
    kind = getattr(next_norm, "fused_kind", None) if next_norm is not None else None
    fuse = kind in ("rms", "dyt")
    n_out = torch.empty(h.shape, dtype=rt.dtype, device=h.device) if fuse else None
    kernels.residual_add_norm(h, terms, n_out, next_norm.weight if fuse else None, next_norm.eps if fuse else 0.0, bias,
                              dyt=(next_norm.alpha, next_norm.shift) if kind == "dyt" else None)
    return h, n_out


class PreNormBlock(Block):
    """Two sublayers one after the other on a float32 stream, each behind a norm of its own and each added with
    the same constant factor: h <- h + c * mixer(norm1(h)), then h <- h + c * feed_forward(norm2(h)); the
    feed-forward (and its norm) may be absent.  Each sum forms the norm of whatever reads the stream next."""
    prompt_capturable = True
    supports_append = True

    def __init__(self, mixer, feed_forward, input_norm, ffn_norm, residual_scale=1.0):
        if (feed_forward is None) != (ffn_norm is None):
            raise ValueError("a feed-forward and its norm come together")
        self.mixer, self.feed_forward, self.input_norm, self.ffn_norm = mixer, feed_forward, input_norm, ffn_norm
        self.residual_scale = float(residual_scale)

    def children(self):
        return [p for p in (self.input_norm, self.mixer, self.ffn_norm, self.feed_forward) if p is not None]

    def state_spec(self):
        return self.mixer.state_spec()

    def _scaled(self, y):
        return kernels.Terms([(e[0], e[1] * self.residual_scale, *e[2:]) for e in _terms(y)])

    def forward(self, rt, batch, h, n, state, next_norm):
        if h.dtype != torch.float32:
            raise ValueError("PreNormBlock works on a float32 residual stream (ModelDefinition.residual_float32)")
        batch.partial_sums_ok = False
        if n is None:
            n = self.input_norm.apply(rt, h)
        y = self._scaled(self.mixer.forward(rt, batch, n, state))
        if self.feed_forward is None:
            return _sum_and_norm(rt, h, y, None, next_norm)
        h, n2 = _sum_and_norm(rt, h, y, None, self.ffn_norm)
        if n2 is None:
            n2 = self.ffn_norm.apply(rt, h)
        return _sum_and_norm(rt, h, self._scaled(self.feed_forward.forward(rt, batch, n2)), None, next_norm)


class LoopEntry(Block):
    prompt_capturable = True
    supports_append = True

    def __init__(self, in_name, step_name, hidden, passes, index):
        self.hidden, self.passes, self.index, self.step_name = hidden, passes, index, step_name
        self.proj = Linear(in_name, hidden, 2 * hidden)
        self.step = None

    def children(self):
        return [self.proj]

    def tensor_specs(self):
        return [TensorSpec(self.step_name, (self.passes, self.hidden), "vector")]

    def bind(self, tensors, rt):
        self.step = tensors[self.step_name].to(torch.float32)[self.index].contiguous()
        self._bound = [self.step]

    def forward(self, rt, batch, h, n, state, next_norm):
        both = torch.empty((h.shape[0], 2 * self.hidden), dtype=rt.dtype, device=h.device)
        kernels.concat_cast(both, h, batch.shared["embedding"])
        h = self.proj.apply(rt, both, out_dtype=torch.float32)
        return _sum_and_norm(rt, h, kernels.Terms(), self.step, next_norm)


register_part("mixer", "side_by_side", SideBySide)
register_part("block", "parallel", ParallelBlock)
register_part("block", "prenorm", PreNormBlock)
register_part("block", "loop_entry", LoopEntry)
