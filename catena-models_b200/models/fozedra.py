"""The Fozedra decoder as parts.

A layer is a `PreNormBlock` on a float32 stream: a dynamic-tanh norm and a mixer, then (if the layer has
one) a dynamic-tanh norm and a squared-ReLU feed-forward, each added with the factor `residual_mult`.  The
mixer is lightning attention (`constant_decay_memory`) or an attention that takes the difference of two
softmax maps behind short causal taps, with a partial rotation rescaled for long contexts and a sliding
window that keeps the first tokens (`diff_attention`).  A layer with `kv_from` attends over another
layer's keys and values: the plan lends it that layer's state unit beside its own.  The output head is the
embedding table.

Tensor names: `embed`, `l<i>.norm1{,.alpha,.b}`, `l<i>.norm2{,.alpha,.b}`, `l<i>.mix.{q,k,v,g,o,norm}` or
`l<i>.mix.{q,k,v}{,.b,.conv}`, `l<i>.mix.{lq1,lk1,lq2,lk2,g,o}`, `l<i>.mlp.{up,down}`, `final.norm{,.alpha,.b}`.
"""
from __future__ import annotations

from ..config.fozedra import FozedraConfig
from ..config.registry import register_architecture
from ..engine.definition import ModelDefinition, PlanEntry
from ..parts import build_part


def _mixer(cfg, i, layer):
    W, m, p = cfg.width, layer.mixer, f"l{i}.mix."
    if layer.type == "lightning":
        return build_part("mixer", "constant_decay_memory", prefix=p, hidden=W, heads=m.heads, dim=m.dim, value_dim=m.vdim,
                          decay=m.decay, eps=cfg.norm_eps, out_dtype="float32")
    if m.rot is None:
        position = build_part("position", "none")
    else:
        position = build_part("position", "partial_yarn_rotary", dims=m.rot.dims, theta=m.rot.base, factor=m.rot.factor,
                              original=m.rot.original, fast=m.rot.fast, slow=m.rot.slow)
    return build_part("mixer", "diff_attention", prefix=p, hidden=W, heads=m.heads, kv_heads=m.kv_heads, dim=m.dim,
                      value_dim=m.vdim, taps=m.taps, window=m.window, keep_first=m.keep_first, position=position,
                      scale=m.scale, diff=m.diff, eps=cfg.norm_eps, shares_kv=m.kv_from is not None, out_dtype="float32")


def define(cfg: FozedraConfig) -> ModelDefinition:
    W = cfg.width
    norm = lambda name: build_part("norm", "dynamic_tanh", name=name, width=W)
    blocks, plan = [], []
    for i, layer in enumerate(cfg.layers):
        ff = None
        if layer.ff:
            ff = build_part("feed_forward", "relu_squared", prefix=f"l{i}.mlp.", hidden=W, intermediate=layer.ff,
                            out_dtype="float32")
        blocks.append(build_part("block", "prenorm", mixer=_mixer(cfg, i, layer), feed_forward=ff,
                                 input_norm=norm(f"l{i}.norm1"), ffn_norm=norm(f"l{i}.norm2") if ff else None,
                                 residual_scale=cfg.residual_mult))
        lender = layer.mixer.kv_from if layer.type == "attention" else None
        plan.append(PlanEntry(block=i, state=i, reads=() if lender is None else (lender,)))
    return ModelDefinition(architecture=cfg.architecture, vocab_size=cfg.vocab, hidden_size=W, embedding_name="embed",
                           blocks=blocks, plan=plan, final_norm=norm("final.norm"), head=None, residual_float32=True)


register_architecture("Fozedra", FozedraConfig, define)
