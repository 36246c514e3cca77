"""The Narasun decoder as parts.

A layer is a `ParallelBlock`: one norm (stored as the weight's distance from one), whose output both the
mixer and the feed-forward read, and one residual sum, kept in float32.  The mixer is either an attention
with a sink beside a decay mix (`side_by_side` of `gqa_attention` and `decay_mix`) or a matrix memory; the
feed-forward a dense gated one, a routed one (sigmoid scores, the weight on the expert's input) or none.
A loop runs layers start .. stop-1 `times` times with the same weights: the plan names the same blocks
again with state units of their own, and every pass begins with a `loop_entry` block (a projection of the
stream and the embedding, plus the pass's learned row).

Tensor names: `embed`, `loop.in`, `loop.step`, `l<i>.norm1`, `l<i>.mix.*` (`left.{q,k,v,o,sink}`,
`right.{r,k,v,g,o,w1,w2,w0,u,norm,mu.{r,k,v,g,w}}`, or `{q,k,v,g,o,norm,i,i.b,f,f.b}`),
`l<i>.mlp.{gate,up,down}` or `l<i>.mlp.{router,e<j>.{gate,up,down}}`, `final.norm`, `head`.
"""
from __future__ import annotations

from ..config.narasun import NarasunConfig
from ..config.registry import register_architecture
from ..engine.definition import ModelDefinition, PlanEntry
from ..parts import build_part
from ..parts.linear import Linear


def _mixer(cfg, i, layer):
    W, eps, p = cfg.width, cfg.norm_eps, f"l{i}.mix."
    if layer.kind == "parallel":
        a, d = layer.mixer.left, layer.mixer.right
        left = build_part("mixer", "gqa_attention", prefix=p + "left.", hidden=W, heads=a.heads, kv_heads=a.kv_heads,
                          head_dim=a.dim, value_dim=a.vdim, window=0, position=build_part("position", "none"),
                          qk_norm_eps=None, output_gate=False, scale=a.scale, sink_name="sink",
                          q_temp=(a.q_temp_coef, a.q_temp_every) if a.q_temp_every else None,
                          names={"q": "q", "k": "k", "v": "v", "out": "o"}, out_dtype="float32")
        right = build_part("mixer", "decay_mix", prefix=p + "right.", hidden=W, heads=d.heads, dim=d.dim, rank=d.rank,
                           eps=eps, out_dtype="float32")
        return build_part("mixer", "side_by_side", a=left, b=right, a_scale=layer.mixer.left_scale,
                          b_scale=layer.mixer.right_scale)
    m = layer.mixer
    return build_part("mixer", "matrix_memory", prefix=p, hidden=W, heads=m.heads, dim=m.dim, value_dim=m.vdim,
                      gate_cap=m.gate_cap, eps=eps, out_dtype="float32")


def _feed_forward(cfg, i, mlp):
    if mlp is None:
        return None
    p = f"l{i}.mlp."
    if mlp.kind == "dense":
        return build_part("feed_forward", "swiglu", prefix=p, hidden=cfg.width, intermediate=mlp.ff,
                          names={"gate": "gate", "up": "up", "down": "down"}, out_dtype="float32")
    return build_part("feed_forward", "routed_swiglu", prefix=p, hidden=cfg.width, intermediate=mlp.ff,
                      experts=mlp.experts, top=mlp.top, gate="sigmoid", renormalize=False, weight_on="input")


def define(cfg: NarasunConfig) -> ModelDefinition:
    W = cfg.width
    if any(l.kind == "parallel" and l.mixer.right.rank == 0 for l in cfg.layers):
        raise ValueError("the decay network's rank is unknown: give 'mixer.right.rank', or load the model from its tensors")
    norm = lambda name: build_part("norm", "rms", name=name, width=W, eps=cfg.norm_eps, weight_offset=1.0)
    blocks = [build_part("block", "parallel", mixer=_mixer(cfg, i, layer), feed_forward=_feed_forward(cfg, i, layer.mlp),
                         input_norm=norm(f"l{i}.norm1")) for i, layer in enumerate(cfg.layers)]
    plan, unit = [], 0
    for layer, begins in cfg.run_order():
        if begins is not None:
            blocks.append(build_part("block", "loop_entry", in_name="loop.in", step_name="loop.step", hidden=W,
                                     passes=cfg.loop.times, index=begins))
            plan.append(PlanEntry(block=len(blocks) - 1, state=unit))       # no state of its own: the unit stays empty
            unit += 1
        plan.append(PlanEntry(block=layer, state=unit))                     # every run of a layer has its own state
        unit += 1
    return ModelDefinition(
        architecture=cfg.architecture, vocab_size=cfg.vocab, hidden_size=W, embedding_name="embed", blocks=blocks,
        plan=plan, final_norm=norm("final.norm"), head=Linear("head", cfg.vocab, W), residual_float32=True,
        keep_embedding=cfg.loop is not None)


register_architecture("Narasun", NarasunConfig, define)
