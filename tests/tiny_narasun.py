"""Small Narasun configurations for the tests, and weights for them that make a fault visible.

The configurations differ from each other in every size, in the order and kinds of layers, in the loop
(inside the stack, over the whole stack, none) and in the constants; sizes that could hide a fault by
being equal (query and value head sizes, heads and key/value heads) or by being 1 (experts used per
token, heads) take both forms.  Weights are drawn so that activations are of order one: matrices
N(0, 1/in), sinks of the order of the scores, decays between 0.2 and 0.99, forget gates near one.
Everything is stored in bfloat16, as a checkpoint is.
"""
import hashlib
import json
import os

import torch


def attention(heads, kv_heads, dim, vdim, scale, coef, every):
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, q_temp=dict(coef=coef, every=every))


def parallel(left, right_heads, right_dim, rank, left_scale, right_scale, mlp, suffix=""):
    return dict(type="parallel" + suffix, mlp=mlp,
                mixer=dict(left=left, right=dict(heads=right_heads, dim=right_dim, rank=rank),
                           left_scale=left_scale, right_scale=right_scale))


def mlstm(heads, dim, vdim, cap, mlp, suffix=""):
    return dict(type="mlstm" + suffix, mlp=mlp, mixer=dict(heads=heads, dim=dim, vdim=vdim, gate_cap=cap))


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(ff, experts, top):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))


# P: a loop inside the stack whose first layer is a matrix memory; two experts per token; a layer without feed-forward;
# a decay network wide enough (rank 32) to run as two products
TINY_P = dict(architecture="Narasun", vocab=200, width=64, norm=dict(eps=1e-5), loop=dict(start=0, stop=2, times=2), layers=[
    mlstm(2, 16, 24, 10.0, moe(40, 5, 2)),
    parallel(attention(4, 2, 16, 16, 0.3, 0.4, 8), 2, 16, 32, 0.7, 1.1, dense(96)),
    mlstm(4, 8, 8, 8.0, None, "_3")])

# Q: no loop; value heads larger than query heads (and no multiple of 16); one key/value head per query head, and one
# for all; a single head; one expert per token
TINY_Q = dict(architecture="Narasun", vocab=130, width=48, norm=dict(eps=1e-6), loop=None, layers=[
    parallel(attention(3, 3, 24, 40, 0.2, 0.3, 5), 3, 8, 4, 1.0, 0.5, moe(24, 3, 1)),
    parallel(attention(2, 1, 32, 32, 0.15, 0.0, 3), 1, 32, 16, 0.9, 0.8, None, "_2"),
    mlstm(1, 32, 16, 15.0, dense(64))])

# R: the loop is the whole stack, three passes, with an attention layer inside it; value heads smaller than query heads
TINY_R = dict(architecture="Narasun", vocab=96, width=32, norm=dict(eps=1e-6), loop=dict(start=0, stop=2, times=3), layers=[
    parallel(attention(2, 2, 16, 8, 0.25, 0.5, 64), 2, 8, 4, 0.8, 0.9, moe(16, 4, 3)),
    mlstm(2, 8, 16, 12.0, dense(48), "_2")])

# D: P with dense feed-forwards in place of the routed ones (nothing in it decides between alternatives)
TINY_D = dict(TINY_P, layers=[mlstm(2, 16, 24, 10.0, dense(40)), TINY_P["layers"][1], TINY_P["layers"][2]])

# O: sizes that are multiples of nothing convenient (width 36, heads of 12 and 20, 77 tokens, rank 5, an inner width of 28)
TINY_O = dict(architecture="Narasun", vocab=77, width=36, norm=dict(eps=1e-5), loop=dict(start=1, stop=2, times=2), layers=[
    parallel(attention(2, 1, 12, 20, 0.3, 0.2, 7), 1, 12, 5, 1.0, 1.0, moe(20, 3, 2)),
    mlstm(3, 12, 20, 9.0, dense(28))])

# one mechanism at a time
ONLY_ATTENTION_MIX = dict(architecture="Narasun", vocab=64, width=32, norm=dict(eps=1e-6), loop=None, layers=[
    parallel(attention(2, 1, 16, 16, 0.25, 0.7, 4), 2, 16, 4, 1.0, 1.0, None)])
ONLY_MEMORY = dict(architecture="Narasun", vocab=64, width=40, norm=dict(eps=1e-6), loop=None, layers=[
    mlstm(2, 24, 40, 6.0, None)])
ONLY_MEMORY_MOE = dict(architecture="Narasun", vocab=64, width=40, norm=dict(eps=1e-6), loop=None, layers=[
    mlstm(1, 8, 8, 6.0, moe(24, 7, 3))])
ONLY_LOOP = dict(architecture="Narasun", vocab=64, width=24, norm=dict(eps=1e-6), loop=dict(start=0, stop=1, times=2), layers=[
    mlstm(1, 8, 8, 6.0, dense(32))])

ALL = {"P": TINY_P, "Q": TINY_Q, "R": TINY_R, "D": TINY_D, "O": TINY_O, "attention_mix": ONLY_ATTENTION_MIX, "memory": ONLY_MEMORY,
       "memory_moe": ONLY_MEMORY_MOE, "loop": ONLY_LOOP}


def _gen(seed, name):
    g = torch.Generator()
    g.manual_seed(int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little") & ((1 << 63) - 1))
    return g


def make_tensors(config, seed):
    """{name: bfloat16 tensor} for a configuration dict."""
    from catena_models_b200.config.registry import config_from_dict

    arch, typed = config_from_dict(config)
    out = {}
    for spec in arch.define(typed).tensor_specs():
        g, name, shape = _gen(seed, spec.name), spec.name, tuple(spec.shape)
        n = lambda std=1.0: torch.randn(shape, generator=g) * std
        u = lambda lo, hi: lo + (hi - lo) * torch.rand(shape, generator=g)
        tail = name.split(".")[-1]
        if name.endswith("norm1") or name == "final.norm":
            t = n(0.1)
        elif name == "embed":
            t = n(1.0)
        elif tail == "sink":
            t = n(1.5)
        elif ".mu." in name:
            t = u(0.0, 1.0)
        elif tail == "w0":
            t = u(-2.5, 0.3)
        elif tail == "u":
            t = n(0.5)
        elif tail == "norm":
            t = 1.0 + n(0.1)
        elif name.endswith("i.b"):
            t = n(1.0)
        elif name.endswith("f.b"):
            t = u(2.0, 5.0)
        elif name == "loop.step":
            t = n(0.2)
        elif tail == "router":
            t = n(1.0 / shape[1] ** 0.5) * 2.0
        else:
            t = n(1.0 / shape[-1] ** 0.5)
        out[name] = t.to(torch.bfloat16)
    return out


def make_folder(tmp, name, seed=0, config=None):
    from catena_models_b200.weights.safetensors_io import write_safetensors

    config = config or ALL[name]
    folder = os.path.join(str(tmp), name)
    os.makedirs(folder, exist_ok=True)
    stored = json.loads(json.dumps(config))
    for layer in stored["layers"]:                      # a checkpoint's config.json does not give the decay network's rank
        if "right" in layer["mixer"]:
            layer["mixer"]["right"].pop("rank", None)
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump(stored, fh)
    write_safetensors(os.path.join(folder, "model.safetensors"), make_tensors(config, seed))
    return folder


def load_plain(folder):
    """(config dict, {name: tensor}) as the plain implementation takes them."""
    from catena_models_b200.weights.safetensors_io import SafetensorsFile

    with open(os.path.join(folder, "config.json")) as fh:
        cfg = json.load(fh)
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    f.close()
    return cfg, tensors


def prompt(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
