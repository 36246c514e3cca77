"""Small Fozedra configurations for the tests, and weights for them that make a fault visible.

The configurations differ from each other in every size, in the order and kinds of layers and in the
constants; sizes that could hide a fault by being equal (key and value head sizes, heads and key/value heads,
turned channels and head size) or by being 1 or 0 (taps, kept first tokens, heads) take both forms.  Weights
are drawn so that activations are of order one: matrices N(0, 1/in), taps of order one, the dynamic tanh's
alpha near one half.  Everything is stored in bfloat16, as a checkpoint is.
"""
import hashlib
import json
import os

import torch


def lightning(heads, dim, vdim, mlp, decay=None):
    decay = decay or [round(0.5 + 0.499 * (i + 1) / heads, 6) for i in range(heads)]
    return dict(type="lightning", mlp=mlp, mixer=dict(heads=heads, dim=dim, vdim=vdim, decay=decay))


def attention(heads, kv_heads, dim, vdim, taps, diff, scale, size, keep, rot_dims, base=10000.0, scaling=None, mlp=None,
              kv_from=None):
    mixer = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=taps, diff=diff, scale=scale,
                 mask=dict(size=size, keep_first=keep),
                 rot=dict(dims=rot_dims, base=base, scaling=scaling or dict(factor=4.0, original=64, fast=16.0, slow=1.0)))
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return dict(type="attention", mlp=mlp, mixer=mixer)


def dense(ff):
    return dict(kind="dense", ff=ff)


def model(vocab, width, eps, mult, layers):
    return dict(architecture="Fozedra", vocab=vocab, width=width, norm=dict(eps=eps), residual_mult=mult, layers=layers)


# A: attention first; a reader of its keys right behind it and another two layers on; value heads smaller than key
# heads; all channels of a vector turned; windows shorter than a tile of keys
_A_ATT = dict(heads=4, kv_heads=2, dim=16, vdim=8, taps=4, diff=0.2, scale=0.25, size=9, keep=3, rot_dims=16)
TINY_A = model(150, 64, 1e-5, 0.7, [
    attention(**_A_ATT, mlp=dense(96)),
    attention(**_A_ATT, mlp=None, kv_from=0),
    lightning(2, 16, 24, dense(40)),
    attention(**_A_ATT, mlp=dense(48), kv_from=0)])

# B: sizes that are multiples of nothing convenient (width 36, heads of 12 and 20, 5 taps); one key/value head for all;
# no kept tokens; a single lightning head; windows that cross a page of 64; no factor on the residual
TINY_B = model(77, 36, 1e-6, 1.0, [
    lightning(1, 12, 20, None, decay=[0.93]),
    attention(3, 1, 12, 20, 5, 0.35, 0.3, 70, 0, 6, base=500.0, scaling=dict(factor=2.0, original=32, fast=8.0, slow=2.0),
              mlp=dense(28)),
    lightning(3, 4, 12, dense(20))])

# C: two taps; as many key/value heads as heads; more kept tokens than the window is wide; a rotation without much
# rescaling; key and value heads of one size
TINY_C = model(96, 32, 1e-6, 0.5, [
    attention(2, 2, 8, 16, 2, 0.5, 0.35, 5, 11, 4, base=100.0, scaling=dict(factor=1.5, original=16, fast=4.0, slow=1.0),
              mlp=dense(64)),
    attention(2, 2, 8, 16, 2, 0.1, 0.4, 33, 2, 4, base=100.0, scaling=dict(factor=1.5, original=16, fast=4.0, slow=1.0),
              mlp=None)])

# M: sizes that the tensor-core kernels take (head sizes that are multiples of 16, a width that is a multiple of 8): the
# bfloat16 engine then runs the attention's prompt form on mma.sync and its products on the tensor-core and streaming kernels
_M_ATT = dict(heads=4, kv_heads=2, dim=32, vdim=64, taps=3, diff=0.4, scale=0.18, size=72, keep=10, rot_dims=16, base=5000.0,
              scaling=dict(factor=3.0, original=128, fast=20.0, slow=1.0))
TINY_M = model(210, 128, 1e-6, 0.6, [
    lightning(2, 32, 64, dense(256)),
    attention(**_M_ATT, mlp=dense(192)),
    attention(**_M_ATT, mlp=None, kv_from=1),
    lightning(4, 16, 32, None)])

# one mechanism at a time
ONLY_LIGHTNING = model(64, 40, 1e-6, 1.0, [lightning(2, 24, 40, None)])
ONLY_ATTENTION = model(64, 32, 1e-6, 1.0, [attention(4, 1, 16, 24, 3, 0.3, 0.25, 12, 4, 8, mlp=None)])    # four query heads a key head
ONLY_TAPS_ONE = model(64, 32, 1e-6, 1.0, [attention(2, 1, 16, 16, 1, 0.3, 0.25, 1000, 0, 8, mlp=None)])
ONLY_FF = model(64, 24, 1e-6, 0.8, [lightning(1, 8, 8, dense(56))])

ALL = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "M": TINY_M, "lightning": ONLY_LIGHTNING, "attention": ONLY_ATTENTION,
       "taps_one": ONLY_TAPS_ONE, "ff": ONLY_FF}


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
        tail = name.split(".")[-1]
        if tail == "alpha":
            t = 0.5 + 0.2 * torch.rand(shape, generator=g)
        elif tail == "b":
            t = n(0.2)
        elif tail in ("norm1", "norm2") or name == "final.norm" or tail == "norm":
            t = 1.0 + n(0.1)
        elif name == "embed":
            t = n(1.0)
        elif tail == "conv":
            t = n(0.6)
        elif tail in ("lq1", "lk1", "lq2", "lk2"):
            t = n(0.3)
        else:
            t = n(1.0 / shape[-1] ** 0.5)
        out[name] = t.to(torch.bfloat16)
    return out


def make_folder(tmp, name, seed=0, config=None, tensors=None):
    from catena_models_b200.weights.safetensors_io import write_safetensors

    config = config or ALL[name]
    folder = os.path.join(str(tmp), name)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump(config, fh)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors or make_tensors(config, seed))
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
