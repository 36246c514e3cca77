"""Configuration of the Narasun decoder.

config.json is nested: `vocab`, `width`, `norm.eps`; `layers`, a list whose entries give `type` (which
mixer the layer has), `mixer` (its sizes and constants) and `mlp` (the feed-forward, or null for none);
`loop` (or null): layers start .. stop-1 run `times` times in a row with the same weights.

Mixer types: `parallel` (an attention with a sink, `mixer.left`, beside a decay mix, `mixer.right`, with
`left_scale` and `right_scale`) and `mlstm` (matrix memory).  A type may carry a numeric suffix
(`mlstm_2`): it names the same mixer.  Feed-forward kinds: `dense` (`ff`) and `moe` (`expert.ff`,
`router.experts`, `router.top`).  The rank of the decay mix's low-rank decay network is not in config.json
of a checkpoint: it is the first dimension of the tensor `l<i>.mix.right.w1` (`with_tensor_shapes`); a
configuration for random weights gives it as `mixer.right.rank`.
"""
from __future__ import annotations

import dataclasses

from ..csrc import limits
from .base import ConfigError, Reader, base_type, section as _section

MIXER_TYPES = ("parallel", "mlstm")
MLP_KINDS = ("dense", "moe")


@dataclasses.dataclass(frozen=True)
class SinkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    q_temp_coef: float
    q_temp_every: int      # 0: no query temperature


@dataclasses.dataclass(frozen=True)
class DecayMixConfig:
    heads: int
    dim: int
    rank: int              # 0 until the tensors have been seen


@dataclasses.dataclass(frozen=True)
class ParallelMixerConfig:
    left: SinkAttentionConfig
    right: DecayMixConfig
    left_scale: float
    right_scale: float


@dataclasses.dataclass(frozen=True)
class MatrixMemoryConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclasses.dataclass(frozen=True)
class MlpConfig:
    kind: str              # dense | moe
    ff: int
    experts: int = 0
    top: int = 0


@dataclasses.dataclass(frozen=True)
class LayerConfig:
    type: str              # as written in config.json
    kind: str              # parallel | mlstm
    mixer: object
    mlp: object            # MlpConfig or None


@dataclasses.dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


@dataclasses.dataclass(frozen=True)
class NarasunConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    layers: tuple
    loop: object           # LoopConfig or None
    raw: dict = dataclasses.field(compare=False, default=None)

    @classmethod
    def from_dict(cls, data, where="config.json"):
        r = Reader(data, where)
        arch = r.string("architecture")
        vocab, width = r.integer("vocab", minimum=1), r.integer("width", minimum=1)
        norm = _section(r, data, "norm", "")
        eps = norm.number("eps", positive=True) if norm else None
        layers = []
        raw_layers = data.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            r.problem("'layers' must be a non-empty list")
            raw_layers = []
        for i, entry in enumerate(raw_layers):
            layers.append(cls._layer(r, entry, f"layers[{i}]."))
        loop = None
        if data.get("loop") is not None:
            lr = _section(r, data, "loop", "")
            if lr:
                loop = LoopConfig(lr.integer("start", minimum=0), lr.integer("stop", minimum=1), lr.integer("times", minimum=1))
        r.finish()
        cfg = cls(arch, vocab, width, eps, tuple(layers), loop, data)
        cfg.validate(where)
        return cfg

    @staticmethod
    def _layer(r, entry, where):
        if not isinstance(entry, dict) or not isinstance(entry.get("type"), str):
            r.problem(f"'{where}type' must be a string")
            return None
        kind = base_type(entry["type"])
        if kind not in MIXER_TYPES:
            r.problem(f"'{where}type' is '{entry['type']}'; known mixers: {', '.join(MIXER_TYPES)}")
            return None
        m = _section(r, entry, "mixer", where)
        mixer = None
        if m and kind == "parallel":
            left, right = _section(r, m.data, "left", where + "mixer."), _section(r, m.data, "right", where + "mixer.")
            lc = rc = None
            if left:
                qt = _section(r, left.data, "q_temp", where + "mixer.left.", required=False)
                heads = left.integer("heads", minimum=1)
                dim = left.integer("dim", minimum=1)
                lc = SinkAttentionConfig(heads, left.integer("kv_heads", default=heads, minimum=1), dim,
                                         left.integer("vdim", default=dim, minimum=1), left.number("scale", positive=True),
                                         qt.number("coef") if qt else 0.0, qt.integer("every", minimum=1) if qt else 0)
            if right:
                rc = DecayMixConfig(right.integer("heads", minimum=1), right.integer("dim", minimum=1),
                                    right.integer("rank", default=0, minimum=0))
            mixer = ParallelMixerConfig(lc, rc, m.number("left_scale", default=1.0), m.number("right_scale", default=1.0))
        elif m:
            dim = m.integer("dim", minimum=1)
            mixer = MatrixMemoryConfig(m.integer("heads", minimum=1), dim, m.integer("vdim", default=dim, minimum=1),
                                       m.number("gate_cap", positive=True))
        mlp = None
        if entry.get("mlp") is not None:
            f = _section(r, entry, "mlp", where)
            kindf = f.string("kind") if f else None
            if kindf == "dense":
                mlp = MlpConfig("dense", f.integer("ff", minimum=1))
            elif kindf == "moe":
                ex, ro = _section(r, f.data, "expert", where + "mlp."), _section(r, f.data, "router", where + "mlp.")
                if ex and ro:
                    mlp = MlpConfig("moe", ex.integer("ff", minimum=1), ro.integer("experts", minimum=1),
                                    ro.integer("top", minimum=1))
            elif kindf is not None:
                r.problem(f"'{where}mlp.kind' is '{kindf}'; known: {', '.join(MLP_KINDS)}")
        return LayerConfig(entry["type"], kind, mixer, mlp)

    def validate(self, where="config"):
        from ..parts.recurrent import scan_fits

        problems = []
        for i, layer in enumerate(self.layers):
            if layer is None or layer.mixer is None:
                continue
            if layer.kind == "parallel":
                a, d = layer.mixer.left, layer.mixer.right
                if a is None or d is None:
                    continue
                if a.heads % a.kv_heads:
                    problems.append(f"layers[{i}]: {a.heads} heads over {a.kv_heads} kv_heads")
                if -(-max(a.dim, a.vdim) // 16) * 16 > limits.MAX_HEAD_DIM:
                    problems.append(f"layers[{i}]: attention heads of {max(a.dim, a.vdim)}: the kernels take up to {limits.MAX_HEAD_DIM}")
                if not scan_fits(d.dim, d.dim):
                    problems.append(f"layers[{i}]: decay-mix heads of {d.dim} channels: the scan kernel takes up to 1024")
            else:
                m = layer.mixer
                if not scan_fits(m.dim, m.vdim):
                    problems.append(f"layers[{i}]: matrix-memory heads of {m.dim} key channels: the scan kernel takes up to 1024")
            if layer.mlp is not None and layer.mlp.kind == "moe" and layer.mlp.top > layer.mlp.experts:
                problems.append(f"layers[{i}]: top {layer.mlp.top} of {layer.mlp.experts} experts")
        if self.loop is not None and not 0 <= self.loop.start < self.loop.stop <= len(self.layers):
            problems.append(f"loop {self.loop.start}..{self.loop.stop} does not lie within {len(self.layers)} layers")
        if problems:
            raise ConfigError(f"{where}: " + "; ".join(problems))

    def with_tensor_shapes(self, shapes):
        """The same configuration with the sizes that only the tensors give (the decay network's rank)."""
        layers = []
        for i, layer in enumerate(self.layers):
            if layer.kind == "parallel" and layer.mixer.right.rank == 0:
                shape = shapes.get(f"l{i}.mix.right.w1")
                if shape is None or len(shape) != 2:
                    raise ConfigError(f"layer {i}: the tensor 'l{i}.mix.right.w1' that gives the decay network's rank is missing")
                right = dataclasses.replace(layer.mixer.right, rank=int(shape[0]))
                layer = dataclasses.replace(layer, mixer=dataclasses.replace(layer.mixer, right=right))
            layers.append(layer)
        return dataclasses.replace(self, layers=tuple(layers))

    def run_order(self):
        """[(layer, pass that begins right before it, or None)] in the order the layers run."""
        L = len(self.layers)
        if self.loop is None:
            return [(l, None) for l in range(L)]
        lo, hi = self.loop.start, self.loop.stop
        out = [(l, None) for l in range(lo)]
        for t in range(self.loop.times):
            out += [(l, t if l == lo else None) for l in range(lo, hi)]
        return out + [(l, None) for l in range(hi, L)]

    def to_dict(self):
        return self.raw
