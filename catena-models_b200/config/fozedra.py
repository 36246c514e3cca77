"""Configuration of the Fozedra decoder.

config.json is nested: `vocab`, `width`, `norm.eps`, `residual_mult`; `layers`, a list whose entries give
`type` (which mixer the layer has), `mixer` (its sizes and constants) and `mlp` (the feed-forward, or null
for none).  Mixer types: `lightning` (`heads`, `dim`, `vdim`, `decay`: one number per head) and `attention`
(`heads`, `kv_heads`, `dim`, `vdim`, `conv`: taps, `diff`, `scale`, `mask.size`, `mask.keep_first`,
`rot.dims`, `rot.base`, `rot.scaling.{factor, original, fast, slow}`, and optionally `kv_from`: the layer
whose keys and values this layer uses).  Feed-forward kind: `dense` (`ff`).
"""
from __future__ import annotations

import dataclasses

from ..csrc import limits
from .base import ConfigError, Reader, base_type, section

MIXER_TYPES = ("lightning", "attention")


@dataclasses.dataclass(frozen=True)
class LightningConfig:
    heads: int
    dim: int
    vdim: int
    decay: tuple


@dataclasses.dataclass(frozen=True)
class RotationConfig:
    dims: int
    base: float
    factor: object           # None: no rescaling
    original: float
    fast: float
    slow: float


@dataclasses.dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    taps: int
    diff: float
    scale: float
    window: int
    keep_first: int
    rot: RotationConfig
    kv_from: object          # a layer index, or None


@dataclasses.dataclass(frozen=True)
class LayerConfig:
    type: str
    mixer: object
    ff: int                  # 0: no feed-forward


@dataclasses.dataclass(frozen=True)
class FozedraConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    layers: tuple
    raw: dict = dataclasses.field(compare=False, default=None)

    @classmethod
    def from_dict(cls, data, where="config.json"):
        r = Reader(data, where)
        arch = r.string("architecture")
        vocab, width = r.integer("vocab", minimum=1), r.integer("width", minimum=1)
        norm = section(r, data, "norm", "")
        eps = norm.number("eps", positive=True) if norm else None
        mult = r.number("residual_mult", default=1.0)
        raw_layers = data.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            r.problem("'layers' must be a non-empty list")
            raw_layers = []
        layers = [cls._layer(r, entry, f"layers[{i}].") for i, entry in enumerate(raw_layers)]
        r.finish()
        cfg = cls(arch, vocab, width, eps, mult, tuple(layers), data)
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
        m = section(r, entry, "mixer", where)
        mixer = None
        if m and kind == "lightning":
            dim = m.integer("dim", minimum=1)
            decay = m.data.get("decay")
            if not isinstance(decay, list) or not all(isinstance(w, (int, float)) and not isinstance(w, bool) for w in decay):
                r.problem(f"'{where}mixer.decay' must be a list of numbers")
                decay = []
            mixer = LightningConfig(m.integer("heads", minimum=1), dim, m.integer("vdim", default=dim, minimum=1),
                                    tuple(float(w) for w in decay))
        elif m:
            heads, dim = m.integer("heads", minimum=1), m.integer("dim", minimum=1)
            mask = section(r, m.data, "mask", where + "mixer.", required=False)
            rot = section(r, m.data, "rot", where + "mixer.", required=False)
            rc = None
            if rot:
                sc = section(r, rot.data, "scaling", where + "mixer.rot.", required=False)
                rc = RotationConfig(rot.integer("dims", minimum=2), rot.number("base", positive=True),
                                    sc.number("factor", positive=True) if sc else None,
                                    sc.number("original", positive=True) if sc else 0.0,
                                    sc.number("fast", positive=True) if sc else 0.0,
                                    sc.number("slow", positive=True) if sc else 0.0)
            mixer = AttentionConfig(heads, m.integer("kv_heads", default=heads, minimum=1), dim,
                                    m.integer("vdim", default=dim, minimum=1), m.integer("conv", default=1, minimum=1),
                                    m.number("diff"), m.number("scale", positive=True),
                                    mask.integer("size", default=0, minimum=0) if mask else 0,
                                    mask.integer("keep_first", default=0, minimum=0) if mask else 0, rc,
                                    m.integer("kv_from", default=None, minimum=0))
        ff = 0
        if entry.get("mlp") is not None:
            f = section(r, entry, "mlp", where)
            kindf = f.string("kind") if f else None
            if kindf == "dense":
                ff = f.integer("ff", minimum=1)
            elif kindf is not None:
                r.problem(f"'{where}mlp.kind' is '{kindf}'; known: dense")
        return LayerConfig(kind, mixer, ff or 0)

    def validate(self, where="config"):
        from ..parts.recurrent import scan_fits

        problems = []
        for i, layer in enumerate(self.layers):
            if layer is None or layer.mixer is None:
                continue
            m = layer.mixer
            if layer.type == "lightning":
                if len(m.decay) != m.heads:
                    problems.append(f"layers[{i}]: {len(m.decay)} decays for {m.heads} heads")
                if any(not 0.0 < w <= 1.0 for w in m.decay):
                    problems.append(f"layers[{i}]: a decay outside (0, 1]")
                if not scan_fits(m.dim, m.vdim):
                    problems.append(f"layers[{i}]: heads of {m.dim} key channels: the scan kernel takes up to 1024")
                continue
            if m.heads % m.kv_heads:
                problems.append(f"layers[{i}]: {m.heads} heads over {m.kv_heads} kv_heads")
            if m.vdim > limits.MAX_HEAD_DIM or 2 * m.dim > 2 * limits.MAX_HEAD_DIM:
                problems.append(f"layers[{i}]: heads of {m.dim} and {m.vdim} channels: the kernels take up to {limits.MAX_HEAD_DIM}")
            if m.taps > limits.MAX_CONV_TAPS:
                problems.append(f"layers[{i}]: {m.taps} taps: the kernels take up to {limits.MAX_CONV_TAPS}")
            if m.rot is not None and (m.rot.dims % 2 or m.rot.dims > m.dim):
                problems.append(f"layers[{i}]: {m.rot.dims} turned channels in vectors of {m.dim}")
            if m.kv_from is not None:
                src = self.layers[m.kv_from] if m.kv_from < i else None
                if src is None or src.type != "attention" or src.mixer is None or src.mixer.kv_from is not None:
                    problems.append(f"layers[{i}]: kv_from {m.kv_from} is no earlier attention layer with keys and values of its own")
                elif (src.mixer.kv_heads, src.mixer.dim, src.mixer.vdim, src.mixer.rot) != (m.kv_heads, m.dim, m.vdim, m.rot):
                    problems.append(f"layers[{i}]: head sizes or rotation differ from layer {m.kv_from}, whose keys and values it uses")
        if problems:
            raise ConfigError(f"{where}: " + "; ".join(problems))

    def to_dict(self):
        return self.raw
