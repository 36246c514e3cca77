"""The Fozedra configuration reader and definition (no device needed)."""
import copy

import pytest

import tiny_fozedra as tiny
from catena_models_b200.cache.spec import CompositeStateSpec, FixedStateSpec, KVStateSpec
from catena_models_b200.config.base import ConfigError
from catena_models_b200.config.registry import config_from_dict


def test_reads_every_size_and_constant():
    arch, cfg = config_from_dict(tiny.TINY_B)
    assert arch.name == "Fozedra" and cfg.vocab == 77 and cfg.width == 36 and cfg.residual_mult == 1.0
    light, att = cfg.layers[0], cfg.layers[1]
    assert light.type == "lightning" and light.mixer.decay == (0.93,) and light.ff == 0
    m = att.mixer
    assert (m.heads, m.kv_heads, m.dim, m.vdim, m.taps, m.window, m.keep_first) == (3, 1, 12, 20, 5, 70, 0)
    assert (m.rot.dims, m.rot.base, m.rot.factor, m.rot.original, m.rot.fast, m.rot.slow) == (6, 500.0, 2.0, 32, 8.0, 2.0)
    assert att.ff == 28 and m.kv_from is None


def test_plan_lends_the_owner_state_to_a_reader():
    arch, cfg = config_from_dict(tiny.TINY_A)
    d = arch.define(cfg)
    assert [e.reads for e in d.plan] == [(), (0,), (), (0,)]
    specs = d.state_specs()
    assert isinstance(specs[0], CompositeStateSpec) and isinstance(specs[0].parts[0], KVStateSpec)
    assert specs[0].parts[0] == KVStateSpec(2, 32, 0)                  # a key row of 2 x 16, a value row of 8: entries of 32
    assert specs[0].parts[1] == FixedStateSpec((4 * (4 * 32 + 2 * 32 + 2 * 8),), "float32")   # a ring of four rows
    assert specs[1] == FixedStateSpec((4 * 4 * 32,), "float32")         # a reader filters its queries only
    names = {s.name for s in d.tensor_specs()}
    assert "l1.mix.q.conv" in names and "l1.mix.k" not in names and "l1.mix.v.b" not in names
    assert "l0.mix.k.conv" in names and "l2.mix.norm" in names and "final.norm.alpha" in names
    assert "l1.norm2" not in names and "l0.norm2.b" in names


@pytest.mark.parametrize("change, words", [
    (lambda c: c["layers"][1]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][1]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][1]["mixer"].update(dim=8), "differ"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "turned"),
    (lambda c: c["layers"][0]["mixer"].update(conv=40), "taps"),
    (lambda c: c["layers"][2]["mixer"].update(decay=[0.5]), "decays"),
    (lambda c: c["layers"][2].update(type="other"), "known mixers"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "mlp.kind"),
    (lambda c: c.pop("width"), "width"),
])
def test_refuses_what_cannot_run(change, words):
    cfg = copy.deepcopy(tiny.TINY_A)
    change(cfg)
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg)
    assert words in str(e.value)


def test_yarn_rates_against_the_plain_statement():
    import plain_fozedra as plain
    from catena_models_b200.parts import build_part

    for dims, base, factor, original, fast, slow in ((20, 40000.0, 6.0, 512, 24.0, 1.5), (6, 500.0, 2.0, 32, 8.0, 2.0),
                                                     (16, 10000.0, 4.0, 64, 16.0, 1.0)):
        part = build_part("position", "partial_yarn_rotary", dims=dims, theta=base, factor=factor, original=original,
                          fast=fast, slow=slow)
        rates, mag = plain.yarn_rates(dims, base, factor, original, fast, slow)
        assert part.rates == pytest.approx(rates, rel=1e-12) and part.magnitude == pytest.approx(mag, rel=1e-12)
        assert len({round(r / f, 6) for r, f in zip(part.rates, [base ** (-2.0 * i / dims) for i in range(dims // 2)])}) > 1
