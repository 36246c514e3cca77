"""Narasun's configuration, definition and cache layout without a device."""
import copy

import pytest

import tiny_narasun as tiny


def typed(config):
    from catena_models_b200.config.registry import config_from_dict
    return config_from_dict(config)


def test_reads_every_size_and_constant():
    arch, cfg = typed(tiny.TINY_Q)
    assert arch.name == "Narasun" and cfg.vocab == 130 and cfg.width == 48 and cfg.norm_eps == 1e-6 and cfg.loop is None
    a = cfg.layers[0].mixer.left
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.q_temp_coef, a.q_temp_every) == (3, 3, 24, 40, 0.2, 0.3, 5)
    assert cfg.layers[1].type == "parallel_2" and cfg.layers[1].kind == "parallel" and cfg.layers[1].mlp is None
    assert cfg.layers[0].mlp.kind == "moe" and (cfg.layers[0].mlp.experts, cfg.layers[0].mlp.top) == (3, 1)
    m = cfg.layers[2].mixer
    assert (m.heads, m.dim, m.vdim, m.gate_cap) == (1, 32, 16, 15.0)


def test_problems_are_collected_with_their_place():
    from catena_models_b200.config.base import ConfigError

    bad = copy.deepcopy(tiny.TINY_P)
    del bad["layers"][1]["mixer"]["left"]["scale"]
    bad["layers"][0]["mixer"]["gate_cap"] = "high"
    bad["layers"][2]["type"] = "convolution"
    with pytest.raises(ConfigError) as e:
        typed(bad)
    text = str(e.value)
    assert "layers[1].mixer.left" in text and "scale" in text and "gate_cap" in text and "convolution" in text
    bad = copy.deepcopy(tiny.TINY_P)
    bad["loop"]["stop"] = 9
    bad["layers"][0]["mlp"]["router"]["top"] = 6
    with pytest.raises(ConfigError) as e:
        typed(bad)
    assert "loop" in str(e.value) and "top 6 of 5" in str(e.value)


def test_run_order_and_plan():
    arch, cfg = typed(tiny.TINY_P)
    assert cfg.run_order() == [(0, 0), (1, None), (0, 1), (1, None), (2, None)]
    d = arch.define(cfg)
    kinds = [type(d.blocks[e.block]).__name__ for e in d.plan]
    assert kinds == ["LoopEntry", "ParallelBlock", "ParallelBlock", "LoopEntry", "ParallelBlock", "ParallelBlock", "ParallelBlock"]
    assert [e.block for e in d.plan if kinds[d.plan.index(e)] == "ParallelBlock"] == [0, 1, 0, 1, 2]
    assert len({e.state for e in d.plan}) == len(d.plan)                   # every run has a state of its own
    assert d.residual_float32 and d.keep_embedding
    _, flat = typed(tiny.TINY_Q)
    assert flat.run_order() == [(0, None), (1, None), (2, None)] and not arch.define(flat).keep_embedding


def test_rank_comes_from_the_tensors():
    from catena_models_b200.config.base import ConfigError

    config = copy.deepcopy(tiny.TINY_Q)
    for layer in config["layers"]:
        layer["mixer"].get("right", {}).pop("rank", None)
    arch, cfg = typed(config)
    with pytest.raises(ValueError):
        arch.define(cfg)
    with pytest.raises(ConfigError):
        cfg.with_tensor_shapes({})
    full = cfg.with_tensor_shapes({"l0.mix.right.w1": (4, 48), "l1.mix.right.w1": (16, 48)})
    assert [l.mixer.right.rank for l in full.layers[:2]] == [4, 16]
    names = {s.name: s.shape for s in arch.define(full).tensor_specs()}
    assert names["l1.mix.right.w2"] == (32, 16) and names["l0.mix.left.sink"] == (3,) and names["head"] == (130, 48)
    assert "loop.in" not in names and names["l0.mlp.e2.down"] == (48, 24) and "l1.mlp.gate" not in names


def test_state_specs_of_a_layer_with_two_mixers():
    from catena_models_b200.cache.spec import CompositeStateSpec, FixedStateSpec, KVStateSpec

    arch, cfg = typed(tiny.TINY_Q)
    specs = arch.define(cfg).state_specs()
    assert isinstance(specs[0], CompositeStateSpec)
    kv, fixed = specs[0].parts
    assert kv == KVStateSpec(3, 48, 0)                          # heads of 24 and 40 share a padded size of 48
    assert fixed == FixedStateSpec((48 + 3 * 8 * 8,), "float32")
    assert specs[2] == FixedStateSpec((1 * (32 * 16 + 32 + 1),), "float32")
    assert specs[0].length_class(300) == (512, 0)


def test_padded_heads_keep_the_product():
    """Heads of unequal sizes are padded with zero rows and columns: the projections' results do not change."""
    import torch
    from catena_models_b200.parts.linear import Linear

    w = torch.randn(3 * 5, 8)
    lin = Linear("w", 15, 8, head_rows=[(3, 5, 16)])
    lin.bind({"w": w}, None)
    assert lin.weight.shape == (48, 8) and lin.out_features == 48
    x = torch.randn(2, 8)
    y = (x @ lin.weight.T).view(2, 3, 16)
    assert torch.allclose(y[:, :, :5].reshape(2, 15), x @ w.T) and bool((y[:, :, 5:] == 0).all())
    o = torch.randn(8, 3 * 5)
    out = Linear("o", 8, 15, head_cols=(3, 5, 16))
    out.bind({"o": o}, None)
    assert torch.allclose(y.reshape(2, 48) @ out.weight.T, y[:, :, :5].reshape(2, 15) @ o.T, atol=1e-6)
