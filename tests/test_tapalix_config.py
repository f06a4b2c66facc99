"""The Tapalix configuration: what it reads, what it refuses, how it is laid out as parts."""

import copy

import pytest

import tapalix_models as tm
from from_scratch_inference_engine_b200.config import ConfigError, config_from_dict
from from_scratch_inference_engine_b200.parts.model import tensor_specs


def test_every_test_configuration_reads_and_round_trips():
    for name, data in tm.CONFIGS.items():
        config = config_from_dict(data)
        assert type(config).__name__ == "TapalixConfig"
        again = config_from_dict(config.to_dict())
        assert again == config, name


def test_run_order_repeats_the_looped_stretch_with_caches_of_its_own():
    spec = config_from_dict(tm.CONFIGS["loop"]).build_spec()
    assert [(c.layer, c.inlet) for c in spec.schedule] == \
        [(0, None), (1, 0), (2, None), (1, 0), (2, None), (3, None)]
    resolved = spec.resolved_schedule()
    assert [entry for _, entry, _ in resolved] == list(range(6))      # every call its own cache entry
    assert spec.embedding_scale == 4.0 and spec.logit_scale == 2.5 and spec.logit_softcap == 12.0
    assert len(spec.inlets) == 1
    first = config_from_dict(tm.CONFIGS["loop_first"]).build_spec()
    assert [(c.layer, c.inlet) for c in first.schedule] == [(0, 0), (1, None)]
    none = config_from_dict(tm.CONFIGS["gated"]).build_spec()
    assert none.inlets == () and all(c.inlet is None for c in none.schedule)


def test_tensor_names_and_shapes():
    specs = {s.name: tuple(s.shape) for s in tensor_specs(config_from_dict(tm.CONFIGS["loop"]).build_spec())}
    assert specs["embed"] == (131, 64) and specs["head"] == (131, 64)
    assert specs["loop.in"] == (64, 128)
    assert specs["final.norm"] == (64,) and specs["final.norm.b"] == (64,)
    assert specs["l0.norm1"] == (64,) and specs["l0.norm1.b"] == (64,)
    assert specs["l0.mix.q"] == (2 * (16 + 8), 64) and specs["l0.mix.dkv"] == (24 + 8, 64)
    assert specs["l0.mix.dkv.norm"] == (24,)
    assert specs["l0.mix.uk"] == (2 * 16, 24) and specs["l0.mix.uv"] == (2 * 12, 24)
    assert specs["l0.mix.o"] == (64, 2 * 12) and "l0.mix.g" not in specs
    assert specs["l1.mix.q"] == (4 * 8, 64) and specs["l1.mix.dkv"] == (40, 64)
    assert specs["l1.mix.g"] == (4 * 16, 64)
    assert specs["l1.mlp.e7.gate"] == (16, 64) and specs["l1.mlp.e7.down"] == (64, 16)
    assert specs["l1.mlp.router"] == (8, 64) and specs["l1.mlp.correction"] == (8,)
    assert specs["l1.mlp.shared.up"] == (48, 64)
    assert not any(name.startswith("l2.mlp") for name in specs)
    assert "l3.mlp.shared.gate" not in specs and "l3.mlp.e3.up" in specs
    assert not any("loop" in s.name for s in tensor_specs(config_from_dict(tm.CONFIGS["gated"]).build_spec()))


def test_cache_needs_follow_the_mixers():
    from from_scratch_inference_engine_b200.parts.model import DecoderModel
    model = DecoderModel(config_from_dict(tm.CONFIGS["loop"]).build_spec())
    needs = model.cache_needs()
    assert len(needs) == 6
    assert (needs[0].head_dim, needs[0].value_dim, needs[0].values_in_keys) == (32, 24, True)
    assert (needs[1].head_dim, needs[1].value_dim) == (40, 40)          # no turned part beside the latent
    assert needs[1] == needs[3] and needs[2] == needs[4]
    assert all(need.window == 0 for need in needs)
    assert all(state is None for state in model.state_needs())


@pytest.mark.parametrize("change,message", [
    (lambda d: d["layers"][0].__setitem__("type", "attention"), "not a mixer"),
    (lambda d: d["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda d: d["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "even"),
    (lambda d: d["layers"][0]["mixer"]["rot"].__setitem__("dims", 10), "at most"),
    (lambda d: d["layers"][0]["mixer"]["rot"]["scaling"].__setitem__("factor", 0), "positive"),
    (lambda d: d["layers"][1]["mlp"]["router"].__setitem__("top", 9), "exceeds"),
    (lambda d: d["layers"][1]["mlp"]["router"]["groups"].__setitem__("count", 3), "groups"),
    (lambda d: d["layers"][1]["mlp"]["router"]["groups"].__setitem__("keep", 3), "groups"),
    (lambda d: d["layers"][0]["mlp"]["router"].__setitem__("top", 5), "groups"),
    (lambda d: d["layers"][1]["mlp"].__setitem__("kind", "other"), "kind"),
    (lambda d: d["loop"].__setitem__("stop", 9), "loop"),
    (lambda d: d["loop"].__setitem__("start", 3), "loop"),
    (lambda d: d["loop"].__setitem__("times", 0), "times"),
    (lambda d: d.__setitem__("logit_softcap", -1.0), "logit_softcap"),
    (lambda d: d.pop("width"), "width"),
])
def test_what_cannot_run_is_refused_with_its_place(change, message):
    data = copy.deepcopy(tm.CONFIGS["loop"])
    change(data)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(data)


def test_stretched_frequency_table_against_the_plain_formula():
    import math
    import numpy as np
    import plain_tapalix as plain
    from from_scratch_inference_engine_b200.parts.rope import rotary_table, yarn_rotary_table
    for rot in ({"base": 50.0, "dims": 12, "scaling": tm.scaling(4.0, 24, 3.0, 1.0)},
                {"base": 1e4, "dims": 32, "scaling": tm.scaling(2.0, 256, 32.0, 1.0)},
                {"base": 100.0, "dims": 4, "scaling": tm.scaling(8.0, 16, 1.0, 0.5)}):
        s = rot["scaling"]
        table = yarn_rotary_table(rot["base"], rot["dims"], 40, s["factor"], s["original"], s["fast"], s["slow"])
        f, m = plain.turn_frequencies(rot)
        half = rot["dims"] // 2
        for p in (0, 1, 17, 39):
            for i in range(half):
                assert abs(table[p, i] - math.cos(p * f[i]) * m) < 1e-6
                assert abs(table[p, half + i] - math.sin(p * f[i]) * m) < 1e-6
        plain_f = [rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(half)]
        # fast pairs keep their frequency, slow ones are divided by the factor, none leaves that range
        assert all(pf / s["factor"] - 1e-12 <= g <= pf + 1e-12 for g, pf in zip(f, plain_f))
        assert m == pytest.approx(0.1 * math.log(s["factor"]) + 1.0)
    # the ramp of the first entry lies inside the pairs: some frequencies are kept, some stretched
    f, _ = plain.turn_frequencies({"base": 50.0, "dims": 12, "scaling": tm.scaling(4.0, 24, 3.0, 1.0)})
    plain_f = [50.0 ** (-2.0 * i / 12) for i in range(6)]
    assert f[0] == plain_f[0] and f[-1] == pytest.approx(plain_f[-1] / 4.0)
    assert np.allclose(rotary_table(50.0, 12, 8)[:, :6], np.cos(np.arange(8)[:, None] * np.asarray(plain_f)[None]))


def test_plain_router_masks_groups_with_minus_infinity_not_zero():
    import torch
    import plain_tapalix as plain
    # every choice score is negative: a masked group at 0 would win, at minus infinity it cannot
    z = torch.tensor([-2.0, -1.0, -3.0, -2.5, 0.5, 0.4], dtype=torch.float64)
    correction = torch.full((6,), -5.0, dtype=torch.float64)
    router = {"experts": 6, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 1}}
    chosen, weights = plain.route(z, correction, router)
    assert chosen == [4, 5]
    s = torch.sigmoid(z)
    assert weights[0] == pytest.approx(float(s[4] / (s[4] + s[5]) * 2.0))
    # a group's score is the sum of its two largest: group 0 (0.9 + 0.1) loses to group 1 (0.6 + 0.6)
    z = torch.logit(torch.tensor([0.9, 0.1, 0.6, 0.6], dtype=torch.float64))
    chosen, _ = plain.route(z, torch.zeros(4, dtype=torch.float64),
                            {"experts": 4, "top": 1, "groups": {"count": 2, "keep": 1}})
    assert chosen == [2]
