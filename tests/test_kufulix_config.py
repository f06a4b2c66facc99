"""The Kufulix configuration: what it reads, what it refuses, how it is laid out as parts; the plain
implementation's own consistency (no GPU)."""

import copy
import math

import numpy as np
import pytest
import torch

import kufulix_models as km
import plain_kufulix as plain
from from_scratch_inference_engine_b200.config import ConfigError, config_from_dict
from from_scratch_inference_engine_b200.parts.model import DecoderModel, tensor_specs


def test_every_test_configuration_reads_and_round_trips():
    for name, data in km.CONFIGS.items():
        config = config_from_dict(data)
        assert type(config).__name__ == "KufulixConfig"
        assert config_from_dict(config.to_dict()) == config, name


def test_layers_that_run_other_layers_tensors_are_calls_of_those_layers():
    spec = config_from_dict(km.CONFIGS["shared"]).build_spec()
    assert len(spec.layers) == 2 and [layer.prefix for layer in spec.layers] == ["l0.", "l1."]
    assert [c.layer for c in spec.schedule] == [0, 1, 0, 1, 0]
    assert [entry for _, entry, _ in spec.resolved_schedule()] == list(range(5))    # a cache entry per call
    model = DecoderModel(spec)
    needs, states = model.cache_needs(), model.state_needs()
    assert needs[0] == needs[2] == needs[4] and needs[1] == needs[3] and needs[0] != needs[1]
    assert (needs[0].kv_heads, needs[0].head_dim, needs[0].v_dim, needs[0].window) == (3, 16, 8, 21)
    assert (needs[1].kv_heads, needs[1].head_dim, needs[1].v_dim, needs[1].window) == (2, 8, 16, 13)
    # the matrices of four heads and the inputs of three earlier tokens, on a 32-byte border
    floats = 4 * 8 * 8 + 3 * (4 * 8 + 2 * 2 * 8)
    assert states[0].shape == (-(-floats // 8) * 8,) and states[1] is None and states[2] == states[0]
    assert spec.logit_softcap == 12.0 and spec.embedding_norm is not None


def test_tensor_names_and_shapes():
    specs = {s.name: tuple(s.shape) for s in tensor_specs(config_from_dict(km.CONFIGS["shared"]).build_spec())
             if not s.optional}
    assert specs["embed"] == (131, 64) and specs["head"] == (131, 64)
    assert specs["embed.norm"] == (64,) and specs["final.norm"] == (64,)
    assert specs["l0.norm1"] == (64,) and specs["l0.norm2"] == (64,)
    assert specs["l0.mix.left.q"] == (48, 64) and specs["l0.mix.left.q.b"] == (48,)
    assert specs["l0.mix.left.v"] == (24, 64) and specs["l0.mix.left.o"] == (64, 24)
    assert specs["l0.mix.left.q.norm"] == (16,) and specs["l0.mix.left.k.norm"] == (16,)
    assert specs["l0.mix.right.in"] == (2 * 32 + 2 * 2 * 8 + 4, 64)
    assert specs["l0.mix.right.conv"] == (32 + 32, 4) and specs["l0.mix.right.conv.b"] == (64,)
    assert specs["l0.mix.right.dt_bias"] == specs["l0.mix.right.A_log"] == specs["l0.mix.right.D"] == (4,)
    assert specs["l0.mix.right.norm"] == (32,) and specs["l0.mix.right.o"] == (64, 32)
    assert specs["l0.mlp.router"] == (8, 64) and specs["l0.mlp.correction"] == (8,)
    assert specs["l0.mlp.e5.up"] == (24, 64) and specs["l0.mlp.e5.down"] == (64, 24)
    assert "l0.mlp.e6.up" not in specs and "l0.mlp.e0.gate" not in specs      # identity experts have no tensors
    assert specs["l1.mix.g"] == (4, 64) and specs["l1.mix.k.b"] == (16,) and "l1.mix.q.norm" not in specs
    assert not any(name.startswith(("l2.", "l3.", "l4.")) for name in specs)
    bare = {s.name for s in tensor_specs(config_from_dict(km.CONFIGS["window"]).build_spec()) if not s.optional}
    assert not any(".mlp." in name or name.endswith("norm2") for name in bare)


def test_refusals_name_the_place():
    def refused(change, name="shared"):
        data = copy.deepcopy(km.CONFIGS[name])
        change(data)
        with pytest.raises(ConfigError) as info:
            config_from_dict(data)
        return str(info.value)

    assert "type" in refused(lambda d: d["layers"][1].update(type="mamba"))
    assert "kv_heads" in refused(lambda d: d["layers"][1]["mixer"].update(heads=3))
    assert "rot.dims" in refused(lambda d: d["layers"][1]["mixer"]["rot"].update(dims=10))
    assert "groups" in refused(lambda d: d["layers"][0]["mixer"]["right"].update(groups=3))
    assert "norm_groups" in refused(lambda d: d["layers"][0]["mixer"]["right"].update(norm_groups=5))
    assert "top" in refused(lambda d: d["layers"][1]["mlp"]["router"].update(top=7))
    assert "groups" in refused(lambda d: d["layers"][0]["mlp"]["router"]["groups"].update(count=3))
    assert "weights_of" in refused(lambda d: d["layers"][2].update(weights_of=2))
    assert "weights_of" in refused(lambda d: d["layers"][4].update(weights_of=2))     # names a layer without tensors
    assert "another layer" in refused(lambda d: d["layers"][2].update(weights_of=1))
    assert "left_scale" in refused(lambda d: d["layers"][0]["mixer"].update(left_scale="wide"))
    assert "mask" in refused(lambda d: d["layers"][1]["mixer"].update(mask=7))


def test_what_may_be_absent():
    data = copy.deepcopy(km.CONFIGS["window"])
    mixer = data["layers"][0]["mixer"]
    mixer.pop("left_scale")
    mixer["left"].pop("mask")
    mixer["left"].pop("rot")
    mixer["right"].pop("groups")
    mixer["right"].pop("norm_groups")
    data.pop("logit_softcap")
    spec = config_from_dict(data).build_spec()
    part = spec.layers[0].mixer
    assert part.params["left_scale"] == 1.0 and part.params["right_scale"] == 1.5
    left, right = part.params["left"].params, part.params["right"].params
    assert left["window"] == 0 and left["chunk"] == 0 and left["position"].kind == "none"
    assert right["groups"] == 1 and right["norm_groups"] == 1 and spec.logit_softcap == 0.0


def test_frequency_table_against_the_formula():
    from from_scratch_inference_engine_b200.parts.rope import llama3_rotary_table, rotary_table
    rot = {"base": 50.0, "dims": 8, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}}
    freqs = plain.turn_frequencies(rot)
    # the three branches all occur: kept, blended, divided by the factor
    plain_f = torch.tensor([50.0 ** (-2.0 * i / 8) for i in range(4)], dtype=torch.float64)
    ratio = (freqs / plain_f).tolist()
    assert ratio[0] == 1.0 and ratio[-1] == 0.25 and any(0.25 < r < 1.0 for r in ratio)
    table = llama3_rotary_table(50.0, 8, 40, 4.0, 32, 1.0, 4.0)
    angle = np.arange(40)[:, None] * freqs.numpy()[None, :]
    assert np.abs(table[:, :4] - np.cos(angle)).max() < 1e-6 and np.abs(table[:, 4:] - np.sin(angle)).max() < 1e-6
    assert np.array_equal(llama3_rotary_table(50.0, 8, 40, 1.0, 32, 1.0, 4.0), rotary_table(50.0, 8, 40))


def test_plain_masks_and_choice():
    w = plain.window_mask(7, 3)
    assert w[5].tolist() == [False, False, False, True, True, True, False]
    assert w[1].tolist() == [True, True, False, False, False, False, False]
    c = plain.chunk_mask(7, 3)
    assert c[5].tolist() == [False, False, False, True, True, True, False]
    assert c[3].tolist() == [False, False, False, True, False, False, False]
    assert c[2].tolist() == [True, True, True, False, False, False, False]
    # groups are masked with minus infinity, not zero: with negative choice values a masked expert
    # at zero would win; the group's score is its largest value, not a sum
    h = torch.eye(4, dtype=torch.float64)[:1]
    weights = {"r.router": torch.zeros(4, 4, dtype=torch.float64),
               "r.correction": torch.tensor([-1.0, -5.0, -3.0, -2.0], dtype=torch.float64)}
    ids, g = plain.route(h, weights, "r.", {"experts": 2, "identity": 2, "top": 2, "groups": {"count": 2, "keep": 1}})
    assert sorted(ids[0].tolist()) == [0, 1] and abs(float(g.sum()) - 1.0) < 1e-12
    ids, _ = plain.route(h, weights, "r.", {"experts": 2, "identity": 2, "top": 2})
    assert sorted(ids[0].tolist()) == [0, 3]


def test_plain_state_space_carries_its_state(tmp_path):
    """The plain recurrence over a whole sequence equals itself run in two halves when the state and
    the convolution's inputs are handed over - and differs when either is dropped: the mechanism
    has state, and the oracle shows it."""
    m = {"heads": 2, "vdim": 4, "state": 3, "groups": 1, "conv": 3, "norm_groups": 1}
    g = torch.Generator().manual_seed(0)
    inner, ch = 8, 8 + 6
    w = {"p.in": torch.randn(2 * inner + 6 + 2, 5, generator=g, dtype=torch.float64),
         "p.conv": torch.randn(ch, 3, generator=g, dtype=torch.float64), "p.conv.b": torch.zeros(ch, dtype=torch.float64),
         "p.dt_bias": torch.zeros(2, dtype=torch.float64), "p.A_log": torch.tensor([-3.0, 0.0], dtype=torch.float64),
         "p.D": torch.ones(2, dtype=torch.float64), "p.norm": torch.ones(inner, dtype=torch.float64),
         "p.o": torch.randn(5, inner, generator=g, dtype=torch.float64)}
    h = torch.randn(12, 5, generator=g, dtype=torch.float64)
    whole = plain.state_space(h, w, "p.", m, 1e-6)
    alone = plain.state_space(h[6:], w, "p.", m, 1e-6)
    assert float((whole[6:] - alone).abs().max()) > 1e-3
    assert torch.equal(whole[:6], plain.state_space(h[:6], w, "p.", m, 1e-6))
