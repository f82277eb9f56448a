"""The Liverax design without a GPU: its configuration reader, its model description against the tensors a checkpoint
holds, its random-weights mode, the distance buckets and the expanded table of the product against the plain
model's, and the plain float64 model against sums written out (layer norm, rotation, masks, sinks, blending)."""
from __future__ import annotations

import copy
import math

import numpy as np
import pytest
import torch

import liverax_models as lm
import plain_liverax as plain
from celeg_b200.config import ConfigError, architecture_of
from celeg_b200.config.liverax import LiveraxConfig


def resolved(raw, seed):
    architecture = architecture_of(raw)
    tensors = lm.make_tensors(raw, seed)
    shapes = {name: tuple(value.shape) for name, value in tensors.items()}
    return architecture, architecture.resolve_config(architecture.parse_config(lm.for_disk(raw)), shapes), tensors


def test_configuration_round_trip_and_tensor_table():
    for name, (raw, seed) in lm.CONFIGS.items():
        architecture, config, tensors = resolved(raw, seed)
        assert architecture.name == "Liverax"
        assert LiveraxConfig.from_dict(config.to_dict()) == config
        spec = architecture.build_spec(config)
        wanted = {ref.name: tuple(ref.shape) for ref in spec.all_tensors()}
        made = {key: tuple(value.shape) for key, value in tensors.items()}
        assert wanted == made, name
        assert len(spec.order) == len(raw["layers"]) and all(entry.cache_of is None for entry in spec.order)


def test_every_constant_comes_from_the_configuration():
    raw, seed = lm.CONFIGS["mixed"]
    architecture, config, _ = resolved(raw, seed)
    first, second, third = config.layers[:3]
    assert (first.heads, first.kv_heads, first.dim, first.vdim, first.window) == (4, 2, 16, 16, 24)
    assert first.rotation.dims == 8 and first.rotation.divide_by == 4.0 and first.value_mix
    assert (second.rot_dim, second.kv_rank, second.q_rank, second.window) == (8, 40, 32, 20) and second.rotation.base == 5000.0
    assert third.scale == pytest.approx(0.3) and third.temperature == (0.5, 16) and third.distance_far == 48
    assert config.distance_buckets == (0, 0, 8, 0, 0, 12) and config.logit_softcap == 25.0
    spec = architecture.build_spec(config)
    assert spec.layers[0].mixer.params["value_mix"] == "first" and spec.layers[2].mixer.params["value_mix"] == "blend"
    assert spec.layers[0].mixer.parts["position"].params["linear_factor"] == 4.0
    assert spec.layers[1].mixer.kind == "latent_attention" and spec.layers[1].mixer.params["window"] == 20
    assert spec.layers[3].feed_forward is None and spec.layers[3].feed_forward_norm is None
    assert spec.layers[0].feed_forward.params["activation"] == "gelu_tanh" and spec.logit_softcap == 25.0
    assert spec.layers[0].mixer_norm.kind == "layernorm" and spec.final_norm.kind == "layernorm"


def test_what_the_configuration_leaves_out():
    raw, seed = lm.CONFIGS["odd"]
    architecture, config, _ = resolved(raw, seed)
    assert config.logit_softcap is None
    assert config.layers[3].window is None and config.layers[3].rotation.divide_by == 1.5 and not config.layers[3].value_mix
    assert config.layers[0].temperature is None and config.layers[4].window is None
    spec = architecture.build_spec(config)
    assert "temperature" not in spec.layers[0].mixer.params and spec.layers[0].mixer.params["value_mix"] == "first"
    assert "value_mix" not in spec.layers[3].mixer.params and "value_mix" not in spec.layers[3].mixer.tensors


def test_faulty_configurations_are_refused():
    raw = lm.for_disk(lm.CONFIGS["mixed"][0])
    for path, value in [(("layers", 0, "type"), "conv"), (("layers", 0, "mixer", "heads"), 3),
                        (("layers", 0, "mixer", "rot", "dims"), 7), (("layers", 0, "mixer", "rot", "dims"), 32),
                        (("layers", 1, "mixer", "rot", "dims"), 4), (("layers", 2, "mixer", "q_temp", "every"), 0),
                        (("layers", 0, "mlp", "kind"), "moe"), (("norm", "eps"), 0.0), (("logit_softcap",), -1.0),
                        (("layers", 3, "mixer", "vdim"), 8), (("layers", 0, "mixer", "mask", "size"), 0)]:
        broken = copy.deepcopy(raw)
        at = broken
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = value
        with pytest.raises(ConfigError):
            LiveraxConfig.from_dict(broken)
    config = LiveraxConfig.from_dict(raw)          # (no checkpoint read yet: the tables' rows are unknown)
    with pytest.raises(ConfigError):
        architecture_of(raw).build_spec(config)


def test_random_weights_mode(tmp_path):
    from celeg_b200.weights.random_init import write_random_model
    from celeg_b200.weights.safetensors_io import TensorRepository
    raw = lm.for_disk(lm.CONFIGS["odd"][0])
    raw["distance_buckets"] = [layer["buckets"] for layer in lm.CONFIGS["odd"][0]["layers"]]
    folder = write_random_model(str(tmp_path / "m"), raw, seed=3)
    repository = TensorRepository(folder)
    shapes = repository.shapes()
    repository.close()
    assert shapes["l0.mix.rel"] == (5, 3) and shapes["l0.mix.vmix"] == () and shapes["l2.mix.sink"] == (5,)
    assert shapes["l2.mix.uq"] == (5 * 10, 7) and shapes["l2.mix.dkv"] == (14, 36)


def test_distance_buckets_and_the_expanded_table():
    from celeg_b200.parts.mixers import distance_bias_table, distance_bucket
    # written out: eight buckets up to distance 64: 0..3 alone, then 4 * 16^(k/4) = 4, 8, 16, 32 open the next ones
    assert [plain.distance_bucket(n, 8, 64) for n in (0, 1, 3, 4, 7, 8, 15, 16, 31, 32, 63, 64, 1000)] == \
        [0, 1, 3, 4, 4, 5, 5, 6, 6, 7, 7, 7, 7]
    for buckets, far in [(8, 64), (5, 9), (12, 100), (32, 512), (4, 300), (6, 40)]:
        rows = [plain.distance_bucket(n, buckets, far) for n in range(far + 50)]
        assert rows == [distance_bucket(n, buckets, float(far)) for n in range(far + 50)]
        assert rows == sorted(rows) and rows[0] == 0 and rows[far] == buckets - 1 and set(rows[far:]) == {buckets - 1}
        table = torch.randn(buckets, 3)
        wide = distance_bias_table(table, far)
        assert wide.shape == (3, far + 1) and wide.dtype == torch.float32
        for n in (0, 1, buckets // 2, far // 2, far - 1, far):
            assert torch.equal(wide[:, n], table[rows[n]])


def test_layer_norm_rotation_and_query_factor_written_out():
    rng = np.random.default_rng(0)
    x = rng.normal(3.0, 2.0, size=(4, 10))
    w = rng.normal(1.0, 0.1, size=10)
    for row, got in zip(x, plain.layer_norm(x, w, 1e-3)):
        mean = sum(row) / 10
        var = sum((v - mean) ** 2 for v in row) / 10
        assert np.allclose(got, [(v - mean) / math.sqrt(var + 1e-3) * s for v, s in zip(row, w)])
    head = rng.normal(size=(1, 1, 6))
    turned = plain.rotate_halves(head, [5], 4, 100.0, 2.0)[0, 0]
    for i in range(2):
        angle = 5 * 100.0 ** (-2 * i / 4) / 2.0
        u, v = head[0, 0, i], head[0, 0, i + 2]
        assert np.allclose([turned[i], turned[i + 2]],
                           [u * math.cos(angle) - v * math.sin(angle), v * math.cos(angle) + u * math.sin(angle)])
    assert np.allclose(turned[4:], head[0, 0, 4:])
    assert plain.query_temperature(0, 0.5, 4) == 1.0 and plain.query_temperature(2, 0.5, 4) == 1.0
    assert plain.query_temperature(3, 0.5, 4) == pytest.approx(1 + 0.5 * math.log(2))
    assert plain.query_temperature(11, 0.5, 4) == pytest.approx(1 + 0.5 * math.log(4))


def test_window_sink_and_blending_written_out():
    scores = np.array([[0.0, 9.0, 9.0, 9.0], [1.0, 2.0, 9.0, 9.0], [3.0, 1.0, 0.5, 9.0], [2.0, 2.0, 2.0, 2.0]])
    weights = plain.masked_softmax_rows(scores, 2)
    assert np.allclose(weights[0], [1, 0, 0, 0]) and weights[2, 0] == 0.0 and weights[3, 1] == 0.0
    assert np.allclose(weights[2, 1:3], np.exp([1.0, 0.5]) / np.exp([1.0, 0.5]).sum())
    sunk = plain.masked_softmax_rows(scores, None, sink=1.5)
    assert np.allclose(sunk[1, :2], np.exp([1.0, 2.0]) / (np.exp([1.0, 2.0]).sum() + math.exp(1.5)))
    assert np.allclose(sunk[0, 0], 1.0 / (1.0 + math.exp(1.5)))
    v, first = np.ones((2, 1, 3)), np.full((2, 1, 3), 5.0)
    assert np.allclose(plain.blend_values(v, first, 0.25), 2.0) and plain.blend_values(v, None, 0.25) is v


def test_the_first_blended_layer_keeps_its_values_and_later_ones_use_them():
    """Zeroing the stored number of a later blended layer must change nothing but that layer; the first one's is
    never read."""
    raw, seed = lm.CONFIGS["mixed"]
    disk = lm.for_disk(raw)
    tensors = plain.as_float64(lm.make_tensors(raw, seed))
    tokens = list(np.random.default_rng(1).integers(0, raw["vocab"], 30))
    base = plain.forward(disk, tensors, tokens)
    changed = dict(tensors)
    changed["l0.mix.vmix"] = np.float64(0.9)
    assert np.array_equal(plain.forward(disk, changed, tokens), base)
    changed["l2.mix.vmix"] = np.float64(0.0)
    assert np.abs(plain.forward(disk, changed, tokens) - base).max() > 1e-3
