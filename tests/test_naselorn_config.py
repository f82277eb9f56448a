"""The Naselorn design without a GPU: its configuration reader, its model description against the tensors a
checkpoint holds, its random-weights mode, and the plain float64 model against itself (each recurrence against its
sum over the past, the chunked mask against a mask written out, the router against a hand-made case)."""
from __future__ import annotations

import copy
import json
import math
import os

import numpy as np
import pytest

import naselorn_models as nm
import plain_naselorn as plain
from celeg_b200.config import ConfigError, architecture_of
from celeg_b200.config.naselorn import NaselornConfig


def test_configuration_round_trip_and_tensor_table():
    for name, (raw, seed) in nm.CONFIGS.items():
        architecture = architecture_of(raw)
        assert architecture.name == "Naselorn"
        config = architecture.parse_config(raw)
        again = NaselornConfig.from_dict(config.to_dict())
        assert again == config
        spec = architecture.build_spec(config)
        wanted = {ref.name: tuple(ref.shape) for ref in spec.all_tensors()}
        made = {key: tuple(value.shape) for key, value in nm.make_tensors(raw, seed).items()}
        assert wanted == made, name
        assert len(spec.order) == len(raw["layers"]) and all(entry.cache_of is None for entry in spec.order)


def test_every_constant_comes_from_the_configuration():
    raw, _ = nm.CONFIGS["mixed"]
    config = architecture_of(raw).parse_config(raw)
    first, third = config.layers[0], config.layers[2]
    assert (first.left.heads, first.left.kv_heads, first.left.dim, first.left.vdim, first.left.chunk) == (4, 2, 16, 32, 16)
    assert first.left.scale == pytest.approx(0.25) and (first.left_scale, first.right_scale) == (1.25, 0.75)
    assert (first.right.width, first.right.blocks, first.right.taps) == (48, 3, 4)
    assert third.left.scale == pytest.approx(0.3) and third.left.chunk == 40
    assert config.layers[1].decay == (0.9, 0.99) and config.embedding_scale == pytest.approx(8.0)
    assert config.layers[0].mlp.top == 3 and config.layers[0].mlp.shared_ff == 48 and config.layers[3].mlp.shared_ff is None
    spec = architecture_of(raw).build_spec(config)
    mixer = spec.layers[0].mixer
    assert mixer.kind == "side_by_side" and mixer.parts["left"].params["chunk"] == 16
    assert mixer.parts["right"].params["gate_factor"] == 8.0
    assert spec.layers[1].feed_forward.params["activation"] == "relu"
    assert spec.layers[0].feed_forward.params["activation"] == "silu"


def test_absent_mask_shows_every_earlier_key_and_absent_feed_forward_is_none():
    raw, _ = nm.CONFIGS["odd"]
    config = architecture_of(raw).parse_config(raw)
    assert config.layers[2].left.chunk is None and config.layers[0].left.chunk == 7
    assert config.layers[1].mlp is None
    spec = architecture_of(raw).build_spec(config)
    assert spec.layers[1].feed_forward is None and spec.layers[1].feed_forward_norm is None


@pytest.mark.parametrize("damage,message", [
    (lambda raw: raw["layers"][0].update(type="sliding"), "unknown layer type"),
    (lambda raw: raw["layers"][0]["mixer"].pop("left"), "left"),
    (lambda raw: raw["layers"][0]["mixer"]["left"].update(kv_heads=3), "multiple"),
    (lambda raw: raw["layers"][0]["mixer"]["right"].update(blocks=5), "multiple"),
    (lambda raw: raw["layers"][0]["mixer"]["right"].update(conv=40), "taps"),
    (lambda raw: raw["layers"][0]["mixer"]["left"]["mask"].update(size=0), "size"),
    (lambda raw: raw["layers"][1]["mixer"].update(decay=[0.5]), "decay"),
    (lambda raw: raw["layers"][1]["mlp"]["router"].update(top=9), "exceeds"),
    (lambda raw: raw["layers"][1]["mlp"].update(kind="sparse"), "unknown kind"),
    (lambda raw: raw.pop("norm"), "norm"),
    (lambda raw: raw.update(layers=[]), "layers"),
])
def test_faulty_configurations_are_refused_with_a_message(damage, message):
    raw = nm.config(64, 32, [nm.with_mlp(nm.parallel(4, 2, 8, 8, 12, 24, 2, 3), nm.dense(48)),
                             nm.with_mlp(nm.lightning(2, 8, 8), nm.moe(8, 2, 16, shared=8))])
    damage(raw)
    with pytest.raises(ConfigError, match=message):
        architecture_of(raw).parse_config(raw)


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    from celeg_b200 import write_random_model
    from celeg_b200.weights.safetensors_io import TensorRepository
    raw, _ = nm.CONFIGS["mixed"]
    folder = write_random_model(str(tmp_path / "random"), raw, seed=3)
    repository = TensorRepository(folder)
    shapes = repository.shapes()
    architecture = architecture_of(raw)
    wanted = {ref.name: tuple(ref.shape) for ref in architecture.build_spec(architecture.parse_config(raw)).all_tensors()}
    assert {key: tuple(value) for key, value in shapes.items()} == wanted
    stored = repository.tensor("l0.norm1").float()
    assert abs(float(stored.mean())) < 0.2                  # the blocks' norm weights lie around zero
    plain_weight = repository.tensor("l1.mix.norm").float()
    assert 0.5 < float(plain_weight.mean()) < 1.5           # the lightning mixer's lies around one
    repository.close()
    assert json.load(open(os.path.join(folder, "config.json")))["architecture"] == "Naselorn"


def test_plain_sinusoid_interleaves_sine_and_cosine():
    table = plain.sinusoid([0, 1, 7], 6)
    assert np.allclose(table[0], [0, 1, 0, 1, 0, 1])
    for i in range(3):
        angle = 7 * 10000.0 ** (-2.0 * i / 6)
        assert table[2, 2 * i] == pytest.approx(math.sin(angle)) and table[2, 2 * i + 1] == pytest.approx(math.cos(angle))
    assert plain.sinusoid([3], 5).shape == (1, 5)           # an odd width ends on a sine


def test_plain_lightning_equals_its_sum_over_the_past():
    raw = nm.single_layer(nm.lightning(2, 4, 3, [0.5, 0.9]))
    tensors = plain.as_float64(nm.make_tensors(raw, 7))
    h = np.random.default_rng(1).normal(size=(9, raw["width"]))
    want = plain.lightning(tensors, "l0.mix.", raw["layers"][0]["mixer"], h, 1e-5)
    q = plain.silu(h @ tensors["l0.mix.q"].T).reshape(9, 2, 4)
    k = plain.silu(h @ tensors["l0.mix.k"].T).reshape(9, 2, 4)
    v = plain.silu(h @ tensors["l0.mix.v"].T).reshape(9, 2, 3)
    read = np.zeros((9, 2, 3))
    for head, decay in enumerate((0.5, 0.9)):
        for t in range(9):
            for s in range(t + 1):
                read[t, head] += decay ** (t - s) * (q[t, head] @ k[s, head]) * v[s, head]
    read = read.reshape(9, 6)
    read = read / np.sqrt((read ** 2).mean(-1, keepdims=True) + 1e-5) * tensors["l0.mix.norm"]     # one norm over both heads
    assert np.allclose((read * plain.sigmoid(h @ tensors["l0.mix.g"].T)) @ tensors["l0.mix.o"].T, want, rtol=1e-10, atol=1e-12)


def test_plain_chunked_attention_equals_a_mask_written_out():
    raw = nm.single_layer(nm.parallel(4, 2, 6, 5, 4, 8, 2, 2, scale=0.7))
    tensors = plain.as_float64(nm.make_tensors(raw, 8))
    mixer = raw["layers"][0]["mixer"]["left"]
    h = np.random.default_rng(2).normal(size=(11, raw["width"]))
    want = plain.chunked_attention(tensors, "l0.mix.left.", mixer, h)
    q = (h @ tensors["l0.mix.left.q"].T + tensors["l0.mix.left.q.b"]).reshape(11, 4, 6)
    k = (h @ tensors["l0.mix.left.k"].T + tensors["l0.mix.left.k.b"]).reshape(11, 2, 6)
    v = (h @ tensors["l0.mix.left.v"].T + tensors["l0.mix.left.v.b"]).reshape(11, 2, 5)
    i, j = np.arange(11)[:, None], np.arange(11)[None, :]
    visible = (j <= i) & (i // 4 == j // 4)
    assert visible[4].sum() == 1 and visible[7].sum() == 4 and visible[10].sum() == 3
    out = np.zeros((11, 4, 5))
    for head in range(4):
        scores = np.where(visible, (q[:, head] @ k[:, head // 2].T) * 0.7, -np.inf)
        p = np.exp(scores - scores.max(-1, keepdims=True))
        out[:, head] = (p / p.sum(-1, keepdims=True)) @ v[:, head // 2]
    assert np.allclose(out.reshape(11, -1) @ tensors["l0.mix.left.o"].T + tensors["l0.mix.left.o.b"], want, rtol=1e-10, atol=1e-12)


def test_plain_recurrent_unit_equals_its_sum_over_the_past_and_starts_from_zero():
    raw = nm.single_layer(nm.parallel(1, 1, 4, 4, None, 6, 2, 3))
    tensors = plain.as_float64(nm.make_tensors(raw, 9))
    base = "l0.mix.right."
    h = np.random.default_rng(3).normal(size=(8, raw["width"]))
    want = plain.gated_recurrent_unit(tensors, base, raw["layers"][0]["mixer"]["right"], h)
    x = h @ tensors[base + "x"].T + tensors[base + "x.b"]
    padded = np.concatenate([np.zeros((2, 6)), x])
    u = sum(tensors[base + "conv"][:, j] * padded[j:j + 8] for j in range(3)) + tensors[base + "conv.b"]
    assert np.allclose(u, plain.causal_conv(x, tensors[base + "conv"], tensors[base + "conv.b"]))
    r, i = np.zeros_like(u), np.zeros_like(u)
    for b in range(2):
        cut = slice(3 * b, 3 * b + 3)
        r[:, cut] = plain.sigmoid(u[:, cut] @ tensors[base + "ra"][b].T + tensors[base + "ra.b"][b])
        i[:, cut] = plain.sigmoid(u[:, cut] @ tensors[base + "ri"][b].T + tensors[base + "ri.b"][b])
    a = np.exp(-8.0 * r * np.log1p(np.exp(tensors[base + "lam"])))
    fed = np.sqrt(1.0 - a ** 2) * i * u
    states = np.zeros_like(u)
    for t in range(8):
        for s in range(t + 1):
            states[t] += np.prod(a[s + 1:t + 1], axis=0) * fed[s]
    assert np.allclose(states[0], fed[0])                 # the first token is fed like every other
    y = plain.gelu_tanh(h @ tensors[base + "y"].T + tensors[base + "y.b"])
    assert np.allclose((states * y) @ tensors[base + "o"].T, want, rtol=1e-10, atol=1e-12)


def test_plain_router_chooses_the_largest_logits_and_weighs_by_their_softmax():
    raw = nm.single_layer(nm.lightning(1, 8, 8), nm.moe(4, 2, 8))
    tensors = plain.as_float64(nm.make_tensors(raw, 6))
    tensors["l0.mlp.router"] = np.zeros((4, raw["width"]))
    tensors["l0.mlp.router"][:, 0] = [3.0, 2.0, 1.0, 0.0]
    tensors["l0.mlp.router.b"] = np.array([0.0, 0.0, 0.0, 4.5])      # the bias lifts the last expert over all others
    h = np.zeros((1, raw["width"]))
    h[0, 0] = 1.0
    chosen, weights = plain.route(tensors, "l0.mlp.", raw["layers"][0]["mlp"], h)
    assert chosen.tolist() == [[3, 0]]
    e = np.exp([4.5, 3.0])
    assert np.allclose(weights[0], e / e.sum())


def test_plain_side_by_side_is_the_weighted_sum_of_its_halves():
    raw = nm.single_layer(nm.parallel(2, 1, 4, 6, 5, 8, 2, 2, left_scale=0.25, right_scale=-2.0))
    tensors = plain.as_float64(nm.make_tensors(raw, 10))
    mixer = copy.deepcopy(raw["layers"][0]["mixer"])
    h = np.random.default_rng(4).normal(size=(7, raw["width"]))
    left = plain.chunked_attention(tensors, "l0.mix.left.", mixer["left"], h)
    right = plain.gated_recurrent_unit(tensors, "l0.mix.right.", mixer["right"], h)
    assert np.allclose(plain.side_by_side(tensors, "l0.mix.", mixer, h), 0.25 * left - 2.0 * right)
