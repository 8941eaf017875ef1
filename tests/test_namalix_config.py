"""Namalix's configuration, description and cache needs, and the plain implementation's mechanisms against facts that can be
worked out by hand, all without a GPU."""

import copy
import math

import numpy as np
import pytest
import torch

import plain_namalix as pn
from namalix_cases import CONFIGS, tensor_shapes

F64 = torch.float64


def _model(cfg):
    from rusty_llama_b200.models.model import Model
    from rusty_llama_b200.parts.base import Runtime
    from rusty_llama_b200.registry import describe_model

    return Model(describe_model(cfg), Runtime.create("cpu", torch.float32))


@pytest.mark.parametrize("name", list(CONFIGS))
def test_the_described_model_asks_for_the_checkpoints_tensors(name):
    cfg = CONFIGS[name]()
    want = tensor_shapes(cfg)
    got = {k: tuple(v.shape) for k, v in _model(cfg).param_infos().items()}
    assert set(got) == set(want)
    for k, shape in want.items():
        assert got[k] == tuple(shape), (k, got[k], shape)


def test_cache_needs_follow_the_layers():
    from rusty_llama_b200.cache import Cache
    from rusty_llama_b200.parts.base import KVNeed, StateNeed

    model = _model(CONFIGS["a"]())
    needs = dict(model.cache_needs())
    assert needs[0] == StateNeed((3, 24, 40), torch.float32)
    assert needs[1] == KVNeed(2, 20, 0, value_dim=12)
    assert needs[2] == (StateNeed((4, 24, 20), torch.float32), StateNeed((2, 2 * 2 * 24 + 4 * 20), torch.float32))
    assert needs[3] == KVNeed(2, 16, 0, value_dim=12)
    assert needs[4] == KVNeed(2, 8, 0)
    needs_b = dict(_model(CONFIGS["b"]()).cache_needs())
    assert needs_b[3] == StateNeed((2, 36, 36), torch.float32)  # a convolution of one tap keeps no inputs
    cache = Cache(model.cache_needs(), 64 * 4, 2, torch.float32, "cpu")
    s = cache.open_sequence()
    cache.view(0).state[s] += 1.0
    cache.view(2)[1].state[s] += 1.0
    cache.reserve([s], [100])
    cache.commit([s], [100])
    cache.check_consistent()
    cache.close_sequence(s)
    assert cache.open_sequence() == s  # the slot is used again, and its records read zero
    assert float(cache.view(0).state[s].abs().sum()) == 0.0 and float(cache.view(2)[1].state[s].abs().sum()) == 0.0


def test_value_mixing_roles_follow_the_order_of_the_layers():
    """The first layer that mixes values is the source, whichever place it has; a layer that does not say so takes no part."""
    from rusty_llama_b200.registry import describe_model

    spec = describe_model(CONFIGS["a"]())
    roles = [layer.mixer.params.get("value_mix") for layer in spec.layers]
    assert roles[0] is None and roles[2] is None and roles[4] is None
    assert roles[1]["role"] == "source" and roles[3]["role"] == "mix" and roles[1]["key"] == roles[3]["key"]
    assert spec.layers[0].block == "shared_norm" and set(spec.layers[0].norms) == {"mixer"}
    assert spec.embedding.params["scale"] == 3.0


def test_configuration_errors_are_named():
    from rusty_llama_b200.errors import ConfigError
    from rusty_llama_b200.registry import describe_model

    def broken(change):
        cfg = copy.deepcopy(CONFIGS["a"]())
        change(cfg)
        with pytest.raises(ConfigError):
            describe_model(cfg)

    broken(lambda c: c["layers"][0].update(type="lightning"))
    broken(lambda c: c["layers"][0]["mixer"].update(decay=[0.5]))
    broken(lambda c: c["layers"][1]["mixer"].update(kv_heads=4))
    broken(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=22))
    broken(lambda c: c["layers"][3]["mixer"].update(vdim=16))  # value mixing between unequal value rows
    broken(lambda c: c["layers"][1]["mlp"]["router"].update(top=6))
    broken(lambda c: c["layers"][0]["mlp"].update(kind="glu"))
    broken(lambda c: c["layers"][2]["mixer"].update(kv_heads=3))
    broken(lambda c: c.pop("width"))


def test_rescaled_frequencies_agree_with_the_librarys_table():
    from rusty_llama_b200.config.rope_scaling import RopeScaling, inverse_frequencies, magnitude

    for base, dims, sc in ((10000.0, 8, {"factor": 2.0, "original": 48, "fast": 4.0, "slow": 0.5}), (10000.0, 32, {"factor": 8.0, "original": 256, "fast": 16.0, "slow": 2.0}),
                           (500.0, 64, {"factor": 4.0, "original": 1000, "fast": 32.0, "slow": 1.0})):
        f, mag = pn.yarn_frequencies(base, dims, sc)
        lib = RopeScaling(kind="yarn", factor=sc["factor"], original_max_position_embeddings=sc["original"], beta_fast=sc["fast"], beta_slow=sc["slow"])
        assert np.allclose(inverse_frequencies(dims, base, lib), f.numpy(), rtol=1e-6)
        assert abs(magnitude(lib) - mag) < 1e-12
        plain = pn.plain_frequencies(base, dims)
        assert float(f[0]) == pytest.approx(float(plain[0]))  # the fastest pair keeps its frequency
        assert float(f[-1]) == pytest.approx(float(plain[-1]) / sc["factor"])  # the slowest is slowed by the factor


def test_rotation_pairs_and_positions():
    x = torch.arange(1.0, 9.0, dtype=F64).view(1, 1, 8).repeat(3, 1, 1)
    pos = torch.tensor([0, 1, 5])
    f = torch.tensor([0.5, 0.25], dtype=F64)
    near = pn.rotate(x, pos, f, 4, True)
    half = pn.rotate(x, pos, f, 4, False)
    assert torch.equal(near[0], x[0]) and torch.equal(half[0], x[0])  # position 0 turns nothing
    assert torch.equal(near[..., 4:], x[..., 4:])  # the rest of a head passes unchanged
    c, s = math.cos(5 * 0.5), math.sin(5 * 0.5)
    assert near[2, 0, 0].item() == pytest.approx(1 * c - 2 * s) and near[2, 0, 1].item() == pytest.approx(2 * c + 1 * s)
    assert half[2, 0, 0].item() == pytest.approx(1 * c - 3 * s) and half[2, 0, 2].item() == pytest.approx(3 * c + 1 * s)
    # a rotation keeps the product of a query and a key a function of their distance
    q, k = torch.randn(1, 1, 8, dtype=F64), torch.randn(1, 1, 8, dtype=F64)
    for pair in (True, False):
        d1 = (pn.rotate(q, torch.tensor([7]), f, 4, pair) * pn.rotate(k, torch.tensor([3]), f, 4, pair)).sum()
        d2 = (pn.rotate(q, torch.tensor([14]), f, 4, pair) * pn.rotate(k, torch.tensor([10]), f, 4, pair)).sum()
        assert d1.item() == pytest.approx(d2.item())


def test_logistic_weights_are_not_normalised_and_are_mixed_after_the_logistic_function():
    T, H = 4, 2
    q = torch.zeros(T, H, 3, dtype=F64)
    k = torch.zeros(T, 1, 3, dtype=F64)
    pb = torch.tensor([0.0, math.log(3.0)], dtype=F64)  # weights 1/2 and 3/4 for every visible key
    w = pn.attention_weights(q, k, {"scale": 1.0, "softcap": 5.0}, pb, torch.eye(H, dtype=F64))
    assert torch.allclose(w[0], torch.tril(torch.full((T, T), 0.5, dtype=F64)))
    assert torch.allclose(w[1], torch.tril(torch.full((T, T), 0.75, dtype=F64)))
    talk = torch.tensor([[1.0, -2.0], [0.5, 0.0]], dtype=F64)
    w = pn.attention_weights(q, k, {"scale": 1.0, "softcap": 5.0}, pb, talk)
    assert torch.allclose(w[0], torch.tril(torch.full((T, T), 0.5 - 1.5, dtype=F64)))
    assert torch.allclose(w[1], torch.tril(torch.full((T, T), 0.25, dtype=F64)))
    # a cap bounds the score before the bias is added
    q[3, 0, 0], k[1, 0, 0] = 100.0, 100.0
    w = pn.attention_weights(q, k, {"scale": 1.0, "softcap": 2.0}, torch.zeros(H, dtype=F64), torch.eye(H, dtype=F64))
    assert w[0, 3, 1].item() == pytest.approx(1 / (1 + math.exp(-2.0 * math.tanh(5000.0))))


def test_short_convolution_sees_the_past_only():
    x = torch.tensor([[1.0], [10.0], [100.0], [1000.0]], dtype=F64)
    w = torch.tensor([[3.0, 2.0, 1.0]], dtype=F64)  # the last column is the current token's
    assert pn.short_convolution(x, w)[:, 0].tolist() == [1.0, 12.0, 123.0, 1230.0]


def test_delta_rule_overwrites_what_a_key_held():
    """With beta = 1 and no decay a key gives back the last value written under it, whatever was there before, and a key at
    right angles to it is left alone."""
    e = torch.eye(4, dtype=F64)
    k = torch.stack([e[0], e[1], e[0], e[1]])[:, None, :]
    v = torch.tensor([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0], [0.0, 0.0]], dtype=F64)[:, None, :]
    q = torch.stack([e[0], e[0], e[0], e[0]])[:, None, :]
    one = torch.ones(4, 1, dtype=F64)
    o = pn.delta_recurrence(q, k, v, one, one)[:, 0]
    assert o.tolist() == [[1.0, 2.0], [1.0, 2.0], [5.0, 6.0], [5.0, 6.0]]
    o = pn.delta_recurrence(q, k, v, 0.5 * one, one)[:, 0]  # half-way toward the new value
    assert o[2].tolist() == [0.5 * 0.5 + 0.5 * 5.0, 0.5 * 1.0 + 0.5 * 6.0]
    o = pn.delta_recurrence(q, k, v, one, 0.5 * one)[:, 0]  # the state halves before every token
    assert o[1].tolist() == [0.5, 1.0]


def test_retention_is_a_decayed_sum():
    q = torch.ones(3, 1, 1, dtype=F64)
    k = torch.ones(3, 1, 1, dtype=F64)
    v = torch.tensor([1.0, 10.0, 100.0], dtype=F64).view(3, 1, 1)
    o = pn.retention_recurrence(q, k, v, torch.tensor([0.5], dtype=F64))
    assert o.view(3).tolist() == [1.0, 10.5, 105.25]


def test_router_choice_and_weights():
    h = torch.eye(3, dtype=F64)
    W = {"r.router": torch.tensor([[0.0, 2.0, -2.0], [1.0, 0.0, 0.0], [-1.0, 0.0, 3.0]], dtype=F64), "r.correction": torch.tensor([0.0, 0.0, 0.6], dtype=F64)}
    chosen, w = pn.route(h, W, "r.", {"top": 2, "scale": 1.5})
    s = pn.logistic(h @ W["r.router"].T)
    # token 0: scores .5, .73, .27; the correction lifts expert 2 to .87: it is chosen, but weighted by its own .27
    assert sorted(chosen[0].tolist()) == [1, 2]
    pick = {e: x for e, x in zip(chosen[0].tolist(), w[0].tolist())}
    assert pick[2] == pytest.approx(1.5 * s[0, 2].item() / (s[0, 1].item() + s[0, 2].item()))
    assert w.sum(dim=1).tolist() == pytest.approx([1.5, 1.5, 1.5])


def test_gelu_and_the_experts_gate():
    z = torch.tensor([-3.0, -0.5, 0.0, 0.5, 3.0], dtype=F64)
    exact = 0.5 * z * (1 + torch.erf(z / math.sqrt(2)))
    assert torch.allclose(pn.gelu_tanh(z), exact, atol=2e-3)
    W = {"e.gate": torch.tensor([[5.0]], dtype=F64), "e.up": torch.tensor([[-5.0]], dtype=F64), "e.down": torch.tensor([[1.0]], dtype=F64)}
    y = pn.expert_ff(torch.tensor([[1.0]], dtype=F64), W, "e.", 2.0)  # gate capped at 2, up clamped to -2
    assert y.item() == pytest.approx(2.0 * (1 / (1 + math.exp(-1.702 * 2.0))) * (-2.0 + 1.0))


def test_the_plain_model_runs_every_configuration():
    from namalix_cases import as_float64, random_weights

    for i, (name, make) in enumerate(CONFIGS.items()):
        cfg = make()
        w = as_float64(random_weights(cfg, seed=5 + i))
        toks = np.random.default_rng(i).integers(0, cfg["vocab"], 40).tolist()
        logits, after = pn.plain_streams(cfg, w, toks)
        assert logits.shape == (40, cfg["vocab"]) and after.shape == (len(cfg["layers"]), 40, cfg["width"])
        assert torch.isfinite(logits).all()
        # causal: the first 25 positions do not change when the rest is replaced
        other = toks[:25] + np.random.default_rng(99).integers(0, cfg["vocab"], 15).tolist()
        assert torch.equal(pn.plain_logits(cfg, w, other)[:25], logits[:25])
