"""Tefavik's configuration, description, run order and cache needs, without a GPU."""

import copy

import pytest
import torch

import plain_tefavik as pt
from tefavik_cases import CONFIGS, DECAY_RANK, tensor_shapes


def _model(cfg):
    from rusty_llama_b200.models.model import Model
    from rusty_llama_b200.parts.base import Runtime
    from rusty_llama_b200.registry import describe_model

    return Model(describe_model(cfg), Runtime.create("cpu", torch.float32))


@pytest.mark.parametrize("name", list(CONFIGS))
def test_the_described_model_asks_for_the_checkpoints_tensors(name):
    """Every tensor of the checkpoint and no other; the inner size of the decay's matrices is left to the checkpoint (-1)."""
    cfg = CONFIGS[name]()
    rank = DECAY_RANK[name]
    want = tensor_shapes(cfg, rank)
    got = {k: tuple(v.shape) for k, v in _model(cfg).param_infos().items()}
    assert set(got) == set(want)
    for k, shape in want.items():
        assert len(got[k]) == len(shape) and all(g in (w, -1) for g, w in zip(got[k], shape)), (k, got[k], shape)
        if -1 in got[k]:
            assert k.endswith(".a1") or k.endswith(".a2")


def test_every_layer_run_gets_storage_of_its_own():
    """A looped layer has one cache or state per pass; the chunked attention's group gives pages of finished chunks back."""
    from rusty_llama_b200.cache import Cache
    from rusty_llama_b200.parts.base import KVNeed, StateNeed

    cfg = CONFIGS["a"]()
    model = _model(cfg)
    needs = dict(model.cache_needs())
    order = pt.layer_order(cfg)
    assert len(needs) == len(order) == 1 + 2 * 3 + 1
    assert needs[0] == (KVNeed(2, 20, 0, value_dim=12, chunk=7), StateNeed((3, 24, 41), torch.float32), StateNeed((3,), torch.float32))
    for run, (layer, _) in enumerate(order):
        if layer == 1:
            assert needs[run] == StateNeed((3, 24, 40), torch.float32)
        if layer == 2:
            assert needs[run] == StateNeed((1, 40, 8), torch.float32)
    assert needs[7][0] == KVNeed(4, 16, 0, value_dim=24, chunk=64)
    cache = Cache(model.cache_needs(), 64 * 6, 2, torch.float32, "cpu")
    s = cache.open_sequence()
    for run in range(1, 7):
        cache.view(run).state[s] += 1.0
    cache.view(0)[1].state[s] += 1.0
    cache.view(0)[2].state[s] += 1.0
    cache.reserve([s], [200])
    cache.commit([s], [200])
    cache.check_consistent()
    cache.close_sequence(s)
    assert cache.open_sequence() == s
    for run in range(1, 7):
        assert float(cache.view(run).state[s].abs().max()) == 0.0
    assert float(cache.view(0)[1].state[s].abs().max()) == 0.0 and float(cache.view(0)[2].state[s].abs().max()) == 0.0
    cache.check_consistent()


def test_run_order_adds_the_embedding_before_every_pass_but_the_first():
    from rusty_llama_b200.registry import describe_model

    for name in CONFIGS:
        cfg = CONFIGS[name]()
        spec = describe_model(cfg)
        runs = [(e.layer, bool(e.add_input)) for e in spec.schedule]
        assert runs == pt.layer_order(cfg), name


def test_configuration_errors_name_the_place():
    from rusty_llama_b200.errors import ConfigError
    from rusty_llama_b200.registry import describe_model

    base = CONFIGS["a"]()
    for change, text in (
        (lambda c: c["layers"][0].update(type="conv"), "layers[0].type"),
        (lambda c: c["layers"][0]["mixer"]["left"].update(heads=5), "kv_heads"),
        (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=22), "rot.dims"),
        (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "mlp.kind"),
        (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "experts"),
        (lambda c: c["loop"].update(stop=9), "loop"),
        (lambda c: c["layers"][1]["mixer"].update(tau=0.0), "tau"),
    ):
        cfg = copy.deepcopy(base)
        change(cfg)
        with pytest.raises(ConfigError) as e:
            describe_model(cfg)
        assert text in str(e.value), (text, str(e.value))
