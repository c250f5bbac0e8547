"""Pagatar on the CPU: configuration, model spec, tensor names, cache and state needs, a folder written and read back,
and properties of the plain mechanisms."""

import copy
import math

import pytest
import torch

import plain_pagatar as plain
from pagedserve_b200.config.pagatar import PagatarConfig, named_config
from pagedserve_b200.config.registry import ConfigError, resolve_architecture
from pagedserve_b200.models.model import Model, init_plan
from pagedserve_b200.models.pagatar import build_pagatar_spec
from pagedserve_b200.parts.base import PartEnv

G, L, A, X = plain.mingru_layer, plain.latent_layer, plain.attention_layer, plain.moe_mlp
CONFIG = plain.make_config(
    [G(80, X(4, 2, 24)),
     L(4, 16, 8, 24, 32, 40, mlp=X(6, 3, 16)),
     A(4, 2, 16, 24, chunk=12, taps=3, scaling=(4.0, 48, 8.0, 1.0), mlp=None),
     A(2, 1, 8, 8, chunk=None, taps=1, rot_dims=0, v_mix=False, mlp=X(3, 1, 8)),
     A(3, 3, 16, 16, chunk=20, taps=2, rot_dims=6, mlp=X(5, 5, 32))],
    width=64, vocab=97, groups=2)


def test_config_round_trip_and_registry():
    name, config_class, builder = resolve_architecture(CONFIG)
    assert name == "Pagatar" and config_class is PagatarConfig and builder is build_pagatar_spec
    config = PagatarConfig.from_dict(CONFIG)
    assert PagatarConfig.from_dict(config.to_dict()).to_dict() == config.to_dict()
    assert config.to_dict() == CONFIG
    assert config.vocabulary_size == 97 and config.norm_groups == 2


def test_keys_that_are_absent_stay_absent():
    """No 'conv': no convolution, no such tensors and nothing kept; no 'kv_heads': as many as query heads."""
    values = plain.make_config([A(4, 2, 16, 24, chunk=None, taps=None, rot_dims=8, v_mix=False, mlp=None)], width=64, vocab=31)
    values["layers"][0]["mixer"].pop("kv_heads")
    config = PagatarConfig.from_dict(values)
    assert config.layers[0]["mixer"]["kv_heads"] == 4 and config.layers[0]["mixer"]["conv"] is None
    assert "conv" not in config.to_dict()["layers"][0]["mixer"]
    spec = build_pagatar_spec(config)
    model = Model(spec, PartEnv(ops=None, dtype=torch.float32, device="cpu"))
    assert model.state_needs()[0] is None
    names = {spec.checkpoint_name(param.name) for param, _ in init_plan(spec)}
    assert not any(name.endswith(".conv") for name in names) and "l0.mix.q.b" in names and "l0.mix.g" in names


@pytest.mark.parametrize("change", [
    lambda c: c.update(vocab=0), lambda c: c.update(width=-3), lambda c: c.pop("norm"),
    lambda c: c["norm"].update(groups=3), lambda c: c["norm"].update(groups=0),
    lambda c: c["layers"][0].update(type="recurrent"), lambda c: c["layers"][0].pop("mixer"),
    lambda c: c["layers"][0]["mixer"].update(width=0),
    lambda c: c["layers"][1]["mixer"].pop("q_rank"), lambda c: c["layers"][1]["mixer"].update(rot_dim=7),
    lambda c: c["layers"][1]["mixer"]["rot"].update(dims=4), lambda c: c["layers"][1]["mixer"].update(kv_rank=1020),
    lambda c: c["layers"][2]["mixer"].pop("scale"), lambda c: c["layers"][2]["mixer"].update(heads=3),
    lambda c: c["layers"][2]["mixer"]["rot"].update(dims=7), lambda c: c["layers"][2]["mixer"]["rot"].update(dims=18),
    lambda c: c["layers"][2]["mixer"]["rot"]["scaling"].pop("fast"), lambda c: c["layers"][2]["mixer"].update(conv=0),
    lambda c: c["layers"][2]["mixer"]["mask"].update(size=0), lambda c: c["layers"][0]["mlp"].update(kind="dense"),
    lambda c: c["layers"][1]["mlp"]["router"].update(top=7), lambda c: c["layers"][1]["mlp"]["expert"].pop("ff"),
    lambda c: c["layers"][4]["mixer"].update(vdim=8)])            # values that are mixed must have one size
def test_inconsistent_configurations_are_refused(change):
    values = copy.deepcopy(CONFIG)
    change(values)
    with pytest.raises(ConfigError):
        PagatarConfig.from_dict(values)


def test_spec_needs_and_tensor_names():
    spec = build_pagatar_spec(PagatarConfig.from_dict(CONFIG))
    assert [(entry.layer, entry.cache_layer) for entry in spec.schedule] == [(i, i) for i in range(5)]
    model = Model(spec, PartEnv(ops=None, dtype=torch.bfloat16, device="cpu"))
    needs, states = model.kv_needs(), model.state_needs()
    assert needs[0] is None and states[0].shape == (80,)
    assert (needs[1].planes, needs[1].n_kv_heads, needs[1].head_dim, needs[1].bounded) == (1, 1, 40, False)
    assert states[1] is None
    # heads of 16 keys and 24 values take 32 numbers in a bfloat16 cache; two kept rows of q | k | v
    assert (needs[2].chunk, needs[2].head_dim, needs[2].planes) == (12, 32, 2)
    assert states[2].shape == (2 * (4 + 2 + 2) * 32,)
    assert needs[3].chunk is None and not needs[3].bounded and states[3] is None         # one tap: nothing is kept
    assert states[4].shape == ((3 + 3 + 3) * 16,)
    # the first layer that mixes values shares them, the later one reads them
    roles = [block.mixer.params.get("value_mix") for block in model.blocks]
    assert roles[2]["role"] == "first" and roles[3] is None and roles[4]["role"] == "later"
    assert model.blocks[2].mixer.step_shared() == {"first_values": (48, torch.float32)}
    assert model.blocks[4].mixer.step_shared() == {}
    assert model.graph_safe
    names = {spec.checkpoint_name(param.name): tuple(param.shape) for param, _ in init_plan(spec)}
    assert names == {name: tuple(shape) for name, shape in plain.tensor_shapes(CONFIG).items()}
    assert spec.normalise_name("l3.norm2") == "l3.norm2.weight" and spec.normalise_name("l3.dwa") == "l3.dwa"


def test_a_random_model_folder_reads_back(tmp_path):
    from pagedserve_b200.weights.random_init import write_random_model
    from pagedserve_b200.weights.safetensors_io import read_safetensors

    config = named_config("pagatar-tiny")
    folder = write_random_model(str(tmp_path), config, seed=7)
    stored = read_safetensors(folder + "/model.safetensors")
    tensors, read_config = plain.read_folder(folder)
    assert set(stored) == set(plain.tensor_shapes(read_config))
    logits = plain.forward(tensors, read_config, [3, 1, 4, 1, 5, 9, 2, 6])
    assert logits.shape == (8, config.vocab) and torch.isfinite(logits).all()
    spec = build_pagatar_spec(PagatarConfig.from_dict(read_config))
    model = Model(spec, PartEnv(ops=None, dtype=torch.float32, device="cpu"))
    model.load_folder(folder)                                   # every tensor found, shaped and cast


def test_stretched_frequencies_match_the_part():
    from pagedserve_b200.parts.positions import RotaryPositions

    for dims, base, scaling in ((16, 10000.0, (4.0, 48, 8.0, 1.0)), (64, 10000.0, (4.0, 512, 16.0, 1.0)),
                                (32, 500.0, (8.0, 64, 16.0, 2.0)), (6, 100.0, None), (40, 20000.0, (2.0, 4096, 4.0, 4.0))):
        named = dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None
        part = RotaryPositions(dict(dims=dims, base=base, interleaved=False, head_dim=dims, scaling=named), "",
                               PartEnv(ops=None, dtype=torch.float32, device="cpu"))
        want, amplitude = plain.stretched_frequencies(dims, base, named, torch.float64)
        split = part.inv_freq_split().double()
        assert torch.allclose(split[:, 0] + split[:, 1], want, rtol=1e-12, atol=0)
        assert torch.allclose(part.inv_freq().double(), want, rtol=1e-6)
        assert math.isclose(part.amplitude, amplitude, rel_tol=1e-12)
    # between the two ends the stretched pairs turn slower by the factor, the fast ones as before
    stretched, _ = plain.stretched_frequencies(64, 10000.0, dict(factor=4.0, original=512, fast=16.0, slow=1.0), torch.float64)
    bare, _ = plain.stretched_frequencies(64, 10000.0, None, torch.float64)
    assert torch.allclose(stretched[:5], bare[:5]) and torch.allclose(stretched[-5:] * 4.0, bare[-5:])
    assert not torch.allclose(stretched[5:15], bare[5:15]) and not torch.allclose(stretched[5:15] * 4.0, bare[5:15])


def test_properties_of_the_plain_mechanisms():
    g = torch.Generator().manual_seed(0)
    # the recurrence is a running blend: a gate of one takes the candidate, a gate of zero keeps the state
    tensors = {"l0.mix.z": torch.zeros(4, 3), "l0.mix.z.b": torch.tensor([40.0, 40.0, -40.0, -40.0]),
               "l0.mix.x": torch.zeros(4, 3), "l0.mix.x.b": torch.tensor([2.0, -3.0, 2.0, -3.0]),
               "l0.mix.g": torch.zeros(4, 3), "l0.mix.g.b": None, "l0.mix.o": torch.eye(4)}
    h = torch.randn(5, 3, generator=g, dtype=torch.float64)
    out = plain.min_gru(tensors, "l0.", {"width": 4}, h)
    assert torch.allclose(out, torch.zeros(5, 4, dtype=torch.float64))               # silu(0) = 0 closes the output
    tensors["l0.mix.g"] = torch.full((4, 3), 0.0)
    # a convolution whose last tap is one and whose others are zero passes its input; one tap back shifts it
    u = torch.randn(6, 2, generator=g, dtype=torch.float64)
    assert torch.equal(plain.short_convolution(u, torch.tensor([[0.0, 0.0, 1.0]] * 2, dtype=torch.float64)), u)
    shifted = plain.short_convolution(u, torch.tensor([[0.0, 1.0, 0.0]] * 2, dtype=torch.float64))
    assert torch.equal(shifted[1:], u[:-1]) and float(shifted[0].abs().max()) == 0.0
    # a chunked mask: position 12 starts a run of its own
    seen = plain.causal_mask(torch.arange(30), 12)
    assert seen[11, 0] and not seen[12, 11] and seen[23, 12] and not seen[24, 23] and not seen[3, 4]
    # groups are normed one by one
    x = torch.cat([torch.full((8,), 1000.0), torch.full((8,), 0.001)]).double()
    normed = plain.group_rms_norm(x, torch.ones(16, dtype=torch.float64), 1e-12, 2)
    assert torch.allclose(normed, torch.ones(16, dtype=torch.float64), atol=1e-5)
    # the correction decides who stands, the weight is the bare score
    tensors = {"router": torch.tensor([[1.0], [0.0], [-1.0]]), "correction": torch.tensor([-5.0, 0.0, 5.0])}
    chosen, weights, _ = plain.router_election(tensors, "", torch.ones(1, 1, dtype=torch.float64), 1)
    assert int(chosen[0, 0]) == 2 and math.isclose(float(weights[0, 0]), 1.0 / (1.0 + math.e), rel_tol=1e-12)
