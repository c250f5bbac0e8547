"""Zositar on the CPU: configuration, model spec, tensor names, the cache's view of chunked masks and borrowed
caches, and properties of the plain mechanisms."""

import copy

import pytest
import torch

import plain_zositar as plain
from pagedserve_b200.cache import CacheManager, KVNeed
from pagedserve_b200.config.registry import ConfigError, resolve_architecture
from pagedserve_b200.config.zositar import ZositarConfig, named_config
from pagedserve_b200.models.model import Model
from pagedserve_b200.models.zositar import build_zositar_spec
from pagedserve_b200.parts.base import PartEnv

A, D, X = plain.attention_layer, plain.dense_mlp, plain.moe_mlp
CONFIG = plain.make_config(
    [A(4, 2, 16, 24, chunk=12, rot_dims=8, mlp=D(48)),
     A(4, 2, 16, 24, chunk=12, rot_dims=8, mlp=X(4, 2, 24, shared_ff=32)),
     A(4, 2, 16, 24, chunk=20, rot_dims=8, mlp=None, kv_from=1),
     A(2, 1, 8, 8, chunk=5, rot_dims=0, mlp=X(6, 3, 16, shared_ff=None)),
     A(4, 2, 16, 24, chunk=12, rot_dims=8, mlp=D(16), kv_from=1)],
    width=64, vocab=97)


def test_config_round_trip_and_registry():
    name, config_class, builder = resolve_architecture(CONFIG)
    assert name == "Zositar" and config_class is ZositarConfig and builder is build_zositar_spec
    config = ZositarConfig.from_dict(CONFIG)
    assert ZositarConfig.from_dict(config.to_dict()).to_dict() == config.to_dict()
    assert config.to_dict() == CONFIG
    assert config.vocabulary_size == 97


@pytest.mark.parametrize("change", [
    lambda c: c.update(vocab=0), lambda c: c.update(width=-3), lambda c: c.pop("norm"),
    lambda c: c["layers"][0].update(type="recurrent"), lambda c: c["layers"][0].pop("mixer"),
    lambda c: c["layers"][0]["mixer"].pop("scale"), lambda c: c["layers"][0]["mixer"].update(heads=3),
    lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18),
    lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), lambda c: c["layers"][0]["mlp"].update(kind="other"),
    lambda c: c["layers"][1]["mlp"]["router"].update(top=5), lambda c: c["layers"][1]["mlp"]["expert"].pop("limit"),
    lambda c: c["layers"][1]["mlp"]["shared"].update(ff=0), lambda c: c["layers"][2]["mixer"].update(kv_from=2),
    lambda c: c["layers"][2]["mixer"].update(kv_from=3), lambda c: c["layers"][4]["mixer"].update(kv_from=2),
    lambda c: c["layers"][2]["mixer"].update(vdim=16), lambda c: c["layers"][2]["mixer"]["rot"].update(base=3.0),
    lambda c: c["layers"][0]["mixer"].update(kv_from=0)])
def test_inconsistent_configurations_are_refused(change):
    values = copy.deepcopy(CONFIG)
    change(values)
    with pytest.raises(ConfigError):
        ZositarConfig.from_dict(values)


def test_spec_schedule_needs_and_tensor_names():
    spec = build_zositar_spec(ZositarConfig.from_dict(CONFIG))
    # a borrower runs on its lender's cache layer
    assert [(entry.layer, entry.cache_layer) for entry in spec.schedule] == [(0, 0), (1, 1), (2, 1), (3, 3), (4, 1)]
    model = Model(spec, PartEnv(ops=None, dtype=torch.float32, device="cpu"))
    needs = model.kv_needs()
    assert [need is not None for need in needs] == [True, True, False, True]      # none behind the last lender
    # a cached head holds the larger of the key and value sizes
    assert (needs[0].n_kv_heads, needs[0].head_dim, needs[0].chunk, needs[0].window) == (2, 24, 12, None)
    # read through chunks of 12 and of 20: rows stay for the longer look back
    assert (needs[1].head_dim, needs[1].chunk, needs[1].window) == (24, None, 20)
    assert (needs[3].n_kv_heads, needs[3].head_dim, needs[3].chunk) == (1, 8, 5)
    assert all(state is None for state in model.state_needs())
    names = {spec.checkpoint_name(param.name) for param in model.param_specs()}
    assert names == set(plain.tensor_shapes(CONFIG))
    shapes = {spec.checkpoint_name(param.name): tuple(param.shape) for param in model.param_specs()}
    assert shapes == plain.tensor_shapes(CONFIG)
    assert model.graph_safe


def test_bfloat16_heads_are_padded_to_the_kernels_sizes():
    values = plain.make_config([A(3, 3, 20, 12, chunk=7, rot_dims=6, mlp=None)], width=32, vocab=11)
    spec = build_zositar_spec(ZositarConfig.from_dict(values))
    need32 = Model(spec, PartEnv(ops=None, dtype=torch.float32, device="cpu")).kv_needs()[0]
    need16 = Model(spec, PartEnv(ops=None, dtype=torch.bfloat16, device="cpu")).kv_needs()[0]
    assert need32.head_dim == 20 and need16.head_dim == 32
    # the stored tensors keep their own shapes either way
    model = Model(spec, PartEnv(ops=None, dtype=torch.bfloat16, device="cpu"))
    shapes = {spec.checkpoint_name(param.name): tuple(param.shape) for param in model.param_specs()}
    assert shapes == plain.tensor_shapes(values)
    tensors = {spec.normalise_name(name): value.float() for name, value in plain.random_model(values, 1).items()}
    model.bind(tensors)
    mixer = model.blocks[0].mixer
    assert mixer.w_in.shape == (3 * 32 * 3, 32) and mixer.w_out.shape == (32, 3 * 32)
    w_in = mixer.w_in.reshape(3, 3, 32, 32)                       # q | k | v, head, slot, width
    assert float(w_in[0, :, 20:].abs().max()) == 0.0 and float(w_in[2, :, 12:].abs().max()) == 0.0
    assert torch.equal(w_in[2, 1, :12], tensors["l0.mix.v"][12:24])
    assert float(mixer.w_out.reshape(32, 3, 32)[:, :, 12:].abs().max()) == 0.0


def test_named_sizes_draw_random_models():
    from pagedserve_b200.weights.random_init import random_tensors

    config = named_config("zositar-tiny")
    tensors = random_tensors(config, seed=1)
    logits = plain.forward(tensors, config.to_dict(), [1, 2, 3, 4, 5, 6, 7])
    assert logits.shape == (7, config.vocab) and torch.isfinite(logits).all()
    assert any(layer["mixer"].get("kv_from") is not None for layer in config.layers)
    assert {layer["mlp"]["kind"] for layer in config.layers} == {"dense", "moe"}


# ------------------------------------------------------------------ what the cache keeps for a chunked mask
def test_first_needed_position_of_chunks_windows_and_both():
    chunked = KVNeed(2, 16, None, chunk=12)
    assert [chunked.first_needed(n) for n in (0, 1, 11, 12, 13, 35, 36)] == [0, 0, 0, 12, 12, 24, 36]
    assert chunked.bounded and not KVNeed(2, 16, None).bounded
    longer = KVNeed(2, 16, None, chunk=20)
    both = chunked.merged(longer)
    assert both == longer.merged(chunked) and (both.window, both.chunk) == (20, None)
    # every key that either mask can still see lies at or behind the merged need's first position
    for length in range(0, 90):
        assert both.first_needed(length) <= min(chunked.first_needed(length), longer.first_needed(length))
    assert chunked.merged(KVNeed(2, 16, None)) == KVNeed(2, 16, None)
    assert chunked.merged(KVNeed(2, 16, 30)).window == 30
    assert chunked.merged(KVNeed(1, 16, None, chunk=12)) is None
    assert chunked.merged(chunked) is chunked


def test_pages_behind_the_current_chunk_are_released_and_used_again():
    cache = CacheManager([KVNeed(1, 8, None, chunk=6), KVNeed(1, 8, None)], [None, None], 4, 8, 2, 64)
    chunked, full = cache.groups
    cache.admit("a")
    cache.extend("a", 13)                    # positions 0..12: the chunk of position 13 begins at 12 = page 3
    assert chunked.allocator.used_pages == 4
    cache.commit("a")
    assert chunked.tables["a"][:3] == [-1, -1, -1] and chunked.tables["a"][3] >= 0
    assert chunked.allocator.used_pages == 1 and full.allocator.used_pages == 4
    cache.extend("a", 5)                     # positions 13..17 (the chunk 12..17 lies in pages 3 and 4)
    cache.commit("a")
    assert chunked.allocator.used_pages == 1         # position 18 opens a chunk and page 4 holds 16..19
    assert [page >= 0 for page in chunked.tables["a"]] == [False, False, False, False, True]
    cache.admit("b")
    cache.extend("b", 9)
    cache.commit("b")
    cache.free("a")
    cache.free("b")
    cache.check_invariants()
    assert chunked.allocator.used_pages == 0 and full.allocator.used_pages == 0


# ------------------------------------------------------------------ the plain mechanisms themselves
def test_plain_chunk_mask():
    mask = plain.chunk_mask(torch.arange(10), 4)
    assert mask[5].tolist() == [False] * 4 + [True, True] + [False] * 4
    assert mask[4].tolist() == [False] * 4 + [True] + [False] * 5
    assert mask[3].tolist() == [True] * 4 + [False] * 6
    shifted = plain.chunk_mask(torch.arange(6, 10), 4)                   # positions, not places in the portion
    assert shifted[2].tolist() == [False, False, True] + [False] and shifted[1].tolist() == [True, True, False, False]
    assert plain.chunk_mask(torch.arange(5), None).tolist() == torch.ones(5, 5).tril().bool().tolist()


def test_plain_attention_sees_its_own_chunk_only():
    tensors = plain.random_model(CONFIG, 3)
    m = CONFIG["layers"][0]["mixer"]
    g = torch.Generator().manual_seed(1)
    h = torch.randn(40, 64, generator=g, dtype=torch.float64)
    run = lambda rows: plain.attention_mixer(tensors, "l0.", m, rows, torch.arange(40), 1e-5,
                                             plain.keys_and_values(tensors, "l0.", m, rows, torch.arange(40), 1e-5))
    out = run(h)
    changed = h.clone()
    changed[15] += 1.0
    moved = (run(changed) - out).abs().max(-1).values
    assert float(moved[:15].max()) == 0.0 and float(moved[15:24].min()) > 0.0 and float(moved[24:].max()) == 0.0


def test_plain_rotation_pairs_halves_and_keeps_sizes():
    g = torch.Generator().manual_seed(2)
    x = torch.randn(3, 2, 12, generator=g, dtype=torch.float64)
    y = plain.rotate_halves(x, torch.tensor([0, 5, 900]), 8, 10000.0)
    assert torch.equal(y[0], x[0]) and torch.equal(y[..., 8:], x[..., 8:])
    for i in range(4):                                                  # number i turns with number i + 4
        pair = torch.stack([x[..., i], x[..., i + 4]]), torch.stack([y[..., i], y[..., i + 4]])
        assert torch.allclose((pair[0] ** 2).sum(0), (pair[1] ** 2).sum(0))
    angle = 5.0 * 10000.0 ** (-2.0 / 8)
    assert torch.allclose(y[1, 0, 1], x[1, 0, 1] * torch.cos(torch.tensor(angle)) - x[1, 0, 5] * torch.sin(torch.tensor(angle)))
    # scores depend on the distance only
    q, k = x[:1, :1], x[1:2, :1]
    at = lambda p, r: (plain.rotate_halves(q, torch.tensor([p]), 8, 50.0) * plain.rotate_halves(k, torch.tensor([r]), 8, 50.0)).sum()
    assert torch.allclose(at(9, 4), at(105, 100))


def test_plain_router_and_experts():
    g = torch.Generator().manual_seed(4)
    router = {"router": torch.randn(6, 16, generator=g, dtype=torch.float64)}
    h = torch.randn(30, 16, generator=g, dtype=torch.float64)
    chosen, weights, margin = plain.router_election(router, "", h, 2)
    scores = torch.sigmoid(h @ router["router"].T)
    assert torch.equal(chosen.sort(-1).values, scores.topk(2).indices.sort(-1).values)
    assert torch.allclose(weights, torch.gather(scores, 1, chosen)) and bool((margin >= 0).all())
    assert float((weights.sum(-1) - 1).abs().max()) > 0.1                # the scores themselves, no renormalizing
    expert = {"gate": torch.eye(4, dtype=torch.float64), "up": torch.eye(4, dtype=torch.float64),
              "down": torch.eye(4, dtype=torch.float64)}
    row = torch.tensor([[3.0, -3.0, 0.5, 0.0]], dtype=torch.float64)
    out = plain.clamped_expert(expert, "", row, 1.0)[0]
    s = lambda z: z * torch.sigmoid(torch.tensor(1.702 * z, dtype=torch.float64))
    assert torch.allclose(out, torch.stack([s(1.0) * 2.0, s(-3.0) * 0.0, s(0.5) * 1.5, s(0.0) * 1.0]))
