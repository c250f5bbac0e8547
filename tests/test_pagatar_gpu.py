"""Pagatar in the engine against the plain implementation (tests/plain_pagatar.py): every mechanism alone, then whole
models through the step function, the trace replay and the scheduler, in float32 and bfloat16.

The configurations are made here, with random weights; sizes differ from model to model so that nothing rests on a
value that happens to be 1 or on two sizes that happen to be equal."""

import io
import json
import os
import tempfile
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import helpers
import plain_pagatar as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"

G = plain.mingru_layer
L = plain.latent_layer
A = plain.attention_layer
X = plain.moe_mlp
STRETCH = (4.0, 48, 8.0, 1.0)                # factor, original, fast, slow
# all three mixers, two key heads for four query heads, values larger than keys (a cached head is padded), chunks
# that are no multiple of a page, a layer without a feed-forward, a second value-mixing layer
CONFIG_A = plain.make_config(
    [G(80, X(4, 2, 24)),
     L(4, 16, 8, 24, 32, 40, mlp=X(6, 3, 16)),
     A(4, 2, 16, 24, chunk=12, taps=3, scaling=STRETCH, mlp=X(4, 2, 24)),
     G(48, None),
     A(4, 2, 16, 24, chunk=20, taps=3, scaling=STRETCH, mlp=X(5, 1, 32)),
     L(2, 32, 16, 16, 48, 24, base=500.0, scale=0.15, mlp=None)],
    width=64, vocab=97, groups=2)
# heads of 64 and 128 numbers and a cached latent row of 128 (the tensor-core attention kernels), chunks that span
# several key tiles, four norm groups, an attention layer that comes first
CONFIG_B = plain.make_config(
    [A(4, 2, 64, 64, chunk=70, taps=4, rot_dims=32, base=500.0, scale=0.11, scaling=(8.0, 64, 16.0, 2.0), mlp=X(8, 2, 32)),
     L(4, 32, 32, 48, 96, 64, base=250000.0, scale=0.12, mlp=X(4, 1, 48)),
     G(160, X(4, 2, 40)),
     A(2, 1, 128, 128, chunk=200, taps=2, base=250000.0, scale=0.07, mlp=None)],
    width=128, vocab=211, eps=1e-6, groups=4)
# nothing a multiple of 8 or 16: three norm groups, a chunk of one token, heads that do not turn, one tap, no mask,
# layers that do not mix values, single heads, every expert chosen, as many key heads as query heads
CONFIG_C = plain.make_config(
    [L(3, 10, 6, 14, 20, 36, scale=0.3, mlp=X(5, 5, 12)),
     A(3, 3, 20, 12, chunk=7, taps=2, rot_dims=6, scale=0.2, mlp=X(3, 1, 36)),
     A(6, 2, 10, 24, chunk=1, taps=1, rot_dims=0, scale=0.3, v_mix=False, mlp=None),
     G(50, X(7, 2, 9)),
     A(1, 1, 48, 36, chunk=None, taps=5, rot_dims=48, base=100.0, scale=0.15, mlp=X(3, 2, 20))],
    width=72, vocab=53, eps=1e-4, groups=3)
# every expert chosen for every token (weights still come from the router): no election that rounding could turn,
# so a bfloat16 run is compared with the plain model at every row; one norm group; a single value-mixing layer
CONFIG_D = plain.make_config(
    [G(96, X(4, 4, 32)),
     A(6, 1, 80, 48, chunk=50, taps=3, rot_dims=20, scale=0.1, scaling=STRETCH, mlp=X(3, 3, 40)),
     L(6, 24, 8, 40, 40, 72, scale=0.18, mlp=X(2, 2, 72)),
     G(64, X(2, 2, 24))],
    width=96, vocab=131, eps=1e-6, groups=1)
# one layer of each kind alone
CONFIG_E = plain.make_config([G(40, X(4, 2, 24))], width=48, vocab=61, groups=2)
CONFIG_F = plain.make_config([A(5, 5, 16, 16, chunk=24, taps=3, rot_dims=4, mlp=X(7, 2, 8))], width=40, vocab=77, groups=5)
# attention layers without a convolution (no 'conv' key, no such tensors): values are still blended in two of them
CONFIG_I = plain.make_config([A(4, 2, 16, 24, chunk=20, taps=None, rot_dims=8, mlp=None),
                              A(2, 1, 32, 48, chunk=None, taps=None, scaling=STRETCH, mlp=X(4, 2, 16)),
                              A(3, 1, 16, 16, chunk=9, taps=None, v_mix=False, mlp=None)],
                             width=56, vocab=71, groups=2)
CONFIG_H = plain.make_config([L(2, 8, 4, 8, 12, 16, mlp=None)], width=32, vocab=41, groups=1)
# latent layers whose turning part has four numbers, so that a head's flat part neither starts nor ends on a multiple
# of eight numbers in the rows of q and in the rows attention reads: cached rows of 128 and of 192 numbers; and a
# cached row of more than 256 numbers (wider than the tensor-core attention kernels take)
CONFIG_G = plain.make_config([L(4, 24, 4, 40, 124, 64, scale=0.15, mlp=None), L(6, 40, 4, 20, 188, 72, scale=0.1, mlp=None),
                              L(3, 16, 8, 24, 300, 40, scale=0.2, mlp=None)],
                             width=80, vocab=89, groups=2)
# layers for keys that stand out: chunks of 12 and of 70, every earlier key hundreds of tokens back, a latent layer
CONFIG_S = plain.make_config(
    [A(4, 2, 16, 16, chunk=12, taps=3, rot_dims=8, scale=0.25, scaling=STRETCH, v_mix=False, mlp=None),
     A(4, 2, 64, 64, chunk=70, taps=3, rot_dims=32, base=500.0, scale=0.11, v_mix=False, mlp=None),
     A(4, 2, 32, 32, chunk=None, taps=3, rot_dims=16, scale=0.18, v_mix=False, mlp=None),
     L(4, 16, 8, 16, 32, 40, scale=0.2, mlp=None)],
    width=96, vocab=67, groups=2)
# layers as wide as a small model's (the tensor-core products and prompt attention run at these sizes), with
# elections (float32) and with every expert chosen (bfloat16)
def _middle(all_chosen):
    top = lambda experts, few: experts if all_chosen else few
    return plain.make_config(
        [G(640, X(16, top(16, 2), 64)),
         L(8, 64, 32, 64, 96, 256, base=20000.0, scale=0.1, mlp=X(6, top(6, 2), 100)),
         A(8, 2, 80, 80, chunk=100, taps=3, rot_dims=40, base=20000.0, scale=0.11, scaling=(8.0, 256, 32.0, 1.0),
           mlp=X(16, top(16, 2), 64)),
         G(512, None),
         A(8, 8, 64, 20, chunk=256, taps=4, rot_dims=16, base=20000.0, scale=0.125, mlp=X(6, top(6, 1), 100)),
         A(16, 1, 96, 160, chunk=32, taps=2, base=500000.0, scale=0.08, mlp=X(6, top(6, 2), 100))],
        width=512, vocab=700, eps=1e-6, groups=2)


CONFIGS = {"a": (CONFIG_A, 1, 16), "b": (CONFIG_B, 2, 16), "c": (CONFIG_C, 3, 8), "d": (CONFIG_D, 4, 32),   # config, seed, page
           "e": (CONFIG_E, 5, 16), "f": (CONFIG_F, 6, 8), "h": (CONFIG_H, 7, 16), "s": (CONFIG_S, 8, 16),
           "g": (CONFIG_G, 9, 16), "i": (CONFIG_I, 10, 16),
           "m": (_middle(False), 21, 16), "n": (_middle(True), 22, 16)}

_FOLDERS, _TENSORS, _LOGITS, _SETTLED = {}, {}, {}, {}
# An election of experts is a close call where the choice score of the last one in leads the first one left out by
# less than this: the rounding of a bfloat16 run may then elect another expert than the plain float64 model does.
CLOSE_CALL = 0.02


def folder_of(which):
    if which not in _FOLDERS:
        from pagedserve_b200.weights.safetensors_io import write_safetensors

        config, seed, _ = CONFIGS[which]
        holder = tempfile.TemporaryDirectory(prefix=f"ps_pagatar_{which}_")
        tensors = plain.random_model(config, seed)
        if which == "s":
            # a convolution that passes the current token only, and large query gains: one key can stand out
            for name in tensors:
                if name.endswith(".conv"):
                    tensors[name] = torch.zeros_like(tensors[name])
                    tensors[name][:, -1] = 1.0
                if name.endswith("mix.q.norm") or name.endswith("mix.dq.norm"):
                    tensors[name] = (tensors[name].float() * 3.0).to(torch.bfloat16)
        _TENSORS[which] = tensors
        with open(os.path.join(holder.name, "config.json"), "w") as handle:
            json.dump(config, handle)
        write_safetensors(os.path.join(holder.name, "model.safetensors"), tensors)
        _FOLDERS[which] = holder
    return _FOLDERS[which].name


def plain_logits(which, sequences):
    folder_of(which)
    out = {}
    for name, tokens in sequences.items():
        key = (which, tuple(tokens))
        if key not in _LOGITS:
            margins = []
            _LOGITS[key] = plain.forward(_TENSORS[which], CONFIGS[which][0], tokens, margins=margins).numpy()
            close = torch.stack(margins).min(0).values < CLOSE_CALL if margins else torch.zeros(len(tokens), dtype=bool)
            _SETTLED[key] = int(close.nonzero()[0]) if close.any() else len(tokens)
        out[name] = _LOGITS[key]
    return out


def assert_rows_close(got, want, dtype, what, mean_factor=1.0):
    """float32: every logit within 3e-5 of the scale (sums differ in order only), the best token the same.
    bfloat16: a row's error is the root mean square over the vocabulary against that of the logits; rounding alone
    gives about 1 % in the mean over the rows and a few per cent at single rows, while a wrong key, a lost state, a
    chunk's edge or an expert moves a row by 30 % and more."""
    assert got.shape == want.shape and np.isfinite(got).all(), what
    if dtype == "float32":
        scale = float(np.abs(want).max())
        error = np.abs(got.astype(np.float64) - want).max(-1)
        assert float(error.max()) <= 3e-5 * scale, \
            f"{what}: row {int(error.argmax())} is off by {float(error.max()):.3e}, scale {scale:.3e}"
        ordered = np.sort(want, axis=-1)
        clear = (ordered[:, -1] - ordered[:, -2]) > 1e-4 * scale
        assert (got.argmax(-1) == want.argmax(-1))[clear].all(), f"{what}: another best token"
        return
    error = np.sqrt(((got - want) ** 2).mean(-1)) / np.sqrt((want ** 2).mean())
    assert float(error.max()) < 0.12, f"{what}: row {int(error.argmax())} is off by {float(error.max()):.3f}"
    assert float(error.mean()) < 0.025 * mean_factor, f"{what}: rows are off by {float(error.mean()):.4f} in the mean"


def settled_rows(which, tokens):
    """How many leading rows of a sequence are free of close calls in the plain model."""
    plain_logits(which, {"x": tokens})
    return _SETTLED[(which, tuple(tokens))]


def build_engine(which, dtype, **options):
    from pagedserve_b200.config.engine_config import EngineConfig
    from pagedserve_b200.engine.engine import Engine

    defaults = dict(dtype=dtype, block_size=CONFIGS[which][2], num_blocks=96, max_num_seqs=4, max_model_len=512)
    defaults.update(options)
    engine = Engine.from_folder(folder_of(which), EngineConfig(**defaults))
    engine.plain_config = CONFIGS[which][0]
    return engine


def sequences_for(which, lengths, seed=0):
    vocab = CONFIGS[which][0]["vocab"]
    return {f"s{i}": helpers.random_tokens(vocab, n, seed=seed + i) for i, n in enumerate(lengths)}


def rel_err(got, want):
    want = want.double()
    return float((got.double().cpu() - want).abs().max() / want.abs().max().clamp_min(1e-30))


# ------------------------------------------------------------------ the replay program on whole models
def run_replay(which, dtype, steps, slots=4):
    from pagedserve_b200.engine import replay as replay_module

    with tempfile.TemporaryDirectory(prefix="ps_out_") as out:
        args = SimpleNamespace(model=folder_of(which), dtype=dtype, out=out, max_tokens=helpers.peak_tokens(steps),
                               block_size=CONFIGS[which][2], max_num_seqs=slots, disable_cuda_graphs=False)
        stdin = io.StringIO("".join(json.dumps(step) + "\n" for step in steps))
        assert replay_module.run(args, stdin=stdin, stdout=io.StringIO()) == 0
        return helpers.collect(out, steps)


def check_replay(which, dtype, steps, sequences, what):
    got = run_replay(which, dtype, steps)
    want = plain_logits(which, sequences)
    for name in sequences:
        rows = len(sequences[name])
        if dtype == "bfloat16":
            # up to the first close call of the plain model's elections the rows must agree; float32 runs of the same
            # schedules compare every row
            rows = settled_rows(which, sequences[name])
            if rows == 0:
                continue
        assert_rows_close(got[name][:rows], want[name][:rows], dtype, f"{what}/{which}/{name}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["a", "b", "c", "d"])
def test_whole_prompts_and_decoded_tails(which, dtype):
    """Each request alone: whole in one step, and most of it in one step with its tail token by token, so that
    prefill and decoding through the cache and the kept state give the same logits.  Sequences of one and two tokens
    (shorter than a convolution) included."""
    sequences = sequences_for(which, [1, 2, 37, 150, 301], seed=10)
    check_replay(which, dtype, helpers.trace_whole(sequences), sequences, "whole")
    check_replay(which, dtype, helpers.trace_tail(sequences, tail=48), sequences, "tail")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["a", "b", "c", "d"])
def test_portions_of_every_size(which, dtype):
    """Portions down to two tokens (fewer than the convolution's taps), cut inside pages, chunks and key tiles."""
    sequences = sequences_for(which, [61, 143, 260], seed=20)
    check_replay(which, dtype, helpers.trace_chunks(sequences, seed=1), sequences, "portions")
    check_replay(which, dtype, helpers.trace_chunks(sequences, seed=2, sizes=(2, 2, 17, 64, 3, 130, 2, 31)), sequences,
                 "portions-2")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["a", "b", "c", "d"])
def test_mixed_batches_reuse_pages_and_slots(which, dtype):
    """Nine unequal requests through four slots: portions of some beside single tokens of others, requests left
    out of steps, pages and state slots handed out again; every request must equal itself alone."""
    sequences = sequences_for(which, [90, 33, 200, 5, 61, 148, 17, 75, 2], seed=30)
    steps = helpers.trace_mixed(sequences, seed=3, live=4, decode_tail=20, max_portion=40)
    assert helpers.peak_tokens(steps) < sum(len(t) for t in sequences.values())
    check_replay(which, dtype, steps, sequences, "mixed")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["e", "f", "h", "g", "i"])
def test_models_of_one_layer(which, dtype):
    sequences = sequences_for(which, [70, 3, 131, 29, 64, 1], seed=70)
    check_replay(which, dtype, helpers.trace_whole(sequences), sequences, "whole")
    steps = helpers.trace_mixed(sequences, seed=5, live=4, decode_tail=16, max_portion=30)
    check_replay(which, dtype, steps, sequences, "mixed")


@pytest.mark.parametrize("dtype,which", [("float32", "m"), ("bfloat16", "n")])
def test_a_model_of_middle_size(dtype, which):
    """A thousand tokens whole, then unequal requests mixed, at layer sizes where the tensor-core kernels run."""
    sequences = sequences_for(which, [1000, 260, 97, 23, 1], seed=60)
    check_replay(which, dtype, helpers.trace_whole(sequences), sequences, "whole")
    steps = helpers.trace_mixed(sequences, seed=6, live=4, decode_tail=24, max_portion=70)
    check_replay(which, dtype, steps, sequences, "mixed")


def test_long_decoding_float32():
    """A short prompt, then hundreds of tokens one by one: the recurrent state and the kept rows of the convolutions
    are carried through every step, chunk after chunk begins and ends among the decoded tokens."""
    sequences = sequences_for("a", [340], seed=40)
    check_replay("a", "float32", helpers.trace_tail(sequences, tail=330), sequences, "long decode")
    sequences = sequences_for("c", [200], seed=41)
    check_replay("c", "float32", helpers.trace_tail(sequences, tail=190), sequences, "long decode")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_in_one_step_and_in_portions(dtype):
    """1,500 tokens: angles of more than a thousand radians, chunks far from the sequence's start, a recurrence
    folded in many segments."""
    which = "b" if dtype == "float32" else "d"          # (bfloat16: the model without elections of experts)
    sequences = sequences_for(which, [1500], seed=80)
    wanted = list(range(0, 1500, 97)) + list(range(1460, 1500))
    whole = [{"step": 0, "entries": [{"id": "s0", "tokens": sequences["s0"], "want": wanted}], "end": ["s0"]}]
    got = run_replay(which, dtype, whole)
    want = plain_logits(which, sequences)["s0"][wanted]
    assert_rows_close(got["s0"], want, dtype, "long prompt in one step")
    steps, number, done = [], 0, 0
    for size in [700, 500, 270] + [1] * 30:
        places = [i for i in range(size) if done + i in wanted]
        steps.append({"step": number, "entries": [{"id": "s0", "tokens": sequences["s0"][done:done + size],
                                                   "want": places}], "end": []})
        number, done = number + 1, done + size
    steps[-1]["end"] = ["s0"]
    got = run_replay(which, dtype, steps)
    assert_rows_close(got["s0"], want, dtype, "long prompt in portions")


def test_cache_and_state_needs():
    engine = build_engine("a", "bfloat16")
    needs, states = engine.model.kv_needs(), engine.model.state_needs()
    assert [need is not None for need in needs] == [False, True, True, False, True, True]
    assert (needs[1].planes, needs[1].n_kv_heads, needs[1].head_dim, needs[1].bounded) == (1, 1, 40, False)
    assert (needs[2].chunk, needs[4].chunk, needs[2].head_dim) == (12, 20, 32)          # heads of 16 and 24: 32
    assert states[0].shape == (80,) and states[3].shape == (48,) and states[1] is None
    assert states[2].shape == (2 * (4 + 2 + 2) * 32,)                                   # taps - 1 rows of q | k | v
    # chunked layers give their pages back while the request lives
    from pagedserve_b200.engine.batch import StepEntry

    tokens = sequences_for("a", [300], seed=50)["s0"]
    for lo in range(0, 300, 50):
        engine.step([StepEntry("r", tokens[lo:lo + 50], [49])])
    used = sorted(group.allocator.used_pages for group in engine.cache.groups)
    assert used[0] <= 3 and used[-1] == 19
    engine.finish("r")
    engine.cache.check_invariants()


# ------------------------------------------------------------------ generation through the scheduler
@pytest.mark.parametrize("strategy", ["orca", "sarathi"])
@pytest.mark.parametrize("which", ["a", "c"])
def test_greedy_generation_equals_the_plain_model(which, strategy):
    from pagedserve_b200.engine.engine import generate

    engine = build_engine(which, "float32", strategy=strategy, prefill_chunk_size=7, max_num_seqs=3)
    prompts = list(sequences_for(which, [9, 30, 3, 55, 1], seed=60).values())
    got = generate(engine, prompts, max_new_tokens=12)
    config, tensors = CONFIGS[which][0], _TENSORS[which]
    for prompt, tokens in zip(prompts, got):
        sequence = list(prompt)
        for _ in range(12):
            logits = plain.forward(tensors, config, sequence)[-1]
            top = torch.topk(logits, 2).values
            if float(top[0] - top[1]) < 1e-3 * float(logits.abs().max()):
                break                                        # a near tie: either token is a correct greedy choice
            sequence.append(int(logits.argmax()))
        made = len(sequence) - len(prompt)
        assert tokens[:made] == sequence[len(prompt):]
    engine.check_status()


def test_command_line_runs_a_model_folder(capsys):
    from pagedserve_b200.main import main

    assert main(["--model", folder_of("c"), "--dtype", "bfloat16", "--max-new-tokens", "4", "--block-size", "8",
                 "--num-blocks", "64", "--max-batch-size", "2", "--prompt-ids", "1 2 3 4 5"]) == 0
    assert "request 0:" in capsys.readouterr().out
    # a named size with random weights
    assert main(["--model", "pagatar-tiny", "--seed", "3", "--dtype", "float32", "--max-new-tokens", "5",
                 "--num-blocks", "32", "--max-batch-size", "2", "--prompt-ids", "7 8 9"]) == 0
    assert "request 0:" in capsys.readouterr().out


# ------------------------------------------------------------------ each part alone
def make_ctx(engine, entries, shared=None):
    from pagedserve_b200.engine.batch import StepEntry

    ctx = engine.runner.prepare([StepEntry(*entry) for entry in entries])
    engine.runner.begin(ctx)
    ctx.shared = shared or {}
    return ctx


def layer_context(engine, index):
    from pagedserve_b200.parts.base import LayerContext

    entry = engine.spec.schedule[index]
    layer = LayerContext(entry.layer, entry.cache_layer, engine.model.positions)
    cache = engine.cache
    group_index = cache.group_of_layer.get(entry.cache_layer)
    if group_index is not None:
        group = cache.groups[group_index]
        layer.k_pool, layer.v_pool = group.layer_views(entry.cache_layer)
        layer.page_stride, layer.page_size = group.page_stride, group.page_size
        layer.pool, layer.pool_layer = group.pool, group.cache_layers.index(entry.cache_layer)
        layer.block_table = cache.slots.table_views[group_index]
    layer.state = cache.state.get(entry.cache_layer)
    return engine.model.blocks[entry.layer], layer


def run_mixer(engine, index, fed, tokens, cuts, first_values=None, name="x", others=()):
    """The mixer of layer ``index`` over ``fed`` [T, W] in portions ``cuts`` (so that later ones start from pages,
    state and kept rows).  ``first_values`` [T, n]: what the first value-mixing layer is taken to have left.
    ``others``: (name, tokens) of requests whose single tokens ride in the last portion's step."""
    block, layer = layer_context(engine, index)
    width = fed.shape[1]
    residual = torch.zeros(fed.shape[0], width, dtype=torch.float32, device=DEV)
    for number, (lo, hi) in enumerate(zip(cuts[:-1], cuts[1:])):
        entries = [(name, tokens[lo:hi], [])]
        rows = fed[lo:hi]
        beside = others if number == len(cuts) - 2 else ()
        if beside:
            entries = [(other, [token], []) for other, token in beside] + entries
            g = torch.Generator().manual_seed(number)
            rows = torch.cat([torch.randn(len(beside), width, generator=g).to(fed.dtype), rows])
        shared = {}
        if first_values is not None:
            pad = torch.zeros(len(beside), first_values.shape[1])
            shared = {"first_values": torch.cat([pad, first_values[lo:hi].float()]).to(DEV).contiguous()}
        elif hasattr(block.mixer, "step_shared"):
            shared = {key: torch.zeros(len(rows), size, dtype=dtype, device=DEV)
                      for key, (size, dtype) in block.mixer.step_shared().items()}
        ctx = make_ctx(engine, entries, shared)
        out = torch.zeros(len(rows), width, dtype=torch.float32, device=DEV)
        block.mixer.forward(rows.to(DEV).contiguous(), out, ctx, layer)
        residual[lo:hi] = out[len(beside):]
        engine.cache.commit_many([entry[0] for entry in entries])
    engine.cache.free(name)
    return residual


def plain_mixer(which, index, fed, first_values=None):
    config, tensors = CONFIGS[which][0], _TENSORS[which]
    entry = config["layers"][index]
    eps, positions = config["norm"]["eps"], torch.arange(fed.shape[0])
    if entry["type"] == "mingru":
        return plain.min_gru(tensors, f"l{index}.", entry["mixer"], fed)
    if entry["type"] == "latent_attention":
        return plain.latent_attention(tensors, f"l{index}.", entry["mixer"], fed, positions, eps)
    return plain.gated_attention(tensors, f"l{index}.", entry["mixer"], fed, positions, eps, first_values)[0]


def mixing_role(which, index):
    """None, "first" or "later": what layer ``index`` does with values shared between layers."""
    layers = CONFIGS[which][0]["layers"]
    if layers[index]["type"] != "attention" or not layers[index]["mixer"].get("v_mix"):
        return None
    earlier = [i for i in range(index) if layers[i]["type"] == "attention" and layers[i]["mixer"].get("v_mix")]
    return "later" if earlier else "first"


@pytest.mark.parametrize("dtype,tol", [("float32", 4e-6), ("bfloat16", 1.5e-2)])
@pytest.mark.parametrize("which", ["a", "b", "c", "d"])
def test_each_part_alone(which, dtype, tol):
    """The norm in groups, the sum behind a norm with the average over depth, every mixer, the experts and the head,
    each fed with the plain implementation's own values.  The mixers run a prompt in three portions (the last of two
    tokens), so the later ones start from pages, state and kept rows."""
    engine = build_engine(which, dtype)
    config, tensors = CONFIGS[which][0], _TENSORS[which]
    eps, groups, compute = config["norm"]["eps"], config["norm"]["groups"], engine.dtype
    count, cuts = 45, [0, 29, 43, 45]
    tokens = helpers.random_tokens(config["vocab"], count, seed=9)
    g = torch.Generator().manual_seed(5)
    width = config["width"]
    stream = torch.randn(count, width, generator=g, dtype=torch.float64) * 2.0
    result = torch.randn(count, width, generator=g, dtype=torch.float64) * 3.0
    ops = engine.model.env.ops
    for index, entry in enumerate(config["layers"]):
        prefix = f"l{index}."
        block = engine.model.blocks[index]
        # x += norm(y), y = 0, the result stored, the average over depth formed, the rounded copy left
        history = torch.randn(len(config["layers"]) + 1, count, width, generator=g, dtype=torch.float64)
        weights = tensors[prefix + "dwa"].double()
        last = "norm2" if entry["mlp"] is not None else "norm1"
        summed = stream + plain.group_rms_norm(result, tensors[prefix + last].double(), eps, groups)
        want = sum(weights[j] * history[j] for j in range(index + 1)) + weights[index + 1] * summed
        x, y = stream.float().to(DEV), result.float().to(DEV)
        kept = history.float().to(DEV)
        copy = torch.empty(count, width, dtype=compute, device=DEV)
        block.norms["post_feed_forward" if entry["mlp"] is not None else "post_mixer"].add_into(
            y, x, copy, kept, index + 2, block.depth_weight)
        assert rel_err(x, want) < 4e-6 and rel_err(kept[index + 1], summed) < 4e-6 and float(y.abs().max()) == 0.0
        assert rel_err(copy, want) < max(tol / 2, 1e-6)
        # the mixer
        fed = (stream * 0.5).to(compute)
        role = mixing_role(which, index)
        first = None
        if role == "later":
            first = torch.randn(count, entry["mixer"]["kv_heads"] * entry["mixer"]["vdim"], generator=g).double()
        want = plain_mixer(which, index, fed.double(), first)
        got = run_mixer(engine, index, fed, tokens, cuts, first)
        assert rel_err(got, want) < tol, (which, index, entry["type"])
        if entry["mlp"] is not None:
            margins = []
            want = plain.routed_ff(tensors, prefix + "mlp.", entry["mlp"], fed.double(), margins)
            clear = margins[0] > 1e-3
            residual = torch.zeros(count, width, dtype=torch.float32, device=DEV)
            ctx = make_ctx(engine, [("y", tokens, [])])
            block.feed_forward.forward(fed.to(DEV), residual, ctx)
            engine.cache.rollback("y")
            engine.cache.free("y")
            assert rel_err(residual.cpu()[clear], want[clear]) < tol, (which, index, "experts")
    # the embedding with its norm, the model's norm on chosen rows, and the head against the token table
    ctx = make_ctx(engine, [("z", tokens, [0, 7, 44])])
    embedded = engine.model.embedding.forward(ctx, engine.model.positions)
    want = plain.group_rms_norm(tensors["embed"].double()[tokens], tensors["embed.norm"].double(), eps, groups)
    assert rel_err(embedded, want) < 4e-6
    picked = engine.model.final_norm.forward(stream.float().to(DEV), rows=ctx.logit_rows)
    logits = engine.model.head.forward(picked, engine.model.embedding)
    want = plain.group_rms_norm(stream, tensors["final.norm"].double(), eps, groups)[[0, 7, 44]] @ tensors["embed"].double().T
    assert rel_err(logits, want) < tol
    engine.cache.rollback("z")
    engine.cache.free("z")
    engine.check_status()


def test_the_first_value_mixing_layer_leaves_its_values():
    """What a layer of role "first" stores is its own values behind the convolution, token by token, also where a
    portion starts from kept rows."""
    engine = build_engine("a", "float32")
    config, tensors = CONFIGS["a"][0], _TENSORS["a"]
    count = 30
    tokens = helpers.random_tokens(config["vocab"], count, seed=4)
    fed = torch.randn(count, config["width"], generator=torch.Generator().manual_seed(3), dtype=torch.float64)
    want = plain.attention_values(tensors, "l2.", config["layers"][2]["mixer"], fed)
    block, layer = layer_context(engine, 2)
    got = []
    for lo, hi in ((0, 17), (17, 19), (19, 30)):
        shared = {"first_values": torch.zeros(hi - lo, want.shape[1], device=DEV)}
        ctx = make_ctx(engine, [("v", tokens[lo:hi], [])], shared)
        block.mixer.forward(fed[lo:hi].float().to(DEV), torch.zeros(hi - lo, config["width"], device=DEV), ctx, layer)
        engine.cache.commit_many(["v"])
        got.append(shared["first_values"].cpu())
    engine.cache.free("v")
    assert rel_err(torch.cat(got), want) < 4e-6


@pytest.mark.parametrize("dtype,tol", [("float32", 4e-6), ("bfloat16", 1.5e-2)])
@pytest.mark.parametrize("which,count", [("a", 300), ("b", 128), ("b", 517), ("c", 260)])
def test_experts_with_many_tokens(which, count, dtype, tol):
    """Steps of many tokens sort their rows by expert (bfloat16): the same sums as token by token.  Tokens whose
    election is a close call are left out: the two sides may elect differently there."""
    engine = build_engine(which, dtype, max_model_len=1024)
    config, tensors = CONFIGS[which][0], _TENSORS[which]
    tokens = helpers.random_tokens(config["vocab"], count, seed=11)
    g = torch.Generator().manual_seed(count)
    fed = torch.randn(count, config["width"], generator=g, dtype=torch.float64).to(engine.dtype)
    for index, entry in enumerate(config["layers"]):
        if entry["mlp"] is None:
            continue
        margins = []
        want = plain.routed_ff(tensors, f"l{index}.mlp.", entry["mlp"], fed.double(), margins)
        clear = margins[0] > 1e-3
        residual = torch.zeros(count, config["width"], dtype=torch.float32, device=DEV)
        ctx = make_ctx(engine, [("y", tokens, [])])
        engine.model.blocks[index].feed_forward.forward(fed.to(DEV), residual, ctx)
        engine.cache.rollback("y")
        engine.cache.free("y")
        assert rel_err(residual.cpu()[clear], want[clear]) < tol, (which, index)
    engine.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("experts,top", [(8, 2), (6, 3), (12, 4), (5, 5), (64, 6), (3, 1)])
def test_the_correction_moves_the_election_and_not_the_weights(dtype, experts, top):
    """Corrections as large as the scores' spread: the elected experts are those of score + correction, their
    weights the plain scores; without the correction other experts would have been chosen."""
    from pagedserve_b200.kernels.ops import Ops

    compute = torch.float32 if dtype == "float32" else torch.bfloat16
    ops = Ops(compute)
    g = torch.Generator().manual_seed(experts * 10 + top)
    tokens, width = 200, 48
    x = torch.randn(tokens, width, generator=g).to(compute)
    router = (torch.randn(experts, width, generator=g) / width ** 0.5).to(compute)
    correction = 0.5 * torch.randn(experts, generator=g)
    tensors = {"router": router, "correction": correction}
    chosen, weights, margin = plain.router_election(tensors, "", x.double(), top)
    dense = torch.empty(tokens, experts, dtype=torch.float32, device=DEV)
    got = torch.empty(tokens, top, dtype=torch.int32, device=DEV)
    got_w = torch.empty(tokens, top, dtype=torch.float32, device=DEV)
    ops.moe_route(x.to(DEV), router.to(DEV), None, dense, got, got_w, None, top, 0, 0, score="sigmoid", normalize=False,
                  correction=correction.to(DEV))
    clear = margin > 1e-2
    assert clear.sum() > tokens // 2
    assert (got.cpu().long().sort(-1).values == chosen.sort(-1).values)[clear].all()
    scores = torch.sigmoid(x.double() @ router.double().T)
    assert rel_err(got_w.cpu()[clear], torch.gather(scores, 1, got.cpu().long())[clear]) < (1e-5 if dtype == "float32" else 2e-2)
    plain_choice = torch.topk(scores, top).indices.sort(-1).values
    if top < experts:
        assert (plain_choice != chosen.sort(-1).values).any()             # the correction does decide elections
    picked = torch.zeros(tokens, experts).scatter_(1, got.cpu().long(), got_w.cpu())
    assert torch.equal(picked, dense.cpu())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,groups", [(64, 1), (64, 2), (72, 3), (40, 5), (512, 4), (1024, 2), (96, 32)])
def test_norm_in_groups(dtype, width, groups):
    """Rows whose runs differ a thousandfold in size: a norm over the whole row would leave the small runs near
    zero.  From float32 rows and from rows of the compute type, gathered, and in place."""
    from pagedserve_b200.kernels.ops import Ops

    compute = torch.float32 if dtype == "float32" else torch.bfloat16
    ops = Ops(compute)
    g = torch.Generator().manual_seed(width + groups)
    rows = torch.randn(37, width, generator=g, dtype=torch.float64)
    rows = (rows.reshape(37, groups, -1) * (10.0 ** (torch.arange(groups) % 4).double())[None, :, None]).reshape(37, width)
    gain = (1.0 + 0.2 * torch.randn(width, generator=g)).float()
    want = plain.group_rms_norm(rows.float().double(), gain.double(), 1e-5, groups)
    picks = torch.tensor([5, 0, 36, 5, 11], dtype=torch.int32)
    out = torch.empty(5, width, dtype=compute, device=DEV)
    ops.group_rms_norm(rows.float().to(DEV), gain.to(DEV), 1e-5, groups, out, rows=picks.to(DEV))
    assert rel_err(out, want[picks.long()]) < (2e-6 if dtype == "float32" else 8e-3)
    assert float(out.float().abs().reshape(5, groups, -1).amax(-1).min()) > 0.3           # every run is of order one
    in_place = rows.float().to(DEV)
    ops.group_rms_norm(in_place, gain.to(DEV), 1e-5, groups, in_place)
    assert rel_err(in_place, want) < 2e-6
    typed = rows.to(compute)
    wide = torch.zeros(37, width + 24, dtype=compute, device=DEV)                          # rows inside wider rows
    wide[:, 8:8 + width] = typed.to(DEV)
    out = torch.empty(37, width, dtype=compute, device=DEV)
    ops.group_rms_norm(wide[:, 8:8 + width], gain.to(DEV), 1e-5, groups, out)
    assert rel_err(out, plain.group_rms_norm(typed.double(), gain.double(), 1e-5, groups)) < (2e-6 if dtype == "float32" else 8e-3)


@pytest.mark.parametrize("width,lengths", [(48, [1, 1, 1]), (50, [2, 17, 1, 300]), (208, [700, 3]), (1024, [129])])
def test_the_recurrence_alone_in_segments_and_token_by_token(width, lengths):
    """The gated recurrence of entries of unequal length in one launch, folded in segments, equals the plain loop;
    the state it leaves is where a next step starts from (slots in another order than the entries)."""
    from pagedserve_b200.kernels.ops import Ops

    ops = Ops(torch.float32)
    g = torch.Generator().manual_seed(width)
    total = sum(lengths)
    zug = torch.randn(total, 3 * width, generator=g) * 2.0
    starts = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    slots = torch.randperm(len(lengths), generator=g).to(torch.int32)
    state = torch.randn(len(lengths) + 1, width, generator=g)
    z, u, gate = zug[:, :width].double(), zug[:, width:2 * width].double(), zug[:, 2 * width:].double()
    candidate = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    want = torch.empty(total, width, dtype=torch.float64)
    final = state.double().clone()
    for item, (lo, hi) in enumerate(zip(starts[:-1], starts[1:])):
        s = state[slots[item]].double()
        for t in range(lo, hi):
            s = (1 - torch.sigmoid(z[t])) * s + torch.sigmoid(z[t]) * candidate[t]
            want[t] = s * torch.nn.functional.silu(gate[t])
        final[slots[item]] = s
    ctx = SimpleNamespace(max_q_len=max(lengths), q_start=torch.from_numpy(starts).to(DEV), item_slot=slots.to(DEV),
                          num_items=len(lengths))
    out = torch.empty(total, width, device=DEV)
    kept = state.to(DEV)
    ops.mingru_scan(zug.to(DEV), width, kept, ctx, out)
    assert rel_err(out, want) < 5e-6 and rel_err(kept, final) < 5e-6


@pytest.mark.parametrize("taps,lengths", [(1, [5, 1]), (2, [1, 1, 9]), (3, [2, 1, 40, 1]), (4, [1, 2, 3, 200]), (7, [3, 3, 1])])
def test_the_convolution_alone_over_kept_rows(taps, lengths):
    """Entries shorter and longer than the convolution, twice in a row: the second step starts from the rows the
    first one kept, which for short entries are partly older kept rows moved up."""
    from pagedserve_b200.kernels.ops import Ops

    ops = Ops(torch.float32)
    g = torch.Generator().manual_seed(taps)
    conv, extra = 40, 12
    weight = torch.randn(conv, taps, generator=g)
    items = len(lengths)
    slots = torch.randperm(items, generator=g).to(torch.int32)
    kept = torch.zeros(items + 1, (taps - 1) * conv, device=DEV) if taps > 1 else None
    history = [torch.zeros(0, conv + extra, dtype=torch.float64) for _ in lengths]
    for step in range(3):
        counts = lengths if step != 1 else lengths[::-1]
        starts = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
        u = torch.randn(int(starts[-1]), conv + extra, generator=g)
        token_item = torch.repeat_interleave(torch.arange(items), torch.tensor(counts)).to(torch.int32)
        want = torch.empty(u.shape, dtype=torch.float64)
        for item, (lo, hi) in enumerate(zip(starts[:-1], starts[1:])):
            before = history[item].shape[0]
            history[item] = torch.cat([history[item], u[lo:hi].double()])
            whole = plain.short_convolution(history[item][:, :conv], weight.double())
            want[lo:hi, :conv] = whole[before:]
            want[lo:hi, conv:] = u[lo:hi, conv:].double()
        ctx = SimpleNamespace(token_item=token_item.to(DEV), q_start=torch.from_numpy(starts).to(DEV),
                              item_slot=slots.to(DEV), num_items=items)
        out = torch.empty(u.shape, device=DEV)
        ops.short_conv(u.to(DEV), weight.to(DEV), taps, conv, kept, ctx, out)
        assert rel_err(out, want) < 3e-6, (taps, step)


# ------------------------------------------------------------------ a key that stands out, at every edge
def standing_out(index, key_at, query_at, count, seed):
    """Rows for the mixer of layer ``index`` of the model whose convolutions pass the current token only, such that
    query head 0 at ``query_at`` points straight along the key of key head 0 at ``key_at`` as attention meets it:
    whether that key is seen decides the head's result.  The norms remove the query's size, so the rows are solved
    for its direction only; the model has large query gains instead."""
    config, tensors = CONFIGS["s"][0], _TENSORS["s"]
    entry = config["layers"][index]
    m, eps = entry["mixer"], config["norm"]["eps"]
    g = torch.Generator().manual_seed(seed)
    rows = torch.randn(count, config["width"], generator=g, dtype=torch.float64)
    t = lambda name: tensors[f"l{index}.mix.{name}"].double()
    where = torch.tensor([key_at - query_at])
    if entry["type"] == "attention":
        d = m["dim"]
        k_pre = (rows[key_at] @ t("k").T + t("k.b"))[:d]
        k_normed = plain.rms_norm(k_pre[None, None], t("k.norm"), eps)
        rot = m["rot"]
        target = plain.rotate_halves(k_normed, where, rot["dims"], rot["base"], rot.get("scaling"))[0, 0]
        wanted = 6.0 * target / t("q.norm") - t("q.b")[:d]
        rows[query_at] = torch.linalg.lstsq(t("q")[:d], wanted[:, None]).solution[:, 0]
        return rows
    d, r, R = m["dim"], m["rot_dim"], m["kv_rank"]
    down = rows[key_at] @ t("dkv").T
    c = plain.rms_norm(down[None, :R], t("dkv.norm"), eps)[0]
    k_flat = (t("uk") @ c)[:d]                                                       # head 0
    k_turn = plain.rotate_neighbours(down[None, R:], where, m["rot"]["dims"], m["rot"]["base"])[0]
    target = torch.cat([k_flat, k_turn])
    latent = torch.linalg.lstsq(t("uq")[:d + r], (6.0 * target)[:, None]).solution[:, 0]
    rows[query_at] = torch.linalg.lstsq(t("dq"), (latent / t("dq.norm"))[:, None]).solution[:, 0]
    return rows


@pytest.mark.parametrize("dtype,tol", [("float32", 1e-5), ("bfloat16", 2.5e-2)])
@pytest.mark.parametrize("index,pairs", [
    (0, ((299, 288), (299, 287), (288, 288), (288, 287), (290, 289))),               # chunks of 12, pages of 16
    (1, ((279, 210), (279, 209), (285, 280), (285, 279), (270, 256))),               # chunks of 70: 210..279, 280..
    (2, ((299, 0), (299, 3), (150, 1), (255, 16), (256, 255))),                      # every earlier key, far back
    (3, ((299, 0), (299, 2), (150, 1), (255, 16), (272, 271), (17, 15)))])            # the latent layer
def test_a_key_that_stands_out_at_edges_and_far_back(index, pairs, dtype, tol):
    """One query made to point at one key, placed at a chunk's first position, one before it, at the query itself,
    at page and tile borders and hundreds of tokens back: in a prompt in one step, in two portions cut between the
    two tokens, with the query decoded alone, and decoded among single tokens of other requests."""
    engine = build_engine("s", dtype)
    config = CONFIGS["s"][0]
    size = (config["layers"][index]["mixer"].get("mask") or {}).get("size")
    count = 300
    tokens = helpers.random_tokens(config["vocab"], count, seed=2)
    # three other requests hold state and pages of their own meanwhile
    for other in ("p", "q", "r"):
        run = helpers.random_tokens(config["vocab"], 20, seed=ord(other))
        from pagedserve_b200.engine.batch import StepEntry

        engine.step([StepEntry(other, run, [])])
    for query_at, key_at in pairs:
        fed = standing_out(index, key_at, query_at, count, seed=query_at + key_at).to(engine.dtype)
        want = plain_mixer("s", index, fed.double())
        if key_at != query_at:
            # the key decides the row: with another key in its place the plain result is another one altogether
            changed = fed.double().clone()
            changed[key_at] = 0.0
            moved = plain_mixer("s", index, changed)[query_at]
            seen = size is None or key_at // size == query_at // size
            assert (float((moved - want[query_at]).abs().max()) > 0.05 * float(want[query_at].abs().max())) == seen
        alone = [0, query_at, query_at + 1, count] if query_at + 1 < count else [0, query_at, count]
        for cuts, others in (([0, count], ()), ([0, key_at + 1, count] if key_at < query_at else [0, 7, count], ()),
                             (alone, ()), (alone[:-1] if len(alone) == 4 else alone, (("p", 1), ("q", 2), ("r", 3)))):
            got = run_mixer(engine, index, fed[:cuts[-1]], tokens, cuts, others=others)
            assert rel_err(got[query_at], want[query_at]) < tol, (index, query_at, key_at, cuts)
            assert rel_err(got, want[:cuts[-1]]) < tol, (index, query_at, key_at, cuts)
    engine.check_status()


@pytest.mark.parametrize("heads,size,positions,window", [
    (8, 128, list(range(623, 635)), None),                      # ten key tiles over eight CTAs: two tiles a CTA
    (8, 128, [5, 70, 130, 200, 260, 330, 390, 450, 520, 580, 640, 700], None),
    (16, 128, list(range(1000, 1012)), None), (8, 64, [631] * 9, None), (4, 48, list(range(900, 940)), None),
    (8, 128, list(range(623, 635)), 128), (8, 112, list(range(700, 710)), -300)])
def test_heads_as_rows_over_far_keys(heads, size, positions, window):
    """Single tokens whose heads all read one cached row per key (the latent layers' attention): the heads of a
    token as the query rows of one tile, its keys shared out over several CTAs that each walk more than one key
    tile, against the CUDA-core kernel.  One row far back is made to stand out for the first head."""
    from pagedserve_b200.kernels.ops import Ops

    ops = Ops(torch.bfloat16)
    g = torch.Generator().manual_seed(size + len(positions))
    page, pages, count = 16, 80, len(positions)
    pool = torch.randn(pages, 1, 1, 1, page, size, generator=g).to(torch.bfloat16).to(DEV)
    rows = pool[:, 0, 0]
    table = torch.arange(pages, dtype=torch.int32, device=DEV)[None].repeat(2, 1).contiguous()
    q = (torch.randn(count, heads * size, generator=g) * 0.3).to(torch.bfloat16)
    q[:, :size] = pool[0, 0, 0, 0, 3].cpu() * 0.5                 # key 3 draws the first head wherever it is seen
    q = q.to(DEV)
    at = torch.tensor(positions, dtype=torch.int32, device=DEV)
    row = torch.zeros(count, dtype=torch.int32, device=DEV)
    want, got = torch.empty_like(q), torch.empty_like(q)
    ops.paged_attention_simt(q, want, rows, rows, pool.stride(0), row, at, table, heads, 1, size, page, window, 0.1)
    ops.shared_position_attention(q, got, rows, rows, pool.stride(0), at, table, row, heads, size, page, window, 0.1,
                                  max_kv_len=max(positions) + 1)
    assert rel_err(got, want.float().cpu()) < 1.2e-2


@pytest.mark.parametrize("rows", [1, 40, 65, 300])
@pytest.mark.parametrize("heads,depth,beside_in,cols,beside_out", [(8, 24, 4, 252, 4), (4, 24, 4, 124, 4), (8, 252, 4, 100, 0),
                                                                   (2, 96, 4, 250, 6), (3, 10, 6, 20, 6), (4, 40, 8, 68, 12)])
def test_products_of_heads_of_ragged_sizes(rows, heads, depth, beside_in, cols, beside_out):
    """Per-head products whose inputs and results are column blocks that neither start nor end on multiples of eight
    numbers (a latent layer with a short turning part): whatever kernels the heads are sent to, every head's result
    is right and the columns beside it stay as they were."""
    from pagedserve_b200.kernels.ops import Ops

    ops = Ops(torch.bfloat16)
    g = torch.Generator().manual_seed(rows + heads)
    a_full = torch.randn(rows, heads * (depth + beside_in), generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(heads * cols, depth, generator=g) * depth ** -0.5).to(torch.bfloat16).to(DEV)
    out_full = torch.full((rows, heads * (cols + beside_out)), 3.0, dtype=torch.bfloat16, device=DEV)
    a = a_full.view(rows, heads, depth + beside_in)[:, :, :depth].permute(1, 0, 2)
    out = out_full.view(rows, heads, cols + beside_out)[:, :, :cols].permute(1, 0, 2)
    ops.linear_grouped(a, w, out, max_rows=64)
    want = torch.einsum("hmk,hnk->hmn", a.float(), w.view(heads, cols, depth).float()).cpu()
    for head in range(heads):
        assert rel_err(out[head].float(), want[head]) < 8e-3, head
    if beside_out:
        assert bool((out_full.view(rows, heads, cols + beside_out)[:, :, cols:] == 3.0).all())
    assert int(ops.status_flag(DEV).item()) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,heads,size,beside,per_head", [(1, 4, 16, 0, True), (70, 3, 10, 6, True), (300, 8, 64, 32, True),
                                                             (300, 8, 64, 32, False), (33, 5, 12, 4, False), (64, 2, 40, 0, False)])
def test_the_gate_on_heads(rows, heads, size, beside, per_head, dtype):
    """The sigmoid gate on the joined heads, one gate per head or per number, on row views with something beside them
    (by pieces of 16 bytes where the sizes allow it, number by number else) against float64; the neighbours stay."""
    from pagedserve_b200.kernels.ops import Ops

    ops = Ops(dtype)
    g = torch.Generator().manual_seed(rows + size)
    width = heads * size
    full = torch.randn(rows, width + beside, generator=g).to(dtype).to(DEV)
    gates_full = (2.0 * torch.randn(rows, (heads if per_head else width) + beside, generator=g)).to(dtype).to(DEV)
    values, gates = full[:, :width], gates_full[:, beside:]
    want = values.double().view(rows, heads, size) * torch.sigmoid(gates.double()).view(rows, heads, -1)
    kept = full[:, width:].clone()
    ops.sigmoid_gate(values, gates, span=size if per_head else 1)
    assert rel_err(values, want.view(rows, width).cpu()) < (1e-6 if dtype == torch.float32 else 5e-3)
    assert torch.equal(full[:, width:], kept)
