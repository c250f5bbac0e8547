"""Zositar in the engine against the plain implementation (tests/plain_zositar.py): every mechanism alone, then whole
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
import plain_zositar as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TORCH_DTYPE = {"float32": torch.float32, "bfloat16": torch.bfloat16}

A = plain.attention_layer
D = plain.dense_mlp
X = plain.moe_mlp
# two key heads for four query heads, chunks that are no multiple of a page, a borrower whose chunk differs from
# its lender's, a layer without a feed-forward, experts with and without a shared one
CONFIG_A = plain.make_config(
    [A(4, 2, 16, 16, chunk=12, rot_dims=8, mlp=D(48)),
     A(4, 2, 16, 16, chunk=12, rot_dims=8, mlp=X(4, 2, 24, shared_ff=32)),
     A(4, 2, 16, 16, chunk=20, rot_dims=8, mlp=None, kv_from=1),
     A(4, 2, 16, 16, chunk=12, rot_dims=8, mlp=X(6, 3, 16, limit=0.8, shared_ff=None), kv_from=1)],
    width=64, vocab=97)
# heads of 64 and 128 numbers (the tensor-core attention kernels), chunks that span several key tiles, whole heads
# that turn, borrowers that come before and after other layers with caches of their own
CONFIG_B = plain.make_config(
    [A(4, 2, 64, 64, chunk=70, rot_dims=32, base=500.0, scale=0.11, mlp=D(96)),
     A(2, 1, 128, 128, chunk=200, rot_dims=128, base=250000.0, scale=0.07, mlp=X(8, 2, 32, shared_ff=64)),
     A(4, 2, 64, 64, chunk=129, rot_dims=32, base=500.0, scale=0.2, mlp=X(4, 1, 48, shared_ff=None), kv_from=0),
     A(2, 1, 128, 128, chunk=200, rot_dims=128, base=250000.0, scale=0.05, mlp=D(40), kv_from=1)],
    width=128, vocab=211, eps=1e-6)
# nothing a multiple of 8 or 16: key and value sizes that differ both ways, a chunk of one token, heads that do not
# turn at all, single heads, every expert chosen, as many key heads as query heads
CONFIG_C = plain.make_config(
    [A(3, 3, 20, 12, chunk=7, rot_dims=6, scale=0.2, mlp=X(5, 5, 12, shared_ff=20)),
     A(6, 2, 10, 24, chunk=1, rot_dims=0, scale=0.3, mlp=None),
     A(3, 3, 20, 12, chunk=33, rot_dims=6, scale=0.25, mlp=D(40), kv_from=0),
     A(1, 1, 48, 32, chunk=64, rot_dims=48, base=100.0, scale=0.15, mlp=X(3, 1, 36, limit=2.5, shared_ff=20, shared_limit=0.5))],
    width=72, vocab=53, eps=1e-4)
# every expert chosen for every token (weights still come from the router): no election that rounding could turn,
# so a bfloat16 run is compared with the plain model at every row; many query heads on one key head, values
# smaller than keys (a cached head is padded)
CONFIG_D = plain.make_config(
    [A(6, 1, 80, 48, chunk=50, rot_dims=20, scale=0.1, mlp=D(64)),
     A(6, 1, 80, 48, chunk=50, rot_dims=20, scale=0.1, mlp=X(4, 4, 32, shared_ff=48)),
     A(6, 1, 80, 48, chunk=90, rot_dims=20, scale=0.12, mlp=X(3, 3, 40, shared_ff=None), kv_from=1),
     A(4, 4, 32, 32, chunk=128, rot_dims=16, scale=0.18, mlp=X(2, 2, 72, shared_ff=24))],
    width=96, vocab=131, eps=1e-6)
# one layer, and a model whose borrowers all follow the first layer
CONFIG_E = plain.make_config([A(2, 1, 32, 16, chunk=16, rot_dims=32, mlp=X(4, 2, 24, shared_ff=8))], width=48, vocab=61)
CONFIG_F = plain.make_config(
    [A(5, 5, 16, 16, chunk=24, rot_dims=4, mlp=D(56)), A(5, 5, 16, 16, chunk=24, rot_dims=4, mlp=D(24), kv_from=0),
     A(5, 5, 16, 16, chunk=9, rot_dims=4, mlp=X(7, 2, 8, shared_ff=16), kv_from=0)], width=40, vocab=77)
# a chunk longer than any prompt of these tests: every earlier key is seen, hundreds of tokens back
CONFIG_G = plain.make_config([A(4, 2, 32, 32, chunk=1000, rot_dims=16, scale=0.18, mlp=None),
                              A(4, 2, 32, 32, chunk=400, rot_dims=16, scale=0.18, mlp=D(32), kv_from=0)], width=56, vocab=67)
# layers as wide as a small model's (the tensor-core products and prompt attention run at these sizes): sixteen
# query heads on one key head of 96, heads of 80, a lender with two borrowers that lie apart, a borrower of a
# borrower's neighbour; and the same with every expert chosen, for bfloat16
def _middle(top):
    return plain.make_config(
        [A(8, 2, 80, 80, chunk=100, rot_dims=40, base=20000.0, scale=0.11, mlp=X(16, top or 2, 64, shared_ff=128)),
         A(8, 2, 80, 80, chunk=100, rot_dims=40, base=20000.0, scale=0.11, mlp=X(16, top or 2, 64, shared_ff=128), kv_from=0),
         A(8, 8, 64, 64, chunk=256, rot_dims=16, base=20000.0, scale=0.125, mlp=D(768)),
         A(8, 2, 80, 80, chunk=100, rot_dims=40, base=20000.0, scale=0.11, mlp=D(256), kv_from=0),
         A(8, 8, 64, 64, chunk=256, rot_dims=16, base=20000.0, scale=0.125,
           mlp=X(6, top or 2, 100, limit=2.5, shared_ff=200, shared_limit=2.0), kv_from=2),
         A(16, 1, 96, 96, chunk=32, rot_dims=96, base=500000.0, scale=0.08,
           mlp=X(6, top or 1, 100, limit=2.5, shared_ff=200, shared_limit=2.0))],
        width=512, vocab=700, eps=1e-6)


CONFIG_M, CONFIG_N = _middle(None), _middle(6)
for _layer in CONFIG_N["layers"]:
    if _layer["mlp"]["kind"] == "moe":
        _layer["mlp"]["router"]["top"] = _layer["mlp"]["router"]["experts"]
CONFIGS = {"m": (CONFIG_M, 21, 16), "n": (CONFIG_N, 22, 16), "a": (CONFIG_A, 1, 16), "b": (CONFIG_B, 2, 16), "c": (CONFIG_C, 3, 8), "d": (CONFIG_D, 4, 32),   # config, seed, page
           "e": (CONFIG_E, 5, 16), "f": (CONFIG_F, 6, 8),
           # the same shapes with query gains three times as large: one key can stand out among hundreds
           "sa": (CONFIG_A, 11, 16), "sb": (CONFIG_B, 12, 16), "sc": (CONFIG_C, 13, 8), "sd": (CONFIG_D, 14, 32),
           "sg": (CONFIG_G, 15, 16)}

_FOLDERS, _TENSORS, _LOGITS, _SETTLED = {}, {}, {}, {}
# An election of experts is a close call where the score of the last one in leads the first one left out by less
# than this: the rounding of a bfloat16 run may then elect another expert than the plain float64 model does, which
# changes that token's row and, through the keys and values made from it, the rows behind it.
CLOSE_CALL = 0.02


def folder_of(which):
    if which not in _FOLDERS:
        from pagedserve_b200.weights.safetensors_io import write_safetensors

        config, seed, _ = CONFIGS[which]
        holder = tempfile.TemporaryDirectory(prefix=f"ps_zositar_{which}_")
        _TENSORS[which] = plain.random_model(config, seed)
        if which.startswith("s"):
            for name in _TENSORS[which]:
                if name.endswith("mix.q.norm"):
                    _TENSORS[which][name] = (_TENSORS[which][name].float() * 3.0).to(torch.bfloat16)
        with open(os.path.join(holder.name, "config.json"), "w") as handle:
            json.dump(config, handle)
        write_safetensors(os.path.join(holder.name, "model.safetensors"), _TENSORS[which])
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
    """float32: every logit within 2e-5 of the scale (sums differ in order only), the best token the same.
    bfloat16: a row's error is taken as the root mean square over the vocabulary against the root mean square of
    the logits; rounding alone gives about 1 % in the mean over the rows and a few per cent at single rows, while a
    wrong key, chunk edge or expert moves a row by 30 % and more."""
    assert got.shape == want.shape and np.isfinite(got).all(), what
    if dtype == "float32":
        scale = float(np.abs(want).max())
        error = np.abs(got.astype(np.float64) - want).max(-1)
        assert float(error.max()) <= 2e-5 * scale, \
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
    engine.plain_config = CONFIGS[which][0]                      # for the helpers below
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
    prefill and decoding through the cache give the same logits.  Sequences of one and two tokens included."""
    sequences = sequences_for(which, [1, 2, 37, 150, 301], seed=10)
    check_replay(which, dtype, helpers.trace_whole(sequences), sequences, "whole")
    check_replay(which, dtype, helpers.trace_tail(sequences, tail=48), sequences, "tail")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["a", "b", "c", "d"])
def test_portions_of_every_size(which, dtype):
    """Portions down to two tokens, cut inside pages, chunks and key tiles."""
    sequences = sequences_for(which, [61, 143, 260], seed=20)
    check_replay(which, dtype, helpers.trace_chunks(sequences, seed=1), sequences, "portions")
    check_replay(which, dtype, helpers.trace_chunks(sequences, seed=2, sizes=(2, 2, 17, 64, 3, 130, 2, 31)), sequences,
                 "portions-2")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["a", "b", "c", "d"])
def test_mixed_batches_reuse_pages_and_slots(which, dtype):
    """Nine unequal requests through four slots: portions of some beside single tokens of others, requests left
    out of steps, pages and slots handed out again; every request must equal itself alone."""
    sequences = sequences_for(which, [90, 33, 200, 5, 61, 148, 17, 75, 2], seed=30)
    steps = helpers.trace_mixed(sequences, seed=3, live=4, decode_tail=20, max_portion=40)
    assert helpers.peak_tokens(steps) < sum(len(t) for t in sequences.values())
    check_replay(which, dtype, steps, sequences, "mixed")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["e", "f"])
def test_small_models_of_other_shapes(which, dtype):
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
    """A short prompt, then 330 tokens one by one: chunk after chunk begins and ends among the decoded tokens, and
    the pages of chunks that have passed are released behind them."""
    sequences = sequences_for("a", [340], seed=40)
    check_replay("a", "float32", helpers.trace_tail(sequences, tail=330), sequences, "long decode")
    sequences = sequences_for("c", [200], seed=41)
    check_replay("c", "float32", helpers.trace_tail(sequences, tail=190), sequences, "long decode")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_in_one_step_and_in_portions(dtype):
    """1,500 tokens: angles of more than a thousand radians, chunks far from the sequence's start."""
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


@pytest.mark.parametrize("dtype,which,most", [("float32", "a", 6), ("bfloat16", "d", 5)])
def test_chunked_layers_give_pages_back(dtype, which, most):
    """Keys of chunks that have passed are never read again: their pages return to the pool while the request
    lives, also where a borrower with a longer chunk reads the same cache layer."""
    engine = build_engine(which, dtype, num_blocks=24)
    tokens = sequences_for(which, [300], seed=50)["s0"]
    from pagedserve_b200.engine.batch import StepEntry

    got = []
    for lo in range(0, 300, 50):
        got.append(engine.step([StepEntry("r", tokens[lo:lo + 50], list(range(50)))]).cpu().numpy())
        # 300 tokens would need 19 pages of 16 (10 of 32) in each group; the chunks keep a few
        assert all(group.allocator.used_pages <= most for group in engine.cache.groups)
    assert_rows_close(np.concatenate(got), plain_logits(which, {"r": tokens})["r"], dtype, "chunk pages")
    engine.finish("r")
    engine.cache.check_invariants()


def test_a_borrower_has_no_pages_of_its_own():
    engine = build_engine("b", "bfloat16")
    schedule = [(entry.layer, entry.cache_layer) for entry in engine.spec.schedule]
    assert schedule == [(0, 0), (1, 1), (2, 0), (3, 1)]
    assert sorted(engine.cache.group_of_layer) == [0, 1]
    needs = engine.model.kv_needs()
    assert len(needs) == 2                                   # no cache layer for the borrowers
    # the lender's rows stay for as long as the longer of the two chunks can look back
    assert (needs[0].chunk, needs[0].window) == (None, 129) and needs[1].chunk == 200


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
    assert main(["--model", "zositar-tiny", "--seed", "3", "--dtype", "float32", "--max-new-tokens", "5",
                 "--num-blocks", "32", "--max-batch-size", "2", "--prompt-ids", "7 8 9"]) == 0
    assert "request 0:" in capsys.readouterr().out


# ------------------------------------------------------------------ each part alone
def make_ctx(engine, entries):
    from pagedserve_b200.engine.batch import StepEntry

    ctx = engine.runner.prepare([StepEntry(*entry) for entry in entries])
    engine.runner.begin(ctx)
    return ctx


def layer_context(engine, index):
    from pagedserve_b200.parts.base import LayerContext

    entry = engine.spec.schedule[index]
    layer = LayerContext(entry.layer, entry.cache_layer, engine.model.positions)
    cache = engine.cache
    group_index = cache.group_of_layer[entry.cache_layer]
    group = cache.groups[group_index]
    layer.k_pool, layer.v_pool = group.layer_views(entry.cache_layer)
    layer.page_stride, layer.page_size = group.page_stride, group.page_size
    layer.pool, layer.pool_layer = group.pool, group.cache_layers.index(entry.cache_layer)
    layer.block_table = cache.slots.table_views[group_index]
    return engine.model.blocks[entry.layer], layer


def run_mixer(engine, index, fed, tokens, cuts, lender_fed=None, name="x"):
    """The mixer of layer ``index`` over ``fed`` [T, W] in portions ``cuts`` (so that later ones start from pages).
    A layer that borrows keys and values runs behind its lender, which is fed ``lender_fed`` in the same steps."""
    config = engine.plain_config
    block, layer = layer_context(engine, index)
    lender = config["layers"][index]["mixer"].get("kv_from")
    if lender is not None:
        lender_block, lender_layer = layer_context(engine, lender)
    residual = torch.zeros(fed.shape[0], fed.shape[1], dtype=torch.float32, device=DEV)
    for lo, hi in zip(cuts[:-1], cuts[1:]):
        ctx = make_ctx(engine, [(name, tokens[lo:hi], [])])
        if lender is not None:
            spare = torch.zeros(hi - lo, fed.shape[1], dtype=torch.float32, device=DEV)
            lender_block.mixer.forward(lender_fed[lo:hi].to(DEV).contiguous(), spare, ctx, lender_layer)
        block.mixer.forward(fed[lo:hi].to(DEV).contiguous(), residual[lo:hi], ctx, layer)
        engine.cache.commit_many([name])
    engine.cache.free(name)
    return residual


def plain_mixer(which, index, fed, lender_fed, count):
    """The plain mixer of layer ``index`` on ``fed`` (its keys and values made from ``lender_fed`` by the lender's
    tensors where it borrows)."""
    config, tensors = CONFIGS[which][0], _TENSORS[which]
    mixer = config["layers"][index]["mixer"]
    eps = config["norm"]["eps"]
    positions = torch.arange(count)
    lender = mixer.get("kv_from")
    if lender is None:
        kv = plain.keys_and_values(tensors, f"l{index}.", mixer, fed, positions, eps)
    else:
        kv = plain.keys_and_values(tensors, f"l{lender}.", config["layers"][lender]["mixer"], lender_fed, positions, eps)
    return plain.attention_mixer(tensors, f"l{index}.", mixer, fed, positions, eps, kv)


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-6), ("bfloat16", 1.2e-2)])
@pytest.mark.parametrize("which", ["a", "b", "c", "d"])
def test_each_part_alone(which, dtype, tol):
    """Norm, the attention of every layer (own keys and borrowed ones), both feed-forwards and the head, each fed
    with the plain implementation's own values.  The mixers run a prompt in two portions, so the second one starts
    from pages."""
    engine = build_engine(which, dtype)
    config, tensors = CONFIGS[which][0], _TENSORS[which]
    eps, compute = config["norm"]["eps"], engine.dtype
    count, cut = 45, 29
    tokens = helpers.random_tokens(config["vocab"], count, seed=9)
    g = torch.Generator().manual_seed(5)
    stream = torch.randn(count, config["width"], generator=g, dtype=torch.float64) * 2.0
    other = torch.randn(count, config["width"], generator=g, dtype=torch.float64) * 2.0
    for index, entry in enumerate(config["layers"]):
        prefix = f"l{index}."
        block = engine.model.blocks[index]
        t = lambda name: tensors[prefix + name].double()
        normed = plain.rms_norm(stream, t("norm1"), eps)
        got_normed = block.norms["pre_mixer"].forward(stream.float().to(DEV))
        assert rel_err(got_normed, normed) < max(tol, 1e-6) / 2
        fed = normed.to(compute)                       # what the mixer is given, as the plain side sees it too
        lender = entry["mixer"].get("kv_from")
        lender_fed = None
        if lender is not None:
            lender_fed = plain.rms_norm(other, tensors[f"l{lender}.norm1"].double(), eps).to(compute)
        want = plain_mixer(which, index, fed.double(), None if lender_fed is None else lender_fed.double(), count)
        got = run_mixer(engine, index, fed, tokens, [0, cut, count], lender_fed)
        assert rel_err(got, want) < tol, (which, index, "attention")
        if entry["mlp"] is not None:
            normed2 = plain.rms_norm(stream, t("norm2"), eps).to(compute)
            if entry["mlp"]["kind"] == "dense":
                want, clear = plain.gated_silu_ff(tensors, prefix + "mlp.", normed2.double()), slice(None)
            else:
                margins = []
                want = plain.routed_ff(tensors, prefix + "mlp.", entry["mlp"], normed2.double(), margins)
                clear = margins[0] > 1e-3
            residual = torch.zeros(count, config["width"], dtype=torch.float32, device=DEV)
            ctx = make_ctx(engine, [("y", tokens, [])])
            block.feed_forward.forward(normed2.to(DEV), residual, ctx)
            engine.cache.rollback("y")
            engine.cache.free("y")
            assert rel_err(residual.cpu()[clear], want[clear]) < tol, (which, index, entry["mlp"]["kind"])
    # the model's norm on chosen rows, and the head with a matrix of its own
    ctx = make_ctx(engine, [("z", tokens, [0, 7, 44])])
    picked = engine.model.final_norm.forward(stream.float().to(DEV), rows=ctx.logit_rows)
    logits = engine.model.head.forward(picked, engine.model.embedding)
    want = plain.rms_norm(stream, tensors["final.norm"].double(), eps)[[0, 7, 44]] @ tensors["head"].double().T
    assert rel_err(logits, want) < tol
    engine.cache.rollback("z")
    engine.cache.free("z")
    engine.check_status()


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-6), ("bfloat16", 1.2e-2)])
@pytest.mark.parametrize("which,count", [("a", 300), ("b", 128), ("b", 517), ("c", 260)])
def test_experts_with_many_tokens(which, count, dtype, tol):
    """Steps of many tokens sort their rows by expert (bfloat16): the same sums as token by token.  Tokens whose
    election is a close call are left out: the two sides may elect differently there."""
    engine = build_engine(which, dtype, max_model_len=1024)
    config, tensors = CONFIGS[which][0], _TENSORS[which]
    eps, compute = config["norm"]["eps"], engine.dtype
    tokens = helpers.random_tokens(config["vocab"], count, seed=11)
    g = torch.Generator().manual_seed(count)
    stream = torch.randn(count, config["width"], generator=g, dtype=torch.float64) * 2.0
    for index, entry in enumerate(config["layers"]):
        if entry["mlp"] is None or entry["mlp"]["kind"] != "moe":
            continue
        prefix = f"l{index}."
        block = engine.model.blocks[index]
        normed = plain.rms_norm(stream, tensors[prefix + "norm2"].double(), eps).to(compute)
        margins = []
        want = plain.routed_ff(tensors, prefix + "mlp.", entry["mlp"], normed.double(), margins)
        clear = margins[0] > 1e-3
        assert int(clear.sum()) > count * 0.9
        residual = torch.zeros(count, config["width"], dtype=torch.float32, device=DEV)
        ctx = make_ctx(engine, [("y", tokens, [])])
        block.feed_forward.forward(normed.to(DEV), residual, ctx)
        engine.cache.rollback("y")
        engine.cache.free("y")
        assert rel_err(residual.cpu()[clear], want[clear]) < tol, (which, index)
    engine.check_status()


def test_the_weight_scales_an_experts_input_not_its_output():
    """With limits that bite, expert(w h) and w expert(h) differ by far more than rounding: the engine gives the
    first.  The plain expert is evaluated both ways on the same election."""
    engine = build_engine("a", "float32")
    config, tensors = CONFIGS["a"][0], _TENSORS["a"]
    entry = config["layers"][3]["mlp"]                                   # limit 0.8, three of six, no shared expert
    g = torch.Generator().manual_seed(3)
    rows = (torch.randn(50, config["width"], generator=g, dtype=torch.float64) * 2.0).float()
    want = plain.routed_ff(tensors, "l3.mlp.", entry, rows.double())
    chosen, weights, _ = plain.router_election(tensors, "l3.mlp.", rows.double(), entry["router"]["top"])
    outside = torch.zeros_like(want)
    for row in range(50):
        for index, weight in zip(chosen[row].tolist(), weights[row]):
            outside[row] += weight * plain.clamped_expert(tensors, f"l3.mlp.e{index}.", rows[row].double()[None],
                                                          entry["expert"]["limit"])[0]
    assert float((outside - want).abs().max()) > 0.05 * float(want.abs().max())
    residual = torch.zeros(50, config["width"], dtype=torch.float32, device=DEV)
    ctx = make_ctx(engine, [("y", helpers.random_tokens(97, 50, seed=1), [])])
    engine.model.blocks[3].feed_forward.forward(rows.to(DEV), residual, ctx)
    engine.cache.rollback("y")
    engine.cache.free("y")
    assert rel_err(residual, want) < 1e-5
    engine.check_status()


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-6), ("bfloat16", 1.2e-2)])
@pytest.mark.parametrize("which,index", [("a", 1), ("b", 0), ("b", 1), ("c", 1), ("d", 1), ("d", 3)])
def test_many_single_tokens_at_once(which, index, dtype, tol):
    """Forty requests of unequal length each bring one token in the same step: every request's row equals the
    plain layer's, whatever stands beside it and wherever its chunk began."""
    engine = build_engine(which, dtype, max_num_seqs=48, num_blocks=600)
    config = CONFIGS[which][0]
    block, layer = layer_context(engine, index)
    g = torch.Generator().manual_seed(7)
    lengths = [int(n) for n in torch.randint(2, 230, (40,), generator=g)]
    chunk = config["layers"][index]["mixer"]["mask"]["size"]
    lengths[:6] = [max(2, n) for n in (2, 17, chunk, chunk + 1, 2 * chunk, 2 * chunk + 1)]
    rows = [torch.randn(n, config["width"], generator=g, dtype=torch.float64).to(engine.dtype) for n in lengths]
    want = [plain_mixer(which, index, fed.double(), None, n)[-1] for fed, n in zip(rows, lengths)]
    tokens = [helpers.random_tokens(config["vocab"], n, seed=n) for n in lengths]
    for first in range(0, 40, 4):                                   # the prompts, four at a time
        names = list(range(first, first + 4))
        ctx = make_ctx(engine, [(i, tokens[i][:-1], []) for i in names])
        host = ctx.host
        fed = torch.cat([rows[i][:-1] for i in host.requests]).to(DEV).contiguous()
        block.mixer.forward(fed, torch.zeros(fed.shape, dtype=torch.float32, device=DEV), ctx, layer)
        engine.cache.commit_many(names)
    ctx = make_ctx(engine, [(i, tokens[i][-1:], []) for i in range(40)])
    order = ctx.host.requests
    fed = torch.stack([rows[i][-1] for i in order]).to(DEV).contiguous()
    residual = torch.zeros(fed.shape, dtype=torch.float32, device=DEV)
    block.mixer.forward(fed, residual, ctx, layer)
    engine.cache.commit_many(list(range(40)))
    assert rel_err(residual, torch.stack([want[i] for i in order])) < tol
    engine.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("experts,top", [(8, 2), (6, 3), (12, 4), (5, 5), (16, 1), (64, 6), (3, 1)])
def test_router_elects_the_plain_experts(dtype, experts, top):
    """Sigmoid scores, the largest win, and the weights are the scores themselves (they do not sum to one)."""
    from pagedserve_b200.kernels.ops import Ops

    compute = TORCH_DTYPE[dtype]
    ops = Ops(compute)
    g = torch.Generator().manual_seed(experts * 7 + top)
    T, width = 203, 72
    x = torch.randn(T, width, generator=g).to(compute)
    router = (torch.randn(experts, width, generator=g) * 0.3).to(compute)
    dense = torch.empty(T, experts, device=DEV)
    chosen = torch.empty(T, top, dtype=torch.int32, device=DEV)
    chosen_w = torch.empty(T, top, device=DEV)
    ops.moe_route(x.to(DEV), router.to(DEV), None, dense, chosen, chosen_w, None, top, 0, 0, score="sigmoid",
                  normalize=False)
    want, want_w, margin = plain.router_election({"router": router}, "", x.double(), top)
    full = torch.zeros(T, experts, dtype=torch.float64).scatter_(1, want, want_w)
    same = (chosen.cpu().sort(-1).values.long() == want.sort(-1).values).all(-1)
    assert bool(same[margin > 1e-5].all())
    assert torch.allclose(dense.cpu().double()[same], full[same], rtol=2e-5, atol=2e-6)
    assert ((dense.cpu() > 0).sum(-1) == top).all()
    if top > 1:
        assert float((chosen_w.cpu().sum(-1) - 1.0).abs().min()) > 1e-3           # not renormalized
    # the election lists the experts from the largest score down
    assert bool((chosen_w.cpu()[:, :-1] >= chosen_w.cpu()[:, 1:]).all())


# ------------------------------------------------------------------ a key that stands out, at every edge
def standing_out(which, index, key_at, query_at, count, seed):
    """Rows for the attention of layer ``index`` (and for its lender, if it borrows) such that query head 0 at
    ``query_at``, after its norm and turning, points straight along the cached key of key head 0 at ``key_at``:
    whether that key is seen decides the head's result.  The norm removes the query's size, so the rows are solved
    for its direction only; the models of this test have large query gains instead."""
    config, tensors = CONFIGS[which][0], _TENSORS[which]
    m = config["layers"][index]["mixer"]
    lender = m.get("kv_from")
    source = index if lender is None else lender
    d, eps = m["dim"], config["norm"]["eps"]
    g = torch.Generator().manual_seed(seed)
    rows = torch.randn(count, config["width"], generator=g, dtype=torch.float64)
    lender_rows = torch.randn(count, config["width"], generator=g, dtype=torch.float64) if lender is not None else None
    key_rows = rows if lender is None else lender_rows
    t = lambda layer, name: tensors[f"l{layer}.mix.{name}"].double()
    k_pre = (key_rows[key_at] @ t(source, "k").T + t(source, "k.b"))[:d]                     # key head 0
    k_normed = plain.rms_norm(k_pre[None, None], t(source, "k.norm"), eps)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    # the two meet at the angle of the distance between their positions
    target = plain.rotate_halves(k_normed, torch.tensor([key_at - query_at]), rot["dims"], rot["base"])[0, 0]
    wanted = 6.0 * target / t(index, "q.norm") - t(index, "q.b")[:d]                      # head 0's projection
    rows[query_at] = torch.linalg.lstsq(t(index, "q")[:d], wanted[:, None]).solution[:, 0]
    return rows, lender_rows


@pytest.mark.parametrize("dtype,tol", [("float32", 1e-5), ("bfloat16", 2e-2)])
@pytest.mark.parametrize("which,index,pairs", [
    ("sa", 1, ((299, 288), (299, 287), (288, 288), (288, 287), (290, 289))),         # chunks of 12, pages of 16
    ("sa", 2, ((299, 280), (299, 279), (280, 279), (296, 281))),                     # borrowed keys, chunks of 20
    ("sb", 0, ((279, 210), (279, 209), (285, 280), (285, 279), (270, 256))),         # chunks of 70: 210..279, 280..
    ("sb", 1, ((299, 200), (299, 199), (199, 0), (199, 1), (200, 199))),             # chunks of 200, heads of 128
    ("sb", 2, ((257, 129), (257, 128), (258, 257), (258, 258))),                     # borrowed, chunks of 129 over 70
    ("sc", 0, ((48, 42), (48, 41), (49, 48), (55, 49))),                             # chunks of 7, pages of 8
    ("sc", 3, ((127, 64), (127, 63), (128, 127), (191, 128))),                       # one head, chunks of 64
    ("sd", 1, ((149, 100), (149, 99), (150, 149), (160, 150))),                      # six heads on one key head
    ("sd", 2, ((179, 90), (179, 89), (180, 179), (269, 180))),                       # borrowed, chunks of 90 over 50
    ("sg", 0, ((299, 0), (299, 3), (150, 1), (255, 16))),                            # every earlier key, far back
    ("sg", 1, ((299, 0), (299, 3), (150, 1), (255, 16)))])
def test_a_key_that_stands_out_just_inside_and_just_outside_the_chunk(which, index, pairs, dtype, tol):
    """One query made to point at one key, placed at the chunk's first position, one before it, at the query itself,
    at page and tile borders and hundreds of tokens back: in a prompt in one step, in two portions cut between the
    two tokens, and with the query decoded alone."""
    engine = build_engine(which, dtype)
    config = CONFIGS[which][0]
    size = config["layers"][index]["mixer"]["mask"]["size"]
    count = 300
    tokens = helpers.random_tokens(config["vocab"], count, seed=2)
    for query_at, key_at in pairs:
        rows, lender_rows = standing_out(which, index, key_at, query_at, count, seed=query_at + key_at)
        fed = rows.to(engine.dtype)
        lender_fed = None if lender_rows is None else lender_rows.to(engine.dtype)
        lent = None if lender_fed is None else lender_fed.double()
        want = plain_mixer(which, index, fed.double(), lent, count)
        if key_at != query_at:
            # the key decides the row: with another key in its place the plain result is another one altogether
            changed, changed_lent = fed.double().clone(), None if lent is None else lent.clone()
            (changed if lent is None else changed_lent)[key_at] = 0.0
            moved = plain_mixer(which, index, changed, changed_lent, count)[query_at]
            seen = key_at // size == query_at // size
            assert (float((moved - want[query_at]).abs().max()) > 0.05 * float(want[query_at].abs().max())) == seen
        for cuts in ([0, count], [0, key_at + 1, count] if key_at < query_at else [0, 7, count],
                     [0, query_at, query_at + 1, count] if query_at + 1 < count else [0, query_at, count]):
            got = run_mixer(engine, index, fed, tokens, cuts, lender_fed)
            assert rel_err(got[query_at], want[query_at]) < tol, (which, index, query_at, key_at, cuts)
            assert rel_err(got, want) < tol, (which, index, query_at, key_at, cuts)
    engine.check_status()


@pytest.mark.parametrize("dtype,tol", [("float32", 1e-5), ("bfloat16", 2e-2)])
def test_a_standing_out_key_among_single_tokens_of_other_requests(dtype, tol):
    """The query decoded alone in a step that also carries single tokens of three other requests: the key at the
    chunk's first position is seen, the one before it is not, whatever else is in the batch."""
    which, index = "sd", 1
    engine = build_engine(which, dtype, num_blocks=200)
    config = CONFIGS[which][0]
    block, layer = layer_context(engine, index)
    g = torch.Generator().manual_seed(21)
    others = {name: torch.randn(n, config["width"], generator=g, dtype=torch.float64).to(engine.dtype)
              for name, n in (("p", 51), ("q", 100), ("r", 7))}
    for query_at, key_at in ((149, 100), (149, 99), (100, 100)):
        rows, _ = standing_out(which, index, key_at, query_at, query_at + 1, seed=key_at)
        fed = dict(others, x=rows.to(engine.dtype))
        tokens = {name: helpers.random_tokens(config["vocab"], value.shape[0], seed=5) for name, value in fed.items()}
        want = {name: plain_mixer(which, index, value.double(), None, value.shape[0])[-1] for name, value in fed.items()}
        ctx = make_ctx(engine, [(name, tokens[name][:-1], []) for name in fed])
        stacked = torch.cat([fed[name][:-1] for name in ctx.host.requests]).to(DEV).contiguous()
        block.mixer.forward(stacked, torch.zeros(stacked.shape, dtype=torch.float32, device=DEV), ctx, layer)
        engine.cache.commit_many(list(fed))
        ctx = make_ctx(engine, [(name, tokens[name][-1:], []) for name in fed])
        order = ctx.host.requests
        last = torch.stack([fed[name][-1] for name in order]).to(DEV).contiguous()
        residual = torch.zeros(last.shape, dtype=torch.float32, device=DEV)
        block.mixer.forward(last, residual, ctx, layer)
        engine.cache.commit_many(list(fed))
        for name in fed:
            engine.cache.free(name)
        assert rel_err(residual, torch.stack([want[name] for name in order])) < tol, (query_at, key_at)
    engine.check_status()


# ------------------------------------------------------------------ the kernel that norms, turns and fills the pages
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,slot,dim,rot_dims,interleaved", [
    (4, 2, 16, 16, 8, False), (16, 16, 64, 64, 32, False), (3, 1, 128, 128, 128, False), (6, 1, 96, 80, 20, False),
    (5, 5, 32, 20, 6, False), (2, 2, 256, 256, 64, False), (3, 3, 20, 20, 6, False), (6, 2, 24, 10, 0, False),
    (2, 1, 18, 18, 10, False), (3, 2, 7, 7, 4, False), (4, 4, 48, 48, 16, True), (2, 1, 10, 10, 6, True)])
def test_heads_are_normed_then_turned_and_cached(dtype, heads, kv_heads, slot, dim, rot_dims, interleaved):
    """Queries in place, keys into the key pages, values into the value pages, against the plain norm and rotation;
    heads padded behind ``dim``, sizes with and without a factor of four (two kernels), rows that are column blocks
    of a wider matrix, a second call that prepares queries only."""
    from types import SimpleNamespace

    from pagedserve_b200.kernels.ops import Ops

    compute = TORCH_DTYPE[dtype]
    ops = Ops(compute)
    g = torch.Generator().manual_seed(heads * 100 + slot)
    T, page, pages = 37, 8, 12
    qw, kw = heads * slot, kv_heads * slot
    projected = torch.randn(T, qw + 2 * kw, generator=g).to(compute)
    base = 10000.0
    freq = base ** (-2.0 * torch.arange(rot_dims // 2, dtype=torch.float64) / max(rot_dims, 1))
    inv_freq = torch.stack([freq.float(), (freq - freq.float().double()).float()], dim=1).contiguous().to(DEV)
    q_gain, k_gain = 1.0 + 0.2 * torch.randn(dim, generator=g), 1.0 + 0.2 * torch.randn(dim, generator=g)
    positions = torch.tensor([5 + 3 * t if t < 20 else 700 + t for t in range(T)], dtype=torch.int32)
    # two requests: tokens 0..19 of slot 1, the rest of slot 0; table rows by slot
    token_slot = torch.tensor([1] * 20 + [0] * 17, dtype=torch.int32)
    table = torch.full((2, 128), -1, dtype=torch.int32)
    order = torch.randperm(pages, generator=g).tolist()
    need = {(int(s), int(p) // page) for s, p in zip(token_slot, positions)}
    assert len(need) <= pages
    for number, (s, index) in enumerate(sorted(need)):
        table[s, index] = order[number]
    pool = torch.zeros(pages, 2, kv_heads, page, slot, dtype=compute, device=DEV)
    layer = SimpleNamespace(k_pool=pool[:, 0], v_pool=pool[:, 1], page_stride=pool.stride(0), page_size=page,
                            block_table=table.to(DEV))
    ctx = SimpleNamespace(token_slot=token_slot.to(DEV), positions=positions.to(DEV))
    device_rows = projected.to(DEV)
    q, k, v = device_rows[:, :qw], device_rows[:, qw:qw + kw], device_rows[:, qw + kw:]
    ops.head_norm_rotary_cache_write(q, k, v, q_gain.to(DEV), k_gain.to(DEV), 1e-5, inv_freq, rot_dims, interleaved, dim,
                                     ctx, layer, heads, kv_heads, slot)

    def plain_heads(rows, count, gain):
        x = rows.double().reshape(T, count, slot)
        normed = plain.rms_norm(x[..., :dim], gain.double(), 1e-5)
        if interleaved:                              # neighbours paired: the halves layout on reordered numbers
            turning = torch.cat([normed[..., 0:rot_dims:2], normed[..., 1:rot_dims:2]], -1)
            turned = plain.rotate_halves(turning, positions.long(), rot_dims, base)
            normed = normed.clone()
            normed[..., 0:rot_dims:2], normed[..., 1:rot_dims:2] = turned[..., :rot_dims // 2], turned[..., rot_dims // 2:]
        else:
            normed = plain.rotate_halves(normed, positions.long(), rot_dims, base)
        return torch.cat([normed, x[..., dim:]], -1)

    tol = 2e-6 if dtype == "float32" else 1e-2
    want_q = plain_heads(projected[:, :qw], heads, q_gain)
    assert rel_err(q.reshape(T, heads, slot), want_q) < tol
    want_k = plain_heads(projected[:, qw:qw + kw], kv_heads, k_gain)
    want_v = projected[:, qw + kw:].reshape(T, kv_heads, slot)
    cached = pool.cpu()
    for t in range(T):
        at = cached[int(table[int(token_slot[t]), int(positions[t]) // page]), :, :, int(positions[t]) % page]
        assert rel_err(at[0], want_k[t]) < tol, t
        assert torch.equal(at[1], want_v[t]), t
    assert torch.equal(device_rows[:, qw:].cpu(), projected[:, qw:])                 # keys and values as projected
    # queries only (a layer that reads another layer's pages): nothing else is touched
    before = pool.clone()
    again = projected[:, :qw].to(DEV).contiguous()
    ops.head_norm_rotary_cache_write(again, None, None, q_gain.to(DEV), None, 1e-5, inv_freq, rot_dims, interleaved, dim,
                                     ctx, layer, heads, kv_heads, slot)
    assert rel_err(again.reshape(T, heads, slot), want_q) < tol and torch.equal(pool, before)
