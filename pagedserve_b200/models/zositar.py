"""Zositar as a ModelSpec.

Token table -> layers in the listed order -> the model's norm -> logits against a head matrix of its own.  Every
layer is pre-norm (h += mixer(norm(h)); h += feed_forward(norm(h)), the second half only where the layer has a
feed-forward); the norm is the RMS form with a plain gain.  The mixer is :class:`RotaryAttention` with biased
projections, a norm per query and key head, halves-paired rotation, a chunked mask and values of their own size; a
layer with ``kv_from`` has no key and value tensors and runs on the cache layer of the layer it names, which has
written the step's keys and values before.  The feed-forward is the gated :class:`DenseMLP`
(W_down (silu(W_gate h) * W_up h)) or :class:`RoutedExperts` with sigmoid scores, weights that are the scores
themselves and scale the experts' inputs, clamped experts and an ungated shared expert.

Tensor names in a checkpoint: ``embed``, ``final.norm``, ``head``, and per layer i ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mix.{q,k,v}`` with ``.b`` biases, ``l<i>.mix.{q,k}.norm``, ``l<i>.mix.o``, ``l<i>.mlp.{gate,up,down}`` or
``l<i>.mlp.router``, ``l<i>.mlp.e<n>.{gate,up,down}``, ``l<i>.mlp.shared.{gate,up,down}``; matrices are stored
``[out, in]``.
"""

from __future__ import annotations

import re
from typing import Optional

from pagedserve_b200.config.registry import register_architecture
from pagedserve_b200.config.zositar import EXPERT_SIGMOID_SLOPE, ZositarConfig
from pagedserve_b200.models.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

# parts shared with other models name their tensors "<name>.weight"; this design stores the bare name
_BARE = re.compile(r"^(embed|head|final\.norm|l\d+\.(norm1|norm2|mlp\.gate|mlp\.up|mlp\.down))$")
_SUFFIX = ".weight"


def _normalise_name(name: str) -> Optional[str]:
    return name + _SUFFIX if _BARE.match(name) else name


def _checkpoint_name(name: str) -> str:
    if name.endswith(_SUFFIX) and _BARE.match(name[:-len(_SUFFIX)]):
        return name[:-len(_SUFFIX)]
    return name


def build_zositar_spec(config: ZositarConfig) -> ModelSpec:
    width = config.width
    norm = dict(width=width, eps=config.norm_eps, has_mean=False, has_bias=False, init_std=0.1)
    width_std = width ** -0.5
    layers, schedule = [], []
    for index, entry in enumerate(config.layers):
        prefix = f"l{index}."
        mixer = entry["mixer"]
        lender = mixer.get("kv_from")
        rot = mixer.get("rot")
        mixer_spec = PartSpec("rotary_attention", dict(
            hidden_size=width, n_heads=mixer["heads"], n_kv_heads=mixer["kv_heads"], head_dim=mixer["dim"],
            v_dim=mixer["vdim"], scale=mixer["scale"], window=None,
            chunk=mixer["mask"]["size"] if mixer.get("mask") else None, softcap=None,
            rotary=dict(dims=rot["dims"], base=rot["base"], interleaved=False) if rot else None,
            q_name="mix.q", k_name="mix.k", v_name="mix.v", out_name="mix.o", sink_name=None, bias=True,
            head_norm=dict(q_name="mix.q.norm", k_name="mix.k.norm", eps=config.norm_eps),
            kv_source=lender is None, init_std=width_std,
            out_init_std=(mixer["heads"] * mixer["vdim"]) ** -0.5), prefix)
        norms = {"pre_mixer": PartSpec("layernorm", dict(norm, name="norm1"), prefix)}
        mlp = entry["mlp"]
        if mlp is None:
            feed_forward = PartSpec("none")
        else:
            norms["pre_feed_forward"] = PartSpec("layernorm", dict(norm, name="norm2"), prefix)
            if mlp["kind"] == "dense":
                feed_forward = PartSpec("dense_mlp", dict(
                    hidden_size=width, inner_size=mlp["ff"], activation="silu", has_bias=False, stored_in_out=False,
                    gate_name="mlp.gate", up_name="mlp.up", down_name="mlp.down", init_std=width_std,
                    out_init_std=mlp["ff"] ** -0.5), prefix)
            else:
                shared = mlp.get("shared")
                feed_forward = PartSpec("routed_experts", dict(
                    hidden_size=width, n_experts=mlp["router"]["experts"], expert_ff=mlp["expert"]["ff"],
                    top=mlp["router"]["top"], groups=0, group_keep=0, shared_ff=shared["ff"] if shared else None,
                    score="sigmoid", normalize=False, shared_gate=False,
                    expert_form=dict(kind="clamped_swish", limit=mlp["expert"]["limit"], alpha=EXPERT_SIGMOID_SLOPE),
                    shared_limit=shared["limit"] if shared else None, init_std=width_std,
                    out_init_std=mlp["expert"]["ff"] ** -0.5), prefix + "mlp.")
        layers.append(LayerSpec(PartSpec("pre_norm"), mixer_spec, feed_forward, norms))
        # a layer that borrows keys and values runs on its lender's cache layer
        schedule.append(ScheduleEntry(index, index if lender is None else lender))
    return ModelSpec(
        architecture=config.architecture,
        hidden_size=width,
        vocab_size=config.vocab,
        max_model_len=config.max_model_len,
        embedding=PartSpec("token_embedding", dict(vocab_size=config.vocab, hidden_size=width, name="embed",
                                                   init_std=1.0)),
        positions=PartSpec("none"),
        layers=layers,
        schedule=schedule,
        final_norm=PartSpec("layernorm", dict(norm, name="final.norm")),
        head=PartSpec("lm_head", dict(vocab_size=config.vocab, hidden_size=width, tied=False, name="head",
                                      init_std=width_std)),
        normalise_name=_normalise_name,
        checkpoint_name=_checkpoint_name,
    )


register_architecture("Zositar", ZositarConfig, build_zositar_spec, replace=True)
