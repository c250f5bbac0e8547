"""Pagatar as a ModelSpec.

Token table, normed in groups -> layers in the listed order -> the model's norm -> logits against the token table.
Every layer is :class:`PostNormBlock`: the sublayers read the residual rows themselves, their results are normed
(RMS norm in groups, plain gain) and added, and the layer ends with a learned average over the embedded rows and all
layers' results so far.  ``mingru`` layers are :class:`MinGRUMixer`; ``latent_attention`` layers
:class:`LatentAttention` with queries through a normed latent, no window and one sigmoid gate per head; ``attention``
layers :class:`RotaryAttention` with biased projections, a short convolution on q, k and v, head norms, a halves-paired
(and possibly stretched) rotation, a chunked mask, values blended with the first such layer's, and a sigmoid gate on
the joined heads.  The feed-forward is :class:`RoutedExperts` with sigmoid scores, an election correction, weights that
are the scores themselves and silu experts, or none.

Tensor names in a checkpoint: ``embed``, ``embed.norm``, ``final.norm``, and per layer i ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.dwa``, ``l<i>.mix.*``, ``l<i>.mlp.router``, ``l<i>.mlp.correction``,
``l<i>.mlp.e<n>.{gate,up,down}``; matrices are stored ``[out, in]``.
"""

from __future__ import annotations

import re
from typing import Optional

from pagedserve_b200.config.pagatar import PagatarConfig
from pagedserve_b200.config.registry import register_architecture
from pagedserve_b200.models.spec import LayerSpec, ModelSpec, PartSpec

# parts shared with other models name their tensors "<name>.weight"; this design stores the bare name
_BARE = re.compile(r"^(embed|embed\.norm|final\.norm|l\d+\.(norm1|norm2))$")
_SUFFIX = ".weight"
# the step's shared rows in which the first value-mixing layer leaves its values
FIRST_VALUES = "first_values"


def _normalise_name(name: str) -> Optional[str]:
    return name + _SUFFIX if _BARE.match(name) else name


def _checkpoint_name(name: str) -> str:
    if name.endswith(_SUFFIX) and _BARE.match(name[:-len(_SUFFIX)]):
        return name[:-len(_SUFFIX)]
    return name


def build_pagatar_spec(config: PagatarConfig) -> ModelSpec:
    width = config.width
    norm = dict(width=width, eps=config.norm_eps, groups=config.norm_groups, init_std=0.1)
    width_std = width ** -0.5
    layers = []
    mixes_seen = False
    for index, entry in enumerate(config.layers):
        prefix = f"l{index}."
        mixer = entry["mixer"]
        if entry["type"] == "mingru":
            mixer_spec = PartSpec("mingru", dict(hidden_size=width, width=mixer["width"], init_std=width_std,
                                                 out_init_std=mixer["width"] ** -0.5), prefix + "mix.")
        elif entry["type"] == "latent_attention":
            inner = mixer["heads"] * mixer["vdim"]
            mixer_spec = PartSpec("latent_attention", dict(
                hidden_size=width, n_heads=mixer["heads"], flat_dim=mixer["dim"], rot_dim=mixer["rot_dim"],
                v_dim=mixer["vdim"], kv_rank=mixer["kv_rank"], q_rank=mixer["q_rank"], gate="head",
                scale=mixer["scale"], window=None, eps=config.norm_eps,
                rotary=dict(dims=mixer["rot"]["dims"], base=mixer["rot"]["base"]),
                init_std=width_std, out_init_std=inner ** -0.5), prefix + "mix.")
        else:
            rot = mixer.get("rot")
            value_mix = None
            if mixer["v_mix"]:
                value_mix = dict(name="mix.vmix", role="later" if mixes_seen else "first", key=FIRST_VALUES)
                mixes_seen = True
            mixer_spec = PartSpec("rotary_attention", dict(
                hidden_size=width, n_heads=mixer["heads"], n_kv_heads=mixer["kv_heads"], head_dim=mixer["dim"],
                v_dim=mixer["vdim"], scale=mixer["scale"], window=None,
                chunk=mixer["mask"]["size"] if mixer.get("mask") else None, softcap=None,
                rotary=dict(dims=rot["dims"], base=rot["base"], interleaved=False,
                            scaling=rot.get("scaling")) if rot else None,
                q_name="mix.q", k_name="mix.k", v_name="mix.v", out_name="mix.o", sink_name=None, bias=True,
                head_norm=dict(q_name="mix.q.norm", k_name="mix.k.norm", eps=config.norm_eps),
                conv=dict(taps=mixer["conv"], suffix=".conv") if mixer.get("conv") else None, value_mix=value_mix,
                gate_name="mix.g",
                init_std=width_std, out_init_std=(mixer["heads"] * mixer["vdim"]) ** -0.5), prefix)
        norms = {"post_mixer": PartSpec("group_rms_norm", dict(norm, name="norm1"), prefix)}
        mlp = entry["mlp"]
        if mlp is None:
            feed_forward = PartSpec("none")
        else:
            norms["post_feed_forward"] = PartSpec("group_rms_norm", dict(norm, name="norm2"), prefix)
            feed_forward = PartSpec("routed_experts", dict(
                hidden_size=width, n_experts=mlp["router"]["experts"], expert_ff=mlp["expert"]["ff"],
                top=mlp["router"]["top"], groups=0, group_keep=0, shared_ff=None, score="sigmoid", normalize=False,
                correction_name="correction", init_std=width_std, out_init_std=mlp["expert"]["ff"] ** -0.5),
                prefix + "mlp.")
        block = PartSpec("post_norm", dict(depth=dict(index=index, name="dwa", entries=len(config.layers) + 1)), prefix)
        layers.append(LayerSpec(block, mixer_spec, feed_forward, norms))
    return ModelSpec(
        architecture=config.architecture,
        hidden_size=width,
        vocab_size=config.vocab,
        max_model_len=config.max_model_len,
        embedding=PartSpec("normed_token_embedding", dict(
            vocab_size=config.vocab, hidden_size=width, name="embed", init_std=1.0,
            norm=dict(name="embed.norm", eps=config.norm_eps, groups=config.norm_groups, init_std=0.1))),
        positions=PartSpec("none"),
        layers=layers,
        schedule=[],
        final_norm=PartSpec("group_rms_norm", dict(norm, name="final.norm")),
        head=PartSpec("lm_head", dict(vocab_size=config.vocab, hidden_size=width, tied=True, tied_to="embed.weight",
                                      name="lm_head", init_std=1.0)),
        normalise_name=_normalise_name,
        checkpoint_name=_checkpoint_name,
    )


register_architecture("Pagatar", PagatarConfig, build_pagatar_spec, replace=True)
