"""Pagatar, plainly: whole sequences, no cache, no batching, one function per mechanism.

Everything here is written from the design's equations for the tests to compare the engine
with; it shares no code with the package.  ``tensors`` maps checkpoint names to tensors,
``config`` is the parsed config.json.  Arithmetic runs in ``dtype`` (float64 unless told
otherwise).

Notation: T tokens, W the model's width, H query heads, G key/value heads, d a head's
query/key size, e its value size, p_t the position of token t (0 for the first token of a
sequence), C the size of a chunk of the mask, R the size of a latent.
"""

import math

import torch


# ------------------------------------------------------------------------------- norms
def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis (plain gain)."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def group_rms_norm(x, w, eps, groups):
    """The last axis in ``groups`` equal runs, each divided by its own root mean square; then the gain."""
    shape = x.shape
    parts = x.reshape(*shape[:-1], groups, shape[-1] // groups)
    parts = parts / torch.sqrt((parts * parts).mean(-1, keepdim=True) + eps)
    return parts.reshape(shape) * w


# ------------------------------------------------------------------------------- rotations
def turn_pairs(first, second, angle, amplitude=1.0):
    cos, sin = torch.cos(angle) * amplitude, torch.sin(angle) * amplitude
    return first * cos - second * sin, second * cos + first * sin


def rotate_neighbours(x, positions, dims, base):
    """x [T, ..., n]: numbers 2i and 2i + 1 (i < dims / 2) turn together by p * base^(-2i/dims)."""
    if not dims:
        return x
    i = torch.arange(dims // 2, dtype=x.dtype)
    angle = positions.to(x.dtype)[:, None] * base ** (-2.0 * i / dims)[None, :]
    while angle.dim() < x.dim():
        angle = angle[:, None]
    out = x.clone()
    out[..., 0:dims:2], out[..., 1:dims:2] = turn_pairs(x[..., 0:dims:2], x[..., 1:dims:2], angle)
    return out


def stretched_frequencies(dims, base, scaling, dtype):
    """(frequencies [dims / 2], amplitude): base^(-2i/dims), and with ``scaling`` (factor, original, fast, slow)
    the blend f / factor * ramp + f * (1 - ramp), ramp rising from 0 at index lo to 1 at index hi, where
    index(t) = dims * ln(original / (2 pi t)) / (2 ln base), lo = max(floor(index(fast)), 0),
    hi = min(ceil(index(slow)), dims - 1); the amplitude 0.1 ln(factor) + 1 multiplies sines and cosines."""
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    index = lambda t: dims * math.log(scaling["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo = max(math.floor(index(scaling["fast"])), 0)
    hi = min(math.ceil(index(scaling["slow"])), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / scaling["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(scaling["factor"]) + 1.0


def rotate_halves(x, positions, dims, base, scaling=None):
    """x [T, heads, d]: numbers i and i + dims / 2 (i < dims / 2) turn together; the rest stays."""
    if not dims:
        return x
    half = dims // 2
    freq, amplitude = stretched_frequencies(dims, base, scaling, x.dtype)
    angle = (positions.to(x.dtype)[:, None] * freq[None, :])[:, None, :]
    out = x.clone()
    out[..., :half], out[..., half:dims] = turn_pairs(x[..., :half], x[..., half:dims], angle, amplitude)
    return out


# ------------------------------------------------------------------------------- masks and softmax
def causal_mask(positions, chunk=None):
    """True where the query at positions[i] may see the key at positions[j]: j not later and, with ``chunk``,
    both in the same run of that many positions counted from position 0."""
    i, j = positions[:, None], positions[None, :]
    seen = j <= i
    if chunk:
        seen = seen & (torch.div(i, chunk, rounding_mode="floor") == torch.div(j, chunk, rounding_mode="floor"))
    return seen


def masked_softmax(scores, mask):
    s = scores.masked_fill(~mask[None], float("-inf"))
    s = s - s.max(-1, keepdim=True).values
    e = torch.exp(s)
    return e / e.sum(-1, keepdim=True)


# ------------------------------------------------------------------------------- mixers
def min_gru(tensors, prefix, m, h):
    """z = sigmoid(W_z h + b_z); u = W_x h + b_x; candidate = u + 1/2 (u >= 0) or sigmoid(u) (u < 0);
    S_t = (1 - z_t) S_(t-1) + z_t candidate_t from S = 0; out = W_o (S_t * silu(W_g h))."""
    t = lambda name: tensors[prefix + "mix." + name].to(h.dtype)
    z = torch.sigmoid(h @ t("z").T + t("z.b"))
    u = h @ t("x").T + t("x.b")
    candidate = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    gate = torch.nn.functional.silu(h @ t("g").T)
    state = torch.zeros(m["width"], dtype=h.dtype)
    rows = []
    for step in range(h.shape[0]):
        state = (1.0 - z[step]) * state + z[step] * candidate[step]
        rows.append(state)
    return (torch.stack(rows) * gate) @ t("o").T


def latent_attention(tensors, prefix, m, h, positions, eps):
    """Queries through a normed latent, keys and values of all heads from one normed latent per token, one
    turning key part for all heads, a sigmoid gate per head."""
    H, d, r, e, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    t = lambda name: tensors[prefix + "mix." + name].to(h.dtype)
    q = (rms_norm(h @ t("dq").T, t("dq.norm"), eps) @ t("uq").T).reshape(T, H, d + r)
    down = h @ t("dkv").T
    c = rms_norm(down[:, :R], t("dkv.norm"), eps)
    dims, base = m["rot"]["dims"], m["rot"]["base"]
    k_turn = rotate_neighbours(down[:, R:], positions, dims, base)                   # [T, r]
    q_turn = rotate_neighbours(q[..., d:], positions, dims, base)                    # [T, H, r]
    k_flat = (c @ t("uk").T).reshape(T, H, d)
    v = (c @ t("uv").T).reshape(T, H, e)
    s = (torch.einsum("ihd,jhd->hij", q[..., :d], k_flat) + torch.einsum("ihr,jr->hij", q_turn, k_turn)) * m["scale"]
    p = masked_softmax(s, causal_mask(positions))
    o = torch.einsum("hij,jhe->ihe", p, v)
    o = o * torch.sigmoid(h @ t("g").T)[:, :, None]
    return o.reshape(T, H * e) @ t("o").T


def short_convolution(u, w):
    """u [T, channels], w [channels, taps]: y_t = sum_j w[:, j] * u_(t - taps + 1 + j), zeros before the start."""
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, u.shape[1], dtype=u.dtype), u])
    return sum(padded[j:j + u.shape[0]] * w[:, j] for j in range(taps))


def projected(tensors, prefix, m, h, name):
    """A biased projection of an attention layer, convolved over time where the layer has a convolution."""
    t = lambda leaf: tensors[prefix + "mix." + leaf].to(h.dtype)
    u = h @ t(name).T + t(name + ".b")
    return short_convolution(u, t(name + ".conv")) if m.get("conv") else u


def attention_values(tensors, prefix, m, h):
    """The values of an attention layer as projected and convolved, before any mixing: [T, G * e]."""
    return projected(tensors, prefix, m, h, "v")


def gated_attention(tensors, prefix, m, h, positions, eps, first_values=None):
    """Biased projections, short convolutions, head norms, halves-paired stretched rotation, chunked mask, values
    blended with ``first_values`` (those of the first layer that mixes values), a sigmoid gate on the joined
    heads.  Returns (output, this layer's values before blending)."""
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    t = lambda name: tensors[prefix + "mix." + name].to(h.dtype)
    q = projected(tensors, prefix, m, h, "q").reshape(T, H, d)
    k = projected(tensors, prefix, m, h, "k").reshape(T, G, d)
    own = attention_values(tensors, prefix, m, h)
    v = own
    if first_values is not None:
        mix = t("vmix")
        v = (1.0 - mix) * v + mix * first_values
    v = v.reshape(T, G, e)
    q = rms_norm(q, t("q.norm"), eps)
    k = rms_norm(k, t("k.norm"), eps)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = rotate_halves(q, positions, rot["dims"], rot["base"], rot.get("scaling"))
    k = rotate_halves(k, positions, rot["dims"], rot["base"], rot.get("scaling"))
    k = k.repeat_interleave(H // G, dim=1)                                 # query head j uses kv head j // (H / G)
    v = v.repeat_interleave(H // G, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    p = masked_softmax(s, causal_mask(positions, (m.get("mask") or {}).get("size")))
    o = torch.einsum("hij,jhe->ihe", p, v).reshape(T, H * e)
    o = o * torch.sigmoid(h @ t("g").T)
    return o @ t("o").T, own


# ------------------------------------------------------------------------------- feed-forward
def expert(tensors, prefix, h):
    """W_down (silu(W_gate h) * (W_up h))."""
    t = lambda name: tensors[prefix + name].to(h.dtype)
    return (torch.nn.functional.silu(h @ t("gate").T) * (h @ t("up").T)) @ t("down").T


def router_election(tensors, prefix, h, top):
    """(chosen [T, top], weights [T, top], margin [T]): s = sigmoid(W_router h); the ``top`` largest of
    s + correction stand (ties: lower index), their weights are their own s; ``margin`` is the gap of the
    choice scores between the last chosen and the first unchosen expert."""
    s = torch.sigmoid(h @ tensors[prefix + "router"].to(h.dtype).T)
    choice = s + tensors[prefix + "correction"].to(h.dtype)
    order = torch.argsort(choice, dim=-1, descending=True, stable=True)
    chosen = order[:, :top]
    weights = torch.gather(s, 1, chosen)
    if top < s.shape[1]:
        ranked = torch.gather(choice, 1, order)
        margin = ranked[:, top - 1] - ranked[:, top]
    else:
        margin = torch.full((h.shape[0],), float("inf"), dtype=h.dtype)
    return chosen, weights, margin


def routed_ff(tensors, prefix, mlp, h, margins=None):
    chosen, weights, margin = router_election(tensors, prefix, h, mlp["router"]["top"])
    if margins is not None:
        margins.append(margin)
    out = torch.zeros_like(h)
    for e in range(mlp["router"]["experts"]):
        rows, places = torch.nonzero(chosen == e, as_tuple=True)
        if rows.numel():
            out[rows] += weights[rows, places][:, None] * expert(tensors, f"{prefix}e{e}.", h[rows])
    return out


# ------------------------------------------------------------------------------- the model
def forward(tensors, config, tokens, dtype=torch.float64, layers_out=None, margins=None):
    """Logits [T, vocab] of one whole sequence.  ``layers_out``: a list that receives the residual rows behind
    every layer; ``margins``: a list that receives every router's margins."""
    eps, groups = config["norm"]["eps"], config["norm"]["groups"]
    t = lambda name: tensors[name].to(dtype)
    ids = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(ids))
    x = group_rms_norm(t("embed")[ids], t("embed.norm"), eps, groups)
    history = [x]
    first_values = None
    for index, layer in enumerate(config["layers"]):
        prefix = f"l{index}."
        m = layer["mixer"]
        if layer["type"] == "mingru":
            y = min_gru(tensors, prefix, m, x)
        elif layer["type"] == "latent_attention":
            y = latent_attention(tensors, prefix, m, x, positions, eps)
        else:
            mixes = bool(m.get("v_mix"))
            y, own = gated_attention(tensors, prefix, m, x, positions, eps, first_values if mixes else None)
            if mixes and first_values is None:
                first_values = own
        x = x + group_rms_norm(y, t(prefix + "norm1"), eps, groups)
        if layer.get("mlp") is not None:
            x = x + group_rms_norm(routed_ff(tensors, prefix + "mlp.", layer["mlp"], x, margins),
                                   t(prefix + "norm2"), eps, groups)
        history.append(x)
        weights = t(prefix + "dwa")
        x = sum(weights[j] * history[j] for j in range(len(history)))
        if layers_out is not None:
            layers_out.append(x)
    x = group_rms_norm(x, t("final.norm"), eps, groups)
    return x @ t("embed").T


def read_folder(folder, dtype=torch.float64):
    """(tensors, config) of a model folder; the safetensors file is read here, byte by byte."""
    import json
    import os
    import struct

    import numpy as np

    with open(os.path.join(folder, "config.json")) as handle:
        config = json.load(handle)
    with open(os.path.join(folder, "model.safetensors"), "rb") as handle:
        size = struct.unpack("<Q", handle.read(8))[0]
        header = json.loads(handle.read(size))
        data = handle.read()
    tensors = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        lo, hi = entry["data_offsets"]
        raw = np.frombuffer(data[lo:hi], dtype=np.uint8)
        if entry["dtype"] == "BF16":
            wide = np.zeros(raw.size // 2, dtype=np.uint32)
            wide[:] = raw.view(np.uint16)
            value = torch.from_numpy((wide << 16).view(np.float32).copy())
        elif entry["dtype"] == "F32":
            value = torch.from_numpy(raw.view(np.float32).copy())
        elif entry["dtype"] == "I32":
            value = torch.from_numpy(raw.view(np.int32).copy())
        else:
            raise ValueError(f"{name}: dtype {entry['dtype']}")
        tensors[name] = value.reshape(entry["shape"]).to(dtype) if value.is_floating_point() else value.reshape(entry["shape"])
    return tensors, config


# ------------------------------------------------------------------------------- random models for the tests
def tensor_shapes(config):
    """{checkpoint name: shape} of a model of ``config``."""
    W, V = config["width"], config["vocab"]
    shapes = {"embed": (V, W), "embed.norm": (W,), "final.norm": (W,)}
    for index, layer in enumerate(config["layers"]):
        p, m = "l%d." % index, layer["mixer"]
        shapes[p + "norm1"] = (W,)
        shapes[p + "dwa"] = (index + 2,)
        if layer["type"] == "mingru":
            n = m["width"]
            shapes.update({p + "mix.z": (n, W), p + "mix.z.b": (n,), p + "mix.x": (n, W), p + "mix.x.b": (n,),
                           p + "mix.g": (n, W), p + "mix.o": (W, n)})
        elif layer["type"] == "latent_attention":
            H, d, r, e, R, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            shapes.update({p + "mix.dq": (Q, W), p + "mix.dq.norm": (Q,), p + "mix.uq": (H * (d + r), Q),
                           p + "mix.dkv": (R + r, W), p + "mix.dkv.norm": (R,), p + "mix.uk": (H * d, R),
                           p + "mix.uv": (H * e, R), p + "mix.g": (H, W), p + "mix.o": (W, H * e)})
        else:
            H, G, d, e, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m.get("conv")
            for name, rows in (("q", H * d), ("k", G * d), ("v", G * e)):
                shapes[p + "mix." + name] = (rows, W)
                shapes[p + "mix." + name + ".b"] = (rows,)
                if taps:
                    shapes[p + "mix." + name + ".conv"] = (rows, taps)
            shapes.update({p + "mix.q.norm": (d,), p + "mix.k.norm": (d,), p + "mix.g": (H * e, W),
                           p + "mix.o": (W, H * e)})
            if m.get("v_mix"):
                shapes[p + "mix.vmix"] = ()
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        shapes[p + "norm2"] = (W,)
        E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
        shapes[p + "mlp.router"] = (E, W)
        shapes[p + "mlp.correction"] = (E,)
        for e in range(E):
            shapes[p + "mlp.e%d.gate" % e] = (ff, W)
            shapes[p + "mlp.e%d.up" % e] = (ff, W)
            shapes[p + "mlp.e%d.down" % e] = (W, ff)
    return shapes


def random_model(config, seed):
    """Random tensors (rounded to bfloat16, stored as such) that keep activations of order one."""
    g = torch.Generator().manual_seed(seed)
    tensors = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.split(".")[-1]
        if name == "embed":
            value = torch.randn(shape, generator=g)
        elif leaf in ("norm1", "norm2", "norm"):
            value = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif leaf == "dwa":
            value = 1.0 / shape[0] + 0.2 * torch.randn(shape, generator=g)
        elif leaf == "b":
            value = 0.5 * torch.randn(shape, generator=g)
        elif leaf == "conv":
            value = torch.randn(shape, generator=g) / math.sqrt(shape[1])
        elif leaf == "vmix":
            value = 0.3 + 0.2 * torch.randn(shape, generator=g)
        elif leaf == "correction":
            value = 0.3 * torch.randn(shape, generator=g)
        elif leaf == "router":
            value = 2.0 * torch.randn(shape, generator=g) / math.sqrt(shape[1])
        else:
            value = torch.randn(shape, generator=g) / math.sqrt(shape[1])
        tensors[name] = value.to(torch.bfloat16)
    return tensors


def moe_mlp(experts=4, top=2, ff=24):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


def mingru_layer(width=48, mlp=None):
    return {"type": "mingru", "mixer": {"width": width}, "mlp": mlp}


def latent_layer(heads=4, dim=16, rot_dim=8, vdim=16, kv_rank=32, q_rank=40, base=10000.0, scale=0.2, mlp=None):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                      "scale": scale, "rot": {"base": base, "dims": rot_dim}}}


def attention_layer(heads=4, kv_heads=2, dim=16, vdim=16, chunk=12, taps=3, rot_dims=None, base=10000.0, scale=0.25,
                    scaling=None, v_mix=True, mlp=None):
    rot = {"base": base, "dims": dim if rot_dims is None else rot_dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot}
    if taps:
        mixer["conv"] = taps
    if chunk:
        mixer["mask"] = {"size": chunk}
    if v_mix:
        mixer["v_mix"] = True
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def make_config(layers, width=64, vocab=97, eps=1e-5, groups=2):
    return {"architecture": "Pagatar", "layers": layers, "norm": {"eps": eps, "groups": groups}, "vocab": vocab,
            "width": width}
