"""Zositar, plainly: whole sequences, no cache, no batching, one function per mechanism.

Everything here is written from the design's equations for the tests to compare the engine
with; it shares no code with the package.  ``tensors`` maps checkpoint names to tensors,
``config`` is the parsed config.json.  Arithmetic runs in ``dtype`` (float64 unless told
otherwise).

Notation: T tokens, W the model's width, H query heads, G key/value heads, d the per-head
query/key size, e the per-head value size, p_t the position of token t (0 for the first
token of a sequence), C the size of a chunk of the mask.
"""

import math

import torch


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis (plain gain)."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def rotate_halves(x, positions, dims, base):
    """x [T, heads, d]: of the first ``dims`` numbers of a head, number i < dims/2 and number i + dims/2 turn
    together by p * base^(-2i/dims); the rest stays."""
    if not dims:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    freq = base ** (-2.0 * i / dims)
    angle = positions.to(x.dtype)[:, None] * freq[None, :]                # [T, half]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    first, second = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = first * cos - second * sin
    out[..., half:dims] = second * cos + first * sin
    return out


def chunk_mask(positions, size):
    """True where the query at positions[i] may see the key at positions[j]: j not later, and both in the same
    run of ``size`` positions counted from position 0 (no size: every earlier key)."""
    i = positions[:, None]
    j = positions[None, :]
    seen = j <= i
    if size:
        seen = seen & (torch.div(i, size, rounding_mode="floor") == torch.div(j, size, rounding_mode="floor"))
    return seen


def masked_softmax(scores, mask):
    s = scores.masked_fill(~mask[None], float("-inf"))
    s = s - s.max(-1, keepdim=True).values
    e = torch.exp(s)
    return e / e.sum(-1, keepdim=True)


def keys_and_values(tensors, prefix, m, h, positions, eps):
    """What an attention layer with projections of its own leaves for itself and for layers that borrow:
    keys [T, G, d] after their norm and turning, values [T, G, e]."""
    G, d, e = m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    t = lambda name: tensors[prefix + "mix." + name].to(h.dtype)
    k = (h @ t("k").T + t("k.b")).reshape(T, G, d)
    v = (h @ t("v").T + t("v.b")).reshape(T, G, e)
    k = rms_norm(k, t("k.norm"), eps)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    return rotate_halves(k, positions, rot["dims"], rot["base"]), v


def attention_mixer(tensors, prefix, m, h, positions, eps, kv):
    """h [T, W] -> [T, W] with the keys and values ``kv`` (the layer's own or a lender's)."""
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    t = lambda name: tensors[prefix + "mix." + name].to(h.dtype)
    q = (h @ t("q").T + t("q.b")).reshape(T, H, d)
    q = rms_norm(q, t("q.norm"), eps)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = rotate_halves(q, positions, rot["dims"], rot["base"])
    k, v = kv
    group = H // G
    k = k.repeat_interleave(group, dim=1)                                 # query head j uses kv head j // group
    v = v.repeat_interleave(group, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    p = masked_softmax(s, chunk_mask(positions, (m.get("mask") or {}).get("size")))
    o = torch.einsum("hij,jhe->ihe", p, v).reshape(T, H * e)
    return o @ t("o").T


def gated_silu_ff(tensors, prefix, h):
    """W_down (silu(W_gate h) * (W_up h))."""
    t = lambda name: tensors[prefix + name].to(h.dtype)
    return (torch.nn.functional.silu(h @ t("gate").T) * (h @ t("up").T)) @ t("down").T


def clamped_expert(tensors, prefix, h, limit):
    """g = min(W_gate h, limit); u = clamp(W_up h, -limit, limit); W_down (g sigmoid(1.702 g) (u + 1))."""
    t = lambda name: tensors[prefix + name].to(h.dtype)
    g = torch.clamp(h @ t("gate").T, max=limit)
    u = torch.clamp(h @ t("up").T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ t("down").T


def router_election(tensors, prefix, h, top):
    """(chosen [T, top], weights [T, top], margin [T]): sigmoid scores of W_router h, the ``top`` largest stand with
    their own scores as weights; ``margin`` is the gap between the last chosen and the first unchosen score
    (infinite when all are chosen)."""
    z = h @ tensors[prefix + "router"].to(h.dtype).T
    s = torch.sigmoid(z)
    order = torch.argsort(s, dim=-1, descending=True, stable=True)
    chosen = order[:, :top]
    weights = torch.gather(s, 1, chosen)
    if top < s.shape[1]:
        margin = weights[:, -1] - torch.gather(s, 1, order[:, top:top + 1])[:, 0]
    else:
        margin = torch.full((h.shape[0],), float("inf"), dtype=h.dtype)
    return chosen, weights, margin


def routed_ff(tensors, prefix, mlp, h, margins=None):
    """sum over the chosen experts of expert(weight * h), plus the shared expert on h itself."""
    chosen, weights, margin = router_election(tensors, prefix, h, mlp["router"]["top"])
    if margins is not None:
        margins.append(margin)
    out = torch.zeros_like(h)
    for row in range(h.shape[0]):
        for index, weight in zip(chosen[row].tolist(), weights[row]):
            out[row] += clamped_expert(tensors, prefix + "e%d." % index, (weight * h[row])[None], mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out = out + clamped_expert(tensors, prefix + "shared.", h, mlp["shared"]["limit"])
    return out


def forward(tensors, config, tokens, dtype=torch.float64, keep_layers=False, margins=None, positions=None):
    """Logits [T, vocab] of one sequence (and the stream after every layer if asked).  ``margins``: a list that
    receives, per layer of experts, how clear every election was."""
    eps = config["norm"]["eps"]
    t = lambda name: tensors[name].to(dtype)
    ids = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(ids)) if positions is None else positions
    x = t("embed")[ids]
    streams, cached = [], {}
    for index, layer in enumerate(config["layers"]):
        prefix = "l%d." % index
        m = layer["mixer"]
        normed = rms_norm(x, t(prefix + "norm1"), eps)
        if m.get("kv_from") is None:
            cached[index] = keys_and_values(tensors, prefix, m, normed, positions, eps)
            kv = cached[index]
        else:
            kv = cached[m["kv_from"]]
        x = x + attention_mixer(tensors, prefix, m, normed, positions, eps, kv)
        mlp = layer.get("mlp")
        if mlp is not None:
            normed = rms_norm(x, t(prefix + "norm2"), eps)
            if mlp["kind"] == "dense":
                x = x + gated_silu_ff(tensors, prefix + "mlp.", normed)
            elif mlp["kind"] == "moe":
                x = x + routed_ff(tensors, prefix + "mlp.", mlp, normed, margins)
            else:
                raise ValueError(mlp["kind"])
        streams.append(x)
    logits = rms_norm(x, t("final.norm"), eps) @ t("head").T
    return (logits, torch.stack(streams)) if keep_layers else logits


# ------------------------------------------------------------------ random models for the tests
def tensor_shapes(config):
    """{checkpoint name: shape} of a model of ``config`` (layers that borrow keys and values store none of theirs)."""
    W, V = config["width"], config["vocab"]
    shapes = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    for index, layer in enumerate(config["layers"]):
        p, m = "l%d." % index, layer["mixer"]
        shapes[p + "norm1"] = (W,)
        shapes[p + "mix.q"] = (m["heads"] * m["dim"], W)
        shapes[p + "mix.q.b"] = (m["heads"] * m["dim"],)
        shapes[p + "mix.q.norm"] = (m["dim"],)
        if m.get("kv_from") is None:
            shapes[p + "mix.k"] = (m["kv_heads"] * m["dim"], W)
            shapes[p + "mix.k.b"] = (m["kv_heads"] * m["dim"],)
            shapes[p + "mix.v"] = (m["kv_heads"] * m["vdim"], W)
            shapes[p + "mix.v.b"] = (m["kv_heads"] * m["vdim"],)
            shapes[p + "mix.k.norm"] = (m["dim"],)
        shapes[p + "mix.o"] = (W, m["heads"] * m["vdim"])
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        shapes[p + "norm2"] = (W,)
        if mlp["kind"] == "dense":
            blocks = [("", mlp["ff"])]
        else:
            shapes[p + "mlp.router"] = (mlp["router"]["experts"], W)
            blocks = [("e%d." % e, mlp["expert"]["ff"]) for e in range(mlp["router"]["experts"])]
            if mlp.get("shared"):
                blocks.append(("shared.", mlp["shared"]["ff"]))
        for name, ff in blocks:
            shapes[p + "mlp." + name + "gate"] = (ff, W)
            shapes[p + "mlp." + name + "up"] = (ff, W)
            shapes[p + "mlp." + name + "down"] = (W, ff)
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
        elif leaf == "b":
            value = 0.3 * torch.randn(shape, generator=g)
        elif leaf == "router":
            value = 2.0 * torch.randn(shape, generator=g) / math.sqrt(shape[1])
        elif leaf in ("gate", "up") and (".mlp.e" in name or ".mlp.shared." in name):
            value = 2.0 * torch.randn(shape, generator=g) / math.sqrt(shape[1])    # so that the limits bite
        else:
            value = torch.randn(shape, generator=g) / math.sqrt(shape[1])
        tensors[name] = value.to(torch.bfloat16)
    return tensors


def attention_layer(heads=4, kv_heads=2, dim=16, vdim=16, chunk=12, rot_dims=8, base=10000.0, scale=0.25,
                    mlp=None, kv_from=None):
    mixer = {"dim": dim, "vdim": vdim, "heads": heads, "kv_heads": kv_heads, "mask": {"size": chunk},
             "rot": {"base": base, "dims": rot_dims}, "scale": scale}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def dense_mlp(ff=48):
    return {"kind": "dense", "ff": ff}


def moe_mlp(experts=4, top=2, ff=24, limit=1.5, shared_ff=32, shared_limit=1.0):
    mlp = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared_ff:
        mlp["shared"] = {"ff": shared_ff, "limit": shared_limit}
    return mlp


def make_config(layers, width=64, vocab=97, eps=1e-5):
    return {"architecture": "Zositar", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
