"""Tefopel, plainly: whole sequences, no cache, no batching, one function per mechanism.

Everything here is written from the design's equations for the tests to compare the engine
with; it shares no code with the package.  ``tensors`` maps checkpoint names to tensors,
``config`` is the parsed config.json.  Arithmetic runs in ``dtype`` (float64 unless told
otherwise).

Notation: T tokens, W the model's width, H query heads, G key/value heads, d the per-head
size, p_t the position of token t (0 for the first token of a sequence).
"""

import math

import torch


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_rms_norm(x, w, eps):
    """The layer norm of this design: unit RMS, then a gain that is stored as its distance from one."""
    return rms_unit(x, eps) * (1.0 + w)


def rotate_interleaved(x, positions, dims, base):
    """x [T, heads, d]: the neighbours (2i, 2i+1), i < dims/2, turn by p * base^(-2i/dims); the rest stays."""
    i = torch.arange(dims // 2, dtype=x.dtype)
    freq = base ** (-2.0 * i / dims)
    angle = positions.to(x.dtype)[:, None] * freq[None, :]                # [T, dims/2]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    even, odd = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = even * cos - odd * sin
    out[..., 1:dims:2] = odd * cos + even * sin
    return out


def attention_scores(q, k, scale, softcap):
    """[H, T, T] capped scores of rotated queries [T, H, d] and keys [T, H, d]."""
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    return softcap * torch.tanh(s / softcap)


def window_mask(T, size):
    """True where query i may see key j: 0 <= i - j < size."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (i - j >= 0) & (i - j < size)


def sink_softmax(scores, mask, sink):
    """Softmax over the visible keys of each row with one more term exp(sink_h) in the denominator only."""
    s = scores.masked_fill(~mask[None], float("-inf"))
    top = torch.maximum(s.max(-1, keepdim=True).values, sink[:, None, None])
    e = torch.exp(s - top)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink[:, None, None] - top))


def attention_mixer(tensors, prefix, m, h, positions):
    """h [T, W] -> [T, W].  The values are the keys as projected, before they are turned."""
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    T = h.shape[0]
    t = lambda name: tensors[prefix + "mix." + name].to(h.dtype)
    q = (h @ t("q").T).reshape(T, H, d)
    k = (h @ t("k").T).reshape(T, G, d)
    v = k
    q = rotate_interleaved(q, positions, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_interleaved(k, positions, m["rot"]["dims"], m["rot"]["base"])
    group = H // G
    k = k.repeat_interleave(group, dim=1)                                 # query head j uses kv head j // group
    v = v.repeat_interleave(group, dim=1)
    s = attention_scores(q, k, m["scale"], m["softcap"])
    p = sink_softmax(s, window_mask(T, m["mask"]["size"]), t("sink"))
    o = torch.einsum("hij,jhd->ihd", p, v).reshape(T, H * d)
    return o @ t("o").T


def token_shift(h, mu, first=None):
    """h + (h' - h) * mu, h' the row before (``first`` or zeros before the first row)."""
    before = torch.zeros_like(h[:1]) if first is None else first[None]
    prev = torch.cat([before, h[:-1]], dim=0)
    return h + (prev - h) * mu


def wkv_decay(tensors, prefix, mix_w):
    """[T, heads * d] decay factors in (0, 1): exp(-exp(low-rank(mix_w) + offset))."""
    t = lambda name: tensors[prefix + "mix." + name].to(mix_w.dtype)
    return torch.exp(-torch.exp(torch.tanh(mix_w @ t("w1").T) @ t("w2").T + t("w0")))


def wkv_recurrence(r, k, v, w, u, state=None):
    """Per head, S [d(key), d(value)]: o_t = (S + diag(u) k_t v_t^T)^T r_t ; S <- diag(w_t) S + k_t v_t^T.
    r, k, v, w: [T, heads, d]; u: [heads, d].  Returns (o [T, heads, d], S)."""
    T, heads, d = r.shape
    S = torch.zeros(heads, d, d, dtype=r.dtype) if state is None else state.clone()
    out = []
    for step in range(T):
        kv = k[step][:, :, None] * v[step][:, None, :]                    # [heads, d, d]
        out.append(torch.einsum("hkv,hk->hv", S + u[:, :, None] * kv, r[step]))
        S = w[step][:, :, None] * S + kv
    return torch.stack(out), S


def wkv_mixer(tensors, prefix, m, h, eps):
    heads, d = m["heads"], m["dim"]
    T = h.shape[0]
    t = lambda name: tensors[prefix + "mix." + name].to(h.dtype)
    mixes = {s: token_shift(h, t("mu." + s)) for s in "rkvgw"}
    r = (mixes["r"] @ t("r").T).reshape(T, heads, d)
    k = (mixes["k"] @ t("k").T).reshape(T, heads, d)
    v = (mixes["v"] @ t("v").T).reshape(T, heads, d)
    gate = torch.nn.functional.silu(mixes["g"] @ t("g").T)
    w = wkv_decay(tensors, prefix, mixes["w"]).reshape(T, heads, d)
    o, _ = wkv_recurrence(r, k, v, w, t("u"))
    o = rms_unit(o, eps).reshape(T, heads * d) * t("norm") * gate
    return o @ t("o").T


def squared_relu_ff(tensors, prefix, h):
    t = lambda name: tensors[prefix + "mlp." + name].to(h.dtype)
    return torch.relu(h @ t("up").T) ** 2 @ t("down").T


def weight_owner(config, index):
    return config["layers"][index].get("weights_of", index)


def forward(tensors, config, tokens, dtype=torch.float64, keep_layers=False):
    """Logits [T, vocab] of one sequence (and the stream after every layer if asked)."""
    eps = config["norm"]["eps"]
    t = lambda name: tensors[name].to(dtype)
    ids = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(ids))
    x = t("embed")[ids]
    streams = []
    for index, layer in enumerate(config["layers"]):
        prefix = "l%d." % weight_owner(config, index)
        normed = offset_rms_norm(x, t(prefix + "norm1"), eps)
        if layer["type"] == "attention":
            x = x + attention_mixer(tensors, prefix, layer["mixer"], normed, positions)
        elif layer["type"] == "wkv":
            x = x + wkv_mixer(tensors, prefix, layer["mixer"], normed, eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            x = x + squared_relu_ff(tensors, prefix, offset_rms_norm(x, t(prefix + "norm2"), eps))
        streams.append(x)
    logits = offset_rms_norm(x, t("final.norm"), eps) @ t("embed").T
    return (logits, torch.stack(streams)) if keep_layers else logits


# ------------------------------------------------------------------ random models for the tests
def tensor_shapes(config, rank=8):
    """{checkpoint name: shape} of a model of ``config`` (layers that borrow weights store none); ``rank`` is the
    inner size of the decay's low-rank pair, which only the tensors' shapes carry."""
    W, V = config["width"], config["vocab"]
    shapes = {"embed": (V, W), "final.norm": (W,)}
    for index, layer in enumerate(config["layers"]):
        if "weights_of" in layer:
            continue
        p, m = "l%d." % index, layer["mixer"]
        shapes[p + "norm1"] = (W,)
        if layer["type"] == "attention":
            shapes[p + "mix.q"] = (m["heads"] * m["dim"], W)
            shapes[p + "mix.k"] = (m["kv_heads"] * m["dim"], W)
            shapes[p + "mix.sink"] = (m["heads"],)
            shapes[p + "mix.o"] = (W, m["heads"] * m["vdim"])
        else:
            inner = m["heads"] * m["dim"]
            for s in "rkvgw":
                shapes[p + "mix.mu." + s] = (W,)
            for s in "rkvg":
                shapes[p + "mix." + s] = (inner, W)
            shapes[p + "mix.w1"] = (rank, W)
            shapes[p + "mix.w2"] = (inner, rank)
            shapes[p + "mix.w0"] = (inner,)
            shapes[p + "mix.u"] = (m["heads"], m["dim"])
            shapes[p + "mix.norm"] = (inner,)
            shapes[p + "mix.o"] = (W, inner)
        if layer.get("mlp") is not None:
            shapes[p + "norm2"] = (W,)
            shapes[p + "mlp.up"] = (layer["mlp"]["ff"], W)
            shapes[p + "mlp.down"] = (W, layer["mlp"]["ff"])
    return shapes


def random_model(config, seed, rank=8):
    """Random tensors (rounded to bfloat16, stored as such) that keep activations of order one."""
    g = torch.Generator().manual_seed(seed)
    W = config["width"]
    tensors = {}
    for name, shape in tensor_shapes(config, rank).items():
        leaf = name.split(".")[-1]
        if name == "embed":
            value = torch.randn(shape, generator=g)
        elif leaf in ("norm1", "norm2") or name == "final.norm":
            value = 0.1 * torch.randn(shape, generator=g)
        elif ".mix.mu." in name:
            value = torch.rand(shape, generator=g)
        elif leaf == "sink":
            value = torch.randn(shape, generator=g)
        elif leaf == "w0":
            value = -1.0 + 1.5 * torch.randn(shape, generator=g)          # decays from nearly 1 down to small
        elif leaf == "u":
            value = 0.5 * torch.randn(shape, generator=g)
        elif leaf == "norm":
            value = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif leaf == "w2":
            value = torch.randn(shape, generator=g) / math.sqrt(shape[1])
        else:
            value = torch.randn(shape, generator=g) / math.sqrt(shape[1])
        tensors[name] = value.to(torch.bfloat16)
    return tensors


def attention_layer(heads=4, kv_heads=2, dim=16, window=12, rot_dims=8, base=10000.0, scale=0.25, softcap=20.0,
                    ff=48):
    return {"type": "attention",
            "mixer": {"dim": dim, "vdim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"size": window},
                      "rot": {"base": base, "dims": rot_dims}, "scale": scale, "softcap": softcap},
            "mlp": None if ff is None else {"ff": ff, "kind": "dense"}}


def wkv_layer(heads=2, dim=16, ff=None, weights_of=None):
    layer = {"type": "wkv", "mixer": {"dim": dim, "heads": heads},
             "mlp": None if ff is None else {"ff": ff, "kind": "dense"}}
    if weights_of is not None:
        layer["weights_of"] = weights_of
    return layer


def make_config(layers, width=64, vocab=97, eps=1e-5):
    return {"architecture": "Tefopel", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
