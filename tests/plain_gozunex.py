"""Gozunex, plainly: whole sequences, no cache, no batching, one function per mechanism.

Everything here is written from the design's equations for the tests to compare the engine
with; it shares no code with the package.  ``tensors`` maps checkpoint names to tensors,
``config`` is the parsed config.json.  Arithmetic runs in ``dtype`` (float64 unless told
otherwise).

Notation: T tokens, W the model's width, S residual streams, H heads, d the unrotated and
r the rotated part of a query head, c the latent of a token (size R), E experts, p_t the
position of token t (0 for the first token of a sequence).
"""

import math

import torch


# ------------------------------------------------------------------------------- small pieces
def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def rotate_pairs(x, positions, dims, base):
    """x [..., T, n]: neighbours (2i, 2i+1), i < dims/2, turn by p_t * base^(-2i/dims); x's axis -2 is T when
    ``x`` is [T, n], or axis 0 when [T, H, n]."""
    i = torch.arange(dims // 2, dtype=x.dtype)
    freq = base ** (-2.0 * i / dims)
    angle = positions.to(x.dtype)[:, None] * freq[None, :]                # [T, dims/2]
    cos, sin = torch.cos(angle), torch.sin(angle)
    while cos.dim() < x.dim():
        cos, sin = cos[:, None], sin[:, None]
    even, odd = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = even * cos - odd * sin
    out[..., 1:dims:2] = odd * cos + even * sin
    return out


def window_mask(T, size):
    """True where query i may see key j: 0 <= i - j (< size, if there is a size)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = i - j >= 0
    if size is not None:
        seen = seen & (i - j < size)
    return seen


# ------------------------------------------------------------------------------- embedding
def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the pair table for every token: a hash of (token before, token); the extra last row for t = 0."""
    rows = []
    for t, token in enumerate(tokens):
        rows.append(buckets if t == 0 else (int(tokens[t - 1]) * mul_prev + int(token) * mul_cur) % buckets)
    return rows


def embed(tensors, config, tokens, dtype):
    e = config.get("embedding", {})
    x = tensors["embed"].to(dtype)[list(tokens)] * e.get("scale", 1.0)
    pair = e.get("bigram")
    if pair:
        rows = bigram_rows(tokens, pair["buckets"], pair["mul_prev"], pair["mul_cur"])
        x = x + tensors["bigram"].to(dtype)[rows]
    return x


# ------------------------------------------------------------------------------- latent attention
def latent_attention(tensors, prefix, m, h, positions, eps):
    """h [T, W] -> [T, W].  Keys and values of every head are made from one small vector per token."""
    H, d, r, R, dv = m["heads"], m["dim"], m["rot_dim"], m["kv_rank"], m["vdim"]
    T = h.shape[0]
    t = lambda name: tensors[prefix + "mix." + name].to(h.dtype)
    q = (h @ t("q").T).reshape(T, H, d + r)
    q_flat, q_turn = q[..., :d], q[..., d:]
    down = h @ t("dkv").T                                                  # [T, R + r]
    c = rms_norm(down[:, :R], t("dkv.norm"), eps)
    k_turn = down[:, R:]                                                   # one for all heads
    k_flat = (c @ t("uk").T).reshape(T, H, d)
    v = (c @ t("uv").T).reshape(T, H, dv)
    dims, base = m["rot"]["dims"], m["rot"]["base"]
    q_turn = rotate_pairs(q_turn, positions, dims, base)
    k_turn = rotate_pairs(k_turn, positions, dims, base)
    s = (torch.einsum("ihd,jhd->hij", q_flat, k_flat) + torch.einsum("ihr,jr->hij", q_turn, k_turn)) * m["scale"]
    size = m["mask"]["size"] if m.get("mask") else None
    s = s.masked_fill(~window_mask(T, size)[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.einsum("hij,jhd->ihd", p, v).reshape(T, H * dv)
    o = o * torch.sigmoid(h @ t("g").T)
    return o @ t("o").T


# ------------------------------------------------------------------------------- wkv
def token_shift(h, mu, before=None):
    """h + (h' - h) * mu with h' the row before (``before`` or zeros for the first)."""
    first = torch.zeros_like(h[:1]) if before is None else before[None]
    prev = torch.cat([first, h[:-1]], dim=0)
    return h + (prev - h) * mu


def wkv_decay(tensors, prefix, mix_w):
    t = lambda name: tensors[prefix + "mix." + name].to(mix_w.dtype)
    return torch.exp(-torch.exp(torch.tanh(mix_w @ t("w1").T) @ t("w2").T + t("w0")))


def wkv_scan(r, k, v, w, u, state=None):
    """Per head: y_t = (S + diag(u) k_t v_t^T)^T r_t, then S <- diag(w_t) S + k_t v_t^T.  r, k, v, w [T, H, d];
    u [H, d]; returns y [T, H, d] and the last S [H, d, d] (key channel x value channel)."""
    T, H, d = r.shape
    S = torch.zeros(H, d, d, dtype=r.dtype) if state is None else state.clone()
    ys = []
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        ys.append(torch.einsum("hkv,hk->hv", S + u[:, :, None] * kv, r[t]))
        S = w[t][:, :, None] * S + kv
    return torch.stack(ys), S


def wkv_mixer(tensors, prefix, m, h, eps):
    H, d = m["heads"], m["dim"]
    T = h.shape[0]
    t = lambda name: tensors[prefix + "mix." + name].to(h.dtype)
    mixes = {s: token_shift(h, t("mu." + s)) for s in "rkvgw"}
    r = (mixes["r"] @ t("r").T).reshape(T, H, d)
    k = (mixes["k"] @ t("k").T).reshape(T, H, d)
    v = (mixes["v"] @ t("v").T).reshape(T, H, d)
    gate = silu(mixes["g"] @ t("g").T)
    w = wkv_decay(tensors, prefix, mixes["w"]).reshape(T, H, d)
    y, _ = wkv_scan(r, k, v, w, t("u").reshape(H, d))
    y = rms_unit(y, eps).reshape(T, H * d) * t("norm") * gate
    return y @ t("o").T


# ------------------------------------------------------------------------------- feed-forward
def gated_expert(tensors, prefix, h):
    t = lambda name: tensors[prefix + name].to(h.dtype)
    return (silu(h @ t("gate").T) * (h @ t("up").T)) @ t("down").T


def route(scores, top, group_count=None, group_keep=None, margins=None):
    """scores [T, E] -> (chosen [T, top], weights [T, top]).  With groups: a group's mark is its best score and only
    experts of the ``group_keep`` best groups stand for election.  ``margins`` (a list) receives, per token, how
    clear the election was: the smallest relative gap between the last one in and the first one left out."""
    T, E = scores.shape
    allowed = torch.ones_like(scores, dtype=torch.bool)
    clear = torch.full((T,), float("inf"), dtype=scores.dtype)
    if group_count:
        per = E // group_count
        marks = scores.reshape(T, group_count, per).max(-1).values
        kept = marks.topk(group_keep, dim=-1).indices
        group_ok = torch.zeros(T, group_count, dtype=torch.bool)
        group_ok.scatter_(1, kept, True)
        allowed = group_ok[:, :, None].expand(T, group_count, per).reshape(T, E)
        if group_keep < group_count:
            ranked = marks.sort(-1, descending=True).values
            clear = torch.minimum(clear, (ranked[:, group_keep - 1] - ranked[:, group_keep]) / ranked[:, group_keep - 1])
    standing = scores.masked_fill(~allowed, float("-inf"))
    chosen = standing.topk(top, dim=-1).indices
    if top < int(allowed.sum(-1).min()):
        ranked = standing.sort(-1, descending=True).values
        clear = torch.minimum(clear, (ranked[:, top - 1] - ranked[:, top]) / ranked[:, top - 1])
    if margins is not None:
        margins.append(clear)
    picked = scores.gather(1, chosen)
    return chosen, picked / (picked.sum(-1, keepdim=True) + 1e-20)


def moe(tensors, prefix, mlp, h, margins=None):
    rt = mlp["router"]
    E = rt["experts"]
    scores = torch.softmax(h @ tensors[prefix + "mlp.router"].to(h.dtype).T, dim=-1)
    groups = rt.get("groups") or {}
    chosen, weights = route(scores, rt["top"], groups.get("count"), groups.get("keep"), margins)
    out = torch.zeros_like(h)
    for e in range(E):
        rows, slot = (chosen == e).nonzero(as_tuple=True)
        if rows.numel():
            out[rows] += weights[rows, slot][:, None] * gated_expert(tensors, f"{prefix}mlp.e{e}.", h[rows])
    if mlp.get("shared"):
        gate = torch.sigmoid(h @ tensors[prefix + "mlp.shared.sg"].to(h.dtype).T)          # [T, 1]
        out = out + gate * gated_expert(tensors, prefix + "mlp.shared.", h)
    return out


# ------------------------------------------------------------------------------- layers and the model
def layer_runs(config):
    """Indices of the layers in the order they run: the looped span several times in a row."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(n))
    span = list(range(loop["start"], loop["stop"]))
    return list(range(loop["start"])) + span * loop["times"] + list(range(loop["stop"], n))


def sublayer(tensors, config, index, which, x, positions, margins=None):
    layer = config["layers"][index]
    prefix = f"l{index}."
    eps = config["norm"]["eps"]
    if which == 1:
        h = rms_norm(x, tensors[prefix + "norm1"].to(x.dtype), eps)
        if layer["type"] == "latent_attention":
            return latent_attention(tensors, prefix, layer["mixer"], h, positions, eps)
        return wkv_mixer(tensors, prefix, layer["mixer"], h, eps)
    h = rms_norm(x, tensors[prefix + "norm2"].to(x.dtype), eps)
    return moe(tensors, prefix, layer["mlp"], h, margins)


def forward(tensors, config, tokens, dtype=torch.float64, trace=None, margins=None):
    """Logits [T, V] of one sequence.  ``trace`` (a list) receives the residual stream after every layer run
    (the sum of the streams where there are several); ``margins`` (a list) one tensor [T] per routed
    feed-forward that ran: how clear each token's election of experts was."""
    T = len(tokens)
    positions = torch.arange(T)
    x0 = embed(tensors, config, tokens, dtype)
    S = config.get("streams")
    streams = [x0.clone() for _ in range(S)] if S else None
    x = x0
    for index in layer_runs(config):
        prefix = f"l{index}."
        for which in (1, 2):
            if which == 2 and config["layers"][index].get("mlp") is None:
                continue
            if streams is None:
                x = x + sublayer(tensors, config, index, which, x, positions, margins)
                continue
            t = lambda name: tensors[f"{prefix}hc{which}.{name}"].to(dtype)
            u = sum(t("in")[s] * streams[s] for s in range(S))
            y = sublayer(tensors, config, index, which, u, positions, margins)
            mix, out = t("mix"), t("out")
            streams = [sum(mix[s, j] * streams[s] for s in range(S)) + out[j] * y for j in range(S)]
        if trace is not None:
            trace.append(sum(streams) if streams is not None else x.clone())
    if streams is not None:
        x = sum(streams)
    x = rms_norm(x, tensors["final.norm"].to(dtype), config["norm"]["eps"])
    return x @ tensors["embed"].to(dtype).T


# ------------------------------------------------------------------------------- configurations and random models
def experts_entry(experts, top, ff, shared_ff=None, groups=None, keep=None):
    router = {"experts": experts, "top": top}
    if groups:
        router["groups"] = {"count": groups, "keep": keep}
    entry = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared_ff:
        entry["shared"] = {"ff": shared_ff}
    return entry


def latent_layer(heads, dim, rot_dim, vdim, kv_rank, window, mlp=None, rot_dims=None, base=10000.0, scale=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
             "scale": (dim + rot_dim) ** -0.5 if scale is None else scale,
             "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}
    if window is not None:
        mixer["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def wkv_layer(heads, dim, mlp=None):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim}, "mlp": mlp}


def make_config(layers, width, vocab, eps=1e-5, streams=None, loop=None, scale=1.0, pair=(61, 5, 3)):
    config = {"architecture": "Gozunex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers,
              "embedding": {"scale": scale}}
    if pair is not None:
        config["embedding"]["bigram"] = {"buckets": pair[0], "mul_prev": pair[1], "mul_cur": pair[2]}
    if streams is not None:
        config["streams"] = streams
    if loop is not None:
        config["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return config


def random_model(config, seed, rank=8):
    """Random tensors under the checkpoint's names, rounded to bfloat16 (stored so)."""
    g = torch.Generator().manual_seed(seed)
    W, V = config["width"], config["vocab"]
    out = {}

    def draw(name, shape, std, centre=0.0):
        values = torch.randn(shape, generator=g) * std
        if isinstance(centre, torch.Tensor) or centre:
            values = values + centre
        out[name] = values.to(torch.bfloat16)

    draw("embed", (V, W), 1.0)
    pair = config["embedding"].get("bigram")
    if pair:
        draw("bigram", (pair["buckets"] + 1, W), 0.7)
    draw("final.norm", (W,), 0.1, 1.0)
    S = config.get("streams")
    for index, layer in enumerate(config["layers"]):
        p = f"l{index}."
        m = layer["mixer"]
        draw(p + "norm1", (W,), 0.1, 1.0)
        if layer["type"] == "latent_attention":
            H, d, r, R, dv = m["heads"], m["dim"], m["rot_dim"], m["kv_rank"], m["vdim"]
            draw(p + "mix.q", (H * (d + r), W), 1.5 * W ** -0.5)
            draw(p + "mix.dkv", (R + r, W), 1.5 * W ** -0.5)
            draw(p + "mix.dkv.norm", (R,), 0.1, 1.0)
            draw(p + "mix.uk", (H * d, R), R ** -0.5)
            draw(p + "mix.uv", (H * dv, R), R ** -0.5)
            draw(p + "mix.g", (H * dv, W), 2.0 * W ** -0.5)
            draw(p + "mix.o", (W, H * dv), (H * dv) ** -0.5)
        else:
            H, d = m["heads"], m["dim"]
            for s in "rkvgw":
                draw(p + "mix.mu." + s, (W,), 0.3, 0.4)
            for s in "rkvg":
                draw(p + "mix." + s, (H * d, W), W ** -0.5)
            draw(p + "mix.w1", (rank, W), W ** -0.5)
            draw(p + "mix.w2", (H * d, rank), 0.4)
            draw(p + "mix.w0", (H * d,), 1.0, -1.5)
            draw(p + "mix.u", (H, d), 0.4)
            draw(p + "mix.norm", (H * d,), 0.1, 1.0)
            draw(p + "mix.o", (W, H * d), (H * d) ** -0.5)
        mlp = layer.get("mlp")
        if mlp is not None:
            draw(p + "norm2", (W,), 0.1, 1.0)
            E, F = mlp["router"]["experts"], mlp["expert"]["ff"]
            draw(p + "mlp.router", (E, W), 4.0 * W ** -0.5)
            names = [(f"e{e}.", F) for e in range(E)]
            if mlp.get("shared"):
                names.append(("shared.", mlp["shared"]["ff"]))
                draw(p + "mlp.shared.sg", (1, W), 2.0 * W ** -0.5)
            for name, ff in names:
                draw(p + "mlp." + name + "gate", (ff, W), 1.5 * W ** -0.5)
                draw(p + "mlp." + name + "up", (ff, W), 1.5 * W ** -0.5)
                draw(p + "mlp." + name + "down", (W, ff), ff ** -0.5)
        if S:
            for which in ((1, 2) if mlp is not None else (1,)):
                draw(f"{p}hc{which}.in", (S,), 0.3, 0.8)
                draw(f"{p}hc{which}.out", (S,), 0.3, 0.9)
                draw(f"{p}hc{which}.mix", (S, S), 0.15, torch.eye(S))
    return out
