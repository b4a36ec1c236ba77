"""A plain, slow float64 implementation of the Tarupel decoder, written from its equations.

One function per mechanism, no cache and no batching: the whole sequence is recomputed from its
first token, the recurrence token by token. It shares no code with the library; the tests compare
the library's logits and intermediate tensors with it.

Notation: h is a sublayer's input [T, width]; W x means x @ W.T for a matrix stored [out, in];
positions count from 0; w is the dictionary of the model's tensors, p a name prefix.
"""
import json
import math
import os
import struct

import torch

F64 = torch.float64


# --------------------------------------------------------------------------- reading a folder
def read_model(folder):
    """(config dict, name -> float64 tensor) of a model folder with one model.safetensors."""
    with open(os.path.join(folder, "config.json")) as handle:
        config = json.load(handle)
    with open(os.path.join(folder, "model.safetensors"), "rb") as handle:
        (size,) = struct.unpack("<Q", handle.read(8))
        header = json.loads(handle.read(size))
        data = handle.read()
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "I32": torch.int32, "F16": torch.float16}
    tensors = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        lo, hi = entry["data_offsets"]
        raw = torch.frombuffer(bytearray(data[lo:hi]), dtype=kinds[entry["dtype"]])
        tensors[name] = raw.reshape(entry["shape"]).to(F64)
    return config, tensors


# --------------------------------------------------------------------------- small pieces
def unit_rms(x, eps):
    """x divided by its root mean square over the last dimension, eps under the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def scalar_norm(x, g, eps):
    """RMS norm whose weight is one number for all coordinates."""
    return unit_rms(x, eps) * g.reshape(())


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def token_shift(h, mu):
    """h_t + (h_(t-1) - h_t) * mu with zeros in front of the first token; h_(t-1) is the
    unshifted row."""
    before = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)
    return h + (before - h) * mu


def causal_conv(x, taps):
    """y_t[c] = sum_j taps[c, j] x_(t - (n-1) + j)[c], zeros before the start, no bias."""
    T, n = x.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros((n - 1, x.shape[1]), dtype=F64), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(n):
        y = y + padded[j:j + T] * taps[:, j]
    return y


def _angles(positions, dims, base):
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    return positions.to(F64)[:, None, None] * freq[None, None, :]


def rotate_halves(x, positions, dims, base):
    """x [T, heads, n]: dimension i pairs with i + dims/2 for i < dims/2; the rest unchanged."""
    a = _angles(positions, dims, base)
    cos, sin = torch.cos(a), torch.sin(a)
    half = dims // 2
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * cos - v * sin
    out[..., half:dims] = v * cos + u * sin
    return out


def rotate_pairs(x, positions, dims, base):
    """x [T, heads, n]: dimension 2i pairs with 2i + 1 for 2i + 1 < dims; the rest unchanged."""
    a = _angles(positions, dims, base)
    cos, sin = torch.cos(a), torch.sin(a)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def softmax_attention(q, k, v, scale, visible):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; visible(i, j) over index tensors says which j <= i a query i sees. Returns [T, H dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[2]), dtype=F64)
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    allowed = (j <= i) & visible(i, j)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        out[:, head] = torch.softmax(s, dim=-1) @ v[:, g]
    return out.reshape(T, -1)


# --------------------------------------------------------------------------- mixers
def general_delta(h, m, w, p, eps):
    """Generalized delta rule with a decay and a removal rate per head and key channel."""
    T, H, d = h.shape[0], m["heads"], m["dim"]
    r, k, v = ((h @ w[p + n].T).reshape(T, H, d) for n in ("r", "k", "v"))
    decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(h @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"]))
    decay = decay.reshape(T, H, d)
    rate = torch.sigmoid(h @ w[p + "a"].T + w[p + "a.b"]).reshape(T, H, d)
    unit = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
    out = torch.zeros((T, H, d), dtype=F64)
    for head in range(H):
        S = torch.zeros((d, d), dtype=F64)  # [key channel, value channel]
        for t in range(T):
            u = unit[t, head]
            old = S
            S = decay[t, head][:, None] * old - torch.outer(rate[t, head] * u, u @ old) \
                + torch.outer(k[t, head], v[t, head])
            out[t, head] = S.T @ r[t, head]
    out = unit_rms(out, eps).reshape(T, H * d) * w[p + "norm"]
    return (out * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def _projections(h, m, w, p):
    T, H, G, d, dv = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ w[p + "q"].T + w[p + "q.b"]
    k = h @ w[p + "k"].T + w[p + "k.b"]
    v = h @ w[p + "v"].T + w[p + "v.b"]
    return T, H, G, d, dv, q, k, v


def chunked_attention(h, m, w, p, eps):
    """Biased projections, a short convolution on each, split-half rotation of a head's first
    dimensions, unit RMS per head after it, keys visible inside the query's own chunk."""
    T, H, G, d, dv, q, k, v = _projections(h, m, w, p)
    q, k, v = (causal_conv(x, w[p + n + ".conv"]) for x, n in ((q, "q"), (k, "k"), (v, "v")))
    positions = torch.arange(T)
    rot = m["rot"]
    q = unit_rms(rotate_halves(q.reshape(T, H, d), positions, rot["dims"], rot["base"]), eps)
    k = unit_rms(rotate_halves(k.reshape(T, G, d), positions, rot["dims"], rot["base"]), eps)
    size = m["mask"]["size"]
    mixed = softmax_attention(q, k, v.reshape(T, G, dv), m["scale"], lambda i, j: i // size == j // size)
    return mixed @ w[p + "o"].T


def window_attention(h, m, w, p, eps):
    """Biased projections, a weighted RMS norm over the whole query row and the whole key row,
    rotation of neighbouring dimensions, keys visible up to size - 1 positions back."""
    T, H, G, d, dv, q, k, v = _projections(h, m, w, p)
    q = unit_rms(q, eps) * w[p + "q.norm"]
    k = unit_rms(k, eps) * w[p + "k.norm"]
    positions = torch.arange(T)
    rot = m["rot"]
    q = rotate_pairs(q.reshape(T, H, d), positions, rot["dims"], rot["base"])
    k = rotate_pairs(k.reshape(T, G, d), positions, rot["dims"], rot["base"])
    size = m["mask"]["size"]
    mixed = softmax_attention(q, k, v.reshape(T, G, dv), m["scale"], lambda i, j: i - j < size)
    return mixed @ w[p + "o"].T


MIXERS = {"general_delta": general_delta, "attention": chunked_attention, "attention_2": window_attention}


# --------------------------------------------------------------------------- feed-forwards
def gated(h, w, p, act):
    return (act(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, f, w, p):
    """(chosen expert ids [T, top], their weights [T, top]) from the scores over all experts."""
    router = f["router"]
    E, top = router["experts"], router["top"]
    scores = torch.softmax(h @ w[p + "router"].T, dim=-1)
    allowed = torch.ones_like(scores, dtype=torch.bool)
    groups = router.get("groups")
    if groups:
        count, keep = groups["count"], groups["keep"]
        best = scores.reshape(-1, count, E // count).max(dim=-1).values
        kept = best.topk(keep, dim=-1).indices
        allowed = torch.zeros((h.shape[0], count), dtype=torch.bool).scatter_(1, kept, True)
        allowed = allowed[:, :, None].expand(-1, -1, E // count).reshape(-1, E)
    ids = scores.masked_fill(~allowed, -1.0).topk(top, dim=-1).indices
    chosen = scores.gather(1, ids)
    weights = chosen / (chosen.sum(dim=-1, keepdim=True) + 1e-20) * router.get("scale", 1.0)
    return ids, weights


def experts(h, f, w, p):
    ids, weights = route(h, f, w, p)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(ids[t].tolist(), weights[t]):
            out[t] += a * gated(h[t:t + 1], w, f"{p}e{e}.", silu)[0]
    if f.get("shared"):
        gate = torch.sigmoid(h @ w[p + "shared.sg"].T)  # [T, 1]
        out = out + gate * gated(h, w, p + "shared.", silu)
    return out


def feed_forward(h, f, w, p):
    return gated(h, w, p, gelu_tanh) if f["kind"] == "dense" else experts(h, f, w, p)


# --------------------------------------------------------------------------- the model
def layer_runs(config):
    """[(layer, pass number or None)]: the pass number stands at the first layer of each pass of
    the looped run."""
    n, loop = len(config["layers"]), config.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, None) for i in range(start)]
    for t in range(times):
        runs += [(i, t if i == start else None) for i in range(start, stop)]
    return runs + [(i, None) for i in range(stop, n)]


def forward(config, w, tokens, layers_out=None, seen=lambda t: t):
    """Logits [T, vocab] of one sequence. `layers_out` (a list) receives the residual stream after
    every layer run; `seen` is applied to what enters a matrix product in a sublayer (the
    identity, or a rounding that mimics a 16-bit product path)."""
    eps, mult = config["norm"]["eps"], config.get("residual_mult", 1.0)
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * config.get("embedding", {}).get("scale", 1.0)
    embedded = x.clone()
    for i, t in layer_runs(config):
        if t is not None:
            if t > 0:
                x = x + embedded
            x = x + w["loop.step"][t]
        layer, p = config["layers"][i], f"l{i}."
        h = token_shift(seen(scalar_norm(x, w[p + "norm1"], eps)), w[p + "shift"])
        x = x + mult * w[p + "ls1"] * MIXERS[layer["type"]](seen(h), layer["mixer"], w, p + "mix.", eps)
        if layer.get("mlp"):
            h = seen(scalar_norm(x, w[p + "norm2"], eps))
            x = x + mult * w[p + "ls2"] * feed_forward(h, layer["mlp"], w, p + "mlp.")
        if layers_out is not None:
            layers_out.append(x.clone())
    return scalar_norm(x, w["final.norm"], eps) @ w["head"].T
