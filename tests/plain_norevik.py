"""A plain, slow float64 implementation of the Norevik decoder, written from its equations.

One function per mechanism, no cache and no batching: the whole sequence is recomputed from
its first token, the state mixers token by token. It shares no code with the library; the tests
compare the library's logits and intermediate tensors with it.

Notation: h is a sublayer's input [T, width] (the residual stream itself: this design has no norm
in front of a sublayer); W x means x @ W.T for a matrix stored [out, in]; positions count from 0.
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
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def layer_norm(x, w, b, eps):
    mean = x.mean(dim=-1, keepdim=True)
    var = ((x - mean) ** 2).mean(dim=-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * w + b


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0.0)


def silu(z):
    return z * torch.sigmoid(z)


def log_sigmoid(z):
    return -softplus(-z)


def rotate_pairs(x, positions, dims, base):
    """Rotate the first `dims` dimensions of x [T, ..., n]: dimension 2i pairs with 2i + 1,
    angle = position * base^(-2i/dims); the rest pass unchanged."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    angle = positions.to(F64)[:, None] * freq[None, :]
    while angle.dim() < x.dim():
        angle = angle.unsqueeze(1)
    cos, sin = torch.cos(angle), torch.sin(angle)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def causal_conv(x, taps, bias):
    """y_t[c] = bias[c] + sum_j taps[c, j] x_(t - (n-1) + j)[c], zeros before the start."""
    T, n = x.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros(n - 1, x.shape[1], dtype=F64), x], dim=0)
    out = torch.zeros_like(x)
    for j in range(n):
        out = out + padded[j:j + T] * taps[:, j]
    return out + bias


# --------------------------------------------------------------------------- state-space mixer
def grouped_unit_rms(y, parts, eps):
    """Each of `parts` equal parts of the last dimension divided by its own root mean square."""
    T, n = y.shape
    return unit_rms(y.reshape(T, parts, n // parts), eps).reshape(T, n)


def mamba2(h, m, w, p, eps):
    """Per head, S [state, vdim] from zero: S <- exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x."""
    H, dv, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * dv
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    T = h.shape[0]
    x = xbc[:, :inner].reshape(T, H, dv)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * dt)                     # [T, H]
    y = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        g = head // (H // G)
        S = torch.zeros(N, dv, dtype=F64)
        for t in range(T):
            S = decay[t, head] * S + dt[t, head] * torch.outer(B[t, g], x[t, head])
            y[t, head] = S.T @ C[t, g] + w[p + "D"][head] * x[t, head]
    y = y.reshape(T, inner) * silu(z)
    y = grouped_unit_rms(y, m["norm_groups"], eps) * w[p + "norm"]
    return y @ w[p + "o"].T


# --------------------------------------------------------------------------- latent attention
def latent_attention(h, m, w, p, eps):
    """Keys and values unfolded from a small normed latent, one rotated key part shared by the
    heads, a sink in the softmax's denominator, an elementwise sigmoid gate."""
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    pos = torch.arange(T)
    q = (h @ w[p + "q"].T).reshape(T, H, d + r)
    down = h @ w[p + "dkv"].T
    c = unit_rms(down[:, :rank], eps) * w[p + "dkv.norm"]
    shared = rotate_pairs(down[:, rank:], pos, m["rot"]["dims"], m["rot"]["base"])       # [T, r]
    q_rot = rotate_pairs(q[..., d:], pos, m["rot"]["dims"], m["rot"]["base"])            # [T, H, r]
    k = (c @ w[p + "uk"].T).reshape(T, H, d)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        s = (q[:, head, :d] @ k[:, head].T + q_rot[:, head] @ shared.T) * m["scale"]     # [T query, T key]
        s = s.masked_fill(pos[None, :] > pos[:, None], -math.inf)
        sink = w[p + "sink"][head]
        top = torch.maximum(s.max(dim=1).values, sink)
        e = torch.exp(s - top[:, None])
        out[:, head] = (e / (e.sum(dim=1) + torch.exp(sink - top))[:, None]) @ v[:, head]
    gate = torch.sigmoid(h @ w[p + "g"].T)
    return (out.reshape(T, H * dv) * gate) @ w[p + "o"].T


# --------------------------------------------------------------------------- matrix memory
def mlstm(h, m, w, p, eps):
    """Per head S [dim, vdim] and n [dim] from zero, with a running maximum m that starts at 0."""
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    T = h.shape[0]
    q = (h @ w[p + "q"].T).reshape(T, H, d) * d ** -0.5
    k = (h @ w[p + "k"].T).reshape(T, H, d)
    v = (h @ w[p + "v"].T).reshape(T, H, dv)
    i_gate = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)
    f_gate = log_sigmoid(cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    out = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        S, n, top = torch.zeros(d, dv, dtype=F64), torch.zeros(d, dtype=F64), torch.zeros((), dtype=F64)
        for t in range(T):
            new = torch.maximum(f_gate[t, head] + top, i_gate[t, head])
            keep, take = torch.exp(f_gate[t, head] + top - new), torch.exp(i_gate[t, head] - new)
            S = keep * S + take * torch.outer(k[t, head], v[t, head])
            n = keep * n + take * k[t, head]
            top = new
            out[t, head] = S.T @ q[t, head] / (torch.maximum((n @ q[t, head]).abs(), torch.exp(-top)) + 1e-6)
    out = unit_rms(out, eps).reshape(T, H * dv) * w[p + "norm"]
    return (out * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


MIXERS = {"mamba2": mamba2, "latent_attention": latent_attention, "mlstm": mlstm}


# --------------------------------------------------------------------------- feed-forwards
def dense(h, f, w, p):
    return torch.relu(h @ w[p + "up"].T) ** 2 @ w[p + "down"].T


def gated_expert(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, f, w, p):
    """(chosen [T, top] over experts + identity experts, their weights [T, top], scores [T, all])."""
    r = f["router"]
    total = r["experts"] + r.get("identity", 0)
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)
    choice = s + w[p + "correction"] if p + "correction" in w else s.clone()
    groups = r.get("groups")
    if groups is not None and groups["count"] > 1:
        size = total // groups["count"]
        best = choice.reshape(-1, groups["count"], size).max(dim=-1).values                 # [T, groups]
        kept = torch.topk(best, groups["keep"], dim=-1).indices
        allowed = torch.zeros_like(best, dtype=torch.bool).scatter_(1, kept, True)
        choice = choice.masked_fill(~allowed.repeat_interleave(size, dim=1), -math.inf)
    chosen = torch.topk(choice, r["top"], dim=-1).indices
    return chosen, torch.gather(s, 1, chosen), s


def experts(h, f, w, p):
    r = f["router"]
    chosen, weights, _ = route(h, f, w, p)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, weight in zip(chosen[t].tolist(), weights[t]):
            if e >= r["experts"]:
                out[t] += weight * h[t]                      # an identity expert
            else:
                out[t] += weight * gated_expert(h[t:t + 1], w, f"{p}e{e}.")[0]
    if f.get("shared") is not None:
        out = out + gated_expert(h, w, p + "shared.")
    return out


def feed_forward(h, f, w, p):
    return dense(h, f, w, p) if f["kind"] == "dense" else experts(h, f, w, p)


# --------------------------------------------------------------------------- the model
def forward(config, w, tokens, layers_out=None, seen=lambda t: t):
    """float64 logits [T, vocab] for one sequence; `layers_out` (a list) receives the residual
    stream after every layer. `seen` is applied to what every sublayer and the head read (the
    identity; a rounding shows how far a row's logits move when only its inputs are rounded)."""
    eps = config["norm"]["eps"]
    x = w["embed"][torch.tensor(list(tokens), dtype=torch.long)] * config.get("embedding", {}).get("scale", 1.0)
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        y = MIXERS[layer["type"]](seen(x), layer["mixer"], w, p + "mix.", eps)
        x = x + layer_norm(y, w[p + "norm1"], w[p + "norm1.b"], eps)
        if layer.get("mlp") is not None:
            y = feed_forward(seen(x), layer["mlp"], w, p + "mlp.")
            x = x + layer_norm(y, w[p + "norm2"], w[p + "norm2.b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    return seen(x) @ w["head"].T
