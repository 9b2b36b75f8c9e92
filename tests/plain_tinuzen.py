"""A plain, slow implementation of the Tinuzen design: one function for each mechanism, on the CPU,
with whole-sequence matrices or token by token.  It shares no code with the package: it takes
config.json's dictionary and a dictionary of tensors by their stored names.

``dt`` is the type everything is computed in (float64 for an oracle).  Nothing here keeps a cache:
a sequence is always run whole, from its first token.
"""
from __future__ import annotations

import torch


def rms_norm(x, w, eps):
    """x * w / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


# ---- embedding --------------------------------------------------------------------------------
def embedding(tokens, W, e):
    """Token rows times a constant, plus a row of a second table picked by a hash of the token and
    the one before it; the sequence's first token takes the table's last row."""
    ids = [int(t) for t in tokens]
    b = e["bigram"]
    rows = [b["buckets"]] + [(ids[t - 1] * b["mul_prev"] + ids[t] * b["mul_cur"]) % b["buckets"]
                             for t in range(1, len(ids))]
    return W["embed"][torch.tensor(ids)] * e["scale"] + W["bigram"][torch.tensor(rows)]


# ---- attention, both kinds --------------------------------------------------------------------
def rotate_neighbours(x, positions, rot):
    """x [T, heads, dim]: columns (2i, 2i + 1) of the first rot['dims'] are turned by the angle
    position * base^(-2i / dims)."""
    dims = rot["dims"]
    i = torch.arange(dims // 2, dtype=x.dtype)
    f = torch.tensor(rot["base"], dtype=x.dtype) ** (-2.0 * i / dims)
    a = positions.to(x.dtype)[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def weigh_and_sum(scores, seen, v, rep, sink):
    """scores [H, T, T], seen [T, T] bool, v [T, G, E] -> [T, H, E].  ``sink``: the weights' sum has one
    more term exp(0), which brings no value."""
    scores = scores.masked_fill(~seen[None], float("-inf"))
    if sink:
        m = torch.clamp(scores.max(-1, keepdim=True).values, min=0.0)
        e = torch.exp(scores - m)
        p = e / (e.sum(-1, keepdim=True) + torch.exp(-m))
    else:
        p = torch.softmax(scores, -1)
    return torch.einsum("hts,she->the", p, v.repeat_interleave(rep, dim=1))


def windowed_attention(h, W, m, eps, pre):
    """The 'attention' mixer: q, k normed over the whole projection, no rotation, a bias that grows with
    the distance (one slope a head), a window that also keeps the sequence's first tokens."""
    T = h.shape[0]
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm(h @ W[pre + "q"].T, W[pre + "q.norm"], eps).view(T, H, D)
    k = rms_norm(h @ W[pre + "k"].T, W[pre + "k.norm"], eps).view(T, G, D)
    v = (h @ W[pre + "v"].T).view(T, G, E)
    rep = H // G
    scores = torch.einsum("thd,shd->hts", q, k.repeat_interleave(rep, dim=1)) * m["scale"]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    slope = 2.0 ** (-8.0 * (torch.arange(H, dtype=h.dtype) + 1) / H)
    scores = scores - slope[:, None, None] * (i - j).to(h.dtype)[None]
    seen = j <= i
    mask = m.get("mask")
    if mask:
        seen = seen & ((i - j < mask["size"]) | (j < mask.get("keep_first", 0)))
    o = weigh_and_sum(scores, seen, v, rep, sink=False)
    return o.reshape(T, H * E) @ W[pre + "o"].T


def sink_attention(h, W, m, pre):
    """The left half of the 'parallel' mixer: the keys, before their rotation, are the values; every
    earlier token is seen; the weights' sum has the extra 1; a sigmoid gate on every output element."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ W[pre + "q"].T).view(T, H, D)
    k = (h @ W[pre + "k"].T).view(T, G, D)
    v = k
    pos = torch.arange(T)
    if m.get("rot"):
        q, k = rotate_neighbours(q, pos, m["rot"]), rotate_neighbours(k, pos, m["rot"])
    rep = H // G
    scores = torch.einsum("thd,shd->hts", q, k.repeat_interleave(rep, dim=1)) * m["scale"]
    seen = pos[None, :] <= pos[:, None]
    o = weigh_and_sum(scores, seen, v, rep, sink=True).reshape(T, H * D)
    o = o * torch.sigmoid(h @ W[pre + "g"].T)
    return o @ W[pre + "o"].T


# ---- the state-space half ---------------------------------------------------------------------
def causal_conv(x, taps, bias):
    """x [T, C]; taps [C, n], the last column on the current token; zeros before the start."""
    T, C = x.shape
    n = taps.shape[1]
    padded = torch.cat([torch.zeros(n - 1, C, dtype=x.dtype), x], 0)
    y = bias.expand(T, C).clone()
    for j in range(n):
        y = y + padded[j: j + T] * taps[:, j]
    return y


def state_space_scan(x, B, C, dt, A_log, D):
    """x [T, H, P], B, C [T, H, N], dt [T, H].  For every head an N x P matrix S, zero at the start:
    S <- exp(-exp(A_log) dt_t) S + dt_t B_t x_t^T;  y_t = S^T C_t + D x_t."""
    T, H, P = x.shape
    N = B.shape[2]
    S = torch.zeros(H, N, P, dtype=x.dtype)
    y = torch.zeros_like(x)
    rate = torch.exp(A_log)
    for t in range(T):
        S = torch.exp(-rate * dt[t])[:, None, None] * S + dt[t][:, None, None] * B[t][:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("hnp,hn->hp", S, C[t]) + D[:, None] * x[t]
    return y


def state_space_mixer(h, W, m, eps, pre):
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    r = h @ W[pre + "in"].T
    z, xbc, dt = r[:, :inner], r[:, inner:2 * inner + 2 * G * N], r[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, W[pre + "conv"], W[pre + "conv.b"]))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N).repeat_interleave(H // G, dim=1)
    C = xbc[:, inner + G * N:].view(T, G, N).repeat_interleave(H // G, dim=1)
    dt = softplus(dt + W[pre + "dt_bias"])
    y = state_space_scan(x, B, C, dt, W[pre + "A_log"], W[pre + "D"]).reshape(T, inner)
    y = y * silu(z)
    parts = m["norm_groups"]
    y = y.view(T, parts, inner // parts)
    y = (y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)).reshape(T, inner) * W[pre + "norm"]
    return y @ W[pre + "o"].T


def side_by_side(h, W, m, eps, pre):
    return m["left_scale"] * sink_attention(h, W, m["left"], pre + "left.") + \
        m["right_scale"] * state_space_mixer(h, W, m["right"], eps, pre + "right.")


# ---- the rest of a layer ----------------------------------------------------------------------
def feed_forward(h, W, pre):
    return (torch.relu(h @ W[pre + "gate"].T) * (h @ W[pre + "up"].T)) @ W[pre + "down"].T


def layer(x, W, L, i, eps):
    """One norm; mixer and feed-forward read its output side by side; each result is multiplied by a
    sigmoid gate made from the same input before it joins the stream."""
    h = rms_norm(x, W[f"l{i}.norm1"], eps)
    if L["type"] == "attention":
        y = windowed_attention(h, W, L["mixer"], eps, f"l{i}.mix.")
    elif L["type"] == "parallel":
        y = side_by_side(h, W, L["mixer"], eps, f"l{i}.mix.")
    else:
        raise ValueError(L["type"])
    out = torch.sigmoid(h @ W[f"l{i}.rg1"].T + W[f"l{i}.rg1.b"]) * y
    if L.get("mlp") is not None:
        out = out + torch.sigmoid(h @ W[f"l{i}.rg2"].T + W[f"l{i}.rg2.b"]) * feed_forward(h, W, f"l{i}.mlp.")
    return x + out


def layer_order(cfg):
    """[(layer, number of the pass it opens or None), ...]: layers start .. stop-1 repeated ``times`` times."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None) for i in range(a)]
    for t in range(times):
        order += [(i, t if i == a else None) for i in range(a, b)]
    return order + [(i, None) for i in range(b, n)]


def forward(cfg, W, tokens, dt=torch.float64, layers_out=None):
    """Logits [T, vocab] of one sequence; ``layers_out``: a list that receives the residual stream
    after every run of a layer."""
    W = {n: (t.to(dt) if t.is_floating_point() else t) for n, t in W.items()}
    eps = cfg["norm"]["eps"]
    x0 = embedding(tokens, W, cfg["embedding"])
    x = x0
    for i, opens in layer_order(cfg):
        if opens is not None:
            if opens > 0:
                x = x + x0
            x = x + W["loop.step"][opens]
        x = layer(x, W, cfg["layers"][i], i, eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, W["final.norm"], eps) @ W["head"].T


def read_folder(model_dir: str):
    """(config.json's dictionary, stored name -> float64 tensor) read with nothing but the file format."""
    import json
    import os
    import struct

    import numpy as np
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    header.pop("__metadata__", None)
    W = {}
    for name, e in header.items():
        raw = data[e["data_offsets"][0]:e["data_offsets"][1]]
        if e["dtype"] == "BF16":
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif e["dtype"] == "F32":
            a = np.frombuffer(raw, dtype="<f4")
        else:
            raise ValueError(f"plain reader: dtype {e['dtype']} of {name}")
        W[name] = torch.from_numpy(a.astype(np.float64).reshape(e["shape"]))
    return cfg, W


def logits(cfg, W, tokens):
    """float64 numpy [T, vocab]."""
    with torch.no_grad():
        return forward(cfg, W, tokens, torch.float64).numpy()
