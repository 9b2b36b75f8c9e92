"""A plain, slow implementation of the Sugizen design: one function for each mechanism, token by
token or with whole-sequence matrices, on the CPU.  It shares no code with the package: it takes
config.json's dictionary and a dictionary of tensors by their stored names.

``dt`` is the type everything is computed in (float64 for an oracle, float32 to see what 32-bit
arithmetic alone does).  Nothing here keeps a cache: a sequence is always run whole.
"""
from __future__ import annotations

import math

import torch


def rms_norm(x, w, eps):
    """x * w / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def short_conv_silu(x, taps):
    """x [T, C]; taps [C, n]: y_t = sum_j taps[:, n-1-j] * x_{t-j} (zeros before the start), then silu."""
    T, C = x.shape
    n = taps.shape[1]
    padded = torch.cat([torch.zeros(n - 1, C, dtype=x.dtype), x], 0)
    y = torch.zeros_like(x)
    for j in range(n):
        y = y + padded[n - 1 - j: n - 1 - j + T] * taps[:, n - 1 - j]
    return y * torch.sigmoid(y)


def unit(x, eps=1e-6):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def delta_rule_scan(q, k, v, beta, decay):
    """q, k [T, H, D] (already unit vectors, q scaled), v [T, H, E], beta [T, H], decay [T, H, D].
    For every head a D x E matrix S, zero at the start:
        S <- decay_t[:, None] * S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t."""
    T, H, D = q.shape
    E = v.shape[2]
    S = torch.zeros(H, D, E, dtype=q.dtype)
    out = torch.zeros(T, H, E, dtype=q.dtype)
    for t in range(T):
        S = decay[t][:, :, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hde,hd->he", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        out[t] = torch.einsum("hde,hd->he", S, q[t])
    return out


def delta_mixer(h, W, m, eps, pre):
    """The gated delta-rule mixer on one sequence h [T, width]; ``pre`` is the tensor-name prefix."""
    T = h.shape[0]
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv_silu(h @ W[pre + "q"].T, W[pre + "q.conv"]).view(T, G, D)
    k = short_conv_silu(h @ W[pre + "k"].T, W[pre + "k.conv"]).view(T, G, D)
    v = short_conv_silu(h @ W[pre + "v"].T, W[pre + "v.conv"]).view(T, H, E)
    q = unit(q) * D ** -0.5
    k = unit(k)
    rep = H // G
    q = q.repeat_interleave(rep, dim=1)
    k = k.repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(h @ W[pre + "b"].T)
    step = softplus((h @ W[pre + "a1"].T) @ W[pre + "a2"].T + W[pre + "dt_bias"]).view(T, H, D)
    decay = torch.exp(-torch.exp(W[pre + "A_log"])[None, :, None] * step)
    o = delta_rule_scan(q, k, v, beta, decay)
    o = rms_norm(o, W[pre + "norm"], eps)
    o = o * torch.sigmoid((h @ W[pre + "g1"].T) @ W[pre + "g2"].T).view(T, H, E)
    return o.reshape(T, H * E) @ W[pre + "o"].T


def rotary_frequencies(rot, dt=torch.float64):
    """f_i = base^(-2i/dims), then the wavelength-dependent scaling if the configuration has one."""
    dims = rot["dims"]
    i = torch.arange(dims // 2, dtype=dt)
    f = torch.tensor(rot["base"], dtype=dt) ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if sc:
        wavelength = 2 * math.pi / f
        short = sc["original"] / sc["high"]
        long_ = sc["original"] / sc["low"]
        s = (sc["original"] / wavelength - sc["low"]) / (sc["high"] - sc["low"])
        mid = (1 - s) * f / sc["factor"] + s * f
        f = torch.where(wavelength < short, f, torch.where(wavelength > long_, f / sc["factor"], mid))
    return f


def rotate(x, positions, rot):
    """x [T, heads, dim]: the first rot['dims'] columns in pairs (i, i + dims/2)."""
    dims = rot["dims"]
    f = rotary_frequencies(rot, x.dtype)
    a = positions.to(x.dtype)[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


def attention_keys_values(h, W, m, eps, pre):
    """Keys (normed, rotated) and values of a layer that owns them, as its cache would hold them."""
    T = h.shape[0]
    G, D, E = m["kv_heads"], m["dim"], m["vdim"]
    k = (h @ W[pre + "k"].T).view(T, G, D)
    v = (h @ W[pre + "v"].T).view(T, G, E)
    k = rms_norm(k, W[pre + "k.norm"], eps)
    if m.get("rot"):
        k = rotate(k, torch.arange(T), m["rot"])
    return k, v


def attention_mixer(h, W, m, eps, pre, kv):
    """kv: (k [T, G, D], v [T, G, E]), the layer's own or another layer's."""
    T = h.shape[0]
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm((h @ W[pre + "q"].T).view(T, H, D), W[pre + "q.norm"], eps)
    if m.get("rot"):
        q = rotate(q, torch.arange(T), m["rot"])
    k, v = kv
    rep = H // G
    scores = torch.einsum("thd,shd->hts", q, k.repeat_interleave(rep, dim=1)) * m["scale"]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if m.get("mask"):
        size = m["mask"]["size"]
        seen = seen & ((i // size) == (j // size))
    scores = scores.masked_fill(~seen[None], float("-inf"))
    p = torch.softmax(scores, -1)
    o = torch.einsum("hts,she->the", p, v.repeat_interleave(rep, dim=1))
    o = o * torch.sigmoid(h @ W[pre + "g"].T)[:, :, None]
    return o.reshape(T, H * E) @ W[pre + "o"].T


def feed_forward(h, W, f, pre):
    g = torch.clamp(h @ W[pre + "gate"].T, max=f["limit"])
    u = torch.clamp(h @ W[pre + "up"].T, -f["limit"], f["limit"])
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ W[pre + "down"].T


def forward(cfg, W, tokens, dt=torch.float64, layers_out=None):
    """Logits [T, vocab] of one sequence; ``layers_out``: a list that receives the residual stream
    after every layer."""
    W = {n: (t.to(dt) if t.is_floating_point() else t) for n, t in W.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    held = {}
    for i, L in enumerate(cfg["layers"]):
        pre, m = f"l{i}.mix.", L["mixer"]
        if L["type"] == "channel_delta":
            y = delta_mixer(x, W, m, eps, pre)
        elif L["type"] == "attention":
            if m.get("kv_from") is not None:
                kv = held[m["kv_from"]]
            else:
                kv = held[i] = attention_keys_values(x, W, m, eps, pre)
            y = attention_mixer(x, W, m, eps, pre, kv)
        else:
            raise ValueError(L["type"])
        x = x + rms_norm(y, W[f"l{i}.norm1"], eps)
        if L.get("mlp") is not None:
            x = x + rms_norm(feed_forward(x, W, L["mlp"], f"l{i}.mlp."), W[f"l{i}.norm2"], eps)
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
