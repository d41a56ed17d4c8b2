"""A plain, slow restatement of the Lifusun family in float64 torch: one function per mechanism, whole sequences
at once, no cache, no state carried between calls.  It shares no code with the engine: it reads config.json and
the checkpoint's tensors by their names.  The tests compare the engine with it.

Notation: x [T, w] is the residual stream of one sequence, positions 0 .. T-1.
"""
import json
import math
import os

import torch
from safetensors import safe_open


def read_model_dir(path):
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    w = {}
    with safe_open(os.path.join(path, "model.safetensors"), "pt") as f:
        for k in f.keys():
            w[k] = f.get_tensor(k).double()
    return cfg, w


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scalar_norm(x, gain, eps):
    """One gain for the whole width."""
    return unit_rms(x, eps) * gain


def short_conv(u, taps):
    """y_t = sum_j taps[:, j] * u_(t - n + 1 + j), zeros before position 0.  u [T, C], taps [C, n]."""
    n = taps.shape[1]
    padded = torch.cat([torch.zeros(n - 1, u.shape[1], dtype=u.dtype), u])
    return sum(taps[:, j] * padded[j:j + u.shape[0]] for j in range(n))


def distance_slopes(heads, exponent=8.0):
    return torch.tensor([2.0 ** (-exponent * (h + 1) / heads) for h in range(heads)], dtype=torch.float64)


def visible(T, chunk):
    i, j = torch.arange(T).view(T, 1), torch.arange(T).view(1, T)
    ok = j <= i
    if chunk:
        ok = ok & (i // chunk == j // chunk)
    return ok


def mixed_scores(q, k, scale, talk):
    """q [T, H, D], k [T, H, D] (already spread over the query heads) -> scores [H, T, T] after the distance bias and
    the mixing of heads."""
    T, H, _ = q.shape
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    dist = (torch.arange(T).view(T, 1) - torch.arange(T).view(1, T)).double()
    s = s - distance_slopes(H).view(H, 1, 1) * dist
    return torch.einsum("hg,gij->hij", talk, s)


def attention_layer(h, m, w, prefix, eps, shared):
    """h [T, w] -> [T, w].  `shared[layer]` = (keys, values) of layers that keep their own, as later layers may read them."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]

    def project(name):
        u = h @ w[prefix + name].T + w[prefix + name + ".b"]
        return short_conv(u, w[prefix + name + ".conv"]) if m.get("conv") else u

    q = unit_rms(project("q"), eps) * w[prefix + "q.norm"]
    if m.get("kv_from") is not None:
        k, v = shared[m["kv_from"]]
    else:
        k = unit_rms(project("k"), eps) * w[prefix + "k.norm"]
        v = unit_rms(project("v").view(T, G, V), eps).reshape(T, G * V)
        shared[prefix] = (k, v)
    rep = H // G
    kh = k.view(T, G, D).repeat_interleave(rep, 1)
    vh = v.view(T, G, V).repeat_interleave(rep, 1)
    a = mixed_scores(q.view(T, H, D), kh, m["scale"], w[prefix + "talk"])
    a = a.masked_fill(~visible(T, (m.get("mask") or {}).get("size", 0)), -math.inf)
    o = torch.einsum("hij,jhv->ihv", torch.softmax(a, -1), vh).reshape(T, H * V)
    return o @ w[prefix + "o"].T


def rotate_half_layout(x, dims, base):
    """x [T, H, D]: dimension i < dims/2 pairs with i + dims/2; the rest passes."""
    if not dims:
        return x
    T, half = x.shape[0], dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64)
    ang = torch.arange(T, dtype=torch.float64).view(T, 1) * freq
    c, s = ang.cos().view(T, 1, half), ang.sin().view(T, 1, half)
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def retention_layer(h, m, w, prefix, eps):
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = rotate_half_layout((h @ w[prefix + "q"].T).view(T, H, D), rot["dims"], rot["base"])
    k = rotate_half_layout((h @ w[prefix + "k"].T).view(T, H, D), rot["dims"], rot["base"]) * D ** -0.5
    v = (h @ w[prefix + "v"].T).view(T, H, V)
    decay = torch.tensor(m["decay"], dtype=torch.float64).view(H, 1, 1)
    S = torch.zeros(H, D, V, dtype=torch.float64)
    o = torch.zeros(T, H, V, dtype=torch.float64)
    for t in range(T):
        S = decay * S + k[t].unsqueeze(-1) * v[t].unsqueeze(-2)
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = unit_rms(o, eps).reshape(T, H * V)
    return (o * torch.nn.functional.silu(h @ w[prefix + "g"].T)) @ w[prefix + "o"].T


def dense_feed_forward(h, w, prefix):
    return (torch.nn.functional.silu(h @ w[prefix + "gate"].T) * (h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def forward(cfg, w, tokens, after_layers=None):
    """Logits [T, vocab] (float64) of one sequence."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)]
    shared = {}
    for i, layer in enumerate(cfg["layers"]):
        h = scalar_norm(x, w[f"l{i}.norm1"], eps)
        if layer["type"] == "attention":
            m = dict(layer["mixer"])
            if m.get("kv_from") is not None:
                m["kv_from"] = f"l{m['kv_from']}.mix."
            x = x + attention_layer(h, m, w, f"l{i}.mix.", eps, shared)
        else:
            x = x + retention_layer(h, layer["mixer"], w, f"l{i}.mix.", eps)
        if layer.get("mlp") is not None:
            x = x + dense_feed_forward(scalar_norm(x, w[f"l{i}.norm2"], eps), w, f"l{i}.mlp.")
        if after_layers is not None:
            after_layers.append(x.clone())
    return scalar_norm(x, w["final.norm"], eps) @ w["head"].T


def greedy_generate(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]
