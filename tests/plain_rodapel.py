"""A plain, slow restatement of the Rodapel family in float64 torch: one function per mechanism, whole sequences
at once, no cache, no state carried between calls.  It shares no code with the engine: it reads config.json and
the checkpoint's tensors by their names.  The tests compare the engine with it.

Notation: x [T, w] is the residual stream of one sequence, positions 0 .. T-1; h is a sub-layer's input (x itself:
the norms of this family sit on the sub-layers' outputs).
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


def rms_norm(x, gain, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * gain


def softmax_over_visible(s, ok):
    """s [H, T, T] scores, ok [T, T] which keys each query sees."""
    return torch.softmax(s.masked_fill(~ok, float("-inf")), dim=-1)


def causal(T):
    i, j = torch.arange(T).view(T, 1), torch.arange(T).view(1, T)
    return j <= i


def sliding(T, size):
    i, j = torch.arange(T).view(T, 1), torch.arange(T).view(1, T)
    return (j <= i) & (i - j < size)


def rotate_pairs(v, base, dims):
    """v [T, H, D]: the leading `dims` numbers of each head are rotated, neighbours (2i, 2i+1) as a pair, by the angle
    position * base^(-2i/dims)."""
    T = v.shape[0]
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64)
    a = torch.arange(T, dtype=torch.float64).view(T, 1, 1) * freq.view(1, 1, half)
    c, s = torch.cos(a), torch.sin(a)
    out = v.clone()
    even, odd = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = even * c - odd * s
    out[..., 1:dims:2] = odd * c + even * s
    return out


def latent_attention(h, w, p, m, eps):
    """Keys and values of all heads rebuilt from one normed latent row per token, and one rotated key part that all
    heads share."""
    T = h.shape[0]
    H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ w[p + "q"].T).view(T, H, D + R)
    q_plain, q_rot = q[..., :D], rotate_pairs(q[..., D:], m["rot"]["base"], m["rot"]["dims"])
    down = h @ w[p + "dkv"].T
    latent = rms_norm(down[:, :C], w[p + "dkv.norm"], eps)
    k_rot = rotate_pairs(down[:, C:].view(T, 1, R), m["rot"]["base"], m["rot"]["dims"])[:, 0]
    k_plain = (latent @ w[p + "uk"].T).view(T, H, D)
    v = (latent @ w[p + "uv"].T).view(T, H, V)
    s = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihr,jr->hij", q_rot, k_rot)) * m["scale"]
    pr = softmax_over_visible(s, causal(T))
    o = torch.einsum("hij,jhv->ihv", pr, v).reshape(T, H * V)
    return o @ w[p + "o"].T


def window_attention(h, w, p, m, eps):
    """Grouped heads, a norm on every query and key head, no rotation, a sliding window, a gate on each head's output."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm((h @ w[p + "q"].T).view(T, H, D), w[p + "q.norm"], eps)
    k = rms_norm((h @ w[p + "k"].T).view(T, G, D), w[p + "k.norm"], eps)
    v = (h @ w[p + "v"].T).view(T, G, V)
    per = H // G
    k, v = k.repeat_interleave(per, dim=1), v.repeat_interleave(per, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    ok = sliding(T, m["mask"]["size"]) if m.get("mask") else causal(T)
    pr = softmax_over_visible(s, ok)
    o = torch.einsum("hij,jhv->ihv", pr, v)
    o = o * torch.sigmoid(h @ w[p + "g"].T).view(T, H, 1)
    return o.reshape(T, H * V) @ w[p + "o"].T


def wkv(h, w, p, m, eps):
    """A matrix state per head with a decay per key channel that the token itself chooses; the current token enters
    its own output through the bonus u instead of the state."""
    T, width = h.shape
    H, D = m["heads"], m["dim"]
    before = torch.cat([torch.zeros(1, width, dtype=h.dtype), h[:-1]])

    def mix(name):
        return h + (before - h) * w[p + "mu." + name]
    r = (mix("r") @ w[p + "r"].T).view(T, H, D)
    k = (mix("k") @ w[p + "k"].T).view(T, H, D)
    v = (mix("v") @ w[p + "v"].T).view(T, H, D)
    gate = torch.nn.functional.silu(mix("g") @ w[p + "g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(mix("w") @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"])).view(T, H, D)
    u = w[p + "u"]
    S = torch.zeros(H, D, D, dtype=h.dtype)                  # [head, key channel, value channel]
    out = torch.zeros(T, H, D, dtype=h.dtype)
    for t in range(T):
        kv = k[t].unsqueeze(2) * v[t].unsqueeze(1)
        out[t] = torch.einsum("hi,hij->hj", r[t], S + u.unsqueeze(2) * kv)
        S = decay[t].unsqueeze(2) * S + kv
    out = out / torch.sqrt((out * out).mean(-1, keepdim=True) + eps)
    return (out.reshape(T, H * D) * w[p + "norm"] * gate) @ w[p + "o"].T


def clamped_glu(h, gate, up, down, limit):
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def routed_experts(h, w, p, mlp):
    """Softmax over all router outputs; the choice adds a correction, the weights do not and are not renormalised;
    the last `identity` outputs stand for experts that hand back their input."""
    r, limit = mlp["router"], mlp["expert"]["limit"]
    E, top = r["experts"], r["top"]
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)
    chosen = torch.topk(s + w[p + "correction"], top, dim=-1).indices
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            if e >= E:
                y = h[t]
            else:
                y = clamped_glu(h[t:t + 1], w[f"{p}e{e}.gate"], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"], limit)[0]
            out[t] += s[t, e] * y
    return out


def feed_forward(h, w, p, mlp):
    if mlp["kind"] == "dense":
        return clamped_glu(h, w[p + "gate"], w[p + "up"], w[p + "down"], mlp["limit"])
    return routed_experts(h, w, p, mlp)


MIXERS = {"latent_attention": latent_attention, "attention": window_attention, "wkv": wkv}


def forward(cfg, w, tokens, layers_out=None):
    """Logits [T, vocab] of one whole sequence; `layers_out` (a list) receives the residual stream after each layer."""
    eps = cfg["norm"]["eps"]
    x = rms_norm(w["embed"][torch.tensor(tokens)], w["embed.norm"], eps)
    for i, layer in enumerate(cfg["layers"]):
        x = x + rms_norm(MIXERS[layer["type"]](x, w, f"l{i}.mix.", layer["mixer"], eps), w[f"l{i}.norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + rms_norm(feed_forward(x, w, f"l{i}.mlp.", layer["mlp"]), w[f"l{i}.norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T


def greedy_generate(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]
