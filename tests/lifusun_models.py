"""Tiny Lifusun configurations for the tests and a writer of random model folders for them.

The writer names the checkpoint's tensors itself (from the configuration alone), so the engine's mapping from its
parameters to tensor names is tested against it.  The sizes differ between the configurations in everything that
a model of this family can vary: widths, head counts, grouped and ungrouped key/value heads, key and value head
sizes that differ, taps, chunk sizes, partial and full rotation, layers without a feed-forward, the order of
layers, which layers lend their keys and values and how many borrow them.
"""
import json
import os

import torch
from safetensors.torch import save_file


def attention(heads, kv_heads, dim, vdim, conv, chunk, scale=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5, "conv": conv,
         "mask": {"size": chunk}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def retention(heads, dim, vdim, decay, rot_dims, base=10000.0):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay, "rot": {"dims": rot_dims, "base": base}}


def layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(width, vocab, eps, layers):
    return {"architecture": "Lifusun", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers}


# attention first, grouped heads, value heads wider than key heads, a borrower without feed-forward, partial rotation
LIF_A = config(64, 160, 1e-5, [
    layer("attention", attention(4, 2, 16, 24, 3, 16, scale=0.3), 96),
    layer("retention", retention(2, 16, 8, [0.9, 0.99], 8), 80),
    layer("attention", attention(4, 2, 16, 24, 5, 16, scale=0.2, kv_from=0), 0),
    layer("retention", retention(3, 24, 40, [0.95, 0.999, 0.8], 24, base=500.0), 72),
])
# two borrowers of one lender, chunks of 32, two taps, a retention layer that rotates nothing, heads of 32
LIF_B = config(96, 131, 1e-6, [
    layer("retention", retention(2, 32, 32, [0.98, 0.9995], 16, base=1e6), 128),
    layer("attention", attention(6, 6, 32, 32, 2, 32), 112),
    layer("attention", attention(6, 6, 32, 32, 4, 32, kv_from=1), 64),
    layer("attention", attention(6, 6, 32, 32, 3, 32, kv_from=1), 0),
    layer("retention", retention(4, 8, 16, [0.5, 0.9, 0.99, 0.999], 0), 40),
])
# retention only (no pages at all), a head size that is not a multiple of 8, one head
LIF_C = config(48, 90, 1e-5, [
    layer("retention", retention(1, 20, 12, [0.97], 10), 56),
    layer("retention", retention(5, 8, 8, [0.9, 0.95, 0.99, 0.995, 0.999], 8), 0),
])
# attention only: one head, a chunk longer than most prompts, sizes that are not multiples of 8, then many heads in chunks of 8
LIF_D = config(40, 77, 2e-5, [
    layer("attention", attention(1, 1, 12, 20, 4, 128), 48),
    layer("attention", attention(20, 5, 8, 16, 2, 8, scale=0.5), 0),
    layer("attention", attention(20, 5, 8, 16, 6, 24, scale=0.25, kv_from=1), 36),
])

CONFIGS = {"A": (LIF_A, 11, 16), "B": (LIF_B, 12, 8), "C": (LIF_C, 13, 16), "D": (LIF_D, 14, 4)}      # config, seed, page size


def make_tensors(cfg, seed, std=0.08):
    """{checkpoint name: bfloat16 tensor}: matrices N(0, std), gains around 1, taps and mixing matrices with a strong
    diagonal / last tap and weaker other entries, biases N(0, 0.1)."""
    g = torch.Generator().manual_seed(seed)

    def normal(*shape, s=std):
        return torch.randn(*shape, generator=g) * s

    w, t = cfg["width"], {}
    t["embed"] = normal(cfg["vocab"], w, s=1.0)
    t["head"] = normal(cfg["vocab"], w)
    t["final.norm"] = torch.tensor(1.1)
    for i, lay in enumerate(cfg["layers"]):
        m, p = lay["mixer"], f"l{i}.mix."
        t[f"l{i}.norm1"] = torch.tensor(0.9 + 0.05 * i)
        if lay["type"] == "attention":
            names = [("q", m["heads"] * m["dim"])]
            if m.get("kv_from") is None:
                names += [("k", m["kv_heads"] * m["dim"]), ("v", m["kv_heads"] * m["vdim"])]
            for name, rows in names:
                t[p + name] = normal(rows, w)
                t[p + name + ".b"] = normal(rows, s=0.1)
                if m.get("conv"):
                    taps = normal(rows, m["conv"], s=0.3)
                    taps[:, -1] += 1.0
                    t[p + name + ".conv"] = taps
                if name != "v":
                    t[p + name + ".norm"] = 1.0 + normal(rows, s=0.1)
            t[p + "talk"] = torch.eye(m["heads"]) + normal(m["heads"], m["heads"], s=0.3)
            t[p + "o"] = normal(w, m["heads"] * m["vdim"])
        else:
            # k leans towards q: a request's first token reads sign(q . k) * v / |v| from a retention layer, which no
            # number format gets right when q . k happens to be next to nothing
            t[p + "q"] = normal(m["heads"] * m["dim"], w)
            t[p + "k"] = t[p + "q"] + 0.6 * normal(m["heads"] * m["dim"], w)
            t[p + "v"], t[p + "g"] = normal(m["heads"] * m["vdim"], w), normal(m["heads"] * m["vdim"], w)
            t[p + "o"] = normal(w, m["heads"] * m["vdim"])
        if lay["mlp"] is not None:
            ff = lay["mlp"]["ff"]
            t[f"l{i}.norm2"] = torch.tensor(1.05)
            t[f"l{i}.mlp.gate"], t[f"l{i}.mlp.up"], t[f"l{i}.mlp.down"] = normal(ff, w), normal(ff, w), normal(w, ff)
    return {k: v.to(torch.bfloat16).contiguous() for k, v in t.items()}


def write_model(cfg, out_dir, seed, std=0.08, tensors=None):
    os.makedirs(out_dir, exist_ok=True)
    save_file(tensors or make_tensors(cfg, seed, std), os.path.join(out_dir, "model.safetensors"))
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f)
    return out_dir
