"""Tiny Rodapel configurations for the tests and a writer of random model folders for them.

The writer names the checkpoint's tensors itself (from the configuration alone), so the engine's mapping from its
parameters to tensor names is tested against it.  The configurations differ in everything a model of this family can
vary: widths, the order of layers, head counts (grouped, ungrouped, one), key and value head sizes that differ, windows
(one token, a page, longer than the prompts), partial and full rotation, latent rows narrower and wider than a head,
expert counts (one, all chosen, identity experts or none), layers without a feed-forward, decay ranks.  The attention
scales are large on purpose: with a peaked softmax one key too many or too few moves the logits far beyond any tolerance.
"""
import json
import os

import torch
from safetensors.torch import save_file


def latent(heads, dim, rot_dim, vdim, rank, scale, rot_dims=None, base=10000.0):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
            "rot": {"dims": rot_dim if rot_dims is None else rot_dims, "base": base}}


def attention(heads, kv_heads, dim, vdim, window, scale):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window}}


def wkv(heads, dim):
    return {"heads": heads, "dim": dim}


def dense(ff, limit=2.0):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, identity, top, ff, limit=2.0):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "identity": identity, "top": top}}


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def config(width, vocab, eps, layers):
    return {"architecture": "Rodapel", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers}


# wkv first; grouped attention with wider values and a window shorter than a page; a latent layer without feed-forward;
# a window of one token (a query sees itself only)
ROD_A = (config(64, 150, 1e-5, [
    layer("wkv", wkv(2, 16), dense(48, limit=1.5)),
    layer("attention", attention(4, 2, 16, 24, 10, 0.6), moe(5, 2, 2, 20, limit=2.5)),
    layer("latent_attention", latent(3, 12, 8, 20, 24, 0.5, base=1000.0), None),
    layer("attention", attention(2, 2, 8, 8, 1, 0.4), dense(40)),
]), {0: 5})
# one latent head with a partly rotated part; every expert chosen; one expert with tensors among identity experts; one
# key/value head for six query heads, a window across pages
ROD_B = (config(96, 131, 1e-6, [
    layer("latent_attention", latent(1, 20, 12, 10, 40, 0.45, rot_dims=6, base=50.0), moe(3, 0, 3, 33)),
    layer("wkv", wkv(3, 24), moe(1, 3, 2, 16, limit=1.0)),
    layer("attention", attention(6, 1, 24, 16, 33, 0.5), moe(4, 1, 1, 24)),
    layer("latent_attention", latent(4, 8, 16, 8, 12, 0.5), dense(64, limit=3.0)),
]), {1: 7})
# wkv only (no page group at all): a head size that is not a multiple of 4, one head, a layer without feed-forward
ROD_C = (config(40, 90, 1e-5, [
    layer("wkv", wkv(1, 7), None),
    layer("wkv", wkv(5, 8), dense(56)),
]), {0: 3, 1: 9})
# attention only: a window longer than most prompts, odd sizes, then a window of exactly one page
ROD_D = (config(48, 77, 2e-5, [
    layer("attention", attention(3, 3, 12, 20, 70, 0.7), dense(36)),
    layer("attention", attention(8, 2, 8, 8, 16, 0.9), moe(2, 2, 2, 12)),
]), {})

CONFIGS = {"A": (ROD_A, 21, 16), "B": (ROD_B, 22, 8), "C": (ROD_C, 23, 16), "D": (ROD_D, 24, 4)}      # (config, ranks), seed, page size


def make_tensors(cfg, ranks, seed, std=0.08, soft=False):
    """{checkpoint name: bfloat16 tensor}.  `ranks`: {layer index: rank of a wkv layer's decay projection}.  `soft`: decays
    that depend less steeply on the token (a decay is exp(-exp(x)): where x is large, bfloat16's rounding of the token's row
    moves the decay by several per cent a token, which compounds in the state)."""
    g = torch.Generator().manual_seed(seed)

    def normal(*shape, s=std):
        return torch.randn(*shape, generator=g) * s

    def gains(n):
        return 1.0 + normal(n, s=0.1)

    w, t = cfg["width"], {}
    t["embed"] = normal(cfg["vocab"], w, s=1.0)
    t["embed.norm"] = gains(w)
    t["head"] = normal(cfg["vocab"], w)
    t["final.norm"] = gains(w)
    for i, lay in enumerate(cfg["layers"]):
        m, p = lay["mixer"], f"l{i}.mix."
        t[f"l{i}.norm1"] = gains(w) * (0.6 + 0.1 * i)
        if lay["type"] == "latent_attention":
            H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            t[p + "q"] = normal(H * (D + R), w, s=0.25)
            t[p + "dkv"] = normal(C + R, w, s=0.25)
            t[p + "dkv.norm"] = gains(C)
            t[p + "uk"], t[p + "uv"] = normal(H * D, C, s=0.3), normal(H * V, C, s=0.2)
            t[p + "o"] = normal(w, H * V)
        elif lay["type"] == "attention":
            H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            t[p + "q"], t[p + "k"], t[p + "v"] = normal(H * D, w), normal(G * D, w), normal(G * V, w)
            t[p + "q.norm"], t[p + "k.norm"] = gains(D) * 1.5, gains(D) * 1.5
            t[p + "g"] = normal(H, w, s=0.3)
            t[p + "o"] = normal(w, H * V)
        else:
            n, rank = m["heads"] * m["dim"], ranks[i]
            for s in "rkvgw":
                t[p + "mu." + s] = torch.rand(w, generator=g)
            t[p + "r"], t[p + "k"], t[p + "v"], t[p + "g"] = (normal(n, w, s=0.2) for _ in range(4))
            t[p + "w1"], t[p + "w2"] = normal(rank, w, s=0.3), normal(n, rank, s=0.2 if soft else 0.8)
            t[p + "w0"] = normal(n, s=0.5 if soft else 1.0) - (2.5 if soft else 1.5)             # decays from almost none to strong
            t[p + "u"] = normal(m["heads"], m["dim"], s=0.5)
            t[p + "norm"] = gains(n)
            t[p + "o"] = normal(w, n)
        mlp = lay["mlp"]
        if mlp is None:
            continue
        t[f"l{i}.norm2"] = gains(w) * 0.8
        q = f"l{i}.mlp."
        if mlp["kind"] == "dense":
            ff = mlp["ff"]
            t[q + "gate"], t[q + "up"], t[q + "down"] = normal(ff, w, s=0.4), normal(ff, w, s=0.4), normal(w, ff)
        else:
            r, ff = mlp["router"], mlp["expert"]["ff"]
            outputs = r["experts"] + r["identity"]
            t[q + "router"] = normal(outputs, w, s=0.5)
            t[q + "correction"] = normal(outputs, s=0.2)
            for e in range(r["experts"]):
                t[f"{q}e{e}.gate"], t[f"{q}e{e}.up"], t[f"{q}e{e}.down"] = normal(ff, w, s=0.4), normal(ff, w, s=0.4), normal(w, ff)
    return {k: v.to(torch.bfloat16).contiguous() for k, v in t.items()}


def write_model(cfg_and_ranks, out_dir, seed, std=0.08, tensors=None, soft=False):
    cfg, ranks = cfg_and_ranks
    os.makedirs(out_dir, exist_ok=True)
    save_file(tensors or make_tensors(cfg, ranks, seed, std, soft), os.path.join(out_dir, "model.safetensors"))
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f)
    return out_dir
