"""Lifusun configurations drawn at random from fixed seeds (layer orders, head counts, grouped heads, key and value head
sizes, taps or none, chunk sizes or none, partial rotation, layers without a feed-forward, several borrowers), each through
the engine in float32 and bfloat16: whole prompts, portions, mixed batches with decoding, against the plain restatement."""
import random

import pytest
import torch

import plain_lifusun as plain
import replay_cases as cases
from helpers import make_engine, rel_err, run_steps
from lifusun_models import attention, config, layer, retention, write_model

pytestmark = pytest.mark.gpu


def draw(seed):
    rng = random.Random(seed)
    width = rng.choice([32, 48, 64, 96, 128, 160, 256])
    layers, lenders = [], []
    for i in range(rng.randint(2, 6)):
        ff = rng.choice([0, 40, 64, 100, 192])
        if rng.random() < 0.55:
            lender = rng.choice(lenders) if lenders and rng.random() < 0.5 else None
            if lender is None:
                kv = rng.choice([1, 2, 3, 4])
                m = attention(kv * rng.choice([1, 2, 4]), kv, rng.choice([8, 16, 24, 32, 64, 96]), rng.choice([8, 16, 32, 48, 64, 128]),
                              rng.choice([0, 2, 3, 4]), rng.choice([0, 8, 16, 32, 64, 128]), scale=rng.choice([None, 0.2, 0.35]))
                lenders.append(i)
            else:
                src = layers[lender]["mixer"]
                m = attention(src["kv_heads"] * rng.choice([1, 2]), src["kv_heads"], src["dim"], src["vdim"], rng.choice([0, 2, 4, 5]),
                              rng.choice([0, 16, 64]), scale=rng.choice([None, 0.3]), kv_from=lender)
            if not m["conv"]:
                del m["conv"]
            if not m["mask"]["size"]:
                del m["mask"]
            layers.append(layer("attention", m, ff))
        else:
            heads, dim = rng.choice([1, 2, 3, 4, 8]), rng.choice([8, 16, 32, 64, 128])
            m = retention(heads, dim, rng.choice([8, 16, 32, 64, 96]), [1.0 - 2.0 ** -rng.uniform(2, 11) for _ in range(heads)],
                          rng.choice([0, dim // 2, dim]), base=rng.choice([1e4, 1e6]))
            if not m["rot"]["dims"]:
                del m["rot"]
            layers.append(layer("retention", m, ff))
    return config(width, rng.choice([64, 131, 300, 512]), rng.choice([1e-5, 1e-6]), layers), rng.choice([4, 8, 16, 32])


@pytest.mark.parametrize("seed", list(range(100, 112)))
def test_random_configuration(tmp_path, seed):
    cfg, page = draw(seed)
    d = write_model(cfg, str(tmp_path / "m"), seed)
    c, w = plain.read_model_dir(d)
    reqs = cases.requests_for(cfg["vocab"], [1, 19, 66, 150, 300], seed)
    ref = {rid: plain.forward(c, w, toks).float() for rid, toks in reqs.items()}
    mixed_steps, peak = cases.mixed(reqs, live=3, seed=seed, decode_tail=12)
    for dtype, tol in (("float32", 1e-4), ("bfloat16", 3e-2)):
        eng = make_engine(d, dtype, page, max(peak // page, 1), max_num_seqs=3)
        for steps in (cases.whole(reqs), cases.portions(reqs), mixed_steps):
            rows = run_steps(eng, steps)
            eng.cache.check()
            worst = max(rel_err(torch.stack([rows[(rid, i)] for i in range(len(toks))]), ref[rid]) for rid, toks in reqs.items())
            assert worst <= tol, (seed, dtype, worst, cfg)
