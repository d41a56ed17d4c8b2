"""Rodapel's configuration, its layers as data, its checkpoint names, sizes that only a tensor's shape gives, and the
trace replay's protocol on a Rodapel folder (CPU)."""
import copy
import io
import json
import os

import numpy as np
import pytest
import torch

import plain_rodapel as plain
from rodapel_models import CONFIGS, ROD_A, ROD_B, make_tensors, write_model

from iitj_llm_coopt_b200.config import ConfigError, load_config
from iitj_llm_coopt_b200.config.rodapel import RodapelConfig
from iitj_llm_coopt_b200.models.decoder import cache_needs
from iitj_llm_coopt_b200.weights.loader import WeightError, expected_tensors


def test_layers_as_data(tmp_path):
    d = write_model(ROD_B, str(tmp_path / "m"), 1)
    _, typed = load_config(d)
    spec = typed.model_spec()
    n = len(ROD_B[0]["layers"])
    assert [c.cache for c in spec.order] == [0, 1, 2, 3] and all(c.write for c in spec.order)
    assert [c.state for c in spec.order] == [None, n + 1, None, None]
    needs = cache_needs(spec)
    assert needs[0].kind == "paged_kv" and needs[0].shared_value and (needs[0].kv_heads, needs[0].head_dim, needs[0].value_dim) == (1, 52, 40)
    assert needs[0].page_elements(8) == 8 * 52
    assert needs[1].kind == "state" and needs[1].state_shape == (3, 24, 24)
    assert needs[2].kind == "paged_kv" and (needs[2].kv_heads, needs[2].head_dim, needs[2].value_dim, needs[2].window) == (1, 24, 16, 33)
    assert needs[n + 1].kind == "state" and needs[n + 1].state_shape == (96,)
    assert [l.arrangement for l in typed.model_spec().layers] == ["branchnorm"] * 4
    a = RodapelConfig.from_dict(ROD_A[0]).with_checkpoint_shapes({"l0.mix.w1": (5, 64)}).model_spec()
    assert a.layers[2].arrangement == "branchnorm_mixer" and a.embedding.kind == "table_norm"
    assert dict(a.layers[0].part("mixer").options)["decay_rank"] == 5
    assert a.layers[1].part("feed_forward").kind == "routed_glu" and a.layers[1].part("feed_forward").experts == 5


def test_decay_rank_comes_from_the_checkpoint_or_the_file():
    with pytest.raises(ConfigError, match="rank"):
        RodapelConfig.from_dict(ROD_A[0]).model_spec()
    cfg = copy.deepcopy(ROD_A[0])
    cfg["layers"][0]["mixer"]["decay_rank"] = 11
    assert dict(RodapelConfig.from_dict(cfg).model_spec().layers[0].part("mixer").options)["decay_rank"] == 11


def test_checkpoint_names_are_the_family_s(tmp_path):
    for name, (cfg, seed, _) in CONFIGS.items():
        d = write_model(cfg, str(tmp_path / name), seed)
        arch, typed = load_config(d)
        assert arch.name == "Rodapel"
        want = expected_tensors(arch, arch.model_spec(typed))
        have = make_tensors(cfg[0], cfg[1], seed)
        assert set(want) == set(have)
        assert all(tuple(want[k][0]) == tuple(have[k].shape) for k in want)


@pytest.mark.parametrize("change,text", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0].update(type="mamba"), "not known"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda c: c["layers"][2]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "mlp.kind"),
    (lambda c: c["layers"][0]["mlp"].pop("limit"), "limit"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=8), "router takes"),
])
def test_bad_configurations_are_refused(change, text):
    cfg = copy.deepcopy(ROD_A[0])
    change(cfg)
    with pytest.raises(ConfigError, match=text):
        RodapelConfig.from_dict(cfg)


def test_missing_and_unexpected_tensors_are_listed(tmp_path):
    from helpers import make_engine
    t = make_tensors(ROD_A[0], ROD_A[1], 1)
    t["l1.mlp.e5.gate"] = t["l1.mlp.e4.gate"].clone()           # the layer has five experts with tensors: e0 .. e4
    del t["l2.mix.dkv.norm"], t["l0.mix.mu.w"], t["embed.norm"]
    d = write_model(ROD_A, str(tmp_path / "m"), 1, tensors=t)
    with pytest.raises(WeightError) as e:
        make_engine(d, "float32", device="cpu")
    assert e.value.missing == ["embed.norm", "l0.mix.mu.w", "l2.mix.dkv.norm"] and e.value.unexpected == ["l1.mlp.e5.gate"]


def test_trace_replay_protocol(tmp_path):
    """bin/trace_run's program on a Rodapel folder (CPU kernel double): files only for steps that want something, a `done`
    line after every step, a request left out of a step that goes on later, two state slots that three requests share."""
    from iitj_llm_coopt_b200 import replay
    from torch_kernels import TorchKernels
    cfg, seed, page = CONFIGS["A"]
    d = write_model(cfg, str(tmp_path / "m"), seed)
    c, w = plain.read_model_dir(d)
    a, b = list(range(3, 40)), list(range(90, 111))
    lines = [json.dumps(x) for x in (
        {"step": 0, "entries": [{"id": "a", "tokens": a[:17], "want": [16]}, {"id": "b", "tokens": b[:2], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[17:19], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": b[2:], "want": [0, 18]}, {"id": "a", "tokens": a[19:20], "want": [0]}], "end": ["b"]},
        {"step": 3, "entries": [{"id": "c", "tokens": b, "want": [20]}, {"id": "a", "tokens": a[20:], "want": [16]}], "end": ["a", "c"]})]
    out = io.StringIO()
    args = replay.parse_args(["--model", d, "--dtype", "float32", "--out", str(tmp_path / "o"), "--max-tokens", "128",
                              "--max-requests", "2", "--device", "cpu"])
    assert replay.run(args, lines, out=out, kernels=TorchKernels()) == 0
    assert out.getvalue().split() == ["done", "0", "done", "1", "done", "2", "done", "3"]
    assert sorted(os.listdir(tmp_path / "o")) == ["0.f32", "2.f32", "3.f32"]
    ra, rb = plain.forward(c, w, a), plain.forward(c, w, b)
    got = {s: np.fromfile(tmp_path / "o" / f"{s}.f32", dtype="<f4").reshape(-1, cfg[0]["vocab"]) for s in (0, 2, 3)}
    want = {0: [ra[16]], 2: [rb[2], rb[20], ra[19]], 3: [rb[20], ra[36]]}
    for s, rows in want.items():
        ref = torch.stack(rows).float().numpy()
        assert np.abs(got[s] - ref).max() <= 1e-4 * np.abs(ref).max()
