"""Lifusun's configuration, its layers as data, its checkpoint names and the trace replay's protocol (CPU)."""
import copy
import io
import json
import os

import numpy as np
import pytest
import torch

import plain_lifusun as plain
import replay_cases as cases
from lifusun_models import CONFIGS, LIF_A, LIF_B, make_tensors, write_model

from iitj_llm_coopt_b200.config import ConfigError, load_config
from iitj_llm_coopt_b200.config.lifusun import LifusunConfig
from iitj_llm_coopt_b200.models.decoder import cache_needs, model_parameter_specs
from iitj_llm_coopt_b200.weights.loader import WeightError, expected_tensors


def test_layers_as_data():
    spec = LifusunConfig.from_dict(LIF_B).model_spec()
    n = len(LIF_B["layers"])
    assert [c.cache for c in spec.order] == [0, 1, 1, 1, 4] and [c.write for c in spec.order] == [True, True, False, False, True]
    assert [c.state for c in spec.order] == [None, n + 1, n + 2, n + 3, None]
    needs = cache_needs(spec)
    assert needs[0].kind == "state" and needs[0].state_shape == (2, 32, 32)
    assert needs[1].kind == "paged_kv" and (needs[1].kv_heads, needs[1].head_dim, needs[1].value_dim) == (6, 32, 32)
    assert needs[2].kind == "none" and needs[3].kind == "none"
    assert needs[n + 1].state_shape == (1, 6 * 32 * 3) and needs[n + 2].state_shape == (3, 6 * 32)      # lender: q, k, v; borrower: q
    assert spec.layers[3].arrangement == "prenorm_mixer" and spec.layers[2].arrangement == "prenorm"


def test_checkpoint_names_are_the_family_s(tmp_path):
    for name, (cfg, seed, _) in CONFIGS.items():
        d = write_model(cfg, str(tmp_path / name), seed)
        arch, typed = load_config(d)
        assert arch.name == "Lifusun" and typed.to_dict() == cfg
        want = expected_tensors(arch, arch.model_spec(typed))
        have = make_tensors(cfg, seed)
        assert set(want) == set(have)
        assert all(tuple(want[k][0]) == tuple(have[k].shape) for k in want)


@pytest.mark.parametrize("change,text", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0].update(type="mamba"), "not known"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "kv_from"),         # layer 1 is no attention layer
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "kv_from"),         # not an earlier layer
    (lambda c: c["layers"][2]["mixer"].update(vdim=8), "other key/value sizes"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "mlp.kind"),
])
def test_bad_configurations_are_refused(change, text):
    cfg = copy.deepcopy(LIF_A)
    change(cfg)
    with pytest.raises(ConfigError, match=text):
        LifusunConfig.from_dict(cfg)


def test_missing_and_unexpected_tensors_are_listed(tmp_path):
    from helpers import make_engine
    t = make_tensors(LIF_A, 1)
    t["l2.mix.k"] = t["l0.mix.k"].clone()           # a borrowing layer has no key tensors
    del t["l0.mix.talk"], t["l3.norm2"]
    d = write_model(LIF_A, str(tmp_path / "m"), 1, tensors=t)
    with pytest.raises(WeightError) as e:
        make_engine(d, "float32", device="cpu")
    assert e.value.missing == ["l0.mix.talk", "l3.norm2"] and e.value.unexpected == ["l2.mix.k"]


def test_trace_replay_protocol(tmp_path):
    """bin/trace_run's program on a Lifusun folder (CPU kernel double): files only for steps that want something, a
    `done` line after every step, a request that is left out of a step and goes on later, slots given back at `end`."""
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
    got = {s: np.fromfile(tmp_path / "o" / f"{s}.f32", dtype="<f4").reshape(-1, cfg["vocab"]) for s in (0, 2, 3)}
    want = {0: [ra[16]], 2: [rb[2], rb[20], ra[19]], 3: [rb[20], ra[36]]}
    for s, rows in want.items():
        ref = torch.stack(rows).float().numpy()
        assert np.abs(got[s] - ref).max() <= 1e-4 * np.abs(ref).max()
