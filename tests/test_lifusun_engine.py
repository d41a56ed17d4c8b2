"""The Lifusun family through the engine's step function, cache manager and entry points, against the plain
restatement of tests/plain_lifusun.py: every way of cutting the same requests into steps (whole, the last tokens
one by one, portions down to two tokens, mixed batches over a pool so small that pages and state slots are used
again), the first tokens, long decoding across many chunks, and greedy generation through `LLM.generate`.
CPU cases run the host logic with the plain-torch kernel double; `-m gpu` cases run the CUDA kernels."""
import pytest
import torch

import plain_lifusun as plain
import replay_cases as cases
from helpers import make_engine, rel_err, run_steps
from lifusun_models import CONFIGS, write_model

FP32_TOL, BF16_TOL = 1e-4, 3e-2
LENGTHS = {"A": [1, 15, 16, 17, 33, 70], "B": [2, 31, 32, 33, 64, 97, 130], "C": [3, 40, 75], "D": [7, 8, 9, 25, 130]}

GPU = pytest.mark.gpu
CASES = [pytest.param("cpu", "float32", n, id=f"cpu-fp32-{n}") for n in "ABCD"] + \
        [pytest.param("cuda:0", dt, n, marks=GPU, id=f"gpu-{dt}-{n}") for dt in ("float32", "bfloat16") for n in "ABCD"]


@pytest.fixture(scope="module")
def lifusun_dirs(tmp_path_factory):
    return {name: write_model(cfg, str(tmp_path_factory.mktemp(f"lif_{name}")), seed) for name, (cfg, seed, _) in CONFIGS.items()}


@pytest.fixture(scope="module")
def refs(lifusun_dirs):
    out = {}
    for name, lens in LENGTHS.items():
        cfg, seed, _ = CONFIGS[name]
        reqs = cases.requests_for(cfg["vocab"], lens, seed + 10)
        c, w = plain.read_model_dir(lifusun_dirs[name])
        out[name] = (reqs, {rid: plain.forward(c, w, toks).float() for rid, toks in reqs.items()})
    return out


def compare(rows, ref, reqs, tol):
    worst = 0.0
    for rid, toks in reqs.items():
        got = torch.stack([rows[(rid, i)] for i in range(len(toks))])
        worst = max(worst, rel_err(got, ref[rid]))
    assert worst <= tol, worst
    return worst


@pytest.mark.parametrize("device,dtype,name", CASES)
def test_every_way_of_cutting(lifusun_dirs, refs, device, dtype, name):
    reqs, ref = refs[name]
    page = CONFIGS[name][2]
    tol = FP32_TOL if dtype == "float32" else BF16_TOL
    mixed_steps, peak = cases.mixed(reqs, live=3, seed=2)
    pages = peak // page
    eng = make_engine(lifusun_dirs[name], dtype, page, pages, device=device, max_num_seqs=3)     # three state slots for all requests
    for steps in (cases.whole(reqs), cases.last_one_by_one(reqs, tail=20), cases.portions(reqs), mixed_steps):
        rows = run_steps(eng, steps)
        eng.cache.check()
        assert eng.cache.num_free == pages and len(eng.cache.free_slots) == 3
        compare(rows, ref, reqs, tol)


@pytest.mark.parametrize("device,dtype,name", CASES)
def test_first_tokens_and_token_by_token(lifusun_dirs, refs, device, dtype, name):
    """A whole request one token a step: the convolution's zeros before position 0, a state that starts empty."""
    reqs, ref = refs[name]
    page = CONFIGS[name][2]
    rid, toks = max(reqs.items(), key=lambda kv: len(kv[1]) if len(kv[1]) <= 40 else 0)
    eng = make_engine(lifusun_dirs[name], dtype, page, 16, device=device, max_num_seqs=2)
    rows = run_steps(eng, [([(rid, toks[i:i + 1], [0])], []) for i in range(len(toks))])
    got = torch.stack([rows[(rid, i)] for i in range(len(toks))])
    assert rel_err(got, ref[rid]) <= (FP32_TOL if dtype == "float32" else BF16_TOL)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding(lifusun_dirs, dtype, name):
    """A short prompt, then hundreds of tokens one by one through many chunks and pages; every position compared."""
    cfg, seed, page = CONFIGS[name]
    total = 330
    reqs = cases.requests_for(cfg["vocab"], [total], seed + 20)
    c, w = plain.read_model_dir(lifusun_dirs[name])
    ref = {rid: plain.forward(c, w, toks).float() for rid, toks in reqs.items()}
    eng = make_engine(lifusun_dirs[name], dtype, page, -(-total // page) + 1, max_num_seqs=2)
    compare(run_steps(eng, cases.last_one_by_one(reqs, tail=total - 21)), ref, reqs, FP32_TOL if dtype == "float32" else BF16_TOL)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["A", "D"])
def test_float32_cuts_agree_closely(lifusun_dirs, refs, name):
    reqs, _ = refs[name]
    eng = make_engine(lifusun_dirs[name], "float32", CONFIGS[name][2], 128, max_num_seqs=4)
    a, b = run_steps(eng, cases.whole(reqs)), run_steps(eng, cases.portions(reqs))
    assert max(rel_err(b[k], a[k]) for k in a) < 1e-5


@pytest.mark.parametrize("device", ["cpu", pytest.param("cuda:0", marks=GPU)])
def test_greedy_generation_through_llm(lifusun_dirs, device):
    """Prompts of unequal length generate together through the scheduler (small token budget: prompts are cut into
    portions, the pool is small enough that requests wait); float32 must choose the plain implementation's tokens."""
    from iitj_llm_coopt_b200 import LLM, SamplingParams
    name = "A"
    cfg, seed, page = CONFIGS[name]
    c, w = plain.read_model_dir(lifusun_dirs[name])
    prompts = [[5, 17, 3, 150, 9], list(range(40, 77)), [159], list(range(20, 39))]
    want = [plain.greedy_generate(c, w, p, 6) for p in prompts]
    kernels = None
    if device == "cpu":
        from torch_kernels import TorchKernels
        kernels = TorchKernels()
    llm = LLM(lifusun_dirs[name], dtype="float32", page_size=page, num_pages=8, max_num_seqs=3, max_num_batched_tokens=24,
              device=device, kernels=kernels)
    outs = llm.generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True))
    assert [o.token_ids for o in outs] == want
