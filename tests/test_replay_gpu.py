"""Replay on the GPU: the same requests whole, with the last 32 tokens one by one, in
portions of changing size, and mixed with other requests over a pool so small that
pages are used again; in float32 and in bfloat16; compared with the plain
implementation.  Once through bin/trace_run as a user runs it, once per cutting
through the engine in this process (so that a failure names the cutting)."""

import numpy as np
import pytest

from tests import traces
from tests.conftest import cuda_or_skip
from tests.plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu

# float32: 1e-4 relative as the architecture's target states; bfloat16: eight bits of
# mantissa through a few layers (the reference allows 3e-2 on its bf16 device path,
# tests/test_gpu_decode.py:433-434).
TOL = {"float32": dict(rtol=1e-4, atol=2e-5), "bfloat16": dict(rtol=2e-2, atol=2e-2)}


def requests_for(cfg, seed=11):
    top = cfg["max_position_embeddings"]
    lengths = [min(n, top) for n in (50, 37, 64, 45, 41, 58, 33, 70)]
    rng = np.random.default_rng(seed)
    return {f"r{i}": rng.integers(0, cfg["vocab_size"], n).tolist() for i, n in enumerate(lengths)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tiny, tmp_path, dtype):
    cuda_or_skip()
    name, model_dir, page = tiny
    cfg, w = plain.load_model(model_dir)
    reqs = requests_for(cfg)
    want = traces.tagged({r: plain.forward(ids, w, cfg) for r, ids in reqs.items()})
    tr = traces.all_modes(reqs)
    out = traces.replay_subprocess(tr, model_dir, dtype, str(tmp_path / "out"), page)
    traces.compare(tr, out, want, what=f"trace_run {name}/{dtype}", **TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["whole", "tail_decode", "portions", "mixed"])
def test_cuttings_in_process(tiny, dtype, mode):
    from sllm_b200.engine import Engine, build_model
    dev = cuda_or_skip()
    name, model_dir, page = tiny
    cfg, w = plain.load_model(model_dir)
    reqs = requests_for(cfg)
    want = {r: plain.forward(ids, w, cfg) for r, ids in reqs.items()}
    tr = getattr(traces, mode)(reqs)
    model, _ = build_model(model_dir, dtype, dev)
    eng = Engine(model, page_size=page, num_pages=tr.max_tokens // page, max_requests=4)
    out = traces.replay_engine(tr, eng)
    traces.compare(tr, out, want, what=f"{name}/{dtype}/{mode}", **TOL[dtype])
    eng.cache.check()
    assert not eng.cache.requests and all(g.pool.used_count == 0 for g in eng.cache.groups)
    if mode == "mixed":
        assert eng.cache.reuse_count > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_cutting_with_freed_pages_poisoned(tiny, dtype):
    """The cache manager's debugging aid fills every page that goes back to the pool with NaN (and
    zeroes a page when it is handed out).  With pages used again and again, a kernel that read a page
    its request does not hold would put NaN into the logits; none may."""
    from sllm_b200.engine import Engine, build_model
    dev = cuda_or_skip()
    name, model_dir, page = tiny
    cfg, w = plain.load_model(model_dir)
    reqs = requests_for(cfg)
    want = {r: plain.forward(ids, w, cfg) for r, ids in reqs.items()}
    tr = traces.mixed(reqs)
    model, _ = build_model(model_dir, dtype, dev)
    eng = Engine(model, page_size=page, num_pages=tr.max_tokens // page, max_requests=4, poison_freed=True)
    assert bool(eng.cache.kv_storage[0].isnan().all())            # nobody holds a page yet
    out = traces.replay_engine(tr, eng)
    assert all(np.isfinite(o).all() for o in out.values())
    traces.compare(tr, out, want, what=f"{name}/{dtype}/mixed, freed pages poisoned", **TOL[dtype])
    assert eng.cache.reuse_count > 0 and bool(eng.cache.kv_storage[0].isnan().all())


def test_float32_cuttings_agree_to_rounding(tiny):
    """In float32 the order of summation for a position does not depend on the cutting,
    so the cuttings agree far more closely with each other than the tolerance against
    the plain implementation demands."""
    from sllm_b200.engine import Engine, build_model
    dev = cuda_or_skip()
    name, model_dir, page = tiny
    cfg, _ = plain.load_model(model_dir)
    reqs = requests_for(cfg)
    rows = {}
    for mode in ("whole", "tail_decode", "portions", "mixed"):
        tr = getattr(traces, mode)(reqs)
        model, _ = build_model(model_dir, "float32", dev)
        eng = Engine(model, page_size=page, num_pages=tr.max_tokens // page, max_requests=4)
        out = traces.replay_engine(tr, eng)
        for s in tr.steps:
            for i, key in enumerate(s["expect"]):
                rows.setdefault(key, {})[mode] = out[s["step"]][i]
    worst = 0.0
    for key, by_mode in rows.items():
        ref = by_mode["whole"]
        for mode, row in by_mode.items():
            worst = max(worst, float(np.abs(row - ref).max()))
    assert worst <= 2e-6, f"cuttings differ by {worst}"
