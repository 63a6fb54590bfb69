"""Vizalix through the engine's own step function, cache manager, scheduler and entry points, against the
plain model: whole prompts, decoding token by token, portions down to two tokens, unequal requests in one
batch, pages and state slots used again, long decoding across windows, greedy generation."""

import json
import os
import subprocess
import sys

import pytest
import torch

import plain_vizalix as pv
import traces
import vizalix_tiny as vt
from engine_harness import run_trace

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# float32 against the plain model in float64; bfloat16 against the plain model that rounds where the engine
# stores 16 bits (a tiny model of several passes can amplify one rounding tenfold, which would say
# nothing about the engine)
TOL = {"float32": 4e-5, "bfloat16": 3e-2}
ROUNDING = {"float32": pv.same, "bfloat16": pv.as_bfloat16}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, cfg in vt.CONFIGS.items():
        w = vt.make_weights(cfg, seed=11 + len(name) + ord(name))
        folder = vt.write_folder(str(tmp_path_factory.mktemp("vz_" + name)), cfg, w)
        out[name] = (folder, cfg, w)
    return out


def runner_for(folder, dtype, **kw):
    from mini_infer_b200.engine.loading import load_model
    from mini_infer_b200.engine.step import ModelRunner
    model, rt, _ = load_model(folder, dtype, "cuda:0")
    args = dict(page_size=8, num_pages=40, max_requests=4, max_tokens_per_step=256, max_context=352)
    args.update(kw)
    return ModelRunner(model, rt, **args)


def check(got, ref, tol):
    worst = 0.0
    for (rid, pos), row in sorted(got.items()):
        scale = float(ref[rid].abs().max())
        err = float((row.double() - ref[rid][pos]).abs().max()) / scale
        worst = max(worst, err)
        assert err <= tol, f"request {rid} position {pos}: {err:.2e} of the largest logit (first failing place)"
    return worst


@pytest.mark.parametrize("name", ["P", "Q", "R", "S", "T"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_cutting_against_the_plain_model(models, name, dtype):
    folder, cfg, w = models[name]
    runner = runner_for(folder, dtype, max_requests=6, num_pages=60)
    reqs = vt.random_requests(cfg, [70, 1, 23, 2, 41, 9], seed=ord(name))
    ref = {rid: pv.forward(cfg, w, toks, rnd=ROUNDING[dtype]) for rid, toks in reqs.items()}
    results = []
    for steps in (traces.whole(reqs), traces.tail_decoded(reqs, tail=36), traces.portions(reqs),
                  traces.portions(reqs, (2,)), traces.mixed(reqs, max_live=3, seed=2, decode_tail=14),
                  traces.decoded_together({r: t for r, t in reqs.items() if len(t) > 1},
                                          {"r0": 30, "r2": 12, "r3": 1, "r4": 40, "r5": 3})):
        got = run_trace(runner, steps)
        check(got, ref, TOL[dtype])
        results.append(got)
        assert runner.cache.used_pages() == [0] * len(runner.cache.pools)
    if name == "T" and dtype == "bfloat16":
        mixers = [l.parts["mixer"] for l in runner.model.layers if "mixer" in l.parts]
        assert [m._tensor_cores for m in mixers if hasattr(m, "_tensor_cores")] == [True, True]
    if dtype == "float32":
        # the 32-bit path gives the same bits however the work was cut and batched
        for other in results[1:5]:
            for key, row in other.items():
                assert torch.equal(row, results[0][key]), key


def test_layer_by_layer(models):
    """The residual stream after every run of a layer (a looped layer counts each time)."""
    folder, cfg, w = models["P"]
    runner = runner_for(folder, "float32")
    toks = vt.random_requests(cfg, [29], 3)["r0"]
    want = []
    pv.forward(cfg, w, toks, residuals=want)
    seen = {}
    runner.model.layer_observer = lambda pos, hidden: seen.__setitem__(pos, hidden.cpu().double())
    runner.add_request("a")
    from mini_infer_b200.engine.step import StepEntry
    runner.step([StepEntry("a", toks, [])])
    runner.release("a")
    runner.model.layer_observer = None
    runs = [pos for pos, e in enumerate(runner.model.spec.schedule) if not e.args.get("auxiliary")]
    assert len(runs) == len(want)
    for n, pos in enumerate(runs):
        assert float((seen[pos] - want[n]).abs().max()) <= 3e-5 * float(want[n].abs().max()), n


def test_long_decoding_beyond_every_window_with_slots_and_pages_used_again(models):
    """Four requests decode 150 tokens each through replayed decode passes while a fifth and sixth wait for a
    slot; the pool holds far fewer pages than all requests together would need."""
    folder, cfg, w = models["P"]
    runner = runner_for(folder, "float32", num_pages=24, max_requests=4, max_context=200)
    reqs = vt.random_requests(cfg, [160, 170, 158, 165, 175, 181], seed=9)
    ref = {rid: pv.forward(cfg, w, toks) for rid, toks in reqs.items()}
    first, second = dict(list(reqs.items())[:4]), dict(list(reqs.items())[4:])
    for part in (first, second):
        got = run_trace(runner, traces.decoded_together(part, 150))
        check(got, ref, TOL["float32"])
    assert runner.graph_replays > 100


def test_states_of_a_finished_request_do_not_leak_into_the_next(models):
    folder, cfg, w = models["Q"]
    runner = runner_for(folder, "float32", max_requests=1)
    reqs = vt.random_requests(cfg, [33, 20, 27], seed=1)
    ref = {rid: pv.forward(cfg, w, toks) for rid, toks in reqs.items()}
    for rid, toks in reqs.items():                       # one slot, used three times
        got = run_trace(runner, traces.portions({rid: toks}, (5, 2, 11)))
        check(got, ref, TOL["float32"])


@pytest.mark.parametrize("name", ["P", "R"])
def test_greedy_generation_through_the_scheduler(models, name):
    from mini_infer_b200.engine.llm import LLM
    from mini_infer_b200.sampling import SamplingParams
    folder, cfg, w = models[name]
    prompts, wants = [], []
    seed = 0
    while len(prompts) < 4:
        seed += 1
        p = vt.random_requests(cfg, [3 + 7 * len(prompts)], seed)["r0"]
        gen = pv.greedy(cfg, w, p, 10)
        logits = pv.forward(cfg, w, p + gen)[len(p) - 1:-1]
        top2 = torch.topk(logits, 2, dim=-1).values
        if float((top2[:, 0] - top2[:, 1]).min()) > 1e-3:          # no near-tie that rounding could turn
            prompts.append(p)
            wants.append(gen)
    llm = LLM(folder, dtype="float32", max_seq_len=96, max_running=3, max_tokens_per_step=16, prefill_chunk=8,
              page_size=8)
    outs = llm.generate(prompts, SamplingParams(greedy=True, max_new_tokens=10))
    assert [o.token_ids for o in outs] == wants
    assert any(s.prefill_tokens and s.decode_tokens for s in llm.last_history)      # portions beside decodes
    assert llm.runner.cache.used_pages() == [0] * len(llm.runner.cache.pools)
    # bfloat16 serves the same model; its tokens are the arg-max of its own logits, checked by error bound
    llm16 = LLM(folder, dtype="bfloat16", max_seq_len=96, max_running=3, max_tokens_per_step=16, page_size=8)
    outs16 = llm16.generate(prompts[:2], SamplingParams(greedy=True, max_new_tokens=4))
    assert all(len(o.token_ids) == 4 for o in outs16)


def test_trace_runner_and_command_line(models, tmp_path):
    folder, cfg, w = models["Q"]
    toks = vt.random_requests(cfg, [19], 2)["r0"]
    ref = pv.forward(cfg, w, toks)
    lines = [json.dumps({"step": 0, "entries": [{"id": "a", "tokens": toks[:12], "want": [0, 11]}], "end": []}),
             json.dumps({"step": 1, "entries": [{"id": "a", "tokens": toks[12:], "want": [6]}], "end": ["a"]})]
    out = str(tmp_path / "out")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                        "--out", out, "--max-tokens", "64"], input="\n".join(lines) + "\n", text=True,
                       capture_output=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1"]
    import numpy as np
    a = torch.from_numpy(np.fromfile(os.path.join(out, "0.f32"), dtype="<f4").reshape(2, -1).copy())
    b = torch.from_numpy(np.fromfile(os.path.join(out, "1.f32"), dtype="<f4").reshape(1, -1).copy())
    scale = float(ref.abs().max())
    assert float((a.double() - ref[[0, 11]]).abs().max()) <= 4e-5 * scale
    assert float((b.double() - ref[[18]]).abs().max()) <= 4e-5 * scale


def test_generate_on_the_command_line_and_random_weights(models, tmp_path):
    folder, cfg, w = models["R"]
    seed = 0
    while True:
        seed += 1
        p = vt.random_requests(cfg, [6], seed)["r0"]
        gen = pv.greedy(cfg, w, p, 6)
        top2 = torch.topk(pv.forward(cfg, w, p + gen)[len(p) - 1:-1], 2, dim=-1).values
        if float((top2[:, 0] - top2[:, 1]).min()) > 1e-3:
            break
    cmd = [sys.executable, os.path.join(ROOT, "bin", "mini_infer"), "generate", "--model", folder, "--prompt-ids",
           ",".join(map(str, p)), "--max-new-tokens", "6", "--greedy", "--dtype", "float32", "--max-seq-len", "64", "--json"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = r.stdout.splitlines()
    assert json.loads(lines[lines.index("--- end ---") + 2])["token_ids"] == gen
    # a folder of seeded random weights for a configuration, written and served by the same entry points
    cfg_path = str(tmp_path / "config.json")
    with open(cfg_path, "w") as f:
        json.dump(vt.CONFIG_S, f)
    out = str(tmp_path / "made")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "mini_infer"), "random-weights", "--config", cfg_path,
                        "--seed", "5", "--out", out], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    runner = runner_for(out, "bfloat16")
    from mini_infer_b200.engine.step import StepEntry
    runner.add_request("a")
    res = runner.step([StepEntry("a", [1, 2, 3], [2])])
    assert res.logits.shape == (1, vt.CONFIG_S["vocab"]) and bool(torch.isfinite(res.logits).all())
