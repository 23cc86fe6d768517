"""The Renadra decoder through the engine on the GPU, in both precisions, against the plain implementation: whole
prompts, the last tokens one by one (replayed as CUDA graphs), portions down to two tokens, mixed batches in which
pages and state slots are used again, decoding from the very first token through windows, kept first keys and several
pages, seeded random configurations, greedy generation through the engine's entry point and the command line, and the
replay program as a subprocess."""

import json
import subprocess
import sys

import numpy as np
import pytest
import torch

import renadra_util as zu
import replay_util as ru
from plain import renadra_plain as plain

pytestmark = pytest.mark.gpu

LENGTHS = (1, 2, 19, 47, 130)
MODES = ["whole", "last32", "portions", "mixed"]


def _check(trace, outputs, expected, dtype):
    """float32: element by element.  bfloat16: every row against its own scale (rounded projections feed forget gates
    and sigmoid weights, so a row's rounding error is a few per cent of its scale; a lost state, a wrong page or a
    window that is one token off misses by the row's whole scale)."""
    if dtype == "bfloat16":
        return ru.compare_rows_to_scale(trace, outputs, expected, rms_bound=0.08, peak_bound=0.3)
    return ru.compare(trace, outputs, expected, dtype)


def _loose(trace, outputs, expected):
    """float32 against float64 for random configurations: recurrences over a hundred tokens and up to three passes
    leave a few 1e-5 of summation order."""
    saved = dict(ru.TOL["float32"])
    ru.TOL["float32"] = dict(atol=2e-4, rtol=2e-4)
    try:
        return ru.compare(trace, outputs, expected, "float32")
    finally:
        ru.TOL["float32"] = saved


def _trace(mode, requests, max_tokens):
    return {"whole": ru.trace_whole, "last32": ru.trace_last_decoded, "portions": ru.trace_portions,
            "mixed": lambda r: ru.trace_mixed(r, max_tokens, seed=5)}[mode](requests)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("name", ["R1", "R2", "R3"])
def test_replay_matches_plain(name, mode, dtype):
    raw, page = zu.CONFIGS[name]
    folder = zu.model_folder(name)
    requests = ru.make_requests(raw["vocab"], LENGTHS + ((70, 45) if mode == "mixed" else ()), seed=11)
    expected = zu.plain_logits(folder, raw, requests)
    max_tokens = 64 * 6
    trace = _trace(mode, requests, max_tokens)
    outputs, engine = ru.run_on_device(folder, dtype, trace, max_tokens, page_size=page, max_seqs=4)
    _check(trace, outputs, expected, dtype)
    if mode == "last32":
        assert engine.runner.graph_replays > 0, "single-token steps were not replayed as CUDA graphs"
    assert engine.manager.free_pages() == [g.pool.count for g in engine.manager.groups]
    engine.manager.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["R1", "R3"])
def test_decoding_from_the_first_token(name, dtype):
    """Every token a step of its own for 150 positions: the windows pass over decoded tokens only, the kept first
    keys were written one at a time, pages behind the windows come back and are used again, and the memories and the
    previous token are carried through 149 steps."""
    raw, page = zu.CONFIGS[name]
    folder = zu.model_folder(name)
    requests = ru.make_requests(raw["vocab"], (150,), seed=31)
    expected = zu.plain_logits(folder, raw, requests)
    trace = ru.trace_last_decoded(requests, last=149)
    outputs, engine = ru.run_on_device(folder, dtype, trace, 192, page_size=page, max_seqs=2)
    _check(trace, outputs, expected, dtype)
    assert engine.runner.graph_replays >= 100


def test_eager_and_captured_single_token_steps_agree():
    """The captured step runs once before it is captured; what that run did to the memories and to the previous token
    is undone (a step's tokens enter the state once)."""
    raw, page = zu.CONFIGS["R1"]
    folder = zu.model_folder("R1")
    requests = ru.make_requests(raw["vocab"], (40, 33), seed=3)
    trace = ru.trace_last_decoded(requests, last=12)
    with_graphs, engine = ru.run_on_device(folder, "float32", trace, 128, page_size=page, max_seqs=4)
    assert engine.runner.graph_replays > 0
    without, _ = ru.run_on_device(folder, "float32", trace, 128, page_size=page, max_seqs=4, cuda_graphs=False)
    for step in trace.expect:
        torch.testing.assert_close(torch.from_numpy(with_graphs[step]), torch.from_numpy(without[step]), atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("seed", list(range(1, 11)))
def test_random_configuration(seed):
    folder = zu.random_model_folder(seed)
    raw, page = zu.CONFIGS[f"random{seed}"]
    requests = ru.make_requests(raw["vocab"], (1, 2, 23, 61, 90, 37), seed=seed)
    expected = zu.plain_logits(folder, raw, requests)
    max_tokens = 64 * 5
    mixed = ru.trace_mixed(requests, max_tokens, seed=seed)
    outputs, engine = ru.run_on_device(folder, "float32", mixed, max_tokens, page_size=page, max_seqs=4)
    _loose(mixed, outputs, expected)
    engine.manager.check_invariants()
    tail = ru.trace_last_decoded(requests, last=20)
    outputs, engine = ru.run_on_device(folder, "float32", tail, max_tokens, page_size=page, max_seqs=4)
    _loose(tail, outputs, expected)
    assert engine.runner.graph_replays > 0
    outputs, engine = ru.run_on_device(folder, "bfloat16", mixed, max_tokens, page_size=page, max_seqs=4)
    assert all(np.isfinite(rows).all() for rows in outputs.values())


@pytest.mark.parametrize("name", ["R1", "R3"])
def test_greedy_generation_through_the_entry_point(name):
    from ampere_kv_engine_b200.engine.engine import Engine
    raw, page = zu.CONFIGS[name]
    folder = zu.model_folder(name)
    w = zu.plain_weights(folder)
    prompts = list(ru.make_requests(raw["vocab"], (3, 30, 61), seed=41).values())
    engine = Engine.from_pretrained(folder, dtype="float32", device="cuda", page_size=page, num_pages=16,
                                    max_batch_tokens=24, max_seqs=4)
    got = engine.generate(prompts, max_new_tokens=8, ignore_eos=True)
    assert got == [plain.greedy_generate(raw, w, p, 8) for p in prompts]
    # five requests through four state slots: one waits, then takes a slot that was used before
    more = prompts + [prompts[1][:7], prompts[2][:11]]
    again = engine.generate(more, max_new_tokens=8, ignore_eos=True)
    assert again[:3] == got and again[3:] == [plain.greedy_generate(raw, w, p, 8) for p in more[3:]]
    engine.manager.check_invariants()
    # bfloat16: every chosen token is (nearly) the best one of the plain logits
    engine = Engine.from_pretrained(folder, dtype="bfloat16", device="cuda", page_size=page, num_pages=16, max_seqs=4)
    for prompt, out in zip(prompts, engine.generate(prompts, max_new_tokens=4, ignore_eos=True)):
        ids = list(prompt)
        for token in out:
            logits = plain.forward(raw, w, ids)[-1]
            assert float(logits.max() - logits[token]) <= 0.05 * float(logits.max() - logits.min()), \
                "bfloat16 picked a token far from the best"
            ids.append(token)


def test_command_line_and_replay_program():
    root = ru.ROOT
    raw, page = zu.CONFIGS["R1"]
    folder = zu.model_folder("R1")
    prompt = list(ru.make_requests(raw["vocab"], (17,), seed=51).values())[0]
    cmd = [sys.executable, "-m", "ampere_kv_engine_b200.runner", "--model", folder, "--mode", "generate", "--dtype",
           "float32", "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "5", "--ignore-eos",
           "--page-size", str(page)]
    proc = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    line = next(l for l in proc.stdout.splitlines() if l.startswith("generated_token_ids"))
    assert json.loads(line.split("=", 1)[1]) == plain.greedy_generate(raw, zu.plain_weights(folder), prompt, 5)
    # the replay program itself, as a user starts it
    requests = ru.make_requests(raw["vocab"], (5, 40), seed=8)
    trace = ru.trace_portions(requests)
    outputs = ru.run_subprocess(folder, "float32", trace, 128, page_size=page)
    ru.compare(trace, outputs, zu.plain_logits(folder, raw, requests), "float32")
