"""The Zavizen decoder through the engine on the GPU, in both precisions, against the plain implementation: whole
prompts, the last tokens one by one (replayed as CUDA graphs), portions down to two tokens, mixed batches in which
pages and state slots are used again, decoding from the very first token, a key far back that decides the softmax
(at page borders, in a prompt and decoded), seeded random configurations, greedy generation through the engine's
entry point and the command line, and the replay program as a subprocess."""

import json
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch
from safetensors.torch import load_file, save_file

import replay_util as ru
import zavizen_util as zu
from plain import zavizen_plain as plain

pytestmark = pytest.mark.gpu

LENGTHS = (1, 2, 19, 47, 130)
MODES = ["whole", "last32", "portions", "mixed"]


def _check(trace, outputs, expected, dtype):
    """float32: element by element against float64 (recurrences over a hundred tokens and several passes leave a few
    1e-5 of summation order).  bfloat16: every row against its own scale (rounded projections feed gates, steps and
    routers, so a row's rounding error is a few per cent of its scale; a lost state, a wrong page or a wrong copy of
    the stream misses by the row's whole scale and goes on missing in the rows after it).  One row in fifty (at least
    one) may miss: at a sequence's first token a retention head reads out (q . k) v of that one token and is then
    divided by its root mean square, so where q . k happens to be a few thousandths of |q| |k| the rounding of q and k
    decides its sign and with it the head's whole output (seen: -0.027 against 7); and the layers before a router are
    rounded too, so a choice that is no close call in exact arithmetic can still change."""
    if dtype == "bfloat16":
        rows = over = 0
        first = None
        for step, wanted in trace.expect.items():
            vocab = next(iter(expected.values())).shape[1]
            got = torch.from_numpy(outputs[step].copy()).view(-1, vocab)
            assert got.shape[0] == len(wanted), f"step {step}: {got.shape[0]} rows written, {len(wanted)} wanted"
            want = torch.stack([expected[rid][pos] for rid, pos in wanted])
            scale = want.square().mean(dim=1).sqrt()
            rms = (got - want).square().mean(dim=1).sqrt() / scale
            peak = (got - want).abs().max(dim=1).values / scale
            assert torch.isfinite(rms).all(), f"step {step}: a row is not finite"
            bad = ((rms > 0.1) | (peak > 0.3)).nonzero().flatten().tolist()
            rows += len(wanted)
            over += len(bad)
            if bad and first is None:
                first = (step, wanted[bad[0]], float(rms[bad[0]]), float(peak[bad[0]]))
        assert over <= max(1, rows // 50), (f"{over} of {rows} rows differ from the plain implementation; the first: step "
                                            f"{first[0]}, request and position {first[1]}, relative RMS error "
                                            f"{first[2]:.4f} (bound 0.1), worst element {first[3]:.4f} (bound 0.3)")
        return over
    saved = dict(ru.TOL["float32"])
    ru.TOL["float32"] = dict(atol=2e-4, rtol=2e-4)
    try:
        return ru.compare(trace, outputs, expected, "float32")
    finally:
        ru.TOL["float32"] = saved


def _trace(mode, requests, max_tokens):
    return {"whole": ru.trace_whole, "last32": ru.trace_last_decoded, "portions": ru.trace_portions,
            "mixed": lambda r: ru.trace_mixed(r, max_tokens, seed=5)}[mode](requests)


def _requests(folder, raw, lengths, seed, dtype):
    """bfloat16 runs take requests whose expert choices are no close calls."""
    if dtype == "bfloat16":
        return zu.decisive_requests(folder, raw, lengths, seed)
    return ru.make_requests(raw["vocab"], lengths, seed=seed)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("name", ["Z1", "Z2", "Z3"])
def test_replay_matches_plain(name, mode, dtype):
    raw, page = zu.CONFIGS[name]
    folder = zu.model_folder(name)
    requests = _requests(folder, raw, LENGTHS + ((70, 45) if mode == "mixed" else ()), 11, dtype)
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
@pytest.mark.parametrize("mode", ["last32", "mixed"])
def test_a_width_at_which_clusters_share_a_row(mode, dtype):
    """Steps of few tokens at width 512: the blocks of a row's cluster add up their sums through distributed shared
    memory, eagerly and inside captured steps."""
    raw, page = zu.CONFIGS["Z4"]
    folder = zu.model_folder("Z4")
    requests = _requests(folder, raw, (1, 2, 19, 47, 70), 13, dtype)
    expected = zu.plain_logits(folder, raw, requests)
    trace = _trace(mode, requests, 64 * 4)
    outputs, engine = ru.run_on_device(folder, dtype, trace, 64 * 4, page_size=page, max_seqs=4)
    _check(trace, outputs, expected, dtype)
    if mode == "last32":
        assert engine.runner.graph_replays > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["Z1", "Z3"])
def test_decoding_from_the_first_token(name, dtype):
    """Every token a step of its own for 150 positions: the keys were written one at a time over several pages, and
    the memories and the convolutions' inputs are carried through 149 steps."""
    raw, page = zu.CONFIGS[name]
    folder = zu.model_folder(name)
    requests = _requests(folder, raw, (150,), 31, dtype)
    expected = zu.plain_logits(folder, raw, requests)
    trace = ru.trace_last_decoded(requests, last=149)
    outputs, engine = ru.run_on_device(folder, dtype, trace, 192, page_size=page, max_seqs=2)
    _check(trace, outputs, expected, dtype)
    assert engine.runner.graph_replays >= 100


def test_eager_and_captured_single_token_steps_agree():
    """The captured step runs once before it is captured; what that run did to the memories and to the convolutions'
    inputs is undone (a step's tokens enter the state once)."""
    raw, page = zu.CONFIGS["Z1"]
    folder = zu.model_folder("Z1")
    requests = ru.make_requests(raw["vocab"], (40, 33), seed=3)
    trace = ru.trace_last_decoded(requests, last=12)
    with_graphs, engine = ru.run_on_device(folder, "float32", trace, 128, page_size=page, max_seqs=4)
    assert engine.runner.graph_replays > 0
    without, _ = ru.run_on_device(folder, "float32", trace, 128, page_size=page, max_seqs=4, cuda_graphs=False)
    for step in trace.expect:
        torch.testing.assert_close(torch.from_numpy(with_graphs[step]), torch.from_numpy(without[step]), atol=1e-5, rtol=1e-5)


def _far_key_model(tmp, page):
    """One parallel layer whose attention side is made so that the query of token ``ask`` finds the key of token
    ``mark`` wherever it stands: both project onto the same dims beyond the rotated ones, every other token's key is
    small there, and the marked token's value alone is large."""
    from ampere_kv_engine_b200.models.registry import config_from_dict
    from ampere_kv_engine_b200.weights.random_init import write_random_model
    raw = {"architecture": "Zavizen", "vocab": 61, "width": 40, "norm": {"eps": 1e-6}, "streams": 2,
           "layers": [zu._layer("parallel", zu._parallel((2, 1, 16, 24, 1.0, zu._rot(4, 100.0)),
                                                         (1, 8, 8, (0.9,), zu._rot(4, 100.0))), None)]}
    _, cfg = config_from_dict(raw)
    folder = write_random_model(cfg, 9, tmp, torch.float32)
    path = os.path.join(folder, "model.safetensors")
    t = load_file(path)
    mark, ask = 7, 11
    embed = 0.05 * torch.randn(61, 40, generator=torch.Generator().manual_seed(2))
    embed[:, [3, 5]] = 0.0
    embed[:, 7] = 1.0                   # what all other tokens share: their keys point along a dim nobody asks for
    embed[mark] = 0.0
    embed[mark, 3] = 4.0
    embed[ask] = 0.0
    embed[ask, 5] = 4.0
    t["embed"] = embed
    t["l0.norm1"] = torch.zeros(40)
    t["l0.hc1.in"] = torch.tensor([1.0, 0.0])
    wq, wk, wv = torch.zeros(32, 40), torch.zeros(16, 40), 0.01 * torch.randn(24, 40, generator=torch.Generator().manual_seed(3))
    wq[[10, 16 + 10], 5] = 1.0          # dim 10 of both query heads (beyond the 4 rotated dims) answers to `ask`
    wk[10, 3] = 1.0                     # dim 10 of the key answers to `mark`
    wk[12, 7] = 1.0
    wq += 0.01 * torch.randn(32, 40, generator=torch.Generator().manual_seed(4))
    wk += 0.01 * torch.randn(16, 40, generator=torch.Generator().manual_seed(5))
    wv[:, 3] = torch.linspace(-2.0, 2.0, 24)
    t["l0.mix.left.q"], t["l0.mix.left.k"], t["l0.mix.left.v"] = wq, wk, wv
    t["l0.mix.left.q.norm"] = torch.full((32,), 4.0)
    t["l0.mix.left.k.norm"] = torch.full((16,), 4.0)
    t["l0.mix.left.o"] = 0.3 * torch.randn(40, 48, generator=torch.Generator().manual_seed(6))
    t["head"] = 0.3 * torch.randn(61, 40, generator=torch.Generator().manual_seed(7))
    save_file({k: v.to(torch.bfloat16).to(torch.float32).contiguous() for k, v in t.items()}, path,
              metadata={"format": "pt"})
    return raw, folder, mark, ask


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page", [16, 64])
def test_one_key_far_back_decides_at_page_borders_in_prompts_and_decoded(dtype, page, tmp_path):
    _far_key_case(dtype, page, tmp_path)


def _far_key_case(dtype, page, tmp_path, run=True):
    raw, folder, mark, ask = _far_key_model(str(tmp_path / "far"), page)
    w = zu.plain_weights(folder)
    g = torch.Generator().manual_seed(1)
    others = [t for t in range(61) if t not in (mark, ask)]
    length = 700
    for where in (0, 1, page - 1, page, page + 1, 5 * page - 1, 5 * page, length - 40):
        tokens = [others[int(i)] for i in torch.randint(0, len(others), (length,), generator=g)]
        tokens[where] = mark
        asks = [length - 33, length - 2]
        for a in asks:
            tokens[a] = ask
        expected = {"r0": plain.forward(raw, w, tokens).float()}
        # the marked key matters: without it the asking rows' logits are others
        blank = list(tokens)
        blank[where] = others[0]
        moved = (plain.forward(raw, w, blank).float()[asks] - expected["r0"][asks]).abs().max()
        assert float(moved) > 0.5, "the test's weights do not make the far key decide"
        requests = {"r0": tokens}
        if not run:
            continue
        # the first asking token inside the prompt's portion, the second decoded alone
        trace = ru.trace_last_decoded(requests, last=20)
        outputs, engine = ru.run_on_device(folder, dtype, trace, 64 * 12, page_size=page, max_seqs=2)
        _check(trace, outputs, expected, dtype)
        whole = ru.trace_whole(requests)
        outputs, _ = ru.run_on_device(folder, dtype, whole, 64 * 12, page_size=page, max_seqs=2)
        _check(whole, outputs, expected, dtype)


@pytest.mark.parametrize("seed", list(range(1, 11)))
def test_random_configuration(seed):
    folder = zu.random_model_folder(seed)
    raw, page = zu.CONFIGS[f"random{seed}"]
    requests = ru.make_requests(raw["vocab"], (1, 2, 23, 61, 90, 37), seed=seed)
    expected = zu.plain_logits(folder, raw, requests)
    max_tokens = 64 * 5
    mixed = ru.trace_mixed(requests, max_tokens, seed=seed)
    outputs, engine = ru.run_on_device(folder, "float32", mixed, max_tokens, page_size=page, max_seqs=4)
    _check(mixed, outputs, expected, "float32")
    engine.manager.check_invariants()
    tail = ru.trace_last_decoded(requests, last=20)
    outputs, engine = ru.run_on_device(folder, "float32", tail, max_tokens, page_size=page, max_seqs=4)
    _check(tail, outputs, expected, "float32")
    assert engine.runner.graph_replays > 0
    outputs, engine = ru.run_on_device(folder, "bfloat16", mixed, max_tokens, page_size=page, max_seqs=4)
    assert all(np.isfinite(rows).all() for rows in outputs.values())


@pytest.mark.parametrize("name", ["Z1", "Z3"])
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
            assert float(logits.max() - logits[token]) <= 0.08 * float(logits.max() - logits.min()), \
                "bfloat16 picked a token far from the best"
            ids.append(token)


def test_command_line_and_replay_program():
    root = ru.ROOT
    raw, page = zu.CONFIGS["Z1"]
    folder = zu.model_folder("Z1")
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
    _check(trace, outputs, zu.plain_logits(folder, raw, requests), "float32")
