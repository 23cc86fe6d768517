"""Renadra without a GPU: configuration, the spec and schedule that are built from it, what its layers ask the cache
manager for (pages of kept first keys, state shares of mixers side by side, the embedding's previous token), and the
engine's host side (batch layout, cache and state manager, step function, scheduler, replay, generation) driven
through the stand-in kernels against the plain implementation; and the plain implementation's own mechanisms against
closed forms."""

import math

import pytest
import torch

import renadra_util as zu
import replay_util as ru
from plain import renadra_plain as plain

LENGTHS = (1, 2, 19, 47, 130)


def test_configuration_reads_every_size_and_names_what_is_wrong():
    from ampere_kv_engine_b200.config.model_config import ConfigError
    from ampere_kv_engine_b200.models.registry import config_from_dict
    arch, cfg = config_from_dict(zu.config("R1"))
    assert arch.name == "Renadra" and cfg.vocab_size == 211 and cfg.width == 72 and len(cfg.layers) == 4
    assert cfg.embedding_scale == 3.0 and cfg.bigram == {"buckets": 97, "mul_prev": 31, "mul_cur": 7}
    assert cfg.loop == {"start": 1, "stop": 3, "times": 3} and cfg.norm_eps == 1e-5
    assert config_from_dict(cfg.to_dict())[1] == cfg
    assert config_from_dict(zu.config("R2"))[1].loop is None
    for path, value, word in ((("layers", 1, "type"), "lstm", "type"), (("layers", 1, "mixer", "dim"), 0, "dim"),
                              (("layers", 2, "mixer", "kv_heads"), 4, "kv_heads"), (("norm", "eps"), 0, "eps"),
                              (("layers", 0, "mlp", "kind"), "routed", "kind"), (("vocab",), -1, "vocab"),
                              (("layers", 0, "mixer", "left", "vdim"), 16, "vdim"),
                              (("layers", 0, "mixer", "left", "rot", "dims"), 15, "dims"),
                              (("layers", 0, "mixer", "left", "rot", "scaling", "factor"), 0, "factor"),
                              (("layers", 0, "mixer", "left", "mask", "keep_first"), -1, "keep_first"),
                              (("layers", 0, "mixer", "right", "decay"), [0.5, 0.9], "decay"),
                              (("layers", 2, "mixer", "rot", "dims"), 18, "dims"),
                              (("layers", 2, "mixer", "mask", "size"), 0, "size"),
                              (("loop", "stop"), 5, "stop"), (("loop", "times"), 0, "times"),
                              (("embedding", "bigram", "buckets"), 0, "buckets")):
        raw = zu.config("R1")
        node = raw
        for key in path[:-1]:
            node = node[key]
        node[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            config_from_dict(raw)


def test_spec_schedules_the_loop_and_gives_layers_their_parts():
    from ampere_kv_engine_b200.kernels import ops
    from ampere_kv_engine_b200.models.decoder import DecoderModel
    from ampere_kv_engine_b200.models.registry import config_from_dict
    arch, cfg = config_from_dict(zu.config("R1"))
    spec = arch.build_spec(cfg)
    assert [l.mixer.kind for l in spec.layers] == ["parallel", "hgrn2", "rotary_attention", "hgrn2"]
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [e.add_embedding for e in spec.schedule] == [False, False, False, True, False, True, False, False]
    assert [None if l.feed_forward is None else l.feed_forward.kind for l in spec.layers] == \
        ["gated_mlp", None, "gated_mlp", "gated_mlp"]
    left = spec.layers[0].mixer.params["left"].params
    assert left["keep_first"] == 5 and left["window"] == 13 and left["weights"] == "sigmoid" and left["value_from_key"]
    assert left["position_encoding"].params["layout"] == "half" and left["position_encoding"].params["scaling"]
    assert spec.layers[2].mixer.params["position_encoding"].params["layout"] == "pairs"
    model = DecoderModel(spec, dtype=torch.float32, device="cpu")
    specs = model.param_specs()
    wanted = {name for name, ps in specs.items() if not ps.optional}
    assert {"embed", "bigram", "final.norm", "head", "l0.mix.left.q", "l0.mix.left.q.b", "l0.mix.left.k.b",
            "l0.mix.left.pb", "l0.mix.left.o", "l0.mix.right.g", "l0.mix.right.norm", "l1.mix.f", "l1.mix.f.b",
            "l1.mix.lower", "l1.mix.norm", "l2.mix.v.b", "l2.mix.o.b", "l3.mlp.down"} <= wanted
    assert not ({"l0.mix.left.v", "l0.mix.left.o.b", "l1.mlp.gate"} & set(specs)) and specs["l1.norm2"].optional
    assert specs["bigram"].shape == (98, 72) and specs["l1.mix.norm"].shape == (12,)
    assert specs["l0.mix.right.norm"].shape == (60,) and specs["l0.mix.left.pb"].shape == (4,)
    # one cache view per schedule position and one more for the embedding's previous token
    caches = model.cache_specs()
    assert len(caches) == len(spec.schedule) + 1 and caches[-1].state_shape == (1,) and caches[-1].kind == "none"
    assert caches[0].kind == "window" and caches[0].keep_first == 5 and caches[0].window == 13
    assert caches[0].state_shape == (ops.linear_scan_state_floats(3, 12, 20),)
    assert caches[1].state_shape == (ops.linear_scan_state_floats(3, 20, 12),) and caches[1].kind == "none"
    # the three appearances of the attention layer share one cache group and have a cache each
    assert caches[2].group_key() == caches[4].group_key() == caches[6].group_key() != caches[0].group_key()


def test_kept_first_pages_stay_while_pages_behind_the_window_come_back():
    from ampere_kv_engine_b200.cache.manager import CacheManager
    from ampere_kv_engine_b200.parts.base import CacheSpec
    spec = CacheSpec(kind="window", num_kv_heads=1, head_dim=8, window=6, keep_first=5)
    m = CacheManager([spec], [None], page_size=4, num_pages=12, max_seqs=2, allocate_storage=False)
    assert m.groups[0].kept_pages == 2
    a = m.open("a")
    held = []
    for step in range(30):
        m.reserve(a, 1)
        m.commit(a, 1)
        m.check_invariants()
        pages = a.pages[0]
        assert pages[0] >= 0 and (len(pages) < 2 or pages[1] >= 0), "a page of the kept first keys was given back"
        # every key the next query can see is backed: the first five, and the window
        for key in list(range(min(5, a.length))) + list(range(max(0, a.length - 5), a.length)):
            m.slot_of(a, 0, key)
        held.append(len(a.held_pages(0)))
    assert max(held) <= 2 + 3 and held[-1] <= 2 + 3            # two kept pages and what a window of six touches
    assert a.pages[0][2] == -1 and a.pages[0][3] == -1
    # a request whose pool is smaller than its length runs on: pages are used again
    b = m.open("b")
    for _ in range(60):
        m.reserve(b, 3)
        m.commit(b, 3)
    m.check_invariants()
    m.close(a)
    m.close(b)
    assert m.free_pages() == [12]
    # the budget of admission counts the kept pages
    assert m.pages_for_tokens(1000, chunk=8)[0] >= 2 + (6 + 8) // 4
    with pytest.raises(ValueError, match="window"):
        CacheManager([CacheSpec(kind="full", num_kv_heads=1, head_dim=8, keep_first=3)], [None], page_size=4,
                     num_pages=4, max_seqs=1, allocate_storage=False)


def test_plain_mechanisms_against_closed_forms():
    # a constant decay: the memory is the decayed sum of outer products
    g = torch.Generator().manual_seed(0)
    T, D, V = 9, 4, 3
    q, k, v = (torch.randn(T, n, generator=g, dtype=torch.float64) for n in (D, D, V))
    out = plain.decayed_memory(q, k, v, torch.full((T, D), 0.8, dtype=torch.float64))
    want = torch.stack([sum(0.8 ** (t - s) * (q[t] @ k[s]) * v[s] for s in range(t + 1)) for t in range(T)])
    torch.testing.assert_close(out, want)
    # a forget gate of one keeps a row as it is, a gate of zero replaces it with the new value
    f = torch.tensor([[0.0, 1.0]] * 3, dtype=torch.float64)
    vals = torch.tensor([[1.0], [2.0], [3.0]], dtype=torch.float64)
    out = plain.decayed_memory(torch.ones(3, 2, dtype=torch.float64), 1.0 - f, vals, f)
    torch.testing.assert_close(out[:, 0], torch.tensor([1.0, 2.0, 3.0], dtype=torch.float64))
    # the rescaled frequencies: fast pairs untouched, slow pairs divided by the factor, the factor on cos and sin
    freq, factor = plain.rotary_frequencies({"dims": 16, "base": 10000.0,
                                             "scaling": {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 1.0}})
    base = 10000.0 ** (-2.0 * torch.arange(8, dtype=torch.float64) / 16)
    assert factor == pytest.approx(0.1 * math.log(4.0) + 1.0)
    assert freq[0] == base[0] and freq[-1] == pytest.approx(float(base[-1]) / 4.0)
    assert all(base[i] / 4.0 <= freq[i] <= base[i] for i in range(8))
    # both layouts turn a pair by the same angle
    x = torch.randn(5, 1, 8, generator=g, dtype=torch.float64)
    rot = {"dims": 8, "base": 100.0}
    half, pairs = plain.rotate(x, rot, "half"), plain.rotate(x[..., [0, 4, 1, 5, 2, 6, 3, 7]], rot, "pairs")
    torch.testing.assert_close(half[..., [0, 4, 1, 5, 2, 6, 3, 7]], pairs)
    # the window with kept first keys
    see = plain.visible(12, 3, 2)
    assert see[10].tolist() == [True, True] + [False] * 6 + [True, True, True, False]
    # the order of layers
    assert plain.layer_order({"layers": [0] * 4, "loop": {"start": 1, "stop": 3, "times": 2}}) == \
        [(0, False), (1, False), (2, False), (1, True), (2, False), (3, False)]


@pytest.mark.parametrize("name", ["R1", "R2"])
@pytest.mark.parametrize("mode", ["whole", "last32", "portions", "mixed"])
def test_replay_matches_plain(fake_ext, name, mode):
    raw, page = zu.CONFIGS[name]
    folder = zu.model_folder(name)
    requests = ru.make_requests(raw["vocab"], LENGTHS + ((70, 45) if mode == "mixed" else ()), seed=11)
    expected = zu.plain_logits(folder, raw, requests)
    max_tokens = 64 * 6
    trace = {"whole": ru.trace_whole, "last32": ru.trace_last_decoded, "portions": ru.trace_portions,
             "mixed": lambda r: ru.trace_mixed(r, max_tokens, seed=5)}[mode](requests)
    outputs = ru.run_inprocess(folder, "float32", trace, max_tokens, page_size=page)
    ru.compare(trace, outputs, expected, "float32")


def test_greedy_generation_through_the_scheduler(fake_ext):
    from ampere_kv_engine_b200.engine.engine import Engine
    raw, page = zu.CONFIGS["R1"]
    folder = zu.model_folder("R1")
    engine = Engine.from_pretrained(folder, dtype="float32", device="cpu", page_size=page, num_pages=12,
                                    max_batch_tokens=24, max_seqs=4)
    prompts = [torch.randint(0, raw["vocab"], (n,), generator=torch.Generator().manual_seed(n)).tolist()
               for n in (3, 30, 61, 1, 17)]
    got = engine.generate(prompts, max_new_tokens=6, ignore_eos=True)
    w = zu.plain_weights(folder)
    assert got == [plain.greedy_generate(raw, w, p, 6) for p in prompts]
    assert engine.manager.free_pages() == [12] * len(engine.manager.groups)
    engine.manager.check_invariants()
    # the same prompts again land in state slots and pages that were used before and give the same tokens
    assert engine.generate(prompts, max_new_tokens=6, ignore_eos=True) == got


def test_a_model_without_a_pair_table_or_a_loop_keeps_no_embedding_state(fake_ext, tmp_path):
    from ampere_kv_engine_b200.engine.engine import Engine
    from ampere_kv_engine_b200.models.registry import config_from_dict
    from ampere_kv_engine_b200.weights.random_init import write_random_model
    raw = zu.config("R2")
    del raw["embedding"]["bigram"]
    raw["layers"] = [raw["layers"][2], raw["layers"][0]]
    _, cfg = config_from_dict(raw)
    folder = write_random_model(cfg, 4, str(tmp_path / "plainer"), torch.float32)
    engine = Engine.from_pretrained(folder, dtype="float32", device="cpu", page_size=16, num_pages=8, max_seqs=2)
    assert len(engine.model.cache_specs()) == 2
    prompt = [5, 7, 11, 13, 17, 19, 23, 29, 31]
    got = engine.generate([prompt], max_new_tokens=5, ignore_eos=True)
    assert got == [plain.greedy_generate(raw, zu.plain_weights(folder), prompt, 5)]


@pytest.mark.parametrize("seed", [1, 4, 7, 11])
def test_random_configuration_on_the_stand_in_kernels(fake_ext, seed):
    """Layer orders, sizes, windows, kept keys, loops and pair tables drawn from the seed, in a mixed trace whose pages
    and state slots are used again."""
    folder = zu.random_model_folder(seed)
    raw, page = zu.CONFIGS[f"random{seed}"]
    requests = ru.make_requests(raw["vocab"], (1, 2, 23, 61, 90, 37), seed=seed)
    expected = zu.plain_logits(folder, raw, requests)
    trace = ru.trace_mixed(requests, 64 * 5, seed=seed)
    outputs = ru.run_inprocess(folder, "float32", trace, 64 * 5, page_size=page)
    saved = dict(ru.TOL["float32"])
    ru.TOL["float32"] = dict(atol=2e-4, rtol=2e-4)
    try:
        ru.compare(trace, outputs, expected, "float32")
    finally:
        ru.TOL["float32"] = saved
