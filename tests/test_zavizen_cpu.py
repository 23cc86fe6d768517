"""Zavizen without a GPU: configuration, the spec and schedule that are built from it, what its layers ask the cache
manager for (pages of the attention side, state shares of mixers side by side, the state-space mixer's memory and
convolution inputs), and the engine's host side (batch layout, cache and state manager, step function, scheduler,
replay, generation) driven through the stand-in kernels against the plain implementation; and the plain
implementation's own mechanisms against closed forms."""

import pytest
import torch

import replay_util as ru
import zavizen_util as zu
from plain import zavizen_plain as plain

LENGTHS = (1, 2, 19, 47, 130)


def test_configuration_reads_every_size_and_names_what_is_wrong():
    from ampere_kv_engine_b200.config.model_config import ConfigError
    from ampere_kv_engine_b200.models.registry import config_from_dict
    arch, cfg = config_from_dict(zu.config("Z1"))
    assert arch.name == "Zavizen" and cfg.vocab_size == 193 and cfg.width == 72 and len(cfg.layers) == 4
    assert cfg.streams == 3 and cfg.loop == {"start": 1, "stop": 3, "times": 2} and cfg.norm_eps == 1e-5
    assert config_from_dict(cfg.to_dict())[1] == cfg
    assert config_from_dict(zu.config("Z2"))[1].loop is None
    for path, value, word in ((("layers", 1, "type"), "lstm", "type"), (("layers", 0, "mixer", "state"), 0, "state"),
                              (("layers", 0, "mixer", "groups"), 3, "groups"), (("norm", "eps"), 0, "eps"),
                              (("layers", 0, "mixer", "norm_groups"), 5, "norm_groups"),
                              (("layers", 1, "mlp", "kind"), "routed", "kind"), (("vocab",), -1, "vocab"),
                              (("streams",), 0, "streams"), (("streams",), 9, "streams"),
                              (("layers", 1, "mixer", "left", "kv_heads"), 3, "kv_heads"),
                              (("layers", 1, "mixer", "left", "rot", "dims"), 15, "dims"),
                              (("layers", 1, "mixer", "left", "rot", "scaling", "factor"), 0, "factor"),
                              (("layers", 1, "mixer", "right", "decay"), [0.5, 0.9], "decay"),
                              (("layers", 1, "mixer", "right", "rot", "dims"), 14, "dims"),
                              (("layers", 0, "mlp", "router", "top"), 5, "top"),
                              (("layers", 0, "mlp", "router", "groups", "count"), 4, "groups"),
                              (("loop", "stop"), 5, "stop"), (("loop", "times"), 0, "times")):
        raw = zu.config("Z1")
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
    arch, cfg = config_from_dict(zu.config("Z1"))
    spec = arch.build_spec(cfg)
    assert spec.streams == 3 and all(l.block == "hyper" for l in spec.layers)
    assert [l.mixer.kind for l in spec.layers] == ["mamba2", "parallel", "parallel", "mamba2"]
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 1, 2, 3] and not any(e.add_embedding for e in spec.schedule)
    assert [None if l.feed_forward is None else l.feed_forward.kind for l in spec.layers] == \
        ["routed_experts", "gated_mlp", None, "routed_experts"]
    moe = spec.layers[0].feed_forward.params
    assert moe["score"] == "softmax" and moe["group_top"] == 1 and moe["groups"] == 3 and moe["keep_groups"] == 2
    assert moe["activation"] == "silu" and not moe["correction"] and moe["shared"] == {"intermediate_size": 40}
    left = spec.layers[1].mixer.params["left"].params
    assert left["row_norm"] and left["position_encoding"].params["scaling"] == {"factor": 2.0}
    assert spec.layers[2].mixer.params["left"].params["position_encoding"].params["scaling"] == {"factor": 1.0}
    model = DecoderModel(spec, dtype=torch.float32, device="cpu")
    specs = model.param_specs()
    wanted = {name for name, ps in specs.items() if not ps.optional}
    assert {"embed", "final.norm", "head", "l0.norm1", "l0.ls2", "l0.hc1.in", "l0.hc2.mix", "l0.mix.in", "l0.mix.conv",
            "l0.mix.conv.b", "l0.mix.A_log", "l0.mix.D", "l0.mix.dt_bias", "l0.mix.norm", "l0.mlp.e5.down",
            "l0.mlp.router", "l0.mlp.shared.up", "l1.mix.left.q.norm", "l1.mix.left.k.norm", "l1.mix.left.out",
            "l1.mix.right.out", "l1.mix.right.g", "l1.mlp.gate", "l3.mlp.e3.gate"} <= wanted
    assert not ({"l3.mlp.shared.up", "l2.mlp.gate", "l1.mix.right.norm"} & set(specs)) and specs["l2.hc2.mix"].optional
    assert specs["l0.mix.in"].shape == (2 * 48 + 2 * 2 * 20 + 4, 72) and specs["l0.mix.conv"].shape == (48 + 80, 3)
    assert specs["l1.mix.left.q.norm"].shape == (96,) and specs["l1.mix.left.k.norm"].shape == (48,)
    assert specs["l0.hc1.mix"].shape == (3, 3) and specs["l1.mix.left.o"].shape == (72, 64)
    caches = model.cache_specs()
    assert len(caches) == len(spec.schedule)
    memory = ops.linear_scan_state_floats(4, 20, 12)
    assert caches[0].kind == "none" and caches[0].state_shape == ((memory + 2 * 128 + 3) // 4 * 4,)
    assert caches[1].kind == "full" and caches[1].state_shape == (ops.linear_scan_state_floats(3, 12, 20),)
    assert [t.width for t in caches[1].stored()] == [24, 16]
    # the two appearances of a parallel layer have a cache each in one group
    assert caches[1].group_key() == caches[3].group_key() != caches[2].group_key()


def test_plain_mechanisms_against_closed_forms():
    g = torch.Generator().manual_seed(0)
    # retention: the decayed sum of outer products, keys scaled by dim^-1/2, no rotation when the angle is zero
    T, D, V = 7, 4, 3
    w = {"m.q": torch.randn(D, 5, generator=g, dtype=torch.float64), "m.k": torch.randn(D, 5, generator=g, dtype=torch.float64),
         "m.v": torch.randn(V, 5, generator=g, dtype=torch.float64), "m.g": torch.randn(V, 5, generator=g, dtype=torch.float64),
         "m.o": torch.eye(V, dtype=torch.float64)}
    h = torch.randn(T, 5, generator=g, dtype=torch.float64)
    m = {"heads": 1, "dim": D, "vdim": V, "decay": [0.8], "rot": {"dims": 2, "base": 10.0}}
    q = plain.rotate_half((h @ w["m.q"].T).view(T, 1, D), m["rot"])[:, 0]
    k = plain.rotate_half((h @ w["m.k"].T).view(T, 1, D), m["rot"])[:, 0] * D ** -0.5
    v = h @ w["m.v"].T
    o = torch.stack([sum(0.8 ** (t - s) * (q[t] @ k[s]) * v[s] for s in range(t + 1)) for t in range(T)])
    want = plain.rms_norm(o, None, 1e-6) * plain.silu(h @ w["m.g"].T)
    torch.testing.assert_close(plain.retention(h, w, "m", m, 1e-6), want)
    # a rotation keeps a pair's length and turns the pair (i, i + dims / 2) by position * frequency
    x = torch.zeros(3, 1, 6, dtype=torch.float64)
    x[:, 0, 1] = 1.0
    r = plain.rotate_half(x, {"dims": 4, "base": 100.0, "scaling": {"factor": 2.0}})
    angle = torch.arange(3, dtype=torch.float64) * (100.0 ** -0.5) / 2.0
    torch.testing.assert_close(r[:, 0, 1], torch.cos(angle), atol=1e-6, rtol=0)
    torch.testing.assert_close(r[:, 0, 3], torch.sin(angle), atol=1e-6, rtol=0)
    assert float(r[:, 0, [0, 2, 4, 5]].abs().max()) == 0.0
    # the short convolution: an impulse comes out as the taps, last column first
    weight = torch.tensor([[1.0, 2.0, 3.0]], dtype=torch.float64)
    imp = torch.zeros(5, 1, dtype=torch.float64)
    imp[1] = 1.0
    assert plain.short_convolution(imp, weight, torch.zeros(1, dtype=torch.float64))[:, 0].tolist() == [0, 3, 2, 1, 0]
    # routing: the best group's experts only; weights sum to the scale
    logits = torch.tensor([[0.0, 5.0, 4.9, 4.8, 1.0, 0.5]], dtype=torch.float64)
    chosen, weights = plain.route(logits, {"experts": 6, "top": 2, "scale": 1.5, "groups": {"count": 3, "keep": 1}})
    assert sorted(chosen[0].tolist()) == [0, 1] and float(weights.sum()) == pytest.approx(1.5)
    chosen, _ = plain.route(logits, {"experts": 6, "top": 2, "scale": 1.5, "groups": {"count": 3, "keep": 2}})
    assert sorted(chosen[0].tolist()) == [1, 2]
    # the order of layers
    assert plain.schedule({"layers": [0] * 4, "loop": {"start": 1, "stop": 3, "times": 2}}) == [0, 1, 2, 1, 2, 3]
    # one copy of the stream read and written with ones is a plain residual sum
    xs = torch.randn(1, 4, 6, generator=g, dtype=torch.float64)
    wts = {"c.in": torch.ones(1, dtype=torch.float64), "c.out": torch.ones(1, dtype=torch.float64),
           "c.mix": torch.ones(1, 1, dtype=torch.float64)}
    new = plain.sublayer(xs, wts, "c", torch.ones(6, dtype=torch.float64), torch.zeros(6, dtype=torch.float64), 1e-6,
                         lambda u: 2.0 * u)
    torch.testing.assert_close(new[0], xs[0] + 2.0 * plain.rms_norm(xs[0], None, 1e-6))


@pytest.mark.parametrize("name", ["Z1", "Z2"])
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
    _loose(trace, outputs, expected)


def _loose(trace, outputs, expected):
    saved = dict(ru.TOL["float32"])
    ru.TOL["float32"] = dict(atol=2e-4, rtol=2e-4)
    try:
        ru.compare(trace, outputs, expected, "float32")
    finally:
        ru.TOL["float32"] = saved


def test_greedy_generation_through_the_scheduler(fake_ext):
    from ampere_kv_engine_b200.engine.engine import Engine
    raw, page = zu.CONFIGS["Z1"]
    folder = zu.model_folder("Z1")
    engine = Engine.from_pretrained(folder, dtype="float32", device="cpu", page_size=page, num_pages=16,
                                    max_batch_tokens=24, max_seqs=4)
    prompts = [torch.randint(0, raw["vocab"], (n,), generator=torch.Generator().manual_seed(n)).tolist()
               for n in (3, 30, 61, 1, 17)]
    got = engine.generate(prompts, max_new_tokens=6, ignore_eos=True)
    w = zu.plain_weights(folder)
    assert got == [plain.greedy_generate(raw, w, p, 6) for p in prompts]
    assert engine.manager.free_pages() == [16] * len(engine.manager.groups)
    engine.manager.check_invariants()
    # the same prompts again land in state slots and pages that were used before and give the same tokens
    assert engine.generate(prompts, max_new_tokens=6, ignore_eos=True) == got


def test_a_model_of_state_space_layers_alone_has_no_pages(fake_ext, tmp_path):
    from ampere_kv_engine_b200.engine.engine import Engine
    from ampere_kv_engine_b200.models.registry import config_from_dict
    from ampere_kv_engine_b200.weights.random_init import write_random_model
    raw = zu.config("Z2")
    raw["layers"] = raw["layers"][1:]
    _, cfg = config_from_dict(raw)
    folder = write_random_model(cfg, 4, str(tmp_path / "ssm"), torch.float32)
    engine = Engine.from_pretrained(folder, dtype="float32", device="cpu", page_size=16, num_pages=8, max_seqs=2)
    assert not engine.manager.groups
    prompt = [5, 7, 11, 13, 17, 19, 23, 29, 31]
    got = engine.generate([prompt], max_new_tokens=5, ignore_eos=True)
    assert got == [plain.greedy_generate(raw, zu.plain_weights(folder), prompt, 5)]


@pytest.mark.parametrize("seed", [1, 4, 7, 11])
def test_random_configuration_on_the_stand_in_kernels(fake_ext, seed):
    """Layer orders, sizes, copies of the stream, loops and routers drawn from the seed, in a mixed trace whose pages
    and state slots are used again."""
    folder = zu.random_model_folder(seed)
    raw, page = zu.CONFIGS[f"random{seed}"]
    requests = ru.make_requests(raw["vocab"], (1, 2, 23, 61, 90, 37), seed=seed)
    expected = zu.plain_logits(folder, raw, requests)
    trace = ru.trace_mixed(requests, 64 * 5, seed=seed)
    outputs = ru.run_inprocess(folder, "float32", trace, 64 * 5, page_size=page)
    _loose(trace, outputs, expected)
