"""Small Zavizen configurations of the tests, model folders with random weights for them (made in a temporary folder,
never committed) and the plain implementation's logits.

The configurations differ from one another in every size, in the order of their layers and in what is present:

* ``Z1``: a state-space layer first (four heads on two groups, three taps, two norm groups) with six experts in three
  groups of which two are kept and a shared expert; then two parallel layers (values narrower than keys and as wide;
  two and one query heads per key head; rotation over part of a head with scaled frequencies and over all of it
  without) of which one has a dense feed-forward and one none; a state-space layer with one group, two taps and four
  experts without groups or a shared one, top 1; layers 1 and 2 run twice in a row; three copies of the stream.
* ``Z2``: one copy of the stream, no loop; a parallel layer with one head on each side; a state-space layer without a
  convolution (one tap) whose experts are all chosen (top equals the experts); a dense feed-forward.
* ``Z3``: sizes at which the 16-byte paths, the tensor-core attention kernels and the small-batch product kernel run:
  attention heads of 128, memories of 64 x 32 and 128 x 64, experts with widths that are multiples of eight; the
  whole model is one loop run twice; four copies of the stream.
* ``Z4``: a width at which the row-wise kernels share a row among the blocks of a cluster on steps of few tokens
  (the stream's write, read and norm; the two normed outputs; the norms over whole q and k rows; the state-space
  preparation cut over channels): width 512, ten q and k heads, 512 convolved channels.

The folders' tensors are made so that mechanisms matter: copies of the stream mix mostly with themselves, routers are
scaled up so that choices vary and are rarely close, step biases spread so that some state-space heads keep their
memory for hundreds of tokens, query and key norm weights scaled up so that single keys can win the softmax.
"""

from __future__ import annotations

import copy
import functools
import os
import tempfile

import torch
from safetensors.torch import load_file, save_file

from plain import zavizen_plain as plain


def _rot(dims, base, factor=None):
    rot = {"dims": dims, "base": base}
    if factor is not None:
        rot["scaling"] = {"factor": factor}
    return rot


def _parallel(left, right):
    heads, kv_heads, dim, vdim, scale, lrot = left
    rheads, rdim, rvdim, decay, rrot = right
    return {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": lrot},
            "right": {"heads": rheads, "dim": rdim, "vdim": rvdim, "decay": list(decay), "rot": rrot}}


def _mamba(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def _moe(experts, top, ff, scale, groups=None, shared=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        mlp["shared"] = {"ff": shared}
    return mlp


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


Z1 = {
    "architecture": "Zavizen", "vocab": 193, "width": 72, "norm": {"eps": 1e-5}, "streams": 3,
    "loop": {"start": 1, "stop": 3, "times": 2},
    "layers": [
        _layer("mamba2", _mamba(4, 12, 20, 2, 3, 2), _moe(6, 2, 24, 2.0, groups=(3, 2), shared=40)),
        _layer("parallel", _parallel((4, 2, 24, 16, 0.2, _rot(16, 500.0, 2.0)),
                                     (3, 12, 20, (0.5, 0.93, 0.999), _rot(12, 100.0))), _dense(96)),
        _layer("parallel", _parallel((3, 3, 16, 16, 0.25, _rot(8, 10000.0)),
                                     (1, 24, 8, (0.97,), _rot(8, 1000.0, 8.0))), None),
        _layer("mamba2", _mamba(2, 40, 8, 1, 2, 1), _moe(4, 1, 32, 1.0)),
    ],
}
Z2 = {
    "architecture": "Zavizen", "vocab": 97, "width": 48, "norm": {"eps": 1e-6}, "streams": 1,
    "layers": [
        _layer("parallel", _parallel((1, 1, 32, 20, 0.18, _rot(32, 100.0)), (1, 8, 40, (1.0,), _rot(2, 50.0))),
               _moe(3, 3, 16, 0.7, shared=8)),
        _layer("mamba2", _mamba(3, 16, 12, 3, 1, 3), _dense(64)),
        _layer("mamba2", _mamba(6, 8, 36, 2, 3, 1), None),
    ],
}
Z3 = {
    "architecture": "Zavizen", "vocab": 320, "width": 256, "norm": {"eps": 1e-6}, "streams": 4,
    "loop": {"start": 0, "stop": 3, "times": 2},
    "layers": [
        _layer("parallel", _parallel((8, 2, 128, 128, 0.09, _rot(64, 1000000.0, 4.0)),
                                     (4, 64, 32, (0.7, 0.9, 0.99, 1.0), _rot(64, 10000.0))), _dense(384)),
        _layer("mamba2", _mamba(4, 64, 128, 1, 4, 2), _moe(8, 3, 128, 1.25, groups=(4, 2), shared=64)),
        _layer("parallel", _parallel((2, 1, 64, 64, 0.125, _rot(32, 10000.0)), (2, 128, 64, (0.95, 0.999), _rot(16, 100.0))),
               _moe(16, 4, 64, 2.5, groups=(4, 2))),
    ],
}
Z4 = {
    "architecture": "Zavizen", "vocab": 150, "width": 512, "norm": {"eps": 1e-6}, "streams": 2,
    "layers": [
        _layer("parallel", _parallel((8, 2, 32, 32, 0.2, _rot(16, 10000.0, 2.0)), (2, 32, 48, (0.9, 0.99), _rot(32, 500.0))),
               _dense(128)),
        _layer("mamba2", _mamba(4, 96, 32, 2, 4, 1), _moe(4, 2, 64, 1.0, shared=32)),
    ],
}
CONFIGS = {"Z1": (Z1, 16), "Z2": (Z2, 32), "Z3": (Z3, 16), "Z4": (Z4, 16)}


def config(name: str) -> dict:
    return copy.deepcopy(CONFIGS[name][0])


def sharpen(tensors: dict, cfg, seed: int) -> dict:
    """Random tensors made so that the mechanisms matter (see the module's text)."""
    g = torch.Generator().manual_seed(seed + 100)
    s = cfg.streams
    for i, layer in enumerate(cfg.layers):
        for which in (1, 2):
            if f"l{i}.hc{which}.mix" in tensors:
                tensors[f"l{i}.hc{which}.mix"] = 0.8 * torch.eye(s) + 0.25 * torch.rand(s, s, generator=g)
                tensors[f"l{i}.hc{which}.in"] = 0.3 + torch.rand(s, generator=g)
                tensors[f"l{i}.hc{which}.out"] = 0.5 + torch.rand(s, generator=g)
        p = f"l{i}.mix"
        if layer.type == "mamba2":
            heads = layer.mixer["heads"]
            # steps from about 0.002 to 0.7: some heads forget within a few tokens, some keep hundreds
            tensors[f"{p}.dt_bias"] = torch.linspace(-6.0, 0.0, heads)[torch.randperm(heads, generator=g)]
            tensors[f"{p}.in"] = tensors[f"{p}.in"] * 4.0
            tensors[f"{p}.conv"] = tensors[f"{p}.conv"] - 0.3
        else:
            tensors[f"{p}.left.q.norm"] = tensors[f"{p}.left.q.norm"] * 1.5
            tensors[f"{p}.left.k.norm"] = tensors[f"{p}.left.k.norm"] * 1.5
            for name in ("q", "k", "v", "g"):
                tensors[f"{p}.right.{name}"] = tensors[f"{p}.right.{name}"] * 10.0
        if f"l{i}.mlp.router" in tensors:
            tensors[f"l{i}.mlp.router"] = tensors[f"l{i}.mlp.router"] * 40.0
    return tensors


@functools.lru_cache(maxsize=None)
def model_folder(name: str, seed: int = 3) -> str:
    from ampere_kv_engine_b200.models.registry import config_from_dict
    from ampere_kv_engine_b200.weights.random_init import write_random_model
    _, cfg = config_from_dict(config(name))
    out = tempfile.mkdtemp(prefix=f"zavizen_{name}_")
    write_random_model(cfg, seed, out, torch.float32)
    path = os.path.join(out, "model.safetensors")
    tensors = sharpen(load_file(path), cfg, seed)
    # bfloat16-representable values: both precisions then run on the same weights
    save_file({k: v.to(torch.bfloat16).to(torch.float32).contiguous() for k, v in tensors.items()}, path,
              metadata={"format": "pt"})
    return out


def plain_weights(folder: str) -> dict:
    return {k: v.double() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}


def plain_logits(folder: str, raw: dict, requests: dict[str, list[int]]) -> dict[str, torch.Tensor]:
    """float64 logits of every request as a whole sequence, as float32."""
    w = plain_weights(folder)
    return {rid: plain.forward(raw, w, toks).float() for rid, toks in requests.items()}


_DECISIVE: dict = {}


def decisive_requests(folder: str, raw: dict, lengths, seed: int, margin: float = 0.5, tries: int = 400
                      ) -> dict[str, list[int]]:
    """Random requests of the given lengths in which no expert choice is a close call: for every token and routed
    layer the chosen experts (and kept groups) lead the others by at least ``margin`` in the router's logits in the
    plain implementation, so that the rounding of the layers before the router cannot change the choice.  Found by trying
    continuations of a few tokens at a time."""
    key = (folder, tuple(lengths), seed, margin)
    if key in _DECISIVE:
        return copy.deepcopy(_DECISIVE[key])
    w = plain_weights(folder)
    g = torch.Generator().manual_seed(seed)
    routed = any((l.get("mlp") or {}).get("kind") == "moe" for l in raw["layers"])
    out = {}
    for i, n in enumerate(lengths):
        toks: list[int] = []
        while len(toks) < n:
            for _ in range(tries):
                cand = toks + torch.randint(0, raw["vocab"], (min(4, n - len(toks)),), generator=g).tolist()
                margins: list = []
                if routed:
                    plain.forward(raw, w, cand, margins=margins)
                if all(float(m[len(toks):].min()) >= margin for m in margins):
                    toks = cand
                    break
            else:
                raise AssertionError("no decisive continuation found; lower the margin")
        out[f"r{i}"] = toks
    _DECISIVE[key] = copy.deepcopy(out)
    return out


def random_config(seed: int) -> dict:
    """A configuration whose every size, constant, layer order and loop is drawn from the seed: three to six layers of
    either mixer (at least one of each), one to five copies of the stream, widths and head sizes that are no multiples
    of 16, scaled frequencies or none, dense or routed feed-forwards or none, groups of experts and shared experts or
    none, a loop or none."""
    g = torch.Generator().manual_seed(2000 + seed)
    pick = lambda *options: options[int(torch.randint(0, len(options), (1,), generator=g))]   # noqa: E731
    num = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=g))                    # noqa: E731

    def rot(dim):
        return _rot(2 * num(1, dim // 2), pick(100.0, 10000.0, 1000000.0), pick(None, None, 2.0, 4.0, 16.0))

    def parallel():
        kv = num(1, 3)
        dim = pick(8, 12, 16, 24, 32, 64)
        rheads = num(1, 4)
        rdim = pick(4, 8, 12, 20, 32, 48, 64)
        return _parallel((kv * num(1, 3), kv, dim, pick(8, 12, 16, 20, 32, dim), round(dim ** -0.5 * pick(0.8, 1.0, 1.5), 4),
                          rot(dim)),
                         (rheads, rdim, pick(4, 8, 12, 20, 32, 40, 64),
                          [round(1.0 - 0.5 ** num(1, 10), 6) for _ in range(rheads)], rot(rdim)))

    def mamba():
        groups = num(1, 3)
        heads = groups * num(1, 3)
        vdim = pick(4, 8, 12, 20, 32, 40)
        parts = pick(1, 1, 2, heads)
        if (heads * vdim) % parts:
            parts = 1
        return _mamba(heads, vdim, pick(4, 8, 12, 20, 32, 48, 64), groups, num(1, 5), parts)

    def mlp():
        kind = pick("none", "dense", "moe", "moe")
        if kind == "none":
            return None
        if kind == "dense":
            return _dense(pick(32, 56, 64, 100))
        count = pick(1, 1, 2, 3)
        per = num(1, 4)
        keep = num(1, count)
        return _moe(count * per, num(1, keep * per), pick(8, 24, 40), pick(0.5, 1.0, 2.5),
                    groups=None if count == 1 and pick(True, False) else (count, keep), shared=pick(None, 16, 48))

    kinds = ["parallel", "mamba2"] + [pick("parallel", "mamba2") for _ in range(num(1, 4))]
    kinds = [kinds[i] for i in torch.randperm(len(kinds), generator=g).tolist()]
    layers = [_layer(kind, parallel() if kind == "parallel" else mamba(), mlp()) for kind in kinds]
    raw = {"architecture": "Zavizen", "vocab": num(50, 300), "width": pick(24, 40, 48, 72, 96, 128),
           "norm": {"eps": pick(1e-5, 1e-6)}, "streams": num(1, 5), "layers": layers}
    if pick(True, True, False):
        start = num(0, len(layers) - 1)
        raw["loop"] = {"start": start, "stop": num(start + 1, len(layers)), "times": num(2, 3)}
    return raw


def random_model_folder(seed: int) -> str:
    name = f"random{seed}"
    if name not in CONFIGS:
        CONFIGS[name] = (random_config(seed), (8, 16, 32)[seed % 3])
    return model_folder(name, seed=seed)
