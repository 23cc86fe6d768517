"""Small Renadra configurations of the tests, model folders with random weights for them (made in a temporary folder,
never committed) and the plain implementation's logits.

The configurations differ from one another in every size, in the order of their layers and in what is present:

* ``R1``: a parallel layer first (rotation over fewer dims than the head has, two query heads per key head, five kept
  first keys behind a window of 13; three memory heads of 12 x 20), then hgrn2 without a feed-forward, attention with
  values narrower than keys, hgrn2; layers 1 and 2 run three times in a row; widths that are no multiple of 16.
* ``R2``: attention first with one head; a parallel layer without kept keys and with as many key heads as query
  heads, whose window is longer than two pages; multipliers of the pair table that are both 1; no loop.
* ``R3``: sizes at which the 16-byte paths, the tensor-core attention kernels and the small-batch product kernel run:
  heads of 64 and 128 dims, memories of 128 x 128 and 64 x 32; the whole model is one loop run twice.

Random matrices of N(0, 0.02) would make every score about zero and every forget gate about its lower bound plus a
half; the folders' query and key matrices are scaled up, the lower bounds spread up to 0.999 and the embedding brought
to the size of the branches, so that a wrong key, a lost state or a window that is off by one shows in the logits.
"""

from __future__ import annotations

import copy
import functools
import os
import tempfile

import torch
from safetensors.torch import load_file, save_file

from plain import renadra_plain as plain


def _rot(dims, base, scaling=None):
    rot = {"dims": dims, "base": base}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return rot


def _attention(heads, kv_heads, dim, vdim, scale, window, rot):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window},
            "rot": rot}


def _left(heads, kv_heads, dim, scale, window, keep, softcap, rot):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale, "softcap": softcap,
            "mask": {"size": window, "keep_first": keep}, "rot": rot}


def _memory(heads, dim, vdim, decay=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim}
    if decay is not None:
        m["decay"] = list(decay)
    return m


def _layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


R1 = {
    "architecture": "Renadra", "vocab": 211, "width": 72, "norm": {"eps": 1e-5},
    "embedding": {"scale": 3.0, "bigram": {"buckets": 97, "mul_prev": 31, "mul_cur": 7}},
    "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        _layer("parallel", {"left": _left(4, 2, 24, 0.2, 13, 5, 8.0, _rot(16, 500.0, (4.0, 32, 8.0, 2.0))),
                            "right": _memory(3, 12, 20, (0.5, 0.93, 0.999)), "left_scale": 0.6, "right_scale": 1.3}, 96),
        _layer("hgrn2", _memory(3, 20, 12), None),
        _layer("attention", _attention(6, 3, 16, 8, 0.25, 9, _rot(16, 10000.0)), 40),
        _layer("hgrn2", _memory(2, 8, 40), 64),
    ],
}
R2 = {
    "architecture": "Renadra", "vocab": 97, "width": 48, "norm": {"eps": 1e-6},
    "embedding": {"scale": 1.0, "bigram": {"buckets": 13, "mul_prev": 1, "mul_cur": 1}},
    "layers": [
        _layer("attention", _attention(1, 1, 32, 32, 0.18, 70, _rot(8, 100.0)), 64),
        _layer("parallel", {"left": _left(3, 3, 16, 0.25, 40, 0, 50.0, _rot(16, 10000.0, (2.0, 64, 16.0, 1.0))),
                            "right": _memory(1, 24, 8, (0.97,)), "left_scale": 1.0, "right_scale": 1.0}, None),
        _layer("hgrn2", _memory(6, 8, 16), 80),
    ],
}
R3 = {
    "architecture": "Renadra", "vocab": 320, "width": 256, "norm": {"eps": 1e-6},
    "embedding": {"scale": 8.0, "bigram": {"buckets": 509, "mul_prev": 3, "mul_cur": 1031}},
    "loop": {"start": 0, "stop": 4, "times": 2},
    "layers": [
        _layer("hgrn2", _memory(2, 128, 128), 512),
        _layer("attention", _attention(4, 2, 128, 128, 0.09, 48, _rot(64, 1000000.0)), 384),
        _layer("parallel", {"left": _left(8, 2, 64, 0.125, 33, 17, 30.0, _rot(64, 1000000.0, (8.0, 128, 32.0, 1.0))),
                            "right": _memory(4, 64, 32, (0.7, 0.9, 0.99, 1.0)), "left_scale": 0.8, "right_scale": 1.1},
               None),
        _layer("attention", _attention(2, 1, 64, 64, 0.125, 200, _rot(32, 10000.0)), 256),
    ],
}
CONFIGS = {"R1": (R1, 16), "R2": (R2, 32), "R3": (R3, 16)}


def config(name: str) -> dict:
    return copy.deepcopy(CONFIGS[name][0])


def sharpen(tensors: dict, cfg, seed: int) -> dict:
    """Random tensors made so that the mechanisms matter (see the module's text)."""
    g = torch.Generator().manual_seed(seed + 100)
    tensors["embed"] = tensors["embed"] * (25.0 / cfg.embedding_scale)
    if "bigram" in tensors:
        tensors["bigram"] = tensors["bigram"] * 25.0
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}.mix"
        if layer.type == "attention":
            for name in ("q", "k"):
                tensors[f"{p}.{name}"] = tensors[f"{p}.{name}"] * 12.0
            for name in ("q.b", "k.b", "v.b", "o.b"):
                tensors[f"{p}.{name}"] = tensors[f"{p}.{name}"] * 10.0
        elif layer.type == "hgrn2":
            n = tensors[f"{p}.lower"].numel()
            # lower bounds from 0 to 0.999: some rows forget at once, some keep what was written for hundreds of tokens
            tensors[f"{p}.lower"] = 1.0 - torch.logspace(-3, 0, n, dtype=torch.float32)[torch.randperm(n, generator=g)]
            tensors[f"{p}.f"] = tensors[f"{p}.f"] * 20.0
            tensors[f"{p}.f.b"] = tensors[f"{p}.f.b"] * 10.0
            tensors[f"{p}.q"] = tensors[f"{p}.q"] * 10.0
        else:
            for name in ("q", "k"):
                tensors[f"{p}.left.{name}"] = tensors[f"{p}.left.{name}"] * 12.0
                tensors[f"{p}.left.{name}.b"] = tensors[f"{p}.left.{name}.b"] * 10.0
            tensors[f"{p}.left.pb"] = tensors[f"{p}.left.pb"] * 10.0 - 1.0
            for name in ("q", "k", "v", "g"):
                tensors[f"{p}.right.{name}"] = tensors[f"{p}.right.{name}"] * 10.0
    return tensors


@functools.lru_cache(maxsize=None)
def model_folder(name: str, seed: int = 3) -> str:
    from ampere_kv_engine_b200.models.registry import config_from_dict
    from ampere_kv_engine_b200.weights.random_init import write_random_model
    _, cfg = config_from_dict(config(name))
    out = tempfile.mkdtemp(prefix=f"renadra_{name}_")
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


def random_config(seed: int) -> dict:
    """A configuration whose every size, constant, layer order and loop is drawn from the seed: three to six layers of
    any mixers (at least one of each family), widths and head sizes that are no multiples of 16, windows shorter and
    longer than a page, kept first keys or none, rescaled frequencies or none, layers without a feed-forward, a pair
    table or none, a loop or none."""
    g = torch.Generator().manual_seed(1000 + seed)
    pick = lambda *options: options[int(torch.randint(0, len(options), (1,), generator=g))]
    num = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=g))

    def rot(dim, scaling):
        dims = 2 * num(1, dim // 2)
        s = (pick(2.0, 4.0, 8.0), pick(32, 64, 256), pick(8.0, 16.0, 32.0), pick(1.0, 2.0)) if scaling else None
        return _rot(dims, pick(100.0, 10000.0, 1000000.0), s)

    def attention():
        kv = num(1, 3)
        dim = pick(8, 12, 16, 24, 32, 64)
        return _attention(kv * num(1, 3), kv, dim, pick(8, 12, 16, 20, 32, dim), round(dim ** -0.5 * pick(0.8, 1.0, 1.5), 4),
                          num(3, 80), rot(dim, False))

    def left():
        kv = num(1, 3)
        dim = pick(8, 12, 16, 24, 32, 64)
        return _left(kv * num(1, 3), kv, dim, round(dim ** -0.5 * pick(0.8, 1.0, 1.5), 4), num(3, 60), pick(0, 1, 7, 20),
                     pick(5.0, 30.0, 50.0), rot(dim, pick(True, True, False)))

    def memory(decay):
        heads = num(1, 5)
        m = _memory(heads, pick(4, 8, 12, 20, 32, 48, 64), pick(4, 8, 12, 20, 32, 40, 64))
        if decay:
            m["decay"] = [round(1.0 - 0.5 ** num(1, 10), 6) for _ in range(heads)]
        return m

    width = pick(24, 40, 48, 72, 96, 128)
    kinds = ["attention", "hgrn2", "parallel"] + [pick("attention", "hgrn2", "parallel") for _ in range(num(0, 3))]
    kinds = [kinds[i] for i in torch.randperm(len(kinds), generator=g).tolist()]
    layers = []
    for kind in kinds:
        ff = pick(None, 32, 56, 64, 100)
        if kind == "attention":
            layers.append(_layer(kind, attention(), ff))
        elif kind == "hgrn2":
            layers.append(_layer(kind, memory(False), ff))
        else:
            layers.append(_layer(kind, {"left": left(), "right": memory(True), "left_scale": pick(0.5, 0.8, 1.0),
                                        "right_scale": pick(0.7, 1.0, 1.2)}, ff))
    raw = {"architecture": "Renadra", "vocab": num(50, 300), "width": width, "norm": {"eps": pick(1e-5, 1e-6)},
           "embedding": {"scale": pick(1.0, 2.5, 9.0)}, "layers": layers}
    if pick(True, True, False):
        raw["embedding"]["bigram"] = {"buckets": pick(7, 61, 257), "mul_prev": num(1, 200), "mul_cur": num(1, 50)}
    if pick(True, True, False):
        start = num(0, len(layers) - 1)
        raw["loop"] = {"start": start, "stop": num(start + 1, len(layers)), "times": num(2, 3)}
    return raw


def random_model_folder(seed: int) -> str:
    name = f"random{seed}"
    if name not in CONFIGS:
        CONFIGS[name] = (random_config(seed), (8, 16, 32)[seed % 3])
    return model_folder(name, seed=seed)
