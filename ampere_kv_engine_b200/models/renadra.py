"""The ``Renadra`` decoder as a model spec.

A scaled token embedding plus the row of a (previous token, token) pair's bucket; pre-norm layers with plain RMS norms
whose mixer is chosen layer by layer, each followed by a SiLU-gated feed-forward or by none; a final norm and an
untied head.  A run of layers may be scheduled several times in a row (the same weights, a cache and a state per
appearance), with the embedding's output added to the stream before every pass but the first.  Mixers:

``attention``  ``rotary_attention`` with queries and keys turned in neighbouring pairs, biases on all four
               projections, unit-RMS values, a window and softmax
``hgrn2``      ``hgrn2``
``parallel``   ``parallel`` of a ``rotary_attention`` (half layout with frequencies rescaled by wavelength, biases on q
               and k, values that are the unrotated keys, capped scores, a window that keeps the first keys, sigmoid
               weights with a bias per head) and a ``lightning_attention``

Tensor names: ``embed``, ``bigram``, ``l<i>.norm1|norm2``, ``l<i>.mix.*`` (``.left.*`` / ``.right.*`` in a parallel
layer; a bias is its matrix's name with ``.b``), ``l<i>.mlp.gate|up|down``, ``final.norm``, ``head``.
"""

from __future__ import annotations

from ..config.model_config import RenadraConfig
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .registry import register_architecture


def _norm(config: RenadraConfig, prefix: str, tensor: str) -> PartSpec:
    return PartSpec("rmsnorm", {"eps": config.norm_eps, "tensor": tensor}, prefix)


def _rope(rot: dict, layout: str) -> PartSpec:
    return PartSpec("rope", {"theta": rot["base"], "rotary_dim": rot["dims"], "layout": layout,
                             "scaling": rot.get("scaling")}, "")


def _attention(config: RenadraConfig, m: dict, prefix: str) -> PartSpec:
    return PartSpec("rotary_attention", {
        "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"], "v_dim": m["vdim"],
        "scale": m["scale"], "position_encoding": _rope(m["rot"], "pairs"), "bias": ("q", "k", "v", "out"),
        "bias_suffix": ".b", "value_norm": True, "norm_eps": config.norm_eps, "softcap": m.get("softcap"),
        "window": m["mask"]["size"], "keep_first": m["mask"].get("keep_first") or 0,
        "names": {"q": "q", "k": "k", "v": "v", "out": "o"}}, prefix)


def _left(m: dict, prefix: str) -> PartSpec:
    return PartSpec("rotary_attention", {
        "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"], "v_dim": m["vdim"],
        "scale": m["scale"], "position_encoding": _rope(m["rot"], "half"), "bias": ("q", "k"), "bias_suffix": ".b",
        "value_from_key": True, "softcap": m.get("softcap"), "window": m["mask"]["size"],
        "keep_first": m["mask"].get("keep_first") or 0, "weights": "sigmoid", "head_bias": True,
        "names": {"q": "q", "k": "k", "out": "o", "head_bias": "pb"}}, prefix)


def _right(config: RenadraConfig, m: dict, prefix: str) -> PartSpec:
    return PartSpec("lightning_attention", {
        "num_heads": m["heads"], "head_dim": m["dim"], "v_dim": m["vdim"], "decay": tuple(m["decay"]),
        "norm_eps": config.norm_eps,
        "names": {"q": "q", "k": "k", "v": "v", "gate": "g", "norm": "norm", "out": "o"}}, prefix)


def build_spec(config: RenadraConfig) -> ModelSpec:
    layers, unused = [], []
    for i, layer in enumerate(config.layers):
        prefix, m = f"l{i}", layer.mixer
        if layer.type == "attention":
            mixer = _attention(config, m, f"{prefix}.mix")
        elif layer.type == "hgrn2":
            mixer = PartSpec("hgrn2", {
                "num_heads": m["heads"], "head_dim": m["dim"], "v_dim": m["vdim"], "norm_eps": config.norm_eps,
                "names": {"q": "q", "gate": "f", "gate_bias": "f.b", "lower": "lower", "v": "v", "norm": "norm",
                          "out": "o"}}, f"{prefix}.mix")
        else:
            mixer = PartSpec("parallel", {
                "left": _left(m["left"], f"{prefix}.mix.left"), "right": _right(config, m["right"], f"{prefix}.mix.right"),
                "left_scale": m["left_scale"], "right_scale": m["right_scale"]}, f"{prefix}.mix")
        ff = ff_norm = None
        if layer.mlp is not None:
            ff = PartSpec("gated_mlp", {"intermediate_size": layer.mlp["ff"], "activation": "silu",
                                        "names": {"gate": "gate", "up": "up", "down": "down"}}, f"{prefix}.mlp")
            ff_norm = _norm(config, prefix, "norm2")
        else:
            unused.append((f"{prefix}.norm2", (config.width,)))     # a layer without a feed-forward may still carry it
        layers.append(LayerSpec(block="prenorm", mixer=mixer, feed_forward=ff, mixer_norm=_norm(config, prefix, "norm1"),
                                feed_forward_norm=ff_norm))
    count = len(layers)
    loop = config.loop or {"start": 0, "stop": count, "times": 1}
    schedule = [ScheduleEntry(i) for i in range(loop["start"])]
    for again in range(loop["times"]):
        schedule += [ScheduleEntry(i, add_embedding=again > 0 and i == loop["start"])
                     for i in range(loop["start"], loop["stop"])]
    schedule += [ScheduleEntry(i) for i in range(loop["stop"], count)]
    pair_table = None
    if config.bigram is not None:
        pair_table = {"tensor": "bigram", "buckets": config.bigram["buckets"], "mul_prev": config.bigram["mul_prev"],
                      "mul_cur": config.bigram["mul_cur"]}
    return ModelSpec(
        hidden_size=config.width,
        vocab_size=config.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": config.vocab, "tensor": "embed",
                                               "scale": config.embedding_scale, "pair_table": pair_table}, ""),
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=_norm(config, "final", "norm"),
        head=PartSpec("linear_head", {"vocab_size": config.vocab, "tied": False, "tensor": "head"}, ""),
        max_position=config.max_position_embeddings,
        eos_token_ids=config.eos_token_id,
        unused_tensors=tuple(unused),
    )


register_architecture("Renadra", RenadraConfig, build_spec)
