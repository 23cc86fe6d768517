"""The ``Zavizen`` decoder as a model spec.

A plain token embedding whose row starts ``streams`` copies of the residual stream; layers of block kind ``hyper``
(every sublayer reads a learned mixture of the copies through an RMS norm whose weight is stored around zero, and
writes its result, times a learned vector over the width, back into all of them); a mixer chosen layer by layer; a
feed-forward chosen layer by layer (a SiLU-gated dense one, ``routed_experts`` with softmax scores, groups scored by
their best expert and plain SiLU experts, or none); a run of layers may be scheduled several times in a row (the same
weights, a cache and a state per appearance); the final norm on the copies' sum, and an untied head.  Mixers:

``parallel``   ``parallel`` of a ``rotary_attention`` (queries and keys normed over their whole projection before a
               partial turn in the half layout with linearly scaled frequencies, full causal softmax) and a
               ``retention`` (constant decay per head, turned queries and keys, a SiLU gate), each side's output
               normed over the model width, half their sum
``mamba2``     ``mamba2``

Tensor names: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.ls1|ls2``, ``l<i>.hc1|hc2.in|out|mix``, ``l<i>.mix.*``
(``.left.*`` / ``.right.*`` in a parallel layer), ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""

from __future__ import annotations

from ..config.model_config import ZavizenConfig
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .registry import register_architecture

#: constants the design fixes
WEIGHT_EPS = 1e-20          # added to the sum the chosen experts' scores are divided by
GROUP_TOP = 1               # a group of experts is scored by its best expert
SIDE_SCALE = 0.5            # a parallel layer's result is half the sum of its normed sides


def _rope(rot: dict) -> PartSpec:
    # a factor of one where the configuration names none: the frequencies are then formed in float64 and rounded once
    return PartSpec("rope", {"theta": rot["base"], "rotary_dim": rot["dims"], "layout": "half",
                             "scaling": rot.get("scaling") or {"factor": 1.0}}, "")


def _connection(config: ZavizenConfig, prefix: str, which: int) -> PartSpec:
    return PartSpec("hyper_connection", {
        "streams": config.streams, "eps": config.norm_eps, "unit_offset": True,
        "names": {"norm": f"norm{which}", "read": f"hc{which}.in", "write": f"hc{which}.out", "mix": f"hc{which}.mix",
                  "scale": f"ls{which}"}}, prefix)


def _mixer(config: ZavizenConfig, kind: str, m: dict, prefix: str) -> PartSpec:
    if kind == "mamba2":
        return PartSpec("mamba2", {
            "num_heads": m["heads"], "v_dim": m["vdim"], "state_dim": m["state"], "groups": m["groups"],
            "taps": m["conv"], "norm_groups": m["norm_groups"], "norm_eps": config.norm_eps,
            "names": {"in": "in", "conv": "conv", "conv_bias": "conv.b", "step_bias": "dt_bias", "rate_log": "A_log",
                      "skip": "D", "norm": "norm", "out": "o"}}, prefix)
    left, right = m["left"], m["right"]
    return PartSpec("parallel", {
        "left": PartSpec("rotary_attention", {
            "num_heads": left["heads"], "num_kv_heads": left["kv_heads"], "head_dim": left["dim"],
            "v_dim": left["vdim"], "scale": left["scale"], "position_encoding": _rope(left["rot"]), "row_norm": True,
            "norm_eps": config.norm_eps,
            "names": {"q": "q", "k": "k", "v": "v", "out": "o", "q_norm": "q.norm", "k_norm": "k.norm"}},
            f"{prefix}.left"),
        "right": PartSpec("retention", {
            "num_heads": right["heads"], "head_dim": right["dim"], "v_dim": right["vdim"],
            "decay": tuple(right["decay"]), "position_encoding": _rope(right["rot"]), "norm_eps": config.norm_eps,
            "names": {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o"}}, f"{prefix}.right"),
        "left_scale": SIDE_SCALE, "right_scale": SIDE_SCALE,
        "out_norm": {"eps": config.norm_eps, "left": "left.out", "right": "right.out"}}, prefix)


def _feed_forward(mlp: dict, prefix: str) -> PartSpec:
    if mlp.get("kind", "dense") == "dense":
        return PartSpec("gated_mlp", {"intermediate_size": mlp["ff"], "activation": "silu",
                                      "names": {"gate": "gate", "up": "up", "down": "down"}}, prefix)
    router, groups = mlp["router"], mlp["router"].get("groups") or {"count": 1, "keep": 1}
    shared = mlp.get("shared")
    return PartSpec("routed_experts", {
        "experts": router["experts"], "top": router["top"], "groups": groups["count"], "keep_groups": groups["keep"],
        "group_top": GROUP_TOP, "route_scale": router["scale"], "weight_eps": WEIGHT_EPS, "score": "softmax",
        "correction": False, "activation": "silu", "intermediate_size": mlp["expert"]["ff"],
        "shared": None if shared is None else {"intermediate_size": shared["ff"]},
        "names": {"expert": "e{}", "gate": "gate", "up": "up", "down": "down", "router": "router",
                  "shared": "shared"}}, prefix)


def build_spec(config: ZavizenConfig) -> ModelSpec:
    layers, unused = [], []
    for i, layer in enumerate(config.layers):
        prefix = f"l{i}"
        parts = {"mixer_connection": _connection(config, prefix, 1)}
        ff = None
        if layer.mlp is not None:
            ff = _feed_forward(layer.mlp, f"{prefix}.mlp")
            parts["feed_forward_connection"] = _connection(config, prefix, 2)
        else:
            # a layer without a feed-forward may still carry the tensors of its second connection
            s = config.streams
            unused += [(f"{prefix}.norm2", (config.width,)), (f"{prefix}.ls2", (config.width,)),
                       (f"{prefix}.hc2.in", (s,)), (f"{prefix}.hc2.out", (s,)), (f"{prefix}.hc2.mix", (s, s))]
        layers.append(LayerSpec(block="hyper", mixer=_mixer(config, layer.type, layer.mixer, f"{prefix}.mix"),
                                feed_forward=ff, parts=parts))
    count = len(layers)
    loop = config.loop or {"start": 0, "stop": count, "times": 1}
    schedule = [ScheduleEntry(i) for i in range(loop["start"])]
    for _ in range(loop["times"]):
        schedule += [ScheduleEntry(i) for i in range(loop["start"], loop["stop"])]
    schedule += [ScheduleEntry(i) for i in range(loop["stop"], count)]
    return ModelSpec(
        hidden_size=config.width,
        vocab_size=config.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": config.vocab, "tensor": "embed"}, ""),
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=PartSpec("rmsnorm", {"eps": config.norm_eps, "tensor": "norm", "unit_offset": True}, "final"),
        head=PartSpec("linear_head", {"vocab_size": config.vocab, "tied": False, "tensor": "head"}, ""),
        max_position=config.max_position_embeddings,
        eos_token_ids=config.eos_token_id,
        unused_tensors=tuple(unused),
        streams=config.streams,
    )


register_architecture("Zavizen", ZavizenConfig, build_spec)
