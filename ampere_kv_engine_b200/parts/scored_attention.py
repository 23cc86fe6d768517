"""Grouped-query attention whose scores are reshaped before the softmax, over paged keys and values of
different widths.

    q, k, v, g = (W_q | W_k | W_v | W_g) x            one product; g: one column per q head (optional)
    q, k       <- each head divided by sqrt(mean(head^2) + eps)          (``unit_norm``)
    q, k       <- times a learned weight per dim, shared by the heads    (``norm_weights``)
    v          <- (1 - lam) v + lam v_first             (``value_blend`` "reader"; a "source" layer publishes its v)
    s(i, j)    = q_i . k_j * scale
    s          <- cap * tanh(s / cap)                   (``softcap``)
    s          <- s - slope_h (i - j),  slope_h = 2 ** (-slope_span (h + 1) / heads)       (``slope_span``)
    i sees j   iff j <= i and both lie in the same block of ``chunk`` positions counted from the sequence's start
    out_h      = softmax(s) v * sigmoid(g_h);   y = W_o out

A mixer without ``own_kv`` has no key and value projections: it reads the pages an earlier schedule position wrote
(the model's schedule names it), with its own queries.  When nothing is done to the scores, keys and values have one
width and the plain attention kernels take that width, those run.

Positions enter through the distance bias and the blocks only.  Keys (after the norm) and values (after the blend)
are what the pages keep; a block's pages are given back once the sequence has moved past it.  Everything between
the first product and the output projection is two kernels (``ops.head_prep``, ``ops.scored_attention``).
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import CacheSpec, CacheTensor, Mixer, ParamSpec, register_mixer


@register_mixer("scored_attention")
class ScoredAttention(Mixer):
    """params: ``num_heads``, ``num_kv_heads``, ``head_dim`` (query / key width), ``v_dim`` (value width),
    ``scale``, ``unit_norm`` (bool) and ``norm_eps``, ``norm_weights`` (bool: the unit-RMS q and k heads are multiplied
    by learned weights ``q_norm`` / ``k_norm``), ``own_kv`` (bool, default True), ``softcap`` (None: none), ``slope_span`` (None: no distance
    bias), ``chunk`` (None: plain causal), ``window`` (None: all keys of the block), ``gated`` (bool),
    ``value_blend`` (None, ``"source"`` or ``"reader"``) and ``blend_key`` (the name under which the source's values
    travel through the step), ``names`` (local tensor names of q, k, v, gate, out, blend)."""

    graph_safe = True
    takes_lazy_norm = True
    adds_residual = True

    NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "gate": "gate_proj.weight",
             "out": "o_proj.weight", "blend": "value_blend", "q_norm": "q_norm.weight", "k_norm": "k_norm.weight"}

    def __init__(self, spec, **kw):
        super().__init__(spec, **kw)
        p = spec.params
        self.num_heads, self.num_kv_heads = int(p["num_heads"]), int(p["num_kv_heads"])
        self.head_dim, self.v_dim = int(p["head_dim"]), int(p["v_dim"])
        if self.num_heads <= 0 or self.num_kv_heads <= 0 or self.num_heads % self.num_kv_heads:
            raise ValueError(f"scored_attention: {self.num_heads} heads are not a multiple of {self.num_kv_heads} kv heads")
        if not (0 < self.head_dim <= 1024 and 0 < self.v_dim <= 512):
            raise ValueError(f"scored_attention: key width {self.head_dim} / value width {self.v_dim} outside what "
                             f"the kernel takes (1024 / 512)")
        self.scale = float(p["scale"]) if p.get("scale") is not None else self.head_dim ** -0.5
        self.unit_norm = bool(p.get("unit_norm", False))
        self.norm_eps = float(p.get("norm_eps", 1e-6))
        self.norm_weights = bool(p.get("norm_weights", False))
        self.own_kv = bool(p.get("own_kv", True))
        if self.norm_weights and not self.unit_norm:
            raise ValueError("scored_attention: norm_weights go with unit_norm")
        self.softcap = float(p["softcap"]) if p.get("softcap") else 0.0
        self.slope_span = float(p["slope_span"]) if p.get("slope_span") is not None else None
        self.chunk = int(p["chunk"]) if p.get("chunk") else 0
        self.window = int(p["window"]) if p.get("window") else 0
        if self.chunk < 0 or self.window < 0 or self.softcap < 0:
            raise ValueError("scored_attention: chunk, window and softcap must not be negative")
        self.gated = bool(p.get("gated", False))
        self.value_blend = p.get("value_blend")
        if self.value_blend not in (None, "source", "reader"):
            raise ValueError(f"scored_attention: value_blend must be None, 'source' or 'reader', got {self.value_blend!r}")
        if self.value_blend is not None and not self.own_kv:
            raise ValueError("scored_attention: a mixer without keys and values of its own has no values to blend")
        self.blend_key = str(p.get("blend_key", "value_blend"))
        self.names = dict(self.NAMES, **(p.get("names") or {}))
        self.slopes = None
        if self.slope_span is not None:
            h = torch.arange(1, self.num_heads + 1, dtype=torch.float64)
            self.slopes = torch.exp2(-self.slope_span * h / self.num_heads).to(torch.float32).to(self.device)
        self.w_in = self.w_o = self.blend_weight = self.q_norm_weight = self.k_norm_weight = None
        #: nothing is done to the scores and keys and values have one width that the plain kernels take
        self.plain_scores = (not self.softcap and self.slope_span is None and not self.chunk and not self.gated
                             and self.head_dim == self.v_dim and self.head_dim % 16 == 0 and self.head_dim <= 256)

    def preferred_q_tile(self):
        if self.head_dim == self.v_dim == 128 or self.plain_scores:
            return ops.attention_q_tile(self.head_dim, self.num_heads // self.num_kv_heads)
        return None

    def cache_spec(self) -> CacheSpec:
        kind = "chunk" if self.chunk else ("window" if self.window else "full")
        return CacheSpec(kind=kind, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim,
                         window=self.window or None, chunk=self.chunk or None,
                         tensors=(CacheTensor("k", self.num_kv_heads, self.head_dim),
                                  CacheTensor("v", self.num_kv_heads, self.v_dim)))

    def param_specs(self):
        h, n = self.hidden_size, self.names
        specs = {n["q"]: ParamSpec((self.num_heads * self.head_dim, h))}
        if self.own_kv:
            specs[n["k"]] = ParamSpec((self.num_kv_heads * self.head_dim, h))
            specs[n["v"]] = ParamSpec((self.num_kv_heads * self.v_dim, h))
        if self.norm_weights:
            specs[n["q_norm"]] = ParamSpec((self.head_dim,), kind="vector", init="norm")
            if self.own_kv:
                specs[n["k_norm"]] = ParamSpec((self.head_dim,), kind="vector", init="norm")
        # a source layer carries the scalar too and does not use it; a layer that does not blend may carry it
        specs[n["blend"]] = ParamSpec((), kind="vector", init="unit_interval", optional=self.value_blend is None)
        if self.gated:
            specs[n["gate"]] = ParamSpec((self.num_heads, h))
        specs[n["out"]] = ParamSpec((h, self.num_heads * self.v_dim))
        return specs

    def load(self, tensors):
        n = self.names
        rows = [tensors[n["q"]]] + ([tensors[n["k"]], tensors[n["v"]]] if self.own_kv else []) \
            + ([tensors[n["gate"]]] if self.gated else [])
        self.w_in = torch.cat(rows, dim=0).contiguous()
        if self.norm_weights:
            self.q_norm_weight = tensors[n["q_norm"]].contiguous()
            self.k_norm_weight = tensors[n["k_norm"]].contiguous() if self.own_kv else None
        self.w_o = tensors[n["out"]].contiguous()
        if self.value_blend == "reader":
            self.blend_weight = tensors[n["blend"]].reshape(1).contiguous()

    def forward(self, x, ctx, cache, residual=None):
        group = ctx.groups[cache.group]
        k_cache, v_cache = cache.tensors["k"], cache.tensors["v"]
        x = ops.linear(x, self.w_in, status=ctx.status)
        tokens = x.shape[0]
        v_keep = v_other = None
        if self.value_blend == "source":
            v_keep = torch.empty((tokens, self.num_kv_heads * self.v_dim), dtype=x.dtype, device=x.device)
            ctx.shared[self.blend_key] = v_keep
        elif self.value_blend == "reader":
            v_other = ctx.shared.get(self.blend_key)
            if v_other is None or v_other.shape != (tokens, self.num_kv_heads * self.v_dim):
                raise ValueError(f"scored_attention: no layer before this one left values of "
                                 f"[{tokens}, {self.num_kv_heads * self.v_dim}] under {self.blend_key!r}")
        writes = cache.writes and self.own_kv
        if cache.writes != self.own_kv:
            raise ValueError("scored_attention: a mixer with keys and values of its own writes its pages, one without "
                             "reads another position's (the schedule's cache_of)")
        q, gate = ops.head_prep(
            x, group.slot_mapping if writes else None, k_cache if writes else None, v_cache if writes else None,
            num_heads=self.num_heads, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim, v_dim=self.v_dim,
            unit_norm=self.unit_norm, eps=self.norm_eps, gated=self.gated, v_keep=v_keep, v_other=v_other,
            blend_weight=self.blend_weight, q_weight=self.q_norm_weight, k_weight=self.k_norm_weight,
            has_kv=self.own_kv, status=ctx.status)
        out = torch.empty((tokens, self.num_heads * self.v_dim), dtype=q.dtype, device=q.device)
        run_attention(ctx, group, q, k_cache, v_cache, out, num_heads=self.num_heads, num_kv_heads=self.num_kv_heads,
                      v_dim=self.v_dim, scale=self.scale, window=self.window, chunk=self.chunk, softcap=self.softcap,
                      slopes=self.slopes, gate=gate, plain=self.plain_scores)
        if residual is not None:
            summed = ops.linear_into_residual(out, self.w_o, residual, status=ctx.status)
            if summed is not None:
                return summed
        return ops.linear(out, self.w_o, partial_ok=True, status=ctx.status)


def run_attention(ctx, group, q, k_cache, v_cache, out, *, num_heads, num_kv_heads, v_dim, scale, window=0, chunk=0,
                  softcap=0.0, slopes=None, gate=None, plain=False, keep_first=0, sigmoid_weights=False, head_bias=None,
                  out_scale=1.0) -> None:
    """``ops.scored_attention`` over the step's tiles: the single-token tiles of a mixed step (they come first) apart
    from the prompt tiles, each with the number of key splits that fills the GPU.  ``plain``: nothing is done to the
    scores and the plain kernels take the sizes: ``ops.paged_attention`` runs instead."""
    group_size = num_heads // num_kv_heads
    plain_tc = plain and ops.attention_takes_tensor_cores(q.dtype, q.shape[1] // num_heads, group_size,
                                                          k_cache.shape[2])
    first = getattr(ctx, "num_decode_tiles", 0)
    for lo, hi, q_tile in ((0, first, 1), (first, ctx.num_tiles, ctx.q_tile)):
        if hi <= lo:
            continue
        longest, mean = ctx.decode_contexts if q_tile == 1 else (ctx.max_context, ctx.max_context)
        for limit in (window + keep_first if window else 0, chunk):
            if limit:
                longest, mean = min(longest, limit), min(mean, limit)
        if plain:
            splits = 1 if q_tile > 1 and plain_tc else ops.choose_splits(
                hi - lo, num_kv_heads, q_tile * group_size, longest, plain_tc, mean_context=mean)
            ops.paged_attention(
                q, k_cache, v_cache, group.block_table, ctx.cu_q, ctx.ctx_lens, ctx.tile_seq[lo:hi], ctx.tile_q0[lo:hi],
                ctx.tile_nq[lo:hi], num_tiles=hi - lo, q_tile=q_tile, num_splits=splits, num_heads=num_heads,
                num_kv_heads=num_kv_heads, window=window, scale=scale, status=ctx.status, out=out)
            continue
        # kept first keys, sigmoid weights and an output factor: the tensor-core kernels take them where keys and
        # values have storage of their own (single tokens: with a positive factor)
        special = bool(keep_first or sigmoid_weights or head_bias is not None or out_scale != 1.0)
        general_only = special and (k_cache is v_cache or (q_tile == 1 and not out_scale > 0.0))
        tensor_core = not general_only and k_cache is not v_cache and ops.scored_takes_tensor_cores(
            q.dtype, q.shape[1] // num_heads, v_dim, group_size, k_cache.shape[2], prompt=q_tile > 1)
        if not general_only and k_cache is v_cache and ops.shared_rows_take_tensor_cores(q.dtype, q.shape[1] // num_heads, v_dim):
            splits = ops.choose_splits_shared_rows(hi - lo, num_kv_heads, q_tile * group_size, longest)
        elif q_tile > 1 and tensor_core:
            splits = 1
        else:
            splits = ops.choose_splits(hi - lo, num_kv_heads, q_tile * group_size, longest, tensor_core,
                                       mean_context=mean)
        ops.scored_attention(
            q, k_cache, v_cache, group.block_table, ctx.cu_q, ctx.ctx_lens, ctx.tile_seq[lo:hi], ctx.tile_q0[lo:hi],
            ctx.tile_nq[lo:hi], num_tiles=hi - lo, q_tile=q_tile, num_splits=splits, num_heads=num_heads,
            num_kv_heads=num_kv_heads, v_dim=v_dim, scale=scale, window=window, chunk=chunk, softcap=softcap,
            slopes=slopes, gate=gate, status=ctx.status, out=out, keep_first=keep_first,
            sigmoid_weights=sigmoid_weights, head_bias=head_bias, out_scale=out_scale)
