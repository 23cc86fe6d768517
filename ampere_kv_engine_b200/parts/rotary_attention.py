"""Grouped-query attention over pages whose queries and keys are turned by position in either layout, with the
options that come with it:

    q, k (, v) = (W_q | W_k (| W_v)) x + biases          one product; biases on q, k, v and the output are optional
    q, k      <- q / sqrt(mean(q^2) + eps) * w_q over ALL of q's heads at once, k likewise (``row_norm``), then
    q, k      <- the first rotary dims of every head turned by the token's position (``position_encoding``: a rope in
                 the half or the neighbouring-pairs layout, possibly with rescaled frequencies and a factor)
    v          = the key head before its turn (``value_from_key``; there is no W_v), or the v head, optionally divided
                 by sqrt(mean(v^2) + eps) (``value_norm``); it is cached so
    s(i, j)    = q_i . k_j * scale;   s <- cap * tanh(s / cap)  (``softcap``)
    i sees j   iff j <= i and (i - j < window or j < keep_first)     (``window``; ``keep_first`` first keys stay
                 visible at their true positions)
    weights    = softmax over the visible keys, or with ``weights="sigmoid"`` sigmoid(s + head_bias[h]) for every
                 visible key, not normalised
    y          = W_o concat_h(out_h) (+ bias), every head's output times ``out_scale`` first (a mixer that runs beside
                 another one scales its share there, in float32, before the one rounding)

Everything between the first product and the output projection is two kernels (``ops.rotary_prep``, then
``ops.paged_attention`` when nothing is done to the scores and the plain kernels take the sizes, else
``ops.scored_attention``).  Pages behind the window are given back; those of the kept first keys are held.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import POSITION_ENCODINGS, CacheSpec, CacheTensor, Mixer, ParamSpec, build_part, register_mixer
from .scored_attention import run_attention


@register_mixer("rotary_attention")
class RotaryAttention(Mixer):
    """params: ``num_heads``, ``num_kv_heads``, ``head_dim``, ``v_dim``, ``scale`` (None: head_dim ** -0.5),
    ``position_encoding`` (a PartSpec of a rope), ``bias`` (a tuple of the projections that carry one, of ``q``, ``k``,
    ``v``, ``out``), ``value_from_key``, ``value_norm`` and ``norm_eps``, ``softcap``, ``window``, ``keep_first``,
    ``weights`` (``"softmax"`` or ``"sigmoid"``), ``head_bias`` (bool: a learned number per head added to the score
    inside the sigmoid), ``out_scale``, ``row_norm`` (bool: a weighted RMS norm over the whole q projection and over
    the whole k projection before the turn, ``norm_eps`` inside the root), ``names`` (local tensor names of q, k, v,
    out, head_bias, q_norm, k_norm; a bias is the matrix's name with ``bias_suffix`` added)."""

    graph_safe = True
    adds_residual = True

    NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "out": "o_proj.weight",
             "head_bias": "head_bias", "q_norm": "q_norm.weight", "k_norm": "k_norm.weight"}

    def __init__(self, spec, **kw):
        super().__init__(spec, **kw)
        p = spec.params
        self.num_heads, self.num_kv_heads = int(p["num_heads"]), int(p["num_kv_heads"])
        self.head_dim, self.v_dim = int(p["head_dim"]), int(p["v_dim"])
        if self.num_heads <= 0 or self.num_kv_heads <= 0 or self.num_heads % self.num_kv_heads:
            raise ValueError(f"rotary_attention: {self.num_heads} heads are not a multiple of {self.num_kv_heads} kv heads")
        if not (0 < self.head_dim <= 1024 and 0 < self.v_dim <= 512):
            raise ValueError(f"rotary_attention: key width {self.head_dim} / value width {self.v_dim} outside what "
                             f"the kernel takes (1024 / 512)")
        self.scale = float(p["scale"]) if p.get("scale") is not None else self.head_dim ** -0.5
        self.bias = tuple(p.get("bias") or ())
        if any(b not in ("q", "k", "v", "out") for b in self.bias):
            raise ValueError(f"rotary_attention: bias names projections of q, k, v, out; got {self.bias}")
        self.out_bias = "out" in self.bias
        self.value_from_key = bool(p.get("value_from_key", False))
        if self.value_from_key and (self.v_dim != self.head_dim or "v" in self.bias):
            raise ValueError("rotary_attention: a value that is its key has the key's width and no projection of its own")
        self.value_norm = bool(p.get("value_norm", False))
        self.norm_eps = float(p.get("norm_eps", 1e-6))
        self.softcap = float(p["softcap"]) if p.get("softcap") else 0.0
        self.window = int(p["window"]) if p.get("window") else 0
        self.keep_first = int(p["keep_first"]) if p.get("keep_first") else 0
        if self.window < 0 or self.keep_first < 0 or self.softcap < 0 or (self.keep_first and not self.window):
            raise ValueError("rotary_attention: window, keep_first and softcap must not be negative, and kept first "
                             "keys go with a window")
        self.weights = str(p.get("weights", "softmax"))
        if self.weights not in ("softmax", "sigmoid"):
            raise ValueError(f"rotary_attention: weights must be 'softmax' or 'sigmoid', got {self.weights!r}")
        self.has_head_bias = bool(p.get("head_bias", False))
        if self.has_head_bias and self.weights != "sigmoid":
            raise ValueError("rotary_attention: a bias per head only matters inside the sigmoid")
        self.out_scale = float(p.get("out_scale", 1.0))
        self.row_norm = bool(p.get("row_norm", False))
        self.q_norm = self.k_norm = None
        self.names = dict(self.NAMES, **(p.get("names") or {}))
        self.bias_suffix = str(p.get("bias_suffix", ".bias"))
        self.position_encoding = build_part(POSITION_ENCODINGS, p["position_encoding"], hidden_size=self.hidden_size,
                                            dtype=self.dtype, device=self.device)
        table = getattr(self.position_encoding, "rotary_table", None)
        if table is None:
            raise ValueError(f"rotary_attention: position encoding {p['position_encoding'].kind!r} has no rotary table")
        self.freq, self.rotary_dims, self.layout, self.factor = table()
        if self.rotary_dims > self.head_dim:
            raise ValueError(f"rotary_attention: {self.rotary_dims} rotary dims in heads of {self.head_dim}")
        self.w_in = self.b_in = self.w_o = self.b_o = self.head_bias = None
        #: nothing is done to the scores and keys and values have one width that the plain kernels take
        self.plain_scores = (self.weights == "softmax" and not self.softcap and not self.keep_first
                             and self.out_scale == 1.0 and self.head_dim == self.v_dim and self.head_dim % 16 == 0
                             and self.head_dim <= 256)

    def children(self):
        return (self.position_encoding,)

    def preferred_q_tile(self):
        if self.plain_scores:
            return ops.attention_q_tile(self.head_dim, self.num_heads // self.num_kv_heads)
        return None

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(kind="window" if self.window else "full", num_kv_heads=self.num_kv_heads,
                         head_dim=self.head_dim, window=self.window or None, keep_first=self.keep_first,
                         tensors=(CacheTensor("k", self.num_kv_heads, self.head_dim),
                                  CacheTensor("v", self.num_kv_heads, self.v_dim)))

    def _projections(self):
        rows = [("q", self.num_heads * self.head_dim), ("k", self.num_kv_heads * self.head_dim)]
        if not self.value_from_key:
            rows.append(("v", self.num_kv_heads * self.v_dim))
        return rows

    def param_specs(self):
        h, n = self.hidden_size, self.names
        specs = {}
        for key, rows in self._projections():
            specs[n[key]] = ParamSpec((rows, h))
            if key in self.bias:
                specs[n[key] + self.bias_suffix] = ParamSpec((rows,), kind="bias")
        if self.has_head_bias:
            specs[n["head_bias"]] = ParamSpec((self.num_heads,), kind="vector", init="around_zero")
        if self.row_norm:
            specs[n["q_norm"]] = ParamSpec((self.num_heads * self.head_dim,), kind="vector", init="norm")
            specs[n["k_norm"]] = ParamSpec((self.num_kv_heads * self.head_dim,), kind="vector", init="norm")
        specs[n["out"]] = ParamSpec((h, self.num_heads * self.v_dim))
        if "out" in self.bias:
            specs[n["out"] + self.bias_suffix] = ParamSpec((h,), kind="bias")
        return specs

    def load(self, tensors):
        n = self.names
        self.w_in = torch.cat([tensors[n[key]] for key, _ in self._projections()], dim=0).contiguous()
        if any(key in self.bias for key, _ in self._projections()):
            self.b_in = torch.cat([tensors[n[key] + self.bias_suffix] if key in self.bias
                                   else torch.zeros(rows, dtype=self.w_in.dtype, device=self.w_in.device)
                                   for key, rows in self._projections()]).contiguous()
        self.w_o = tensors[n["out"]].contiguous()
        if "out" in self.bias:
            self.b_o = tensors[n["out"] + self.bias_suffix].contiguous()
        if self.has_head_bias:
            self.head_bias = tensors[n["head_bias"]].float().contiguous()
        if self.row_norm:
            self.q_norm = tensors[n["q_norm"]].float().contiguous()
            self.k_norm = tensors[n["k_norm"]].float().contiguous()

    def in_projection(self) -> tuple[torch.Tensor, torch.Tensor | None]:
        """The matrix (and bias) of the one product that makes q, k (and v): a mixer that runs beside another one on
        the same input may have it computed together with the other's and handed in as ``projected``."""
        return self.w_in, self.b_in

    def heads_forward(self, x, ctx, cache, projected=None) -> torch.Tensor:
        """Everything before the output projection: [tokens, heads * v_dim], each head's output times ``out_scale``.
        ``projected``: (a product that holds this mixer's q, k (and v) columns, the column where they begin)."""
        group = ctx.groups[cache.group]
        k_cache, v_cache = cache.tensors["k"], cache.tensors["v"]
        if not cache.writes:
            raise ValueError("rotary_attention: the mixer writes its own pages")
        if projected is not None:
            x, x_off = projected
        else:
            x, x_off = ops.linear(x, self.w_in, self.b_in, status=ctx.status), 0
        q = ops.rotary_prep(x, ctx.positions, group.slot_mapping, self.freq, k_cache, v_cache,
                            num_heads=self.num_heads, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim,
                            v_dim=self.v_dim, rotary_dims=self.rotary_dims, layout=self.layout, factor=self.factor,
                            value_from_key=self.value_from_key, value_norm=self.value_norm, eps=self.norm_eps,
                            status=ctx.status, q_norm=self.q_norm, k_norm=self.k_norm, row_norm_eps=self.norm_eps,
                            x_off=x_off)
        out = torch.empty((q.shape[0], self.num_heads * self.v_dim), dtype=q.dtype, device=q.device)
        run_attention(ctx, group, q, k_cache, v_cache, out, num_heads=self.num_heads, num_kv_heads=self.num_kv_heads,
                      v_dim=self.v_dim, scale=self.scale, window=self.window, softcap=self.softcap,
                      plain=self.plain_scores, keep_first=self.keep_first, sigmoid_weights=self.weights == "sigmoid",
                      head_bias=self.head_bias, out_scale=self.out_scale)
        return out

    def out_projection(self) -> tuple[torch.Tensor, torch.Tensor | None]:
        return self.w_o, self.b_o

    def forward(self, x, ctx, cache, residual=None):
        out = self.heads_forward(x, ctx, cache)
        if residual is not None and self.b_o is None:
            summed = ops.linear_into_residual(out, self.w_o, residual, status=ctx.status)
            if summed is not None:
                return summed
        return ops.linear(out, self.w_o, self.b_o, partial_ok=self.b_o is None, status=ctx.status)
