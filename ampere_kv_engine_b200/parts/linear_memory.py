"""Linear-attention mixers whose memory is one matrix per head, carried from token to token in float32:

    S_t = diag(a_t) S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t            S: [head_dim, v_dim] per (request, head)

``hgrn2``: a row is written with one minus its forget gate.

    q = silu(W_q x);  v = W_v x;  f = lower + (1 - lower) * sigmoid(W_f x + bias);   a = f,  k = 1 - f
    y = W_o concat_h( o_h / sqrt(mean(o_h^2) + eps) * norm )          one norm weight [v_dim] shared by the heads

``lightning_attention``: a constant decay per head.

    q, k, v = silu(W_q x), silu(W_k x), silu(W_v x);   a = decay[head] for every row
    y = W_o ( concat_h(o_h) / sqrt(mean over all heads of o^2 + eps) * norm * sigmoid(W_g x) )     norm: [heads * v_dim]

``retention``: a constant decay per head, queries and keys turned by position, no activation.

    q, k = rope(W_q x), rope(W_k x) * head_dim^-1/2;   v = W_v x;   a = decay[head] for every row
    y = W_o ( concat_h( o_h / sqrt(mean(o_h^2) + eps) ) * silu(W_g x) )          no norm weight

One product makes all projections of a token; ``ops.linear_scan`` applies the activations and gates in float32 and
walks the step's tokens of every sequence in order, from and into the request's state slot (so the memory after a
token is the same however the tokens were cut into steps); ``ops.group_norm_gate`` norms what was read out.  A
request's state is its memory alone, in the scan kernel's own order.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import POSITION_ENCODINGS, CacheSpec, Mixer, ParamSpec, build_part, register_mixer


class _LinearMemory(Mixer):
    graph_safe = True

    def _sizes(self, p, what: str):
        self.num_heads, self.head_dim, self.v_dim = int(p["num_heads"]), int(p["head_dim"]), int(p["v_dim"])
        if self.num_heads <= 0 or ops.linear_scan_shape(self.head_dim, self.v_dim) is None:
            raise ValueError(f"{what}: {self.num_heads} heads of key width {self.head_dim} and value width {self.v_dim} "
                             f"are outside what the kernel takes (each up to {ops.LINEAR_SCAN_MAX_DIM})")
        self.norm_eps = float(p.get("norm_eps", 1e-6))
        self.out_scale = float(p.get("out_scale", 1.0))
        self.qk_width = self.num_heads * self.head_dim
        self.v_width = self.num_heads * self.v_dim
        self.state_floats = ops.linear_scan_state_floats(self.num_heads, self.head_dim, self.v_dim)

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(kind="none", state_shape=(self.state_floats,))

    def out_projection(self):
        return self.w_o, None

    def forward(self, x, ctx, cache, residual=None):
        return ops.linear(self.heads_forward(x, ctx, cache), self.w_o, status=ctx.status)


@register_mixer("hgrn2")
class Hgrn2(_LinearMemory):
    """params: ``num_heads``, ``head_dim`` (width of q and of the forget gate per head), ``v_dim``, ``norm_eps``,
    ``out_scale`` (on the normed output), ``names`` (local tensor names of q, gate, gate_bias, lower, v, norm, out)."""

    NAMES = {"q": "q_proj.weight", "gate": "f_proj.weight", "gate_bias": "f_proj.bias", "lower": "lower_bound",
             "v": "v_proj.weight", "norm": "o_norm.weight", "out": "o_proj.weight"}

    def __init__(self, spec, **kw):
        super().__init__(spec, **kw)
        self._sizes(spec.params, "hgrn2")
        self.names = dict(self.NAMES, **(spec.params.get("names") or {}))
        self.w_in = self.w_o = self.gate_bias = self.lower = self.norm_weight = None

    def param_specs(self):
        h, n = self.hidden_size, self.names
        return {
            n["q"]: ParamSpec((self.qk_width, h)),
            n["gate"]: ParamSpec((self.qk_width, h)),
            n["gate_bias"]: ParamSpec((self.qk_width,), kind="vector", init="around_zero"),
            n["lower"]: ParamSpec((self.qk_width,), kind="vector", init="unit_interval"),
            n["v"]: ParamSpec((self.v_width, h)),
            n["norm"]: ParamSpec((self.v_dim,), kind="vector", init="norm"),
            n["out"]: ParamSpec((h, self.v_width)),
        }

    def load(self, tensors):
        n = self.names
        self.w_in = torch.cat([tensors[n[k]] for k in ("q", "gate", "v")], dim=0).contiguous()     # [q | f | v]
        self.gate_bias = tensors[n["gate_bias"]].float().contiguous()
        self.lower = tensors[n["lower"]].float().contiguous()
        self.norm_weight = tensors[n["norm"]].float().contiguous()
        self.w_o = tensors[n["out"]].contiguous()

    def heads_forward(self, x, ctx, cache):
        if cache.state is None:
            raise ValueError("hgrn2: the cache manager gave this position no state")
        x = ops.linear(x, self.w_in, status=ctx.status)
        o = ops.linear_scan(x, cache.state, ctx.cu_q, ctx.state_slots, num_heads=self.num_heads,
                            head_dim=self.head_dim, v_dim=self.v_dim, mode="gated_write", q_off=0,
                            k_off=self.qk_width, v_off=2 * self.qk_width, gate_bias=self.gate_bias, lower=self.lower)
        return ops.group_norm_gate(o, self.norm_weight, group=self.v_dim, eps=self.norm_eps, out_dtype=x.dtype,
                                   factor=self.out_scale)


@register_mixer("lightning_attention")
class LightningAttention(_LinearMemory):
    """params: ``num_heads``, ``head_dim``, ``v_dim``, ``decay`` (a number per head), ``norm_eps``, ``out_scale``,
    ``names`` (local tensor names of q, k, v, gate, norm, out)."""

    NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "gate": "g_proj.weight",
             "norm": "o_norm.weight", "out": "o_proj.weight"}

    def __init__(self, spec, **kw):
        super().__init__(spec, **kw)
        self._sizes(spec.params, "lightning_attention")
        decay = [float(d) for d in spec.params["decay"]]
        if len(decay) != self.num_heads:
            raise ValueError(f"lightning_attention: {len(decay)} decay rates for {self.num_heads} heads")
        self.decay = torch.tensor(decay, dtype=torch.float64).to(torch.float32).to(self.device)
        self.names = dict(self.NAMES, **(spec.params.get("names") or {}))
        self.w_in = self.w_o = self.norm_weight = None

    def param_specs(self):
        h, n = self.hidden_size, self.names
        return {
            n["q"]: ParamSpec((self.qk_width, h)),
            n["k"]: ParamSpec((self.qk_width, h)),
            n["v"]: ParamSpec((self.v_width, h)),
            n["gate"]: ParamSpec((self.v_width, h)),
            n["out"]: ParamSpec((h, self.v_width)),
            n["norm"]: ParamSpec((self.v_width,), kind="vector", init="norm"),
        }

    def load(self, tensors):
        n = self.names
        self.w_in = torch.cat([tensors[n[k]] for k in ("q", "k", "v", "gate")], dim=0).contiguous()   # [q | k | v | g]
        self.norm_weight = tensors[n["norm"]].float().contiguous()
        self.w_o = tensors[n["out"]].contiguous()

    def heads_forward(self, x, ctx, cache):
        if cache.state is None:
            raise ValueError("lightning_attention: the cache manager gave this position no state")
        x = ops.linear(x, self.w_in, status=ctx.status)
        o = ops.linear_scan(x, cache.state, ctx.cu_q, ctx.state_slots, num_heads=self.num_heads,
                            head_dim=self.head_dim, v_dim=self.v_dim, mode="constant_decay", q_off=0,
                            k_off=self.qk_width, v_off=2 * self.qk_width, decay=self.decay)
        return ops.group_norm_gate(o, self.norm_weight, group=self.v_width, eps=self.norm_eps, out_dtype=x.dtype,
                                   factor=self.out_scale, x=x, gate_off=2 * self.qk_width + self.v_width)


@register_mixer("retention")
class Retention(_LinearMemory):
    """params: ``num_heads``, ``head_dim``, ``v_dim``, ``decay`` (a number per head), ``position_encoding`` (a
    PartSpec of a rope in the half layout), ``key_scale`` (None: ``head_dim ** -0.5``, applied after the turn),
    ``norm_eps``, ``names`` (local tensor names of q, k, v, gate, out).  Each head's read-out is divided by its root
    mean square (no weight) and multiplied by ``silu`` of the gate projection."""

    NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "gate": "g_proj.weight",
             "out": "o_proj.weight"}

    def __init__(self, spec, **kw):
        super().__init__(spec, **kw)
        self._sizes(spec.params, "retention")
        decay = [float(d) for d in spec.params["decay"]]
        if len(decay) != self.num_heads:
            raise ValueError(f"retention: {len(decay)} decay rates for {self.num_heads} heads")
        self.decay = torch.tensor(decay, dtype=torch.float64).to(torch.float32).to(self.device)
        key_scale = spec.params.get("key_scale")
        self.key_scale = float(key_scale) if key_scale is not None else self.head_dim ** -0.5
        self.names = dict(self.NAMES, **(spec.params.get("names") or {}))
        self.position_encoding = build_part(POSITION_ENCODINGS, spec.params["position_encoding"],
                                            hidden_size=self.hidden_size, dtype=self.dtype, device=self.device)
        table = getattr(self.position_encoding, "rotary_table", None)
        if table is None:
            raise ValueError("retention: the position encoding has no rotary table")
        self.freq, self.rotary_dims, layout, factor = table()
        if layout != "half" or factor != 1.0 or self.rotary_dims > self.head_dim:
            raise ValueError("retention: queries and keys are turned in the half layout, without a factor, over at "
                             "most the head's width")
        self.w_in = self.w_o = None

    def children(self):
        return (self.position_encoding,)

    def param_specs(self):
        h, n = self.hidden_size, self.names
        return {
            n["q"]: ParamSpec((self.qk_width, h)),
            n["k"]: ParamSpec((self.qk_width, h)),
            n["v"]: ParamSpec((self.v_width, h)),
            n["gate"]: ParamSpec((self.v_width, h)),
            n["out"]: ParamSpec((h, self.v_width)),
        }

    def load(self, tensors):
        n = self.names
        self.w_in = torch.cat([tensors[n[k]] for k in ("q", "k", "v", "gate")], dim=0).contiguous()   # [q | k | v | g]
        self.w_o = tensors[n["out"]].contiguous()

    def in_projection(self):
        return self.w_in, None

    def heads_forward(self, x, ctx, cache, projected=None):
        """``projected``: (a product that holds this mixer's q, k, v and gate columns, the column where they begin)."""
        if cache.state is None:
            raise ValueError("retention: the cache manager gave this position no state")
        if projected is not None:
            x, off = projected
        else:
            x, off = ops.linear(x, self.w_in, status=ctx.status), 0
        rows = ops.rotary_rows(x, ctx.positions, self.freq, num_heads=self.num_heads, head_dim=self.head_dim,
                               v_dim=self.v_dim, rotary_dims=self.rotary_dims, q_off=off, k_off=off + self.qk_width,
                               v_off=off + 2 * self.qk_width, k_scale=self.key_scale)
        o = ops.linear_scan(rows, cache.state, ctx.cu_q, ctx.state_slots, num_heads=self.num_heads,
                            head_dim=self.head_dim, v_dim=self.v_dim, mode="plain_decay", q_off=0,
                            k_off=self.qk_width, v_off=2 * self.qk_width, decay=self.decay)
        return ops.group_norm_gate(o, None, group=self.v_dim, eps=self.norm_eps, out_dtype=x.dtype,
                                   factor=self.out_scale, x=x, gate_off=off + 2 * self.qk_width + self.v_width,
                                   gate="silu")
