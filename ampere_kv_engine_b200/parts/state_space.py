"""A selective state-space mixer (Mamba-2, the state-space duality form): a matrix memory per head with one scalar
decay per head and token, behind a short causal convolution.

    [z | xBC | step] = W_in h                       z: heads * v_dim, xBC: heads * v_dim + 2 * groups * state, step: heads
    xBC   <- silu(conv(xBC) + conv_bias)            per channel over time, zeros before the sequence's start
    dt     = softplus(step + step_bias);   a = exp(-exp(rate_log) * dt)                       one of each per head
    S     <- a S + dt B x^T;   y = S^T C + skip * x           per head, S: [state, v_dim]; head h reads group
                                                              h // (heads / groups) of B and C
    y     <- y * silu(z), RMS-normed in ``norm_groups`` equal parts of the width, times a weight, then W_o

What a request carries from step to step is float32 and lives in its state slot: every head's S in the scan kernel's
own order, then the last ``taps - 1`` inputs of the convolved channels.  One product makes all projections of a token;
``ops.ssm_prep`` turns them into the float32 rows of a scan with q = C, k = B, v = dt x and a decay per token
(``ops.linear_scan(mode="token_decay")``, which walks a sequence's tokens in order whatever the step holds);
``ops.group_norm_gate`` adds the skip term, gates, and norms; ``ops.conv_tail`` keeps the convolutions' inputs.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import CacheSpec, Mixer, ParamSpec, register_mixer


@register_mixer("mamba2")
class Mamba2(Mixer):
    """params: ``num_heads``, ``v_dim`` (a head's width), ``state_dim``, ``groups`` (of B and C), ``taps`` (of the
    convolution; 1: none), ``norm_groups``, ``norm_eps``, ``names`` (local tensor names of in, conv, conv_bias,
    step_bias, rate_log, skip, norm, out)."""

    graph_safe = True

    NAMES = {"in": "in_proj.weight", "conv": "conv1d.weight", "conv_bias": "conv1d.bias", "step_bias": "dt_bias",
             "rate_log": "A_log", "skip": "D", "norm": "norm.weight", "out": "out_proj.weight"}

    def __init__(self, spec, **kw):
        super().__init__(spec, **kw)
        p = spec.params
        self.num_heads, self.v_dim, self.state_dim = int(p["num_heads"]), int(p["v_dim"]), int(p["state_dim"])
        self.groups, self.taps, self.norm_groups = int(p["groups"]), int(p["taps"]), int(p.get("norm_groups", 1))
        if self.num_heads <= 0 or self.groups <= 0 or self.num_heads % self.groups:
            raise ValueError(f"mamba2: {self.num_heads} heads are not a multiple of {self.groups} groups")
        if self.num_heads > ops.SSM_MAX_HEADS or ops.linear_scan_shape(self.state_dim, self.v_dim) is None:
            raise ValueError(f"mamba2: {self.num_heads} heads with a state of {self.state_dim} x {self.v_dim} are outside "
                             f"what the kernels take ({ops.SSM_MAX_HEADS} heads, each size up to {ops.LINEAR_SCAN_MAX_DIM})")
        if not 1 <= self.taps <= ops.CONV_MAX_TAPS:
            raise ValueError(f"mamba2: {self.taps} taps outside what the kernel takes (1 to {ops.CONV_MAX_TAPS})")
        self.inner = self.num_heads * self.v_dim
        if self.norm_groups <= 0 or self.inner % self.norm_groups:
            raise ValueError(f"mamba2: {self.norm_groups} norm groups do not divide the inner width {self.inner}")
        self.norm_eps = float(p.get("norm_eps", 1e-6))
        self.names = dict(self.NAMES, **(p.get("names") or {}))
        self.channels = self.inner + 2 * self.groups * self.state_dim          # what the convolution runs over
        self.in_width = 2 * self.inner + 2 * self.groups * self.state_dim + self.num_heads
        # a request's state: the memories, then the convolution's last inputs, rounded up to a multiple of four floats
        self.memory = ops.linear_scan_state_floats(self.num_heads, self.state_dim, self.v_dim)
        self.state_floats = (self.memory + (self.taps - 1) * self.channels + 3) // 4 * 4
        self.w_in = self.w_o = self.conv = self.conv_bias = self.step_bias = self.rate_log = self.skip = None
        self.norm_weight = None

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(kind="none", state_shape=(self.state_floats,))

    def param_specs(self):
        h, n = self.hidden_size, self.names
        return {
            n["in"]: ParamSpec((self.in_width, h)),
            n["conv"]: ParamSpec((self.channels, self.taps), kind="vector", init="unit_interval"),
            n["conv_bias"]: ParamSpec((self.channels,), kind="vector", init="around_zero"),
            n["step_bias"]: ParamSpec((self.num_heads,), kind="vector", init="around_zero"),
            n["rate_log"]: ParamSpec((self.num_heads,), kind="vector", init="around_zero"),
            n["skip"]: ParamSpec((self.num_heads,), kind="vector", init="norm"),
            n["norm"]: ParamSpec((self.inner,), kind="vector", init="norm"),
            n["out"]: ParamSpec((h, self.inner)),
        }

    def load(self, tensors):
        n = self.names
        self.w_in = tensors[n["in"]].contiguous()
        for attr, key in (("conv", "conv"), ("conv_bias", "conv_bias"), ("step_bias", "step_bias"),
                          ("rate_log", "rate_log"), ("skip", "skip"), ("norm_weight", "norm")):
            setattr(self, attr, tensors[n[key]].float().contiguous())
        self.w_o = tensors[n["out"]].contiguous()

    def out_projection(self):
        return self.w_o, None

    def heads_forward(self, x, ctx, cache):
        """Everything before the output projection: [tokens, heads * v_dim]."""
        if cache.state is None:
            raise ValueError("mamba2: the cache manager gave this position no state")
        gn = self.groups * self.state_dim
        x = ops.linear(x, self.w_in, status=ctx.status)
        rows = ops.ssm_prep(x, self.conv, self.conv_bias, self.step_bias, self.rate_log, cache.state, ctx.cu_q,
                            ctx.state_slots, tail_off=self.memory, num_heads=self.num_heads, v_dim=self.v_dim,
                            state_dim=self.state_dim, groups=self.groups, taps=self.taps, conv_off=self.inner,
                            step_off=self.inner + self.channels)
        o = ops.linear_scan(rows, cache.state, ctx.cu_q, ctx.state_slots, num_heads=self.num_heads,
                            head_dim=self.state_dim, v_dim=self.v_dim, mode="token_decay", q_off=0, k_off=gn,
                            v_off=2 * gn, qk_group=self.num_heads // self.groups, decay_off=2 * gn + self.inner)
        ops.conv_tail(x, cache.state, ctx.cu_q, ctx.state_slots, tail_off=self.memory, conv_off=self.inner,
                      channels=self.channels, taps=self.taps)
        return ops.group_norm_gate(o, self.norm_weight, group=self.inner // self.norm_groups, eps=self.norm_eps,
                                   out_dtype=x.dtype, x=x, gate_off=0, gate="silu", gate_first=True, skip=rows,
                                   skip_off=2 * gn + self.inner + self.num_heads, skip_coef=self.skip,
                                   skip_head=self.v_dim)

    def forward(self, x, ctx, cache):
        return ops.linear(self.heads_forward(x, ctx, cache), self.w_o, status=ctx.status)
