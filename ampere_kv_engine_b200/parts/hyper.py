"""A residual stream kept in several copies ("hyper-connections") and the block kind that runs a layer on it.

Every token has ``streams`` copies x_1 .. x_S of the stream (all equal to the embedding's row at the start; the model
reads their sum at the end).  A sublayer with its connection (``read`` [S], ``write`` [S], ``mix`` [S, S] from -> to,
an optional ``scale`` vector over the width) does

    u    = sum_s read[s] x_s
    y    = sublayer(norm(u))                                     norm: RMS with a weight, possibly stored around zero
    x_t <- sum_s mix[s, t] x_s + write[t] * (scale * y)          all t at once from the old copies

The write of one sublayer and the read and norm of the next are one kernel (``ops.hyper_step``): what a connection
hands on is an ``ops.HyperPending``.  The copies, the mixtures and the norm are float32.  A connection with
``streams == 0`` stands for a plain residual stream: one copy, read and written with ones.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import CONNECTIONS, Block, Connection, ParamSpec, register_block, register_connection


@register_connection("hyper_connection")
class HyperConnection(Connection):
    """params: ``streams``, ``eps`` and ``unit_offset`` of the norm, ``learned`` (default True: the connection has
    ``read``, ``write`` and ``mix`` tensors; False: ones and the identity), ``names`` (local tensor names of ``norm``,
    ``read``, ``write``, ``mix`` and ``scale``; a ``scale`` of None means no scale vector)."""

    graph_safe = True

    NAMES = {"norm": "norm.weight", "read": "read", "write": "write", "mix": "mix", "scale": None}

    def __init__(self, spec, **kw):
        super().__init__(spec, **kw)
        p = spec.params
        self.streams = int(p["streams"])
        if not 1 <= self.streams <= ops.HYPER_MAX_STREAMS:
            raise ValueError(f"hyper_connection: {self.streams} streams outside what the kernel takes "
                             f"(1 to {ops.HYPER_MAX_STREAMS})")
        self.eps = float(p["eps"])
        self.unit_offset = bool(p.get("unit_offset", False))
        self.learned = bool(p.get("learned", True))
        self.names = dict(self.NAMES, **(p.get("names") or {}))
        self.weight = self.read_coef = self.write_coef = self.mix = self.scale = None

    def param_specs(self):
        n, s = self.names, self.streams
        specs = {n["norm"]: ParamSpec((self.hidden_size,), kind="vector",
                                      init="around_zero" if self.unit_offset else "norm")}
        if self.learned:
            specs[n["read"]] = ParamSpec((s,), kind="vector", init="norm")
            specs[n["write"]] = ParamSpec((s,), kind="vector", init="norm")
            specs[n["mix"]] = ParamSpec((s, s), kind="vector", init="unit_interval")
        if n["scale"] is not None:
            specs[n["scale"]] = ParamSpec((self.hidden_size,), kind="vector", init="norm")
        return specs

    def load(self, tensors):
        n, s = self.names, self.streams
        norm = tensors[n["norm"]].float()
        self.weight = (norm + 1.0 if self.unit_offset else norm).contiguous()
        if self.learned:
            self.read_coef = tensors[n["read"]].float().contiguous()
            self.write_coef = tensors[n["write"]].float().contiguous()
            self.mix = tensors[n["mix"]].float().contiguous()
        else:
            self.read_coef = torch.ones(s, dtype=torch.float32, device=norm.device)
            self.write_coef = torch.ones(s, dtype=torch.float32, device=norm.device)
            self.mix = torch.eye(s, dtype=torch.float32, device=norm.device)
        self.scale = tensors[n["scale"]].float().contiguous() if n["scale"] is not None else None

    def read(self, streams, pending, ctx):
        return ops.hyper_step(streams, pending, self.read_coef, self.weight, self.eps, self.dtype,
                              status=getattr(ctx, "status", None))

    def write(self, y):
        if y.dim() == 3:            # a stack of split-K partial sums
            y = y.sum(0)
        return ops.HyperPending(y, self.mix, self.write_coef, self.scale)


@register_block("hyper")
class HyperBlock(Block):
    """roles: ``mixer_connection``, ``mixer``, ``feed_forward_connection``, ``feed_forward`` (the last two may be
    absent).  ``hidden`` is [tokens, streams, width]; what travels between blocks in place of a pending delta is the
    last sublayer's unwritten result (``ops.HyperPending``)."""

    def __init__(self, layer, **kw):
        super().__init__(layer, **kw)
        self.mixer_connection = self.build_role("mixer_connection", CONNECTIONS)
        self.mixer = self.build_role("mixer")
        self.feed_forward = self.feed_forward_connection = None
        if layer.feed_forward is not None:
            self.feed_forward_connection = self.build_role("feed_forward_connection", CONNECTIONS)
            self.feed_forward = self.build_role("feed_forward")

    def forward(self, hidden, delta, ctx, cache):
        if hidden.dim() != 3 or hidden.shape[1] != self.mixer_connection.streams:
            raise ValueError(f"block kind 'hyper': the stream must come in {self.mixer_connection.streams} copies "
                             f"[tokens, streams, width], got {tuple(hidden.shape)}")
        if delta is not None and not isinstance(delta, ops.HyperPending):
            raise ValueError("block kind 'hyper' follows a block that leaves something else than an unwritten "
                             "sublayer result")
        x = self.mixer_connection.read(hidden, delta, ctx)
        pending = self.mixer_connection.write(self.mixer.forward(x, ctx, cache))
        if self.feed_forward is not None:
            x = self.feed_forward_connection.read(hidden, pending, ctx)
            pending = self.feed_forward_connection.write(self.feed_forward.forward(x, ctx))
        return hidden, pending
