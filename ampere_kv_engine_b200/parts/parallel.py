"""Two mixers side by side: both read the same input, and the layer's branch is ``left_scale * left(x) +
right_scale * right(x)``.

Each side is a registered mixer kind of its own.  The layer has one cache view, so at most one side keeps pages; a
side that keeps a state gets its share of the position's state (the sides' floats lie one behind the other in a
request's slot).  When both sides offer ``heads_forward`` / ``out_projection`` (everything before the output
projection, with an ``out_scale`` applied in float32 before the one rounding) and neither output projection has a
bias, the two output projections run as one product over the sides' outputs laid next to each other; otherwise each
side runs whole and ``ops.scaled_sum`` adds them up (sides with a bias on their output projection, or kinds that do
not offer the two methods).

With ``out_norm`` each side's output is first RMS-normed over the model width with a learned weight of its own:
``left_scale * norm_l(left(x)) + right_scale * norm_r(right(x))``.  The sides' output products then leave float32
(the accumulators as they are), and one kernel norms both and adds them up (``ops.normed_pair_sum``).
"""

from __future__ import annotations

import dataclasses

import torch

from ..config.spec import PartSpec
from ..kernels import ops
from .base import MIXERS, CacheSpec, Mixer, ParamSpec, build_part, register_mixer


@register_mixer("parallel")
class ParallelMixers(Mixer):
    """params: ``left`` and ``right`` (PartSpecs of registered mixer kinds), ``left_scale``, ``right_scale``,
    ``out_norm`` (None, or ``{"eps", "left", "right"}``: the epsilon and the local names of the two norm weights)."""

    adds_residual = True

    def __init__(self, spec, **kw):
        super().__init__(spec, **kw)
        p = spec.params
        self.scales = (float(p.get("left_scale", 1.0)), float(p.get("right_scale", 1.0)))
        self.out_norm = dict(p["out_norm"]) if p.get("out_norm") else None
        self.norm_weights = None
        self.w_in = None            # both sides' first projections as one matrix (made at the first step), or False
        self.in_split = 0
        sides = []
        for side, scale in zip((p["left"], p["right"]), self.scales):
            if not isinstance(side, PartSpec):
                raise ValueError("parallel: 'left' and 'right' are part specs of mixers")
            sides.append(side)
        built = [build_part(MIXERS, side, hidden_size=self.hidden_size, dtype=self.dtype, device=self.device)
                 for side in sides]
        # one product for both output projections, if both sides can hand over what stands before theirs
        self.joined = self.out_norm is None and all(hasattr(m, "heads_forward") and hasattr(m, "out_projection")
                                                    and not getattr(m, "out_bias", False) for m in built)
        if self.joined:
            built = [build_part(MIXERS, PartSpec(side.kind, dict(side.params, out_scale=scale), side.prefix),
                                hidden_size=self.hidden_size, dtype=self.dtype, device=self.device)
                     for side, scale in zip(sides, self.scales)]
        self.sides = tuple(built)
        specs = [m.cache_spec() for m in self.sides]
        paged = [s for s in specs if s.kind != "none"]
        if len(paged) > 1:
            raise ValueError("parallel: only one side may keep pages (a schedule position has one cache)")
        self.state_sizes = []
        for s in specs:
            if len(s.state_shape) > 1:
                raise ValueError("parallel: a side's state must be a flat run of floats")
            self.state_sizes.append(int(s.state_shape[0]) if s.state_shape else 0)
        base = paged[0] if paged else CacheSpec()
        total = sum(self.state_sizes)
        self._cache_spec = dataclasses.replace(base, state_shape=(total,) if total else ())
        self.w_o = None

    @property
    def graph_safe(self):
        return all(m.graph_safe for m in self.sides)

    def children(self):
        return self.sides

    def preferred_q_tile(self):
        wishes = {m.preferred_q_tile() for m in self.sides} - {None}
        return wishes.pop() if len(wishes) == 1 else None

    def cache_spec(self) -> CacheSpec:
        return self._cache_spec

    def param_specs(self):
        if self.out_norm is None:
            return {}
        return {self.out_norm[side]: ParamSpec((self.hidden_size,), kind="vector", init="norm")
                for side in ("left", "right")}

    def load(self, tensors):
        """The sides have their tensors by now (children load first is not promised, so the joined matrix is made at
        the first step)."""
        if self.out_norm is not None:
            self.norm_weights = tuple(tensors[self.out_norm[side]].float().contiguous() for side in ("left", "right"))

    def _projected(self, x, ctx):
        """One product for both sides' first projections, where both sides take theirs from a shared product and
        neither has a bias there: ((product, first column of the left side's), (product, first column of the
        right side's)), else (None, None)."""
        if self.w_in is None:
            self.w_in = False
            if all(hasattr(m, "in_projection") and hasattr(m, "heads_forward") and hasattr(m, "out_projection")
                   and m.out_projection()[1] is None and m.in_projection()[1] is None for m in self.sides):
                self.w_in = torch.cat([m.in_projection()[0] for m in self.sides], dim=0).contiguous()
                self.in_split = self.sides[0].in_projection()[0].shape[0]
                # the sides keep views of the one matrix, not copies of their parts
                self.sides[0].w_in, self.sides[1].w_in = self.w_in[:self.in_split], self.w_in[self.in_split:]
        if self.w_in is False:
            return None, None
        both = ops.linear(x, self.w_in, status=ctx.status)
        return (both, 0), (both, self.in_split)

    @staticmethod
    def _float_output(side, x, ctx, cache, projected=None):
        """A side's output in float32: its last product's accumulators where the side lets us run that product."""
        if hasattr(side, "heads_forward") and hasattr(side, "out_projection") and side.out_projection()[1] is None:
            heads = (side.heads_forward(x, ctx, cache, projected=projected) if projected is not None
                     else side.heads_forward(x, ctx, cache))
            return ops.linear(heads, side.out_projection()[0], out_dtype=torch.float32, status=ctx.status)
        return side.forward(x, ctx, cache).float()

    def _views(self, cache):
        views, at = [], 0
        for size in self.state_sizes:
            state = None
            if size:
                state = cache.state[:, at:at + size]
                at += size
            views.append(dataclasses.replace(cache, state=state))
        return views

    def forward(self, x, ctx, cache, residual=None):
        left, right = self.sides
        cl, cr = self._views(cache)
        if self.out_norm is not None:
            pl, pr = self._projected(x, ctx)
            return ops.normed_pair_sum(self._float_output(left, x, ctx, cl, pl), self._float_output(right, x, ctx, cr, pr),
                                       *self.norm_weights, eps=float(self.out_norm["eps"]), sa=self.scales[0],
                                       sb=self.scales[1], out_dtype=torch.float32)
        if self.joined:
            if self.w_o is None:
                self.w_o = torch.cat((left.out_projection()[0], right.out_projection()[0]), dim=1).contiguous()
            both = torch.cat((left.heads_forward(x, ctx, cl), right.heads_forward(x, ctx, cr)), dim=1)
            if residual is not None:
                summed = ops.linear_into_residual(both, self.w_o, residual, status=ctx.status)
                if summed is not None:
                    return summed
            return ops.linear(both, self.w_o, partial_ok=True, status=ctx.status)
        return ops.scaled_sum(left.forward(x, ctx, cl), right.forward(x, ctx, cr), *self.scales)
