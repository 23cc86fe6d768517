"""Position encodings.

``rope``: rotate-half rotary embedding over the first ``rotary_dim`` dims of every head
(the whole head for Qwen3).  ``inv_freq[j] = 1 / theta^(2j / rotary_dim)`` is computed once
in float32 on the host from an int64 ``arange`` exactly as the reference does
(ampere_kv/runner.py:41-44); angles ``position * inv_freq`` and their cos/sin are float32
in the kernel (runner.py:86-93).  ``none``: positions do not enter the mixer.

``rope`` also knows the layout that pairs neighbouring dims (``layout="pairs"``) and a rescaling of the
frequencies by wavelength (``scaling``): with ``turns(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta)``,
``lo = max(floor(turns(fast)), 0)``, ``hi = min(ceil(turns(slow)), rotary_dim - 1)`` and
``ramp_j = clamp((j - lo) / max(hi - lo, 0.001), 0, 1)`` the frequency of pair j becomes
``f_j / factor * ramp_j + f_j * (1 - ramp_j)`` (slow pairs are stretched by ``factor``, fast ones kept) and cos and
sin are multiplied by ``0.1 ln(factor) + 1``.  Such a table is formed in float64 and rounded once.
"""

from __future__ import annotations

import math

import torch

from .base import PositionEncoding, register_position_encoding


@register_position_encoding("rope")
class RotaryEmbedding(PositionEncoding):
    """params: ``theta``, ``rotary_dim``, ``layout`` (``"half"``, the default: dim i pairs with i + rotary_dim / 2;
    ``"pairs"``: dim 2i with 2i + 1), ``scaling`` (None; ``factor`` alone: every frequency divided by it; or
    ``factor``, ``original``, ``fast``, ``slow`` of the rescaling by wavelength)."""

    graph_safe = True


    def __init__(self, spec, **kw):
        super().__init__(spec, **kw)
        self.theta = float(spec.params["theta"])
        self.rotary_dim = int(spec.params["rotary_dim"])
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ValueError(f"rope: rotary_dim must be a positive even number, got {self.rotary_dim}")
        self.layout = str(spec.params.get("layout", "half"))
        if self.layout not in ("half", "pairs"):
            raise ValueError(f"rope: layout must be 'half' or 'pairs', got {self.layout!r}")
        scaling = spec.params.get("scaling")
        self.factor = 1.0
        if scaling is not None and "original" not in scaling:
            # linear scaling: every frequency divided by one factor (positions stretched); float64, rounded once
            stretch = float(scaling["factor"])
            if stretch <= 0:
                raise ValueError("rope: linear scaling needs a positive factor")
            j = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
            self.inv_freq = (self.theta ** (-2.0 * j / self.rotary_dim) / stretch).to(torch.float32).to(self.device)
        elif scaling is None and self.layout == "half":
            exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.int64).float() / self.rotary_dim
            self.inv_freq = (1.0 / (self.theta ** exponent)).to(self.device)
        elif scaling is None:
            j = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
            self.inv_freq = (self.theta ** (-2.0 * j / self.rotary_dim)).to(torch.float32).to(self.device)
        else:
            stretch, original = float(scaling["factor"]), float(scaling["original"])
            if stretch <= 0 or original <= 0 or self.theta <= 1:
                raise ValueError("rope: scaling needs a positive factor and original length and a base above 1")
            j = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
            freq = self.theta ** (-2.0 * j / self.rotary_dim)

            def turns(t: float) -> float:
                return self.rotary_dim * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(self.theta))

            lo = max(math.floor(turns(float(scaling["fast"]))), 0)
            hi = min(math.ceil(turns(float(scaling["slow"]))), self.rotary_dim - 1)
            ramp = ((j - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
            self.inv_freq = (freq / stretch * ramp + freq * (1.0 - ramp)).to(torch.float32).to(self.device)
            self.factor = 0.1 * math.log(stretch) + 1.0

    def fused_rotary(self):
        """The table of the fused rotate-half kernels, which know neither the other layout nor a factor."""
        if self.layout != "half" or self.factor != 1.0:
            return None
        return self.inv_freq, self.rotary_dim

    def rotary_table(self) -> tuple[torch.Tensor, int, str, float]:
        """(frequency per pair float32 [rotary_dim / 2], rotary_dim, layout, factor on cos and sin) for kernels that
        take all four (``ops.rotary_prep``)."""
        return self.inv_freq, self.rotary_dim, self.layout, self.factor

    def apply(self, q, k, positions):
        raise NotImplementedError("rope: this layout or scaling is applied by ops.rotary_prep (mixer "
                                  "'rotary_attention'), not on dense q and k")


@register_position_encoding("none")
class NoPositionEncoding(PositionEncoding):
    graph_safe = True
    def fused_rotary(self):
        return None, 0
