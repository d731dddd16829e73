"""Position encodings.

``rotary``: rotation of query and key halves by position-dependent angles, with the
optional Llama 3 frequency scaling.  Frequencies follow engine/model/layers.py:55-73 and
angles engine/model/layers.py:75-79: everything is 32-bit; the table holds cos and sin of
``position * inv_freq`` for every position the engine can feed, so the kernels read the
same values a whole-sequence computation would.
"""

from __future__ import annotations

import math

from .base import BuildEnv, PositionEncoding
from .registry import register_part


def rotary_inv_freq(rotary_dim: int, theta: float, scaling: dict | None):
    """``inv_freq[j] = theta^(-2j/dim)``; with ``scaling`` (llama3) long wavelengths are
    divided by ``factor``, short ones kept, the band between interpolated."""
    import torch

    inv_freq = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.int64).float() / rotary_dim))
    if not scaling:
        return inv_freq
    factor = float(scaling["factor"])
    low_f, high_f = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    low_wavelen, high_wavelen = orig / low_f, orig / high_f
    wavelen = 2 * math.pi / inv_freq
    scaled = torch.where(wavelen > low_wavelen, inv_freq / factor, inv_freq)
    smooth = (orig / wavelen - low_f) / (high_f - low_f)
    smoothed = (1 - smooth) * scaled / factor + smooth * scaled
    medium = ~(wavelen < high_wavelen) & ~(wavelen > low_wavelen)
    return torch.where(medium, smoothed, scaled)


@register_part("position", "rotary")
class RotaryEncoding(PositionEncoding):
    def __init__(self, rotary_dim: int, theta: float, scaling: dict | None,
                 max_positions: int) -> None:
        if rotary_dim % 2:
            raise ValueError(f"rotary_dim ({rotary_dim}) must be even")
        self.rotary_dim, self.theta, self.scaling = int(rotary_dim), float(theta), scaling
        self.max_positions = int(max_positions)
        self.inv_freq = self._table = None

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        return cls(params["rotary_dim"], params["theta"], params.get("scaling"),
                   env.max_positions)

    def bind(self, tensors, env: BuildEnv) -> None:
        """No stored tensor (the reference keeps ``inv_freq`` out of checkpoints,
        engine/model/layers.py:52-53): the table is computed here, on the device."""
        import torch

        self.inv_freq = rotary_inv_freq(self.rotary_dim, self.theta, self.scaling).to(env.device)
        pos = torch.arange(self.max_positions, device=env.device).float()
        freqs = pos[:, None] * self.inv_freq.float()[None, :]
        self._table = torch.stack((freqs.cos(), freqs.sin()), dim=1).contiguous()  # [P, 2, half]

    def rotary_table(self):
        return self._table


@register_part("position", "none")
class NoPositionEncoding(PositionEncoding):
    """Leaves queries, keys and embeddings as they are."""

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        return cls()
