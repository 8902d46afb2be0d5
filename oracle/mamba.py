"""Oracle (test infrastructure): Mamba2/SSD linear branch = ``oracle.gdn`` with
``rule='mamba'`` (no beta, no WY transform, decay clamp of
src/nats/ops/mamba/chunk_h.py:177).  The op does not L2-normalise q/k (the layer
does it with separate modules, src/nats/layers/natsl_attn_mamba2.py:193-194,
469-470) and uses ``scale = 1`` (natsl_attn_mamba2.py:505).
"""
from __future__ import annotations

from .gdn import linear_chunk, linear_recurrent


def mamba_recurrent(q, k, v, g, sel, nbs=64, scale=1.0, h0=None, decay=True):
    return linear_recurrent(q, k, v, g, None, sel, nbs=nbs, scale=scale, h0=h0, decay=decay,
                            use_l2norm=False, rule="mamba")


def mamba_chunk(q, k, v, g, sel, nbs=64, scale=1.0, h0=None, decay=True, **kw):
    return linear_chunk(q, k, v, g, None, sel, nbs=nbs, scale=scale, h0=h0, decay=decay,
                        use_l2norm=False, rule="mamba", **kw)
