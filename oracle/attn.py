"""Oracle (test infrastructure): the chunk-masked softmax branch.

The boolean mask is the one the reference's own debug script builds to check its
kernel (src/nats/ops/attns/attns.py:2041-2058): key s is visible to query t when
the key's block is softmax-selected and lies entirely before t, or when both
are in the same block and s <= t.  The kernel realises the same object in two
stages (attns.py:173-217 selected past blocks, :271-340 own span).

Outputs follow the kernel's conventions: rows without any visible key give
o = 0 and lse = 0 (attns.py:343-350); lse is base-2 of the scaled scores
(attns.py:158-159, 347).
"""
from __future__ import annotations

import math

import torch


def attn_mask(sel_attn: torch.Tensor, T: int, nbs: int, HQ: int, own_chunk: bool = True) -> torch.Tensor:
    """sel_attn [B,TN,HN] (column 0 of the block types) -> bool mask [B,HQ,T,T].

    Softmax head hq uses selection head ``hq // (HQ // HN)`` (attns.py:101).
    ``own_chunk=False`` is the ``'gated_delta_net'`` / ``'mamba'`` mode where the
    softmax branch only sees fully-past selected blocks (attns.py:319-320).
    """
    B, TN, HN = sel_attn.shape
    t = torch.arange(T)
    blk = t // nbs
    sel = sel_attn.to(torch.bool).repeat_interleave(HQ // HN, dim=2).permute(0, 2, 1)   # [B,HQ,TN]
    col_sel = sel[:, :, blk]                                                            # [B,HQ,T] over keys
    past = t[:, None] >= (blk[None, :] + 1) * nbs                                       # [T,T]
    m = col_sel[:, :, None, :] & past[None, None]
    if own_chunk:
        own = (blk[:, None] == blk[None, :]) & (t[:, None] >= t[None, :])
        m = m | own[None, None]
    return m


def attn_mask_rows(sel_attn: torch.Tensor, T: int, nbs: int, HQ: int, t0: int, t1: int, own_chunk: bool = True) -> torch.Tensor:
    """Rows [t0, t1) of ``attn_mask`` -> bool [B,HQ,t1-t0,T], for sequences whose full mask does not fit in memory."""
    B, TN, HN = sel_attn.shape
    s = torch.arange(T)
    t = torch.arange(t0, t1)
    blk_s, blk_t = s // nbs, t // nbs
    sel = sel_attn.to(torch.bool).repeat_interleave(HQ // HN, dim=2).permute(0, 2, 1)   # [B,HQ,TN]
    col_sel = sel[:, :, blk_s]                                                          # [B,HQ,T]
    past = t[:, None] >= (blk_s[None, :] + 1) * nbs
    m = col_sel[:, :, None, :] & past[None, None]
    if own_chunk:
        own = (blk_t[:, None] == blk_s[None, :]) & (t[:, None] >= s[None, :])
        m = m | own[None, None]
    return m


def attn_sdpa(q, k, v, mask, scale=None):
    """q [B,T,HQ,K]; k [B,T,HKV,K]; v [B,T,HKV,V]; mask [B,HQ,T,T] bool.
    Returns (o [B,T,HQ,V], lse [B,T,HQ] base-2)."""
    B, T, HQ, K = q.shape
    HKV = k.shape[2]
    if scale is None:
        scale = K ** -0.5
    G = HQ // HKV
    qh = q.permute(0, 2, 1, 3)
    kh = k.permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
    vh = v.permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
    s = (qh @ kh.transpose(-1, -2)) * scale
    s = s.masked_fill(~mask, float("-inf"))
    valid = mask.any(-1)
    m = s.amax(-1, keepdim=True)
    m = torch.where(valid[..., None], m, torch.zeros_like(m))
    p = (s - m).exp()
    den = p.sum(-1, keepdim=True)
    o = (p @ vh) / torch.where(valid[..., None], den, torch.ones_like(den))
    o = torch.where(valid[..., None], o, torch.zeros_like(o))
    lse = (m.squeeze(-1) + den.squeeze(-1).clamp_min(1e-38).log()) / math.log(2.0)
    lse = torch.where(valid, lse, torch.zeros_like(lse))
    return o.permute(0, 2, 1, 3).contiguous(), lse.permute(0, 2, 1).contiguous()
