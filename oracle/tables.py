"""Oracle (test infrastructure): selection decisions and the integer tables.

Restates, in plain torch-on-CPU integer code:
  * ``hard_softmax``                      src/nats/layers/natsl_attn_gdn.py:47-61
  * last-block forcing                    src/nats/layers/natsl_attn_gdn.py:553-554
  * round / index sort / block counts     src/nats/ops/mixed_ops/mixed_attn_gdn.py:88-100
  * ``prepare_nats_block_indices``        src/nats/ops/nats_util.py:6-32
  * ``prepare_nats_chunk_offsets``        src/nats/ops/nats_util.py:35-64
  * ``compute_attn_n_iters_per_block``    src/nats/ops/nats_util.py:67-121
  * ``compute_starting_idx_for_chunks``   src/nats/ops/nats_util.py:124-162

Column 0 of the last axis is the softmax-attention op, column 1 the linear op
(``OFFSET_ATTN = 0``, ``OFFSET_GATED_DELTA_NET = 1``, mixed_attn_gdn.py:107-108).
Only ``nats_block_size >= 64`` with ``nats_block_size % 64 == 0`` is restated
(the reference asserts ``nats_block_size >= CHUNK_SIZE``, mixed_attn_gdn.py:90).
"""
from __future__ import annotations

import torch

OFFSET_ATTN = 0
OFFSET_LINEAR = 1
CHUNK = 64


def cdiv(a: int, b: int) -> int:
    return -(-a // b)


def hard_softmax(logits: torch.Tensor) -> torch.Tensor:
    """One-hot of the first maximum of softmax(logits) over the last axis.

    natsl_attn_gdn.py:55-60 — the maximum is taken over the *softmax output*
    (in the logits' dtype), not over the logits, so ties created by rounding in
    the softmax resolve to the lowest index.  Forward value only.
    """
    y_soft = logits.softmax(-1)
    index = y_soft.max(-1, keepdim=True)[1]
    return torch.zeros_like(logits).scatter_(-1, index, 1.0)


def force_last_block(types: torch.Tensor) -> torch.Tensor:
    """natsl_attn_gdn.py:553 — the last block is selected for every op."""
    types = types.clone()
    types[:, -1] = 1
    return types


def build_tables(types: torch.Tensor, T: int, nbs: int = 64, attn_bt: int = 128,
                 attn_bs: int = 64) -> dict:
    """All integer tables the reference derives from ``nats_block_types``.

    types: [B, TN, HN, 2] (any float dtype; rounded first, mixed_attn_gdn.py:88).
    Returns int64 tensors:
      types_i        [B, TN, HN, 2]   0/1
      indices        [B, TN, HN, 2]   sorted selected block ids, TN = "absent"
      n_blocks       [B, HN, 2]
      chunk_indices  [Nsel, 2]        (b*HN+hn, local j) for the linear op
      offsets        [B*HN + 1]       exclusive prefix sum of selected 64-chunks
      starting_h_idx [B, NT, HN]      stored-state index chunk i reads
      attn_n_iters   [B, NTq, HN]     selected attention blocks fully before tile i
    """
    assert nbs >= CHUNK and nbs % CHUNK == 0
    B, TN, HN, NOPS = types.shape
    assert NOPS == 2 and TN == cdiv(T, nbs)
    ti = torch.round(types.float()).to(torch.int64)
    ar = torch.arange(TN, dtype=torch.int64).view(1, TN, 1, 1)
    indices = torch.where(ti == 1, ar, torch.full_like(ti, TN)).sort(1)[0]
    n_blocks = ti.sum(1)

    # nats_util.py:29-32 / :63-64 — per (b, hn) the number of 64-token compute
    # chunks covered by the selected linear blocks, listed and prefix-summed.
    n_chunks = (n_blocks[..., OFFSET_LINEAR] * nbs + CHUNK - 1) // CHUNK
    flat = n_chunks.flatten()
    rows = []
    for bh, n in enumerate(flat.tolist()):
        for j in range(n):
            rows.append((bh, j))
    chunk_indices = torch.tensor(rows, dtype=torch.int64).reshape(-1, 2)
    offsets = torch.zeros(B * HN + 1, dtype=torch.int64)
    offsets[1:] = flat.cumsum(0)

    # nats_util.py:159-161 — count selected linear blocks that start before chunk i.
    NT = cdiv(T, CHUNK)
    start = torch.arange(NT, dtype=torch.int64) * CHUNK
    lin = indices[..., OFFSET_LINEAR]                                   # [B, TN, HN]
    starting_h_idx = (lin.unsqueeze(1) * nbs < start.view(1, NT, 1, 1)).sum(2)

    # nats_util.py:114-120 — count selected attention blocks that end at or before
    # the first row of query tile i.
    NTq = cdiv(T, attn_bt)
    qstart = torch.arange(NTq, dtype=torch.int64) * attn_bt
    att = indices[..., OFFSET_ATTN]
    attn_n_iters = ((att.unsqueeze(1) + 1) * nbs <= qstart.view(1, NTq, 1, 1)).sum(2)
    return dict(types_i=ti, indices=indices, n_blocks=n_blocks, chunk_indices=chunk_indices,
                offsets=offsets, starting_h_idx=starting_h_idx, attn_n_iters=attn_n_iters)


def synth_types(B: int, TN: int, HN: int, p_attn: float, seed: int,
                force_last: bool = True, dtype=torch.float32) -> torch.Tensor:
    """Seeded synthetic selection: logits ~ N(0,1) with the attention logit shifted
    so that P(softmax op) = p_attn, passed through ``hard_softmax``.
    """
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(B, TN, HN, 2, generator=g, dtype=torch.float32)
    # logit_attn - logit_lin ~ N(shift, 2); P(>0) = p_attn  =>  shift = sqrt(2) * Phi^-1(p_attn)
    shift = (2.0 ** 0.5) * torch.distributions.Normal(0.0, 1.0).icdf(torch.tensor(float(p_attn))).item()
    logits[..., OFFSET_ATTN] += shift
    types = hard_softmax(logits.to(dtype))
    if force_last:
        types = force_last_block(types)
    return types
