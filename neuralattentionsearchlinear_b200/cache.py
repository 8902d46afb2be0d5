"""Decoding state of the NAtSL layers: what a layer keeps between a prefill and the following single-token steps.

The reference's ``NAtSLayerCache`` / ``NAtSCache`` (src/nats/models/utils.py:34-670, 671-853) hold, per layer, the softmax
branch's keys and values, the linear state and the state at the start of the current block, the convolution tails and
the running sum of the layer input over the current block (the selection of a block is decided when its last token has
arrived).  This is a compact restatement of the same bookkeeping for batches without padding:

* keys / values of every token are kept together with the 0/1 types of the finished blocks; visibility of a key for a
  query is evaluated from the types (``generate_msk``), the same object the reference's ``generate_msk`` (:209-287) builds.
  (The reference additionally drops the keys of unselected blocks to save memory; outputs do not depend on that.)
* ``state`` / ``state_block_start`` / ``g_block``: the current recurrent state, the state the current block started from
  and the log decay accumulated in the current block (re-roll at the block end needs all three).
"""
from __future__ import annotations

from typing import List, Optional

import torch


class NAtSLayerCache:
    def __init__(self, nats_block_size: int = 64):
        self.nats_block_size = nats_block_size
        self.n_tokens = 0                               # tokens seen so far
        self.k_attn: Optional[torch.Tensor] = None      # [B, n_tokens, HKV, DK]
        self.v_attn: Optional[torch.Tensor] = None      # [B, n_tokens, HKV, DV]
        self.block_types: Optional[torch.Tensor] = None  # [B, finished blocks, HN, 2] sampled types
        self.state: Optional[torch.Tensor] = None        # [B, H, K, V] fp32: current state
        self.state_block_start: Optional[torch.Tensor] = None
        self.g_block: Optional[torch.Tensor] = None      # [B, H] fp32: log decay of the current block so far
        self.pool_sum: Optional[torch.Tensor] = None     # [B, D] fp32: sum of the layer input over the current block
        self.conv_state = None                           # (q, k, v) tails of the short convolutions

    @property
    def n_tokens_in_nats_block(self) -> int:
        return self.n_tokens % self.nats_block_size

    @property
    def n_finished_blocks(self) -> int:
        return self.n_tokens // self.nats_block_size

    def append_kv(self, k: torch.Tensor, v: torch.Tensor) -> None:
        self.k_attn = k if self.k_attn is None else torch.cat([self.k_attn, k], 1)
        self.v_attn = v if self.v_attn is None else torch.cat([self.v_attn, v], 1)

    def append_types(self, types: torch.Tensor) -> None:
        self.block_types = types if self.block_types is None else torch.cat([self.block_types, types], 1)

    def generate_msk(self, n_data: int, HQ: int, own_chunk: bool = True) -> torch.Tensor:
        """Boolean mask [B, HQ, n_data, n_keys] for the last ``n_data`` tokens as queries over all cached keys (the new
        tokens' keys already appended): a key is visible when its block is finished, softmax-selected and lies before
        the query's block, or when both are in the same block and the key is not later than the query."""
        nbs = self.nats_block_size
        n_keys = self.k_attn.shape[1]
        dev = self.k_attn.device
        B = self.k_attn.shape[0]
        t = torch.arange(n_keys - n_data, n_keys, device=dev)
        s = torch.arange(n_keys, device=dev)
        blk_t, blk_s = t // nbs, s // nbs
        n_done = 0 if self.block_types is None else self.block_types.shape[1]
        if n_done:
            HN = self.block_types.shape[2]
            sel = (self.block_types[..., 0] > 0.5).repeat_interleave(HQ // HN, dim=2).permute(0, 2, 1)     # [B,HQ,n_done]
            col_sel = torch.zeros(B, HQ, n_keys, dtype=torch.bool, device=dev)
            inside = blk_s < n_done
            col_sel[:, :, inside] = sel[:, :, blk_s[inside]]
        else:
            col_sel = torch.zeros(B, HQ, n_keys, dtype=torch.bool, device=dev)
        past = blk_s[None, :] < blk_t[:, None]
        m = col_sel[:, :, None, :] & past[None, None]
        if own_chunk:
            own = (blk_s[None, :] == blk_t[:, None]) & (s[None, :] <= t[:, None])
            m = m | own[None, None]
        return m


class NAtSCache:
    """One ``NAtSLayerCache`` per layer, indexed by ``layer_idx`` (created on first use)."""

    def __init__(self):
        self.layers: List[NAtSLayerCache] = []

    def __len__(self) -> int:
        return len(self.layers)

    def __getitem__(self, layer_idx: int) -> NAtSLayerCache:
        return self.layers[layer_idx]

    def layer(self, layer_idx: int, nats_block_size: int) -> NAtSLayerCache:
        while len(self.layers) <= layer_idx:
            self.layers.append(NAtSLayerCache(nats_block_size))
        return self.layers[layer_idx]

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self.layers[layer_idx].n_tokens if len(self.layers) > layer_idx else 0
