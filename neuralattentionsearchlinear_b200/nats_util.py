"""Selection tables on the device (host-side mirror of ``src/nats/ops/nats_util.py`` and of the
op prologue ``src/nats/ops/mixed_ops/mixed_attn_gdn.py:88-100`` of the reference).

The reference builds these tables with several torch ops plus a Python loop over a device
tensor (a device-to-host sync, nats_util.py:29-32).  Here one C-ABI call
(``natsl_build_tables``) produces all of them on the current stream, with no sync.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib

CHUNK_SIZE = 64
OFFSET_ATTN = 0
OFFSET_LINEAR = 1

_TYPE_CODES = {torch.bfloat16: _lib.DT_BF16, torch.float32: _lib.DT_F32, torch.float16: _lib.DT_F16,
               torch.int32: _lib.DT_I32}


def cdiv(a: int, b: int) -> int:
    return -(-a // b)


def current_stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


@dataclass
class SelectionTables:
    """All int32, on the device.  Shapes: types_i / indices [B,TN,HN,2]; n_blocks [B,HN,2];
    n_chunks_lin [B*HN]; offsets [B*HN+1]; chunk_indices [B*HN*NT, 2] (first offsets[-1] rows are
    valid); starting_h_idx [B,NT,HN]; attn_n_iters [B,cdiv(T,128),HN]."""
    types_i: torch.Tensor
    indices: torch.Tensor
    n_blocks: torch.Tensor
    n_chunks_lin: torch.Tensor
    offsets: torch.Tensor
    chunk_indices: torch.Tensor
    starting_h_idx: torch.Tensor
    attn_n_iters: torch.Tensor
    T: int
    nats_block_size: int

    def compact_chunk_indices(self) -> torch.Tensor:
        """The reference's ``prepare_nats_block_indices`` result [Nsel, 2] (needs one host sync)."""
        n = int(self.offsets[-1].item())
        return self.chunk_indices[:n]


def build_selection_tables(nats_block_types: torch.Tensor, T: int, nats_block_size: int = 64,
                           with_chunk_indices: bool = False) -> SelectionTables:
    """nats_block_types [B,TN,HN,2] (float 0/1; rounded like mixed_attn_gdn.py:88) -> tables."""
    if not nats_block_types.is_cuda:
        raise ValueError("nats_block_types must be a CUDA tensor (there is no CPU path)")
    if nats_block_types.dtype not in _TYPE_CODES:
        raise TypeError(f"unsupported nats_block_types dtype {nats_block_types.dtype}")
    assert nats_block_size >= CHUNK_SIZE, "nats_block_size must be >= 64"      # mixed_attn_gdn.py:90
    types = nats_block_types.contiguous()
    B, TN, HN, n_ops = types.shape
    if n_ops != 2:
        raise NotImplementedError("selection tables are specified for n_ops == 2")
    dev = types.device
    NT, NTq = cdiv(T, CHUNK_SIZE), cdiv(T, _lib.ATTN_BT)
    i32 = dict(dtype=torch.int32, device=dev)
    t = SelectionTables(
        types_i=torch.empty(B, TN, HN, 2, **i32), indices=torch.empty(B, TN, HN, 2, **i32),
        n_blocks=torch.empty(B, HN, 2, **i32), n_chunks_lin=torch.empty(B * HN, **i32),
        offsets=torch.empty(B * HN + 1, **i32),
        chunk_indices=torch.empty(B * HN * NT if with_chunk_indices else 0, 2, **i32),
        starting_h_idx=torch.empty(B, NT, HN, **i32), attn_n_iters=torch.empty(B, NTq, HN, **i32),
        T=T, nats_block_size=nats_block_size)
    _lib.call("natsl_build_tables", types.data_ptr(), _TYPE_CODES[types.dtype], B, TN, HN, T, nats_block_size,
              _lib.ATTN_BT, t.types_i.data_ptr(), t.indices.data_ptr(), t.n_blocks.data_ptr(),
              t.n_chunks_lin.data_ptr(), t.offsets.data_ptr(),
              t.chunk_indices.data_ptr() if with_chunk_indices else None,
              t.starting_h_idx.data_ptr(), t.attn_n_iters.data_ptr(), current_stream_ptr(dev))
    return t
