"""Sequence-parallel NAtSL-Mamba2 hybrid attention for long sequences (one contiguous segment of the sequence
per rank, in rank order; every segment but the last a multiple of the block size).

Linear branch: the carried state obeys ``h_out = a * h_in + S_loc`` over a segment (scalar decay), so each rank
  1. runs the recurrence on its segment from a zero state            -> S_loc, a
  2. all-gathers (a, S_loc) (a few MB) and folds the earlier ranks   -> h_in
  3. reruns recurrence + output from h_in.
Softmax branch: a rank needs only the *selected* key/value blocks of earlier ranks; they are packed per head,
all-gathered, and placed in front of the rank's own keys, and the attention kernel runs on that virtual sequence
with the query window set to the rank's own tokens.

The reference has no sequence parallelism; results equal the single-device op on the whole sequence with the
decay carried over all skipped blocks (the layers always select the last block, where the reference's handling
of trailing skipped blocks makes no difference).

The collectives are ``torch.distributed`` (NCCL on GPUs); everything else goes through ``backend`` — the CUDA
ops by default.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import _lib, _ops
from .nats_util import build_selection_tables, current_stream_ptr


class CudaSegmentOps:
    """Compute steps of one rank, on the CUDA kernels of this package."""

    def tables(self, types, T, nbs):
        return build_selection_tables(types, T, nbs)

    def linear(self, q, k, v, g, tables, scale, h0, decay, skip_out):
        o, ht, inter = _ops.linear_fwd(_lib.RULE_MAMBA, q, k, v, g, None, tables, scale, h0, decay, False, True,
                                       trailing_quirk=False, return_intermediates=True, skip_out=skip_out)
        return o, ht, inter['gcs']

    def segment_decay(self, gcs, tables, decay):
        B, T, H = gcs.shape
        HN = tables.types_i.shape[2]
        a = torch.empty(B, H, dtype=torch.float32, device=gcs.device)
        trail = torch.empty_like(a)
        _lib.call("natsl_sp_segment_decay", gcs.data_ptr(), tables.types_i.data_ptr(), a.data_ptr(), trail.data_ptr(),
                  B, T, H, HN, tables.nats_block_size, _lib.FLAG_DECAY_SKIPPED if decay else 0,
                  current_stream_ptr(gcs.device))
        return a, trail

    def state_combine(self, a_all, S_all, rank):
        R, B, H, K, V = S_all.shape
        h_in = torch.empty(B, H, K, V, dtype=torch.float32, device=S_all.device)
        _lib.call("natsl_sp_state_combine", a_all.data_ptr(), S_all.data_ptr(), h_in.data_ptr(), rank, R, B, H, K, V,
                  current_stream_ptr(S_all.device))
        return h_in

    def pack(self, x, tables, cap_blocks):
        B, T, H, D = x.shape
        nbs = tables.nats_block_size
        packed = torch.zeros(B, cap_blocks * nbs, H, D, dtype=x.dtype, device=x.device)
        _lib.call("natsl_pack_selected_blocks", x.data_ptr(), tables.indices.data_ptr(), tables.n_blocks.data_ptr(),
                  packed.data_ptr(), B, T, H, tables.types_i.shape[2], D, nbs, 0, cap_blocks,
                  current_stream_ptr(x.device))
        return packed

    def attn(self, q, k, v, tables, scale, own_chunk, q_off):
        return _ops.attn_fwd(q, k, v, tables, scale, own_chunk, q_off=q_off)[0]

    def n_attn_blocks(self, tables):
        return tables.n_blocks[..., 0].contiguous()          # [B, HN] int32


def _all_gather(x: torch.Tensor, world: int, group) -> torch.Tensor:
    """[...] -> [world, ...] (rank order)."""
    x = x.contiguous()
    out = torch.empty((world * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x, group=group)
    return out.view((world,) + tuple(x.shape))


def virtual_attn_types(n_all: torch.Tensor, rank: int, cap: int, types_local: torch.Tensor) -> torch.Tensor:
    """Block types of the virtual key sequence [world x cap gathered slots | own blocks].
    n_all [world, B, HN]: softmax-selected block counts of every rank.  Slot j of rank r' is selected iff
    r' < rank and j < n_all[r'].  The linear column is unused by the softmax branch and left zero."""
    R, B, HN = n_all.shape
    dev = types_local.device
    j = torch.arange(cap, device=dev).view(1, 1, cap, 1)
    earlier = (torch.arange(R, device=dev) < rank).view(R, 1, 1, 1)
    sel = (j < n_all.view(R, B, 1, HN)) & earlier                              # [R,B,cap,HN]
    remote = sel.permute(1, 0, 2, 3).reshape(B, R * cap, HN).to(types_local.dtype)
    attn_col = torch.cat([remote, types_local[..., 0]], 1)
    return torch.stack([attn_col, torch.zeros_like(attn_col)], -1).contiguous()


def nats_mixed_attn_mamba_sp(q_attn, k_attn, v_attn, q_lattn, k_lattn, v_lattn, g, nats_block_types, *,
                             nats_block_size: int = 256, scale_attn=None, scale_lattn=1.0,
                             ops_for_incomplete_chunks: str = 'all', decay_for_non_mamba_blocks: bool = True,
                             group=None, backend=None):
    """One rank's share of ``nats_mixed_attn_mamba`` on a sequence split over the ranks of ``group``.
    All tensors are this rank's segment ([B, T_local, ...]; block types [B, TN_local, HN, 2]).
    -> (o_mamba [B,T_local,H,V], o_attn [B,T_local,HQ,V_attn], final_state [B,H,K,V] fp32)."""
    if ops_for_incomplete_chunks not in ('all', 'mamba'):
        raise NotImplementedError("only own-block linear attention ('all', 'mamba') is built")
    be = backend or CudaSegmentOps()
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    nbs = nats_block_size
    B, T_loc, H, K = q_lattn.shape
    V = v_lattn.shape[-1]
    if scale_attn is None:
        scale_attn = k_attn.shape[-1] ** -0.5
    if rank < world - 1 and T_loc % max(nbs, 128):
        raise ValueError("every segment but the last must be a multiple of the block size (and of 128)")
    own = ops_for_incomplete_chunks == 'all'
    tb = be.tables(nats_block_types, T_loc, nbs)

    # ---- linear branch
    if world == 1:
        o_lin, ht, _ = be.linear(q_lattn, k_lattn, v_lattn, g, tb, scale_lattn, None, decay_for_non_mamba_blocks, False)
    else:
        _, S_loc, gcs = be.linear(q_lattn, k_lattn, v_lattn, g, tb, scale_lattn, None, decay_for_non_mamba_blocks, True)
        a, trail = be.segment_decay(gcs, tb, decay_for_non_mamba_blocks)
        S_end = (S_loc * trail[..., None, None]).contiguous()
        a_all, S_all = _all_gather(a, world, group), _all_gather(S_end, world, group)
        h_in = be.state_combine(a_all, S_all, rank)
        o_lin, ht, _ = be.linear(q_lattn, k_lattn, v_lattn, g, tb, scale_lattn, h_in, decay_for_non_mamba_blocks, False)

    # ---- softmax branch
    if world == 1:
        o_attn = be.attn(q_attn, k_attn, v_attn, tb, scale_attn, own, 0)
    else:
        n_loc = be.n_attn_blocks(tb)
        n_all = _all_gather(n_loc, world, group)
        cap = int(n_all[:world - 1].max().item()) if world > 1 else 0       # one host sync: capacity of the gather
        step = max(1, 128 // nbs)
        cap = -(-cap // step) * step                                          # keep the query offset a multiple of 128
        if cap == 0:
            o_attn = be.attn(q_attn, k_attn, v_attn, tb, scale_attn, own, 0)
        else:
            k_pack, v_pack = be.pack(k_attn.contiguous(), tb, cap), be.pack(v_attn.contiguous(), tb, cap)
            k_all, v_all = _all_gather(k_pack, world, group), _all_gather(v_pack, world, group)
            # [R, B, cap*nbs, H, D] -> [B, R*cap*nbs, H, D], own keys behind
            cat = lambda allp, own_x: torch.cat([allp.permute(1, 0, 2, 3, 4).reshape(B, world * cap * nbs, *own_x.shape[2:]),
                                                 own_x], 1).contiguous()
            k_virt, v_virt = cat(k_all, k_attn), cat(v_all, v_attn)
            types_virt = virtual_attn_types(n_all.to(torch.int64), rank, cap, nats_block_types)
            q_off = world * cap * nbs
            tb_v = be.tables(types_virt, q_off + T_loc, nbs)
            o_attn = be.attn(q_attn, k_virt, v_virt, tb_v, scale_attn, own, q_off)
    return o_lin, o_attn, (ht if rank == world - 1 else None)
