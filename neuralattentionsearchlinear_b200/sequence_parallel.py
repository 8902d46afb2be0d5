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


def segment_ids(rank: int, world: int, layout: str) -> list:
    """Global indices of the segments a rank holds, in the order they are laid out in its tensors.
    'contiguous': one segment per rank.  'zigzag': the sequence is cut into 2*world segments and rank r holds
    segments r and 2*world-1-r, which balances the softmax branch (a query sees about a fixed fraction of all
    earlier keys, so late segments are expensive)."""
    if layout == 'contiguous':
        return [rank]
    if layout == 'zigzag':
        return [rank, 2 * world - 1 - rank]
    raise ValueError(f"unknown layout {layout!r}")


def nats_mixed_attn_mamba_sp(q_attn, k_attn, v_attn, q_lattn, k_lattn, v_lattn, g, nats_block_types, *,
                             nats_block_size: int = 256, scale_attn=None, scale_lattn=1.0,
                             ops_for_incomplete_chunks: str = 'all', decay_for_non_mamba_blocks: bool = True,
                             layout: str = 'contiguous', group=None, backend=None):
    """One rank's share of ``nats_mixed_attn_mamba`` on a sequence split over the ranks of ``group``.
    All tensors hold this rank's segment(s) along the time axis ([B, T_local, ...]; block types
    [B, TN_local, HN, 2]); with ``layout='zigzag'`` T_local covers the rank's two equally long segments one after
    the other (see ``segment_ids``).
    -> (o_mamba [B,T_local,H,V], o_attn [B,T_local,HQ,V_attn], final_state [B,H,K,V] fp32 on the rank that holds
    the last segment, else None)."""
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
    own = ops_for_incomplete_chunks == 'all'
    seg = segment_ids(rank, world, layout)
    n_seg = len(seg)
    n_glob = world * n_seg
    last_holder = (n_glob - 1) in seg
    if n_seg > 1 or not last_holder:
        if T_loc % (n_seg * max(nbs, 128)):
            raise ValueError("every segment but the last of the sequence must be a multiple of the block size (and of 128)")
    if world == 1:
        tb = be.tables(nats_block_types, T_loc, nbs)
        o_lin, ht, _ = be.linear(q_lattn, k_lattn, v_lattn, g, tb, scale_lattn, None, decay_for_non_mamba_blocks, False)
        o_attn = be.attn(q_attn, k_attn, v_attn, tb, scale_attn, own, 0)
        return o_lin, o_attn, ht
    L = T_loc // n_seg

    def split(x):                       # [B, n_seg*n, ...] -> [n_seg*B, n, ...]   (segment-major batch)
        if n_seg == 1:
            return x.contiguous()
        n = x.shape[1] // n_seg
        return x.reshape(B, n_seg, n, *x.shape[2:]).transpose(0, 1).reshape(n_seg * B, n, *x.shape[2:]).contiguous()

    def merge(x):                       # inverse of split
        if n_seg == 1:
            return x
        n = x.shape[1]
        return x.reshape(n_seg, B, n, *x.shape[2:]).transpose(0, 1).reshape(B, n_seg * n, *x.shape[2:]).contiguous()

    TNs = nats_block_types.shape[1] // n_seg
    types_s = split(nats_block_types) if n_seg > 1 else nats_block_types.contiguous()
    assert types_s.shape[1] == TNs
    qa, ka, va, ql, kl, vl, gs = (split(x) for x in (q_attn, k_attn, v_attn, q_lattn, k_lattn, v_lattn, g))
    tb = be.tables(types_s, L, nbs)
    # global order of the gathered segments: entry [r', j] of a gathered [world, n_seg, ...] array is segment
    # segment_ids(r', world, layout)[j]; `order` lists (r', j) flat indices by increasing global segment index
    flat_ids = [sid for r in range(world) for sid in segment_ids(r, world, layout)]
    order = sorted(range(n_glob), key=lambda i: flat_ids[i])

    def to_global(x_all):               # [world, n_seg*B, ...] -> [n_glob, B, ...] in sequence order
        y = x_all.reshape(world * n_seg, B, *x_all.shape[2:])
        return y[torch.tensor(order, device=y.device)].contiguous()

    # ---- linear branch
    _, S_loc, gcs = be.linear(ql, kl, vl, gs, tb, scale_lattn, None, decay_for_non_mamba_blocks, True)
    a, trail = be.segment_decay(gcs, tb, decay_for_non_mamba_blocks)
    S_end = (S_loc * trail[..., None, None]).contiguous()
    a_glob, S_glob = to_global(_all_gather(a, world, group)), to_global(_all_gather(S_end, world, group))
    h_in = torch.cat([be.state_combine(a_glob, S_glob, sid) for sid in seg], 0)          # [n_seg*B, H, K, V]
    o_lin, ht, _ = be.linear(ql, kl, vl, gs, tb, scale_lattn, h_in, decay_for_non_mamba_blocks, False)
    final = ht[(seg.index(n_glob - 1)) * B:(seg.index(n_glob - 1) + 1) * B] if last_holder else None

    # ---- softmax branch
    n_loc = be.n_attn_blocks(tb)                                                         # [n_seg*B, HN]
    n_glob_t = to_global(_all_gather(n_loc, world, group))                               # [n_glob, B, HN]
    cap = int(n_glob_t[:n_glob - 1].max().item())            # one host sync: capacity of the gather
    step = max(1, 128 // nbs)
    cap = -(-cap // step) * step                             # keep the query offset a multiple of 128
    if cap == 0:
        o_attn = be.attn(qa, ka, va, tb, scale_attn, own, 0)
    else:
        k_glob = to_global(_all_gather(be.pack(ka, tb, cap), world, group))              # [n_glob, B, cap*nbs, H, D]
        v_glob = to_global(_all_gather(be.pack(va, tb, cap), world, group))
        q_off = n_glob * cap * nbs
        flat = lambda x: x.permute(1, 0, 2, 3, 4).reshape(B, q_off, *x.shape[3:])
        k_rem, v_rem = flat(k_glob), flat(v_glob)
        outs = []
        for j, sid in enumerate(seg):
            sl = slice(j * B, (j + 1) * B)
            k_virt, v_virt = torch.cat([k_rem, ka[sl]], 1).contiguous(), torch.cat([v_rem, va[sl]], 1).contiguous()
            types_virt = virtual_attn_types(n_glob_t.to(torch.int64), sid, cap, types_s[sl])
            tb_v = be.tables(types_virt, q_off + L, nbs)
            outs.append(be.attn(qa[sl].contiguous(), k_virt, v_virt, tb_v, scale_attn, own, q_off))
        o_attn = torch.cat(outs, 0)
    return merge(o_lin), merge(o_attn), final
