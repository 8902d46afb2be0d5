"""Sequence-parallel NAtSL-Mamba2 hybrid attention for long sequences.

The sequence is cut into segments; a rank holds one segment ('contiguous') or two ('zigzag': segments r and
2R-1-r of 2R, which balances the softmax branch).  Every segment but the last of the sequence is a multiple of
the block size.

Linear branch: over a segment the carried state obeys ``h_out = a * h_in + S_loc`` (scalar decay), so
  1. every segment is cut further into short sub-segments that run side by side as batch entries (the
     recurrence is serial over chunks, so this is also what keeps one GPU busy at batch 1), each from a zero
     state                                                                        -> S_loc, a per sub-segment
  2. the sub-segments of a segment are folded locally, the per-segment (a, S) pairs (a few MB) are all-gathered
     and folded over the earlier segments                                         -> h_in of every sub-segment
  3. recurrence + output are rerun from h_in.
Softmax branch: a segment needs only the *selected* key/value blocks of earlier segments; they are packed per
head and all-gathered, and the attention kernel reads its keys from two places: the gathered buffer (shared by
the rank's segments) and the segment's own keys, with the query window set to the segment's own tokens.

The two branches run on two streams; the one host read (the capacity of the key/value gather) happens while
the linear branch is already enqueued.  The reference has no sequence parallelism; results equal the
single-device op on the whole sequence with the decay carried over all skipped blocks (the layers always
select the last block, where the reference's handling of trailing skipped blocks makes no difference).

The collectives are ``torch.distributed`` (NCCL on GPUs); everything else goes through ``backend`` — the CUDA
ops by default.
"""
from __future__ import annotations

import contextlib
import functools
import os

import torch
import torch.distributed as dist

from . import _lib, _ops
from .nats_util import build_selection_tables, current_stream_ptr

_side_streams: dict = {}
last_kv_capacity = None          # (blocks per head, pairs) the last call without ``kv_capacity`` read back


class CudaSegmentOps:
    """Compute steps of one rank, on the CUDA kernels of this package."""

    def side_stream(self, device):
        idx = device.index if device.index is not None else torch.cuda.current_device()
        if idx not in _side_streams:
            _side_streams[idx] = torch.cuda.Stream(device=idx)
        return _side_streams[idx]

    def tables(self, types, T, nbs):
        return build_selection_tables(types, T, nbs)

    def linear(self, q, k, v, g, tables, scale, h0, decay, skip_out):
        o, ht, inter = _ops.linear_fwd(_lib.RULE_MAMBA, q, k, v, g, None, tables, scale, h0, decay, False, True,
                                       trailing_quirk=False, skip_out=skip_out)
        return o, ht, (inter['gcs'] if inter else None)

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

    def prefix_states(self, a, S, h0, want_prefix):
        N, B, H, K, V = S.shape
        dev = S.device
        prefix = torch.empty_like(S) if want_prefix else None
        tot_S = torch.empty(B, H, K, V, dtype=torch.float32, device=dev)
        tot_a = torch.empty(B, H, dtype=torch.float32, device=dev)
        _lib.call("natsl_sp_prefix_states", a.data_ptr(), S.data_ptr(), _lib.ptr(h0), _lib.ptr(prefix), tot_S.data_ptr(),
                  tot_a.data_ptr(), N, B, H, K, V, current_stream_ptr(dev))
        return prefix, tot_S, tot_a

    def pack(self, x, tables, cap_blocks):
        B, T, H, D = x.shape
        nbs = tables.nats_block_size
        # slots past a head's number of selected blocks stay unwritten: they are never selected in the virtual sequence
        packed = torch.empty(B, cap_blocks * nbs, H, D, dtype=x.dtype, device=x.device)
        _lib.call("natsl_pack_selected_blocks", x.data_ptr(), tables.indices.data_ptr(), tables.n_blocks.data_ptr(),
                  packed.data_ptr(), B, T, H, tables.types_i.shape[2], D, nbs, 0, cap_blocks,
                  current_stream_ptr(x.device))
        return packed

    def attn(self, q, k, v, tables, scale, own_chunk, q_off):
        return _ops.attn_fwd(q, k, v, tables, scale, own_chunk, q_off=q_off)[0]

    def pack_pairs(self, x, tables, cap_pairs, max_per_head=0):
        B, T, H, D = x.shape
        nbs = tables.nats_block_size
        packed = torch.empty(B, cap_pairs * nbs, D, dtype=x.dtype, device=x.device)     # the tail past the last pair is never read
        _lib.call("natsl_pack_selected_pairs", x.data_ptr(), tables.indices.data_ptr(), tables.n_blocks.data_ptr(),
                  packed.data_ptr(), B, T, H, tables.types_i.shape[2], D, nbs, 0, cap_pairs, int(max_per_head),
                  current_stream_ptr(x.device))
        return packed

    def attn_split(self, q, k_rem, v_rem, k, v, tables, scale, own_chunk, rem_base, rem_slots):
        return _ops.attn_fwd_split(q, k_rem, v_rem, k, v, tables, scale, own_chunk, rem_base, rem_slots)

    def n_attn_blocks(self, tables):
        return tables.n_blocks[..., 0].contiguous()          # [B, HN] int32


def _all_gather(x: torch.Tensor, world: int, group) -> torch.Tensor:
    """[...] -> [world, ...] (rank order)."""
    x = x.contiguous()
    out = torch.empty((world * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x, group=group)
    return out.view((world,) + tuple(x.shape))


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


@functools.lru_cache(maxsize=None)
def _layout_constants(world: int, layout: str, device_str: str):
    """(global id of every gathered segment [world*n_seg] in gathered order, permutation gathered -> sequence order)."""
    flat_ids = [sid for r in range(world) for sid in segment_ids(r, world, layout)]
    order = sorted(range(len(flat_ids)), key=lambda i: flat_ids[i])
    dev = torch.device(device_str)
    return torch.tensor(flat_ids, device=dev), torch.tensor(order, device=dev)


@functools.lru_cache(maxsize=None)
def _ids_tensor(ids: tuple, device_str: str) -> torch.Tensor:
    return torch.tensor(list(ids), device=torch.device(device_str))


def virtual_attn_types(n_all: torch.Tensor, gathered_ids: torch.Tensor, my_ids, cap: int,
                       types_local: torch.Tensor) -> torch.Tensor:
    """Block types of the virtual key sequences [G x cap gathered slots | own blocks] of the rank's segments.
    n_all [G, B, HN]: softmax-selected block counts of every gathered segment (gathered order); gathered_ids [G]:
    their global segment index; my_ids: global indices of the n local segments; types_local [n*B, TN, HN, 2]
    (segment-major batch).  Slot j of gathered segment g is selected for local segment i iff
    gathered_ids[g] < my_ids[i] and j < n_all[g].  The linear column is unused by the softmax branch (zero)."""
    G, B, HN = n_all.shape
    dev = types_local.device
    n = len(my_ids)
    mine = _ids_tensor(tuple(my_ids), str(dev)).view(n, 1, 1, 1, 1)       # cached: no host copy inside a graph capture
    slot = torch.arange(cap, device=dev).view(1, 1, 1, cap, 1)
    vis = gathered_ids.to(dev).view(1, 1, G, 1, 1) < mine
    sel = vis & (slot < n_all.permute(1, 0, 2).reshape(1, B, G, 1, HN))                  # [n,B,G,cap,HN]
    remote = sel.reshape(n * B, G * cap, HN).to(types_local.dtype)
    attn_col = torch.cat([remote, types_local[..., 0]], 1)
    return torch.stack([attn_col, torch.zeros_like(attn_col)], -1).contiguous()


def pick_linear_splits(L: int, nbs: int, target_tokens: int = 1024) -> int:
    """Number of equal sub-segments (multiples of the block size and of 128 tokens) a segment of L tokens is cut
    into for the linear branch; 1 for a ragged segment."""
    unit = max(nbs, 128)
    if L % unit:
        return 1
    best = 1
    for s in range(1, L // unit + 1):
        if L % (s * unit) == 0 and L // s >= target_tokens:
            best = s
    return best


def _split(x, B, n):                    # [B, n*m, ...] -> [n*B, m, ...]   (segment-major batch)
    if n == 1:
        return x.contiguous()
    m = x.shape[1] // n
    return x.reshape(B, n, m, *x.shape[2:]).transpose(0, 1).reshape(n * B, m, *x.shape[2:]).contiguous()


def _merge(x, B, n):                    # inverse of _split
    if n == 1:
        return x
    m = x.shape[1]
    return x.reshape(n, B, m, *x.shape[2:]).transpose(0, 1).reshape(B, n * m, *x.shape[2:]).contiguous()


def nats_mixed_attn_mamba_sp(q_attn, k_attn, v_attn, q_lattn, k_lattn, v_lattn, g, nats_block_types, *,
                             nats_block_size: int = 256, scale_attn=None, scale_lattn=1.0,
                             ops_for_incomplete_chunks: str = 'all', decay_for_non_mamba_blocks: bool = True,
                             layout: str = 'contiguous', linear_splits=None, kv_capacity=None, group=None,
                             linear_group=None, backend=None):
    """One rank's share of ``nats_mixed_attn_mamba`` on a sequence split over the ranks of ``group`` (also usable
    with a single rank, where only the sub-segment split of the linear branch remains).
    All tensors hold this rank's segment(s) along the time axis ([B, T_local, ...]; block types
    [B, TN_local, HN, 2]); with ``layout='zigzag'`` T_local covers the rank's two equally long segments one after
    the other (see ``segment_ids``).  ``linear_splits``: sub-segments per segment in the linear branch (default:
    about 1024 tokens each).  ``kv_capacity`` = (softmax-selected blocks per head, selected (block, head) pairs) a
    segment may have at most: sizes the key/value gather without reading the counts back to the host (no host
    synchronisation, so the call can be captured in a CUDA graph); if a segment exceeds it the device status
    (``natsl_device_status``) reads 3 and the outputs are invalid.  Without it the exact maxima are read back (one
    host synchronisation) and left in ``last_kv_capacity``.  ``linear_group``: a second process group over the same
    ranks for the collectives of the linear branch, so that they do not queue behind the key/value gather.
    -> (o_mamba [B,T_local,H,V], o_attn [B,T_local,HQ,V_attn], final_state [B,H,K,V] fp32 on the rank that holds
    the last segment, else None)."""
    if ops_for_incomplete_chunks not in ('all', 'mamba'):
        raise NotImplementedError("only own-block linear attention ('all', 'mamba') is built")
    be = backend or CudaSegmentOps()
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    nbs = nats_block_size
    B, T_loc, H, K = q_lattn.shape
    dev = q_lattn.device
    if scale_attn is None:
        scale_attn = k_attn.shape[-1] ** -0.5
    own = ops_for_incomplete_chunks == 'all'
    decay = decay_for_non_mamba_blocks
    seg = segment_ids(rank, world, layout)
    n_seg = len(seg)
    n_glob = world * n_seg
    last_holder = (n_glob - 1) in seg
    if n_seg > 1 or not last_holder:
        if T_loc % (n_seg * max(nbs, 128)):
            raise ValueError("every segment but the last of the sequence must be a multiple of the block size (and of 128)")
    L = T_loc // n_seg
    s_lin = int(linear_splits) if linear_splits else pick_linear_splits(L, nbs)
    if s_lin > 1 and L % (s_lin * max(nbs, 128)):
        raise ValueError(f"linear_splits={s_lin} does not cut a {L}-token segment into multiples of the block size")
    n_sub = n_seg * s_lin
    gathered_ids, order = _layout_constants(world, layout, str(dev))

    def to_global(x_all):               # [world, n_seg*B, ...] -> [n_glob, B, ...] in sequence order
        y = x_all.reshape(world * n_seg, B, *x_all.shape[2:])
        return y if layout == 'contiguous' else y[order].contiguous()

    side = be.side_stream(dev) if hasattr(be, 'side_stream') else None
    cur = torch.cuda.current_stream(dev) if side is not None else None
    on_side = (lambda: torch.cuda.stream(side)) if side is not None else contextlib.nullcontext
    made_on_side = []

    # ---- softmax branch, part 1 (main stream): per-segment tables and the selected-block counts of every segment
    types_s = _split(nats_block_types, B, n_seg)
    qa, ka, va = (_split(x, B, n_seg) for x in (q_attn, k_attn, v_attn))
    tb = be.tables(types_s, L, nbs)
    if side is not None:
        side.wait_stream(cur)
    if world > 1:
        n_all = _all_gather(be.n_attn_blocks(tb), world, group)                          # [world, n_seg*B, HN]

    # ---- linear branch, part 1 (side stream): every sub-segment from a zero state, folded per segment
    with on_side():
        types_l = _split(nats_block_types, B, n_sub)
        ql, kl, vl, gl = (_split(x, B, n_sub) for x in (q_lattn, k_lattn, v_lattn, g))
        tbl = tb if n_sub == n_seg else be.tables(types_l, L // s_lin, nbs)
        if world > 1 or s_lin > 1:
            _, S_loc, gcs = be.linear(ql, kl, vl, gl, tbl, scale_lattn, None, decay, True)
            a, trail = be.segment_decay(gcs, tbl, decay)
            S_end = S_loc * trail[..., None, None]
            a_sub = a.view(n_seg, s_lin, B, H)
            S_sub = S_end.view(n_seg, s_lin, B, H, K, -1)
            if s_lin > 1:
                tot = [be.prefix_states(a_sub[j], S_sub[j], None, False) for j in range(n_seg)]
                S_seg = torch.stack([t[1] for t in tot]).reshape(n_seg * B, H, K, -1)
                a_seg = torch.stack([t[2] for t in tot]).reshape(n_seg * B, H)
            else:
                S_seg, a_seg = S_end, a

    # ---- softmax branch, part 2 (main stream): gather the selected blocks, one attention launch for all segments
    cap = 0
    if world > 1:
        HKV = ka.shape[2]
        n_g = n_all.reshape(n_glob, B, -1).to(torch.int64)                               # gathered order
        n_h = n_g.repeat_interleave(HKV // n_g.shape[2], dim=2)                          # per key/value head
        if kv_capacity is not None:
            cap, cap_pairs = (int(x) for x in kv_capacity)
            limit = cap
        else:
            # the one host read: virtual slots per head and capacity (in pairs) of the gather
            cap, cap_pairs = (int(x) for x in torch.stack([n_g.max(), n_h.sum(2).max()]).tolist())
            limit = 0
            global last_kv_capacity
            last_kv_capacity = (cap, cap_pairs)
        step = max(1, 128 // nbs)
        cap = -(-cap // step) * step                         # keeps the query offset a multiple of 128
        if kv_capacity is not None:
            # a caller-given capacity always takes the packed path (also when it is zero), so that segments holding
            # more selected blocks than promised set device status 3 instead of being left out silently
            cap, cap_pairs = max(step, cap), max(1, cap_pairs)
            limit = cap
    if cap == 0:
        o_attn = be.attn(qa, ka, va, tb, scale_attn, own, 0)
    else:
        # selected (block, head) pairs of every segment, packed back to back: [world, n_seg*B, cap_pairs*nbs, D]
        k_all = _all_gather(be.pack_pairs(ka, tb, cap_pairs, limit), world, group)
        v_all = _all_gather(be.pack_pairs(va, tb, cap_pairs, limit), world, group)

        def flat(x):                    # -> [B, n_glob*cap_pairs*nbs, D], gathered order (a view when B = 1)
            x = x.reshape(n_glob, B, cap_pairs * nbs, x.shape[-1])
            return x.permute(1, 0, 2, 3).reshape(B, n_glob * cap_pairs * nbs, x.shape[-1]).contiguous()

        seg_base = torch.arange(n_glob, device=dev).view(n_glob, 1, 1) * cap_pairs
        rem_base = (n_h.cumsum(2) - n_h + seg_base).permute(1, 0, 2).to(torch.int32).contiguous()   # [B, n_glob, HKV]
        types_virt = virtual_attn_types(n_g, gathered_ids, seg, cap, types_s)
        tb_v = be.tables(types_virt, n_glob * cap * nbs + L, nbs)
        o_attn = be.attn_split(qa, flat(k_all), flat(v_all), ka, va, tb_v, scale_attn, own, rem_base, cap)

    # ---- linear branch, part 2 (side stream): fold the earlier segments, rerun from the true starting states
    with on_side():
        if world > 1 or s_lin > 1:
            if world > 1:
                lg = linear_group if linear_group is not None else group
                a_glob, S_glob = to_global(_all_gather(a_seg, world, lg)), to_global(_all_gather(S_seg, world, lg))
                h_seg = [be.state_combine(a_glob, S_glob, sid) for sid in seg]           # state each segment starts from
            else:
                h_seg = [None] * n_seg
            if s_lin > 1:
                h_in = torch.cat([be.prefix_states(a_sub[j], S_sub[j], h_seg[j], True)[0] for j in range(n_seg)], 0)
                h_in = h_in.reshape(n_sub * B, H, K, -1)
            else:
                h_in = torch.cat(h_seg, 0)
        else:
            h_in = None
        o_lin, ht, _ = be.linear(ql, kl, vl, gl, tbl, scale_lattn, h_in, decay, False)
        final = None
        if last_holder:
            j = seg.index(n_glob - 1)
            e = (j * s_lin + s_lin - 1) * B
            final = ht[e:e + B]
        o_lin = _merge(o_lin, B, n_sub)
        made_on_side = [o_lin] + ([final] if final is not None else [])
    if side is not None:
        cur.wait_stream(side)
        for t_ in made_on_side:
            t_.record_stream(cur)
        for t_ in (q_lattn, k_lattn, v_lattn, g, nats_block_types):
            t_.record_stream(side)
    return o_lin, _merge(o_attn, B, n_seg), final


class GraphedMambaSP:
    """Plan / replay form of ``nats_mixed_attn_mamba_sp`` for a fixed shape (several ranks, CUDA kernels).

    At this scale a rank's share is a few hundred microseconds of GPU work, less than the host needs to issue the
    ~100 small launches of the eager function.  The plan binds to the caller's tensors (update their contents in
    place between runs), sizes the key/value gather from ``kv_capacity`` (see ``nats_mixed_attn_mamba_sp``) and
    captures the compute in four CUDA graphs; the NCCL all-gathers (two group calls: counts + keys + values, and the
    (a, S) pairs) stay eager, between the graphs:

        graph A  tables, block counts, packed selected (block, head) pairs
        gather   counts, packed keys, packed values          (asynchronous, default group; runs under B, C)
        graph B  linear branch from zero states, per-segment (a, S)
        gather   (a, S)                                       (``linear_group``, its own communicator)
        graph C  state fold, recurrence and output from the true starting states
        graph D  virtual tables + attention                   (after the key/value gather has arrived)

    ``run()`` returns the same triple as the eager function; the tensors are reused by the next run.
    """

    def __init__(self, q_attn, k_attn, v_attn, q_lattn, k_lattn, v_lattn, g, nats_block_types, *, kv_capacity,
                 nats_block_size: int = 256, scale_attn=None, scale_lattn=1.0, ops_for_incomplete_chunks: str = 'all',
                 decay_for_non_mamba_blocks: bool = True, layout: str = 'zigzag', linear_splits=None, group=None,
                 linear_group=None, gather_under_linear=None):
        if ops_for_incomplete_chunks not in ('all', 'mamba'):
            raise NotImplementedError("only own-block linear attention ('all', 'mamba') is built")
        if not dist.is_initialized() or dist.get_world_size(group) < 2:
            raise ValueError("the plan form is for several ranks; use nats_mixed_attn_mamba_sp on one")
        be = CudaSegmentOps()
        self.group, self.lin_group = group, (linear_group if linear_group is not None else group)
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        self.world = world
        # order of a step: True = the key/value gather runs under the whole linear branch and the attention follows;
        # False = both gathers first, then the two branches side by side on two streams (measured within 3 % of each
        # other at 4 and 8 ranks)
        self.gather_under_linear = (world >= 8) if gather_under_linear is None else bool(gather_under_linear)
        self._side = be.side_stream(q_lattn.device)
        nbs = nats_block_size
        B, T_loc, H, K = q_lattn.shape
        dev = q_lattn.device
        self.dev = dev
        if scale_attn is None:
            scale_attn = k_attn.shape[-1] ** -0.5
        own = ops_for_incomplete_chunks == 'all'
        decay = decay_for_non_mamba_blocks
        seg = segment_ids(rank, world, layout)
        n_seg = len(seg)
        n_glob = world * n_seg
        if T_loc % (n_seg * max(nbs, 128)):
            raise ValueError("every segment must be a multiple of the block size (and of 128)")
        L = T_loc // n_seg
        s_lin = int(linear_splits) if linear_splits else pick_linear_splits(L, nbs)
        n_sub = n_seg * s_lin
        gathered_ids, order = _layout_constants(world, layout, str(dev))
        cap, cap_pairs = (int(x) for x in kv_capacity)
        limit = cap
        step = max(1, 128 // nbs)
        cap = max(step, -(-cap // step) * step)
        cap_pairs = max(1, cap_pairs)
        HKV = k_attn.shape[2]
        last_holder = (n_glob - 1) in seg
        st = {}                          # tensors handed from one stage to the next (static once captured)

        def to_global(x_all):
            y = x_all.reshape(world * n_seg, B, *x_all.shape[2:])
            return y if layout == 'contiguous' else y[order].contiguous()

        def stage_a():
            st['types_s'] = _split(nats_block_types, B, n_seg)
            st['qa'], st['ka'], st['va'] = (_split(x, B, n_seg) for x in (q_attn, k_attn, v_attn))
            st['tb'] = be.tables(st['types_s'], L, nbs)
            st['n_loc'] = be.n_attn_blocks(st['tb'])
            st['pk'] = be.pack_pairs(st['ka'], st['tb'], cap_pairs, limit)
            st['pv'] = be.pack_pairs(st['va'], st['tb'], cap_pairs, limit)

        def stage_b():
            types_l = _split(nats_block_types, B, n_sub)
            st['lin_in'] = tuple(_split(x, B, n_sub) for x in (q_lattn, k_lattn, v_lattn, g))
            ql, kl, vl, gl = st['lin_in']
            st['tbl'] = be.tables(types_l, L // s_lin, nbs)
            _, S_loc, gcs = be.linear(ql, kl, vl, gl, st['tbl'], scale_lattn, None, decay, True)
            a, trail = be.segment_decay(gcs, st['tbl'], decay)
            S_end = S_loc * trail[..., None, None]
            st['a_sub'] = a.view(n_seg, s_lin, B, H)
            st['S_sub'] = S_end.view(n_seg, s_lin, B, H, K, -1)
            if s_lin > 1:
                tot = [be.prefix_states(st['a_sub'][j], st['S_sub'][j], None, False) for j in range(n_seg)]
                st['S_seg'] = torch.stack([t[1] for t in tot]).reshape(n_seg * B, H, K, -1).contiguous()
                st['a_seg'] = torch.stack([t[2] for t in tot]).reshape(n_seg * B, H).contiguous()
            else:
                st['S_seg'], st['a_seg'] = S_end.contiguous(), a.contiguous()

        def stage_c():                   # linear branch from the true starting states; needs the (a, S) gather only
            a_glob, S_glob = to_global(st['a_all']), to_global(st['S_all'])
            h_seg = [be.state_combine(a_glob, S_glob, sid) for sid in seg]
            if s_lin > 1:
                h_in = torch.cat([be.prefix_states(st['a_sub'][j], st['S_sub'][j], h_seg[j], True)[0]
                                  for j in range(n_seg)], 0).reshape(n_sub * B, H, K, -1)
            else:
                h_in = torch.cat(h_seg, 0)
            ql, kl, vl, gl = st['lin_in']
            o_lin, ht, _ = be.linear(ql, kl, vl, gl, st['tbl'], scale_lattn, h_in, decay, False)
            final = None
            if last_holder:
                j = seg.index(n_glob - 1)
                e = (j * s_lin + s_lin - 1) * B
                final = ht[e:e + B]
            st['o_lin'], st['final'] = _merge(o_lin, B, n_sub), final

        def stage_d():                   # softmax branch; needs the key/value gather
            n_g = st['n_all'].reshape(n_glob, B, -1).to(torch.int64)
            n_h = n_g.repeat_interleave(HKV // n_g.shape[2], dim=2)

            def flat(x):
                x = x.reshape(n_glob, B, cap_pairs * nbs, x.shape[-1])
                return x.permute(1, 0, 2, 3).reshape(B, n_glob * cap_pairs * nbs, x.shape[-1]).contiguous()

            seg_base = torch.arange(n_glob, device=dev).view(n_glob, 1, 1) * cap_pairs
            rem_base = (n_h.cumsum(2) - n_h + seg_base).permute(1, 0, 2).to(torch.int32).contiguous()
            types_virt = virtual_attn_types(n_g, gathered_ids, seg, cap, st['types_s'])
            tb_v = be.tables(types_virt, n_glob * cap * nbs + L, nbs)
            o_attn = be.attn_split(st['qa'], flat(st['k_all']), flat(st['v_all']), st['ka'], st['va'], tb_v, scale_attn,
                                   own, rem_base, cap)
            st['out'] = (st['o_lin'], _merge(o_attn, B, n_seg), st['final'])

        self.coalesce = os.environ.get("NATSL_SP_COALESCE", "1") == "1"
        self._stages = (stage_a, stage_b, stage_c, stage_d)
        self._st = st
        self._graphs = None
        # one eager pass: creates the communicators' buffers, the library's per-device state and the gather outputs
        self._issue(stage_a, stage_b, stage_c, stage_d, first=True)
        torch.cuda.synchronize(dev)

    def _gather(self, out, inp, group):
        return dist.all_gather_into_tensor(out.view((-1,) + tuple(out.shape[2:])), inp, group=group, async_op=True)

    def _gather_many(self, pairs, group):
        """Several all-gathers as one group call (one launch on the communicator's stream instead of one per tensor);
        falls back to one call per tensor where the backend has no grouped form.  -> list of handles with wait()."""
        manager = getattr(dist, "_coalescing_manager", None)
        if manager is not None and self.coalesce:
            try:
                with manager(group=group, async_ops=True) as cm:
                    for out, inp in pairs:
                        dist.all_gather_into_tensor(out.view((-1,) + tuple(out.shape[2:])), inp, group=group)
                return [cm]
            except (RuntimeError, ValueError, NotImplementedError):
                self.coalesce = False
        return [self._gather(out, inp, group) for out, inp in pairs]

    def _issue(self, a, b, c, d, first=False):
        """One step: the key/value gather (default group) runs under the whole linear branch, whose own small
        gather goes through ``linear_group``; the attention starts when the keys have arrived."""
        st = self._st
        a()
        if first:
            for dst, src in (('n_all', 'n_loc'), ('k_all', 'pk'), ('v_all', 'pv')):
                st[dst] = torch.empty((self.world,) + tuple(st[src].shape), dtype=st[src].dtype, device=self.dev)
        kv = self._gather_many([(st['n_all'], st['n_loc']), (st['k_all'], st['pk']), (st['v_all'], st['pv'])], self.group)
        b()
        if first:
            st['a_all'] = torch.empty((self.world,) + tuple(st['a_seg'].shape), dtype=torch.float32, device=self.dev)
            st['S_all'] = torch.empty((self.world,) + tuple(st['S_seg'].shape), dtype=torch.float32, device=self.dev)
        lin = self._gather_many([(st['a_all'], st['a_seg']), (st['S_all'], st['S_seg'])], self.lin_group)
        if self.gather_under_linear:
            for h in lin:
                h.wait()
            c()
            for h in kv:
                h.wait()
            d()
        else:
            for h in lin + kv:
                h.wait()
            cur = torch.cuda.current_stream(self.dev)
            self._side.wait_stream(cur)
            with torch.cuda.stream(self._side):
                c()
            d()
            cur.wait_stream(self._side)

    def capture(self):
        """Captures the compute stages into CUDA graphs (call once, after construction, on every rank)."""
        graphs = []
        for stage in self._stages:
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                stage()
            graphs.append(gr)
        torch.cuda.synchronize(self.dev)
        self._graphs = graphs

    def run(self):
        if self._graphs is None:
            self._issue(*self._stages)
        else:
            self._issue(*(g.replay for g in self._graphs))
        return self._st['out']
