"""Thin launch wrappers: allocate outputs with torch, pass raw pointers to the C ABI."""
from __future__ import annotations

import os

import torch

from . import _lib
from .nats_util import SelectionTables, cdiv, current_stream_ptr

BF16 = torch.bfloat16
USE_MAMBA_WALK = os.environ.get("NATSL_MAMBA_WALK", "1") != "0"    # natsl_mamba_walk_fused (K = 128, V = 64)
USE_FUSED_WALK = True        # K = V = 128, block 64: recurrence + output fused on tcgen05 (natsl_gdn_walk_fused)
# value dimension of the fused walk split over two CTAs (natsl_gdn_walk_fused_vsplit, T <= 8192): half an SM per CTA.
# Off by default: measured alone it is no faster than the one-CTA walk (0.204 vs 0.189 ms at B=8, T=4096, H=16), and
# the kernels of the two branches do not overlap in practice (the block scheduler drains one grid before the next).
WALK_VSPLIT = os.environ.get("NATSL_WALK_VSPLIT", "0") == "1"
# chunk preparation on tcgen05 for K = V = 128 (natsl_gdn_chunk_prep_tc); "0" keeps the mma.sync kernel for every shape
PREP_TC = os.environ.get("NATSL_PREP_TC", "1") != "0"


# softmax branch with persistent CTAs (two per SM working through the query tiles) instead of one CTA per query tile.
# Off by default: parity-green but measured slower (0.43 vs 0.29 ms at B=8, T=4096, H=16).
ATTN_PERSISTENT = os.environ.get("NATSL_ATTN_PERSISTENT", "0") == "1"


def _attn_flags(own_chunk: bool) -> int:
    return (_lib.FLAG_ATTN_OWN_CHUNK if own_chunk else 0) | (_lib.FLAG_ATTN_PERSISTENT if ATTN_PERSISTENT else 0)


def prep_entry(K: int, V: int) -> str:
    """Name of the chunk-preparation entry point for these head dims (both take the arguments of ``..._prep_ex``)."""
    return "natsl_gdn_chunk_prep_tc" if (PREP_TC and K == 128 and V == 128) else "natsl_gdn_chunk_prep_ex"


def _need(cond: bool, msg: str, exc=ValueError):
    if not cond:
        raise exc(msg)


def _check_qkv(q, k, v, tables, what: str, same_heads: bool):
    """Shapes that the kernels take on trust: the same batch, key and value sequences of one length, matching head
    counts and head dims, tables built for this batch, everything on one CUDA device."""
    _need(q.dim() == 4 and k.dim() == 4 and v.dim() == 4, f"{what}: q, k, v must be [B, T, H, D]")
    _need(q.is_cuda and k.device == q.device and v.device == q.device, f"{what}: q, k, v must be on one CUDA device")
    _need(k.shape[0] == q.shape[0] and v.shape[0] == q.shape[0], f"{what}: q, k, v differ in batch size")
    _need(k.shape[3] == q.shape[3], f"{what}: q and k differ in head dim ({q.shape[3]} vs {k.shape[3]})")
    _need(v.shape[1] == k.shape[1] and v.shape[2] == k.shape[2],
          f"{what}: k {tuple(k.shape)} and v {tuple(v.shape)} differ in length or heads")
    if same_heads:
        _need(k.shape[1] == q.shape[1] and k.shape[2] == q.shape[2], f"{what}: q {tuple(q.shape)} and k {tuple(k.shape)} differ")
    else:
        _need(q.shape[2] % k.shape[2] == 0, f"{what}: {q.shape[2]} query heads over {k.shape[2]} key/value heads")
    _need(tables.types_i.shape[0] == q.shape[0] and tables.types_i.device == q.device,
          f"{what}: the selection tables were built for another batch or device")


def attn_fwd(q, k, v, tables: SelectionTables, scale: float, own_chunk: bool, mma_sync: bool = False, q_off: int = 0):
    """q [B,Tq,HQ,DK], k [B,T,HKV,DK], v [B,T,HKV,DV] bf16 -> (o [B,Tq,HQ,DV] bf16, lse [B,Tq,HQ] fp32 base-2).
    The queries are the tokens [q_off, q_off+Tq) of the T-key sequence (q_off = 0 and Tq = T normally)."""
    _need(q.dtype == BF16 and k.dtype == BF16 and v.dtype == BF16, "softmax branch needs bf16 q/k/v", TypeError)
    _check_qkv(q, k, v, tables, "softmax branch", same_heads=False)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    B, Tq, HQ, DK = q.shape
    T, HKV, DV = k.shape[1], k.shape[2], v.shape[3]
    _need(tables.T == T, f"tables were built for T={tables.T}, keys have T={T}")
    _need(0 <= q_off and q_off + Tq <= T, f"queries [{q_off}, {q_off + Tq}) do not lie inside the {T} keys")
    HN = tables.types_i.shape[2]
    o = torch.empty(B, Tq, HQ, DV, dtype=BF16, device=q.device)
    lse = torch.empty(B, Tq, HQ, dtype=torch.float32, device=q.device)
    flags = _attn_flags(own_chunk) | (_lib.FLAG_ATTN_MMA_SYNC if mma_sync else 0)
    _lib.call("natsl_attn_fwd_ex", q.data_ptr(), k.data_ptr(), v.data_ptr(), tables.types_i.data_ptr(),
              tables.indices.data_ptr(), tables.attn_n_iters.data_ptr(), o.data_ptr(), lse.data_ptr(),
              B, T, Tq, int(q_off), HQ, HKV, HN, DK, DV, tables.nats_block_size, float(scale), flags,
              current_stream_ptr(q.device))
    return o, lse


def attn_fwd_split(q, k_rem, v_rem, k, v, tables: SelectionTables, scale: float, own_chunk: bool, rem_base=None,
                   rem_slots: int = 0):
    """Softmax branch over a key sequence held in two parts: keys [0, S) gathered from other segments (shared by the
    B / B_rem local segments that sit segment-major in the batch of q, k, v) and keys [S, S+L) in k, v [B, L, HKV, .];
    the queries q [B, L, HQ, DK] are the tokens [S, S+L).  Gathered part: k_rem, v_rem [B_rem, S, HKV, .], or with
    ``rem_base`` [B_rem, G, HKV] int32 the packed selected (block, head) pairs [B_rem, tokens, .] of G segments with
    ``rem_slots`` virtual blocks per head each (S = G * rem_slots * block size).  -> o [B, L, HQ, DV] bf16."""
    for t_ in (q, k_rem, v_rem, k, v):
        _need(t_.dtype == BF16 and t_.is_contiguous(), "softmax branch needs contiguous bf16 tensors", TypeError)
    B, L, HQ, DK = q.shape
    HKV, DV = k.shape[2], v.shape[3]
    B_rem = k_rem.shape[0]
    nbs = tables.nats_block_size
    if rem_base is None:
        S, rem_tokens = k_rem.shape[1], 0
    else:
        _need(rem_base.dtype == torch.int32 and rem_base.is_contiguous() and rem_base.shape[0] == B_rem
              and rem_base.shape[2] == HKV, "rem_base must be a contiguous int32 [B_rem, G, HKV] tensor")
        S, rem_tokens = rem_base.shape[1] * int(rem_slots) * nbs, k_rem.shape[1]
    _need(tables.T == S + L, f"tables were built for T={tables.T}, keys have T={S + L}")
    o = torch.empty(B, L, HQ, DV, dtype=BF16, device=q.device)
    lse = torch.empty(B, L, HQ, dtype=torch.float32, device=q.device)
    _lib.call("natsl_attn_fwd_split", q.data_ptr(), k_rem.data_ptr(), v_rem.data_ptr(), _lib.ptr(rem_base), int(rem_slots),
              int(rem_tokens), k.data_ptr(), v.data_ptr(), tables.types_i.data_ptr(), tables.indices.data_ptr(),
              tables.attn_n_iters.data_ptr(), o.data_ptr(), lse.data_ptr(), B, B_rem, S + L, L, S, S, HQ, HKV,
              tables.types_i.shape[2], DK, DV, nbs, float(scale), _attn_flags(own_chunk), current_stream_ptr(q.device))
    return o


def attn_dense_mask(tables: SelectionTables, HQ: int, own_chunk: bool) -> torch.Tensor:
    """Debug: the dense boolean mask [B,HQ,T,T] the attention kernel realises."""
    B, TN, HN, _ = tables.types_i.shape
    T = tables.T
    mask = torch.empty(B, HQ, T, T, dtype=torch.uint8, device=tables.types_i.device)
    flags = _lib.FLAG_ATTN_OWN_CHUNK if own_chunk else 0
    _lib.call("natsl_attn_dense_mask", tables.types_i.data_ptr(), tables.indices.data_ptr(),
              tables.attn_n_iters.data_ptr(), mask.data_ptr(), B, T, HQ, HN, tables.nats_block_size, flags,
              current_stream_ptr(mask.device))
    return mask.bool()


def linear_fwd(rule: int, q, k, v, g, beta, tables: SelectionTables, scale: float, h0, decay: bool,
               use_l2norm: bool, output_final_state: bool, trailing_quirk: bool = True,
               return_intermediates: bool = False, skip_out: bool = False, own_chunk: bool = True, tables_event=None):
    """Linear branch forward (prep -> state recurrence -> output).  Returns (o, ht, inter); with ``skip_out``
    only the recurrence runs (o is None).  ``own_chunk=False``: the output keeps only the state term (the mode
    in which the softmax branch alone covers the current chunk); ``tables`` must then be per 64-token chunk.
    ``tables_event``: CUDA event after which the tables (built on another stream) are valid; the chunk preparation
    does not read them and is launched before the wait."""
    _need(q.dtype == BF16 and k.dtype == BF16 and v.dtype == BF16, "linear branch needs bf16 q/k/v", TypeError)
    _check_qkv(q, k, v, tables, "linear branch", same_heads=True)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    B, T, H, K = q.shape
    V = v.shape[3]
    dev = q.device
    _need(tables.T == T, f"tables were built for T={tables.T}, the sequence has T={T}")
    _need(tuple(g.shape) == (B, T, H) and g.device == dev, f"g must be [B,T,H] = {(B, T, H)} on {dev}, got {tuple(g.shape)}")
    _need(beta is None or (tuple(beta.shape) == (B, T, H) and beta.device == dev),
          f"beta must be [B,T,H] = {(B, T, H)} on {dev}")
    _need(rule != _lib.RULE_GDN or beta is not None, "the gated delta rule needs beta")
    HN = tables.types_i.shape[2]
    _need(H % HN == 0, f"{H} heads over {HN} selection heads")
    NT = cdiv(T, 64)
    nbs = tables.nats_block_size
    if K not in (64, 128) or V not in (64, 128, 256):
        # head dims the chunk kernels have no tiles for (the 760M configuration: K = 192, V = 384): the token recurrence
        # with re-roll computes the same function for any K in {32, 64, 96, 128, 192, 256} and V a multiple of 8 --
        # correct, not fast, forward only
        if return_intermediates or skip_out or not own_chunk:
            raise NotImplementedError(f"head dims K={K}, V={V} run the token recurrence, which has no chunk intermediates "
                                      "(backward pass, state-only and mode 'attn' need K in {64,128}, V in {64,128,256})")
        if tables_event is not None:
            torch.cuda.current_stream(dev).wait_event(tables_event)
        o, ht, _ = linear_recurrent(rule, q, k, v, g, beta, tables, scale, h0, decay, use_l2norm)
        return o, (ht if output_final_state else None), None
    st = current_stream_ptr(dev)
    g = g.float().contiguous()
    gcs = torch.empty(B, T, H, dtype=torch.float32, device=dev)
    fused = (rule == _lib.RULE_GDN and K == 128 and V == 128 and nbs == 64 and NT <= 1024 and not return_intermediates
             and not skip_out and own_chunk and USE_FUSED_WALK)
    # Mamba2 with state dim 128 and head dim 64: recurrence + output (or the recurrence alone) in one tcgen05 walk
    mamba_fused = (rule == _lib.RULE_MAMBA and K == 128 and V == 64 and NT <= 1024 and not return_intermediates
                   and own_chunk and USE_MAMBA_WALK and (not skip_out or output_final_state))
    if rule == _lib.RULE_GDN:
        beta = beta.contiguous()
        _need(beta.dtype in (BF16, torch.float32), "beta must be bf16 or fp32", TypeError)
        w = torch.empty(B, T, H, K, dtype=BF16, device=dev)
        u = torch.empty(B, T, H, V, dtype=BF16, device=dev)
        krstd = torch.empty(B, T, H, dtype=torch.float32, device=dev)
        qrstd = torch.empty(B, T, H, dtype=torch.float32, device=dev) if fused else None
        pmat = torch.empty(B, T, H, 64, dtype=BF16, device=dev) if fused else None
        _lib.call(prep_entry(K, V), q.data_ptr() if fused else None, k.data_ptr(), v.data_ptr(), g.data_ptr(),
                  beta.data_ptr(), _lib.DT_BF16 if beta.dtype == BF16 else _lib.DT_F32, w.data_ptr(), u.data_ptr(),
                  gcs.data_ptr(), krstd.data_ptr(), _lib.ptr(qrstd), _lib.ptr(pmat), B, T, H, K, V, int(use_l2norm), st)
    else:
        w, u, krstd = None, v, None
        _lib.call("natsl_chunk_local_cumsum", g.data_ptr(), gcs.data_ptr(), B, T, H, st)
    if tables_event is not None:
        torch.cuda.current_stream(dev).wait_event(tables_event)
    ht = torch.empty(B, H, K, V, dtype=torch.float32, device=dev) if output_final_state else None
    if h0 is not None:
        h0 = h0.float().contiguous()
        _need(tuple(h0.shape) == (B, H, K, V), f"initial state must be [B,H,K,V], got {tuple(h0.shape)}")
    flags = (_lib.FLAG_DECAY_SKIPPED if decay else 0) | (0 if trailing_quirk else _lib.FLAG_NO_TRAILING_QUIRK)
    if fused:
        # recurrence + output in one tcgen05 walk; the per-chunk states are never materialised
        o = torch.empty(B, T, H, V, dtype=BF16, device=dev)
        entry = "natsl_gdn_walk_fused_vsplit" if (WALK_VSPLIT and NT <= 128) else "natsl_gdn_walk_fused"
        _lib.call(entry, q.data_ptr(), k.data_ptr(), w.data_ptr(), u.data_ptr(), pmat.data_ptr(),
                  gcs.data_ptr(), krstd.data_ptr(), qrstd.data_ptr(), tables.types_i.data_ptr(),
                  tables.indices.data_ptr(), tables.n_blocks.data_ptr(), _lib.ptr(h0), o.data_ptr(), _lib.ptr(ht),
                  B, T, H, HN, K, V, nbs, float(scale), flags, st)
        return o, ht, None
    if mamba_fused:
        o = None if skip_out else torch.empty(B, T, H, V, dtype=BF16, device=dev)
        _lib.call("natsl_mamba_walk_fused", None if skip_out else q.data_ptr(), k.data_ptr(), v.data_ptr(), gcs.data_ptr(),
                  tables.types_i.data_ptr(), tables.indices.data_ptr(), tables.n_blocks.data_ptr(), _lib.ptr(h0),
                  _lib.ptr(o), _lib.ptr(ht), B, T, H, HN, K, V, nbs, float(scale), flags, st)
        return o, ht, (dict(gcs=gcs) if skip_out else None)
    state_only = skip_out and ht is not None and not return_intermediates
    h = None if state_only else torch.empty(B, NT, H, K, V, dtype=BF16, device=dev)
    carry = None if state_only else torch.empty(B, NT, H, dtype=torch.float32, device=dev)
    _lib.call("natsl_linear_fwd_h", rule, k.data_ptr(), _lib.ptr(w), u.data_ptr(), gcs.data_ptr(), _lib.ptr(krstd),
              tables.types_i.data_ptr(), tables.indices.data_ptr(), tables.n_blocks.data_ptr(), _lib.ptr(h0),
              _lib.ptr(h), _lib.ptr(carry), _lib.ptr(ht), B, T, H, HN, K, V, nbs, flags, st)
    inter = dict(w=w, u=u, gcs=gcs, k_rstd=krstd, h=h, carry=carry) if return_intermediates else None
    if skip_out:
        return None, ht, (inter or dict(gcs=gcs))
    o = torch.empty(B, T, H, V, dtype=BF16, device=dev)
    _lib.call("natsl_linear_fwd_o", rule, q.data_ptr(), k.data_ptr(), _lib.ptr(w), u.data_ptr(), gcs.data_ptr(),
              _lib.ptr(krstd), h.data_ptr(), carry.data_ptr(), o.data_ptr(), B, T, H, K, V, float(scale),
              int(use_l2norm and rule == _lib.RULE_GDN) | (0 if own_chunk else 2), st)
    return o, ht, inter


def _dt_code(t):
    if t.dtype == torch.float32:
        return _lib.DT_F32
    if t.dtype == BF16:
        return _lib.DT_BF16
    raise TypeError(f"unsupported dtype {t.dtype} (fp32 or bf16)")


def linear_recurrent(rule: int, q, k, v, g, beta, tables: SelectionTables, scale: float, h0, decay: bool,
                     use_l2norm: bool):
    """Reference-precision linear branch: token recurrence with re-roll (fp32 math; fp32 or bf16 tensors).
    Returns (o, ht, hstart): output, state after the last selected block, block-start state at the end."""
    _need(q.dtype == k.dtype == v.dtype, "q, k, v must share a dtype", TypeError)
    code = _dt_code(q)
    _check_qkv(q, k, v, tables, "linear branch (recurrent form)", same_heads=True)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    B, T, H, K = q.shape
    V = v.shape[3]
    dev = q.device
    _need(tables.T == T, f"tables were built for T={tables.T}, the sequence has T={T}")
    _need(tuple(g.shape) == (B, T, H), f"g must be [B,T,H] = {(B, T, H)}, got {tuple(g.shape)}")
    _need(beta is None or tuple(beta.shape) == (B, T, H), f"beta must be [B,T,H] = {(B, T, H)}")
    g = g.float().contiguous()
    if beta is not None:
        beta = beta.to(q.dtype).contiguous()
    if h0 is not None:
        h0 = h0.float().contiguous()
    o = torch.empty(B, T, H, V, dtype=q.dtype, device=dev)
    ht = torch.empty(B, H, K, V, dtype=torch.float32, device=dev)
    hstart = torch.empty_like(ht)
    _lib.call("natsl_linear_recurrent_fwd", rule, code, q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(),
              _lib.ptr(beta), tables.types_i.data_ptr(), _lib.ptr(h0), o.data_ptr(), ht.data_ptr(), hstart.data_ptr(),
              B, T, H, tables.types_i.shape[2], K, V, tables.nats_block_size, float(scale),
              _lib.FLAG_DECAY_SKIPPED if decay else 0, int(use_l2norm), current_stream_ptr(dev))
    return o, ht, hstart


def linear_recurrent_step(rule: int, q, k, v, g, beta, block_types, state, state_block_start, g_block, t_off: int, nbs: int,
                          scale: float, decay: bool, use_l2norm: bool):
    """Decoding step of the linear branch: the T new tokens continue a block that already holds ``t_off`` tokens.
    ``block_types`` [B, cdiv(t_off + T, nbs), HN, 2] (0/1 floats or ints) are read only where a block ends inside the
    call.  -> (o [B,T,H,V], new current state, new block-start state), states fp32 [B,H,K,V]."""
    code = _dt_code(q)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    B, T, H, K = q.shape
    V = v.shape[3]
    dev = q.device
    g = g.float().contiguous()
    if beta is not None:
        beta = beta.to(q.dtype).contiguous()
    types_i = torch.round(block_types.float()).to(torch.int32).contiguous()
    _need(types_i.shape[1] == cdiv(t_off + T, nbs) and types_i.shape[3] == 2, "block_types must cover the blocks the step touches")
    state = state.float().contiguous()
    start = state_block_start.float().contiguous()
    g_block = g_block.float().contiguous()
    _need(tuple(state.shape) == (B, H, K, V) and tuple(start.shape) == (B, H, K, V) and tuple(g_block.shape) == (B, H),
          "states must be [B,H,K,V] and the block decay [B,H]")
    o = torch.empty(B, T, H, V, dtype=q.dtype, device=dev)
    new_state, new_start = torch.empty_like(state), torch.empty_like(start)
    _lib.call("natsl_linear_recurrent_step", rule, code, q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), _lib.ptr(beta),
              types_i.data_ptr(), state.data_ptr(), start.data_ptr(), g_block.data_ptr(), int(t_off), o.data_ptr(),
              new_state.data_ptr(), new_start.data_ptr(), B, T, H, types_i.shape[2], K, V, int(nbs), float(scale),
              _lib.FLAG_DECAY_SKIPPED if decay else 0, int(use_l2norm), current_stream_ptr(dev))
    return o, new_state, new_start


def attn_fwd_fp32(q, k, v, tables: SelectionTables, scale: float, own_chunk: bool):
    """Reference-precision softmax branch (fp32 math; fp32 or bf16 tensors).  Returns (o, lse base-2)."""
    _need(q.dtype == k.dtype == v.dtype, "q, k, v must share a dtype", TypeError)
    code = _dt_code(q)
    _check_qkv(q, k, v, tables, "softmax branch (fp32 form)", same_heads=False)
    _need(k.shape[1] == q.shape[1] and tables.T == q.shape[1], "q, k and the tables must cover the same sequence")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    B, T, HQ, DK = q.shape
    HKV, DV = k.shape[2], v.shape[3]
    o = torch.empty(B, T, HQ, DV, dtype=q.dtype, device=q.device)
    lse = torch.empty(B, T, HQ, dtype=torch.float32, device=q.device)
    _lib.call("natsl_attn_fwd_fp32", code, q.data_ptr(), k.data_ptr(), v.data_ptr(), tables.types_i.data_ptr(),
              o.data_ptr(), lse.data_ptr(), B, T, HQ, HKV, tables.types_i.shape[2], DK, DV, tables.nats_block_size,
              float(scale), _lib.FLAG_ATTN_OWN_CHUNK if own_chunk else 0, current_stream_ptr(q.device))
    return o, lse


# ------------------------------------------------------------------------------------------------ backward
class StageTimer:
    """Optional per-stage device timing of the backward pass: CUDA events on the launching stream around every C-ABI
    call; ``result()`` synchronises and returns {stage: milliseconds} (summed over repeated calls)."""

    def __init__(self):
        self.events = []

    def call(self, stage: str, name: str, *args):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        _lib.call(name, *args)
        e1.record()
        self.events.append((stage, e0, e1))

    def result(self) -> dict:
        torch.cuda.synchronize()
        out = {}
        for stage, e0, e1 in self.events:
            out[stage] = out.get(stage, 0.0) + e0.elapsed_time(e1)
        return out


def _call(timer, stage, name, *args):
    if timer is None:
        _lib.call(name, *args)
    else:
        timer.call(stage, name, *args)


def attn_bwd(q, k, v, o, lse, do, tables: SelectionTables, scale: float, own_chunk: bool, reference_compat: bool = False,
             timer: StageTimer | None = None):
    """Backward of the softmax branch.  -> (dq, dk, dv bf16, dnats_attn [B,TN,HN] fp32): ``dnats_attn`` is the sum of the
    score gradients of the keys of a softmax-selected block over the queries of later blocks, summed over the heads
    of a selection group and zero for the other blocks (src/nats/ops/attns/attns.py:922, 975-978, 1625-1629, 1749-1755).
    ``reference_compat``: leave out every own-block term like the reference's default backward."""
    for t_ in (q, k, v, o, do):
        _need(t_.dtype == BF16, "softmax-branch backward needs bf16 tensors", TypeError)
    _check_qkv(q, k, v, tables, "softmax branch (backward)", same_heads=False)
    q, k, v, o, do, lse = (t_.contiguous() for t_ in (q, k, v, o, do, lse))
    B, T, HQ, DK = q.shape
    HKV, DV = k.shape[2], v.shape[3]
    _need(k.shape[1] == T and tables.T == T, "q, k and the tables must cover the same sequence")
    _need(tuple(do.shape) == (B, T, HQ, DV) and tuple(o.shape) == (B, T, HQ, DV), "o and do must be [B,T,HQ,DV]")
    TN, HN = tables.types_i.shape[1], tables.types_i.shape[2]
    nbs = tables.nats_block_size
    NT = cdiv(T, 64)
    dev = q.device
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    delta = torch.empty(B, T, HQ, dtype=torch.float32, device=dev)
    part = torch.empty(B, NT, HQ, dtype=torch.float32, device=dev)
    flags = (_lib.FLAG_ATTN_OWN_CHUNK if own_chunk else 0) | (_lib.FLAG_BWD_REFERENCE_COMPAT if reference_compat else 0)
    _call(timer, "attn_bwd", "natsl_attn_bwd", q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(),
              tables.types_i.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), delta.data_ptr(), part.data_ptr(),
              B, T, HQ, HKV, HN, DK, DV, nbs, float(scale), flags, current_stream_ptr(dev))
    cpb = nbs // 64
    if NT != TN * cpb:                                        # ragged last block: pad the tile axis
        part = torch.nn.functional.pad(part, (0, 0, 0, TN * cpb - NT))
    per_block = part.view(B, TN, cpb, HN, HQ // HN).sum((2, 4))
    dnats = per_block * (tables.types_i[..., 0] != 0)
    return dq, dk, dv, dnats


def linear_bwd(rule: int, q, k, v, g, beta, tables: SelectionTables, scale: float, h0, decay: bool, use_l2norm: bool,
               do, dht=None, invalid_dnats: bool = True, trailing_quirk: bool = True, return_intermediates: bool = False,
               timer: StageTimer | None = None):
    """Backward of the linear branch (block size 64).  Recomputes the forward's preparation and recurrence, then runs the
    five backward stages.  -> dict(dq, dk, dv bf16; dg fp32; dbeta fp32 or None; dh0 fp32 or None; dnats [B,NT,HN] fp32
    = the reference's dnats column for the linear branch, src/nats/ops/common/chunk_o.py:440-443, 459-492, 1568-1575)."""
    gdn = rule == _lib.RULE_GDN
    for t_ in (q, k, v, do):
        _need(t_.dtype == BF16, "linear-branch backward needs bf16 tensors", TypeError)
    _check_qkv(q, k, v, tables, "linear branch (backward)", same_heads=True)
    _need(tables.nats_block_size == 64, "the backward pass is built for nats_block_size = 64", NotImplementedError)
    q, k, v, do = q.contiguous(), k.contiguous(), v.contiguous(), do.contiguous()
    B, T, H, K = q.shape
    V = v.shape[3]
    _need(K in (64, 128) and V in (64, 128), f"backward head dims K={K} V={V}: 64 or 128 each", NotImplementedError)
    _need(tables.T == T, f"tables were built for T={tables.T}, the sequence has T={T}")
    dev = q.device
    HN = tables.types_i.shape[2]
    NT = cdiv(T, 64)
    st = current_stream_ptr(dev)
    g = g.float().contiguous()
    bf = dict(dtype=BF16, device=dev)
    f32 = dict(dtype=torch.float32, device=dev)
    gcs = torch.empty(B, T, H, **f32)
    # ---- forward recompute: w, u, gcs; the state and the carried decay every chunk reads
    if gdn:
        beta = beta.contiguous()
        _need(beta.dtype in (BF16, torch.float32), "beta must be bf16 or fp32", TypeError)
        w, u = torch.empty(B, T, H, K, **bf), torch.empty(B, T, H, V, **bf)
        krs0 = torch.empty(B, T, H, **f32)
        _call(timer, "recompute_prep", prep_entry(K, V), None, k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(),
                  _lib.DT_BF16 if beta.dtype == BF16 else _lib.DT_F32, w.data_ptr(), u.data_ptr(), gcs.data_ptr(),
                  krs0.data_ptr(), None, None, B, T, H, K, V, int(use_l2norm), st)
    else:
        w, u, krs0 = None, v, None
        _call(timer, "recompute_prep", "natsl_chunk_local_cumsum", g.data_ptr(), gcs.data_ptr(), B, T, H, st)
    if h0 is not None:
        h0 = h0.float().contiguous()
    flags = (_lib.FLAG_DECAY_SKIPPED if decay else 0) | (0 if trailing_quirk else _lib.FLAG_NO_TRAILING_QUIRK)
    h = torch.empty(B, NT, H, K, V, **bf)
    carry = torch.empty(B, NT, H, **f32)
    _call(timer, "recompute_scan", "natsl_linear_fwd_h", rule, k.data_ptr(), _lib.ptr(w), u.data_ptr(), gcs.data_ptr(), _lib.ptr(krs0),
              tables.types_i.data_ptr(), tables.indices.data_ptr(), tables.n_blocks.data_ptr(), _lib.ptr(h0),
              h.data_ptr(), carry.data_ptr(), None, B, T, H, HN, K, V, 64, flags, st)
    # ---- 1: normalised q, k and the chunk-local part of dv'
    l2 = bool(use_l2norm and gdn)
    if l2:
        qn, kn = torch.empty_like(q), torch.empty_like(k)
        qrs, krs = torch.empty(B, T, H, **f32), torch.empty(B, T, H, **f32)
    else:
        qn, kn, qrs, krs = q, k, None, None
    dvl = torch.empty(B, T, H, V, **bf)
    _call(timer, "bwd_pre", "natsl_linear_bwd_pre", q.data_ptr(), k.data_ptr(), do.data_ptr(), gcs.data_ptr(), _lib.ptr(qn if l2 else None),
              _lib.ptr(kn if l2 else None), _lib.ptr(qrs), _lib.ptr(krs), dvl.data_ptr(), B, T, H, K, V, float(scale), int(l2), st)
    # ---- 2: reverse walk
    dS_all = torch.empty(B, NT, H, K, V, **bf)
    dvp = torch.empty(B, T, H, V, **bf)
    dh0 = torch.empty(B, H, K, V, **f32) if h0 is not None else None
    if dht is not None:
        dht = dht.float().contiguous()
    _call(timer, "bwd_dh", "natsl_linear_bwd_dh", rule, qn.data_ptr(), kn.data_ptr(), _lib.ptr(w), do.data_ptr(), dvl.data_ptr(),
              gcs.data_ptr(), carry.data_ptr(), tables.types_i.data_ptr(), tables.indices.data_ptr(),
              tables.n_blocks.data_ptr(), _lib.ptr(dht), dS_all.data_ptr(), dvp.data_ptr(), _lib.ptr(dh0), B, T, H, HN, K, V,
              float(scale), st)
    # ---- 3: everything that contracts with the state or its gradient
    vp = torch.empty(B, T, H, V, **bf) if gdn else v
    dw = torch.empty(B, T, H, K, **bf) if gdn else None
    dq1, dk1 = torch.empty(B, T, H, K, **bf), torch.empty(B, T, H, K, **bf)
    dkd = torch.empty(B, T, H, **f32)
    scal = torch.empty(B, NT, H, 4, **f32)
    dn_lin = torch.empty(B, NT, H, **f32)
    _call(timer, "bwd_state", "natsl_linear_bwd_state", rule, kn.data_ptr(), _lib.ptr(v if gdn else None), _lib.ptr(w), u.data_ptr(),
              do.data_ptr(), dvp.data_ptr(), gcs.data_ptr(), h.data_ptr(), carry.data_ptr(), dS_all.data_ptr(),
              tables.types_i.data_ptr(), tables.indices.data_ptr(), tables.n_blocks.data_ptr(),
              tables.starting_h_idx.data_ptr(), _lib.ptr(vp if gdn else None), _lib.ptr(dw), dq1.data_ptr(), dk1.data_ptr(),
              dkd.data_ptr(), scal.data_ptr(), dn_lin.data_ptr(), B, T, H, HN, K, V, float(scale), int(invalid_dnats), st)
    # ---- 4: the 64 x 64 part, the WY transform and the l2 norm
    dq, dk = torch.empty_like(q), torch.empty_like(k)
    dv = torch.empty_like(v) if gdn else dvp
    dbeta = torch.empty(B, T, H, **f32) if gdn else None
    dg_tok = torch.empty(B, T, H, **f32)
    _call(timer, "bwd_intra", "natsl_linear_bwd_intra", rule, qn.data_ptr(), kn.data_ptr(), _lib.ptr(v if gdn else None), _lib.ptr(w),
              _lib.ptr(u if gdn else None), vp.data_ptr(), _lib.ptr(dvp if gdn else None), _lib.ptr(dw), do.data_ptr(),
              dq1.data_ptr(), dk1.data_ptr(), gcs.data_ptr(), _lib.ptr(beta if gdn else None),
              _lib.DT_BF16 if (gdn and beta.dtype == BF16) else _lib.DT_F32, _lib.ptr(qrs), _lib.ptr(krs), dkd.data_ptr(),
              tables.types_i.data_ptr(), dq.data_ptr(), dk.data_ptr(), _lib.ptr(dv if gdn else None), _lib.ptr(dbeta),
              dg_tok.data_ptr(), scal.data_ptr(), B, T, H, HN, K, V, float(scale), int(l2), st)
    # ---- 5: decay gradients
    dg = torch.empty(B, T, H, **f32)
    _call(timer, "bwd_dg", "natsl_linear_bwd_dg", dg_tok.data_ptr(), scal.data_ptr(), tables.types_i.data_ptr(), tables.indices.data_ptr(),
              tables.n_blocks.data_ptr(), dg.data_ptr(), B, T, H, HN, flags, st)
    dnats = dn_lin.view(B, NT, HN, H // HN).sum(-1)
    out = dict(dq=dq, dk=dk, dv=dv, dg=dg, dbeta=dbeta, dh0=dh0, dnats=dnats)
    if return_intermediates:
        out.update(dS=dS_all, dvp=dvp, dw=dw, vp=vp, h=h, carry=carry, gcs=gcs, w=w, u=u)
    return out
