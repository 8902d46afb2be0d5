"""``nats_mixed_attn_gdn``: softmax branch + gated-delta-rule branch of the NAtSL-GDN layer.

Same function names, argument order, defaults and return values as the reference's
``src/nats/ops/mixed_ops/mixed_attn_gdn.py:286-325`` (training / prefill op) and ``:328-440``
(chunk-inference op); the work is done by the C-ABI CUDA kernels.
"""
from __future__ import annotations

import contextlib
import os

import torch

from . import _lib, _ops
from .nats_util import CHUNK_SIZE, OFFSET_ATTN, OFFSET_LINEAR, build_selection_tables  # noqa: F401

# which branches also compute the query's own (possibly incomplete) block — mixed_attn_gdn.py:29-42
all_incomplete_ops = {
    'all': dict(attn=True, gated_delta_net=True),
    'attn': dict(attn=True, gated_delta_net=False),
    'gated_delta_net': dict(attn=False, gated_delta_net=True),
}


_attn_streams: dict = {}


def _get_attn_stream(device: torch.device) -> torch.cuda.Stream:
    """One side stream per device for the softmax branch (mixed_attn_gdn.py:19-26 of the reference)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _attn_streams:
        _attn_streams[idx] = torch.cuda.Stream(device=idx)
    return _attn_streams[idx]


_lin_streams: dict = {}
# The linear branch (chunk preparation -> walk) runs on a high-priority stream, so that its CTAs are placed ahead of the
# softmax branch's remaining ones whenever an SM frees up: the serial walk then starts earlier and the attention CTAs
# fill in around it.  Measured with the step replayed from a CUDA graph: 0.621 - 0.633 ms against 0.640 - 0.644 ms
# (three runs each); NATSL_LINEAR_PRIORITY=0 puts the branch back on the caller's stream.
LINEAR_BRANCH_PRIORITY = os.environ.get("NATSL_LINEAR_PRIORITY", "1") != "0"


def _get_linear_stream(device: torch.device) -> torch.cuda.Stream:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _lin_streams:
        _lin_streams[idx] = torch.cuda.Stream(device=idx, priority=-1)
    return _lin_streams[idx]


def _check_common(ops_for_incomplete_chunks, nats_block_size, attn_sw_size, cu_seqlens, use_g_for_attn, table):
    if ops_for_incomplete_chunks not in table:
        raise KeyError(ops_for_incomplete_chunks)
    assert nats_block_size >= CHUNK_SIZE                                  # mixed_attn_gdn.py:90
    if nats_block_size % CHUNK_SIZE:
        raise NotImplementedError("nats_block_size must be a multiple of 64")
    if attn_sw_size is not None:
        raise NotImplementedError("sliding-window softmax (attn_sw_size) is not built")
    if cu_seqlens is not None:
        raise NotImplementedError("variable-length batches (cu_seqlens) are not built")
    if use_g_for_attn:
        raise NotImplementedError("use_g_for_attn is not built (the layers always pass False)")


def per_chunk_tables(nats_block_types, T, nats_block_size):
    """Selection tables of the linear branch when the softmax branch alone covers the current chunk
    (ops_for_incomplete_chunks='attn'): the recurrence then walks 64-token chunks (every chunk of a selected block
    updates the state, chunks of other blocks only decay it; src/nats/ops/common/chunk_delta_h.py:189-324), which
    is the plain walk on the block types repeated per chunk."""
    cpb = nats_block_size // CHUNK_SIZE
    NT = -(-T // CHUNK_SIZE)
    per_chunk = torch.round(nats_block_types).repeat_interleave(cpb, dim=1)[:, :NT].contiguous()
    return build_selection_tables(per_chunk, T, CHUNK_SIZE)


# The reference's softmax-branch backward leaves out every own-block term of dq, dk, dv with the default settings
# (the flag it passes in backward is tied to sliding windows: mixed_attn_gdn.py:237 against :115 in the forward), so
# it is not the gradient of its own forward.  The default here is the true gradient; set this switch (or the
# environment variable NATSL_REFERENCE_COMPAT_BWD=1) to reproduce the reference's numbers instead.
REFERENCE_COMPAT_BWD = os.environ.get("NATSL_REFERENCE_COMPAT_BWD", "0") == "1"


@contextlib.contextmanager
def reference_compat_bwd(enabled: bool = True):
    """Within this context the ops record ``enabled`` as their softmax-branch backward mode."""
    global REFERENCE_COMPAT_BWD
    old, REFERENCE_COMPAT_BWD = REFERENCE_COMPAT_BWD, bool(enabled)
    try:
        yield
    finally:
        REFERENCE_COMPAT_BWD = old


def _zeros_like_or_none(t):
    return None if t is None else torch.zeros_like(t)


def hybrid_backward(ctx, rule, do_lin, do_attn, dht):
    """Shared backward of the two hybrid ops: softmax-branch dq/dk/dv, linear-branch dq/dk/dv/dg/dbeta/dh0 and the
    ``dnats`` pair (mixed_attn_gdn.py:196-283; mixed_attn_mamba.py:194-292)."""
    if not ctx.bwd_ok:
        raise NotImplementedError(ctx.bwd_why)
    q_attn, k_attn, v_attn, o_attn, lse, q, k, v, g, beta, h0 = ctx.saved_tensors
    tables = ctx.tables
    if do_attn is None:
        do_attn = torch.zeros_like(o_attn)
    if do_lin is None:
        do_lin = torch.zeros(q.shape[:3] + (v.shape[3],), dtype=q.dtype, device=q.device)
    dqa, dka, dva, dn_attn = _ops.attn_bwd(q_attn, k_attn, v_attn, o_attn, lse, do_attn.to(o_attn.dtype), tables,
                                           ctx.scale_attn, ctx.own_attn, reference_compat=ctx.compat)
    r = _ops.linear_bwd(rule, q, k, v, g, beta, tables, ctx.scale_lattn, h0, ctx.decay, ctx.use_l2norm,
                        do_lin.to(q.dtype), dht=dht, invalid_dnats=ctx.invalid_dnats_linear)
    dnats = torch.stack([dn_attn, r['dnats']], -1).to(ctx.types_dtype)
    dg = r['dg'].to(g.dtype)
    dbeta = None if r['dbeta'] is None else r['dbeta'].to(beta.dtype)
    dh0 = None if (h0 is None or r['dh0'] is None) else r['dh0'].to(h0.dtype)
    return dqa, dka, dva, r['dq'], r['dk'], r['dv'], dh0, dg, dbeta, dnats


class NAtSMixedAttentionGDN(torch.autograd.Function):
    """Forward and backward of mixed_attn_gdn.py:47-283."""

    @staticmethod
    def forward(ctx, q_attn, k_attn, v_attn, q_lattn, k_lattn, v_lattn, initial_state_gated_delta, g, beta,
                nats_block_types, n_nats_blocks, scale_attn, scale_lattn, cu_seqlens, cu_seqlens_nats,
                nats_block_size, attn_sw_size=None, ops_for_incomplete_chunks='gated_delta_net',
                output_final_state_gated_delta=False, compute_dnats_for_invalid_blocks_attn=False,
                compute_dnats_for_invalid_blocks_linear_att=True, decay_for_non_gdn_blocks=False,
                incomplete_block_start_with_ht=True, use_g_for_attn=True, lattn_use_qk_l2norm_in_kernel=True):
        _check_common(ops_for_incomplete_chunks, nats_block_size, attn_sw_size, cu_seqlens, use_g_for_attn,
                      all_incomplete_ops)
        strategy = all_incomplete_ops[ops_for_incomplete_chunks]
        own_linear = strategy['gated_delta_net']
        if own_linear and not incomplete_block_start_with_ht:
            raise NotImplementedError("incomplete_block_start_with_ht=False is not built")
        T = q_lattn.shape[1]
        ctx.bwd_ok, ctx.bwd_why = True, ""
        if q_lattn.dtype == torch.float32:
            if not own_linear:
                raise NotImplementedError("ops_for_incomplete_chunks='attn' is built for bf16 tensors only")
            # fp32 tensors take the reference-precision kernels (token recurrence with re-roll, fp32 softmax)
            tables = build_selection_tables(nats_block_types, T, nats_block_size)
            o_attn, lse = _ops.attn_fwd_fp32(q_attn, k_attn, v_attn, tables, scale_attn, own_chunk=strategy['attn'])
            o_gdn, ht, _ = _ops.linear_recurrent(_lib.RULE_GDN, q_lattn, k_lattn, v_lattn, g, beta, tables, scale_lattn,
                                                 initial_state_gated_delta, decay_for_non_gdn_blocks,
                                                 lattn_use_qk_l2norm_in_kernel)
            ctx.bwd_ok, ctx.bwd_why = False, "the backward pass is built for bf16 tensors (fp32 tensors run forward only)"
            return o_gdn, o_attn, (ht if output_final_state_gated_delta else None)
        # The two branches are independent: the softmax branch runs on a side stream (as the reference does for
        # its Mamba2 / DeltaNet ops, src/nats/ops/mixed_ops/mixed_attn_mamba.py:114-124) and joins before returning.
        # The selection tables are built on the side stream too: the chunk preparation of the linear branch does not
        # read them, so it starts at once and only the recurrence waits for the tables.
        cur = torch.cuda.current_stream(q_attn.device)
        side = _get_attn_stream(q_attn.device)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            tables = build_selection_tables(nats_block_types, T, nats_block_size)
            lin_tables = tables if own_linear else per_chunk_tables(nats_block_types, T, nats_block_size)
            tables_ready = torch.cuda.Event()
            tables_ready.record(side)
            o_attn, lse = _ops.attn_fwd(q_attn, k_attn, v_attn, tables, scale_attn, own_chunk=strategy['attn'])
        lin = _get_linear_stream(q_attn.device) if LINEAR_BRANCH_PRIORITY else cur
        if lin is not cur:
            lin.wait_stream(cur)
        with torch.cuda.stream(lin):
            o_gdn, ht, _ = _ops.linear_fwd(_lib.RULE_GDN, q_lattn, k_lattn, v_lattn, g, beta, lin_tables, scale_lattn,
                                           initial_state_gated_delta, decay_for_non_gdn_blocks,
                                           lattn_use_qk_l2norm_in_kernel, output_final_state_gated_delta,
                                           own_chunk=own_linear, tables_event=tables_ready)
        cur.wait_stream(side)
        if lin is not cur:
            cur.wait_stream(lin)
            for t_ in (o_gdn, ht):
                if t_ is not None:
                    t_.record_stream(cur)
            for t_ in (q_lattn, k_lattn, v_lattn, g, beta, initial_state_gated_delta):
                if t_ is not None:
                    t_.record_stream(lin)
        for t_ in (tables.types_i, tables.indices, tables.n_blocks, tables.starting_h_idx, lin_tables.types_i,
                   lin_tables.indices, lin_tables.n_blocks, o_attn, lse):
            t_.record_stream(cur)                      # allocated on the side stream, read on the current one
            if lin is not cur:
                t_.record_stream(lin)
        for t_ in (q_attn, k_attn, v_attn, nats_block_types):
            t_.record_stream(side)                     # allocated elsewhere, read on the side stream
        if not own_linear:
            ctx.bwd_ok, ctx.bwd_why = False, "the backward pass is not built for ops_for_incomplete_chunks='attn'"
        elif nats_block_size != CHUNK_SIZE:
            ctx.bwd_ok, ctx.bwd_why = False, "the backward pass is built for nats_block_size = 64"
        elif q_lattn.shape[-1] not in (64, 128) or v_lattn.shape[-1] not in (64, 128):
            ctx.bwd_ok, ctx.bwd_why = False, "the backward pass is built for linear-branch head dims 64 and 128"
        ctx.save_for_backward(q_attn, k_attn, v_attn, o_attn, lse, q_lattn, k_lattn, v_lattn, g, beta,
                              initial_state_gated_delta)
        ctx.tables = tables
        ctx.scale_attn, ctx.scale_lattn, ctx.own_attn = float(scale_attn), float(scale_lattn), strategy['attn']
        ctx.decay, ctx.use_l2norm = bool(decay_for_non_gdn_blocks), bool(lattn_use_qk_l2norm_in_kernel)
        ctx.invalid_dnats_linear = bool(compute_dnats_for_invalid_blocks_linear_att)
        ctx.compat = REFERENCE_COMPAT_BWD
        ctx.types_dtype = nats_block_types.dtype
        return o_gdn, o_attn, ht

    @staticmethod
    def backward(ctx, do_gdn, do_attn, dht):
        grads = hybrid_backward(ctx, _lib.RULE_GDN, do_gdn, do_attn, dht)
        dqa, dka, dva, dq, dk, dv, dh0, dg, dbeta, dnats = grads
        return (dqa, dka, dva, dq, dk, dv, dh0, dg, dbeta, dnats) + (None,) * 15


def nats_mixed_attn_gdn(
        q_attn: torch.Tensor, k_attn: torch.Tensor, v_attn: torch.Tensor,
        q_lattn: torch.Tensor, k_lattn: torch.Tensor, v_lattn: torch.Tensor,
        initial_state_gated_delta: torch.Tensor,
        g: torch.Tensor,
        beta: torch.Tensor,
        nats_block_types: torch.Tensor,
        n_nats_blocks: torch.Tensor,
        scale_attn=None, scale_lattn=None,
        cu_seqlens=None, cu_seqlens_nats=None,
        nats_block_size: int = 64,
        attn_sw_size: int | None = None,
        ops_for_incomplete_chunks: str = 'gated_delta_net',
        output_final_state_gated_delta: bool = False,
        compute_dnats_for_invalid_blocks_attn: bool = False,
        compute_dnats_for_invalid_blocks_linear_att: bool = True,
        decay_for_non_gdn_blocks: bool = False,
        incomplete_block_start_with_ht: bool = True,
        use_g_for_attn: bool = False,
        lattn_use_qk_l2norm_in_kernel: bool = True,
):
    """-> (o_gated_delta [B,T,H,V], o_attn [B,T,HQ,V_attn], final_state [B,H,K,V] fp32 or None).

    Differentiable (bf16 tensors, block size 64, modes 'all' and 'gated_delta_net'): gradients flow to q/k/v of both
    branches, g, beta, the initial state and, as the reference's ``dnats``, to ``nats_block_types``.  Configurations
    without a backward raise ``NotImplementedError`` when ``backward`` is reached.
    ``n_nats_blocks`` is accepted for signature parity; the counts are recomputed on the device
    from ``nats_block_types``."""
    if scale_attn is None:
        scale_attn = k_attn.shape[-1] ** -0.5
    if scale_lattn is None:
        scale_lattn = k_lattn.shape[-1] ** -0.5
    return NAtSMixedAttentionGDN.apply(
        q_attn, k_attn, v_attn, q_lattn, k_lattn, v_lattn, initial_state_gated_delta, g, beta,
        nats_block_types, n_nats_blocks, scale_attn, scale_lattn, cu_seqlens, cu_seqlens_nats,
        nats_block_size, attn_sw_size, ops_for_incomplete_chunks, output_final_state_gated_delta,
        compute_dnats_for_invalid_blocks_attn, compute_dnats_for_invalid_blocks_linear_att,
        decay_for_non_gdn_blocks, incomplete_block_start_with_ht, use_g_for_attn,
        lattn_use_qk_l2norm_in_kernel)


def _chunk_start_state(inter, ht, gcs, tables, op_type_last_chunk, T, nbs, decay):
    """State at the start of the block that follows / contains the last token, as the reference
    extracts it for decoding (src/nats/ops/gated_delta_rule/chunk_fwd.py:178-206)."""
    cpb = nbs // CHUNK_SIZE
    TN = tables.types_i.shape[1]
    c0 = (TN - 1) * cpb                                   # first compute chunk of the last block
    h_last = inter['h'][:, c0].float()                    # [B,H,K,V]
    carry_last = inter['carry'][:, c0]                    # [B,H]
    start = h_last * carry_last.exp()[..., None, None]
    if T % nbs == 0:
        assert op_type_last_chunk is not None
        H = h_last.shape[1]
        HN = op_type_last_chunk.shape[1]
        was_linear = (op_type_last_chunk[..., OFFSET_LINEAR] > 0).repeat_interleave(H // HN, dim=1)
        if decay:
            blk_g = gcs[:, c0 * CHUNK_SIZE:].view(gcs.shape[0], cpb, CHUNK_SIZE, H)[:, :, -1].sum(1)
            start = start * blk_g.exp()[..., None, None]
        start = torch.where(was_linear[..., None, None], ht, start)
    return start


def nats_mixed_attn_gdn_chunk_inference(
        q_attn: torch.Tensor, k_attn: torch.Tensor, v_attn: torch.Tensor,
        q_lattn: torch.Tensor, k_lattn: torch.Tensor, v_lattn: torch.Tensor,
        initial_state_gated_delta_chunk_start: torch.Tensor,
        g: torch.Tensor,
        beta: torch.Tensor,
        nats_block_types: torch.Tensor,
        op_type_last_chunk: torch.Tensor | None,
        n_nats_blocks: torch.Tensor,
        n_tokens_in_current_block: int = 0,
        scale_attn=None, scale_lattn=None,
        cu_seqlens=None, cu_seqlens_nats=None,
        nats_block_size: int = 64,
        attn_sw_size: int | None = None,
        ops_for_incomplete_chunks: str = 'gated_delta_net',
        output_final_state_gated_delta: bool = False,
        decay_for_non_gdn_blocks: bool = False,
        incomplete_block_start_with_ht: bool = True,
        use_g_for_attn: bool = False,
        lattn_use_qk_l2norm_in_kernel: bool = True,
):
    """Prefill under eval (mixed_attn_gdn.py:328-440): same kernels as ``nats_mixed_attn_gdn`` plus
    the block-start state for the decoder.
    -> (o_gated_delta, o_attn, final_state, chunk_start_state)."""
    _check_common(ops_for_incomplete_chunks, nats_block_size, attn_sw_size, cu_seqlens, use_g_for_attn,
                  all_incomplete_ops)
    if n_tokens_in_current_block:
        raise NotImplementedError("continued prefill into a partially filled block is not built")
    strategy = all_incomplete_ops[ops_for_incomplete_chunks]
    if not strategy['gated_delta_net'] or not incomplete_block_start_with_ht:
        raise NotImplementedError("only own-block linear attention starting from the carried state is built")
    if scale_attn is None:
        scale_attn = k_attn.shape[-1] ** -0.5
    if scale_lattn is None:
        scale_lattn = k_lattn.shape[-1] ** -0.5
    T = q_lattn.shape[1]
    with torch.no_grad():
        tables = build_selection_tables(nats_block_types, T, nats_block_size)
        o_attn, _ = _ops.attn_fwd(q_attn, k_attn, v_attn, tables, scale_attn, own_chunk=strategy['attn'])
        o_gdn, ht, inter = _ops.linear_fwd(_lib.RULE_GDN, q_lattn, k_lattn, v_lattn, g, beta, tables, scale_lattn,
                                           initial_state_gated_delta_chunk_start, decay_for_non_gdn_blocks,
                                           lattn_use_qk_l2norm_in_kernel, True, return_intermediates=True)
        if not output_final_state_gated_delta:
            return o_gdn, o_attn, None, None
        start = _chunk_start_state(inter, ht, inter['gcs'], tables, op_type_last_chunk, T, nats_block_size,
                                   decay_for_non_gdn_blocks)
    return o_gdn, o_attn, ht, start


def repeat_masks(attn_msk: torch.Tensor, n_rep: int) -> torch.Tensor:
    """[B, HN, q, k] -> [B, HN * n_rep, q, k] (src/nats/ops/attns/attn_utils.py:3-13)."""
    return attn_msk if n_rep == 1 else attn_msk.repeat_interleave(n_rep, dim=1)


def _masked_sdpa(q_attn, k_attn, v_attn, attn_msk, scale_attn):
    """Softmax branch of a decoding step: the new queries against all cached keys under the cache's visibility mask
    (mixed_attn_gdn.py:475-483 of the reference does the same with torch's SDPA)."""
    HQ, HKV = q_attn.shape[2], k_attn.shape[2]
    msk = repeat_masks(attn_msk, HQ // attn_msk.shape[1])
    kk, vv = k_attn.transpose(1, 2), v_attn.transpose(1, 2)
    if HKV != HQ:
        kk, vv = kk.repeat_interleave(HQ // HKV, dim=1), vv.repeat_interleave(HQ // HKV, dim=1)
    o = torch.nn.functional.scaled_dot_product_attention(q_attn.transpose(1, 2), kk, vv, attn_mask=msk, scale=scale_attn)
    o = torch.where(msk.any(-1, keepdim=True), o, torch.zeros_like(o))       # a query without any visible key gives 0
    return o.transpose(1, 2).contiguous()


def nats_mixed_attn_gdn_recurrent(
        q_attn: torch.Tensor, k_attn: torch.Tensor, v_attn: torch.Tensor,
        q_lattn: torch.Tensor, k_lattn: torch.Tensor, v_lattn: torch.Tensor,
        attn_msk: torch.Tensor,
        initial_state_gated_delta: torch.Tensor,
        initial_state_gated_delta_chunk_start: torch.Tensor,
        g: torch.Tensor,
        g_cumsum: torch.Tensor,
        beta: torch.Tensor,
        nats_block_types: torch.Tensor,
        n_tokens_in_current_block: int = 0,
        scale_attn=None, scale_lattn=None,
        cu_seqlens=None, cu_seqlens_nats=None,
        nats_block_size: int = 64,
        attn_sw_size: int | None = None,
        ops_for_incomplete_chunks: str = 'gated_delta_net',
        output_final_state_gated_delta: bool = False,
        decay_for_non_gdn_blocks: bool = False,
        incomplete_block_start_with_ht: bool = True,
        use_g_for_attn: bool = False,
        lattn_use_qk_l2norm_in_kernel: bool = True,
):
    """Decoding step (mixed_attn_gdn.py:443-590): a few new tokens that continue a block holding
    ``n_tokens_in_current_block`` tokens.  k_attn / v_attn are all cached keys / values including the new tokens',
    ``attn_msk`` [B, HN or HQ, new tokens, keys] their visibility; ``initial_state_gated_delta`` is the current state,
    ``..._chunk_start`` the state the current block started from and ``g_cumsum`` [B,H] the block's log decay so far.
    -> (o_gated_delta, o_attn, state after the new tokens, state at the start of the then-current block)."""
    _check_common(ops_for_incomplete_chunks, nats_block_size, attn_sw_size, cu_seqlens, use_g_for_attn, all_incomplete_ops)
    if not all_incomplete_ops[ops_for_incomplete_chunks]['gated_delta_net'] or not incomplete_block_start_with_ht:
        raise NotImplementedError("decoding is built for own-block linear attention starting from the carried state")
    if scale_attn is None:
        scale_attn = k_attn.shape[-1] ** -0.5
    if scale_lattn is None:
        scale_lattn = k_lattn.shape[-1] ** -0.5
    with torch.no_grad():
        o_attn = _masked_sdpa(q_attn, k_attn, v_attn, attn_msk, scale_attn)
        B, _, H, _ = q_lattn.shape
        o_gdn, state, start = _ops.linear_recurrent_step(
            _lib.RULE_GDN, q_lattn, k_lattn, v_lattn, g, beta, nats_block_types, initial_state_gated_delta,
            initial_state_gated_delta_chunk_start, g_cumsum.reshape(B, H), int(n_tokens_in_current_block), nats_block_size,
            scale_lattn, decay_for_non_gdn_blocks, lattn_use_qk_l2norm_in_kernel)
    return o_gdn, o_attn, state, start
