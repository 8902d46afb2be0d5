"""``nats_mixed_attn_mamba``: softmax branch + Mamba2/SSD branch of the NAtSL-Mamba2 layer.

Mirrors ``src/nats/ops/mixed_ops/mixed_attn_mamba.py:295-332`` (op) and ``:363-457``
(chunk inference).  q = C, k = B (already L2-normalised by the layer), v = x * dt, g = A * dt.
"""
from __future__ import annotations

import torch

from . import _lib, _ops
from . import mixed_attn_gdn as gdn_ops
from .mixed_attn_gdn import _check_common, _chunk_start_state, per_chunk_tables
from .nats_util import build_selection_tables

# mixed_attn_mamba.py:33-46
all_incomplete_ops = {
    'all': dict(attn=True, mamba=True),
    'attn': dict(attn=True, mamba=False),
    'mamba': dict(attn=False, mamba=True),
}


class NAtSMixedAttentionMamba(torch.autograd.Function):
    """Forward and backward of mixed_attn_mamba.py:51-292."""

    @staticmethod
    def forward(ctx, q_attn, k_attn, v_attn, q_lattn, k_lattn, v_lattn, initial_state_mamba, g, nats_block_types,
                n_nats_blocks, scale_attn, scale_lattn, cu_seqlens, cu_seqlens_nats, nats_block_size, attn_sw_size,
                ops_for_incomplete_chunks, output_final_state_mamba, compute_dnats_for_invalid_blocks_attn,
                compute_dnats_for_invalid_blocks_linear_att, decay_for_non_mamba_blocks, incomplete_block_start_with_ht,
                use_g_for_attn):
        _check_common(ops_for_incomplete_chunks, nats_block_size, attn_sw_size, cu_seqlens, use_g_for_attn,
                      all_incomplete_ops)
        strategy = all_incomplete_ops[ops_for_incomplete_chunks]
        own_linear = strategy['mamba']
        if own_linear and not incomplete_block_start_with_ht:
            raise NotImplementedError("incomplete_block_start_with_ht=False is not built")
        T = q_lattn.shape[1]
        tables = build_selection_tables(nats_block_types, T, nats_block_size)
        lin_tables = tables if own_linear else per_chunk_tables(nats_block_types, T, nats_block_size)
        ctx.bwd_ok, ctx.bwd_why = True, ""
        if q_lattn.dtype == torch.float32:
            if not own_linear:
                raise NotImplementedError("ops_for_incomplete_chunks='attn' is built for bf16 tensors only")
            o_attn, _ = _ops.attn_fwd_fp32(q_attn, k_attn, v_attn, tables, scale_attn, own_chunk=strategy['attn'])
            o_m, ht, _ = _ops.linear_recurrent(_lib.RULE_MAMBA, q_lattn, k_lattn, v_lattn, g, None, tables, scale_lattn,
                                               initial_state_mamba, decay_for_non_mamba_blocks, False)
            ctx.bwd_ok, ctx.bwd_why = False, "the backward pass is built for bf16 tensors (fp32 tensors run forward only)"
            return o_m, o_attn, (ht if output_final_state_mamba else None)
        o_attn, lse = _ops.attn_fwd(q_attn, k_attn, v_attn, tables, scale_attn, own_chunk=strategy['attn'])
        o_m, ht, _ = _ops.linear_fwd(_lib.RULE_MAMBA, q_lattn, k_lattn, v_lattn, g, None, lin_tables, scale_lattn,
                                     initial_state_mamba, decay_for_non_mamba_blocks, False,
                                     output_final_state_mamba, own_chunk=own_linear)
        if not own_linear:
            ctx.bwd_ok, ctx.bwd_why = False, "the backward pass is not built for ops_for_incomplete_chunks='attn'"
        elif nats_block_size != 64:
            ctx.bwd_ok, ctx.bwd_why = False, "the backward pass is built for nats_block_size = 64"
        ctx.save_for_backward(q_attn, k_attn, v_attn, o_attn, lse, q_lattn, k_lattn, v_lattn, g, None, initial_state_mamba)
        ctx.tables = tables
        ctx.scale_attn, ctx.scale_lattn, ctx.own_attn = float(scale_attn), float(scale_lattn), strategy['attn']
        ctx.decay, ctx.use_l2norm = bool(decay_for_non_mamba_blocks), False
        ctx.invalid_dnats_linear = bool(compute_dnats_for_invalid_blocks_linear_att)
        ctx.compat = gdn_ops.REFERENCE_COMPAT_BWD
        ctx.types_dtype = nats_block_types.dtype
        return o_m, o_attn, ht

    @staticmethod
    def backward(ctx, do_m, do_attn, dht):
        dqa, dka, dva, dq, dk, dv, dh0, dg, _, dnats = gdn_ops.hybrid_backward(ctx, _lib.RULE_MAMBA, do_m, do_attn, dht)
        return (dqa, dka, dva, dq, dk, dv, dh0, dg, dnats) + (None,) * 14


def nats_mixed_attn_mamba(
        q_attn: torch.Tensor, k_attn: torch.Tensor, v_attn: torch.Tensor,
        q_lattn: torch.Tensor, k_lattn: torch.Tensor, v_lattn: torch.Tensor,
        initial_state_mamba: torch.Tensor,
        g: torch.Tensor,
        nats_block_types: torch.Tensor,
        n_nats_blocks: torch.Tensor,
        scale_attn=None, scale_lattn=None,
        cu_seqlens=None, cu_seqlens_nats=None,
        nats_block_size: int = 64,
        attn_sw_size: int | None = None,
        ops_for_incomplete_chunks: str = 'all',
        output_final_state_mamba: bool = False,
        compute_dnats_for_invalid_blocks_attn: bool = False,
        compute_dnats_for_invalid_blocks_linear_att: bool = True,
        decay_for_non_mamba_blocks: bool = False,
        incomplete_block_start_with_ht: bool = True,
        use_g_for_attn: bool = False,
):
    """-> (o_mamba [B,T,H,V], o_attn [B,T,HQ,V_attn], final_state [B,H,K,V] fp32 or None).  Differentiable for bf16
    tensors with block size 64 in the modes 'all' and 'mamba' (other configurations raise in ``backward``)."""
    if scale_attn is None:
        scale_attn = k_attn.shape[-1] ** -0.5
    if scale_lattn is None:
        scale_lattn = 1                                                     # mixed_attn_mamba.py:318-319
    return NAtSMixedAttentionMamba.apply(
        q_attn, k_attn, v_attn, q_lattn, k_lattn, v_lattn, initial_state_mamba, g, nats_block_types, n_nats_blocks,
        scale_attn, scale_lattn, cu_seqlens, cu_seqlens_nats, nats_block_size, attn_sw_size, ops_for_incomplete_chunks,
        output_final_state_mamba, compute_dnats_for_invalid_blocks_attn, compute_dnats_for_invalid_blocks_linear_att,
        decay_for_non_mamba_blocks, incomplete_block_start_with_ht, use_g_for_attn)


def nats_mixed_attn_mamba_chunk_inference(
        q_attn: torch.Tensor, k_attn: torch.Tensor, v_attn: torch.Tensor,
        q_lattn: torch.Tensor, k_lattn: torch.Tensor, v_lattn: torch.Tensor,
        initial_state_mamba_start: torch.Tensor,
        g: torch.Tensor,
        nats_block_types: torch.Tensor,
        op_type_last_chunk: torch.Tensor | None,
        n_nats_blocks: torch.Tensor,
        n_tokens_in_current_block: int = 0,
        scale_attn=None, scale_lattn=None,
        cu_seqlens=None, cu_seqlens_nats=None,
        nats_block_size: int = 64,
        ops_for_incomplete_chunks: str = 'all',
        output_final_state_mamba: bool = True,
        decay_for_non_mamba_blocks: bool = True,
        incomplete_block_start_with_ht: bool = True,
        use_g_for_attn: bool = False,
):
    """-> (o_mamba, o_attn, final_state, chunk_start_state)  (mixed_attn_mamba.py:363-457)."""
    _check_common(ops_for_incomplete_chunks, nats_block_size, None, cu_seqlens, use_g_for_attn, all_incomplete_ops)
    if n_tokens_in_current_block:
        raise NotImplementedError("continued prefill into a partially filled block is not built")
    strategy = all_incomplete_ops[ops_for_incomplete_chunks]
    if not strategy['mamba'] or not incomplete_block_start_with_ht:
        raise NotImplementedError("only own-block linear attention starting from the carried state is built")
    if scale_attn is None:
        scale_attn = k_attn.shape[-1] ** -0.5
    if scale_lattn is None:
        scale_lattn = k_lattn.shape[-1] ** -0.5                             # mixed_attn_mamba.py:389-390
    T = q_lattn.shape[1]
    with torch.no_grad():
        tables = build_selection_tables(nats_block_types, T, nats_block_size)
        o_attn, _ = _ops.attn_fwd(q_attn, k_attn, v_attn, tables, scale_attn, own_chunk=strategy['attn'])
        o_m, ht, inter = _ops.linear_fwd(_lib.RULE_MAMBA, q_lattn, k_lattn, v_lattn, g, None, tables, scale_lattn,
                                         initial_state_mamba_start, decay_for_non_mamba_blocks, False, True,
                                         return_intermediates=True)
        if not output_final_state_mamba:
            return o_m, o_attn, None, None
        start = _chunk_start_state(inter, ht, inter['gcs'], tables, op_type_last_chunk, T, nats_block_size,
                                   decay_for_non_mamba_blocks)
    return o_m, o_attn, ht, start


def nats_mixed_attn_mamba_recurrent(
        q_attn: torch.Tensor, k_attn: torch.Tensor, v_attn: torch.Tensor,
        q_lattn: torch.Tensor, k_lattn: torch.Tensor, v_lattn: torch.Tensor,
        attn_msk: torch.Tensor,
        initial_state_mamba: torch.Tensor,
        initial_state_mamba_chunk_start: torch.Tensor,
        g: torch.Tensor,
        g_cumsum: torch.Tensor,
        nats_block_types: torch.Tensor,
        n_tokens_in_current_block: int = 0,
        scale_attn=None, scale_lattn=None,
        cu_seqlens=None, cu_seqlens_nats=None,
        nats_block_size: int = 64,
        ops_for_incomplete_chunks: str = 'all',
        output_final_state_mamba: bool = False,
        decay_for_non_mamba_blocks: bool = False,
        incomplete_block_start_with_ht: bool = True,
        use_g_for_attn: bool = False,
):
    """Decoding step of the NAtSL-Mamba2 op (mixed_attn_mamba.py:460-593): see ``nats_mixed_attn_gdn_recurrent``.
    -> (o_mamba, o_attn, state after the new tokens, state at the start of the then-current block)."""
    _check_common(ops_for_incomplete_chunks, nats_block_size, None, cu_seqlens, use_g_for_attn, all_incomplete_ops)
    if not all_incomplete_ops[ops_for_incomplete_chunks]['mamba'] or not incomplete_block_start_with_ht:
        raise NotImplementedError("decoding is built for own-block linear attention starting from the carried state")
    if scale_attn is None:
        scale_attn = k_attn.shape[-1] ** -0.5
    if scale_lattn is None:
        scale_lattn = k_lattn.shape[-1] ** -0.5
    with torch.no_grad():
        o_attn = gdn_ops._masked_sdpa(q_attn, k_attn, v_attn, attn_msk, scale_attn)
        B, _, H, _ = q_lattn.shape
        o_m, state, start = _ops.linear_recurrent_step(
            _lib.RULE_MAMBA, q_lattn, k_lattn, v_lattn, g, None, nats_block_types, initial_state_mamba,
            initial_state_mamba_chunk_start, g_cumsum.reshape(B, H), int(n_tokens_in_current_block), nats_block_size,
            scale_lattn, decay_for_non_mamba_blocks, False)
    return o_m, o_attn, state, start
