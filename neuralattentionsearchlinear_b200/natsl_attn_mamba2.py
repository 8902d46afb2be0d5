"""``NeuralAttentionSearchLinearAttnMamba``: the NAtSL layer on the Mamba2/SSD parameterisation, with the
constructor arguments, parameter names and forward signature of the reference layer
(src/nats/layers/natsl_attn_mamba2.py:66-599).  q = C and k = B are L2-normalised by the layer,
dt = softplus(a_proj + dt_bias), v <- v * dt, g = -exp(A_log) * dt (natsl_attn_mamba2.py:469-474).

Built: full-sequence training / prefill (``mode='chunk'``) and, with a ``NAtSCache`` in ``cache_params``, prefill into the
cache followed by decoding steps of fewer than 64 tokens; forward returns the projected output like the reference.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .decoding import forward_cached
from .mixed_attn_mamba import (nats_mixed_attn_mamba, nats_mixed_attn_mamba_chunk_inference,
                               nats_mixed_attn_mamba_recurrent)
from .modules import FusedMultiInputRMSNormGated, L2Norm, RMSNorm, ShortConvolution, hard_softmax, mean_pooling


class NeuralAttentionSearchLinearAttnMamba(nn.Module):
    def __init__(
            self,
            hidden_size: int = 2048,
            expand_v: float = 2,
            head_dim: int = 256,
            num_heads: int = 6,
            num_attn_heads: int = 24,
            num_v_heads: int = None,
            n_ops: int = 2,
            num_nats_head: Optional[int] = None,
            nats_block_size: int = 64,
            nats_block_agg_type: str = 'mean',
            nats_sample_strategy: str = 'argmax',
            ops_for_incomplete_chunks: str = 'gated_delta_net',
            mode: str = 'chunk',
            use_gate: bool = True,
            use_short_conv: bool = True,
            allow_neg_eigval: bool = False,
            conv_size: int = 4,
            conv_bias: bool = False,
            conv_activation: str | None = 'silu',
            outputs_are_wighted: bool = True,
            attn_qk_norm: bool = False,
            attn_with_short_conv: bool = False,
            compute_dnats_for_invalid_blocks_attn: bool = False,
            compute_dnats_for_invalid_blocks_linear_att: bool = False,
            decay_for_non_mamba_blocks: bool = True,
            incomplete_block_start_with_ht: bool = True,
            attn_apply_pos_encoding: bool = False,
            attn_rope_theta: Optional[float] = 10000.,
            attn_max_position_embeddings: Optional[int] = None,
            layer_idx: int = None,
            norm_eps: float = 1e-5,
            **kwargs
    ):
        super().__init__()
        self.mode = mode
        self.hidden_size = hidden_size
        self.expand_v = expand_v
        self.use_gate = use_gate
        self.use_short_conv = use_short_conv
        self.head_dim = head_dim
        self.num_heads = num_heads
        self.num_v_heads = num_v_heads if num_v_heads is not None else num_heads
        self.n_ops = n_ops
        self.head_k_dim = head_dim
        self.head_v_dim = int(self.head_dim * self.expand_v)
        self.key_dim = int(self.num_heads * self.head_k_dim)
        self.value_dim = int(self.num_v_heads * self.head_v_dim)
        self.layer_idx = layer_idx
        self.attn_qk_norm = attn_qk_norm
        self.num_attn_heads = num_attn_heads
        self.head_attn_k_dim = self.key_dim // self.num_attn_heads
        self.head_attn_v_dim = self.value_dim // self.num_attn_heads
        self.attn_with_short_conv = attn_with_short_conv
        if self.attn_qk_norm:
            self.q_norm = RMSNorm(self.head_attn_k_dim, eps=norm_eps)
            self.k_norm = RMSNorm(self.head_attn_k_dim, eps=norm_eps)
        self.q_norm2 = L2Norm(eps=norm_eps)
        self.k_norm2 = L2Norm(eps=norm_eps)
        if attn_apply_pos_encoding:
            raise NotImplementedError("attn_apply_pos_encoding=True (rotary) is not built")
        self.compute_dnats_for_invalid_blocks_attn = compute_dnats_for_invalid_blocks_attn
        self.compute_dnats_for_invalid_blocks_linear_att = compute_dnats_for_invalid_blocks_linear_att
        self.incomplete_block_start_with_ht = incomplete_block_start_with_ht
        self.decay_for_non_mamba_blocks = decay_for_non_mamba_blocks
        self.usg_for_attn = False
        if num_nats_head is None:
            num_nats_head = num_heads
        self.nats_block_size = nats_block_size
        self.num_nats_head = num_nats_head
        # the reference's default string names the GDN mode; for this layer it means "linear branch only"
        self.ops_for_incomplete_chunks = 'mamba' if ops_for_incomplete_chunks == 'gated_delta_net' else ops_for_incomplete_chunks
        if self.num_v_heads > self.num_heads:
            raise NotImplementedError("grouped value heads (num_v_heads > num_heads) are not built")
        if not math.isclose(head_dim * expand_v, self.head_v_dim, rel_tol=1e-5):
            raise ValueError(f"expand_v={expand_v} does not produce an integer head_v_dim")
        assert mode in ['chunk', 'fused_recurrent'], f"Not supported mode `{mode}`."

        self.q_proj = nn.Linear(hidden_size, self.key_dim, bias=False)
        self.k_proj = nn.Linear(hidden_size, self.key_dim, bias=False)
        self.v_proj = nn.Linear(hidden_size, self.value_dim, bias=False)
        self.a_proj = nn.Linear(hidden_size, self.num_v_heads, bias=False)
        if nats_block_agg_type != 'mean':
            raise NotImplementedError(f"Pooling system {nats_block_agg_type} is not supported!")
        self.pooling_func = mean_pooling
        self.nats_sample_func = (lambda x: F.gumbel_softmax(x, hard=True, dim=-1)) if nats_sample_strategy == 'gumble' else hard_softmax
        self.nats_layer = nn.Linear(hidden_size, self.n_ops * self.num_nats_head, bias=False)
        self.dt_bias = nn.Parameter(torch.ones(self.num_heads))
        self.A_log = nn.Parameter(torch.log(torch.arange(1, self.num_heads + 1).float()))
        self.A_log._no_weight_decay = True
        self.dt_bias._no_weight_decay = True
        self.outputs_are_wighted = outputs_are_wighted
        if self.outputs_are_wighted:
            self.nats_out_weights_layer = nn.Linear(self.key_dim, self.n_ops * self.num_attn_heads, bias=False)
        if use_short_conv:
            self.q_conv1d = ShortConvolution(self.key_dim, conv_size, bias=conv_bias, activation=conv_activation)
            self.k_conv1d = ShortConvolution(self.key_dim, conv_size, bias=conv_bias, activation=conv_activation)
            self.v_conv1d = ShortConvolution(self.value_dim, conv_size, bias=conv_bias, activation=conv_activation)
        if use_gate:
            self.g_proj = nn.Linear(hidden_size, self.value_dim, bias=False)
            self.o_norm = FusedMultiInputRMSNormGated(self.head_attn_v_dim, eps=norm_eps)
        else:
            raise NotImplementedError("use_gate=False is not built for the Mamba2 layer")
        self.o_proj = nn.Linear(self.value_dim, hidden_size, bias=False)
        self.attn_fraction = torch.zeros(1)

    def select(self, pooled: torch.Tensor) -> torch.Tensor:
        """Block-mean layer input [B, NB, D] -> sampled 0/1 block types [B, NB, HN, n_ops] (natsl_attn_mamba2.py:352-365)."""
        logits = self.nats_layer(pooled).unflatten(-1, (self.num_nats_head, self.n_ops))
        return self.nats_sample_func(logits)

    def project_qkv(self, hidden_states: torch.Tensor, conv_state=None, want_conv_state: bool = False) -> dict:
        """q = C, k = B, v = x * dt of the linear branch, q/k/v of the softmax branch, the mixing weights and the log decay
        from the layer input (natsl_attn_mamba2.py:366-474).  ``conv_state``: the (q, k, v) convolution tails of a cache."""
        cq, ck, cv = conv_state if conv_state is not None else (None, None, None)
        new_state = None
        if self.use_short_conv:
            if self.attn_with_short_conv:
                q, sq = self.q_conv1d(self.q_proj(hidden_states), cache=cq, output_final_state=want_conv_state)
                k, sk = self.k_conv1d(self.k_proj(hidden_states), cache=ck, output_final_state=want_conv_state)
                v, sv = self.v_conv1d(self.v_proj(hidden_states), cache=cv, output_final_state=want_conv_state)
                q_attn, k_attn, v_attn = q, k, v
            else:
                q_attn, k_attn, v_attn = self.q_proj(hidden_states), self.k_proj(hidden_states), self.v_proj(hidden_states)
                q, sq = self.q_conv1d(q_attn, cache=cq, output_final_state=want_conv_state)
                k, sk = self.k_conv1d(k_attn, cache=ck, output_final_state=want_conv_state)
                v, sv = self.v_conv1d(v_attn, cache=cv, output_final_state=want_conv_state)
            new_state = (sq, sk, sv)
        else:
            if self.attn_with_short_conv:
                q, k, v = (F.silu(p(hidden_states)) for p in (self.q_proj, self.k_proj, self.v_proj))
                q_attn, k_attn, v_attn = q, k, v
            else:
                q_attn, k_attn, v_attn = self.q_proj(hidden_states), self.k_proj(hidden_states), self.v_proj(hidden_states)
                q, k, v = F.silu(q_attn), F.silu(k_attn), F.silu(v_attn)
        o_weights = None
        if self.outputs_are_wighted:
            o_weights = self.nats_out_weights_layer(q).unflatten(-1, (self.num_attn_heads, self.n_ops)).softmax(-1)
        q = q.unflatten(-1, (-1, self.head_k_dim))
        k = k.unflatten(-1, (-1, self.head_k_dim))
        v = v.unflatten(-1, (-1, self.head_v_dim))
        q_attn = q_attn.unflatten(-1, (-1, self.head_attn_k_dim)).contiguous()
        k_attn = k_attn.unflatten(-1, (-1, self.head_attn_k_dim)).contiguous()
        v_attn = v_attn.unflatten(-1, (-1, self.head_attn_v_dim)).contiguous()
        if self.attn_qk_norm:
            q_attn, k_attn = self.q_norm(q_attn), self.k_norm(k_attn)
        q, k = self.q_norm2(q), self.k_norm2(k)
        dt = F.softplus(self.a_proj(hidden_states).float() + self.dt_bias)
        v = (v * dt.unsqueeze(-1)).to(v.dtype)
        g = -self.A_log.float().exp() * dt
        return dict(q=q, k=k, v=v, q_attn=q_attn, k_attn=k_attn, v_attn=v_attn, g=g, o_weights=o_weights,
                    conv_state=new_state)

    def project(self, hidden_states: torch.Tensor, want_conv_state: bool = False) -> dict:
        """Everything the hybrid-attention op consumes, computed from the layer input (natsl_attn_mamba2.py:355-474)."""
        B, T, dim = hidden_states.shape
        hs_reduced = self.pooling_func(hidden_states.unsqueeze(-2), chunk_size=self.nats_block_size).view(B, -1, dim)
        types_raw = self.select(hs_reduced)
        p = self.project_qkv(hidden_states, want_conv_state=want_conv_state)
        types = types_raw.clone()
        op_type_last = types[:, -1].clone()
        types[:, -1] = 1
        n_blocks = types.int().sum(1)
        self.attn_fraction = (n_blocks.float()[..., 0] / types.shape[1]).mean(0).detach()
        p.update(types=types, types_raw=types_raw, n_blocks=n_blocks, op_type_last=op_type_last)
        return p

    # ------------------------------------------------------------------------------------------------ decoding
    def _ops_for_cache(self) -> dict:
        """The two ops the cached forward (``decoding.forward_cached``) runs for this layer."""
        common = dict(nats_block_size=self.nats_block_size, ops_for_incomplete_chunks=self.ops_for_incomplete_chunks,
                      output_final_state_mamba=True, decay_for_non_mamba_blocks=self.decay_for_non_mamba_blocks,
                      incomplete_block_start_with_ht=True, use_g_for_attn=self.usg_for_attn, scale_lattn=1)

        def chunk(p, T):
            return nats_mixed_attn_mamba_chunk_inference(
                q_attn=p['q_attn'], k_attn=p['k_attn'], v_attn=p['v_attn'], q_lattn=p['q'], k_lattn=p['k'], v_lattn=p['v'],
                initial_state_mamba_start=None, g=p['g'], nats_block_types=p['types'],
                op_type_last_chunk=p['op_type_last'] if T % self.nats_block_size == 0 else None, n_nats_blocks=p['n_blocks'],
                scale_attn=p['k_attn'].shape[-1] ** -0.5, **common)

        def step(p, cache, msk, types_new, t_off):
            return nats_mixed_attn_mamba_recurrent(
                q_attn=p['q_attn'], k_attn=cache.k_attn, v_attn=cache.v_attn, q_lattn=p['q'], k_lattn=p['k'], v_lattn=p['v'],
                attn_msk=msk, initial_state_mamba=cache.state, initial_state_mamba_chunk_start=cache.state_block_start,
                g=p['g'], g_cumsum=cache.g_block, nats_block_types=types_new, n_tokens_in_current_block=t_off,
                scale_attn=p['k_attn'].shape[-1] ** -0.5, **common)

        return dict(chunk=chunk, step=step)

    def mix(self, hidden_states, o_mamba, o_attn, o_weights):
        g = self.g_proj(hidden_states)
        if self.outputs_are_wighted:
            o = self.o_norm(o_mamba.reshape(o_attn.shape), o_attn, g.reshape(o_attn.shape), o_weights)
        else:
            o = self.o_norm(o_mamba, o_attn.reshape(o_mamba.shape), g.reshape(o_mamba.shape))
        return self.o_proj(o.flatten(-2))

    def forward(
            self,
            hidden_states: torch.Tensor,
            attention_mask: Optional[torch.Tensor] = None,
            cache_params=None,
            use_cache: Optional[bool] = False,
            output_attentions: Optional[bool] = False,
            **kwargs: Dict
    ):
        if attention_mask is not None:
            assert len(attention_mask.shape) == 2
        if kwargs.get('cu_seqlens', None) is not None:
            raise NotImplementedError("variable-length batches are not built")
        B, T, _ = hidden_states.shape
        if cache_params is not None:                        # prefill into / decode from a NAtSCache
            o_m, o_attn, o_w = forward_cached(self, hidden_states, cache_params)
            with torch.no_grad():
                return self.mix(hidden_states, o_m, o_attn, o_w)
        if T < 64 or self.mode != 'chunk':
            raise NotImplementedError("fewer than 64 tokens (decoding) need a NAtSCache in cache_params")
        p = self.project(hidden_states)
        common = dict(scale_attn=p['k_attn'].shape[-1] ** -0.5, scale_lattn=1, cu_seqlens=None, cu_seqlens_nats=None,
                      nats_block_size=self.nats_block_size, ops_for_incomplete_chunks=self.ops_for_incomplete_chunks,
                      incomplete_block_start_with_ht=self.incomplete_block_start_with_ht,
                      decay_for_non_mamba_blocks=self.decay_for_non_mamba_blocks, use_g_for_attn=self.usg_for_attn)
        if self.training:
            o_m, o_attn, _ = nats_mixed_attn_mamba(
                q_attn=p['q_attn'], k_attn=p['k_attn'], v_attn=p['v_attn'], q_lattn=p['q'], k_lattn=p['k'], v_lattn=p['v'],
                initial_state_mamba=None, g=p['g'], nats_block_types=p['types'], n_nats_blocks=p['n_blocks'],
                output_final_state_mamba=use_cache,
                compute_dnats_for_invalid_blocks_attn=self.compute_dnats_for_invalid_blocks_attn,
                compute_dnats_for_invalid_blocks_linear_att=self.compute_dnats_for_invalid_blocks_linear_att, **common)
        else:
            o_m, o_attn, _, _ = nats_mixed_attn_mamba_chunk_inference(
                q_attn=p['q_attn'], k_attn=p['k_attn'], v_attn=p['v_attn'], q_lattn=p['q'], k_lattn=p['k'], v_lattn=p['v'],
                initial_state_mamba_start=None, g=p['g'], nats_block_types=p['types'],
                op_type_last_chunk=p['op_type_last'] if T % self.nats_block_size == 0 else None,
                n_nats_blocks=p['n_blocks'], output_final_state_mamba=use_cache, **common)
        return self.mix(hidden_states, o_m, o_attn, p['o_weights'])
