"""``NeuralAttentionSearchLinearAttnGDN``: the NAtSL layer on the Gated DeltaNet parameterisation, with the
constructor arguments, parameter names and forward signature of the reference layer
(src/nats/layers/natsl_attn_gdn.py:64-666).  The hybrid attention itself runs in the CUDA ops of this package;
projections and the small modules around it are plain PyTorch.

Built: full-sequence prefill and training (``mode='chunk'``), and decoding with a ``NAtSCache`` in ``past_key_values``
(prefill into the empty cache, then steps of fewer than 64 tokens).  Variable-length batches and rotary embeddings
raise ``NotImplementedError``.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .mixed_attn_gdn import nats_mixed_attn_gdn, nats_mixed_attn_gdn_chunk_inference, nats_mixed_attn_gdn_recurrent
from .decoding import forward_cached
from .modules import FusedMultiInputRMSNormGated, RMSNorm, ShortConvolution, hard_softmax, mean_pooling


class NeuralAttentionSearchLinearAttnGDN(nn.Module):
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
            ops_for_incomplete_chunks: str = 'all',
            mode: str = 'chunk',
            use_gate: bool = True,
            use_short_conv: bool = True,
            allow_neg_eigval: bool = False,
            conv_size: int = 4,
            conv_bias: bool = False,
            conv_activation: str | None = 'silu',
            outputs_are_weighted: bool = True,
            attn_qk_norm: bool = True,
            attn_with_short_conv: bool = True,
            compute_dnats_for_invalid_blocks_attn: bool = False,
            compute_dnats_for_invalid_blocks_linear_att: bool = False,
            decay_for_non_gdn_blocks: bool = True,
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
        self.allow_neg_eigval = allow_neg_eigval
        self.hidden_size = hidden_size
        self.expand_v = expand_v
        self.use_gate = use_gate
        self.use_short_conv = use_short_conv
        self.conv_size = conv_size
        self.conv_bias = conv_bias
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
        self.attn_groups = num_attn_heads // num_heads
        self.num_attn_v_heads = self.attn_groups * self.num_v_heads
        self.attn_with_short_conv = attn_with_short_conv
        self.attn_rope_theta = attn_rope_theta
        self.attn_max_position_embeddings = attn_max_position_embeddings
        if self.attn_qk_norm:
            self.q_norm = RMSNorm(self.head_attn_k_dim, eps=norm_eps)
            self.k_norm = RMSNorm(self.head_attn_k_dim, eps=norm_eps)
        self.attn_apply_pos_encoding = attn_apply_pos_encoding
        if attn_apply_pos_encoding:
            raise NotImplementedError("attn_apply_pos_encoding=True (rotary) is not built; the trained configs set False")
        self.rotary = None
        self.compute_dnats_for_invalid_blocks_attn = compute_dnats_for_invalid_blocks_attn
        self.compute_dnats_for_invalid_blocks_linear_att = compute_dnats_for_invalid_blocks_linear_att
        self.incomplete_block_start_with_ht = incomplete_block_start_with_ht
        self.decay_for_non_gdn_blocks = decay_for_non_gdn_blocks
        self.usg_for_attn = False
        if num_nats_head is None:
            num_nats_head = num_heads
        self.nats_block_size = nats_block_size
        self.num_nats_head = num_nats_head
        self.nats_block_agg_type = nats_block_agg_type
        self.ops_for_incomplete_chunks = ops_for_incomplete_chunks

        if not math.isclose(self.num_v_heads * self.head_dim * expand_v, self.value_dim, rel_tol=1e-5):
            raise ValueError(f"expand_v={expand_v} does not produce an integer value_dim")
        if self.num_v_heads > self.num_heads:
            raise NotImplementedError("grouped value heads (num_v_heads > num_heads) are not built")
        if self.num_attn_heads > self.num_heads and self.num_attn_heads % self.num_heads != 0:
            raise ValueError(f"num_attn_heads={self.num_attn_heads} must be divisible by num_heads={self.num_heads}.")
        if not math.isclose(head_dim * expand_v, self.head_v_dim, rel_tol=1e-5):
            raise ValueError(f"expand_v={expand_v} does not produce an integer head_v_dim")
        assert mode in ['chunk', 'fused_recurrent'], f"Not supported mode `{mode}`."

        self.q_proj = nn.Linear(hidden_size, self.key_dim, bias=False)
        self.k_proj = nn.Linear(hidden_size, self.key_dim, bias=False)
        self.v_proj = nn.Linear(hidden_size, self.value_dim, bias=False)
        self.a_proj = nn.Linear(hidden_size, self.num_v_heads, bias=False)
        self.b_proj = nn.Linear(hidden_size, self.num_v_heads, bias=False)
        if nats_block_agg_type != 'mean':
            raise NotImplementedError(f"Pooling system {nats_block_agg_type} is not supported!")
        self.pooling_func = mean_pooling
        self.nats_sample_strategy = nats_sample_strategy
        if nats_sample_strategy == 'gumble':
            self.nats_sample_func = lambda x: F.gumbel_softmax(x, hard=True, dim=-1)
        else:
            self.nats_sample_func = hard_softmax
        self.nats_layer = nn.Linear(hidden_size, self.n_ops * self.num_nats_head, bias=False)

        A = torch.empty(self.num_v_heads, dtype=torch.float32).uniform_(0, 16)
        self.A_log = nn.Parameter(torch.log(A))
        self.A_log._no_weight_decay = True
        dt_min, dt_max, dt_init_floor = 0.001, 0.1, 1e-4
        dt = torch.exp(torch.rand(self.num_v_heads) * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min))
        dt = torch.clamp(dt, min=dt_init_floor)
        self.dt_bias = nn.Parameter(dt + torch.log(-torch.expm1(-dt)))
        self.dt_bias._no_weight_decay = True

        self.outputs_are_weighted = outputs_are_weighted
        if self.outputs_are_weighted:
            self.nats_out_weights_layer = nn.Linear(self.key_dim, self.n_ops * self.num_attn_heads, bias=False)
        if use_short_conv:
            self.q_conv1d = ShortConvolution(self.key_dim, conv_size, bias=conv_bias, activation=conv_activation)
            self.k_conv1d = ShortConvolution(self.key_dim, conv_size, bias=conv_bias, activation=conv_activation)
            self.v_conv1d = ShortConvolution(self.value_dim, conv_size, bias=conv_bias, activation=conv_activation)
        if use_gate:
            self.g_proj = nn.Linear(hidden_size, self.value_dim, bias=False)
            self.o_norm = FusedMultiInputRMSNormGated(self.head_attn_v_dim, eps=norm_eps)
        else:
            self.o_norm = nn.ModuleList([RMSNorm(self.head_v_dim, eps=norm_eps), RMSNorm(self.head_attn_v_dim, eps=norm_eps)])
        self.o_proj = nn.Linear(self.value_dim, hidden_size, bias=False)
        self.attn_fraction = torch.zeros(1)

    # ------------------------------------------------------------------------------------------------
    def select(self, pooled: torch.Tensor) -> torch.Tensor:
        """Block-mean layer input [B, NB, D] -> sampled 0/1 block types [B, NB, HN, n_ops] (natsl_attn_gdn.py:411-420)."""
        logits = self.nats_layer(pooled).unflatten(-1, (self.num_nats_head, self.n_ops))
        return self.nats_sample_func(logits)

    def project_qkv(self, hidden_states: torch.Tensor, conv_state=None, want_conv_state: bool = False) -> dict:
        """q, k, v of both branches, the mixing weights, beta and the log decay from the layer input
        (natsl_attn_gdn.py:425-530).  ``conv_state``: the (q, k, v) convolution tails of a decoding cache."""
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
        if self.outputs_are_weighted:
            o_weights = self.nats_out_weights_layer(q).unflatten(-1, (self.num_attn_heads, self.n_ops)).softmax(-1)
        q = q.unflatten(-1, (-1, self.head_k_dim))
        k = k.unflatten(-1, (-1, self.head_k_dim))
        v = v.unflatten(-1, (-1, self.head_v_dim))
        q_attn = q_attn.unflatten(-1, (-1, self.head_attn_k_dim))
        k_attn = k_attn.unflatten(-1, (-1, self.head_attn_k_dim))
        v_attn = v_attn.unflatten(-1, (-1, self.head_attn_v_dim))
        if self.attn_qk_norm:
            q_attn, k_attn = self.q_norm(q_attn), self.k_norm(k_attn)
        beta = self.b_proj(hidden_states).sigmoid()
        if self.allow_neg_eigval:
            beta = beta * 2.
        g = -self.A_log.float().exp() * F.softplus(self.a_proj(hidden_states).float() + self.dt_bias)
        return dict(q=q, k=k, v=v, q_attn=q_attn, k_attn=k_attn, v_attn=v_attn, beta=beta, g=g, o_weights=o_weights,
                    conv_state=new_state)

    def project(self, hidden_states: torch.Tensor, want_conv_state: bool = False) -> dict:
        """Everything the hybrid-attention op consumes, computed from the layer input
        (natsl_attn_gdn.py:411-530, 553-555)."""
        B, T, dim = hidden_states.shape
        hs_reduced = self.pooling_func(hidden_states.unsqueeze(-2), chunk_size=self.nats_block_size).view(B, -1, dim)
        types_raw = self.select(hs_reduced)
        p = self.project_qkv(hidden_states, want_conv_state=want_conv_state)
        types = types_raw.clone()
        op_type_last = types[:, -1].clone()
        types[:, -1] = 1                                   # natsl_attn_gdn.py:553
        n_blocks = types.int().sum(1)
        self.attn_fraction = (n_blocks.float()[..., 0] / types.shape[1]).mean(0).detach()
        p.update(types=types, types_raw=types_raw, n_blocks=n_blocks, op_type_last=op_type_last)
        return p

    def mix(self, hidden_states, o_gated_delta, o_attn, o_weights):
        """Norm, mix, gate and project the two branch outputs (natsl_attn_gdn.py:652-666)."""
        if self.use_gate:
            g = self.g_proj(hidden_states).unflatten(-1, (-1, self.head_v_dim))
            if self.outputs_are_weighted:
                o = self.o_norm(o_gated_delta.reshape(o_attn.shape), o_attn, g.reshape(o_attn.shape), o_weights)
            else:
                o = self.o_norm(o_gated_delta, o_attn.reshape(o_gated_delta.shape), g)
        else:
            o1 = self.o_norm[0](o_gated_delta)
            o2 = self.o_norm[1](o_attn)
            o = o1 + o2.reshape(o1.shape)
        return self.o_proj(o.flatten(-2))

    def forward(
            self,
            hidden_states: torch.Tensor,
            attention_mask: Optional[torch.Tensor] = None,
            past_key_values=None,
            use_cache: Optional[bool] = False,
            output_attentions: Optional[bool] = False,
            **kwargs: Dict
    ) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[object]]:
        if attention_mask is not None:
            assert len(attention_mask.shape) == 2
            if len(attention_mask) > 1:
                raise NotImplementedError("Attention with variable length is not supported yet!")
        if kwargs.get('cu_seqlens', None) is not None:
            raise NotImplementedError("variable-length batches are not built")
        B, T, _ = hidden_states.shape
        if past_key_values is not None:
            return self._forward_cached(hidden_states, past_key_values)
        if T < 64 or self.mode != 'chunk':
            raise NotImplementedError("fewer than 64 tokens (decoding) need a NAtSCache in past_key_values")
        p = self.project(hidden_states)
        common = dict(scale_attn=p['k_attn'].shape[-1] ** -0.5, scale_lattn=p['k'].shape[-1] ** -0.5,
                      cu_seqlens=None, cu_seqlens_nats=None, nats_block_size=self.nats_block_size,
                      ops_for_incomplete_chunks=self.ops_for_incomplete_chunks,
                      incomplete_block_start_with_ht=self.incomplete_block_start_with_ht,
                      decay_for_non_gdn_blocks=self.decay_for_non_gdn_blocks, use_g_for_attn=self.usg_for_attn,
                      lattn_use_qk_l2norm_in_kernel=True)
        if self.training:
            o_gd, o_attn, _ = nats_mixed_attn_gdn(
                q_attn=p['q_attn'], k_attn=p['k_attn'], v_attn=p['v_attn'], q_lattn=p['q'], k_lattn=p['k'], v_lattn=p['v'],
                initial_state_gated_delta=None, g=p['g'], beta=p['beta'], nats_block_types=p['types'],
                n_nats_blocks=p['n_blocks'], output_final_state_gated_delta=use_cache,
                compute_dnats_for_invalid_blocks_attn=self.compute_dnats_for_invalid_blocks_attn,
                compute_dnats_for_invalid_blocks_linear_att=self.compute_dnats_for_invalid_blocks_linear_att, **common)
        else:
            o_gd, o_attn, _, _ = nats_mixed_attn_gdn_chunk_inference(
                q_attn=p['q_attn'], k_attn=p['k_attn'], v_attn=p['v_attn'], q_lattn=p['q'], k_lattn=p['k'], v_lattn=p['v'],
                initial_state_gated_delta_chunk_start=None, g=p['g'], beta=p['beta'], nats_block_types=p['types'],
                op_type_last_chunk=p['op_type_last'] if T % self.nats_block_size == 0 else None,
                n_nats_blocks=p['n_blocks'], output_final_state_gated_delta=use_cache, **common)
        o = self.mix(hidden_states, o_gd, o_attn, p['o_weights'])
        return o, None, past_key_values

    # ------------------------------------------------------------------------------------------------ decoding
    def _ops_for_cache(self) -> dict:
        """The two ops the cached forward (``decoding.forward_cached``) runs for this layer."""
        common = dict(nats_block_size=self.nats_block_size, ops_for_incomplete_chunks=self.ops_for_incomplete_chunks,
                      output_final_state_gated_delta=True, decay_for_non_gdn_blocks=self.decay_for_non_gdn_blocks,
                      incomplete_block_start_with_ht=True, use_g_for_attn=self.usg_for_attn, lattn_use_qk_l2norm_in_kernel=True)

        def chunk(p, T):
            return nats_mixed_attn_gdn_chunk_inference(
                q_attn=p['q_attn'], k_attn=p['k_attn'], v_attn=p['v_attn'], q_lattn=p['q'], k_lattn=p['k'], v_lattn=p['v'],
                initial_state_gated_delta_chunk_start=None, g=p['g'], beta=p['beta'], nats_block_types=p['types'],
                op_type_last_chunk=p['op_type_last'] if T % self.nats_block_size == 0 else None, n_nats_blocks=p['n_blocks'],
                scale_attn=p['k_attn'].shape[-1] ** -0.5, scale_lattn=p['k'].shape[-1] ** -0.5, **common)

        def step(p, cache, msk, types_new, t_off):
            return nats_mixed_attn_gdn_recurrent(
                q_attn=p['q_attn'], k_attn=cache.k_attn, v_attn=cache.v_attn, q_lattn=p['q'], k_lattn=p['k'], v_lattn=p['v'],
                attn_msk=msk, initial_state_gated_delta=cache.state,
                initial_state_gated_delta_chunk_start=cache.state_block_start, g=p['g'], g_cumsum=cache.g_block,
                beta=p['beta'], nats_block_types=types_new, n_tokens_in_current_block=t_off,
                scale_attn=p['k_attn'].shape[-1] ** -0.5, scale_lattn=p['k'].shape[-1] ** -0.5, **common)

        return dict(chunk=chunk, step=step)

    def _forward_cached(self, hidden_states: torch.Tensor, past_key_values):
        """Prefill into an empty cache (64 tokens or more, chunk kernels) or a decoding step of fewer than 64 tokens
        (token recurrence with re-roll + masked attention over the cached keys), natsl_attn_gdn.py:389-410, 576-650."""
        o_gd, o_attn, o_w = forward_cached(self, hidden_states, past_key_values)
        with torch.no_grad():
            return self.mix(hidden_states, o_gd, o_attn, o_w), None, past_key_values
