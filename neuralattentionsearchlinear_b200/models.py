"""Decoder model around the NAtSL-GDN layer, for the model-level benchmark configurations: embeddings, pre-norm
blocks (hybrid attention layer + SwiGLU MLP), final norm, LM head and next-token loss.

Plain ``nn.Module`` classes with the class names, configuration fields, parameter names and initialisation of the
reference's HuggingFace classes (src/nats/models/natsl_attn_gdn/configuration_natsl_attn_gdn.py:8-132,
modeling_natsl_attn_gdn.py:55-149 block, :163-191 initialisation, :220-320 model, :323-509 causal LM), so that a state
dict of the reference loads by name.  Everything outside the hybrid attention op is ordinary PyTorch; the HuggingFace
base classes (generation, cache, checkpoint I/O) are not restated: prefill and training only.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _lib
from .modules import RMSNorm, swiglu
from .nats_util import current_stream_ptr
from .natsl_attn_gdn import NeuralAttentionSearchLinearAttnGDN


@dataclass
class NeuralAttentionSearchLineraAttnGDNConfig:
    """Fields and defaults of configuration_natsl_attn_gdn.py:12-62 (the class name keeps the reference's spelling)."""
    attn_mode: str = "chunk"
    hidden_size: int = 2048
    expand_v: float = 2.0
    use_gate: bool = True
    use_short_conv: bool = True
    allow_neg_eigval: bool = False
    conv_size: int = 4
    conv_bias: bool = False
    head_dim: int = 256
    num_heads: int = 6
    num_attn_heads: int = 12
    num_v_heads: Optional[int] = None
    n_ops: int = 2
    num_nats_head: Optional[int] = None
    nats_block_size: int = 64
    nats_block_agg_type: str = 'mean'
    nats_sample_strategy: str = 'argmax'
    ops_for_incomplete_chunks: str = 'all'
    max_position_embeddings: int = 2048
    hidden_ratio: Optional[int] = 4
    intermediate_size: Optional[int] = None
    hidden_act: str = "swish"
    outputs_are_wighted: bool = True
    attn_qk_norm: bool = False
    attn_with_short_conv: bool = False
    compute_dnats_for_invalid_blocks_attn: bool = False
    compute_dnats_for_invalid_blocks_linear_att: bool = False
    incomplete_block_start_with_ht: bool = True
    decay_for_non_gdn_blocks: bool = False
    attn_apply_pos_encoding: bool = True
    attn_rope_theta: Optional[float] = 10000.
    attn_max_position_embeddings: Optional[int] = None
    num_hidden_layers: int = 21
    norm_eps: float = 1e-6
    use_cache: bool = True
    pad_token_id: Optional[int] = None
    bos_token_id: int = 1
    eos_token_id: int = 2
    tie_word_embeddings: bool = False
    initializer_range: float = 0.02
    fuse_norm: bool = True
    fuse_swiglu: bool = True
    fuse_cross_entropy: bool = True
    use_l2warp: bool = False
    vocab_size: int = 32000
    gdn_layers: List[int] = field(default_factory=list)


class GatedMLP(nn.Module):
    """down(swish(gate(x)) * up(x)), no biases; default width 256 * ceil(hidden * ratio * 2/3 / 256)
    (the MLP of modeling_natsl_attn_gdn.py:111-117)."""

    def __init__(self, hidden_size: int, hidden_ratio: Optional[int] = None, intermediate_size: Optional[int] = None,
                 hidden_act: str = 'swish', fuse_swiglu: bool = True):
        super().__init__()
        if hidden_ratio is None:
            hidden_ratio = 4
        if intermediate_size is None:
            intermediate_size = 256 * ((int(hidden_size * hidden_ratio * 2 / 3) + 255) // 256)
        if hidden_act not in ('swish', 'silu'):
            raise ValueError(f"Unsupported hidden_act: {hidden_act}")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.gate_proj = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.up_proj = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.down_proj = nn.Linear(intermediate_size, hidden_size, bias=False)

    def forward(self, x, **kwargs):
        return self.down_proj(swiglu(self.gate_proj(x), self.up_proj(x)))


class NeuralAttentionSearchLinearAttnGDNBlock(nn.Module):
    """modeling_natsl_attn_gdn.py:55-149.  The reference passes ``outputs_are_wighted=`` to a layer whose parameter is
    spelt ``outputs_are_weighted`` (the value is swallowed by **kwargs and the layer default True applies) and gives
    ``compute_dnats_for_invalid_blocks_linear_att`` the value of the softmax-branch flag (:97, :101); both are kept."""

    def __init__(self, config: NeuralAttentionSearchLineraAttnGDNConfig, layer_idx: int):
        super().__init__()
        self.config, self.layer_idx = config, layer_idx
        if layer_idx in config.gdn_layers:
            raise NotImplementedError("plain Gated DeltaNet layers (gdn_layers) are not built; use gdn_layers=[]")
        self.attn_norm = RMSNorm(config.hidden_size, eps=config.norm_eps)
        self.attn = NeuralAttentionSearchLinearAttnGDN(
            hidden_size=config.hidden_size, expand_v=config.expand_v, head_dim=config.head_dim,
            num_heads=config.num_heads, num_attn_heads=config.num_attn_heads, num_v_heads=config.num_v_heads,
            n_ops=config.n_ops, num_nats_head=config.num_nats_head, nats_block_size=config.nats_block_size,
            nats_block_agg_type=config.nats_block_agg_type, nats_sample_strategy=config.nats_sample_strategy,
            ops_for_incomplete_chunks=config.ops_for_incomplete_chunks, use_gate=config.use_gate,
            use_short_conv=config.use_short_conv, allow_neg_eigval=config.allow_neg_eigval, conv_size=config.conv_size,
            conv_bias=config.conv_bias, outputs_are_wighted=config.outputs_are_wighted, attn_qk_norm=config.attn_qk_norm,
            attn_with_short_conv=config.attn_with_short_conv,
            compute_dnats_for_invalid_blocks_attn=config.compute_dnats_for_invalid_blocks_attn,
            compute_dnats_for_invalid_blocks_linear_att=config.compute_dnats_for_invalid_blocks_attn,
            incomplete_block_start_with_ht=config.incomplete_block_start_with_ht,
            decay_for_non_gdn_blocks=config.decay_for_non_gdn_blocks, attn_rope_theta=config.attn_rope_theta,
            attn_apply_pos_encoding=config.attn_apply_pos_encoding,
            attn_max_position_embeddings=config.attn_max_position_embeddings, norm_eps=config.norm_eps, layer_idx=layer_idx)
        self.mlp_norm = RMSNorm(config.hidden_size, eps=config.norm_eps)
        self.mlp = GatedMLP(config.hidden_size, config.hidden_ratio, config.intermediate_size, config.hidden_act,
                            config.fuse_swiglu)

    def forward(self, hidden_states, attention_mask=None, past_key_values=None, use_cache=False, output_attentions=False,
                **kwargs):
        residual = hidden_states
        hidden_states = self.attn_norm(hidden_states)
        hidden_states, attentions, past_key_values = self.attn(
            hidden_states=hidden_states, attention_mask=attention_mask, past_key_values=past_key_values,
            use_cache=use_cache, output_attentions=output_attentions, **kwargs)
        hidden_states, residual = self.mlp_norm(hidden_states, residual, True)      # fused pre-norm residual, :138-139
        hidden_states = residual + self.mlp(hidden_states, **kwargs)
        return hidden_states, attentions, past_key_values


def init_weights(model: nn.Module, initializer_range: float = 0.02) -> None:
    """modeling_natsl_attn_gdn.py:163-191: Linear / Conv1d / Embedding weights ~ N(0, initializer_range), biases zero;
    A_log = log U(0, 16); dt_bias = softplus^-1 of exp(U * (ln 0.1 - ln 0.001) + ln 0.001) clamped at 1e-4."""
    for module in model.modules():
        if isinstance(module, NeuralAttentionSearchLinearAttnGDN):
            with torch.no_grad():
                module.A_log.copy_(nn.init.uniform_(module.A_log, a=0, b=16).log())
                dt = torch.exp(nn.init.uniform_(module.dt_bias) * (math.log(0.1) - math.log(0.001)) + math.log(0.001)).clamp(min=1e-4)
                module.dt_bias.copy_(dt + torch.log(-torch.expm1(-dt)))
        elif isinstance(module, (nn.Linear, nn.Conv1d)):
            nn.init.normal_(module.weight, mean=0.0, std=initializer_range)
            if module.bias is not None:
                nn.init.zeros_(module.bias)
        elif isinstance(module, nn.Embedding):
            nn.init.normal_(module.weight, mean=0.0, std=initializer_range)


class NeuralAttentionSearchLinearAttnGDNModel(nn.Module):
    """modeling_natsl_attn_gdn.py:220-320 (prefill / training; no cache)."""

    def __init__(self, config: NeuralAttentionSearchLineraAttnGDNConfig):
        super().__init__()
        self.config = config
        self.padding_idx, self.vocab_size = config.pad_token_id, config.vocab_size
        self.embeddings = nn.Embedding(config.vocab_size, config.hidden_size, self.padding_idx)
        self.layers = nn.ModuleList([NeuralAttentionSearchLinearAttnGDNBlock(config, i)
                                     for i in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, eps=config.norm_eps)

    def forward(self, input_ids=None, attention_mask=None, inputs_embeds=None, past_key_values=None, use_cache=None,
                **kwargs):
        if (input_ids is None) == (inputs_embeds is None):
            raise ValueError("You have to specify exactly one of input_ids and inputs_embeds")
        if past_key_values is not None or use_cache:
            raise NotImplementedError("decoding with a cache is not built (prefill and training only)")
        hidden_states = self.embeddings(input_ids) if inputs_embeds is None else inputs_embeds
        for layer in self.layers:
            hidden_states, _, _ = layer(hidden_states, attention_mask=attention_mask, **kwargs)
        return self.norm(hidden_states)


class _ChunkedLinearCrossEntropy(torch.autograd.Function):
    """mean next-token cross entropy of (hidden @ W^T) without keeping the [tokens, vocab] logits: the tokens are
    processed in slices, and the gradients with respect to hidden and W are formed slice by slice in the forward (the
    role of the reference's FusedLinearCrossEntropyLoss, modeling_natsl_attn_gdn.py:474-491)."""

    @staticmethod
    def forward(ctx, hidden, weight, labels, ignore_index, slice_tokens):
        n = hidden.shape[0]
        valid = labels != ignore_index
        denom = valid.sum().clamp_min(1).float()
        d_hidden = torch.empty_like(hidden)
        d_weight = torch.zeros_like(weight, dtype=torch.float32)
        loss = torch.zeros((), dtype=torch.float32, device=hidden.device)
        use_kernel = (hidden.is_cuda and hidden.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
                      and weight.shape[0] % 8 == 0)
        for s in range(0, n, slice_tokens):
            h, y = hidden[s:s + slice_tokens], labels[s:s + slice_tokens]
            if use_kernel:
                # one kernel turns the slice's logits into their gradient in place (unscaled: 1/denom is applied to the
                # two products below, on the device) and returns the rows' losses
                p = h @ weight.t()
                rows_loss = torch.empty(p.shape[0], dtype=torch.float32, device=p.device)
                _lib.call("natsl_xent_rows", p.data_ptr(), y.long().contiguous().data_ptr(), rows_loss.data_ptr(), p.shape[0],
                          p.shape[1], int(ignore_index), 1.0, current_stream_ptr(p.device))
                loss += rows_loss.sum()
                d_hidden[s:s + slice_tokens] = ((p @ weight).float() / denom).to(hidden.dtype)
                d_weight += (p.t() @ h).float()
                continue
            logits = (h @ weight.t()).float()
            lse = torch.logsumexp(logits, -1)
            ok = y != ignore_index
            tgt = logits.gather(1, y.clamp_min(0)[:, None])[:, 0]
            loss += ((lse - tgt) * ok).sum()
            p = torch.softmax(logits, -1)
            p.scatter_add_(1, y.clamp_min(0)[:, None], -torch.ones_like(tgt)[:, None])
            p = (p * (ok[:, None] / denom)).to(hidden.dtype)
            d_hidden[s:s + slice_tokens] = p @ weight
            d_weight += (p.t() @ h).float()
        if use_kernel:
            d_weight /= denom
        ctx.save_for_backward(d_hidden, d_weight.to(weight.dtype))
        return loss / denom

    @staticmethod
    def backward(ctx, dloss):
        d_hidden, d_weight = ctx.saved_tensors
        return d_hidden * dloss, d_weight * dloss, None, None, None


class NeuralAttentionSearchLinearAttnGDNForCausalLM(nn.Module):
    """modeling_natsl_attn_gdn.py:323-509: ``forward(input_ids, labels=None, logits_to_keep=0)`` ->
    dict(loss, logits, attn_frac).  With labels under training the loss is computed without materialising the logits
    (``fuse_cross_entropy``) and ``logits`` is None, as in the reference."""

    def __init__(self, config: NeuralAttentionSearchLineraAttnGDNConfig):
        super().__init__()
        self.config = config
        self.model = NeuralAttentionSearchLinearAttnGDNModel(config)
        self.vocab_size = config.vocab_size
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        init_weights(self, config.initializer_range)
        if config.tie_word_embeddings:
            self.lm_head.weight = self.model.embeddings.weight

    def forward(self, input_ids=None, attention_mask=None, inputs_embeds=None, labels=None, logits_to_keep: Optional[int] = 0,
                **kwargs):
        hidden_states = self.model(input_ids=input_ids, attention_mask=attention_mask, inputs_embeds=inputs_embeds, **kwargs)
        fused = self.config.fuse_cross_entropy and self.training and labels is not None
        loss, logits = None, None
        if not fused:
            logits = self.lm_head(hidden_states if logits_to_keep is None else hidden_states[:, -logits_to_keep:])
        if labels is not None:
            ignore = -100
            labels = torch.cat((labels[..., 1:], torch.full_like(labels[:, :1], ignore)), 1)      # shift, :490
            if fused:
                loss = _ChunkedLinearCrossEntropy.apply(hidden_states.flatten(0, 1), self.lm_head.weight, labels.flatten(),
                                                        ignore, 8192)
            else:
                loss = F.cross_entropy(logits.flatten(0, 1).float(), labels.flatten(), ignore_index=ignore)
        attn_frac = torch.mean(torch.stack([layer.attn.attn_fraction.float().reshape(-1).mean() for layer in self.model.layers]))
        return dict(loss=loss, logits=logits, attn_frac=attn_frac)
