"""Cached forward shared by the two NAtSL layers: prefill into an empty ``NAtSLayerCache`` with the chunk kernels, then
steps of fewer than ``nats_block_size`` tokens with the token recurrence (re-roll at block ends) and masked attention over
the cached keys (src/nats/layers/natsl_attn_gdn.py:389-410, 576-650; src/nats/layers/natsl_attn_mamba2.py:330-352, 520-590).

A layer plugs in through four hooks:
  ``layer.project(hidden, want_conv_state=True)``        everything the chunk op consumes (+ ``types_raw``, ``conv_state``)
  ``layer.project_qkv(hidden, conv_state, want_conv_state)`` the same without the selection, for a few new tokens
  ``layer.select(pooled)``                               block-mean layer input -> sampled 0/1 block types
  ``layer._ops_for_cache()``                             dict(chunk=(p, T) -> (o_lin, o_attn, state, block-start state),
                                                              step=(p, cache, mask, types, t_off) -> the same four)
"""
from __future__ import annotations

import torch


@torch.no_grad()
def forward_cached(layer, hidden_states: torch.Tensor, cache_container):
    """-> (o_linear, o_attn, o_weights) for ``hidden_states`` [B, T, D]; updates the layer's cache."""
    if layer.layer_idx is None:
        raise ValueError("a layer used with a cache needs its layer_idx")
    if layer.ops_for_incomplete_chunks == 'attn' or not layer.incomplete_block_start_with_ht:
        raise NotImplementedError("decoding is built for the modes in which the linear branch covers the own block")
    hooks = layer._ops_for_cache()
    cache = cache_container.layer(layer.layer_idx, layer.nats_block_size)
    B, T, _ = hidden_states.shape
    nbs = layer.nats_block_size
    own_attn = layer.ops_for_incomplete_chunks == 'all'
    dev = hidden_states.device
    if cache.n_tokens == 0 and T >= 64:
        p = layer.project(hidden_states, want_conv_state=True)
        o_lin, o_attn, ht, start = hooks['chunk'](p, T)
        r, n_done = T % nbs, T // nbs
        cache.append_kv(p['k_attn'].contiguous(), p['v_attn'].contiguous())
        if n_done:
            cache.append_types(p['types_raw'][:, :n_done].contiguous())
        cache.state_block_start = start
        cache.state = start.clone() if r == 0 else ht
        H = p['g'].shape[2]
        cache.g_block = p['g'][:, T - r:].float().sum(1) if r else torch.zeros(B, H, device=dev)
        cache.pool_sum = hidden_states[:, T - r:].float().sum(1) if r else torch.zeros(B, hidden_states.shape[2], device=dev)
        cache.conv_state = p['conv_state']
        cache.n_tokens = T
        return o_lin, o_attn, p['o_weights']
    if T >= 64:
        raise NotImplementedError("continuing a prefill of 64 tokens or more into a filled cache is not built; "
                                  "feed the continuation in pieces of fewer than 64 tokens")
    if cache.n_tokens == 0:                                 # a short prompt: start from empty states
        H, K, V = layer.num_heads, layer.head_k_dim, layer.head_v_dim
        cache.state = torch.zeros(B, H, K, V, device=dev)
        cache.state_block_start = torch.zeros(B, H, K, V, device=dev)
        cache.g_block = torch.zeros(B, H, device=dev)
        cache.pool_sum = torch.zeros(B, hidden_states.shape[2], device=dev)
    outs_l, outs_a, weights = [], [], []
    a = 0
    while a < T:
        t_off = cache.n_tokens % nbs
        b_ = min(T, a + (nbs - t_off))                      # a piece never crosses a block boundary
        hs = hidden_states[:, a:b_]
        n = b_ - a
        completes = (t_off + n) == nbs
        cache.pool_sum = cache.pool_sum + hs.float().sum(1)
        if completes:
            pooled = (cache.pool_sum / nbs).to(hs.dtype)[:, None, :]
            types_new = layer.select(pooled)                 # decided once the block's last token is known
        else:
            types_new = torch.ones(B, 1, layer.num_nats_head, layer.n_ops, device=dev, dtype=hs.dtype)
        p = layer.project_qkv(hs, conv_state=cache.conv_state, want_conv_state=True)
        cache.append_kv(p['k_attn'].contiguous(), p['v_attn'].contiguous())
        msk = cache.generate_msk(n, layer.num_attn_heads, own_chunk=own_attn)
        o_lin, o_attn, state, start = hooks['step'](p, cache, msk, types_new, t_off)
        cache.state, cache.state_block_start = state, start
        if completes:
            cache.append_types(types_new)
            cache.g_block = torch.zeros_like(cache.g_block)
            cache.pool_sum = torch.zeros_like(cache.pool_sum)
        else:
            cache.g_block = cache.g_block + p['g'].float().sum(1)
        cache.conv_state = p['conv_state']
        cache.n_tokens += n
        outs_l.append(o_lin)
        outs_a.append(o_attn)
        weights.append(p['o_weights'])
        a = b_
    o_w = torch.cat(weights, 1) if weights[0] is not None else None
    return torch.cat(outs_l, 1), torch.cat(outs_a, 1), o_w
