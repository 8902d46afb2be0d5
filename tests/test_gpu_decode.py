"""GPU test (-m gpu) of decoding with a cache: prefill + token-by-token steps must reproduce the one-shot forward of the
whole sequence (the self-consistency check of the reference's own layer script,
src/nats/layers/natsl_attn_gdn.py:669-777: prefill, then the last tokens decoded one by one)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _layer(mode="all", seed=0):
    from neuralattentionsearchlinear_b200 import NeuralAttentionSearchLinearAttnGDN
    torch.manual_seed(seed)
    layer = NeuralAttentionSearchLinearAttnGDN(hidden_size=256, expand_v=1, head_dim=64, num_heads=4, num_attn_heads=4,
                                               nats_block_size=64, ops_for_incomplete_chunks=mode, layer_idx=0,
                                               decay_for_non_gdn_blocks=True, norm_eps=1e-6)
    return layer.cuda().bfloat16().eval()


def _close(got, ref, what, tol=2e-2):
    got, ref = got.float().cpu(), ref.float().cpu()
    assert torch.isfinite(got).all(), what
    s = max(1.0, float(ref.abs().max()))
    err = (got - ref).abs()
    assert bool((err <= tol * s + tol * ref.abs()).all()), f"{what}: max err {err.max().item():.4g} (ref max {ref.abs().max().item():.4g})"


@pytest.mark.parametrize("mode,T0,T,piece", [("all", 230, 300, 1), ("all", 256, 330, 5), ("gated_delta_net", 200, 280, 1),
                                             ("all", 64, 200, 7)])
def test_prefill_then_decode_matches_one_shot(mode, T0, T, piece):
    from neuralattentionsearchlinear_b200 import NAtSCache
    layer = _layer(mode, seed=T0)
    x = torch.randn(2, T, 256, generator=torch.Generator().manual_seed(T)).bfloat16().cuda()
    with torch.no_grad():
        full, _, _ = layer(x)
        cache = NAtSCache()
        outs = [layer(x[:, :T0], past_key_values=cache, use_cache=True)[0]]
        t = T0
        while t < T:
            n = min(piece, T - t)
            outs.append(layer(x[:, t:t + n], past_key_values=cache, use_cache=True)[0])
            t += n
    got = torch.cat(outs, 1)
    assert cache[0].n_tokens == T and cache[0].block_types.shape[1] == T // 64
    _close(got[:, :T0], full[:, :T0], "prefill part")
    _close(got[:, T0:], full[:, T0:], "decoded part")


def test_short_prompt_decodes_from_an_empty_cache():
    from neuralattentionsearchlinear_b200 import NAtSCache
    layer = _layer("all", seed=3)
    T = 150
    x = torch.randn(1, T, 256, generator=torch.Generator().manual_seed(9)).bfloat16().cuda()
    with torch.no_grad():
        full, _, _ = layer(x)
        cache = NAtSCache()
        outs = [layer(x[:, t:t + 10], past_key_values=cache, use_cache=True)[0] for t in range(0, T, 10)]
    _close(torch.cat(outs, 1), full, "decoded from scratch")


def _mamba_layer(mode, nbs, head_dim, expand_v, seed):
    from neuralattentionsearchlinear_b200 import NeuralAttentionSearchLinearAttnMamba
    torch.manual_seed(seed)
    layer = NeuralAttentionSearchLinearAttnMamba(hidden_size=256, expand_v=expand_v, head_dim=head_dim, num_heads=256 // head_dim,
                                                 num_attn_heads=256 // head_dim, nats_block_size=nbs,
                                                 ops_for_incomplete_chunks=mode, layer_idx=0, norm_eps=1e-6)
    return layer.cuda().bfloat16().eval()


@pytest.mark.parametrize("mode,nbs,head_dim,expand_v,T0,T,piece", [("all", 64, 64, 1, 230, 300, 1), ("mamba", 64, 64, 1, 192, 270, 3),
                                                                    ("all", 128, 128, 0.5, 300, 400, 1)])
def test_mamba_layer_prefill_then_decode_matches_one_shot(mode, nbs, head_dim, expand_v, T0, T, piece):
    """The same self-consistency check for the Mamba2 layer (src/nats/layers/natsl_attn_mamba2.py:520-590)."""
    from neuralattentionsearchlinear_b200 import NAtSCache
    layer = _mamba_layer(mode, nbs, head_dim, expand_v, seed=T0)
    x = torch.randn(2, T, 256, generator=torch.Generator().manual_seed(T)).bfloat16().cuda()
    with torch.no_grad():
        full = layer(x)
        cache = NAtSCache()
        outs = [layer(x[:, :T0], cache_params=cache, use_cache=True)]
        t = T0
        while t < T:
            n = min(piece, T - t)
            outs.append(layer(x[:, t:t + n], cache_params=cache, use_cache=True))
            t += n
    got = torch.cat(outs, 1)
    assert cache[0].n_tokens == T and cache[0].block_types.shape[1] == T // nbs
    _close(got[:, :T0], full[:, :T0], "prefill part")
    _close(got[:, T0:], full[:, T0:], "decoded part")


@pytest.mark.parametrize("rule,decay,T,piece,dtype", [("gdn", True, 200, 1, torch.float32), ("gdn", False, 192, 5, torch.float32),
                                                      ("mamba", True, 200, 1, torch.float32), ("mamba", False, 256, 7, torch.float32),
                                                      ("mamba", True, 150, 3, torch.bfloat16), ("gdn", True, 150, 3, torch.bfloat16)])
def test_recurrent_step_op_matches_the_token_recurrence(rule, decay, T, piece, dtype):
    """The step entry of the linear branch fed piece by piece from empty states against the oracle's token recurrence over
    the whole sequence: outputs of every token, and the block-start state a decoder continues from."""
    from neuralattentionsearchlinear_b200 import _lib, _ops
    from oracle import gdn as ogdn
    from oracle import tables as otab
    from tests.helpers import synth_gdn_inputs, synth_mamba_inputs
    B, H, HN, K, V, nbs = 2, 4, 2, 64, 64, 64
    if rule == "gdn":
        q, k, v, g, beta, _ = synth_gdn_inputs(B, T, H, K, V, seed=T, dtype=dtype, normalize_qk=False)
        scale, l2 = K ** -0.5, True
    else:
        q, k, v, g, _ = synth_mamba_inputs(B, T, H, K, V, seed=T, dtype=dtype)
        beta, scale, l2 = None, 1.0, False
    NB = -(-T // nbs)
    raw = otab.synth_types(B, NB, HN, 0.5, seed=T + 1, force_last=False)
    types = raw.clone()
    if T % nbs:
        types[:, -1] = 1
    f = lambda x: None if x is None else x.float()
    o_ref, _, start_ref = ogdn.linear_recurrent(f(q), f(k), f(v), g, f(beta), types[..., 1], nbs=nbs, scale=scale, decay=decay,
                                                use_l2norm=l2, rule=rule, return_block_start=True)
    dev = torch.device("cuda")
    c = lambda x: None if x is None else x.to(dev)
    state = torch.zeros(B, H, K, V, device=dev)
    start = torch.zeros(B, H, K, V, device=dev)
    g_block = torch.zeros(B, H, device=dev)
    code = _lib.RULE_GDN if rule == "gdn" else _lib.RULE_MAMBA
    outs, t = [], 0
    while t < T:
        t_off = t % nbs
        n = min(piece, T - t, nbs - t_off)
        ends = t_off + n == nbs
        ty = raw[:, t // nbs:t // nbs + 1] if ends else torch.ones(B, 1, HN, 2)
        sl = slice(t, t + n)
        o, state, start = _ops.linear_recurrent_step(code, c(q[:, sl]), c(k[:, sl]), c(v[:, sl]), c(g[:, sl]),
                                                     None if beta is None else c(beta[:, sl]), c(ty), state, start, g_block,
                                                     t_off, nbs, scale, decay, l2)
        g_block = torch.zeros_like(g_block) if ends else g_block + c(g[:, sl]).float().sum(1)
        outs.append(o)
        t += n
    tol = 2e-4 if dtype == torch.float32 else 1e-2
    _close(torch.cat(outs, 1), o_ref, f"{rule} step outputs", tol)
    _close(start, start_ref, f"{rule} block-start state", tol)
