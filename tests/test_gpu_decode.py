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
