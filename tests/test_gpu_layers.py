"""The drop-in layer modules on the GPU: output mixing kernel vs its formula, and both layers' forward
against the oracle ops applied to the layer's own projected tensors (same selection, same inputs)."""
import pytest
import torch

from oracle import attn as oattn
from oracle import gdn as ogdn
from tests.helpers import assert_close

pytestmark = pytest.mark.gpu


def _mix_reference(x1, x2, g, xw, w1, w2, eps):
    x1, x2, g, xw = x1.float(), x2.float(), g.float(), xw.float()
    r1 = torch.rsqrt(x1.pow(2).mean(-1, keepdim=True) + eps)
    r2 = torch.rsqrt(x2.pow(2).mean(-1, keepdim=True) + eps)
    y = x1 * r1 * w1.float() * xw[..., :1] + x2 * r2 * w2.float() * xw[..., 1:]
    return y * g * torch.sigmoid(g)


@pytest.mark.parametrize("D", [64, 128, 256])
def test_norm_gate_mix_kernel(D):
    from neuralattentionsearchlinear_b200.modules import FusedMultiInputRMSNormGated
    gen = torch.Generator().manual_seed(D)
    x1 = torch.randn(3, 70, 4, D, generator=gen).bfloat16().cuda()
    x2 = torch.randn(3, 70, 4, D, generator=gen).bfloat16().cuda()
    g = torch.randn(3, 70, 4, D, generator=gen).bfloat16().cuda()
    xw = torch.rand(3, 70, 4, 2, generator=gen).bfloat16().cuda()
    m = FusedMultiInputRMSNormGated(D, eps=1e-5).cuda()
    m.weight1.data = torch.randn(D, generator=gen).cuda()
    m.weight2.data = torch.randn(D, generator=gen).cuda()
    y = m(x1, x2, g, xw)
    ref = _mix_reference(x1.cpu(), x2.cpu(), g.cpu(), xw.cpu(), m.weight1.data.cpu(), m.weight2.data.cpu(), 1e-5)
    assert_close(y, ref, 1e-2, "norm_gate_mix")


def _oracle_from_projection(layer, p, rule):
    f = lambda x: x.detach().float().cpu()
    types = f(p['types'])
    T = p['q'].shape[1]
    nbs = layer.nats_block_size
    if rule == "gdn":
        o_l, _ = ogdn.linear_chunk(f(p['q']), f(p['k']), f(p['v']), f(p['g']), f(p['beta']), types[..., 1], nbs=nbs,
                                   decay=layer.decay_for_non_gdn_blocks)
    else:
        o_l, _ = ogdn.linear_chunk(f(p['q']), f(p['k']), f(p['v']), f(p['g']), None, types[..., 1], nbs=nbs, scale=1.0,
                                   decay=layer.decay_for_non_mamba_blocks, use_l2norm=False, rule="mamba")
    own = layer.ops_for_incomplete_chunks in ('all', 'attn')
    mask = oattn.attn_mask(types[..., 0], T, nbs, p['q_attn'].shape[2], own_chunk=own)
    o_a, _ = oattn.attn_sdpa(f(p['q_attn']), f(p['k_attn']), f(p['v_attn']), mask)
    return o_l, o_a


def test_gdn_layer_forward_matches_oracle_ops():
    import neuralattentionsearchlinear_b200 as nat
    torch.manual_seed(0)
    layer = nat.NeuralAttentionSearchLinearAttnGDN(hidden_size=256, expand_v=1, head_dim=64, num_heads=4,
                                                   num_attn_heads=4, nats_block_size=64).cuda().bfloat16().eval()
    x = torch.randn(2, 320, 256, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        y, _, _ = layer(x)
        p = layer.project(x)
        o_l, o_a = _oracle_from_projection(layer, p, "gdn")
        y_ref = layer.mix(x, o_l.cuda().bfloat16(), o_a.cuda().bfloat16(), p['o_weights'])
    assert y.shape == x.shape and torch.isfinite(y.float()).all()
    assert_close(y, y_ref, 3e-2, "gdn layer output")
    assert 0.0 < float(layer.attn_fraction.mean()) < 1.0
    layer.train()
    with torch.no_grad():
        y2, _, _ = layer(x)
    assert_close(y2, y_ref, 3e-2, "gdn layer output (training-mode op)")


def test_mamba_layer_forward_matches_oracle_ops():
    import neuralattentionsearchlinear_b200 as nat
    torch.manual_seed(1)
    layer = nat.NeuralAttentionSearchLinearAttnMamba(hidden_size=256, expand_v=0.5, head_dim=128, num_heads=2,
                                                     num_attn_heads=2, nats_block_size=128,
                                                     ops_for_incomplete_chunks='all').cuda().bfloat16().eval()
    x = torch.randn(1, 512, 256, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        y = layer(x)
        p = layer.project(x)
        o_l, o_a = _oracle_from_projection(layer, p, "mamba")
        y_ref = layer.mix(x, o_l.cuda().bfloat16(), o_a.cuda().bfloat16(), p['o_weights'])
    assert y.shape == x.shape
    assert_close(y, y_ref, 3e-2, "mamba layer output")


def test_layers_refuse_unbuilt_paths():
    import neuralattentionsearchlinear_b200 as nat
    layer = nat.NeuralAttentionSearchLinearAttnGDN(hidden_size=128, expand_v=1, head_dim=64, num_heads=2,
                                                   num_attn_heads=2).cuda().bfloat16()
    x = torch.randn(1, 32, 128, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(NotImplementedError):
        layer(x)
    with pytest.raises(ValueError):                      # a cache needs the layer's index
        layer(torch.randn(1, 128, 128, device="cuda", dtype=torch.bfloat16), past_key_values=nat.NAtSCache())
    mamba = nat.NeuralAttentionSearchLinearAttnMamba(hidden_size=128, expand_v=1, head_dim=64, num_heads=2,
                                                     num_attn_heads=2).cuda().bfloat16()
    with pytest.raises(ValueError):
        mamba(torch.randn(1, 128, 128, device="cuda", dtype=torch.bfloat16), cache_params=nat.NAtSCache())
    with pytest.raises(NotImplementedError):             # fewer than 64 tokens without a cache
        mamba(x)


@pytest.mark.parametrize("rule", ["gdn", "mamba"])
def test_ops_replay_from_a_cuda_graph(rule):
    """Both ops can be captured into a CUDA graph after one eager call (they fork and join their side streams with
    events, allocate through torch and never synchronise the host); a replay on new input contents equals the eager op."""
    import neuralattentionsearchlinear_b200 as nat
    from oracle import tables as otab
    from tests.helpers import synth_gdn_inputs, synth_mamba_inputs
    B, T, H, K, V, nbs = 2, 512, 4, 128, 128, 64
    dev = torch.device("cuda")

    def inputs(seed):
        if rule == "gdn":
            q, k, v, g, beta, _ = synth_gdn_inputs(B, T, H, K, V, seed=seed)
        else:
            q, k, v, g, _ = synth_mamba_inputs(B, T, H, K, V, seed=seed)
            beta = torch.zeros(B, T, H).bfloat16()
        types = otab.synth_types(B, T // nbs, H, 0.3, seed=seed + 1)
        return [x.to(dev) for x in (q, k, v, g, beta, types)]

    def op(q, k, v, g, beta, types):
        if rule == "gdn":
            return nat.nats_mixed_attn_gdn(q, k, v, q, k, v, None, g, beta, types, None, nats_block_size=nbs,
                                           ops_for_incomplete_chunks="all", output_final_state_gated_delta=True,
                                           decay_for_non_gdn_blocks=True)
        return nat.nats_mixed_attn_mamba(q, k, v, q, k, v, None, g, types, None, scale_attn=K ** -0.5, nats_block_size=nbs,
                                         ops_for_incomplete_chunks="all", output_final_state_mamba=True,
                                         decay_for_non_mamba_blocks=True)

    static = inputs(1)
    with torch.no_grad():
        op(*static)                                        # eager warm-up (per-device look-ups happen here)
        torch.cuda.synchronize()
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                outs = op(*static)
        torch.cuda.current_stream().wait_stream(side)
        fresh = inputs(7)
        for dst, src in zip(static, fresh):
            dst.copy_(src)
        graph.replay()
        torch.cuda.synchronize()
        ref = op(*fresh)
        torch.cuda.synchronize()
    for a, b in zip(outs, ref):
        assert torch.equal(a, b)
    from neuralattentionsearchlinear_b200 import _lib
    assert _lib.load().natsl_device_status() == 0
