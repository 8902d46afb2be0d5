"""GPU parity tests (-m gpu) of the pieces around the kernels: the device-side selection decisions against the oracle,
the two extra states of the chunk-inference ops, and the long-context Mamba2 configuration at its real shape."""
import pytest
import torch

from oracle import attn as oattn
from oracle import gdn as ogdn
from oracle import tables as otab
from tests.helpers import assert_close, synth_gdn_inputs, synth_mamba_inputs

pytestmark = pytest.mark.gpu
TOL = 1e-2


@pytest.fixture(scope="module")
def nat():
    import neuralattentionsearchlinear_b200 as n
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    return n


# ------------------------------------------------------------------------------------------------ selection decisions
def _decide_on_device(logits):
    """What the layers do on the device (natsl_attn_gdn.py:47-61, 553 of the reference): hard_softmax, last block forced."""
    from neuralattentionsearchlinear_b200.modules import hard_softmax
    types = hard_softmax(logits.cuda()).clone()
    types[:, -1] = 1
    return types.cpu()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_selection_decisions_bit_exact(nat, dtype):
    """Seeded logits (the benchmark's distribution) and exact ties: the 0/1 decisions computed on the device equal the
    oracle's, bit for bit, and so do the tables built from them."""
    gen = torch.Generator().manual_seed(7)
    logits = torch.randn(8, 64, 16, 2, generator=gen)
    logits[..., 0] -= 0.95                                     # about 25 % softmax blocks
    logits[1, :, :, 1] = logits[1, :, :, 0]                    # exact ties: the first operation wins (torch.max)
    logits[2, ::2, :, 0] = 0.0
    logits[2, ::2, :, 1] = 0.0
    logits = logits.to(dtype)
    got = _decide_on_device(logits)
    ref = otab.force_last_block(otab.hard_softmax(logits))
    assert torch.equal(got.float(), ref.float())
    assert set(got.float().unique().tolist()) <= {0.0, 1.0}
    assert bool((got[1, :-1, :, 0] == 1).all()) and bool((got[1, :-1, :, 1] == 0).all())
    tb = nat.build_selection_tables(got.cuda(), 4096, 64)
    rt = otab.build_tables(ref, 4096, 64)
    assert torch.equal(tb.indices.cpu().long(), rt["indices"]) and torch.equal(tb.n_blocks.cpu().long(), rt["n_blocks"])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_selection_decisions_near_ties(nat, dtype):
    """Pairs of logits one unit in the last place apart, at many magnitudes, in both orders.  Whether the two rounded
    probabilities tie (then the first operation wins, torch.max) depends on the last-place rounding of the exponential
    inside softmax, which differs between the CPU and the CUDA math libraries; the reference itself runs this softmax
    on the device.  So the oracle pins these cases only up to that rounding: every device decision must be one-hot and
    admissible (the larger logit, or the first operation on a tie of the probabilities), and away from the
    one-unit-apart cases it is bit-exact (previous test).  In bf16 the rounded probabilities tie the same way on both
    sides and the decisions are equal."""
    base = torch.cat([torch.linspace(-8, 8, 4001), torch.logspace(-6, 1, 2000), -torch.logspace(-6, 1, 2000)]).to(dtype)
    if dtype == torch.float32:
        up = torch.nextafter(base, torch.full_like(base, 1e9))
    else:
        bits = base.view(torch.int16).int()
        up = torch.where(base >= 0, bits + 1, bits - 1).to(torch.int16).view(torch.bfloat16)
        up = torch.where(base == 0, torch.full_like(base, 1e-30), up)
    n = base.numel()
    logits = torch.stack([torch.stack([base, up], -1), torch.stack([up, base], -1)], 0).view(2, n, 1, 2)
    logits = torch.cat([logits, logits[:, :1]], 1)             # one more block: the forced last block is not a test case
    got = _decide_on_device(logits).float()[:, :-1]
    ref = otab.force_last_block(otab.hard_softmax(logits)).float()[:, :-1]
    assert bool((got.sum(-1) == 1).all()) and set(got.unique().tolist()) <= {0.0, 1.0}
    larger = logits[:, :-1].float().argmax(-1)
    picked = got.argmax(-1)
    assert bool(((picked == larger) | (picked == 0)).all()), "a decision is neither the larger logit nor a tie"
    if dtype == torch.bfloat16:
        assert torch.equal(got, ref)
    else:
        # the oracle (CPU softmax) is admissible in the same sense; the two may differ only on these near-ties
        picked_ref = ref.argmax(-1)
        assert bool(((picked_ref == larger) | (picked_ref == 0)).all())


# ------------------------------------------------------------------------------------------------ chunk-inference states
@pytest.mark.parametrize("rule,T,nbs,decay", [("gdn", 512, 64, True), ("gdn", 500, 64, True), ("gdn", 512, 128, False),
                                              ("mamba", 512, 64, True), ("mamba", 600, 128, True)])
def test_chunk_inference_states(nat, rule, T, nbs, decay):
    """The 4-tuple of the chunk-inference ops: final state and the state a decoder continues from
    (src/nats/ops/gated_delta_rule/chunk_fwd.py:178-206), against the token recurrence with re-roll."""
    B, H, K, V = 2, 4, 64, 64
    TN = -(-T // nbs)
    dev = torch.device("cuda")
    types_raw = otab.synth_types(B, TN, H, 0.4, seed=T + nbs, force_last=False)
    types = otab.force_last_block(types_raw.clone())
    op_last = types_raw[:, -1].clone()
    c = lambda x: None if x is None else x.to(dev)
    if rule == "gdn":
        q, k, v, g, beta, h0 = synth_gdn_inputs(B, T, H, K, V, seed=T, normalize_qk=False)
        o, oa, ht, start = nat.nats_mixed_attn_gdn_chunk_inference(
            c(q), c(k), c(v), c(q), c(k), c(v), c(h0), c(g), c(beta), c(types), c(op_last) if T % nbs == 0 else None, None,
            nats_block_size=nbs, ops_for_incomplete_chunks="all", output_final_state_gated_delta=True,
            decay_for_non_gdn_blocks=decay)
        kw = dict(nbs=nbs, h0=h0.float(), decay=decay, use_l2norm=True, rule="gdn")
        args = (q.float(), k.float(), v.float(), g, beta.float())
    else:
        q, k, v, g, h0 = synth_mamba_inputs(B, T, H, K, V, seed=T)
        o, oa, ht, start = nat.nats_mixed_attn_mamba_chunk_inference(
            c(q), c(k), c(v), c(q), c(k), c(v), c(h0), c(g), c(types), c(op_last) if T % nbs == 0 else None, None,
            scale_lattn=1.0, nats_block_size=nbs, ops_for_incomplete_chunks="all", output_final_state_mamba=True,
            decay_for_non_mamba_blocks=decay)
        kw = dict(nbs=nbs, scale=1.0, h0=h0.float(), decay=decay, use_l2norm=False, rule="mamba")
        args = (q.float(), k.float(), v.float(), g, None)
    o_ref, fin_ref = ogdn.linear_recurrent(*args, types[..., 1], **kw)
    # the state the decoder continues from follows the sampled type of the last block, not the forced one
    _, _, start_ref = ogdn.linear_recurrent(*args, types_raw[..., 1] if T % nbs == 0 else types[..., 1],
                                            return_block_start=True, **kw)
    assert_close(o, o_ref, TOL, "o")
    assert_close(ht, fin_ref, TOL, "final state")
    assert_close(start, start_ref, TOL, "block-start state")


# ------------------------------------------------------------------------------------------------ long context, real shape
def test_mamba_long_context_real_shape(nat):
    """B=1, T=65536, H=32, state dim 128, head dim 64, block 256, ~10 % softmax blocks: the whole layer op runs on the
    device; heads 0-1 of the linear branch and three 128-query windows of the softmax branch (first, middle, last)
    are compared with the oracle."""
    T, H, K, V, nbs = 65536, 32, 128, 64, 256
    hs = 2
    q, k, v, g, _ = synth_mamba_inputs(1, T, H, K, V, seed=4)
    types = otab.synth_types(1, T // nbs, H, 0.10, seed=5)
    dev = torch.device("cuda")
    scale_attn = K ** -0.5
    o_m, o_a, ht = nat.nats_mixed_attn_mamba(q.to(dev), k.to(dev), v.to(dev), q.to(dev), k.to(dev), v.to(dev), None, g.to(dev),
                                             types.to(dev), None, scale_attn=scale_attn, nats_block_size=nbs,
                                             ops_for_incomplete_chunks="all", output_final_state_mamba=True,
                                             decay_for_non_mamba_blocks=True)
    from neuralattentionsearchlinear_b200 import _lib
    assert _lib.load().natsl_device_status() == 0
    sl = lambda x: x[:, :, :hs].float().contiguous()
    o_ref, fin_ref = ogdn.linear_chunk(sl(q), sl(k), sl(v), g[:, :, :hs].contiguous(), None, types[:, :, :hs, 1], nbs=nbs,
                                       scale=1.0, decay=True, use_l2norm=False, rule="mamba")
    assert_close(o_m[:, :, :hs], o_ref, TOL, "o_mamba (heads 0-1, T=65536)")
    assert_close(ht[:, :hs], fin_ref, TOL, "final state (heads 0-1)")
    for t0 in (0, T // 2, T - 128):
        mask = oattn.attn_mask_rows(types[:, :, :hs, 0], T, nbs, hs, t0, t0 + 128)
        oa_ref, _ = oattn.attn_sdpa(sl(q)[:, t0:t0 + 128], sl(k), sl(v), mask, scale_attn)
        assert_close(o_a[:, t0:t0 + 128, :hs], oa_ref, TOL, f"o_attn (queries {t0}..{t0 + 127})")
