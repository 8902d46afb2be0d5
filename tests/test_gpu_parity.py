"""GPU parity tests (-m gpu): the CUDA path, called through the C ABI, against the CPU oracle on
the same seeded inputs.  Integer tables and masks bit-exact; bf16 outputs within
rtol = atol = 1e-2 of the oracle evaluated in fp32 on the same bf16-rounded inputs."""
import os

import numpy as np
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


def _tables_equal(tb, ref, B, HN):
    assert torch.equal(tb.types_i.cpu().long(), ref["types_i"])
    assert torch.equal(tb.indices.cpu().long(), ref["indices"])
    assert torch.equal(tb.n_blocks.cpu().long(), ref["n_blocks"])
    assert torch.equal(tb.offsets.cpu().long(), ref["offsets"])
    assert torch.equal(tb.starting_h_idx.cpu().long(), ref["starting_h_idx"])
    assert torch.equal(tb.attn_n_iters.cpu().long(), ref["attn_n_iters"])
    assert torch.equal(tb.compact_chunk_indices().cpu().long(), ref["chunk_indices"])


@pytest.mark.parametrize("B,T,HN,nbs,p,dtype", [
    (1, 512, 2, 64, 0.4, torch.float32), (2, 512, 4, 64, 0.5, torch.bfloat16), (3, 1000, 3, 64, 0.25, torch.float32),
    (2, 1024, 2, 128, 0.3, torch.float16), (8, 4096, 16, 64, 0.25, torch.bfloat16), (1, 65536, 32, 256, 0.1, torch.float32),
    (2, 130, 2, 64, 0.5, torch.float32), (1, 64, 1, 64, 0.5, torch.float32), (1, 40000, 1, 64, 0.9, torch.float32)])
def test_tables_bit_exact(nat, B, T, HN, nbs, p, dtype):
    TN = -(-T // nbs)
    types = otab.synth_types(B, TN, HN, p, seed=B + T + HN, dtype=dtype)
    ref = otab.build_tables(types, T, nbs)
    tb = nat.build_selection_tables(types.cuda(), T, nbs, with_chunk_indices=True)
    _tables_equal(tb, ref, B, HN)


def test_tables_against_reference_generated_golden(nat, golden_dir):
    z = np.load(os.path.join(golden_dir, "tables_ref.npz"))
    for n in sorted({k.split("_")[0] for k in z.files}):
        B, T, HN, nbs = z[f"{n}_meta"].tolist()
        tb = nat.build_selection_tables(torch.from_numpy(z[f"{n}_types"]).cuda(), T, nbs, with_chunk_indices=True)
        for key, got in [("indices", tb.indices), ("n_blocks", tb.n_blocks), ("offsets", tb.offsets),
                         ("starting_h_idx", tb.starting_h_idx), ("attn_n_iters", tb.attn_n_iters),
                         ("chunk_indices", tb.compact_chunk_indices())]:
            assert np.array_equal(got.cpu().numpy().astype(np.int64), z[f"{n}_{key}"]), (n, key)


def test_tables_all_or_nothing(nat):
    for fill in (0.0, 1.0):
        types = torch.full((2, 8, 2, 2), fill)
        ref = otab.build_tables(types, 512, 64)
        tb = nat.build_selection_tables(types.cuda(), 512, 64, with_chunk_indices=True)
        _tables_equal(tb, ref, 2, 2)


@pytest.mark.parametrize("B,T,HQ,HN,nbs,own", [(2, 512, 4, 4, 64, True), (1, 700, 4, 2, 64, True), (2, 1024, 2, 2, 128, True),
                                                (1, 1500, 2, 1, 256, True), (2, 512, 4, 4, 64, False), (1, 1024, 2, 2, 128, False),
                                                (1, 100, 2, 2, 64, True)])
def test_dense_mask_bit_exact(nat, B, T, HQ, HN, nbs, own):
    from neuralattentionsearchlinear_b200 import _ops
    TN = -(-T // nbs)
    types = otab.synth_types(B, TN, HN, 0.4, seed=T + nbs)
    tb = nat.build_selection_tables(types.cuda(), T, nbs)
    got = _ops.attn_dense_mask(tb, HQ, own).cpu()
    ref = oattn.attn_mask(types[..., 0], T, nbs, HQ, own_chunk=own)
    assert torch.equal(got, ref)


@pytest.mark.parametrize("B,T,HQ,HKV,HN,DK,DV,nbs,own", [
    (2, 512, 4, 4, 4, 64, 64, 64, True), (1, 700, 4, 2, 2, 128, 128, 64, True), (2, 1024, 2, 2, 2, 64, 128, 128, True),
    (1, 1100, 2, 2, 1, 128, 64, 256, True), (2, 512, 4, 4, 4, 64, 64, 64, False), (1, 2048, 2, 2, 2, 128, 128, 64, True)])
def test_attention_forward(nat, B, T, HQ, HKV, HN, DK, DV, nbs, own, monkeypatch):
    from neuralattentionsearchlinear_b200 import _ops
    gen = torch.Generator().manual_seed(T + DK)
    q = torch.randn(B, T, HQ, DK, generator=gen).bfloat16()
    k = torch.randn(B, T, HKV, DK, generator=gen).bfloat16()
    v = torch.randn(B, T, HKV, DV, generator=gen).bfloat16()
    types = otab.synth_types(B, -(-T // nbs), HN, 0.3, seed=T)
    tb = nat.build_selection_tables(types.cuda(), T, nbs)
    o, lse = _ops.attn_fwd(q.cuda(), k.cuda(), v.cuda(), tb, DK ** -0.5, own)
    mask = oattn.attn_mask(types[..., 0], T, nbs, HQ, own_chunk=own)
    o_ref, lse_ref = oattn.attn_sdpa(q.float(), k.float(), v.float(), mask, DK ** -0.5)
    assert_close(o, o_ref, TOL, "o_attn")
    assert_close(lse, lse_ref, TOL, "lse")
    from neuralattentionsearchlinear_b200 import _lib
    assert _lib.load().natsl_device_status() == 0
    # the mma.sync comparison kernel realises the same function
    o2, lse2 = _ops.attn_fwd(q.cuda(), k.cuda(), v.cuda(), tb, DK ** -0.5, own, mma_sync=True)
    assert_close(o2, o_ref, TOL, "o_attn (mma.sync)")
    assert_close(lse2, lse_ref, TOL, "lse (mma.sync)")
    # the persistent form (optional) walks the same tiles in the same order with the same arithmetic: identical bits
    monkeypatch.setattr(_ops, "ATTN_PERSISTENT", not _ops.ATTN_PERSISTENT)
    o3, lse3 = _ops.attn_fwd(q.cuda(), k.cuda(), v.cuda(), tb, DK ** -0.5, own)
    assert _lib.load().natsl_device_status() == 0
    assert torch.equal(o3, o) and torch.equal(lse3, lse)


@pytest.mark.parametrize("DK,DV,nbs", [(128, 128, 64), (128, 64, 256), (64, 64, 128)])
def test_attention_growing_scores(nat, DK, DV, nbs):
    """Keys whose norm grows along the sequence: the running row maximum keeps rising by more than the lazy
    threshold, so the accumulator in tensor memory is rescaled many times; plus run-to-run and batch-subset
    bit-identity (no race between the rescale and the tensor core)."""
    from neuralattentionsearchlinear_b200 import _lib, _ops
    B, T, HQ, HKV = 3, 2048, 4, 2
    gen = torch.Generator().manual_seed(DK + nbs)
    ramp = (1.0 + 9.0 * torch.arange(T) / T).view(1, T, 1, 1)
    q = torch.randn(B, T, HQ, DK, generator=gen).bfloat16()
    k = (torch.randn(B, T, HKV, DK, generator=gen) * ramp).bfloat16()
    v = torch.randn(B, T, HKV, DV, generator=gen).bfloat16()
    types = otab.synth_types(B, T // nbs, HKV, 0.5, seed=nbs)
    tb = nat.build_selection_tables(types.cuda(), T, nbs)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    o, lse = _ops.attn_fwd(qc, kc, vc, tb, DK ** -0.5, True)
    mask = oattn.attn_mask(types[..., 0], T, nbs, HQ)
    o_ref, lse_ref = oattn.attn_sdpa(q.float(), k.float(), v.float(), mask, DK ** -0.5)
    assert_close(o, o_ref, TOL, "o_attn")
    assert_close(lse, lse_ref, TOL, "lse")
    o_again, _ = _ops.attn_fwd(qc, kc, vc, tb, DK ** -0.5, True)
    assert torch.equal(o, o_again)
    tb1 = nat.build_selection_tables(types[1:2].cuda().contiguous(), T, nbs)
    o_one, _ = _ops.attn_fwd(qc[1:2].contiguous(), kc[1:2].contiguous(), vc[1:2].contiguous(), tb1, DK ** -0.5, True)
    assert torch.equal(o[1:2], o_one)
    assert _lib.load().natsl_device_status() == 0


def test_attention_more_key_tiles_than_the_shared_list_holds(nat):
    """A long, densely selected sequence: the late query tiles walk more key tiles (≈ 150) than the per-CTA tile list
    in shared memory holds (128), so the descriptors past it are recomputed on the fly."""
    from neuralattentionsearchlinear_b200 import _lib, _ops
    B, T, HQ, HKV, DK, DV, nbs = 1, 10240, 1, 1, 128, 64, 64
    gen = torch.Generator().manual_seed(77)
    q = torch.randn(B, T, HQ, DK, generator=gen).bfloat16()
    k = torch.randn(B, T, HKV, DK, generator=gen).bfloat16()
    v = torch.randn(B, T, HKV, DV, generator=gen).bfloat16()
    types = otab.synth_types(B, T // nbs, 1, 0.9, seed=78)
    assert int(types[..., 0].sum()) > 135                  # the last query tile sees more than 128 key tiles
    tb = nat.build_selection_tables(types.cuda(), T, nbs)
    o, lse = _ops.attn_fwd(q.cuda(), k.cuda(), v.cuda(), tb, DK ** -0.5, True)
    mask = oattn.attn_mask(types[..., 0], T, nbs, HQ)
    o_ref, lse_ref = oattn.attn_sdpa(q.float(), k.float(), v.float(), mask, DK ** -0.5)
    assert_close(o, o_ref, TOL, "o_attn")
    assert_close(lse, lse_ref, TOL, "lse")
    assert _lib.load().natsl_device_status() == 0


GDN_CASES = [  # B, T, H, HN, K, V, nbs, decay, use_h0
    (2, 512, 4, 4, 64, 64, 64, True, False),
    (1, 700, 4, 2, 128, 128, 64, True, True),
    (2, 384, 2, 2, 64, 128, 64, False, True),
    (1, 1024, 2, 2, 128, 64, 128, True, True),
    (1, 1100, 2, 1, 128, 256, 256, True, False),
    (1, 64, 2, 2, 128, 128, 64, True, True),
    (1, 50, 2, 2, 64, 64, 64, True, False),
]


@pytest.mark.parametrize("B,T,H,HN,K,V,nbs,decay,use_h0", GDN_CASES)
def test_gdn_linear_branch(nat, B, T, H, HN, K, V, nbs, decay, use_h0):
    from neuralattentionsearchlinear_b200 import _lib, _ops
    q, k, v, g, beta, h0 = synth_gdn_inputs(B, T, H, K, V, seed=T + K, normalize_qk=False)
    if not use_h0:
        h0 = None
    types = otab.synth_types(B, -(-T // nbs), HN, 0.35, seed=T + 1)
    tb = nat.build_selection_tables(types.cuda(), T, nbs)
    o, ht, inter = _ops.linear_fwd(_lib.RULE_GDN, q.cuda(), k.cuda(), v.cuda(), g.cuda(), beta.cuda(), tb, K ** -0.5,
                                   None if h0 is None else h0.cuda(), decay, True, True, return_intermediates=True)
    o_ref, s_ref, ir = ogdn.linear_chunk(q.float(), k.float(), v.float(), g, beta.float(), types[..., 1], nbs=nbs,
                                         h0=h0, decay=decay, return_intermediates=True)
    assert_close(inter["gcs"], ir["gcs"], 1e-4, "gcs")
    assert_close(inter["k_rstd"], ir["k_rstd"], 1e-3, "k_rstd")
    assert_close(inter["carry"], ir["carry"], 1e-4, "carry")
    assert_close(inter["u"], ir["u"], TOL, "u")
    assert_close(inter["w"], ir["w"], TOL, "w")
    assert_close(inter["h"], ir["h"], 2 * TOL, "h")
    assert_close(o, o_ref, TOL, "o_gdn")
    assert_close(ht, s_ref, 2 * TOL, "final_state")


@pytest.mark.parametrize("B,T,H,HN,K,V,nbs,decay", [(1, 1024, 4, 4, 128, 64, 256, True), (2, 512, 2, 2, 64, 64, 64, True),
                                                     (1, 900, 2, 1, 128, 128, 128, False)])
def test_mamba_linear_branch(nat, B, T, H, HN, K, V, nbs, decay):
    from neuralattentionsearchlinear_b200 import _lib, _ops
    q, k, v, g, h0 = synth_mamba_inputs(B, T, H, K, V, seed=T)
    types = otab.synth_types(B, -(-T // nbs), HN, 0.2, seed=T + 1)
    tb = nat.build_selection_tables(types.cuda(), T, nbs)
    o, ht, _ = _ops.linear_fwd(_lib.RULE_MAMBA, q.cuda(), k.cuda(), v.cuda(), g.cuda(), None, tb, 1.0, h0.cuda(),
                               decay, False, True)
    o_ref, s_ref = ogdn.linear_chunk(q.float(), k.float(), v.float(), g, None, types[..., 1], nbs=nbs, scale=1.0,
                                     h0=h0, decay=decay, use_l2norm=False, rule="mamba")
    assert_close(o, o_ref, TOL, "o_mamba")
    assert_close(ht, s_ref, 2 * TOL, "final_state")


def test_op_level_gdn_matches_recurrent_oracle(nat):
    """The public op (both branches) on the CPU-sized configuration against the token recurrence."""
    B, T, H, K, V = 2, 512, 4, 64, 64
    q, k, v, g, beta, _ = synth_gdn_inputs(B, T, H, K, V, seed=0)
    types = otab.synth_types(B, 8, H, 0.5, seed=0)
    cu = lambda x: x.cuda()
    o_l, o_a, ht = nat.nats_mixed_attn_gdn(cu(q), cu(k), cu(v), cu(q), cu(k), cu(v), None, cu(g), cu(beta), cu(types),
                                           None, nats_block_size=64, ops_for_incomplete_chunks='all',
                                           output_final_state_gated_delta=True, decay_for_non_gdn_blocks=True)
    o_ref, s_ref = ogdn.linear_recurrent(q.float(), k.float(), v.float(), g, beta.float(), types[..., 1], nbs=64)
    mask = oattn.attn_mask(types[..., 0], T, 64, H)
    oa_ref, _ = oattn.attn_sdpa(q.float(), k.float(), v.float(), mask)
    assert_close(o_l, o_ref, TOL, "o_gdn")
    assert_close(o_a, oa_ref, TOL, "o_attn")
    assert_close(ht, s_ref, 2 * TOL, "final_state")


@pytest.mark.parametrize("mode", ["all", "attn", "gated_delta_net"])
@pytest.mark.parametrize("T,nbs,K,V", [(512, 64, 64, 64), (700, 128, 128, 128), (1024, 256, 128, 64)])
def test_ops_for_incomplete_chunks_modes_gdn(nat, mode, T, nbs, K, V):
    """The three modes of mixed_attn_gdn.py:35-42: which branch covers the current chunk."""
    B, H = 2, 4
    q, k, v, g, beta, _ = synth_gdn_inputs(B, T, H, K, V, seed=T)
    types = otab.synth_types(B, -(-T // nbs), 2, 0.5, seed=nbs)
    types[:, -1] = 1
    cu = lambda x: x.cuda()
    o_l, o_a, ht = nat.nats_mixed_attn_gdn(cu(q), cu(k), cu(v), cu(q), cu(k), cu(v), None, cu(g), cu(beta), cu(types),
                                           None, nats_block_size=nbs, ops_for_incomplete_chunks=mode,
                                           output_final_state_gated_delta=True, decay_for_non_gdn_blocks=True)
    o_ref, s_ref = ogdn.linear_chunk(q.float(), k.float(), v.float(), g, beta.float(), types[..., 1], nbs=nbs,
                                     own_chunk=(mode != "attn"))
    mask = oattn.attn_mask(types[..., 0], T, nbs, H, own_chunk=(mode != "gated_delta_net"))
    oa_ref, _ = oattn.attn_sdpa(q.float(), k.float(), v.float(), mask)
    assert_close(o_l, o_ref, TOL, f"o_gdn ({mode})")
    assert_close(o_a, oa_ref, TOL, f"o_attn ({mode})")
    assert_close(ht, s_ref, 2 * TOL, f"final_state ({mode})")


@pytest.mark.parametrize("mode", ["attn", "mamba"])
def test_ops_for_incomplete_chunks_modes_mamba(nat, mode):
    B, T, H, K, V, nbs = 1, 1024, 4, 128, 64, 256
    q, k, v, g, _ = synth_mamba_inputs(B, T, H, K, V, seed=5)
    types = otab.synth_types(B, T // nbs, H, 0.4, seed=6)
    types[:, -1] = 1
    cu = lambda x: x.cuda()
    o_l, o_a, ht = nat.nats_mixed_attn_mamba(cu(q), cu(k), cu(v), cu(q), cu(k), cu(v), None, cu(g), cu(types), None,
                                             scale_attn=K ** -0.5, nats_block_size=nbs, ops_for_incomplete_chunks=mode,
                                             output_final_state_mamba=True, decay_for_non_mamba_blocks=True)
    o_ref, s_ref = ogdn.linear_chunk(q.float(), k.float(), v.float(), g, None, types[..., 1], nbs=nbs, scale=1.0,
                                     use_l2norm=False, rule="mamba", own_chunk=(mode != "attn"))
    mask = oattn.attn_mask(types[..., 0], T, nbs, H, own_chunk=(mode != "mamba"))
    oa_ref, _ = oattn.attn_sdpa(q.float(), k.float(), v.float(), mask, K ** -0.5)
    assert_close(o_l, o_ref, TOL, f"o_mamba ({mode})")
    assert_close(o_a, oa_ref, TOL, f"o_attn ({mode})")
    assert_close(ht, s_ref, 2 * TOL, f"final_state ({mode})")


def test_error_paths(nat):
    from neuralattentionsearchlinear_b200 import _lib
    types = otab.synth_types(1, 4, 2, 0.5, seed=0).cuda()
    with pytest.raises(_lib.NatslError):
        _lib.call("natsl_build_tables", types.data_ptr(), 1, 1, 4, 2, 256, 96, 128, None, None, None, None, None, None,
                  None, None, None)
    q = torch.zeros(1, 256, 2, 96, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_lib.NatslError):
        nat.nats_mixed_attn_gdn(q, q, q, q, q, q, None, torch.zeros(1, 256, 2, device="cuda"),
                                torch.zeros(1, 256, 2, device="cuda"), types, None)
    with pytest.raises(NotImplementedError):
        nat.nats_mixed_attn_gdn(q, q, q, q, q, q, None, None, None, types, None, attn_sw_size=16)


def test_full_size_layer_config(nat):
    """The benchmark configuration (B=8, T=4096, H=16, d=128, block 64, ~25 % softmax blocks) at full
    size: two batch elements against the oracle, and batch-independence (a size-independent property:
    (batch, head) units never interact)."""
    import bench
    B, T, H, K, V, nbs = (bench.CFG[n] for n in ("B", "T", "H", "K", "V", "nbs"))
    host = bench.make_inputs(0, B, H)
    d = {n: t.cuda() for n, t in host.items()}
    run = lambda x: nat.nats_mixed_attn_gdn(x["q"], x["k"], x["v"], x["q"], x["k"], x["v"], None, x["g"], x["beta"],
                                            x["types"], None, nats_block_size=nbs, ops_for_incomplete_chunks="all",
                                            output_final_state_gated_delta=True, decay_for_non_gdn_blocks=True)
    o_l, o_a, ht = run(d)
    frac = host["types"][:, :-1, :, 0].float().mean().item()
    assert 0.2 < frac < 0.3
    for b in (0, B - 1):
        s = {n: t[b:b + 1] for n, t in host.items()}
        ty = s["types"].float()
        o_ref, s_ref = ogdn.linear_chunk(s["q"].float(), s["k"].float(), s["v"].float(), s["g"], s["beta"].float(),
                                         ty[..., 1], nbs=nbs)
        assert_close(o_l[b:b + 1], o_ref, TOL, f"o_gdn[b={b}]")
        assert_close(ht[b:b + 1], s_ref, 2 * TOL, f"final_state[b={b}]")
        mask = oattn.attn_mask(ty[..., 0], T, nbs, H)
        oa_ref, _ = oattn.attn_sdpa(s["q"].float(), s["k"].float(), s["v"].float(), mask)
        assert_close(o_a[b:b + 1], oa_ref, TOL, f"o_attn[b={b}]")
    sub = {n: t[3:5].contiguous() for n, t in d.items()}
    o_l2, o_a2, ht2 = run(sub)
    assert torch.equal(o_l2, o_l[3:5]) and torch.equal(o_a2, o_a[3:5]) and torch.equal(ht2, ht[3:5])


@pytest.mark.parametrize("vsplit", [False, True])
@pytest.mark.parametrize("B,T,H,HN,decay,use_h0", [(2, 512, 4, 4, True, False), (1, 700, 4, 2, True, True),
                                                    (2, 384, 2, 2, False, True), (1, 64, 2, 2, True, True),
                                                    (1, 50, 2, 1, True, False), (1, 2048, 2, 2, True, True)])
def test_gdn_fused_walk(nat, B, T, H, HN, decay, use_h0, vsplit, monkeypatch):
    """Recurrence + output fused on tcgen05 (K = V = 128, block 64) against the oracle, and against the
    two-kernel path it replaces; both forms of the walk (one CTA per (batch, head), and the value dimension split
    over two CTAs)."""
    from neuralattentionsearchlinear_b200 import _lib, _ops
    monkeypatch.setattr(_ops, "WALK_VSPLIT", vsplit)
    K = V = 128
    q, k, v, g, beta, h0 = synth_gdn_inputs(B, T, H, K, V, seed=T + 5, normalize_qk=False)
    if not use_h0:
        h0 = None
    types = otab.synth_types(B, -(-T // 64), HN, 0.35, seed=T + 2)
    tb = nat.build_selection_tables(types.cuda(), T, 64)
    args = (_lib.RULE_GDN, q.cuda(), k.cuda(), v.cuda(), g.cuda(), beta.cuda(), tb, K ** -0.5,
            None if h0 is None else h0.cuda(), decay, True, True)
    assert _ops.USE_FUSED_WALK
    o, ht, inter = _ops.linear_fwd(*args)
    assert inter is None                                   # fused path: no per-chunk states
    assert _lib.load().natsl_device_status() == 0
    o_ref, s_ref = ogdn.linear_chunk(q.float(), k.float(), v.float(), g, beta.float(), types[..., 1], nbs=64, h0=h0,
                                     decay=decay)
    assert_close(o, o_ref, TOL, "o_gdn (fused walk)")
    assert_close(ht, s_ref, 2 * TOL, "final_state (fused walk)")
    o2, ht2, _ = _ops.linear_fwd(*args, return_intermediates=True)      # scan + out kernels
    assert_close(o, o2.float(), TOL, "fused vs two-kernel o")
    assert_close(ht, ht2, 2 * TOL, "fused vs two-kernel state")
    # run-to-run bit-identity: the walk's warps run up to a chunk apart and meet only through mbarriers
    for _ in range(4):
        o3, ht3, _ = _ops.linear_fwd(*args)
        assert torch.equal(o3, o) and torch.equal(ht3, ht)


@pytest.mark.parametrize("nbs,decay,T", [(64, True, 512), (128, False, 400), (64, True, 100)])
def test_fp32_path_matches_naive_recurrent_form(nat, nbs, decay, T):
    """fp32 tensors (the CPU-sized configuration: B=2, H=4, d=64): the reference-precision kernels against the
    naive recurrent form within 1e-4, through the public op."""
    B, H, K, V = 2, 4, 64, 64
    q, k, v, g, beta, h0 = synth_gdn_inputs(B, T, H, K, V, seed=0, dtype=torch.float32)
    types = otab.synth_types(B, -(-T // nbs), H, 0.5, seed=0)
    cu = lambda x: x.cuda()
    o_l, o_a, ht = nat.nats_mixed_attn_gdn(cu(q), cu(k), cu(v), cu(q), cu(k), cu(v), cu(h0), cu(g), cu(beta), cu(types),
                                           None, nats_block_size=nbs, ops_for_incomplete_chunks='all',
                                           output_final_state_gated_delta=True, decay_for_non_gdn_blocks=decay)
    assert o_l.dtype == torch.float32
    o_ref, s_ref = ogdn.linear_recurrent(q.double(), k.double(), v.double(), g.double(), beta.double(), types[..., 1],
                                         nbs=nbs, h0=h0.double(), decay=decay)
    mask = oattn.attn_mask(types[..., 0], T, nbs, H)
    oa_ref, _ = oattn.attn_sdpa(q.double(), k.double(), v.double(), mask)
    assert_close(o_l, o_ref.float(), 1e-4, "o_gdn fp32")
    assert_close(o_a, oa_ref.float(), 1e-4, "o_attn fp32")
    assert_close(ht, s_ref.float(), 1e-4, "final_state fp32")
    # Mamba2 rule
    o_m, o_a2, htm = nat.nats_mixed_attn_mamba(cu(q), cu(k), cu(v), cu(q), cu(k), cu(v), cu(h0), cu(g), cu(types), None,
                                               nats_block_size=nbs, ops_for_incomplete_chunks='all',
                                               output_final_state_mamba=True, decay_for_non_mamba_blocks=decay)
    om_ref, sm_ref = ogdn.linear_recurrent(q.double(), k.double(), v.double(), g.double(), None, types[..., 1], nbs=nbs,
                                           scale=1.0, h0=h0.double(), decay=decay, use_l2norm=False, rule="mamba")
    assert_close(o_m, om_ref.float(), 1e-4, "o_mamba fp32")
    assert_close(htm, sm_ref.float(), 1e-4, "mamba final_state fp32")


def test_gdn_op_with_the_760m_head_dims(nat):
    """K = 192, V = 384 (experiments/configs/natsl_760M.json: head_dim 192, expand_v 2; softmax heads 64 / 128): no chunk
    kernel has tiles for these; the op takes the token recurrence for the linear branch -- correct, not fast, forward only."""
    B, T, H, HQ, K, V, nbs = 1, 300, 2, 6, 192, 384, 64
    q, k, v, g, beta, _ = synth_gdn_inputs(B, T, H, K, V, seed=7)
    gen = torch.Generator().manual_seed(3)
    qa = torch.randn(B, T, HQ, K * H // HQ, generator=gen).bfloat16()
    ka = torch.randn(B, T, HQ, K * H // HQ, generator=gen).bfloat16()
    va = torch.randn(B, T, HQ, V * H // HQ, generator=gen).bfloat16()
    types = otab.synth_types(B, -(-T // nbs), H, 0.3, seed=2)
    c = lambda x: x.cuda()
    qg = c(q).requires_grad_(True)
    o_l, o_a, ht = nat.nats_mixed_attn_gdn(c(qa), c(ka), c(va), qg, c(k), c(v), None, c(g), c(beta), c(types), None,
                                           nats_block_size=nbs, ops_for_incomplete_chunks="all",
                                           output_final_state_gated_delta=True, decay_for_non_gdn_blocks=True)
    o_ref, s_ref = ogdn.linear_chunk(q.float(), k.float(), v.float(), g, beta.float(), types[..., 1], nbs=nbs)
    assert_close(o_l, o_ref, TOL, "o_gdn (K=192, V=384)")
    assert_close(ht, s_ref, TOL, "final state (K=192, V=384)")
    mask = oattn.attn_mask(types[..., 0], T, nbs, HQ)
    oa_ref, _ = oattn.attn_sdpa(qa.float(), ka.float(), va.float(), mask)
    assert_close(o_a, oa_ref, TOL, "o_attn (64 / 128)")
    with pytest.raises(NotImplementedError):
        o_l.float().sum().backward()
