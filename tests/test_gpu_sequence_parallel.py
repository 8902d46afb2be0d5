"""Sequence-parallel Mamba2 hybrid attention on 2 GPUs (NCCL): every rank's share against the single-GPU op on
the whole sequence (which the other GPU tests check against the oracle); skipped with fewer than 2 GPUs.
On one GPU: the sub-segment split of the linear branch and the two-source attention entry point."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import tables as otab
from tests.helpers import synth_mamba_inputs

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, B, T, H, K, V, nbs, layout, splits, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import neuralattentionsearchlinear_b200 as nat
        from neuralattentionsearchlinear_b200.sequence_parallel import nats_mixed_attn_mamba_sp
        q, k, v, g, _ = synth_mamba_inputs(B, T, H, K, V, seed=7)
        types = otab.synth_types(B, T // nbs, H, 0.15, seed=8)
        dev = torch.device("cuda", rank)
        from neuralattentionsearchlinear_b200.sequence_parallel import segment_ids
        ids = segment_ids(rank, world, layout)
        per = (T // nbs) // (world * len(ids))             # blocks per segment
        sl = torch.cat([torch.arange(s * per * nbs, (s + 1) * per * nbs) for s in ids])
        bsel = torch.cat([torch.arange(s * per, (s + 1) * per) for s in ids])
        c = lambda x: x.to(dev).contiguous()
        o_l, o_a, ht = nats_mixed_attn_mamba_sp(c(q[:, sl]), c(k[:, sl]), c(v[:, sl]), c(q[:, sl]), c(k[:, sl]), c(v[:, sl]),
                                                c(g[:, sl]), c(types[:, bsel]), nats_block_size=nbs,
                                                scale_attn=K ** -0.5, decay_for_non_mamba_blocks=True, layout=layout,
                                                linear_splits=splits)
        torch.cuda.synchronize()
        # again with the gather capacity given (no host read) and the state exchange on its own communicator
        from neuralattentionsearchlinear_b200 import sequence_parallel as sp
        o_l2, o_a2, _ = nats_mixed_attn_mamba_sp(c(q[:, sl]), c(k[:, sl]), c(v[:, sl]), c(q[:, sl]), c(k[:, sl]), c(v[:, sl]),
                                                 c(g[:, sl]), c(types[:, bsel]), nats_block_size=nbs,
                                                 scale_attn=K ** -0.5, decay_for_non_mamba_blocks=True, layout=layout,
                                                 linear_splits=splits, kv_capacity=sp.last_kv_capacity,
                                                 linear_group=dist.new_group())
        torch.cuda.synchronize()
        assert torch.equal(o_l, o_l2) and torch.equal(o_a, o_a2)
        # plan / replay form: compute captured in CUDA graphs, collectives eager between them
        xs = [c(q[:, sl]), c(k[:, sl]), c(v[:, sl])]
        lin_group = dist.new_group()
        for under in (True, False):                        # both orders of a step
            plan = sp.GraphedMambaSP(xs[0], xs[1], xs[2], xs[0], xs[1], xs[2], c(g[:, sl]), c(types[:, bsel]),
                                     kv_capacity=sp.last_kv_capacity, nats_block_size=nbs, scale_attn=K ** -0.5,
                                     layout=layout, linear_splits=splits, linear_group=lin_group,
                                     gather_under_linear=under)
            p_l, p_a, _ = plan.run()
            torch.cuda.synchronize()
            assert torch.equal(o_l, p_l) and torch.equal(o_a, p_a)
            plan.capture()
            for _ in range(2):
                p_l, p_a, _ = plan.run()
            torch.cuda.synchronize()
            assert torch.equal(o_l, p_l) and torch.equal(o_a, p_a)
        # single-GPU op on the whole sequence, on this rank's GPU
        r_l, r_a, r_ht = nat.nats_mixed_attn_mamba(c(q), c(k), c(v), c(q), c(k), c(v), None, c(g), c(types), None,
                                                   scale_attn=K ** -0.5, nats_block_size=nbs,
                                                   ops_for_incomplete_chunks='all', output_final_state_mamba=True,
                                                   decay_for_non_mamba_blocks=True)
        sl = sl.to(dev)
        err_l = (o_l.float() - r_l[:, sl].float()).abs().max().item()
        err_a = (o_a.float() - r_a[:, sl].float()).abs().max().item()
        err_h = (ht - r_ht).abs().max().item() if ht is not None else 0.0
        ref_mag = max(r_l.float().abs().max().item(), r_a.float().abs().max().item())
        from neuralattentionsearchlinear_b200 import _lib
        ret[rank] = (err_l, err_a, err_h, ref_mag, _lib.load().natsl_device_status())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("B,T,nbs,layout,splits", [(1, 4096, 256, "contiguous", None), (1, 2048, 64, "contiguous", 1),
                                                   (1, 4096, 256, "zigzag", None), (2, 2048, 128, "zigzag", 2)])
def test_sp_two_gpus_matches_single_gpu(B, T, nbs, layout, splits):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world, H, K, V = 2, 4, 128, 64
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), B, T, H, K, V, nbs, layout, splits, ret), nprocs=world, join=True)
    for r in range(world):
        err_l, err_a, err_h, mag, status = ret[r]
        assert status == 0
        # both sides are the same bf16 kernels; they differ by the order of the state fold only
        assert err_l <= 2e-2 * max(1.0, mag), (r, err_l)
        assert err_a <= 2e-2 * max(1.0, mag), (r, err_a)
        assert err_h <= 2e-2 * max(1.0, mag), (r, err_h)


@pytest.mark.parametrize("B,T,nbs,splits,decay", [(1, 8192, 256, 8, True), (2, 2048, 64, 4, False), (1, 4096, 128, None, True)])
def test_sub_segment_split_matches_plain_op(B, T, nbs, splits, decay):
    """One GPU, no process group: the linear branch cut into sub-segments against the plain op."""
    import neuralattentionsearchlinear_b200 as nat
    from neuralattentionsearchlinear_b200 import _lib
    from neuralattentionsearchlinear_b200.sequence_parallel import nats_mixed_attn_mamba_sp
    H, K, V = 4, 128, 64
    dev = torch.device("cuda", 0)
    q, k, v, g, _ = synth_mamba_inputs(B, T, H, K, V, seed=17)
    types = otab.synth_types(B, T // nbs, H, 0.2, seed=18)
    types[:, -1] = 1
    q, k, v, g, types = (x.to(dev) for x in (q, k, v, g, types))
    o_l, o_a, ht = nats_mixed_attn_mamba_sp(q, k, v, q, k, v, g, types, nats_block_size=nbs, scale_attn=K ** -0.5,
                                            decay_for_non_mamba_blocks=decay, linear_splits=splits)
    r_l, r_a, r_ht = nat.nats_mixed_attn_mamba(q, k, v, q, k, v, None, g, types, None, scale_attn=K ** -0.5,
                                               nats_block_size=nbs, ops_for_incomplete_chunks='all',
                                               output_final_state_mamba=True, decay_for_non_mamba_blocks=decay)
    torch.cuda.synchronize()
    mag = max(1.0, r_l.float().abs().max().item())
    assert (o_l.float() - r_l.float()).abs().max().item() <= 2e-2 * mag
    assert torch.equal(o_a, r_a)                           # same kernel, same inputs
    assert (ht - r_ht).abs().max().item() <= 2e-2 * mag
    assert _lib.load().natsl_device_status() == 0


@pytest.mark.parametrize("persistent", [False, True])
@pytest.mark.parametrize("DK,DV,nbs", [(128, 64, 256), (64, 128, 64), (128, 128, 128)])
def test_attn_split_equals_concatenated_keys(DK, DV, nbs, persistent, monkeypatch):
    """Keys held in two tensors (gathered part shared by two local segments + own part) against one call per
    segment on the concatenated keys: bit-identical (both forms of the kernel)."""
    from neuralattentionsearchlinear_b200 import _lib, _ops
    monkeypatch.setattr(_ops, "ATTN_PERSISTENT", persistent)
    from neuralattentionsearchlinear_b200.nats_util import build_selection_tables
    dev = torch.device("cuda", 0)
    B_rem, n_loc, S, L, HQ, HKV = 2, 2, 1024, 768, 4, 2
    gen = torch.Generator().manual_seed(23)
    rnd = lambda *s: torch.randn(*s, generator=gen).bfloat16().to(dev)
    q, k, v = rnd(n_loc * B_rem, L, HQ, DK), rnd(n_loc * B_rem, L, HKV, DK), rnd(n_loc * B_rem, L, HKV, DV)
    k_rem, v_rem = rnd(B_rem, S, HKV, DK), rnd(B_rem, S, HKV, DV)
    types = otab.synth_types(n_loc * B_rem, (S + L) // nbs, HKV, 0.4, seed=24).to(dev)
    tb = build_selection_tables(types, S + L, nbs)
    o = _ops.attn_fwd_split(q, k_rem, v_rem, k, v, tb, DK ** -0.5, True)
    for j in range(n_loc):
        sl = slice(j * B_rem, (j + 1) * B_rem)
        tbj = build_selection_tables(types[sl].contiguous(), S + L, nbs)
        kc, vc = torch.cat([k_rem, k[sl]], 1).contiguous(), torch.cat([v_rem, v[sl]], 1).contiguous()
        oj, _ = _ops.attn_fwd(q[sl].contiguous(), kc, vc, tbj, DK ** -0.5, True, q_off=S)
        assert torch.equal(o[sl], oj)
    assert _lib.load().natsl_device_status() == 0


@pytest.mark.parametrize("persistent", [False, True])
@pytest.mark.parametrize("DK,DV,nbs,HKV,HN", [(128, 64, 128, 4, 2), (64, 64, 256, 2, 2)])
def test_attn_split_packed_pairs_equals_head_major(DK, DV, nbs, HKV, HN, persistent, monkeypatch):
    """The gathered keys as packed (block, head) pairs against the padded head-major layout: bit-identical."""
    from neuralattentionsearchlinear_b200 import _lib, _ops
    monkeypatch.setattr(_ops, "ATTN_PERSISTENT", persistent)
    from neuralattentionsearchlinear_b200.sequence_parallel import CudaSegmentOps, virtual_attn_types
    dev = torch.device("cuda", 0)
    be = CudaSegmentOps()
    G, B, n_loc, Lr, L, HQ = 3, 1, 2, 1024, 512, 4
    gen = torch.Generator().manual_seed(31)
    rnd = lambda *s: torch.randn(*s, generator=gen).bfloat16().to(dev)
    k_g, v_g = rnd(G, Lr, HKV, DK), rnd(G, Lr, HKV, DV)                  # the G remote segments as a batch
    types_g = otab.synth_types(G, Lr // nbs, HN, 0.5, seed=32).to(dev)
    tb_g = be.tables(types_g, Lr, nbs)
    n_g = tb_g.n_blocks[..., 0].to(torch.int64).view(G, B, HN)
    n_h = n_g.repeat_interleave(HKV // HN, dim=2)
    vcap, cap_pairs = int(n_g.max()), int(n_h.sum(2).max())
    assert vcap > 0
    q, k, v = rnd(n_loc * B, L, HQ, DK), rnd(n_loc * B, L, HKV, DK), rnd(n_loc * B, L, HKV, DV)
    types_l = otab.synth_types(n_loc * B, L // nbs, HN, 0.5, seed=33).to(dev)
    types_v = virtual_attn_types(n_g, torch.tensor([0, 1, 2]), [3, 4], vcap, types_l)
    tb_v = be.tables(types_v, G * vcap * nbs + L, nbs)
    hm = lambda x: be.pack(x, tb_g, vcap).reshape(1, G * vcap * nbs, HKV, x.shape[-1])
    o_hm = be.attn_split(q, hm(k_g), hm(v_g), k, v, tb_v, DK ** -0.5, True, None, 0)
    pp = lambda x: be.pack_pairs(x, tb_g, cap_pairs).reshape(1, G * cap_pairs * nbs, x.shape[-1])
    seg_base = torch.arange(G, device=dev).view(G, 1, 1) * cap_pairs
    rem_base = (n_h.cumsum(2) - n_h + seg_base).permute(1, 0, 2).to(torch.int32).contiguous()
    o_pp = be.attn_split(q, pp(k_g), pp(v_g), k, v, tb_v, DK ** -0.5, True, rem_base, vcap)
    torch.cuda.synchronize()
    assert torch.equal(o_hm, o_pp)
    assert _lib.load().natsl_device_status() == 0


def test_pack_pairs_capacity_overflow_sets_status():
    from neuralattentionsearchlinear_b200 import _lib
    from neuralattentionsearchlinear_b200.sequence_parallel import CudaSegmentOps
    dev = torch.device("cuda", 0)
    be = CudaSegmentOps()
    x = torch.zeros(1, 1024, 2, 64, dtype=torch.bfloat16, device=dev)
    types = torch.ones(1, 8, 2, 2, device=dev)                       # every block selected: 16 pairs, 8 per head
    tb = be.tables(types, 1024, 128)
    assert _lib.load().natsl_device_status() == 0
    be.pack_pairs(x, tb, 16, 8)
    assert _lib.load().natsl_device_status() == 0
    be.pack_pairs(x, tb, 12, 0)                                      # too few pairs
    assert _lib.load().natsl_device_status() == 3
    be.pack_pairs(x, tb, 16, 4)                                      # more blocks per head than announced
    assert _lib.load().natsl_device_status() == 3
    assert _lib.load().natsl_device_status() == 0                    # reading clears it
