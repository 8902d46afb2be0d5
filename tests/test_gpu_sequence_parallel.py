"""Sequence-parallel Mamba2 hybrid attention on 2 GPUs (NCCL): every rank's share against the single-GPU op on
the whole sequence (which the other GPU tests check against the oracle).  Skipped with fewer than 2 GPUs."""
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


def _worker(rank, world, port, B, T, H, K, V, nbs, layout, ret):
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
                                                scale_attn=K ** -0.5, decay_for_non_mamba_blocks=True, layout=layout)
        torch.cuda.synchronize()
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


@pytest.mark.parametrize("T,nbs,layout", [(4096, 256, "contiguous"), (2048, 64, "contiguous"), (4096, 256, "zigzag"),
                                          (2048, 128, "zigzag")])
def test_sp_two_gpus_matches_single_gpu(T, nbs, layout):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world, B, H, K, V = 2, 1, 4, 128, 64
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), B, T, H, K, V, nbs, layout, ret), nprocs=world, join=True)
    for r in range(world):
        err_l, err_a, err_h, mag, status = ret[r]
        assert status == 0
        # both sides are the same bf16 kernels; they differ by the order of the state fold only
        assert err_l <= 2e-2 * max(1.0, mag), (r, err_l)
        assert err_a <= 2e-2 * max(1.0, mag), (r, err_a)
        assert err_h <= 2e-2 * max(1.0, mag), (r, err_h)
