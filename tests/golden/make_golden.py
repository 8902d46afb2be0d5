"""Generates the committed golden vectors under tests/golden/.

Run once in a container that has the reference checkout (read-only) and the
third-party ``flash-linear-attention`` package on disk:

    python tests/golden/make_golden.py --reference /path/to/reference

Outputs (small .npz files, committed):
  tables_ref.npz      integer tables produced by the REFERENCE's own
                      ``src/nats/ops/nats_util.py`` (loaded by file path, CPU) with the
                      op prologue of ``src/nats/ops/mixed_ops/mixed_attn_gdn.py:88-100``
                      applied to seeded block types.
  gdn_fla_naive.npz   outputs of flash-linear-attention's pure-PyTorch
                      ``naive_recurrent_gated_delta_rule`` (the package whose kernels the
                      reference's debug scripts compare against) on seeded inputs.
  oracle_config0.npz  the oracle's own outputs on the CPU-sized configuration
                      (B=2, T=512, H=4, K=V=64, block 64, seed 0), as a regression pin.
"""
from __future__ import annotations

import argparse
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import attn as oattn  # noqa: E402
from oracle import gdn as ogdn  # noqa: E402
from oracle import tables as otab  # noqa: E402


def load_by_path(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def reference_tables(nu, types, T, nbs, attn_bt=128, attn_bs=64):
    """mixed_attn_gdn.py:88-139 and attns.py's n_iters call, using the reference's functions."""
    types = torch.round(types)
    TN = types.shape[1]
    idx = torch.where(types == 1., torch.arange(TN, dtype=torch.int32).view(1, -1, 1, 1), TN)
    idx = idx.sort(1)[0]
    n_blocks = types.int().sum(1)
    ci = nu.prepare_nats_block_indices(n_blocks[..., 1], nbs, 64)
    off = nu.prepare_nats_chunk_offsets(n_blocks, types, nbs, 64, 1)
    sh = nu.compute_starting_idx_for_chunks(nats_block_indices=idx, T=T, BT=64, NAtS_Block_Size=nbs, offset_op=1)
    ni = nu.compute_attn_n_iters_per_block(idx, T, attn_bt, attn_bs, nbs, 0)
    return dict(indices=idx, n_blocks=n_blocks, chunk_indices=ci, offsets=off, starting_h_idx=sh, attn_n_iters=ni)


def config0_inputs(seed=0, B=2, T=512, H=4, K=64, V=64, dtype=torch.float32):
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(B, T, H, K, generator=gen, dtype=dtype)
    k = torch.randn(B, T, H, K, generator=gen, dtype=dtype)
    v = torch.randn(B, T, H, V, generator=gen, dtype=dtype)
    q, k = ogdn.l2norm(q), ogdn.l2norm(k)
    beta = torch.randn(B, T, H, generator=gen, dtype=dtype).sigmoid()
    g = -torch.nn.functional.softplus(torch.randn(B, T, H, generator=gen, dtype=dtype))
    return q, k, v, g, beta


def grad_pin_inputs():
    """Small float64 inputs of the backward pin (B=1, T=256, H=2, K=8, V=6, block 64)."""
    gen = torch.Generator().manual_seed(21)
    dt = torch.float64
    B, T, H, K, V = 1, 256, 2, 8, 6
    r = lambda *s: torch.randn(*s, generator=gen, dtype=dt)
    types = otab.synth_types(B, T // 64, 2, 0.5, seed=22, dtype=dt)
    types[:, -1] = 1
    return dict(q=r(B, T, H, K), k=r(B, T, H, K), v=r(B, T, H, V), g=-torch.nn.functional.softplus(r(B, T, H)) * 0.3,
                beta=r(B, T, H).sigmoid(), do=r(B, T, H, V), dht=r(B, H, K, V), types=types)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of a checkout of automl/NeuralAttentionSearchLinear")
    ap.add_argument("--fla-naive", default=None, help="path to fla/ops/gated_delta_rule/naive.py")
    args = ap.parse_args()

    # ---- 1. tables from the reference's own nats_util.py -------------------------------
    nu = load_by_path("ref_nats_util", os.path.join(args.reference, "src/nats/ops/nats_util.py"))
    out = {}
    cases = [  # (name, B, T, HN, nbs, p_attn, seed)
        ("a", 1, 512, 2, 64, 0.4, 11), ("b", 2, 512, 4, 64, 0.5, 0), ("c", 3, 1000, 3, 64, 0.25, 5),
        ("d", 2, 1024, 2, 128, 0.3, 7), ("e", 1, 4096, 16, 64, 0.25, 3), ("f", 2, 2048, 4, 256, 0.1, 9),
        ("g", 2, 130, 2, 64, 0.5, 13),
    ]
    for name, B, T, HN, nbs, p, seed in cases:
        TN = -(-T // nbs)
        types = otab.synth_types(B, TN, HN, p, seed)
        ref = reference_tables(nu, types, T, nbs)
        out[f"{name}_meta"] = np.array([B, T, HN, nbs], dtype=np.int64)
        out[f"{name}_types"] = types.numpy()
        for k_, v_ in ref.items():
            out[f"{name}_{k_}"] = v_.numpy().astype(np.int64)
    np.savez_compressed(os.path.join(HERE, "tables_ref.npz"), **out)

    # ---- 2. third-party naive GDN (all blocks selected) ----------------------------------
    naive_path = args.fla_naive
    if naive_path is None:
        import sysconfig
        naive_path = os.path.join(sysconfig.get_paths()["purelib"], "fla/ops/gated_delta_rule/naive.py")
    naive = load_by_path("fla_naive", naive_path)
    gen = torch.Generator().manual_seed(0)
    B, T, H, K, V = 2, 192, 2, 32, 32
    q = torch.randn(B, T, H, K, generator=gen)
    k = ogdn.l2norm(torch.randn(B, T, H, K, generator=gen))
    v = torch.randn(B, T, H, V, generator=gen)
    beta = torch.randn(B, T, H, generator=gen).sigmoid()
    g = -torch.nn.functional.softplus(torch.randn(B, T, H, generator=gen))
    h0 = torch.randn(B, H, K, V, generator=gen)
    o_n, s_n = naive.naive_recurrent_gated_delta_rule(q, k, v, beta, g, scale=K ** -0.5, initial_state=h0,
                                                      output_final_state=True)
    np.savez_compressed(os.path.join(HERE, "gdn_fla_naive.npz"), q=q.numpy(), k=k.numpy(), v=v.numpy(),
                        beta=beta.numpy(), g=g.numpy(), h0=h0.numpy(), o=o_n.float().numpy(), s=s_n.float().numpy())

    # ---- 3. oracle regression pin on the CPU-sized configuration -------------------------
    q, k, v, g, beta = config0_inputs()
    types = otab.synth_types(2, 8, 4, 0.5, seed=0)
    o_l, s_l = ogdn.linear_chunk(q, k, v, g, beta, types[..., 1], nbs=64)
    mask = oattn.attn_mask(types[..., 0], 512, 64, 4)
    o_a, lse = oattn.attn_sdpa(q, k, v, mask)
    np.savez_compressed(os.path.join(HERE, "oracle_config0.npz"), types=types.numpy(),
                        o_lin=o_l[:, ::7].numpy(), s_lin=s_l.numpy(), o_attn=o_a[:, ::7].numpy(), lse=lse[:, ::7].numpy(),
                        mask_rowsum=mask.sum(-1).numpy().astype(np.int32))
    # ---- 4. regression pin of the no-own-chunk mode and of the backward oracle (float64, small) -------------
    from oracle import grad as ograd
    x = grad_pin_inputs()
    sel = x["types"][..., 1]
    o_na, s_na = ogdn.linear_chunk(x["q"], x["k"], x["v"], x["g"], x["beta"], sel, nbs=64, own_chunk=False)
    gr = ograd.linear_chunk_backward(x["q"], x["k"], x["v"], x["g"], x["beta"], sel, x["do"], x["dht"], decay=True)
    dn = ograd.dnats_linear(x["q"], x["k"], x["v"], x["g"], x["beta"], sel, x["do"], x["dht"], decay=True)
    ga = ograd.attn_grads(x["q"], x["k"], x["v"], x["types"][..., 0], x["do"], nbs=64, reference_compat=True)
    np.savez_compressed(os.path.join(HERE, "oracle_grad_pin.npz"), o_no_own=o_na[:, ::5].numpy(), s_no_own=s_na.numpy(),
                        dq=gr["dq"][:, ::5].numpy(), dk=gr["dk"][:, ::5].numpy(), dv=gr["dv"][:, ::5].numpy(),
                        dg=gr["dg"].numpy(), dbeta=gr["dbeta"].numpy(), dnats_lin=dn.numpy(),
                        dq_attn_compat=ga["dq"][:, ::5].numpy(), dk_attn_compat=ga["dk"][:, ::5].numpy(),
                        dnats_attn=ga["dnats"].numpy())
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
