"""The oracle's integer tables against (1) tables produced by the reference's own
nats_util.py (tests/golden/tables_ref.npz, see make_golden.py) and (2) a
known-answer vector produced by that code for B=1, TN=8, HN=2, block 64."""
import os

import numpy as np
import torch

from oracle import tables as otab

KEYS = ["indices", "n_blocks", "chunk_indices", "offsets", "starting_h_idx", "attn_n_iters"]


def test_tables_match_reference_generated(golden_dir):
    z = np.load(os.path.join(golden_dir, "tables_ref.npz"))
    names = sorted({k.split("_")[0] for k in z.files})
    assert len(names) >= 7
    for n in names:
        B, T, HN, nbs = z[f"{n}_meta"].tolist()
        types = torch.from_numpy(z[f"{n}_types"])
        mine = otab.build_tables(types, T, nbs)
        for k in KEYS:
            ref = z[f"{n}_{k}"]
            got = mine[k].numpy()
            assert got.shape == ref.shape, (n, k, got.shape, ref.shape)
            assert np.array_equal(got, ref), (n, k)


def test_known_answer_vector():
    attn = torch.tensor([[1, 0, 0, 1, 0, 0, 1, 1], [0, 0, 1, 0, 0, 0, 0, 1]])
    lin = torch.tensor([[0, 1, 1, 0, 1, 1, 0, 1], [1, 1, 0, 1, 1, 1, 1, 1]])
    types = torch.stack([attn.T, lin.T], -1).unsqueeze(0).float()        # [1,8,2,2]
    t = otab.build_tables(types, 512, 64)
    assert t["indices"][0, :, 0, 0].tolist() == [0, 3, 6, 7, 8, 8, 8, 8]
    assert t["indices"][0, :, 1, 0].tolist() == [2, 7, 8, 8, 8, 8, 8, 8]
    assert t["indices"][0, :, 0, 1].tolist() == [1, 2, 4, 5, 7, 8, 8, 8]
    assert t["indices"][0, :, 1, 1].tolist() == [0, 1, 3, 4, 5, 6, 7, 8]
    assert t["n_blocks"].tolist() == [[[4, 5], [2, 7]]]
    assert t["chunk_indices"].tolist() == [[0, 0], [0, 1], [0, 2], [0, 3], [0, 4], [1, 0], [1, 1], [1, 2],
                                           [1, 3], [1, 4], [1, 5], [1, 6]]
    assert t["offsets"].tolist() == [0, 5, 12]
    assert t["starting_h_idx"][0].tolist() == [[0, 0], [0, 1], [1, 2], [2, 2], [2, 3], [3, 4], [4, 5], [4, 6]]
    assert t["attn_n_iters"][0].tolist() == [[0, 0], [1, 0], [2, 1], [2, 1]]
    t64 = otab.build_tables(types, 512, 64, attn_bt=64)
    assert t64["attn_n_iters"][0].tolist() == [[0, 0], [1, 0], [1, 0], [1, 1], [2, 1], [2, 1], [2, 1], [3, 1]]


def test_hard_softmax_first_max_and_one_hot():
    logits = torch.tensor([[0.3, 0.3], [1.0, -1.0], [-2.0, 5.0]])
    y = otab.hard_softmax(logits)
    assert y.tolist() == [[1.0, 0.0], [1.0, 0.0], [0.0, 1.0]]
    yb = otab.hard_softmax(torch.randn(64, 2, dtype=torch.bfloat16))
    assert set(yb.float().flatten().tolist()) <= {0.0, 1.0} and bool((yb.sum(-1) == 1).all())


def test_synth_fraction():
    ty = otab.synth_types(8, 64, 16, 0.25, seed=0, force_last=False)
    frac = ty[..., 0].mean().item()
    assert 0.22 < frac < 0.28
