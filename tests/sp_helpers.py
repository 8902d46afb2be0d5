"""CPU stand-in for the per-rank compute steps of the sequence-parallel path, built on the oracle, so that the
exchange / combine / virtual-sequence logic can be tested with gloo ranks and no GPU (test infrastructure)."""
from __future__ import annotations

from types import SimpleNamespace

import torch

from oracle import attn as oattn
from oracle import gdn as ogdn
from oracle import tables as otab


class OracleSegmentOps:
    def tables(self, types, T, nbs):
        t = otab.build_tables(types, T, nbs)
        return SimpleNamespace(types_i=t["types_i"], indices=t["indices"], n_blocks=t["n_blocks"], nats_block_size=nbs,
                               T=T, types=types)

    def linear(self, q, k, v, g, tables, scale, h0, decay, skip_out):
        o, ht, inter = ogdn.linear_chunk(q, k, v, g, None, tables.types_i[..., 1], nbs=tables.nats_block_size, scale=scale,
                                         h0=h0, decay=decay, use_l2norm=False, rule="mamba",
                                         reference_trailing_carry=False, return_intermediates=True)
        return (None if skip_out else o), ht, inter["gcs"]

    def segment_decay(self, gcs, tables, decay):
        B, T, H = gcs.shape
        nbs = tables.nats_block_size
        HN = tables.types_i.shape[2]
        a = torch.zeros(B, H, dtype=gcs.dtype)
        trail = torch.zeros(B, H, dtype=gcs.dtype)
        for b in range(B):
            for h in range(H):
                acc = tr = 0.0
                for c in range(-(-T // 64)):
                    sel = int(tables.types_i[b, (c * 64) // nbs, h // (H // HN), 1])
                    gl = float(gcs[b, min(c * 64 + 63, T - 1), h])
                    if decay or sel:
                        acc += gl
                    tr = 0.0 if sel else (tr + gl if decay else tr)
                a[b, h], trail[b, h] = acc, tr
        return a.exp(), trail.exp()

    def state_combine(self, a_all, S_all, rank):
        h_in = torch.zeros_like(S_all[0])
        f = torch.ones_like(a_all[0])
        for r in range(rank - 1, -1, -1):
            h_in += f[..., None, None] * S_all[r]
            f = f * a_all[r]
        return h_in

    def prefix_states(self, a, S, h0, want_prefix):
        p = torch.zeros_like(S[0]) if h0 is None else h0.clone()
        f = torch.ones_like(a[0])
        pre = []
        for n in range(S.shape[0]):
            pre.append(p.clone())
            p = a[n][..., None, None] * p + S[n]
            f = f * a[n]
        return (torch.stack(pre) if want_prefix else None), p, f

    def pack_pairs(self, x, tables, cap_pairs, max_per_head=0):
        B, T, H, D = x.shape
        nbs = tables.nats_block_size
        HN = tables.types_i.shape[2]
        out = torch.zeros(B, cap_pairs * nbs, D, dtype=x.dtype)
        for b in range(B):
            p = 0
            for h in range(H):
                hn = h // (H // HN)
                for j in range(int(tables.n_blocks[b, hn, 0])):
                    blk = int(tables.indices[b, j, hn, 0])
                    seg = x[b, blk * nbs:(blk + 1) * nbs, h]
                    if p < cap_pairs:
                        out[b, p * nbs:p * nbs + seg.shape[0]] = seg
                    p += 1
        return out

    def attn_split(self, q, k_rem, v_rem, k, v, tables, scale, own_chunk, rem_base, rem_slots):
        nbs = tables.nats_block_size
        B_rem, G, HKV = rem_base.shape
        S = G * rem_slots * nbs

        def unpack(x):                                     # pairs -> [B_rem, S, HKV, D] virtual layout (zeros elsewhere)
            out = torch.zeros(B_rem, S, HKV, x.shape[-1], dtype=x.dtype)
            n_pairs = x.shape[1] // nbs
            for b in range(B_rem):
                for g in range(G):
                    for h in range(HKV):
                        for j in range(rem_slots):
                            p = int(rem_base[b, g, h]) + j
                            if p < n_pairs:
                                out[b, (g * rem_slots + j) * nbs:(g * rem_slots + j + 1) * nbs, h] = x[b, p * nbs:(p + 1) * nbs]
            return out

        rep = q.shape[0] // B_rem                          # the gathered keys are shared by the local segments
        k_virt = torch.cat([unpack(k_rem).repeat(rep, 1, 1, 1), k], 1)
        v_virt = torch.cat([unpack(v_rem).repeat(rep, 1, 1, 1), v], 1)
        return self.attn(q, k_virt, v_virt, tables, scale, own_chunk, S)

    def pack(self, x, tables, cap_blocks):
        B, T, H, D = x.shape
        nbs = tables.nats_block_size
        HN = tables.types_i.shape[2]
        out = torch.zeros(B, cap_blocks * nbs, H, D, dtype=x.dtype)
        for b in range(B):
            for h in range(H):
                hn = h // (H // HN)
                for j in range(min(int(tables.n_blocks[b, hn, 0]), cap_blocks)):
                    blk = int(tables.indices[b, j, hn, 0])
                    seg = x[b, blk * nbs:(blk + 1) * nbs, h]
                    out[b, j * nbs:j * nbs + seg.shape[0], h] = seg
        return out

    def attn(self, q, k, v, tables, scale, own_chunk, q_off):
        T = k.shape[1]
        mask = oattn.attn_mask(tables.types_i[..., 0], T, tables.nats_block_size, q.shape[2], own_chunk=own_chunk)
        mask = mask[:, :, q_off:q_off + q.shape[1]]
        B, Tq, HQ, K = q.shape
        G = HQ // k.shape[2]
        s = torch.einsum("bthk,bshk->bhts", q, k.repeat_interleave(G, 2)) * scale
        s = s.masked_fill(~mask, float("-inf"))
        p = torch.softmax(s, -1)
        p = torch.where(mask.any(-1, keepdim=True), p, torch.zeros_like(p))
        return torch.einsum("bhts,bshv->bthv", p, v.repeat_interleave(G, 2))

    def n_attn_blocks(self, tables):
        return tables.n_blocks[..., 0].to(torch.int32).contiguous()
