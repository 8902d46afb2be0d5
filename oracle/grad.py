"""Oracle (test infrastructure): gradients of the hybrid attention op, for the backward pass that the
CUDA path does not have yet.

Two kinds of quantities are restated here.

* True gradients: autograd through the oracle's own forward (token recurrence with re-roll,
  ``oracle/gdn.py``; masked softmax, ``oracle/attn.py``) in the caller's dtype (use float64).
* What the reference returns instead where it deviates from the true gradient
  (src/nats/ops/mixed_ops/mixed_attn_gdn.py:196-283):
    - its softmax-branch backward drops the own-chunk terms of dq, dk, dv while normalising with the forward's
      lse (the forward passes ``compute_incomplete_chunk_scores`` from the strategy, mixed_attn_gdn.py:115; the
      backward passes it only for sliding windows, :237; kernels src/nats/ops/attns/attns.py:590-591, 842, 884);
    - ``dnats`` is not a derivative of the forward with respect to the 0/1 block types: column 0 is the gradient
      with respect to an additive logit bias on the keys of a softmax-selected block as seen by later blocks' queries
      (attns.py:922-978, zero for unselected blocks, :1625-1629), column 1 the gradient with respect to a gate on the
      block's state write (src/nats/ops/common/chunk_o.py:440-443), for selected blocks — and for the other blocks,
      when ``compute_dnats_for_invalid_blocks_linear_att`` is set, the same expression evaluated with the raw
      values and the state gradient of the next selected block (chunk_o.py:459-492); both are summed over the heads
      of a selection group (chunk_o.py:1568-1575, attns.py:1749-1755).

Block size 64 only (one compute chunk per block): the reference's chunk kernels are not self-consistent for
larger blocks (src/nats/ops/gated_delta_rule/chunk.py:47-50).
"""
from __future__ import annotations

import torch

from . import attn as oattn
from . import gdn as ogdn

C = ogdn.CHUNK


def _leaf(x):
    return None if x is None else x.detach().clone().requires_grad_(True)


def linear_true_grads(q, k, v, g, beta, sel, do, dht=None, *, scale=None, h0=None, decay=True, use_l2norm=True,
                      rule="gdn", nbs=64):
    """Autograd through the token recurrence with re-roll.  do [B,T,H,V]; dht [B,H,K,V] or None.
    -> dict(dq, dk, dv, dg, dbeta (None for Mamba2), dh0 (None without h0))."""
    q_, k_, v_, g_ = _leaf(q), _leaf(k), _leaf(v), _leaf(g)
    b_ = _leaf(beta) if rule == "gdn" else None
    h_ = _leaf(h0)
    o, sfin = ogdn.linear_recurrent(q_, k_, v_, g_, b_, sel, nbs=nbs, scale=scale, h0=h_, decay=decay,
                                    use_l2norm=use_l2norm, rule=rule)
    loss = (o * do).sum()
    if dht is not None:
        loss = loss + (sfin * dht).sum()
    loss.backward()
    return dict(dq=q_.grad, dk=k_.grad, dv=v_.grad, dg=g_.grad, dbeta=None if b_ is None else b_.grad,
                dh0=None if h_ is None else h_.grad)


def chunk_forward_with_probes(q, k, v, g, beta, sel, *, scale=None, h0=None, decay=True, use_l2norm=True, rule="gdn",
                              write_gate=None):
    """The chunk form of ``oracle.gdn.linear_chunk`` for block size 64, written so that autograd can see two extra
    things: ``write_gate`` [B,NT,H] multiplies the state write of every chunk (1 = the forward), and a zero tensor
    is added to the state after every chunk (``probes``; its gradient is the gradient with respect to that state).
    -> (o [B,T,H,V], final state [B,H,K,V], probes list of NT tensors [B,H,K,V], writes list of NT tensors
    [B,H,K,V] = the term each chunk would add to the state, from the processed values v' of selected chunks and the raw
    values of the others)."""
    B, T, H, K = q.shape
    V = v.shape[-1]
    dt = q.dtype
    assert T % C == 0, "the backward oracle takes whole chunks"
    if scale is None:
        scale = K ** -0.5
    if use_l2norm:
        q, k = ogdn.l2norm(q), ogdn.l2norm(k)
    NT = T // C
    if beta is None:
        beta = torch.ones(B, T, H, dtype=dt)
    ch = lambda x, D: x.view(B, NT, C, H, D).permute(0, 3, 1, 2, 4)          # [B,H,NT,C,D]
    qc, kc, vc = ch(q, K), ch(k, K), ch(v, V)
    gc = g.view(B, NT, C, H).permute(0, 3, 1, 2).cumsum(-1)
    bc = beta.view(B, NT, C, H).permute(0, 3, 1, 2)
    gam = gc[..., :, None] - gc[..., None, :]
    tril_s = torch.tril(torch.ones(C, C, dtype=torch.bool), -1)
    tril_i = torch.tril(torch.ones(C, C, dtype=torch.bool), 0)
    zero = torch.zeros((), dtype=dt)
    if rule == "gdn":
        A = torch.where(tril_s, bc[..., :, None] * (kc @ kc.transpose(-1, -2)) * gam.exp(), zero)
        eye = torch.eye(C, dtype=dt)
        Ai = torch.linalg.solve_triangular(eye + A, eye.expand_as(A).contiguous(), upper=False)
        u = Ai @ (vc * bc[..., None])
        w = Ai @ (kc * (bc * gc.exp())[..., None])
    else:
        u, w = vc, torch.zeros_like(kc)
    P = torch.where(tril_i, (qc @ kc.transpose(-1, -2)) * gam.exp(), zero)
    gL = gc[..., -1]
    selh = ogdn._expand_sel(sel, H).permute(0, 2, 1)                           # [B,H,NT]
    S = torch.zeros(B, H, K, V, dtype=dt) if h0 is None else h0
    Sfin = S
    carry = torch.zeros(B, H, dtype=dt)
    outs, probes, writes = [], [], []
    for c in range(NT):
        act = selh[..., c]
        ec = carry.exp()[..., None, None]
        vprime = u[:, :, c] - ec * (w[:, :, c] @ S)
        outs.append(scale * ((gc[:, :, c] + carry[..., None]).exp()[..., None] * (qc[:, :, c] @ S) + P[:, :, c] @ vprime))
        gl = gL[:, :, c]
        kdec = (gl[..., None] - gc[:, :, c]).exp() if rule == "gdn" else torch.clamp(gl[..., None] - gc[:, :, c], max=0.0).exp()
        write = kc[:, :, c].transpose(-1, -2) @ (vprime * kdec[..., None])
        # what the reference evaluates for a block that does not update the state: the raw values
        writes.append(torch.where(act[..., None, None], write, kc[:, :, c].transpose(-1, -2) @ (vc[:, :, c] * kdec[..., None])))
        gate = 1.0 if write_gate is None else write_gate[:, c].unsqueeze(-1).unsqueeze(-1)
        S_new = (gl + carry).exp()[..., None, None] * S + gate * write
        S = torch.where(act[..., None, None], S_new, S)
        probe = torch.zeros(B, H, K, V, dtype=dt, requires_grad=True)
        probes.append(probe)
        S = S + probe
        carry = torch.where(act, torch.zeros_like(carry), carry + gl if decay else carry)
        Sfin = torch.where(act[..., None, None], S, Sfin)
    o = torch.stack(outs, 2).permute(0, 2, 3, 1, 4).reshape(B, T, H, V)
    return o, Sfin, probes, writes


def dnats_linear(q, k, v, g, beta, sel, do, dht=None, *, invalid_blocks=True, **kw):
    """Column 1 of the reference's ``dnats`` [B,NT,HN]: for a selected block the gradient with respect to a gate on its
    state write, <write_c, dS_after_c>; for the other blocks (when ``invalid_blocks``) the same inner product with
    the raw-value write and the state gradient of the next selected block (zero when there is none), summed over
    the heads of a selection group."""
    q_, k_, v_, g_ = (x.detach() for x in (q, k, v, g))
    o, sfin, probes, writes = chunk_forward_with_probes(q_, k_, v_, g_, None if beta is None else beta.detach(), sel, **kw)
    loss = (o * do).sum()
    if dht is not None:
        loss = loss + (sfin * dht).sum()
    grads = torch.autograd.grad(loss, probes, allow_unused=True)
    B, T, H, K = q.shape
    NT, HN = T // C, sel.shape[2]
    selh = ogdn._expand_sel(sel, H)                                            # [B,NT,H]
    out = torch.zeros(B, NT, H, dtype=q.dtype)
    nxt = None                                                                 # dS after the next selected block
    for c in range(NT - 1, -1, -1):
        gS = grads[c] if grads[c] is not None else torch.zeros_like(writes[c])
        m = selh[:, c]
        nxt = gS if nxt is None else torch.where(m[..., None, None], gS, nxt)
        has_next = selh[:, c:].any(1)
        val = (writes[c].detach() * nxt).sum((-1, -2))
        val = torch.where(has_next, val, torch.zeros_like(val))
        out[:, c] = val if invalid_blocks else torch.where(m, val, torch.zeros_like(val))
    return out.view(B, NT, HN, H // HN).sum(-1)


def attn_grads(q, k, v, sel_attn, do, *, nbs=64, scale=None, own_chunk=True, reference_compat=False):
    """Gradients of the softmax branch, o = softmax(mask(scale q k^T)) v, with respect to q, k, v.
    ``reference_compat``: the own-chunk entries of the score-gradient matrix are dropped (they still count in the
    normaliser and in delta = rowsum(do * o)), as the reference's backward does for the default settings.
    Also returns ``dnats`` [B,TN,HN], column 0 of the reference's: sum of the score gradients of the keys of a
    selected block over the queries of later blocks, summed over the heads of a selection group."""
    B, T, HQ, K = q.shape
    HKV = k.shape[2]
    G = HQ // HKV
    if scale is None:
        scale = K ** -0.5
    mask = oattn.attn_mask(sel_attn, T, nbs, HQ, own_chunk=own_chunk)          # [B,HQ,T,T]
    qh = q.permute(0, 2, 1, 3)
    kh = k.permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
    vh = v.permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
    doh = do.permute(0, 2, 1, 3)
    s = (qh @ kh.transpose(-1, -2)) * scale
    s = s.masked_fill(~mask, float("-inf"))
    valid = mask.any(-1, keepdim=True)
    p = torch.softmax(s, -1)
    p = torch.where(valid, p, torch.zeros_like(p))
    o = p @ vh
    delta = (doh * o).sum(-1, keepdim=True)
    dp = doh @ vh.transpose(-1, -2)
    ds = p * (dp - delta)                                                      # gradient w.r.t. the scaled scores
    blk = torch.arange(T) // nbs
    past = (torch.arange(T)[:, None] >= (blk[None, :] + 1) * nbs)[None, None]  # key block entirely before the query
    p_used, ds_used = (torch.where(past, p, torch.zeros_like(p)), torch.where(past, ds, torch.zeros_like(ds))) \
        if reference_compat else (p, ds)
    dq = (ds_used @ kh) * scale
    dk = (ds_used.transpose(-1, -2) @ qh) * scale
    dv = p_used.transpose(-1, -2) @ doh
    fold = lambda x: x.view(B, HKV, G, T, -1).sum(2).permute(0, 2, 1, 3).contiguous()
    TN, HN = sel_attn.shape[1], sel_attn.shape[2]
    ds_past = torch.where(past, ds, torch.zeros_like(ds)).sum(2)               # [B,HQ,T]: per key, over later queries
    pad = TN * nbs - T
    if pad:
        ds_past = torch.cat([ds_past, torch.zeros(B, HQ, pad, dtype=ds.dtype)], -1)
    per_block = ds_past.view(B, HQ, TN, nbs).sum(-1)                           # [B,HQ,TN]
    per_block = per_block.view(B, HN, HQ // HN, TN).sum(2).permute(0, 2, 1)    # [B,TN,HN]
    dnats = torch.where(sel_attn.to(torch.bool), per_block, torch.zeros_like(per_block))
    return dict(dq=dq.permute(0, 2, 1, 3).contiguous(), dk=fold(dk), dv=fold(dv), dnats=dnats)
