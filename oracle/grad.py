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


def linear_chunk_backward(q, k, v, g, beta, sel, do, dht=None, *, scale=None, h0=None, decay=True, use_l2norm=True,
                          rule="gdn"):
    """The backward of the chunk form written out (block size 64), in the order a kernel pipeline would take
    (the reference's order: src/nats/ops/gated_delta_rule/chunk.py:199-332): recompute the forward per chunk,
    walk the chunks in reverse carrying dS (gradient with respect to the state after the chunk) and the gradient with
    respect to the carried decay, and push every chunk's gradients through the WY transform, the decays and the l2
    normalisation.  No autograd; ``tests/test_oracle_grad.py`` checks it against ``linear_true_grads``.
    -> dict(dq, dk, dv, dg, dbeta, dh0) plus the per-chunk intermediates a kernel test wants:
       dS [B,NT,H,K,V] (gradient w.r.t. the state after chunk c), dvp [B,T,H,V] (gradient w.r.t. v'),
       dw [B,T,H,K], du [B,T,H,V]."""
    B, T, H, K = q.shape
    V = v.shape[-1]
    dt = q.dtype
    assert T % C == 0
    if scale is None:
        scale = K ** -0.5
    NT = T // C
    gdn = rule == "gdn"
    if beta is None:
        beta = torch.ones(B, T, H, dtype=dt)
    q_rstd = torch.rsqrt((q * q).sum(-1) + 1e-6) if use_l2norm else torch.ones(B, T, H, dtype=dt)
    k_rstd = torch.rsqrt((k * k).sum(-1) + 1e-6) if use_l2norm else torch.ones(B, T, H, dtype=dt)
    qn, kn = q * q_rstd[..., None], k * k_rstd[..., None]
    ch = lambda x, D: x.view(B, NT, C, H, D).permute(0, 3, 1, 2, 4)          # [B,H,NT,C,D]
    chs = lambda x: x.view(B, NT, C, H).permute(0, 3, 1, 2)                   # [B,H,NT,C]
    qc, kc, vc, doc = ch(qn, K), ch(kn, K), ch(v, V), ch(do, V)
    gc = chs(g).cumsum(-1)
    bc = chs(beta)
    gam = (gc[..., :, None] - gc[..., None, :]).exp()
    tril_s = torch.tril(torch.ones(C, C, dtype=torch.bool), -1)
    tril_i = torch.tril(torch.ones(C, C, dtype=torch.bool), 0)
    zero = torch.zeros((), dtype=dt)
    kk = kc @ kc.transpose(-1, -2)
    if gdn:
        A = torch.where(tril_s, bc[..., :, None] * kk * gam, zero)
        eye = torch.eye(C, dtype=dt)
        Ai = torch.linalg.solve_triangular(eye + A, eye.expand_as(A).contiguous(), upper=False)
        zu = vc * bc[..., None]                                               # right-hand sides of the WY solve
        zw = kc * (bc * gc.exp())[..., None]
        u, w = Ai @ zu, Ai @ zw
    else:
        u, w = vc, torch.zeros_like(kc)
    qk = qc @ kc.transpose(-1, -2)
    P = torch.where(tril_i, qk * gam, zero)
    gL = gc[..., -1]
    selh = ogdn._expand_sel(sel, H).permute(0, 2, 1)                           # [B,H,NT]
    # ---- forward recurrence: the state and the carry every chunk reads
    S = torch.zeros(B, H, K, V, dtype=dt) if h0 is None else h0.clone()
    carry = torch.zeros(B, H, dtype=dt)
    S_read, carry_read, vps = [], [], []
    last_sel = -1
    for c in range(NT):
        act = selh[..., c]
        S_read.append(S)
        carry_read.append(carry)
        vp = u[:, :, c] - carry.exp()[..., None, None] * (w[:, :, c] @ S)
        vps.append(vp)
        gl = gL[:, :, c]
        kd = (gl[..., None] - gc[:, :, c]).exp() if gdn else torch.clamp(gl[..., None] - gc[:, :, c], max=0.0).exp()
        S_new = (gl + carry).exp()[..., None, None] * S + kc[:, :, c].transpose(-1, -2) @ (vp * kd[..., None])
        S = torch.where(act[..., None, None], S_new, S)
        carry = torch.where(act, torch.zeros_like(carry), carry + gl if decay else carry)
    # ---- reverse walk
    # the final state the forward returns is the state after the last selected chunk of each (b, h)
    idx = torch.arange(NT).view(1, 1, NT)
    last = torch.where(selh, idx, torch.full_like(idx, -1)).amax(-1)          # [B,H], -1 if none
    dS = torch.zeros(B, H, K, V, dtype=dt)
    dcar = torch.zeros(B, H, dtype=dt)                                         # gradient w.r.t. the carry after the chunk
    dh0_extra = torch.zeros(B, H, K, V, dtype=dt)
    if dht is not None:
        dh0_extra = torch.where((last < 0)[..., None, None], dht, dh0_extra)   # no selected chunk: final state = h0
    dqn = torch.zeros_like(qc)
    dkn = torch.zeros_like(kc)
    dvc = torch.zeros_like(vc)
    dgc = torch.zeros_like(gc)                                                 # w.r.t. the chunk-local cumsum
    dbc = torch.zeros_like(bc)
    dS_all = torch.zeros(B, NT, H, K, V, dtype=dt)
    dvp_all, dw_all, du_all = torch.zeros_like(vc), torch.zeros_like(kc), torch.zeros_like(vc)
    for c in range(NT - 1, -1, -1):
        act = selh[..., c]
        a3 = act[..., None, None]
        if dht is not None:
            dS = dS + torch.where((last == c)[..., None, None], dht, torch.zeros_like(dht))
        dS_all[:, c] = dS
        S_c, car = S_read[c], carry_read[c]
        vp, gl, g_c = vps[c], gL[:, :, c], gc[:, :, c]
        ec = car.exp()
        kraw = gl[..., None] - g_c
        kd = kraw.exp() if gdn else torch.clamp(kraw, max=0.0).exp()
        k_c, q_c, do_c = kc[:, :, c], qc[:, :, c], doc[:, :, c]
        # state update (selected chunks): S+ = e^{gl+car} S + k^T (vp * kd)
        kdS = k_c @ dS                                                         # [C,V]
        dvp = torch.where(a3, kdS * kd[..., None], torch.zeros_like(vp))
        dk_c = torch.where(a3, (vp * kd[..., None]) @ dS.transpose(-1, -2), torch.zeros_like(k_c))
        dkd = torch.where(act[..., None], (kdS * vp).sum(-1) * kd, torch.zeros_like(kd))   # w.r.t. log kd
        if not gdn:
            dkd = torch.where(kraw < 0, dkd, torch.zeros_like(dkd))            # clamp(min(.,0)) passes no gradient above 0
        dec = (gl + car).exp()
        ddec = (dS * S_c).sum((-1, -2)) * dec                                  # w.r.t. (gl + car), selected only
        dgl = torch.where(act, ddec + dkd.sum(-1), torch.zeros_like(gl))
        dg_tok = -dkd                                                          # w.r.t. the local cumsum of each token
        dcar_in = torch.where(act, ddec, dcar)                                 # a selected chunk resets the carry
        if decay:
            dgl = dgl + torch.where(act, torch.zeros_like(dcar), dcar)
        dS_prev = torch.where(a3, dec[..., None, None] * dS, dS)
        # output: o = s [ (e^{g+car} q) S + P vp ]
        E = (g_c + car[..., None]).exp()
        dvp = dvp + scale * (P[:, :, c].transpose(-1, -2) @ do_c)
        dP = torch.where(tril_i, scale * (do_c @ vp.transpose(-1, -2)), zero)
        dEq = scale * (do_c @ S_c.transpose(-1, -2))                           # w.r.t. (E q)
        dS_prev = dS_prev + scale * ((q_c * E[..., None]).transpose(-1, -2) @ do_c)
        dq_c = dEq * E[..., None]
        dE = (dEq * q_c).sum(-1) * E                                           # w.r.t. (g + car) per token
        dg_tok = dg_tok + dE
        dcar_in = dcar_in + dE.sum(-1)
        # v' = u - e^{car} w S
        du = dvp
        dw = -ec[..., None, None] * (dvp @ S_c.transpose(-1, -2))
        dS_prev = dS_prev - ec[..., None, None] * (w[:, :, c].transpose(-1, -2) @ dvp)
        dcar_in = dcar_in - ec * ((w[:, :, c] @ S_c) * dvp).sum((-1, -2))
        dvp_all[:, :, c], dw_all[:, :, c], du_all[:, :, c] = dvp, dw, du
        # P = tril(q k^T Gamma)
        dqk = dP * gam[:, :, c]
        dq_c = dq_c + dqk @ k_c
        dk_c = dk_c + dqk.transpose(-1, -2) @ q_c
        dGam = dP * qk[:, :, c] * gam[:, :, c]                                 # w.r.t. (g_i - g_j)
        if gdn:
            # u = Ai zu, w = Ai zw, Ai = (I + A)^-1
            Ai_c = Ai[:, :, c]
            dzu, dzw = Ai_c.transpose(-1, -2) @ du, Ai_c.transpose(-1, -2) @ dw
            dAi = du @ zu[:, :, c].transpose(-1, -2) + dw @ zw[:, :, c].transpose(-1, -2)
            dA = torch.where(tril_s, -(Ai_c.transpose(-1, -2) @ dAi @ Ai_c.transpose(-1, -2)), zero)
            b_c = bc[:, :, c]
            # A = beta_i (k k^T)_ij Gamma_ij
            dkk = dA * b_c[..., :, None] * gam[:, :, c]
            dk_c = dk_c + dkk @ k_c + dkk.transpose(-1, -2) @ k_c
            db = (dA * kk[:, :, c] * gam[:, :, c]).sum(-1)
            dGam = dGam + dA * A[:, :, c]
            # zu = v beta ; zw = k beta e^{g}
            dvc[:, :, c] = dzu * b_c[..., None]
            db = db + (dzu * vc[:, :, c]).sum(-1)
            eg = g_c.exp()
            dk_c = dk_c + dzw * (b_c * eg)[..., None]
            zk = (dzw * k_c).sum(-1)
            db = db + zk * eg
            dg_tok = dg_tok + zk * b_c * eg
            dbc[:, :, c] = db
        else:
            dvc[:, :, c] = du
        dg_tok = dg_tok + dGam.sum(-1) - dGam.sum(-2)
        dg_tok[..., -1] = dg_tok[..., -1] + dgl                                # g_last is the cumsum at the last token
        dgc[:, :, c] = dg_tok
        dqn[:, :, c], dkn[:, :, c] = dq_c, dk_c
        dS, dcar = dS_prev, dcar_in
    dh0 = dS + dh0_extra
    # ---- back through the chunk-local cumsum and the l2 normalisation
    dg = torch.flip(torch.flip(dgc, [-1]).cumsum(-1), [-1])                    # reverse cumsum inside each chunk
    un = lambda x, D: x.permute(0, 2, 3, 1, 4).reshape(B, T, H, D)
    uns = lambda x: x.permute(0, 2, 3, 1).reshape(B, T, H)
    dqn_t, dkn_t = un(dqn, K), un(dkn, K)
    if use_l2norm:
        dq = q_rstd[..., None] * (dqn_t - qn * (dqn_t * qn).sum(-1, keepdim=True))
        dk = k_rstd[..., None] * (dkn_t - kn * (dkn_t * kn).sum(-1, keepdim=True))
    else:
        dq, dk = dqn_t, dkn_t
    return dict(dq=dq, dk=dk, dv=un(dvc, V), dg=uns(dg), dbeta=uns(dbc) if gdn else None,
                dh0=dh0 if h0 is not None else None, dS=dS_all, dvp=un(dvp_all, V), dw=un(dw_all, K), du=un(du_all, V))
