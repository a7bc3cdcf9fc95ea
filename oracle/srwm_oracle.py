"""CPU oracle for the two recurrent operators (TEST INFRASTRUCTURE, not product code).

This file restates, in plain PyTorch on the CPU, the arithmetic of the reference's
own per-step test loops:

* SRWM:   supervised_learning/self_ref_v0/__init__.py:296-356  (loop used as ground truth
          by the reference's ``__main__`` check) together with the kernel-side facts that the
          loop leaves out: the update is applied at *every* step including the last and the
          final state is written back into the caller's tensors
          (supervised_learning/self_ref_v0/self_ref_v0.cu:317-350, 420-431).
* delta:  supervised_learning/fast_weight/__init__.py:167-191 (ground-truth loop) and
          supervised_learning/fast_weight/fast_weight_cuda.cu:101-169 (saved v_old/v_insert,
          state written back in place).

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference arm of
``bench.py`` may import this module, and only as the checker or as the timed CPU baseline.
The shipped operators never call into it.

Parity pin: ``oracle/pin_reference_main.py`` runs the reference's two ``__main__`` self
tests on the CPU with the functions below standing in for the CUDA extension, so the
reference's own assertions (max relative error < 1e-3 against its autograd loop) are
what validate the explicit forward/backward here; the tensors of those runs are stored
under ``tests/golden/``.

Two families of functions:

``*_loop``       differentiable per-step loops (gradients by torch.autograd) -- the
                 authoritative semantics; O(L) graph, use for small/medium sizes.
``*_explicit``   hand-written forward + reverse-time backward (the recipe the CUDA
                 kernels implement: rebuild W_{t-1} by undoing the rank-1 update),
                 batched over (N, H); no autograd graph, so usable at larger sizes.

All functions work in the dtype of their inputs (use float64 for tolerance checks,
float32 for timing).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------------------
# SRWM
# --------------------------------------------------------------------------------------

def srwm_loop(x, W_y, W_q, W_k, w_b, update_last=True):
    """Differentiable per-step SRWM loop.

    Shapes: x [N,H,L,E]; W_y,W_q,W_k [N,H,E,E]; w_b [N,H,E,4].
    Row-vector convention: ``out[m] = sum_e v[e] * W[e][m]``
    (supervised_learning/self_ref_v0/self_ref_v0.cu:150,170-172).
    Returns (out [N,H,L,E], (W_y,W_q,W_k,w_b) after the last step).
    ``update_last=False`` reproduces the reference loop exactly (it skips the update at
    the last position, __init__.py:321); outputs are identical either way.
    """
    N, H, L, E = x.shape
    Wy, Wq, Wk, wb = W_y, W_q, W_k, w_b
    outs = []
    for t in range(L):
        xt = x[:, :, t, :].unsqueeze(2)                      # [N,H,1,E]
        y = torch.matmul(xt, Wy).squeeze(2)
        outs.append(y)
        if t == L - 1 and not update_last:
            break
        q = F.softmax(torch.matmul(xt, Wq).squeeze(2), dim=-1)
        k = F.softmax(torch.matmul(xt, Wk).squeeze(2), dim=-1)
        beta = torch.sigmoid(torch.matmul(xt, wb).squeeze(2))  # [N,H,4]
        dqk = (q - k).unsqueeze(2)                            # [N,H,1,E]
        kcol = k.unsqueeze(3)                                 # [N,H,E,1]
        y_ins = beta[..., 0:1] * torch.matmul(dqk, Wy).squeeze(2)
        q_ins = beta[..., 1:2] * torch.matmul(dqk, Wq).squeeze(2)
        k_ins = beta[..., 2:3] * torch.matmul(dqk, Wk).squeeze(2)
        b_ins = beta[..., 3:4] * torch.matmul(dqk, wb).squeeze(2)
        Wy = Wy + kcol * y_ins.unsqueeze(2)
        Wq = Wq + kcol * q_ins.unsqueeze(2)
        Wk = Wk + kcol * k_ins.unsqueeze(2)
        wb = wb + kcol * b_ins.unsqueeze(2)
    return torch.stack(outs, dim=2), (Wy, Wq, Wk, wb)


def srwm_forward_explicit(x, W_y, W_q, W_k, w_b):
    """Forward pass that also produces what the kernel saves for backward.

    Returns dict with out, q, k, beta (post-sigmoid), y_diff, q_diff, k_diff, beta_diff
    (the ``q.W - k.W`` differences, self_ref_v0.cu:374-385,403-406) and the final state.
    Inputs are not modified.
    """
    N, H, L, E = x.shape
    Wy, Wq, Wk, wb = W_y.clone(), W_q.clone(), W_k.clone(), w_b.clone()
    out = x.new_empty(N, H, L, E)
    qs = x.new_empty(N, H, L, E)
    ks = x.new_empty(N, H, L, E)
    betas = x.new_empty(N, H, L, 4)
    yd = x.new_empty(N, H, L, E)
    qd = x.new_empty(N, H, L, E)
    kd = x.new_empty(N, H, L, E)
    bd = x.new_empty(N, H, L, 4)
    for t in range(L):
        xt = x[:, :, t, :].unsqueeze(2)
        out[:, :, t] = torch.matmul(xt, Wy).squeeze(2)
        q = F.softmax(torch.matmul(xt, Wq).squeeze(2), dim=-1)
        k = F.softmax(torch.matmul(xt, Wk).squeeze(2), dim=-1)
        beta = torch.sigmoid(torch.matmul(xt, wb).squeeze(2))
        dqk = (q - k).unsqueeze(2)
        dy = torch.matmul(dqk, Wy).squeeze(2)
        dq = torch.matmul(dqk, Wq).squeeze(2)
        dk = torch.matmul(dqk, Wk).squeeze(2)
        db = torch.matmul(dqk, wb).squeeze(2)
        kcol = k.unsqueeze(3)
        Wy += kcol * (beta[..., 0:1] * dy).unsqueeze(2)
        Wq += kcol * (beta[..., 1:2] * dq).unsqueeze(2)
        Wk += kcol * (beta[..., 2:3] * dk).unsqueeze(2)
        wb += kcol * (beta[..., 3:4] * db).unsqueeze(2)
        qs[:, :, t], ks[:, :, t], betas[:, :, t] = q, k, beta
        yd[:, :, t], qd[:, :, t], kd[:, :, t], bd[:, :, t] = dy, dq, dk, db
    return dict(out=out, q=qs, k=ks, beta=betas, y_diff=yd, q_diff=qd, k_diff=kd,
                beta_diff=bd, W_y=Wy, W_q=Wq, W_k=Wk, w_b=wb)


def srwm_backward_explicit(x, q, k, beta, y_diff, q_diff, k_diff, beta_diff, grad_out,
                           W_y, W_q, W_k, w_b, grad_state=None):
    """Reverse-time SRWM backward that rebuilds W_{t-1} by undoing the rank-1 updates.

    ``W_*`` are the FINAL states (what the forward left in the caller's tensors).
    ``grad_state`` = optional (gWy,gWq,gWk,gwb): gradient flowing into the returned final
    state (stateful variant); the result is the mathematically correct dL/dW_0 (the
    reference's stateful backward double-counts the incoming gradient,
    supervised_learning/self_ref_v0/__init__.py:182-210 with self_ref_v0.cu:676,1213).
    Follows self_ref_v0.cu:694-1187 block by block.  Returns
    (grad_x, grad_W_y, grad_W_q, grad_W_k, grad_w_b, (W_y0, W_q0, W_k0, w_b0)).
    """
    N, H, L, E = x.shape
    W = [W_y.clone(), W_q.clone(), W_k.clone(), w_b.clone()]
    if grad_state is None:
        G = [torch.zeros_like(w) for w in W]
    else:
        G = [g.clone() for g in grad_state]
    diffs = [y_diff, q_diff, k_diff, beta_diff]
    gx = torch.zeros_like(x)
    for t in range(L - 1, -1, -1):
        xt, qt, kt, bt = x[:, :, t], q[:, :, t], k[:, :, t], beta[:, :, t]
        g = grad_out[:, :, t]
        kcol, krow = kt.unsqueeze(3), kt.unsqueeze(2)
        gq = torch.zeros_like(qt)
        gk = torch.zeros_like(kt)
        gb_pre = x.new_zeros(N, H, 4)
        for z in range(4):
            bz = bt[..., z:z + 1]                         # [N,H,1]
            dz = diffs[z][:, :, t]                        # [N,H,Mz]
            ins = bz * dz
            r = torch.matmul(krow, G[z]).squeeze(2)       # sum_e k[e] G[e][m]   (old G)
            gk = gk + torch.matmul(G[z], ins.unsqueeze(3)).squeeze(3)
            gb_pre[..., z] = (r * dz).sum(-1) * (bz * (1 - bz)).squeeze(-1)
            W[z] = W[z] - kcol * ins.unsqueeze(2)         # undo update -> W_{t-1}
            gd = bz * r
            G[z] = G[z] + (qt - kt).unsqueeze(3) * gd.unsqueeze(2)
            u = torch.matmul(W[z], gd.unsqueeze(3)).squeeze(3)
            gq = gq + u
            gk = gk - u
        gq_pre = qt * (gq - (gq * qt).sum(-1, keepdim=True))
        gk_pre = kt * (gk - (gk * kt).sum(-1, keepdim=True))
        pre = [g, gq_pre, gk_pre, gb_pre]
        gxt = torch.zeros_like(xt)
        for z in range(4):
            gxt = gxt + torch.matmul(W[z], pre[z].unsqueeze(3)).squeeze(3)
            G[z] = G[z] + xt.unsqueeze(3) * pre[z].unsqueeze(2)
        gx[:, :, t] = gxt
    return gx, G[0], G[1], G[2], G[3], tuple(W)


# --------------------------------------------------------------------------------------
# Delta rule
# --------------------------------------------------------------------------------------

def delta_loop(Q, K, V, beta, W0):
    """Differentiable per-step delta-rule loop.

    Shapes: Q,K [N,H,L,E]; V [N,H,L,M]; beta [N,H,L,1] (post-sigmoid); W0 [N,H,E,M].
    ``v_old = k.W ; ins = beta*(v - v_old) ; W += k^T ins ; out = q.W`` with the
    POST-update W (supervised_learning/fast_weight/__init__.py:186-191; the reference loop
    stores the transpose [M,E], the kernel [E,M] -- fast_weight_cuda.cu:97,108-109).
    Returns (out [N,H,L,M], W_L).
    """
    N, H, L, E = Q.shape
    W = W0
    outs = []
    for t in range(L):
        kt = K[:, :, t]
        v_old = torch.matmul(kt.unsqueeze(2), W).squeeze(2)
        ins = beta[:, :, t] * (V[:, :, t] - v_old)
        W = W + kt.unsqueeze(3) * ins.unsqueeze(2)
        outs.append(torch.matmul(Q[:, :, t].unsqueeze(2), W).squeeze(2))
    return torch.stack(outs, dim=2), W


def delta_forward_explicit(Q, K, V, beta, W0):
    """Forward that also returns the kernel's saved tensors v_old / v_insert
    (fast_weight_cuda.cu:146-168) and the final state."""
    N, H, L, E = Q.shape
    M = V.shape[-1]
    W = W0.clone()
    out = Q.new_empty(N, H, L, M)
    v_old = Q.new_empty(N, H, L, M)
    v_ins = Q.new_empty(N, H, L, M)
    for t in range(L):
        kt = K[:, :, t]
        vo = torch.matmul(kt.unsqueeze(2), W).squeeze(2)
        ins = beta[:, :, t] * (V[:, :, t] - vo)
        W += kt.unsqueeze(3) * ins.unsqueeze(2)
        out[:, :, t] = torch.matmul(Q[:, :, t].unsqueeze(2), W).squeeze(2)
        v_old[:, :, t], v_ins[:, :, t] = vo, ins
    return dict(out=out, v_old=v_old, v_insert=v_ins, W=W)


def delta_backward_explicit(Q, K, V, beta, v_old, v_insert, grad_out, W_final):
    """Single-pass reverse-time delta-rule backward (the reference does the same math
    in two kernels, fast_weight_cuda.cu:489-552 and :336-389).  ``W_final`` is W_L; the
    initial state W_0 is rebuilt and returned (the reference restores it in place,
    fast_weight_cuda.cu:391).  Returns (gQ, gK, gV, gbeta, W_0, dL/dW_0); the reference's
    autograd function discards dL/dW_0 (fast_weight/__init__.py:96 returns None)."""
    N, H, L, E = Q.shape
    W = W_final.clone()
    G = torch.zeros_like(W)
    gQ, gK = torch.zeros_like(Q), torch.zeros_like(K)
    gV, gB = torch.zeros_like(V), torch.zeros_like(beta)
    for t in range(L - 1, -1, -1):
        qt, kt, g = Q[:, :, t], K[:, :, t], grad_out[:, :, t]
        bt = beta[:, :, t]                                  # [N,H,1]
        ins = v_insert[:, :, t]
        G = G + qt.unsqueeze(3) * g.unsqueeze(2)
        gQ[:, :, t] = torch.matmul(W, g.unsqueeze(3)).squeeze(3)
        r = torch.matmul(kt.unsqueeze(2), G).squeeze(2)     # [N,H,M]
        gV[:, :, t] = bt * r
        gvo = -bt * r
        gB[:, :, t] = (r * (V[:, :, t] - v_old[:, :, t])).sum(-1, keepdim=True)
        gk = torch.matmul(G, ins.unsqueeze(3)).squeeze(3)
        W = W - kt.unsqueeze(3) * ins.unsqueeze(2)          # -> W_{t-1}
        gk = gk + torch.matmul(W, gvo.unsqueeze(3)).squeeze(3)
        gK[:, :, t] = gk
        G = G + kt.unsqueeze(3) * gvo.unsqueeze(2)
    return gQ, gK, gV, gB, W, G


# --------------------------------------------------------------------------------------
# helpers shared by tests / bench
# --------------------------------------------------------------------------------------

def max_relative_error(a, b, eps=1e-6):
    """The reference's own parity metric (self_ref_v0/__init__.py:232-233)."""
    return float(torch.abs((b - a) / (torch.abs(b) + eps)).max().item())


def rel_l2(a, b):
    """||a-b|| / ||b||, a scale-free whole-tensor error (robust to near-zero entries)."""
    a = a.double()
    b = b.double()
    return float((a - b).norm() / (b.norm() + 1e-300))


def rel_max(a, b):
    """max|a-b| / max|b|."""
    a = a.double()
    b = b.double()
    return float((a - b).abs().max() / (b.abs().max() + 1e-300))


def rel_elem(a, b, floor=1e-3):
    """Element-wise relative error max |a-b| / |b| over the elements with |b| > floor * max|b|:
    the reference's metric (self_ref_v0/__init__.py:232-233) with its absolute 1e-6 guard replaced
    by a floor relative to the tensor's scale, so that it means the same for tensors of any scale."""
    a = a.double()
    b = b.double()
    m = b.abs() > floor * b.abs().max()
    if not bool(m.any()):
        return 0.0
    return float(((a - b).abs()[m] / b.abs()[m]).max())
