"""The reference's SRWM and delta-rule layers on top of the fused layer-level calls.

Same constructor arguments, parameter names (so a reference ``state_dict`` loads) and
``forward`` signatures as

* ``SRWMlayer``    supervised_learning/layer.py:112-209
* ``SRlayer``      reinforcement_learning/torchbeast/layer.py:340-421
* ``FastFFlayer``  supervised_learning/layer.py:49-108 (``norm_eps=0``, fresh zero fast weights
                   per call) and reinforcement_learning/torchbeast/layer.py:127-189
                   (``FastFFlayerRL``: ``norm_eps=1e-5``, fast weights carried as state)

but the per-call work around the operator -- input softmax, four ``W.repeat(bsz,1,1,1)``,
``shift + repeat``, the ``[L,B,H*d] -> [B,H,L,d]`` layout change and back, the four
``W_bc - W.repeat`` subtractions; for the delta rule the four-way split of the slow net's rows,
``elu + 1``, the sum normalisation and the sigmoid -- is done inside the kernels
(``layer_ops.srwm_layer`` / ``layer_ops.delta_layer``).
``SRlayer.unroll`` additionally runs the learner's one-step-at-a-time loop with episode
resets (reinforcement_learning/torchbeast_procgen/model.py:1180-1197) as ONE call.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from .layer_ops import delta_layer, srwm_layer


def _heads(h, num_head, dim_head):
    """[L, B, H*d] -> the [B, H, L, d] view the operator reads in place."""
    slen, bsz, _ = h.shape
    return h.reshape(slen, bsz, num_head, dim_head).permute(1, 2, 0, 3)


def _merge(out):
    """[B, H, L, d] laid out like the input view -> [L, B, H*d] (a view, no copy)."""
    bsz, num_head, slen, dim_head = out.shape
    return out.transpose(1, 2).reshape(bsz, slen, num_head * dim_head).transpose(0, 1)


class SRWMlayer(nn.Module):
    """Self-referential weight matrix layer of the supervised-learning models."""

    def __init__(self, num_head, dim_head, in_dim, dropout, use_ln=True, use_input_softmax=False,
                 beta_init=-1.0, stateful=False):
        super().__init__()
        self.num_head, self.dim_head, self.in_dim = num_head, dim_head, in_dim
        self.use_ln, self.use_input_softmax, self.stateful = use_ln, use_input_softmax, stateful
        self.W_y = nn.Parameter(torch.empty(1, num_head, dim_head, dim_head))
        self.W_q = nn.Parameter(torch.empty(1, num_head, dim_head, dim_head))
        self.W_k = nn.Parameter(torch.empty(1, num_head, dim_head, dim_head))
        self.w_b = nn.Parameter(torch.empty(1, num_head, dim_head, 4))
        if use_ln:
            self.layer_norm = nn.LayerNorm(in_dim)
        self.out_linear = nn.Linear(num_head * dim_head, in_dim, bias=False)
        self.drop = nn.Dropout(dropout)
        self.reset_parameters(beta_init)

    def reset_parameters(self, beta_init):
        std = 1.0 / math.sqrt(self.dim_head)
        for w in (self.W_y, self.W_q, self.W_k):
            nn.init.normal_(w, mean=0.0, std=std)
        nn.init.normal_(self.w_b, mean=beta_init, std=std)

    def forward(self, h, state=None, get_state=False):
        x = _heads(h, self.num_head, self.dim_head)
        # stateful: gradients flow through the carried state (stateful_self_ref_v0); otherwise
        # the returned state carries none, as with the reference's in-place mutated buffers
        out, shift = srwm_layer(x, self.W_y, self.W_q, self.W_k, self.w_b, shift=state,
                                input_softmax=self.use_input_softmax)
        out = self.drop(self.out_linear(_merge(out)))
        out = (self.layer_norm(h) if self.use_ln else h) + out
        if get_state:
            if not self.stateful:
                shift = tuple(s.detach() for s in shift)
            return out, shift
        return out


class SRlayer(nn.Module):
    """Self-referential weight matrix layer of the reinforcement-learning agents: the input
    softmax is always on, the state (shift from the slow weights) is required and comes
    back detached."""

    def __init__(self, num_head, dim_head, in_dim, dropout):
        super().__init__()
        self.num_head, self.dim_head, self.in_dim = num_head, dim_head, in_dim
        self.W_y = nn.Parameter(torch.empty(1, num_head, dim_head, dim_head))
        self.W_q = nn.Parameter(torch.empty(1, num_head, dim_head, dim_head))
        self.W_k = nn.Parameter(torch.empty(1, num_head, dim_head, dim_head))
        self.w_b = nn.Parameter(torch.empty(1, num_head, dim_head, 4))
        self.layer_norm = nn.LayerNorm(in_dim)
        self.out_linear = nn.Linear(num_head * dim_head, in_dim, bias=False)
        self.drop = nn.Dropout(dropout)
        self.reset_rec_parameters()

    def reset_rec_parameters(self):
        std = 1.0 / math.sqrt(self.dim_head)
        for w in (self.W_y, self.W_q, self.W_k, self.w_b):
            nn.init.normal_(w, mean=0.0, std=std)

    def forward(self, h, state=None):
        assert state is not None
        x = _heads(h, self.num_head, self.dim_head)
        out, shift = srwm_layer(x, self.W_y, self.W_q, self.W_k, self.w_b, shift=state, input_softmax=True)
        out = h + self.drop(self.out_linear(_merge(out)))
        return out, tuple(s.detach() for s in shift)

    def unroll(self, h, done, state):
        """The learner's loop over ``h [T, B, D]`` with ``done [T, B]`` as one call: before
        step t the state of the samples with ``done[t]`` goes back to zero, every step sees a
        detached state.  Returns (out [T, B, D], state after the last step)."""
        assert state is not None
        x = _heads(h, self.num_head, self.dim_head)
        out, shift = srwm_layer(x, self.W_y, self.W_q, self.W_k, self.w_b, shift=state, done=done.t(),
                                input_softmax=True, detach_state=True)
        out = h + self.drop(self.out_linear(_merge(out)))
        return out, shift


class FastFFlayer(nn.Module):
    """Delta-rule fast-weight layer of the supervised-learning models: layer norm, slow net,
    then -- in one call on the slow net's raw rows -- the q/k/beta preparation and the
    recurrence, starting from zero fast weights."""

    norm_eps = 0.0

    def __init__(self, num_head, dim_head, in_dim, dropout):
        super().__init__()
        self.num_head, self.dim_head, self.in_dim = num_head, dim_head, in_dim
        self.slow_net = nn.Linear(in_dim, num_head * (3 * dim_head + 1), bias=False)
        self.layer_norm = nn.LayerNorm(in_dim)
        self.out_linear = nn.Linear(num_head * dim_head, in_dim, bias=False)
        self.drop = nn.Dropout(dropout)

    def _rows(self, x):
        slen, bsz, _ = x.shape
        qkvb = self.slow_net(self.layer_norm(x))
        return qkvb.view(slen, bsz, self.num_head, 3 * self.dim_head + 1).permute(1, 2, 0, 3)

    def forward(self, x):
        rows = self._rows(x)
        W = torch.empty(rows.shape[0], self.num_head, self.dim_head, self.dim_head, device=x.device)
        out = delta_layer(rows, W, norm_eps=self.norm_eps, zero_init=True)
        return x + self.drop(self.out_linear(_merge(out)))


class FastFFlayerRL(FastFFlayer):
    """The agents' variant: 1e-5 in the normalisers, the fast weights are the carried state
    (given, updated in place by the call, returned as a copy)."""

    norm_eps = 1e-5

    def forward(self, x, state=None):
        assert state is not None
        out = delta_layer(self._rows(x), state, norm_eps=self.norm_eps)
        return x + self.drop(self.out_linear(_merge(out))), state.clone()

