"""CPU oracle for the layer-level SRWM calls (TEST INFRASTRUCTURE, not product code).

Restates, in plain differentiable PyTorch on the CPU, what the reference's layers do around
the SRWM operator, so that the fused layer-level entry points can be checked against it:

* ``srwm_layer``     the core of ``SRWMlayer.forward`` (supervised_learning/layer.py:156-209)
                     and ``SRlayer.forward`` (reinforcement_learning/torchbeast/layer.py:378-421):
                     optional softmax over the head dimension of the input, the carried state
                     stored as a SHIFT from the slow weights (``W_bc = shift + W.repeat(bsz)``),
                     the SRWM recurrence, and the new shift ``W_L - W.repeat(bsz)``.
* ``srwm_unroll_detached``  the learner's unroll (reinforcement_learning/torchbeast_procgen/
                     model.py:1180-1197): one step per call, the state multiplied by
                     ``notdone`` before every step and DETACHED after it (layer.py:412-421).
* ``delta_layer``    the preparation in ``FastFFlayer.forward`` (supervised_learning/layer.py:66-96,
                     reinforcement_learning/torchbeast/layer.py:136-176): the four-way split of
                     the slow net's rows, sigmoid, ``elu + 1`` and the sum normalisation (with
                     the agents' 1e-5 in the denominator, layer.py:30-33), then the delta rule.

The recurrence itself is ``srwm_oracle.srwm_loop`` / ``delta_loop`` (pinned against the reference's
own self test).  Parity pin of these wrappers: ``oracle/pin_reference_layers.py`` runs the
reference's own layer classes (``SRWMlayer``, both ``FastFFlayer`` s, ``SRlayer`` under the learner's
loop) on the CPU in float64 and stores every tensor of those runs under ``tests/golden/layer_*.pt``;
``tests/test_layer_golden.py`` checks the functions below against them (outputs to 1e-10, all
gradients to 1e-9).

Only ``tests/`` may import this module.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from srwm_oracle import delta_loop, srwm_loop


def srwm_layer(x, base, shift=None, input_softmax=True):
    """x [N,H,L,E] (raw activations when ``input_softmax``); base = (W_y, W_q, W_k, w_b) with
    batch size 1 (``[1,H,E,.]``); shift = optional 4 tensors ``[N,H,E,.]``.

    layer.py:162-163 (softmax), :166-177 (shift + repeat), :179-182 (operator),
    :200-204 (new shift).  Returns (out [N,H,L,E], new shift (4 tensors)).
    """
    N = x.shape[0]
    if input_softmax:
        x = F.softmax(x, dim=-1)
    W = [b.repeat(N, 1, 1, 1) for b in base]
    if shift is not None:
        W = [s + w for s, w in zip(shift, W)]
    out, WL = srwm_loop(x, *W)
    new_shift = tuple(wl - b.repeat(N, 1, 1, 1) for wl, b in zip(WL, base))
    return out, new_shift


def srwm_unroll_detached(x, base, shift, done, input_softmax=True):
    """The learner's unroll: x [N,H,T,E], done [N,T] (bool / 0-1), shift = 4 tensors [N,H,E,.].

    Per step t (model.py:1180-1197): ``shift = notdone_t * shift``; one-step layer call with
    ``state = shift`` (layer.py:392-397); the returned state is detached (layer.py:412-421).
    Returns (out [N,H,T,E], final shift (detached)).
    """
    N, H, T, E = x.shape
    shift = [s.detach() for s in shift]
    outs = []
    for t in range(T):
        nd = (1.0 - done[:, t].to(x.dtype)).view(N, 1, 1, 1)
        shift = [nd * s for s in shift]
        o, shift = srwm_layer(x[:, :, t:t + 1, :], base, shift, input_softmax=input_softmax)
        shift = [s.detach() for s in shift]
        outs.append(o)
    return torch.cat(outs, dim=2), tuple(shift)


def delta_layer(qkvb, W0, norm_eps=0.0):
    """qkvb [N,H,L,3E+1] raw rows (q | k | v | b); W0 [N,H,E,E].
    layer.py:74-79 (split, sigmoid), :86-90 (elu + 1, sum normalisation), :96 (operator).
    Returns (out [N,H,L,E], final W)."""
    E = (qkvb.shape[-1] - 1) // 3
    q, k, v, b = torch.split(qkvb, (E, E, E, 1), -1)
    b = torch.sigmoid(b)
    q = F.elu(q, 1.0, False) + 1.0
    k = F.elu(k, 1.0, False) + 1.0
    q = q / (q.sum(-1, keepdim=True) + norm_eps)
    k = k / (k.sum(-1, keepdim=True) + norm_eps)
    return delta_loop(q, k, v, b, W0)

