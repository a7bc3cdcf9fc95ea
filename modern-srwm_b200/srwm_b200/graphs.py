"""CUDA-graph replay of a launch-bound inference step.

An actor step of the reinforcement-learning agents is one tiny kernel per layer (L = 1, a few
dozen sequences) wrapped in a few hundred microseconds of Python and launch overhead
(reinforcement_learning/torchbeast/layer.py:378-421 called once per environment step).
``GraphedSRStep`` captures the step of a stack of ``SRlayer`` + feed-forward blocks once and
replays it: the carried state lives in static buffers that the captured kernels update in
place, the input is copied into a static buffer, the output is read from one.
"""
from __future__ import annotations

import torch

from .layer_ops import srwm_layer_forward
from .layers import _heads, _merge


class GraphedSRStep:
    """One inference step (L = 1) of ``layers`` = [(SRlayer, feed-forward module or None), ...]
    with optional ``pre`` / ``post`` modules, as a CUDA graph.

        step = GraphedSRStep(layers, state, example_input, pre=input_proj)
        out = step(h)            # h: [1, B, in_dim]; the state buffers advance in place

    ``state``: per layer the four shift tensors [B, H, d, .]; they are copied into the graph's
    static buffers, readable (and resettable) through ``step.state``.  The slow weights are
    read at replay time, so parameter updates are seen without re-capturing.
    """

    def __init__(self, layers, state, example_input, pre=None, post=None, warmup=3):
        self.layers, self.pre, self.post = layers, pre, post
        dev = example_input.device
        self.static_in = example_input.detach().clone()
        self.state = [[t.detach().to(torch.float32).contiguous().clone() for t in st] for st in state]
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side), torch.no_grad():
            keep = [[t.clone() for t in st] for st in self.state]
            for _ in range(warmup):          # also sets the kernels' attributes outside the capture
                self._step()
            for st, k in zip(self.state, keep):
                for t, v in zip(st, k):
                    t.copy_(v)
        torch.cuda.current_stream(dev).wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(self.graph):
            self.static_out = self._step()
        # the capture itself does not run the kernels: the state is still the given one

    def _step(self):
        h = self.static_in if self.pre is None else self.pre(self.static_in)
        for (sr, ff), st in zip(self.layers, self.state):
            x = _heads(h, sr.num_head, sr.dim_head)
            out, _, _ = srwm_layer_forward(x, (sr.W_y, sr.W_q, sr.W_k, sr.w_b), st, None, True, save=False,
                                           inplace_state=True)
            h = h + sr.drop(sr.out_linear(_merge(out)))
            if ff is not None:
                h = ff(h)
        return h if self.post is None else self.post(h)

    def __call__(self, h):
        self.static_in.copy_(h)
        self.graph.replay()
        return self.static_out

    def reset(self, mask=None):
        """Zero the carried state (of the samples where ``mask`` [B] is set)."""
        for st in self.state:
            for t in st:
                if mask is None:
                    t.zero_()
                else:
                    t.mul_((~mask).to(t.dtype).view(-1, 1, 1, 1))
