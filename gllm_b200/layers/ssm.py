"""Recurrent mixers. `Mamba1Mixer`: input projection -> [x | z]; causal depthwise convolution + SiLU on x;
low-rank projection -> [dt | B | C]; dt projection + softplus; diagonal selective state-space recurrence in fp32;
gate by SiLU(z); output projection.

Per-sequence state lives in slot-indexed device tensors owned by the engine's cache (one set per layer run):
the last taps - 1 convolution inputs and the fp32 [state, channels] recurrence matrix. A chunk that starts at
position 0 starts from zeros, any other chunk continues from its slot.
"""
from __future__ import annotations

import torch
from torch import nn

from gllm_b200.layers import functional as Fn


class Mamba1Mixer(nn.Module):
    uses_pages = False

    def __init__(self, hidden: int, inner: int, nstate: int, dt_rank: int, taps: int, dtype, device):
        super().__init__()
        self.hidden, self.inner, self.nstate, self.dt_rank, self.taps = hidden, inner, nstate, dt_rank, taps

        def par(*shape, dt=dtype):
            return nn.Parameter(torch.zeros(*shape, dtype=dt, device=device), requires_grad=False)

        f32 = torch.float32
        self.in_w = par(2 * inner, hidden)
        self.conv_w = par(inner, taps, dt=f32)
        self.conv_b = par(inner, dt=f32)
        self.x_w = par(dt_rank + 2 * nstate, inner)
        self.dt_w = par(inner, dt_rank)
        self.dt_b = par(inner, dt=f32)
        self.a = par(inner, nstate, dt=f32)         # A = -exp(A_log), fp32
        self.d_skip = par(inner, dt=f32)
        self.o_w = par(hidden, inner)

    def cache_entry(self):
        return {"kind": "ssm", "channels": self.inner, "nstate": self.nstate, "taps": self.taps}

    def forward(self, inp, h: torch.Tensor, cache, run_id: int) -> torch.Tensor:
        conv_state = cache.conv_state[run_id] if cache is not None else None
        ssm_state = cache.ssm_state[run_id] if cache is not None else None
        xz = Fn.linear_any(h, self.in_w)
        xc = Fn.causal_conv_silu(xz, self.inner, self.conv_w, self.conv_b, conv_state, inp)
        proj = Fn.linear_any(xc, self.x_w)
        dt_raw = Fn.linear_any(proj[:, : self.dt_rank], self.dt_w)
        y = Fn.selective_scan(xc, dt_raw, proj, xz, self.a, self.d_skip, self.dt_b, ssm_state, inp, self.inner,
                              self.nstate, self.dt_rank)
        return Fn.linear_any(y, self.o_w)
