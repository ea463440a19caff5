"""Sliding-window grouped-query attention over the paged cache with an optional softmax sink.

Mechanism (parameters, so other designs can use it):
  * per-head RMS norm of queries and keys with one weight vector shared by all heads (`qk_norm`);
  * no positional rotation — scores depend on content only;
  * `window`: position i attends to j with 0 <= i - j < window (None = the whole past);
  * `use_sink`: one learned logit per query head joins the softmax denominator and carries no value;
  * `values="key"`: there is no value projection, the values are the keys as projected (before their norm). The
    K cache holds the normed keys and the V cache the raw keys, so the attention kernel itself is an ordinary
    paged K/V attention.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from gllm_b200.layers import functional as Fn


class SinkWindowAttention(nn.Module):
    uses_pages = True
    state_shapes = None

    def __init__(self, hidden: int, heads: int, kv_heads: int, dim: int, scale: float, window: Optional[int],
                 eps: float, dtype, device, use_sink: bool = True, qk_norm: bool = True, values: str = "key"):
        super().__init__()
        assert values == "key", "only key-valued attention is implemented"
        assert heads % kv_heads == 0, (heads, kv_heads)
        self.hidden, self.heads, self.kv_heads, self.dim = hidden, heads, kv_heads, dim
        self.scale, self.window, self.eps = float(scale), window, eps

        def par(*shape, dt=dtype):
            return nn.Parameter(torch.zeros(*shape, dtype=dt, device=device), requires_grad=False)

        self.qk_w = par((heads + kv_heads) * dim, hidden)        # [q rows ; k rows]
        self.q_norm_w = par(dim) if qk_norm else None
        self.k_norm_w = par(dim) if qk_norm else None
        self.sink = par(heads, dt=torch.float32) if use_sink else None
        self.o_w = par(hidden, heads * dim)

    def cache_entry(self):
        return {"kind": "kv", "heads": self.kv_heads, "dim": self.dim}

    def forward(self, inp, h: torch.Tensor, cache, run_id: int) -> torch.Tensor:
        qk = Fn.linear_any(h, self.qk_w)
        hd = self.heads * self.dim
        if cache is None:      # memory probe without a cache
            return Fn.linear_any(qk[:, :hd].contiguous(), self.o_w)
        kc, vc = cache.k_cache[run_id], cache.v_cache[run_id]
        q = Fn.qk_norm_kv_write(qk, self.heads, self.kv_heads, self.dim, self.q_norm_w, self.k_norm_w, self.eps,
                                kc, vc, inp.slot_mapping)
        a = Fn.window_attention(q, kc, vc, inp, self.scale, self.heads, self.dim, self.window, self.sink)
        return Fn.linear_any(a, self.o_w)


class RotaryChunkCore(nn.Module):
    """Grouped-query softmax attention over the paged cache with
      * per-head RMS norm of q and k (weights shared by the heads), applied before the rotation;
      * rotary positions on the first `rot_dims` entries of each head, entry i paired with i + rot_dims / 2;
      * a mask made of the causal rule and, optionally, a sliding `window` and / or a `chunk`: position i sees j only
        if floor(i / chunk) == floor(j / chunk), chunks counted from the start of the sequence;
      * values of their own width `v_dim`.
    A core in the sense of layers/parallel_mixer.py: it reads [q | k | v] rows of a joint projection."""
    uses_pages, uses_state = True, False
    in_names = ("q", "k", "v")

    def __init__(self, heads: int, kv_heads: int, dim: int, v_dim: int, scale: float, rot_dims: int, rot_base: float,
                 chunk: Optional[int], window: Optional[int], eps: float, dtype, device, qk_norm: bool = True):
        super().__init__()
        assert heads % kv_heads == 0, (heads, kv_heads)
        assert rot_dims % 2 == 0 and rot_dims <= dim, (rot_dims, dim)
        self.heads, self.kv_heads, self.dim, self.v_dim = heads, kv_heads, dim, v_dim
        self.scale, self.rot_dims, self.rot_base, self.chunk, self.window, self.eps = \
            float(scale), int(rot_dims), float(rot_base), chunk, window, eps
        self.in_rows = (heads * dim, kv_heads * dim, kv_heads * v_dim)
        self.n_in, self.n_out = sum(self.in_rows), heads * v_dim
        self.q_norm_w = nn.Parameter(torch.zeros(dim, dtype=dtype, device=device), requires_grad=False) if qk_norm \
            else None
        self.k_norm_w = nn.Parameter(torch.zeros(dim, dtype=dtype, device=device), requires_grad=False) if qk_norm \
            else None

    def cache_entry(self):
        return {"kind": "kv", "heads": self.kv_heads, "dim": self.dim, "vdim": self.v_dim}

    def core(self, inp, proj, cache, run_id, out, out_scale=1.0):
        if cache is None:      # memory probe without a cache
            out.zero_()
            return out
        kc, vc = cache.k_cache[run_id], cache.v_cache[run_id]
        q = Fn.qk_norm_rope_kv_write(proj, self.heads, self.kv_heads, self.dim, self.v_dim, self.q_norm_w,
                                     self.k_norm_w, self.eps, inp.positions, self.rot_dims, self.rot_base, kc, vc,
                                     inp.slot_mapping)
        return Fn.masked_attention(q, kc, vc, inp, self.scale, self.heads, self.dim, self.v_dim, self.window,
                                   self.chunk, None, out_scale, out)

    def load_extra(self, reader, pre, put):
        if self.q_norm_w is not None:
            put(self.q_norm_w, reader.get(pre + "q.norm"))
            put(self.k_norm_w, reader.get(pre + "k.norm"))
