"""Plain, slow restatement of the Femolix design: one function per mechanism, whole sequences, no cache, no batching.
Shares no code with gllm_b200. `weights` maps checkpoint names to tensors; `cfg` is the parsed config.json.

    block:     x <- norm1(alpha x + mixer(x));  x <- norm2(alpha x + ff(x))        (norm after the sum)
    delta:     gated delta rule with short convolutions on q / k / v, unit-length q / k, per-head decay and write gate
    parallel:  lambda_l * chunk-masked rotary softmax attention  +  lambda_r * constant-decay linear attention
    ff:        gated SiLU feed-forward, dense or a top-k mixture (softmax over the chosen logits)
    logits:    cap * tanh(head . norm(x) / cap)
"""
import math

import torch
import torch.nn.functional as F


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def short_conv_silu(x, w):
    """x [T, C], w [C, taps]; output t = silu(sum_j w[:, j] * x[t - (taps - 1) + j]), zeros before the start."""
    t, c = x.shape
    taps = w.shape[1]
    xp = torch.cat([x.new_zeros(taps - 1, c), x], 0)
    acc = x.new_zeros(t, c)
    for j in range(taps):
        acc = acc + xp[j:j + t] * w[:, j]
    return F.silu(acc)


def delta_mixer(h, w, p, m, eps):
    t = h.shape[0]
    nh, g, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv_silu(h @ w[p + "q"].T, w[p + "q.conv"]).reshape(t, g, d)
    k = short_conv_silu(h @ w[p + "k"].T, w[p + "k.conv"]).reshape(t, g, d)
    v = short_conv_silu(h @ w[p + "v"].T, w[p + "v.conv"]).reshape(t, nh, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                             # [T, H]
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * F.softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    gate = F.silu(h @ w[p + "g"].T).reshape(t, nh, dv)
    out = h.new_zeros(t, nh, dv)
    for hd in range(nh):
        kv = hd // (nh // g)
        s = h.new_zeros(d, dv)
        for i in range(t):
            s = decay[i, hd] * s
            u = beta[i, hd] * (v[i, hd] - s.T @ k[i, kv])
            s = s + torch.outer(k[i, kv], u)
            out[i, hd] = s.T @ q[i, kv]
    out = rms(out, eps) * w[p + "norm"] * gate
    return out.reshape(t, nh * dv) @ w[p + "o"].T


def rotate(x, pos, dims, base):
    """x [T, heads, D]: the first `dims` entries rotate, entry i pairs with i + dims / 2."""
    half = dims // 2
    freq = base ** (-2.0 * torch.arange(half, dtype=x.dtype) / dims)
    ang = pos.to(x.dtype)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], -1)


def chunk_attention(h, w, p, m, eps):
    t = h.shape[0]
    nh, g, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(t, nh, d)
    k = (h @ w[p + "k"].T).reshape(t, g, d)
    v = (h @ w[p + "v"].T).reshape(t, g, dv)
    q = rms(q, eps) * w[p + "q.norm"]
    k = rms(k, eps) * w[p + "k.norm"]
    pos = torch.arange(t)
    q = rotate(q, pos, m["rot"]["dims"], m["rot"]["base"])
    k = rotate(k, pos, m["rot"]["dims"], m["rot"]["base"])
    size = m["mask"]["size"]
    i, j = pos[:, None], pos[None, :]
    seen = (j <= i) & (i // size == j // size)
    out = h.new_zeros(t, nh, dv)
    for hd in range(nh):
        kv = hd // (nh // g)
        sc = (q[:, hd] @ k[:, kv].T) * m["scale"]
        sc = sc.masked_fill(~seen, float("-inf"))
        out[:, hd] = torch.softmax(sc, -1) @ v[:, kv]
    return out.reshape(t, nh * dv) @ w[p + "o"].T


def decay_linear_attention(h, w, p, m, eps):
    t = h.shape[0]
    nh, d, dv = m["heads"], m["dim"], m["vdim"]
    q = F.silu(h @ w[p + "q"].T).reshape(t, nh, d)
    k = F.silu(h @ w[p + "k"].T).reshape(t, nh, d)
    v = F.silu(h @ w[p + "v"].T).reshape(t, nh, dv)
    out = h.new_zeros(t, nh, dv)
    for hd in range(nh):
        s = h.new_zeros(d, dv)
        for i in range(t):
            s = m["decay"][hd] * s + torch.outer(k[i, hd], v[i, hd])
            out[i, hd] = s.T @ q[i, hd]
    out = rms(out.reshape(t, nh * dv), eps) * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps):
    return m["left_scale"] * chunk_attention(h, w, p + "left.", m["left"], eps) + \
        m["right_scale"] * decay_linear_attention(h, w, p + "right.", m["right"], eps)


def gated_ff(h, w, p):
    return (F.silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def mixture_ff(h, w, p, mlp):
    z = h @ w[p + "router"].T
    top = mlp["router"]["top"]
    val, idx = torch.topk(z, top, dim=-1)
    wt = torch.softmax(val, -1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            out[t] += wt[t, j] * gated_ff(h[t:t + 1], w, "%se%d." % (p, e))[0]
    return out


def forward(cfg, weights, tokens, dtype=torch.float64, trace=None):
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, L in enumerate(cfg["layers"]):
        p = "l%d." % i
        if L["type"] == "delta":
            y = delta_mixer(x, w, p + "mix.", L["mixer"], eps)
        elif L["type"] == "parallel":
            y = parallel_mixer(x, w, p + "mix.", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = rms(alpha * x + y, eps) * w[p + "norm1"]
        mlp = L.get("mlp")
        if mlp is not None:
            y = gated_ff(x, w, p + "mlp.") if mlp["kind"] == "dense" else mixture_ff(x, w, p + "mlp.", mlp)
            x = rms(alpha * x + y, eps) * w[p + "norm2"]
        if trace is not None:
            trace.append(x.clone())
    z = (rms(x, eps) * w["final.norm"]) @ w["head"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(z / cap) if cap else z
