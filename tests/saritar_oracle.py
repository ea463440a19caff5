"""Plain, slow fp64/fp32 restatement of the Saritar layer equations, one function per mechanism.

Shares no code with the product path (gllm_b200): plain torch tensor arithmetic only, whole sequences at once,
no cache, no batching. The tests compare the engine against these functions.

Notation: x [T, W] residual stream of one sequence, h the normed input of a sublayer.
"""
import math

import torch


def rms(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def sink_window_attention(h, p, heads, kv_heads, dim, scale, window, eps):
    """Sliding-window GQA whose values are the un-normed keys, RMS-normed q/k, no positional rotation, one
    learned sink logit per head in the softmax denominator."""
    t = h.shape[0]
    q = (h @ p["q"].T).view(t, heads, dim)
    k = (h @ p["k"].T).view(t, kv_heads, dim)
    v = k.clone()
    q = rms(q, p["q.norm"], eps)
    k = rms(k, p["k.norm"], eps)
    rep = heads // kv_heads
    out = torch.zeros(t, heads, dim, dtype=h.dtype)
    i = torch.arange(t)
    d = i[:, None] - i[None, :]
    allowed = (d >= 0) & (d < window)
    for hd in range(heads):
        g = hd // rep
        s = (q[:, hd] @ k[:, g].T) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        m = torch.maximum(s.max(-1).values, p["sink"][hd].expand(t))
        e = torch.exp(s - m[:, None])
        den = e.sum(-1) + torch.exp(p["sink"][hd] - m)
        out[:, hd] = (e / den[:, None]) @ v[:, g]
    return out.reshape(t, heads * dim) @ p["o"].T


def mamba1(h, p, inner, state, dt_rank, taps):
    """Selective scan with a causal depthwise convolution in front, token by token."""
    t = h.shape[0]
    xz = h @ p["in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    xp = torch.cat([torch.zeros(taps - 1, inner, dtype=h.dtype), x], 0)
    xc = torch.zeros_like(x)
    for j in range(taps):
        xc = xc + xp[j:j + t] * p["conv"][:, j]
    xc = xc + p["conv.b"]
    xc = xc * torch.sigmoid(xc)
    proj = xc @ p["x"].T
    dt, b, c = proj[:, :dt_rank], proj[:, dt_rank:dt_rank + state], proj[:, dt_rank + state:]
    dt = torch.nn.functional.softplus(dt @ p["dt"].T + p["dt.b"])
    a = -torch.exp(p["A_log"])
    s = torch.zeros(inner, state, dtype=h.dtype)
    ys = []
    for i in range(t):
        s = torch.exp(dt[i][:, None] * a) * s + (dt[i] * xc[i])[:, None] * b[i][None, :]
        ys.append(s @ c[i] + p["D"] * xc[i])
    y = torch.stack(ys) * (z * torch.sigmoid(z))
    return y @ p["o"].T


def relu2_mlp(h, p):
    return torch.relu(h @ p["up"].T) ** 2 @ p["down"].T


def forward(cfg, weights, tokens, dtype=torch.float64, return_layers=False):
    """Logits [T, vocab] of one whole sequence. `weights`: name -> tensor (checkpoint names)."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x0 = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    x = x0.clone()
    layers = cfg["layers"]
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    order = []
    for i in range(loop["start"]):
        order.append((i, False))
    for r in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            order.append((i, r > 0 and i == loop["start"]))
    for i in range(loop["stop"], len(layers)):
        order.append((i, False))
    trace = []
    for i, add_embed in order:
        L = layers[i]
        m = L["mixer"]
        pre = "l%d." % i
        if add_embed:
            x = x + x0
        p = {k[len(pre) + 4:]: v for k, v in w.items() if k.startswith(pre + "mix.")}
        h = rms(x, w[pre + "norm1"], eps)
        if L["type"] == "attention":
            y = sink_window_attention(h, p, m["heads"], m["kv_heads"], m["dim"], m["scale"], m["mask"]["size"], eps)
        elif L["type"] == "mamba1":
            y = mamba1(h, p, m["inner"], m["state"], m["dt_rank"], m["conv"])
        else:
            raise ValueError(L["type"])
        x = x + rms(y, w[pre + "norm1b"], eps)
        if L.get("mlp") is not None:
            pm = {k[len(pre) + 4:]: v for k, v in w.items() if k.startswith(pre + "mlp.")}
            h = rms(x, w[pre + "norm2"], eps)
            x = x + rms(relu2_mlp(h, pm), w[pre + "norm2b"], eps)
        trace.append(x.clone())
    logits = rms(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(trace)) if return_layers else logits
