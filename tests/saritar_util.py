"""Helpers of the Saritar tests: small random checkpoints on disk, the replay session, comparisons."""
import json
import os

import numpy as np
import torch

import saritar_oracle as oracle
from conftest import scratch_dir


def attn(heads=4, kv_heads=2, dim=16, window=7, scale=0.25):
    return {"type": "attention", "mixer": {"dim": dim, "vdim": dim, "heads": heads, "kv_heads": kv_heads,
                                           "mask": {"size": window}, "scale": scale}, "mlp": None}


def mamba(inner=24, state=5, dt_rank=3, conv=3):
    return {"type": "mamba1", "mixer": {"conv": conv, "dt_rank": dt_rank, "inner": inner, "state": state}, "mlp": None}


def with_mlp(layer, ff=40):
    return {**layer, "mlp": {"kind": "dense", "ff": ff}}


def make_config(layers, vocab=61, width=24, loop=None, embed_scale=2.0, eps=1e-5):
    cfg = {"architecture": "Saritar", "vocab": vocab, "width": width, "embedding": {"scale": embed_scale},
           "norm": {"eps": eps}, "layers": layers}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def random_weights(cfg, seed=0):
    """name -> bf16-representable fp32 tensor, in checkpoint naming."""
    g = torch.Generator().manual_seed(seed)
    w = {}

    def rnd(*shape, std=1.0):
        return (torch.randn(*shape, generator=g) * std).bfloat16().float()

    wd, v = cfg["width"], cfg["vocab"]
    w["embed"] = rnd(v, wd, std=0.5)
    w["head"] = rnd(v, wd, std=wd ** -0.5)
    w["final.norm"] = 1 + rnd(wd, std=0.2)
    for i, L in enumerate(cfg["layers"]):
        p, m = "l%d." % i, L["mixer"]
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if L["mlp"] else ()):
            w[p + n] = 1 + rnd(wd, std=0.2)
        if L["type"] == "attention":
            h, g_, d = m["heads"], m["kv_heads"], m["dim"]
            w[p + "mix.q"] = rnd(h * d, wd, std=wd ** -0.5)
            w[p + "mix.k"] = rnd(g_ * d, wd, std=wd ** -0.5)
            w[p + "mix.q.norm"] = 1 + rnd(d, std=0.3)
            w[p + "mix.k.norm"] = 1 + rnd(d, std=0.3)
            w[p + "mix.sink"] = rnd(h, std=1.0)
            w[p + "mix.o"] = rnd(wd, h * d, std=(h * d) ** -0.5)
        else:
            c, n, r, t = m["inner"], m["state"], m["dt_rank"], m["conv"]
            w[p + "mix.in"] = rnd(2 * c, wd, std=wd ** -0.5)
            w[p + "mix.conv"] = rnd(c, t, std=0.5)
            w[p + "mix.conv.b"] = rnd(c, std=0.3)
            w[p + "mix.x"] = rnd(r + 2 * n, c, std=c ** -0.5)
            w[p + "mix.dt"] = rnd(c, r, std=r ** -0.5)
            w[p + "mix.dt.b"] = rnd(c, std=1.0) - 1.0
            w[p + "mix.A_log"] = rnd(c, n, std=0.7)
            w[p + "mix.D"] = rnd(c, std=1.0)
            w[p + "mix.o"] = rnd(wd, c, std=c ** -0.5)
        if L["mlp"]:
            w[p + "mlp.up"] = rnd(L["mlp"]["ff"], wd, std=wd ** -0.5)
            w[p + "mlp.down"] = rnd(wd, L["mlp"]["ff"], std=L["mlp"]["ff"] ** -0.5)
    return {k: v.bfloat16().float() for k, v in w.items()}     # exactly what the bf16 checkpoint holds


def save_model(cfg, weights):
    from safetensors.torch import save_file
    d = scratch_dir("saritar_")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.bfloat16().contiguous() for k, v in weights.items()}, os.path.join(d, "model.safetensors"))
    return d


def session(path, dtype="float32", device="cpu", max_tokens=256, page_size=4, state_slots=4):
    from gllm_b200.entrypoints.trace_run import TraceSession
    return TraceSession(path, dtype, max_tokens, device, page_size, state_slots)


def expected_logits(cfg, weights, tokens):
    return oracle.forward(cfg, weights, tokens, torch.float64).float().numpy()


def rel_err(got, want):
    """root mean square of the difference over the vocabulary (means removed) / rms of the expected row, worst row"""
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return float((np.sqrt((d ** 2).mean(-1)) / (np.sqrt((w ** 2).mean(-1)) + 1e-9)).max())


def run_chunks(sess, rid, tokens, cuts):
    """Feed `tokens` of request `rid` alone in portions of the sizes `cuts` (the rest one by one); all logits."""
    outs, at = [], 0
    sizes = list(cuts)
    while at < len(tokens):
        n = min(sizes.pop(0) if sizes else 1, len(tokens) - at)
        end = [rid] if at + n == len(tokens) else []
        outs.append(sess.step([{"id": rid, "tokens": tokens[at:at + n], "want": list(range(n))}], end))
        at += n
    return np.concatenate(outs, 0)
