"""Helpers of the Femolix tests: small random checkpoints on disk, the replay session, comparisons."""
import json
import os

import numpy as np
import torch

import femolix_oracle as oracle
from conftest import scratch_dir


def delta(heads=4, kv_heads=2, dim=8, vdim=12, conv=3, mlp=None):
    return {"type": "delta", "mixer": {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim},
            "mlp": mlp}


def parallel(heads=4, kv_heads=2, dim=12, vdim=20, chunk=7, rot=8, base=50.0, scale=0.3, rheads=3, rdim=10, rvdim=6,
             decay=(0.5, 0.9, 0.99), ls=1.3, rs=0.7, mlp=None):
    return {"type": "parallel",
            "mixer": {"left": {"dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim, "mask": {"size": chunk},
                               "rot": {"base": base, "dims": rot}, "scale": scale},
                      "right": {"decay": list(decay), "dim": rdim, "heads": rheads, "vdim": rvdim},
                      "left_scale": ls, "right_scale": rs},
            "mlp": mlp}


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=16):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def make_config(layers, vocab=67, width=24, alpha=1.7, cap=9.0, eps=1e-5):
    return {"architecture": "Femolix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "postln_alpha": alpha,
            "logit_softcap": cap, "layers": layers}


def random_weights(cfg, seed=0):
    """name -> bf16-representable fp32 tensor, in checkpoint naming."""
    g = torch.Generator().manual_seed(seed)
    w = {}

    def rnd(*shape, std=1.0):
        return (torch.randn(*shape, generator=g) * std).bfloat16().float()

    wd, v = cfg["width"], cfg["vocab"]
    w["embed"] = rnd(v, wd, std=1.0)
    w["head"] = rnd(v, wd, std=3.0 * wd ** -0.5)
    w["final.norm"] = 1 + rnd(wd, std=0.2)

    def lin(name, out, inp, gain=1.0):
        w[name] = rnd(out, inp, std=gain * inp ** -0.5)

    for i, L in enumerate(cfg["layers"]):
        p, m = "l%d." % i, L["mixer"]
        w[p + "norm1"] = 1 + rnd(wd, std=0.2)
        if L["type"] == "delta":
            h, g_, d, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            for n, rows in (("q", g_ * d), ("k", g_ * d), ("v", h * dv)):
                lin(p + "mix." + n, rows, wd, 2.0)
                w[p + "mix." + n + ".conv"] = rnd(rows, taps, std=0.6)
            lin(p + "mix.g", h * dv, wd)
            lin(p + "mix.b", h, wd, 2.0)
            lin(p + "mix.a", h, wd, 2.0)
            w[p + "mix.A_log"] = rnd(h, std=0.7)
            w[p + "mix.dt_bias"] = rnd(h, std=1.0)
            w[p + "mix.norm"] = 1 + rnd(dv, std=0.3)
            lin(p + "mix.o", wd, h * dv, 2.0)
        else:
            l, r = m["left"], m["right"]
            h, g_, d, dv = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
            lin(p + "mix.left.q", h * d, wd, 2.0)
            lin(p + "mix.left.k", g_ * d, wd, 2.0)
            lin(p + "mix.left.v", g_ * dv, wd, 2.0)
            w[p + "mix.left.q.norm"] = 1 + rnd(d, std=0.3)
            w[p + "mix.left.k.norm"] = 1 + rnd(d, std=0.3)
            lin(p + "mix.left.o", wd, h * dv, 2.0)
            rh, rd, rv = r["heads"], r["dim"], r["vdim"]
            lin(p + "mix.right.q", rh * rd, wd, 2.0)
            lin(p + "mix.right.k", rh * rd, wd, 2.0)
            lin(p + "mix.right.v", rh * rv, wd, 2.0)
            lin(p + "mix.right.g", rh * rv, wd)
            w[p + "mix.right.norm"] = 1 + rnd(rh * rv, std=0.3)
            lin(p + "mix.right.o", wd, rh * rv, 2.0)
        mlp = L["mlp"]
        if mlp:
            w[p + "norm2"] = 1 + rnd(wd, std=0.2)
            if mlp["kind"] == "dense":
                lin(p + "mlp.gate", mlp["ff"], wd, 2.0)
                lin(p + "mlp.up", mlp["ff"], wd, 2.0)
                lin(p + "mlp.down", wd, mlp["ff"], 2.0)
            else:
                lin(p + "mlp.router", mlp["router"]["experts"], wd, 4.0)
                for e in range(mlp["router"]["experts"]):
                    f = mlp["expert"]["ff"]
                    lin("%smlp.e%d.gate" % (p, e), f, wd, 2.0)
                    lin("%smlp.e%d.up" % (p, e), f, wd, 2.0)
                    lin("%smlp.e%d.down" % (p, e), wd, f, 2.0)
    return {k: t.bfloat16().float() for k, t in w.items()}     # exactly what the bf16 checkpoint holds


def save_model(cfg, weights):
    from safetensors.torch import save_file
    d = scratch_dir("femolix_")
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


def run_plan(sess, reqs, plan):
    """plan: steps of [(request, n tokens)]; -> {request: logits of all its tokens}"""
    at = {k: 0 for k in reqs}
    got = {k: [] for k in reqs}
    for step in plan:
        entries, end = [], []
        for k, n in step:
            entries.append({"id": k, "tokens": reqs[k][at[k]:at[k] + n], "want": list(range(n))})
            at[k] += n
            if at[k] == len(reqs[k]):
                end.append(k)
        out = sess.step(entries, end)
        o = 0
        for k, n in step:
            got[k].append(out[o:o + n])
            o += n
    assert all(at[k] == len(reqs[k]) for k in reqs)
    return {k: np.concatenate(v, 0) for k, v in got.items()}
