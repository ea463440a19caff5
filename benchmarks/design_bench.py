"""Prefill / decode throughput of the Saritar design beside the closest existing decoder (Qwen3: GQA attention with
q/k norm + gated MLP) at matched width, depth and parameter count, through the public `LLM.generate` API with
random weights, plus the device time of each new kernel against its roofline and against the like kernel of the
existing path. Invoked as `python bench.py --design saritar` (the default benchmark is untouched).

Prints ONE JSON line: {"design": ..., "sizes": [{"width", ..., "saritar": {...}, "qwen3": {...}}], "kernels": [...]}
"""
from __future__ import annotations

import json
import os
import time

import torch


def _saritar_cfg(width, n_pairs, heads, kv, dim, window, ff, vocab):
    att = {"type": "attention", "mixer": {"dim": dim, "vdim": dim, "heads": heads, "kv_heads": kv,
                                          "mask": {"size": window}, "scale": dim ** -0.5},
           "mlp": {"kind": "dense", "ff": ff}}
    mam = {"type": "mamba1", "mixer": {"conv": 4, "dt_rank": width // 16, "inner": 2 * width, "state": 16},
           "mlp": None}
    return {"architecture": "Saritar", "vocab": vocab, "width": width, "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-5}, "layers": [att, mam] * n_pairs, "loop": {"start": 0, "stop": 0, "times": 1}}


def _qwen3_cfg(width, layers, heads, kv, dim, inter, vocab):
    return {"architectures": ["Qwen3ForCausalLM"], "hidden_size": width, "num_hidden_layers": layers,
            "num_attention_heads": heads, "num_key_value_heads": kv, "head_dim": dim, "intermediate_size": inter,
            "vocab_size": vocab, "rms_norm_eps": 1e-6, "rope_theta": 1e6, "max_position_embeddings": 8192,
            "tie_word_embeddings": False, "torch_dtype": "bfloat16"}


def _throughput(cfg, vocab, warmup, steps):
    from gllm_b200.engine.llm_engine import LLM
    llm = LLM(cfg, load_format="dummy", maxp=8192, maxd=256, max_cuda_graph_bs=64, model_max_length=4096,
              enable_prefix_caching=False, log_stats=False, launch_mode="inproc", num_gpu_pages=4096,
              num_state_slots=64)
    params = sum(p.numel() for p in llm.worker.runner.model.parameters())
    g = torch.Generator().manual_seed(0)

    def prompts(n, length):
        return [torch.randint(0, vocab, (length,), generator=g).tolist() for _ in range(n)]

    res = {"params_m": round(params / 1e6, 1)}
    for name, n, plen, olen in (("prefill", 16, 2048, 1), ("decode", 64, 16, 128)):
        best = None
        for it in range(warmup + steps):
            ps = prompts(n, plen)                      # fresh ids every pass
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            llm.generate(tokens=ps, output_lens=[olen] * n, temperature=0.0, top_k=1)
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            if it >= warmup:
                best = dt if best is None else min(best, dt)
        tok = n * plen if name == "prefill" else n * olen
        res[name + "_tok_s"] = round(tok / best, 1)
    llm.worker.runner.close()
    llm.worker.runner.kv_cache = llm.worker.runner.model = None
    del llm
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    return res


def _time(fn, iters=10):
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(3):
        fn()
    tot = 0.0
    for _ in range(iters):
        flush.zero_()                                   # L2 flush between timed launches
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        tot += a.elapsed_time(b)
    return tot / iters


def _kernels(peaks):
    """Device time of the new kernels at layer-like sizes; bytes are the algorithmic minimum."""
    from gllm_b200.ops import ref, sm100, sm100_seq as S
    dev, bf = "cuda", torch.bfloat16
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    out = []

    def row(name, ms, nbytes, like=None):
        r = {"kernel": name, "ms": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 1),
             "frac_hbm": round(nbytes / ms / 1e6 / hbm, 3)}
        if like:
            r["like"] = like
        out.append(r)

    T, W = 8192, 4096
    x = torch.randn(T, W, device=dev)
    y, w1, w2 = torch.randn(T, W, device=dev).to(bf), torch.ones(W, device=dev).to(bf), torch.ones(W, device=dev).to(bf)
    row("resid_norm (post-norm + add + pre-norm, fp32 stream)", _time(lambda: S.resid_norm(x, y, w1, None, w2, 1e-5, bf)),
        T * W * (4 + 4 + 2 + 2))
    res = torch.randn(T, W, device=dev).to(bf)
    row("rmsnorm + residual (existing bf16 path)", _time(lambda: sm100.rmsnorm(y, w1, 1e-5, res)), T * W * (2 + 2 + 2 + 2),
        like="resid_norm")
    C, N, R = 8192, 16, 256
    for label, qlens in (("prefill 4 x 2048", [2048] * 4), ("decode 256 x 1", [1] * 256)):
        Tt, B = sum(qlens), len(qlens)
        qsl = torch.tensor([0] + torch.tensor(qlens).cumsum(0).tolist(), dtype=torch.int32, device=dev)
        sl = torch.tensor([q + 100 for q in qlens], dtype=torch.int32, device=dev)
        rs = torch.arange(B, dtype=torch.int32, device=dev)
        xz = torch.randn(Tt, 2 * C, device=dev).to(bf)
        cw, cb = torch.randn(C, 4, device=dev), torch.randn(C, device=dev)
        cs = torch.zeros(B, 3, C, device=dev).to(bf)
        xc = S.causal_conv_silu(xz, C, cw, cb, cs, rs, sl, qsl)
        row("conv_silu " + label, _time(lambda: S.causal_conv_silu(xz, C, cw, cb, cs, rs, sl, qsl)),
            Tt * C * 4 + B * 3 * C * 4)
        proj, dtr = torch.randn(Tt, R + 2 * N, device=dev).to(bf), torch.randn(Tt, C, device=dev).to(bf)
        A, Dk, db = -torch.rand(C, N, device=dev), torch.randn(C, device=dev), torch.randn(C, device=dev)
        ss = torch.zeros(B, N, C, device=dev)
        row("selective_scan " + label,
            _time(lambda: S.selective_scan(xc, dtr, proj, xz, A, Dk, db, ss, rs, sl, qsl, C, N, R)),
            Tt * C * 2 * 4 + B * N * C * 8)
    H, G, D, ps = 32, 8, 128, 16
    for label, qlens, ctx, win in (("prefill 4 x 2048, window 1024", [2048] * 4, 0, 1024),
                                   ("decode 256 x 1 at 2048, window 1024", [1] * 256, 2047, 1024)):
        Tt, B = sum(qlens), len(qlens)
        qsl = torch.tensor([0] + torch.tensor(qlens).cumsum(0).tolist(), dtype=torch.int32, device=dev)
        sl = torch.tensor([q + ctx for q in qlens], dtype=torch.int32, device=dev)
        npp = (max(qlens) + ctx + ps - 1) // ps
        bt = torch.arange(B * npp, dtype=torch.int32, device=dev).reshape(B, npp)
        kshape = ref.kv_cache_shape(B * npp + 1, G, D, ps)
        kc, vc = torch.randn(kshape, device=dev).to(bf), torch.randn(kshape, device=dev).to(bf)
        pos = torch.cat([torch.arange(ctx, ctx + q) for q in qlens]).to(torch.int32).to(dev)
        q = torch.randn(Tt, H * D, device=dev).to(bf)
        sink = torch.zeros(H, device=dev)
        keys = sum(min(p + 1, win) for ql in qlens for p in range(ctx, ctx + ql))
        nd = B if qlens[0] == 1 else 0
        ms = _time(lambda: S.window_attention(q, kc, vc, bt, sl, qsl, pos, D ** -0.5, H, D, win, sink,
                                              num_decode_seqs=nd, max_q_len=max(qlens)), iters=5)
        r = {"kernel": "window_attention " + label, "ms": round(ms, 4),
             "tflops": round(4.0 * keys * H * D / ms / 1e9, 2)}
        ms2 = _time(lambda: sm100.paged_attention(q, kc, vc, bt, sl, qsl, D ** -0.5, H, D,
                                                  B if qlens[0] == 1 else 0, B, max(qlens), max(qlens) + ctx), iters=3)
        full = sum(p + 1 for ql in qlens for p in range(ctx, ctx + ql))
        r["like"] = {"kernel": "paged_attention (existing, full causal)", "ms": round(ms2, 4),
                     "tflops": round(4.0 * full * H * D / ms2 / 1e9, 2)}
        out.append(r)
    return out


def run(args):
    peaks = {}
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            peaks = json.load(f)
    vocab = 32000
    kernels = _kernels(peaks)
    sizes = []
    for width, pairs, heads, kv in ((1024, 4, 8, 2), (2048, 4, 16, 4), (4096, 2, 32, 8)):
        s_cfg = _saritar_cfg(width, pairs, heads, kv, 128, 1024, 4 * width, vocab)
        q_cfg = _qwen3_cfg(width, 2 * pairs, heads, kv, 128, 3 * width, vocab)
        sizes.append({"width": width, "layers": 2 * pairs,
                      "saritar": _throughput(s_cfg, vocab, args.warmup, args.steps),
                      "qwen3": _throughput(q_cfg, vocab, args.warmup, args.steps)})
    line = {"design": "saritar", "dtype": "bf16", "data": "synthetic", "warmup": args.warmup, "steps": args.steps,
            "timing": "wall clock around LLM.generate with synchronize (sizes); CUDA events, L2 flushed (kernels)",
            "peaks": peaks, "sizes": sizes, "kernels": kernels}
    print(json.dumps(line))
    return line
