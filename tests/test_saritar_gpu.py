"""Saritar on the sm_100a kernels: every kernel of csrc/seq against its unfused PyTorch form, and the engine
scenarios of test_saritar_cpu.py (chunking, mixed batches, page / slot re-use, generation, CUDA-graph decode) against
the plain oracle, in fp32 (tight) and bf16 (rounding-sized tolerance)."""
import numpy as np
import pytest
import torch

import saritar_oracle as oracle
import saritar_util as U
from test_saritar_cpu import CONFIGS, toks

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOLS = {"float32": 2e-4, "bfloat16": 6e-2}


def close(a, b, tol):
    return (a.float() - b.float()).abs().max().item() <= tol * (b.float().abs().max().item() + 1e-9)


@pytest.mark.parametrize("dt,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
def test_kernels_against_unfused_ops(dt, tol):
    from gllm_b200.ops import ref, sm100_seq as S
    torch.manual_seed(0)
    T, W = 37, 200
    x = torch.randn(T, W, device=DEV)
    y, wp, wq = (torch.randn(*s, device=DEV).to(dt) for s in ((T, W), (W,), (W,)))
    add = torch.randn(T, W, device=DEV)
    x1, x2 = x.clone(), x.clone()
    assert close(S.resid_norm(x1, y, wp, add, wq, 1e-5, dt), ref.resid_norm(x2, y, wp, add, wq, 1e-5, dt), tol)
    assert close(x1, x2, 1e-5)
    x3 = x.clone()
    assert S.resid_norm(x3, y, wp, None, None, 1e-5, dt) is None and not torch.equal(x3, x)
    for m, k, n in ((45, 72, 50), (1, 10, 3), (130, 192, 768), (3, 384, 64), (70, 64, 192)):
        a, w = torch.randn(m, k, device=DEV).to(dt), torch.randn(n, k, device=DEV).to(dt)
        assert close(S.linear_any(a, w), (a.float() @ w.float().T).to(dt), tol), (m, k, n)
    for D, N, taps in ((48, 24, 4), (64, 16, 2), (8, 1, 1), (128, 40, 3)):
        H, G, ps, win = 6, 2, 16, 20
        qlens, ctx = [5, 1, 30], [17, 40, 0]
        Tt = sum(qlens)
        qsl = torch.tensor([0, 5, 6, 36], dtype=torch.int32, device=DEV)
        sl = torch.tensor([c + q for c, q in zip(ctx, qlens)], dtype=torch.int32, device=DEV)
        kshape = ref.kv_cache_shape(32, G, D, ps)
        kc, vc = torch.randn(kshape, device=DEV).to(dt), torch.randn(kshape, device=DEV).to(dt)
        bt = torch.randperm(31)[:12].reshape(3, 4).to(torch.int32).to(DEV)
        pos = torch.cat([torch.arange(c, c + q) for c, q in zip(ctx, qlens)]).to(torch.int32).to(DEV)
        seqi = torch.cat([torch.full((q,), i) for i, q in enumerate(qlens)]).to(DEV)
        slots = (bt[seqi, (pos // ps).long()] * ps + pos % ps).to(torch.int32)
        qk = torch.randn(Tt, (H + G) * D, device=DEV).to(dt)
        qn, kn = torch.randn(D, device=DEV).to(dt), torch.randn(D, device=DEV).to(dt)
        kc2, vc2 = kc.clone(), vc.clone()
        q1 = S.qk_norm_kv_write(qk, H, G, D, qn, kn, 1e-5, kc, vc, slots)
        q2 = ref.qk_norm_kv_write(qk, H, G, D, qn, kn, 1e-5, kc2, vc2, slots)
        assert close(q1, q2, tol) and close(kc, kc2, tol) and torch.equal(vc, vc2)
        sink = torch.randn(H, device=DEV)
        for wn, sk in ((win, sink), (None, None), (3, sink), (1, None)):
            a1 = S.window_attention(q2, kc2, vc2, bt, sl, qsl, pos, 0.2, H, D, wn, sk)
            a2 = ref.window_attention(q2, kc2, vc2, bt, sl, qsl, 0.2, H, D, wn, sk)
            assert close(a1, a2, tol), (D, wn)
        C, R = 100, 10
        xz = torch.randn(Tt, 2 * C, device=DEV).to(dt)
        cw, cb = torch.randn(C, taps, device=DEV), torch.randn(C, device=DEV)
        cs = torch.randn(5, max(taps - 1, 1), C, device=DEV).to(dt)
        cs2 = cs.clone()
        rs = torch.tensor([3, 0, 2], dtype=torch.int32, device=DEV)
        c1 = S.causal_conv_silu(xz, C, cw, cb, cs, rs, sl, qsl)
        c2 = ref.causal_conv_silu(xz, C, cw, cb, cs2, rs, sl, qsl)
        assert close(c1, c2, tol) and (taps == 1 or torch.equal(cs, cs2))
        proj, dtr = torch.randn(Tt, R + 2 * N, device=DEV).to(dt), torch.randn(Tt, C, device=DEV).to(dt)
        A, Dk, db = -torch.rand(C, N, device=DEV) * 2, torch.randn(C, device=DEV), torch.randn(C, device=DEV)
        ss = torch.randn(5, N, C, device=DEV)
        ss2 = ss.clone()
        y1 = S.selective_scan(c2, dtr, proj, xz, A, Dk, db, ss, rs, sl, qsl, C, N, R)
        y2 = ref.selective_scan(c2, dtr, proj, xz, A, Dk, db, ss2, rs, sl, qsl, C, N, R)
        assert close(y1, y2, tol) and close(ss, ss2, 1e-5)
        assert torch.equal(S.relu2(xz), ref.relu2(xz))


@pytest.mark.parametrize("dt,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("N,C", [(16, 96), (24, 100), (8, 64), (40, 32)])
def test_scan_and_conv_on_long_chunks(dt, tol, N, C):
    """few long sequences take the 4-threads-per-channel scan"""
    from gllm_b200.ops import ref, sm100_seq as S
    torch.manual_seed(2)
    qlens, ctx, R, taps = [70, 33], [0, 9], 6, 4
    Tt = sum(qlens)
    qsl = torch.tensor([0, 70, 103], dtype=torch.int32, device=DEV)
    sl = torch.tensor([c + q for c, q in zip(ctx, qlens)], dtype=torch.int32, device=DEV)
    rs = torch.tensor([1, 0], dtype=torch.int32, device=DEV)
    xz = torch.randn(Tt, 2 * C, device=DEV).to(dt)
    cw, cb = torch.randn(C, taps, device=DEV), torch.randn(C, device=DEV)
    cs = torch.randn(3, taps - 1, C, device=DEV).to(dt)
    cs2 = cs.clone()
    c1 = S.causal_conv_silu(xz, C, cw, cb, cs, rs, sl, qsl)
    c2 = ref.causal_conv_silu(xz, C, cw, cb, cs2, rs, sl, qsl)
    assert close(c1, c2, tol) and torch.equal(cs, cs2)
    proj, dtr = torch.randn(Tt, R + 2 * N, device=DEV).to(dt), torch.randn(Tt, C, device=DEV).to(dt)
    A, Dk, db = -torch.rand(C, N, device=DEV) * 2, torch.randn(C, device=DEV), torch.randn(C, device=DEV)
    ss = torch.randn(3, N, C, device=DEV)
    ss2 = ss.clone()
    y1 = S.selective_scan(c2, dtr, proj, xz, A, Dk, db, ss, rs, sl, qsl, C, N, R)
    y2 = ref.selective_scan(c2, dtr, proj, xz, A, Dk, db, ss2, rs, sl, qsl, C, N, R)
    assert close(y1, y2, tol) and close(ss, ss2, 1e-5)


@pytest.mark.parametrize("D", [64, 128])
def test_window_and_sink_on_the_tensor_core_attention(D):
    """decode rows first, then prompt portions; contexts over several 64-key tiles; windows that end inside, at
    and beyond tile and page borders."""
    from gllm_b200.ops import ref, sm100_seq as S
    torch.manual_seed(1)
    bf, H, G, ps = torch.bfloat16, 8, 2, 16
    qlens, ctx = [1, 1, 1, 70, 5, 200], [0, 63, 300, 130, 64, 0]
    B, Tt = len(qlens), sum(qlens)
    qsl = torch.tensor([0] + torch.tensor(qlens).cumsum(0).tolist(), dtype=torch.int32, device=DEV)
    sl = torch.tensor([c + q for c, q in zip(ctx, qlens)], dtype=torch.int32, device=DEV)
    npp = 20
    bt = torch.randperm(B * npp)[: B * npp].reshape(B, npp).to(torch.int32).to(DEV)
    kshape = ref.kv_cache_shape(B * npp + 1, G, D, ps)
    kc, vc = torch.randn(kshape, device=DEV).to(bf), torch.randn(kshape, device=DEV).to(bf)
    pos = torch.cat([torch.arange(c, c + q) for c, q in zip(ctx, qlens)]).to(torch.int32).to(DEV)
    q = torch.randn(Tt, H * D, device=DEV).to(bf)
    sink = torch.randn(H, device=DEV) * 2
    for wn, sk in ((72, sink), (64, sink), (65, None), (1, sink), (16, None), (None, sink), (None, None), (250, sink)):
        want = ref.window_attention(q, kc, vc, bt, sl, qsl, D ** -0.5, H, D, wn, sk)
        got = S.window_attention(q, kc, vc, bt, sl, qsl, pos, D ** -0.5, H, D, wn, sk, num_decode_seqs=3,
                                 max_q_len=max(qlens))
        plain = S.window_attention(q, kc, vc, bt, sl, qsl, pos, D ** -0.5, H, D, wn, sk, simt=True)
        assert close(got, want, 2e-2), (D, wn, sk is not None)
        assert close(plain, want, 2e-2), (D, wn, sk is not None)


@pytest.fixture(scope="module")
def models():
    out = {}
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        w = U.random_weights(cfg, seed=10 + i)
        out[name] = (cfg, w, U.save_model(cfg, w))
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_chunked_and_decoded_match_oracle(models, name, dtype):
    cfg, w, path = models[name]
    t = toks(45, cfg["vocab"], 2)
    want = U.expected_logits(cfg, w, t)
    s = U.session(path, dtype=dtype, device=DEV)
    for k, cuts in enumerate(([len(t)], [], [2, 2, 3, 17, 2], [30])):
        assert U.rel_err(U.run_chunks(s, "r%d" % k, t, cuts), want) < TOLS[dtype], cuts


def test_engine_on_the_tensor_core_attention_path():
    cfg = U.make_config([U.with_mlp(U.attn(heads=4, kv_heads=2, dim=64, window=40, scale=0.125), ff=96),
                         U.mamba(inner=64, state=16, dt_rank=8, conv=4),
                         U.attn(heads=2, kv_heads=1, dim=128, window=70, scale=0.09)], width=64, loop=(0, 2, 2))
    w = U.random_weights(cfg, seed=77)
    path = U.save_model(cfg, w)
    t = toks(150, cfg["vocab"], 4)
    want = U.expected_logits(cfg, w, t)
    s = U.session(path, dtype="bfloat16", device=DEV, max_tokens=512, page_size=16)
    for k, cuts in enumerate(([len(t)], [100] + [1] * 50, [2, 62, 3, 64, 17, 2])):
        assert U.rel_err(U.run_chunks(s, "r%d" % k, t, cuts), want) < TOLS["bfloat16"], cuts


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_reuse_pages_and_slots(models, dtype):
    cfg, w, path = models["mixed_loop"]
    v = cfg["vocab"]
    reqs = {k: toks(n, v, 20 + i) for i, (k, n) in enumerate([("a", 30), ("b", 9), ("c", 17), ("d", 2), ("e", 26), ("f", 12)])}
    want = {k: U.expected_logits(cfg, w, t) for k, t in reqs.items()}
    s = U.session(path, dtype=dtype, device=DEV, max_tokens=64, page_size=4, state_slots=3)
    at, got = {k: 0 for k in reqs}, {k: [] for k in reqs}
    plan = [[("a", 11), ("b", 9)], [("a", 1), ("c", 5)], [("a", 2), ("c", 1)], [("c", 11), ("a", 16), ("d", 2)],
            [("e", 3)], [("e", 1), ("f", 12)], [("e", 22)]]
    for step in plan:
        entries, end = [], []
        for k, n in step:
            entries.append({"id": k, "tokens": reqs[k][at[k]:at[k] + n], "want": list(range(n))})
            at[k] += n
            if at[k] == len(reqs[k]):
                end.append(k)
        out, o = s.step(entries, end), 0
        for k, n in step:
            got[k].append(out[o:o + n])
            o += n
    for k in reqs:
        assert U.rel_err(np.concatenate(got[k], 0), want[k]) < TOLS[dtype], k


@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_on_the_gpu(models, graphs):
    from gllm_b200.engine.llm_engine import LLM
    cfg, w, path = models["mixed_loop"]
    llm = LLM(path, dtype="float32", page_size=4, maxp=32, maxd=8, num_gpu_pages=64, model_max_length=96,
              log_stats=False, num_state_slots=3, disable_cuda_graph=not graphs, max_cuda_graph_bs=4)
    prompts = [toks(21, cfg["vocab"], 31), toks(3, cfg["vocab"], 32), toks(9, cfg["vocab"], 33)]
    lens = [7, 12, 5]
    seqs = llm.generate(tokens=prompts, output_lens=lens, temperature=0.0, top_k=1)
    if graphs:
        assert llm.worker.runner.stats["graph_steps"] > 0
    for p, n, s in zip(prompts, lens, seqs):
        cur = list(p)
        for _ in range(n):
            cur.append(int(oracle.forward(cfg, w, cur, torch.float64)[-1].argmax()))
        assert s.token_ids == cur
