"""Femolix on the sm_100a kernels: every new kernel of csrc/seq against its unfused PyTorch form, and the engine
scenarios of test_femolix_cpu.py (chunking, mixed batches, page / slot re-use, generation, CUDA-graph decode) against
the plain oracle, in fp32 (tight) and bf16 (rounding-sized tolerance)."""
import numpy as np
import pytest
import torch

import femolix_oracle as oracle
import femolix_util as U
from test_femolix_cpu import CONFIGS, _chunk_probe, toks

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL32 = 2e-4


def row_errs(got, want):
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return np.sqrt((d ** 2).mean(-1)) / (np.sqrt((w ** 2).mean(-1)) + 1e-9)


class Expect:
    """What a run is held to. fp32: the oracle, tightly. bf16: the error that rounding alone causes is measured by
    running the unfused PyTorch forms on the CPU with the same rounding points (bf16 weights, activations and cache,
    fp32 accumulation); the kernels may be at most twice as far from the oracle, on the median row and, for models
    without discrete choices, on the worst row. In models with a router, one bf16 rounding can flip a close call
    in these tiny sizes and move every later row by tens of percent on either device: there only the median is held,
    loosely; their exactness is what the fp32 runs and the kernel tests establish."""

    def __init__(self, cfg, w, path, tokens, dtype):
        self.want = U.expected_logits(cfg, w, tokens)
        self.dtype = dtype
        self.routed = any(L["mlp"] and L["mlp"]["kind"] == "moe" and
                          L["mlp"]["router"]["top"] < L["mlp"]["router"]["experts"] for L in cfg["layers"])
        if dtype == "bfloat16":
            s = U.session(path, "bfloat16", "cpu", max_tokens=max(256, len(tokens) + 64), page_size=16)
            got = s.step([{"id": "r", "tokens": tokens, "want": list(range(len(tokens)))}], ["r"])
            self.noise = row_errs(got, self.want)

    def check(self, got):
        e = row_errs(got, self.want)
        if self.dtype == "float32":
            assert e.max() < TOL32
        elif self.routed:
            assert np.median(e) < max(2 * np.median(self.noise), 0.25)
        else:
            assert np.median(e) <= 2 * np.median(self.noise) + 1e-2
            assert e.max() <= 2 * self.noise.max() + 2e-2


def close(a, b, tol):
    return (a.float() - b.float()).abs().max().item() <= tol * (b.float().abs().max().item() + 1e-9)


def _batch(qlens, ctx, ps, pages):
    qsl = torch.tensor([0] + np.cumsum(qlens).tolist(), dtype=torch.int32, device=DEV)
    sl = torch.tensor([c + q for c, q in zip(ctx, qlens)], dtype=torch.int32, device=DEV)
    per = max((c + q + ps - 1) // ps for c, q in zip(ctx, qlens))
    bt = torch.randperm(pages - 1)[: len(qlens) * per].reshape(len(qlens), per).to(torch.int32).to(DEV)
    pos = torch.cat([torch.arange(c, c + q) for c, q in zip(ctx, qlens)]).to(torch.int32).to(DEV)
    seqi = torch.cat([torch.full((q,), i) for i, q in enumerate(qlens)]).to(DEV)
    slots = (bt[seqi, (pos // ps).long()] * ps + pos % ps).to(torch.int32)
    return qsl, sl, bt, pos, slots


@pytest.mark.parametrize("dt,tol", [(torch.float32, 3e-5), (torch.bfloat16, 2e-2)])
def test_kernels_against_unfused_ops(dt, tol):
    from gllm_b200.ops import ref, sm100_seq as S
    torch.manual_seed(0)
    T, W = 37, 200
    x = torch.randn(T, W, device=DEV)
    y, w = torch.randn(T, W, device=DEV).to(dt), (torch.rand(W, device=DEV) + 0.5).to(dt)
    x1, x2 = x.clone(), x.clone()
    h1, h2 = S.postnorm(x1, y, 1.75, w, 1e-5, dt), ref.postnorm(x2, y, 1.75, w, 1e-5, dt)
    assert close(h1, h2, tol) and close(x1, x2, 1e-5)
    gu = torch.randn(T, 2 * 50, device=DEV).to(dt)
    assert close(S.silu_mul(gu), ref.silu_mul(gu), tol)
    z = (torch.randn(T, 77, device=DEV) * 20).to(dt)
    assert close(S.softcap(z.clone(), 12.0), ref.softcap(z, 12.0), tol)
    # router: ids exact (random logits have no near ties), weights close
    hh, wr = torch.randn(T, W, device=DEV).to(dt), torch.randn(11, W, device=DEV).to(dt)
    for k in (1, 2, 11):
        w2, i2 = ref.router_topk(hh, wr, k)
        for path in ("token", "gemm"):
            w1, i1 = S.router_topk(hh, wr, k, force=path)
            assert torch.equal(i1, i2) and close(w1, w2, 1e-4), (k, path)
    if dt == torch.bfloat16:          # tensor-core logits: ragged token and expert counts, two expert tiles
        for tt, ee, ww in ((37, 11, 208), (300, 70, 64), (64, 8, 16), (1000, 64, 512)):
            hb = torch.randn(tt, ww + 16, device=DEV).to(dt)[:, :ww]
            wb = torch.randn(ee, ww, device=DEV).to(dt)
            w2, i2 = ref.router_topk(hb, wb, 2)
            w1, i1 = S.router_topk(hb, wb, 2, force="mma")
            assert torch.equal(i1, i2) and close(w1, w2, 1e-4), (tt, ee, ww)
    # plain experts
    E, F = 5, 24
    w13, w2_ = (torch.randn(E, 2 * F, W, device=DEV) * W ** -0.5).to(dt), (torch.randn(E, W, F, device=DEV) * F ** -0.5).to(dt)
    wt, ids = ref.router_topk(hh, wr[:E], 2)
    assert close(S.routed_experts(hh, w13, w2_, wt, ids), ref.fused_experts(hh, w13, w2_, wt, ids, None), tol)
    # q/k norm + rotation + cache write, then chunk / window attention on the plain kernel, odd head sizes
    for D, Dv, rot in ((40, 72, 24), (8, 4, 6), (64, 64, 32), (20, 36, 0)):
        H, G, ps = 6, 2, 16
        qlens, ctx = [5, 1, 30], [17, 40, 0]
        qsl, sl, bt, pos, slots = _batch(qlens, ctx, ps, 32)
        Tt = sum(qlens)
        kc = torch.randn(ref.kv_cache_shape(32, G, D, ps), device=DEV).to(dt)
        vc = torch.randn(ref.kv_cache_shape(32, G, Dv, ps), device=DEV).to(dt)
        qkv = torch.randn(Tt, H * D + G * D + G * Dv + 8, device=DEV).to(dt)
        qn, kn = torch.randn(D, device=DEV).to(dt), torch.randn(D, device=DEV).to(dt)
        kc2, vc2 = kc.clone(), vc.clone()
        big = pos + 5000                                   # far positions: angles need more than fp32 products
        q1 = S.qk_norm_rope_kv_write(qkv, H, G, D, Dv, qn, kn, 1e-5, big, rot, 5000.0, kc, vc, slots)
        q2 = ref.qk_norm_rope_kv_write(qkv, H, G, D, Dv, qn, kn, 1e-5, big, rot, 5000.0, kc2, vc2, slots)
        assert close(q1, q2, tol) and close(kc, kc2, tol) and torch.equal(vc, vc2)
        sink = torch.randn(H, device=DEV)
        for wn, ch, sk in ((None, 7, None), (None, 16, None), (5, 12, sink), (None, 1, None), (None, None, None)):
            joint = torch.zeros(Tt, H * Dv + 8, device=DEV).to(dt)
            a1 = S.window_attention(q2, kc2, vc2, bt, sl, qsl, pos, 0.2, H, D, wn, sk, chunk=ch, v_dim=Dv,
                                    out_scale=1.2, out=joint[:, 8:])
            a2 = ref.window_attention(q2, kc2, vc2, bt, sl, qsl, 0.2, H, D, wn, sk, chunk=ch, v_dim=Dv, out_scale=1.2)
            assert close(a1, a2, tol), (D, wn, ch)
            assert joint[:, :8].abs().max().item() == 0
    # matrix-state recurrences with carried state, grouped heads, padded value columns
    for Hh, Gq, D, V, delta in ((4, 2, 32, 24, True), (2, 2, 64, 48, False), (3, 1, 5, 3, True), (2, 2, 48, 40, False),
                                (1, 1, 128, 16, True), (2, 1, 128, 40, True), (2, 2, 192, 8, False)):
        # head sizes above 64 take the 8-lanes-per-column form when the chunks are long
        qlens, ctx = ([40, 1, 70], [17, 40, 0]) if (D > 64 and V != 16) else ([5, 1, 30], [17, 40, 0])
        qsl, sl, _, _, _ = _batch(qlens, ctx, 16, 32)
        Tt = sum(qlens)
        rs = torch.tensor([2, 0, 3], dtype=torch.int32, device=DEV)
        q, k = torch.randn(Tt, Gq * D + 3, device=DEV).to(dt), torch.randn(Tt, Gq * D, device=DEV).to(dt)
        v = torch.randn(Tt, Hh * V, device=DEV).to(dt)
        beta, a = torch.randn(Tt, Hh, device=DEV).to(dt), torch.randn(Tt, Hh, device=DEV).to(dt)
        neg_a, dtb = -torch.rand(Hh, device=DEV) * 2, torch.randn(Hh, device=DEV)
        decay = torch.tensor([0.9, 1.0, 0.5, 0.99][:Hh], device=DEV)
        st1 = torch.randn(5, Hh, D, V, device=DEV) * 0.3
        st2 = st1.clone()
        args = (beta, a, neg_a, dtb, None) if delta else (None, None, None, None, decay)
        o1 = S.linear_state_scan(q[:, :Gq * D], k, v, *args, st1, rs, sl, qsl, Hh, Gq, D, V, not delta, delta,
                                 D ** -0.5 if delta else 1.0, delta)
        o2 = ref.linear_state_scan(q[:, :Gq * D], k, v, *args, st2, rs, sl, qsl, Hh, Gq, D, V, not delta, delta,
                                   D ** -0.5 if delta else 1.0, delta)
        assert close(o1, o2, 2e-4), (Hh, D, V, delta)
        assert close(st1, st2, 2e-4)
        assert torch.equal(st1[1], st2[1]) and torch.equal(st1[4], st2[4])      # untouched slots
        gate, nw = torch.randn(Tt, Hh * V + 5, device=DEV).to(dt), torch.randn(V, device=DEV).to(dt)
        for group, wv, act in ((V, nw, "silu"), (Hh * V, torch.randn(Hh * V, device=DEV).to(dt), "sigmoid")):
            joint = torch.zeros(Tt, Hh * V + 2, device=DEV).to(dt)
            g1 = S.gated_group_norm(o2, gate[:, :Hh * V], wv, group, 1e-5, act, 0.5, joint[:, 2:])
            g2 = ref.gated_group_norm(o2, gate[:, :Hh * V], wv, group, 1e-5, act, 0.5, None, dt)
            assert close(g1, g2, tol)


def test_tensor_core_attention_with_chunk_mask_and_strided_output():
    """bf16, head size 64 / 128 with equal value size: the chunk mask runs on the tensor-core kernels (decode and
    prefill) and must agree with the plain kernel and the PyTorch form, also when it writes a scaled column slice."""
    from gllm_b200.ops import ref, sm100_seq as S
    torch.manual_seed(1)
    dt = torch.bfloat16
    for D, ps, ch in ((64, 16, 24), (128, 16, 100), (64, 64, 7), (128, 8, 64)):
        H, G = 8, 2
        for qlens, ctx in (([1, 1, 1], [130, 63, 0]), ([70, 3, 150], [17, 140, 0]), ([1, 1, 90], [99, 5, 31])):
            qsl, sl, bt, pos, _ = _batch(qlens, ctx, ps, 64)
            Tt = sum(qlens)
            nd = sum(1 for q in qlens if q == 1) if qlens[0] == 1 else 0
            nd = nd if all(q == 1 for q in qlens[:nd]) else 0
            kc = torch.randn(ref.kv_cache_shape(64, G, D, ps), device=DEV).to(dt)
            vc = torch.randn(ref.kv_cache_shape(64, G, D, ps), device=DEV).to(dt)
            q = torch.randn(Tt, H * D, device=DEV).to(dt)
            joint = torch.zeros(Tt, H * D + 64, device=DEV).to(dt)
            a1 = S.window_attention(q, kc, vc, bt, sl, qsl, pos, D ** -0.5, H, D, None, None, num_decode_seqs=nd,
                                    max_q_len=max(qlens), chunk=ch, v_dim=D, out_scale=1.2, out=joint[:, 64:])
            a0 = S.window_attention(q, kc, vc, bt, sl, qsl, pos, D ** -0.5, H, D, None, None, simt=True, chunk=ch,
                                    v_dim=D, out_scale=1.2)
            a2 = ref.window_attention(q, kc, vc, bt, sl, qsl, D ** -0.5, H, D, None, None, chunk=ch, v_dim=D,
                                      out_scale=1.2)
            assert close(a0, a2, 2e-2) and close(a1, a2, 2e-2), (D, ps, ch, qlens)
            assert joint[:, :64].abs().max().item() == 0


def test_grouped_gemm_experts_match_plain_experts():
    from gllm_b200.layers.moe import SelectedSoftmaxMoE
    torch.manual_seed(2)
    W, F, E = 384, 128, 8
    m = SelectedSoftmaxMoE(E, 2, W, F, torch.bfloat16, DEV)
    assert m.interleaved
    m.router_w.data.copy_(torch.randn(E, W) * 0.3)
    gates = [torch.randn(F, W) * W ** -0.5 for _ in range(E)]
    ups = [torch.randn(F, W) * W ** -0.5 for _ in range(E)]
    downs = [torch.randn(W, F) * F ** -0.5 for _ in range(E)]
    for e in range(E):
        m.load_expert(e, gates[e].bfloat16().to(DEV), ups[e].bfloat16().to(DEV), downs[e].bfloat16().to(DEV))
    h = torch.randn(150, W, device=DEV).bfloat16()
    got = m(h).float().cpu()
    hd = h.double().cpu()
    z = hd @ m.router_w.double().cpu().T
    val, idx = torch.topk(z, 2, -1)
    wt = torch.softmax(val, -1)
    want = torch.zeros(150, W, dtype=torch.float64)
    for t in range(150):
        for j in range(2):
            e = int(idx[t, j])
            g, u, d = gates[e].bfloat16().double(), ups[e].bfloat16().double(), downs[e].bfloat16().double()
            want[t] += wt[t, j] * (d @ (torch.nn.functional.silu(g @ hd[t]) * (u @ hd[t])))
    assert close(got, want.float(), 3e-2)


@pytest.fixture(scope="module")
def models():
    out = {}
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        w = U.random_weights(cfg, seed=40 + i)
        out[name] = (cfg, w, U.save_model(cfg, w))
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_and_decoding(models, name, dtype):
    cfg, w, path = models[name]
    t = toks(45, cfg["vocab"], 1)
    ex = Expect(cfg, w, path, t, dtype)
    s = U.session(path, dtype, DEV)
    ex.check(U.run_chunks(s, "a", t, [len(t)]))
    ex.check(U.run_chunks(s, "b", t, [20]))
    ex.check(U.run_chunks(s, "c", t, [2, 2, 7, 1, 1, 13, 2]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_reuse_pages_and_slots(models, dtype):
    cfg, w, path = models["mixed"]
    v = cfg["vocab"]
    reqs = {k: toks(n, v, 20 + i) for i, (k, n) in enumerate([("a", 30), ("b", 9), ("c", 17), ("d", 2), ("e", 26),
                                                              ("f", 12)])}
    ex = {k: Expect(cfg, w, path, t, dtype) for k, t in reqs.items()}
    s = U.session(path, dtype, DEV, max_tokens=64, page_size=4, state_slots=3)
    plan = [[("a", 11), ("b", 9)], [("a", 1), ("c", 5)], [("a", 2), ("c", 1)], [("c", 11), ("a", 16), ("d", 2)],
            [("e", 3)], [("e", 1), ("f", 12)], [("e", 22)]]
    got = U.run_plan(s, reqs, plan)
    for k in reqs:
        ex[k].check(got[k])
    mm = s.scheduler.mm
    assert mm.get_num_free_state_slots() == 3 and mm.get_num_free_pages() == mm.usable_pages


@pytest.mark.parametrize("chunk,page_size", [(8, 4), (5, 4), (16, 16), (6, 8)])
def test_chunk_edges_on_the_kernels(chunk, page_size):
    for back in range(0, chunk + 2):
        want, outs, offset = _chunk_probe(chunk, page_size, back, DEV, torch.float32)
        for o in outs:
            assert torch.allclose(o, want, atol=1e-4, rtol=1e-4), (chunk, back)
        assert (outs[0][-1, 0].item() > 2.5) == (back <= offset)


def test_tensor_core_sized_model_in_bf16():
    """Head size 64 = value size, ff % 64 == 0, width % 128 == 0: tcgen05 GEMMs, tensor-core chunk attention and
    the grouped expert GEMMs carry the model; logits must stay within rounding of the oracle."""
    cfg = U.make_config([U.parallel(heads=4, kv_heads=2, dim=64, vdim=64, chunk=24, rot=32, rheads=2, rdim=32,
                                    rvdim=32, decay=(0.9, 0.99), mlp=U.moe(experts=8, top=2, ff=64)),
                         U.delta(heads=4, kv_heads=2, dim=32, vdim=32, mlp=U.dense(128))], width=128, vocab=96)
    w = U.random_weights(cfg, 5)
    path = U.save_model(cfg, w)
    t = toks(150, cfg["vocab"], 4)
    s = U.session(path, "bfloat16", DEV, max_tokens=512, page_size=16)
    ex = Expect(cfg, w, path, t, "bfloat16")
    ex.check(U.run_chunks(s, "a", t, [150]))
    ex.check(U.run_chunks(s, "b", t, [100, 30, 2]))
    # the same sizes without a router: every row within twice the rounding noise
    cfg2 = U.make_config([U.parallel(heads=4, kv_heads=2, dim=64, vdim=64, chunk=24, rot=32, rheads=2, rdim=32,
                                     rvdim=32, decay=(0.9, 0.99), mlp=U.dense(128)),
                          U.delta(heads=4, kv_heads=2, dim=32, vdim=32, mlp=U.dense(256))], width=128, vocab=96)
    w2 = U.random_weights(cfg2, 6)
    path2 = U.save_model(cfg2, w2)
    s2 = U.session(path2, "bfloat16", DEV, max_tokens=512, page_size=16)
    ex2 = Expect(cfg2, w2, path2, t, "bfloat16")
    ex2.check(U.run_chunks(s2, "a", t, [150]))
    ex2.check(U.run_chunks(s2, "b", t, [100, 30, 2]))


def test_greedy_generation_with_cuda_graphs(models):
    from gllm_b200.engine.llm_engine import LLM
    cfg, w, path = models["mixed"]
    llm = LLM(path, dtype="float32", page_size=4, maxp=16, maxd=8, num_gpu_pages=64, model_max_length=96,
              log_stats=False, num_state_slots=4, max_cuda_graph_bs=4)
    prompts = [toks(21, cfg["vocab"], 31), toks(3, cfg["vocab"], 32), toks(9, cfg["vocab"], 33)]
    lens = [7, 12, 5]
    seqs = llm.generate(tokens=prompts, output_lens=lens, temperature=0.0, top_k=1)
    assert llm.worker.runner.stats["graph_steps"] > 0
    for p, n, s in zip(prompts, lens, seqs):
        cur = list(p)
        for _ in range(n):
            cur.append(int(oracle.forward(cfg, w, cur, torch.float64)[-1].argmax()))
        assert s.token_ids == cur
