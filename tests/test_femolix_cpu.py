"""Femolix through the engine (scheduler bookkeeping, page / state-slot managers, batch builder, runner) against the
plain oracle in femolix_oracle.py: mechanisms alone, chunking, batching, re-use of pages and slots, chunk and page
edges, degenerate sizes, greedy generation. Runs on the CPU path in fp32; test_femolix_gpu.py repeats the scenarios
on the kernels."""
import numpy as np
import pytest
import torch

import femolix_oracle as oracle
import femolix_util as U

TOL = 2e-4


def toks(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


CONFIGS = {
    "delta_only": U.make_config([U.delta(mlp=U.dense()), U.delta(heads=3, kv_heads=3, dim=6, vdim=6, conv=2)]),
    "parallel_only": U.make_config([U.parallel(mlp=U.dense()), U.parallel(heads=2, kv_heads=2, dim=8, vdim=8, chunk=3,
                                                                           rot=4, rheads=1, decay=(0.8,))]),
    "moe_only": U.make_config([U.delta(mlp=U.moe()), U.parallel(mlp=U.moe(experts=5, top=3, ff=8))]),
    "mixed": U.make_config([U.parallel(mlp=U.moe()), U.delta(mlp=U.dense()), U.delta(conv=4, mlp=U.moe(top=1)),
                            U.parallel(chunk=5, rot=12, mlp=None)]),
    "ones": U.make_config([U.delta(heads=1, kv_heads=1, dim=4, vdim=4, conv=1, mlp=U.moe(experts=1, top=1, ff=4)),
                           U.parallel(heads=1, kv_heads=1, dim=4, vdim=4, chunk=1, rot=2, rheads=1, rdim=4, rvdim=4,
                                      decay=(1.0,), ls=1.0, rs=1.0, mlp=U.moe(experts=3, top=3, ff=4)),
                           U.parallel(heads=3, kv_heads=1, dim=8, vdim=4, chunk=64, rot=0, mlp=U.dense(8))],
                          width=16, alpha=1.0, cap=30.0),
}


@pytest.fixture(scope="module")
def models():
    out = {}
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        w = U.random_weights(cfg, seed=40 + i)
        out[name] = (cfg, w, U.save_model(cfg, w))
    return out


# -- each mechanism alone, against its own oracle function -----------------------------------------------------
def _mixer_alone(layer_cfg, seed, n=19, cuts=((19,), (7, 1, 1, 2, 8), (2,) * 9 + (1,)), page_size=4, width=24):
    """One mixer driven directly through the cache and batch builder, whole and in portions."""
    from gllm_b200.input_data import InputData, build_batch
    from gllm_b200.memory_manager import HybridCache, MemoryManager
    from gllm_b200.models.hybrid import HybridSpec, make_mixer
    from gllm_b200.scheduler import ScheduledSeq
    from gllm_b200.sequence import Sequence
    cfg = U.make_config([layer_cfg], width=width)
    w = U.random_weights(cfg, seed)
    spec = HybridSpec("femolix", width, cfg["vocab"], 1e-5, 1.0, cfg["layers"], dtype=torch.float32)
    m = make_mixer(layer_cfg["type"], layer_cfg["mixer"], spec, "cpu")

    class R:
        def get(self, name):
            return w[name]

    def put(p, t):
        p.data.copy_(t)

    m.load(R(), "l0.mix.", put)
    h = torch.randn(n, width, generator=torch.Generator().manual_seed(seed))
    wd = {k: v.double() for k, v in w.items()}
    fn = oracle.delta_mixer if layer_cfg["type"] == "delta" else oracle.parallel_mixer
    want = fn(h.double(), wd, "l0.mix.", layer_cfg["mixer"], 1e-5).float()
    for cut in cuts:
        mm = MemoryManager(64, page_size, num_state_slots=2)
        cache = HybridCache([m.cache_entry()], 64, page_size, 2, torch.float32, "cpu")
        inp = InputData(64, 4, 32, "cpu")
        seq = Sequence(0, list(range(n)), [])
        assert mm.acquire_state(seq)
        got, at = [], 0
        for c in cut:
            seq.scheduled_token_num = at + c
            mm.pre_allocate_page([seq])
            inp.load(build_batch([ScheduledSeq(seq, at, c)], page_size, 100))
            got.append(m(inp, h[at:at + c], cache, 0))
            at += c
        assert torch.allclose(torch.cat(got), want, atol=2e-4, rtol=2e-4), cut


def test_delta_mixer_alone():
    _mixer_alone(U.delta(), 1)
    _mixer_alone(U.delta(heads=2, kv_heads=1, dim=5, vdim=3, conv=4), 2)
    _mixer_alone(U.delta(heads=1, kv_heads=1, dim=4, vdim=4, conv=1), 3)


def test_parallel_mixer_alone():
    _mixer_alone(U.parallel(), 4)
    _mixer_alone(U.parallel(heads=2, kv_heads=1, dim=6, vdim=2, chunk=4, rot=6, rheads=2, decay=(0.3, 1.0)), 5)
    _mixer_alone(U.parallel(chunk=1, rot=0, ls=0.0), 6)       # only the linear-attention side contributes
    _mixer_alone(U.parallel(chunk=100, rs=0.0), 7)            # only the softmax side, one chunk


def test_ops_against_oracle_functions():
    from gllm_b200.ops import ref
    g = torch.Generator().manual_seed(0)
    x = torch.randn(9, 16, generator=g)
    pos = torch.tensor([0, 1, 2, 3, 50, 51, 1000, 1001, 70000], dtype=torch.int32)
    got = ref.rotate_half_pairs(x.reshape(9, 2, 8), pos, 6, 100.0)
    # the oracle rotates by running position; build its answer position by position
    ref_rows = []
    for i, p in enumerate(pos.tolist()):
        full = torch.zeros(p + 1, 2, 8, dtype=torch.float64)
        full[p] = x[i].double().reshape(2, 8)
        ref_rows.append(oracle.rotate(full, torch.arange(p + 1), 6, 100.0)[p])
    assert torch.allclose(got.double(), torch.stack(ref_rows), atol=1e-5)
    h = torch.randn(5, 12, generator=g)
    wr = torch.randn(7, 12, generator=g)
    wt, ids = ref.router_topk(h, wr, 3)
    z = h @ wr.T
    for t in range(5):
        top = sorted(range(7), key=lambda e: -z[t, e].item())[:3]
        assert sorted(ids[t].tolist()) == sorted(top)
        e = torch.exp(z[t, ids[t].long()] - z[t, ids[t].long()].max())
        assert torch.allclose(wt[t], e / e.sum(), atol=1e-6)
    assert torch.allclose(ref.softcap(z, 2.0), 2.0 * torch.tanh(z / 2.0))
    xs, y, wn = torch.randn(4, 12, generator=g), torch.randn(4, 12, generator=g), torch.rand(12, generator=g) + 0.5
    want = oracle.rms(1.5 * xs + y, 1e-5) * wn
    hh = ref.postnorm(xs, y, 1.5, wn, 1e-5, torch.float32)
    assert hh is xs and torch.allclose(xs, want, atol=1e-6)


# -- whole models ----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_matches_oracle(models, name):
    cfg, w, path = models[name]
    t = toks(37, cfg["vocab"], 1)
    s = U.session(path)
    got = s.step([{"id": "a", "tokens": t, "want": list(range(len(t)))}], ["a"])
    assert U.rel_err(got, U.expected_logits(cfg, w, t)) < TOL


def test_residual_stream_after_every_layer(models):
    cfg, w, path = models["mixed"]
    t = toks(11, cfg["vocab"], 8)
    trace = []
    oracle.forward(cfg, w, t, torch.float64, trace)
    s = U.session(path)
    s.runner.model.trace = []
    s.step([{"id": "a", "tokens": t, "want": []}], ["a"])
    got = s.runner.model.trace
    assert len(got) == len(trace)
    for a, b in zip(got, trace):
        assert torch.allclose(a.double(), b, atol=1e-4)


@pytest.mark.parametrize("name", ["mixed", "ones", "delta_only"])
def test_token_by_token_equals_prefill(models, name):
    cfg, w, path = models[name]
    t = toks(45, cfg["vocab"], 2)        # long decoding: crosses 11 pages and every chunk several times
    want = U.expected_logits(cfg, w, t)
    s = U.session(path)
    assert U.rel_err(U.run_chunks(s, "a", t, []), want) < TOL
    assert U.rel_err(U.run_chunks(s, "b", t, [len(t)]), want) < TOL


@pytest.mark.parametrize("cuts", [[2, 2, 2, 3, 5], [7, 1, 1, 2, 9, 4], [16, 2], [1, 30], [33, 2, 2], [6, 1, 7, 7]])
def test_portions(models, cuts):
    cfg, w, path = models["mixed"]
    t = toks(41, cfg["vocab"], 3)
    s = U.session(path)
    assert U.rel_err(U.run_chunks(s, "a", t, cuts), U.expected_logits(cfg, w, t)) < TOL


def test_mixed_batch_equals_alone_and_reuses_pages_and_slots(models):
    cfg, w, path = models["mixed"]
    v = cfg["vocab"]
    reqs = {k: toks(n, v, 20 + i) for i, (k, n) in enumerate([("a", 30), ("b", 9), ("c", 17), ("d", 2), ("e", 26),
                                                              ("f", 12)])}
    want = {k: U.expected_logits(cfg, w, t) for k, t in reqs.items()}
    # pool of 64 tokens and 3 slots: the six requests cannot all be resident, pages and slots are handed on
    s = U.session(path, max_tokens=64, page_size=4, state_slots=3)
    plan = [[("a", 11), ("b", 9)], [("a", 1), ("c", 5)], [("a", 2), ("c", 1)], [("c", 11), ("a", 16), ("d", 2)],
            [("e", 3)], [("e", 1), ("f", 12)], [("e", 22)]]
    got = U.run_plan(s, reqs, plan)
    for k in reqs:
        assert U.rel_err(got[k], want[k]) < TOL, k
    mm = s.scheduler.mm
    assert mm.get_num_free_state_slots() == 3 and mm.get_num_free_pages() == mm.usable_pages


def test_stale_slot_and_page_contents_do_not_leak(models):
    cfg, w, path = models["mixed"]
    s = U.session(path, max_tokens=32, page_size=4, state_slots=1)
    a, b = toks(19, cfg["vocab"], 5), toks(7, cfg["vocab"], 6)
    U.run_chunks(s, "a", a, [10, 9])
    assert U.rel_err(U.run_chunks(s, "b", b, [3, 2, 2]), U.expected_logits(cfg, w, b)) < TOL


def test_first_tokens_of_a_sequence(models):
    cfg, w, path = models["mixed"]
    t = toks(6, cfg["vocab"], 9)
    want = U.expected_logits(cfg, w, t)
    s = U.session(path)
    for cuts in ([1], [1, 1, 1], [2, 1], [3, 3]):
        assert U.rel_err(U.run_chunks(s, "x%d" % len(cuts), t, cuts), want) < TOL


# -- edges that random weights would hide ----------------------------------------------------------------------
def _chunk_probe(chunk, page_size, back, device="cpu", dtype=torch.float32):
    """The softmax side alone with identity projections: the key `back` positions before the last query carries a
    huge score. Returns (oracle output, framework outputs for three ways of cutting, marked value of the last row)."""
    from gllm_b200.input_data import InputData, build_batch
    from gllm_b200.layers.parallel_mixer import CoreMixer
    from gllm_b200.layers.window_attention import RotaryChunkCore
    from gllm_b200.memory_manager import HybridCache, MemoryManager
    from gllm_b200.scheduler import ScheduledSeq
    from gllm_b200.sequence import Sequence
    torch.manual_seed(0)
    H, G, D, Dv = 2, 1, 8, 4
    W = H * D + G * D + G * Dv
    n = back + 1 + (chunk * 2 + 3)             # the last query sits a few chunks in
    core = RotaryChunkCore(H, G, D, Dv, 1.0, 0, 10000.0, chunk, None, 1e-6, dtype, device)
    m = CoreMixer(W, [core], [""], [1.0], dtype, device)
    m.in_w.data[:W].copy_(torch.eye(W).to(dtype))          # rows beyond W are GEMM padding
    core.q_norm_w.data.fill_(1.0)
    core.k_norm_w.data.fill_(1.0)
    m.o_w.data.copy_(torch.eye(W)[:, : H * Dv].to(dtype))
    h = torch.randn(n, W) * 0.1
    tgt = n - 1 - back
    h[tgt, H * D:H * D + D] = torch.tensor([9.0, 0, 0, 0, 0, 0, 0, 0])
    h[tgt, H * D + D:] = torch.tensor([5.0, 0, 0, 0])                       # its value
    h[n - 1, :D] = torch.tensor([30.0, 0, 0, 0, 0, 0, 0, 0])                # the last query looks for it
    wd = {"q": m.in_w[: H * D], "k": m.in_w[H * D:H * D + D], "v": m.in_w[H * D + D:W], "q.norm": core.q_norm_w,
          "k.norm": core.k_norm_w, "o": m.o_w}
    mc = {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": 1.0, "mask": {"size": chunk},
          "rot": {"dims": 0, "base": 10000.0}}
    want = oracle.chunk_attention(h.double(), {k: v.double().cpu() for k, v in wd.items()}, "", mc, 1e-6).float()
    outs = []
    for cuts in ([n], [n - 1, 1], [2] * (n // 2) + [1] * (n % 2)):
        mm = MemoryManager(128, page_size)
        cache = HybridCache([m.cache_entry()], 128, page_size, 0, dtype, device)
        inp = InputData(256, 4, 64, device)
        seq = Sequence(0, list(range(n)), [])
        got, at = [], 0
        for c in cuts:
            seq.scheduled_token_num = at + c
            mm.pre_allocate_page([seq])
            inp.load(build_batch([ScheduledSeq(seq, at, c)], page_size, 100))
            got.append(m(inp, h[at:at + c].to(device=device, dtype=dtype), cache, 0).float().cpu())
            at += c
        outs.append(torch.cat(got))
    return want, outs, (n - 1) % chunk


@pytest.mark.parametrize("chunk,page_size", [(8, 4), (5, 4), (16, 16), (6, 8), (2, 4)])
def test_chunk_edges_and_page_borders(chunk, page_size):
    for back in range(0, chunk + 2):
        want, outs, offset = _chunk_probe(chunk, page_size, back)
        inside = back <= offset                  # the marked key lies in the last query's chunk
        for o in outs:
            assert torch.allclose(o, want, atol=1e-4, rtol=1e-4), (chunk, back)
        marked = outs[0][-1, 0].item()
        assert (marked > 2.5) == inside, (chunk, back, marked)


def test_far_state_survives_long_decoding():
    """A decay of exactly 1 keeps the first token's write for ever; it must still be read hundreds of tokens later,
    through prefill, portions and single tokens alike."""
    cfg = U.make_config([U.parallel(heads=1, kv_heads=1, dim=4, vdim=4, chunk=4, rot=0, rheads=2, rdim=6, rvdim=5,
                                    decay=(1.0, 0.97), ls=0.1, rs=2.0, mlp=None)], width=16, vocab=11)
    w = U.random_weights(cfg, 77)
    path = U.save_model(cfg, w)
    t = [3] + [5] * 300
    t2 = [7] + [5] * 300                      # differs in the first token only
    a, b = U.expected_logits(cfg, w, t), U.expected_logits(cfg, w, t2)
    assert np.abs(a[-1] - b[-1]).max() > 1e-3            # the oracle itself still sees the first token
    s = U.session(path, max_tokens=512, page_size=16)
    assert U.rel_err(U.run_chunks(s, "a", t, [200, 50, 2, 2]), a) < TOL
    assert U.rel_err(U.run_chunks(s, "b", t2, [1, 250]), b) < TOL


def test_greedy_generation_through_the_engine(models):
    from gllm_b200.engine.llm_engine import LLM
    cfg, w, path = models["mixed"]
    llm = LLM(path, dtype="float32", page_size=4, maxp=16, maxd=8, num_cpu_pages=64, model_max_length=96,
              log_stats=False, device="cpu", num_state_slots=2)
    prompts = [toks(21, cfg["vocab"], 31), toks(3, cfg["vocab"], 32), toks(9, cfg["vocab"], 33)]
    lens = [7, 12, 5]
    seqs = llm.generate(tokens=prompts, output_lens=lens, temperature=0.0, top_k=1)
    for p, n, s in zip(prompts, lens, seqs):
        cur = list(p)
        for _ in range(n):
            cur.append(int(oracle.forward(cfg, w, cur, torch.float64)[-1].argmax()))
        assert s.token_ids == cur
