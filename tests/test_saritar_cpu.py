"""Saritar through the engine (scheduler bookkeeping, page / state-slot managers, batch builder, runner) against the
plain oracle in saritar_oracle.py: mechanisms alone, chunking, batching, re-use of pages and slots, window and page
edges, degenerate sizes, greedy generation. Runs on the CPU path in fp32; test_saritar_gpu.py repeats the scenarios
on the kernels."""
import numpy as np
import pytest
import torch

import saritar_oracle as oracle
import saritar_util as U

TOL = 2e-4


def toks(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


CONFIGS = {
    "attention_only": U.make_config([U.with_mlp(U.attn()), U.attn(heads=2, kv_heads=2, dim=8, window=3)]),
    "mamba_only": U.make_config([U.mamba(), U.with_mlp(U.mamba(inner=16, state=3, dt_rank=2, conv=2))]),
    "mixed_loop": U.make_config([U.mamba(), U.with_mlp(U.attn(window=6)), U.mamba(conv=4), U.attn(heads=4, kv_heads=1)],
                                loop=(1, 3, 3)),
    "loop_from_zero": U.make_config([U.with_mlp(U.attn(window=5)), U.mamba()], loop=(0, 2, 2), embed_scale=1.0),
    "ones": U.make_config([U.attn(heads=1, kv_heads=1, dim=8, window=1), U.mamba(inner=8, state=1, dt_rank=1, conv=1),
                           U.attn(heads=3, kv_heads=3, dim=8, window=64)], loop=(0, 1, 1), width=16),
}


@pytest.fixture(scope="module")
def models():
    out = {}
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        w = U.random_weights(cfg, seed=10 + i)
        out[name] = (cfg, w, U.save_model(cfg, w))
    return out


@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_matches_oracle(models, name):
    cfg, w, path = models[name]
    t = toks(37, cfg["vocab"], 1)
    s = U.session(path)
    got = s.step([{"id": "a", "tokens": t, "want": list(range(len(t)))}], ["a"])
    assert U.rel_err(got, U.expected_logits(cfg, w, t)) < TOL


@pytest.mark.parametrize("name", ["mixed_loop", "ones", "mamba_only"])
def test_token_by_token_equals_prefill(models, name):
    cfg, w, path = models[name]
    t = toks(45, cfg["vocab"], 2)        # long decoding: crosses 11 pages and every window several times
    want = U.expected_logits(cfg, w, t)
    s = U.session(path)
    assert U.rel_err(U.run_chunks(s, "a", t, []), want) < TOL
    assert U.rel_err(U.run_chunks(s, "b", t, [len(t)]), want) < TOL


@pytest.mark.parametrize("cuts", [[2, 2, 2, 3, 5], [7, 1, 1, 2, 9, 4], [16, 2], [1, 30], [33, 2, 2]])
def test_portions(models, cuts):
    cfg, w, path = models["mixed_loop"]
    t = toks(41, cfg["vocab"], 3)
    s = U.session(path)
    assert U.rel_err(U.run_chunks(s, "a", t, cuts), U.expected_logits(cfg, w, t)) < TOL


def test_mixed_batch_equals_alone_and_reuses_pages_and_slots(models):
    cfg, w, path = models["mixed_loop"]
    v = cfg["vocab"]
    reqs = {k: toks(n, v, 20 + i) for i, (k, n) in enumerate([("a", 30), ("b", 9), ("c", 17), ("d", 2), ("e", 26), ("f", 12)])}
    want = {k: U.expected_logits(cfg, w, t) for k, t in reqs.items()}
    # pool of 64 tokens and 3 slots: the six requests cannot all be resident, pages and slots are handed on
    s = U.session(path, max_tokens=64, page_size=4, state_slots=3)
    at = {k: 0 for k in reqs}
    got = {k: [] for k in reqs}
    plan = [[("a", 11), ("b", 9)], [("a", 1), ("c", 5)], [("a", 2), ("c", 1)], [("c", 11), ("a", 16), ("d", 2)],
            [("e", 3)], [("e", 1), ("f", 12)], [("e", 22)]]
    for step in plan:
        entries, end = [], []
        for k, n in step:
            entries.append({"id": k, "tokens": reqs[k][at[k]:at[k] + n], "want": list(range(n))})
            at[k] += n
            if at[k] == len(reqs[k]):
                end.append(k)
        out = s.step(entries, end)
        o = 0
        for k, n in step:
            got[k].append(out[o:o + n])
            o += n
    for k in reqs:
        assert at[k] == len(reqs[k])
        assert U.rel_err(np.concatenate(got[k], 0), want[k]) < TOL, k
    mm = s.scheduler.mm
    assert mm.get_num_free_state_slots() == 3 and mm.get_num_free_pages() == mm.usable_pages


def test_stale_slot_and_page_contents_do_not_leak(models):
    cfg, w, path = models["mamba_only"]
    s = U.session(path, max_tokens=32, page_size=4, state_slots=1)
    a, b = toks(19, cfg["vocab"], 5), toks(7, cfg["vocab"], 6)
    U.run_chunks(s, "a", a, [10, 9])
    assert U.rel_err(U.run_chunks(s, "b", b, [3, 2, 2]), U.expected_logits(cfg, w, b)) < TOL


def _attention_probe(window, page_size, far):
    """One attention layer driven directly: key `far` positions back carries a huge score; inside the window it must
    dominate the output, outside it must not appear at all."""
    from gllm_b200.layers.window_attention import SinkWindowAttention
    from gllm_b200.input_data import InputData, build_batch
    from gllm_b200.memory_manager import HybridCache, MemoryManager
    from gllm_b200.scheduler import ScheduledSeq
    from gllm_b200.sequence import Sequence
    torch.manual_seed(0)
    H, G, D = 2, 1, 8
    W = (H + G) * D
    n = far + 3
    m = SinkWindowAttention(W, H, G, D, 1.0, window, 1e-6, torch.float32, "cpu")
    m.qk_w.data.copy_(torch.eye(W))
    m.q_norm_w.data.fill_(1.0)
    m.k_norm_w.data.fill_(1.0)
    m.sink.data.fill_(-2.0)
    m.o_w.data.copy_(torch.eye(W)[:, : H * D])
    h = torch.randn(n, W) * 0.1
    tgt = n - 1 - far
    h[tgt, H * D:] = torch.tensor([9.0, 0, 0, 0, 0, 0, 0, 0])          # the marked key (its value is the raw key)
    h[n - 1, :D] = torch.tensor([30.0, 0, 0, 0, 0, 0, 0, 0])            # last query looks for it
    p = {"q": m.qk_w[: H * D], "k": m.qk_w[H * D:], "q.norm": m.q_norm_w, "k.norm": m.k_norm_w, "sink": m.sink, "o": m.o_w}
    want = oracle.sink_window_attention(h.double(), {k: v.double() for k, v in p.items()}, H, G, D, 1.0, window, 1e-6)
    outs = []
    for cuts in ([n], [n - 1, 1], [2] * (n // 2) + [1] * (n % 2)):
        mm = MemoryManager(64, page_size)
        cache = HybridCache([m.cache_entry()], 64, page_size, 0, torch.float32, "cpu")
        inp = InputData(64, 4, 32, "cpu")
        seq = Sequence(0, list(range(n)), [])
        got, at = [], 0
        for c in cuts:
            seq.scheduled_token_num = at + c
            mm.pre_allocate_page([seq])
            inp.load(build_batch([ScheduledSeq(seq, at, c)], page_size, 100))
            got.append(m(inp, h[at:at + c], cache, 0))
            at += c
        outs.append(torch.cat(got))
    return want.float(), outs, tgt


@pytest.mark.parametrize("window,page_size", [(8, 4), (5, 4), (16, 16), (1, 4)])
def test_window_edges_and_page_borders(window, page_size):
    for far, inside in ((window - 1, True), (window, False)):
        want, outs, tgt = _attention_probe(window, page_size, far)
        for o in outs:
            assert torch.allclose(o, want, atol=1e-4, rtol=1e-4)
        marked = outs[0][-1, 0].item()
        assert (marked > 4.0) == inside, (window, far, marked)      # the marked value is 9 * weight


def test_far_key_through_many_pages():
    want, outs, _ = _attention_probe(40, 4, 39)
    assert outs[1][-1, 0].item() > 4.0
    for o in outs:
        assert torch.allclose(o, want, atol=1e-4, rtol=1e-4)


def test_sink_takes_probability_mass():
    want, outs, _ = _attention_probe(4, 4, 2)
    assert torch.allclose(outs[0], want, atol=1e-4)
    # without keys of any weight the first token's output is its own value scaled by 1 / (1 + exp(sink - score))
    assert outs[0][0].abs().max() < want[0].abs().max() * 1.0001 + 1e-6


def test_first_tokens_of_a_sequence(models):
    cfg, w, path = models["mixed_loop"]
    t = toks(6, cfg["vocab"], 9)
    want = U.expected_logits(cfg, w, t)
    s = U.session(path)
    for cuts in ([1], [1, 1, 1], [2, 1], [3, 3]):
        assert U.rel_err(U.run_chunks(s, "x%d" % len(cuts), t, cuts), want) < TOL


def test_greedy_generation_through_the_engine(models):
    from gllm_b200.engine.llm_engine import LLM
    cfg, w, path = models["mixed_loop"]
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
