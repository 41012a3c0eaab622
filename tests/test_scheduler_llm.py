"""The scheduler's decisions (no GPU): admission, budgets, portions, preemption with
recompute, finishing; and the Python entry point end to end with the plain kernel references
standing in for the CUDA kernels, token-exact against the plain implementation."""
import pytest
import torch

from mini_inference_b200.cache import CacheManager
from mini_inference_b200.engine.llm import LLM
from mini_inference_b200.engine.request import Request, SamplingParams
from mini_inference_b200.engine.scheduler import Scheduler
from mini_inference_b200.parts.base import KVCacheNeed
from tests.helpers import random_tokens
from tests.plain import qwen3_plain as plain
from tests.ref_ops import TorchRefOps
from tests.ref_sampling import perturbed_scores


def sched(pages=8, page=4, seqs=4, budget=64, chunked=False, watermark=0.0):
    cache = CacheManager([KVCacheNeed(1, 16)], page, pages, seqs, 4096, allocate=False, watermark=watermark)
    return Scheduler(cache, seqs, budget, 4096, chunked_prefill=chunked), cache


def req(n, new=4):
    return Request(prompt_ids=list(range(n)), params=SamplingParams(max_new_tokens=new))


def advance(chunks, token=1):
    """What the engine does after a step: mark computed, append a token when a request's prompt is done."""
    for r, s, e in chunks:
        r.num_computed = e
        if e == r.total_len:
            r.output_ids.append(token)
        r.seq.num_tokens = e


def test_whole_prompts_fifo_and_batch_limit():
    s, cache = sched(pages=100, seqs=2)
    a, b, c = req(5), req(7), req(3)
    for r in (a, b, c):
        s.add(r)
    chunks = s.schedule()
    assert [(r.id, st, e) for r, st, e in chunks] == [(a.id, 0, 5), (b.id, 0, 7)]      # max_num_seqs 2
    advance(chunks)
    chunks = s.schedule()
    assert [(st, e) for _, st, e in chunks] == [(5, 6), (7, 8)]                          # decode: one token each
    s.finish(a)
    chunks = s.schedule()
    assert [r.id for r, _, _ in chunks] == [b.id, c.id]
    assert s.stats()["steps"] == 3 and s.decode_tokens == 3


def test_token_budget_without_chunking():
    s, _ = sched(pages=100, budget=10)
    a, b = req(6), req(8)
    s.add(a); s.add(b)
    assert [r.id for r, _, _ in s.schedule()] == [a.id]          # b (8) exceeds what is left of the budget
    big, _ = sched(pages=100, budget=10)
    big.add(req(30))
    assert [(st, e) for _, st, e in big.schedule()] == [(0, 30)]  # a long prompt may still run alone


def test_chunked_prefill_budget_and_order():
    s, _ = sched(pages=100, budget=8, chunked=True)
    a, b = req(3), req(20)
    s.add(a); s.add(b)
    c1 = s.schedule()
    assert [(r.id, st, e) for r, st, e in c1] == [(a.id, 0, 3), (b.id, 0, 5)]
    advance(c1)
    c2 = s.schedule()                                            # decode first, then the unfinished prompt
    assert [(r.id, st, e) for r, st, e in c2] == [(a.id, 3, 4), (b.id, 5, 12)]
    assert s.max_step_tokens <= 8 and s.prefill_chunks == 2 and s.mixed_steps == 1


def test_admission_is_head_of_line_and_respects_watermark():
    s, cache = sched(pages=6, page=4, watermark=0.1)
    a, b, c = req(16), req(12), req(2)
    for r in (a, b, c):
        s.add(r)
    chunks = s.schedule()
    assert [r.id for r, _, _ in chunks] == [a.id]                # b needs 3 + 1 watermark > 2 free; c waits behind b
    assert [r.id for r in s.waiting] == [b.id, c.id]


def test_pages_run_out_newest_is_preempted_and_recomputed():
    s, cache = sched(pages=4, page=4)
    a, b = req(7, new=20), req(7, new=20)
    s.add(a); s.add(b)
    advance(s.schedule())                                        # both admitted: 2 pages each, pool empty
    advance(s.schedule())                                        # 8 tokens each still fit
    advance(s.schedule())                                        # the 9th token of each needs a 3rd page
    assert s.preemptions == 1 and b.preemptions == 1 and b.state == "waiting"
    assert s.waiting[0] is b and b.num_computed == 0 and b.seq is None and len(b.output_ids) == 2
    assert [r.id for r in s.running] == [a.id]
    cache.check_invariants()
    s.finish(a)
    chunks = s.schedule()
    assert [(r.id, st, e) for r, st, e in chunks] == [(b.id, 0, 9)]      # prompt + generated, from position 0
    cache.check_invariants()


def test_chunked_preemption_refunds_budget():
    s, cache = sched(pages=4, page=4, budget=32, chunked=True)
    a, b = req(8, new=20), req(7, new=20)
    s.add(a); s.add(b)
    advance(s.schedule())                                        # a: 2 pages (8 tokens), b: 2 pages (7 tokens)
    chunks = s.schedule()                                        # a's 9th token needs a page -> b (newest) is preempted
    assert [(r.id, st, e) for r, st, e in chunks] == [(a.id, 8, 9)]
    assert s.preemptions == 1 and s.waiting[0] is b
    cache.check_invariants()


def test_abort_all_frees_everything():
    s, cache = sched(pages=10)
    for n in (5, 6):
        s.add(req(n))
    s.schedule()
    assert len(s.abort_all()) == 2 and cache.free_pages() == 10 and not s.running


# ---------------------------------------------------------------- entry point, CPU stand-in kernels
def llm(d, **kw):
    kw.setdefault("kv_cache_tokens", 512)
    return LLM(d, dtype="float32", device="cpu", ops=TorchRefOps(), **kw)


@pytest.mark.parametrize("name", ["A", "B", "W"])
def test_generate_greedy_matches_plain(tiny_dirs, name):
    d, cfg, page = tiny_dirs[name]
    prompts = [random_tokens(cfg["vocab_size"], n, seed=20 + n) for n in (5, 11, 17)]
    c, w = plain.load_model_dir(d)
    want = [plain.greedy_generate(c, w, p, 8) for p in prompts]
    for kw in (dict(), dict(chunked_prefill=True, max_batched_tokens=4), dict(max_num_seqs=1)):
        eng = llm(d, kv_block_size=page, **kw)
        got = eng.generate(prompts, SamplingParams(max_new_tokens=8))
        assert got == want, kw
        st = eng.stats()
        assert st["running"] == 0 and st["kv_blocks_used"] == 0
        eng.cache.check_invariants()


def test_preemption_keeps_outputs_exact(tiny_dirs):
    """A pool of 6 pages of 8 tokens for 4 requests that each grow to 29 tokens."""
    d, cfg, _ = tiny_dirs["A"]
    prompts = [random_tokens(cfg["vocab_size"], 9, seed=40 + i) for i in range(4)]
    c, w = plain.load_model_dir(d)
    want = [plain.greedy_generate(c, w, p, 20) for p in prompts]
    for chunked in (False, True):
        eng = llm(d, kv_block_size=8, kv_cache_tokens=48, kv_watermark=0.0, chunked_prefill=chunked, max_batched_tokens=16)
        assert eng.generate(prompts, SamplingParams(max_new_tokens=20)) == want
        assert eng.stats()["preemptions"] > 0
        eng.cache.check_invariants()
        assert eng.cache.free_pages() == 6


def test_arrivals_mid_run_and_temperature(tiny_dirs):
    """Config B's workload: requests of lengths 1, 3, 9, 14, 30 arriving while others run, portions
    of 7 tokens, temperature 0.8 with a fixed seed: a request's draws do not depend on its company."""
    d, cfg, page = tiny_dirs["B"]
    prompts = [random_tokens(cfg["vocab_size"], n, seed=60 + n) for n in (1, 3, 9, 14, 30)]
    sp = [SamplingParams(max_new_tokens=12, temperature=0.8, seed=100 + i) for i in range(5)]
    alone = [llm(d, kv_block_size=page).generate([p], s)[0] for p, s in zip(prompts, sp)]
    eng = llm(d, kv_block_size=page, chunked_prefill=True, max_batched_tokens=7)
    reqs = []
    for i, (p, s) in enumerate(zip(prompts, sp)):
        reqs.append(eng.add_request(p, s))
        eng.step()
        eng.step()
    while eng.has_work():
        eng.step()
    assert [r.output_ids for r in reqs] == alone
    assert eng.stats()["mixed_steps"] > 0 and eng.stats()["prefill_chunks"] > 0
    # and each drawn token is the argmax of logits/T + gumbel noise of (seed, tokens so far)
    c, w = plain.load_model_dir(d)
    ids = prompts[2] + alone[2]
    logits = plain.forward_logits(c, w, ids)
    for k in range(12):
        row = logits[len(prompts[2]) - 1 + k][None]
        sc = perturbed_scores(row, torch.tensor([0.8]), torch.tensor([102]), torch.tensor([k]))[0]
        assert sc[alone[2][k]] >= sc.max() - 1e-3


@pytest.mark.parametrize("case", range(6))
def test_random_workloads_and_settings(tiny_dirs, case):
    """Workloads and engine settings drawn at random (arrival steps, prompt and output lengths, page pools from roomy to
    barely enough for the longest request, step budgets, portions on or off, batch limits): every request's greedy tokens are
    the plain implementation's, the cache manager's invariants hold after every step, and all pages come back."""
    random_workload(tiny_dirs, case, llm)


def random_workload(tiny_dirs, case, llm):
    import numpy as np
    rng = np.random.default_rng(100 + case)
    name = ("A", "B", "W")[case % 3]
    d, cfg, page = tiny_dirs[name]
    c, w = plain.load_model_dir(d)
    n = int(rng.integers(3, 8))
    lens = [int(rng.integers(1, 40)) for _ in range(n)]
    news = [int(rng.integers(1, 14)) for _ in range(n)]
    arrive = sorted(int(rng.integers(0, 12)) for _ in range(n))
    prompts = [random_tokens(cfg["vocab_size"], L, seed=500 + 10 * case + i) for i, L in enumerate(lens)]
    want = [plain.greedy_generate(c, w, p, k) for p, k in zip(prompts, news)]
    longest = max(L + k for L, k in zip(lens, news))
    pages_longest = -(-longest // page)
    pool_pages = int(rng.integers(pages_longest + 1, 4 * pages_longest + 2))
    chunked = bool(rng.integers(0, 2))
    budget = int(rng.integers(2, 24)) if chunked else int(rng.integers(max(lens), 3 * max(lens) + 1))
    eng = llm(d, kv_block_size=page, kv_cache_tokens=pool_pages * page, kv_watermark=0.0, chunked_prefill=chunked,
              max_batched_tokens=budget, max_num_seqs=int(rng.integers(1, 5)))
    total_pages = eng.cache.free_pages()
    reqs, step = [None] * n, 0
    while any(r is None for r in reqs) or eng.has_work():
        for i in range(n):
            if reqs[i] is None and arrive[i] <= step:
                reqs[i] = eng.add_request(prompts[i], SamplingParams(max_new_tokens=news[i]))
        eng.step()
        eng.cache.check_invariants()
        step += 1
        assert step < 3000, "the engine does not finish"
    setting = dict(config=name, pool_pages=pool_pages, chunked=chunked, budget=budget, lens=lens, news=news, arrive=arrive)
    assert [r.output_ids for r in reqs] == want, setting
    assert all(r.error is None for r in reqs), setting
    assert eng.cache.free_pages() == total_pages and eng.stats()["running"] == 0, setting


def test_limits_and_errors(tiny_dirs):
    d, cfg, page = tiny_dirs["A"]
    eng = llm(d, kv_block_size=8, kv_cache_tokens=64)
    with pytest.raises(ValueError, match="empty"):
        eng.add_request([])
    with pytest.raises(ValueError, match="limit"):
        eng.add_request([1] * 64)
    with pytest.raises(ValueError, match="token id"):
        eng.add_request([cfg["vocab_size"]])
    r = eng.add_request([1] * 60, SamplingParams(max_new_tokens=50))
    assert r.params.max_new_tokens == 4                           # capped by the limit (custom_engine.py:194)
    # eos stops a request
    c, w = plain.load_model_dir(d)
    first = plain.greedy_generate(c, w, [3, 4, 5], 6)
    k = next((i for i in range(1, 6) if first[i] not in first[:i]), 0)
    eng2 = llm(d, kv_block_size=8)
    eng2.eos_ids = {first[k]}
    out = eng2.generate([[3, 4, 5]], SamplingParams(max_new_tokens=10))[0]
    assert out == first[:k + 1]
    assert eng2.generate([[3, 4, 5]], SamplingParams(max_new_tokens=6, ignore_eos=True))[0] == first
    # a failing step aborts the batch, frees the cache and keeps the engine usable
    eng3 = llm(d, kv_block_size=8)
    real = eng3.runner.step
    eng3.runner.step = lambda *a, **k: (_ for _ in ()).throw(RuntimeError("boom"))
    rq = eng3.add_request([1, 2, 3])
    done = eng3.step()
    assert done == [rq] and rq.finish_reason == "error" and "boom" in rq.error
    assert eng3.cache.free_pages() == eng3.cache.num_pages
    eng3.runner.step = real
    assert eng3.generate([[3, 4, 5]], SamplingParams(max_new_tokens=6))[0] == first
    # score(): all-position logits through the cache
    sc = eng3.score([3, 4, 5, 6])
    assert torch.allclose(sc, plain.forward_logits(c, w, [3, 4, 5, 6]), atol=1e-5)
