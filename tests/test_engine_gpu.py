"""The engine on the GPU with its own kernels, in float32 and in bfloat16, against the plain
implementation: whole prompts, decoding token by token, portions, mixed batches with page
re-use, long decoding."""
import pytest
import torch

from tests.helpers import check_cuts, check_mixed, make_engine, plain_logits, random_tokens, rel_err, run_cuts

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOLS = {"float32": 2e-5, "bfloat16": 4e-2}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "W", "F", "V"])
def test_whole_decode_and_portions(tiny_dirs, name, dtype):
    d, cfg, page = tiny_dirs[name]
    check_cuts(make_engine(d, page, 64, dtype=dtype, device=DEV), d, cfg["vocab_size"], TOLS[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "W", "F", "V"])
def test_mixed_batches_reuse_pages(tiny_dirs, name, dtype):
    d, cfg, page = tiny_dirs[name]
    check_mixed(lambda pages: make_engine(d, page, pages, dtype=dtype, device=DEV), d, cfg["vocab_size"], page,
                TOLS[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "W", "F", "V"])
def test_long_decoding(tiny_dirs, name, dtype):
    """A short prompt and 300 tokens one by one: several splits, many pages, window edges."""
    d, cfg, page = tiny_dirs[name]
    ids = random_tokens(cfg["vocab_size"], 310, seed=11)
    want = plain_logits(d, ids)
    runner = make_engine(d, page, 128, dtype=dtype, device=DEV)
    runner.ops.force_splits = 3
    try:
        got = run_cuts(runner, "long", ids, [10] + [1] * 300)
    finally:
        runner.ops.force_splits = None
    assert rel_err(got, want) < TOLS[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generate_through_entry_point(tiny_dirs, dtype):
    """Greedy generation through LLM.generate, with and without CUDA graphs, chunked or not."""
    from mini_inference_b200 import LLM, SamplingParams
    from tests.plain import qwen3_plain as plain
    d, cfg, page = tiny_dirs["B"]
    prompts = [random_tokens(cfg["vocab_size"], n, seed=20 + n) for n in (1, 3, 9, 14, 30)]
    c, w = plain.load_model_dir(d)
    want = [plain.greedy_generate(c, w, p, 12) for p in prompts]
    outs = []
    for kw in (dict(), dict(cuda_graphs=True), dict(chunked_prefill=True, max_batched_tokens=7, cuda_graphs=True)):
        llm = LLM(d, dtype=dtype, device=DEV, kv_block_size=page, kv_cache_tokens=1024, **kw)
        outs.append(llm.generate(prompts, SamplingParams(max_new_tokens=12)))
        llm.cache.check_invariants()
        assert llm.cache.free_pages() == llm.cache.num_pages
        if kw.get("cuda_graphs"):
            assert llm.stats()["graph_replays"] > 0
    if dtype == "float32":
        assert all(o == want for o in outs)
    else:       # bfloat16 rounding may flip a near-tie: every generated token is judged at its own position
        for o in outs:
            for p, g in zip(prompts, o):
                ref = plain.forward_logits(c, w, p + g)
                err = (llm.score(p + g).float().cpu() - ref).abs().max().item()
                assert err < TOLS[dtype] * ref.abs().max().item()
                assert all(ref[len(p) - 1 + k][t] >= ref[len(p) - 1 + k].max() - 2 * err for k, t in enumerate(g))


def test_overlapped_decode_is_token_exact(tiny_dirs):
    """Launching the next decode step before this one's tokens are read changes no token: greedy and sampled, requests
    of different lengths (length stops at different steps), stops on EOS found mid-way (the step launched in vain is
    dropped), and a request that arrives while a step is in flight."""
    from mini_inference_b200 import LLM, SamplingParams
    d, cfg, page = tiny_dirs["B"]
    prompts = [random_tokens(cfg["vocab_size"], n, seed=80 + n) for n in (2, 5, 9, 14)]
    sps = [SamplingParams(max_new_tokens=m, temperature=t, seed=7 + i)
           for i, (m, t) in enumerate([(17, 0.0), (9, 0.9), (25, 0.0), (13, 0.7)])]
    runs = {}
    for overlap in (False, True):
        llm = LLM(d, dtype="float32", device=DEV, kv_block_size=page, kv_cache_tokens=1024, cuda_graphs=True,
                  overlap_decode=overlap)
        plain_out = llm.generate(prompts, sps)
        # a token that some request produces in the middle of its output becomes the end-of-sequence token
        eos = plain_out[2][10]
        llm.eos_ids = {eos}
        eos_out = llm.generate(prompts, sps)
        # a late arrival: two requests run, the third is added after a few steps
        llm.eos_ids = set()
        reqs = [llm.add_request(p, sp) for p, sp in zip(prompts[:2], sps[:2])]
        for _ in range(4):
            llm.step()
        reqs.append(llm.add_request(prompts[2], sps[2]))
        while llm.has_work():
            llm.step()
        late_out = [list(r.output_ids) for r in reqs]
        llm.cache.check_invariants()
        assert llm.cache.free_pages() == llm.cache.num_pages
        runs[overlap] = (plain_out, eos_out, late_out, llm.stats()["graph_replays"])
    assert runs[True][:3] == runs[False][:3]
    assert [len(o) for o in runs[True][0]] == [17, 9, 25, 13]
    assert len(runs[True][1][2]) == 11 and runs[True][1][2] == runs[True][0][2][:11]      # stopped on the chosen token
    assert runs[True][2] == [runs[True][0][0], runs[True][0][1], runs[True][0][2]]
    assert runs[True][3] >= runs[False][3]                 # a few steps were launched in vain, none was lost


def test_temperature_sampling_does_not_depend_on_company(tiny_dirs):
    from mini_inference_b200 import LLM, SamplingParams
    d, cfg, page = tiny_dirs["B"]
    prompts = [random_tokens(cfg["vocab_size"], n, seed=60 + n) for n in (3, 9, 14)]
    sp = [SamplingParams(max_new_tokens=12, temperature=0.8, seed=100 + i) for i in range(3)]
    llm = LLM(d, dtype="float32", device=DEV, kv_block_size=page, kv_cache_tokens=1024, cuda_graphs=True)
    alone = [llm.generate([p], s)[0] for p, s in zip(prompts, sp)]
    assert llm.generate(prompts, sp) == alone
    assert alone != llm.generate(prompts, [SamplingParams(max_new_tokens=12, temperature=0.8, seed=7)] * 3)


def test_preemption_on_gpu(tiny_dirs):
    from mini_inference_b200 import LLM, SamplingParams
    from tests.plain import qwen3_plain as plain
    d, cfg, _ = tiny_dirs["A"]
    prompts = [random_tokens(cfg["vocab_size"], 9, seed=40 + i) for i in range(4)]
    c, w = plain.load_model_dir(d)
    want = [plain.greedy_generate(c, w, p, 20) for p in prompts]
    llm = LLM(d, dtype="float32", device=DEV, kv_block_size=8, kv_cache_tokens=48, kv_watermark=0.0, cuda_graphs=True)
    assert llm.generate(prompts, SamplingParams(max_new_tokens=20)) == want
    assert llm.stats()["preemptions"] > 0


def test_linear_tuning_table():
    """The start-up timing fills a table per (row bucket, shape) and the chosen kernels still compute the product."""
    from mini_inference_b200.ops import get_ops
    ops = get_ops(DEV)
    g = torch.Generator().manual_seed(0)
    ws = [(torch.randn(512, 256, generator=g) * 0.05).to(torch.bfloat16).to(DEV) for _ in range(3)]
    saved = ops._linear_choice
    try:
        report = ops.tune_linear(ws, iters=4, min_bytes=0)
        assert set(ops._linear_choice) == {(m, 512, 256) for m in ops.ROW_BUCKETS}
        assert all(v["best"] in ("library", "stream", "skinny") for v in report.values())
        x = torch.randn(5, 256, generator=g).to(torch.bfloat16).to(DEV)
        want = x.float() @ ws[0].float().T
        got = ops.linear(x, ws[0], out_dtype=torch.float32)
        assert ((got - want).abs().max() / want.abs().max()).item() < 1e-4
    finally:
        ops._linear_choice = saved


def test_run_engine_command_line(tmp_path):
    import json
    import os
    import subprocess
    from tests.conftest import ROOT
    out = tmp_path / "r.json"
    r = subprocess.run([os.path.join(ROOT, "bin", "run_engine"), "--random-weights", "tiny", "-n", "5", "-c", "3", "--warmup", "1",
                        "--max-new-tokens", "12", "--prompt-len", "3:20", "--kv-tokens", "512", "--cuda-graphs", "on",
                        "--chunked-prefill", "on", "--max-batched-tokens", "16", "--temperature", "0.7", "--out", str(out)],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    data = json.loads(out.read_text())
    assert data["summary"]["num_prompts"] == 5 and len(data["runs"]) == 5
    assert all(run["generated_tokens"] == 12 and run["error"] is None for run in data["runs"])
    assert data["summary"]["throughput_tok_s"] > 0 and data["summary"]["graph_replays"] > 0


LAYER_SIZES = {      # the benchmark configurations' layer sizes (two layers, a cut-down vocabulary)
    "4b": dict(hidden_size=2560, num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=9728,
               tie_word_embeddings=True),
    "8b": dict(hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
               tie_word_embeddings=False),
    "14b": dict(hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, head_dim=128, intermediate_size=17408,
                tie_word_embeddings=False),
}


def sized_model(tmp_path, size, vocab=4099, seed=3):
    from mini_inference_b200.weights import write_random_model
    cfg = dict(LAYER_SIZES[size], architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, vocab_size=vocab,
               rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=4096)
    d = str(tmp_path / f"sizes_{size}")
    write_random_model(cfg, d, seed=seed, std=0.02)
    return d, cfg


def test_run_engine_command_line_with_a_model_folder(tiny_dirs, tmp_path):
    """--model DIR (a folder with config.json and model.safetensors), float32, with the roofline figures in the summary."""
    import json
    import os
    import subprocess
    from tests.conftest import ROOT
    d, cfg, page = tiny_dirs["B"]
    out = tmp_path / "m.json"
    r = subprocess.run([os.path.join(ROOT, "bin", "run_engine"), "--model", d, "--dtype", "float32", "-n", "4", "-c", "2",
                        "--warmup", "1", "--max-new-tokens", "9", "--prompt-len", "5:30", "--kv-tokens", "512", "--page-size",
                        str(page), "--roofline", "--out", str(out)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    data = json.loads(out.read_text())
    sm = data["summary"]
    assert sm["engine"]["model"] == d and sm["engine"]["architecture"] == "Qwen3ForCausalLM" and sm["engine"]["dtype"] == "float32"
    assert all(run["generated_tokens"] == 9 and run["error"] is None for run in data["runs"])
    assert sm["decode_achieved_gb_s"] > 0 and 0 < sm["decode_fraction_of_hbm_peak"] < 1
    assert sm["prefill_or_mixed_achieved_tflop_s"] >= 0 and sm["peaks"] in ("measured", "fallback")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("size", ["4b", "8b", "14b"])
def test_benchmark_layer_sizes(tmp_path, dtype, size):
    """The layer sizes of the benchmark configurations (Qwen3-4B, 8B, 14B: widths 2560 / 4096 / 5120, groups of 4 and 5
    query heads, untied heads), two layers and a cut-down vocabulary: whole, the last 32 tokens one by one, portions,
    and one mixed step (a portion of one request beside decoded tokens of two others), against the plain implementation."""
    from mini_inference_b200.engine.batch import StepEntry
    d, cfg = sized_model(tmp_path, size)
    ids = random_tokens(cfg["vocab_size"], 200, seed=1)
    want = plain_logits(d, ids)
    runner = make_engine(d, 16, 64, dtype=dtype, device=DEV)
    tol = 1e-4 if dtype == "float32" else 5e-2
    for name, cuts in (("whole", [200]), ("decode", [168] + [1] * 32), ("portions", [90, 7, 2, 64, 35, 2])):
        got = run_cuts(runner, name, ids, cuts)
        assert rel_err(got, want) < tol, (name, rel_err(got, want))
    a, b, c = (runner.cache.admit(k) for k in "abc")
    runner.step([StepEntry(a, ids[:150], []), StepEntry(b, ids[:37], []), StepEntry(c, ids[:64], [])])
    mixed = runner.step([StepEntry(a, ids[150:151], [0]), StepEntry(c, ids[64:160], range(96)), StepEntry(b, ids[37:38], [0])])
    ref = torch.cat([want[150:151], want[64:160], want[37:38]])
    assert rel_err(mixed.float().cpu(), ref) < tol, ("mixed", rel_err(mixed.float().cpu(), ref))
    if hasattr(runner.ops, "check_errors"):
        runner.ops.check_errors()


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("first_products", ["library", "stream"])
def test_benchmarked_decode_path(tmp_path, dtype, first_products):
    """The state the decode benchmark times, checked against the plain implementation: a start-up table that sends the
    out-projection and the down-projection to the weight-streaming kernel with their sums left for the next norm kernel
    to add up (and qkv / gate-up to the library or to the same kernel), weight-prefetch hints on, the step replayed as a
    CUDA graph from a bucket larger than the live batch, sampling on the device and the sampled tokens fed back there."""
    from mini_inference_b200 import LLM, SamplingParams
    from mini_inference_b200.engine.batch import StepEntry
    from mini_inference_b200.engine.graphs import DecodeGraphs
    from mini_inference_b200.ops import DeferredSum
    from tests.plain import qwen3_plain as plain
    d, cfg = sized_model(tmp_path, "4b")
    V, L = cfg["vocab_size"], LAYER_SIZES["4b"]
    llm = LLM(d, dtype=dtype, device=DEV, kv_block_size=16, kv_cache_tokens=2048, max_num_seqs=4, cuda_graphs=False)
    ops = llm.ops
    hidden, q_dim, inter = L["hidden_size"], L["num_attention_heads"] * L["head_dim"], L["intermediate_size"]
    qkv_rows = q_dim + 2 * L["num_key_value_heads"] * L["head_dim"]
    table = {}
    for m in ops.ROW_BUCKETS:
        table[(m, hidden, q_dim)] = table[(m, hidden, inter)] = table[(m, V, hidden)] = "stream"
        table[(m, qkv_rows, hidden)] = table[(m, 2 * inter, hidden)] = first_products
    deferred, hinted = [], []
    inner = ops.add_rmsnorm

    def counting(x, delta, weight, eps, rows=None, next_weight=None):
        deferred.append(isinstance(delta, DeferredSum))
        hinted.append(next_weight is not None)
        return inner(x, delta, weight, eps, rows, next_weight=next_weight)
    saved = ops._linear_choice
    ops._linear_choice, ops.add_rmsnorm = table, counting
    try:
        assert llm.model.blocks[0].hint1 and llm.model.blocks[0].hint2
        llm.graphs = DecodeGraphs(llm.runner, 4, buckets=[4])
        llm.graphs.capture()
        if dtype == "bfloat16":
            # two norms per layer + the final norm; all but the first get partial sums, all but the last a hint
            assert sum(deferred) >= 4 and sum(hinted) >= 4, (sum(deferred), sum(hinted))
        tol = 5e-2 if dtype == "bfloat16" else 1e-4
        lens = (40, 100, 203)
        seqs_ids = [random_tokens(V, n + 32, seed=30 + n) for n in lens]
        want = [plain_logits(d, ids) for ids in seqs_ids]
        seqs = [llm.cache.admit(("t", i), len(ids)) for i, ids in enumerate(seqs_ids)]
        for s, ids, n in zip(seqs, seqs_ids, lens):
            llm.runner.step([StepEntry(s, ids[:n], [])])
        G = llm.graphs
        worst = 0.0
        for k in range(32):                                  # 32 teacher-forced tokens through the graph, 3 live rows of 4
            for s in seqs:
                assert llm.cache.ensure(s, s.num_tokens + 1)
            G.fill(4, seqs, [ids[n + k] for ids, n in zip(seqs_ids, lens)])
            G.replay(4)
            got = G.logits_out[4][:3].float().cpu()
            for s in seqs:
                llm.cache.commit(s, s.num_tokens + 1)
            ref = torch.stack([w[n + k] for w, n in zip(want, lens)])
            worst = max(worst, rel_err(got, ref))
        assert worst < tol, ("graph decode", worst)
        # a mixed eager step under the same table: a portion of a fourth request beside a decoded token of the others
        for s in seqs[1:]:
            llm.cache.free(s)
        extra_ids = random_tokens(V, 30, seed=77)
        extra = llm.cache.admit(("t", 9), 64)
        # (request 0 is complete: its last fed token was position lens[0] + 31; feed one more to decode)
        more = random_tokens(V, 1, seed=78)
        full0 = seqs_ids[0] + more
        mixed = llm.runner.step([StepEntry(extra, extra_ids[:23], range(23)), StepEntry(seqs[0], more, [0])]).float().cpu()
        ref = torch.cat([plain_logits(d, extra_ids)[:23], plain_logits(d, full0)[-1:]])
        assert rel_err(mixed, ref) < tol, ("mixed", rel_err(mixed, ref))
        llm.cache.free(extra)
        llm.cache.free(seqs[0])
        # generation through the entry point: overlapped decode, the sampled tokens never leave the device between steps
        prompts = [random_tokens(V, n, seed=50 + n) for n in (7, 33, 90)]
        outs = llm.generate(prompts, SamplingParams(max_new_tokens=24))
        assert llm.stats()["graph_replays"] >= 32 + 20
        c, w = plain.load_model_dir(d)
        for p, g in zip(prompts, outs):
            ref = plain.forward_logits(c, w, p + g)
            err = (llm.score(p + g).float().cpu() - ref).abs().max().item()
            assert err < tol * ref.abs().max().item()
            for k, tok in enumerate(g):
                row = ref[len(p) - 1 + k]
                assert row[tok] >= row.max() - 2 * err, ("fed-back token", k)
        ops.check_errors()
        llm.cache.check_invariants()
    finally:
        ops._linear_choice = saved
        del ops.add_rmsnorm


@pytest.mark.parametrize("case", [1, 2, 3, 5])
def test_random_workloads_on_the_kernels(tiny_dirs, case):
    """The randomised workloads and settings of the scheduler tests (arrivals, lengths, pools down to barely enough, budgets,
    portions, batch limits) on the float32 kernels, with decode graphs on for half of them: tokens as the plain implementation's."""
    from mini_inference_b200.engine.llm import LLM
    from tests.test_scheduler_llm import random_workload

    def llm(d, **kw):
        return LLM(d, dtype="float32", device=DEV, cuda_graphs=case % 2 == 1, **kw)
    random_workload(tiny_dirs, case, llm)


def test_scheduler_in_bfloat16_is_judged_by_logits(tiny_dirs):
    """Chunked prompts, CUDA graphs, overlapped decode and a pool small enough to preempt, in bfloat16: every generated
    token is judged at its own position against the plain implementation (the logits of prompt + generated, and the token
    being the plain argmax up to twice the logits' error), not by comparing a few leading tokens."""
    from mini_inference_b200 import LLM, SamplingParams
    from tests.plain import qwen3_plain as plain
    d, cfg, page = tiny_dirs["F"]
    prompts = [random_tokens(cfg["vocab_size"], n, seed=90 + n) for n in (9, 30, 17, 41, 5, 26)]
    c, w = plain.load_model_dir(d)
    llm = LLM(d, dtype="bfloat16", device=DEV, kv_block_size=page, kv_cache_tokens=16 * 14, kv_watermark=0.0, max_num_seqs=4,
              chunked_prefill=True, max_batched_tokens=24, cuda_graphs=True, overlap_decode=True)
    outs = llm.generate(prompts, SamplingParams(max_new_tokens=40))
    st = llm.stats()
    assert st["preemptions"] > 0 and st["graph_replays"] > 0 and st["prefill_chunks"] > 0 and st["mixed_steps"] > 0
    llm.cache.check_invariants()
    assert llm.cache.free_pages() == llm.cache.num_pages
    for p, g in zip(prompts, outs):
        assert len(g) == 40
        ref = plain.forward_logits(c, w, p + g)
        mine = llm.score(p + g).float().cpu()
        err = (mine - ref).abs().max().item()
        assert err < TOLS["bfloat16"] * ref.abs().max().item()
        for k, tok in enumerate(g):
            row = ref[len(p) - 1 + k]
            assert row[tok] >= row.max() - 2 * err, (k, tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompts_under_page_pressure(tmp_path, dtype):
    """The long-context workload in small: 14B layer sizes (two layers), requests with prompts of ~1,500 tokens fed in
    portions of 512, a pool too small for all of them, so that the newest is preempted and recomputed; graphs on.  float32:
    the tokens equal those of a run with a large pool.  bfloat16: every token is judged at its position by its logits."""
    from mini_inference_b200 import LLM, SamplingParams
    from tests.plain import qwen3_plain as plain
    d, cfg = sized_model(tmp_path, "14b", vocab=1031)
    prompts = [random_tokens(cfg["vocab_size"], n, seed=200 + n) for n in (1500, 1409, 1333, 1467)]
    runs = {}
    small_pool = 364 * 16           # the four prompts take 359 pages, their 48 new tokens would need 371
    for pool in (small_pool, 16384):
        llm = LLM(d, dtype=dtype, device=DEV, kv_block_size=16, kv_cache_tokens=pool, kv_watermark=0.0, max_num_seqs=4,
                  max_model_len=2048, chunked_prefill=True, max_batched_tokens=512, cuda_graphs=True)
        runs[pool] = (llm.generate(prompts, SamplingParams(max_new_tokens=48)), llm.stats()["preemptions"])
        llm.cache.check_invariants()
        assert llm.cache.free_pages() == llm.cache.num_pages
        llm.ops.check_errors()
    (small, pre_small), (large, pre_large) = runs[small_pool], runs[16384]
    assert pre_small > 0 and pre_large == 0
    if dtype == "float32":
        assert small == large
        return
    c, w = plain.load_model_dir(d)
    for p, g in zip(prompts[:2], small[:2]):
        ref = plain.forward_logits(c, w, p + g)[len(p) - 1:]
        mine = llm.score(p + g).float().cpu()[len(p) - 1:]
        err = (mine - ref).abs().max().item()
        assert err < 5e-2 * ref.abs().max().item()
        assert all(ref[k][t] >= ref[k].max() - 2 * err for k, t in enumerate(g))


def test_start_up_choice_of_many_row_kernels(tmp_path):
    """The start-up timing of prompt-step products on the model's own weights: every shape and row bucket gets an answer, the
    parts' probes are used (gate/up with its activation, q/k/v with norm, rotation and cache write), only answers for the own
    kernel are kept, and a prompt step after it still gives the plain implementation's logits."""
    d, cfg = sized_model(tmp_path, "4b")
    ids = random_tokens(cfg["vocab_size"], 600, seed=3)
    want = plain_logits(d, ids)
    runner = make_engine(d, 16, 64, dtype="bfloat16", device=DEV)
    ops, model = runner.ops, runner.model
    probes = model.first_product_probes(ops)
    qkv_shape, gate_up_shape = tuple(model.blocks[0].parts["mixer"].qkv.shape), tuple(model.blocks[0].parts["feed_forward"].gate_up.shape)
    assert set(probes) == {qkv_shape, gate_up_shape}
    before = dict(ops._many_choice)
    try:
        report = ops.tune_many_rows(model.matrix_weights(), probes, iters=2, min_bytes=0)
        shapes = {tuple(int(v) for v in k.split(" ")[0].split("x")) for k in report}
        assert {qkv_shape, gate_up_shape} <= shapes and len(report) >= 2 * len(ops.MANY_BUCKETS)
        assert all(v["best"] in ("library", "tc2") and v["library"] > 0 and v["tc2"] > 0 for v in report.values())
        assert set(ops._many_choice.values()) <= {"tc2"}
        assert sorted(ops._many_choice) == sorted((int(k.split("<=")[1]), *(int(v) for v in k.split(" ")[0].split("x")))
                                                  for k, v in report.items() if v["best"] == "tc2")
        # whatever the clock said: the own kernel for every bucket of the gate/up shape and the library elsewhere is a legal table
        ops._many_choice = {(b, *gate_up_shape): "tc2" for b in ops.MANY_BUCKETS}
        got = run_cuts(runner, "chosen", ids, [600])
        assert rel_err(got, want) < 5e-2, rel_err(got, want)
    finally:
        ops._many_choice = before
    ops.check_errors()


def test_own_tensor_core_gemm_in_the_engine(tmp_path):
    """Prompt steps with every many-row product on this package's two-block tcgen05 GEMM (by default only where the start-up
    timing finds it faster), the gate/up product with the activation in its epilogue: same logits as the plain implementation."""
    d, cfg = sized_model(tmp_path, "4b")
    ids = random_tokens(cfg["vocab_size"], 700, seed=2)
    want = plain_logits(d, ids)
    runner = make_engine(d, 16, 64, dtype="bfloat16", device=DEV)
    saved = runner.ops.tc_gemm
    runner.ops.tc_gemm = True
    calls = []
    inner = runner.ops._gemm_tc
    runner.ops._gemm_tc = lambda *a: calls.append(a[0].shape[0]) or inner(*a)
    try:
        for name, cuts in (("whole", [700]), ("portions", [300, 257, 143])):
            got = run_cuts(runner, name, ids, cuts)
            assert rel_err(got, want) < 5e-2, (name, rel_err(got, want))
    finally:
        runner.ops.tc_gemm = saved
        del runner.ops._gemm_tc
    runner.ops.check_errors()
    assert calls and min(calls) >= 128          # qkv, o and down of every layer and step went through it
