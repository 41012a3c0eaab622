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
    else:       # bfloat16 rounding may flip a near-tie late in a sequence; the ways of running agree on the start
        assert all([x[:3] for x in o] == [x[:3] for x in want] for o in outs)


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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_benchmark_layer_sizes(tmp_path, dtype):
    """The layer sizes of the benchmark (Qwen3-4B: width 2560, 32/8 heads of 128, feed-forward 9728), two layers and
    a cut-down vocabulary: whole, the last 32 tokens one by one, and portions, against the plain implementation.  This
    is where the tensor-core attention, the TMA weight-streaming products and the deferred sums run at their real shapes."""
    from mini_inference_b200.weights import write_random_model
    cfg = {"architectures": ["Qwen3ForCausalLM"], "hidden_size": 2560, "num_hidden_layers": 2, "num_attention_heads": 32,
           "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 9728, "vocab_size": 4099, "rope_theta": 1000000.0,
           "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 4096}
    d = str(tmp_path / "bench_sizes")
    write_random_model(cfg, d, seed=3, std=0.02)
    ids = random_tokens(cfg["vocab_size"], 200, seed=1)
    want = plain_logits(d, ids)
    runner = make_engine(d, 16, 64, dtype=dtype, device=DEV)
    tol = 1e-4 if dtype == "float32" else 5e-2
    for name, cuts in (("whole", [200]), ("decode", [168] + [1] * 32), ("portions", [90, 7, 2, 64, 35, 2])):
        got = run_cuts(runner, name, ids, cuts)
        assert rel_err(got, want) < tol, (name, rel_err(got, want))
    if hasattr(runner.ops, "check_errors"):
        runner.ops.check_errors()
