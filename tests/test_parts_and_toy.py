"""Each part of a layer alone, and the generality of the assembly: a toy mixer with state of
its own, defined here, is registered, built into a model next to attention layers, and stepped
through the framework's runner, cache manager and batch without touching the framework's files;
the execution order names a layer twice and lets a step read another step's cache."""
import pytest
import torch

from mini_inference_b200.cache import CacheManager
from mini_inference_b200.config.spec import ExecStep, LayerSpec, ModelSpec, PartSpec
from mini_inference_b200.engine.batch import StepBatch, StepEntry
from mini_inference_b200.engine.runner import ModelRunner
from mini_inference_b200.parts import (DecoderModel, KVCacheNeed, Part, StateNeed, StepContext, WeightSpec, build_part,
                                       register_mixer)
from tests.helpers import random_cuts, rel_err
from tests.plain import qwen3_plain as plain
from tests.ref_ops import TorchRefOps

DEVICES = ["cpu", pytest.param("cuda:0", marks=pytest.mark.gpu)]


def get_ops(device):
    if device == "cpu":
        return TorchRefOps()
    from mini_inference_b200.ops import get_ops
    return get_ops(device)


# ---------------------------------------------------------------- a toy mixer with state
@register_mixer("toy_ema")
class ToyEMA(Part):
    """y_t = W s_t with s_t = a * s_{t-1} + (1 - a) * h_t: a running average kept per request
    in a state slot, advanced token by token in position order."""
    def __init__(self, spec):
        super().__init__(spec)
        self.hidden, self.decay = spec.get("hidden_size"), spec.get("decay")

    def weight_specs(self):
        return [WeightSpec("mix", (self.hidden, self.hidden))]

    def cache_need(self):
        return StateNeed((self.hidden,), "float32")

    def load(self, tensors, dtype, device):
        self.mix = tensors["mix"]

    def forward(self, h, ctx, cache, position, owns_cache=True):
        out = torch.empty_like(h)
        q = ctx.batch.host["seg_q_start"]
        for s, slot in enumerate(ctx.batch.host["seg_slot"]):
            state = cache.state[slot]
            for t in range(q[s], q[s + 1]):
                state.mul_(self.decay).add_(h[t].float(), alpha=1 - self.decay)
                out[t] = state.to(h.dtype)
        return ctx.ops.linear(out, self.mix)


def toy_spec(hidden=64, vocab=97):
    norm = PartSpec.of("rmsnorm", size=hidden, eps=1e-5)
    pos = PartSpec.of("rotary", head_dim=16, theta=10000.0)
    ffn = PartSpec.of("swiglu", hidden_size=hidden, intermediate_size=96)
    attn = PartSpec.of("gqa_attention", hidden_size=hidden, num_heads=4, num_kv_heads=2, head_dim=16, scale=0.25,
                       qk_norm=True, qk_norm_eps=1e-5, window=None)
    win = PartSpec.of("gqa_attention", hidden_size=hidden, num_heads=4, num_kv_heads=2, head_dim=16, scale=0.25,
                      qk_norm=False, window=7)
    toy = PartSpec.of("toy_ema", hidden_size=hidden, decay=0.8)

    def names(i, mixer_tensors):
        p = f"l{i}."
        d = {"norm1.weight": p + "n1", "norm2.weight": p + "n2", "feed_forward.gate_proj": p + "g",
             "feed_forward.up_proj": p + "u", "feed_forward.down_proj": p + "d"}
        d.update({f"mixer.{t}": p + t for t in mixer_tensors})
        return tuple(sorted(d.items()))
    qkvo = ["q_proj", "k_proj", "v_proj", "o_proj"]
    layers = (LayerSpec("prenorm", attn, ffn, norm, pos, names(0, qkvo + ["q_norm", "k_norm"])),
              LayerSpec("prenorm", toy, ffn, norm, PartSpec.of("none"), names(1, ["mix"])),
              LayerSpec("prenorm", win, ffn, norm, pos, names(2, qkvo)))
    # layer 0 runs twice (own caches); the last step re-reads the keys and values of step 0
    order = (ExecStep(0), ExecStep(1), ExecStep(2), ExecStep(0), ExecStep(0, cache_from=0))
    return ModelSpec(hidden_size=hidden, vocab_size=vocab, layers=layers, order=order, final_norm=norm,
                     embedding_name="emb", final_norm_name="fn", lm_head_name="head", max_position=512)


def random_weights(model, dtype, device, seed=0):
    g = torch.Generator().manual_seed(seed)
    tensors = {}
    for name, ws in model.weight_table():
        t = torch.rand(ws.shape, generator=g) + 0.5 if ws.init == "norm" else torch.randn(ws.shape, generator=g) * 0.08
        tensors[name] = t.to(torch.bfloat16).to(dtype).to(device)
    model.load(dict(tensors), dtype, device)
    return {k: v.float().cpu() for k, v in tensors.items()}


def toy_plain(w, ids, hidden=64):
    """Whole-sequence statement of the toy model, from the plain implementation's parts."""
    cfg = {"num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "rms_norm_eps": 1e-5}
    x = plain.embed(ids, w["emb"])
    n = len(ids)
    cos, sin = plain.rotary_tables(torch.arange(n), 16, 10000.0, x.dtype)

    def attn(i, h, window, qk_norm, kv=None):
        q = (h @ w[f"l{i}.q_proj"].T).view(n, 4, 16)
        if qk_norm:
            q = plain.rms_norm(q, w[f"l{i}.q_norm"], 1e-5)
        q = plain.apply_rope(q, cos, sin)
        if kv is None:
            k = (h @ w[f"l{i}.k_proj"].T).view(n, 2, 16)
            if qk_norm:
                k = plain.rms_norm(k, w[f"l{i}.k_norm"], 1e-5)
            kv = (plain.apply_rope(k, cos, sin), (h @ w[f"l{i}.v_proj"].T).view(n, 2, 16))
        o = plain.causal_attention(q, kv[0], kv[1], 0.25, window)
        return o.reshape(n, 64) @ w[f"l{i}.o_proj"].T, kv

    def ema(i, h):
        s, out = torch.zeros(hidden), []
        for t in range(n):
            s = 0.8 * s + 0.2 * h[t]
            out.append(s.clone())
        return torch.stack(out) @ w[f"l{i}.mix"].T

    kv0 = None
    for step, (i, shared) in enumerate([(0, False), (1, False), (2, False), (0, False), (0, True)]):
        h = plain.rms_norm(x, w[f"l{i}.n1"], 1e-5)
        if i == 1:
            a = ema(i, h)
        elif i == 2:
            a, _ = attn(i, h, 7, False)
        else:
            a, kv = attn(i, h, None, True, kv0 if shared else None)
            if step == 0:
                kv0 = kv
        x = x + a
        h = plain.rms_norm(x, w[f"l{i}.n2"], 1e-5)
        x = x + (torch.nn.functional.silu(h @ w[f"l{i}.g"].T) * (h @ w[f"l{i}.u"].T)) @ w[f"l{i}.d"].T
    return plain.rms_norm(x, w["fn"], 1e-5) @ w["head"].T


@pytest.mark.parametrize("device", DEVICES)
def test_toy_mixer_is_registered_built_and_stepped(device):
    model = DecoderModel(toy_spec())
    w = random_weights(model, torch.float32, device)
    needs = model.cache_needs()
    assert [type(n).__name__ if n else None for n in needs] == ["KVCacheNeed", "StateNeed", "KVCacheNeed", "KVCacheNeed", None]
    cache = CacheManager(needs, 4, 64, 4, 512, dtype=torch.float32, device=device)
    assert len(cache.kv_groups) == 2 and len(cache.state_groups) == 1        # full keys (2 steps) and a window
    runner = ModelRunner(model, cache, get_ops(device))
    g = torch.Generator().manual_seed(3)
    seqs = {k: torch.randint(0, 97, (n,), generator=g).tolist() for k, n in (("a", 29), ("b", 17))}
    want = {k: toy_plain(w, ids) for k, ids in seqs.items()}
    # whole, then in portions, then both requests interleaved (the state slot is per request)
    for cuts_of in (lambda n: [n], lambda n: random_cuts(n, __import__("random").Random(5)), lambda n: [n - 8] + [1] * 8):
        live = {k: (cache.admit(k), cuts_of(len(ids)), [0], []) for k, ids in seqs.items()}
        while any(c for _, c, _, _ in live.values()):
            entries, owners = [], []
            for k, (seq, cuts, at, out) in live.items():
                if cuts:
                    n = cuts.pop(0)
                    entries.append(StepEntry(seq, seqs[k][at[0]:at[0] + n], range(n)))
                    owners.append((k, n))
                    at[0] += n
            logits = runner.step(entries).float().cpu()
            row = 0
            for k, n in owners:
                live[k][3].append(logits[row:row + n])
                row += n
        for k, (seq, _, _, out) in live.items():
            assert rel_err(torch.cat(out), want[k]) < 3e-5, k
            cache.free(seq)
        cache.check_invariants()


# ---------------------------------------------------------------- each built-in part alone
def ctx_for(device, entries_lens, cache, dtype=torch.float32):
    seqs = [cache.admit(i) for i in range(len(entries_lens))]
    entries = []
    for s, n in zip(seqs, entries_lens):
        cache.ensure(s, n)
        entries.append(StepEntry(s, [1] * n, []))
    batch = StepBatch(entries, cache, device)
    return StepContext(get_ops(device), batch, dtype, device), seqs


@pytest.mark.parametrize("device", DEVICES)
def test_norm_part(device):
    part = build_part("norm", PartSpec.of("rmsnorm", size=72, eps=1e-3))
    assert [(w.name, w.shape, w.kind) for w in part.weight_specs()] == [("weight", (72,), "vector")]
    g = torch.Generator().manual_seed(0)
    w, x, d = torch.rand(72, generator=g) + 0.5, torch.randn(5, 72, generator=g), torch.randn(5, 72, generator=g)
    part.load({"weight": w.to(device)}, torch.float32, device)
    ctx = StepContext(get_ops(device), None, torch.float32, device)
    xs = x.clone().to(device)
    y = part.forward(xs, d.to(device), ctx)
    assert torch.allclose(xs.cpu(), x + d, atol=1e-6)                      # the residual stream took the delta
    assert torch.allclose(y.cpu(), plain.rms_norm(x + d, w, 1e-3), atol=1e-5)
    rows = torch.tensor([4, 1], dtype=torch.int32, device=device)
    y2 = part.forward(x.clone().to(device), None, ctx, rows=rows)
    assert torch.allclose(y2.cpu(), plain.rms_norm(x[[4, 1]], w, 1e-3), atol=1e-5)


@pytest.mark.parametrize("device", DEVICES)
def test_feed_forward_part(device):
    part = build_part("feed_forward", PartSpec.of("swiglu", hidden_size=40, intermediate_size=56))
    g = torch.Generator().manual_seed(1)
    w = {n: torch.randn(s.shape, generator=g) * 0.2 for s in part.weight_specs() for n in [s.name]}
    part.load({k: v.to(device) for k, v in w.items()}, torch.float32, device)
    assert part.gate_up.shape == (112, 40)
    h = torch.randn(7, 40, generator=g)
    y = part.forward(h.to(device), StepContext(get_ops(device), None, torch.float32, device))
    named = {"p.mlp.gate_proj.weight": w["gate_proj"], "p.mlp.up_proj.weight": w["up_proj"], "p.mlp.down_proj.weight": w["down_proj"]}
    assert torch.allclose(y.cpu(), plain.swiglu_mlp(h, named, "p."), atol=1e-5)


@pytest.mark.parametrize("device", DEVICES)
def test_position_part(device):
    part = build_part("position", PartSpec.of("rotary", head_dim=48, theta=5000.0))
    part.load({}, torch.float32, device)
    inv = part.rotary_inv_freq().cpu()
    assert torch.equal(inv, 1.0 / (5000.0 ** (torch.arange(0, 48, 2, dtype=torch.float32) / 48)))
    assert build_part("position", PartSpec.of("none")).rotary_inv_freq() is None


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("window,qk_norm", [(None, True), (6, False)])
def test_attention_part(device, window, qk_norm):
    H, KV, D, hid = 6, 2, 16, 40
    part = build_part("mixer", PartSpec.of("gqa_attention", hidden_size=hid, num_heads=H, num_kv_heads=KV, head_dim=D,
                                           scale=0.3, qk_norm=qk_norm, qk_norm_eps=1e-4, window=window))
    assert part.cache_need() == KVCacheNeed(KV, D, window)
    pos = build_part("position", PartSpec.of("rotary", head_dim=D, theta=777.0))
    pos.load({}, torch.float32, device)
    g = torch.Generator().manual_seed(2)
    w = {s.name: (torch.rand(s.shape, generator=g) + 0.5 if s.init == "norm" else torch.randn(s.shape, generator=g) * 0.3)
         for s in part.weight_specs()}
    part.load({k: v.to(device) for k, v in w.items()}, torch.float32, device)
    cache = CacheManager([part.cache_need()], 4, 32, 2, 256, dtype=torch.float32, device=device)
    lens = [19, 11]
    ctx, seqs = ctx_for(device, lens, cache)
    h = torch.randn(sum(lens), hid, generator=g)
    y = part.forward(h.to(device), ctx, cache.layer_caches[0], pos).cpu()
    at = 0
    for n in lens:
        hs = h[at:at + n]
        cos, sin = plain.rotary_tables(torch.arange(n), D, 777.0, torch.float32)
        q, k = (hs @ w["q_proj"].T).view(n, H, D), (hs @ w["k_proj"].T).view(n, KV, D)
        if qk_norm:
            q, k = plain.rms_norm(q, w["q_norm"], 1e-4), plain.rms_norm(k, w["k_norm"], 1e-4)
        o = plain.causal_attention(plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin),
                                   (hs @ w["v_proj"].T).view(n, KV, D), 0.3, window)
        assert torch.allclose(y[at:at + n], o.reshape(n, H * D) @ w["o_proj"].T, atol=2e-5)
        at += n
