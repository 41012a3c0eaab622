"""Each part of a layer alone, and the generality of the assembly: a toy mixer with state of
its own, defined here, is registered, built into a model next to attention layers, and stepped
through the framework's runner, cache manager and batch without touching the framework's files;
the execution order names a layer twice and lets a step read another step's cache."""
import pytest
import torch

from mini_inference_b200.cache import CacheManager
from mini_inference_b200.config.spec import ExecStep, LayerSpec, ModelSpec, PartSpec
from mini_inference_b200.engine.batch import BatchBuilder, StepEntry
from mini_inference_b200.engine.runner import ModelRunner
from mini_inference_b200.parts import (DecoderModel, KVCacheNeed, Part, StateNeed, StepContext, WeightSpec, build_part,
                                       register_block, register_mixer)
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
    in a state slot, advanced token by token in position order.  It asks the step builder for a per-entry array of
    its own (the flat row behind each entry's last token), which reaches it on the device beside the built-in fields."""
    step_arrays_key = "toy_ema"

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden, self.decay = spec.get("hidden_size"), spec.get("decay")

    def weight_specs(self):
        return [WeightSpec("mix", (self.hidden, self.hidden))]

    def cache_need(self):
        return StateNeed((self.hidden,), "float32")

    def load(self, tensors, dtype, device):
        self.mix = tensors["mix"]

    def step_arrays(self, facts):
        return {"seg_end": facts.q_start[1:].copy()}

    def forward(self, h, ctx, cache, position, owns_cache=True):
        out = torch.empty_like(h)
        q = ctx.batch.host["seg_q_start"]
        ends = ctx.batch.extras["toy_ema"]["seg_end"]                  # the array this mixer asked for, on the device
        assert ends.device == h.device and ends.dtype == torch.int32
        assert ends.tolist() == list(ctx.batch.extras_host["toy_ema"]["seg_end"]) == [int(v) for v in q[1:]]
        ends = ends.tolist()
        for s, slot in enumerate(ctx.batch.host["seg_slot"]):
            state = cache.state[slot]
            for t in range(q[s], ends[s]):
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
    def layer(mixer, position, weight_names):
        return LayerSpec.of("prenorm", weight_names, mixer=mixer, feed_forward=ffn, norm1=norm, norm2=norm, position=position)
    layers = (layer(attn, pos, names(0, qkvo + ["q_norm", "k_norm"])),
              layer(toy, PartSpec.of("none"), names(1, ["mix"])),
              layer(win, pos, names(2, qkvo)))
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
    assert set(runner.builder.hooks) == {"paged_attention", "toy_ema"}      # one hook per kind of part, not per layer
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
def ctx_for(device, entries_lens, cache, dtype=torch.float32, part=None):
    seqs = [cache.admit(i) for i in range(len(entries_lens))]
    entries = []
    for s, n in zip(seqs, entries_lens):
        cache.ensure(s, n)
        entries.append(StepEntry(s, [1] * n, []))
    hooks = {part.step_arrays_key: part.step_arrays} if part is not None else {}
    batch = BatchBuilder(cache, device, hooks).build(entries)
    batch.apply_table_updates(get_ops(device))
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
    ctx, seqs = ctx_for(device, lens, cache, part=part)
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


# ---------------------------------------------------------------- a toy routed feed-forward and a toy learned position encoding
from mini_inference_b200.parts import register_feed_forward, register_position  # noqa: E402


@register_feed_forward("toy_routed")
class ToyRouted(Part):
    """Top-2 of E small experts: router logits and the softmax over the two chosen in float32, the experts' products
    through the kernel namespace, an integer table that says where each router column's expert is stored."""
    def __init__(self, spec):
        super().__init__(spec)
        self.hidden, self.inter, self.E = spec.get("hidden_size"), spec.get("intermediate_size"), spec.get("experts")

    def weight_specs(self):
        return [WeightSpec("router", (self.E, self.hidden)), WeightSpec("w_in", (self.E * self.inter, self.hidden)),
                WeightSpec("w_out", (self.E * self.hidden, self.inter)), WeightSpec("place", (self.E,), kind="table")]

    def load(self, tensors, dtype, device):
        self.router, self.place = tensors["router"], tensors["place"]
        self.w_in = tensors["w_in"].view(self.E, self.inter, self.hidden)
        self.w_out = tensors["w_out"].view(self.E, self.hidden, self.inter)

    def forward(self, h, ctx):
        logits = h.float() @ self.router.float().T
        top, idx = logits.topk(2, dim=-1)
        gate = torch.softmax(top, dim=-1)
        out = torch.zeros(h.shape, dtype=torch.float32, device=h.device)
        for e in range(self.E):
            rows, which = (idx == e).nonzero(as_tuple=True)
            if rows.numel():
                slot = int(self.place[e])
                y = ctx.ops.linear(torch.relu(ctx.ops.linear(h[rows].contiguous(), self.w_in[slot])), self.w_out[slot])
                out.index_add_(0, rows, y.float() * gate[rows, which, None])
        return out.to(h.dtype)


@register_position("toy_learned")
class ToyLearnedPosition(Part):
    """A learned absolute encoding: a row of its own table is added to each token's embedding; nothing is rotated."""
    def __init__(self, spec):
        super().__init__(spec)
        self.size, self.max_pos = spec.get("hidden_size"), spec.get("max_position")

    def weight_specs(self):
        return [WeightSpec("table", (self.max_pos, self.size))]

    def load(self, tensors, dtype, device):
        self.table = tensors["table"]

    def rotary_inv_freq(self):
        return None

    def on_embedding(self, x, ctx):
        return (x.float() + self.table[ctx.batch.positions.long()].float()).to(x.dtype)


def routed_spec(hidden=48, vocab=61, inter=40, experts=4):
    norm = PartSpec.of("rmsnorm", size=hidden, eps=1e-5)
    pos = PartSpec.of("toy_learned", hidden_size=hidden, max_position=128)
    attn = PartSpec.of("gqa_attention", hidden_size=hidden, num_heads=3, num_kv_heads=1, head_dim=16, scale=0.25,
                       qk_norm=False, window=None)
    routed = PartSpec.of("toy_routed", hidden_size=hidden, intermediate_size=inter, experts=experts)
    dense = PartSpec.of("swiglu", hidden_size=hidden, intermediate_size=inter)

    def names(i, ffn_tensors):
        p = f"l{i}."
        d = {"norm1.weight": p + "n1", "norm2.weight": p + "n2", "position.table": "pos_table"}
        d.update({f"mixer.{t}": p + t for t in ("q_proj", "k_proj", "v_proj", "o_proj")})
        d.update({f"feed_forward.{t}": p + t for t in ffn_tensors})
        return tuple(sorted(d.items()))
    def layer(ffn, weight_names):
        return LayerSpec.of("prenorm", weight_names, mixer=attn, feed_forward=ffn, norm1=norm, norm2=norm, position=pos)
    layers = (layer(routed, names(0, ["router", "w_in", "w_out", "place"])),
              layer(dense, names(1, ["gate_proj", "up_proj", "down_proj"])),
              layer(routed, names(2, ["router", "w_in", "w_out", "place"])))
    return ModelSpec(hidden_size=hidden, vocab_size=vocab, layers=layers, order=tuple(ExecStep(i) for i in range(3)),
                     final_norm=norm, embedding_name="emb", final_norm_name="fn", lm_head_name=None, max_position=128)


def routed_plain(w, ids, hidden=48, inter=40, experts=4):
    n = len(ids)
    x = plain.embed(ids, w["emb"]) + w["pos_table"][:n]
    for i in range(3):
        h = plain.rms_norm(x, w[f"l{i}.n1"], 1e-5)
        q = (h @ w[f"l{i}.q_proj"].T).view(n, 3, 16)                 # nothing is rotated
        k = (h @ w[f"l{i}.k_proj"].T).view(n, 1, 16)
        v = (h @ w[f"l{i}.v_proj"].T).view(n, 1, 16)
        x = x + plain.causal_attention(q, k, v, 0.25, None).reshape(n, hidden) @ w[f"l{i}.o_proj"].T
        h = plain.rms_norm(x, w[f"l{i}.n2"], 1e-5)
        if i == 1:
            x = x + (torch.nn.functional.silu(h @ w[f"l{i}.gate_proj"].T) * (h @ w[f"l{i}.up_proj"].T)) @ w[f"l{i}.down_proj"].T
            continue
        logits = h @ w[f"l{i}.router"].T
        top, idx = logits.topk(2, dim=-1)
        gate = torch.softmax(top, dim=-1)
        w_in = w[f"l{i}.w_in"].view(experts, inter, hidden)
        w_out = w[f"l{i}.w_out"].view(experts, hidden, inter)
        y = torch.zeros(n, hidden)
        for t in range(n):
            for j in range(2):
                slot = int(w[f"l{i}.place"][idx[t, j]])
                y[t] += gate[t, j] * (torch.relu(h[t] @ w_in[slot].T) @ w_out[slot].T)
        x = x + y
    return plain.rms_norm(x, w["fn"], 1e-5) @ w["emb"].T


@pytest.mark.parametrize("device", DEVICES)
def test_toy_routed_feed_forward_and_learned_position(device):
    """A feed-forward with routing (float32 router, an integer table among its tensors) and a position encoding with a
    table of its own are registered here, chosen layer by layer beside a dense feed-forward, and stepped in portions."""
    model = DecoderModel(routed_spec())
    table = dict(model.weight_table())
    assert table["pos_table"].shape == (128, 48) and table["l0.place"].kind == "table"
    assert sum(name == "pos_table" for name, _ in model.weight_table()) == 1          # shared by the layers, loaded once
    g = torch.Generator().manual_seed(11)
    tensors = {}
    for name, ws in model.weight_table():
        if ws.kind == "table":
            t = torch.randperm(ws.shape[0], generator=g).to(torch.int32)
        elif ws.init == "norm":
            t = torch.rand(ws.shape, generator=g) + 0.5
        else:
            t = torch.randn(ws.shape, generator=g) * 0.15
        tensors[name] = t.to(device)
    model.load(dict(tensors), torch.float32, device)
    w = {k: (v.cpu() if v.dtype == torch.int32 else v.float().cpu()) for k, v in tensors.items()}
    cache = CacheManager(model.cache_needs(), 4, 64, 4, 128, dtype=torch.float32, device=device)
    runner = ModelRunner(model, cache, get_ops(device))
    ids = torch.randint(0, 61, (37,), generator=g).tolist()
    want = routed_plain(w, ids)
    for cuts in ([37], [20] + [1] * 17, random_cuts(37, __import__("random").Random(9))):
        seq, at, out = cache.admit("r"), 0, []
        for n in cuts:
            out.append(runner.step([StepEntry(seq, ids[at:at + n], range(n))]).float().cpu())
            at += n
        cache.free(seq)
        assert rel_err(torch.cat(out), want) < 3e-5, cuts
    cache.check_invariants()


# ---------------------------------------------------------------- a toy arrangement with roles of its own
@register_block("toy_parallel")
class ToyParallelBlock(Part):
    """x = x + mixer(n(x)) + feed_forward(n(x)) with ONE norm n shared by both branches, and a second norm of another
    size-less kind ("post") applied to the feed-forward's output: an arrangement whose roles are not the pre-norm block's."""
    roles = {"mixer": "mixer", "feed_forward": "feed_forward", "norm": "norm", "post": "norm", "position": "position"}

    def __init__(self, spec, parts):
        super().__init__(spec)
        self.parts = dict(parts)
        self.mixer = parts["mixer"]

    def forward(self, x, delta, ctx, cache, owns_cache=True):
        p = self.parts
        h = p["norm"].forward(x, delta, ctx)
        a = p["mixer"].forward(h, ctx, cache, p["position"], owns_cache)
        f = p["feed_forward"].forward(h, ctx)
        rows = torch.arange(f.shape[0], dtype=torch.int32, device=f.device)
        f = p["post"].forward(f, None, ctx, rows=rows)
        return x, (a.float() + f.float()).to(x.dtype)


def test_a_block_names_its_own_roles():
    """The layer description is a mapping role -> part that the block interprets: a block with one shared norm and a
    post-norm is built and stepped without touching the framework; a layer that gives the wrong roles is refused."""
    hidden = 48
    norm = PartSpec.of("rmsnorm", size=hidden, eps=1e-5)
    attn = PartSpec.of("gqa_attention", hidden_size=hidden, num_heads=3, num_kv_heads=1, head_dim=16, scale=0.25,
                       qk_norm=False, window=None)
    ffn = PartSpec.of("swiglu", hidden_size=hidden, intermediate_size=40)
    pos = PartSpec.of("rotary", head_dim=16, theta=10000.0)
    names = {"norm.weight": "n", "post.weight": "pn", "mixer.q_proj": "q", "mixer.k_proj": "k", "mixer.v_proj": "v",
             "mixer.o_proj": "o", "feed_forward.gate_proj": "g", "feed_forward.up_proj": "u", "feed_forward.down_proj": "d"}
    layer = LayerSpec.of("toy_parallel", names, mixer=attn, feed_forward=ffn, norm=norm, post=norm, position=pos)
    spec = ModelSpec(hidden_size=hidden, vocab_size=53, layers=(layer,), order=(ExecStep(0), ExecStep(0)), final_norm=norm,
                     embedding_name="emb", final_norm_name="fn", lm_head_name=None, max_position=64)
    model = DecoderModel(spec)
    assert {n for n, _ in model.weight_table()} == {"emb", "fn", *names.values()}
    w = random_weights(model, torch.float32, "cpu", seed=4)
    cache = CacheManager(model.cache_needs(), 4, 32, 2, 64, dtype=torch.float32, device="cpu")
    runner = ModelRunner(model, cache, TorchRefOps())
    ids = [5, 9, 2, 44, 17, 30, 8, 8, 21]
    n = len(ids)
    x = plain.embed(ids, w["emb"])
    cos, sin = plain.rotary_tables(torch.arange(n), 16, 10000.0, x.dtype)
    for _ in range(2):
        h = plain.rms_norm(x, w["n"], 1e-5)
        q = plain.apply_rope((h @ w["q"].T).view(n, 3, 16), cos, sin)
        k = plain.apply_rope((h @ w["k"].T).view(n, 1, 16), cos, sin)
        a = plain.causal_attention(q, k, (h @ w["v"].T).view(n, 1, 16), 0.25, None).reshape(n, hidden) @ w["o"].T
        f = (torch.nn.functional.silu(h @ w["g"].T) * (h @ w["u"].T)) @ w["d"].T
        x = x + a + plain.rms_norm(f, w["pn"], 1e-5)
    want = plain.rms_norm(x, w["fn"], 1e-5) @ w["emb"].T
    seq, out = cache.admit("p"), []
    for a0, b0 in ((0, 4), (4, 6), (6, 9)):
        out.append(runner.step([StepEntry(seq, ids[a0:b0], range(b0 - a0))]))
    assert rel_err(torch.cat(out), want) < 3e-5
    with pytest.raises(KeyError, match="roles"):
        DecoderModel(ModelSpec(hidden_size=hidden, vocab_size=53, order=(ExecStep(0),), final_norm=norm, embedding_name="emb",
                               final_norm_name="fn", lm_head_name=None, max_position=64,
                               layers=(LayerSpec.of("prenorm", names, mixer=attn, feed_forward=ffn, norm=norm, position=pos),)))


def test_optional_protocol_is_declared_not_probed():
    """Every optional fast-path name exists on Part with a default that means "not offered"; the built-in parts override
    what they offer, and the pre-norm block finds the attention mixer's first weight (the qkv matrix) for its hint."""
    base = Part(PartSpec.of("x"))
    assert (base.offers_open, base.open_weight, base.first_weight, base.accepts_deferred, base.takes_next_weight,
            base.step_arrays_key) == (False, None, None, False, False, None)
    model = DecoderModel(toy_spec())
    random_weights(model, torch.float32, "cpu")
    block = model.blocks[0]
    assert block.open_mixer and block.open_ffn and block.hint1 and block.hint2
    assert block.mixer.first_weight is block.mixer.qkv and block.feed_forward.first_weight is block.feed_forward.gate_up
    assert block.mixer.open_weight is block.mixer.o
    assert not model.blocks[1].open_mixer                                  # the toy mixer offers nothing
    assert model.deferrable_shapes() == {(64, 64), (64, 96)}
