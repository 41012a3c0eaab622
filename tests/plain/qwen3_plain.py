"""Plain, slow Qwen3-dense forward pass: whole sequences, no cache, no batching.

This file is the oracle the engine is compared with.  It shares no code with the
package: every function below is written from the formulas the reference engine
executes (paths are relative to the davidjoyme/mini-inference project root).
The reference re-uses the norm / rotary / MLP modules of the model object it
loads, so for those parts the formula is the one the reference was observed to
compute (checked numerically once, see tests/golden/).

Everything runs in the dtype of the weights it is given (float32 in the tests);
softmax, norm statistics and rotation angles are always float32.
"""
from __future__ import annotations

import math

import torch


def embed(token_ids, table):
    """x_t = E[id_t]  (engine/core/model_runner.py:115)."""
    return table[torch.as_tensor(token_ids, dtype=torch.long)]


def rms_norm(x, weight, eps):
    """y = w * cast(x32 * rsqrt(mean(x32^2) + eps)); statistics in float32, eps inside the
    square root, weight applied after the cast back (engine/core/model_runner.py:120-121,133
    call the model's norm modules; per-head use at :149-150)."""
    x32 = x.float()
    var = x32.pow(2).mean(dim=-1, keepdim=True)
    return weight * (x32 * torch.rsqrt(var + eps)).to(x.dtype)


def rotary_tables(positions, head_dim, theta, dtype):
    """cos/sin [n, D]: inv_freq_i = 1 / theta^(2i/D), angle = pos * inv_freq, the half-size
    angle vector repeated twice (engine/core/model_runner.py:116-117 takes them from the
    model's rotary module; the layout is fixed by rotate_half at :6-8)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    ang = torch.as_tensor(positions, dtype=torch.float32)[:, None] * inv_freq[None, :]
    ang = torch.cat([ang, ang], dim=-1)
    return ang.cos().to(dtype), ang.sin().to(dtype)


def rotate_half(x):
    """cat(-x[D/2:], x[:D/2])  (engine/core/model_runner.py:6-8)."""
    half = x.shape[-1] // 2
    return torch.cat([-x[..., half:], x[..., :half]], dim=-1)


def apply_rope(x, cos, sin):
    """x*cos + rotate_half(x)*sin with cos/sin broadcast over heads
    (engine/core/model_runner.py:151-152).  x: [n, heads, D]; cos/sin: [n, D]."""
    return x * cos[:, None, :] + rotate_half(x) * sin[:, None, :]


def causal_attention(q, k, v, scale, window=None):
    """softmax_j(scale * q_p . k_j) over keys j <= p (engine/core/model_runner.py:165-172;
    decode sees j < seq_len, kernels/paged_attention/decode_triton.py:25-30,43); query head h
    reads kv head h // (H / KV) (kernels/paged_attention/reference.py:14,25-26).  With a
    window W only keys p - W < j <= p are visible.  q: [n, H, D]; k, v: [n, KV, D]."""
    n, H, D = q.shape
    group = H // k.shape[1]
    kk = k.repeat_interleave(group, dim=1).float()
    vv = v.repeat_interleave(group, dim=1).float()
    scores = torch.einsum("phd,jhd->hpj", q.float(), kk) * scale
    pos = torch.arange(n)
    visible = pos[None, :] <= pos[:, None]
    if window is not None:
        visible &= pos[None, :] > pos[:, None] - window
    scores = scores.masked_fill(~visible[None], float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    out = torch.einsum("hpj,jhd->phd", probs, vv)
    return out.to(q.dtype)


def attention_block(h, w, prefix, cfg, cos, sin, window=None, kv_override=None):
    """q/k/v projections, per-head q/k RMSNorm before RoPE, attention, output projection
    (engine/core/model_runner.py:137-196).  Returns (out, (k, v)) so that a later layer may
    re-use this layer's keys and values."""
    n = h.shape[0]
    H, KV, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    q = (h @ w[prefix + "self_attn.q_proj.weight"].T).view(n, H, D)
    q = rms_norm(q, w[prefix + "self_attn.q_norm.weight"], cfg["rms_norm_eps"])
    q = apply_rope(q, cos, sin)
    if kv_override is None:
        k = (h @ w[prefix + "self_attn.k_proj.weight"].T).view(n, KV, D)
        v = (h @ w[prefix + "self_attn.v_proj.weight"].T).view(n, KV, D)
        k = rms_norm(k, w[prefix + "self_attn.k_norm.weight"], cfg["rms_norm_eps"])
        k = apply_rope(k, cos, sin)
    else:
        k, v = kv_override
    o = causal_attention(q, k, v, D ** -0.5, window)
    return o.reshape(n, H * D) @ w[prefix + "self_attn.o_proj.weight"].T, (k, v)


def swiglu_mlp(h, w, prefix):
    """down(silu(gate(h)) * up(h))  (engine/core/model_runner.py:124-131;
    engine/core/fused_linear.py:173-177)."""
    g = h @ w[prefix + "mlp.gate_proj.weight"].T
    u = h @ w[prefix + "mlp.up_proj.weight"].T
    return (torch.nn.functional.silu(g) * u) @ w[prefix + "mlp.down_proj.weight"].T


def layer_windows(cfg):
    """Per-layer window (None = all keys) from the config keys layer_types / sliding_window /
    use_sliding_window / max_window_layers.  The reference refuses such models
    (engine/models.py:17-22); the oracle defines the meaning the engine implements."""
    L = cfg["num_hidden_layers"]
    W = cfg.get("sliding_window")
    types = cfg.get("layer_types")
    if types:
        return [W if "sliding" in t else None for t in types]
    if cfg.get("use_sliding_window") and W:
        first = cfg.get("max_window_layers", L)
        return [W if i >= first else None for i in range(L)]
    return [None] * L


def normalise_config(cfg):
    """Fill the keys that config.json may leave out (engine/core/model_runner.py:77-79)."""
    cfg = dict(cfg)
    cfg.setdefault("num_key_value_heads", cfg["num_attention_heads"])
    if not cfg.get("head_dim"):
        cfg["head_dim"] = cfg["hidden_size"] // cfg["num_attention_heads"]
    if "rope_theta" not in cfg:
        cfg["rope_theta"] = cfg["rope_parameters"]["rope_theta"]
    cfg.setdefault("rms_norm_eps", 1e-6)
    cfg.setdefault("tie_word_embeddings", False)
    return cfg


def forward_logits(cfg, w, token_ids, order=None, share=None):
    """Logits [n, vocab] (float32) for every position of one whole sequence
    (engine/core/model_runner.py:112-135, all_logits=True).

    order: execution order as a list of layer indices (default 0..L-1; a layer may appear
    twice).  share: {step index -> earlier step index} whose keys/values the step attends to
    instead of its own."""
    cfg = normalise_config(cfg)
    n = len(token_ids)
    x = embed(token_ids, w["model.embed_tokens.weight"])
    cos, sin = rotary_tables(torch.arange(n), cfg["head_dim"], cfg["rope_theta"], x.dtype)
    windows = layer_windows(cfg)
    order = list(range(cfg["num_hidden_layers"])) if order is None else order
    share = share or {}
    kvs = {}
    for step, i in enumerate(order):
        p = f"model.layers.{i}."
        h = rms_norm(x, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
        a, kv = attention_block(h, w, p, cfg, cos, sin, windows[i],
                                kv_override=kvs[share[step]] if step in share else None)
        kvs[step] = kv
        x = x + a
        h = rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        x = x + swiglu_mlp(h, w, p)
    x = rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return (x @ head.T).float()


def greedy_generate(cfg, w, prompt_ids, max_new_tokens):
    """Argmax continuation, recomputing the whole sequence for every new token
    (engine/core/sampler.py:4 is the argmax; ties go to the lowest id)."""
    ids = list(prompt_ids)
    for _ in range(max_new_tokens):
        ids.append(int(forward_logits(cfg, w, ids)[-1].argmax()))
    return ids[len(prompt_ids):]


def softmax_temperature(logits, temperature):
    """probs = softmax(logits / max(temperature, 1e-5))  (engine/core/sampler.py:7)."""
    return torch.softmax(logits.float() / max(temperature, 1e-5), dim=-1)


def read_safetensors(path):
    """Minimal reader of the safetensors container, independent of the package's own
    (8-byte little-endian header length, JSON header, raw little-endian data)."""
    import json
    import struct
    kinds = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16,
             "I32": torch.int32, "I64": torch.int64}
    with open(path, "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(hlen))
        data = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        t = torch.frombuffer(bytearray(data[a:b]), dtype=kinds[info["dtype"]])
        out[name] = t.reshape(info["shape"]).clone()
    return out


def load_model_dir(path, dtype=torch.float32):
    """(config dict, weights dict cast to dtype) of a model folder."""
    import json
    import os
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    w = {k: v.to(dtype) for k, v in read_safetensors(os.path.join(path, "model.safetensors")).items()}
    return cfg, w


__all__ = [name for name in dir() if not name.startswith("_") and name not in ("math", "torch")]
