"""The generic decoder: embedding, the layers of a ModelSpec run in the spec's order, final
norm on the rows whose logits are wanted, and the head (engine/core/model_runner.py:112-135).
It is built from the spec alone; which family the spec came from is unknown here."""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from ..config.spec import ModelSpec, PartSpec
from .base import Part, WeightSpec, build_part, lookup


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self._positions: Dict = {}
        self.blocks = []
        self._owned: List[Tuple[str, WeightSpec, Part]] = []      # (checkpoint name, spec, owner)
        for li, layer in enumerate(spec.layers):
            names = dict(layer.weight_names)
            block_cls = lookup("block", layer.block)
            given = dict(layer.parts)
            if set(given) != set(block_cls.roles):
                raise KeyError(f"layer {li}: block '{layer.block}' arranges the roles {sorted(block_cls.roles)}, "
                               f"the layer gives {sorted(given)}")
            parts = {}
            for role, family in block_cls.roles.items():
                pspec = given[role]
                if family == "position":               # one position part per distinct spec, shared by its layers;
                    part = self._positions.get(pspec)  # its tensors (if any) are named by the first layer that uses it
                    if part is not None:
                        parts[role] = part
                        continue
                    part = self._positions[pspec] = build_part(family, pspec)
                else:
                    part = build_part(family, pspec)
                parts[role] = part
                for ws in part.weight_specs():
                    key = f"{role}.{ws.name}"
                    if key not in names:
                        raise KeyError(f"layer {li}: weight_names has no entry for '{key}'")
                    self._owned.append((names[key], ws, part))
            self.blocks.append(block_cls(PartSpec.of(layer.block), parts))
        self.final_norm = build_part("norm", spec.final_norm)
        norms = [p for b in self.blocks for role, p in b.parts.items() if b.roles[role] == "norm"] + [self.final_norm]
        self._norms_accept_deferred = all(n.accepts_deferred for n in norms)
        for ws in self.final_norm.weight_specs():
            self._owned.append((spec.final_norm_name, ws, self.final_norm))
        self.embedding = None
        self.lm_head = None
        self.dtype = None
        self.device = None

    # ---------------------------------------------------------------- weights
    def weight_table(self) -> List[Tuple[str, WeightSpec]]:
        """Every tensor the checkpoint must hold: (checkpoint name, spec)."""
        table = [(self.spec.embedding_name, WeightSpec("embedding", (self.spec.vocab_size, self.spec.hidden_size)))]
        table += [(name, ws) for name, ws, _ in self._owned]
        if self.spec.lm_head_name is not None:
            table.append((self.spec.lm_head_name, WeightSpec("lm_head", (self.spec.vocab_size, self.spec.hidden_size))))
        return table

    def ignorable_names(self):
        """Tensors a checkpoint may hold that the model does not read (a tied head's copy)."""
        return {"lm_head.weight"} if self.spec.lm_head_name is None else set()

    def load(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype, device) -> None:
        """tensors: checkpoint name -> tensor already on the device in its runtime dtype."""
        self.dtype, self.device = dtype, torch.device(device)
        per_part: Dict[int, Dict[str, torch.Tensor]] = {}
        for name, ws, part in self._owned:
            per_part.setdefault(id(part), {})[ws.name] = tensors[name]
        seen = set()
        for _, _, part in self._owned:
            if id(part) not in seen:
                seen.add(id(part))
                part.load(per_part[id(part)], dtype, self.device)
        for position in self._positions.values():
            if id(position) not in seen:
                position.load({}, dtype, self.device)
        self.embedding = tensors[self.spec.embedding_name]
        self.lm_head = self.embedding if self.spec.lm_head_name is None else tensors[self.spec.lm_head_name]

    def matrix_weights(self):
        """The matrices the model multiplies by (after the parts fused what they fuse)."""
        out = []
        for block in self.blocks:
            for part in block.parts.values():
                out += [v for v in vars(part).values() if isinstance(v, torch.Tensor) and v.dim() == 2 and v.is_floating_point()]
        out.append(self.lm_head)
        return out

    def deferrable_shapes(self):
        """(N, K) of the products whose only reader is a norm (the last product of a mixer or feed-forward that offers
        forward_open), when every norm accepts deferred sums: the kernel namespace may time them accordingly."""
        if not self._norms_accept_deferred:
            return frozenset()
        shapes = set()
        for block in self.blocks:
            for part in block.parts.values():
                w = part.open_weight
                if part.offers_open and isinstance(w, torch.Tensor) and w.dim() == 2:
                    shapes.add((w.shape[0], w.shape[1]))
        return frozenset(shapes)

    def gated_shapes(self):
        """(N, K) of the matrices that go through ctx.ops.gated_linear."""
        shapes = set()
        for block in self.blocks:
            for part in block.parts.values():
                w = part.gated_weight
                if isinstance(w, torch.Tensor) and w.dim() == 2:
                    shapes.add((w.shape[0], w.shape[1]))
        return frozenset(shapes)

    def first_product_probes(self, ops):
        """{(N, K) of a part's first weight: probe(rows) -> run(weight)} for the parts that offer one (see Part)."""
        probes = {}
        for block in self.blocks:
            for part in block.parts.values():
                w = part.first_weight
                if isinstance(w, torch.Tensor) and w.dim() == 2 and (w.shape[0], w.shape[1]) not in probes:
                    if part.first_product_probe(ops, 1) is not None:
                        probes[(w.shape[0], w.shape[1])] = (lambda rows, part=part: part.first_product_probe(ops, rows))
        return probes

    def step_flops(self, rows: int, pairs: int, logit_rows: int) -> int:
        """Floating-point operations of a step that feeds `rows` tokens which see `pairs` (query, key) pairs in all and
        wants logits for `logit_rows` of them: 2 per weight element and row, plus what the mixers report."""
        total = 2 * logit_rows * self.lm_head.numel()
        for step in self.spec.order:
            for part in self.blocks[step.layer].parts.values():
                total += 2 * rows * sum(v.numel() for v in vars(part).values()
                                        if isinstance(v, torch.Tensor) and v.dim() == 2 and v.is_floating_point())
                total += part.step_flops(rows, pairs)
        return total

    def step_array_hooks(self):
        """{key: part.step_arrays} of the parts that ask for per-step arrays of their own, one per key."""
        hooks = {}
        for block in self.blocks:
            for part in block.parts.values():
                if part.step_arrays_key is not None:
                    hooks.setdefault(part.step_arrays_key, part.step_arrays)
        return hooks

    # ---------------------------------------------------------------- cache needs
    def cache_needs(self):
        """Per execution step: the mixer's need, or None when the step reads another's cache."""
        needs = []
        for step in self.spec.order:
            needs.append(None if step.cache_from is not None else self.blocks[step.layer].mixer.cache_need())
        return needs

    # ---------------------------------------------------------------- one step
    def forward(self, ctx, caches):
        """caches[i]: LayerCache of execution step i.  Returns float32 logits for
        ctx.batch.logit_rows, or None when no row wants logits."""
        b, ops = ctx.batch, ctx.ops
        ctx.defer_ok = self._norms_accept_deferred and getattr(ops, "deferred", False)
        ctx.hints_ok = getattr(ops, "takes_hints", False)
        x = ops.embedding(b.token_ids, self.embedding)
        for position in self._positions.values():
            x = position.on_embedding(x, ctx)
        delta = None
        for i, step in enumerate(self.spec.order):
            src = i if step.cache_from is None else step.cache_from
            x, delta = self.blocks[step.layer].forward(x, delta, ctx, caches[src], step.cache_from is None)
        if b.num_logit_rows == 0:
            return None
        h = self.final_norm.forward(x, delta, ctx, rows=b.logit_rows)
        return ops.linear(h, self.lm_head, out_dtype=torch.float32)
