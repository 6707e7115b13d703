"""A model built from a `ModelSpec`: its parts, the tensors they expect, and one forward pass over
a step's batch.

The forward pass is the reference's layer loop (src/main.zig:846-861 for a prompt portion,
:1189-1217 for a decoded token: layers, final RMSNorm, lm_head) run once for a flattened batch of
several requests; the head is computed only at the rows whose logits are wanted (the reference
computes the last row, src/main.zig:867-881).
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..parts.base import ModelSpec, ParamDecl, Residual, make_part


class Model:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.hidden_size, self.vocab_size = spec.hidden_size, spec.vocab_size
        self.blocks = []
        for ls in spec.layers:
            mixer = make_part("mixer", ls.mixer)
            ff = make_part("feed_forward", ls.feed_forward)
            n1 = make_part("norm", ls.mixer_norm)
            n2 = make_part("norm", ls.ff_norm)
            self.blocks.append(make_part("block", ls.block, mixer, ff, n1, n2))
        self.final_norm = make_part("norm", spec.final_norm)
        for k, call in enumerate(spec.order):
            if not 0 <= call.layer < len(self.blocks):
                raise ValueError(f"order[{k}] names layer {call.layer}, but there are {len(self.blocks)} layers")
            if call.cache_of is not None:
                if not 0 <= call.cache_of < k or spec.order[call.cache_of].cache_of is not None:
                    raise ValueError(f"order[{k}].cache_of should name an earlier entry that owns its cache")
                a = self.blocks[spec.order[call.cache_of].layer].mixer.cache_need()
                b = self.blocks[call.layer].mixer.cache_need()
                if a != b:
                    raise ValueError(f"order[{k}] cannot read the cache of order[{call.cache_of}]: {b} != {a}")
        self.embed_name = spec.embedding.params["weight"]
        self.head_name = spec.head.params["weight"]
        self.tied = bool(spec.head.params["tied"])
        self.table = None
        self.head_w = None
        self.dtype = None

    # ------------------------------------------------------------------ tensors
    def _parts_of(self, block):
        return [block, block.mixer_norm, block.mixer, block.ff_norm, block.feed_forward]

    def param_decls(self) -> Dict[str, ParamDecl]:
        """Every tensor the model expects, by full name."""
        decls = {self.embed_name: ParamDecl((self.vocab_size, self.hidden_size), "table")}
        if not self.tied:
            decls[self.head_name] = ParamDecl((self.vocab_size, self.hidden_size), "matrix")
        for ls, block in zip(self.spec.layers, self.blocks):
            for part in self._parts_of(block):
                for local, decl in part.params().items():
                    decls[ls.prefix + local] = decl
        for local, decl in self.final_norm.params().items():
            decls[local] = decl
        return decls

    def bind(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype) -> None:
        """Hand each part its tensors (already on the device, in their kept dtypes)."""
        self.dtype = dtype
        self.table = tensors[self.embed_name]
        self.head_w = self.table if self.tied else tensors[self.head_name]
        for ls, block in zip(self.spec.layers, self.blocks):
            for part in self._parts_of(block):
                names = part.params()
                if names:
                    part.bind({local: tensors[ls.prefix + local] for local in names}, dtype)
        self.final_norm.bind({n: tensors[n] for n in self.final_norm.params()}, dtype)

    # ------------------------------------------------------------------ cache needs
    def cache_needs(self) -> List:
        """For every entry of the running order: the cache need of its mixer, or the index of the
        entry whose cache it reads."""
        out = []
        for call in self.spec.order:
            if call.cache_of is not None:
                out.append(("shared", call.cache_of))
            else:
                out.append(("own", self.blocks[call.layer].mixer.cache_need()))
        return out

    # ------------------------------------------------------------------ forward
    def forward(self, step, cache) -> torch.Tensor:
        """Run the step's tokens through the layers; return 32-bit logits [wanted, vocab]."""
        ops = step.ops
        begin = getattr(ops, "begin_forward", None)
        if begin:
            begin()
        try:
            return self._forward(step, cache, ops)
        finally:
            if begin:
                ops.end_forward()

    def _forward(self, step, cache, ops) -> torch.Tensor:
        step.scratch.clear()                # per-step tables are computed anew (also inside a graph capture)
        h = Residual(ops.embed(step.token_ids, self.table))
        pending = None
        for k, call in enumerate(self.spec.order):
            view = cache.view(k, step)
            h, pending = self.blocks[call.layer].forward(h, pending, step, view, call.cache_of is None)
        if step.n_wanted == 0:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=h.data.device)
        n = self.final_norm.forward(h, pending, step, lazy=True, rows=step.logit_rows)
        return ops.linear(n, self.head_w, out_dtype=torch.float32)
