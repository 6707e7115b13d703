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

from ..parts.base import ModelSpec, ParamDecl, Residual, make_block, make_part


class Model:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.hidden_size, self.vocab_size = spec.hidden_size, spec.vocab_size
        sizes = dict(vocab=spec.vocab_size, hidden=spec.hidden_size)
        self.embedding = make_part("embedding", spec.embedding, **sizes)
        self.blocks = [make_block(ls) for ls in spec.layers]
        self.final_norm = make_part("norm", spec.final_norm)
        self.head = make_part("head", spec.head, **sizes)
        for k, call in enumerate(spec.order):
            if not 0 <= call.layer < len(self.blocks):
                raise ValueError(f"order[{k}] names layer {call.layer}, but there are {len(self.blocks)} layers")
            if call.cache_of is not None:
                if not 0 <= call.cache_of < k or spec.order[call.cache_of].cache_of is not None:
                    raise ValueError(f"order[{k}].cache_of should name an earlier entry that owns its cache")
                a = self.blocks[spec.order[call.cache_of].layer].cache_needs()
                b = self.blocks[call.layer].cache_needs()
                if a != b:
                    raise ValueError(f"order[{k}] cannot read the cache of order[{call.cache_of}]: {b} != {a}")
        self.dtype = None

    # ------------------------------------------------------------------ tensors
    def _owners(self):
        """(prefix of the tensor names, part) for every part that may own tensors."""
        out = [("", self.embedding)]
        for ls, block in zip(self.spec.layers, self.blocks):
            out += [(ls.prefix, part) for part in [block] + list(block.parts().values())]
        return out + [("", self.final_norm), ("", self.head)]

    def all_parts(self) -> List:
        return [part for _, part in self._owners()]

    def param_decls(self) -> Dict[str, ParamDecl]:
        """Every tensor the model expects, by full name."""
        decls = {}
        for prefix, part in self._owners():
            for local, decl in part.params().items():
                decls[prefix + local] = decl
        return decls

    def bind(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype) -> None:
        """Hand each part its tensors (already on the device, in their kept dtypes)."""
        self.dtype = dtype
        for prefix, part in self._owners():
            names = part.params()
            if names or part in (self.embedding, self.head):
                part.bind({local: tensors[prefix + local] for local in names}, dtype)
        if getattr(self.head, "tied", False):
            self.head.tie(self.embedding)

    # ------------------------------------------------------------------ cache needs
    def cache_needs(self) -> List:
        """For every entry of the running order: ("own", the cache needs of its block's parts, a
        tuple), or ("shared", the index of the entry whose cache it reads)."""
        out = []
        for call in self.spec.order:
            if call.cache_of is not None:
                out.append(("shared", call.cache_of))
            else:
                out.append(("own", self.blocks[call.layer].cache_needs()))
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
        h = Residual(self.embedding.forward(step.token_ids, step))
        pending = None
        for k, call in enumerate(self.spec.order):
            h, pending = self.blocks[call.layer].forward(h, pending, step, cache.views(k, step), call.cache_of is None)
        if step.n_wanted == 0:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=h.data.device)
        n = self.final_norm.forward(h, pending, step, lazy=getattr(self.head, "accepts_lazy_input", False),
                                    rows=step.logit_rows)
        return self.head.forward(n, step)
