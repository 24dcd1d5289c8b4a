"""A model built from a `ModelSpec`: instantiated parts, the checkpoint tensors
they expect, and the forward pass of one step over the residual stream."""
from __future__ import annotations

import inspect
from dataclasses import dataclass
from typing import Dict, List, Tuple

import torch

from ..parts.base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, Part, PartSpec, WeightDecl)
from .spec import ModelSpec, ScheduleEntry


@dataclass
class BuiltLayer:
    block: Part
    mixer: Part
    ffn: Part
    mixer_norm: Part
    ffn_norm: Part


class Model:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.embedding = EMBEDDINGS.build(spec.embedding)
        self.final_norm = NORMS.build(spec.final_norm)
        self.head = HEADS.build(spec.head)
        self.layers: List[BuiltLayer] = []
        self._bound: List[Tuple[Part, PartSpec]] = [(self.embedding, spec.embedding),
                                                    (self.final_norm, spec.final_norm), (self.head, spec.head)]
        for ls in spec.layers:
            bl = BuiltLayer(BLOCKS.build(ls.block), MIXERS.build(ls.mixer), FEED_FORWARDS.build(ls.ffn),
                            NORMS.build(ls.mixer_norm), NORMS.build(ls.ffn_norm))
            self.layers.append(bl)
            self._bound += [(bl.block, ls.block), (bl.mixer, ls.mixer), (bl.ffn, ls.ffn),
                            (bl.mixer_norm, ls.mixer_norm), (bl.ffn_norm, ls.ffn_norm)]
        self.schedule: List[ScheduleEntry] = spec.resolved_schedule()
        # blocks written before `next_norm` existed (or that have no use for it) are called without it
        self._takes_next_norm = ["next_norm" in inspect.signature(bl.block.forward).parameters for bl in self.layers]
        self.act_dtype: torch.dtype | None = None
        # a position encoding is built inside its mixer; it counts too
        self.replayable = all(getattr(part, "replayable", True) and
                              getattr(getattr(part, "pos", None), "replayable", True) for part, _ in self._bound)

    # ---- weights -----------------------------------------------------------
    def expected_tensors(self) -> Dict[str, WeightDecl]:
        """Checkpoint tensor name -> declaration, over all parts.  A tensor that two
        parts share (a tied head) must be declared alike by both."""
        out: Dict[str, WeightDecl] = {}
        for part, ps in self._bound:
            for local, decl in part.weight_decls().items():
                if local not in ps.tensors:
                    raise KeyError(f"{ps.kind}: no checkpoint tensor name given for weight {local!r}")
                name = ps.tensors[local]
                if name in out and (out[name].shape != decl.shape or out[name].role != decl.role):
                    raise ValueError(f"tensor {name!r} is shared by parts that expect different shapes: "
                                     f"{out[name].shape} and {decl.shape}")
                out.setdefault(name, decl)
        return out

    def bind_weights(self, tensors: Dict[str, torch.Tensor], act_dtype: torch.dtype) -> None:
        self.act_dtype = act_dtype
        for part, ps in self._bound:
            local = {l: tensors[ps.tensors[l]] for l in part.weight_decls()}
            part.bind(local, act_dtype)

    def reserve(self, device, max_rows: int, max_context: int) -> None:
        """Lets every part size its scratch memory, and the products theirs for the widest matrix."""
        for part, _ in self._bound:
            part.reserve(device, max_rows, max_context)
        if self.act_dtype == torch.bfloat16:
            from ..kernels import ops
            mats = [d.shape for d in self.expected_tensors().values() if d.role == "matrix" and len(d.shape) == 2]
            if mats:
                # stacked matrices (q|k|v, gate|up, B|C|x) are up to three times as tall as a declared one
                ops.reserve_product_workspace(device, 3 * max(m[0] for m in mats), max(m[1] for m in mats))

    # ---- cache -------------------------------------------------------------
    def storage_needs(self) -> List[object]:
        """What each cache storage must hold, indexed by storage number (None: nothing)."""
        n = max((e.storage for e in self.schedule), default=-1) + 1
        needs: List[object] = [None] * n
        owner_seen = [False] * n
        for e in self.schedule:
            need = self.layers[e.layer].mixer.cache_need()
            if e.reads_only:
                continue
            if owner_seen[e.storage]:
                raise ValueError(f"cache storage {e.storage} is written by more than one schedule entry")
            owner_seen[e.storage] = True
            needs[e.storage] = need
        for e in self.schedule:
            if e.reads_only:
                if not owner_seen[e.storage]:
                    raise ValueError(f"schedule entry for layer {e.layer} reads storage {e.storage}, which no entry writes")
                if self.layers[e.layer].mixer.cache_need() != needs[e.storage]:
                    raise ValueError(f"layer {e.layer} reads storage {e.storage} but needs a different cache shape")
        return needs

    # ---- one step ----------------------------------------------------------
    def forward(self, ctx, storages) -> torch.Tensor:
        """Runs the tokens of `ctx` through the schedule; returns fp32 logits [n_wanted, vocab]."""
        x = self.embedding.forward(ctx)
        for i, e in enumerate(self.schedule):
            layer = self.layers[e.layer]
            if self._takes_next_norm[e.layer]:
                # the norm that reads the residual after this layer: the next entry's first norm, or the final one
                nxt = self.layers[self.schedule[i + 1].layer].mixer_norm if i + 1 < len(self.schedule) else (
                    self.final_norm if ctx.wants_all_rows else None)
                layer.block.forward(ctx, x, layer, storages[e.storage], e.reads_only, next_norm=nxt)
            else:
                layer.block.forward(ctx, x, layer, storages[e.storage], e.reads_only)
        return self.head.forward(ctx, x, self.final_norm)
