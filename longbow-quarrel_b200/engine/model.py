"""A model built from its description: embedding, blocks, the order they run in,
final norm, head.  It owns the parts and their weights; it owns no cache."""
from __future__ import annotations

import torch

from ..kernels import linear
from ..parts.base import Runtime, StepContext
from ..parts.registry import make_part
from ..parts.spec import ModelSpec, PartSpec
from ..weights.spec import WeightSpec


class Model:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        self.spec, self.runtime = spec, runtime
        self.embedding = make_part("embedding", spec.embedding, runtime)
        self.blocks = [make_part("block", PartSpec(layer.arrangement, dict(layer.params)), runtime, layer=layer)
                       for layer in spec.layers]
        self.final_norm = make_part("norm", spec.final_norm, runtime)
        self.head = make_part("head", spec.head, runtime)
        self._order_known = False
        # probe(run, x, ctx): called with the residual stream after the embedding (run -1) and after every
        # scheduled run of a layer, for looking into a step (trace replay's per-layer statistics).  Steps
        # with a probe are not replayed from CUDA graphs.
        self.probe = None
        for n, entry in enumerate(spec.schedule):
            if not 0 <= entry.layer < len(self.blocks):
                raise ValueError(f"schedule entry {n} names layer {entry.layer}; the model has {len(self.blocks)}")
        self._keeps_embedding = any(getattr(b, "reads_embedding", False) for b in self.blocks)
        writers = [e.cache for e in spec.schedule if e.writes_cache]
        if len(set(writers)) != len(writers):
            raise ValueError("schedule: two runs write the same cache entry")
        for e in spec.schedule:
            if not e.writes_cache and e.cache not in writers:
                raise ValueError(f"schedule: a run reads cache entry {e.cache}, which no run writes")
        # State that parts keep for each sequence beside the mixers' cache entries (`state_need`: the embedding's, and
        # every run of a block's own) gets cache entries of its own, numbered after the schedule's.
        free = max([e.cache for e in spec.schedule], default=-1) + 1
        self._state_entries: dict = {}
        need = getattr(self.embedding, "state_need", lambda: None)()
        if need is not None:
            self._state_entries["embedding"] = (free, need)
            free += 1
        for n, entry in enumerate(spec.schedule):
            need = getattr(self.blocks[entry.layer], "state_need", lambda: None)()
            if need is not None:
                self._state_entries[n] = (free, need)
                free += 1

    # ------------------------------------------------------------------ weights
    def _named_parts(self):
        yield "", self.embedding
        for block in self.blocks:
            yield block.prefix, block
        yield "", self.final_norm
        yield "", self.head

    def weight_table(self) -> dict[str, WeightSpec]:
        """Every tensor the model reads, by its full name."""
        table: dict[str, WeightSpec] = {}
        for prefix, part in self._named_parts():
            for name, spec in part.weights().items():
                full = prefix + name
                if full in table:
                    raise ValueError(f"two parts name the tensor {full!r}")
                table[full] = spec
        return table

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        for prefix, part in self._named_parts():
            mine = {}
            for name, spec in part.weights().items():
                if prefix + name in tensors:
                    mine[name] = tensors[prefix + name]
                elif spec.fallback is None:
                    raise KeyError(prefix + name)
            for full in part.borrows():              # tensors of other parts that this one reads as well
                if full in tensors:
                    mine[full] = tensors[full]
            part.load(mine)

    @property
    def graph_safe(self) -> bool:
        """Every part allows its steps to be captured in a CUDA graph."""
        return all(part.graph_safe for _, part in self._named_parts())

    def cache_needs(self) -> dict:
        """Cache entry -> what the mixer that writes it needs."""
        needs = {e.cache: self.blocks[e.layer].cache_need() for e in self.spec.schedule if e.writes_cache}
        needs.update({entry: need for entry, need in self._state_entries.values()})
        return needs

    def step_needs(self) -> dict:
        """Name -> builder of every per-step integer array that some part asks for (see Part.step_needs)."""
        out = {}
        for _, part in self._named_parts():
            out.update(part.step_needs())
        return out

    def kernel_libraries(self) -> tuple:
        """Kernel libraries that parts of this model name beyond the ones every model uses (built before the first step)."""
        found = set()
        for _, part in self._named_parts():
            for p in (part, *(part.parts() if hasattr(part, "parts") else ())):
                found.update(getattr(p, "kernel_libraries", ()))
        return tuple(sorted(found))

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for _, part in self._named_parts():
            for t in _tensors_of(part):
                if t.data_ptr() not in seen:
                    seen.add(t.data_ptr())
                    total += t.numel() * t.element_size()
        return total

    # ------------------------------------------------------------------ forward
    def forward(self, ctx: StepContext, cache) -> torch.Tensor | None:
        """Run this step's rows through every scheduled layer; logits [wanted, vocab]
        (float32) at ctx.want_rows, or None when nothing is wanted."""
        if not self._order_known:
            # The first step also notes in which order the weights are read (it is the same in every step).
            self._order_known = True
            with linear.recording():
                return self.forward(ctx, cache)
        states = self._state_entries
        if "embedding" in states:
            x = self.embedding.forward(ctx.tokens, ctx=ctx, state=cache.view(states["embedding"][0]))
        else:
            x = self.embedding.forward(ctx.tokens)
        schedule = self.spec.schedule
        probe = self.probe
        if probe is not None:
            probe(-1, x, ctx)
        # A block that reads the embedding's rows again later (`reads_embedding`) gets a copy: the stream changes in place.
        embedded = x.clone() if self._keeps_embedding else None
        normed = None           # rows of the next layer's first norm, when this layer's last product made them
        for i, entry in enumerate(schedule):
            block = self.blocks[entry.layer]
            if getattr(block, "replaces_stream", False):
                # A block that makes a new stream out of the old one (and the embedding's rows); it is no layer, and
                # the probe is not called for it.
                x = block.forward(x, ctx, embedded=embedded)
                normed = None
                continue
            if i in states:
                # A block with state of its own (it folds no norms: what the layer ahead left unfinished is finished first).
                block.forward(x, ctx, cache.view(entry.cache), entry.writes_cache, state=cache.view(states[i][0]))
                normed = None
                if probe is not None:
                    probe(i, x, ctx)
                continue
            if not getattr(block, "folds_norm", False):
                block.forward(x, ctx, cache.view(entry.cache), entry.writes_cache)
                normed = None
                if probe is not None:
                    probe(i, x, ctx)
                continue
            after = self.blocks[schedule[i + 1].layer] if i + 1 < len(schedule) else None
            emit = after.input_norm(x.shape[0]) if getattr(after, "folds_norm", False) else None
            normed = block.forward(x, ctx, cache.view(entry.cache), entry.writes_cache, normed=normed, emit=emit)
            if probe is not None:
                probe(i, x, ctx)
        if ctx.want_rows is None or ctx.want_rows.numel() == 0:
            return None
        h = self.final_norm.forward(x, rows=ctx.want_rows)
        return self.head.forward(h)


def _tensors_of(obj, depth: int = 0):
    if depth > 3:
        return
    for value in vars(obj).values():
        if isinstance(value, torch.Tensor):
            yield value
        elif hasattr(value, "tensor") and isinstance(getattr(value, "tensor"), torch.Tensor):
            yield value.tensor
        elif hasattr(value, "__dict__") and not isinstance(value, (Runtime, type)) and hasattr(value, "weights"):
            yield from _tensors_of(value, depth + 1)
