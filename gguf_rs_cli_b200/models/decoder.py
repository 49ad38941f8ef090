"""The generic decoder: builds parts from a ModelSpec and runs them in the spec's
order.  It is the only model class; architectures differ in the spec they build.

forward: embedding -> for each run of the schedule, that layer's block on the
residual stream -> final norm on the wanted rows only -> head.  The reference runs
the head for every token and throws all but the last logits away
(src/main.rs:248-254); here only the rows that are asked for reach the final norm
and the head.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..cache.cache import Cache, CacheLayout
from ..config.specs import LayerSpec, ModelSpec, PartSpec
from ..parts.base import HostBatch, RunView, StepContext, Stream, plan_key_of
from ..parts.registry import BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS
from ..weights.loader import TensorRequest, WeightStore


class Layer:
    def __init__(self, spec: LayerSpec, dtype, device, positions: Dict[str, object]):
        position = None
        if spec.position is not None:
            key = spec.position.key()
            if key not in positions:          # layers with equal constants share one table
                positions[key] = POSITIONS.get(spec.position.kind)(spec.position, dtype, device)
            position = positions[key]
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, dtype, device, position=position)
        self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, dtype, device)
        self.norms = {name: NORMS.get(s.kind)(s, dtype, device) for name, s in spec.norms.items()}
        self.block = BLOCKS.get(spec.block)(self.mixer, self.feed_forward, self.norms)

    def parts(self):
        return [self.mixer, self.feed_forward] + list(self.norms.values())


def _requests_of(spec: ModelSpec, parts) -> List[TensorRequest]:
    seen, out = set(), []
    for p in parts:
        for r in p.tensor_requests():
            if (r.name, r.fallback) not in seen:
                seen.add((r.name, r.fallback))
                out.append(r)
    return out


class Decoder:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device):
        spec.validate()
        self.spec, self.dtype, self.device = spec, dtype, device
        self.positions: Dict[str, object] = {}
        self.embedding = EMBEDDINGS.get(spec.embedding.kind)(spec.embedding, dtype, device)
        self.layers = [Layer(ls, dtype, device, self.positions) for ls in spec.layers]
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm, dtype, device)
        self.head = HEADS.get(spec.head.kind)(spec.head, dtype, device)
        for r, run in enumerate(spec.schedule):
            mixer = self.layers[run.layer].mixer
            owns = mixer.kv_spec() is not None
            if run.cache_of is not None and owns:
                raise ValueError(f"schedule[{r}] reads the cache of run {run.cache_of}, but its mixer keeps keys and "
                                 f"values of its own (build it with shares_kv)")
            if run.cache_of is None and not owns and getattr(mixer, "shares_kv", False):
                raise ValueError(f"schedule[{r}]: the mixer of layer {run.layer} has no keys and values of its own; "
                                 f"the entry must name the run whose cache it reads (cache_of)")
            if run.cache_of is not None:
                src = self.layers[spec.schedule[run.cache_of].layer].mixer.kv_spec()
                if src is None or src != mixer.reads_kv_spec():
                    raise ValueError(f"schedule[{r}] cannot read the cache of run {run.cache_of}: {src} does not match "
                                     f"{mixer.reads_kv_spec()}")

        # parts that lay out index arrays on the host, one per plan key, and what decides whether and how a
        # decode step is captured: every computing part's graph_class (constant, callable, or missing)
        self.planners = []
        self._graph_constants, self._graph_callables, self.capturable = [], [], True
        seen_plans, seen_classes = set(), set()
        computing = [self.embedding, self.final_norm, self.head]
        for r in spec.schedule:
            l = self.layers[r.layer]
            computing += [l.block, l.mixer, l.feed_forward] + list(l.norms.values())
        for part in computing:
            key = plan_key_of(part)
            if hasattr(part, "plan") and key not in seen_plans:
                seen_plans.add(key)
                self.planners.append((key, part))
            if key in seen_classes:
                continue
            seen_classes.add(key)
            gc = getattr(part, "graph_class", None)
            if gc is None:
                self.capturable = False
            elif callable(gc):
                self._graph_callables.append(gc)
            else:
                self._graph_constants.append(gc)

    def graph_class(self, batch: HostBatch):
        """Hashable class of a decode step for capture in a CUDA graph, or None when a part of the model
        cannot be captured."""
        if not self.capturable:
            return None
        classes = []
        for fn in self._graph_callables:
            c = fn(batch)
            if c is None:
                return None
            classes.append(c)
        return tuple(classes)

    # ---------------------------------------------------------------- weights
    def parts(self):
        out = [self.embedding]
        for l in self.layers:
            out += l.parts()
        return out + [self.final_norm, self.head]

    def tensor_requests(self) -> List[TensorRequest]:
        return _requests_of(self.spec, self.parts())

    def load(self, store: WeightStore) -> "Decoder":
        store.check(self.tensor_requests(), allow_unused=self.spec.ignored_tensors)
        for p in self.parts():
            p.load(store)
        store.release()
        for layer in self.layers:
            fuse = getattr(layer.block, "fuse", None)
            if fuse:
                fuse()
        return self

    # ------------------------------------------------------------------ cache
    def cache_layout(self) -> CacheLayout:
        """Keys and values for every run whose mixer keeps them, and the fixed-size state
        every run's mixer declares (named run<r>.<name>)."""
        layout = CacheLayout()
        for r, run in enumerate(self.spec.schedule):
            mixer = self.layers[run.layer].mixer
            kv = mixer.kv_spec()
            if kv is not None and run.cache_of is None:
                layout.kv[r] = kv
            for name, sd in mixer.state_spec().items():
                layout.states[f"run{r}.{name}"] = sd
        return layout

    def run_views(self, cache: Cache) -> List[RunView]:
        views = []
        for r, run in enumerate(self.spec.schedule):
            src = r if run.cache_of is None else run.cache_of
            if src in cache.group_of_run:
                gi, i = cache.group_of_run[src]
                g = cache.groups[gi]
                views.append(RunView(r, run.layer, run.cache_of is None, gi, g.k[i], g.v[i], g.ring_pages, g.spec))
            else:
                views.append(RunView(r, run.layer, False))
        return views

    # ---------------------------------------------------------------- forward
    def forward(self, ctx: StepContext, runs: List[RunView], want_rows: torch.Tensor) -> torch.Tensor:
        """Logits float32 [len(want_rows), V] at the packed token rows asked for."""
        make = getattr(self.embedding, "forward_stream", None)
        stream = make(ctx.tokens, ctx) if make else Stream(self.embedding.forward(ctx.tokens, ctx))
        ctx.mark("embed")
        for view in runs:
            ctx.mark_detail = view.index == 0         # stages are stamped in the first run only, as the reference does
            self.layers[view.layer].block.forward(stream, ctx, view)
        ctx.mark_detail = True
        ctx.mark("layers")
        h = self.final_norm.apply(stream, ctx, rows=want_rows, buffer="final_normed")
        logits = self.head.forward(h, ctx)
        ctx.mark("head")
        return logits


def tensor_requests(spec: ModelSpec) -> List[TensorRequest]:
    """The tensors a model of this spec asks for, without building anything on a device."""
    return Decoder(spec, torch.float32, "meta").tensor_requests()
