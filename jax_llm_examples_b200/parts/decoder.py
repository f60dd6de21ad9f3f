"""A decoder put together from blocks, and the order in which they run.

The order is data: ``schedule`` is a list of :class:`LayerRun`.  A block may be named twice
(shared weights; each run has its own cache), and a run may read the cache that another run
fills (``writes=False``), in which case it stores no keys or values of its own.
"""

from __future__ import annotations

import dataclasses

import torch

from ..cache.manager import Retention
from ..kernels import api as K
from .base import Block, KVNeed, LayerCache, Norm, Runtime, StateNeed, StepContext, walk_parts
from .linear import linear


@dataclasses.dataclass(frozen=True)
class LayerRun:
    block: int  # index into the model's blocks
    cache: int | None = None  # index of the cache it reads (None: the mixer keeps no keys and values)
    writes: bool = True  # False: another run fills that cache
    state: "int | tuple[int, ...] | None" = None  # its per-request state slab(s) (None: stateless)

    @property
    def state_indices(self) -> tuple:
        return () if self.state is None else ((self.state,) if isinstance(self.state, int) else tuple(self.state))


@dataclasses.dataclass(frozen=True)
class CachePlan:
    caches: tuple[KVNeed, ...]  # one entry per cache index
    groups: tuple[Retention, ...]  # distinct retentions; each gets a page pool and a block table
    group_of: tuple[int, ...]  # cache index -> group index
    states: tuple[StateNeed, ...]  # one entry per state index


class DecoderModel:
    """Embedding, scheduled blocks, final norm, LM head (llama4/llama4_jax/model.py:1186-1204)."""

    def __init__(self, runtime: Runtime, embedding: torch.Tensor, blocks: list[Block], final_norm: Norm,
                 lm_head: torch.Tensor, schedule: list[LayerRun] | None = None, config=None, embedding_scale: float = 1.0,
                 residual_streams: int | None = None):
        self.runtime, self.embedding, self.blocks = runtime, embedding, blocks
        # None: one residual row per token.  A number S: every token carries S rows (x is [N, S * D]), all equal to
        # the embedding's output at the start; the blocks' and the final norms are the kind that keeps streams.
        self.residual_streams = residual_streams
        self.final_norm, self.lm_head, self.config = final_norm, lm_head, config
        self.embedding_scale = float(embedding_scale)  # the residual stream starts as scale * embedding row
        self.vocab_size, self.hidden_size = embedding.shape
        if schedule is None:
            schedule = self.schedule_of([(i,) for i in range(len(blocks))], blocks)
        self.schedule = list(schedule)
        self.plan = self._make_plan()
        # a block that wants the embedding's output later on (to feed it in again) gets a copy of it in
        # ``ctx.scratch["embedding_output"]``
        self.keeps_embedding_output = any(getattr(b, "wants_embedding_output", False) for b in blocks)

    @staticmethod
    def schedule_of(order, blocks: list[Block]) -> list[LayerRun]:
        """The schedule that runs ``blocks[i]`` for every ``(i, ...)`` of ``order`` in turn, every run with a cache
        and state slabs of its own (a block named twice shares its weights between runs, nothing else)."""
        schedule, c, s = [], 0, 0
        for i, *_ in order:
            mixer = blocks[i].mixer
            has_kv = mixer is not None and mixer.kv_need() is not None
            n_state = 0 if mixer is None else len(mixer.state_needs())
            state = None if n_state == 0 else (s if n_state == 1 else tuple(range(s, s + n_state)))
            schedule.append(LayerRun(i, c if has_kv else None, True, state))
            c += has_kv
            s += n_state
        return schedule

    def _make_plan(self) -> CachePlan:
        caches: dict[int, KVNeed] = {}
        writers: dict[int, int] = {}
        states: dict[int, StateNeed] = {}
        for pos, run in enumerate(self.schedule):
            mixer = self.blocks[run.block].mixer
            if mixer is None:
                if run.cache is not None or run.state is not None:
                    raise ValueError(f"schedule entry {pos}: a block without a mixer has no cache and no state")
                continue
            need = mixer.kv_need()
            if (need is None) != (run.cache is None):
                raise ValueError(f"schedule entry {pos}: the block's mixer {'needs' if need else 'has'} no cache index")
            if need is not None:
                if run.writes:
                    if run.cache in writers:
                        raise ValueError(f"schedule entry {pos}: cache {run.cache} already has a writer (entry {writers[run.cache]})")
                    writers[run.cache] = pos
                    caches[run.cache] = need
                else:
                    if run.cache not in writers:
                        raise ValueError(f"schedule entry {pos}: reads cache {run.cache} before any entry fills it")
                    w = caches[run.cache]
                    if (w.num_kv_heads, w.head_dim, w.planes) != (need.num_kv_heads, need.head_dim, need.planes):
                        raise ValueError(f"schedule entry {pos}: cache {run.cache} has other head sizes than this mixer")
                    if w.retention != need.retention:
                        # the reader must not need keys that the writer's group gives back: the writer keeps everything,
                        # or both look back over a window and the writer's is at least as long
                        wide = w.retention.kind == need.retention.kind == Retention.window(1).kind and w.retention.size >= need.retention.size
                        if w.retention != Retention.all() and not wide:
                            raise ValueError(f"schedule entry {pos}: reads a cache whose pages are released by another rule")
            needs = mixer.state_needs()
            if len(needs) != len(run.state_indices):
                raise ValueError(f"schedule entry {pos}: state index does not match the mixer's need")
            for idx, sn in zip(run.state_indices, needs):
                if idx in states:
                    raise ValueError(f"schedule entry {pos}: state {idx} is used twice")
                states[idx] = sn
        if sorted(caches) != list(range(len(caches))) or sorted(states) != list(range(len(states))):
            raise ValueError("cache and state indices must be 0..n-1 without gaps")
        groups: list[Retention] = []
        group_of = []
        for c in range(len(caches)):
            r = caches[c].retention
            if r not in groups:
                groups.append(r)
            group_of.append(groups.index(r))
        return CachePlan(tuple(caches[c] for c in range(len(caches))), tuple(groups), tuple(group_of),
                         tuple(states[s] for s in range(len(states))))

    def required_libraries(self) -> tuple[str, ...]:
        libs = ["elementwise", "gemm_simt"] + ([] if self.runtime.dtype == torch.float32 else ["gemm_stream"])
        for p in self.parts():
            libs.extend(p.required_libraries(self.runtime))
        return tuple(dict.fromkeys(libs))

    def parts(self):
        """Every part of the model, parts inside parts included."""
        for top in (*self.blocks, self.final_norm):
            yield from walk_parts(top)

    def step_planners(self) -> tuple:
        """The distinct host planners of all parts, in a fixed order (see Part.step_planners)."""
        return tuple(dict.fromkeys(f for p in self.parts() for f in p.step_planners()))

    @property
    def capturable(self) -> bool:
        """False if a part does host work per step that a captured CUDA graph would freeze."""
        return all(p.capturable for p in self.parts())

    def weight_bytes(self) -> int:
        seen, total = set(), 0

        def walk(o):
            nonlocal total
            if isinstance(o, torch.Tensor):
                store = o.untyped_storage()
                if store.data_ptr() not in seen:  # views (a shared expert inside the experts' tensor) count once
                    seen.add(store.data_ptr())
                    total += store.nbytes()
            elif hasattr(o, "__dict__"):
                for v in vars(o).values():
                    walk(v)
            elif isinstance(o, (list, tuple)):
                for v in o:
                    walk(v)

        walk([self.embedding, self.lm_head, self.final_norm, self.blocks])
        return total

    def forward(self, ctx: StepContext, kv: list[torch.Tensor], states: list[torch.Tensor],
                block_tables: list[torch.Tensor]) -> torch.Tensor:
        """Runs the step's tokens through the schedule; returns float32 logits [M, V] at ctx.logit_rows."""
        rt = self.runtime
        x = torch.empty((ctx.n_tokens, self.hidden_size), dtype=torch.float32, device=rt.device)
        K.embed(ctx.token_ids, self.embedding, x, ctx.status, self.embedding_scale)
        if self.keeps_embedding_output:
            ctx.scratch["embedding_output"] = x.clone()
        if self.residual_streams is not None:
            # the first norm writes the streams from the embedding's rows while it reads them
            ctx.scratch["streams_start"] = x
            x = torch.empty((ctx.n_tokens, self.residual_streams * self.hidden_size), dtype=torch.float32, device=rt.device)
        delta = None
        for run in self.schedule:
            slabs = tuple(states[i] for i in run.state_indices)
            first = slabs[0] if slabs else None
            if run.cache is None:
                cache = LayerCache(None, None, False, first, slabs)
            else:
                cache = LayerCache(kv[run.cache], block_tables[self.plan.group_of[run.cache]], run.writes, first, slabs)
            delta = self.blocks[run.block].forward(ctx, x, delta, cache)
        if ctx.n_logit_rows == 0:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=rt.device)
        h = self.final_norm.forward(ctx, x, delta, out_dtype=rt.dtype, row_index=ctx.logit_rows)[0]
        return linear(ctx, h, self.lm_head, torch.float32)
