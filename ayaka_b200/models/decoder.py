"""The one model class: a decoder assembled from a :class:`ModelSpec`.

It owns the embedding, the position encoding, one block per layer, the final norm and the
head, and runs the layers in the order the spec lists. It knows nothing of GPT-2: another
architecture is another spec.
"""

from __future__ import annotations

import torch

from ayaka_b200.kernels import native, ops
from ayaka_b200.parts.base import BuildContext, CacheNeed, Part, StateNeed, build_part
from ayaka_b200.parts.context import LayerCache, StepContext
from ayaka_b200.parts.spec import ModelSpec

__all__ = ["DecoderModel"]


class DecoderModel(Part):
    """Embedding -> runs of blocks -> final norm on the wanted rows -> head (fp32 logits).

    Parameter names: ``embedding.weight``, ``position.*``, ``layers.<i>.<part>.*``,
    ``final_norm.*`` and, when the head is not tied, ``head.weight``.
    """

    def __init__(self, spec: ModelSpec, ctx: BuildContext) -> None:
        super().__init__(ctx)
        self.spec = spec
        self.embedding = self.add_child(
            "embedding", build_part("embedding", spec.embedding.kind, spec.embedding, ctx))
        self.position = self.add_child(
            "position", build_part("position", spec.position.kind, spec.position, ctx))
        layers = Part(ctx)
        self.add_child("layers", layers)
        self.blocks: list[Part] = []
        for index, layer in enumerate(spec.layers):
            block = build_part("block", layer.block, layer, ctx, self.position)
            layers.add_child(str(index), block)
            self.blocks.append(block)
        self.final_norm = self.add_child(
            "final_norm", build_part("norm", spec.final_norm.kind, spec.final_norm, ctx))
        self.head = self.add_child(
            "head", build_part("head", spec.head.kind, spec.head, ctx, self.embedding))
        for position, run in enumerate(spec.order):
            if not 0 <= run.layer < len(self.blocks):
                raise ValueError(f"order[{position}] names layer {run.layer}, which does not "
                                 "exist")
            if run.reads_cache_of is not None and not 0 <= run.reads_cache_of < position:
                raise ValueError(f"order[{position}] must read the cache of an earlier run")
        self._runs: dict[tuple[int, int], object] = {}
        self._keep: list[object] = []

    def needs(self) -> list[tuple[CacheNeed | None, StateNeed | None]]:
        """For each run of the order: the pages and the state its mixer asks for."""
        out = []
        for run in self.spec.order:
            mixer = self.blocks[run.layer].mixer  # type: ignore[attr-defined]
            out.append((mixer.cache_need(), mixer.state_need()))
        return out

    def _native_runs(self, step: StepContext, caches: list[LayerCache]):  # noqa: ANN202
        """The execution order packed for the C++ host code (once per list of caches and
        workspace), or ``None`` when some layer has a part that code does not know."""
        key = (id(caches), id(step.workspace))
        if key not in self._runs:
            entries = []
            for index, run in enumerate(self.spec.order):
                block = self.blocks[run.layer]
                cache = caches[index]
                halves = block.native_run(step.workspace) \
                    if hasattr(block, "native_run") and cache.k_pages is not None else None
                if halves is None:
                    entries = None
                    break
                entries.append((*halves, cache))
            self._runs[key] = None if entries is None else native.LayerRuns(entries)
            self._keep.append(caches)  # the key is an id: keep its object alive
        return self._runs[key]

    def forward(self, step: StepContext, caches: list[LayerCache],
                want_rows: torch.Tensor | None, num_want: int) -> torch.Tensor | None:
        """Run the step's rows; return fp32 logits ``[num_want, vocab]`` (a view of a
        persistent buffer) at the rows listed in ``want_rows``, or ``None`` if none is wanted."""
        spec = self.spec
        residual = step.workspace.buffer("model.residual", spec.hidden_size, torch.float32)
        self.embedding.forward(  # type: ignore[attr-defined]
            step, residual, self.position.added_rows(step))  # type: ignore[attr-defined]
        runs = self._native_runs(step, caches) if ops.NATIVE_STEP else None
        if runs is not None:
            # every layer can run from the C++ host code: one call walks the whole order
            native.run_layers(runs, native.step_args(step, residual.device), residual)
        else:
            for index, run in enumerate(spec.order):
                self.blocks[run.layer].forward(residual, step, caches[index])  # type: ignore
        if num_want == 0 or want_rows is None:
            return None
        chosen = step.workspace.buffer("model.head_in", spec.hidden_size, self.ctx.dtype,
                                       rows=num_want)
        logits = step.workspace.buffer("model.logits", spec.vocab_size, torch.float32,
                                       rows=num_want)
        if hasattr(self.head, "forward_normed") and \
                getattr(self.final_norm, "fusable_layer_norm", False):
            self.head.forward_normed(self.final_norm, residual, want_rows,  # type: ignore
                                     chosen, logits, count=num_want)
        else:
            self.final_norm.forward(residual, chosen, count=num_want,  # type: ignore
                                    rows=want_rows)
            self.head.forward(chosen, logits, count=num_want)  # type: ignore[attr-defined]
        return logits[:num_want]
