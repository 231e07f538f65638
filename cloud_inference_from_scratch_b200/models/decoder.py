"""A decoder put together from a ``ModelSpec``: embedding (times a constant), scheduled layers,
final norm, head, logits (times a constant, softly capped).

This is the only model class of the framework; an architecture contributes a
description, not a class.  The forward pass is the reference's
``Qwen2CausalLM.forward`` (src/cloud_engine/model.py:194-228) restated over parts:
gather embeddings into the float32 residual stream, run the schedule, normalise only
the rows whose logits are wanted (the reference normalises all rows and then selects,
model.py:221-225), multiply by the head and return float32 logits.

Beyond the reference: a description may ask for a learned vector per position that is added to the
embedding rows (``position_tensor``), for a sinusoid of the position instead (``position_wave_base``),
for several copies of the residual stream side by side (``residual_streams``, [T, streams * H]; the
blocks of such a model read and write the copies and the final norm reads their sum), for a stored
vector that is added to the stream right before a run of a layer (``ScheduleEntry.entry_offset``), for the
embedding rows to be added once more there (``ScheduleEntry.adds_embedding``), and for a constant on every
sublayer's result (``residual_scale``).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from ..config.spec import ModelSpec
from ..parts.base import (
    Block,
    CacheSpec,
    Norm,
    Part,
    StateSpec,
    TensorSpec,
    build_part,
    part_class,
)


@dataclass
class LayerParts:
    """The built parts of one layer by slot name, their arrangement, and the tensor-name prefix of
    each part in the weight files."""

    prefix: str
    parts: dict[str, Part]
    families: dict[str, str]
    block: Block
    prefixes: dict[str, str]

    def named_parts(self):
        for slot, part in self.parts.items():
            yield self.prefixes[slot], part

    @property
    def cache_part(self) -> Part | None:
        """The part whose cache the layer's binding belongs to (at most one part of a layer keeps one)."""
        return self.parts.get(self.block.cache_slot)

    def __getattr__(self, name: str) -> Part:      # layer.mixer, layer.feed_forward, ...
        try:
            return self.__dict__["parts"][name]
        except KeyError:
            raise AttributeError(name) from None


@dataclass(frozen=True)
class CacheNeed:
    """What one schedule entry needs of the cache manager (``owner`` is the entry whose
    cache it uses: itself, or the earlier entry it reads)."""

    entry: int
    owner: int
    pages: CacheSpec | None
    state: StateSpec | None


class DecoderModel:
    def __init__(self, spec: ModelSpec) -> None:
        spec.validate()
        self.spec = spec
        self.layers: list[LayerParts] = []
        for layer in spec.layers:
            parts = {slot: build_part(part.family, part) for slot, part in layer.parts.items()}
            block = part_class("block", layer.block.kind)(parts, **layer.block.params)
            keepers = [slot for slot, part in parts.items()
                       if getattr(part, "cache_spec", None) and (part.cache_spec() or part.state_spec())]
            if any(slot != block.cache_slot for slot in keepers):
                raise ValueError(
                    f"layer {layer.prefix!r}: the parts {keepers} keep a cache, but the block binds only "
                    f"{block.cache_slot!r} to one"
                )
            self.layers.append(
                LayerParts(
                    prefix=layer.prefix, parts=parts, block=block,
                    families={slot: part.family for slot, part in layer.parts.items()},
                    prefixes={slot: layer.prefix + part.prefix for slot, part in layer.parts.items()},
                )
            )
        self.final_norm: Norm = build_part("norm", spec.final_norm)
        # a projection may add itself into the residual stream only if whoever normalises next
        # understands that the sum is already there
        norms = [self.final_norm] + [part for layer in self.layers for slot, part in layer.parts.items()
                                     if layer.families[slot] == "norm"]
        self.norms_accept_accumulated = all(getattr(norm, "accepts_accumulated", False) for norm in norms)
        # A decode step may be recorded and run as one persistent kernel only if every kernel of every
        # part is a method of ``Ops`` (which then keeps the order of recorded and launched work); a part
        # says so itself, and a part that launches anything of its own (torch ops included) does not.
        self.records_programs = all(
            getattr(part, "kernels_through_ops", False)
            for layer in self.layers for part in [layer.block, *layer.parts.values()])
        # a callable (schedule entry, residual, pending update) run after every layer, for whoever wants to look
        # at the stream (tests); the stream after the layer is ``residual`` plus what is still pending
        self.after_layer: Any = None
        self.embedding: Any = None
        self.position_table: Any = None
        self.head: Any = None
        self.runtime: Any = None

    # ------------------------------------------------------------------ tensors
    def tensor_table(self) -> dict[str, TensorSpec]:
        """Every tensor the model reads, by its name in the weight files."""
        spec = self.spec
        table: dict[str, TensorSpec] = {
            spec.embedding_tensor: TensorSpec((spec.vocab_size, spec.hidden_size))
        }
        if spec.head_tensor != spec.embedding_tensor:
            table[spec.head_tensor] = TensorSpec((spec.vocab_size, spec.hidden_size))
        if spec.position_tensor:
            table[spec.position_tensor] = TensorSpec((spec.max_positions, spec.hidden_size))
        for name, rows in spec.offset_tensors:
            table[name] = TensorSpec((rows, spec.hidden_size), role="vector")
        for layer in self.layers:
            for prefix, part in layer.named_parts():
                for name, tensor in part.tensor_specs().items():
                    table[prefix + name] = tensor
        for name, tensor in self.final_norm.tensor_specs().items():
            table[spec.final_norm_prefix + name] = tensor
        return table

    def cache_needs(self) -> list[CacheNeed]:
        needs: list[CacheNeed] = []
        for index, entry in enumerate(self.spec.schedule):
            keeper = self.layers[entry.layer].cache_part
            owner = index if entry.reads_cache_of is None else entry.reads_cache_of
            pages = keeper.cache_spec() if keeper is not None and hasattr(keeper, "cache_spec") else None
            state = keeper.state_spec() if keeper is not None and hasattr(keeper, "state_spec") else None
            needs.append(CacheNeed(index, owner, pages, state))
        for need in needs:
            if need.owner != need.entry:
                owner = needs[need.owner]
                if (owner.pages, owner.state) != (need.pages, need.state):
                    raise ValueError(
                        f"schedule entry {need.entry} reads the cache of entry {need.owner}, "
                        "whose mixer keeps a different kind of cache"
                    )
        return needs

    # ------------------------------------------------------------------ binding
    def bind(self, tensors: Any, runtime: Any) -> None:
        """``tensors(name)`` returns the tensor on the device in the dtype its role asks for."""
        self.runtime = runtime
        spec = self.spec
        self.embedding = runtime.ops.prepare_weight(tensors(spec.embedding_tensor))
        self.position_table = (runtime.ops.prepare_weight(tensors(spec.position_tensor))
                               if spec.position_tensor else None)
        self.head = (
            self.embedding
            if spec.head_tensor == spec.embedding_tensor
            else runtime.ops.prepare_weight(tensors(spec.head_tensor))
        )
        self.offsets = {name: tensors(name).contiguous() for name, _ in spec.offset_tensors}
        self.wave = None
        if spec.position_wave_base is not None:
            import torch

            # frequencies in double precision, rounded once; the kernel multiplies by the position in float32
            pairs = torch.arange((spec.hidden_size + 1) // 2, dtype=torch.float64)
            wave = torch.pow(torch.tensor(float(spec.position_wave_base), dtype=torch.float64),
                             -2.0 * pairs / spec.hidden_size)
            self.wave = wave.to(device=runtime.device, dtype=torch.float32).contiguous()
        for layer in self.layers:
            for prefix, part in layer.named_parts():
                part.bind({name: tensors(prefix + name) for name in part.tensor_specs()}, runtime)
        self.final_norm.bind(
            {name: tensors(spec.final_norm_prefix + name) for name in self.final_norm.tensor_specs()},
            runtime,
        )

    # ------------------------------------------------------------------ forward
    def forward(self, ctx: Any) -> Any:
        """Runs the tokens of ``ctx`` and returns float32 logits [wanted rows, vocab]."""
        import torch

        rt = self.runtime
        spec = self.spec
        streams = spec.residual_streams
        residual = rt.workspace.get("residual", ctx.num_tokens, spec.hidden_size * streams, torch.float32)
        if self.wave is not None:
            rt.ops.embedding(ctx.token_ids, self.embedding, residual, spec.embedding_scale,
                             positions=ctx.positions, wave=self.wave)
        elif streams > 1 or self.position_table is not None:
            # the stream copies lie side by side in a token's row; a learned position vector is added
            rt.ops.embedding(ctx.token_ids, self.embedding, residual, spec.embedding_scale,
                             positions=ctx.positions, position_table=self.position_table, streams=streams)
        else:
            rt.ops.embedding(ctx.token_ids, self.embedding, residual, spec.embedding_scale)
        embedded = None
        if any(entry.adds_embedding for entry in spec.schedule):
            # the stream as it is before the first layer, kept for the runs that add it again
            if self.wave is not None or streams > 1 or self.position_table is not None:
                raise ValueError("adding the embedding rows again is built for a plain embedding")
            embedded = rt.workspace.get("embedded", ctx.num_tokens, spec.hidden_size, torch.float32)
            rt.ops.embedding(ctx.token_ids, self.embedding, embedded, spec.embedding_scale)
        sink = rt.ops.residual_sink(residual) if self.norms_accept_accumulated and streams == 1 else None
        ctx.residual_sink = sink
        pending = None
        recorded = self.records_programs and sink is not None and rt.ops.begin_program(ctx)
        for index, entry in enumerate(spec.schedule):
            if sink is not None:
                # what the block after this layer wants to know of its first norm (the final norm
                # takes plain rows)
                sink.following_gain = None
                if index + 1 < len(spec.schedule):
                    sink.following_gain = self.layers[spec.schedule[index + 1].layer].block.entry_gain()
            if entry.entry_offset is not None or entry.adds_embedding:
                vector = None
                if entry.entry_offset is not None:
                    name, row = entry.entry_offset
                    vector = self.offsets[name][row]
                rt.ops.add_rows(residual, pending, vector, base=embedded if entry.adds_embedding else None,
                                scale=spec.residual_scale)
                pending = None
            pending = self.layers[entry.layer].block.forward(
                residual, pending, ctx, ctx.bindings[index]
            )
            if self.after_layer is not None:
                self.after_layer(index, residual, pending)
        if recorded:
            rt.ops.end_program()
        if ctx.num_logit_rows == 0:
            return None
        x = self.final_norm.forward(residual, pending, ctx, rows=ctx.logit_rows)
        logits = rt.workspace.get("logits", ctx.num_logit_rows, spec.vocab_size, torch.float32,
                                  per_request=True)
        rt.ops.linear(x, self.head, None, logits)
        rt.ops.shape_logits(logits, spec.logit_scale, spec.logit_softcap)
        return logits
