"""The declarative description of a model: parts and parameters layer by layer, and the run order.

``ModelSpec.layers`` are the layers that own weights; ``ModelSpec.schedule`` is the order in which
they run, as data.  An entry may name a layer that already ran (its weights are reused, with a cache
and state of its own), and may read the cache that an earlier entry wrote instead of writing one.
"""

from __future__ import annotations

from dataclasses import dataclass, field


@dataclass(frozen=True)
class ScheduleEntry:
    layer: int                         # index into ModelSpec.layers
    read_cache_of: int | None = None   # schedule position whose cache this entry reads (it writes none)


@dataclass
class ModelSpec:
    name: str
    vocab_size: int
    hidden_size: int
    embedding_name: str
    layers: list[tuple[str, dict]]             # ("block part name", params) per layer
    final_norm: tuple[str, dict]
    head_name: str | None                      # None with tied_head: the embedding table is the head
    tied_head: bool = False
    schedule: list[ScheduleEntry] = field(default_factory=list)
    ignored_prefixes: tuple[str, ...] = ()     # checkpoint tensors that are not this model's and are skipped
    name_aliases: tuple[tuple[str, str], ...] = ()   # (prefix in file, prefix in spec) rewrites
    # ("embedding part name", params) and ("head part name", params); None: the token table and the
    # normed linear head described by the fields above
    embedding: tuple[str, dict] | None = None
    head: tuple[str, dict] | None = None

    def __post_init__(self):
        if self.embedding is None:
            self.embedding = ("token_table", dict(vocab_size=self.vocab_size, hidden_size=self.hidden_size,
                                                  weight_name=self.embedding_name))
        if self.head is None:
            self.head = ("linear", dict(vocab_size=self.vocab_size, hidden_size=self.hidden_size, norm=self.final_norm,
                                        weight_name=self.head_name,
                                        tied_to=self.embedding_name if self.tied_head else None))
        if not self.schedule:
            self.schedule = [ScheduleEntry(i) for i in range(len(self.layers))]
        for pos, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule[{pos}] names layer {e.layer}; the model has {len(self.layers)}")
            if e.read_cache_of is not None:
                src = e.read_cache_of
                if not 0 <= src < pos:
                    raise ValueError(f"schedule[{pos}] reads the cache of entry {src}, which does not run before it")
                if self.schedule[src].read_cache_of is not None:
                    raise ValueError(f"schedule[{pos}] reads the cache of entry {src}, which writes none")
