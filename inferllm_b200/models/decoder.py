"""The generic decoder: embedding, blocks run in the order of the schedule, final norm, head.

It is built from a `ModelSpec` alone: each layer's block arrangement, mixer, feed-forward and
norm are looked up by kind in the part registries and built with the spec's parameters, so
layers of one model may differ, a layer may run twice, and a layer may read another layer's
cache.  The reference builds its module list the same way from a per-model `construct_llm`
(src/graph/llama_like.cpp:54-109) and runs it in `Graph::execute` (src/core/graph.cpp:166-197).
"""
from __future__ import annotations

from typing import Dict, List

from ..config.base import ModelSpec
from ..parts.base import PagedKV, TensorDecl, build_part, lookup
from ..parts.embedding import Embedding, LMHead


class DecoderModel:
    def __init__(self, spec: ModelSpec, runtime):
        spec.validate()
        self.spec = spec
        self.rt = runtime
        self.embedding = Embedding(spec.embedding, runtime)
        self.blocks = []
        self._names: List[Dict[str, tuple]] = []  # per layer: full tensor name -> (part, local name)
        for ls in spec.layers:
            block_cls = lookup("block", ls.block)
            mixer = build_part("mixer", ls.mixer, runtime)
            ffn = build_part("feed_forward", ls.ffn, runtime)
            norms = {role: build_part("norm", ls.norm, runtime) for role in block_cls.norm_roles()}
            self.blocks.append(block_cls(mixer, ffn, norms))
        self.final_norm = build_part("norm", spec.final_norm, runtime)
        self.head = LMHead(spec.head, runtime)

    # ---- tensors

    def _owners(self):
        """(tensor-name prefix, part) for every part that owns tensors."""
        out = [(self.spec.embedding["name"], self.embedding)]
        for ls, block in zip(self.spec.layers, self.blocks):
            out.append((ls.prefix + ls.names["mixer"], block.mixer))
            out.append((ls.prefix + ls.names["ffn"], block.ffn))
            for role, norm in block.norms.items():
                out.append((ls.prefix + ls.names[role], norm))
        out.append((self.spec.final_norm["name"], self.final_norm))
        out.append((self.spec.head["name"], self.head))
        return out

    def tensor_decls(self) -> Dict[str, TensorDecl]:
        """Every tensor the model reads from a weight file, by its name there."""
        decls = {}
        for prefix, part in self._owners():
            for local, decl in part.tensors().items():
                decls[prefix + local] = decl
        return decls

    def load_tensors(self, fetch) -> None:
        """`fetch(name)` returns the tensor on the device; each part takes its own and packs
        them, one part at a time so that at most one part's tensors exist twice."""
        for prefix, part in self._owners():
            names = part.tensors()
            if names or part is self.head:
                part.load({local: fetch(prefix + local) for local in names})
        if self.head.tied:
            self.head.tie(self.embedding)

    # ---- cache

    def cache_requests(self) -> Dict[int, object]:
        """Cache entry number -> what its writing layer's mixer asks for."""
        return {e.cache: self.blocks[e.layer].mixer.cache_request()
                for e in self.spec.schedule if e.writes}

    # ---- one step

    def forward(self, ctx):
        """Run the tokens of one step; returns float32 logits [len(ctx.want_rows), vocab]."""
        stream = self.embedding.forward(ctx.ids, ctx)
        for e in self.spec.schedule:
            self.blocks[e.layer].forward(stream, ctx, ctx.cache_view(e.cache, e.writes), e.writes)
        if ctx.want_rows.numel() == 0:
            import torch
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=stream.x.device)
        y = self.final_norm.forward(stream, rows=ctx.want_rows)
        return self.head.forward(y)

    def graph_safe(self) -> bool:
        """True if a one-token-per-sequence step launches the same kernels every time, i.e. no
        part reads host-side fields of the step context (a mixer says so with `graph_safe`)."""
        return all(getattr(b.mixer, "graph_safe", False) and getattr(b.ffn, "graph_safe", True)
                   for b in self.blocks)

    def pad_safe(self) -> bool:
        """True if a single prompt may be run with tokens appended behind its own (see
        `parts.Mixer.pad_safe`) and launches the same kernels for the same token count."""
        return self.graph_safe() and all(getattr(b.mixer, "pad_safe", False) for b in self.blocks)
