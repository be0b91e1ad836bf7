"""A decoder model as the interpretation of a ModelPlan.

The embedding part starts the residual stream, the blocks run in the plan's order, the final
norm reads the wanted rows and the head part makes logits of them
(src/flexengine/inference/models/qwen2.py:90-136).  Nothing here names an architecture or
does arithmetic of its own: sizes and parts come from the plan.
"""
from __future__ import annotations

from .base import block_factory, build_part
from .spec import ModelPlan, PartSpec


class DecoderModel:
    def __init__(self, plan: ModelPlan):
        plan.validate()
        self.plan = plan
        self.blocks = [block_factory(layer.block)(layer) for layer in plan.layers]
        self.final_norm = build_part("norm", plan.final_norm)
        sizes = {"vocab_size": plan.vocab_size, "hidden_size": plan.hidden_size}
        self.embedding = build_part("embedding", plan.embedding or PartSpec("token_table", sizes))
        self.head = build_part("head", plan.head or PartSpec("linear", sizes))
        self.dtype = None
        self.device = None

    # --- weights ----------------------------------------------------------------------
    def parameter_shapes(self) -> dict:
        """{target tuple: (shape, kind)} for every tensor the model holds."""
        shapes = {}
        for where, part in self._outer_parts():
            for name, (shape, kind) in part.parameter_shapes().items():
                shapes[(where, name)] = (shape, kind)
        for i, block in enumerate(self.blocks):
            for part_name, part in block.parts().items():
                for name, (shape, kind) in part.parameter_shapes().items():
                    shapes[("layer", i, part_name, name)] = (shape, kind)
        return shapes

    def bind(self, tensors: dict, dtype, device) -> None:
        """``tensors``: {target tuple: tensor}, complete and shape-checked by the loader."""
        self.dtype, self.device = dtype, device
        for where, part in self._outer_parts():
            part.bind({k[1]: t for k, t in tensors.items() if k[0] == where})
        for i, block in enumerate(self.blocks):
            for part_name, part in block.parts().items():
                part.bind({k[3]: t for k, t in tensors.items()
                           if k[0] == "layer" and k[1] == i and k[2] == part_name})

    def _outer_parts(self):
        """The parts outside the layers, under the names their bindings use."""
        return (("embedding", self.embedding), ("final_norm", self.final_norm), ("lm_head", self.head))

    @property
    def lm_head(self):
        """The head's matrix (the embedding's storage when tied)."""
        return getattr(self.head, "weight", None)

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        def visit(t):
            nonlocal total
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        for part in [p for _, p in self._outer_parts()] + [p for b in self.blocks for p in b.parts().values()]:
            for name in part.parameter_shapes():
                visit(getattr(part, name.replace(".", "_"), None))
        return total

    @staticmethod
    def _knows_next_norm(block) -> bool:
        known = getattr(block, "_knows_next_norm", None)
        if known is None:
            import inspect
            names = inspect.signature(block.forward).parameters
            known = block._knows_next_norm = "next_norm" in names and "next_reads" in names
        return known

    # --- forward -----------------------------------------------------------------------
    def forward(self, ctx):
        """Run the tokens of ``ctx``; returns float32 logits [len(ctx.logit_rows), V] (or None)."""
        residual = self.embedding.forward(ctx)
        pending = None
        run = self.plan.run
        for at, entry in enumerate(run):
            block = self.blocks[entry.layer]
            # a block that can make use of it is told which norm reads the residual after it
            after = self.blocks[run[at + 1].layer] if at + 1 < len(run) else None
            if after is not None and getattr(after, "takes_prenormed", False) and self._knows_next_norm(block):
                reads = getattr(after, "mixer", None)
                pending = block.forward(ctx, residual, pending, entry, next_norm=after.input_norm,
                                        next_reads=reads.reads_first() if reads is not None else None)
            else:
                pending = block.forward(ctx, residual, pending, entry)
        if ctx.num_logit_rows == 0:
            # the last branch output only matters to rows whose logits are wanted
            return None
        h = self.final_norm.forward(ctx, residual, pending, rows=ctx.logit_rows)
        return self.head.forward(ctx, h)
