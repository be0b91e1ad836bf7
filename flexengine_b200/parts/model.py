"""A decoder model as the interpretation of a ModelPlan.

Embedding, the run order over blocks, the final norm on the wanted rows and the
vocabulary projection (src/flexengine/inference/models/qwen2.py:90-136).  Nothing
here names an architecture; sizes come from the plan.
"""
from __future__ import annotations

from .base import block_factory, build_part
from .spec import ModelPlan


class DecoderModel:
    def __init__(self, plan: ModelPlan):
        plan.validate()
        self.plan = plan
        self.blocks = [block_factory(layer.block)(layer) for layer in plan.layers]
        self.final_norm = build_part("norm", plan.final_norm)
        self.embedding = None     # [V, H]
        self.lm_head = None       # [V, H]; the same storage as the embedding when tied
        self.dtype = None
        self.device = None

    # --- weights ----------------------------------------------------------------------
    def parameter_shapes(self) -> dict:
        """{target tuple: (shape, kind)} for every tensor the model holds."""
        v, h = self.plan.vocab_size, self.plan.hidden_size
        shapes = {("embedding", "weight"): ((v, h), "matrix"), ("lm_head", "weight"): ((v, h), "matrix")}
        for name, (shape, kind) in self.final_norm.parameter_shapes().items():
            shapes[("final_norm", name)] = (shape, kind)
        for i, block in enumerate(self.blocks):
            for part_name, part in block.parts().items():
                for name, (shape, kind) in part.parameter_shapes().items():
                    shapes[("layer", i, part_name, name)] = (shape, kind)
        return shapes

    def bind(self, tensors: dict, dtype, device) -> None:
        """``tensors``: {target tuple: tensor}, complete and shape-checked by the loader."""
        self.dtype, self.device = dtype, device
        self.embedding = tensors[("embedding", "weight")]
        self.lm_head = tensors[("lm_head", "weight")]
        self.final_norm.bind({k[1]: t for k, t in tensors.items() if k[0] == "final_norm"})
        for i, block in enumerate(self.blocks):
            for part_name, part in block.parts().items():
                part.bind({k[3]: t for k, t in tensors.items()
                           if k[0] == "layer" and k[1] == i and k[2] == part_name})

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        def visit(t):
            nonlocal total
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        visit(self.embedding), visit(self.lm_head)
        for part in [self.final_norm] + [p for b in self.blocks for p in b.parts().values()]:
            for name in part.parameter_shapes():
                visit(getattr(part, name.replace(".", "_"), None))
        return total

    # --- forward -----------------------------------------------------------------------
    def forward(self, ctx):
        """Run the tokens of ``ctx``; returns float32 logits [len(ctx.logit_rows), V] (or None)."""
        ops = ctx.ops
        residual = ops.embedding(ctx.token_ids, self.embedding)
        pending = None
        for entry in self.plan.run:
            pending = self.blocks[entry.layer].forward(ctx, residual, pending, entry)
        if ctx.num_logit_rows == 0:
            # the last branch output only matters to rows whose logits are wanted
            return None
        h = self.final_norm.forward(ctx, residual, pending, rows=ctx.logit_rows)
        return ops.linear(h, self.lm_head, None, out_float32=True)
