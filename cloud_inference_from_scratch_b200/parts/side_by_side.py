"""Two mixers side by side: both read the same normalised input and the layer's update is
``left_scale * left(h) + right_scale * right(h)``, summed in float32.

Each side is any registered mixer (a ``PartSpec``); its tensors lie under the side's prefix.  At most one
side may keep pages and at most one may keep per-request state: the layer's binding carries one of each, and
both sides are handed the same binding.  Work lists that a side wants in a step's metadata are found through
``subparts``.
"""

from __future__ import annotations

from ..config.spec import PartSpec
from .base import Mixer, build_part, register_part


class SideBySide(Mixer):
    def __init__(self, left: PartSpec, right: PartSpec, left_scale: float = 1.0, right_scale: float = 1.0) -> None:
        self.sides = (build_part("mixer", left), build_part("mixer", right))
        self.prefixes = (left.prefix, right.prefix)
        self.scales = (float(left_scale), float(right_scale))
        if sum(side.cache_spec() is not None for side in self.sides) > 1:
            raise ValueError("side_by_side: both mixers keep pages; a layer binds one page cache")
        if sum(side.state_spec() is not None for side in self.sides) > 1:
            raise ValueError("side_by_side: both mixers keep per-request state; a layer binds one state")
        self.state_in_graphs = all(side.state_in_graphs or side.state_spec() is None for side in self.sides)
        self.kernels_through_ops = False

    def subparts(self):
        return self.sides

    def cache_spec(self):
        return next((spec for spec in (side.cache_spec() for side in self.sides) if spec is not None), None)

    def state_spec(self):
        return next((spec for spec in (side.state_spec() for side in self.sides) if spec is not None), None)

    def tensor_specs(self):
        return {prefix + name: spec for side, prefix in zip(self.sides, self.prefixes)
                for name, spec in side.tensor_specs().items()}

    def bind(self, tensors, runtime) -> None:
        self.runtime = runtime
        for side, prefix in zip(self.sides, self.prefixes):
            side.bind({name: tensors[prefix + name] for name in side.tensor_specs()}, runtime)

    def forward(self, x, ctx, binding):
        import torch

        rt = self.runtime
        total = rt.workspace.get("side_by_side.sum", x.shape[0], x.shape[1], torch.float32)
        sink, ctx.residual_sink = getattr(ctx, "residual_sink", None), None   # neither side adds itself into the stream
        for index, (side, scale) in enumerate(zip(self.sides, self.scales)):
            y = side.forward(x, ctx, binding)
            if not torch.is_tensor(y):
                y = rt.ops.resolve(y, rt.workspace.get("side_by_side.term", x.shape[0], x.shape[1], torch.float32))
            if y.dtype != torch.float32:
                y = y.float()
            rt.ops.scaled_sum(total, y, scale, accumulate=index > 0)
        ctx.residual_sink = sink
        return total


register_part("mixer", "side_by_side", SideBySide, replace=True)
