"""SwiGLU feed-forward: ``down(silu(gate(x)) * up(x))``, no biases.

Reference: ``Qwen2MLP.forward`` (src/cloud_engine/model.py:86-100) runs gate and up as
two matrix products and three elementwise kernels.  Here gate and up are stacked into
one weight [2I, H] and one product; SiLU and the multiply run in float32 registers in
one kernel that writes [T, I].
"""

from __future__ import annotations

from .base import FeedForward, TensorSpec, register_part


class SwiGLU(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int) -> None:
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {
            "gate_proj.weight": TensorSpec((self.intermediate_size, self.hidden_size)),
            "up_proj.weight": TensorSpec((self.intermediate_size, self.hidden_size)),
            "down_proj.weight": TensorSpec((self.hidden_size, self.intermediate_size)),
        }

    def bind(self, tensors, runtime) -> None:
        self.runtime = runtime
        self.w_gate_up = runtime.ops.prepare_gate_up(tensors["gate_proj.weight"], tensors["up_proj.weight"])
        self.w_down = runtime.ops.prepare_weight(tensors["down_proj.weight"])

    takes_normed_input = True   # x goes to ops.gate_up only
    kernels_through_ops = True  # every kernel of this part is a method of ``Ops``: a decode step may be recorded

    def forward(self, x, ctx):
        rt = self.runtime
        tokens = x.shape[0]
        hidden = rt.workspace.get("swiglu.hidden", tokens, self.intermediate_size, rt.dtype)
        rt.ops.gate_up(x, self.w_gate_up, hidden, rt.workspace)
        update = rt.workspace.get("feed_forward.update", tokens, self.hidden_size, rt.dtype)
        return rt.ops.linear(hidden, self.w_down, None, update, allow_partials=True,
                             tag="feed_forward.update", residual=getattr(ctx, "residual_sink", None))


register_part("feed_forward", "swiglu", SwiGLU, replace=True)


class ClampedGLU(FeedForward):
    """Gated feed-forward with biases, a capped gate and a shifted up branch:
    ``g = min(W_gate x + b_gate, limit)``, ``u = clamp(W_up x + b_up, -limit, limit)``,
    ``y = g * sigmoid(slope * g) * (u + shift)``, result ``W_down y + b_down``.  Gate and up are one
    stacked product with float32 results; biases, bounds and activation run in float32 in one kernel.
    The result is float32 (a term of the residual sum).  Tensor names: ``gate``, ``gate.b``, ``up``,
    ``up.b``, ``down``, ``down.b``."""

    def __init__(self, hidden_size: int, intermediate_size: int, limit: float, slope: float = 1.702,
                 shift: float = 1.0) -> None:
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.limit = float(limit)
        self.slope = float(slope)
        self.shift = float(shift)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        inter, hidden = self.intermediate_size, self.hidden_size
        return {
            "gate": TensorSpec((inter, hidden)), "gate.b": TensorSpec((inter,), role="vector"),
            "up": TensorSpec((inter, hidden)), "up.b": TensorSpec((inter,), role="vector"),
            "down": TensorSpec((hidden, inter)), "down.b": TensorSpec((hidden,), role="vector"),
        }

    def bind(self, tensors, runtime) -> None:
        import torch

        self.runtime = runtime
        self.w_gate_up = runtime.ops.prepare_weight(torch.cat([tensors["gate"], tensors["up"]]))
        self.b_gate_up = torch.cat([tensors["gate.b"], tensors["up.b"]]).contiguous()
        self.w_down = runtime.ops.prepare_weight(tensors["down"])
        self.b_down = tensors["down.b"].contiguous()

    def forward(self, x, ctx):
        import torch

        rt = self.runtime
        tokens = x.shape[0]
        both = rt.workspace.get("glu.gate_up", tokens, 2 * self.intermediate_size, torch.float32)
        rt.ops.linear(x, self.w_gate_up, None, both)
        hidden = rt.workspace.get("glu.hidden", tokens, self.intermediate_size, rt.dtype)
        rt.ops.gated_act(both, self.b_gate_up, hidden, self.slope, self.limit, self.shift)
        update = rt.workspace.get("feed_forward.update32", tokens, self.hidden_size, torch.float32)
        return rt.ops.linear(hidden, self.w_down, self.b_down, update)


register_part("feed_forward", "clamped_glu", ClampedGLU, replace=True)


class DenseActivation(FeedForward):
    """Feed-forward without a gate: ``W_down act(W_up x)``, no biases.  ``activation`` "relu2": the square of
    relu.  The up product has float32 results, the activation runs in float32 and is rounded once; the result
    is float32 (a term of the residual sum).  Tensor names: ``up``, ``down``."""

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "relu2") -> None:
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        if activation not in ("relu2",):
            raise ValueError(f"dense feed-forward: activation {activation!r} is not built (known: relu2)")
        self.activation = activation

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {"up": TensorSpec((self.intermediate_size, self.hidden_size)),
                "down": TensorSpec((self.hidden_size, self.intermediate_size))}

    def bind(self, tensors, runtime) -> None:
        self.runtime = runtime
        self.w_up = runtime.ops.prepare_weight(tensors["up"])
        self.w_down = runtime.ops.prepare_weight(tensors["down"])

    def forward(self, x, ctx):
        import torch

        rt = self.runtime
        tokens = x.shape[0]
        raised = rt.workspace.get("dense.up", tokens, self.intermediate_size, torch.float32)
        rt.ops.linear(x, self.w_up, None, raised)
        hidden = rt.workspace.get("dense.hidden", tokens, self.intermediate_size, rt.dtype)
        rt.ops.unary_act(raised, hidden, self.activation)
        update = rt.workspace.get("feed_forward.update32", tokens, self.hidden_size, torch.float32)
        return rt.ops.linear(hidden, self.w_down, None, update)


register_part("feed_forward", "dense_activation", DenseActivation, replace=True)


class GatedDense(FeedForward):
    """Gated feed-forward with an activation by name: ``W_down (act(W_gate x) * (W_up x))``, no biases;
    ``activation`` "gelu_tanh" (``0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))``) or "silu".  Gate and up are
    one stacked product with float32 results; the activation and the multiply run in float32 in one kernel and
    are rounded once; the result is float32 (a term of the residual sum).  Tensor names: ``gate``, ``up``,
    ``down``."""

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "gelu_tanh") -> None:
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        if activation not in ("gelu_tanh", "silu"):
            raise ValueError(f"gated feed-forward: activation {activation!r} is not built (known: gelu_tanh, silu)")
        self.activation = activation

    def tensor_specs(self) -> dict[str, TensorSpec]:
        inter, hidden = self.intermediate_size, self.hidden_size
        return {"gate": TensorSpec((inter, hidden)), "up": TensorSpec((inter, hidden)),
                "down": TensorSpec((hidden, inter))}

    def bind(self, tensors, runtime) -> None:
        import torch

        self.runtime = runtime
        self.w_gate_up = runtime.ops.prepare_weight(torch.cat([tensors["gate"], tensors["up"]]))
        self.w_down = runtime.ops.prepare_weight(tensors["down"])

    kernels_through_ops = True

    def forward(self, x, ctx):
        import torch

        rt = self.runtime
        tokens = x.shape[0]
        both = rt.workspace.get("glu.gate_up", tokens, 2 * self.intermediate_size, torch.float32)
        rt.ops.linear(x, self.w_gate_up, None, both)
        hidden = rt.workspace.get("glu.hidden", tokens, self.intermediate_size, rt.dtype)
        rt.ops.glu_act(both, hidden, self.activation)
        update = rt.workspace.get("feed_forward.update32", tokens, self.hidden_size, torch.float32)
        return rt.ops.linear(hidden, self.w_down, None, update)


register_part("feed_forward", "gated_dense", GatedDense, replace=True)
