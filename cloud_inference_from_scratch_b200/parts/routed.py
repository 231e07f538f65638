"""Routed experts: every token runs through the ``top`` of ``experts`` small SwiGLU feed-forwards.

Router logits ``z = W_router h`` in float32; scores ``s = softmax(z)`` over all experts; the
experts with the largest ``s + correction`` are chosen (``correction`` is a stored vector that only
steers the choice); the mixing weights are the chosen experts' ``s`` themselves, renormalised to
sum 1 only if ``renormalize`` says so.  The result is the weighted sum of
``W_down (silu(W_gate h) * (W_up h))`` over the chosen experts, added up in float32 in the order
the experts were chosen.

The experts' matrices are stacked into three tensors at load time ([E, F, H], [E, F, H], [E, H, F];
for bfloat16 with sizes the tensor-core kernels take, gate and up as one [E, 2F, H] with their rows
interleaved in blocks of 16);
Two options: ``router_bias`` adds a stored vector to the logits, and ``score="chosen_softmax"`` chooses the
experts with the largest logits and weights them by the softmax over the chosen logits alone.

the kernels group the (token, expert) pairs by expert on the device and never tell the host how
many tokens an expert got, so a step is one fixed sequence of launches.
"""

from __future__ import annotations

from .base import FeedForward, TensorSpec, register_part


class RoutedExperts(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int, top: int,
                 correction: bool = True, renormalize: bool = False,
                 names: dict[str, str] | None = None, router_bias: bool = False, score: str = "softmax") -> None:
        if not 1 <= top <= num_experts:
            raise ValueError("top must lie in 1..num_experts")
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.num_experts = int(num_experts)
        self.top = int(top)
        self.correction = bool(correction)
        self.renormalize = bool(renormalize)
        self.router_bias = bool(router_bias)
        if score not in ("softmax", "chosen_softmax"):
            raise ValueError(f"routed experts: score {score!r} is not built (known: softmax, chosen_softmax)")
        if score == "chosen_softmax" and correction:
            raise ValueError("routed experts: a correction steers a choice among softmax scores, not among logits")
        self.score = score
        self.names = dict(router="router", correction="correction", expert="e{}.", gate="gate", up="up", down="down",
                          router_bias="router.b")
        self.names.update(names or {})

    def _expert(self, index: int, which: str) -> str:
        return self.names["expert"].format(index) + self.names[which]

    def tensor_specs(self) -> dict[str, TensorSpec]:
        specs = {self.names["router"]: TensorSpec((self.num_experts, self.hidden_size), role="vector")}
        if self.correction:
            specs[self.names["correction"]] = TensorSpec((self.num_experts,), role="vector")
        if self.router_bias:
            specs[self.names["router_bias"]] = TensorSpec((self.num_experts,), role="vector")
        for e in range(self.num_experts):
            specs[self._expert(e, "gate")] = TensorSpec((self.intermediate_size, self.hidden_size))
            specs[self._expert(e, "up")] = TensorSpec((self.intermediate_size, self.hidden_size))
            specs[self._expert(e, "down")] = TensorSpec((self.hidden_size, self.intermediate_size))
        return specs

    def bind(self, tensors, runtime) -> None:
        import torch

        self.runtime = runtime
        self.router = tensors[self.names["router"]].contiguous()
        self.bias = tensors[self.names["correction"]].contiguous() if self.correction else None
        self.logit_bias = tensors[self.names["router_bias"]].contiguous() if self.router_bias else None
        stack = lambda which: runtime.ops.prepare_weight(  # noqa: E731
            torch.stack([tensors[self._expert(e, which)] for e in range(self.num_experts)]))
        self.w_gate, self.w_up, self.w_down = stack("gate"), stack("up"), stack("down")
        if runtime.ops.moe_interleaves(self.hidden_size, self.intermediate_size):
            # one tensor for gate and up, rows interleaved in blocks of 16: the tensor-core kernels
            # finish SiLU(gate) * up in their epilogue
            self.w_gate, self.w_up = runtime.ops.interleave_gate_up(self.w_gate, self.w_up), None

    def forward(self, x, ctx):
        import torch

        rt = self.runtime
        update = rt.workspace.get("feed_forward.update32", x.shape[0], self.hidden_size, torch.float32)
        return rt.ops.routed_experts(x, self.router, self.bias, self.w_gate, self.w_up, self.w_down,
                                     self.top, self.renormalize, update, rt.workspace, router_bias=self.logit_bias,
                                     chosen_softmax=self.score == "chosen_softmax")


register_part("feed_forward", "routed_experts", RoutedExperts, replace=True)
