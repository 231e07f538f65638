"""Gated linear attention: linear attention whose state decays per key channel by a gate read from the input.

For input ``h``: ``q = W_q h * dim^(-1/2)``, ``k = W_k h`` (heads x dim), ``v = W_v h`` (heads x vdim) and a decay
per head and key channel ``alpha = sigmoid(z)^(1 / tau)`` with ``z = W_a2 (W_a1 h) + b`` (a projection through a
narrow inner width).  Per head a state matrix ``S`` [dim, vdim] runs through the request's tokens,
``S <- diag(alpha) S + k v^T`` and ``o = S^T q``; it starts at zero, is float32 and lives in the request's
state slot between steps.  Every head of ``o`` is divided by its own root mean square and multiplied by a gain
vector of a head's size that all heads share; the heads side by side are multiplied by ``silu(W_g h)`` and
projected by ``W_o``.

q, k, v and the gate come from ONE matrix product with float32 results that are not rounded again before the
recurrence; the decay's logarithm, the exponentials and the state are float32.  A step of single tokens runs the
recurrence token by token; a step with prompt portions runs it in chunks of 32 tokens (the same sums in another
order).  The mixer holds no pages: its cache is the state alone.

Tensor names (after the part's prefix): ``q``, ``k``, ``v``, ``g``, ``o``, ``norm``, ``a1``, ``a2``, ``a2.b``;
``names`` maps them to others.  The inner width of the decay projection is ``decay_rank``, or, if None, whatever
the stored ``a1`` has.
"""

from __future__ import annotations

from .base import Mixer, StateSpec, TensorSpec, register_part

NAMES = ("q", "k", "v", "g", "o", "norm", "a1", "a2", "a2.b")


class GatedLinearAttention(Mixer):
    state_in_graphs = True   # the kernels read the step's numbers on the device and honour request_active
    kernels_through_ops = True

    def __init__(self, hidden_size: int, num_heads: int, key_dim: int, value_dim: int, tau: float, eps: float,
                 q_scale: float | None = None, decay_rank: int | None = None,
                 names: dict[str, str] | None = None) -> None:
        if not tau > 0:
            raise ValueError("gated linear attention: tau must be positive")
        self.hidden_size = int(hidden_size)
        self.num_heads = int(num_heads)
        self.key_dim = int(key_dim)
        self.value_dim = int(value_dim)
        self.tau = float(tau)
        self.eps = float(eps)
        self.decay_rank = int(decay_rank) if decay_rank else -1     # -1: the file says
        self.q_scale = float(q_scale) if q_scale is not None else self.key_dim ** -0.5
        self.qk_width = self.num_heads * self.key_dim
        self.v_width = self.num_heads * self.value_dim
        self.names = {key: key for key in NAMES}
        self.names.update(names or {})

    @property
    def plan_key(self):
        return ("gla",)

    def plan(self, host, cache):
        """Chunk work lists for a step with prompt portions (one list serves every such layer)."""
        return self.runtime.ops.plan_gla(host)

    def state_spec(self) -> StateSpec:
        return StateSpec((self.num_heads, self.key_dim, self.value_dim), "float32")

    def tensor_specs(self) -> dict[str, TensorSpec]:
        n, hidden = self.names, self.hidden_size
        return {
            n["q"]: TensorSpec((self.qk_width, hidden)),
            n["k"]: TensorSpec((self.qk_width, hidden)),
            n["v"]: TensorSpec((self.v_width, hidden)),
            n["g"]: TensorSpec((self.v_width, hidden)),
            n["o"]: TensorSpec((hidden, self.v_width)),
            n["norm"]: TensorSpec((self.value_dim,), init="gain", role="vector"),
            n["a1"]: TensorSpec((self.decay_rank, hidden)),
            n["a2"]: TensorSpec((self.qk_width, self.decay_rank)),
            n["a2.b"]: TensorSpec((self.qk_width,), role="vector"),
        }

    def bind(self, tensors, runtime) -> None:
        import torch

        self.runtime = runtime
        ops, n = runtime.ops, self.names
        largest = ops.require_gla()
        if self.key_dim > largest:
            raise ValueError(f"the gated-linear-attention kernels take keys of up to {largest}, got {self.key_dim}")
        self.rank = int(tensors[n["a1"]].shape[0])
        if tensors[n["a2"]].shape[1] != self.rank:
            raise ValueError("the two decay projections disagree about their inner width")
        self.w_in = ops.prepare_weight(torch.cat([tensors[n[key]] for key in ("q", "k", "v", "g")]))
        self.w_narrow = ops.prepare_weight(tensors[n["a1"]])
        self.w_decay = ops.prepare_weight(tensors[n["a2"]])
        self.w_out = ops.prepare_weight(tensors[n["o"]])
        self.decay_bias = tensors[n["a2.b"]].contiguous()
        self.gain = tensors[n["norm"]].contiguous()

    def forward(self, x, ctx, binding):
        import torch

        rt = self.runtime
        ops = rt.ops
        tokens, f32 = x.shape[0], torch.float32
        qk, vw = self.qk_width, self.v_width
        proj = rt.workspace.get("gla.proj", tokens, 2 * qk + 2 * vw, f32)
        ops.linear(x, self.w_in, None, proj)
        narrow = rt.workspace.get("gla.narrow", tokens, self.rank, rt.dtype)
        ops.linear(x, self.w_narrow, None, narrow)
        logits = rt.workspace.get("gla.decay", tokens, qk, f32)
        ops.linear(narrow, self.w_decay, None, logits)
        mixed = rt.workspace.get("gla.o", tokens, vw, f32)
        plan = getattr(ctx, "extras", {}).get(self.plan_key) or None
        ops.gla(proj, (0, qk, 2 * qk), logits, self.decay_bias, self.tau, self.q_scale, mixed, binding.state, ctx,
                self.num_heads, self.key_dim, self.value_dim, plan=plan)
        gated = rt.workspace.get("gla.gated", tokens, vw, rt.dtype)
        ops.head_norm_gate(mixed, proj[:, 2 * qk + vw:], self.gain, self.eps, gated, self.num_heads, gate_act="silu")
        update = rt.workspace.get("mixer.update32", tokens, self.hidden_size, f32)
        return ops.linear(gated, self.w_out, None, update)


register_part("mixer", "gla", GatedLinearAttention, replace=True)
