"""Gated delta rule: a recurrent mixer whose state forgets by ONE decay per head and corrects what it reads
back under the current key.

For input ``h``: ``q = W_q h`` and ``k = W_k h`` (kv_heads x dim), ``v = W_v h`` (heads x vdim); value head
``j`` reads q/k head ``j // (heads / kv_heads)``.  Each of q, k, v passes a short causal convolution over time
per channel (``taps`` taps, the last one the current token's, zeros before the start of a request) and SiLU.
Then q and k are made unit vectors per head (``x / sqrt(sum(x^2) + 1e-6)``) and q is multiplied by
``dim^(-1/2)``.  Per head a write strength ``b = sigmoid(W_b h)`` and a decay
``g = exp(-exp(A) * softplus(W_a h + dt))``.  The state ``S`` [dim, vdim] of a head runs

    S <- g S;    u = b (v - S^T k);    S <- S + k u^T;    o = S^T q

so the read-out sees the current token's write.  Every head of ``o`` is divided by its own root mean square,
multiplied by a gain vector of a head's size (shared by the heads) and by ``silu(W_g h)``, and projected by
``W_o``.

q, k, v, the gate and both rate projections come from ONE matrix product with float32 results; from there to
the normalised output everything is float32.  A request's state is the matrices of its heads and the inputs of
the convolution's last ``taps - 1`` tokens, float32, in its state slot; the mixer holds no pages.

Tensor names (after the part's prefix): ``q``, ``q.conv``, ``k``, ``k.conv``, ``v``, ``v.conv``, ``b``, ``a``,
``A_log``, ``dt_bias``, ``g``, ``norm``, ``o``.
"""

from __future__ import annotations

from .base import Mixer, StateSpec, TensorSpec, register_part


class GatedDelta(Mixer):
    state_in_graphs = True   # the kernels read the step's numbers on the device and honour request_active

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int,
                 taps: int, eps: float, names: dict[str, str] | None = None) -> None:
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if taps < 1:
            raise ValueError("the short convolution needs at least one tap")
        self.hidden_size = int(hidden_size)
        self.num_heads = int(num_heads)
        self.num_kv_heads = int(num_kv_heads)
        self.key_dim = int(key_dim)
        self.value_dim = int(value_dim)
        self.taps = int(taps)
        self.eps = float(eps)
        self.qk_width = self.num_kv_heads * self.key_dim
        self.v_width = self.num_heads * self.value_dim
        self.channels = 2 * self.qk_width + self.v_width          # what passes the convolution
        self.matrix_floats = self.num_heads * self.key_dim * self.value_dim
        self.names = {key: key for key in ("q", "q.conv", "k", "k.conv", "v", "v.conv", "b", "a", "A_log",
                                           "dt_bias", "g", "norm", "o")}
        self.names.update(names or {})

    @property
    def plan_key(self):
        return ("memory.chunks",)       # the matrix memory's chunks: one list serves both mixers

    def plan(self, host, cache):
        """Chunk work lists for a step with prompt portions."""
        return self.runtime.ops.plan_memory_chunks(host)

    def state_spec(self) -> StateSpec:
        # the heads' matrices, then the convolution's history [taps - 1, channels]
        return StateSpec((self.matrix_floats + (self.taps - 1) * self.channels,), "float32")

    def tensor_specs(self) -> dict[str, TensorSpec]:
        n, hidden = self.names, self.hidden_size
        specs = {
            n["q"]: TensorSpec((self.qk_width, hidden)), n["k"]: TensorSpec((self.qk_width, hidden)),
            n["v"]: TensorSpec((self.v_width, hidden)), n["g"]: TensorSpec((self.v_width, hidden)),
            n["b"]: TensorSpec((self.num_heads, hidden)), n["a"]: TensorSpec((self.num_heads, hidden)),
            n["A_log"]: TensorSpec((self.num_heads,), role="vector"),
            n["dt_bias"]: TensorSpec((self.num_heads,), role="vector"),
            n["norm"]: TensorSpec((self.value_dim,), init="gain", role="vector"),
            n["o"]: TensorSpec((hidden, self.v_width)),
        }
        for key, width in (("q.conv", self.qk_width), ("k.conv", self.qk_width), ("v.conv", self.v_width)):
            specs[n[key]] = TensorSpec((width, self.taps), role="vector")
        return specs

    def bind(self, tensors, runtime) -> None:
        import torch

        self.runtime = runtime
        ops, n = runtime.ops, self.names
        largest, longest = ops.require_recurrent()
        if self.key_dim > largest:
            raise ValueError(f"the scan kernels take key sizes of up to {largest}, got {self.key_dim}")
        if self.taps > longest:
            raise ValueError(f"the short convolution takes up to {longest} taps, got {self.taps}")
        self.w_in = ops.prepare_weight(torch.cat([tensors[n[key]] for key in ("q", "k", "v", "g", "b", "a")]))
        self.w_out = ops.prepare_weight(tensors[n["o"]])
        self.w_conv = torch.cat([tensors[n[key]] for key in ("q.conv", "k.conv", "v.conv")]).float().contiguous()
        self.a_log = tensors[n["A_log"]].contiguous()
        self.dt_bias = tensors[n["dt_bias"]].contiguous()
        self.gain = tensors[n["norm"]].contiguous()

    def forward(self, x, ctx, binding):
        import torch

        rt = self.runtime
        ops = rt.ops
        tokens, f32 = x.shape[0], torch.float32
        qk, vv, heads = self.qk_width, self.v_width, self.num_heads
        proj = rt.workspace.get("gated_delta.proj", tokens, self.channels + vv + 2 * heads, f32)
        ops.linear(x, self.w_in, None, proj)
        conv = rt.workspace.get("gated_delta.conv", tokens, self.channels, f32)
        ops.short_conv(proj, self.w_conv, binding.state[:, self.matrix_floats:], conv, ctx)
        mixed = rt.workspace.get("gated_delta.o", tokens, vv, f32)
        ops.gated_delta_scan(conv, (0, qk, 2 * qk), proj, (self.channels + vv, self.channels + vv + heads),
                             self.a_log, self.dt_bias, self.key_dim ** -0.5, mixed, binding.state, ctx, heads,
                             self.num_kv_heads, self.key_dim, self.value_dim,
                             plan=getattr(ctx, "extras", {}).get(self.plan_key) or None)
        gated = rt.workspace.get("gated_delta.gated", tokens, vv, rt.dtype)
        ops.head_norm_gate(mixed, proj[:, self.channels:self.channels + vv], self.gain, self.eps, gated, heads,
                           gate_act="silu")
        update = rt.workspace.get("mixer.update32", tokens, self.hidden_size, f32)
        return ops.linear(gated, self.w_out, None, update)


register_part("mixer", "gated_delta", GatedDelta, replace=True)
