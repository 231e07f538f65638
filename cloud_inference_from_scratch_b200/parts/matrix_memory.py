"""Matrix memory (the mLSTM of xLSTM): a recurrent mixer with a matrix state per head and exponential gates
that are kept in range by a running maximum.

For input ``h``: ``q = W_q h * dim^(-1/2)``, ``k = W_k h`` (heads x dim), ``v = W_v h`` (heads x vdim); per
head a log input gate ``i = cap * tanh((W_i h + b_i) / cap)`` and a log forget gate
``f = logsigmoid(cap * tanh((W_f h + b_f) / cap))``.  The state of a head is a matrix ``S`` [dim, vdim], a
vector ``n`` [dim] and a running maximum ``m``, all zero at the start of a request:

    m_t = max(f + m_(t-1), i)
    S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T          (n_t likewise with k alone)
    o_t = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6)

Every head of ``o`` is divided by its own root mean square; the heads side by side are multiplied by a gain
vector and by ``sigmoid(W_g h)`` and projected by ``W_o``.

q, k, v, the output gate and both gate projections come from ONE matrix product with float32 results; from
there to the normalised output everything is float32.  The state is float32 and lives in the request's state
slot between steps; the mixer holds no pages.

Tensor names (after the part's prefix): ``q``, ``k``, ``v``, ``g``, ``i``, ``i.b``, ``f``, ``f.b``, ``norm``, ``o``.
"""

from __future__ import annotations

from .base import Mixer, StateSpec, TensorSpec, register_part


NORMALISER_COLUMNS = 32     # as the scan kernel lays a head's state out


class MatrixMemory(Mixer):
    state_in_graphs = True   # the scan reads the step's numbers on the device and honours request_active

    def __init__(self, hidden_size: int, num_heads: int, key_dim: int, value_dim: int, gate_cap: float, eps: float,
                 names: dict[str, str] | None = None) -> None:
        self.hidden_size = int(hidden_size)
        self.num_heads = int(num_heads)
        self.key_dim = int(key_dim)
        self.value_dim = int(value_dim)
        self.gate_cap = float(gate_cap)
        if not self.gate_cap > 0.0:
            raise ValueError("the gate cap must be positive")
        self.eps = float(eps)
        self.qk_width = self.num_heads * self.key_dim
        self.v_width = self.num_heads * self.value_dim
        self.names = {key: key for key in ("q", "k", "v", "g", "i", "i.b", "f", "f.b", "norm", "o")}
        self.names.update(names or {})

    @property
    def plan_key(self):
        return ("memory.chunks",)

    def plan(self, host, cache):
        """Chunk work lists for a step with prompt portions (one list serves every matrix memory)."""
        return self.runtime.ops.plan_memory_chunks(host)

    def state_spec(self) -> StateSpec:
        # per head: the matrix, then the normaliser vector and the running maximum once for every
        # NORMALISER_COLUMNS value columns (the blocks of a scan share no word that one of them writes)
        copies = -(-self.value_dim // NORMALISER_COLUMNS)
        return StateSpec((self.num_heads * (self.key_dim * self.value_dim + copies * (self.key_dim + 1)),), "float32")

    def tensor_specs(self) -> dict[str, TensorSpec]:
        n, hidden = self.names, self.hidden_size
        return {
            n["q"]: TensorSpec((self.qk_width, hidden)), n["k"]: TensorSpec((self.qk_width, hidden)),
            n["v"]: TensorSpec((self.v_width, hidden)), n["g"]: TensorSpec((self.v_width, hidden)),
            n["i"]: TensorSpec((self.num_heads, hidden)), n["i.b"]: TensorSpec((self.num_heads,), role="vector"),
            n["f"]: TensorSpec((self.num_heads, hidden)), n["f.b"]: TensorSpec((self.num_heads,), role="vector"),
            n["norm"]: TensorSpec((self.v_width,), init="gain", role="vector"),
            n["o"]: TensorSpec((hidden, self.v_width)),
        }

    def bind(self, tensors, runtime) -> None:
        import torch

        self.runtime = runtime
        ops, n = runtime.ops, self.names
        largest, _ = ops.require_recurrent()
        if ops.normaliser_columns != NORMALISER_COLUMNS:
            raise RuntimeError("the scan kernel and this part disagree on the layout of a head's state")
        if self.key_dim > largest:
            raise ValueError(f"the scan kernels take key sizes of up to {largest}, got {self.key_dim}")
        self.w_in = ops.prepare_weight(torch.cat([tensors[n[key]] for key in ("q", "k", "v", "g", "i", "f")]))
        self.w_out = ops.prepare_weight(tensors[n["o"]])
        self.input_bias = tensors[n["i.b"]].contiguous()
        self.forget_bias = tensors[n["f.b"]].contiguous()
        self.gain = tensors[n["norm"]].contiguous()

    def forward(self, x, ctx, binding):
        import torch

        rt = self.runtime
        ops = rt.ops
        tokens, f32 = x.shape[0], torch.float32
        qk, vv, heads = self.qk_width, self.v_width, self.num_heads
        proj = rt.workspace.get("memory.proj", tokens, 2 * qk + 2 * vv + 2 * heads, f32)
        ops.linear(x, self.w_in, None, proj)
        mixed = rt.workspace.get("memory.o", tokens, vv, f32)
        below = ops.mlstm_scan(proj, (0, qk, 2 * qk, 2 * qk + 2 * vv, 2 * qk + 2 * vv + heads), self.input_bias,
                               self.forget_bias, self.gate_cap, self.key_dim ** -0.5, mixed, binding.state, ctx,
                               heads, self.key_dim, self.value_dim,
                               plan=getattr(ctx, "extras", {}).get(self.plan_key) or None)
        gated = rt.workspace.get("memory.gated", tokens, vv, rt.dtype)
        ops.head_norm_gate(mixed, proj[:, 2 * qk + vv:2 * qk + 2 * vv], self.gain, self.eps, gated, heads,
                           denominators=below)
        update = rt.workspace.get("memory.update32", tokens, self.hidden_size, f32)
        return ops.linear(gated, self.w_out, None, update)


register_part("mixer", "matrix_memory", MatrixMemory, replace=True)
