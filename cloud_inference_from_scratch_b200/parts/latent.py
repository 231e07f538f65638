"""Attention whose keys and values are linear maps of a cached latent ("latent attention").

For input ``h`` [T, width], with ``H`` heads, per head ``dim`` plain and ``rot_dim`` rotated
query/key elements, value size ``vdim``, latent size ``kv_rank`` and query latent size ``q_rank``:

* ``c_q = rmsnorm(W_dq h) * g_q``; ``q = W_uq c_q``, head by head [dim plain | rot_dim rotated];
* ``W_dkv h`` = [latent (kv_rank) | key part (rot_dim)]; ``c = rmsnorm(latent) * g_kv`` and the key part,
  rotated by the token's position, are all the pages keep (one row each per token, for all heads);
* head j: key = [W_uk[j] c | rotated key part], value = W_uv[j] c, score = q . key * scale, causal;
* softmax, optionally with one more term exp(sink_j) in the denominator (``sink``: a stored number per
  head that has no key and no value and is not scaled);
* optionally the heads side by side are multiplied by sigmoid(W_g h) (``gate``); then ``W_o``.

The maps are linear, so keys and values are never expanded: the plain query part is carried into
the latent space (``q' = W_uk[j]^T q_plain``: a product per head), attention runs over the rows
[c | key part] for all heads at once and sums latents, and ``W_uv[j]`` is applied to the sum (again a
product per head, with the gate in its epilogue).  Scores, weights, norms and angles are float32.

``shares_cache``: the layer has no ``W_dkv`` and no latent norm of its own; it reads the rows another
layer of equal ``kv_rank``, ``rot_dim`` and rotation wrote (the schedule's ``reads_cache_of``).

``q_rank`` 0: no query latent; ``q = W_q h`` straight from the input (tensor ``q``).  ``window`` > 0: a query at
position i sees the keys j with 0 <= i - j < window only, and the pages behind the window are given back.

Tensor names (after the part's prefix): ``dq``, ``dq.norm``, ``uq``, ``dkv``, ``dkv.norm``, ``uk``, ``uv``,
``sink``, ``g``, ``o``, and ``q`` when there is no query latent; ``names`` maps them to others.
"""

from __future__ import annotations

from types import SimpleNamespace

from ..config.spec import PartSpec
from .base import CacheSpec, Mixer, TensorSpec, build_part, register_part

NAMES = ("dq", "dq.norm", "uq", "dkv", "dkv.norm", "uk", "uv", "sink", "g", "o", "q")


class LatentAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int, value_dim: int,
                 kv_rank: int, q_rank: int, scale: float, position: PartSpec, norm_eps: float,
                 sink: bool = False, gate: bool = False, shares_cache: bool = False,
                 names: dict[str, str] | None = None, window: int = 0) -> None:
        self.hidden_size = int(hidden_size)
        self.num_heads = int(num_heads)
        self.head_dim = int(head_dim)
        self.rot_dim = int(rot_dim)
        self.value_dim = int(value_dim)
        self.kv_rank = int(kv_rank)
        self.q_rank = int(q_rank)
        self.scale = float(scale)
        self.norm_eps = float(norm_eps)
        self.sink = bool(sink)
        self.gate = bool(gate)
        self.shares_cache = bool(shares_cache)
        self.window = int(window)
        if self.window < 0 or self.q_rank < 0:
            raise ValueError("latent attention: window and q_rank must not be negative")
        self.position = build_part("position", position)
        if self.position.rotary_dim > self.rot_dim:
            raise ValueError("the rotation covers more elements than the rotated part has")
        self.q_head = self.head_dim + self.rot_dim
        self.out_width = self.num_heads * self.value_dim
        self.names = {key: key for key in NAMES}
        self.names.update(names or {})

    def cache_spec(self) -> CacheSpec:
        # one row of "keys" per token holds the latent, one row of "values" the rotated key part
        return CacheSpec(kv_heads=1, head_dim=self.kv_rank, window=self.window,
                         value_dim=0 if self.rot_dim == self.kv_rank else self.rot_dim)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        n, heads = self.names, self.num_heads
        specs = {
            n["uk"]: TensorSpec((heads * self.head_dim, self.kv_rank)),
            n["uv"]: TensorSpec((heads * self.value_dim, self.kv_rank)),
            n["o"]: TensorSpec((self.hidden_size, self.out_width)),
        }
        if self.q_rank:
            specs[n["dq"]] = TensorSpec((self.q_rank, self.hidden_size))
            specs[n["dq.norm"]] = TensorSpec((self.q_rank,), init="gain", role="vector")
            specs[n["uq"]] = TensorSpec((heads * self.q_head, self.q_rank))
        else:
            specs[n["q"]] = TensorSpec((heads * self.q_head, self.hidden_size))
        if not self.shares_cache:
            specs[n["dkv"]] = TensorSpec((self.kv_rank + self.rot_dim, self.hidden_size))
            specs[n["dkv.norm"]] = TensorSpec((self.kv_rank,), init="gain", role="vector")
        if self.sink:
            specs[n["sink"]] = TensorSpec((heads,), role="vector")
        if self.gate:
            specs[n["g"]] = TensorSpec((self.out_width, self.hidden_size))
        return specs

    def bind(self, tensors, runtime) -> None:
        import torch

        self.runtime = runtime
        ops, n, heads = runtime.ops, self.names, self.num_heads
        largest = ops.require_latent()
        if self.kv_rank > largest:
            raise ValueError(f"latent attention kernels take a latent of up to {largest}, got {self.kv_rank}")
        # one product for everything that reads h: query latent (or, without one, the queries themselves), then
        # latent and key part, then the gate
        stacked = [tensors[n["dq"] if self.q_rank else n["q"]]]
        self.q_columns = stacked[0].shape[0]
        if not self.shares_cache:
            stacked.append(tensors[n["dkv"]])
        self.gate_column = sum(t.shape[0] for t in stacked)
        if self.gate:
            stacked.append(tensors[n["g"]])
        self.w_down = ops.prepare_weight(torch.cat(stacked))
        self.w_uq = ops.prepare_weight(tensors[n["uq"]]) if self.q_rank else None
        # per head [K, N]: the plain query part times W_uk[j] (dim -> kv_rank) is W_uk[j] as stored;
        # the latent sum times W_uv[j]^T (kv_rank -> vdim) is the stored [vdim, kv_rank] transposed
        self.w_absorb = ops.prepare_weight(tensors[n["uk"]]).view(heads, self.head_dim, self.kv_rank).contiguous()
        self.w_expand = (ops.prepare_weight(tensors[n["uv"]]).view(heads, self.value_dim, self.kv_rank)
                         .transpose(1, 2).contiguous())
        self.w_o = ops.prepare_weight(tensors[n["o"]])
        self.q_gain = tensors[n["dq.norm"]].contiguous() if self.q_rank else None
        self.kv_gain = tensors[n["dkv.norm"]].contiguous() if not self.shares_cache else None
        self.sinks = tensors[n["sink"]].contiguous() if self.sink else None
        self.position.bind({}, runtime)
        inv_freq = torch.tensor(self.position.frequencies(), dtype=torch.float64).to(torch.float32)
        self.rotation = SimpleNamespace(
            inv_freq=inv_freq.to(runtime.device).contiguous(), magnitude=self.position.magnitude,
            interleaved=self.position.pairing == "interleaved", dims=self.position.rotary_dim)

    def forward(self, x, ctx, binding):
        import torch

        rt = self.runtime
        ops = rt.ops
        tokens, heads, f32 = x.shape[0], self.num_heads, torch.float32
        if binding.owns_cache == self.shares_cache:
            raise ValueError("a latent-attention layer either makes its own latent or reads another layer's")
        kv = binding.kv
        down = rt.workspace.get("latent.down", tokens, self.w_down.shape[0], f32)
        ops.linear(x, self.w_down, None, down)
        if self.q_rank:
            q_latent = rt.workspace.get("latent.q_latent", tokens, self.q_rank, rt.dtype)
            ops.latent_prepare(down, q_latent, self.q_gain, self.kv_gain, ctx, kv, self.rotation, self.q_rank,
                               self.kv_rank, self.rot_dim, self.norm_eps, not self.shares_cache, binding.owns_cache)
            q = rt.workspace.get("latent.q", tokens, heads * self.q_head, f32)
            ops.linear(q_latent, self.w_uq, None, q)
        else:
            # the queries are columns of the one product; what follows them is normalised, rotated and cached
            q = down[:, :self.q_columns]
            if not self.shares_cache:
                ops.latent_prepare(down[:, self.q_columns:], None, None, self.kv_gain, ctx, kv, self.rotation, 0,
                                   self.kv_rank, self.rot_dim, self.norm_eps, True, binding.owns_cache)
        q_absorbed = rt.workspace.get("latent.q_absorbed", tokens, heads * self.kv_rank, f32)
        ops.head_linear(q, self.q_head, self.w_absorb, q_absorbed, self.kv_rank, heads)
        summed = rt.workspace.get("latent.sum", tokens, heads * self.kv_rank, f32)
        ops.latent_attention(q_absorbed, q[:, self.head_dim:], self.q_head, summed, ctx, kv, self.rotation,
                             self.sinks, heads, self.kv_rank, self.rot_dim, self.scale, window=self.window)
        mixed = rt.workspace.get("latent.out", tokens, self.out_width, rt.dtype)
        ops.head_linear(summed, self.kv_rank, self.w_expand, mixed, self.value_dim, heads,
                        gate=down[:, self.gate_column:] if self.gate else None)
        update = rt.workspace.get("mixer.update32", tokens, self.hidden_size, f32)
        return ops.linear(mixed, self.w_o, None, update)


register_part("mixer", "latent_attention", LatentAttention, replace=True)
