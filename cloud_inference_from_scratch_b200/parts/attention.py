"""Grouped-query causal attention over the paged cache.

Reference formulas: projections with bias, head-major split (src/cloud_engine/model.py:132-137);
rotary on q and k (attention.py:83-85); keys and values written to the pages before
attention so that a portion attends to itself through the cache (attention.py:193,225;
cache.py:398-425); per q head h the kv head h // (Hq/Hkv), keys 0..pos inclusive,
scale 1/sqrt(head_dim), float32 softmax (kernel.py:356-405; attention.py:88-112,129);
output projection without bias (model.py:128-130).

Here q, k and v come from ONE matrix product with the three weights stacked, the
rotation is fused with the write of k and v into the pages, and attention reads the
pages directly through the block table.  ``window`` > 0 limits a query at position p
to keys p-window+1..p.

Options beyond the reference, each a constant of the part so that any description may use it:

* ``value_dim``: value heads of a size of their own (the pages then keep keys and values in two
  tensors);
* ``qk_norm="projection"``: q and k are each divided by the root mean square of their whole
  projection (all heads together, before the split into heads) and multiplied by a stored gain
  vector of that size; keys are cached so;
* ``qk_norm="head"``: every q and k head is divided by its OWN root mean square and multiplied by a
  stored gain vector of a head's size that all heads share; keys are cached so;
* ``value_norm``: every value head is divided by its own root mean square (no gain) before it is
  cached;
* ``keep_first``: with a window, a query also sees the request's first ``keep_first`` keys (at their true
  positions), however far the window has moved on;
* ``gate``: the heads side by side are multiplied by ``sigmoid(W_g h)`` before the output projection
  (the gate's weight is stacked under q, k and v: one product);
* ``distance_penalty``: the score of query position i and key position j is lowered by
  ``r1_h * ln(1 + r2_h * (i - j))`` with two stored numbers per query head;
* ``sink``: the softmax denominator of every query head holds one more term ``exp(sink_h)``, a stored number
  per head that has no key and no value and is not scaled;
* ``projection_float32``: q, k and v leave their product as float32 and are not rounded before the norms and
  the rotation;
* ``position=None``: no rotation;
* ``names``: the tensor names, where a model stores them under others.

With any of these but the last two the layer runs product -> norms + rotation + cache write -> attention ->
output projection with the kernels of those options; scores, softmax, norms and angles are float32.  On that
path the rotation (after the norms) takes either pairing, a part of the head, blended frequencies and a
magnitude factor on cos and sin, all from the position part.
"""

from __future__ import annotations

import math

from ..config.spec import PartSpec
from .base import CacheSpec, Mixer, TensorSpec, build_part, register_part


class Attention(Mixer):
    def __init__(
        self,
        hidden_size: int,
        num_heads: int,
        num_kv_heads: int,
        head_dim: int,
        qkv_bias: bool,
        position: PartSpec | None,
        window: int = 0,
        scale: float | None = None,
        value_dim: int | None = None,
        qk_norm: str | None = None,
        value_norm: bool = False,
        distance_penalty: bool = False,
        norm_eps: float = 1e-6,
        names: dict[str, str] | None = None,
        keep_first: int = 0,
        gate: bool = False,
        sink: bool = False,
        projection_float32: bool = False,
    ) -> None:
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.hidden_size = int(hidden_size)
        self.num_heads = int(num_heads)
        self.num_kv_heads = int(num_kv_heads)
        self.head_dim = int(head_dim)
        self.qkv_bias = bool(qkv_bias)
        self.window = int(window)
        self.keep_first = int(keep_first) if self.window > 0 else 0
        if keep_first < 0:
            raise ValueError("keep_first must not be negative")
        self.gate = bool(gate)
        self.sink = bool(sink)
        self.projection_float32 = bool(projection_float32)
        self.position = build_part("position", position) if position is not None else None
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.scale *= float(getattr(self.position, "attention_factor", 1.0))
        self.q_width = self.num_heads * self.head_dim
        self.kv_width = self.num_kv_heads * self.head_dim
        self.value_dim = int(value_dim) if value_dim else self.head_dim
        self.v_width = self.num_kv_heads * self.value_dim
        self.out_width = self.num_heads * self.value_dim
        self.qkv_width = self.q_width + self.kv_width + self.v_width
        if qk_norm not in (None, "projection", "head"):
            raise ValueError(f"qk_norm must be None, 'projection' or 'head', got {qk_norm!r}")
        self.qk_norm = qk_norm
        self.value_norm = bool(value_norm)
        self.distance_penalty = bool(distance_penalty)
        self.norm_eps = float(norm_eps)
        # the options that the rotary kernels and the tensor-core attention kernels do not know
        self.general = bool(self.qk_norm or self.value_norm or self.distance_penalty
                            or self.value_dim != self.head_dim or self.keep_first or self.gate or self.sink
                            or self.projection_float32)
        if not self.general and (getattr(self.position, "magnitude", 1.0) != 1.0
                                 or getattr(self.position, "keep_pairing", False)):
            raise ValueError("the fused rotary kernels rotate without a magnitude factor and pair (j, j + R/2) only")
        if self.gate and self.qkv_bias:
            raise ValueError("the output gate is built for projections without biases")
        self.names = {key: key for key in ("q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight",
                                           "q_proj.bias", "k_proj.bias", "v_proj.bias", "q_norm", "k_norm",
                                           "r1", "r2", "gate", "sink")}
        self.names.update(names or {})
        self.tiled = False      # set at bind: whether prompt portions run on the tensor-core kernel

    @property
    def plan_key(self):
        if self.general and not self.tiled:      # its attention kernel walks the batch itself: no work lists
            return None
        return ("attention", self.num_heads // self.num_kv_heads)

    def plan(self, host, cache):
        """Work lists for this step's attention kernels, added to the step's metadata copy."""
        return self.runtime.ops.plan_attention(host, self.num_heads // self.num_kv_heads)

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(kv_heads=self.num_kv_heads, head_dim=self.head_dim, window=self.window,
                         value_dim=0 if self.value_dim == self.head_dim else self.value_dim,
                         keep_first=self.keep_first)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        n = self.names
        specs = {
            n["q_proj.weight"]: TensorSpec((self.q_width, self.hidden_size)),
            n["k_proj.weight"]: TensorSpec((self.kv_width, self.hidden_size)),
            n["v_proj.weight"]: TensorSpec((self.v_width, self.hidden_size)),
            n["o_proj.weight"]: TensorSpec((self.hidden_size, self.out_width)),
        }
        if self.qkv_bias:
            specs[n["q_proj.bias"]] = TensorSpec((self.q_width,), role="vector")
            specs[n["k_proj.bias"]] = TensorSpec((self.kv_width,), role="vector")
            specs[n["v_proj.bias"]] = TensorSpec((self.v_width,), role="vector")
        if self.qk_norm:
            per_head = self.qk_norm == "head"
            specs[n["q_norm"]] = TensorSpec((self.head_dim if per_head else self.q_width,), init="gain", role="vector")
            specs[n["k_norm"]] = TensorSpec((self.head_dim if per_head else self.kv_width,), init="gain", role="vector")
        if self.gate:
            specs[n["gate"]] = TensorSpec((self.out_width, self.hidden_size))
        if self.sink:
            specs[n["sink"]] = TensorSpec((self.num_heads,), role="vector")
        if self.distance_penalty:
            specs[n["r1"]] = TensorSpec((self.num_heads,), init="gain", role="vector")
            specs[n["r2"]] = TensorSpec((self.num_heads,), init="gain", role="vector")
        return specs

    def bind(self, tensors, runtime) -> None:
        import torch

        self.runtime = runtime
        ops = runtime.ops
        # With a rotary encoding whose sizes allow it, the q and k rows are kept in the paired
        # layout: a decode step then rotates and stores inside the projection's kernel, and the
        # separate rotary kernel (prompt portions) reads the same layout.
        rotary = self.position.rotary_dim if self.position is not None else 0
        self.paired = bool(self.position is not None and not self.general and getattr(ops, "can_pair_rotary", None)
                           and ops.can_pair_rotary(self.head_dim, rotary))

        # an encoding may want the elements of every q and k head stored in another order (its
        # pairs side by side for the kernels); scores do not change when q and k move together.  The kernel
        # of the general path rotates either pairing where the elements stand (gains of a q/k norm are stored
        # by element and stay where they are)
        order = None if self.general else getattr(self.position, "row_order", lambda: None)()

        def reorder(rows, heads):
            index = (torch.arange(heads).view(-1, 1) * self.head_dim + torch.tensor(order).view(1, -1)).reshape(-1)
            return rows.index_select(0, index.to(rows.device)).contiguous()

        def stacked(suffix):
            q, k, v = (tensors[self.names[f"{name}_proj.{suffix}"]] for name in "qkv")
            if order is not None:
                q, k = reorder(q, self.num_heads), reorder(k, self.num_kv_heads)
            if self.paired:
                q = ops.pair_rotary_rows(q, self.num_heads, self.head_dim, rotary)
                k = ops.pair_rotary_rows(k, self.num_kv_heads, self.head_dim, rotary)
            if self.gate and suffix == "weight":
                return torch.cat([q, k, v, tensors[self.names["gate"]]]).contiguous()
            return torch.cat([q, k, v]).contiguous()

        self.w_qkv = ops.prepare_weight(stacked("weight"))
        self.b_qkv = stacked("bias") if self.qkv_bias else None
        self.w_o = runtime.ops.prepare_weight(tensors[self.names["o_proj.weight"]])
        self.rotation = None
        if self.position is not None:
            self.position.bind({}, runtime)
            if self.general:
                from types import SimpleNamespace

                inv_freq = torch.tensor(self.position.frequencies(), dtype=torch.float64).to(torch.float32)
                self.rotation = SimpleNamespace(
                    inv_freq=inv_freq.to(runtime.device).contiguous(), magnitude=self.position.magnitude,
                    interleaved=self.position.pairing == "interleaved", dims=self.position.rotary_dim)
        self.sinks = tensors[self.names["sink"]].contiguous() if self.sink else None
        self.q_gain = tensors[self.names["q_norm"]].contiguous() if self.qk_norm else None
        self.k_gain = tensors[self.names["k_norm"]].contiguous() if self.qk_norm else None
        self.distance = ((tensors[self.names["r1"]].contiguous(), tensors[self.names["r2"]].contiguous())
                         if self.distance_penalty else None)
        # the tensor-core kernels take bfloat16 heads of a multiple of 16 elements, values as large as keys
        self.tiled = bool(self.value_dim == self.head_dim and self.head_dim % 16 == 0 and self.head_dim <= 256
                          and runtime.dtype_name == "bfloat16")
        if not self.general or self.tiled:
            runtime.ops.require_attention(self.head_dim)

    takes_normed_input = True   # x goes to ops.linear only
    kernels_through_ops = True  # every kernel of this part is a method of ``Ops``: a decode step may be recorded

    def forward_general(self, x, ctx, binding):
        """The layer with q/k norm, value norm, rotation after the norms, distance penalty, a sink or a value size of
        its own."""
        import torch

        rt = self.runtime
        tokens = x.shape[0]
        kv = binding.kv
        width = self.qkv_width + (self.out_width if self.gate else 0)
        if self.projection_float32:
            qkv = rt.workspace.get("attention.qkv32", tokens, width, torch.float32)
            qkv = rt.ops.linear(x, self.w_qkv, self.b_qkv, qkv)
        else:
            qkv = rt.workspace.get("attention.qkv", tokens, width, rt.dtype)
            qkv = rt.ops.linear(x, self.w_qkv, self.b_qkv, qkv, tag="attention.qkv", defer_bias=True)
        q = rt.workspace.get("attention.q", tokens, self.q_width, rt.dtype)
        rt.ops.norm_kv_write(qkv, ctx, kv, self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim,
                             self.q_gain, self.k_gain, self.value_norm, self.norm_eps, q,
                             write_cache=binding.owns_cache, per_head=self.qk_norm == "head",
                             rotation=self.rotation)
        mixed = rt.workspace.get("attention.out", tokens, self.out_width, rt.dtype)
        rt.ops.attention_penalised(q, mixed, ctx, kv, self.num_heads, self.num_kv_heads, self.head_dim,
                                   self.value_dim, self.scale, self.window, self.distance,
                                   keep_first=self.keep_first, sinks=self.sinks)
        if self.gate:
            if self.projection_float32:
                raise ValueError("the output gate reads a projection of the compute dtype")
            rt.ops.sigmoid_gate(mixed, qkv[:, self.qkv_width:])
        update = rt.workspace.get("mixer.update32", tokens, self.hidden_size, torch.float32)
        return rt.ops.linear(mixed, self.w_o, None, update)

    def forward(self, x, ctx, binding):
        if self.general:
            return self.forward_general(x, ctx, binding)
        rt = self.runtime
        tokens = x.shape[0]
        kv = binding.kv
        q_buffer = rt.workspace.get("attention.q", tokens, self.q_width, rt.dtype)
        q = None
        if self.paired:   # a few decode tokens: projection, rotation and cache write in one kernel
            q = rt.ops.qkv_rope(x, self.w_qkv, self.b_qkv, ctx, kv, self.position, self.num_heads,
                                self.num_kv_heads, self.head_dim, binding.owns_cache, q_buffer)
        if q is None:
            qkv = rt.workspace.get("attention.qkv", tokens, self.qkv_width, rt.dtype)
            # for few tokens the projection may come back as partial sums that the next kernel adds up
            qkv = rt.ops.linear(x, self.w_qkv, self.b_qkv, qkv, allow_partials=True, tag="attention.qkv",
                                defer_bias=True)
            q = rt.ops.rope_kv_write(
                qkv, ctx, kv, self.position, self.num_heads, self.num_kv_heads, self.head_dim,
                write_cache=binding.owns_cache, q_buffer=q_buffer, paired=self.paired,
            )
        mixed = rt.workspace.get("attention.out", tokens, self.q_width, rt.dtype)
        rt.ops.attention(
            q, mixed, ctx, kv, self.num_heads, self.num_kv_heads, self.head_dim,
            self.scale, self.window,
        )
        update = rt.workspace.get("mixer.update", tokens, self.hidden_size, rt.dtype)
        return rt.ops.linear(mixed, self.w_o, None, update, allow_partials=True, tag="mixer.update",
                             residual=getattr(ctx, "residual_sink", None))


register_part("mixer", "attention", Attention, replace=True)
