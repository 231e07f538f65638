"""RMSNorm over the float32 residual stream, fused with the pending residual add.

Formula (src/cloud_engine/attention.py:52-57): ``w * (x * rsqrt(mean(x^2) + eps))`` with
the statistics in float32.  The reference keeps the residual in float16 and adds in
float16 (model.py:217-220); here the stream is float32, the add is a 32-bit sum inside
the same kernel, and the result is rounded once to the compute dtype.
"""

from __future__ import annotations

from ..lazy import Accumulated, NormedInput
from .base import Norm, TensorSpec, register_part


class RMSNorm(Norm):
    """``gain_offset``: the stored vector w lies around zero and the gain is ``gain_offset + w`` (formed
    once, in float32, when the tensors are bound).  ``name``: the tensor's name after the part's prefix."""

    def __init__(self, hidden_size: int, eps: float, gain_offset: float = 0.0, name: str = "weight") -> None:
        self.hidden_size = int(hidden_size)
        self.eps = float(eps)
        self.gain_offset = float(gain_offset)
        self.name = str(name)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        init = "gain" if self.gain_offset == 0.0 else "normal"
        return {self.name: TensorSpec((self.hidden_size,), init=init, role="vector")}

    def bind(self, tensors, runtime) -> None:
        self.runtime = runtime
        self.weight = tensors[self.name]
        if self.gain_offset != 0.0:
            self.weight = (self.weight.float() + self.gain_offset).contiguous()

    accepts_accumulated = True   # ``update`` may be an ``Accumulated``: the sum is already in the stream
    kernels_through_ops = True  # every kernel of this part is a method of ``Ops``: a decode step may be recorded

    def forward(self, residual, update, ctx, rows=None):
        rt = self.runtime
        count = residual.shape[0] if rows is None else rows.shape[0]
        out = rt.workspace.get("norm.out" if rows is None else "norm.rows", count,
                               self.hidden_size, rt.dtype, per_request=rows is not None)
        rt.ops.add_rmsnorm(residual, update, self.weight, self.eps, out, rows)
        return out

    @property
    def lazy_gain(self):
        """The gain vector a projection may pre-multiply the new residual rows with for this norm
        (see ``forward_lazy``)."""
        return self.weight

    def forward_lazy(self, residual, update, ctx):
        """For a consumer that finishes the norm itself (``takes_normed_input``): when the sum is
        already in the stream, scaled by this norm's gain, and its sums of squares are known,
        nothing runs here."""
        if isinstance(update, Accumulated) and update.scaled is not None and update.gain is self.weight:
            return NormedInput(update, self.eps, materialize=lambda: self.forward(residual, None, ctx))
        return self.forward(residual, update, ctx)


register_part("norm", "rmsnorm", RMSNorm, replace=True)


class LayerNorm(Norm):
    """Layer norm with gain and bias over the float32 stream, fused with the pending residual add:
    ``gain * (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) + bias``, statistics in float32, one rounding.
    ``update_scale``: the pending update is multiplied by this constant as it is added to the stream (a model
    that scales every sublayer's result).  ``names``: the tensors' names after the part's prefix (``weight``,
    ``bias``); ``bias=False``: no bias tensor."""

    def __init__(self, hidden_size: int, eps: float, update_scale: float = 1.0, bias: bool = True,
                 names: dict[str, str] | None = None) -> None:
        self.hidden_size = int(hidden_size)
        self.eps = float(eps)
        self.update_scale = float(update_scale)
        self.has_bias = bool(bias)
        self.names = dict(weight="weight", bias="bias")
        self.names.update(names or {})

    def tensor_specs(self) -> dict[str, TensorSpec]:
        specs = {self.names["weight"]: TensorSpec((self.hidden_size,), init="gain", role="vector")}
        if self.has_bias:
            specs[self.names["bias"]] = TensorSpec((self.hidden_size,), role="vector")
        return specs

    def bind(self, tensors, runtime) -> None:
        self.runtime = runtime
        self.weight = tensors[self.names["weight"]].contiguous()
        self.bias = tensors[self.names["bias"]].contiguous() if self.has_bias else None

    kernels_through_ops = True

    def forward(self, residual, update, ctx, rows=None):
        rt = self.runtime
        count = residual.shape[0] if rows is None else rows.shape[0]
        out = rt.workspace.get("norm.out" if rows is None else "norm.rows", count,
                               self.hidden_size, rt.dtype, per_request=rows is not None)
        rt.ops.add_layernorm(residual, update, self.weight, self.bias, self.eps, out, rows,
                             update_scale=self.update_scale)
        return out


register_part("norm", "layernorm", LayerNorm, replace=True)


class StreamRMSNorm(Norm):
    """RMS norm of what a sublayer reads from ``streams`` side-by-side copies of the residual
    stream (``residual``: float32 [T, streams * H]; one stream is the ordinary case):
    ``gain * u / sqrt(mean(u^2) + eps)`` with ``u = sum_t read[t] * stream_t``.  The gain is a
    vector [H] or, with ``single_gain``, one number for all coordinates (stored as a tensor without
    axes).  A pending ``StreamUpdate`` (or a plain tensor: the residual add) is applied to the
    streams first, in the same kernel, in float32."""

    def __init__(self, hidden_size: int, eps: float, single_gain: bool = False) -> None:
        self.hidden_size = int(hidden_size)
        self.eps = float(eps)
        self.single_gain = bool(single_gain)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        if self.single_gain:
            return {"": TensorSpec((), init="gain", role="vector")}
        return {"weight": TensorSpec((self.hidden_size,), init="gain", role="vector")}

    def bind(self, tensors, runtime) -> None:
        self.runtime = runtime
        self.weight = tensors["" if self.single_gain else "weight"].reshape(-1).contiguous()

    def forward(self, residual, update, ctx, rows=None, read=None):
        rt = self.runtime
        streams = residual.shape[1] // self.hidden_size
        count = residual.shape[0] if rows is None else rows.shape[0]
        out = rt.workspace.get("norm.out" if rows is None else "norm.rows", count,
                               self.hidden_size, rt.dtype, per_request=rows is not None)
        rt.ops.stream_norm(residual, streams, update, read, self.weight, self.eps, out, rows)
        return out


register_part("norm", "stream_rmsnorm", StreamRMSNorm, replace=True)
