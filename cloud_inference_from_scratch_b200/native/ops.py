"""Python face of the CUDA kernels: one method per kernel family, bound to a device and a dtype.

Every method launches hand-written sm_100a code from ``csrc/`` on the current CUDA stream
through a C interface (ctypes); nothing here computes on the host and there is no fallback
when a library cannot be built or the device is not a CUDA device.  Which kernel a call
reaches is decided by sizes only (for example: the tensor-core attention kernels take head
sizes that are multiples of 16 up to 256, other shapes go to the generic kernel); a size no
kernel takes raises.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_void_p
from typing import Any

from ..lazy import Accumulated, GateUpWeight, NormedInput, Partials, ResidualSink, StreamUpdate  # noqa: F401  (re-exported)
from .build import load_library

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def _ptr(tensor: Any) -> int | None:
    return None if tensor is None else tensor.data_ptr()


# More rows than this go to the tile kernels (tcgen05 or the library).  The streaming kernel
# multiplies with mma.sync, 8 tokens an instruction: built for 32 and 64 rows it was bound by that
# tensor path (the gate/up product of 64 tokens took 30 us against the library's 17) and its
# epilogues, which finish a token row per warp, by the number of rows.
STREAM_MAX_ROWS = 16
# Up to this many rows a projection adds itself into the residual stream, or rotates and stores
# q/k/v (cluster epilogues of the streaming kernel): every row count that kernel takes.
FUSED_RESIDUAL_MAX_ROWS = STREAM_MAX_ROWS


class _Lib:
    """A loaded library whose entry points return 0 or set ``cie_last_error``."""

    def __init__(self, handle: ctypes.CDLL) -> None:
        self.handle = handle
        handle.cie_last_error.restype = ctypes.c_char_p

    def function(self, name: str, argtypes: list[Any]):
        fn = getattr(self.handle, name)
        fn.argtypes = argtypes
        fn.restype = c_int
        last_error = self.handle.cie_last_error

        def call(*args: Any) -> None:
            if fn(*args) != 0:
                raise KernelError(last_error().decode(errors="replace"))

        return call


class Ops:
    def __init__(self, device: Any, dtype: Any, gemm: str | None = None) -> None:
        import torch

        self.torch = torch
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise KernelError(
                f"this engine runs on a CUDA device (sm_100a) only; got device {self.device}"
            )
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device is available; there is no CPU path")
        if dtype not in (torch.float32, torch.bfloat16):
            raise KernelError(f"compute dtype must be float32 or bfloat16, got {dtype}")
        self.dtype = dtype
        self.code = F32 if dtype == torch.float32 else BF16
        self.gemm_mode = gemm or ("simt" if self.code == F32 else os.environ.get("CIE_GEMM", "cublas"))
        if self.code == F32 and self.gemm_mode != "simt":
            raise KernelError("the 32-bit path multiplies on the CUDA cores only (gemm='simt')")
        if self.gemm_mode not in ("simt", "tensor", "cublas"):
            raise KernelError(f"unknown gemm mode {self.gemm_mode!r}")
        self.error_word = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.launches = 0
        self.max_rows = 0             # most tokens of a step, if the runtime knows (0: not known)
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count

        v, i, f = c_void_p, c_int, c_float
        ew = _Lib(load_library("elementwise.cu"))
        self._embedding = ew.function("cie_embedding", [v, v, v, i, i, i, f, i, v, v])
        ll = ctypes.c_longlong
        self._shape_logits = ew.function("cie_shape_logits", [v, ll, f, f, v])
        self._add_rmsnorm = ew.function("cie_add_rmsnorm", [v, v, i, ll, v, v, v, v, i, i, f, i, v])
        self._rope_kv_write = ew.function(
            "cie_rope_kv_write",
            [v, i, ll, v, v, i, v, v, v, i, i, v, v, v, i, i, i, i, i, i, i, i, i, v, v],
        )
        self._silu_mul = ew.function("cie_silu_mul", [v, v, i, i, i, i, v])
        self._gated_act = ew.function("cie_gated_act", [v, i, v, v, i, i, f, f, f, i, v])
        self._embedding_wave = ew.function("cie_embedding_wave", [v, v, v, v, v, i, i, i, f, i, v, v])
        self._add_rows = ew.function("cie_add_rows", [v, v, i, ll, f, v, v, i, i, v])
        self._add_layernorm = ew.function("cie_add_layernorm", [v, v, i, ll, f, v, v, v, v, i, i, f, i, v])
        self._glu_act = ew.function("cie_glu_act", [v, i, v, i, i, i, i, v])
        self._unary_act = ew.function("cie_unary_act", [v, v, ll, i, i, v])
        self._sigmoid_gate = ew.function("cie_sigmoid_gate", [v, v, i, i, i, i, v])
        self._scaled_sum = ew.function("cie_scaled_sum", [v, v, f, f, ll, v])
        gs = _Lib(load_library("gemm_simt.cu"))
        self._gemm_simt = gs.function("cie_gemm_simt", [v, v, v, v, i, i, i, i, i, i, v])
        ag = _Lib(load_library("attention_generic.cu"))
        self._attention_generic_sink = ag.function(
            "cie_attention_generic_sink",
            [v, i, v, i, v, v, v, v, v, i, i, i, i, i, i, i, i, f, i, v, v, i, v, v, i, v, i, v, v],
        )
        self._group_share_floats = int(ag.handle.cie_attention_group_share_floats())
        self._group_tickets = None
        # libraries that only some models need are built and loaded when a part first asks for them
        self._streams_lib = None
        self._lightning_lib = None
        self._latent_lib = None
        self._delta_lib = None
        self._gla_lib = None
        self._recurrent_lib = None
        self._moe_lib = None
        self._sample = None   # sampling.cu is built when something is first sampled
        self._tensor_gemm = None
        self._fold_gemm_held = None
        # from this many rows on, projections fold the residual add / the norm / the activation
        # into the persistent tcgen05 kernel instead of running library products and separate
        # kernels (0: never)
        self.fold_rows = int(os.environ.get("CIE_FOLD_ROWS", "0"))
        # which products of 17 to 256 rows go to the weight-streaming tcgen05 kernel instead of the
        # library: "0" none, "gate_up" the gate/up product with its activation (the default: 64
        # requests decode in 3.23 instead of 3.31 ms a step, 32 in 2.80 instead of 2.88; a prompt in
        # 256-token portions takes 24.7 instead of 25.0 ms), "all" every product (for measurements)
        self.skinny_products = os.environ.get("CIE_SKINNY", "gate_up")
        if self.skinny_products == "0":
            self.skinny_products = ""
        self._skinny = None
        self._tensor_attention: dict[int, Any] = {}
        self._gemm_stream = None
        self._gemm_stream_ex = None
        self._gemm_stream_rope = None
        self.fuse_norm = False
        self._partial_buffers: dict[str, Any] = {}
        self.scratch_frozen = False
        self.scratch_generation = 0   # counts scratch buffers replaced by larger ones
        self.program = None           # recorder of decode programs (native/program.py), made on first use
        if self.code == BF16 and self.gemm_mode != "simt":
            st = _Lib(load_library("gemm_stream.cu"))
            self._gemm_stream = st.function("cie_gemm_stream", [v, v, v, v, i, i, i, i, i, i, v, v])
            self._gemm_stream_ex = st.function(
                "cie_gemm_stream_ex", [v, v, i, f, v, v, v, v, v, v, v, i, i, i, i, i, i, i, v, v])
            self._gemm_stream_rope = st.function(
                "cie_gemm_stream_rope",
                [v, v, i, f, v, v, v, i, v, v, v, i, i, v, v, v, i, i, i, i, i, i, i, i, i, v, v])
            self.fuse_norm = os.environ.get("CIE_FUSE_NORM", "1") != "0"
        if self.code == BF16 and self.gemm_mode == "tensor":
            from .tensor_gemm import TensorGemm

            self._tensor_gemm = TensorGemm(self)

    # ------------------------------------------------------------------ helpers
    @property
    def stream(self) -> int:
        return self.torch.cuda.current_stream(self.device).cuda_stream

    # ------------------------------------------------------------------ decode programs
    def begin_program(self, ctx: Any) -> bool:
        """Starts recording the streaming products and the decode attention of this step instead of
        launching them (see native/program.py), if the step is one the persistent kernel takes: a
        bfloat16 step of at most 16 tokens, each the single next token of its request.  Everything
        else that runs through ``Ops`` meanwhile flushes what was recorded first.  ``end_program``
        runs the rest."""
        from . import program

        if (self.code != BF16 or self._gemm_stream is None or not self.fuse_norm or not program.enabled()
                or ctx.num_tokens > program.MAX_ROWS or ctx.num_tokens != ctx.num_requests
                or ctx.num_single != ctx.num_requests):
            return False
        if self.program is None:
            self.program = program.DecodeProgram(self)
        self.program.begin()
        return True

    def end_program(self) -> None:
        if self.program is not None:
            self.program.end()

    def _flush(self) -> None:
        """Before a kernel that is not recorded: what was recorded so far runs first."""
        if self.program is not None and self.program.calls:
            self.program.flush()

    @property
    def recording(self) -> bool:
        return self.program is not None and self.program.recording

    def _code_of(self, tensor: Any) -> int:
        if tensor.dtype == self.torch.float32:
            return F32
        if tensor.dtype == self.torch.bfloat16:
            return BF16
        raise KernelError(f"unsupported tensor dtype {tensor.dtype}")

    def prepare_weight(self, weight: Any) -> Any:
        """A matrix [N, K] as the matrix products want it: compute dtype, contiguous."""
        return weight.to(device=self.device, dtype=self.dtype).contiguous()

    def attention_penalised(self, q: Any, out: Any, ctx: Any, kv: Any, q_heads: int, kv_heads: int,
                            head_dim: int, value_dim: int, scale: float, window: int, distance: Any,
                            keep_first: int = 0, sinks: Any = None) -> None:
        """Attention with the options of ``attention_generic`` (a value size of its own, a distance
        penalty, kept first keys), softmax weights float32 throughout.  bfloat16 prompt portions whose value heads have
        the size of the key heads run on the tensor cores (mma.sync; the weights enter the value
        product as two bfloat16 terms); single tokens, the 32-bit path and every other shape run on
        the kernel that takes one warp per (token, head)."""
        fast = (self._tensor_attention.get(head_dim)
                if value_dim == head_dim and self.code == BF16 else None)
        singles = ctx.num_single
        if (fast is None or singles == ctx.num_requests or q.shape[1] % 8 or out.shape[1] % 8
                or os.environ.get("CIE_PENALISED_TC", "1") == "0"):
            self.attention_generic(q, out, ctx, kv, q_heads, kv_heads, head_dim, scale, window,
                                   value_dim=value_dim, distance=distance,
                                   few_tokens=singles == ctx.num_requests, keep_first=keep_first, sinks=sinks)
            return
        if singles:     # the leading rows of a mixed step are its single tokens
            self.attention_generic(q[:singles], out[:singles], ctx, kv, q_heads, kv_heads, head_dim, scale,
                                   window, value_dim=value_dim, distance=distance, few_tokens=True,
                                   keep_first=keep_first, sinks=sinks)
        plan = ctx.extras.get(("attention", q_heads // kv_heads)) or None
        fast.run_portions(q, out, ctx, kv, q_heads, kv_heads, scale, window, plan, distance, True,
                          keep_first=keep_first, sinks=sinks)

    def require_attention(self, head_dim: int) -> None:
        """Builds, at model set-up, the attention kernels a head size needs."""
        if self.code == BF16:
            from . import tensor_attention

            if head_dim not in self._tensor_attention and tensor_attention.supports(head_dim):
                self._tensor_attention[head_dim] = tensor_attention.TensorAttention(self, head_dim)

    def plan_attention(self, host: Any, group: int) -> dict[str, Any]:
        """Integer work lists the attention kernels want in a step's metadata (may be empty)."""
        if self.code != BF16 or host.num_single == host.num_requests:
            return {}
        from . import tensor_attention

        return tensor_attention.plan_tiles(host.query_lens, group, skip=host.num_single)

    def check_errors(self) -> None:
        """Reads the device error word (synchronises) and raises if a kernel flagged a fault."""
        word = int(self.error_word.item())
        if word:
            self.error_word.zero_()
            faults = [name for bit, name in ((1, "a token had no valid cache page"),
                                              (2, "a token id was outside the vocabulary"),
                                              (4, "a request index was outside the batch"),
                                              (8, "a bounded wait for a tensor copy or a tensor-core "
                                                  "product ran out"))
                      if word & bit]
            if word & ~15:
                faults.append(f"unknown bits {word & ~15:#x}")
            raise KernelError("device error word set: " + "; ".join(faults))

    # ------------------------------------------------------------------ kernels
    def embedding(self, token_ids: Any, table: Any, residual: Any, scale: float = 1.0,
                  positions: Any = None, position_table: Any = None, streams: int = 1,
                  wave: Any = None) -> None:
        """residual[t] = table[token_ids[t]] * scale (+ position_table[positions[t]]), float32, in each
        of ``streams`` side-by-side copies ([T, streams * H]).  ``wave``: float32 frequencies [ceil(H / 2)];
        then sin(p * wave[i]) is added to entry 2i and cos(p * wave[i]) to entry 2i + 1, p the position."""
        self._flush()
        tokens = residual.shape[0]
        hidden = residual.shape[1] // streams
        self.launches += 1
        if wave is not None:
            if position_table is not None or streams > 1:
                raise KernelError("embedding: a sinusoid goes with one stream and no learned position vector")
            self._embedding_wave(_ptr(token_ids), _ptr(positions), _ptr(table), _ptr(wave), _ptr(residual), tokens,
                                 hidden, table.shape[0], float(scale), self._code_of(table), _ptr(self.error_word),
                                 self.stream)
            return
        if position_table is not None or streams > 1:
            self._load_streams()
            self._embedding_streams(_ptr(token_ids), _ptr(positions), _ptr(table), _ptr(position_table),
                                    _ptr(residual), tokens, hidden, table.shape[0],
                                    0 if position_table is None else position_table.shape[0], streams,
                                    float(scale), self._code_of(table), _ptr(self.error_word), self.stream)
            return
        self._embedding(_ptr(token_ids), _ptr(table), _ptr(residual), tokens, hidden,
                        table.shape[0], float(scale), self._code_of(table), _ptr(self.error_word), self.stream)

    def shape_logits(self, logits: Any, scale: float = 1.0, softcap: float = 0.0) -> None:
        """logits = softcap * tanh(logits * scale / softcap) (or logits * scale), float32, in place."""
        self._flush()
        if scale == 1.0 and softcap == 0.0:
            return
        self.launches += 1
        self._shape_logits(_ptr(logits), logits.numel(), float(scale), float(softcap), self.stream)

    def residual_sink(self, residual: Any) -> "ResidualSink":
        """The float32 stream as a target that projections may add themselves into."""
        return ResidualSink(residual)

    def add_rmsnorm(self, residual: Any, update: Any, gain: Any, eps: float, out: Any,
                    rows: Any = None) -> None:
        """``update``: None, a tensor [T, H] of the compute dtype, or ``Partials``."""
        self._flush()
        count, hidden = out.shape
        self.launches += 1
        if isinstance(update, Accumulated):
            update = None   # its kernel has added it already
        if isinstance(update, Partials) and update.splits == 0:
            update = self.resolve(update, None)
        if (update is not None and not isinstance(update, Partials) and update.dtype == self.torch.float32
                and self.code != F32):
            # a float32 result in a bfloat16 run: one float32 term still to be added
            update = Partials(update, 1, update.shape[0], update.shape[1], None)
        if isinstance(update, Partials):
            self._add_rmsnorm(_ptr(residual), _ptr(update.data), update.splits,
                              update.stride, _ptr(update.bias), _ptr(gain), _ptr(out),
                              _ptr(rows), count, hidden, eps, self._code_of(out), self.stream)
        else:
            self._add_rmsnorm(_ptr(residual), _ptr(update), 0, 0, None, _ptr(gain), _ptr(out),
                              _ptr(rows), count, hidden, eps, self._code_of(out), self.stream)

    def add_layernorm(self, residual: Any, update: Any, gain: Any, bias: Any, eps: float, out: Any,
                      rows: Any = None, update_scale: float = 1.0) -> None:
        """The layer norm with gain and bias of ``residual + update_scale * update`` (the sum stays in the float32
        stream unless ``rows`` selects rows): ``update`` is None, a tensor [T, H] of the compute dtype or of
        float32, or ``Partials`` without a pending bias."""
        self._flush()
        count, hidden = out.shape
        self.launches += 1
        if isinstance(update, Accumulated):
            raise KernelError("add_layernorm: an update that is already in the stream cannot be scaled")
        if isinstance(update, Partials) and (update.splits == 0 or update.bias is not None):
            update = self.resolve(update, self.torch.empty(update.shape, dtype=self.torch.float32, device=self.device))
        if (update is not None and not isinstance(update, Partials) and update.dtype == self.torch.float32
                and self.code != F32):
            update = Partials(update, 1, update.shape[0], update.shape[1], None)
        if isinstance(update, Partials):
            self._add_layernorm(_ptr(residual), _ptr(update.data), update.splits, update.stride, float(update_scale),
                                _ptr(gain), _ptr(bias), _ptr(out), _ptr(rows), count, hidden, float(eps),
                                self._code_of(out), self.stream)
        else:
            self._add_layernorm(_ptr(residual), _ptr(update), 0, 0, float(update_scale), _ptr(gain), _ptr(bias),
                                _ptr(out), _ptr(rows), count, hidden, float(eps), self._code_of(out), self.stream)

    def add_rows(self, residual: Any, update: Any, vector: Any, base: Any = None, scale: float = 1.0) -> None:
        """residual[t] += vector + base[t] + scale * update, float32 in place: the stream as a run of layers that
        starts with a learned offset finds it.  ``vector`` (float32 [H]) and ``base`` (float32 [T, H]) may be None;
        ``update``: None, an ``Accumulated`` (already added; only with scale 1), or float32 terms as ``Partials``."""
        self._flush()
        if isinstance(update, Accumulated):
            if scale != 1.0:
                raise KernelError("add_rows: an update that is already in the stream cannot be scaled")
            update = None
        if update is not None and not isinstance(update, Partials):
            if update.dtype != self.torch.float32:
                update = update.float()
            update = Partials(update.contiguous(), 1, update.shape[0], update.shape[1], None)
        if isinstance(update, Partials) and (update.splits == 0 or update.bias is not None):
            data = self.resolve(update, self.torch.empty(update.shape, dtype=self.torch.float32, device=self.device))
            update = Partials(data.float().contiguous(), 1, update.rows, update.width, None)
        tokens, hidden = residual.shape
        self.launches += 1
        if update is None:
            self._add_rows(_ptr(residual), None, 0, 0, 1.0, _ptr(base), _ptr(vector), tokens, hidden, self.stream)
        else:
            self._add_rows(_ptr(residual), _ptr(update.data), update.splits, update.stride, float(scale), _ptr(base),
                           _ptr(vector), tokens, hidden, self.stream)

    def glu_act(self, gate_up: Any, out: Any, kind: str = "silu") -> None:
        """out = act(gate) * up for contiguous ``gate_up`` [T, 2 * I] = [gate | up] (float32 or the compute dtype), in
        float32, rounded once; ``kind``: "silu" or "gelu_tanh"."""
        self._flush()
        kinds = {"silu": 0, "gelu_tanh": 1}
        if kind not in kinds:
            raise KernelError(f"glu_act: unknown activation {kind!r} (known: {sorted(kinds)})")
        self.launches += 1
        self._glu_act(_ptr(gate_up), self._code_of(gate_up), _ptr(out), out.shape[0], out.shape[1], kinds[kind],
                      self._code_of(out), self.stream)

    def unary_act(self, x: Any, out: Any, kind: str = "relu2") -> None:
        """out = act(x) for contiguous float32 ``x``, rounded once; "relu2": the square of relu."""
        self._flush()
        kinds = {"relu2": 0}
        if kind not in kinds:
            raise KernelError(f"unary_act: unknown activation {kind!r} (known: {sorted(kinds)})")
        self.launches += 1
        self._unary_act(_ptr(x), _ptr(out), x.numel(), kinds[kind], self._code_of(out), self.stream)

    def sigmoid_gate(self, x: Any, gate: Any) -> None:
        """x *= sigmoid(gate) in place; ``gate`` is a view of columns of a wider row of the same dtype."""
        self._flush()
        self.launches += 1
        self._sigmoid_gate(_ptr(x), _ptr(gate), gate.stride(0), x.shape[0], x.shape[1], self._code_of(x), self.stream)

    def scaled_sum(self, out: Any, a: Any, alpha: float, accumulate: bool) -> None:
        """out = alpha * a, or out += alpha * a; contiguous float32."""
        self._flush()
        self.launches += 1
        self._scaled_sum(_ptr(out), _ptr(a), float(alpha), 1.0 if accumulate else 0.0, a.numel(), self.stream)

    # ------------------------------------------------------------------ recurrent mixers with one gate a head
    def _load_recurrent(self) -> None:
        if self._recurrent_lib is None:
            v, i, f, ll = c_void_p, c_int, c_float, ctypes.c_longlong
            lib = _Lib(load_library("recurrent.cu"))
            self._mlstm_scan = lib.function(
                "cie_mlstm_scan", [v, i, i, i, i, i, i, v, v, f, f, v, i, v, ll, v, v, v, i, i, i, i, i, v, v])
            self._gated_delta_scan = lib.function(
                "cie_gated_delta_scan", [v, i, i, i, i, v, i, i, i, v, v, f, v, i, v, ll, v, v, v, i, i, i, i, i, i, v, v])
            self._short_conv = lib.function("cie_short_conv", [v, i, v, i, v, ll, v, i, v, v, v, v, i, i, i, i, v, v])
            self._head_norm_gate = lib.function("cie_head_norm_gate", [v, i, v, v, i, v, i, i, v, i, i, i, i, f, i, v])
            self._mlstm_stream = lib.function(
                "cie_mlstm_stream", [v, i, i, i, i, i, i, v, v, f, f, v, v, i, v, v, ll, v, v, v, i, i, i, i, i, i, v, v])
            self._gated_delta_stream = lib.function(
                "cie_gated_delta_stream",
                [v, i, i, i, i, v, i, i, i, v, v, f, v, v, i, v, ll, v, v, v, i, i, i, i, i, i, i, v, v])
            lib.handle.cie_recurrent_stream_floats.restype = ctypes.c_longlong
            self._recurrent_stream_floats = lib.handle.cie_recurrent_stream_floats
            self.stream_max_dim = int(lib.handle.cie_stream_max_dim())
            self._mlstm_chunked = lib.function(
                "cie_mlstm_chunked", [v, i, i, i, i, i, i, v, v, f, f, v, v, i, v, ll, v, v, v, v, v, v, i, i, i, i, i, i, i, v, v])
            self._gated_delta_chunked = lib.function(
                "cie_gated_delta_chunked",
                [v, i, i, i, i, v, i, i, i, v, v, f, v, v, i, v, ll, v, v, v, v, v, i, i, i, i, i, i, i, i, v, v])
            lib.handle.cie_gated_delta_chunk_floats.restype = ctypes.c_longlong
            self._gated_delta_chunk_floats = lib.handle.cie_gated_delta_chunk_floats
            lib.handle.cie_mlstm_chunk_floats.restype = ctypes.c_longlong
            self._mlstm_chunk_floats = lib.handle.cie_mlstm_chunk_floats
            self.mlstm_chunk_tokens = int(lib.handle.cie_mlstm_chunk_tokens())
            self.mlstm_chunk_max_dim = int(lib.handle.cie_mlstm_chunk_max_dim())
            self.scan_max_dim = int(lib.handle.cie_scan_max_dim())
            self.conv_max_taps = int(lib.handle.cie_conv_max_taps())
            self.normaliser_columns = int(lib.handle.cie_normaliser_columns())
            self._recurrent_lib = lib

    def require_recurrent(self) -> tuple[int, int]:
        """Builds, at model set-up, the kernels of the recurrent mixers with one gate a head; returns the largest
        key size and the longest short convolution they take."""
        self._load_recurrent()
        return self.scan_max_dim, self.conv_max_taps

    def _streams(self, tokens: int, ctx: Any, dim: int) -> bool:
        """Whether a step runs the recurrences as prepare + stream: prompt portions (eight tokens a request or
        more on average) and keys the stream kernel's registers hold."""
        return (tokens >= 8 * ctx.num_requests and dim <= self.stream_max_dim
                and os.environ.get("CIE_RECURRENT_STREAM", "1") != "0")

    def plan_memory_chunks(self, host: Any) -> dict[str, Any]:
        """Work lists of the matrix memory's chunked form for a step that holds prompt portions (first token
        row and token count of every chunk; where every request's chunks start).  A step of single tokens
        needs none."""
        if host.num_single == host.num_requests:
            return {}
        self._load_recurrent()
        return self._plan_chunks(host, self.mlstm_chunk_tokens)

    def _stream_scratch(self, tokens: int, heads: int, dim: int, vdim: int, memory: bool) -> Any:
        floats = self._recurrent_stream_floats
        return self.scratch(f"recurrent.packed.{heads}x{dim}x{vdim}.{int(memory)}",
                            int(floats(tokens, heads, dim, vdim, int(memory))),
                            reserve=int(floats(max(tokens, self.max_rows), heads, dim, vdim, int(memory))))

    def mlstm_scan(self, proj: Any, offsets: tuple[int, int, int, int, int], input_bias: Any, forget_bias: Any,
                   cap: float, q_scale: float, out: Any, state: Any, ctx: Any, heads: int, dim: int, vdim: int,
                   plan: dict[str, Any] | None = None) -> Any:
        """Runs the matrix memory (mLSTM) over every request's new tokens from the state in its slot
        (``state``: float32 [slots, heads * (dim * vdim + copies * (dim + 1))]: per head the matrix and then
        the normaliser and the running maximum, once for every ``normaliser_columns`` value columns).  ``proj``
        float32 rows hold q, k, v and the two gate projections from the columns ``offsets``; ``out`` float32
        [T, heads * vdim].  A step of single tokens runs one kernel and ``out`` is the mixer's output; a step with
        prompt portions first packs what the recurrence reads for all tokens at once and then streams it: ``out``
        then holds the numerators and the float32 [T, heads] tensor that is returned what ``head_norm_gate`` is to
        divide them by (None otherwise).  With ``plan`` (``plan_memory_chunks``, on the device) and key and value
        sizes that the chunk kernels take, prompt portions run in chunks instead: the gates of all tokens, chunk
        sums in parallel, a short walk over each request's chunks, outputs in parallel; ``out`` is the mixer's
        output."""
        self._flush()
        self._load_recurrent()
        q_off, k_off, v_off, i_off, f_off = offsets
        tokens = proj.shape[0]
        if (plan and tokens >= 8 * ctx.num_requests and max(dim, vdim) <= self.mlstm_chunk_max_dim
                and os.environ.get("CIE_RECURRENT_CHUNKS", "1") != "0"):
            chunks = plan["chunk_row"].shape[0]
            floats = int(self._mlstm_chunk_floats(tokens, chunks, heads, dim, vdim))
            rows = max(tokens, self.max_rows)
            reserve = int(self._mlstm_chunk_floats(rows, -(-rows // self.mlstm_chunk_tokens) + ctx.num_requests,
                                                   heads, dim, vdim))
            scratch = self.scratch(f"recurrent.chunks.{heads}x{dim}x{vdim}", floats, reserve=max(floats, reserve))
            self.launches += 5
            self._mlstm_chunked(_ptr(proj), proj.stride(0), q_off, k_off, v_off, i_off, f_off, _ptr(input_bias),
                                _ptr(forget_bias), float(cap), float(q_scale), _ptr(scratch), _ptr(out), out.stride(0),
                                _ptr(state), state.stride(0), _ptr(ctx.query_start), _ptr(ctx.slots),
                                _ptr(ctx.request_active), _ptr(plan["chunk_row"]), _ptr(plan["chunk_count"]),
                                _ptr(plan["request_chunk_start"]), tokens, chunks, ctx.num_requests, heads, dim, vdim,
                                state.shape[0], _ptr(self.error_word), self.stream)
            return None
        if self._streams(tokens, ctx, dim):
            packed = self._stream_scratch(tokens, heads, dim, vdim, True)
            below = self.scratch(f"recurrent.denominators.{heads}", tokens * heads,
                                 reserve=max(tokens, self.max_rows) * heads)[:tokens * heads].view(tokens, heads)
            self.launches += 2
            self._mlstm_stream(_ptr(proj), proj.stride(0), q_off, k_off, v_off, i_off, f_off, _ptr(input_bias),
                               _ptr(forget_bias), float(cap), float(q_scale), _ptr(packed), _ptr(out), out.stride(0),
                               _ptr(below), _ptr(state), state.stride(0), _ptr(ctx.query_start), _ptr(ctx.slots),
                               _ptr(ctx.request_active), tokens, ctx.num_requests, heads, dim, vdim, state.shape[0],
                               _ptr(self.error_word), self.stream)
            return below
        self.launches += 1
        self._mlstm_scan(_ptr(proj), proj.stride(0), q_off, k_off, v_off, i_off, f_off, _ptr(input_bias),
                         _ptr(forget_bias), float(cap), float(q_scale), _ptr(out), out.stride(0), _ptr(state),
                         state.stride(0), _ptr(ctx.query_start), _ptr(ctx.slots), _ptr(ctx.request_active),
                         ctx.num_requests, heads, dim, vdim, state.shape[0], _ptr(self.error_word), self.stream)
        return None

    def short_conv(self, proj: Any, weight: Any, history: Any, out: Any, ctx: Any) -> None:
        """out[t, c] = silu(sum_j weight[c, j] * x[t - (taps - 1 - j), c]) for the first ``weight.shape[0]``
        columns of float32 ``proj``; inputs before this step come from ``history`` (a view [slots, (taps - 1) *
        channels] of the requests' state, oldest first), which then takes this step's last inputs."""
        self._flush()
        self._load_recurrent()
        channels, taps = weight.shape
        self.launches += 2 if taps > 1 else 1
        self._short_conv(_ptr(proj), proj.stride(0), _ptr(weight), taps, _ptr(history), history.stride(0), _ptr(out),
                         out.stride(0), _ptr(ctx.query_start), _ptr(ctx.request_of_token), _ptr(ctx.slots),
                         _ptr(ctx.request_active), proj.shape[0], ctx.num_requests, channels, history.shape[0],
                         _ptr(self.error_word), self.stream)

    def gated_delta_scan(self, conv: Any, offsets: tuple[int, int, int], proj: Any, gate_offsets: tuple[int, int],
                         a_log: Any, dt_bias: Any, q_scale: float, out: Any, state: Any, ctx: Any, heads: int,
                         kv_heads: int, dim: int, vdim: int, plan: dict[str, Any] | None = None) -> None:
        """Runs the gated delta rule over every request's new tokens from the state in its slot (``state``:
        float32 [slots, >= heads * dim * vdim], a head's matrix after the other).  ``conv`` float32 rows hold
        q, k (kv_heads x dim) and v (heads x vdim) after convolution and SiLU from the columns ``offsets``;
        ``proj`` float32 rows hold the write-strength and decay projections (heads each) from ``gate_offsets``;
        ``out`` float32 [T, heads * vdim].  Single tokens: one kernel.  Prompt portions with ``plan``
        (``plan_memory_chunks``, on the device), keys and values up to ``mlstm_chunk_max_dim`` and values a multiple
        of 4: in chunks (a triangular system per chunk, a walk over each request's chunks, outputs in parallel);
        other prompt portions: prepare + stream."""
        self._flush()
        self._load_recurrent()
        q_off, k_off, v_off = offsets
        b_off, a_off = gate_offsets
        tokens = conv.shape[0]
        if (plan and tokens >= 8 * ctx.num_requests and max(dim, vdim) <= self.mlstm_chunk_max_dim and vdim % 4 == 0
                and os.environ.get("CIE_RECURRENT_CHUNKS", "1") != "0"):
            chunks = plan["chunk_row"].shape[0]
            floats = int(self._gated_delta_chunk_floats(tokens, chunks, heads, dim, vdim))
            rows = max(tokens, self.max_rows)
            reserve = int(self._gated_delta_chunk_floats(rows, -(-rows // self.mlstm_chunk_tokens) + ctx.num_requests,
                                                         heads, dim, vdim))
            scratch = self.scratch(f"recurrent.delta_chunks.{heads}x{dim}x{vdim}", floats, reserve=max(floats, reserve))
            self.launches += 4
            self._gated_delta_chunked(_ptr(conv), conv.stride(0), q_off, k_off, v_off, _ptr(proj), proj.stride(0),
                                      b_off, a_off, _ptr(a_log), _ptr(dt_bias), float(q_scale), _ptr(scratch), _ptr(out),
                                      out.stride(0), _ptr(state), state.stride(0), _ptr(ctx.slots),
                                      _ptr(ctx.request_active), _ptr(plan["chunk_row"]), _ptr(plan["chunk_count"]),
                                      _ptr(plan["request_chunk_start"]), tokens, chunks, ctx.num_requests, heads,
                                      kv_heads, dim, vdim, state.shape[0], _ptr(self.error_word), self.stream)
            return
        if self._streams(tokens, ctx, dim):       # prompt portions: pack for all tokens at once, then stream
            packed = self._stream_scratch(tokens, heads, dim, vdim, False)
            self.launches += 2
            self._gated_delta_stream(_ptr(conv), conv.stride(0), q_off, k_off, v_off, _ptr(proj), proj.stride(0),
                                     b_off, a_off, _ptr(a_log), _ptr(dt_bias), float(q_scale), _ptr(packed), _ptr(out),
                                     out.stride(0), _ptr(state), state.stride(0), _ptr(ctx.query_start),
                                     _ptr(ctx.slots), _ptr(ctx.request_active), tokens, ctx.num_requests, heads,
                                     kv_heads, dim, vdim, state.shape[0], _ptr(self.error_word), self.stream)
            return
        self.launches += 1
        self._gated_delta_scan(_ptr(conv), conv.stride(0), q_off, k_off, v_off, _ptr(proj), proj.stride(0), b_off,
                               a_off, _ptr(a_log), _ptr(dt_bias), float(q_scale), _ptr(out), out.stride(0),
                               _ptr(state), state.stride(0), _ptr(ctx.query_start), _ptr(ctx.slots),
                               _ptr(ctx.request_active), ctx.num_requests, heads, kv_heads, dim, vdim,
                               state.shape[0], _ptr(self.error_word), self.stream)

    def head_norm_gate(self, o: Any, gate: Any, gain: Any, eps: float, out: Any, heads: int,
                       gate_act: str = "sigmoid", denominators: Any = None) -> None:
        """Every head (``out.shape[1] / heads`` columns) of float32 ``o`` divided by its own root mean square,
        times ``gain`` (one number per column, or a vector of a head's size for all heads), times sigmoid or
        SiLU of ``gate`` (float32, may be a view of columns).  With ``denominators`` (float32 [T, heads],
        contiguous) every head is first divided by its number."""
        self._flush()
        self._load_recurrent()
        size = out.shape[1] // heads
        if gain.numel() not in (size, out.shape[1]):
            raise KernelError(f"head_norm_gate: a gain of {gain.numel()} numbers for heads of {size}")
        shared = 1 if gain.numel() == size and heads > 1 else 0
        acts = {"sigmoid": 0, "silu": 1}
        self.launches += 1
        self._head_norm_gate(_ptr(o), o.stride(0), _ptr(denominators), _ptr(gate), gate.stride(0), _ptr(gain), shared, acts[gate_act],
                             _ptr(out), out.stride(0), out.shape[0], heads, size, float(eps), self._code_of(out),
                             self.stream)

    # ------------------------------------------------------------------ residual streams
    def _load_streams(self) -> None:
        if self._streams_lib is None:
            v, i, f = c_void_p, c_int, c_float
            lib = _Lib(load_library("streams.cu"))
            self._embedding_streams = lib.function("cie_embedding_streams", [v, v, v, v, v, i, i, i, i, i, f, i, v, v])
            self._stream_norm = lib.function("cie_stream_norm", [v, i, v, i, v, v, v, v, i, v, v, i, i, f, i, v])
            self._norm_kv_write = lib.function(
                "cie_norm_kv_write",
                [v, v, v, i, v, v, v, i, i, v, v, v, v, i, i, i, i, i, i, i, i, f, i, i, i, v, i, f, i, i, v, v])
            self._streams_lib = lib

    def stream_norm(self, residual: Any, streams: int, update: Any, read: Any, gain: Any, eps: float,
                    out: Any, rows: Any = None) -> None:
        """The boundary between two sublayers over ``streams`` copies of the residual stream
        (``residual``: float32 [T, streams * H]): applies ``update`` (a ``StreamUpdate``, a plain
        tensor to add to every stream, or None) in place, reads ``sum_t read[t] * stream_t`` (``read``
        None: the plain sum) and writes its RMS norm times ``gain`` (a vector [H] or one number) to
        ``out``.  With ``rows`` only those token rows are read and nothing is written back."""
        self._flush()
        self._load_streams()
        if isinstance(update, Accumulated):
            update = None
        if isinstance(update, Partials):
            update = self.resolve(update, self.torch.empty(update.shape, dtype=self.torch.float32, device=self.device))
        if update is not None and not isinstance(update, StreamUpdate):
            update = StreamUpdate(update)
        if update is not None and isinstance(update.y, Partials):
            update.y = self.resolve(update.y, self.torch.empty(update.y.shape, dtype=self.torch.float32, device=self.device))
        count, hidden = out.shape
        y = update.y if update is not None else None
        self.launches += 1
        self._stream_norm(_ptr(residual), streams, _ptr(y), self._code_of(y) if y is not None else 0,
                          _ptr(update.mix) if update is not None else None,
                          _ptr(update.out) if update is not None else None, _ptr(read), _ptr(gain),
                          1 if gain.numel() == 1 else 0, _ptr(out), _ptr(rows), count, hidden, float(eps),
                          self._code_of(out), self.stream)

    def norm_kv_write(self, qkv: Any, ctx: Any, kv: Any, q_heads: int, kv_heads: int, dim: int, vdim: int,
                      q_gain: Any, k_gain: Any, value_norm: bool, eps: float, q_buffer: Any,
                      write_cache: bool = True, per_head: bool = False, rotation: Any = None) -> Any:
        """q and k of every token divided by the root mean square of their whole projection and
        multiplied by a gain vector (``q_gain`` None: left as they are), every value head divided by
        its own root mean square (``value_norm``); q goes to ``q_buffer``, k and v into the pages.
        ``per_head``: every q and k head is divided by its OWN root mean square instead, and the gains
        are vectors of a head's size that all heads share.
        ``rotation`` (``inv_freq`` float32 [dims / 2], ``dims``, ``magnitude``, ``interleaved``): after the norms
        the first ``dims`` elements of every q and k head turn by the token's position.
        ``qkv`` is a tensor [T, (Hq + Hkv) * dim + Hkv * vdim] of the compute dtype or of float32 (its rows may
        go on with other columns, which are left alone) or ``Partials`` with its bias pending."""
        self._flush()
        self._load_streams()
        bias = None
        if isinstance(qkv, Partials):
            if qkv.splits:
                qkv = self.resolve(qkv, self.torch.empty(qkv.shape, dtype=self.dtype, device=self.device))
            else:
                qkv, bias = qkv.data, qkv.bias
        table = ctx.block_tables[kv.group]
        self.launches += 1
        self._norm_kv_write(_ptr(qkv), _ptr(bias), _ptr(q_buffer), q_buffer.shape[1], _ptr(ctx.positions),
                            _ptr(ctx.request_of_token), _ptr(table), table.shape[1], kv.num_pages, _ptr(kv.k),
                            _ptr(kv.v), _ptr(q_gain), _ptr(k_gain), qkv.shape[0], q_heads, kv_heads, dim, vdim,
                            kv.page_size, 0 if q_gain is None else (2 if per_head else 1), 1 if value_norm else 0,
                            float(eps), 1 if write_cache else 0, qkv.stride(0), self._code_of(qkv),
                            _ptr(rotation.inv_freq) if rotation is not None else None,
                            int(rotation.dims) if rotation is not None else 0,
                            float(rotation.magnitude) if rotation is not None else 1.0,
                            int(rotation.interleaved) if rotation is not None else 0,
                            self._code_of(q_buffer), _ptr(self.error_word), self.stream)
        return q_buffer

    # ------------------------------------------------------------------ linear attention with decay
    def _load_lightning(self) -> None:
        if self._lightning_lib is None:
            v, i, f = c_void_p, c_int, c_float
            lib = _Lib(load_library("lightning.cu"))
            self._lightning_scan = lib.function("cie_lightning_scan", [v, i, v, i, v, v, v, v, v, i, i, i, i, i, i, v, v])
            self._lightning_gate_norm = lib.function("cie_lightning_gate_norm", [v, i, v, i, v, v, i, i, f, i, v])
            self._lightning_chunked = lib.function(
                "cie_lightning_chunked", [v, i, v, i, v, v, v, v, v, v, v, v, i, i, i, i, i, i, i, v, v])
            self.lightning_chunk_tokens = int(lib.handle.cie_lightning_chunk_tokens())
            self._lightning_lib = lib

    LIGHTNING_CHUNK_MAX_DIM = 128     # largest key and value size of the chunked kernels

    def plan_lightning(self, host: Any) -> dict[str, Any]:
        """Work lists of the chunked form for a step that holds prompt portions: every request's new
        tokens cut into chunks (first token row and token count of each) and, per request, where its
        chunks start.  A step of single tokens runs the recurrence directly and needs none."""
        import numpy as np

        if host.num_single == host.num_requests:
            return {}
        self._load_lightning()
        return self._plan_chunks(host, self.lightning_chunk_tokens)

    @staticmethod
    def _plan_chunks(host: Any, size: int) -> dict[str, Any]:
        """Every request's new tokens cut into chunks of ``size`` from its first new token."""
        import numpy as np

        rows, counts, starts = [], [], [0]
        for first, length in zip(host.query_start[:-1].tolist(), host.query_lens.tolist()):
            for offset in range(0, length, size):
                rows.append(first + offset)
                counts.append(min(size, length - offset))
            starts.append(len(rows))
        return {"chunk_row": np.asarray(rows, dtype=np.int32), "chunk_count": np.asarray(counts, dtype=np.int32),
                "request_chunk_start": np.asarray(starts, dtype=np.int32)}

    def lightning_chunked(self, proj: Any, out: Any, state: Any, decay: Any, ctx: Any, plan: dict[str, Any],
                          heads: int, dim: int, vdim: int) -> None:
        """The same recurrence as ``lightning_scan`` for a step with prompt portions, in chunks (see
        ``plan_lightning``): chunk sums in parallel, a short walk over each request's chunks, outputs
        in parallel.  Float32 throughout."""
        self._flush()
        self._load_lightning()
        chunks = plan["chunk_row"].shape[0]
        scratch = self.scratch("lightning.chunks", chunks * heads * dim * vdim)
        self.launches += 3
        self._lightning_chunked(_ptr(proj), proj.stride(0), _ptr(out), out.stride(0), _ptr(state), _ptr(scratch),
                                _ptr(decay), _ptr(plan["chunk_row"]), _ptr(plan["chunk_count"]),
                                _ptr(plan["request_chunk_start"]), _ptr(ctx.slots), _ptr(ctx.request_active),
                                chunks, ctx.num_requests, heads, dim, vdim, state.shape[0], self._code_of(proj),
                                _ptr(self.error_word), self.stream)

    def lightning_scan(self, proj: Any, out: Any, state: Any, decay: Any, ctx: Any, heads: int, dim: int,
                       vdim: int) -> None:
        """Runs S <- decay * S + k v^T, o = S^T q over every request's new tokens from the state in
        its slot (``state``: float32 [slots, heads, dim, vdim]).  ``proj`` rows are [q | k | v | ...]
        before their SiLU; ``out`` is float32 [T, heads * vdim]."""
        self._flush()
        self._load_lightning()
        self.launches += 1
        self._lightning_scan(_ptr(proj), proj.stride(0), _ptr(out), out.stride(0), _ptr(state), _ptr(decay),
                             _ptr(ctx.query_start), _ptr(ctx.slots), _ptr(ctx.request_active), ctx.num_requests,
                             heads, dim, vdim, state.shape[0], self._code_of(proj), _ptr(self.error_word),
                             self.stream)

    def lightning_gate_norm(self, o: Any, gate: Any, gain: Any, eps: float, out: Any) -> None:
        """out = gain * o / rms(o) * sigmoid(gate), the norm over the whole row (all heads together);
        ``gate`` is a view of columns of the projection (its row stride is used)."""
        self._flush()
        self._load_lightning()
        self.launches += 1
        self._lightning_gate_norm(_ptr(o), o.stride(0), _ptr(gate), gate.stride(0), _ptr(gain), _ptr(out),
                                  out.shape[0], out.shape[1], float(eps), self._code_of(out), self.stream)

    # ------------------------------------------------------------------ gated linear attention
    def _load_gla(self) -> None:
        if self._gla_lib is None:
            v, i, f = c_void_p, c_int, c_float
            lib = _Lib(load_library("gla.cu"))
            self._gla_scan = lib.function(
                "cie_gla_scan", [v, i, i, i, i, v, i, v, f, f, v, i, v, v, v, v, i, i, i, i, i, v, v])
            self._gla_chunked = lib.function(
                "cie_gla_chunked",
                [v, i, i, i, i, v, i, v, f, f, v, i, v, v, v, v, v, v, v, v, i, i, i, i, i, i, v, v])
            self.gla_scan_max_dim = int(lib.handle.cie_gla_scan_max_dim())
            self.gla_chunk_tokens = int(lib.handle.cie_gla_chunk_tokens())
            self.gla_chunk_max_dim = int(lib.handle.cie_gla_chunk_max_dim())
            self._gla_lib = lib

    def require_gla(self) -> int:
        """Builds, at model set-up, the kernels of gated linear attention; returns the largest key size they take."""
        self._load_gla()
        return self.gla_scan_max_dim

    def plan_gla(self, host: Any) -> dict[str, Any]:
        """Chunk work lists of gated linear attention for a step that holds prompt portions (one list serves
        every such layer); a step of single tokens runs the recurrence directly and needs none."""
        if host.num_single == host.num_requests:
            return {}
        self._load_gla()
        return self._plan_chunks(host, self.gla_chunk_tokens)

    def gla(self, proj: Any, offsets: tuple[int, int, int], z: Any, z_bias: Any, tau: float, q_scale: float,
            out: Any, state: Any, ctx: Any, heads: int, dim: int, vdim: int,
            plan: dict[str, Any] | None = None) -> None:
        """Gated linear attention over every request's new tokens from the state in its slot (``state``: float32
        [slots, heads, dim, vdim]): ``S <- diag(alpha) S + k v^T``, ``o = S^T (q * q_scale)`` with
        ``alpha = sigmoid(z + z_bias)^(1 / tau)`` per head and key channel.  ``proj`` is float32 [T, *] with q, k
        and v at the columns ``offsets``; ``z`` float32 [T, heads * dim] (the chunked form overwrites it);
        ``out`` float32 [T, heads * vdim].  With
        ``plan`` (chunk lists of a step with prompt portions) and sizes the chunked kernels take, the recurrence
        runs in chunks; else token by token."""
        self._flush()
        self._load_gla()
        if proj.dtype != self.torch.float32 or z.dtype != self.torch.float32:
            raise KernelError("gla: the projections enter the recurrence as float32 rows")
        head = (_ptr(proj), proj.stride(0), int(offsets[0]), int(offsets[1]), int(offsets[2]), _ptr(z), z.stride(0),
                _ptr(z_bias), 1.0 / float(tau), float(q_scale), _ptr(out), out.stride(0), _ptr(state))
        chunked = (plan and dim <= self.gla_chunk_max_dim and vdim <= self.gla_chunk_max_dim
                   and os.environ.get("CIE_GLA_CHUNKS", "1") != "0")
        if chunked:
            chunks = plan["chunk_row"].shape[0]
            # room for the chunks of the largest step the runtime knows of (and a partial chunk for many requests),
            # so that a long prompt after captured steps does not have to grow the buffers
            most = max(chunks, self.max_rows // self.gla_chunk_tokens + 64)
            sums = self.scratch(f"gla.chunks.{heads}x{dim}x{vdim}", chunks * heads * dim * vdim,
                                reserve=most * heads * dim * vdim)
            decays = self.scratch(f"gla.decays.{heads}x{dim}", chunks * heads * dim, reserve=most * heads * dim)
            self.launches += 4
            self._gla_chunked(*head, _ptr(sums), _ptr(decays), _ptr(plan["chunk_row"]), _ptr(plan["chunk_count"]),
                              _ptr(plan["request_chunk_start"]), _ptr(ctx.slots), _ptr(ctx.request_active), chunks,
                              ctx.num_requests, heads, dim, vdim, state.shape[0], _ptr(self.error_word), self.stream)
            return
        self.launches += 1
        self._gla_scan(*head, _ptr(ctx.query_start), _ptr(ctx.slots), _ptr(ctx.request_active), ctx.num_requests,
                       heads, dim, vdim, state.shape[0], _ptr(self.error_word), self.stream)

    # ------------------------------------------------------------------ attention over a cached latent
    def _load_latent(self) -> None:
        if self._latent_lib is None:
            v, i, f = c_void_p, c_int, c_float
            lib = _Lib(load_library("latent.cu"))
            self._latent_prepare = lib.function(
                "cie_latent_prepare", [v, i, v, v, v, v, v, v, i, i, v, v, v, f, i, i, i, i, i, i, i, f, i, i, i, v, v])
            self._head_linear = lib.function("cie_head_linear", [v, i, i, v, v, i, i, v, i, i, i, i, i, i, i, v])
            self._latent_attention = lib.function(
                "cie_latent_attention",
                [v, v, i, i, v, v, v, v, v, v, v, i, i, v, f, i, i, v, i, i, i, i, i, f, i, i, i, i, v, v])
            self._latent_merge = lib.function("cie_latent_merge", [v, v, v, v, i, i, i, i, i, i, v])
            self._head_gather = lib.function("cie_head_gather", [v, i, i, v, i, i, i, v])
            self._head_scatter = lib.function("cie_head_scatter", [v, v, i, i, v, i, i, i, i, i, v])
            self.latent_max_rank = int(lib.handle.cie_latent_attention_max_rank())
            self._latent_lib = lib
            self._latent_tensor = None
            if self.code == BF16 and os.environ.get("CIE_LATENT_TENSOR", "1") != "0":
                tensor = _Lib(load_library("latent_tensor.cu"))
                self._latent_tensor = tensor.function(
                    "cie_latent_attention_tensor",
                    [v, v, i, i, v, v, v, v, v, v, v, i, i, v, f, i, i, v, i, i, i, i, i, f, i, i, i, i, v, v])
                self._latent_tensor_supports = tensor.handle.cie_latent_attention_tensor_supports

    def require_latent(self) -> int:
        """Builds, at model set-up, the kernels of attention over a cached latent; returns the largest latent they take."""
        self._load_latent()
        return self.latent_max_rank

    def latent_prepare(self, down: Any, q_out: Any, q_gain: Any, kv_gain: Any, ctx: Any, kv: Any, rotation: Any,
                       q_rank: int, rank: int, rot: int, eps: float, has_kv: bool, write_cache: bool) -> None:
        """Per token of ``down`` (float32 [T, q_rank (+ rank + rot)]): the query latent divided by its
        root mean square times ``q_gain`` goes to ``q_out``; with ``has_kv`` and ``write_cache`` the
        latent, normalised likewise with ``kv_gain``, and the key part, rotated by the token's position,
        go into the pages (``kv.k``: latents, ``kv.v``: rotated key parts).  ``rotation`` gives
        ``inv_freq``, ``magnitude``, ``interleaved`` and ``dims``."""
        self._flush()
        self._load_latent()
        table = ctx.block_tables[kv.group]
        self.launches += 1
        self._latent_prepare(_ptr(down), down.stride(0), _ptr(q_out), _ptr(q_gain), _ptr(kv_gain), _ptr(ctx.positions),
                             _ptr(ctx.request_of_token), _ptr(table), table.shape[1], kv.num_pages, _ptr(kv.k),
                             _ptr(kv.v), _ptr(rotation.inv_freq), float(rotation.magnitude), int(rotation.interleaved),
                             int(rotation.dims), down.shape[0], q_rank, rank, rot, kv.page_size, float(eps),
                             1 if has_kv else 0, 1 if write_cache else 0, self.code, _ptr(self.error_word), self.stream)

    def head_linear(self, x: Any, x_head: int, weight: Any, out: Any, out_head: int, heads: int, gate: Any = None) -> None:
        """A product per head: ``out[t, h, :N] = x[t, h, :K] @ weight[h]`` with ``weight`` [heads, K, N] in
        the compute dtype, ``x`` float32 (head h of a row starts at column ``h * x_head``), ``out`` float32
        or the compute dtype (head h at column ``h * out_head``); sums in float32, k ascending.  With
        ``gate`` (float32 [T, heads * N], may be a view of columns) the result is multiplied by sigmoid(gate).

        More than 16 tokens in bfloat16 run as ONE batched library product (the framework's rule for
        matrix products of that many rows): the rows are gathered head-major and rounded to bfloat16, the
        product's bfloat16 result is carried back (with the gate) by a second small kernel."""
        self._flush()
        self._load_latent()
        _, depth, width = weight.shape
        tokens = x.shape[0]
        if (self.code == BF16 and tokens > STREAM_MAX_ROWS and weight.dtype == self.torch.bfloat16
                and os.environ.get("CIE_HEAD_BATCHED", "1") != "0"):
            torch = self.torch
            most = max(tokens, self.max_rows)
            rows = self.scratch(f"head.rows.{heads}x{depth}", (heads * tokens * depth + 1) // 2, reserve=(heads * most * depth + 1) // 2)
            rows = rows.view(torch.bfloat16)
            rows = rows[: heads * tokens * depth].view(heads, tokens, depth)
            result = self.scratch(f"head.result.{heads}x{width}", (heads * tokens * width + 1) // 2, reserve=(heads * most * width + 1) // 2)
            result = result.view(torch.bfloat16)
            result = result[: heads * tokens * width].view(heads, tokens, width)
            self.launches += 3
            self._head_gather(_ptr(x), x.stride(0), x_head, _ptr(rows), tokens, heads, depth, self.stream)
            torch.bmm(rows, weight, out=result)
            self._head_scatter(_ptr(result), _ptr(out), out.stride(0), out_head, _ptr(gate),
                               gate.stride(0) if gate is not None else 0, tokens, heads, width, self._code_of(out),
                               self.stream)
            return
        self.launches += 1
        self._head_linear(_ptr(x), x.stride(0), x_head, _ptr(weight), _ptr(out), out.stride(0), out_head, _ptr(gate),
                          gate.stride(0) if gate is not None else 0, x.shape[0], heads, depth, width,
                          self._code_of(weight), self._code_of(out), self.stream)

    def latent_attention(self, q_latent: Any, q_raw: Any, q_raw_head: int, out: Any, ctx: Any, kv: Any, rotation: Any,
                         sink: Any, heads: int, rank: int, rot: int, scale: float, window: int = 0) -> None:
        """Causal softmax attention of every (token, head) over the rows [latent | rotated key part] its
        request holds in the pages: ``q_latent`` float32 [T, heads, rank] meets the latents, the rotated
        part of ``q_raw`` (float32; head h starts at column ``h * q_raw_head``; rotated here) meets the key
        parts; ``out`` float32 [T, heads, rank] is the weighted sum of the latents.  ``sink`` (float32
        [heads] or None) adds exp(sink_h) to the softmax denominator.  ``window`` > 0: a token sees only its
        last ``window`` keys, itself included.  With few tokens the keys are cut
        into ranges over CTAs and joined by a second kernel.  bfloat16 pages whose two parts are multiples
        of 8 elements run on the tensor cores (16 heads of a token a tile), everything else on the plain
        kernel (8 heads a CTA, a warp each)."""
        self._flush()
        self._load_latent()
        tokens = q_latent.shape[0]
        table = ctx.block_tables[kv.group]
        tensor = self._latent_tensor is not None and bool(self._latent_tensor_supports(rank, rot))
        groups = -(-heads // (16 if tensor else 8))
        ranges, range_keys, scratch = 1, 1 << 30, None
        if tokens * groups < self.sm_count:
            # about two CTAs an SM: ranges of a multiple of 128 keys, counted over the longest context the tables hold
            longest = table.shape[1] * kv.page_size
            if window > 0:
                longest = min(longest, window)
            wanted = -(-2 * self.sm_count // (tokens * groups))
            range_keys = max(128, (-(-longest // wanted) + 127) // 128 * 128)
            ranges = max(1, -(-longest // range_keys))
        if ranges > 1:
            # tokens x groups x ranges stays within a few CTAs an SM, which bounds the scratch memory whatever the
            # step: made once at that size, it need not grow under a captured graph
            reserve = 8 * self.sm_count * (heads // groups + 1) * (rank + 2)
            scratch = self.scratch(f"latent.ranges.{heads}x{rank}", tokens * heads * ranges * (rank + 2), reserve=reserve)
        else:
            ranges, range_keys = 1, 1 << 30
        self.launches += 2 if ranges > 1 else 1
        if tensor:
            self._latent_tensor(_ptr(q_latent), _ptr(q_raw), q_raw.stride(0), q_raw_head, _ptr(out), _ptr(scratch),
                                _ptr(kv.k), _ptr(kv.v), _ptr(ctx.positions), _ptr(ctx.request_of_token), _ptr(table),
                                table.shape[1], kv.num_pages, _ptr(rotation.inv_freq), float(rotation.magnitude),
                                int(rotation.interleaved), int(rotation.dims), _ptr(sink), tokens, heads, rank, rot,
                                kv.page_size, float(scale), range_keys, ranges,
                                0 if os.environ.get("CIE_LATENT_PAIRS", "1") == "0" else 1, int(window),
                                _ptr(self.error_word), self.stream)
            if ranges > 1:
                self._latent_merge(_ptr(scratch), _ptr(out), _ptr(ctx.positions), _ptr(sink), tokens, heads, rank,
                                   range_keys, ranges, int(window), self.stream)
            return
        self._latent_attention(_ptr(q_latent), _ptr(q_raw), q_raw.stride(0), q_raw_head, _ptr(out), _ptr(scratch),
                               _ptr(kv.k), _ptr(kv.v), _ptr(ctx.positions), _ptr(ctx.request_of_token), _ptr(table),
                               table.shape[1], kv.num_pages, _ptr(rotation.inv_freq), float(rotation.magnitude),
                               int(rotation.interleaved), int(rotation.dims), _ptr(sink), tokens, heads, rank, rot,
                               kv.page_size, float(scale), range_keys, ranges, int(window), self.code,
                               _ptr(self.error_word), self.stream)

    # ------------------------------------------------------------------ generalized delta rule
    def _load_delta(self) -> None:
        if self._delta_lib is None:
            v, i, f = c_void_p, c_int, c_float
            lib = _Lib(load_library("delta.cu"))
            self._tanh_rows = lib.function("cie_tanh_rows", [v, i, v, i, i, i, v])
            self._delta_scan = lib.function(
                "cie_delta_scan", [v, i, i, i, i, i, v, i, v, v, v, i, v, v, v, v, i, i, i, i, v, v])
            self._group_gate_norm = lib.function("cie_group_gate_norm", [v, i, v, i, v, v, i, i, i, i, f, i, v])
            self._delta_stream = lib.function(
                "cie_delta_stream", [v, i, i, i, i, i, v, i, v, v, v, v, i, v, v, v, v, i, i, i, i, i, v, v])
            lib.handle.cie_delta_stream_floats.restype = ctypes.c_longlong
            self.delta_max_dim = int(lib.handle.cie_delta_max_dim())
            self.delta_stream_max_dim = int(lib.handle.cie_delta_stream_max_dim())
            self._delta_lib = lib

    def require_delta(self) -> int:
        """Builds, at model set-up, the kernels of the generalized delta rule; returns the largest head size they take."""
        self._load_delta()
        return self.delta_max_dim

    def tanh_rows(self, x: Any, out: Any) -> None:
        """out = tanh(x) for float32 ``x`` (may be a view of columns), rounded to ``out``'s dtype."""
        self._flush()
        self._load_delta()
        self.launches += 1
        self._tanh_rows(_ptr(x), x.stride(0), _ptr(out), out.shape[0], out.shape[1], self._code_of(out), self.stream)

    def delta_scan(self, proj: Any, offsets: tuple[int, int, int, int], decay: Any, decay_bias: Any,
                   removal_bias: Any, out: Any, state: Any, ctx: Any, heads: int, dim: int) -> None:
        """Runs the generalized delta rule over every request's new tokens from the state in its slot
        (``state``: float32 [slots, heads, dim, dim]).  ``proj`` float32 rows hold r, k, v and the
        removal projection from the columns ``offsets``; ``decay`` float32 [T, heads * dim] is the decay
        projection; both biases are added here; ``out`` float32 [T, heads * dim].  A step of single tokens
        runs one kernel that works the rates out as it goes; a step with prompt portions (eight tokens a
        request or more on average) first works out, for all tokens at once, what the recurrence reads
        and then streams it through a ring of copies: the same additions in the same order."""
        self._flush()
        self._load_delta()
        r_off, k_off, v_off, a_off = offsets
        tokens = proj.shape[0]
        if (tokens >= 8 * ctx.num_requests and dim <= self.delta_stream_max_dim
                and os.environ.get("CIE_DELTA_STREAM", "1") != "0"):
            floats = self._delta_lib.handle.cie_delta_stream_floats
            packed = self.scratch(f"delta.packed.{heads}x{dim}", int(floats(tokens, heads, dim)),
                                  reserve=int(floats(max(tokens, self.max_rows), heads, dim)))
            self.launches += 2
            self._delta_stream(_ptr(proj), proj.stride(0), r_off, k_off, v_off, a_off, _ptr(decay), decay.stride(0),
                               _ptr(decay_bias), _ptr(removal_bias), _ptr(packed), _ptr(out), out.stride(0), _ptr(state),
                               _ptr(ctx.query_start), _ptr(ctx.slots), _ptr(ctx.request_active), tokens,
                               ctx.num_requests, heads, dim, state.shape[0], _ptr(self.error_word), self.stream)
            return
        self.launches += 1
        self._delta_scan(_ptr(proj), proj.stride(0), r_off, k_off, v_off, a_off, _ptr(decay), decay.stride(0),
                         _ptr(decay_bias), _ptr(removal_bias), _ptr(out), out.stride(0), _ptr(state),
                         _ptr(ctx.query_start), _ptr(ctx.slots), _ptr(ctx.request_active), ctx.num_requests, heads, dim,
                         state.shape[0], _ptr(self.error_word), self.stream)

    def group_gate_norm(self, o: Any, gate: Any, gain: Any, eps: float, out: Any, groups: int) -> None:
        """Every group of ``out.shape[1] / groups`` columns of float32 ``o`` divided by its own root mean
        square, times ``gain`` (all columns), times sigmoid(``gate``) (float32, may be a view of columns)."""
        self._flush()
        self._load_delta()
        self.launches += 1
        self._group_gate_norm(_ptr(o), o.stride(0), _ptr(gate), gate.stride(0), _ptr(gain), _ptr(out), out.stride(0),
                              out.shape[0], groups, out.shape[1] // groups, float(eps), self._code_of(out), self.stream)

    def gated_act(self, gate_up: Any, bias: Any, out: Any, slope: float, limit: float, shift: float) -> None:
        """out[t, c] = g * sigmoid(slope * g) * (u + shift) with g, u the columns c and inter + c of
        ``gate_up`` (float32 or the compute dtype) plus ``bias`` (or None), g capped at ``limit`` and u
        clamped to +-``limit`` when ``limit`` > 0."""
        self._flush()
        self.launches += 1
        self._gated_act(_ptr(gate_up), self._code_of(gate_up), _ptr(bias), _ptr(out), out.shape[0], out.shape[1],
                        float(slope), float(limit), float(shift), self._code_of(out), self.stream)

    # ------------------------------------------------------------------ routed experts
    def _load_moe(self) -> None:
        if self._moe_lib is None:
            v, i = c_void_p, c_int
            lib = _Lib(load_library("moe.cu"))
            self._moe_route = lib.function("cie_moe_route", [v, v, v, v, v, v, v, v, v, v, v, i, i, i, i, i, v, i, i, v])
            self._moe_gate_up_simt = lib.function("cie_moe_gate_up_simt", [v, v, v, v, v, v, v, i, i, i, i, i, i, v])
            self._moe_down_simt = lib.function("cie_moe_down_simt", [v, v, v, v, v, v, i, i, i, i, i, i, v])
            self._moe_combine = lib.function("cie_moe_combine", [v, v, v, i, i, i, i, v])
            self._moe_gate_up_tc = lib.function("cie_moe_gate_up_tc", [v, v, v, v, v, v, v, i, i, i, i, i, v])
            self._moe_down_tc = lib.function("cie_moe_down_tc", [v, v, v, v, v, v, i, i, i, i, i, v])
            self.moe_row_tile = int(lib.handle.cie_moe_row_tile())
            self._moe_lib = lib
            self._moe_tcgen05_lib = None

    def _load_moe_tcgen05(self) -> None:
        if self._moe_tcgen05_lib is None:
            v, i = c_void_p, c_int
            lib = _Lib(load_library("moe_tcgen05.cu"))
            self._moe_gate_up_tcgen05 = lib.function(
                "cie_moe_gate_up_tcgen05", [v, v, v, v, v, v, v, i, i, i, i, i, i, v, v])
            self._moe_down_tcgen05 = lib.function(
                "cie_moe_down_tcgen05", [v, v, v, v, v, v, i, i, i, i, i, i, v, v])
            self._moe_tcgen05_lib = lib

    def moe_interleaves(self, hidden: int, ff: int) -> bool:
        """Whether the gate and up matrices of routed experts are kept as one tensor with their rows
        interleaved in blocks of 16 ([E, 2F, H]), the layout of the tensor-core kernels that finish
        SiLU(gate) * up in their epilogue."""
        return self.code == BF16 and hidden % 8 == 0 and ff % 16 == 0

    def interleave_gate_up(self, gate: Any, up: Any) -> Any:
        """[E, F, H] twice -> [E, 2F, H]: 16 gate rows, their 16 up rows, the next 16 gate rows, ..."""
        experts, ff, hidden = gate.shape
        both = self.torch.stack([gate.view(experts, ff // 16, 16, hidden), up.view(experts, ff // 16, 16, hidden)], dim=2)
        return both.reshape(experts, 2 * ff, hidden).contiguous()

    def routed_experts(self, x: Any, router: Any, correction: Any, w_gate: Any, w_up: Any, w_down: Any,
                       top: int, renormalize: bool, out: Any, workspace: Any, router_bias: Any = None,
                       chosen_softmax: bool = False) -> Any:
        """out[t] = sum over the ``top`` chosen experts e of score_e * down_e(SiLU(gate_e x) * up_e x).
        ``router`` float32 [E, H]; ``w_gate``/``w_up`` [E, F, H], or ``w_up`` None and ``w_gate`` the
        interleaved [E, 2F, H] of ``interleave_gate_up``; ``w_down`` [E, H, F]; ``out`` float32 or the
        activation type.  ``router_bias`` (float32 [E]) is added to the router's logits; ``chosen_softmax``: the
        experts with the largest logits are chosen and weighted by the softmax over their logits alone."""
        self._flush()
        self._load_moe()
        torch = self.torch
        tokens, hidden = x.shape
        experts, ff = w_gate.shape[0], w_gate.shape[1] // (2 if w_up is None else 1)
        pairs = tokens * top
        ids = workspace.get("moe.ids", tokens, top, torch.int32)
        weights = workspace.get("moe.weights", tokens, top, torch.float32)
        place_to_pair = workspace.get("moe.places", tokens, top, torch.int32)
        # counts, offsets, cursors, the tile count and the tile list (three numbers a tile; at most one
        # tile per 64 pairs plus one per expert) share one integer buffer that holds them for any
        # number of tokens
        plan = workspace.get("moe.plan", tokens, 6 * experts + 8 + (3 * top + 63) // 64, torch.int32).view(-1)
        counts, offsets, cursors = plan[:experts], plan[experts:2 * experts + 1], plan[2 * experts + 1:3 * experts + 1]
        tile_count, tiles = plan[3 * experts + 1:3 * experts + 2], plan[3 * experts + 2:]
        assert tiles.numel() >= 3 * (-(-pairs // self.moe_row_tile) + experts)
        act = workspace.get("moe.act", tokens, top * ff, self.dtype)
        rows = workspace.get("moe.rows", tokens, top * hidden, torch.float32)
        code = self._code_of(x)
        self.launches += 5
        self._moe_route(_ptr(x), _ptr(router), _ptr(correction), _ptr(ids), _ptr(weights), _ptr(counts),
                        _ptr(offsets), _ptr(cursors), _ptr(place_to_pair), _ptr(tiles), _ptr(tile_count), tokens,
                        hidden, experts, top, 1 if renormalize else 0, _ptr(router_bias), 1 if chosen_softmax else 0,
                        code, self.stream)
        aligned = (x.data_ptr() | w_gate.data_ptr() | w_down.data_ptr() | act.data_ptr()) % 16 == 0
        if w_up is None and not (code == BF16 and aligned):
            raise KernelError("routed_experts: interleaved gate/up weights are for aligned bfloat16 operands")
        if w_up is None and os.environ.get("CIE_MOE_TCGEN05", "1") != "0":
            # tcgen05: the rows of every expert gathered side by side, tiles by TMA, accumulators in
            # tensor memory
            self._load_moe_tcgen05()
            gathered = workspace.get("moe.sorted", tokens, top * hidden, self.dtype)
            self._moe_gate_up_tcgen05(_ptr(x), _ptr(gathered), _ptr(w_gate), _ptr(act), _ptr(place_to_pair),
                                      _ptr(tiles), _ptr(tile_count), tokens, top, experts, ff, hidden,
                                      self.moe_row_tile, _ptr(self.error_word), self.stream)
            self._moe_down_tcgen05(_ptr(act), _ptr(w_down), _ptr(rows), _ptr(place_to_pair), _ptr(tiles),
                                   _ptr(tile_count), tokens, top, experts, ff, hidden, self.moe_row_tile,
                                   _ptr(self.error_word), self.stream)
            self.launches += 1
        elif (code == BF16 and hidden % 8 == 0 and ff % 8 == 0 and aligned
                and (w_up is None or (os.environ.get("CIE_MOE_TC", "1") != "0" and w_up.data_ptr() % 16 == 0))):
            # bfloat16 on the tensor cores (mma.sync, float32 accumulators)
            self._moe_gate_up_tc(_ptr(x), _ptr(w_gate), _ptr(w_up), _ptr(act), _ptr(place_to_pair), _ptr(tiles),
                                 _ptr(tile_count), tokens, top, experts, ff, hidden, self.stream)
            self._moe_down_tc(_ptr(act), _ptr(w_down), _ptr(rows), _ptr(place_to_pair), _ptr(tiles),
                              _ptr(tile_count), tokens, top, experts, ff, hidden, self.stream)
        else:
            self._moe_gate_up_simt(_ptr(x), _ptr(w_gate), _ptr(w_up), _ptr(act), _ptr(place_to_pair), _ptr(tiles),
                                   _ptr(tile_count), tokens, top, experts, ff, hidden, code, self.stream)
            self._moe_down_simt(_ptr(act), _ptr(w_down), _ptr(rows), _ptr(place_to_pair), _ptr(tiles),
                                _ptr(tile_count), tokens, top, experts, ff, hidden, code, self.stream)
        self._moe_combine(_ptr(rows), _ptr(weights), _ptr(out), tokens, hidden, top, self._code_of(out), self.stream)
        return out

    def stream_plan(self, m: int, n: int, k: int, allow_partials: bool) -> tuple[int, int] | None:
        """(weight rows per CTA, splits along K) for the streaming kernel, or None if the shape
        is not its kind (more than 16 rows, or K not a multiple of 8)."""
        if self._gemm_stream is None or m > STREAM_MAX_ROWS or k % 8 or k < 8:
            return None
        block_rows = 32
        tiles = -(-n // block_rows)
        splits = 1
        if allow_partials:
            # K is cut until the CTAs fill the slots the device has for them: an SM holds five CTAs
            # of the kernel, one is left free for the kernel that follows
            splits = max(1, min(-(-4 * self.sm_count // tiles), k // 256, 8))
        return block_rows, splits

    def scratch(self, tag: str, elements: int, reserve: int = 0) -> Any:
        """Float32 scratch memory by name.  A buffer is made for ``max(elements, reserve)`` at
        first use and may grow later, but not once ``freeze_scratch`` was called (a CUDA graph
        then holds its address)."""
        torch = self.torch
        held = self._partial_buffers.get(tag)
        if held is None or held.numel() < elements:
            if held is not None and self.scratch_frozen:
                raise KernelError(
                    f"scratch buffer {tag!r} would have to grow from {held.numel()} to {elements} "
                    "elements while a CUDA graph that uses it is alive"
                )
            if held is not None:
                self.scratch_generation += 1
            held = torch.empty(max(elements, reserve, 1), dtype=torch.float32, device=self.device)
            self._partial_buffers[tag] = held
        return held

    def freeze_scratch(self) -> None:
        self.scratch_frozen = True

    def _stream(self, x: Any, weight: Any, bias: Any, out: Any, m: int, n: int, k: int, splits: int,
                mode: int, residual: Any = None, sq: Any = None, scaled: Any = None,
                next_gain: Any = None, early_trigger: bool = False, tag: str = "linear") -> None:
        """One launch of the streaming kernel; ``x`` is a tensor or a ``NormedInput``."""
        row_sq, tiles, eps = None, 0, 0.0
        if isinstance(x, NormedInput):
            row_sq, tiles, eps, x = x.accumulated.sq, x.accumulated.tiles, x.eps, x.accumulated.scaled
        if (self.recording and mode != 2 and weight.data_ptr() % 16 == 0 and (mode != 3 or n % 32 == 0)
                and x.data_ptr() % 16 == 0 and x.stride(0) % 8 == 0):
            self.program.gemm(x, row_sq, tiles, eps, weight, bias, out, residual, sq, scaled, next_gain,
                              m, n, k, mode, tag)
            return
        self._flush()
        self.launches += 1
        self._gemm_stream_ex(_ptr(x), _ptr(row_sq), tiles, eps, _ptr(weight), _ptr(bias), _ptr(out),
                             _ptr(residual), _ptr(sq), _ptr(scaled), _ptr(next_gain), m, n, k, splits,
                             mode, 32, 1 if early_trigger else 0, _ptr(self.error_word), self.stream)

    def linear(self, x: Any, weight: Any, bias: Any, out: Any, allow_partials: bool = False,
               tag: str = "", defer_bias: bool = False, residual: Any = None) -> Any:
        """out[M, N] = x[M, K] @ weight[N, K]^T (+ bias); out is the compute dtype or float32.

        Returns ``out``; or, when ``allow_partials`` and the product was cut along K, a
        ``Partials`` that a consuming kernel adds up (then ``out`` was not written); or, when the
        caller names the ``ResidualSink`` its result is to be added to and the streaming kernel
        takes the shape, an ``Accumulated`` (the sum is in the residual stream, ``out`` was not
        written).  ``x`` may be a ``NormedInput``."""
        m, k = x.shape
        n = weight.shape[0]
        if weight.shape[1] != k or tuple(out.shape) != (m, n):
            raise KernelError(f"linear: shapes x{tuple(x.shape)} w{tuple(weight.shape)} out{tuple(out.shape)}")
        if m == 0:
            return out
        plan = self.stream_plan(m, n, k, allow_partials) if self.code == BF16 else None
        if plan is None and self.code == BF16 and self.fold_rows and m >= self.fold_rows:
            done = self._linear_folded(x, weight, bias, out, m, n, k, allow_partials, tag, residual)
            if done is not None:
                return done
        if plan is None and isinstance(x, NormedInput):
            x = x.materialize()
        if plan is not None:
            block_rows, splits = plan
            if residual is not None and self.fuse_norm and allow_partials and m <= FUSED_RESIDUAL_MAX_ROWS:
                cluster = 1
                while cluster * 2 <= splits:
                    cluster *= 2
                tiles = -(-n // 32)
                sq = self.scratch("sq." + (tag or "linear"), m * tiles, reserve=STREAM_MAX_ROWS * tiles)
                gain = residual.gain if n % 8 == 0 else None
                scaled = None
                if gain is not None:
                    scaled = self.scratch("scaled." + (tag or "linear"), (m * n + 1) // 2,
                                          reserve=STREAM_MAX_ROWS * n // 2)
                    scaled = scaled.view(self.torch.bfloat16)[: m * n].view(m, n)
                self._stream(x, weight, bias, None, m, n, k, cluster, 4, residual=residual.tensor, sq=sq,
                             scaled=scaled, next_gain=gain, early_trigger=residual.early_trigger,
                             tag=tag or "linear")
                return Accumulated(residual.tensor, sq, tiles, scaled, gain)
            if splits > 1:
                scratch = self.scratch("partials." + (tag or "linear"), splits * m * n,
                                       reserve=splits * STREAM_MAX_ROWS * n)
                self._stream(x, weight, None, scratch, m, n, k, splits, 2)
                return Partials(scratch, splits, m, n, bias)
            self._stream(x, weight, bias, out, m, n, k, 1, 1 if out.dtype == self.torch.float32 else 0,
                         tag=tag or "linear")
            return out
        self._flush()
        if self.skinny_products == "all" and self.code == BF16 and x.dtype == self.torch.bfloat16:
            skinny = self._skinny_gemm()
            if skinny.supports(x, weight, m, n, k, False, out):
                skinny.launch(x, weight, bias, out, 1 if out.dtype == self.torch.float32 else 0)
                return out
        if self._tensor_gemm is not None and self._tensor_gemm.run(x, weight, bias, out):
            return out
        if self.gemm_mode == "cublas" and self.code == BF16:
            if defer_bias and bias is not None and out.dtype == self.dtype:
                self._cublas_linear(x, weight, None, out)
                return Partials(out, 0, m, n, bias)   # the consumer adds the bias in float32
            self._cublas_linear(x, weight, bias, out)
            return out
        self.launches += 1
        self._gemm_simt(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), m, n, k, self._code_of(x),
                        self._code_of(out), 0 if self.code == F32 else 1, self.stream)
        return out

    def _skinny_gemm(self) -> Any:
        if self._skinny is None:
            from .skinny import SkinnyGemm

            self._skinny = SkinnyGemm(self)
        return self._skinny

    def _fold_gemm(self) -> Any:
        if self._tensor_gemm is not None:
            return self._tensor_gemm
        if self._fold_gemm_held is None:
            from .tensor_gemm import TensorGemm

            self._fold_gemm_held = TensorGemm(self)
        return self._fold_gemm_held

    def _linear_folded(self, x: Any, weight: Any, bias: Any, out: Any, m: int, n: int, k: int,
                       allow_partials: bool, tag: str, residual: Any) -> Any:
        """Many rows on the persistent tcgen05 kernel where that saves a whole pass over the
        activations: a projection that adds itself into the residual stream, or a product whose
        input rows are still to be divided by their root mean square.  None: not its case."""
        self._flush()
        gemm = self._fold_gemm()
        if k % 8 or weight.data_ptr() % 16:
            return None
        if isinstance(x, NormedInput):
            acc = x.accumulated
            gemm.launch_fused(acc.scaled, weight, bias, out, 1 if out.dtype == self.torch.float32 else 0,
                              row_sq=acc.sq, row_tiles=acc.tiles, eps=x.eps)
            return out
        if residual is not None and allow_partials and self.fuse_norm and x.data_ptr() % 16 == 0:
            tiles = -(-n // 32)
            sq = self.scratch("sq.rows." + (tag or "linear"), m * tiles)
            gain = residual.gain if n % 8 == 0 else None
            scaled = None
            if gain is not None:
                scaled = self.scratch("scaled.rows." + (tag or "linear"), (m * n + 1) // 2)
                scaled = scaled.view(self.torch.bfloat16)[: m * n].view(m, n)
            gemm.launch_fused(x, weight, bias, None, 4, residual=residual.tensor, sq=sq, scaled=scaled, next_gain=gain)
            return Accumulated(residual.tensor, sq, tiles, scaled, gain)
        return None

    def resolve(self, value: Any, out: Any) -> Any:
        """A plain tensor for a part that cannot consume ``Partials`` itself."""
        self._flush()
        if not isinstance(value, Partials):
            return value
        if value.splits == 0:
            if value.bias is not None:
                value.data.add_(value.bias.to(value.data.dtype))
            return value.data
        if value.stride != value.rows * value.width:
            raise KernelError("partial sums that lie apart are added up by the norm kernel only")
        total = value.data[: value.splits * value.rows * value.width].view(value.splits, value.rows, value.width).sum(0)
        if value.bias is not None:
            total = total + value.bias
        out.copy_(total)
        return out

    def prepare_gate_up(self, gate: Any, up: Any) -> GateUpWeight:
        """Stacks gate and up; for bfloat16, interleaved in blocks of 16 rows when the channel
        count allows, so that the streaming kernel can apply SiLU(gate) * up in its epilogue."""
        torch = self.torch
        inter = gate.shape[0]
        block = inter
        if self._gemm_stream is not None and inter % 16 == 0:
            block = 16
            hidden = gate.shape[1]
            stacked = torch.stack([gate.view(inter // block, block, hidden),
                                   up.view(inter // block, block, hidden)], dim=1)
            weight = stacked.reshape(2 * inter, hidden)
        else:
            weight = torch.cat([gate, up])
        return GateUpWeight(self.prepare_weight(weight), inter, block)

    def gate_up(self, x: Any, weight: GateUpWeight, hidden_out: Any, workspace: Any) -> Any:
        """hidden_out[T, I] = SiLU(x Wg^T) * (x Wu^T)."""
        m, k = x.shape
        inter = weight.inter
        if self.code == BF16 and weight.block == 16:
            plan = self.stream_plan(m, 2 * inter, k, False)
            if plan is not None:
                self._stream(x, weight.weight, None, hidden_out, m, 2 * inter, k, 1, 3, tag="gate_up")
                return hidden_out
        if (isinstance(x, NormedInput) and self.code == BF16 and weight.block == 16 and self.fold_rows
                and m >= self.fold_rows and k % 8 == 0):
            acc = x.accumulated
            self._flush()
            self._fold_gemm().launch_fused(acc.scaled, weight.weight, None, hidden_out, 3, row_sq=acc.sq,
                                              row_tiles=acc.tiles, eps=x.eps)
            return hidden_out
        if isinstance(x, NormedInput):
            x = x.materialize()
        if self.skinny_products and self.code == BF16 and weight.block == 16 and x.dtype == self.torch.bfloat16:
            skinny = self._skinny_gemm()
            if skinny.supports(x, weight.weight, m, 2 * inter, k, True, hidden_out):
                self._flush()
                skinny.launch(x, weight.weight, None, hidden_out, 3)
                return hidden_out
        both = workspace.get("swiglu.gate_up", m, 2 * inter, self.dtype)
        self.linear(x, weight.weight, None, both)
        self.silu_mul(both, hidden_out, weight.block)
        return hidden_out

    def _cublas_linear(self, x: Any, weight: Any, bias: Any, out: Any) -> None:
        """Library matrix product (cuBLAS through torch), as the reference uses for every
        projection; kept as a yardstick for the hand-written tensor-core kernel."""
        self._flush()
        torch = self.torch
        if out.dtype == torch.float32:
            torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)   # float32 straight into the caller's buffer
        else:
            torch.mm(x, weight.t(), out=out)
        if bias is not None:
            out.add_(bias.to(out.dtype))

    def rope_kv_write(self, qkv: Any, ctx: Any, kv: Any, position: Any, q_heads: int,
                      kv_heads: int, head_dim: int, write_cache: bool = True,
                      q_buffer: Any = None, paired: bool = False) -> Any:
        """Rotates q and k, writes k and v into the pages; returns the tensor that holds the
        rotated q (head h of token t at [t, h * head_dim]).  ``qkv`` is a tensor (q is rotated in
        place) or ``Partials`` (then q goes to ``q_buffer``).  ``paired``: the q and k columns of
        ``qkv`` are in the paired layout of ``pair_rotary_rows``; q then always goes to ``q_buffer``."""
        self._flush()
        rot = position.rotary_dim if position is not None else 0
        inv_freq = position.inv_freq if position is not None else None
        table = ctx.block_tables[kv.group]
        self.launches += 1
        if isinstance(qkv, Partials) and qkv.splits == 0:
            tokens = qkv.rows
            src, splits, stride, bias = qkv.data, 0, 0, qkv.bias
            target = qkv.data
        elif isinstance(qkv, Partials):
            tokens = qkv.rows
            src, splits, stride, bias = qkv.data, qkv.splits, qkv.rows * qkv.width, qkv.bias
            target = q_buffer
        else:
            tokens = qkv.shape[0]
            src, splits, stride, bias = qkv, 0, 0, None
            target = qkv
        if paired:
            if q_buffer is None:
                raise KernelError("rope_kv_write: the paired layout needs a q buffer")
            target = q_buffer
        self._rope_kv_write(_ptr(src), splits, stride, _ptr(bias), _ptr(target), target.shape[1],
                            _ptr(ctx.positions), _ptr(ctx.request_of_token), _ptr(table),
                            table.shape[1], kv.num_pages, _ptr(kv.k), _ptr(kv.v), _ptr(inv_freq),
                            tokens, q_heads, kv_heads, head_dim, rot, kv.page_size,
                            1 if write_cache else 0, 1 if paired else 0, self._code_of(target),
                            _ptr(self.error_word), self.stream)
        return target

    # ------------------------------------------------------------------ rotary epilogue of the q/k/v product
    def can_pair_rotary(self, head_dim: int, rotary_dim: int) -> bool:
        """Whether the stacked q/k/v weight of an attention layer may be kept in the paired
        layout, which lets a decode step rotate and store inside the projection's own kernel."""
        return (self._gemm_stream_rope is not None and os.environ.get("CIE_FUSE_ROPE", "1") != "0"
                and head_dim % 32 == 0 and rotary_dim % 32 == 0 and 32 <= rotary_dim <= head_dim)

    def pair_rotary_rows(self, rows: Any, heads: int, head_dim: int, rotary_dim: int) -> Any:
        """Rows [heads * head_dim, ...] of a q or k projection (weight or bias) in the paired
        layout: inside every head, blocks of 16 rotary elements followed by their 16 partners."""
        torch = self.torch
        half = rotary_dim // 2
        order = torch.empty(head_dim, dtype=torch.long)
        for d in range(head_dim):
            if d >= rotary_dim:
                column = d
            elif d < half:
                column = (d // 16) * 32 + d % 16
            else:
                column = ((d - half) // 16) * 32 + 16 + (d - half) % 16
            order[column] = d
        index = (torch.arange(heads).view(-1, 1) * head_dim + order.view(1, -1)).reshape(-1).to(rows.device)
        return rows.index_select(0, index).contiguous()

    def qkv_rope(self, x: Any, weight: Any, bias: Any, ctx: Any, kv: Any, position: Any, q_heads: int,
                 kv_heads: int, head_dim: int, write_cache: bool, q_buffer: Any) -> Any:
        """The stacked q/k/v projection (paired layout) of a few decode tokens, rotated and stored
        by the product's own kernel; returns ``q_buffer``, or None when the shape is not its kind
        (the caller then runs the product and ``rope_kv_write(..., paired=True)``)."""
        m, k = x.shape
        n = weight.shape[0]
        if (self._gemm_stream_rope is None or position is None or m > FUSED_RESIDUAL_MAX_ROWS
                or self.stream_plan(m, n, k, True) is None
                or not self.can_pair_rotary(head_dim, position.rotary_dim)):
            return None
        tiles, k_tiles = -(-n // 32), -(-k // 128)
        # K slices per block of weight rows (the size of a cluster): about two and a half CTAs an SM
        # was measured best for this small product (its successor, attention, cannot start beside it)
        splits = 8
        while splits > 1 and (2 * tiles * splits > 5 * self.sm_count or k_tiles // splits < 2):
            splits //= 2
        row_sq, row_tiles, eps = None, 0, 0.0
        if isinstance(x, NormedInput):
            row_sq, row_tiles, eps, x = x.accumulated.sq, x.accumulated.tiles, x.eps, x.accumulated.scaled
        table = ctx.block_tables[kv.group]
        if self.recording and weight.data_ptr() % 16 == 0 and x.data_ptr() % 16 == 0 and x.stride(0) % 8 == 0:
            self.program.rope(x, row_sq, row_tiles, eps, weight, bias, q_buffer, ctx.positions,
                              ctx.request_of_token, table, kv.num_pages, kv.k, kv.v, position.inv_freq, m,
                              q_heads, kv_heads, head_dim, position.rotary_dim, kv.page_size, write_cache, k)
            return q_buffer
        self._flush()
        self.launches += 1
        self._gemm_stream_rope(_ptr(x), _ptr(row_sq), row_tiles, eps, _ptr(weight), _ptr(bias),
                               _ptr(q_buffer), q_buffer.shape[1], _ptr(ctx.positions),
                               _ptr(ctx.request_of_token), _ptr(table), table.shape[1], kv.num_pages,
                               _ptr(kv.k), _ptr(kv.v), _ptr(position.inv_freq), m, q_heads, kv_heads,
                               head_dim, position.rotary_dim, kv.page_size, 1 if write_cache else 0, k,
                               splits, _ptr(self.error_word), self.stream)
        return q_buffer

    def attention(self, qkv: Any, out: Any, ctx: Any, kv: Any, q_heads: int, kv_heads: int,
                  head_dim: int, scale: float, window: int) -> None:
        fast = self._tensor_attention.get(head_dim)
        if fast is None:
            self._flush()
        if fast is not None:
            plan = ctx.extras.get(("attention", q_heads // kv_heads)) or None
            if fast.run(qkv, out, ctx, kv, q_heads, kv_heads, scale, window, plan):
                return
        self.attention_generic(qkv, out, ctx, kv, q_heads, kv_heads, head_dim, scale, window)

    def attention_generic(self, qkv: Any, out: Any, ctx: Any, kv: Any, q_heads: int,
                          kv_heads: int, head_dim: int, scale: float, window: int,
                          value_dim: int | None = None, distance: Any = None, few_tokens: bool = False,
                          keep_first: int = 0, sinks: Any = None) -> None:
        """``keep_first``: with a window, the request's first so many keys stay visible behind it.
        ``value_dim``: size of a value head when it is not ``head_dim``; ``distance``: (r1, r2),
        float32 [q_heads] each, of the penalty r1 * log(1 + r2 * (query position - key position)).
        ``sinks``: float32 [q_heads]; exp(sinks[h]) joins the softmax denominator of head h.
        ``few_tokens``: the rows are single tokens of a decode step; their keys are then cut into
        ranges with a CTA each where the device would otherwise stand mostly idle."""
        self._flush()
        table = ctx.block_tables[kv.group]
        self.launches += 1
        tokens = qkv.shape[0]
        splits, shares, tickets = 1, None, None
        if few_tokens:
            units = tokens * kv_heads * -(-(q_heads // kv_heads) // 8)
            keys = table.shape[1] * kv.page_size
            if window > 0:
                keys = min(keys, window + keep_first)
            # a range keeps at least 128 keys; no more CTAs than one an SM
            splits = max(1, min(keys // 128, self.sm_count // max(units, 1), 16))
            if splits > 1:
                shares = self.scratch("attention.shares", units * splits * self._group_share_floats)
                if self._group_tickets is None or self._group_tickets.numel() < units:
                    self._group_tickets = self.torch.zeros(max(units, 1024), dtype=self.torch.int32, device=self.device)
                    self.scratch_generation += 1
                tickets = self._group_tickets
        r1, r2 = distance if distance is not None else (None, None)
        self._attention_generic_sink(
            _ptr(qkv), qkv.shape[1], _ptr(out), out.shape[1], _ptr(kv.k), _ptr(kv.v), _ptr(ctx.positions),
            _ptr(ctx.request_of_token), _ptr(table), table.shape[1], kv.num_pages, tokens, q_heads, kv_heads,
            head_dim, value_dim or head_dim, kv.page_size, scale, window, _ptr(r1), _ptr(r2), splits,
            _ptr(shares), _ptr(tickets), int(keep_first), _ptr(sinks), self._code_of(qkv),
            _ptr(self.error_word), self.stream)

    def silu_mul(self, gate_up: Any, out: Any, block: int | None = None) -> None:
        self._flush()
        tokens, inter = out.shape
        self.launches += 1
        self._silu_mul(_ptr(gate_up), _ptr(out), tokens, inter, inter if block is None else block,
                       self._code_of(out), self.stream)

    def _load_sampling(self) -> None:
        if self._sample is None:
            v, i = c_void_p, c_int
            lib = _Lib(load_library("sampling.cu"))
            self._sample = lib.function("cie_sample", [v, i, i, v, v, v, v, v])
            self._feed_tokens = lib.function("cie_feed_tokens", [v, v, i, i, v])
            self._sample_slices = int(lib.handle.cie_sample_slices())

    def sample(self, logits: Any, temperature: Any, keys: Any, out: Any) -> None:
        """logits float32 [R, V]; temperature float32 [R] or None (greedy); keys int64 [R]."""
        self._flush()
        rows, vocab = logits.shape
        self._load_sampling()
        # the row maxima are searched by several CTAs a row first (two launches)
        scratch = self.scratch("sample.maxima", 2 * rows * self._sample_slices, reserve=2 * 1024 * self._sample_slices)
        self.launches += 2 if vocab >= 4096 else 1
        self._sample(_ptr(logits), rows, vocab, _ptr(temperature), _ptr(keys), _ptr(out), _ptr(scratch), self.stream)

    def feed_tokens(self, sampled: Any, token_ids: Any, real: int) -> None:
        """token_ids[i] = sampled[min(i, real - 1)] (int32, on the device): the token ids of a decode step
        that is launched before the step before it has been read back."""
        self._flush()
        self._load_sampling()
        self.launches += 1
        self._feed_tokens(_ptr(sampled), _ptr(token_ids), token_ids.shape[0], real, self.stream)
