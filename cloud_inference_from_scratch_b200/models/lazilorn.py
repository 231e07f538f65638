"""Lazilorn: from its typed configuration to a model description.

Token embedding times a constant plus a sinusoid of the position; pre-norm layers (RMS norm with a plain
gain) whose mixer is either two mixers side by side (softmax attention without rotation, with q and k
normalised per head, a sliding window that keeps the request's first tokens, and an output gate; and a matrix
memory with exponential gates) or the gated delta rule with short convolutions; an optional feed-forward
``W_down relu(W_up x)^2``; a final norm, a head of its own and a constant on the logits.  A run of
consecutive layers may be passed several times (``loop``): every pass is a further run of those layers in the
schedule, with a cache and a state of its own, and starts by adding its row of ``loop.step`` to the stream.

Tensor names: ``embed``, ``head``, ``final.norm``, ``loop.step``; per layer ``l<i>.`` + ``norm1``, ``norm2``,
``mix.*`` (``mix.left.*`` and ``mix.right.*`` for two mixers side by side), ``mlp.*``.
"""

from __future__ import annotations

from ..config.lazilorn_config import GatedDeltaConfig, LazilornConfig, ParallelMixerConfig
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MAX_POSITIONS = 1 << 20     # the design names no limit; positions and angles are float32
WAVE_BASE = 10000.0         # the sinusoid's frequencies are WAVE_BASE^(-2i / width)
LOOP_TENSOR = "loop.step"

ATTENTION_NAMES = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o",
                   "q_norm": "q.norm", "k_norm": "k.norm", "gate": "g"}


def _mixer(config: LazilornConfig, mixer: ParallelMixerConfig | GatedDeltaConfig) -> PartSpec:
    if isinstance(mixer, GatedDeltaConfig):
        return PartSpec("gated_delta", dict(hidden_size=config.width, num_heads=mixer.heads,
                                            num_kv_heads=mixer.kv_heads, key_dim=mixer.dim, value_dim=mixer.vdim,
                                            taps=mixer.conv, eps=config.norm_eps), prefix="mix.")
    left, right = mixer.left, mixer.right
    attention = PartSpec(
        "attention",
        dict(hidden_size=config.width, num_heads=left.heads, num_kv_heads=left.kv_heads, head_dim=left.dim,
             value_dim=left.vdim, qkv_bias=False, position=None, window=left.window, keep_first=left.keep_first,
             scale=left.scale, qk_norm="head", gate=True, norm_eps=config.norm_eps, names=ATTENTION_NAMES),
        prefix="left.")
    memory = PartSpec(
        "matrix_memory",
        dict(hidden_size=config.width, num_heads=right.heads, key_dim=right.dim, value_dim=right.vdim,
             gate_cap=right.gate_cap, eps=config.norm_eps),
        prefix="right.")
    return PartSpec("side_by_side", dict(left=attention, right=memory, left_scale=mixer.left_scale,
                                         right_scale=mixer.right_scale), prefix="mix.")


def lazilorn_spec(config: LazilornConfig) -> ModelSpec:
    norm = dict(hidden_size=config.width, eps=config.norm_eps, name="")
    layers: list[LayerSpec] = []
    for index, layer in enumerate(config.layers):
        parts = dict(mixer=_mixer(config, layer.mixer), mixer_norm=PartSpec("rmsnorm", norm, prefix="norm1"))
        if layer.mlp is not None:
            parts["feed_forward"] = PartSpec(
                "dense_activation", dict(hidden_size=config.width, intermediate_size=layer.mlp.ff, activation="relu2"),
                prefix="mlp.")
            parts["feed_forward_norm"] = PartSpec("rmsnorm", norm, prefix="norm2")
        layers.append(LayerSpec(prefix=f"l{index}.", block=PartSpec("prenorm_residual"), parts=parts))
    count = len(layers)
    loop = config.loop
    if loop is None:
        schedule = [ScheduleEntry(layer=i) for i in range(count)]
    else:
        schedule = [ScheduleEntry(layer=i) for i in range(loop.start)]
        for number in range(loop.times):
            schedule += [ScheduleEntry(layer=i, entry_offset=(LOOP_TENSOR, number) if i == loop.start else None)
                         for i in range(loop.start, loop.stop)]
        schedule += [ScheduleEntry(layer=i) for i in range(loop.stop, count)]
    return ModelSpec(
        architecture=config.architecture,
        vocab_size=config.vocab,
        hidden_size=config.width,
        embedding_tensor="embed",
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=PartSpec("rmsnorm", norm),
        final_norm_prefix="final.norm",
        head_tensor="head",
        max_positions=MAX_POSITIONS,
        eos_token_id=None,
        embedding_scale=config.embedding_scale,
        logit_scale=config.logit_scale,
        position_wave_base=WAVE_BASE,
        offset_tensors=((LOOP_TENSOR, loop.times),) if loop is not None else (),
    )


register_architecture("Lazilorn", "lazilorn", LazilornConfig.from_dict, lazilorn_spec, replace=True)
