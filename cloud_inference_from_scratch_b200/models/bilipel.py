"""Bilipel: from its typed configuration to a model description.

Token embedding; pre-norm layers (layer norm with gain and bias) whose mixer is softmax attention with grouped
key/value heads (q and k normalised over their whole projection, a part of every head rotated in rotate-half
pairs with blended frequencies, a sink term in the softmax), attention over a cached latent (interleaved rotary
pairs on a key part that all heads share, a sliding window, a sink term) or gated linear attention (a decay per
key channel read from the input); a feed-forward that is dense and gated (tanh form of GELU) or routed (softmax
over the chosen experts' logits), or none; every sublayer's result times one constant; a run of consecutive
layers may be passed several times (``loop``): every pass is a further run of those layers in the schedule, with
a cache and a state of its own, starts by adding its row of ``loop.step`` to the stream and, from the second
pass on, the embedding rows once more.  A final layer norm and a head of its own.

Tensor names: ``embed``, ``head``, ``final.norm`` (+ ``.b``), ``loop.step``; per layer ``l<i>.`` + ``norm1``,
``norm2`` (+ ``.b``), ``mix.*``, ``mlp.*``.
"""

from __future__ import annotations

from ..config.bilipel_config import BilipelConfig, GlaConfig, LatentMixerConfig, RotationConfig, SinkAttentionConfig
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MAX_POSITIONS = 1 << 20     # the design names no limit; positions and angles are float32
LOOP_TENSOR = "loop.step"

ATTENTION_NAMES = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o",
                   "q_norm": "q.norm", "k_norm": "k.norm", "sink": "sink"}
NORM_NAMES = {"weight": "", "bias": ".b"}


def _rotation(rot: RotationConfig, head_dim: int, pairing: str) -> PartSpec:
    return PartSpec("rope_neox", dict(head_dim=head_dim, rotary_dim=rot.dims, theta=rot.base,
                                      max_positions=MAX_POSITIONS, pairing=pairing, ramp=rot.scaling,
                                      keep_pairing=True))


def _mixer(config: BilipelConfig, mixer: SinkAttentionConfig | LatentMixerConfig | GlaConfig) -> PartSpec:
    if isinstance(mixer, GlaConfig):
        return PartSpec("gla", dict(hidden_size=config.width, num_heads=mixer.heads, key_dim=mixer.dim,
                                    value_dim=mixer.vdim, tau=mixer.tau, eps=config.norm_eps,
                                    decay_rank=mixer.decay_rank), prefix="mix.")
    if isinstance(mixer, LatentMixerConfig):
        return PartSpec(
            "latent_attention",
            dict(hidden_size=config.width, num_heads=mixer.heads, head_dim=mixer.dim, rot_dim=mixer.rot_dim,
                 value_dim=mixer.vdim, kv_rank=mixer.kv_rank, q_rank=0, scale=mixer.scale,
                 position=_rotation(mixer.rot, mixer.rot_dim, "interleaved"), norm_eps=config.norm_eps, sink=True,
                 window=mixer.window),
            prefix="mix.")
    return PartSpec(
        "attention",
        dict(hidden_size=config.width, num_heads=mixer.heads, num_kv_heads=mixer.kv_heads, head_dim=mixer.dim,
             value_dim=mixer.vdim, qkv_bias=False, position=_rotation(mixer.rot, mixer.dim, "half"),
             scale=mixer.scale, qk_norm="projection", sink=True, projection_float32=True,
             norm_eps=config.norm_eps, names=ATTENTION_NAMES),
        prefix="mix.")


def bilipel_spec(config: BilipelConfig) -> ModelSpec:
    norm = dict(hidden_size=config.width, eps=config.norm_eps, update_scale=config.residual_mult, names=NORM_NAMES)
    layers: list[LayerSpec] = []
    for index, layer in enumerate(config.layers):
        parts = dict(mixer=_mixer(config, layer.mixer), mixer_norm=PartSpec("layernorm", norm, prefix="norm1"))
        if layer.mlp is not None:
            if layer.mlp.kind == "dense":
                parts["feed_forward"] = PartSpec(
                    "gated_dense", dict(hidden_size=config.width, intermediate_size=layer.mlp.ff,
                                        activation="gelu_tanh"), prefix="mlp.")
            else:
                parts["feed_forward"] = PartSpec(
                    "routed_experts", dict(hidden_size=config.width, intermediate_size=layer.mlp.ff,
                                           num_experts=layer.mlp.experts, top=layer.mlp.top, correction=False,
                                           router_bias=True, score="chosen_softmax"), prefix="mlp.")
            parts["feed_forward_norm"] = PartSpec("layernorm", norm, prefix="norm2")
        layers.append(LayerSpec(prefix=f"l{index}.", block=PartSpec("prenorm_residual"), parts=parts))
    count = len(layers)
    loop = config.loop
    if loop is None:
        schedule = [ScheduleEntry(layer=i) for i in range(count)]
    else:
        schedule = [ScheduleEntry(layer=i) for i in range(loop.start)]
        for number in range(loop.times):
            for i in range(loop.start, loop.stop):
                first = i == loop.start
                schedule.append(ScheduleEntry(layer=i, entry_offset=(LOOP_TENSOR, number) if first else None,
                                              adds_embedding=first and number > 0))
        schedule += [ScheduleEntry(layer=i) for i in range(loop.stop, count)]
    return ModelSpec(
        architecture=config.architecture,
        vocab_size=config.vocab,
        hidden_size=config.width,
        embedding_tensor="embed",
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=PartSpec("layernorm", norm),
        final_norm_prefix="final.norm",
        head_tensor="head",
        max_positions=MAX_POSITIONS,
        eos_token_id=None,
        offset_tensors=((LOOP_TENSOR, loop.times),) if loop is not None else (),
        residual_scale=config.residual_mult,
    )


register_architecture("Bilipel", "bilipel", BilipelConfig.from_dict, bilipel_spec, replace=True)
