"""The Bilipel configuration reader, its model description, its tensor names, its run order and the plain
implementation's own small checks (no GPU)."""

import copy
import math

import pytest
import torch

import plain_bilipel as plain
from cloud_inference_from_scratch_b200 import models, parts  # noqa: F401  (registries)
from cloud_inference_from_scratch_b200.config import ConfigError, resolve_config
from cloud_inference_from_scratch_b200.config.bilipel_config import BilipelConfig
from cloud_inference_from_scratch_b200.models import DecoderModel


def raw_config():
    rot = dict(base=3000.0, dims=4, scaling=dict(factor=4.0, original=64, fast=8.0, slow=0.5))
    attention = dict(heads=6, kv_heads=3, dim=8, vdim=10, scale=0.3, rot=rot)
    latent = dict(heads=3, dim=8, rot_dim=6, vdim=5, kv_rank=24, scale=0.25, rot=dict(base=500.0, dims=6),
                  mask=dict(size=7))
    gla = dict(heads=2, dim=12, vdim=10, tau=8.0, decay_rank=5)
    moe = dict(kind="moe", expert=dict(ff=16), router=dict(experts=5, top=2))
    return dict(architecture="Bilipel", vocab=50, width=24, norm=dict(eps=1e-5), residual_mult=0.5,
                loop=dict(start=1, stop=3, times=3),
                layers=[dict(type="attention", mixer=attention, mlp=dict(kind="dense", ff=14)),
                        dict(type="gla", mixer=gla, mlp=moe),
                        dict(type="latent_attention", mixer=latent, mlp=None),
                        dict(type="latent_attention", mixer=dict(latent, heads=2, mask=None), mlp=moe)])


def test_reads_back_what_it_wrote_and_is_found_by_its_name():
    raw = raw_config()
    del raw["layers"][3]["mixer"]["mask"]
    arch, config, spec = resolve_config(raw)
    assert arch.name == "Bilipel" and isinstance(config, BilipelConfig)
    assert BilipelConfig.from_dict(config.to_dict()) == config and config.to_dict() == raw
    assert spec.residual_scale == 0.5 and spec.offset_tensors == (("loop.step", 3),)


def test_run_order_of_a_loop():
    """Every pass names the looped layers again; its first run adds its row of the offsets, and from the second
    pass on the embedding rows too."""
    _, _, spec = resolve_config(raw_config())
    got = [(entry.layer, entry.entry_offset, entry.adds_embedding) for entry in spec.schedule]
    step = "loop.step"
    assert got == [(0, None, False),
                   (1, (step, 0), False), (2, None, False),
                   (1, (step, 1), True), (2, None, False),
                   (1, (step, 2), True), (2, None, False),
                   (3, None, False)]
    assert [(layer, number) for layer, number in plain.run_order(raw_config())] == [
        (0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    raw = raw_config()
    del raw["loop"]
    spec = resolve_config(raw)[2]
    assert [entry.layer for entry in spec.schedule] == [0, 1, 2, 3] and spec.offset_tensors == ()


def test_tensor_names_shapes_and_caches():
    _, _, spec = resolve_config(raw_config())
    model = DecoderModel(spec)
    table = model.tensor_table()
    assert table["embed"].shape == (50, 24) and table["head"].shape == (50, 24)
    assert table["final.norm"].shape == (24,) and table["final.norm.b"].shape == (24,) and table["loop.step"].shape == (3, 24)
    assert table["l0.norm1"].shape == (24,) and table["l0.norm1.b"].shape == (24,) and table["l0.norm2.b"].shape == (24,)
    assert table["l0.mix.q"].shape == (48, 24) and table["l0.mix.k"].shape == (24, 24) and table["l0.mix.v"].shape == (30, 24)
    assert table["l0.mix.q.norm"].shape == (48,) and table["l0.mix.k.norm"].shape == (24,)
    assert table["l0.mix.sink"].shape == (6,) and table["l0.mix.o"].shape == (24, 60)
    assert table["l0.mlp.gate"].shape == (14, 24) and table["l0.mlp.up"].shape == (14, 24) and table["l0.mlp.down"].shape == (24, 14)
    assert table["l1.mix.q"].shape == (24, 24) and table["l1.mix.v"].shape == (20, 24) and table["l1.mix.g"].shape == (20, 24)
    assert table["l1.mix.a1"].shape == (5, 24) and table["l1.mix.a2"].shape == (24, 5) and table["l1.mix.a2.b"].shape == (24,)
    assert table["l1.mix.norm"].shape == (10,) and table["l1.mix.o"].shape == (24, 20)
    assert table["l1.mlp.router"].shape == (5, 24) and table["l1.mlp.router.b"].shape == (5,)
    assert table["l1.mlp.e4.gate"].shape == (16, 24) and table["l1.mlp.e0.down"].shape == (24, 16) and "l1.mlp.e5.up" not in table
    assert table["l2.mix.q"].shape == (42, 24) and table["l2.mix.dkv"].shape == (30, 24) and table["l2.mix.dkv.norm"].shape == (24,)
    assert table["l2.mix.uk"].shape == (24, 24) and table["l2.mix.uv"].shape == (15, 24) and table["l2.mix.sink"].shape == (3,)
    assert "l2.mix.dq" not in table and "l2.mix.uq" not in table and "l2.norm2" not in table
    assert not any(name.startswith("l2.mlp") for name in table)
    needs = model.cache_needs()
    assert [need.owner for need in needs] == list(range(8))        # every run, looped ones too, keeps its own
    assert (needs[0].pages.kv_heads, needs[0].pages.head_dim, needs[0].pages.value_size, needs[0].pages.window) == (3, 8, 10, 0)
    assert needs[1].pages is None and needs[1].state.shape == (2, 12, 10) and needs[3].state.shape == (2, 12, 10)
    assert (needs[2].pages.kv_heads, needs[2].pages.head_dim, needs[2].pages.value_size, needs[2].pages.window) == (1, 24, 6, 7)
    assert needs[7].pages.window == 0


def test_the_decay_width_may_be_left_to_the_file():
    raw = raw_config()
    del raw["layers"][1]["mixer"]["decay_rank"]
    table = DecoderModel(resolve_config(raw)[2]).tensor_table()
    assert table["l1.mix.a1"].shape == (-1, 24) and table["l1.mix.a2"].shape == (24, -1)


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="conv"), "mixer type"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "more than a head"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=3), "even"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=4), "must equal"),
    (lambda c: c["layers"][1]["mixer"].update(tau=0), "positive"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=6), "more than"),
    (lambda c: c["layers"][0]["mlp"].update(kind="conv"), "not built"),
    (lambda c: c["loop"].update(stop=5), "loop"),
    (lambda c: c.pop("width"), "width"),
])
def test_refusals(change, message):
    raw = copy.deepcopy(raw_config())
    change(raw)
    with pytest.raises(ConfigError, match=message):
        BilipelConfig.from_dict(raw)


def test_plain_mechanisms_against_their_definitions():
    """The oracle's own pieces on inputs whose answer is known."""
    g = torch.Generator().manual_seed(1)
    x = torch.randn(3, 10, generator=g, dtype=torch.float64)
    y = plain.layer_norm(x, torch.ones(10, dtype=torch.float64), torch.zeros(10, dtype=torch.float64), 0.0)
    assert torch.allclose(y.mean(-1), torch.zeros(3, dtype=torch.float64), atol=1e-12)
    assert torch.allclose((y * y).mean(-1), torch.ones(3, dtype=torch.float64), atol=1e-12)
    # a sink far below every score changes nothing; a sink far above takes all the weight
    scores = torch.randn(4, 4, generator=g, dtype=torch.float64)
    seen = plain.visibility(4)
    plain_softmax = torch.softmax(scores.masked_fill(~seen, -math.inf), -1)
    assert torch.allclose(plain.softmax_with_sink(scores, seen, torch.tensor(-200.0, dtype=torch.float64)), plain_softmax)
    assert plain.softmax_with_sink(scores, seen, torch.tensor(200.0, dtype=torch.float64)).max() < 1e-60
    # a sink equal to the only score halves the first token's weight
    assert math.isclose(float(plain.softmax_with_sink(scores, seen, scores[0, 0])[0, 0]), 0.5)
    assert plain.visibility(6, 2).sum(-1).tolist() == [1, 2, 2, 2, 2, 2]
    # a decay of one keeps everything: the recurrence is a running sum of k v^T
    q, k = torch.randn(5, 2, 3, generator=g, dtype=torch.float64), torch.randn(5, 2, 3, generator=g, dtype=torch.float64)
    v = torch.randn(5, 2, 4, generator=g, dtype=torch.float64)
    out = plain.gla_recurrence(q, k, v, torch.ones(5, 2, 3, dtype=torch.float64))
    want = torch.einsum("thd,shd,shv->tshv", q, k, v)
    want = torch.stack([want[t, : t + 1].sum(0) for t in range(5)])
    assert torch.allclose(out, want)
    # the rotation keeps lengths (times the magnitude) and turns pair i by position * f_i
    rot = dict(base=100.0, dims=4, scaling=dict(factor=3.0, original=16, fast=4.0, slow=0.5))
    head = torch.randn(7, 1, 6, generator=g, dtype=torch.float64)
    freq, magnitude = plain.rotary_frequencies(rot)
    for interleaved in (False, True):
        turned = plain.rotate(head, torch.arange(7), rot, interleaved)
        assert torch.allclose(turned[..., 4:], head[..., 4:])
        assert torch.allclose(turned[..., :4].norm(dim=-1), head[..., :4].norm(dim=-1) * magnitude)
    assert math.isclose(magnitude, 0.1 * math.log(3.0) + 1.0)
