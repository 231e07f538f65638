"""The Bilipel design in the engine against the plain implementation of ``plain_bilipel.py``: each mechanism
alone, whole prompts against decoding, portions down to two tokens, unequal batches, pages and state slots that
are used again, window and page edges, far keys, first tokens, long decoding, sizes of every kind, and greedy
generation through the public entry point."""

import json
import math
import subprocess
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_bilipel as plain
from helpers import peak_tokens, random_tokens, replay, requests_in, trace_mixed, trace_portions, trace_tail, trace_whole

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
F = torch.float64

# worst |logit difference| of a row over the standard deviation of the request's reference logits
GATE = {"float32": 2e-4, "bfloat16": 0.1}


# ------------------------------------------------------------------ configurations
def attention(heads=4, kv_heads=2, dim=16, vdim=24, rot_dims=8, scale=0.3, base=1000.0, scaling=True):
    rot = dict(base=base, dims=rot_dims)
    if scaling:
        rot["scaling"] = dict(factor=4.0, original=32, fast=8.0, slow=0.5)
    return dict(type="attention", mixer=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, rot=rot))


def latent(heads=3, dim=8, rot_dim=4, vdim=12, kv_rank=20, window=9, scale=0.3, base=300.0):
    mixer = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, scale=scale,
                 rot=dict(base=base, dims=rot_dim))
    if window:
        mixer["mask"] = dict(size=window)
    return dict(type="latent_attention", mixer=mixer)


def gla(heads=2, dim=12, vdim=20, tau=4.0, rank=5):
    return dict(type="gla", mixer=dict(heads=heads, dim=dim, vdim=vdim, tau=tau, decay_rank=rank))


def dense(layer, ff=40):
    return dict(layer, mlp=dict(kind="dense", ff=ff))


def moe(layer, ff=16, experts=5, top=2):
    return dict(layer, mlp=dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top)))


def bare(layer):
    return dict(layer, mlp=None)


def config(layers, width=64, vocab=211, loop=None, eps=1e-5, mult=0.5):
    raw = dict(architecture="Bilipel", vocab=vocab, width=width, norm=dict(eps=eps), residual_mult=mult,
               layers=list(layers))
    if loop is not None:
        raw["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
    return raw


CONFIGS = {
    # all three mixers, a loop over the middle that is passed three times, value sizes unlike key sizes, every
    # kind of feed-forward and none
    "mixed": config([dense(attention()), moe(latent()), bare(gla()), moe(attention(heads=2, kv_heads=2, rot_dims=16, scaling=False)),
                     dense(latent(window=0))], loop=(1, 4, 3)),
    # no loop; every query head its own key head; the whole head rotated; a window of one key; one expert of one;
    # a constant of one on the sublayers
    "plain": config([moe(gla(heads=1, dim=16, vdim=16, tau=1.0, rank=3), ff=24, experts=1, top=1),
                     dense(attention(heads=2, kv_heads=2, dim=32, vdim=32, rot_dims=32, scale=0.2), ff=32),
                     bare(latent(heads=1, dim=16, rot_dim=16, vdim=16, kv_rank=16, window=1))],
                    width=48, vocab=130, mult=1.0),
    # one key head; sizes that are no multiples of eight; the whole model looped; all experts chosen
    "narrow": config([moe(attention(heads=3, kv_heads=1, dim=20, vdim=12, rot_dims=6, scale=0.5), ff=10, experts=3, top=3),
                      dense(latent(heads=5, dim=6, rot_dim=10, vdim=7, kv_rank=18, window=5), ff=7),
                      bare(gla(heads=3, dim=10, vdim=6, tau=16.0, rank=2))],
                     width=36, vocab=77, loop=(0, 3, 2), eps=1e-6, mult=0.35),
    # sizes that the tensor-core kernels take: heads of 64 with values as large, a latent of 64 + 32, sixteen
    # latent heads, keys and values of 64 and 128 for the chunked recurrence, a window over several key tiles and
    # one longer than any request
    "tiles": config([moe(attention(heads=4, kv_heads=2, dim=64, vdim=64, rot_dims=32, scale=0.15), ff=32, experts=8, top=2),
                     dense(latent(heads=16, dim=32, rot_dim=32, vdim=32, kv_rank=64, window=70, scale=0.15), ff=64),
                     bare(gla(heads=2, dim=64, vdim=128, tau=16.0, rank=16)),
                     dense(latent(heads=4, dim=16, rot_dim=8, vdim=16, kv_rank=32, window=400), ff=32)],
                    width=128, loop=(1, 3, 2)),
    # no attention at all: no pages, only state slots
    "recurrent": config([dense(gla(heads=2, dim=16, vdim=16), ff=16), moe(gla(heads=2, dim=8, vdim=24, tau=2.0))],
                        width=32, vocab=90, loop=(1, 2, 3)),
}
PAGE = {"mixed": 4, "plain": 16, "narrow": 8, "tiles": 16, "recurrent": 8}
# N(0, 0.05) weights leave sinks, biases, offsets and decays close to nothing
SCALES = {"embed": 10.0, "head": 6.0, "sink": 30.0, "a2.b": 40.0, "mix.a1": 4.0, "mix.a2": 8.0, "loop.step": 10.0,
          "mix.q": 2.0, "mix.k": 2.0, "mix.v": 2.0, "mlp.router": 8.0, "router.b": 10.0, "norm1.b": 4.0, "norm2.b": 4.0,
          "final.norm.b": 4.0, "mlp.e": 3.0}
# the bfloat16 runs of whole models let the stored bias alone choose the experts (the router still sets the
# weights): with the choice left to the logits, one token in ten has two experts within bfloat16 rounding of each
# other and goes either way
SCALES_BF16 = dict(SCALES, **{"router.b": 2000.0, "mlp.router": 4.0})


def make_model(folder, raw, seed, std=0.05, scales=None):
    from cloud_inference_from_scratch_b200.weights import write_random_model

    return write_random_model(folder, raw, seed, std=std, scales=scales or SCALES)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("bilipel")
    out = {}
    for index, (name, raw) in enumerate(CONFIGS.items()):
        out[name, "float32"] = make_model(root / name, raw, 5 + index)
        out[name, "bfloat16"] = make_model(root / (name + "-fixed"), raw, 5 + index, scales=SCALES_BF16)
    return out


def core_for(folder, dtype, page, pages, slots=4, step_tokens=0):
    from cloud_inference_from_scratch_b200.engine.core import build_core

    return build_core(folder, dtype=dtype, page_size=page, num_pages=pages, max_requests=slots,
                      max_model_len=pages * page, max_tokens_per_step=step_tokens)


PLAIN_LOGITS = {}


def plain_logits(folder, tokens, round_inputs=False):
    key = (str(folder), tuple(tokens), round_inputs)
    if key not in PLAIN_LOGITS:
        raw, tensors = plain.read_folder(folder)
        PLAIN_LOGITS[key] = plain.forward(raw, tensors, tokens, round_inputs=round_inputs).numpy()
    return PLAIN_LOGITS[key]


def check(folder, got, dtype, gate=None, skip_what_rounding_decides=False):
    """Every row against the plain model run on the whole request.  ``skip_what_rounding_decides`` (bfloat16 only,
    where float32 has held every row to a far sharper gate): positions whose plain logits move by more than a
    quarter of the gate when the sublayers' inputs are rounded to bfloat16 and everything else stays exact are
    not held to it; there a recurrent head's output is nearly nothing before its norm (its query at right angles
    to the few keys written so far), and the norm blows the rounding up."""
    limit = gate or GATE[dtype]
    worst = 0.0
    for rid, tokens in got["fed"].items():
        ref = plain_logits(folder, tokens)
        rows = got["logits"][rid]
        assert sorted(rows) == list(range(len(tokens))), f"{rid}: positions missing"
        mine = np.stack([rows[p] for p in range(len(tokens))])
        errors = np.abs(mine - ref).max(axis=1) / ref.std()
        if skip_what_rounding_decides:
            moved = np.abs(plain_logits(folder, tokens, True) - ref).max(axis=1) / ref.std() > limit / 4
            assert moved.sum() <= max(4, len(tokens) // 4), f"{rid}: rounding decides {int(moved.sum())} rows"
            errors = np.where(moved, 0.0, errors)
        worst = max(worst, float(errors.max()))
        assert errors.max() <= limit, (
            f"{rid}: first wrong position {int(np.argmax(errors > limit))} of {len(tokens)}, error {errors.max():.3e}")
    return worst


def run_trace(core, steps):
    return {"logits": replay(core, steps), "fed": requests_in(steps)}


def requests_for(raw, lengths, seed):
    return {f"r{i}": random_tokens(raw["vocab"], n, seed + i) for i, n in enumerate(lengths)}


# ------------------------------------------------------------------ the whole model, every cutting
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompts_decoding_portions_and_batches(folders, name, dtype):
    page, folder = PAGE[name], folders[name, dtype]
    # lengths: one token, two, a page's edge and one past it, several windows, several pages and chunks
    requests = requests_for(CONFIGS[name], [1, 2, page, page + 1, 23, 61, 97], seed=10)
    for steps in (trace_whole(requests), trace_tail(requests, tail=40), trace_portions(requests),
                  trace_mixed(requests, seed=3, live_limit=3)):
        # a pool that holds what is live and no more, and three slots: pages and slots come back
        pages = -(-peak_tokens(steps, round_to=page) // page) + 1
        core = core_for(folder, dtype, page, pages, slots=3)
        check(folder, run_trace(core, steps), dtype, skip_what_rounding_decides=dtype == "bfloat16")
        assert core.cache.free_pages(0) == core.cache.total_pages(0)


def drawn_configuration(seed):
    """A configuration drawn from the whole space of sizes: widths, any layer kind in any order, head counts, key
    and value sizes (multiples of 8 and 16 and others, above and below what the chunked and tensor-core kernels
    take), rotated parts from two elements to the whole head with and without blended frequencies, windows from
    one key to more than a request has or none, latent sizes, decay temperatures and inner widths, experts from
    one to many with one to all chosen, layers without feed-forward, loops anywhere or none, any constant on the
    sublayers."""
    import random

    rng = random.Random(seed)
    layers = []
    for _ in range(rng.randint(1, 5)):
        kind = rng.choice(["attention", "latent", "gla"])
        if kind == "attention":
            kv, group = rng.choice([1, 2, 4]), rng.choice([1, 2, 3, 8])
            dim = rng.choice([8, 16, 24, 32, 48, 64, 96, 128])
            vdim = dim if rng.random() < 0.5 else rng.choice([8, 16, 40, 64, 128, 160])
            layer = attention(kv * group, kv, dim, vdim, rng.choice([2, dim // 2, dim]) // 2 * 2,
                              rng.choice([0.4, 1.2, 3.0]) / dim ** 0.5, rng.choice([100.0, 10000.0, 500000.0]),
                              rng.random() < 0.5)
        elif kind == "latent":
            rot_dim, dim = rng.choice([2, 8, 16, 32, 64]), rng.choice([4, 16, 32, 64, 128])
            layer = latent(rng.choice([1, 2, 5, 8, 16, 20]), dim, rot_dim,
                           rng.choice([8, 32, 64, 100]), rng.choice([8, 24, 64, 96, 256, 520]),
                           rng.choice([0, 1, 2, 5, 16, 17, 33, 64, 100, 500]),
                           rng.choice([0.4, 1.2, 3.0]) / (dim + rot_dim) ** 0.5, rng.choice([100.0, 10000.0]))
        else:
            layer = gla(rng.choice([1, 2, 3, 8]), rng.choice([4, 16, 32, 64, 128, 160]), rng.choice([8, 32, 64, 128, 136]),
                        rng.choice([1.0, 4.0, 16.0]), rng.choice([1, 4, 16, 24]))
        feed = rng.choice(["none", "dense", "moe", "moe"])
        if feed == "dense":
            layer = dense(layer, rng.choice([8, 24, 100]))
        elif feed == "moe":
            experts = rng.choice([1, 2, 4, 8, 13])
            layer = moe(layer, rng.choice([8, 16, 24, 40]), experts, rng.randint(1, min(experts, 4)))
        else:
            layer = bare(layer)
        layers.append(layer)
    loop = None
    if rng.random() < 0.7:
        start = rng.randrange(len(layers))
        loop = (start, rng.randint(start + 1, len(layers)), rng.randint(1, 3))
    return config(layers, width=rng.choice([64, 96, 128, 256]), vocab=rng.choice([50, 211, 450]), loop=loop,
                  eps=rng.choice([1e-6, 1e-5]), mult=rng.choice([0.25, 0.5, 1.0, 1.4]))


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6, 7, 8])
def test_drawn_configurations(seed, tmp_path):
    raw = drawn_configuration(seed)
    requests = requests_for(raw, [1, 2, 37, 150], seed=seed)
    for dtype, scales, gate in (("float32", SCALES, 4e-4), ("bfloat16", SCALES_BF16, 0.2)):
        folder = make_model(tmp_path / dtype, raw, 100 + seed, scales=scales)
        for steps in (trace_whole(requests), trace_mixed(requests, seed=seed, live_limit=3)):
            pages = -(-peak_tokens(steps, round_to=16) // 16) + 1
            core = core_for(folder, dtype, 16, pages, slots=3)
            check(folder, run_trace(core, steps), dtype, gate=gate, skip_what_rounding_decides=dtype == "bfloat16")


def test_float32_rows_do_not_depend_on_the_cut_or_the_batch(folders):
    """The same position through four cuttings: equal to rounding of the order of additions at most."""
    raw = CONFIGS["mixed"]
    requests = requests_for(raw, [50, 31, 77], seed=40)
    seen = []
    for steps in (trace_whole(requests), trace_tail(requests, tail=20), trace_portions(requests),
                  trace_mixed(requests, seed=9, live_limit=3)):
        core = core_for(folders["mixed", "float32"], "float32", 4, 64, slots=3)
        seen.append(replay(core, steps))
    for rid, tokens in requests.items():
        base = np.stack([seen[0][rid][p] for p in range(len(tokens))])
        for other in seen[1:]:
            mine = np.stack([other[rid][p] for p in range(len(tokens))])
            assert np.abs(mine - base).max() <= 5e-5 * base.std()


def test_long_decoding_past_windows_and_pages(folders):
    """160 tokens decoded one by one after a short prompt: the window passes over decoded tokens many times, pages
    behind it are given back, and the recurrent state is carried for every token."""
    for name in ("mixed", "narrow"):
        requests = requests_for(CONFIGS[name], [170, 165], seed=70)
        steps = trace_tail(requests, tail=160)
        for dtype in ("float32", "bfloat16"):
            core = core_for(folders[name, dtype], dtype, PAGE[name], 400 // PAGE[name], slots=2)
            check(folders[name, dtype], run_trace(core, steps), dtype, skip_what_rounding_decides=dtype == "bfloat16")


def test_a_state_slot_that_is_used_again_starts_from_zero(folders):
    """One slot only: every request inherits the slot of the one before it."""
    for name in ("plain", "recurrent"):
        requests = requests_for(CONFIGS[name], [30, 8, 19], seed=90)
        core = core_for(folders[name, "float32"], "float32", 16, 4, slots=1)
        check(folders[name, "float32"], run_trace(core, trace_portions(requests)), "float32")


# ------------------------------------------------------------------ mechanisms alone
def runtime(dtype):
    from cloud_inference_from_scratch_b200.engine.runtime import Runtime

    return Runtime("cuda:0", dtype)


def rand(*shape, scale=1.0, seed=0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def close(got, want, dtype, scale=None, loose=3e-2, tight=2e-5):
    want = want.double().cpu()
    error = float((got.double().cpu() - want).abs().max() / (scale or want.std()))
    assert error <= (tight if dtype == "float32" else loose), error


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [40, 33, 192, 2048, 9000])
def test_layer_norm_adds_the_scaled_update_into_the_stream(dtype, width):
    """A mean far from zero beside a small spread (the variance is taken from the deviations), an update of one
    float32 term, of two, of the compute dtype and none, all rows and selected rows."""
    from cloud_inference_from_scratch_b200.lazy import Partials

    rt = runtime(dtype)
    rows, eps, mult = 6, 1e-5, 0.6
    stream = rand(rows, width, seed=1) * 0.1 + 7.0
    gain, bias = 1 + rand(width, scale=0.2, seed=2), rand(width, scale=0.5, seed=3)
    first, second = rand(rows, width, seed=4), rand(rows, width, seed=5)
    both = torch.stack([first, second]).cuda().contiguous()
    cases = [(None, None), (first.cuda(), first), (Partials(both, 2, rows, width, None), first + second),
             (first.to(rt.dtype).cuda(), first.to(rt.dtype))]
    for update, added in cases:
        residual = stream.clone().cuda()
        out = torch.empty(rows, width, dtype=rt.dtype).cuda()
        rt.ops.add_layernorm(residual, update, gain.cuda(), bias.cuda(), eps, out, update_scale=mult)
        total = stream.double() + (mult * added.double() if added is not None else 0.0)
        close(residual, total, "float32", scale=1.0, tight=2e-6)
        close(out, plain.layer_norm(total, gain.double(), bias.double(), eps), dtype, scale=1.0, tight=1e-4)
        # selected rows: nothing is written back
        residual = stream.clone().cuda()
        chosen = torch.tensor([4, 0, 4], dtype=torch.int32).cuda()
        picked = torch.empty(3, width, dtype=rt.dtype).cuda()
        rt.ops.add_layernorm(residual, update, gain.cuda(), bias.cuda(), eps, picked, chosen, update_scale=mult)
        assert torch.equal(residual.cpu(), stream)
        close(picked, plain.layer_norm(total, gain.double(), bias.double(), eps)[[4, 0, 4]], dtype, scale=1.0, tight=1e-4)


def test_rows_added_before_a_pass():
    """The stream takes the scaled pending update, the embedding rows once more and the pass's own vector."""
    rt = runtime("float32")
    stream, update, base, vector = rand(5, 70, seed=1), rand(5, 70, seed=2), rand(5, 70, seed=3), rand(70, seed=4)
    for use_update, use_base, use_vector in [(1, 1, 1), (0, 1, 1), (1, 0, 1), (1, 1, 0), (0, 0, 1)]:
        residual = stream.clone().cuda()
        rt.ops.add_rows(residual, update.cuda() if use_update else None, vector.cuda() if use_vector else None,
                        base=base.cuda() if use_base else None, scale=0.6)
        want = stream.double() + 0.6 * update.double() * use_update + base.double() * use_base + vector.double() * use_vector
        close(residual, want, "float32", scale=1.0, tight=1e-6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gated_activations(dtype):
    rt = runtime(dtype)
    both = rand(7, 2 * 37, scale=3.0, seed=1)
    for kind, act in (("gelu_tanh", plain.gelu_tanh), ("silu", plain.silu)):
        out = torch.empty(7, 37, dtype=rt.dtype).cuda()
        rt.ops.glu_act(both.cuda(), out, kind)
        want = act(both[:, :37].double()) * both[:, 37:].double()
        close(out, want, dtype, scale=float(want.abs().max()), loose=5e-3, tight=1e-6)


def fake_step(lengths, contexts, page, dtype, heads, dim, vdim, seed=0):
    """Positions, tables and empty pools for requests that hold ``contexts`` tokens and bring ``lengths``."""
    total = [c + n for c, n in zip(contexts, lengths)]
    pages_per = [-(-t // page) for t in total]
    order = torch.randperm(sum(pages_per) + 2, generator=torch.Generator().manual_seed(seed)).tolist()
    table = torch.full((len(lengths), max(pages_per)), -1, dtype=torch.int32)
    cursor = 0
    for r, count in enumerate(pages_per):
        table[r, :count] = torch.tensor(order[cursor:cursor + count], dtype=torch.int32)
        cursor += count
    positions = torch.cat([torch.arange(c, c + n) for c, n in zip(contexts, lengths)]).int()
    request_of = torch.cat([torch.full((n,), r) for r, n in enumerate(lengths)]).int()
    kv = SimpleNamespace(group=0, num_pages=len(order), page_size=page,
                         k=torch.zeros(len(order), heads, page, dim, dtype=dtype).cuda(),
                         v=torch.zeros(len(order), heads, page, vdim, dtype=dtype).cuda())
    singles = 0
    while singles < len(lengths) and lengths[singles] == 1:
        singles += 1
    starts = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    ctx = SimpleNamespace(positions=positions.cuda(), request_of_token=request_of.cuda(),
                          block_tables=[table.cuda()], num_requests=len(lengths), num_single=singles, extras={},
                          context_lens=torch.tensor(contexts, dtype=torch.int32).cuda(),
                          query_lens=torch.tensor(lengths, dtype=torch.int32).cuda(),
                          query_start=torch.from_numpy(starts).cuda(),
                          slots=torch.arange(len(lengths), dtype=torch.int32).cuda(),
                          request_active=torch.ones(len(lengths), dtype=torch.int32).cuda(),
                          host=SimpleNamespace(query_lens=np.asarray(lengths, dtype=np.int32), num_single=singles,
                                               num_requests=len(lengths),
                                               query_start=starts))
    return ctx, kv


def plan_into(ctx, rt, group):
    plan = rt.ops.plan_attention(ctx.host, group)
    if plan:
        ctx.extras[("attention", group)] = {name: torch.from_numpy(np.asarray(a)).cuda() for name, a in plan.items()}


def rotation_of(rot, interleaved):
    freq, magnitude = plain.rotary_frequencies(rot)
    return SimpleNamespace(inv_freq=freq.float().cuda(), magnitude=magnitude, interleaved=interleaved, dims=rot["dims"])


def softmax_rows(q, k, v, scale, sink, window=0, offset=0):
    """q [n, heads, d] at positions offset.. against all of k, v [m, groups, *]: plain attention with a sink."""
    n, heads, _ = q.shape
    m, groups, _ = k.shape
    i = torch.arange(offset, offset + n).view(-1, 1)
    j = torch.arange(m).view(1, -1)
    seen = j <= i
    if window:
        seen &= (i - j) < window
    out = []
    for head in range(heads):
        group = head // (heads // groups)
        weights = plain.softmax_with_sink(q[:, head] @ k[:, group].T * scale, seen, sink[head])
        out.append(weights @ v[:, group])
    return torch.stack(out, 1)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim,vdim,rot_dims", [(16, 24, 8), (64, 64, 16), (20, 12, 20), (128, 128, 64)])
def test_attention_norm_rotation_sink_and_one_far_key_that_stands_out(dtype, dim, vdim, rot_dims):
    """float32 q, k, v go through the norm over the whole projection and the rotation into pages; then, for the
    last query of a request of 300 tokens, one key far back (and, in turn, the first key, one at a page's edge and
    the query's own) is turned along that query so that it takes nearly all the weight against a sink that would
    take it otherwise.  Prompt, a portion over cached keys, and single tokens."""
    rt = runtime(dtype)
    heads, groups, page, eps, scale = 4, 2, 16, 1e-5, 1.7 / dim ** 0.5
    rot = dict(base=1000.0, dims=rot_dims, scaling=dict(factor=4.0, original=64, fast=8.0, slow=0.5))
    n = 300
    rt.ops.require_attention(dim)
    width = heads * dim + groups * (dim + vdim)
    q_gain, k_gain = 1 + rand(heads * dim, scale=0.2, seed=3), 1 + rand(groups * dim, scale=0.2, seed=4)
    sink = torch.tensor([4.0, -3.0, 0.5, 9.0])
    for edge in (0, 37, page * 9 - 1, page * 9, n - 1):
        qkv = rand(n, width, seed=1)
        # the key of group 0 at `edge`, after norm and rotation, points along head 0 of the last query: un-rotate it
        full = qkv.double()
        q = plain.rms_norm(full[:, :heads * dim], q_gain.double(), eps).view(n, heads, dim)
        q = plain.rotate(q, torch.arange(n), rot, False)
        target = plain.rotate(q[n - 1:n, :1], torch.tensor([-edge]), rot, False)      # turned back by the key's position
        qkv[edge, heads * dim:heads * dim + dim] = (target[0, 0] / k_gain[:dim].double() * 30.0 / target.norm()).float()
        full = qkv.double()
        k = plain.rms_norm(full[:, heads * dim:heads * dim + groups * dim], k_gain.double(), eps).view(n, groups, dim)
        k = plain.rotate(k, torch.arange(n), rot, False)
        v = full[:, heads * dim + groups * dim:].view(n, groups, vdim)
        want = softmax_rows(q, k, v, scale, sink.double())
        for lengths, contexts in (([n], [0]), ([n - 250], [250]), ([1], [n - 1])):
            # what the request holds already goes into the pages by a step of its own
            ctx, kv = fake_step([n], [0], page, rt.dtype, groups, dim, vdim, seed=2)
            held = contexts[0]
            q_all = torch.empty(n, heads * dim, dtype=rt.dtype).cuda()
            rt.ops.norm_kv_write(qkv.cuda(), ctx, kv, heads, groups, dim, vdim, q_gain.cuda(), k_gain.cuda(), False, eps,
                                 q_all, rotation=rotation_of(rot, False))
            step, _ = fake_step(lengths, contexts, page, rt.dtype, groups, dim, vdim, seed=2)
            plan_into(step, rt, heads // groups)
            out = torch.empty(n - held, heads * vdim, dtype=rt.dtype).cuda()
            rt.ops.attention_penalised(q_all[held:].contiguous(), out, step, kv, heads, groups, dim, vdim, scale, 0, None,
                                       sinks=sink.cuda())
            rt.ops.check_errors()
            # the key that stands out scores up to 40: float32 rounding of that score moves its weight by 1e-5
            close(out.view(n - held, heads, vdim), want[held:], dtype, scale=1.0, loose=6e-2, tight=1e-4)
        # float32 angles: at position 300 the angle carries an error of 300 * 2^-24
        close(q_all.view(n, heads, dim), q, dtype, scale=1.0, loose=4e-2, tight=1e-4)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,rank,rot_dim", [(3, 20, 4), (16, 64, 32), (8, 96, 32), (5, 18, 10)])
@pytest.mark.parametrize("window", [1, 7, 40, 64, 65, 200, 0])
def test_latent_attention_window_edges_with_one_key_that_stands_out(dtype, window, heads, rank, rot_dim):
    """Latents and key parts go through norm and rotation into pages; then, for the last query of a request of 230
    tokens, one key at a time is made to stand out: the window's first key, the one before it (which must not
    show), one far back, the query's own.  Whole prompt, a portion over cached rows, and a single token; keys at
    page borders are among them.  A window that is one token off shows as a wrong latent sum."""
    rt = runtime(dtype)
    rt.ops.require_latent()
    page, eps, scale, n = 16, 1e-5, 0.2, 230
    rot = dict(base=300.0, dims=rot_dim)
    gain = 1 + rand(rank, scale=0.2, seed=3)
    sink = rand(heads, scale=3.0, seed=5)
    edges = [n - 1, 3]
    if window:
        edges += [p for p in (n - window, n - 1 - window) if 0 <= p < n]
    for edge in edges:
        down = rand(n, rank + rot_dim, seed=1)
        q_latent = rand(n, heads, rank, scale=0.5, seed=6)
        q_raw = rand(n, heads, rot_dim, scale=0.5, seed=7)
        q_latent[n - 1, 0] *= 4.0
        down[edge, :rank] = q_latent[n - 1, 0] / gain * 12.0        # the latent of `edge` along head 0's last query
        latent_rows = plain.rms_norm(down[:, :rank].double(), gain.double(), eps)
        key_part = plain.rotate(down[:, rank:].double().view(n, 1, rot_dim), torch.arange(n), rot, True)[:, 0]
        turned = plain.rotate(q_raw.double(), torch.arange(n), rot, True)
        keys = torch.cat([latent_rows, key_part], -1).view(n, 1, rank + rot_dim)
        if dtype == "bfloat16":      # the pages hold bfloat16 rows
            keys = keys.to(torch.bfloat16).double()
        want = softmax_rows(torch.cat([q_latent.double(), turned], -1), keys.expand(n, heads, -1).contiguous(),
                            keys[..., :rank].expand(n, heads, -1).contiguous(), scale, sink.double(), window)
        for lengths, contexts in (([n], [0]), ([n - 180], [180]), ([1], [n - 1])):
            ctx, kv = fake_step([n], [0], page, rt.dtype, 1, rank, rot_dim, seed=2)
            kv.k, kv.v = kv.k.view(-1, page, rank), kv.v.view(-1, page, rot_dim)
            rt.ops.latent_prepare(down.cuda(), None, None, gain.cuda(), ctx, kv, rotation_of(rot, True), 0, rank, rot_dim,
                                  eps, True, True)
            held = contexts[0]
            step, _ = fake_step(lengths, contexts, page, rt.dtype, 1, rank, rot_dim, seed=2)
            out = torch.empty(n - held, heads * rank, dtype=torch.float32).cuda()
            rt.ops.latent_attention(q_latent[held:].reshape(n - held, -1).contiguous().cuda(),
                                    q_raw[held:].reshape(n - held, -1).contiguous().cuda(), rot_dim, out, step, kv,
                                    rotation_of(rot, True), sink.cuda(), heads, rank, rot_dim, scale, window=window)
            rt.ops.check_errors()
            close(out.view(n - held, heads, rank), want[held:], dtype, scale=1.0, loose=5e-2, tight=3e-5)


def gla_inputs(tokens, heads, dim, vdim, seed):
    pad = 7 if heads == 2 else 8          # columns before q: rows that allow 16-byte loads, and rows that do not
    proj = rand(tokens, pad + 2 * heads * dim + heads * vdim, seed=seed)
    z = rand(tokens, heads * dim, scale=3.0, seed=seed + 1)
    bias = rand(heads * dim, scale=2.0, seed=seed + 2)
    bias[0] = -60.0         # one channel forgets everything at once
    bias[1] = 60.0          # one keeps everything
    return proj, z, bias


@pytest.mark.parametrize("heads,dim,vdim", [(2, 12, 20), (1, 64, 128), (3, 128, 64), (2, 5, 33), (1, 160, 40), (2, 32, 136)])
@pytest.mark.parametrize("tau", [1.0, 16.0])
def test_gated_linear_attention_token_by_token_and_in_chunks(heads, dim, vdim, tau):
    """Both forms against the plain recurrence, from states that are not zero, with requests of one token, of a
    chunk's length, one more and several chunks, and a request that is not active (its state must stay)."""
    rt = runtime("float32")
    rt.ops.require_gla()
    lengths = [1, 32, 33, 100, 2]
    tokens, slots = sum(lengths), len(lengths) + 1
    proj, z, bias = gla_inputs(tokens, heads, dim, vdim, seed=3)
    q_off = proj.shape[1] - 2 * heads * dim - heads * vdim
    k_off, v_off = q_off + heads * dim, q_off + 2 * heads * dim
    start = rand(slots, heads, dim, vdim, seed=9)
    q_scale = dim ** -0.5
    q = proj[:, q_off:k_off].double().view(tokens, heads, dim) * q_scale
    k = proj[:, k_off:v_off].double().view(tokens, heads, dim)
    v = proj[:, v_off:].double().view(tokens, heads, vdim)
    alpha = torch.sigmoid(z.double() + bias.double()).pow(1.0 / tau).view(tokens, heads, dim)
    order = [3, 0, 5, 1, 2]                       # the slot of every request
    want, final = [], start.double().clone()
    first = 0
    for r, count in enumerate(lengths):
        state = start[order[r]].double().clone()
        for t in range(first, first + count):
            state = alpha[t].unsqueeze(-1) * state + k[t].unsqueeze(-1) * v[t].unsqueeze(-2)
            want.append(torch.einsum("hdv,hd->hv", state, q[t]))
        if r != 2:
            final[order[r]] = state
        first += count
    want = torch.stack(want)
    for chunked in (False, True):
        ctx, _ = fake_step(lengths, [0] * len(lengths), 16, torch.float32, 1, 8, 8)
        ctx.slots = torch.tensor(order, dtype=torch.int32).cuda()
        ctx.request_active = torch.tensor([1, 1, 0, 1, 1], dtype=torch.int32).cuda()
        plan = None
        if chunked:
            plan = {name: torch.from_numpy(a).cuda() for name, a in rt.ops.plan_gla(ctx.host).items()}
            if dim > rt.ops.gla_chunk_max_dim or vdim > rt.ops.gla_chunk_max_dim:
                continue
        state = start.clone().cuda()
        out = torch.empty(tokens, heads * vdim, dtype=torch.float32).cuda()
        rt.ops.gla(proj.cuda(), (q_off, k_off, v_off), z.cuda(), bias.cuda(), tau, q_scale, out, state, ctx, heads, dim,
                   vdim, plan=plan)
        rt.ops.check_errors()
        close(out.view(tokens, heads, vdim), want, "float32", tight=2e-5)
        close(state, final, "float32", tight=2e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("experts,top,hidden,ff", [(5, 2, 48, 16), (1, 1, 40, 24), (8, 8, 64, 32), (13, 3, 36, 10)])
def test_routed_experts_with_a_bias_and_weights_over_the_chosen_logits(dtype, experts, top, hidden, ff):
    """The part alone: the bias moves who is chosen; the weights are the softmax over the chosen logits only."""
    from cloud_inference_from_scratch_b200.config import PartSpec
    from cloud_inference_from_scratch_b200.parts import build_part

    rt = runtime(dtype)
    part = build_part("feed_forward", PartSpec("routed_experts", dict(
        hidden_size=hidden, intermediate_size=ff, num_experts=experts, top=top, correction=False, router_bias=True,
        score="chosen_softmax")))
    tensors = {"router": rand(experts, hidden, scale=0.5, seed=1), "router.b": rand(experts, scale=2.0, seed=2)}
    for e in range(experts):
        tensors[f"e{e}.gate"] = rand(ff, hidden, scale=0.3, seed=10 + e).to(rt.dtype)
        tensors[f"e{e}.up"] = rand(ff, hidden, scale=0.3, seed=40 + e).to(rt.dtype)
        tensors[f"e{e}.down"] = rand(hidden, ff, scale=0.3, seed=70 + e).to(rt.dtype)
    part.bind({name: t.cuda() for name, t in tensors.items()}, rt)
    x = rand(21, hidden, seed=5).to(rt.dtype)
    got = part.forward(x.cuda(), SimpleNamespace())
    rt.ops.check_errors()
    mlp = dict(router=dict(top=top))
    want = plain.routed_feed_forward(x.double(), {name: t.double() for name, t in tensors.items()}, mlp)
    close(got, want, dtype, loose=4e-2, tight=2e-5)
    if top < experts:      # without the bias other experts are chosen for some token
        other = plain.routed_feed_forward(x.double(), dict({n: t.double() for n, t in tensors.items()},
                                                           **{"router.b": torch.zeros(experts, dtype=F)}), mlp)
        assert (other - want).abs().max() > 1e-3


# ------------------------------------------------------------------ the public entry point and the replay program
def test_greedy_generation_through_the_engine(folders):
    from cloud_inference_from_scratch_b200 import generate

    folder = folders["mixed", "float32"]
    raw, tensors = plain.read_folder(folder)
    prompts = [random_tokens(raw["vocab"], n, 300 + n) for n in (5, 19, 33)]
    want = [plain.greedy(raw, tensors, prompt, 8) for prompt in prompts]
    results = generate(folder, prompts, max_output_tokens=8, dtype="float32", block_size=4, kv_cache_blocks=64,
                       prefill_chunk_size=16, max_batched_tokens=40)
    assert [result.token_ids for result in results] == want


def test_the_replay_program_on_a_bilipel_folder(folders, tmp_path):
    folder = folders["narrow", "float32"]
    requests = requests_for(CONFIGS["narrow"], [9, 30], seed=500)
    steps = trace_mixed(requests, seed=4, live_limit=2)
    out = tmp_path / "out"
    done = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out),
                           "--max-tokens", "128"], input="\n".join(json.dumps(step) for step in steps) + "\n",
                          capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [line for line in done.stdout.splitlines() if line.startswith("done")] == [f"done {s['step']}" for s in steps]
    position = {rid: 0 for rid in requests}
    for step in steps:
        rows = np.fromfile(out / f"{step['step']}.f32", dtype="<f4").reshape(-1, CONFIGS["narrow"]["vocab"])
        row = 0
        for entry in step["entries"]:
            ref = plain_logits(folder, requests[entry["id"]])
            for place in entry["want"]:
                assert np.abs(rows[row] - ref[position[entry["id"]] + place]).max() <= 2e-4 * ref.std()
                row += 1
            position[entry["id"]] += len(entry["tokens"])
        assert row == len(rows)
