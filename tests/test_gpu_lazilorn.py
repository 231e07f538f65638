"""The Lazilorn design in the engine against the plain implementation of ``plain_lazilorn.py``:
each mechanism alone, whole prompts against decoding, portions down to two tokens, unequal batches,
pages and state slots that are used again, window and page edges, kept first keys, far keys, first
tokens, long decoding, sizes of every kind, and greedy generation through the public entry point."""

import json
import subprocess
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_lazilorn as plain
from helpers import peak_tokens, random_tokens, replay, requests_in, trace_mixed, trace_portions, trace_tail, trace_whole

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
F = torch.float64

# worst |logit difference| of a row over the standard deviation of the request's reference logits
GATE = {"float32": 2e-4, "bfloat16": 0.1}


# ------------------------------------------------------------------ configurations
def window_attention(heads=4, kv_heads=2, dim=16, vdim=24, window=9, keep=2, scale=0.45):
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, mask=dict(size=window, keep_first=keep))


def memory(heads=3, dim=8, vdim=20, cap=9.0):
    return dict(heads=heads, dim=dim, vdim=vdim, gate_cap=cap)


def parallel(left=None, right=None, left_scale=0.7, right_scale=1.3, ff=40):
    return dict(type="parallel", mixer=dict(left=left or window_attention(), right=right or memory(),
                                            left_scale=left_scale, right_scale=right_scale),
                mlp=dict(kind="dense", ff=ff) if ff else None)


def delta(heads=4, kv_heads=2, dim=12, vdim=20, conv=3, ff=0):
    return dict(type="delta", mixer=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv),
                mlp=dict(kind="dense", ff=ff) if ff else None)


def config(layers, width=64, vocab=211, loop=None, eps=1e-5, embedding_scale=6.0, logit_scale=0.7):
    raw = dict(architecture="Lazilorn", vocab=vocab, width=width, norm=dict(eps=eps),
               embedding=dict(scale=embedding_scale), logit_scale=logit_scale, layers=list(layers))
    if loop is not None:
        raw["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
    return raw


CONFIGS = {
    # both mixers, a loop over a parallel and a delta layer in the middle, value sizes unlike key sizes
    "mixed": config([parallel(), delta(), parallel(ff=0), delta(ff=24), parallel()], loop=(1, 3, 3)),
    # no loop; every query head its own key head; no kept keys; a window of one key; a convolution of two taps
    "plain": config([delta(heads=2, kv_heads=2, dim=16, vdim=16, conv=2, ff=32),
                     parallel(window_attention(heads=2, kv_heads=2, dim=32, vdim=16, window=1, keep=0, scale=0.3),
                              memory(heads=1, dim=24, vdim=24, cap=15.0), left_scale=1.0, right_scale=1.0, ff=0)],
                    width=48, vocab=130, embedding_scale=1.0, logit_scale=1.0),
    # one key head; sizes that are no multiples of eight; more kept keys than a page and than the window;
    # one tap (no convolution history); the whole model looped
    "narrow": config([parallel(window_attention(heads=3, kv_heads=1, dim=20, vdim=12, window=5, keep=11, scale=0.5),
                               memory(heads=2, dim=5, vdim=33, cap=3.0), ff=10),
                      delta(heads=3, kv_heads=1, dim=10, vdim=6, conv=1, ff=7)],
                     width=36, vocab=77, loop=(0, 2, 2), eps=1e-6),
    # head sizes that the tensor-core attention kernel takes, keys of 64 and more for the scans, a window
    # that is no multiple of anything and one longer than any request
    "tiles": config([parallel(window_attention(heads=4, kv_heads=2, dim=32, vdim=32, window=21, keep=3, scale=0.3),
                              memory(heads=2, dim=64, vdim=64), ff=32),
                     delta(heads=2, kv_heads=1, dim=64, vdim=128, conv=4),
                     parallel(window_attention(heads=2, kv_heads=1, dim=64, vdim=64, window=400, keep=1, scale=0.2),
                              memory(heads=1, dim=128, vdim=32), ff=32)], loop=(1, 2, 2)),
    # no attention at all: no pages, only state slots
    "recurrent": config([delta(heads=2, kv_heads=1, dim=16, vdim=16, conv=4, ff=16),
                         delta(heads=2, kv_heads=2, dim=8, vdim=24, conv=5)], width=32, vocab=90, loop=(1, 2, 3)),
}
PAGE = {"mixed": 4, "plain": 16, "narrow": 8, "tiles": 16, "recurrent": 8}
# N(0, 0.05) weights leave biases, rates and taps close to nothing
SCALES = {"embed": 4.0, "head": 6.0, ".conv": 8.0, "i.b": 40.0, "f.b": 60.0, "A_log": 20.0, "dt_bias": 20.0,
          "mix.right.i": 3.0, "mix.right.f": 3.0, "mix.a": 3.0, "mix.b": 3.0, "loop.step": 10.0,
          "left.q": 2.0, "left.k": 2.0}


def make_model(folder, raw, seed, std=0.05, scales=None):
    from cloud_inference_from_scratch_b200.weights import write_random_model

    return write_random_model(folder, raw, seed, std=std, scales=scales or SCALES)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("lazilorn")
    return {name: make_model(root / name, raw, 5 + index) for index, (name, raw) in enumerate(CONFIGS.items())}


def core_for(folder, dtype, page, pages, slots=4, step_tokens=0):
    from cloud_inference_from_scratch_b200.engine.core import build_core

    return build_core(folder, dtype=dtype, page_size=page, num_pages=pages, max_requests=slots,
                      max_model_len=pages * page, max_tokens_per_step=step_tokens)


PLAIN_LOGITS = {}


def plain_logits(folder, tokens):
    key = (str(folder), tuple(tokens))
    if key not in PLAIN_LOGITS:
        raw, tensors = plain.read_folder(folder)
        PLAIN_LOGITS[key] = plain.forward(tokens, tensors, raw).numpy()
    return PLAIN_LOGITS[key]


ROUNDED_LOGITS = {}


def rows_that_rounding_decides(folder, tokens, limit):
    """Positions whose plain logits move by more than a quarter of the limit when the sublayers' inputs are
    rounded to bfloat16 and everything else stays exact: there a recurrent head's output is nearly nothing
    before its norm (its query at right angles to the few keys written so far), and the norm blows the
    rounding up.  No implementation in bfloat16 can be held to the exact row at such a position."""
    key = (str(folder), tuple(tokens))
    if key not in ROUNDED_LOGITS:
        raw, tensors = plain.read_folder(folder)
        ROUNDED_LOGITS[key] = plain.forward(tokens, tensors, raw, round_inputs=True).numpy()
    ref = plain_logits(folder, tokens)
    return np.abs(ROUNDED_LOGITS[key] - ref).max(axis=1) / ref.std() > limit / 4


def check(folder, got, dtype, gate=None, skip_what_rounding_decides=False, loose_first=0):
    """Every row against the plain model run on the whole request.  ``loose_first``: that many first positions
    are not held to the gate (bfloat16 only, where float32 has held them to a far sharper one): a recurrent
    head that has written one or two keys puts out next to nothing when its query is nearly at right angles
    to them, its norm divides by that, and one sample of the rounding does not bound another."""
    worst = 0.0
    for rid, tokens in got["fed"].items():
        ref = plain_logits(folder, tokens)
        rows = got["logits"][rid]
        assert sorted(rows) == list(range(len(tokens))), f"{rid}: positions missing"
        mine = np.stack([rows[p] for p in range(len(tokens))])
        errors = np.abs(mine - ref).max(axis=1) / ref.std()
        if skip_what_rounding_decides:
            skipped = rows_that_rounding_decides(folder, tokens, gate or GATE[dtype])
            assert skipped.sum() <= max(3, len(tokens) // 10), f"{rid}: rounding decides {int(skipped.sum())} rows"
            errors = np.where(skipped, 0.0, errors)
            errors[:loose_first] = 0.0
        worst = max(worst, float(errors.max()))
        limit = gate or GATE[dtype]
        assert errors.max() <= limit, (
            f"{rid}: first wrong position {int(np.argmax(errors > limit))} of {len(tokens)}, error {errors.max():.3e}")
    return worst


def run_trace(core, steps):
    return {"logits": replay(core, steps), "fed": requests_in(steps)}


def requests_for(raw, lengths, seed):
    return {f"r{i}": random_tokens(raw["vocab"], n, seed + i) for i, n in enumerate(lengths)}


def steady_requests(folder, lengths, seed):
    """Requests whose FIRST token leaves no recurrent head with q nearly at right angles to k: there the
    head's first output is (k . q) v up to a positive factor, the head norm keeps only the sign of k . q,
    and bfloat16 rounding of the input would decide the row."""
    raw, tensors = plain.read_folder(folder)
    out = {}
    for index, n in enumerate(lengths):
        for attempt in range(50):
            tokens = random_tokens(raw["vocab"], n, seed + index + 1000 * attempt)
            if plain.first_token_margin(raw, tensors, tokens) >= 0.05:
                break
        out[f"r{index}"] = tokens
    return out


# ------------------------------------------------------------------ the whole model, every cutting
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompts_decoding_portions_and_batches(folders, name, dtype):
    page = PAGE[name]
    # lengths: one token, two, a page's edge and one past it, several windows, several pages
    requests = steady_requests(folders[name], [1, 2, page, page + 1, 23, 61, 97], seed=10)
    for steps in (trace_whole(requests), trace_tail(requests, tail=40), trace_portions(requests),
                  trace_mixed(requests, seed=3, live_limit=3)):
        # a pool that holds what is live and no more, and three slots: pages and slots come back
        pages = -(-peak_tokens(steps, round_to=page) // page) + 1
        core = core_for(folders[name], dtype, page, pages, slots=3)
        check(folders[name], run_trace(core, steps), dtype)
        assert core.cache.free_pages(0) == core.cache.total_pages(0)


def drawn_configuration(seed):
    """A configuration drawn from the whole space of sizes: widths, either layer kind in any order, head
    counts, key and value sizes (multiples of 8 and 16 and others, above and below what the chunked and
    tensor-core kernels take), windows from one key to more than a request has, kept keys from none to
    several pages, convolutions of one to seven taps, gate caps, layers with and without feed-forward,
    loops anywhere or none."""
    import random

    rng = random.Random(seed)
    layers = []
    for _ in range(rng.randint(1, 5)):
        ff = rng.choice([0, 8, 24, 100])
        if rng.random() < 0.55:
            kv, group = rng.choice([1, 2, 4]), rng.choice([1, 2, 3, 8])
            dim = rng.choice([8, 16, 24, 32, 48, 64, 96, 128])
            vdim = dim if rng.random() < 0.5 else rng.choice([8, 16, 40, 64, 128, 160])
            left = window_attention(kv * group, kv, dim, vdim, rng.choice([1, 2, 5, 16, 17, 33, 64, 100, 500]),
                                    rng.choice([0, 0, 1, 3, 4, 16, 40]), rng.choice([0.4, 1.2, 4.0]) / dim ** 0.5)
            right = memory(rng.choice([1, 2, 3, 8]), rng.choice([4, 16, 32, 64, 128, 160]),
                           rng.choice([8, 32, 64, 128, 136]), rng.choice([1.0, 8.0, 15.0, 30.0]))
            layers.append(parallel(left, right, rng.choice([0.25, 0.8, 1.0]), rng.choice([0.5, 1.0, 2.0]), ff))
        else:
            kv, group = rng.choice([1, 2, 3]), rng.choice([1, 2, 4])
            layers.append(delta(kv * group, kv, rng.choice([4, 16, 32, 64, 128, 160]),
                                rng.choice([8, 32, 64, 128, 136]), rng.randint(1, 7), ff))
    loop = None
    if rng.random() < 0.7:
        start = rng.randrange(len(layers))
        loop = (start, rng.randint(start + 1, len(layers)), rng.randint(1, 3))
    return config(layers, width=rng.choice([64, 96, 128, 256]), vocab=rng.choice([50, 211, 448]), loop=loop,
                  eps=rng.choice([1e-6, 1e-5]), embedding_scale=rng.choice([1.0, 8.0, 16.0]),
                  logit_scale=rng.choice([0.25, 1.0, 2.0]))


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6, 7, 8])
def test_drawn_configurations(seed, tmp_path):
    raw = drawn_configuration(seed)
    folder = make_model(tmp_path / "model", raw, 100 + seed)
    requests = steady_requests(folder, [1, 2, 37, 150], seed=seed)
    for dtype, gate in (("float32", 4e-4), ("bfloat16", 0.2)):
        for steps in (trace_whole(requests), trace_mixed(requests, seed=seed, live_limit=3)):
            pages = -(-peak_tokens(steps, round_to=16) // 16) + 1
            core = core_for(folder, dtype, 16, pages, slots=3)
            check(folder, run_trace(core, steps), dtype, gate=gate, skip_what_rounding_decides=dtype == "bfloat16",
                  loose_first=2 if dtype == "bfloat16" else 0)


def test_float32_rows_do_not_depend_on_the_cut_or_the_batch(folders):
    """The same position through four cuttings: equal to rounding of the order of additions at most."""
    raw = CONFIGS["mixed"]
    requests = requests_for(raw, [50, 31, 77], seed=40)
    seen = []
    for steps in (trace_whole(requests), trace_tail(requests, tail=20), trace_portions(requests),
                  trace_mixed(requests, seed=9, live_limit=3)):
        core = core_for(folders["mixed"], "float32", 4, 64, slots=3)
        seen.append(replay(core, steps))
    for rid, tokens in requests.items():
        base = np.stack([seen[0][rid][p] for p in range(len(tokens))])
        for other in seen[1:]:
            mine = np.stack([other[rid][p] for p in range(len(tokens))])
            assert np.abs(mine - base).max() <= 5e-5 * base.std()


def test_long_decoding_past_windows_and_pages(folders):
    """160 tokens decoded one by one after a short prompt: the window passes over decoded tokens many
    times, pages behind it are given back while the pages of the kept first keys stay, and the state of
    both recurrent mixers is carried for every token."""
    for name in ("mixed", "narrow"):
        requests = steady_requests(folders[name], [170, 165], seed=70)
        steps = trace_tail(requests, tail=160)
        for dtype in ("float32", "bfloat16"):
            core = core_for(folders[name], dtype, PAGE[name], 400 // PAGE[name], slots=2)
            check(folders[name], run_trace(core, steps), dtype)


def test_a_state_slot_that_is_used_again_starts_from_zero(folders):
    """One slot only: every request inherits the slot of the one before it (matrices, normaliser, running
    maximum, convolution history)."""
    for name in ("plain", "recurrent"):
        requests = requests_for(CONFIGS[name], [30, 8, 19], seed=90)
        core = core_for(folders[name], "float32", 16, 4, slots=1)
        check(folders[name], run_trace(core, trace_portions(requests)), "float32")


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
@pytest.mark.parametrize("width", [40, 33, 512])
def test_embedding_adds_the_sinusoid_of_the_position(dtype, width):
    """Positions far from zero too: the angle is a float32 product of the position and the frequency."""
    rt = runtime(dtype)
    table = rand(50, width, seed=1).to(rt.dtype)
    ids = torch.tensor([3, 49, 0, 3, 7], dtype=torch.int32)
    where = torch.tensor([0, 29, 7, 1, 3000], dtype=torch.int32)
    wave = torch.pow(torch.tensor(10000.0, dtype=F), -2.0 * torch.arange((width + 1) // 2, dtype=F) / width)
    out = torch.empty(5, width, dtype=torch.float32).cuda()
    rt.ops.embedding(ids.cuda(), table.cuda(), out, scale=3.5, positions=where.cuda(), wave=wave.float().cuda())
    rt.ops.check_errors()
    weights = {"embed": table.float()}
    for row, (token, p) in enumerate(zip(ids.tolist(), where.tolist())):
        want = plain.embed_tokens([0] * p + [token], weights, dict(width=width, embedding=dict(scale=3.5)), F)[p]
        # float32 angles: at position 3000 the angle carries an error of 3000 * 2^-24
        close(out[row], want, "float32", scale=1.0, tight=2e-6 + p * 2.0 ** -23)


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
                          host=SimpleNamespace(query_lens=np.asarray(lengths, dtype=np.int32), num_single=singles,
                                               num_requests=len(lengths)))
    return ctx, kv, table, positions, request_of


def plan_into(ctx, rt, group):
    plan = rt.ops.plan_attention(ctx.host, group)
    if plan:
        ctx.extras[("attention", group)] = {name: torch.from_numpy(np.asarray(a)).cuda() for name, a in plan.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim,vdim", [(16, 24), (32, 32), (20, 12), (128, 128)])
@pytest.mark.parametrize("window,keep", [(1, 0), (7, 3), (16, 1), (17, 16), (5, 9), (0, 0)])
def test_attention_window_edges_and_kept_first_keys_with_one_key_that_stands_out(dtype, window, keep, dim, vdim):
    """Keys go through the per-head q/k norm into pages; then, for the last query of the long request, one
    key at a time is turned along that query so that it takes nearly all the weight where the query may see
    it and must not show where it may not: just inside and just outside the window, the last kept key and
    the first key that is not kept.  A window or a count that is one token off shows as a wrong value row."""
    rt = runtime(dtype)
    heads, groups, page, eps, scale = 4, 2, 8, 1e-5, 2.4 / dim ** 0.5
    lengths, n = [1, 44, 25], 44       # a single token leads the step, as the step function lays it out
    tokens = sum(lengths)
    rt.ops.require_attention(dim)
    width = heads * dim + groups * (dim + vdim)
    q_gain, k_gain = 1 + rand(dim, scale=0.2, seed=3), 1 + rand(dim, scale=0.2, seed=4)
    last = 1 + n - 1                    # the row of the long request's last query, position n - 1
    edges = [n - 1]
    if window > 0:
        edges += [p for p in (n - window, n - 1 - window, keep - 1, keep) if 0 <= p < n]
    for edge in edges:
        qkv = rand(tokens, width, seed=1)
        target = qkv[last, :dim] * q_gain            # head 0 of the query after its norm, up to a factor
        qkv[1 + edge, heads * dim:heads * dim + dim] = target / k_gain * 40.0 / target.norm()
        qkv = qkv.to(rt.dtype)
        ctx, kv, _, _, _ = fake_step(lengths, [0, 0, 0], page, rt.dtype, groups, dim, vdim)
        plan_into(ctx, rt, heads // groups)
        q_out = torch.empty(tokens, heads * dim, dtype=rt.dtype).cuda()
        rt.ops.norm_kv_write(qkv.cuda(), ctx, kv, heads, groups, dim, vdim, q_gain.cuda(), k_gain.cuda(), False, eps,
                             q_out, per_head=True)
        out = torch.empty(tokens, heads * vdim, dtype=rt.dtype).cuda()
        rt.ops.attention_penalised(q_out, out, ctx, kv, heads, groups, dim, vdim, scale, window, None, keep_first=keep)
        rt.ops.check_errors()
        full = qkv.double()
        q = plain.rms(full[:, :heads * dim].view(tokens, heads, dim), eps) * q_gain.double()
        k = plain.rms(full[:, heads * dim:heads * dim + groups * dim].view(tokens, groups, dim), eps) * k_gain.double()
        v = full[:, heads * dim + groups * dim:].view(tokens, groups, vdim)
        first = 0
        for count in lengths:
            rows = slice(first, first + count)
            want = plain.windowed_softmax(q[rows], k[rows], v[rows], scale, window, keep)
            close(out[rows].view(count, heads, vdim), want, dtype, scale=1.0, loose=6e-2)
            first += count


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim", [32, 64])
@pytest.mark.parametrize("window,keep", [(70, 5), (70, 70), (64, 64), (130, 1), (33, 100), (200, 0), (1, 129)])
def test_attention_prompt_portions_far_from_their_kept_keys(dtype, dim, window, keep):
    """A prompt of 400 tokens at once, and its last 150 tokens as a portion over 250 cached ones (values as
    large as keys, so bfloat16 portions run on the tensor cores): the kept keys lie several key tiles before
    the window, in the tile next to it, or in the tile where it starts.  One key at a time is turned along
    the last query: the last kept one, the first that is not kept, the window's first, the one before it."""
    rt = runtime(dtype)
    heads, groups, page, eps, scale, n, cut = 4, 2, 16, 1e-5, 2.4 / dim ** 0.5, 400, 250
    rt.ops.require_attention(dim)
    width = heads * dim + groups * 2 * dim
    ones = torch.ones(dim)
    for edge in [p for p in (n - window, n - 1 - window, keep - 1, keep) if 0 <= p < n]:
        qkv = rand(n, width, seed=5)
        target = qkv[n - 1, :dim]
        qkv[edge, heads * dim:heads * dim + dim] = target * 40.0 / target.norm()
        qkv = qkv.to(rt.dtype)
        ctx, kv, _, _, _ = fake_step([n], [0], page, rt.dtype, groups, dim, dim, seed=2)
        plan_into(ctx, rt, heads // groups)
        q_out = torch.empty(n, heads * dim, dtype=rt.dtype).cuda()
        rt.ops.norm_kv_write(qkv.cuda(), ctx, kv, heads, groups, dim, dim, ones.cuda(), ones.cuda(), False, eps, q_out,
                             per_head=True)
        full = qkv.double()
        q = plain.rms(full[:, :heads * dim].view(n, heads, dim), eps)
        k = plain.rms(full[:, heads * dim:heads * dim + groups * dim].view(n, groups, dim), eps)
        v = full[:, heads * dim + groups * dim:].view(n, groups, dim)
        want = plain.windowed_softmax(q, k, v, scale, window, keep)
        out = torch.empty(n, heads * dim, dtype=rt.dtype).cuda()
        rt.ops.attention_penalised(q_out, out, ctx, kv, heads, groups, dim, dim, scale, window, None, keep_first=keep)
        rt.ops.check_errors()
        close(out.view(n, heads, dim), want, dtype, scale=1.0, loose=6e-2)
        part, pools, _, _, _ = fake_step([n - cut], [cut], page, rt.dtype, groups, dim, dim, seed=2)   # the same pages
        plan_into(part, rt, heads // groups)
        out = torch.empty(n - cut, heads * dim, dtype=rt.dtype).cuda()
        rt.ops.attention_penalised(q_out[cut:].contiguous(), out, part, kv, heads, groups, dim, dim, scale, window, None,
                                   keep_first=keep)
        rt.ops.check_errors()
        close(out.view(n - cut, heads, dim), want[cut:], dtype, scale=1.0, loose=6e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window,keep,stand_out", [(0, 0, 2), (64, 4, 3), (64, 4, 4), (64, 4, 237), (64, 4, 236),
                                                   (300, 0, 1), (301, 0, 0), (5, 40, 39), (5, 40, 40)])
def test_attention_decodes_over_a_context_with_a_far_key(dtype, window, keep, stand_out):
    """Single queries over 300 cached keys; one key far back (a kept one, the first that is not kept, the
    first of the window, the one before it) is turned along the last query."""
    rt = runtime(dtype)
    heads, groups, dim, vdim, page, eps, scale = 2, 1, 32, 8, 16, 1e-6, 1.0
    n = 301
    width = heads * dim + groups * (dim + vdim)
    qkv = rand(n, width, seed=11)
    qkv[stand_out, heads * dim:heads * dim + dim] = qkv[n - 1, :dim] * 25.0
    qkv = qkv.to(rt.dtype)
    ones = torch.ones(dim)
    ctx, kv, table, _, _ = fake_step([n - 1], [0], page, rt.dtype, groups, dim, vdim)
    q_out = torch.empty(n, heads * dim, dtype=rt.dtype).cuda()
    rt.ops.norm_kv_write(qkv[: n - 1].cuda(), ctx, kv, heads, groups, dim, vdim, ones.cuda(), ones.cuda(), False, eps,
                         q_out[: n - 1], per_head=True)
    ctx.positions = torch.tensor([n - 1], dtype=torch.int32).cuda()
    ctx.request_of_token = torch.tensor([0], dtype=torch.int32).cuda()
    rt.ops.norm_kv_write(qkv[n - 1:].cuda(), ctx, kv, heads, groups, dim, vdim, ones.cuda(), ones.cuda(), False, eps,
                         q_out[n - 1:], per_head=True)
    full = qkv.double()
    q = plain.rms(full[:, :heads * dim].view(n, heads, dim), eps)
    k = plain.rms(full[:, heads * dim:heads * dim + dim].view(n, groups, dim), eps)
    v = full[:, heads * dim + dim:].view(n, groups, vdim)
    want = plain.windowed_softmax(q[n - 1:], k, v, scale, window, keep, first_position=n - 1)
    for few_tokens in (False, True):      # True: the keys are cut into ranges with a CTA each, joined by tickets
        for _ in range(2):                # twice: the tickets must be back at zero
            out = torch.zeros(1, heads * vdim, dtype=rt.dtype).cuda()
            rt.ops.attention_generic(q_out[n - 1:], out, ctx, kv, heads, groups, dim, scale, window, value_dim=vdim,
                                     few_tokens=few_tokens, keep_first=keep)
            rt.ops.check_errors()
            close(out.view(1, heads, vdim), want, dtype, scale=1.0)


def scan_ctx(lengths, slots, active):
    starts = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    request_of = np.concatenate([np.full(n, r, dtype=np.int32) for r, n in enumerate(lengths)])
    singles = 0
    while singles < len(lengths) and lengths[singles] == 1:
        singles += 1
    host = SimpleNamespace(num_single=singles, num_requests=len(lengths), query_start=starts,
                           query_lens=np.asarray(lengths, dtype=np.int32))
    ctx = SimpleNamespace(query_start=torch.from_numpy(starts).cuda(), slots=torch.tensor(slots, dtype=torch.int32).cuda(),
                          num_requests=len(lengths), num_single=singles, extras={}, host=host,
                          request_of_token=torch.from_numpy(request_of).cuda(),
                          request_active=torch.tensor(active, dtype=torch.int32).cuda())
    return ctx, starts


def memory_gates(rows_i, rows_f, bias_i, bias_f, cap):
    log_in = cap * torch.tanh((rows_i + bias_i) / cap)
    log_keep = torch.nn.functional.logsigmoid(cap * torch.tanh((rows_f + bias_f) / cap))
    return log_in, log_keep


@pytest.mark.parametrize("heads,dim,vdim,cap", [(3, 20, 36, 9.0), (2, 64, 64, 15.0), (1, 128, 32, 4.0), (2, 5, 130, 1.0),
                                                (2, 160, 8, 30.0), (1, 64, 300, 9.0), (2, 200, 136, 9.0), (2, 6, 30, 9.0),
                                                (1, 7, 127, 12.0)])
@pytest.mark.parametrize("streams", ["chunks", "1", "0"])
def test_matrix_memory_carries_matrix_normaliser_and_maximum_between_steps(heads, dim, vdim, cap, streams, monkeypatch):
    """Prompt portions in chunks (keys and values up to 128), as prepare + stream (keys up to 128) or on the
    token-by-token kernel.  Three steps of unequal requests (portions of 1 to 100 tokens, so every kernel for prompts and for
    single tokens runs) from states that are not zero, one request inactive in the second step (its state
    must stay); gates with large biases either way, so that the running maximum moves and the floor
    exp(-m) of the denominator is what counts for some tokens and |n . q| for others."""
    monkeypatch.setenv("CIE_RECURRENT_STREAM", "0" if streams == "0" else "1")
    rt = runtime("float32")
    qk, vv = heads * dim, heads * vdim
    width = 2 * qk + 2 * vv + 2 * heads
    offsets = (0, qk, 2 * qk, 2 * qk + 2 * vv, 2 * qk + 2 * vv + heads)
    bias_i, bias_f = rand(heads, scale=3.0, seed=1), rand(heads, scale=3.0, seed=2) + 2.0
    slots = [2, 0, 3, 5]
    # a head's state: the matrix, then the normaliser and the maximum once for every 32 value columns
    copies = -(-vdim // 32)
    per_head = dim * vdim + copies * (dim + 1)
    matrices, vectors = rand(6, heads, dim * vdim, scale=0.5, seed=4), rand(6, heads, dim, scale=0.5, seed=6)
    maxima = rand(6, heads, 1, scale=3.0, seed=5)                # running maxima of either sign
    start = torch.cat([matrices] + [vectors, maxima] * copies, dim=2)
    state = start.clone().view(6, heads * per_head).cuda()
    known = {r: (matrices[s].view(heads, dim, vdim).double(), vectors[s].double(), maxima[s, :, 0].double())
             for r, s in enumerate(slots)}
    for step, (lengths, active) in enumerate((([1, 13, 100, 33], [1, 1, 1, 1]), ([1, 1, 6, 64], [1, 0, 1, 1]),
                                              ([1, 1, 1, 1], [1, 1, 1, 1]))):
        tokens = sum(lengths)
        proj = rand(tokens, width, seed=20 + step)
        proj[:, offsets[3]:] *= 4.0
        ctx, starts = scan_ctx(lengths, slots, active)
        out = torch.empty(tokens, vv, dtype=torch.float32).cuda()
        plan = None
        if streams == "chunks":
            plan = {name: torch.from_numpy(a).cuda() for name, a in rt.ops.plan_memory_chunks(ctx.host).items()}
        below = rt.ops.mlstm_scan(proj.cuda(), offsets, bias_i.cuda(), bias_f.cuda(), cap, dim ** -0.5, out, state,
                                  ctx, heads, dim, vdim, plan=plan)
        rt.ops.check_errors()
        wide = tokens >= 8 * len(lengths)
        chunked = streams == "chunks" and wide and bool(plan) and max(dim, vdim) <= 128
        assert (below is not None) == (streams != "0" and not chunked and dim <= 128 and wide)
        if below is not None:          # the stream leaves numerators and what the head norm divides them by
            out = (out.view(tokens, heads, vdim) / below.unsqueeze(2)).view(tokens, vv)
        for r in range(len(lengths)):
            rows = proj[starts[r]:starts[r + 1]].double()
            q = rows[:, :qk].view(-1, heads, dim) * dim ** -0.5
            k = rows[:, qk:2 * qk].view(-1, heads, dim)
            v = rows[:, 2 * qk:2 * qk + vv].view(-1, heads, vdim)
            log_in, log_keep = memory_gates(rows[:, offsets[3]:offsets[3] + heads], rows[:, offsets[4]:], bias_i.double(),
                                            bias_f.double(), cap)
            want, after = plain.memory_recurrence(q, k, v, log_in, log_keep, known[r])
            close(out[starts[r]:starts[r + 1]].view(-1, heads, vdim), want, "float32", scale=float(want.abs().max()),
                  tight=3e-4)     # a gate of 30 carries 2e-6 of rounding into every factor of 100 tokens
            if active[r]:
                known[r] = after
            mine = state[slots[r]].view(heads, per_head).cpu()
            close(mine[:, :dim * vdim].reshape(heads, dim, vdim), known[r][0], "float32",
                  scale=max(1.0, float(known[r][0].abs().max())), tight=1e-4)
            for copy in range(copies):
                at = dim * vdim + copy * (dim + 1)
                close(mine[:, at:at + dim], known[r][1], "float32", scale=max(1.0, float(known[r][1].abs().max())), tight=1e-4)
                close(mine[:, at + dim], known[r][2], "float32", scale=1.0, tight=1e-5)
    assert torch.equal(state[1].cpu(), start[1].view(-1)) and torch.equal(state[4].cpu(), start[4].view(-1))


def test_matrix_memory_starts_its_maximum_at_zero_and_not_below():
    """A first token whose input gate is far below zero: with the maximum started at zero the write is
    exp(i) k v^T and the floor of the denominator is one; a maximum started at minus infinity would give
    the write weight one."""
    rt = runtime("float32")
    heads, dim, vdim, cap = 1, 8, 8, 20.0
    proj = rand(2, 2 * dim + 2 * vdim + 2, seed=3)
    proj[:, -2] = -9.0       # input gate
    proj[:, -1] = 9.0        # forget gate
    ctx, _ = scan_ctx([2], [0], [1])
    state = torch.zeros(1, dim * vdim + dim + 1).cuda()
    out = torch.empty(2, vdim).cuda()
    offsets = (0, dim, 2 * dim, 2 * dim + 2 * vdim, 2 * dim + 2 * vdim + 1)
    zero = torch.zeros(1).cuda()
    rt.ops.mlstm_scan(proj.cuda(), offsets, zero, zero, cap, 1.0, out, state, ctx, heads, dim, vdim)
    rows = proj.double()
    log_in, log_keep = memory_gates(rows[:, -2:-1], rows[:, -1:], 0.0, 0.0, cap)
    want, after = plain.memory_recurrence(rows[:, :dim].view(2, 1, dim), rows[:, dim:2 * dim].view(2, 1, dim),
                                          rows[:, 2 * dim:2 * dim + vdim].view(2, 1, vdim), log_in, log_keep)
    assert float(want.abs().max()) < 1e-2          # the tiny write shows: nothing near the size of v
    close(out.view(2, 1, vdim), want, "float32", scale=float(want.abs().max()), tight=1e-4)
    assert abs(float(state[0, -1]) - float(after[2])) < 1e-6


@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_short_convolution_reads_and_leaves_its_history(taps):
    """Portions shorter and longer than the taps, a request that is inactive (its history must stay), and
    history rows that are not zero."""
    rt = runtime("float32")
    channels, extra = 70, 9
    weight = rand(channels, taps, seed=1)
    slots = [3, 0, 2, 1]
    history = rand(5, 11 + (taps - 1) * channels, seed=2).cuda()      # 11 floats of something else come first
    view = history[:, 11:]
    before = {r: view[s].cpu().view(taps - 1, channels).double() for r, s in enumerate(slots)}
    for step, (lengths, active) in enumerate((([1, 2, 9, 1], [1, 1, 1, 1]), ([1, 5, 2, 3], [1, 0, 1, 1]))):
        tokens = sum(lengths)
        proj = rand(tokens, channels + extra, seed=5 + step)
        ctx, starts = scan_ctx(lengths, slots, active)
        out = torch.empty(tokens, channels).cuda()
        rt.ops.short_conv(proj.cuda(), weight.cuda(), view, out, ctx)
        rt.ops.check_errors()
        for r in range(4):
            x = proj[starts[r]:starts[r + 1], :channels].double()
            want = torch.nn.functional.silu(plain.short_convolution(x, weight.double(), before[r]))
            close(out[starts[r]:starts[r + 1]], want, "float32", scale=1.0)
            if active[r]:
                before[r] = torch.cat([before[r], x])[x.shape[0]:]
            if taps > 1:        # one tap: no history
                close(view[slots[r]].view(taps - 1, channels), before[r], "float32", scale=1.0, tight=0.0)
    assert torch.equal(history[4].cpu(), rand(5, 11 + (taps - 1) * channels, seed=2)[4])


@pytest.mark.parametrize("heads,groups,dim,vdim", [(4, 2, 12, 20), (2, 1, 64, 128), (2, 2, 128, 64), (3, 1, 5, 130),
                                                   (1, 1, 160, 8), (2, 2, 10, 36), (2, 1, 33, 30)])
@pytest.mark.parametrize("streams", ["chunks", "1", "0"])
def test_gated_delta_rule_carries_its_state_between_steps(heads, groups, dim, vdim, streams, monkeypatch):
    """Three steps of unequal requests from states that are not zero; one request inactive in the second.
    Prompt portions in chunks (keys and values up to 128, values a multiple of 4), as prepare + stream (keys up
    to 128) or on the token-by-token kernel."""
    monkeypatch.setenv("CIE_RECURRENT_STREAM", "0" if streams == "0" else "1")
    rt = runtime("float32")
    qk, vv = groups * dim, heads * vdim
    a_log, dt = rand(heads, scale=0.7, seed=1), rand(heads, scale=1.0, seed=2)
    slots = [2, 0, 3, 5]
    start = rand(6, heads * dim * vdim + 13, scale=0.3, seed=4)
    state = start.clone().cuda()
    known = {r: start[s, :heads * dim * vdim].view(heads, dim, vdim).double() for r, s in enumerate(slots)}
    for step, (lengths, active) in enumerate((([1, 13, 100, 33], [1, 1, 1, 1]), ([1, 1, 6, 64], [1, 0, 1, 1]),
                                              ([1, 1, 1, 1], [1, 1, 1, 1]))):
        tokens = sum(lengths)
        conv = rand(tokens, 2 * qk + vv, seed=30 + step)
        gates = rand(tokens, 3 + 2 * heads, scale=2.0, seed=40 + step)
        ctx, starts = scan_ctx(lengths, slots, active)
        out = torch.empty(tokens, vv, dtype=torch.float32).cuda()
        plan = None
        if streams == "chunks":
            plan = {name: torch.from_numpy(a).cuda() for name, a in rt.ops.plan_memory_chunks(ctx.host).items()}
        before = rt.ops.launches
        rt.ops.gated_delta_scan(conv.cuda(), (0, qk, 2 * qk), gates.cuda(), (3, 3 + heads), a_log.cuda(), dt.cuda(),
                                dim ** -0.5, out, state, ctx, heads, groups, dim, vdim, plan=plan)
        rt.ops.check_errors()
        wide = tokens >= 8 * len(lengths)
        chunked = streams == "chunks" and wide and max(dim, vdim) <= 128 and vdim % 4 == 0
        assert rt.ops.launches - before == (4 if chunked else 2 if wide and streams != "0" and dim <= 128 else 1)
        for r in range(len(lengths)):
            rows, g = conv[starts[r]:starts[r + 1]].double(), gates[starts[r]:starts[r + 1]].double()
            q, k = rows[:, :qk].view(-1, groups, dim), rows[:, qk:2 * qk].view(-1, groups, dim)
            q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
            k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
            v = rows[:, 2 * qk:].view(-1, heads, vdim)
            beta = torch.sigmoid(g[:, 3:3 + heads])
            decay = torch.exp(-torch.exp(a_log.double()) * torch.nn.functional.softplus(g[:, 3 + heads:] + dt.double()))
            want, after = plain.delta_recurrence(q, k, v, beta, decay, known[r])
            close(out[starts[r]:starts[r + 1]].view(-1, heads, vdim), want, "float32", scale=float(want.abs().max()),
                  tight=1e-4)
            if active[r]:
                known[r] = after
            close(state[slots[r], :heads * dim * vdim].view(heads, dim, vdim), known[r], "float32",
                  scale=max(1.0, float(known[r].abs().max())), tight=1e-4)
    assert torch.equal(state[:, heads * dim * vdim:].cpu(), start[:, heads * dim * vdim:])      # what follows the matrices
    assert torch.equal(state[1].cpu(), start[1]) and torch.equal(state[4].cpu(), start[4])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,size,shared,act", [(3, 20, True, "silu"), (2, 64, False, "sigmoid"), (1, 130, True, "sigmoid"),
                                                   (5, 7, False, "silu")])
@pytest.mark.parametrize("divided", [False, True])
def test_heads_divided_by_their_own_root_mean_square_times_gain_and_gate(dtype, heads, size, shared, act, divided):
    """``divided``: every head is first divided by a number of its token and head (the numerators and
    denominators that the streamed matrix memory leaves)."""
    rt = runtime(dtype)
    tokens = 9
    o = rand(tokens, heads * size, seed=1)
    o[2] *= 1e-3                                         # a row where eps counts
    below = (0.05 + rand(tokens, heads, seed=7).abs() * 3.0) if divided else None
    wide = rand(tokens, 5 + heads * size, seed=2)
    gain = 1 + rand(size if shared else heads * size, scale=0.3, seed=3)
    out = torch.empty(tokens, heads * size, dtype=rt.dtype).cuda()
    rt.ops.head_norm_gate(o.cuda(), wide.cuda()[:, 5:], gain.cuda(), 1e-5, out, heads, gate_act=act,
                          denominators=below.cuda() if divided else None)
    o = o.double().view(tokens, heads, size)
    if divided:
        o = o / below.double().unsqueeze(2)
    normed = plain.rms(o, 1e-5)
    normed = normed * gain.double() if shared else normed * gain.double().view(heads, size)
    gate = wide[:, 5:].double()
    gate = torch.sigmoid(gate) if act == "sigmoid" else torch.nn.functional.silu(gate)
    close(out, normed.reshape(tokens, heads * size) * gate, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tokens", [1, 5, 200])
def test_squared_relu_feed_forward_part(dtype, tokens):
    from cloud_inference_from_scratch_b200.config import PartSpec
    from cloud_inference_from_scratch_b200.parts import build_part

    rt = runtime(dtype)
    hidden, ff = 40, 56
    part = build_part("feed_forward", PartSpec("dense_activation", dict(hidden_size=hidden, intermediate_size=ff,
                                                                        activation="relu2")))
    tensors = {"up": rand(ff, hidden, scale=0.3, seed=1).to(rt.dtype), "down": rand(hidden, ff, scale=0.3, seed=2).to(rt.dtype)}
    assert set(part.tensor_specs()) == set(tensors)
    part.bind({name: value.cuda() for name, value in tensors.items()}, rt)
    x = rand(tokens, hidden, seed=3).to(rt.dtype)
    got = part.forward(x.cuda(), SimpleNamespace(residual_sink=None))
    want = plain.squared_relu_feed_forward(x.double(), {name: value.double() for name, value in tensors.items()}, "", F)
    close(got, want, dtype)


# ------------------------------------------------------------------ the public entry point
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(folders, dtype):
    from cloud_inference_from_scratch_b200 import generate

    raw, tensors = plain.read_folder(folders["mixed"])
    prompts = list(steady_requests(folders["mixed"], [1, 9, 30, 17], seed=100).values())
    results = generate(folders["mixed"], prompts, max_output_tokens=12, dtype=dtype, block_size=4,
                       kv_cache_blocks=40, prefill_chunk_size=8, max_batched_tokens=20, max_active_sequences=3)
    for prompt, result in zip(prompts, results):
        got = result.token_ids
        assert len(got) == 12
        # every token is the argmax of the plain model's logits given the engine's own tokens so far
        # (a near tie may go the other way under bfloat16 rounding: then the logits must be close)
        logits = plain.forward(prompt + got, tensors, raw).numpy()
        for index, token in enumerate(got):
            row = logits[len(prompt) + index - 1]
            assert row[token] >= row.max() - (1e-3 if dtype == "float32" else 0.15) * logits.std()


def test_trace_program_replays_a_lazilorn_model(folders, tmp_path):
    raw, tensors = plain.read_folder(folders["narrow"])
    tokens = random_tokens(raw["vocab"], 21, 7)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": tokens[:13], "want": [0, 12]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": tokens[13:], "want": [7]},
                                     {"id": "b", "tokens": tokens[:2], "want": []}], "end": ["a", "b"]}]
    out = tmp_path / "out"
    done = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(folders["narrow"]), "--dtype", "float32",
                           "--out", str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                          capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [line for line in done.stdout.splitlines() if line.startswith("done")] == ["done 0", "done 1"]
    ref = plain.forward(tokens, tensors, raw).numpy()
    first = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1)
    second = np.fromfile(out / "1.f32", dtype="<f4").reshape(1, -1)
    assert np.abs(first - ref[[0, 12]]).max() <= 1e-4 * ref.std()
    assert np.abs(second - ref[[20]]).max() <= 1e-4 * ref.std()
