"""A plain, slow Lazilorn: one function per mechanism, token by token, in float64 (or float32) on the CPU.

Written from the design's equations only; it shares no code with the engine.  ``weights`` maps tensor
names to torch tensors, ``config`` is the config.json dictionary.

Notation: ``h`` the normalised input of a sublayer [T, width]; ``p`` a token's position in its request.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch

# When a list: the recurrent mixers append, for a request's FIRST token, |cos(q, k)| of every head.  There the
# state holds one write, a head puts out (k . q) v up to a positive factor, and the head norm that follows
# keeps only the sign of k . q: where the cosine is nearly zero, rounding of the input decides the row.
FIRST_TOKEN_COSINES = None


def _note_first_token(q0, k0):
    if FIRST_TOKEN_COSINES is not None:
        cos = (q0 * k0).sum(-1) / (q0.norm(dim=-1) * k0.norm(dim=-1) + 1e-30)
        FIRST_TOKEN_COSINES.extend(float(c) for c in cos.abs().reshape(-1))


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def embed_tokens(tokens, weights, config, dtype):
    """Embedding row times a constant plus the sinusoid of the position: entry 2i is sin(p w_i), entry
    2i + 1 is cos(p w_i), w_i = 10000^(-2i / width)."""
    width = config["width"]
    x = weights["embed"].to(dtype)[torch.as_tensor(tokens)] * config["embedding"]["scale"]
    p = torch.arange(len(tokens), dtype=dtype).unsqueeze(1)
    pair = torch.arange((width + 1) // 2, dtype=dtype)
    angle = p * torch.pow(torch.tensor(10000.0, dtype=dtype), -2.0 * pair / width)
    wave = torch.zeros(len(tokens), 2 * angle.shape[1], dtype=dtype)
    wave[:, 0::2] = torch.sin(angle)
    wave[:, 1::2] = torch.cos(angle)
    return x + wave[:, :width]


def windowed_softmax(q, k, v, scale, window, keep, first_position=0):
    """Softmax attention of queries q [Tq, heads, dim] at positions first_position.. over keys k [Tk, groups,
    dim] and values v [Tk, groups, vdim] at positions 0..: query i sees key j <= i if i - j < window or
    j < keep (window 0: every earlier key)."""
    heads, groups = q.shape[1], k.shape[1]
    out = torch.zeros(q.shape[0], heads, v.shape[2], dtype=q.dtype)
    for row in range(q.shape[0]):
        i = first_position + row
        seen = [j for j in range(i + 1) if window <= 0 or i - j < window or j < keep]
        for head in range(heads):
            g = head // (heads // groups)
            weight = torch.softmax((k[seen, g] @ q[row, head]) * scale, 0)
            out[row, head] = (weight.unsqueeze(1) * v[seen, g]).sum(0)
    return out


def window_attention(h, w, prefix, sizes, eps, dtype):
    """Softmax attention without rotation: q and k normalised per head (one gain vector of the head's
    size for all heads), grouped key/value heads, a sliding window that also keeps the first tokens,
    and an output gate sigmoid(W_g h) on the concatenated heads."""
    heads, groups, dim, vdim = sizes["heads"], sizes["kv_heads"], sizes["dim"], sizes["vdim"]
    window, keep = sizes["mask"]["size"], sizes["mask"]["keep_first"]
    tokens = h.shape[0]
    q = (h @ w[prefix + "q"].to(dtype).T).view(tokens, heads, dim)
    k = (h @ w[prefix + "k"].to(dtype).T).view(tokens, groups, dim)
    v = (h @ w[prefix + "v"].to(dtype).T).view(tokens, groups, vdim)
    q = rms(q, eps) * w[prefix + "q.norm"].to(dtype)
    k = rms(k, eps) * w[prefix + "k.norm"].to(dtype)
    out = windowed_softmax(q, k, v, sizes["scale"], window, keep)
    gate = torch.sigmoid(h @ w[prefix + "g"].to(dtype).T)
    return (out.reshape(tokens, heads * vdim) * gate) @ w[prefix + "o"].to(dtype).T


def memory_recurrence(q, k, v, log_in, log_keep, state=None):
    """The matrix memory's recurrence alone.  q, k [T, heads, dim] (q already scaled), v [T, heads, vdim], log
    gates [T, heads]; ``state`` (S [heads, dim, vdim], n [heads, dim], m [heads]) or None for zeros.  Returns
    the unnormalised head outputs [T, heads, vdim] and the state after the last token."""
    tokens, heads, dim = q.shape
    vdim, dtype = v.shape[2], q.dtype
    if state is None:
        S = torch.zeros(heads, dim, vdim, dtype=dtype)
        n = torch.zeros(heads, dim, dtype=dtype)
        m = torch.zeros(heads, dtype=dtype)
    else:
        S, n, m = (part.clone().to(dtype) for part in state)
    out = torch.zeros(tokens, heads, vdim, dtype=dtype)
    for t in range(tokens):
        m_new = torch.maximum(log_keep[t] + m, log_in[t])
        keep = torch.exp(log_keep[t] + m - m_new)
        take = torch.exp(log_in[t] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t].unsqueeze(2) * v[t].unsqueeze(1)
        n = keep[:, None] * n + take[:, None] * k[t]
        m = m_new
        top = torch.einsum("hdv,hd->hv", S, q[t])
        bottom = torch.maximum((n * q[t]).sum(1).abs(), torch.exp(-m)) + 1e-6
        out[t] = top / bottom.unsqueeze(1)
    return out, (S, n, m)


def matrix_memory(h, w, prefix, sizes, eps, dtype):
    """mLSTM: per head a matrix S [dim, vdim], a vector n [dim] and a running maximum m (0 at the start)."""
    heads, dim, vdim, cap = sizes["heads"], sizes["dim"], sizes["vdim"], sizes["gate_cap"]
    tokens = h.shape[0]
    q = (h @ w[prefix + "q"].to(dtype).T).view(tokens, heads, dim) * dim ** -0.5
    k = (h @ w[prefix + "k"].to(dtype).T).view(tokens, heads, dim)
    v = (h @ w[prefix + "v"].to(dtype).T).view(tokens, heads, vdim)
    log_in = cap * torch.tanh((h @ w[prefix + "i"].to(dtype).T + w[prefix + "i.b"].to(dtype)) / cap)
    log_keep = torch.nn.functional.logsigmoid(
        cap * torch.tanh((h @ w[prefix + "f"].to(dtype).T + w[prefix + "f.b"].to(dtype)) / cap))
    _note_first_token(q[0], k[0])
    out, _ = memory_recurrence(q, k, v, log_in, log_keep)
    out = rms(out, eps).reshape(tokens, heads * vdim) * w[prefix + "norm"].to(dtype)
    out = out * torch.sigmoid(h @ w[prefix + "g"].to(dtype).T)
    return out @ w[prefix + "o"].to(dtype).T


def side_by_side(h, w, prefix, sizes, eps, dtype):
    left = window_attention(h, w, prefix + "left.", sizes["left"], eps, dtype)
    right = matrix_memory(h, w, prefix + "right.", sizes["right"], eps, dtype)
    return sizes["left_scale"] * left + sizes["right_scale"] * right


def short_convolution(x, taps_weight, history=None):
    """Causal convolution over time per channel; the last tap is the current token's.  ``history``
    [taps - 1, channels]: the inputs before x's first row (zeros before the start of a request)."""
    tokens, channels = x.shape
    taps = taps_weight.shape[1]
    before = torch.zeros(taps - 1, channels, dtype=x.dtype) if history is None else history.to(x.dtype)
    padded = torch.cat([before, x])
    out = torch.zeros_like(x)
    for j in range(taps):
        out = out + padded[j:j + tokens] * taps_weight[:, j]
    return out


def delta_recurrence(q, k, v, beta, decay, state=None):
    """The gated delta rule alone.  q, k [T, groups, dim] (unit vectors, q scaled), v [T, heads, vdim], beta and
    decay [T, heads]; ``state`` S [heads, dim, vdim] or None for zeros.  Returns the head outputs and the state."""
    tokens, groups, dim = q.shape
    heads, vdim, dtype = v.shape[1], v.shape[2], q.dtype
    S = torch.zeros(heads, dim, vdim, dtype=dtype) if state is None else state.clone().to(dtype)
    out = torch.zeros(tokens, heads, vdim, dtype=dtype)
    for t in range(tokens):
        for head in range(heads):
            g = head // (heads // groups)
            S[head] = decay[t, head] * S[head]
            u = beta[t, head] * (v[t, head] - S[head].T @ k[t, g])
            S[head] = S[head] + torch.outer(k[t, g], u)
            out[t, head] = S[head].T @ q[t, g]
    return out, S


def gated_delta(h, w, prefix, sizes, eps, dtype):
    """Gated delta rule with short convolutions, unit q and k, one decay and one write strength per head."""
    heads, groups, dim, vdim = sizes["heads"], sizes["kv_heads"], sizes["dim"], sizes["vdim"]
    tokens = h.shape[0]
    silu = torch.nn.functional.silu
    q = silu(short_convolution(h @ w[prefix + "q"].to(dtype).T, w[prefix + "q.conv"].to(dtype))).view(tokens, groups, dim)
    k = silu(short_convolution(h @ w[prefix + "k"].to(dtype).T, w[prefix + "k.conv"].to(dtype))).view(tokens, groups, dim)
    v = silu(short_convolution(h @ w[prefix + "v"].to(dtype).T, w[prefix + "v.conv"].to(dtype))).view(tokens, heads, vdim)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    _note_first_token(q[0], k[0])
    beta = torch.sigmoid(h @ w[prefix + "b"].to(dtype).T)
    rate = torch.exp(w[prefix + "A_log"].to(dtype))
    decay = torch.exp(-rate * torch.nn.functional.softplus(h @ w[prefix + "a"].to(dtype).T + w[prefix + "dt_bias"].to(dtype)))
    out, _ = delta_recurrence(q, k, v, beta, decay)
    out = rms(out, eps) * w[prefix + "norm"].to(dtype)
    out = out.reshape(tokens, heads * vdim) * silu(h @ w[prefix + "g"].to(dtype).T)
    return out @ w[prefix + "o"].to(dtype).T


def squared_relu_feed_forward(h, w, prefix, dtype):
    return torch.relu(h @ w[prefix + "up"].to(dtype).T) ** 2 @ w[prefix + "down"].to(dtype).T


MIXERS = {"parallel": side_by_side, "delta": gated_delta}


def run_order(config):
    """(layer, number of the pass whose first layer this run is, or None) in the order the layers run."""
    count = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None) for i in range(count)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None) for i in range(start)]
    for t in range(times):
        order += [(i, t if i == start else None) for i in range(start, stop)]
    return order + [(i, None) for i in range(stop, count)]


def forward(tokens, weights, config, dtype=torch.float64, layers_out=None, round_inputs=False):
    """Logits [T, vocab] of one whole request; ``layers_out`` (a list) gets the stream after every layer run.
    ``round_inputs`` rounds every sublayer's normalised input to bfloat16 and nothing else: how far a row then
    moves tells how much of it rounding alone decides."""
    eps = config["norm"]["eps"]
    rounded = (lambda h: h.to(torch.bfloat16).to(dtype)) if round_inputs else (lambda h: h)
    x = embed_tokens(tokens, weights, config, dtype)
    for index, first_of_pass in run_order(config):
        layer = config["layers"][index]
        name = f"l{index}."
        if first_of_pass is not None:
            x = x + weights["loop.step"].to(dtype)[first_of_pass]
        h = rounded(rms(x, eps) * weights[name + "norm1"].to(dtype))
        x = x + MIXERS[layer["type"]](h, weights, name + "mix.", layer["mixer"], eps, dtype)
        if layer["mlp"] is not None:
            h = rounded(rms(x, eps) * weights[name + "norm2"].to(dtype))
            x = x + squared_relu_feed_forward(h, weights, name + "mlp.", dtype)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = rms(x, eps) * weights["final.norm"].to(dtype)
    return x @ weights["head"].to(dtype).T * config["logit_scale"]


def read_folder(folder):
    """(config.json dictionary, tensors as float32) of a model folder."""
    import safetensors.torch

    folder = Path(folder)
    raw = json.loads((folder / "config.json").read_text())
    tensors = {name: t.float() for name, t in safetensors.torch.load_file(str(folder / "model.safetensors")).items()}
    return raw, tensors


def first_token_margin(config, weights, tokens):
    """The smallest |cos(q, k)| over all recurrent heads of all layer runs at the request's first token."""
    global FIRST_TOKEN_COSINES
    FIRST_TOKEN_COSINES = []
    try:
        forward(tokens[:1], weights, config)
        return min(FIRST_TOKEN_COSINES, default=1.0)
    finally:
        FIRST_TOKEN_COSINES = None


def tensor_shapes(config):
    """Name -> shape of every tensor a model of this configuration stores."""
    width = config["width"]
    shapes = {"embed": (config["vocab"], width), "head": (config["vocab"], width), "final.norm": (width,)}
    if config.get("loop"):
        shapes["loop.step"] = (config["loop"]["times"], width)
    for index, layer in enumerate(config["layers"]):
        name = f"l{index}."
        shapes[name + "norm1"] = (width,)
        m = layer["mixer"]
        if layer["type"] == "parallel":
            a, b = m["left"], m["right"]
            p = name + "mix.left."
            shapes.update({p + "q": (a["heads"] * a["dim"], width), p + "k": (a["kv_heads"] * a["dim"], width),
                           p + "v": (a["kv_heads"] * a["vdim"], width), p + "q.norm": (a["dim"],),
                           p + "k.norm": (a["dim"],), p + "g": (a["heads"] * a["vdim"], width),
                           p + "o": (width, a["heads"] * a["vdim"])})
            p = name + "mix.right."
            shapes.update({p + "q": (b["heads"] * b["dim"], width), p + "k": (b["heads"] * b["dim"], width),
                           p + "v": (b["heads"] * b["vdim"], width), p + "g": (b["heads"] * b["vdim"], width),
                           p + "o": (width, b["heads"] * b["vdim"]), p + "norm": (b["heads"] * b["vdim"],),
                           p + "i": (b["heads"], width), p + "i.b": (b["heads"],),
                           p + "f": (b["heads"], width), p + "f.b": (b["heads"],)})
        else:
            p = name + "mix."
            qk, vv = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"]
            shapes.update({p + "q": (qk, width), p + "q.conv": (qk, m["conv"]), p + "k": (qk, width),
                           p + "k.conv": (qk, m["conv"]), p + "v": (vv, width), p + "v.conv": (vv, m["conv"]),
                           p + "b": (m["heads"], width), p + "A_log": (m["heads"],), p + "norm": (m["vdim"],),
                           p + "a": (m["heads"], width), p + "dt_bias": (m["heads"],), p + "g": (vv, width),
                           p + "o": (width, vv)})
        if layer["mlp"] is not None:
            shapes[name + "norm2"] = (width,)
            shapes[name + "mlp.up"] = (layer["mlp"]["ff"], width)
            shapes[name + "mlp.down"] = (width, layer["mlp"]["ff"])
    return shapes


def random_weights(config, seed, spread=1.0):
    """Random tensors (bfloat16-representable float32) for a configuration; gains around one."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm2") or name.endswith("norm"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=gen)
        elif len(shape) == 1:
            t = 0.5 * torch.randn(shape, generator=gen)
        elif leaf == "conv":
            t = torch.randn(shape, generator=gen) / math.sqrt(shape[1])
        elif name in ("embed", "loop.step"):
            t = torch.randn(shape, generator=gen) * (0.05 if name == "embed" else 0.2)
        else:
            t = torch.randn(shape, generator=gen) * spread / math.sqrt(shape[1])
        out[name] = t.to(torch.bfloat16).float()
    return out
