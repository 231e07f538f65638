"""Bilipel in plain double-precision PyTorch: one function per mechanism, whole sequences only, no cache.

The oracle of the Bilipel tests.  It shares nothing with the product path: it takes the configuration as the
dictionary that config.json holds and the weights as a dictionary of tensors by their stored names, and walks
a whole sequence at once (the recurrence token by token), so every cutting of a prompt, every batch and every
page layout of the engine is held to the same numbers.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def layer_norm(x, gain, bias, eps):
    centred = x - x.mean(-1, keepdim=True)
    return centred / torch.sqrt((centred * centred).mean(-1, keepdim=True) + eps) * gain + bias


def rms_norm(x, gain, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * gain


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def rotary_frequencies(rot):
    """f_i for i < dims / 2; with ``scaling`` every frequency is blended between itself and itself / factor."""
    dims, base = int(rot["dims"]), float(rot["base"])
    plain = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    scaling = rot.get("scaling")
    if not scaling:
        return torch.tensor(plain, dtype=F64), 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_index(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    low = max(math.floor(pair_index(float(scaling["fast"]))), 0)
    high = min(math.ceil(pair_index(float(scaling["slow"]))), dims - 1)
    blended = []
    for i, f in enumerate(plain):
        ramp = min(max((i - low) / max(high - low, 0.001), 0.0), 1.0)
        blended.append(f / factor * ramp + f * (1.0 - ramp))
    return torch.tensor(blended, dtype=F64), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot, interleaved):
    """x: [T, heads, size]; the first rot.dims elements of every head turn by position * f_i."""
    dims = int(rot["dims"])
    freq, magnitude = rotary_frequencies(rot)
    angle = positions.to(F64).view(-1, 1, 1) * freq.view(1, 1, -1)
    cos, sin = torch.cos(angle) * magnitude, torch.sin(angle) * magnitude
    out = x.clone()
    if interleaved:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * cos - v * sin
        out[..., 1:dims:2] = v * cos + u * sin
    else:
        u, v = x[..., : dims // 2], x[..., dims // 2: dims]
        out[..., : dims // 2] = u * cos - v * sin
        out[..., dims // 2: dims] = v * cos + u * sin
    return out


def softmax_with_sink(scores, visible, sink):
    """scores [T, T] of one head; ``visible`` a boolean mask; ``sink`` one number that joins the denominator."""
    scores = scores.masked_fill(~visible, -math.inf)
    top = torch.maximum(scores.max(-1, keepdim=True).values, torch.as_tensor(sink, dtype=F64))
    weights = torch.exp(scores - top)
    return weights / (weights.sum(-1, keepdim=True) + torch.exp(sink - top))


def visibility(tokens, window=0):
    i = torch.arange(tokens).view(-1, 1)
    j = torch.arange(tokens).view(1, -1)
    seen = j <= i
    if window:
        seen &= (i - j) < window
    return seen


def attention_mixer(h, w, m, eps):
    heads, groups, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    tokens = h.shape[0]
    positions = torch.arange(tokens)
    q = rms_norm(h @ w["q"].T, w["q.norm"], eps).view(tokens, heads, dim)
    k = rms_norm(h @ w["k"].T, w["k.norm"], eps).view(tokens, groups, dim)
    v = (h @ w["v"].T).view(tokens, groups, vdim)
    q, k = rotate(q, positions, m["rot"], False), rotate(k, positions, m["rot"], False)
    seen = visibility(tokens)
    out = []
    for head in range(heads):
        group = head // (heads // groups)
        weights = softmax_with_sink(q[:, head] @ k[:, group].T * m["scale"], seen, w["sink"][head])
        out.append(weights @ v[:, group])
    return torch.cat(out, -1) @ w["o"].T


def latent_mixer(h, w, m, eps):
    heads, dim, rot_dim, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    tokens = h.shape[0]
    positions = torch.arange(tokens)
    rot = dict(m["rot"], dims=rot_dim)
    q = (h @ w["q"].T).view(tokens, heads, dim + rot_dim)
    q_plain, q_turned = q[..., :dim], rotate(q[..., dim:], positions, rot, True)
    down = h @ w["dkv"].T
    latent = rms_norm(down[:, :rank], w["dkv.norm"], eps)
    k_turned = rotate(down[:, rank:].view(tokens, 1, rot_dim), positions, rot, True)[:, 0]
    k_plain = (latent @ w["uk"].T).view(tokens, heads, dim)
    values = (latent @ w["uv"].T).view(tokens, heads, vdim)
    seen = visibility(tokens, (m.get("mask") or {}).get("size", 0))
    out = []
    for head in range(heads):
        scores = (q_plain[:, head] @ k_plain[:, head].T + q_turned[:, head] @ k_turned.T) * m["scale"]
        out.append(softmax_with_sink(scores, seen, w["sink"][head]) @ values[:, head])
    return torch.cat(out, -1) @ w["o"].T


def gla_recurrence(q, k, v, alpha):
    """q, k, alpha [T, heads, dim], v [T, heads, vdim]: S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T q_t."""
    tokens, heads, dim = q.shape
    state = torch.zeros(heads, dim, v.shape[-1], dtype=F64)
    out = []
    for t in range(tokens):
        state = alpha[t].unsqueeze(-1) * state + k[t].unsqueeze(-1) * v[t].unsqueeze(-2)
        out.append(torch.einsum("hdv,hd->hv", state, q[t]))
    return torch.stack(out)


def gla_mixer(h, w, m, eps):
    heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
    tokens = h.shape[0]
    q = (h @ w["q"].T).view(tokens, heads, dim) * dim ** -0.5
    k = (h @ w["k"].T).view(tokens, heads, dim)
    v = (h @ w["v"].T).view(tokens, heads, vdim)
    z = (h @ w["a1"].T) @ w["a2"].T + w["a2.b"]
    alpha = torch.sigmoid(z).pow(1.0 / m["tau"]).view(tokens, heads, dim)
    o = rms_norm(gla_recurrence(q, k, v, alpha), w["norm"], eps).reshape(tokens, heads * vdim)
    return (o * silu(h @ w["g"].T)) @ w["o"].T


def dense_feed_forward(h, w):
    return (gelu_tanh(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def routed_feed_forward(h, w, mlp):
    logits = h @ w["router"].T + w["router.b"]
    chosen = torch.topk(logits, int(mlp["router"]["top"]), dim=-1)
    share = torch.softmax(chosen.values, -1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for slot, expert in enumerate(chosen.indices[t].tolist()):
            e = f"e{expert}."
            y = (silu(h[t] @ w[e + "gate"].T) * (h[t] @ w[e + "up"].T)) @ w[e + "down"].T
            out[t] += share[t, slot] * y
    return out


MIXERS = {"attention": attention_mixer, "latent_attention": latent_mixer, "gla": gla_mixer}


def sub(weights, prefix):
    return {name[len(prefix):]: tensor.to(F64) for name, tensor in weights.items() if name.startswith(prefix)}


def rounded(h, on):
    """The sublayer's input as a bfloat16 product would see it (``on``), or as it is."""
    return h.to(torch.bfloat16).to(F64) if on else h


def run_layer(x, config, weights, index, round_inputs=False):
    layer, eps, mult = config["layers"][index], config["norm"]["eps"], config.get("residual_mult", 1.0)
    w = sub(weights, f"l{index}.")
    h = rounded(layer_norm(x, w["norm1"], w["norm1.b"], eps), round_inputs)
    x = x + mult * MIXERS[layer["type"]](h, sub(w, "mix."), layer["mixer"], eps)
    if layer.get("mlp"):
        h = rounded(layer_norm(x, w["norm2"], w["norm2.b"], eps), round_inputs)
        ff = sub(w, "mlp.")
        x = x + mult * (dense_feed_forward(h, ff) if layer["mlp"]["kind"] == "dense"
                        else routed_feed_forward(h, ff, layer["mlp"]))
    return x


def run_order(config):
    """(layer, pass number or None): pass numbers mark a looped run's first layer."""
    count, loop = len(config["layers"]), config.get("loop")
    if not loop:
        return [(i, None) for i in range(count)]
    order = [(i, None) for i in range(loop["start"])]
    for number in range(loop["times"]):
        order += [(i, number if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return order + [(i, None) for i in range(loop["stop"], count)]


def read_folder(folder):
    """config.json as a dictionary and the stored tensors by name."""
    import json
    from pathlib import Path

    import safetensors.torch

    with open(Path(folder) / "config.json", encoding="utf-8") as handle:
        config = json.load(handle)
    return config, safetensors.torch.load_file(str(Path(folder) / "model.safetensors"))


def greedy(config, weights, prompt, count):
    """``count`` tokens after ``prompt``, each the argmax (lowest index on ties) of the whole sequence so far."""
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(int(torch.argmax(forward(config, weights, tokens)[-1])))
    return tokens[len(prompt):]


def forward(config, weights, tokens, streams=None, round_inputs=False):
    """Logits [T, vocab] of one sequence in float64.  ``streams``: a list that receives the stream after every layer
    run.  ``round_inputs``: every sublayer reads its input rounded to bfloat16 (everything else stays exact)."""
    w = {name: tensor.to(F64) for name, tensor in weights.items()}
    embedded = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x = embedded
    for index, number in run_order(config):
        if number is not None:
            if number > 0:
                x = x + embedded
            x = x + w["loop.step"][number]
        x = run_layer(x, config, weights, index, round_inputs)
        if streams is not None:
            streams.append(x)
    x = layer_norm(x, w["final.norm"], w["final.norm.b"], config["norm"]["eps"])
    return x @ w["head"].T
