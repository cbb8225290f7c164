"""Plain, slow Gulazen forward pass: whole sequences, no cache, one function per mechanism.

The oracle of the Gulazen tests.  It shares no code with the package under test: it reads a model folder through the
``safetensors`` library, builds every attention as a dense [T, T] table per head, takes the short convolution as a
loop over its taps and runs every expert of a token in a Python loop.

A Gulazen layer reads the residual x itself and norms what a sublayer hands back:

    x <- x + ls1 * N1(mixer(x + conv(x)))        x <- x + ls2 * N2(ff(x))

with N(y) = y / sqrt(mean(y^2) + eps) * (1 + w).  The mixer is grouped-query attention without rotation, with an RMS
norm over a token's whole query (and key) projection, soft-capped scores that are mixed across heads before the
softmax, a sliding window that keeps a sequence's first tokens visible, and a learned sink in the softmax's
denominator.  The feed-forward is dense (one matrix up, a two-sided activation with two learned numbers, one matrix
down) or a mixture of gated experts chosen by their logits, with a shared expert.  The embedding takes a sinusoidal
position vector, and the output head is the embedding table.

Everything here is 32-bit.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch
from safetensors import safe_open


def read_folder(folder):
    """config.json as a dict and every tensor of the folder's *.safetensors files (floats widened to float32)."""
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    tensors = {}
    for path in sorted(folder.glob("*.safetensors")):
        with safe_open(str(path), framework="pt", device="cpu") as f:
            for name in f.keys():
                t = f.get_tensor(name)
                tensors[name] = t.to(torch.float32) if t.is_floating_point() else t
    return cfg, tensors


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def one_plus_norm(x, weight, eps):
    """RMS norm whose weight is stored around zero."""
    return unit_rms(x, eps) * (1.0 + weight)


# ---- embedding ---------------------------------------------------------------------------


def sinusoid(positions, width):
    """[T, width]: column 2i holds sin(p * 10000^(-2i / width)), column 2i + 1 the cosine of the same angle."""
    out = torch.zeros(len(positions), width)
    p = positions.to(torch.float32)
    for c in range(width):
        i = c // 2
        angle = p * torch.tensor(10000.0 ** (-2.0 * i / width), dtype=torch.float32)
        out[:, c] = torch.sin(angle) if c % 2 == 0 else torch.cos(angle)
    return out


# ---- the short convolution ---------------------------------------------------------------


def causal_conv(h, w):
    """h [T, width], w [width, taps]: out_t = sum_j w[:, j] * h_(t - taps + 1 + j), zeros before the start."""
    T, taps = h.shape[0], w.shape[1]
    out = torch.zeros_like(h)
    for t in range(T):
        for j in range(taps):
            src = t - taps + 1 + j
            if src >= 0:
                out[t] += w[:, j] * h[src]
    return out


# ---- the mixer ---------------------------------------------------------------------------


def visible(T, size, keep_first):
    """[T, T] True where key j is visible to query i: j <= i and (i - j < size or j < keep_first).  No size: causal."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if size is not None:
        seen &= ((i - j) < int(size)) | (j < int(keep_first))
    return seen


def raw_scores(q, k, m):
    """[H, T, T] scaled and capped scores of every query head against its key head."""
    H, G = m["heads"], m["kv_heads"]
    T = q.shape[0]
    s = torch.zeros(H, T, T)
    for head in range(H):
        s[head] = (q[:, head] @ k[:, head // (H // G)].T) * m["scale"]
    cap = m.get("softcap")
    if cap:
        s = cap * torch.tanh(s / cap)
    return s


def talk(scores, table):
    """New score of head h = sum over heads g of table[h, g] * score of head g."""
    return torch.einsum("hg,gij->hij", table, scores)


def sink_softmax(scores, seen, sink):
    """Softmax over the visible keys whose denominator also holds exp(sink) (one per head, or none)."""
    scores = scores.masked_fill(~seen, float("-inf"))
    if sink is None:
        return torch.softmax(scores, dim=-1)
    H, T, _ = scores.shape
    wide = torch.cat([scores, sink.reshape(H, 1, 1).expand(H, T, 1)], dim=-1)
    return torch.softmax(wide, dim=-1)[..., :-1]


def attention(h, w, m, eps):
    """h [T, width]; w: the mixer's tensors by short name; m: the mixer's config entry."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T)
    k = (h @ w["k"].T)
    v = (h @ w["v"].T).reshape(T, G, V)
    q = (unit_rms(q, eps) * w["q.norm"]).reshape(T, H, D)          # over the whole projection, before the heads are cut
    k = (unit_rms(k, eps) * w["k.norm"]).reshape(T, G, D)
    s = raw_scores(q, k, m)
    if "talk" in w:
        s = talk(s, w["talk"])
    mask = m.get("mask") or {}
    seen = visible(T, mask.get("size"), mask.get("keep_first", 0))
    p = sink_softmax(s, seen, w.get("sink"))
    out = torch.zeros(T, H, V)
    for head in range(H):
        out[:, head] = p[head] @ v[:, head // (H // G)]
    return out.reshape(T, H * V) @ w["o"].T


# ---- feed-forwards -----------------------------------------------------------------------


def xielu(z, p, q):
    """softplus(p) z^2 + z / 2 for z > 0;  (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2 for z <= 0."""
    ap = torch.nn.functional.softplus(p)
    an = 0.5 + torch.nn.functional.softplus(q)
    pos = ap * z * z + 0.5 * z
    neg = an * (torch.exp(torch.clamp(z, max=0.0)) - 1.0 - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def dense_ff(h, w):
    return xielu(h @ w["up"].T, w["act"][0], w["act"][1]) @ w["down"].T


def gated_expert(h, w, prefix):
    g = h @ w[prefix + "gate"].T
    return (g * torch.sigmoid(g) * (h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def route(h, w, top):
    """(chosen [T, top], weights [T, top]): the largest logits, softmax over the chosen logits only."""
    z = h @ w["router"].T + w["router.b"]
    best = torch.topk(z, top, dim=-1)
    return best.indices, torch.softmax(best.values, dim=-1)


def moe_ff(h, w, mlp):
    top = int(mlp["router"]["top"])
    chosen, weights = route(h, w, top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(top):
            e = int(chosen[t, c])
            out[t] += weights[t, c] * gated_expert(h[t:t + 1], w, f"e{e}.")[0]
    if mlp.get("shared") is not None:
        out = out + gated_expert(h, w, "shared.")
    return out


# ---- the model ---------------------------------------------------------------------------


def sub(tensors, prefix):
    return {name[len(prefix):]: t for name, t in tensors.items() if name.startswith(prefix)}


def layer(x, i, cfg, tensors, trace=None):
    entry = cfg["layers"][i]
    eps = float(cfg["norm"]["eps"])
    p = f"l{i}."
    h = x
    if p + "canon1" in tensors:
        h = h + causal_conv(h, tensors[p + "canon1"])
    if entry["type"] != "attention":
        raise ValueError(f"no mixer of type {entry['type']!r}")
    y = attention(h, sub(tensors, p + "mix."), entry["mixer"], eps)
    y = one_plus_norm(y, tensors[p + "norm1"], eps)
    if p + "ls1" in tensors:
        y = y * tensors[p + "ls1"]
    x = x + y
    mlp = entry.get("mlp")
    if mlp is not None:
        w = sub(tensors, p + "mlp.")
        y = dense_ff(x, w) if mlp["kind"] == "dense" else moe_ff(x, w, mlp)
        y = one_plus_norm(y, tensors[p + "norm2"], eps)
        if p + "ls2" in tensors:
            y = y * tensors[p + "ls2"]
        x = x + y
    return x


def hidden(cfg, tensors, tokens, layers_out=None):
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = tensors["embed"][ids] + sinusoid(torch.arange(len(ids)), int(cfg["width"]))
    for i in range(len(cfg["layers"])):
        x = layer(x, i, cfg, tensors)
        if layers_out is not None:
            layers_out.append(x.clone())
    return x


def forward(cfg, tensors, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence at every position."""
    x = hidden(cfg, tensors, tokens, layers_out)
    return one_plus_norm(x, tensors["final.norm"], float(cfg["norm"]["eps"])) @ tensors["embed"].T


def generate(cfg, tensors, prompts, n_new):
    """Greedy continuation of every prompt by ``n_new`` tokens: the whole sequence is run again for every token."""
    out = []
    for prompt in prompts:
        seq, new = list(prompt), []
        for _ in range(n_new):
            tok = int(forward(cfg, tensors, seq)[-1].argmax())
            new.append(tok)
            seq.append(tok)
        out.append(new)
    return out
