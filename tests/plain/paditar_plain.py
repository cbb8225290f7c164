"""Plain, slow Paditar forward pass: whole sequences, no cache, one function per mechanism.

The oracle of the Paditar tests.  It shares no code with the package under test: it reads a model folder through the
``safetensors`` library, builds every attention as a dense [T, T] table per head and map, takes the short convolution
as a loop over its taps and walks the matrix memory token by token.

A Paditar layer norms a sublayer's input and what the sublayer hands back:

    x <- x + N1b(mixer(N1(x)))        x <- x + N2b(ff(N2(x)))

with N(y) = y / sqrt(mean(y^2) + eps) * (1 + w).  A run of layers repeats with the same weights; before every pass but
the first the embedding output is added to x, and before every pass a vector of that pass.  The mixer is either an
attention with two score maps per head (partly rotated, joined as a1 - lambda a2, unit-normed per head, gated element
by element) or two mixers side by side: an attention whose values are its keys (biases, a short convolution, per-head
norms, a query temperature, a softmax with 1 in the denominator, a gate per head) and an mLSTM matrix memory.  The
feed-forward is up, squared relu, down, and the output head is the embedding table.

Everything here is 64-bit, so that what is compared against it is the library's rounding and nothing else.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch
from safetensors import safe_open

F = torch.float64


def read_folder(folder):
    """config.json as a dict and every tensor of the folder's *.safetensors files (floats widened to float64)."""
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    tensors = {}
    for path in sorted(folder.glob("*.safetensors")):
        with safe_open(str(path), framework="pt", device="cpu") as f:
            for name in f.keys():
                t = f.get_tensor(name)
                tensors[name] = t.to(F) if t.is_floating_point() else t
    return cfg, tensors


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def one_plus_norm(x, weight, eps):
    """RMS norm whose weight is stored around zero."""
    return unit_rms(x, eps) * (1.0 + weight)


def causal_table(T):
    return torch.ones(T, T, dtype=torch.bool).tril()


# ---- attention with two score maps ----------------------------------------------------------


def rotate_half(t, positions, base, dims):
    """t [T, ..., D]: of the first ``dims`` columns, column i turns with column i + dims / 2 by positions * base^(-2i / dims)."""
    half = dims // 2
    out = t.clone()
    for i in range(half):
        angle = positions.to(F) * base ** (-2.0 * i / dims)
        c, s = torch.cos(angle), torch.sin(angle)
        shape = (-1,) + (1,) * (t.dim() - 2)
        c, s = c.reshape(shape), s.reshape(shape)
        u, v = t[..., i], t[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


def softmax_attention(q, k, v, scale, extra_one=False):
    """One head: q [T, D], k [T, D], v [T, V]; causal; ``extra_one`` adds 1 to the softmax's denominator."""
    T = q.shape[0]
    s = (q @ k.T) * scale
    s = s.masked_fill(~causal_table(T), float("-inf"))
    top = s.max(dim=-1, keepdim=True).values
    if extra_one:
        top = top.clamp(min=0.0)
    e = torch.exp(s - top)
    total = e.sum(dim=-1, keepdim=True)
    if extra_one:
        total = total + torch.exp(-top)
    return (e / total) @ v


def diff_lambda(w, diff):
    return math.exp(float((w["lq1"] * w["lk1"]).sum())) - math.exp(float((w["lq2"] * w["lk2"]).sum())) + diff


def diff_attention(h, w, m, eps):
    """h [T, width]; w: the mixer's tensors by their last name; m: the mixer's entry of config.json."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).reshape(T, H, 2, D)
    k = (h @ w["k"].T).reshape(T, G, 2, D)
    v = (h @ w["v"].T).reshape(T, G, V)
    if m.get("rot") is not None:
        pos = torch.arange(T)
        q = rotate_half(q, pos, float(m["rot"]["base"]), int(m["rot"]["dims"]))
        k = rotate_half(k, pos, float(m["rot"]["base"]), int(m["rot"]["dims"]))
    lam = diff_lambda(w, float(m["diff"]))
    heads = []
    for head in range(H):
        g = head // (H // G)
        a1 = softmax_attention(q[:, head, 0], k[:, g, 0], v[:, g], float(m["scale"]))
        a2 = softmax_attention(q[:, head, 1], k[:, g, 1], v[:, g], float(m["scale"]))
        heads.append(unit_rms(a1 - lam * a2, eps) * (1.0 - float(m["diff"])))
    o = torch.cat(heads, dim=-1) * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


# ---- attention whose values are its keys ------------------------------------------------------


def short_convolution(u, weight):
    """u [T, C], weight [C, taps]: y_t = sum_j weight[:, j] * u_(t - taps + 1 + j), zeros before the start."""
    T, C = u.shape
    taps = weight.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            src = t - taps + 1 + j
            if src >= 0:
                y[t] += weight[:, j] * u[src]
    return y


def query_temperature(T, coef, every):
    return torch.tensor([1.0 + coef * math.log((p + 1) // every + 1) for p in range(T)], dtype=F)


def key_value_attention(h, w, m, eps):
    """The left side.  w: {"q", "q.b", "k", "k.b", "q.conv", "k.conv", "q.norm", "k.norm", "g", "o", "o.b"}."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = h @ w["q"].T + w["q.b"]
    k = h @ w["k"].T + w["k.b"]
    if m.get("conv"):
        q, k = short_convolution(q, w["q.conv"]), short_convolution(k, w["k.conv"])
    values = k.reshape(T, G, D)
    q = unit_rms(q.reshape(T, H, D), eps) * w["q.norm"]
    kn = unit_rms(k.reshape(T, G, D), eps) * w["k.norm"]
    if m.get("q_temp") is not None:
        q = q * query_temperature(T, float(m["q_temp"]["coef"]), int(m["q_temp"]["every"]))[:, None, None]
    gate = torch.sigmoid(h @ w["g"].T)
    heads = []
    for head in range(H):
        g = head // (H // G)
        heads.append(softmax_attention(q[:, head], kn[:, g], values[:, g], float(m["scale"]), extra_one=True) * gate[:, head:head + 1])
    return torch.cat(heads, dim=-1) @ w["o"].T + w["o.b"]


# ---- the matrix memory -------------------------------------------------------------------------


def matrix_memory(h, w, m, eps):
    """The right side.  w: {"q", "k", "v", "g", "o", "norm", "i", "i.b", "f", "f.b"}."""
    T = h.shape[0]
    H, D, V, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ w["q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ w["k"].T).reshape(T, H, D)
    v = (h @ w["v"].T).reshape(T, H, V)
    log_i = cap * torch.tanh((h @ w["i"].T + w["i.b"]) / cap)
    log_f = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w["f"].T + w["f.b"]) / cap))
    out = torch.zeros(T, H, V, dtype=F)
    for head in range(H):
        S = torch.zeros(D, V, dtype=F)
        n = torch.zeros(D, dtype=F)
        top = 0.0
        for t in range(T):
            new_top = max(float(log_f[t, head]) + top, float(log_i[t, head]))
            keep, take = math.exp(float(log_f[t, head]) + top - new_top), math.exp(float(log_i[t, head]) - new_top)
            S = keep * S + take * torch.outer(k[t, head], v[t, head])
            n = keep * n + take * k[t, head]
            top = new_top
            out[t, head] = (S.T @ q[t, head]) / (max(abs(float(n @ q[t, head])), math.exp(-top)) + 1e-6)
    o = unit_rms(out, eps).reshape(T, H * V) * w["norm"] * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def side_by_side(h, w_left, w_right, m, eps):
    return (float(m["left_scale"]) * key_value_attention(h, w_left, m["left"], eps)
            + float(m["right_scale"]) * matrix_memory(h, w_right, m["right"], eps))


# ---- feed-forward, layers, the model ------------------------------------------------------------


def feed_forward(h, up, down):
    return torch.relu(h @ up.T) ** 2 @ down.T


def below(tensors, prefix):
    """{name without the prefix: tensor} of the tensors whose names start with it."""
    return {name[len(prefix):]: t for name, t in tensors.items() if name.startswith(prefix)}


def layer(x, cfg, tensors, i):
    entry, eps, p = cfg["layers"][i], float(cfg["norm"]["eps"]), f"l{i}."
    h = one_plus_norm(x, tensors[p + "norm1"], eps)
    if entry["type"] == "attention":
        y = diff_attention(h, below(tensors, p + "mix."), entry["mixer"], eps)
    else:
        y = side_by_side(h, below(tensors, p + "mix.left."), below(tensors, p + "mix.right."), entry["mixer"], eps)
    x = x + one_plus_norm(y, tensors[p + "norm1b"], eps)
    if entry.get("mlp") is not None:
        h = one_plus_norm(x, tensors[p + "norm2"], eps)
        x = x + one_plus_norm(feed_forward(h, tensors[p + "mlp.up"], tensors[p + "mlp.down"]), tensors[p + "norm2b"], eps)
    return x


def layer_runs(cfg):
    """[(layer, number of the pass that starts here or None)] in the order the layers run."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if loop is None:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg, tensors, tokens, layers_out=None):
    """Logits [T, vocab] (32-bit) of one sequence; ``layers_out`` receives the residual after every layer run."""
    embedded = tensors["embed"][torch.tensor(tokens)]
    x = embedded.clone()
    for i, t in layer_runs(cfg):
        if t is not None:
            if t > 0:
                x = x + embedded
            x = x + tensors["loop.step"][t]
        x = layer(x, cfg, tensors, i)
        if layers_out is not None:
            layers_out.append(x.to(torch.float32))
    x = one_plus_norm(x, tensors["final.norm"], float(cfg["norm"]["eps"]))
    return (x @ tensors["embed"].T).to(torch.float32)


def generate(cfg, tensors, prompts, n_new):
    """Greedy continuation of every prompt by ``n_new`` tokens, each from a full forward pass."""
    out = []
    for prompt in prompts:
        seq = list(prompt)
        for _ in range(n_new):
            seq.append(int(forward(cfg, tensors, seq)[-1].argmax()))
        out.append(seq[len(prompt):])
    return out
