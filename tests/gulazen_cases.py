"""Small Gulazen configurations for the tests, and the plain implementation's logits for them.

The configurations differ from one another in every size and option: convolutions of 1, 2, 4 and 5 taps and none; fewer
key/value heads than query heads, as many, and a single head; key and value widths that differ; windows of 7, 20, one
page and more, and none; 0, 1, 3 and more kept first tokens than a window is long; caps from 2 to 50 and none; experts
with and without a shared expert, one choice, all experts chosen; a layer without feed-forward; dense and expert layers
in different orders.
"""

from __future__ import annotations

import copy

import torch

from plain import gulazen_plain as plain
from starter_b200.config import config_from_dict
from starter_b200.weights import write_model_folder


def _attention(heads, kv_heads, dim, vdim, window=None, keep=0, softcap=None, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale}
    if softcap is not None:
        m["softcap"] = softcap
    if window is not None:
        m["mask"] = {"size": window, "keep_first": keep}
    return {"type": "attention", "mixer": m}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff, shared=None):
    mlp = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared is not None:
        mlp["shared"] = {"ff": shared}
    return mlp


def _with(entry, mlp):
    entry = copy.deepcopy(entry)
    entry["mlp"] = copy.deepcopy(mlp)
    return entry


def _model(vocab, width, eps, taps, layers):
    raw = {"architecture": "Gulazen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if taps:
        raw["canon"] = {"taps": taps}
    return raw


CASES = {
    # four taps; windows of 20 and 7 with 3 and 1 kept tokens, and one without a window; a last layer without feed-forward
    "A": _model(211, 96, 1e-5, 4, [
        _with(_attention(6, 2, 16, 24, window=20, keep=3, softcap=8.0, scale=0.4), _moe(5, 3, 40, shared=56)),
        _with(_attention(4, 4, 8, 16, window=7, keep=1, softcap=50.0), _dense(136)),
        _with(_attention(3, 1, 24, 8, softcap=2.0), _moe(4, 1, 72)),
        _with(_attention(6, 3, 16, 16, window=33, keep=0, softcap=15.0), None)]),
    # sizes the tensor-core kernels take (keys of 32 and 64 columns, values of 64 and 128, a window of one page and one
    # of 100), two taps, all experts chosen
    "B": _model(300, 128, 1e-6, 2, [
        _with(_attention(8, 2, 32, 64, window=64, keep=5, softcap=20.0), _dense(256)),
        _with(_attention(2, 1, 64, 128, window=100, keep=70, softcap=30.0, scale=0.2), _moe(3, 3, 80, shared=96)),
        _with(_attention(4, 4, 64, 64, window=130, keep=2, softcap=10.0), _moe(6, 2, 64, shared=32)),
        _with(_attention(16, 4, 32, 64, window=70, keep=64), _dense(192))]),
    # no convolution, single heads, widths that are no multiples of 8, more kept tokens than the window is long
    "C": _model(97, 40, 1e-4, 0, [
        _with(_attention(1, 1, 20, 12, window=5, keep=9, softcap=5.0), _dense(52)),
        _with(_attention(3, 1, 6, 10, softcap=12.0), _moe(2, 2, 24, shared=16)),
        _with(_attention(5, 5, 12, 4, window=40, keep=1), _dense(20))]),
    # five taps over a short window
    "D": _model(64, 32, 1e-5, 5, [_with(_attention(2, 2, 8, 8, window=3, keep=0, softcap=4.0), _moe(2, 1, 16)),
                                  _with(_attention(2, 1, 8, 16, window=4, keep=2, softcap=6.0), None)]),
    # one tap (the convolution keeps no state), a window of one token, a width that is no multiple of 4, 24 heads (two
    # per warp of the tensor-core kernel), all experts chosen and none shared, a single head without a window
    "E": _model(77, 30, 1e-5, 1, [_with(_attention(2, 2, 6, 10, window=1, keep=0, softcap=3.0), _dense(14)),
                                  _with(_attention(24, 8, 16, 64, window=50, keep=3, softcap=20.0), _moe(3, 3, 10)),
                                  _with(_attention(1, 1, 4, 4), None)]),
}
SEEDS = {"A": 25, "B": 26, "C": 27, "D": 28, "E": 29}


def config(name):
    return config_from_dict(copy.deepcopy(CASES[name]))


def write_folder(name, folder, dtype=torch.bfloat16, shards=1):
    return write_model_folder(config(name), SEEDS[name], folder, dtype=dtype, shards=shards)


def plain_logits(folder, seqs):
    cfg, tensors = plain.read_folder(folder)
    return [plain.forward(cfg, tensors, s) for s in seqs]
