"""Small Paditar configurations for the tests, and the plain implementation's logits for them.

The configurations differ from one another in every size and option: loops over the first layers, over inner layers, up
to the last layer, of one pass, and none; rotations over part of a head, over the whole head, and none; fewer key/value
heads than query heads, as many, and a single head; convolutions of 1, 2, 3 and 5 taps and none; a query temperature
that steps at every position, every 5, every 64, and none; matrix memories with keys wider than 128 columns and values
wider than 64 (the recurrence kernel's other paths), caps from 1.5 to 30; scales of the two sides that are equal, 1 and
far apart; a layer without feed-forward; widths that are no multiples of 8 or of 4, and odd head sizes.
"""

from __future__ import annotations

import copy

import torch

from plain import paditar_plain as plain
from starter_b200.config import config_from_dict
from starter_b200.weights import write_model_folder


def _attention(heads, kv_heads, dim, vdim, diff, rot=None, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff, "scale": dim ** -0.5 if scale is None else scale}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return {"type": "attention", "mixer": m}


def _parallel(left, right, left_scale, right_scale):
    heads, kv_heads, dim, conv, temp, scale = left
    lm = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5 if scale is None else scale}
    if conv is not None:
        lm["conv"] = conv
    if temp is not None:
        lm["q_temp"] = {"coef": temp[0], "every": temp[1]}
    rh, rd, rv, cap = right
    return {"type": "parallel", "mixer": {"left": lm, "right": {"heads": rh, "dim": rd, "vdim": rv, "gate_cap": cap},
                                          "left_scale": left_scale, "right_scale": right_scale}}


def _with(entry, ff):
    entry = copy.deepcopy(entry)
    entry["mlp"] = {"kind": "dense", "ff": ff} if ff else None
    return entry


def _model(vocab, width, eps, loop, layers):
    raw = {"architecture": "Paditar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop is not None:
        raw["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return raw


CASES = {
    # three passes over the two inner layers; part of a head rotated; three taps; a temperature that steps every 5 positions
    "A": _model(211, 96, 1e-5, (1, 3, 3), [
        _with(_attention(6, 2, 16, 24, 0.7, rot=(500.0, 8), scale=0.4), 136),
        _with(_parallel((4, 2, 24, 3, (0.5, 5), None), (3, 16, 24, 8.0), 1.5, 0.25), 72),
        _with(_attention(4, 4, 8, 16, 0.2, rot=(10000.0, 8)), None),
        _with(_parallel((2, 1, 32, 2, (1.0, 1), 0.3), (2, 40, 72, 15.0), 1.0, 1.0), 40)]),
    # sizes the tensor-core kernels take; two passes from the first layer on; a temperature that steps once a page
    "B": _model(300, 128, 1e-6, (0, 2, 2), [
        _with(_parallel((4, 1, 64, 4, (0.25, 64), None), (2, 64, 64, 11.0), 0.8, 1.3), 256),
        _with(_attention(8, 2, 32, 64, 0.5, rot=(1000000.0, 16)), 192),
        _with(_attention(2, 1, 64, 128, 0.8, rot=(10000.0, 64), scale=0.2), 64)]),
    # no loop, no rotation, single heads, one tap and no convolution at all, no temperature, widths that are no multiples
    # of 8, keys of the memory wider than 128 columns and values wider than 64
    "C": _model(97, 40, 1e-4, None, [
        _with(_parallel((1, 1, 20, 1, None, None), (1, 136, 12, 1.5), 2.0, 0.5), 52),
        _with(_attention(1, 1, 20, 12, 0.9), 20),
        _with(_parallel((3, 3, 6, None, (0.1, 7), None), (2, 10, 130, 30.0), 0.5, 2.0), None),
        _with(_attention(5, 5, 12, 4, 0.4, rot=(100.0, 4)), 24)]),
    # one pass (the loop's vector is still added), the loop reaches the last layer, five taps
    "D": _model(64, 32, 1e-5, (1, 2, 1), [_with(_attention(2, 2, 8, 8, 0.6, rot=(10000.0, 2)), 16),
                                          _with(_parallel((2, 2, 8, 5, (2.0, 3), None), (4, 8, 8, 5.0), 1.0, 0.7), 48)]),
    # a width that is no multiple of 4, odd head sizes everywhere (rows that no 16-byte read fits), an odd vocabulary, the loop
    # over all layers, eight taps, twelve query heads on one key head
    "E": _model(131, 30, 1e-6, (0, 3, 2), [
        _with(_parallel((3, 1, 7, 8, (0.7, 2), 0.5), (3, 5, 3, 4.0), 0.9, 1.1), 14),
        _with(_attention(3, 1, 5, 7, 0.35, rot=(50.0, 2)), 22),
        _with(_parallel((12, 1, 4, 2, None, None), (1, 9, 65, 9.0), 1.0, 0.3), None)]),
}
SEEDS = {"A": 35, "B": 36, "C": 37, "D": 38, "E": 39}


def config(name):
    return config_from_dict(copy.deepcopy(CASES[name]))


def write_folder(name, folder, dtype=torch.bfloat16, shards=1):
    return write_model_folder(config(name), SEEDS[name], folder, dtype=dtype, shards=shards)


def plain_logits(folder, seqs):
    cfg, tensors = plain.read_folder(folder)
    return [plain.forward(cfg, tensors, s) for s in seqs]
