"""Gulazen through the library's own cache, step function and generation loop on a CPU (the kernels' meaning restated
in torch, tests/emulated_ops.py), against the plain implementation: what is tested here is the host side, i.e. the
configuration, the layer's two cache entries, the pinned pages of the kept first tokens, the cutting of work into steps."""

import copy
import json

import pytest
import torch

import gulazen_cases as cases
from conftest import random_tokens
from emulated_ops import EmulatedOps
from helpers import assert_close, run_ragged_batches, run_tail_by_one, run_whole
from plain import gulazen_plain as plain
from starter_b200.cache import KVGroup, StateGroup
from starter_b200.cache.cache import PAGE
from starter_b200.config import ConfigError, config_from_dict, load_config
from starter_b200.engine import Engine
from starter_b200.engine.session import Session


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: cases.write_folder(name, tmp_path_factory.mktemp(f"gulazen_{name}"), dtype=torch.float32) for name in cases.CASES}


def session(folder, **kw):
    args = dict(dtype="float32", device="cpu", ops=EmulatedOps(), max_tokens=64 * 12, max_seqs=4)
    args.update(kw)
    return Session(folder, **args)


def test_configuration_round_trip_and_parts(folders):
    cfg = load_config(folders["A"])
    assert cfg.architecture == "Gulazen" and config_from_dict(cfg.to_dict()) == cfg
    spec = cfg.model_spec()
    assert spec.residual_float32 and spec.tie_embeddings and spec.position_embedding.base == 10000.0
    assert [b.kind for b in spec.layers] == ["postnorm"] * 4 and [b.mixer.kind for b in spec.layers] == ["talking_attention"] * 4
    assert [b.ff.kind if b.ff is not None else None for b in spec.layers] == ["moe", "act_mlp", "moe", None]
    m = spec.layers[0].mixer
    assert (m.window, m.keep_first, m.softcap, m.scale, m.v_dim) == (20, 3, 8.0, 0.4, 24)
    assert spec.layers[2].mixer.window is None and spec.layers[2].mixer.keep_first == 0
    assert spec.layers[3].mixer.softcap == 15.0 and spec.layers[3].ff_norm is None and spec.layers[0].conv.taps == 4
    assert spec.layers[0].ff.over_chosen and spec.layers[0].ff.router_bias and spec.layers[0].ff.shared.intermediate_size == 56
    assert spec.layers[2].ff.shared is None and spec.layers[2].ff.top == 1
    names = cfg.tensor_names()
    assert names.layers[0]["mixer"]["q_norm"] == "l0.mix.q.norm" and names.layers[0]["ff"]["router_bias"] == "l0.mlp.router.b"
    assert names.layers[1]["ff"]["act"] == "l1.mlp.act" and names.layers[2]["ff_norm"]["scale"] == "l2.ls2"
    assert names.layers[3]["conv"]["weight"] == "l3.canon1" and "ff" not in names.layers[3]
    bare = cases.config("C")
    assert bare.model_spec().layers[0].conv is None and "conv" not in bare.tensor_names().layers[0]
    assert bare.model_spec().layers[2].mixer.softcap is None


@pytest.mark.parametrize("change, what", [
    (lambda r: r["layers"][0].update(type="conv"), "unknown"),
    (lambda r: r["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=4), "evenly"),
    (lambda r: r["layers"][0]["mixer"].update(softcap=0.0), "softcap"),
    (lambda r: r["layers"][0]["mixer"]["mask"].pop("size"), "size"),
    (lambda r: r["layers"][0]["mixer"]["mask"].update(keep_first=-1), "keep_first"),
    (lambda r: r["layers"][0]["mlp"].update(kind="gated"), "not built"),
    (lambda r: r["layers"][0]["mlp"]["router"].update(top=9), "chooses"),
    (lambda r: r["layers"][1]["mlp"].pop("ff"), "ff"),
    (lambda r: r["canon"].update(taps=0), "taps"),
    (lambda r: r.pop("norm"), "norm"),
])
def test_bad_configurations_are_refused(change, what):
    raw = copy.deepcopy(cases.CASES["A"])
    change(raw)
    with pytest.raises(ConfigError, match=what):
        config_from_dict(raw)


def test_cache_entries_pinned_pages_and_state_records(folders):
    sess = session(folders["A"], max_tokens=64 * 40, max_seq_tokens=64 * 20, max_step_tokens=24)
    layers = sess.cache.layers
    assert len(layers) == 4 and all(isinstance(l.group, KVGroup) for l in layers)
    assert all(isinstance(l.aux.group, StateGroup) for l in layers)                 # every layer: the convolution's last inputs
    assert layers[0].aux.group is layers[3].aux.group and layers[0].aux.index != layers[3].aux.index
    assert layers[0].aux.state.shape[1:] == (3, 96) and layers[0].aux.state.dtype == torch.float32
    g = layers[0].group
    assert g.request.keep_first == 3 and g.pinned_pages == 1 and g.ring_pages > 0 and g.table_width == 1 + g.ring_pages
    assert g.k.shape[-1] == 16 and g.v.shape[-1] == 24
    assert layers[2].group.ring_pages == 0                                          # no window: every key stays
    assert layers[3].group.pinned_pages == 0 and layers[3].group.ring_pages > 0     # a window that keeps nothing
    bare = session(folders["C"]).cache.layers
    assert all(l.aux is None for l in bare)                                         # no convolution, no record
    wide = session(folders["B"], max_tokens=64 * 40, max_seq_tokens=64 * 20, max_step_tokens=16).cache.layers
    assert wide[1].group.pinned_pages == 2 and wide[3].group.pinned_pages == 1      # 70 and 64 kept tokens
    assert PAGE == 64


@pytest.mark.parametrize("name", list(cases.CASES))
def test_every_cutting_matches_plain(folders, name):
    folder = folders[name]
    seqs = random_tokens(cases.CASES[name]["vocab"], (5, 90, 41, 1, 64, 65, 2), seed=3)
    ref = cases.plain_logits(folder, seqs)
    sess = session(folder, max_step_tokens=24, max_rows=50)     # prompts go through in portions of 24 tokens at most
    assert_close(run_whole(sess, seqs), ref, "float32", "alone and whole")
    assert_close(run_whole(sess, seqs[:3], together=True), ref[:3], "float32", "one ragged step")
    assert_close(run_tail_by_one(sess, seqs, tail=30), ref, "float32", "tail one by one")
    assert_close(run_ragged_batches(sess, seqs, batch_size=3, poison=True), ref, "float32", "ragged batches, freed pages poisoned")
    assert sess.cache.slots.n_held == 0


def test_portions_down_to_two_tokens(folders):
    seqs = random_tokens(211, (37,), seed=4)
    ref = cases.plain_logits(folders["A"], seqs)
    for portion in (2, 3, 7, 20, 21):
        sess = session(folders["A"], max_step_tokens=portion)
        assert_close(run_whole(sess, seqs), ref, "float32", f"portions of {portion}")


def test_the_ring_turns_under_the_pinned_pages(folders):
    """A sequence far longer than the ring: the window's pages are used again and again, the kept tokens' pages stay, and
    every position still matches a run that holds all keys."""
    seqs = random_tokens(300, (700,), seed=12)
    ref = cases.plain_logits(folders["B"], seqs)
    sess = session(folders["B"], max_tokens=64 * 30, max_seq_tokens=64 * 16, max_step_tokens=16)
    g = sess.cache.layers[1].group
    assert g.pinned_pages == 2 and g.table_width < 700 // 64
    assert_close(run_tail_by_one(sess, seqs, tail=300), ref, "float32", "long decoding through a turning ring")
    assert_close(run_whole(sess, seqs), ref, "float32", "a long prompt in portions through a turning ring")


def test_state_of_a_freed_slot_does_not_leak(folders):
    """A slot that held a sequence is used again: the convolution starts from zeros, not from the last inputs left there."""
    sess = session(folders["D"], max_seqs=1)
    seqs = random_tokens(64, (70, 9, 3), seed=5)
    ref = cases.plain_logits(folders["D"], seqs)
    assert_close(run_whole(sess, seqs), ref, "float32", "later sequences in the first one's slot")
    assert_close(run_tail_by_one(sess, seqs, tail=8), ref, "float32", "and decoded")


def test_layers_match_plain(folders):
    """The residual after every layer, taken from the library's own stream, beside the plain model's."""
    cfg, tensors = plain.read_folder(folders["A"])
    tokens = random_tokens(211, (19,), seed=9)[0]
    want = []
    plain.forward(cfg, tensors, tokens, want)
    sess = session(folders["A"])
    seen = []
    for block in sess.model.blocks:
        inner = block.forward

        def spy(ctx, stream, layer_cache, inner=inner):
            inner(ctx, stream, layer_cache)
            seen.append(stream.x.clone())
        block.forward = spy
    run_whole(sess, [tokens])
    assert len(seen) == len(want) == 4
    for i, (got, ref) in enumerate(zip(seen, want)):
        assert got.dtype == torch.float32
        assert float((got - ref).abs().max()) <= 1e-4 * float(ref.abs().max()), f"layer {i}"


def test_greedy_generation_through_the_entry_point(folders):
    cfg, tensors = plain.read_folder(folders["C"])
    prompts = random_tokens(97, (3, 11, 1), seed=6)
    want = plain.generate(cfg, tensors, prompts, 10)
    engine = Engine.from_session(session(folders["C"]), use_graphs=False)
    assert engine.generate_all(prompts, 10) == want
    assert engine.session.cache.slots.n_held == 0


def test_random_weights_from_the_command_line(tmp_path):
    from starter_b200.cli import main
    (tmp_path / "config.json").write_text(json.dumps(cases.CASES["D"]))
    assert main(["random-weights", "--config", str(tmp_path / "config.json"), "--seed", "3", "--out", str(tmp_path / "model")]) == 0
    sess = session(tmp_path / "model")
    assert sess.model.spec.vocab_size == 64 and len(sess.model.blocks) == 2
    seqs = random_tokens(64, (12,), seed=8)
    assert_close(run_whole(sess, seqs), cases.plain_logits(tmp_path / "model", seqs), "float32", "folder from the command line")
