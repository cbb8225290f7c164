"""Paditar through the library's own cache, step function and generation loop on a CPU (the kernels' meaning restated
in torch, tests/emulated_ops.py), against the plain implementation: what is tested here is the host side, i.e. the
configuration, the order of the passes with a cache entry per layer run, a layer's chain of cache entries (keys, the
convolution's record, the memory's record), and the cutting of work into steps."""

import copy
import json

import pytest
import torch

import paditar_cases as cases
from conftest import random_tokens
from emulated_ops import EmulatedOps
from helpers import assert_close, run_ragged_batches, run_tail_by_one, run_whole
from plain import paditar_plain as plain
from starter_b200.cache import KVGroup, StateGroup
from starter_b200.config import ConfigError, config_from_dict, load_config
from starter_b200.engine import Engine
from starter_b200.engine.session import Session


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: cases.write_folder(name, tmp_path_factory.mktemp(f"paditar_{name}"), dtype=torch.float32) for name in cases.CASES}


def session(folder, **kw):
    args = dict(dtype="float32", device="cpu", ops=EmulatedOps(), max_tokens=64 * 12, max_seqs=4)
    args.update(kw)
    return Session(folder, **args)


def test_configuration_round_trip_and_parts(folders):
    cfg = load_config(folders["A"])
    assert cfg.architecture == "Paditar" and config_from_dict(cfg.to_dict()) == cfg
    spec = cfg.model_spec()
    assert spec.residual_float32 and spec.tie_embeddings and (spec.loop.start, spec.loop.stop, spec.loop.times) == (1, 3, 3)
    assert spec.execution_order() == (0, 1, 2, 1, 2, 1, 2, 3) and spec.pass_starts() == {1: 0, 3: 1, 5: 2}
    assert [b.kind for b in spec.layers] == ["sandwich"] * 4
    assert [b.mixer.kind for b in spec.layers] == ["diff_attention", "pair", "diff_attention", "pair"]
    assert [b.ff.activation if b.ff is not None else None for b in spec.layers] == ["relu2", "relu2", None, "relu2"]
    m = spec.layers[0].mixer
    assert (m.gate, m.diff, m.scale, m.v_dim, m.position.rotary_dim, m.position.theta) == (True, 0.7, 0.4, 24, 8, 500.0)
    pair = spec.layers[1].mixer
    assert (pair.left_scale, pair.right_scale) == (1.5, 0.25)
    assert (pair.left.kind, pair.left.taps, pair.left.temp_coef, pair.left.temp_every) == ("key_value_attention", 3, 0.5, 5)
    assert pair.left.bias and pair.left.unit_sink and pair.left.head_gate and pair.left.qk_norm_eps == 1e-5
    assert (pair.right.kind, pair.right.num_heads, pair.right.head_dim, pair.right.v_dim, pair.right.gate_cap) == ("mlstm", 3, 16, 24, 8.0)
    assert spec.layers[0].mixer_norm.offset == 1.0 and spec.layers[0].mixer_out_norm.kind == "branch_rmsnorm"
    names = cfg.tensor_names()
    assert names.loop_step == "loop.step" and names.layers[0]["mixer"]["lq2"] == "l0.mix.lq2"
    assert names.layers[1]["mixer"]["left.q_bias"] == "l1.mix.left.q.b" and names.layers[1]["mixer"]["left.k_conv"] == "l1.mix.left.k.conv"
    assert names.layers[1]["mixer"]["right.f_bias"] == "l1.mix.right.f.b" and names.layers[1]["mixer_out_norm"]["weight"] == "l1.norm1b"
    assert "ff" not in names.layers[2] and names.layers[3]["ff_out_norm"]["weight"] == "l3.norm2b"
    bare = cases.config("C")
    assert bare.model_spec().loop is None and bare.model_spec().layers[1].mixer.position is None
    assert bare.model_spec().layers[2].mixer.left.taps == 0 and "left.q_conv" not in bare.tensor_names().layers[2]["mixer"]
    assert bare.model_spec().layers[0].mixer.left.temp_every == 0


@pytest.mark.parametrize("change, what", [
    (lambda r: r["layers"][0].update(type="conv"), "unknown"),
    (lambda r: r["layers"][0]["mixer"].pop("diff"), "diff"),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=4), "evenly"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=18), "at most dim"),
    (lambda r: r["layers"][1]["mixer"]["left"].update(vdim=8), "values are the keys"),
    (lambda r: r["layers"][1]["mixer"]["left"]["q_temp"].update(every=0), "every"),
    (lambda r: r["layers"][1]["mixer"]["right"].update(gate_cap=0.0), "gate_cap"),
    (lambda r: r["layers"][1]["mixer"].pop("right_scale"), "right_scale"),
    (lambda r: r["layers"][0]["mlp"].update(kind="moe"), "not built"),
    (lambda r: r["loop"].update(stop=5), "loop runs"),
    (lambda r: r["loop"].update(times=0), "times"),
    (lambda r: r.pop("norm"), "norm"),
])
def test_bad_configurations_are_refused(change, what):
    raw = copy.deepcopy(cases.CASES["A"])
    change(raw)
    with pytest.raises(ConfigError, match=what):
        config_from_dict(raw)


def test_a_cache_entry_per_layer_run_and_a_chain_per_layer(folders):
    sess = session(folders["A"])
    layers = sess.cache.layers
    assert len(layers) == 8                                                   # layers 1 and 2 run three times each
    assert all(isinstance(l.group, KVGroup) for l in layers)
    runs_of_1 = [layers[i] for i in (1, 3, 5)]
    assert len({(id(l.group), l.index) for l in runs_of_1}) == 3              # every pass keeps keys of its own
    for l in runs_of_1:
        assert isinstance(l.aux.group, StateGroup) and l.aux.state.shape[1:] == (2, (4 + 2) * 24)          # the convolution's record
        assert isinstance(l.aux.aux.group, StateGroup) and l.aux.aux.state.shape[1:] == (3 * 16 * 24 + 3 * 16 + 3,)   # S, n, m
        assert l.group.v.shape[-1] == l.group.k.shape[-1] == 24 and l.aux.aux.aux is None
    assert len({(id(l.aux.aux.group), l.aux.aux.index) for l in runs_of_1}) == 3
    assert layers[0].aux is None and layers[0].group.k.shape[2] == 2 * 2 and layers[0].group.v.shape[2] == 2   # two key maps, one value
    bare = session(folders["C"]).cache.layers
    assert isinstance(bare[0].aux.group, StateGroup) and bare[0].aux.aux is None      # one tap keeps no record: the memory's comes next
    assert bare[0].aux.state.shape[1:] == (136 * 12 + 136 + 1,) and bare[2].aux.state.shape[1:] == (2 * 10 * 130 + 2 * 10 + 2,)


@pytest.mark.parametrize("name", list(cases.CASES))
def test_every_cutting_matches_plain(folders, name):
    folder = folders[name]
    seqs = random_tokens(cases.CASES[name]["vocab"], (5, 90, 41, 1, 64, 65, 2), seed=3)
    ref = cases.plain_logits(folder, seqs)
    sess = session(folder, max_rows=50)     # a step of more than 50 rows goes through in several forward passes
    assert_close(run_whole(sess, seqs), ref, "float32", "alone and whole")
    assert_close(run_whole(sess, seqs[:3], together=True), ref[:3], "float32", "one ragged step")
    assert_close(run_tail_by_one(sess, seqs, tail=30), ref, "float32", "tail one by one")
    assert_close(run_ragged_batches(sess, seqs, batch_size=3, poison=True), ref, "float32", "ragged batches, freed pages poisoned")
    assert sess.cache.slots.n_held == 0


def test_portions_down_to_two_tokens(folders):
    seqs = random_tokens(211, (37,), seed=4)
    ref = cases.plain_logits(folders["A"], seqs)
    for portion in (2, 3, 7, 20, 21):
        sess = session(folders["A"], max_rows=portion)
        assert_close(run_whole(sess, seqs), ref, "float32", f"portions of {portion}")


def test_state_of_a_freed_slot_does_not_leak(folders):
    """A slot that held a sequence is used again: the convolution starts from zeros and the memory from S = n = m = 0, not
    from what the last sequence left there."""
    sess = session(folders["D"], max_seqs=1)
    seqs = random_tokens(64, (70, 9, 3), seed=5)
    ref = cases.plain_logits(folders["D"], seqs)
    assert_close(run_whole(sess, seqs), ref, "float32", "later sequences in the first one's slot")
    assert_close(run_tail_by_one(sess, seqs, tail=8), ref, "float32", "and decoded")


def test_layer_runs_match_plain(folders):
    """The residual after every layer run (a looped layer counts each time), taken from the library's own stream."""
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
    assert len(seen) == len(want) == 8
    for i, (got, ref) in enumerate(zip(seen, want)):
        assert got.dtype == torch.float32
        assert float((got - ref).abs().max()) <= 1e-4 * float(ref.abs().max()), f"layer run {i}"


def test_the_embedding_output_survives_the_layers_before_the_loop(folders):
    """Layers change the residual in place; the rows that later passes add again must be the embedding's, untouched."""
    sess = session(folders["A"])
    kept = []
    inner = sess.runtime.ops.add_rows

    def spy(x, rows_too=None, vector=None, out=None):
        if rows_too is not None:
            kept.append(rows_too.clone())
        return inner(x, rows_too, vector, out)
    sess.runtime.ops.add_rows = spy
    tokens = random_tokens(211, (7,), seed=2)[0]
    run_whole(sess, [tokens])
    table = sess.model.embedding.float()
    assert len(kept) == 2 and all(torch.equal(k, table[torch.tensor(tokens)]) for k in kept)


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
