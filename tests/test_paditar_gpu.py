"""Paditar on the GPU against the plain implementation: every mechanism alone, then whole models in every way of
cutting the work; a key that stands out far back, at page borders and on both sides of the causal edge; the sink's
share; the temperature's steps; states of several sequences and of a slot that is used again; long decoding; and greedy
generation through the entry point."""

import math

import pytest
import torch

import paditar_cases as cases
from conftest import random_tokens
from helpers import assert_close, make_session, run_ragged_batches, run_tail_by_one, run_whole
from plain import paditar_plain as plain
from starter_b200.cache import Cache
from starter_b200.config import ActMLPSpec, DiffAttentionSpec, KeyValueAttentionSpec, MLSTMSpec, PairMixerSpec, ScaledHalfRopeSpec
from starter_b200.engine import Engine
from starter_b200.engine.context import Runtime, StepContext
from starter_b200.parts import build_part

pytestmark = pytest.mark.gpu
MODES = ["float32", "bfloat16"]
REL = {"float32": 3e-5, "bfloat16": 2.5e-2}
EPS = 1e-5


def runtime(mode):
    from starter_b200.csrc.ops import get_ops
    return Runtime(dtype=getattr(torch, mode), device=torch.device("cuda"), ops=get_ops(verbose=False))


def rand(shape, seed, scale=1.0, mean=0.0):
    g = torch.Generator().manual_seed(seed)
    return (mean + torch.randn(shape, generator=g) * scale).to(torch.bfloat16).float()   # bfloat16 numbers, so both modes read the same


def close(got, want, mode, what, rel=None):
    rel = rel or REL[mode]
    want = want.float()
    scale = float(want.abs().max())
    err = float((got.float().cpu() - want).abs().max())
    assert err <= rel * scale, f"{what}: {err:.3g} > {rel * scale:.3g}"


def mostly_close(got, want, mode, what, share=0.97, worst=0.15):
    """32-bit runs: every row within the tolerance.  bfloat16 runs of a mechanism that divides by what may nearly cancel
    (the memory's normaliser, a unit norm of a difference): the same roundings taken in torch leave a few rows in a
    hundred up to 0.08 of the scale away from the 64-bit result, so most rows stay within the tolerance and none strays
    far.  What a wrong key, state or page does shows in the 32-bit run of the same cutting."""
    if mode == "float32":
        return close(got, want, mode, what)
    want = want.float()
    errs = (got.float().cpu() - want).abs().max(dim=1).values / float(want.abs().max())
    within = float((errs <= REL[mode]).float().mean())
    assert within >= share and float(errs.max()) < worst, f"{what}: {within:.3f} of the rows within the tolerance, worst {float(errs.max()):.3g}"


def model_close(got, ref, mode, what):
    """The same for whole models: every branch is normed on its way back, so a rounded branch output enters the residual
    at full size, layer after layer."""
    if mode == "float32":
        return assert_close(got, ref, mode, what)
    for g, r in zip(got, ref):
        assert g.shape == r.shape
    mostly_close(torch.cat(list(got)), torch.cat(list(ref)), mode, what)


def context(rt, cache, slots, q_lens):
    for s, n in zip(slots, q_lens):
        cache.reserve(s, cache.lengths_host[s] + n)
    cache.flush()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    row_seq = [b for b, n in enumerate(q_lens) for _ in range(n)]
    return StepContext(runtime=rt, cache=cache, n_seqs=len(slots), n_rows=cu[-1], max_q_len=max(q_lens),
                       kv_bound=max(cache.lengths_host[s] + n for s, n in zip(slots, q_lens)), seq_slot=i32(slots), cu_q=i32(cu),
                       row_seq=i32(row_seq), lengths=cache.lengths, status=torch.zeros(1, dtype=torch.int32, device="cuda"))


def run_part(rt, part, h, cuts, pages=16):
    """A mixer with its cache entries over one sequence whose rows h come in pieces of the given sizes; the outputs of
    all pieces in order."""
    cache = Cache([part.cache_request()], n_slots=2, max_tokens=64 * pages, dtype=rt.dtype, device="cuda")
    cache.alloc()                      # the sequence under test sits in the second slot
    slot = cache.alloc()
    outs, at = [], 0
    for n in cuts:
        ctx = context(rt, cache, [slot], [n])
        outs.append(part.forward(ctx, h[at:at + n].to(rt.dtype).cuda().contiguous(), cache.layers[0]))
        rt.ops.advance_lengths(ctx)
        cache.advance_host(slot, n)
        assert int(ctx.status.item()) == 0
        at += n
    return torch.cat(outs)


def cuttings(n):
    """Whole; a tail token by token; portions of two; two unequal portions; every token alone."""
    return [[n], [n - 9] + [1] * 9, [2] * (n // 2) + [1] * (n % 2), [n // 3, n - n // 3], [1] * n]


ROLES = {"q.b": "q_bias", "k.b": "k_bias", "o.b": "o_bias", "q.conv": "q_conv", "k.conv": "k_conv", "q.norm": "q_norm", "k.norm": "k_norm",
         "i.b": "i_bias", "f.b": "f_bias"}


def role(name):
    """A tensor's last name in a checkpoint -> the role the part knows it by ("left.q.b" -> "left.q_bias")."""
    for side in ("left.", "right."):
        if name.startswith(side):
            return side + ROLES.get(name[len(side):], name[len(side):])
    return ROLES.get(name, name)


def part_of(rt, spec, w):
    return build_part("mixer", spec, {role(k): v.to(rt.dtype).cuda() for k, v in w.items()}, rt)


# ---- rows: the start of a pass, the squared relu ---------------------------------------------------------------

@pytest.mark.parametrize("width", [40, 96, 1030])
def test_a_pass_starts_from_residual_plus_embedding_plus_vector(width):
    ops = runtime("float32").ops
    x, e, s = rand((37, width), 1).cuda(), rand((37, width), 2).cuda(), rand((width,), 3).cuda()
    assert torch.equal(ops.add_rows(x, e, s), x + e + s) and torch.equal(ops.add_rows(x, None, s), x + s)
    copy = ops.add_rows(x)
    assert torch.equal(copy, x) and copy.data_ptr() != x.data_ptr()
    want = x + e + s
    assert ops.add_rows(x, e, s, out=x) is x and torch.equal(x, want)


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("width, ff, rows", [(96, 136, 5), (40, 52, 70), (1024, 2048, 16), (1024, 2048, 300)])
def test_squared_relu_feed_forward_alone(mode, width, ff, rows):
    rt = runtime(mode)
    up, down = rand((ff, width), 4, width ** -0.5), rand((width, ff), 5, ff ** -0.5)
    part = build_part("ff", ActMLPSpec(hidden_size=width, intermediate_size=ff, activation="relu2"),
                      {"up": up.to(rt.dtype).cuda(), "down": down.to(rt.dtype).cuda()}, rt)
    h = rand((rows, width), 6)
    close(part.forward(None, h.to(rt.dtype).cuda()), plain.feed_forward(h.double(), up.double(), down.double()), mode, "up, squared relu, down")


# ---- attention with two score maps and an output gate ----------------------------------------------------------

def diff_spec(H, G, D, V, diff, rot=None, scale=None, width=80):
    position = ScaledHalfRopeSpec(theta=rot[0], rotary_dim=rot[1]) if rot is not None else None
    return DiffAttentionSpec(hidden_size=width, num_heads=H, num_kv_heads=G, head_dim=D, v_dim=V, scale=D ** -0.5 if scale is None else scale,
                             diff=diff, norm_eps=EPS, position=position, gate=True)


def diff_weights(s, seed):
    H, G, D, V, h = s.num_heads, s.num_kv_heads, s.head_dim, s.v_dim, s.hidden_size
    w = {"q": rand((H * 2 * D, h), seed, h ** -0.5), "k": rand((G * 2 * D, h), seed + 1, h ** -0.5), "v": rand((G * V, h), seed + 2, h ** -0.5),
         "g": rand((H * V, h), seed + 3, h ** -0.5), "o": rand((h, H * V), seed + 4, (H * V) ** -0.5)}
    w.update({n: rand((D,), seed + 5 + i, 0.15) for i, n in enumerate(("lq1", "lk1", "lq2", "lk2"))})
    return w


def diff_entry(s):
    m = {"heads": s.num_heads, "kv_heads": s.num_kv_heads, "dim": s.head_dim, "vdim": s.v_dim, "scale": s.scale, "diff": s.diff}
    if s.position is not None:
        m["rot"] = {"base": s.position.theta, "dims": s.position.rotary_dim}
    return m


def plain_diff(h, w, s):
    return plain.diff_attention(h.double(), {k: v.double() for k, v in w.items()}, diff_entry(s), EPS)


DIFF_SIZES = [
    dict(H=6, G=2, D=16, V=24, diff=0.7, rot=(500.0, 8), scale=0.4),        # the general kernel; part of a head rotated
    dict(H=8, G=2, D=32, V=64, diff=0.5, rot=(1e6, 16)),                    # sizes the tensor-core kernels take
    dict(H=2, G=1, D=64, V=128, diff=0.8, rot=(1e4, 64), scale=0.2),        # the whole head rotated
    dict(H=1, G=1, D=20, V=12, diff=0.9),                                   # one head, no rotation
    dict(H=4, G=4, D=128, V=128, diff=0.3, rot=(1e4, 32)),                  # as many key/value heads as query heads
    dict(H=5, G=5, D=12, V=4, diff=0.4, rot=(100.0, 4)),
]


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("sizes", DIFF_SIZES)
def test_two_map_attention_with_its_gate_alone(mode, sizes):
    rt = runtime(mode)
    spec = diff_spec(**sizes)
    w = diff_weights(spec, 20)
    part = part_of(rt, spec, w)
    n = 150
    h = rand((n, spec.hidden_size), 3)
    want = plain_diff(h, w, spec)
    for cuts in cuttings(n):
        close(run_part(rt, part, h, cuts), want, mode, f"cut {cuts[:3]}..")


def test_the_gate_is_taken_element_by_element():
    """Gate weights that shut every column but a few: what passes is exactly those columns."""
    rt = runtime("float32")
    spec = diff_spec(H=2, G=1, D=16, V=8, diff=0.5, width=32)
    w = diff_weights(spec, 40)
    w["g"] = torch.zeros_like(w["g"])
    h = rand((20, 32), 7)
    h[:, 0] = 1.0
    open_columns = [1, 9, 15]
    w["g"][:, 0] = -60.0
    for c in open_columns:
        w["g"][c, 0] = 60.0
    w["o"] = torch.zeros(32, 16)
    w["o"][:16] = torch.eye(16)                               # the output shows the gated columns themselves
    got = run_part(rt, part_of(rt, spec, w), h, [20]).cpu()
    want = plain_diff(h, w, spec).float()
    close(got, want, "float32", "gated columns")
    shut = [c for c in range(16) if c not in open_columns]
    assert float(got[:, shut].abs().max()) < 1e-12 and float(got[:, open_columns].abs().min()) > 1e-3


# ---- attention whose values are its keys -----------------------------------------------------------------------

def kva_spec(H, G, D, taps=4, temp=(0.25, 64), scale=None, width=80):
    return KeyValueAttentionSpec(hidden_size=width, num_heads=H, num_kv_heads=G, head_dim=D, scale=D ** -0.5 if scale is None else scale,
                                 bias=True, taps=taps or 0, qk_norm_eps=EPS, temp_coef=temp[0] if temp else 0.0,
                                 temp_every=temp[1] if temp else 0, unit_sink=True, head_gate=True)


def kva_weights(s, seed):
    H, G, D, h = s.num_heads, s.num_kv_heads, s.head_dim, s.hidden_size
    w = {"q": rand((H * D, h), seed, h ** -0.5), "k": rand((G * D, h), seed + 1, h ** -0.5), "g": rand((H, h), seed + 2, h ** -0.5),
         "o": rand((h, H * D), seed + 3, (H * D) ** -0.5), "q.b": rand((H * D,), seed + 4, 0.3), "k.b": rand((G * D,), seed + 5, 0.3),
         "o.b": rand((h,), seed + 6, 0.3), "q.norm": rand((D,), seed + 7, 0.2, 1.5), "k.norm": rand((D,), seed + 8, 0.2, 1.5)}
    if s.taps:
        w.update({"q.conv": rand((H * D, s.taps), seed + 9, 0.5), "k.conv": rand((G * D, s.taps), seed + 10, 0.5)})
    return w


def kva_entry(s):
    m = {"heads": s.num_heads, "kv_heads": s.num_kv_heads, "dim": s.head_dim, "vdim": s.head_dim, "scale": s.scale}
    if s.taps:
        m["conv"] = s.taps
    if s.temp_every:
        m["q_temp"] = {"coef": s.temp_coef, "every": s.temp_every}
    return m


def plain_kva(h, w, s):
    return plain.key_value_attention(h.double(), {k: v.double() for k, v in w.items()}, kva_entry(s), EPS)


KVA_SIZES = [
    dict(H=4, G=2, D=24, taps=3, temp=(0.5, 5)),                 # the general kernel
    dict(H=4, G=1, D=64, taps=4, temp=(0.25, 64)),                # sizes the tensor-core kernels take; the temperature steps once a page
    dict(H=8, G=2, D=128, taps=2, temp=(1.0, 1), scale=0.05),    # a step at every position
    dict(H=1, G=1, D=20, taps=1, temp=None),                     # one tap keeps no record
    dict(H=3, G=3, D=6, taps=None, temp=(0.1, 7)),               # no convolution at all
    dict(H=2, G=2, D=8, taps=5, temp=(2.0, 3)),
    dict(H=16, G=4, D=64, taps=3, temp=(0.4, 32)),
]


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("sizes", KVA_SIZES)
def test_key_value_attention_alone(mode, sizes):
    rt = runtime(mode)
    spec = kva_spec(**sizes)
    w = kva_weights(spec, 30)
    part = part_of(rt, spec, w)
    n = 150
    h = rand((n, spec.hidden_size), 3)
    want = plain_kva(h, w, spec)
    for cuts in cuttings(n):
        close(run_part(rt, part, h, cuts), want, mode, f"cut {cuts[:3]}..")


@pytest.mark.parametrize("mode", MODES)
def test_key_value_attention_without_its_norm(mode):
    """The spec's norm is an option: without it queries and keys go on as they are.  The expected output is put together
    here from the plain helpers (temperature, softmax with a 1 in its denominator), since the plain mixer always norms."""
    import dataclasses
    rt = runtime(mode)
    spec = dataclasses.replace(kva_spec(H=2, G=1, D=16, taps=None, temp=(0.5, 4), scale=0.3, width=32), qk_norm_eps=None)
    w = kva_weights(dataclasses.replace(spec, qk_norm_eps=EPS), 33)
    w.pop("q.norm"), w.pop("k.norm")
    n = 40
    h = rand((n, 32), 11)
    # the plain attention by hand, from the plain helpers, without the unit norms
    q = (h.double() @ w["q"].double().T + w["q.b"].double()).reshape(n, 2, 16) * plain.query_temperature(n, 0.5, 4)[:, None, None]
    k = (h.double() @ w["k"].double().T + w["k.b"].double()).reshape(n, 1, 16)
    gate = torch.sigmoid(h.double() @ w["g"].double().T)
    heads = [plain.softmax_attention(q[:, i], k[:, 0], k[:, 0], 0.3, extra_one=True) * gate[:, i:i + 1] for i in range(2)]
    want = torch.cat(heads, dim=-1) @ w["o"].double().T + w["o.b"].double()
    for cuts in ([n], [n - 9] + [1] * 9):
        close(run_part(rt, part_of(rt, spec, w), h, cuts), want, mode, f"cut {cuts[:3]}..")


def standout(spec, n, at, seed, strength=5.0):
    """Rows and weights in which the key at position ``at`` stands out for every later query of head 0: ordinary rows
    share a direction u and have nothing along a second direction z; the row at ``at`` is a multiple of z; the first key
    head's matrix maps z onto what the first query head makes of u, and the convolution's last tap passes it on.  The
    value at ``at`` is large with the row, so seeing or not seeing that key moves the output."""
    h = spec.hidden_size
    w = kva_weights(spec, seed)
    D = spec.head_dim
    u, z = torch.zeros(h), torch.zeros(h)
    u[0], z[1] = 1.0, 1.0
    rows = rand((n, h), seed + 20, 0.05)
    rows[:, 1] = 0.0
    rows = rows + 2.0 * u
    rows[at] = strength * z
    for name in ("q.b", "k.b"):
        w[name] = w[name] * 0.05
    if spec.taps:
        for name in ("q.conv", "k.conv"):
            w[name] = w[name] * 0.05
            w[name][:, -1] = 1.0
    w["k"][:, 1] = 0.0
    w["k"][:D, 1] = w["q"][:D, 0]
    return rows.to(torch.bfloat16).float(), {k: v.to(torch.bfloat16).float() for k, v in w.items()}


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("n, at", [(330, 0), (330, 1), (200, 63), (200, 64), (200, 65), (330, 127), (330, 128), (700, 5), (150, 149)])
def test_a_key_that_stands_out_far_back_and_at_page_borders(mode, n, at):
    rt = runtime(mode)
    spec = kva_spec(H=4, G=2, D=64, taps=2, temp=(0.25, 64), scale=0.6)
    h, w = standout(spec, n, at, 50)
    want = plain_kva(h, w, spec)
    if 0 < at < n - 1:    # the test can tell: with an ordinary row in the key's place the later outputs move by a good part of their size
        plainer = h.clone()
        plainer[at] = h[at - 1]
        moved = (plain_kva(plainer, w, spec)[at + 1:] - want[at + 1:]).abs().mean()
        assert float(moved) > 0.2 * float(want[at + 1:].abs().mean())
    part = part_of(rt, spec, w)
    tail = n - max(at - 1, 1)          # decoding starts one position before the key
    for cuts in ([n], [n - tail] + [1] * tail if tail <= 140 else [n - 40] + [1] * 40, [max(at, 1), n - max(at, 1)]):
        cuts = [c for c in cuts if c > 0]
        close(run_part(rt, part, h, cuts, pages=24), want, mode, f"key at {at}, cut {cuts[:3]}..")


@pytest.mark.parametrize("mode", MODES)
def test_the_sink_takes_its_share(mode):
    """With a scale so small that every score is 0, position p spreads its weight evenly over p + 1 keys and the sink:
    the output is the sum of the values so far divided by p + 2."""
    rt = runtime(mode)
    spec = kva_spec(H=2, G=1, D=16, taps=None, temp=None, scale=1e-9, width=32)
    w = kva_weights(spec, 60)
    w["g"] = torch.zeros_like(w["g"])                      # every gate is one half
    w["o"] = torch.zeros(32, 32)                           # the output shows the first head's columns themselves
    w["o"][:16, :16] = torch.eye(16)
    w["o.b"] = torch.zeros(32)
    h = rand((40, 32), 8)
    got = run_part(rt, part_of(rt, spec, w), h, [30] + [1] * 10).float().cpu()
    values = h.double() @ w["k"].double().T + w["k.b"].double()
    want = 0.5 * torch.cumsum(values, dim=0) / (torch.arange(40, dtype=torch.float64)[:, None] + 2.0)
    close(got[:, :16], want, mode, "even weights with one share for the sink")
    close(got, plain_kva(h, w, spec), mode, "and the plain attention agrees")


@pytest.mark.parametrize("mode", MODES)
def test_the_temperature_steps_where_it_should(mode):
    """A large coefficient: a query one position early or late with its step would show."""
    rt = runtime(mode)
    spec = kva_spec(H=2, G=2, D=32, taps=3, temp=(4.0, 16), scale=0.3)
    w = kva_weights(spec, 70)
    n = 70
    h = rand((n, spec.hidden_size), 9)
    want = plain_kva(h, w, spec)
    for cuts in ([n], [14] + [1] * (n - 14), [15, 1, 16, 15, 17, 6]):
        close(run_part(rt, part_of(rt, spec, w), h, cuts), want, mode, f"cut {cuts[:3]}..")


def test_records_of_two_sequences_and_a_slot_used_again():
    """Two sequences side by side in one step, each with its own convolution record and keys; then the first slot is
    freed and taken by a new sequence, which must start from zeros."""
    rt = runtime("float32")
    spec = kva_spec(H=2, G=1, D=16, taps=4, temp=(0.5, 3), width=32)
    w = kva_weights(spec, 80)
    part = part_of(rt, spec, w)
    cache = Cache([part.cache_request()], n_slots=2, max_tokens=64 * 8, dtype=rt.dtype, device="cuda")
    a, b, c = rand((21, 32), 1), rand((9, 32), 2), rand((12, 32), 3)
    sa, sb = cache.alloc(), cache.alloc()

    def step(slots, pieces):
        ctx = context(rt, cache, slots, [len(p) for p in pieces])
        out = part.forward(ctx, torch.cat(pieces).cuda(), cache.layers[0])
        rt.ops.advance_lengths(ctx)
        for s, p in zip(slots, pieces):
            cache.advance_host(s, len(p))
        assert int(ctx.status.item()) == 0
        return out.cpu()

    first = step([sa, sb], [a[:10], b[:2]])
    second = step([sb, sa], [b[2:], a[10:]])
    got_a, got_b = torch.cat([first[:10], second[7:]]), torch.cat([first[10:], second[:7]])
    close(got_a, plain_kva(a, w, spec), "float32", "first sequence")
    close(got_b, plain_kva(b, w, spec), "float32", "second sequence")
    cache.free(sa)
    sc = cache.alloc()
    assert sc == sa
    close(step([sc], [c]), plain_kva(c, w, spec), "float32", "a new sequence in the freed slot")


# ---- the matrix memory -----------------------------------------------------------------------------------------

def mem_spec(H, D, V, cap, width=80):
    return MLSTMSpec(hidden_size=width, num_heads=H, head_dim=D, v_dim=V, gate_cap=cap, norm_eps=EPS)


def mem_weights(s, seed, gate_scale=1.0):
    H, D, V, h = s.num_heads, s.head_dim, s.v_dim, s.hidden_size
    return {"q": rand((H * D, h), seed, h ** -0.5), "k": rand((H * D, h), seed + 1, h ** -0.5), "v": rand((H * V, h), seed + 2, h ** -0.5),
            "g": rand((H * V, h), seed + 3, h ** -0.5), "o": rand((h, H * V), seed + 4, (H * V) ** -0.5),
            "norm": rand((H * V,), seed + 5, 0.2, 1.0), "i": rand((H, h), seed + 6, gate_scale * h ** -0.5), "i.b": rand((H,), seed + 7, 0.5),
            "f": rand((H, h), seed + 8, gate_scale * h ** -0.5), "f.b": rand((H,), seed + 9, 0.5, 2.0)}


def mem_entry(s):
    return {"heads": s.num_heads, "dim": s.head_dim, "vdim": s.v_dim, "gate_cap": s.gate_cap}


def plain_mem(h, w, s):
    return plain.matrix_memory(h.double(), {k: v.double() for k, v in w.items()}, mem_entry(s), EPS)


MEM_SIZES = [
    dict(H=3, D=16, V=24, cap=8.0),
    dict(H=2, D=64, V=64, cap=11.0),
    dict(H=4, D=128, V=128, cap=15.0),      # a head's columns shared out over two blocks
    dict(H=1, D=136, V=12, cap=1.5),        # keys wider than the registers hold: the state stays in memory
    dict(H=2, D=10, V=130, cap=30.0),       # three blocks of columns, the last one nearly empty
    dict(H=4, D=48, V=64, cap=5.0),
    dict(H=5, D=1, V=1, cap=3.0),           # a scalar memory
]


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("sizes", MEM_SIZES)
def test_matrix_memory_alone(mode, sizes):
    rt = runtime(mode)
    spec = mem_spec(**sizes)
    w = mem_weights(spec, 90)
    part = part_of(rt, spec, w)
    n = 100
    h = rand((n, spec.hidden_size), 3)
    want = plain_mem(h, w, spec)
    # the unit norm of a single value is its sign unless the value is tiny: there a rounded input shows in full
    rel = 8e-2 if mode == "bfloat16" and spec.v_dim == 1 else None
    for cuts in cuttings(n):
        close(run_part(rt, part, h, cuts), want, mode, f"cut {cuts[:3]}..", rel=rel)


@pytest.mark.parametrize("mode", MODES)
def test_gates_that_swing_move_the_running_maximum(mode):
    """Gate matrices ten times larger: the input gate reaches its cap, the forget gate closes and opens, and the running
    maximum climbs and falls over a long sequence; the record carries S, n and m from step to step."""
    rt = runtime(mode)
    spec = mem_spec(H=2, D=32, V=32, cap=10.0)
    w = mem_weights(spec, 100, gate_scale=10.0)
    part = part_of(rt, spec, w)
    n = 600
    h = rand((n, spec.hidden_size), 4)
    want = plain_mem(h, w, spec)
    for cuts in ([n], [n - 200] + [1] * 200, [33] * 18 + [6]):
        mostly_close(run_part(rt, part, h, cuts), want, mode, f"cut {cuts[:3]}..")


def test_the_first_token_divides_by_one():
    """At a sequence's first token with a closed input gate m stays 0 and |n . q| is tiny: the divisor is exp(-0) = 1."""
    rt = runtime("float32")
    spec = mem_spec(H=1, D=8, V=8, cap=20.0, width=16)
    w = mem_weights(spec, 110)
    w["i"], w["i.b"] = torch.zeros_like(w["i"]), torch.full((1,), -15.0)
    h = rand((3, 16), 5)
    close(run_part(rt, part_of(rt, spec, w), h, [1, 2]), plain_mem(h, w, spec), "float32", "closed input gate")


def test_memory_records_of_two_sequences_and_a_slot_used_again():
    rt = runtime("float32")
    spec = mem_spec(H=2, D=16, V=24, cap=6.0, width=32)
    w = mem_weights(spec, 120)
    part = part_of(rt, spec, w)
    cache = Cache([part.cache_request()], n_slots=2, max_tokens=64 * 8, dtype=rt.dtype, device="cuda")
    a, b, c = rand((21, 32), 1), rand((9, 32), 2), rand((12, 32), 3)
    sa, sb = cache.alloc(), cache.alloc()

    def step(slots, pieces):
        ctx = context(rt, cache, slots, [len(p) for p in pieces])
        out = part.forward(ctx, torch.cat(pieces).cuda(), cache.layers[0])
        rt.ops.advance_lengths(ctx)
        for s, p in zip(slots, pieces):
            cache.advance_host(s, len(p))
        return out.cpu()

    first = step([sa, sb], [a[:10], b[:2]])
    second = step([sb, sa], [b[2:], a[10:]])
    close(torch.cat([first[:10], second[7:]]), plain_mem(a, w, spec), "float32", "first sequence")
    close(torch.cat([first[10:], second[:7]]), plain_mem(b, w, spec), "float32", "second sequence")
    cache.free(sa)
    assert cache.alloc() == sa
    close(step([sa], [c]), plain_mem(c, w, spec), "float32", "a new sequence in the freed slot")


# ---- two mixers side by side -----------------------------------------------------------------------------------

@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("scales", [(1.5, 0.25), (1.0, 1.0), (0.0, 2.0)])
def test_two_mixers_side_by_side(mode, scales):
    rt = runtime(mode)
    left, right = kva_spec(H=4, G=2, D=24, taps=3, temp=(0.5, 5)), mem_spec(H=3, D=16, V=24, cap=8.0)
    spec = PairMixerSpec(left=left, right=right, left_scale=scales[0], right_scale=scales[1])
    wl, wr = kva_weights(left, 130), mem_weights(right, 140)
    w = {"left." + k: v for k, v in wl.items()}
    w.update({"right." + k: v for k, v in wr.items()})
    part = part_of(rt, spec, w)
    n = 90
    h = rand((n, 80), 6)
    entry = {"left": kva_entry(left), "right": mem_entry(right), "left_scale": scales[0], "right_scale": scales[1]}
    want = plain.side_by_side(h.double(), {k: v.double() for k, v in wl.items()}, {k: v.double() for k, v in wr.items()}, entry, EPS)
    for cuts in cuttings(n):
        close(run_part(rt, part, h, cuts), want, mode, f"cut {cuts[:3]}..")


# ---- whole models ------------------------------------------------------------------------------------------------

@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name in cases.CASES:
        out[name, "bfloat16"] = cases.write_folder(name, tmp_path_factory.mktemp(f"paditar_{name}_bf16"))
        out[name, "float32"] = cases.write_folder(name, tmp_path_factory.mktemp(f"paditar_{name}_f32"), dtype=torch.float32, shards=2)
    return out


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("name", list(cases.CASES))
def test_every_cutting_matches_plain(folders, name, mode):
    folder = folders[name, mode]
    seqs = random_tokens(cases.CASES[name]["vocab"], (5, 90, 41, 1, 64, 65, 2, 130), seed=3)
    ref = cases.plain_logits(folder, seqs)
    sess = make_session(folder, mode, max_tokens=64 * 16, max_seqs=4, max_rows=100)
    model_close(run_whole(sess, seqs), ref, mode, "alone and whole")
    model_close(run_whole(sess, seqs[:4], together=True), ref[:4], mode, "one ragged step")
    model_close(run_tail_by_one(sess, seqs, tail=40), ref, mode, "tail one by one")
    model_close(run_ragged_batches(sess, seqs, batch_size=3, poison=True), ref, mode, "ragged batches, freed pages poisoned")
    assert sess.cache.slots.n_held == 0


@pytest.mark.parametrize("mode", MODES)
def test_portions_down_to_two_tokens(folders, mode):
    seqs = random_tokens(211, (37,), seed=4)
    ref = cases.plain_logits(folders["A", mode], seqs)
    for portion in (2, 3, 7, 21):
        sess = make_session(folders["A", mode], mode, max_tokens=64 * 4, max_seqs=2, max_rows=portion)
        model_close(run_whole(sess, seqs), ref, mode, f"portions of {portion}")


@pytest.mark.parametrize("mode", MODES)
def test_long_decoding_in_a_batch(folders, mode):
    seqs = random_tokens(300, (420, 333), seed=12)
    ref = cases.plain_logits(folders["B", mode], seqs)
    sess = make_session(folders["B", mode], mode, max_tokens=64 * 16, max_seqs=2)
    model_close(run_ragged_batches(sess, seqs, batch_size=2, prefix_fraction=0.2), ref, mode, "hundreds of tokens decoded side by side")


def test_layer_runs_match_plain(folders):
    cfg, tensors = plain.read_folder(folders["A", "float32"])
    tokens = random_tokens(211, (19,), seed=9)[0]
    want = []
    plain.forward(cfg, tensors, tokens, want)
    sess = make_session(folders["A", "float32"], "float32", max_tokens=64 * 4, max_seqs=2)
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
        assert float((got.cpu() - ref).abs().max()) <= 2e-5 * float(ref.abs().max()), f"layer run {i}"


def test_the_residual_is_32_bit_in_a_bfloat16_run(folders):
    sess = make_session(folders["D", "bfloat16"], "bfloat16", max_tokens=64 * 4, max_seqs=2)
    kinds = []
    for block in sess.model.blocks:
        inner = block.forward

        def spy(ctx, stream, layer_cache, inner=inner):
            inner(ctx, stream, layer_cache)
            kinds.append(stream.x.dtype)
        block.forward = spy
    run_whole(sess, random_tokens(64, (9,), seed=1))
    assert kinds == [torch.float32] * 2


@pytest.mark.parametrize("mode", MODES)
def test_greedy_generation_through_the_entry_point(folders, mode):
    cfg, tensors = plain.read_folder(folders["C", "float32"])
    prompts = random_tokens(97, (3, 11, 1, 30), seed=6)
    want = plain.generate(cfg, tensors, prompts, 12)
    engine = Engine.from_session(make_session(folders["C", "float32"], "float32", max_tokens=64 * 8, max_seqs=4))   # graphs on
    assert engine.generate_all(prompts, 12) == want
    assert engine.session.cache.slots.n_held == 0
    engine = Engine.from_session(make_session(folders["C", "float32"], "float32", max_tokens=64 * 8, max_seqs=4), use_graphs=False)
    assert engine.generate_all(prompts, 12) == want
    if mode == "bfloat16":      # rounding may turn a close call: every request still ends with its tokens
        engine = Engine.from_session(make_session(folders["C", "bfloat16"], "bfloat16", max_tokens=64 * 8, max_seqs=4))
        got = engine.generate_all(prompts, 12)
        assert [len(g) for g in got] == [12] * 4 and engine.session.cache.slots.n_held == 0


def test_the_trace_runner_replays_this_design(folders, tmp_path):
    import json
    import subprocess
    import sys
    from pathlib import Path
    import numpy as np
    root = Path(__file__).resolve().parent.parent
    folder = folders["D", "float32"]
    seqs = random_tokens(64, (20, 9), seed=2)
    ref = cases.plain_logits(folder, seqs)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": seqs[0][:15], "want": [14]}, {"id": "b", "tokens": seqs[1][:8], "want": [0, 7]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": seqs[0][15:16], "want": [0]}, {"id": "b", "tokens": seqs[1][8:9], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": seqs[0][16:17], "want": []}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": seqs[0][17:20], "want": [2]}], "end": ["a"]}]
    proc = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(tmp_path),
                           "--max-tokens", "64"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == ["done", "0", "done", "1", "done", "2", "done", "3"] and not (tmp_path / "2.f32").exists()
    read = lambda i: torch.from_numpy(np.fromfile(tmp_path / f"{i}.f32", dtype="<f4").reshape(-1, 64).copy())
    want = {0: torch.stack([ref[0][14], ref[1][0], ref[1][7]]), 1: torch.stack([ref[0][15], ref[1][8]]), 3: ref[0][19:20]}
    for i, r in want.items():
        assert float((read(i) - r).abs().max()) <= 1e-4 * float(r.abs().max()), f"step {i}"
