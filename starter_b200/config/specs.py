"""Typed descriptions of the parts a model is put together from.

A spec is plain data: every size and constant a part needs, and nothing about
the model the part sits in.  An architecture turns its ``config.json`` into a
``ModelSpec``; the builder turns each spec into a part by looking its ``kind``
up in the part registry.  A new kind of part is a new spec class with a
``kind`` of its own plus one registered part class; nothing here has to change.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """Root-mean-square norm over the last axis: y = w * x * rsqrt(mean(x^2) + eps)."""

    size: int
    eps: float
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class RopeSpec:
    """Rotary position encoding, rotate-half pairing (d, d + rotary_dim/2),
    angle(p, j) = p / theta**(2j / rotary_dim)."""

    theta: float
    rotary_dim: int
    kind: str = "rope"


@dataclass(frozen=True)
class GroupedNormSpec:
    """Root-mean-square norm in groups: the last axis is cut into ``groups`` equal consecutive parts, each divided by
    its own sqrt(mean(part^2) + eps); then the whole is multiplied by w (by ``offset`` + w when the checkpoint keeps
    its weights around zero).  One group is the plain norm."""

    size: int
    eps: float
    groups: int = 1
    offset: float = 0.0     # the stored weight stands for offset + w (1.0: a weight stored around zero)
    kind: str = "grouped_rmsnorm"


@dataclass(frozen=True)
class PairRopeSpec:
    """Rotary position encoding over neighbouring columns: (2j, 2j + 1) of the first ``rotary_dim`` columns turn
    by angle(p, j) = p * theta**(-2j / rotary_dim); angles, sines and the rotation itself are 32-bit."""

    theta: float
    rotary_dim: int
    kind: str = "rope_pairs"


@dataclass(frozen=True)
class ScaledHalfRopeSpec:
    """Rotary position encoding over the first ``rotary_dim`` columns of a head, column i paired with column
    i + rotary_dim/2, with 32-bit angles taken in the kernels (no table) and, when ``factor`` is given, frequencies
    stretched by wavelength: with d(t) = rotary_dim ln(original / (2 pi t)) / (2 ln theta), pairs below d(fast) keep
    f_i = theta**(-2i / rotary_dim), pairs above d(slow) turn ``factor`` times slower, a linear ramp in between, and
    cosines and sines grow by 0.1 ln(factor) + 1."""

    theta: float
    rotary_dim: int
    factor: Optional[float] = None
    original: Optional[float] = None
    fast: Optional[float] = None
    slow: Optional[float] = None
    kind: str = "rope_half_scaled"


@dataclass(frozen=True)
class SinusoidSpec:
    """A position vector added to the embedded rows (kind "sinusoid"): column 2i of position p holds
    sin(p * base**(-2i / size)), column 2i + 1 the cosine of the same angle; angles, sines and the sum are 32-bit."""

    size: int
    base: float = 10000.0
    kind: str = "sinusoid"


@dataclass(frozen=True)
class CausalConvSpec:
    """A short causal convolution over time on every channel, added to its input (kind "causal_conv"):
    out_t = h_t + sum_j w[:, j] * h_(t - taps + 1 + j), zeros before a sequence's start.  The last ``taps`` - 1
    inputs of a sequence are its state."""

    size: int
    taps: int
    kind: str = "causal_conv"


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention over a key/value cache.

    ``window``: a query at position p sees the keys n with p - window < n <= p;
    None means every earlier key.  ``kv_from``: index of another layer whose
    cache this layer reads instead of projecting and storing keys and values.
    """

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    qk_norm: Optional[NormSpec] = None
    position: Optional[Any] = None
    window: Optional[int] = None
    kv_from: Optional[int] = None
    kind: str = "attention"


@dataclass(frozen=True)
class BiasedAttentionSpec:
    """Causal grouped-query attention whose scores carry more than a scale, over keys of ``head_dim`` and values of
    ``v_dim`` columns (kind "biased_attention").  Every option is off when None:

    * ``value_norm_eps``: each head's value is divided by its root mean square before it is cached;
    * ``head_temperature``: a learned number per query head multiplies the scaled score;
    * ``slope_log2``: c takes slope_h * (i - j) off the score of query i and key j, slope_h = 2**(-c (h + 1) / heads);
    * ``chunk``: key j is visible to query i only if i // chunk == j // chunk (counted from the sequence's start);
    * ``window``: only the last ``window`` keys are visible.
    """

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    v_dim: int
    scale: float
    value_norm_eps: Optional[float] = None
    head_temperature: bool = False
    slope_log2: Optional[float] = None
    chunk: Optional[int] = None
    window: Optional[int] = None
    kind: str = "biased_attention"


@dataclass(frozen=True)
class TalkingAttentionSpec:
    """Causal grouped-query attention whose scores meet across heads before the softmax (kind "talking_attention"),
    over keys of ``head_dim`` and values of ``v_dim`` columns, nothing rotated.  Every option is off when None / False / 0:

    * ``qk_norm_eps``: a token's whole query projection (all heads side by side) is divided by its root mean square and
      multiplied by a weight of that size before it is cut into heads; the same for the key projection;
    * ``softcap`` c: a scaled score s becomes c * tanh(s / c);
    * ``talk``: a learned [heads, heads] table T; head h's score against a key becomes sum_g T[h, g] * (head g's score);
    * ``window`` with ``keep_first``: key j is visible to query i if j <= i and (i - j < window or j < keep_first);
    * ``sink``: the softmax's denominator holds exp(s_h) once more, a learned number per head with no key or value.
    """

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    v_dim: int
    scale: float
    qk_norm_eps: Optional[float] = None
    softcap: Optional[float] = None
    talk: bool = False
    sink: bool = False
    window: Optional[int] = None
    keep_first: int = 0
    kind: str = "talking_attention"


@dataclass(frozen=True)
class DiffAttentionSpec:
    """Causal grouped-query attention with two score maps per head over the same values (kind "diff_attention"):
    queries and keys hold [map 1 | map 2] of ``head_dim`` columns each, every map is a softmax attention of its own, and
    a head's output is (a1 - lambda a2) divided by its root mean square over ``v_dim`` (eps ``norm_eps``) times
    (1 - ``diff``), with lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + ``diff`` from four learned vectors.  ``window``:
    only the last ``window`` keys are visible (None: all); ``position``: a position part applied to every map;
    ``gate``: the heads' outputs, side by side, are multiplied element by element with sigmoid(W_g h) before the
    output projection."""

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    v_dim: int
    scale: float
    diff: float
    norm_eps: float
    window: Optional[int] = None
    position: Optional[Any] = None
    gate: bool = False
    kind: str = "diff_attention"


@dataclass(frozen=True)
class KeyValueAttentionSpec:
    """Causal grouped-query attention whose values are its keys (kind "key_value_attention"): q = W_q h, k = W_k h,
    no value projection; v = k as it stands before the key norm.  Every option is off when None / False / 0:

    * ``bias``: the query, key and output projections take a bias;
    * ``taps``: queries and keys pass a short causal convolution over time per channel, right after the projection,
      y_t = sum_j w[:, j] u_(t - taps + 1 + j) (not added to its input); the last ``taps`` - 1 projections are state;
    * ``qk_norm_eps``: per head, queries and keys are divided by their root mean square and multiplied by a weight of
      ``head_dim`` values that all heads share;
    * ``temp_coef``, ``temp_every``: the query at position p is multiplied by 1 + coef * ln(floor((p + 1) / every) + 1);
    * ``unit_sink``: the softmax's denominator holds one more term exp(0), with no key or value;
    * ``head_gate``: head h's output is multiplied by sigmoid(W_g h)_h, one number per head."""

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    bias: bool = False
    taps: int = 0
    qk_norm_eps: Optional[float] = None
    temp_coef: float = 0.0
    temp_every: int = 0
    unit_sink: bool = False
    head_gate: bool = False
    kind: str = "key_value_attention"


@dataclass(frozen=True)
class MLSTMSpec:
    """The matrix memory of an mLSTM layer (kind "mlstm"): per head a [head_dim, v_dim] state S and a normaliser n with a
    running maximum m (all zero at a sequence's start).  q = W_q h / sqrt(head_dim), k = W_k h, v = W_v h; per head a log
    input gate i = cap tanh((W_i h + b_i) / cap) and a log forget gate f = logsigmoid(cap tanh((W_f h + b_f) / cap));
    m_t = max(f + m_(t-1), i); S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T, n_t likewise with k alone;
    o = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6); each head's o is divided by its root mean square (``norm_eps``),
    multiplied by a weight over all heads' columns and by sigmoid(W_g h), then projected."""

    hidden_size: int
    num_heads: int
    head_dim: int
    v_dim: int
    gate_cap: float
    norm_eps: float
    kind: str = "mlstm"


@dataclass(frozen=True)
class PairMixerSpec:
    """Two mixers side by side that read the same input (kind "pair"): left_scale * left(h) + right_scale * right(h)."""

    left: Any
    right: Any
    left_scale: float = 1.0
    right_scale: float = 1.0
    kind: str = "pair"


@dataclass(frozen=True)
class GLASpec:
    """Gated linear attention (kind "gla"): per head a [head_dim, v_dim] state S <- diag(a_t) S + k_t v_t^T read as
    o_t = S^T q_t, with a decay per key channel a = sigmoid(W2 (W1 h) + b)**(1 / tau) through two small matrices of
    inner size ``decay_rank``; the head's output is RMS-normed over ``v_dim`` with a weight shared by the heads and
    gated by silu(W_g h)."""

    hidden_size: int
    num_heads: int
    head_dim: int
    v_dim: int
    tau: float
    decay_rank: int
    norm_eps: float
    kind: str = "gla"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Causal attention through low-rank latents (kind "latent_attention").

    Queries: RMSNorm(W_dq h) of ``q_rank`` columns, up-projected to ``num_heads`` heads of [head_dim plain | rot_dim
    rotated] columns.  Keys and values: W_dkv h gives ``kv_rank`` columns that are normed (the latent) and ``rot_dim``
    more that are rotated and shared by all heads; a head's plain key and its value (``v_dim`` columns) are
    up-projections of the latent.  Only the latent and the rotated part are cached.  ``sink``: the softmax's
    denominator holds one more term exp(s_h), a learned number per head with no key or value.
    """

    hidden_size: int
    num_heads: int
    head_dim: int
    rot_dim: int
    v_dim: int
    q_rank: int
    kv_rank: int
    scale: float
    norm_eps: float
    position: Optional[Any] = None
    sink: bool = False
    kind: str = "latent_attention"


@dataclass(frozen=True)
class WKVSpec:
    """Linear recurrence with a [head_dim, head_dim] state per head and a data-dependent decay per key channel
    (kind "wkv"); ``decay_rank`` is the inner size of the decay's two small matrices, ``norm_eps`` the eps of the
    per-head unit norm of the output."""

    hidden_size: int
    num_heads: int
    head_dim: int
    decay_rank: int
    norm_eps: float
    kind: str = "wkv"


@dataclass(frozen=True)
class GatedMLPSpec:
    """Dense gated feed-forward: down(act(gate(x)) * up(x)).

    ``activation`` "silu": silu(g) * u.  "clamped_swish": g' = min(g, limit), u' = clamp(u, -limit, limit),
    g' * sigmoid(alpha * g') * (u' + 1)."""

    hidden_size: int
    intermediate_size: int
    activation: str = "silu"
    limit: Optional[float] = None
    alpha: float = 1.702
    kind: str = "gated_mlp"


@dataclass(frozen=True)
class ActMLPSpec:
    """Dense feed-forward without a gate (kind "act_mlp"): down(act(up(x))).  ``activation`` "xielu": with two learned
    numbers p, q (stored with the layer), act(z) = softplus(p) z^2 + z / 2 for z > 0 and
    (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2 otherwise.  "relu2": act(z) = max(z, 0)^2, no learned numbers."""

    hidden_size: int
    intermediate_size: int
    activation: str = "xielu"
    kind: str = "act_mlp"


@dataclass(frozen=True)
class MoESpec:
    """Mixture of experts (kind "moe"): a 32-bit router over ``n_experts`` gated feed-forwards (``expert``: the
    GatedMLPSpec every one of them has) and ``n_identity`` further outputs that stand for experts which hand their
    input back.  s = softmax(router logits) over all of them; the ``top`` largest of s + correction are chosen; their
    weights are their s divided by the chosen ones' sum (+ 1e-20), times ``route_scale``.  ``shared``: a feed-forward
    that every token runs and that is added.

    ``router_bias``: the router's logits take a learned bias.  ``correction`` False: the router has no correction
    vector.  ``over_chosen``: the ``top`` largest logits (+ correction) are chosen and the weights are the softmax over
    the chosen logits only (the same numbers as above, without the softmax over all outputs in between)."""

    hidden_size: int
    n_experts: int
    n_identity: int
    top: int
    route_scale: float
    expert: Any
    shared: Optional[Any] = None
    router_bias: bool = False
    correction: bool = True
    over_chosen: bool = False
    kind: str = "moe"


@dataclass(frozen=True)
class StreamNormSpec:
    """The way a branch meets a residual kept in ``streams`` copies X_1 .. X_S (kind "stream_rmsnorm"): it reads
    RMSNorm(sum_s in[s] X_s) * weight, and its output y returns as X'_t = sum_s mix[s, t] X_s + mult out[t] y, all
    streams at once from the old ones, in 32-bit.  ``streams`` 0: one plain residual, x += mult y, no learned
    in / out / mix."""

    size: int
    eps: float
    streams: int = 0
    mult: float = 1.0
    kind: str = "stream_rmsnorm"


@dataclass(frozen=True)
class StreamBlockSpec:
    """One layer over a residual in streams: the mixer, then the feed-forward (which may be absent), each read and
    written through its own StreamNormSpec."""

    mixer_norm: Any
    mixer: Any
    ff_norm: Any = None
    ff: Any = None
    kind: str = "streams"


@dataclass(frozen=True)
class BranchNormSpec:
    """RMS norm of a branch's OUTPUT on its way into the residual (kind "branch_rmsnorm"):
    x += y / sqrt(mean(y^2) + eps) * (offset + w) * s, with ``layer_scale`` a learned vector s per column (else 1)."""

    size: int
    eps: float
    offset: float = 0.0
    layer_scale: bool = False
    kind: str = "branch_rmsnorm"


@dataclass(frozen=True)
class PostNormBlockSpec:
    """One layer whose branches read the residual itself and are normed on the way back (kind "postnorm"):
    x += N1(mixer(conv(x))); x += N2(ff(x)).  ``conv``: what the mixer reads goes through this part first (None: the
    residual as it is); ``ff`` may be absent."""

    mixer: Any
    mixer_norm: Any
    conv: Any = None
    ff: Any = None
    ff_norm: Any = None
    kind: str = "postnorm"


@dataclass(frozen=True)
class SandwichBlockSpec:
    """One layer whose branches are normed on the way in and on the way back (kind "sandwich"):
    x += N1b(mixer(N1(x))); x += N2b(ff(N2(x))).  The inner norms are of a kind that reads the residual
    ("grouped_rmsnorm"), the outer ones of a kind that adds to it ("branch_rmsnorm"); ``ff`` may be absent."""

    mixer_norm: Any
    mixer: Any
    mixer_out_norm: Any
    ff_norm: Any = None
    ff: Any = None
    ff_out_norm: Any = None
    kind: str = "sandwich"


@dataclass(frozen=True)
class LoopSpec:
    """Layers ``start`` .. ``stop`` - 1 run ``times`` times in a row with the same weights, each pass with a cache of its
    own; the rest follow.  Before each pass but the first the embedding output is added to the residual; before every
    pass, after that, row t of a learned [times, hidden] table (t the number of the pass)."""

    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class BlockSpec:
    """One layer: x += mixer(norm(x)); x += ff(norm(x)) for kind "prenorm"."""

    mixer_norm: Any
    mixer: Any
    ff_norm: Any
    ff: Any
    kind: str = "prenorm"


@dataclass(frozen=True)
class ParallelBlockSpec:
    """One layer with a single norm that both branches read: x += mixer(norm(x)) + ff(norm(x)); ``ff`` may be None."""

    norm: Any
    mixer: Any
    ff: Any = None
    kind: str = "parallel"


@dataclass(frozen=True)
class ModelSpec:
    """A decoder: embedding, layers, the order they run in, final norm, output head.

    ``schedule`` lists layer indices in execution order; an index may appear
    more than once: the layer then runs again with the same weights, and each occurrence keeps
    a cache entry of its own.

    Three optional constants of the outer model, None where an architecture has none (Qwen3 has
    none): ``embedding_scale`` multiplies the embedded rows, ``logit_scale`` the logits, and
    ``logit_softcap`` c turns a logit x into c * tanh(x / c), after the scale.

    ``residual_float32``: the residual stream is kept and summed in 32-bit also in a bfloat16 run (the norms then
    read 32-bit rows and hand the run's dtype to the branches).

    ``streams``: the residual is kept in this many 32-bit copies side by side ([rows, streams * hidden], all equal to
    the embedding output at the start, summed before the final norm); the layers are then of kind "streams".

    ``position_embedding``: a position part that enters at the embedding (its ``embed`` makes the first residual
    from the token ids and the rows' positions); None: positions enter in the mixers only.

    ``loop``: a run of layers that repeats (see LoopSpec); it takes the place of ``schedule`` and needs a 32-bit residual.
    """

    hidden_size: int
    vocab_size: int
    layers: Tuple[BlockSpec, ...]
    final_norm: Any
    tie_embeddings: bool
    schedule: Tuple[int, ...] = field(default=())
    embedding_scale: Optional[float] = None
    logit_scale: Optional[float] = None
    logit_softcap: Optional[float] = None
    residual_float32: bool = False
    streams: Optional[int] = None
    position_embedding: Optional[Any] = None
    loop: Optional[LoopSpec] = None

    def execution_order(self) -> Tuple[int, ...]:
        if self.loop is not None:
            lo, hi, n = self.loop.start, self.loop.stop, len(self.layers)
            return tuple(range(lo)) + tuple(range(lo, hi)) * self.loop.times + tuple(range(hi, n))
        return self.schedule if self.schedule else tuple(range(len(self.layers)))

    def pass_starts(self):
        """{place in the execution order: number of the pass that starts there} for a model with a loop."""
        if self.loop is None:
            return {}
        lo, hi = self.loop.start, self.loop.stop
        return {lo + t * (hi - lo): t for t in range(self.loop.times)}
