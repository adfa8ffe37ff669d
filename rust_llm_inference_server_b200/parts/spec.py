"""A model as data: which parts each layer is made of, with every size and constant as a
parameter, and the order in which layers run.

Nothing here knows an architecture.  An architecture's `describe(config)` returns a `ModelSpec`;
`parts.build` turns each spec into a part by its `kind` through the part registries.
The reference builds its one model imperatively (crates/model/src/llama.rs:142-170); the specs
carry the same information: tensor names (llama.rs:25-28,144-156; attention.rs:47-51;
layers.rs:171-173) and constants (config.rs:5-26).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass(frozen=True)
class RMSNormSpec:
    """y = x / sqrt(mean(x^2) + eps) * (offset + w).  `offset` 1 is a weight stored around zero."""
    dim: int
    eps: float
    weight: str                      # tensor name, shape (dim,)
    offset: float = 0.0
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class RopeSpec:
    """Rotate-half rotary encoding; `scaling` as in config.RopeScaling (llama3) or None.  `head_dim` is the number
    of entries that turn (entry i with entry i + head_dim / 2): a mixer that rotates itself may apply it to the
    first entries of a longer head and let the rest pass."""
    head_dim: int
    theta: float
    scaling: Any = None
    # True: the frequencies are worked out in float64 and rounded to float32 once (the default keeps the
    # reference's float32 arithmetic, crates/model/src/rope.rs:19-49)
    exact: bool = False
    kind: str = "rope"


@dataclass(frozen=True)
class YarnRopeSpec:
    """Rotate-half rotary encoding over the first `dims` entries of a vector (the rest pass
    unchanged) with YaRN's frequency blend: with dim(t) = dims ln(original / (2 pi t)) / (2 ln base),
    lo = max(floor(dim(fast)), 0), hi = min(ceil(dim(slow)), dims - 1) and ramp_i = clamp((i - lo) /
    max(hi - lo, 0.001), 0, 1), frequency i is f_i / factor * ramp_i + f_i (1 - ramp_i), f_i =
    base^(-2i / dims), and cos and sin are multiplied by 0.1 ln(factor) + 1.  `factor` None: the plain
    frequencies f_i and no multiplier.  `pairing` says which entries turn together: "half" (entry i with
    entry i + dims / 2) or "adjacent" (entry 2i with entry 2i + 1); a mixer takes the one its kernels know."""
    dims: int
    base: float
    factor: Optional[float] = None
    original: float = 0.0
    fast: float = 0.0
    slow: float = 0.0
    pairing: str = "half"
    kind: str = "yarn_rope"


@dataclass(frozen=True)
class NoPositionSpec:
    kind: str = "none"


@dataclass(frozen=True)
class GQAAttentionSpec:
    """Causal grouped-query attention.  `window`: keys visible to a query (None = all earlier
    ones).  `scale`: score multiplier (None = 1 / sqrt(head_dim), the reference's fixed choice,
    crates/model/src/attention.rs:147,210)."""
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    q_proj: str                      # (n_heads * head_dim, hidden)
    k_proj: str                      # (n_kv_heads * head_dim, hidden)
    v_proj: str
    o_proj: str                      # (hidden, n_heads * head_dim)
    position: Any = field(default_factory=NoPositionSpec)
    window: Optional[int] = None
    scale: Optional[float] = None
    kind: str = "gqa_attention"


@dataclass(frozen=True)
class DistanceBiasSpec:
    """A learned bias added to a score by how far back its key lies: row bucket(n) of `table`
    (rows, n_heads) for a key n positions before the query.  With half = rows // 2: bucket(n) = n below
    half; from there on the rows are spaced evenly in ln(n) up to `far`, bucket(n) = min(rows - 1,
    half + floor(ln(n / half) / ln(far / half) * (rows - half)))."""
    table: str                       # (rows, n_heads)
    rows: Optional[int]              # None: as many as the checkpoint's tensor has
    far: float
    kind: str = "log_buckets"


@dataclass(frozen=True)
class BiasedAttentionSpec:
    """Causal grouped-query attention without rotation: queries and keys are RMS-normed per head
    (weights `q_norm`, `k_norm` of size `dim`, shared by the heads; None: no norm), score = scale *
    q . k + bias by distance (`bias`, None: none), values have a width of their own (`v_dim`).
    `value_mix` names a scalar lambda: the layer caches and uses (1 - lambda) v + lambda v_src, v_src
    being the values that the layer with `value_source` made of the same token (that layer's own values
    stay unmixed).  `head_gate` (n_heads, hidden): head h's output is multiplied by sigmoid of row h
    applied to the mixer's input.

    Further options, each off by default.  `v_proj` None: the values are the keys as projected (before rotation
    and norm; v_dim = dim).  `rotation`: a rotary spec with adjacent pairing, applied to queries and keys before
    their norms.  `unit_norm`: queries and keys are divided by their root mean square per head without a weight
    (instead of `q_norm` / `k_norm`).  `q_temp` = (coef, every): queries are multiplied by 1 + coef ln(floor((p +
    1) / every) + 1) at position p.  `slopes`: one number a head, slope * distance is subtracted from a score.
    `sink` (n_heads,): exp(sink_h) joins the denominator of head h's softmax, without a key or a value.
    `rotation` may also be a rotate-half spec (`RopeSpec`, or a yarn spec with pairing "half").  `q_bias`, `k_bias`,
    `v_bias`: biases of the three projections.  `out_gate` (n_heads * v_dim, hidden): every channel of every head's
    output is multiplied by sigmoid of its row applied to the mixer's input (instead of `head_gate`)."""
    hidden: int
    n_heads: int
    n_kv_heads: int
    dim: int
    v_dim: int
    scale: float
    eps: float
    q_proj: str                      # (n_heads * dim, hidden)
    k_proj: str                      # (n_kv_heads * dim, hidden)
    v_proj: Optional[str]            # (n_kv_heads * v_dim, hidden)
    o_proj: str                      # (hidden, n_heads * v_dim)
    q_norm: Optional[str] = None     # (dim,)
    k_norm: Optional[str] = None     # (dim,)
    bias: Any = None                 # a DistanceBiasSpec
    head_gate: Optional[str] = None  # (n_heads, hidden)
    value_mix: Optional[str] = None  # scalar tensor
    value_source: bool = False
    window: Optional[int] = None
    rotation: Any = None
    unit_norm: bool = False
    q_temp: Optional[tuple] = None   # (coef, every)
    slopes: Optional[tuple] = None   # one a head
    sink: Optional[str] = None       # (n_heads,)
    q_bias: Optional[str] = None     # (n_heads * dim,)
    k_bias: Optional[str] = None     # (n_kv_heads * dim,)
    v_bias: Optional[str] = None     # (n_kv_heads * v_dim,)
    out_gate: Optional[str] = None   # (n_heads * v_dim, hidden)
    kind: str = "biased_attention"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Causal attention whose keys and values are linear maps of a cached latent.  Per token the
    cache holds [c | k_rot]: c = rmsnorm(W_dkv h)[:kv_rank] * kv_norm and the rotated key part
    (`rot_dim` wide, shared by all heads).  Queries: q = W_uq (rmsnorm(W_dq h) * q_norm), per head
    [dim unrotated | rot_dim rotated].  Head h: key = [W_uk_h c | k_rot], value = W_uv_h c, score =
    scale * q . key.  `sink`: a tensor (n_heads,) whose exp joins each head's softmax denominator.
    `kv_down` None: the layer has no W_dkv and reads the cache slot of another call."""
    hidden: int
    n_heads: int
    dim: int                         # unrotated query/key entries per head
    rot_dim: int                     # rotated entries per head
    v_dim: int
    q_rank: int
    kv_rank: int
    scale: float
    eps: float
    q_down: str                      # (q_rank, hidden)
    q_norm: str                      # (q_rank,)
    q_up: str                        # (n_heads * (dim + rot_dim), q_rank)
    kv_down: Optional[str]           # (kv_rank + rot_dim, hidden)
    kv_norm: Optional[str]           # (kv_rank,)
    k_up: str                        # (n_heads * dim, kv_rank)
    v_up: str                        # (n_heads * v_dim, kv_rank)
    o_proj: str                      # (hidden, n_heads * v_dim)
    sink: Optional[str] = None       # (n_heads,)
    position: Any = field(default_factory=NoPositionSpec)
    window: Optional[int] = None
    kind: str = "latent_attention"


@dataclass(frozen=True)
class LightningAttentionSpec:
    """Linear attention with a per-head decay: q, k = silu(W h) (n_heads x dim), v = silu(W_v h)
    (n_heads x v_dim); S_t = decay_h S_(t-1) + k_t v_t^T (float32 state per request), o_t = S_t^T q_t;
    out = W_o (rmsnorm(o) * out_norm * sigmoid(W_g h))."""
    hidden: int
    n_heads: int
    dim: int
    v_dim: int
    decay: tuple                     # one factor per head
    eps: float
    q_proj: str                      # (n_heads * dim, hidden)
    k_proj: str
    v_proj: str                      # (n_heads * v_dim, hidden)
    gate_proj: str                   # (n_heads * v_dim, hidden)
    out_norm: str                    # (n_heads * v_dim,)
    o_proj: str                      # (hidden, n_heads * v_dim)
    kind: str = "lightning_attention"


@dataclass(frozen=True)
class RetentionSpec:
    """A decayed outer-product state read by the query as it is (scores are neither exponentiated nor normalised), one fixed decay a head: q, k = W h (n_heads x dim), rotated by
    position where `rotation` (a rotate-half spec over the first entries of a head) is given, k times `k_scale`
    (None: dim^(-1/2)); v = W_v h (n_heads x v_dim); S_t = decay_h S_(t-1) + k_t v_t^T (float32 state per request),
    o_t = S_t^T q_t; each head's o is divided by its root mean square (times `out_norm` (v_dim,), None: no weight);
    out = W_o (o * act(W_g h)) with `gate_act` "silu" or "sigmoid" (`gate_proj` None: no gate)."""
    hidden: int
    n_heads: int
    dim: int
    v_dim: int
    decay: tuple                     # one factor a head
    eps: float
    q_proj: str                      # (n_heads * dim, hidden)
    k_proj: str
    v_proj: str                      # (n_heads * v_dim, hidden)
    o_proj: str                      # (hidden, n_heads * v_dim)
    gate_proj: Optional[str] = None  # (n_heads * v_dim, hidden)
    gate_act: str = "silu"
    out_norm: Optional[str] = None   # (v_dim,)
    rotation: Any = None
    k_scale: Optional[float] = None
    kind: str = "retention"


@dataclass(frozen=True)
class ForgetGateRecurrenceSpec:
    """A linear recurrence with one gate a channel that keeps f of the state and writes 1 - f of the new value (HGRN2): q = silu(W_q h) (n_heads x dim), v =
    W_v h (n_heads x v_dim), a forget gate per head and channel f = l + (1 - l) sigmoid(W_f h + f_bias) above the
    lower bound l = `lower` (n_heads * dim,); S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T (float32 state per request),
    o_t = S_t^T q_t; out = W_o (rmsnorm_per_head(o) * out_norm) with `out_norm` (v_dim,) shared by the heads."""
    hidden: int
    n_heads: int
    dim: int
    v_dim: int
    eps: float
    q_proj: str                      # (n_heads * dim, hidden)
    f_proj: str                      # (n_heads * dim, hidden)
    lower: str                       # (n_heads * dim,)
    v_proj: str                      # (n_heads * v_dim, hidden)
    o_proj: str                      # (hidden, n_heads * v_dim)
    f_bias: Optional[str] = None     # (n_heads * dim,)
    out_norm: Optional[str] = None   # (v_dim,)
    kind: str = "forget_gate_recurrence"


@dataclass(frozen=True)
class GatedDeltaSpec:
    """The gated delta rule: q, k = W h (n_qk_heads x dim), v = W_v h (n_heads x v_dim); each passes a causal
    convolution over time per channel (`conv` taps, weights `<projection>.conv`-like tensors (channels, taps), the
    last tap on the current token) and silu; q and k become unit vectors per head (x / sqrt(sum x^2 + unit_eps)),
    q times dim^(-1/2); beta = sigmoid(W_b h) and decay g = exp(-exp(a_log) softplus(W_a h + dt_bias)), one a
    head; per head S <- g S, u = beta (v - S^T k), S <- S + k u^T, o = S^T q (float32 state per request); out =
    W_o (rmsnorm_per_head(o) * out_norm * silu(W_g h)).  Head h reads q and k of head h / (n_heads / n_qk_heads)."""
    hidden: int
    n_heads: int
    n_qk_heads: int
    dim: int
    v_dim: int
    conv: int
    eps: float
    q_proj: str                      # (n_qk_heads * dim, hidden)
    k_proj: str
    v_proj: str                      # (n_heads * v_dim, hidden)
    q_conv: str                      # (n_qk_heads * dim, conv)
    k_conv: str
    v_conv: str                      # (n_heads * v_dim, conv)
    beta_proj: str                   # (n_heads, hidden)
    decay_proj: str                  # (n_heads, hidden)
    a_log: str                       # (n_heads,)
    dt_bias: str                     # (n_heads,)
    gate_proj: str                   # (n_heads * v_dim, hidden)
    out_norm: str                    # (v_dim,)
    o_proj: str                      # (hidden, n_heads * v_dim)
    unit_eps: float = 1e-6
    kind: str = "gated_delta"


@dataclass(frozen=True)
class ParallelMixerSpec:
    """Several mixers side by side on the same input: the result is the mean of their outputs, each first
    RMS-normed over the model width with a weight of its own (`out_norms`, one tensor name a branch).  At most
    one branch keeps a paged cache and at most one a per-request state.  `out_norms` None: the outputs join as they
    are.  `coefficients` (one number a branch; None: 1 / branches): the result is their weighted sum."""
    hidden: int
    branches: tuple                  # of mixer specs
    out_norms: Optional[tuple]       # of tensor names, shape (hidden,)
    eps: float
    coefficients: Optional[tuple] = None
    kind: str = "parallel"


@dataclass(frozen=True)
class DenseFFSpec:
    """W_down act(W_up h + b_up) + b_down; `activation` "relu2" is the square of max(., 0).  The
    biases are optional tensors."""
    hidden: int
    intermediate: int
    up_proj: str                     # (intermediate, hidden)
    down_proj: str                   # (hidden, intermediate)
    up_bias: Optional[str] = None    # (intermediate,)
    down_bias: Optional[str] = None  # (hidden,)
    activation: str = "relu2"
    kind: str = "dense_ff"


@dataclass(frozen=True)
class SwiGLUSpec:
    """W_down (g sigmoid(slope g) (u + up_shift)) with g = W_gate h and u = W_up h; with a `limit`, g is
    cut at limit from above and u clipped to [-limit, limit] first.  The defaults are SwiGLU.  A `slope` of
    +infinity is the limit max(g, 0) (u + up_shift): a unit gated by relu."""
    hidden: int
    intermediate: int
    gate_proj: str                   # (intermediate, hidden)
    up_proj: str
    down_proj: str                   # (hidden, intermediate)
    slope: float = 1.0
    limit: Optional[float] = None
    up_shift: float = 0.0
    kind: str = "swiglu"


@dataclass(frozen=True)
class RoutedFFSpec:
    """A mixture of `n_experts` gated feed-forwards (each as SwiGLUSpec describes, `intermediate` wide) of
    which a token uses `top`.  Scores s = sigmoid(W_router h) in float32; the experts with the largest
    s + correction are chosen; their outputs are summed with weights s * route_scale (not renormalised).
    `scoring` "softmax_chosen": the logits z = W_router h + router_bias choose, and the weights are the softmax
    over the chosen logits alone.
    Tensor names of expert e are the patterns with {e} filled in.  `shared`: a SwiGLUSpec that every token
    runs through, added after multiplication by sigmoid(W_shared_gate h) where `shared_gate` is given.

    `scoring` "softmax": s = softmax(W_router h) over all router outputs.  `n_identity`: the router has that many
    outputs more than there are experts (its last rows); they are scored, grouped and chosen like experts, and a
    chosen one hands the token's input back (times its weight).  `groups` = (count, keep): the router outputs form
    `count` equal groups of neighbours; a group ranks by its largest s + correction, and only outputs of the `keep`
    best groups can be chosen.  `normalize`: the chosen scores are divided by their sum (+ 1e-20) before
    route_scale."""
    hidden: int
    intermediate: int
    n_experts: int
    top: int
    router: str                      # (n_experts, hidden)
    gate_proj: str                   # pattern, (intermediate, hidden)
    up_proj: str
    down_proj: str                   # pattern, (hidden, intermediate)
    correction: Optional[str] = None  # (n_experts,)
    route_scale: float = 1.0
    slope: float = 1.0
    limit: Optional[float] = None
    up_shift: float = 0.0
    shared: Any = None
    shared_gate: Optional[str] = None  # (1, hidden)
    router_bias: Optional[str] = None  # (n_experts,)
    scoring: str = "sigmoid"
    n_identity: int = 0
    groups: Optional[tuple] = None   # (count, keep)
    normalize: bool = False
    kind: str = "routed_ff"


@dataclass(frozen=True)
class EmbeddingSpec:
    """Token table: row `id` of `weight` (vocab, dim) starts the residual stream, multiplied by
    `scale` if one is given (the reference's Llama has none, crates/model/src/llama.rs:256-262), then
    normed where `norm` (an RMSNormSpec) is given."""
    vocab_size: int
    dim: int
    weight: str
    scale: Optional[float] = None
    norm: Any = None
    kind: str = "embedding"


@dataclass(frozen=True)
class LMHeadSpec:
    """Logits = h · weight^T in float32 (crates/model/src/llama.rs:279-285), then, where given,
    multiplied by `logit_scale` and capped smoothly: cap · tanh(logits / cap).  `weight` may name
    the embedding's tensor (tied)."""
    vocab_size: int
    dim: int
    weight: str
    logit_scale: Optional[float] = None
    soft_cap: Optional[float] = None
    kind: str = "lm_head"


@dataclass(frozen=True)
class LayerSpec:
    """One block.  arrangement "prenorm": x += mixer(norm1(x)); x += feed_forward(norm2(x))
    (crates/model/src/llama.rs:264-271; `feed_forward` None leaves the second line out, norm2 is then None too).
    arrangement "sandwich": each sublayer's result is normed
    and scaled before it joins the stream, x += scale1 * post_norm1(mixer(norm1(x))) and the same
    with norm2, feed_forward, post_norm2, scale2; `feed_forward` None leaves the second sublayer out
    (norm2, post_norm2 and scale2 are then None too).  arrangement "outnorm": the sublayers read the
    stream itself and only their results are normed, x += residual_mult * norm1(mixer(x)), then x +=
    residual_mult * norm2(feed_forward(x)), the second line only with a feed-forward.  arrangement "postnorm": the
    sum is normed, x = norm1(stream_mult * x + mixer(x)), then x = norm2(stream_mult * x + feed_forward(x)), the
    sublayers reading x itself and the second line only with a feed-forward."""
    norm1: Any
    mixer: Any
    norm2: Any
    feed_forward: Any
    arrangement: str = "prenorm"
    post_norm1: Any = None
    post_norm2: Any = None
    scale1: Optional[str] = None     # tensor name, shape (hidden,): per-channel scale of the sublayer's result
    scale2: Optional[str] = None
    residual_mult: float = 1.0
    stream_mult: float = 1.0


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order: run `layer` with cache slot `cache`.  A layer may be named by
    several calls (its weights are shared, each call has a cache slot and state of its own unless
    it names another call's slot).  `writes_cache=False`: the call stores nothing and reads the
    slot that an earlier call of the same step has filled."""
    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    vocab_size: int
    hidden: int
    embedding: Any                   # an EmbeddingSpec, or just the tensor's name (vocab, hidden)
    layers: tuple
    order: tuple                     # of LayerCall
    final_norm: Any
    lm_head: Any                     # an LMHeadSpec, or just the tensor's name (the embedding's when tied)
    max_positions: int
    # names that a checkpoint may hold although the model does not read them
    ignorable: tuple = ()
    eos_token_ids: tuple = ()
