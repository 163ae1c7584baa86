"""Typed descriptions of a model: what each part is and which constants it has.

A specification is plain, frozen data.  It holds every size and constant that a
part needs, so that the part itself never looks at a model's configuration.  A
``ModelSpec`` is a list of layer specifications plus the order in which the
layers run; one model can therefore have different mixers and feed-forwards in
different layers, run a layer twice, or let a layer read another layer's cache.

Every specification has a ``kind``: the key under which the implementing class
is registered in ``parts``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


class ConfigError(ValueError):
    """A configuration that is incomplete or inconsistent."""


@dataclass(frozen=True)
class RMSNormSpec:
    """y = x * w / sqrt(mean(x^2) + eps)  (reference: src/models/jiuge/jiuge.cpp:198).  ``weight_name`` is appended to the
    part's prefix.  ``one_plus``: the checkpoint stores the weight around zero and the norm multiplies by 1 + w."""
    size: int
    eps: float
    weight_name: str = "weight"
    one_plus: bool = False
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class RopeSpec:
    """Rotary position encoding of query and key heads.

    Angle of pair ``j`` at position ``p``: ``p / theta ** (j / (head_dim / 2))``
    (reference: src/models/jiuge/jiuge_weight.hpp:134-186).  ``interleaved``
    False pairs element ``j`` with ``j + head_dim/2`` (the checkpoint's own
    layout); True pairs ``2j`` with ``2j+1`` (the layout the reference's loader
    permutes the rows to, scripts/jiuge.py:217-227).
    """
    head_dim: int
    theta: float
    max_positions: int
    interleaved: bool = False
    kind: str = "rope"


@dataclass(frozen=True)
class AttentionSpec:
    """Causal softmax attention over a paged key/value cache.

    ``window`` None: every earlier key is seen.  ``window`` W: a query at
    position p sees keys at positions p-W+1 .. p.
    """
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    softmax_scale: float
    position: Optional[RopeSpec] = None
    window: Optional[int] = None
    bias: bool = False
    kind: str = "attention"


@dataclass(frozen=True)
class SwiGLUSpec:
    """down(silu(gate(x)) * up(x))  (reference: src/models/jiuge/jiuge.cpp:247-249)."""
    hidden_size: int
    intermediate_size: int
    kind: str = "swiglu"


@dataclass(frozen=True)
class LayerNormSpec:
    """y = (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * w + b, in float32.  ``weight_name`` and ``bias_name`` are
    appended to the part's prefix."""
    size: int
    eps: float
    weight_name: str = "weight"
    bias_name: str = "bias"
    kind: str = "layernorm"


@dataclass(frozen=True)
class FrequencyRampSpec:
    """Stretching of a rotation for sequences longer than ``original`` positions: pair i keeps its frequency f_i where its
    wavelength fits more than ``fast`` times into ``original``, gets f_i / ``factor`` where it fits fewer than ``slow`` times,
    and a mixture between: with where(t) = dims ln(original / (2 pi t)) / (2 ln base), lo = max(floor(where(fast)), 0),
    hi = min(ceil(where(slow)), dims - 1), ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), the frequency is
    f_i / factor * ramp_i + f_i (1 - ramp_i).  Cos and sin are multiplied by ``magnitude_slope`` ln(factor) + 1."""
    factor: float
    original: float
    fast: float
    slow: float
    magnitude_slope: float = 0.1


@dataclass(frozen=True)
class PairRotarySpec:
    """Rotation of the first ``dims`` elements of a head in pairs by the angle ``p * base ** (-2i / dims)``, formed in
    float32 from the position; the other elements pass unchanged.  ``layout`` "pairs": pair i is elements (2i, 2i+1);
    "halves": elements (i, i + dims / 2).  Needs no table and no longest position.  ``scaling`` stretches the frequencies
    (``FrequencyRampSpec``)."""
    dims: int
    base: float
    scaling: Optional[FrequencyRampSpec] = None
    layout: str = "pairs"
    kind: str = "pair_rotary"

    def frequencies(self):
        """(f_i for i < dims / 2 in float64, the factor of cos and sin)."""
        import math
        f = [float(self.base) ** (-2.0 * i / self.dims) for i in range(self.dims // 2)]
        s = self.scaling
        if s is None:
            return f, 1.0
        where = lambda turns: self.dims * math.log(s.original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))
        lo, hi = max(math.floor(where(s.fast)), 0), min(math.ceil(where(s.slow)), self.dims - 1)
        ramp = [min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(self.dims // 2)]
        return [fi / s.factor * r + fi * (1.0 - r) for fi, r in zip(f, ramp)], s.magnitude_slope * math.log(s.factor) + 1.0


@dataclass(frozen=True)
class ConvAttentionSpec:
    """Softmax attention over a paged cache with grouped heads whose keys and values may differ in size, and with these
    options, each a parameter: a short causal convolution over time on every channel of the q, k and v projections
    (``conv_taps`` taps, 0 for none), an RMS norm over the WHOLE q and the whole k projection (``qk_norm``), a rotation
    (``position``), after it a division of every head of q and k by its root mean square (``head_norm``, eps
    ``qk_norm_eps``), a cap on the scores (``score_cap`` c > 0: s <- c tanh(s / c)), a sliding window that may keep the
    first ``keep_first`` positions visible for good, a sink (a key of score 0 without a value in every softmax), one output gate per
    head (sigmoid of a projection of the mixer's input), and ``shares_kv``: the layer makes queries only and reads the
    keys and values that another layer wrote into its cache.  The names are those of the checkpoint's tensors below the
    mixer's prefix: projection ``q``, its convolution ``q`` + ``conv_suffix``, its norm ``q`` + ``norm_suffix``.

    Further options: ``bias``: q, k and v have biases (``q`` + ``bias_suffix``), added in the projection; ``head_norm``
    "before_rotation": every head of q and k passes an RMS norm BEFORE the rotation, with one weight of ``head_dim`` per
    projection shared by its heads (``q`` + ``norm_suffix``), eps ``qk_norm_eps``; ``chunk`` C (instead of a window): a query
    at position i sees the keys j <= i with floor(j / C) = floor(i / C), chunks counted from position 0 of the sequence."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    v_head_dim: int
    softmax_scale: float
    window: Optional[int] = None
    conv_taps: int = 0
    qk_norm: bool = False
    qk_norm_eps: float = 1e-6
    position: Optional[PairRotarySpec] = None
    sink: bool = False
    head_gate: bool = False
    shares_kv: bool = False
    head_norm: object = False          # False, True (after the rotation, no weight) or "before_rotation" (weights of head_dim)
    score_cap: float = 0.0
    keep_first: int = 0
    q_name: str = "q"
    k_name: str = "k"
    v_name: str = "v"
    gate_name: str = "g"
    o_name: str = "o"
    conv_suffix: str = ".conv"
    norm_suffix: str = ".norm"
    bias: bool = False
    bias_suffix: str = ".b"
    chunk: Optional[int] = None
    kind: str = "conv_attention"


@dataclass(frozen=True)
class LinearAttentionSpec:
    """Linear attention as a recurrence per head: S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, with the state
    S [head_dim, v_head_dim] in float32 per request.

    ``decay``: one constant per head (then a_t is that constant for every key channel), or None with ``decay_rank`` > 0:
    a_t = sigmoid(W2 (W1 h) + b2) ** (1 / decay_tau), one value per key channel and token (W1: ``decay_down_name``,
    [rank, hidden]; W2: ``decay_up_name`` [heads * head_dim, rank] with bias ``decay_up_name`` + ``bias_suffix``).
    ``qkv_act`` acts on q, k and v ("none" or "silu"); q is multiplied by ``q_scale``.  The output passes an RMS norm,
    over all heads at once with a weight of heads * v_head_dim (``norm_per_head`` False) or per head with one weight of
    v_head_dim shared by the heads, is multiplied by ``gate_act`` of a projection of the mixer's input, and projected.

    Options that another recurrence of this family takes: ``token_shift``: each of q, k, v, the gate and the decay's
    projection reads its own mixture h_t + (h_(t-1) - h_t) * mu of a row and the row before it (mu: ``shift_prefix`` + the
    projection's name; the decay's is ``shift_prefix`` + ``decay_shift_name``), the last row being part of the request's
    state; ``bonus_name``: a tensor u [heads, head_dim], and a row reads the state BEFORE its own decay with a bonus for its
    own key, o_t = (S_(t-1) + diag(u) k_t v_t^T)^T q_t; ``decay_form`` "exp_neg_exp": a_t = exp(-exp(z)) instead of
    sigmoid(z) ** (1 / tau); ``decay_act``: an activation on W1's output; ``decay_bias_name`` names the bias of W2;
    ``norm_per_head`` "unit": the mean per head, a weight of heads * v_head_dim."""
    hidden_size: int
    num_heads: int
    head_dim: int
    v_head_dim: int
    norm_eps: float
    qkv_act: str = "none"
    q_scale: float = 1.0
    decay: Optional[Tuple[float, ...]] = None
    decay_rank: int = 0
    decay_tau: float = 1.0
    norm_per_head: bool = False
    gate_act: str = "sigmoid"
    q_name: str = "q"
    k_name: str = "k"
    v_name: str = "v"
    gate_name: str = "g"
    o_name: str = "o"
    norm_name: str = "norm"
    decay_down_name: str = "a1"
    decay_up_name: str = "a2"
    bias_suffix: str = ".b"
    token_shift: bool = False
    shift_prefix: str = "mu."
    decay_shift_name: str = "w"
    bonus_name: Optional[str] = None
    decay_form: str = "sigmoid_pow"
    decay_act: str = "none"
    decay_bias_name: Optional[str] = None
    kind: str = "linear_attention"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Causal softmax attention whose keys and values are made from one latent vector per position.

    A query head has ``head_dim`` plain and ``rot_dim`` rotated elements.  The down projection ``kv_down_name`` gives
    ``latent_size`` elements, RMS-normed with the weight ``kv_down_name`` + ``norm_suffix`` into the latent vector c, and
    ``rot_dim`` more that are rotated and serve every head as the rotated part of its key.  Head h's plain key is
    ``k_up_name``[h] c, its value ``v_up_name``[h] c (``v_head_dim`` elements); score = (q_plain . k_plain + q_rot . k_rot) *
    ``softmax_scale``.  The cache holds c and the rotated part only.  ``output_gate``: the heads' outputs side by side are
    multiplied by sigmoid(``gate_name`` h) before the output product.

    ``q_rank`` > 0: the queries go through a latent of their own, c_q = RMSnorm(``q_down_name`` h) with the weight
    ``q_down_name`` + ``norm_suffix``, q = ``q_up_name`` c_q.  ``window`` W: a query at position i sees the keys j with
    0 <= i - j < W.  ``rot_dim`` may be 0 (no rotated part)."""
    hidden_size: int
    num_heads: int
    head_dim: int
    rot_dim: int
    v_head_dim: int
    latent_size: int
    softmax_scale: float
    norm_eps: float
    position: Optional[PairRotarySpec] = None
    output_gate: bool = True
    window: Optional[int] = None
    q_rank: int = 0
    q_down_name: str = "dq"
    q_up_name: str = "uq"
    q_name: str = "q"
    kv_down_name: str = "dkv"
    k_up_name: str = "uk"
    v_up_name: str = "uv"
    gate_name: str = "g"
    o_name: str = "o"
    norm_suffix: str = ".norm"
    kind: str = "latent_attention"


@dataclass(frozen=True)
class SelectiveScanSpec:
    """A state-space mixer with input-dependent step sizes: the in-projection gives [x | z] of ``inner`` channels each; x
    passes a causal convolution of ``conv_taps`` taps per channel (with bias) and silu; ``x_name`` projects it to
    [dt part (``dt_rank``) | B (``state_size``) | C (``state_size``)]; dt = softplus(``dt_name`` dt part + bias) per
    channel; A = -exp(``a_log_name``) [inner, state_size]; S <- exp(dt A) S + dt x B, y = S C + D x; y silu(z) is projected
    out.  The state S [inner, state_size] and the convolution's last taps - 1 inputs are kept per request, in float32."""
    hidden_size: int
    inner: int
    state_size: int
    dt_rank: int
    conv_taps: int
    in_name: str = "in"
    conv_name: str = "conv"
    x_name: str = "x"
    dt_name: str = "dt"
    a_log_name: str = "A_log"
    d_name: str = "D"
    o_name: str = "o"
    bias_suffix: str = ".b"
    kind: str = "selective_scan"


@dataclass(frozen=True)
class RoutedExpertsSpec:
    """A feed-forward of ``num_experts`` small gated units of which each row uses ``top``: scores are sigmoid(router h) in
    float32; the ``top`` largest choose the experts; an expert sees score * h (``scale_input``) and the outputs add up
    without renormalising.  ``shared``: a gated unit that every row passes, added on top.

    ``score_form`` "softmax_renorm": scores are softmax(router h) over all experts, the chosen ones' scores are divided by
    their sum (+ 1e-20) and multiply the units' OUTPUTS (``scale_input`` False); that is the softmax over the chosen
    logits alone.  ``act`` "swish_clamp": a unit's inner value is g' sigmoid(1.702 g') (u' + 1) with g' = min(gate h, limit),
    u' = clamp(up h, -limit, limit).  ``router_bias``: the logits are router h + ``router_name`` + ``bias_suffix``.
    ``shared_gate_name``: the shared unit's output is multiplied by sigmoid(w . h), one number per row, w that tensor
    ([1, hidden], below ``shared_prefix``)."""
    hidden_size: int
    num_experts: int
    top: int
    expert_size: int
    act: str = "silu"
    shared: Optional[object] = None
    scale_input: bool = True
    score_form: str = "sigmoid"
    limit: float = 0.0
    router_name: str = "router"
    router_bias: bool = False
    bias_suffix: str = ".b"
    shared_gate_name: Optional[str] = None
    expert_prefix: str = "e{}."
    shared_prefix: str = "shared."
    gate_name: str = "gate"
    up_name: str = "up"
    down_name: str = "down"
    kind: str = "routed_experts"


@dataclass(frozen=True)
class ReinjectSpec:
    """A step between two layers that feeds the embedding's output in again: x <- W [x | x0] + b, with W ``weight_name``
    [hidden, 2 hidden] and b row ``step_index`` of ``step_name`` [steps, hidden] (None: no b)."""
    hidden_size: int
    steps: int
    step_index: int
    weight_name: str = "loop.in"
    step_name: Optional[str] = "loop.step"
    kind: str = "reinject"


@dataclass(frozen=True)
class StepVectorSpec:
    """A step between two layers that adds one row of a table to every row of the stream: x <- x + ``table_name``[``index``]
    (the table [``steps``, hidden]; a vector per pass of a repeated span, say)."""
    hidden_size: int
    steps: int
    index: int
    table_name: str = "loop.step"
    kind: str = "step_vector"


@dataclass(frozen=True)
class DeltaRuleSpec:
    """The gated delta rule, a recurrence per head with the state S [head_dim, v_head_dim] in float32 per request:

        S <- g_t S;   w_t = beta_t (v_t - S^T k_t);   S <- S + k_t w_t^T;   o_t = S^T q_t

    q and k have ``num_kv_heads`` heads of ``head_dim`` (query head h uses head h // (num_heads / num_kv_heads)), v has
    ``num_heads`` heads of ``v_head_dim``; none has a bias.  Each passes a causal convolution over time per channel
    (``conv_taps`` taps, tensor ``q`` + ``conv_suffix`` [channels, taps], the last column the current row's, zeros before
    the sequence) and ``conv_act``; q and k then become unit vectors per head, x / sqrt(sum(x^2) + ``unit_eps``), q also
    times ``q_scale`` (None: head_dim ** -0.5).  beta_t = sigmoid(``beta_name`` h) and g_t = exp(-exp(``a_log_name``)
    softplus(``decay_name`` h + ``dt_bias_name``)), one each per head.  The heads' outputs are divided by their root mean
    square over v_head_dim (``norm_eps``), times the weight ``norm_name`` [v_head_dim] shared by the heads, times
    ``gate_act`` of ``gate_name`` h, and projected by ``o_name``.  The convolutions' last taps - 1 inputs are state too."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    v_head_dim: int
    conv_taps: int
    norm_eps: float
    unit_eps: float = 1e-6
    q_scale: Optional[float] = None
    conv_act: str = "silu"
    gate_act: str = "silu"
    q_name: str = "q"
    k_name: str = "k"
    v_name: str = "v"
    beta_name: str = "b"
    decay_name: str = "a"
    a_log_name: str = "A_log"
    dt_bias_name: str = "dt_bias"
    gate_name: str = "g"
    norm_name: str = "norm"
    o_name: str = "o"
    conv_suffix: str = ".conv"
    kind: str = "delta_rule"


@dataclass(frozen=True)
class SandwichBlockSpec:
    """One layer with a norm before and after each sublayer: x += norm_b(mixer(norm_a(x))); x += norm_d(ff(norm_c(x))).
    ``feed_forward`` None: the layer has a mixer only."""
    mixer: object
    feed_forward: Optional[object]
    mixer_norm: object
    mixer_post_norm: object
    ffn_norm: Optional[object]
    ffn_post_norm: Optional[object]
    mixer_prefix: str = "mix."
    ffn_prefix: str = "mlp."
    mixer_norm_prefix: str = "norm1"
    mixer_post_norm_prefix: str = "norm1b"
    ffn_norm_prefix: str = "norm2"
    ffn_post_norm_prefix: str = "norm2b"
    kind: str = "sandwich"


@dataclass(frozen=True)
class GLUSpec:
    """down(act(gate(x)) * up(x)) with ``act`` "silu", "relu" or "gelu_tanh" (0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))),
    or "swish_clamp": down(g' sigmoid(1.702 g') (u' + 1)) with g' = min(gate x, limit), u' = clamp(up x, -limit, limit)."""
    hidden_size: int
    intermediate_size: int
    act: str = "gelu_tanh"
    limit: float = 0.0
    gate_name: str = "gate"
    up_name: str = "up"
    down_name: str = "down"
    kind: str = "glu"


@dataclass(frozen=True)
class MLPSpec:
    """down(act(up(x))): a feed-forward without a gate; ``act`` "gelu_erf" (0.5 z (1 + erf(z / sqrt 2))), "gelu_tanh", "silu" or
    "relu"."""
    hidden_size: int
    intermediate_size: int
    act: str = "gelu_erf"
    up_name: str = "up"
    down_name: str = "down"
    kind: str = "mlp"


@dataclass(frozen=True)
class ParallelMixerSpec:
    """Two mixers side by side that read the same input: ``left_scale`` * left(h) + ``right_scale`` * right(h).  Each is any
    mixer's specification; at most one of them keeps pages."""
    left: object
    right: object
    left_scale: float = 1.0
    right_scale: float = 1.0
    left_prefix: str = "left."
    right_prefix: str = "right."
    kind: str = "parallel"


@dataclass(frozen=True)
class PostNormBlockSpec:
    """One layer whose norms sit on the sublayers' outputs: x += norm_a(mixer(x)); x += norm_b(feed_forward(x)).  The
    sublayers read the stream itself.  ``feed_forward`` None: the layer has a mixer only."""
    mixer: object
    feed_forward: Optional[object]
    mixer_norm: object
    ffn_norm: Optional[object]
    mixer_prefix: str = "mix."
    ffn_prefix: str = "mlp."
    mixer_norm_prefix: str = "norm1"
    ffn_norm_prefix: str = "norm2"
    kind: str = "postnorm"


@dataclass(frozen=True)
class BlockSpec:
    """One layer: x += s * mixer(norm_a(x)); x += s * feed_forward(norm_b(x)).  ``feed_forward`` None: the layer has a
    mixer only.

    The four ``*_prefix`` strings are the names, below the layer's own prefix,
    under which the checkpoint stores each part's tensors.
    """
    mixer: object
    feed_forward: Optional[object]
    mixer_norm: object
    ffn_norm: Optional[object]
    residual_scale: float = 1.0
    mixer_prefix: str = "self_attn."
    ffn_prefix: str = "mlp."
    mixer_norm_prefix: str = "input_layernorm."
    ffn_norm_prefix: str = "post_attention_layernorm."
    kind: str = "prenorm"


@dataclass(frozen=True)
class RunEntry:
    """One entry of the execution order.

    ``layer`` indexes ``ModelSpec.layers`` (whose weights run), ``cache`` names
    the cache the mixer works on.  ``writes_cache`` False means the mixer only
    reads what an earlier entry with the same ``cache`` wrote in this step.
    """
    layer: int
    cache: int
    writes_cache: bool = True
    before: Optional[object] = None     # a step on the stream that runs before the layer (``ReinjectSpec``), or None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    layers: Tuple[BlockSpec, ...]
    order: Tuple[RunEntry, ...]
    final_norm: object
    embed_scale: float = 1.0
    logit_scale: float = 1.0
    logit_softcap: float = 0.0         # c > 0: logits <- c tanh(logits / c)
    position_table_name: Optional[str] = None      # a learned vector per position [position_rows, hidden], added to the embedding
    position_rows: int = 0
    tie_embeddings: bool = False
    embed_name: str = "model.embed_tokens.weight"
    lm_head_name: str = "lm_head.weight"
    final_norm_prefix: str = "model.norm."
    layer_prefix: str = "model.layers.{}."
    eos_token_ids: Tuple[int, ...] = field(default_factory=tuple)

    def __post_init__(self):
        n = len(self.layers)
        writers = {}
        for pos, e in enumerate(self.order):
            if not 0 <= e.layer < n:
                raise ConfigError(f"order[{pos}] names layer {e.layer}, but there are {n} layers")
            if e.writes_cache:
                if e.cache in writers:
                    raise ConfigError(
                        f"order[{pos}] and order[{writers[e.cache]}] both write cache {e.cache}")
                writers[e.cache] = pos
            elif e.cache not in writers:
                raise ConfigError(
                    f"order[{pos}] reads cache {e.cache} before any entry has written it")

    @property
    def num_caches(self) -> int:
        return 1 + max(e.cache for e in self.order) if self.order else 0


def default_order(num_layers: int) -> Tuple[RunEntry, ...]:
    """Every layer once, in sequence, each with a cache of its own."""
    return tuple(RunEntry(layer=i, cache=i) for i in range(num_layers))
