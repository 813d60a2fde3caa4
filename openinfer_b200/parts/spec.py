"""Plain-data descriptions of a model's parts.

An architecture turns its config into a ``ModelSpec``: a list of ``BlockSpec``
(each naming its mixer, feed-forward and norms with all their sizes and
constants), the order in which the blocks run, and the embedding / final norm /
head. Parts are built from these specs through the registries in
``parts.registry``; a spec's ``kind`` is the registry key. Nothing here knows
which architecture produced it.
"""
from __future__ import annotations

import dataclasses
from typing import Any, List, Optional, Tuple, Union


@dataclasses.dataclass(frozen=True)
class ParamInfo:
    """One tensor a part wants from the checkpoint.

    ``init`` is how the random-weights mode draws it: ("normal", std),
    ("one_plus_normal", std) or ("normal_around", std, mean). ``integer`` tensors are kept as int32.
    """

    shape: Tuple[int, ...]
    init: Tuple = ("normal", 0.02)
    integer: bool = False
    free_dims: Tuple[int, ...] = ()   # dimensions whose size the checkpoint decides (``shape`` there: what random weights use)


@dataclasses.dataclass(frozen=True)
class NormSpec:
    kind: str = "rms"
    size: int = 0
    eps: float = 1e-6
    weight_offset: float = 0.0  # scale is (weight_offset + w)
    param_name: str = "weight"  # local tensor name (appended to the prefix the enclosing part gives the norm)
    # kind "dyt" (Dynamic Tanh: tanh(alpha x) w + b, no mean and no variance; eps is not used): the bias vector and the
    # scalar alpha are stored beside the weight under its name + these suffixes
    bias_suffix: str = ".b"
    alpha_suffix: str = ".alpha"


@dataclasses.dataclass(frozen=True)
class PositionSpec:
    """Position encoding applied to queries and keys inside a mixer."""

    kind: str = "rope"          # "rope" or "none"
    rotary_dim: int = 0         # leading dims of each head that rotate (<= head_dim, even)
    theta: float = 10000.0
    max_positions: int = 0
    interleaved: bool = False   # angle d turns the neighbours (2 d, 2 d + 1) instead of (d, d + rotary_dim / 2)
    # long waves stretched, (factor, low, high, original): a frequency f with wavelength l = 2 pi / f stays for
    # l < original / high, becomes f / factor for l > original / low, and in between (1 - s) f / factor + s f with
    # s = (original / l - low) / (high - low)
    scaling: Optional[Tuple[float, float, float, float]] = None
    precise: bool = False       # frequencies and angles in float64 (cos and sin rounded once); False: float32 throughout
    # another way to stretch the waves ("YaRN"), (factor, original, fast, slow): with turns(t) = rotary_dim ln(original /
    # (2 pi t)) / (2 ln theta), lo = max(floor(turns(fast)), 0), hi = min(ceil(turns(slow)), rotary_dim - 1) and
    # r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), frequency i becomes r_i f_i / factor + (1 - r_i) f_i, and cos and
    # sin are both multiplied by 0.1 ln(factor) + 1. Tables in float64, rounded once.
    yarn: Optional[Tuple[float, float, float, float]] = None


@dataclasses.dataclass(frozen=True)
class AttentionSpec:
    kind: str = "attention"
    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    softmax_scale: float = 0.0
    position: PositionSpec = PositionSpec(kind="none")
    qk_norm: Optional[NormSpec] = None      # per-head norm over head_dim, before the rotation
    window: Optional[int] = None            # keys visible to a query, itself included; None = all
    # queries / keys and values of other sizes than head_dim (None: head_dim). head_dim is then the cached row, a multiple
    # of 8 that holds both; the projections are padded with zero rows at load time and the norm's constants follow
    qk_dim: Optional[int] = None
    v_dim: Optional[int] = None
    q_name: str = "q_proj.weight"
    k_name: str = "k_proj.weight"
    v_name: str = "v_proj.weight"
    o_name: str = "o_proj.weight"
    q_norm_name: str = "q_norm.weight"
    k_norm_name: str = "k_norm.weight"
    # a short causal filter over time on every channel of q, k and v, directly behind the projections (no bias, no
    # activation): ``conv_taps`` taps, tensors q_name / k_name / v_name + ``conv_suffix`` of shape [channels, taps]; the last
    # taps - 1 projected rows of a request are state
    conv_taps: int = 0
    conv_suffix: str = ".conv"
    # the query at position p is multiplied by 1 + coef * ln(floor((p + 1) / every) + 1): (coef, every)
    q_temperature: Optional[Tuple[float, int]] = None
    score_cap: float = 0.0                  # > 0: score <- cap * tanh(score / cap)
    # > 0: head h (of H) takes 2^(-e (h + 1) / H) * (i - j) off the score of key j for query i, e this exponent
    distance_slope_exponent: float = 0.0
    sink: bool = False                      # a learned number per head in the softmax's denominator (``sink_name`` [heads])
    sink_name: str = "sink"
    head_gate: bool = False                 # head h's output is multiplied by sigmoid(W_g x)_h (``gate_name`` [heads, hidden])
    gate_name: str = "g"
    qkv_bias: bool = False                  # q, k and v have biases (tensor name + ``bias_suffix``), added in the projection
    bias_suffix: str = ".b"
    # > 0: AFTER the rotation q and k heads are divided by their root mean square over qk_dim numbers (no weight), with
    # this eps inside the root; takes the place of ``qk_norm``, which norms before the rotation
    unit_norm_after_rotation_eps: float = 0.0
    # with a window: the first ``keep_first`` keys of a sequence stay visible to every later query (at their true
    # positions), and their pages are never given back
    keep_first: int = 0


@dataclasses.dataclass(frozen=True)
class LatentAttentionSpec:
    """Attention over a low-rank latent: one vector c of ``latent_rank`` numbers per position is cached, and every head
    forms its keys and values from it (k = Wuk_h c, v = Wuv_h c). No position encoding."""

    kind: str = "latent_attention"
    hidden_size: int = 0
    num_heads: int = 0
    qk_dim: int = 0                         # per head: size of queries and keys
    v_dim: int = 0                          # per head: size of values
    latent_rank: int = 0
    softmax_scale: float = 0.0
    latent_norm: Optional[NormSpec] = None  # norm of the latent before it is cached and used
    window: Optional[int] = None            # keys visible to a query, itself included; None = all
    output_gate: bool = False               # head h's output is multiplied by sigmoid(Wg x)_h
    has_latent: bool = True                 # False: the layer reads the latent of an earlier layer and has no down-projection
    # how the per-head up-projections are applied: "weights" multiplies them into the query and output projections
    # once at load time; "runtime" applies them to the queries and to the attention's output in every step
    absorb: str = "weights"
    q_name: str = "q"
    down_name: str = "dkv"
    latent_norm_name: str = "dkv.norm"
    up_k_name: str = "uk"
    up_v_name: str = "uv"
    gate_name: str = "g"
    out_name: str = "o"
    # a rotated part beside the latent: every head's query has ``rope_dim`` more numbers behind its ``qk_dim`` unrotated
    # ones, the down-projection ``rope_dim`` more rows behind the latent's (one key part shared by all heads, not normed);
    # both are turned by ``position`` and their dot product is added to the score. The cached row is [latent, key part].
    rope_dim: int = 0
    position: Optional[PositionSpec] = None
    sink: bool = False                      # a learned number per head in the softmax's denominator (``sink_name`` [heads])
    sink_name: str = "sink"
    # "head": one gate per head (``gate_name`` [heads, hidden]); "element": one per output number ([heads * v_dim, hidden]),
    # which sits between the value up-projection and the output projection, so the values' up-projection runs in every step
    gate_per: str = "head"


@dataclasses.dataclass(frozen=True)
class DenseMlpSpec:
    """down( act(up x) ) with one up-projection. ``activation`` "xielu": the two shape numbers are a tensor."""

    kind: str = "dense_mlp"
    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "xielu"
    up_name: str = "up"
    down_name: str = "down"
    act_name: str = "act"


@dataclasses.dataclass(frozen=True)
class ShortConvSpec:
    """Causal convolution over time on each channel; the last ``taps - 1`` inputs are per-request state."""

    kind: str = "short_conv"
    channels: int = 0
    taps: int = 0
    add_input: bool = True                  # out = x + conv(x) rather than conv(x)
    param_name: str = ""


@dataclasses.dataclass(frozen=True)
class DepthAverageSpec:
    """After a layer, the stream becomes a weighted sum of the outputs of all layers so far (and of the embedding
    output): ``terms`` weights, one tensor."""

    kind: str = "depth_average"
    terms: int = 0
    param_name: str = ""


@dataclasses.dataclass(frozen=True)
class TokenInputSpec:
    """A per-layer input that depends on the token id alone: y = proj (gelu_tanh(gate x) * e) with e the ``dim`` numbers
    at ``offset`` of the token's row in a table shared by all layers (``table_name``, an absolute tensor name,
    [vocab_size, table_width]); the stream takes x + rms(y) * weight."""

    kind: str = "token_input"
    hidden_size: int = 0
    dim: int = 0
    offset: int = 0
    vocab_size: int = 0
    table_width: int = 0
    eps: float = 1e-6
    table_name: str = "/side.embed"          # a leading "/" makes a tensor name absolute (no block or part prefix)
    gate_name: str = "gate"
    proj_name: str = "proj"
    norm_name: str = "norm"


@dataclasses.dataclass(frozen=True)
class StreamCoefficientsSpec:
    """How one sublayer reads S residual streams and writes back to them (three small tensors)."""

    kind: str = "stream_coefficients"
    streams: int = 1
    in_name: str = "in"
    mix_name: str = "mix"
    out_name: str = "out"


@dataclasses.dataclass(frozen=True)
class GatedMlpSpec:
    kind: str = "gated_mlp"
    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "silu"
    limit: float = 0.0                      # of activations that clamp ("swiglu_clamp")
    gate_name: str = "gate_proj.weight"
    up_name: str = "up_proj.weight"
    down_name: str = "down_proj.weight"


@dataclasses.dataclass(frozen=True)
class RoutedExpertsSpec:
    """``experts`` gated feed-forwards of which every row uses the ``top`` with the largest router logits, weighted by
    the softmax over those logits. Tensors: ``router_name`` [experts, hidden] and per expert ``expert_prefix`` + index +
    "." + gate / up / down names."""

    kind: str = "routed_experts"
    hidden_size: int = 0
    intermediate_size: int = 0
    experts: int = 0
    top: int = 0
    activation: str = "swiglu_clamp"
    limit: float = 0.0
    router_name: str = "router"
    expert_prefix: str = "e"
    gate_name: str = "gate"
    up_name: str = "up"
    down_name: str = "down"
    # "softmax_top": the ``top`` largest router logits, weighted by their softmax. "table": no router; an integer tensor
    # ``table_name`` [vocab_size, top] gives every token id its experts, each weighted 1 / top. "sigmoid_groups": scores
    # s = sigmoid(logit); the choice goes by s + a stored correction (``correction_name`` [experts]) among the experts of
    # the ``keep_groups`` best of ``groups`` equal groups of neighbours (a group's score: the sum of its two largest choice
    # scores); the weights are the chosen experts' s divided by their sum
    routing: str = "softmax_top"
    correction_name: str = "correction"
    groups: int = 1
    keep_groups: int = 1
    table_name: str = "table"
    vocab_size: int = 0
    # an expert of the same form that every row uses, added to the routed sum (a GatedMlpSpec; tensors under ``shared_name``)
    shared: Any = None
    shared_name: str = "shared."


@dataclasses.dataclass(frozen=True)
class MatrixMemorySpec:
    """A recurrent mixer with a matrix C [qk_dim, v_dim], a normaliser n and a running maximum m per head (the mLSTM cell):
    exponential input gate and sigmoid forget gate in the log domain, both soft-capped at ``gate_cap``."""

    kind: str = "matrix_memory"
    hidden_size: int = 0
    num_heads: int = 0
    qk_dim: int = 0
    v_dim: int = 0
    gate_cap: float = 0.0
    eps: float = 1e-6                       # of the per-head unit norm of the read-out


@dataclasses.dataclass(frozen=True)
class GatedDeltaSpec:
    """A recurrent mixer with a matrix C [qk_dim, v_dim] per head updated by the delta rule, one decay per head and key
    channel; queries, keys and values pass a short causal filter over time and silu first. The decay and the output
    gate come through low-rank products whose inner sizes the checkpoint decides."""

    kind: str = "gated_delta"
    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    qk_dim: int = 0
    v_dim: int = 0
    conv_taps: int = 0
    eps: float = 1e-6
    decay_rank: int = 0                     # what random weights use; a checkpoint's own sizes win
    gate_rank: int = 0


@dataclasses.dataclass(frozen=True)
class LinearAttentionSpec:
    """Linear attention with one fixed decay per head ("lightning attention"): q, k (``qk_dim``) and v (``v_dim``) through
    silu; per head S <- decay_h S + k v^T, read-out S^T q with no other scale; the concatenated heads are RMS-normed together
    (weight ``norm_name`` [heads * v_dim]), multiplied by sigmoid(W_g x) and projected out. S is float32 state per request."""

    kind: str = "linear_attention"
    hidden_size: int = 0
    num_heads: int = 0
    qk_dim: int = 0
    v_dim: int = 0
    decays: Tuple[float, ...] = ()          # one per head
    eps: float = 1e-6
    q_name: str = "q"
    k_name: str = "k"
    v_name: str = "v"
    gate_name: str = "g"
    out_name: str = "o"
    norm_name: str = "norm"


@dataclasses.dataclass(frozen=True)
class ParallelMixerSpec:
    """Two mixers side by side that read the same input; the result is left_scale * left + right_scale * right."""

    kind: str = "parallel"
    left: Any = None
    right: Any = None
    left_scale: float = 1.0
    right_scale: float = 1.0
    left_name: str = "left."
    right_name: str = "right."


@dataclasses.dataclass(frozen=True)
class BlockSpec:
    """One layer: its parts and the tensor-name prefixes under which they live."""

    kind: str = "prenorm"
    name: str = ""                               # e.g. "model.layers.3."
    mixer: Any = None
    feed_forward: Any = None
    input_norm: Optional[NormSpec] = None
    post_norm: Optional[NormSpec] = None
    mixer_name: str = "self_attn."
    feed_forward_name: str = "mlp."
    input_norm_name: str = "input_layernorm."
    post_norm_name: str = "post_attention_layernorm."
    input_conv: Any = None                       # blocks that filter the mixer's input over time (ShortConvSpec)
    input_conv_name: str = "conv."
    depth_average: Any = None                    # blocks whose result is averaged with earlier layers' (DepthAverageSpec)
    depth_average_name: str = "depth."
    # blocks over several residual streams ("hyper"): how many, whether the layer has the three coefficient tensors per
    # sublayer, and their names
    streams: int = 1
    stream_coefficients: bool = False
    mixer_streams_name: str = "hc1."
    feed_forward_streams_name: str = "hc2."
    token_input: Any = None                      # blocks that end with a per-token input (TokenInputSpec)
    token_input_name: str = "side."
    # blocks that also norm their sublayers' OUTPUTS ("sandwich": x <- x + out_norm(f(in_norm(x)))): ``input_norm`` and
    # ``post_norm`` are the norms of the two inputs, these the norms of the two results
    mixer_out_norm: Optional[NormSpec] = None
    feed_forward_out_norm: Optional[NormSpec] = None
    mixer_out_norm_name: str = "norm1b"
    feed_forward_out_norm_name: str = "norm2b"


@dataclasses.dataclass(frozen=True)
class LayerCall:
    """One entry of the run order: which block runs, and whose cache it reads.

    ``read_cache_of`` is the index (in the order list) of an EARLIER call whose
    keys and values this call's mixer reads instead of writing its own.
    """

    layer: int
    read_cache_of: Optional[int] = None


@dataclasses.dataclass(frozen=True)
class ModelSpec:
    vocab_size: int
    hidden_size: int
    blocks: Tuple[BlockSpec, ...]
    order: Tuple[Union[int, LayerCall], ...]
    final_norm: NormSpec
    embedding_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm."
    head_name: Optional[str] = "lm_head.weight"   # None: the head is the embedding table (tied)
    max_positions: int = 0
    stop_token_ids: Tuple[int, ...] = ()
    embedding_scale: float = 1.0     # the embedded rows are multiplied by this (1: as stored, the reference's Qwen3)
    logit_soft_cap: float = 0.0      # > 0: logits = cap * tanh(logits / cap)
    logit_scale: float = 1.0         # the logits are multiplied by this
    residual_dtype: str = "model"    # "model": the stream between layers has the model's type; "float32": always 32-bit
    streams: int = 1                 # residual streams a row travels as ([tokens, streams, hidden]; blocks of kind "hyper")
    embedding_norm: Optional[NormSpec] = None     # a norm applied to the embedded rows before the first block
    embedding_init: Tuple = ("normal", 0.02)      # how random weights draw the embedding table
    embedding_norm_name: str = "embed.norm"

    def calls(self) -> List[LayerCall]:
        return [c if isinstance(c, LayerCall) else LayerCall(int(c)) for c in self.order]
