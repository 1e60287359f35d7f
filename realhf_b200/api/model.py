"""Model-side contracts: configs, Model / Engine / Backend / Interface ABCs and registries.

Parity: `realhf/api/core/model_api.py` (GenerationHyperparameters :25-94, ReaLMoEConfig :98-140,
ReaLModelConfig :144-264, ModelVersion, FinetuneSpec, PipelinableEngine :305-461, Model :465-510,
ModelBackend :513-545, ModelInterface :564-632, registries :635-738).
"""

from __future__ import annotations

import abc
import dataclasses
from typing import Any, Callable, Dict, List, Optional, Tuple, Union

import torch

from realhf_b200.api.config import (ModelAbstraction, ModelBackendAbstraction, ModelInterfaceAbstraction, ModelName,
                                    ModelWrapperAbstraction)
from realhf_b200.api.data import SequenceSample


@dataclasses.dataclass
class GenerationHyperparameters:
    max_new_tokens: int = 256
    min_new_tokens: int = 256
    greedy: bool = False
    top_p: float = 0.9
    top_k: int = 200
    temperature: float = 1.0
    use_cuda_graph: bool = False
    force_cudagraph_recapture: bool = True
    force_no_logits_mask: bool = False
    # B200 addition (no reference counterpart): decode with e4m3 weights / activations on the fp8 tensor cores.  Sampled
    # tokens and the returned log-probs are those of the quantised policy (see docs/generation_fp8.md).
    fp8_weights: bool = False

    def __post_init__(self):
        if self.temperature == 0.0:
            self.greedy, self.temperature = True, 1.0
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError("top_p must be in (0, 1]")
        if self.top_k <= 0:
            raise ValueError("top_k must be positive")
        if self.min_new_tokens > self.max_new_tokens:
            raise ValueError("min_new_tokens > max_new_tokens")


@dataclasses.dataclass
class ReaLMoEConfig:
    num_experts: int = 8
    top_k: int = 2
    routing_type: str = "aux_loss"  # aux_loss | sinkhorn | none
    aux_loss_coeff: float = 1e-3
    capacity_factor: Optional[float] = None
    pad_to_capacity: bool = False   # accepted for compatibility: dropped assignments get a zero routing weight and the grouped GEMM
                                    # takes device-side row offsets, so no expert batch needs padding to a static capacity
    token_drop_policy: str = "probs"  # probs | position
    z_loss_coeff: float = 0.0
    input_jitter_eps: float = 0.0
    use_grouped_gemm: bool = True
    expert_parallel: bool = False  # partition experts over the TP group (all-to-all dispatch); reference: not available
    # ---- routing variants of heterogeneous stacks (B200 addition).  routing_type "softmax_all": scores = softmax over ALL router
    # outputs; the top_k largest of (scores + `mlp.router.correction`, when `score_correction`) are chosen; the weights are the
    # chosen experts' scores, divided by their sum only with `renormalize`.
    score_correction: bool = False
    renormalize: bool = True
    identity_experts: int = 0      # the router has num_experts + identity_experts outputs; the last ones pass their input through
    shared_ff: Optional[int] = None  # a shared expert of this width runs for every token, times sigmoid(w_sg . x) (one number per token)
    # routing_type "sigmoid": scores = sigmoid(logit) of every router output on its own, the top_k largest are chosen and weigh.
    scale_input: bool = False      # the routing weight multiplies the expert's INPUT, expert(w x), instead of its output
    shared_gate: bool = True       # False: the shared expert's output is added as it is (no `mlp.shared.sg.weight`)
    shared_limit: Optional[float] = None  # clamp limit of the shared expert when the experts are clamped units (None: the experts' own)

    @property
    def n_router_outputs(self) -> int:
        return self.num_experts + self.identity_experts


@dataclasses.dataclass
class RotaryConfig:
    """Rotation of the pairs (2i, 2i + 1) (`interleaved`) of the first `dims` dimensions of a vector by the angle pos * f_i,
    f_i = base^(-2i / dims).  With `factor` (YaRN rescaling of a model trained on `original` positions): with
    dim(t) = dims ln(original / (2 pi t)) / (2 ln base), lo = max(floor(dim(fast)), 0), hi = min(ceil(dim(slow)), dims - 1) and
    ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1) the frequency becomes f_i / factor * ramp_i + f_i (1 - ramp_i), and cos and
    sin are multiplied by 0.1 ln(factor) + 1."""
    dims: int
    base: float = 10000.0
    interleaved: bool = True
    factor: Optional[float] = None
    original: int = 0
    fast: float = 32.0
    slow: float = 1.0

    def frequencies(self) -> Tuple[List[float], float]:
        """(f_i for i < dims / 2 in double precision, the factor on cos and sin)."""
        import math
        n = self.dims // 2
        f = [self.base ** (-2.0 * i / self.dims) for i in range(n)]
        if self.factor is None:
            return f, 1.0

        def dim_of(turns: float) -> float:
            return self.dims * math.log(self.original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))
        lo = max(math.floor(dim_of(self.fast)), 0)
        hi = min(math.ceil(dim_of(self.slow)), self.dims - 1)
        out = []
        for i in range(n):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            out.append(f[i] / self.factor * ramp + f[i] * (1.0 - ramp))
        return out, 0.1 * math.log(self.factor) + 1.0


@dataclasses.dataclass
class LatentAttentionConfig:
    """Attention whose keys and values are up-projections of one shared low-rank latent per token (only the latent is cached).
    `window`: a query at position i sees positions (i - window, i]; None = the whole prefix.
    `kv_from`: 0-based index of an EARLIER block whose cached latent this block reads instead of projecting its own.
    Further mechanisms, each a switch or a size:
      * `rot_dim` > 0: every head's query / key gets `rot_dim` more dimensions that carry the position (`rotary`); the key part is
        ONE vector per token shared by all heads, the last `rot_dim` outputs of the down-projection, cached beside the latent
        (a cache row is [latent | rotated key part]).  `qk_dim` counts the unrotated dimensions only; `scale` multiplies the
        whole score;
      * `q_rank`: queries are the up-projection of an RMS-normalised latent of this rank (None: one projection);
      * `sink`: a learned per-head logit in the softmax denominator (no key, no value);
      * `out_gate`: the concatenated heads are multiplied element by element by sigmoid(W_g x), x the mixer's input."""
    n_heads: int
    qk_dim: int
    v_dim: int
    kv_rank: int
    scale: float
    window: Optional[int] = None
    kv_from: Optional[int] = None
    rot_dim: int = 0
    rotary: Optional[RotaryConfig] = None
    q_rank: Optional[int] = None
    sink: bool = False
    out_gate: bool = False

    def __post_init__(self):
        if isinstance(self.rotary, dict):
            self.rotary = RotaryConfig(**self.rotary)
        if self.rot_dim:
            if self.rotary is None or self.rotary.dims != self.rot_dim or self.rot_dim % 2 or not self.rotary.interleaved:
                raise ValueError("rot_dim > 0 needs an interleaved `rotary` over exactly rot_dim (even) dimensions")
            if self.kv_from is not None or self.window is not None:
                raise ValueError("the rotated form has its own latent and no window")

    @property
    def rotated(self) -> bool:
        """The mixer of `models.hetero_block._latent_rope_*` (any of rot_dim / q_rank / sink / out_gate set)."""
        return bool(self.rot_dim or self.q_rank or self.sink or self.out_gate)

    @property
    def cache_width(self) -> int:
        return self.kv_rank + self.rot_dim


@dataclasses.dataclass
class WindowAttentionConfig:
    """Softmax attention over cached keys / values with grouped key / value heads (query head h reads head h // (n_heads /
    n_kv_heads)).  Every further mechanism is a switch or a constant, so that families can combine them:

      * `rotary`: queries and keys are rotated by their position over the first `rotary.dims` dimensions of every head (pairs
        (2i, 2i + 1) when `rotary.interleaved`, else (i, i + dims / 2)); keys are cached rotated.  None: no rotation;

      * `window` / `keep_first`: query i sees key j <= i when i - j < window or j < keep_first (window None: all j <= i).  The
        cache of a sequence is then `keep_first` fixed rows plus a ring of `window` rows, whatever the sequence's length;
      * `value_norm`: every head's value is divided by its root mean square (no weight) before it is cached;
      * `head_temp`: a learned per-head factor on the scaled score;
      * `slope_base` b: the score loses slope_h * (i - j), slope_h = 2^(-b (h + 1) / n_heads) (None: no distance term);
      * `sink`: a learned per-head logit added to the softmax denominator as exp(sink_h): a key-less, value-less entry;
      * `out_gate`: head h's output is multiplied by sigmoid(w_g . x)_h, x being the mixer's input;
      * `qk_norm`: every query / key head is RMS-normalised over qk_dim with a weight (one for queries, one for keys);
      * `n_maps` = 2: differential attention.  Queries and keys have two maps per head ([map 1 | map 2], 2 qk_dim wide), each a
        softmax attention of its own over the same values; with lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + `diff` (learned vectors
        of size qk_dim, one number per layer) head h's output is o = a1 - lambda a2, then o / sqrt(mean(o^2) + eps) * (1 - diff)."""
    n_heads: int
    n_kv_heads: int
    qk_dim: int
    v_dim: int
    scale: float
    window: Optional[int] = None
    keep_first: int = 0
    qkv_bias: bool = True
    value_norm: bool = True
    head_temp: bool = True
    slope_base: Optional[float] = 8.0
    sink: bool = True
    out_gate: bool = True
    qk_norm: bool = False
    n_maps: int = 1
    diff: float = 0.0
    rotary: Optional[RotaryConfig] = None

    def __post_init__(self):
        if isinstance(self.rotary, dict):
            self.rotary = RotaryConfig(**self.rotary)
        if self.rotary is not None and (self.rotary.dims % 2 or not 0 < self.rotary.dims <= self.qk_dim or self.n_maps != 1):
            raise ValueError("rotary.dims: even, at most qk_dim, one score map")
        if self.n_heads % self.n_kv_heads:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        if self.n_maps not in (1, 2):
            raise ValueError("n_maps: 1 (plain) or 2 (differential)")
        if self.n_maps == 2 and (self.out_gate or self.sink or self.head_temp or self.slope_base is not None or self.value_norm or self.qkv_bias):
            raise ValueError("differential attention combines with qk_norm and the window only")
        if self.window is None:
            self.keep_first = 0
        elif self.window < 1 or self.keep_first < 0:
            raise ValueError("window >= 1 and keep_first >= 0 expected")

    def cache_rows(self, max_len: int) -> int:
        """Rows a sequence of at most max_len tokens needs: position p lives in row p when p < keep_first, else in row
        keep_first + (p - keep_first) % (rows - keep_first)."""
        return max_len if self.window is None else max(1, min(max_len, self.keep_first + self.window))


@dataclasses.dataclass
class DeltaRuleConfig:
    """Gated delta-rule mixer: a per-head matrix state S [qk_dim, v_dim] (fp32), updated per token by
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q,  with a scalar decay g in (0, 1) and a write strength beta in
    (0, 1) per head and token.  q / k have `n_kv_heads` heads (head h reads q / k head h // (n_heads / n_kv_heads)), pass a causal
    depthwise convolution of `conv_taps` taps and SiLU (so does v), and are scaled to unit length; o is RMS-normalised per head
    and gated by SiLU of a projection.  A sequence's decode state is S plus the last conv_taps - 1 projection outputs."""
    n_heads: int
    n_kv_heads: int
    qk_dim: int
    v_dim: int
    conv_taps: int
    unit_eps: float = 1e-6         # q, k <- x / sqrt(sum(x^2) + unit_eps)

    def __post_init__(self):
        if self.n_heads % self.n_kv_heads:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        if self.conv_taps < 1:
            raise ValueError("conv_taps >= 1 expected (1 = the current token only)")

    @property
    def conv_channels(self) -> int:
        return 2 * self.n_kv_heads * self.qk_dim + self.n_heads * self.v_dim


@dataclasses.dataclass
class MLSTMConfig:
    """Matrix-memory LSTM mixer: per head a matrix state S [qk_dim, v_dim], a normaliser n [qk_dim] and a running maximum m (from
    0) of the log gates, all fp32.  With i = cap tanh((w_i . x + b_i) / cap), f = logsigmoid(cap tanh((w_f . x + b_f) / cap)):
    m' = max(f + m, i);  S <- exp(f + m - m') S + exp(i - m') k v^T;  n likewise with k;  o = S^T q / (max(|n . q|, exp(-m')) + 1e-6),
    q scaled by qk_dim^(-1/2).  Each head's o is divided by its root mean square, the concatenation multiplied by a weight and by
    sigmoid(W_g x)."""
    n_heads: int
    qk_dim: int
    v_dim: int
    gate_cap: float = 15.0


@dataclasses.dataclass
class DecayConfig:
    """Linear attention with a fixed decay per head (retention, lightning attention): per head a matrix state S [qk_dim, v_dim]
    (fp32, from zero), S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; no softmax, no denominator.  Switches:

      * `act`: "silu" puts SiLU on the projected q, k and v; "none" leaves them;
      * `rotary`: q and k are rotated by the position (fp32) over the first `rotary.dims` dimensions of every head, in the half
        layout (i, i + dims / 2) or the interleaved one;
      * `k_scale`: a factor on k (after the rotation), e.g. qk_dim^(-1/2);
      * `out_norm`: "head": every head's o is divided by its root mean square (no weight); "full": the concatenated heads are
        RMS-normalised together, times a weight [n_heads * v_dim];
      * `gate`: the normalised output is multiplied by silu(W_g x) ("silu") or sigmoid(W_g x) ("sigmoid"), x the mixer's input.
    The projection row is [q (H d) | k (H d) | v (H dv) | gate (H dv)]."""
    n_heads: int
    qk_dim: int
    v_dim: int
    decay: List[float]
    act: str = "none"              # none | silu
    rotary: Optional[RotaryConfig] = None
    k_scale: float = 1.0
    out_norm: str = "head"         # head | full
    gate: str = "silu"             # silu | sigmoid

    def __post_init__(self):
        if isinstance(self.rotary, dict):
            self.rotary = RotaryConfig(**self.rotary)
        self.decay = [float(g) for g in self.decay]
        if len(self.decay) != self.n_heads:
            raise ValueError("`decay` needs one value per head")
        if self.act not in ("none", "silu") or self.out_norm not in ("head", "full") or self.gate not in ("silu", "sigmoid"):
            raise ValueError("act: none | silu; out_norm: head | full; gate: silu | sigmoid")
        if self.rotary is not None and (self.rotary.dims % 2 or not 0 < self.rotary.dims <= self.qk_dim):
            raise ValueError("rotary.dims: even and at most qk_dim")

    @property
    def width(self) -> int:
        """Columns of the projection row."""
        return 2 * self.n_heads * (self.qk_dim + self.v_dim)


@dataclasses.dataclass
class LoopConfig:
    """Blocks start .. stop - 1 (0-based) run `times` times in a row with the same weights, every pass with a cache / state of its
    own.  With `inject`, the embedding output x0 is mixed back in at the start of a pass: mode "linear": every pass,
    x <- W_in [x; x0], W_in [hidden, 2 hidden]; mode "add": every pass but the first, x <- x + x0."""
    start: int
    stop: int
    times: int
    inject: bool = True
    inject_mode: str = "linear"    # linear | add


@dataclasses.dataclass
class BlockMLPConfig:
    """Feed-forward of one block of a heterogeneous stack.  kind `clamped_glu`: y = g * sigmoid(alpha g) * (u + 1) with
    g = min(gate, limit), u = clamp(up, -limit, limit); kind `moe`: `moe.num_experts` SiLU-gated experts of width `ff`, the
    `moe.top_k` largest router logits (with a router bias) are chosen and weighted by the softmax over the chosen logits;
    kind `relu2`: down(relu(up(x))^2), no gate; kind `glu`: down(act(gate(x)) * up(x)) with `act` silu or gelu_tanh.  The experts
    of kind `moe` are SiLU-gated units of width `ff`, or, with `limit` > 0, clamped units (the `clamped_glu` form with `limit` and
    `alpha`); routing variants are fields of `moe`."""
    kind: str                      # clamped_glu | moe | relu2 | glu
    ff: int
    limit: float = 0.0
    alpha: float = 1.702
    moe: Optional[ReaLMoEConfig] = None
    act: str = "silu"


@dataclasses.dataclass
class BlockConfig:
    """One entry of `ReaLModelConfig.blocks` (a stack whose blocks differ from each other)."""
    mixer: str                     # latent_attention | window_attention | delta | mlstm | decay | parallel
    attn: Optional[LatentAttentionConfig] = None
    mlp: Optional[BlockMLPConfig] = None   # None: the block has no feed-forward sublayer
    wattn: Optional[WindowAttentionConfig] = None
    delta: Optional[DeltaRuleConfig] = None
    mlstm: Optional[MLSTMConfig] = None
    decay: Optional[DecayConfig] = None
    # mixer "parallel": `wattn` and `decay` read the same input side by side; the result is branch_scales[0] * window attention +
    # branch_scales[1] * decayed linear attention (each after its own output projection)
    branch_scales: Tuple[float, float] = (1.0, 1.0)

    def __post_init__(self):
        if isinstance(self.attn, dict):
            self.attn = LatentAttentionConfig(**self.attn)
        if isinstance(self.wattn, dict):
            self.wattn = WindowAttentionConfig(**self.wattn)
        if isinstance(self.delta, dict):
            self.delta = DeltaRuleConfig(**self.delta)
        if isinstance(self.mlstm, dict):
            self.mlstm = MLSTMConfig(**self.mlstm)
        if isinstance(self.decay, dict):
            self.decay = DecayConfig(**self.decay)
        self.branch_scales = (float(self.branch_scales[0]), float(self.branch_scales[1]))
        want = {"latent_attention": self.attn, "window_attention": self.wattn, "delta": self.delta, "mlstm": self.mlstm, "decay": self.decay,
                "parallel": self.wattn if self.decay is not None else None}
        if self.mixer not in want:
            raise ValueError(f"unknown mixer `{self.mixer}`")
        if want[self.mixer] is None:
            raise ValueError(f"a `{self.mixer}` block needs its mixer config")
        if isinstance(self.mlp, dict):
            self.mlp = BlockMLPConfig(**self.mlp)
        if self.mlp is not None and isinstance(self.mlp.moe, dict):
            self.mlp.moe = ReaLMoEConfig(**self.mlp.moe)


@dataclasses.dataclass
class ReaLModelConfig:
    n_layers: int
    n_kv_heads: int
    n_q_heads: int
    hidden_dim: int
    intermediate_dim: int
    vocab_size: int
    head_dim: Optional[int] = None
    n_positions: Optional[int] = None
    embd_pdrop: float = 0.1
    resid_pdrop: float = 0.1
    attn_pdrop: float = 0.1
    layer_norm_epsilon: float = 1e-5
    activation_function: str = "gelu"
    scale_attn_by_inverse_layer_idx: bool = True
    scale_attn_weights: bool = True
    use_attention_bias: bool = True
    use_attn_proj_bias: bool = True
    use_mlp_bias: bool = True
    layer_norm_type: Optional[str] = None  # None (LayerNorm) | "rms" | "gemma" | "layer" (heterogeneous stacks: LayerNorm, no bias)
    mlp_type: Optional[str] = None  # None (plain MLP) | "llama" | "moe"
    apply_rotary: bool = False
    rotary_base: float = 10000.0
    rotary_interleaved: bool = False
    rotary_scaling: Optional[float] = None
    rotary_scaling_type: Optional[str] = None
    normalize_embed: bool = False
    abs_position_embedding_offset: int = 0
    do_layernorm_before: bool = True
    tied_embedding: bool = False
    sliding_window: Optional[int] = None
    moe: Optional[ReaLMoEConfig] = None
    is_critic: bool = False
    # ---- heterogeneous stacks (B200 addition, no reference counterpart): `blocks[i]` describes block i + 1; the homogeneous fields
    # above (heads, intermediate_dim, mlp_type, ...) are then only summaries.  The remaining fields are mechanisms any family may use.
    blocks: Optional[List[BlockConfig]] = None
    norm_groups: int = 1                 # RMSNorm in `norm_groups` equal consecutive parts, each with its own root mean square
    sandwich_norm: bool = False          # a second norm on every sublayer's OUTPUT, before the residual add
    conv_taps: int = 0                   # h <- h + causal depthwise conv(h) over time on every sublayer's input (0 = none);
                                         # the last conv_taps - 1 inputs are part of a sequence's decode state
    logit_softcap: Optional[float] = None  # logits <- cap * tanh(logits / cap)
    fp32_residual: bool = False          # the residual stream is kept in fp32 whatever the compute dtype
    sinusoidal_positions: bool = False   # x <- embed + pe(p), pe[2i] = sin(p base^(-2i/H)), pe[2i+1] = cos(same), angles in fp32
    sinusoid_base: float = 10000.0
    logit_scale: Optional[float] = None  # logits <- logits * logit_scale (fp32)
    loop: Optional[LoopConfig] = None    # a range of blocks that runs several times (heterogeneous stacks only)
    embed_scale: Optional[float] = None  # the embedding output is multiplied by this constant
    residual_mult: float = 1.0           # x <- x + residual_mult * branch ("layer" stacks)
    layer_scale: bool = False            # every branch output (after its output norm) times a learned vector (`attn.ls.weight`,
                                         # `mlp.ls.weight`) before it joins the stream ("layer" stacks)

    def layer_runs(self) -> List[Tuple[int, bool]]:
        """(1-based block index, the run starts a pass of the loop) for every block run, in execution order."""
        L, lp = self.n_layers, self.loop
        if lp is None:
            return [(i, False) for i in range(1, L + 1)]
        runs = [(i + 1, False) for i in range(lp.start)]
        for p in range(lp.times):
            runs += [(i + 1, i == lp.start and (p > 0 or lp.inject_mode == "linear")) for i in range(lp.start, lp.stop)]
        return runs + [(i + 1, False) for i in range(lp.stop, L)]

    def __post_init__(self):
        if isinstance(self.loop, dict):
            self.loop = LoopConfig(**self.loop)
        if self.loop is not None:
            if self.blocks is None:
                raise ValueError("`loop` needs a heterogeneous stack (`blocks`)")
            if not (0 <= self.loop.start < self.loop.stop <= self.n_layers and self.loop.times >= 1):
                raise ValueError("loop: 0 <= start < stop <= n_layers and times >= 1 expected")
            if self.loop.inject_mode not in ("linear", "add"):
                raise ValueError("loop.inject_mode: linear | add")
        if self.is_critic and self.tied_embedding:
            raise ValueError("a critic cannot tie its embedding and output weights")
        if self.blocks is not None:
            self.blocks = [BlockConfig(**b) if isinstance(b, dict) else b for b in self.blocks]
            if len(self.blocks) != self.n_layers:
                raise ValueError("`blocks` must describe every layer")
            if self.layer_norm_type == "layer" and (self.norm_groups != 1 or self.conv_taps or not self.sandwich_norm):
                raise ValueError("\"layer\" stacks: one norm group, no convolution, norms on both sides of every sublayer")
            if self.layer_norm_type != "layer" and (self.layer_scale or self.residual_mult != 1.0
                                                    or any(b.mixer in ("decay", "parallel") for b in self.blocks)):
                raise ValueError("layer_scale, residual_mult and the decay / parallel mixers live in \"layer\" stacks")
            for i, b in enumerate(self.blocks):
                if b.mixer != "latent_attention":
                    continue
                if b.attn.rotated and (self.norm_groups != 1 or self.sandwich_norm or self.conv_taps):
                    raise ValueError("rotated latent attention lives in plain pre-norm stacks")
                src = b.attn.kv_from
                if src is not None and not (0 <= src < i and self.blocks[src].attn.kv_from is None
                                            and self.blocks[src].attn.kv_rank == b.attn.kv_rank):
                    raise ValueError(f"block {i}: kv_from must name an earlier block that projects a latent of the same rank")
        if self.head_dim is None:
            self.head_dim = self.hidden_dim // self.n_q_heads
        if isinstance(self.moe, dict):
            self.moe = ReaLMoEConfig(**self.moe)

    def n_params(self) -> int:
        """Parameter count (used by the PP partitioner, the FLOP model and the allocation search)."""
        h, f, v = self.hidden_dim, self.intermediate_dim, self.vocab_size
        if self.blocks is not None:
            n = 2 * v * h + h
            norms = (2 if self.sandwich_norm else 1) + self.conv_taps + int(self.layer_scale)   # per sublayer: norm(s), taps, scale
            for b in self.blocks:
                if b.mixer in ("decay", "parallel"):
                    a = b.decay
                    n += h * a.width + a.n_heads * a.v_dim * (h + (1 if a.out_norm == "full" else 0)) + norms * h
                    if b.mixer == "parallel":
                        w = b.wattn
                        n += h * (w.n_heads * w.qk_dim + w.n_kv_heads * (w.qk_dim + w.v_dim)) + w.n_heads * w.v_dim * h
                elif b.mixer == "window_attention":
                    a = b.wattn
                    qkv = a.n_heads * a.qk_dim + a.n_kv_heads * (a.qk_dim + a.v_dim)
                    qkv += (a.n_maps - 1) * (a.n_heads + a.n_kv_heads) * a.qk_dim
                    n += h * (qkv + (a.n_heads if a.out_gate else 0)) + (qkv if a.qkv_bias else 0) + a.n_heads * a.v_dim * h
                    n += a.n_heads * (int(a.head_temp) + int(a.sink)) + norms * h
                    n += (2 * a.qk_dim if a.qk_norm else 0) + (4 * a.qk_dim if a.n_maps == 2 else 0)
                elif b.mixer == "delta":
                    a = b.delta
                    n += h * (2 * a.n_kv_heads * a.qk_dim + 2 * a.n_heads * a.v_dim + 2 * a.n_heads) + a.n_heads * a.v_dim * h
                    n += a.conv_channels * a.conv_taps + 2 * a.n_heads + a.v_dim + norms * h
                elif b.mixer == "mlstm":
                    a = b.mlstm
                    n += h * (2 * a.n_heads * a.qk_dim + 2 * a.n_heads * a.v_dim + 2 * a.n_heads) + 2 * a.n_heads
                    n += a.n_heads * a.v_dim * (h + 1) + norms * h
                elif b.attn.rotated:
                    a = b.attn
                    dq = a.qk_dim + a.rot_dim
                    n += (h * a.q_rank + a.q_rank + a.q_rank * a.n_heads * dq) if a.q_rank else h * a.n_heads * dq
                    n += h * a.cache_width + a.kv_rank + a.kv_rank * a.n_heads * (a.qk_dim + a.v_dim) + a.n_heads * a.v_dim * h
                    n += (a.n_heads if a.sink else 0) + (h * a.n_heads * a.v_dim if a.out_gate else 0) + norms * h
                else:
                    a = b.attn
                    n += h * a.n_heads * a.qk_dim + (h * a.kv_rank + a.kv_rank if a.kv_from is None else 0)
                    n += a.kv_rank * a.n_heads * (a.qk_dim + a.v_dim) + a.n_heads * a.v_dim * h + norms * h
                if b.mlp is not None:
                    e = b.mlp.moe.num_experts if b.mlp.kind == "moe" else 1
                    mats = 2 if b.mlp.kind == "relu2" else 3
                    n += e * mats * h * b.mlp.ff + norms * h
                    if b.mlp.kind == "moe":
                        mo = b.mlp.moe
                        if mo.routing_type in ("softmax_all", "sigmoid"):
                            n += mo.n_router_outputs * (h + (1 if mo.score_correction else 0))
                            n += (3 * h * mo.shared_ff + (h if mo.shared_gate else 0)) if mo.shared_ff else 0
                        else:
                            n += e * (h + 1)
            if self.loop is not None and self.loop.inject and self.loop.inject_mode == "linear":
                n += 2 * h * h
            return n
        qkv = h * self.head_dim * (self.n_q_heads + 2 * self.n_kv_heads)
        attn = qkv + self.n_q_heads * self.head_dim * h
        if self.mlp_type == "moe":
            mlp = self.moe.num_experts * 3 * h * f + h * self.moe.num_experts
        elif self.mlp_type == "llama":
            mlp = 3 * h * f
        else:
            mlp = 2 * h * f
        emb = v * h + (self.n_positions * h if (not self.apply_rotary and self.n_positions) else 0)
        head = h if self.is_critic else (0 if self.tied_embedding else v * h)
        return self.n_layers * (attn + mlp + 2 * h) + emb + head + h


@dataclasses.dataclass
class ModelVersion:
    epoch: int = 0
    epoch_step: int = 0
    global_step: int = 0


@dataclasses.dataclass
class FinetuneSpec:
    total_train_epochs: int
    total_train_steps: int
    steps_per_epoch: int


class PipelinableEngine(abc.ABC):
    """What an interface drives: the same four calls regardless of the (dp,tp,pp) layout behind them."""

    def train_batch(self, input_: SequenceSample, loss_fn: Callable, version_steps: int,
                    num_micro_batches: Optional[int] = None) -> Dict[str, Any]:
        raise NotImplementedError()

    def eval_batch(self, input_: SequenceSample, loss_fn: Callable, num_micro_batches: Optional[int] = None):
        raise NotImplementedError()

    def forward(self, input_: SequenceSample, num_micro_batches: Optional[int] = None,
                post_hook: Optional[Callable] = None, aggregate_fn: Callable = torch.cat):
        raise NotImplementedError()

    def generate(self, input_: SequenceSample, tokenizer, gconfig: GenerationHyperparameters = None,
                 num_micro_batches: Optional[int] = None):
        raise NotImplementedError()


@dataclasses.dataclass
class Model:
    """A model shard plus what travels with it (tokenizer, device, version counter, backend name)."""

    name: ModelName
    module: Any
    tokenizer: Any
    device: Union[str, torch.device]
    dtype: Optional[torch.dtype] = None
    version: ModelVersion = dataclasses.field(default_factory=ModelVersion)
    ft_spec: Optional[FinetuneSpec] = None
    backend_name: Optional[str] = None
    module_config: Optional[ReaLModelConfig] = None
    hf_family: Optional[str] = None

    def __post_init__(self):
        try:
            self.module = self.module.to(self.device)
        except (ValueError, AttributeError, NotImplementedError):
            pass

    def inc_version(self):
        self.version.global_step += 1
        self.version.epoch_step += 1
        if self.ft_spec and self.version.epoch_step >= self.ft_spec.steps_per_epoch:
            self.version.epoch += 1
            self.version.epoch_step = 0


class ModelBackend(abc.ABC):
    """Wraps `model.module` into a PipelinableEngine (optimizer, sharding, schedules)."""

    @abc.abstractmethod
    def _initialize(self, model: Model, spec: FinetuneSpec) -> Model:
        ...

    def initialize(self, model: Model, spec: FinetuneSpec) -> Model:
        model.ft_spec = spec
        return self._initialize(model, spec)

    def destroy(self, model: Model):
        pass

    def save(self, model: Model, save_dir: str):
        """Optimizer / scheduler state (the reference saves none; we do for `recover`)."""

    def load(self, model: Model, load_dir: str):
        pass


class NullBackend(ModelBackend):
    def _initialize(self, model, spec):
        return model


def null_model(name: ModelName, device) -> Model:
    return Model(name, torch.nn.Identity(), None, device)


def tokenizer_only_model(name: ModelName, device, tokenizer_path: str) -> Model:
    from realhf_b200.api.data import load_hf_tokenizer
    return Model(name, torch.nn.Identity(), load_hf_tokenizer(tokenizer_path), device)


class ModelInterface(abc.ABC):
    """An algorithm's view of a model: what `generate / inference / train_step` mean for it."""

    def save(self, model: Model, save_dir: str):
        pass

    def state_dict(self) -> Dict:
        """Algorithm state that lives outside the model (KL controller, value normaliser, ...): written with the recover
        states and restored on a recover run.  (The reference loses this state on recovery)"""
        return {}

    def load_state_dict(self, sd: Dict):
        pass

    def evaluate(self, model: Model, eval_dataloader) -> Dict:
        return {}

    def inference(self, model: Model, data: SequenceSample, n_mbs: Optional[int] = None) -> Optional[SequenceSample]:
        raise NotImplementedError()

    def generate(self, model: Model, data: SequenceSample, n_mbs: Optional[int] = None) -> Optional[SequenceSample]:
        raise NotImplementedError()

    def train_step(self, model: Model, data: SequenceSample, n_mbs: Optional[int] = None) -> Dict:
        raise NotImplementedError()

    # used by the profiler to fabricate inputs of the right shape
    def _mock_generate(self, model: Model, data: SequenceSample):
        return data

    def _mock_inference(self, model: Model, data: SequenceSample):
        return data

    def _mock_train_step(self, model: Model, data: SequenceSample):
        return data

    def mock(self, type_: str, model: Model, data: SequenceSample) -> SequenceSample:
        return getattr(self, f"_mock_{type_}")(model, data)


class NullInterface(ModelInterface):
    def inference(self, model, data, n_mbs=None):
        scores = torch.zeros(data.bs, dtype=torch.float32, device=model.device)
        return SequenceSample.from_default(seqlens=[1] * data.bs, ids=data.ids, data={"rewards": scores})

    def train_step(self, model, data, n_mbs=None):
        model.inc_version()
        return {}

    def save(self, model, save_dir):
        pass


ALL_MODEL_CLASSES: Dict[str, Callable] = {}
ALL_INTERFACE_CLASSES: Dict[str, Callable] = {}
ALL_BACKEND_CLASSES: Dict[str, Callable] = {}
ALL_WRAPPER_CLASSES: Dict[str, Callable] = {}
SUPPORTED_HF_FAMILIES: Dict[str, "HFFamilySpec"] = {}


def register_model(name: str, fn):
    if name in ALL_MODEL_CLASSES:
        raise KeyError(f"model `{name}` already registered")
    ALL_MODEL_CLASSES[name] = fn


def register_interface(name: str, cls):
    if name in ALL_INTERFACE_CLASSES:
        raise KeyError(f"interface `{name}` already registered")
    ALL_INTERFACE_CLASSES[name] = cls


def register_backend(name: str, cls):
    if name in ALL_BACKEND_CLASSES:
        raise KeyError(f"backend `{name}` already registered")
    ALL_BACKEND_CLASSES[name] = cls


def register_wrapper(name: str, cls):
    ALL_WRAPPER_CLASSES[name] = cls


def make_model_wrapper(cfg: ModelWrapperAbstraction) -> Callable[[Model], Model]:
    return ALL_WRAPPER_CLASSES[cfg.type_](**cfg.args)


def make_model(cfg: ModelAbstraction, name: ModelName, device) -> Model:
    model = ALL_MODEL_CLASSES[cfg.type_](**cfg.args, name=name, device=device)
    for w in cfg.wrappers:
        model = make_model_wrapper(w)(model)
    return model


def make_interface(cfg: ModelInterfaceAbstraction) -> ModelInterface:
    return ALL_INTERFACE_CLASSES[cfg.type_](**cfg.args)


def make_backend(cfg: ModelBackendAbstraction) -> ModelBackend:
    return ALL_BACKEND_CLASSES[cfg.type_](**cfg.args)


register_backend("null", NullBackend)
register_model("null", null_model)
register_model("tokenizer", tokenizer_only_model)
register_interface("null", NullInterface)


@dataclasses.dataclass
class HFFamilySpec:
    """How one HuggingFace family maps to ReaLModelConfig and parameter names (api/from_hf/*)."""

    name: str
    hf_cls_name: str
    config_from_hf: Callable[[Any, bool], ReaLModelConfig]
    config_to_hf: Callable[[ReaLModelConfig], Any]
    sd_from_hf: Callable[[Dict[str, torch.Tensor], ReaLModelConfig], Dict[str, torch.Tensor]]
    sd_to_hf: Callable[[Dict[str, torch.Tensor], ReaLModelConfig], Dict[str, torch.Tensor]]
    embedding_param_names: Callable[[ReaLModelConfig], List[str]]
    tblock_param_names: Callable[[ReaLModelConfig, int], List[str]]
    head_param_names: Callable[[ReaLModelConfig], List[str]]
    make_test_config: Optional[Callable[[], ReaLModelConfig]] = None
    real_config_maker: Optional[Callable] = None
    # families without a `transformers` class: `config.json` is read and written as a plain dict, and all weights live in one file
    config_from_dict: Optional[Callable[[dict, bool], ReaLModelConfig]] = None
    config_to_dict: Optional[Callable[[ReaLModelConfig], dict]] = None
    weight_file: Optional[str] = None


def register_hf_family(name: str, hf_cls_name: str, config_from_hf_converter, config_to_hf_converter,
                       sd_from_hf_converter, sd_to_hf_converter, embedding_param_names, tblock_param_names,
                       head_param_names, real_config_maker=None, make_test_config=None, config_from_dict=None, config_to_dict=None,
                       weight_file=None):
    if name in SUPPORTED_HF_FAMILIES:
        raise KeyError(f"HF family `{name}` already registered")
    SUPPORTED_HF_FAMILIES[name] = HFFamilySpec(name, hf_cls_name, config_from_hf_converter, config_to_hf_converter,
                                               sd_from_hf_converter, sd_to_hf_converter, embedding_param_names,
                                               tblock_param_names, head_param_names, make_test_config,
                                               real_config_maker, config_from_dict, config_to_dict, weight_file)
