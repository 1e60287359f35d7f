"""Blocks of a heterogeneous stack (`ReaLModelConfig.blocks`): packed (prefill / inference) and one-token (decode) forms.

A block is  x <- x + post_norm(mixer(conv(norm(x))));  x <- x + post_norm(ff(conv(norm(x))))  on a residual stream that stays
fp32 when `fp32_residual` is set (post_norm and conv are optional: `sandwich_norm`, `conv_taps`).  `ReaLModel.forward` /
`ReaLModel.decode_step` own the loop over block RUNS (`ReaLModelConfig.layer_runs`: a block inside `config.loop` runs several times,
each run with its own state), the embedding and the head; `models.generation.DecodeState` owns the per-sequence state, two tensors
per run (`state.k[r]`, `state.v[r]`), by mixer:

  * latent attention: `k[r]` the latent ring [n_slots, R, kv_rank] (model dtype; position p in row p % R; a block with
    `kv_from = j` holds the SAME tensor as block j), `v[r]` the convolution state [2, n_slots, taps - 1, hidden] fp32 (the normalised
    inputs of the last taps - 1 tokens of the mixer [0] and the feed-forward [1]);
  * window attention: `k[r]` keys [n_slots, G, rows, d], `v[r]` normalised values [n_slots, G, rows, dv] (model dtype); position p
    in row p below `keep_first`, else in a ring of the remaining rows (`WindowAttentionConfig.cache_rows`);
  * delta rule: `k[r]` the matrix states [n_slots, H, d, dv] fp32, `v[r]` the last taps - 1 projection outputs
    [n_slots, taps - 1, C] fp32;
  * differential window attention (`n_maps` = 2): `k[r]` [n_slots, 2G, rows, d] (both maps' keys), `v[r]` [n_slots, G, rows, dv];
  * rotated latent attention: `k[r]` the ring [n_slots, R, kv_rank + rot_dim] of rows [latent | rotated key part], `v[r]` empty;
  * matrix-memory LSTM: `k[r]` the states with the normaliser as last column [n_slots, H, d, dv + 1] fp32, `v[r]` the running
    maxima [n_slots, H] fp32;
  * decayed linear attention (`decay`): `k[r]` the matrix states [n_slots, H, d, dv] fp32, `v[r]` empty;
  * `parallel` (window attention beside decayed linear attention): `k[r]`, `v[r]` the rotated keys / values as for window
    attention, and a third tensor `state.m[r]` with the matrix states [n_slots, H, d, dv] fp32 (`m[r]` is None for other mixers).

A stack with `layer_norm_type == "layer"` runs  x <- x + mult * ls * LN_post(mixer(LN(x)))  and the same for the feed-forward, LN
being the bias-free LayerNorm; the add, the branch's output norm and the next sublayer's input norm are one kernel
(`ops.functional.residual_add_centred_norm_`).

Inference only (no autograd through these kernels) and not tensor-parallel.  A stack with a loop runs on one pipeline stage.
"""

from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional

import torch

from realhf_b200.ops import attention as attn_ops
from realhf_b200.ops import functional as OF
from realhf_b200.ops import recurrent as rec_ops


@dataclasses.dataclass
class PackedMeta:
    """Per-token indices of a packed batch, and where (if anywhere) the blocks leave the sequences' decode state."""
    pos: torch.Tensor                      # [T] int32 position inside the sequence
    remain: torch.Tensor                   # [T] int32 tokens that follow in the same sequence
    tok_slot: torch.Tensor                 # [T] int32 state slot of the token's sequence, -1 = keep no state
    k: Optional[List[torch.Tensor]] = None   # DecodeState.k / .v, indexed by local block
    v: Optional[List[torch.Tensor]] = None
    latents: Dict[int, torch.Tensor] = dataclasses.field(default_factory=dict)   # block index (0-based) -> packed latent [T, rank]
    cu_seqlens: Optional[torch.Tensor] = None
    max_seqlen: Optional[int] = None
    seq_slot: Optional[torch.Tensor] = None   # [n_seqs] int32 state slot of every sequence (None: keep no state)
    m: Optional[List[Optional[torch.Tensor]]] = None   # DecodeState.m


def packed_meta(cu_seqlens: torch.Tensor, total: int, slots: Optional[torch.Tensor] = None, state=None,
                max_seqlen: Optional[int] = None) -> PackedMeta:
    dev = cu_seqlens.device
    idx = torch.arange(total, device=dev, dtype=torch.int32)
    seq = torch.searchsorted(cu_seqlens[1:].contiguous(), idx, right=True).clamp_(max=cu_seqlens.numel() - 2).long()
    pos = (idx - cu_seqlens[seq]).int()
    remain = (cu_seqlens[seq + 1] - 1 - idx).int()
    if slots is None:
        tok_slot = torch.full((total,), -1, dtype=torch.int32, device=dev)
    else:
        tok_slot = slots.to(dev).int()[seq].contiguous()
    return PackedMeta(pos, remain, tok_slot, state.k if state is not None else None, state.v if state is not None else None,
                      cu_seqlens=cu_seqlens.int().contiguous(), max_seqlen=max_seqlen,
                      seq_slot=slots.to(dev).int().contiguous() if slots is not None else None,
                      m=getattr(state, "m", None) if state is not None else None)


def _mlp(model, i: int, h: torch.Tensor, mcfg) -> torch.Tensor:
    p = model.p
    if mcfg.kind == "moe":
        from realhf_b200.models import moe
        return moe.moe_forward(model, i, h, mcfg.moe, clamp=(mcfg.limit, mcfg.alpha) if mcfg.limit > 0 else None)
    if mcfg.kind == "relu2":
        return OF.linear(OF.relu2_linear(h, p[f"{i}.mlp.up.weight"]), p[f"{i}.mlp.down.weight"])
    if mcfg.kind == "glu":
        return OF.linear(OF.gated_linear(h, p[f"{i}.mlp.gate_up.weight"], mcfg.act), p[f"{i}.mlp.down.weight"])
    a = OF.clamped_gated_linear(h, p[f"{i}.mlp.gate_up.weight"], mcfg.limit, mcfg.alpha)
    return OF.linear(a, p[f"{i}.mlp.down.weight"])


def _window_attention_packed(model, i: int, li: int, h: torch.Tensor, meta: PackedMeta) -> torch.Tensor:
    c, p = model.config, model.p
    a = c.blocks[i - 1].wattn
    keep = meta.k is not None
    qkvg = OF.linear(h, p[f"{i}.attn.qkvg.weight"], p.get(f"{i}.attn.qkvg.bias"))
    if a.n_maps == 2:
        o = attn_ops.diff_window_attention(qkvg, a, p[f"{i}.attn.q_norm.weight"], p[f"{i}.attn.k_norm.weight"], p[f"{i}.attn.lambda.weight"],
                                           c.layer_norm_epsilon, meta.k[li] if keep else None, meta.v[li] if keep else None, meta.tok_slot,
                                           meta.pos, meta.remain, meta.cu_seqlens, meta.max_seqlen)
        return OF.linear(o, p[f"{i}.attn.o.weight"])
    if a.rotary is not None:
        attn_ops.rotate_qk_(qkvg, a, pos=meta.pos)
    v_n = attn_ops.value_norm_store(qkvg, a, c.layer_norm_epsilon, meta.k[li] if keep else None, meta.v[li] if keep else None,
                                    meta.tok_slot, meta.pos, meta.remain)
    o = attn_ops.sink_window_attention(qkvg, v_n, a, p.get(f"{i}.attn.temp.weight"), p.get(f"{i}.attn.sink.weight"), meta.pos,
                                       meta.cu_seqlens, meta.max_seqlen)
    return OF.linear(o, p[f"{i}.attn.o.weight"])


def _window_attention_decode(model, i: int, li: int, h: torch.Tensor, k_caches, v_caches, cache_lens, slots) -> torch.Tensor:
    c, p = model.config, model.p
    a = c.blocks[i - 1].wattn
    qkvg = OF.linear(h, p[f"{i}.attn.qkvg.weight"], p.get(f"{i}.attn.qkvg.bias"))
    if a.n_maps == 2:
        o = attn_ops.diff_window_decode_attention(qkvg, a, p[f"{i}.attn.q_norm.weight"], p[f"{i}.attn.k_norm.weight"], p[f"{i}.attn.lambda.weight"],
                                                  c.layer_norm_epsilon, k_caches[li], v_caches[li], cache_lens, slots)
        return OF.linear(o, p[f"{i}.attn.o.weight"])
    if a.rotary is not None:
        attn_ops.rotate_qk_(qkvg, a, cache_lens=cache_lens, slots=slots)
    o = attn_ops.sink_window_decode_attention(qkvg, a, p.get(f"{i}.attn.temp.weight"), p.get(f"{i}.attn.sink.weight"), k_caches[li],
                                              v_caches[li], cache_lens, slots, c.layer_norm_epsilon)
    return OF.linear(o, p[f"{i}.attn.o.weight"])


def _delta_packed(model, i: int, li: int, h: torch.Tensor, meta: PackedMeta) -> torch.Tensor:
    c, p = model.config, model.p
    d = c.blocks[i - 1].delta
    keep = meta.k is not None
    proj = OF.linear(h, p[f"{i}.attn.in.weight"])
    u = rec_ops.delta_prepare(proj, p[f"{i}.attn.conv.weight"], p[f"{i}.attn.A_log.weight"], p[f"{i}.attn.dt_bias.weight"], d, meta.pos,
                              meta.v[li] if keep else None, meta.tok_slot, meta.remain)
    o = rec_ops.delta_rule_scan(u, d, meta.cu_seqlens, meta.k[li] if keep else None, meta.seq_slot if keep else None)
    return OF.linear(_delta_out(model, i, d, o, proj), p[f"{i}.attn.o.weight"])


def _delta_out(model, i: int, d, o: torch.Tensor, proj: torch.Tensor) -> torch.Tensor:
    g0 = 2 * d.n_kv_heads * d.qk_dim + d.n_heads * d.v_dim
    return rec_ops.gated_head_norm(o, model.p[f"{i}.attn.o_norm.weight"], proj[:, g0:g0 + d.n_heads * d.v_dim],
                                   model.config.layer_norm_epsilon, model.dtype)


def _delta_decode(model, i: int, li: int, h: torch.Tensor, k_caches, v_caches, slots) -> torch.Tensor:
    c, p = model.config, model.p
    d = c.blocks[i - 1].delta
    proj = OF.linear(h, p[f"{i}.attn.in.weight"])
    u = rec_ops.delta_prepare_step(proj, p[f"{i}.attn.conv.weight"], p[f"{i}.attn.A_log.weight"], p[f"{i}.attn.dt_bias.weight"], d,
                                   v_caches[li], slots)
    o = rec_ops.delta_rule_step(u, d, k_caches[li], slots)
    return OF.linear(_delta_out(model, i, d, o, proj), p[f"{i}.attn.o.weight"])


def _mlstm_packed(model, i: int, li: int, h: torch.Tensor, meta: PackedMeta) -> torch.Tensor:
    c, p = model.config, model.p
    m = c.blocks[i - 1].mlstm
    keep = meta.k is not None
    proj = OF.linear(h, p[f"{i}.attn.in.weight"])
    o, mx = rec_ops.mlstm_scan(proj, p[f"{i}.attn.gate_bias.weight"], m, meta.cu_seqlens, meta.k[li] if keep else None,
                               meta.v[li] if keep else None, meta.seq_slot if keep else None)
    return OF.linear(_mlstm_out(model, i, m, o, mx, proj), p[f"{i}.attn.o.weight"])


def _mlstm_out(model, i: int, m, o, mx, proj) -> torch.Tensor:
    g0 = 2 * m.n_heads * m.qk_dim + m.n_heads * m.v_dim
    return rec_ops.mlstm_out(o, mx, model.p[f"{i}.attn.o_norm.weight"], proj[:, g0:g0 + m.n_heads * m.v_dim], model.config.layer_norm_epsilon,
                             model.dtype)


def _mlstm_decode(model, i: int, li: int, h: torch.Tensor, k_caches, v_caches, slots) -> torch.Tensor:
    p = model.p
    m = model.config.blocks[i - 1].mlstm
    proj = OF.linear(h, p[f"{i}.attn.in.weight"])
    o, mx = rec_ops.mlstm_step(proj, p[f"{i}.attn.gate_bias.weight"], m, k_caches[li], v_caches[li], slots)
    return OF.linear(_mlstm_out(model, i, m, o, mx, proj), p[f"{i}.attn.o.weight"])


def _latent_rope_queries(model, i: int, a, proj: torch.Tensor, cq: Optional[torch.Tensor]) -> torch.Tensor:
    """[rows, H (d + rot)] queries, not yet rotated: the up-projection of the normalised query latent, or a section of `proj`."""
    if a.q_rank:
        return OF.linear(cq, model.p[f"{i}.attn.uq.weight"])
    q0 = a.cache_width + (a.n_heads * a.v_dim if a.out_gate else 0)
    return proj[:, q0:q0 + a.n_heads * (a.qk_dim + a.rot_dim)]


def _latent_rope_gate(a, o: torch.Tensor, proj: torch.Tensor) -> torch.Tensor:
    if a.out_gate:
        g0 = (a.q_rank or 0) + a.cache_width
        attn_ops.sigmoid_gate_(o, proj[:, g0:g0 + a.n_heads * a.v_dim])
    return o


def _latent_rope_packed(model, i: int, li: int, h: torch.Tensor, meta: PackedMeta) -> torch.Tensor:
    c, p = model.config, model.p
    a = c.blocks[i - 1].attn
    keep = meta.k is not None
    proj = OF.linear(h, p[f"{i}.attn.in.weight"])
    cq, lat = attn_ops.latent_rope_prepare(proj, a, p.get(f"{i}.attn.q_ln.weight"), p[f"{i}.attn.dkv_ln.weight"], c.layer_norm_epsilon, meta.pos,
                                           meta.k[li] if keep else None, meta.tok_slot, meta.remain)
    q = _latent_rope_queries(model, i, a, proj, cq)
    kv = OF.linear(lat[:, : a.kv_rank], p[f"{i}.attn.ukv.weight"])
    o = attn_ops.latent_rope_attention(q, kv, lat, a, p.get(f"{i}.attn.sink.weight"), meta.pos, meta.cu_seqlens, meta.max_seqlen)
    return OF.linear(_latent_rope_gate(a, o, proj), p[f"{i}.attn.o.weight"])


def _latent_rope_decode(model, i: int, li: int, h: torch.Tensor, k_caches, cache_lens, slots) -> torch.Tensor:
    c, p = model.config, model.p
    a = c.blocks[i - 1].attn
    proj = OF.linear(h, p[f"{i}.attn.in.weight"])
    cq, _ = attn_ops.latent_rope_prepare(proj, a, p.get(f"{i}.attn.q_ln.weight"), p[f"{i}.attn.dkv_ln.weight"], c.layer_norm_epsilon, None,
                                         k_caches[li], cache_lens=cache_lens, slots=slots, want_lat=False)
    q = _latent_rope_queries(model, i, a, proj, cq)
    o = attn_ops.latent_rope_decode_attention(q, a, p[f"{i}.attn.ukv.weight"], p.get(f"{i}.attn.sink.weight"), k_caches[li], cache_lens, slots)
    return OF.linear(_latent_rope_gate(a, o, proj), p[f"{i}.attn.o.weight"])


def _decay_branch(model, i: int, d, proj: torch.Tensor, o: torch.Tensor) -> torch.Tensor:
    """Output norm and gate of a decayed-linear-attention branch; `proj` is the branch's projection row [q | k | v | gate]."""
    g0 = 2 * d.n_heads * d.qk_dim + d.n_heads * d.v_dim
    return rec_ops.decay_out(o, d, model.p.get(f"{i}.attn.o_norm.weight"), proj[:, g0:g0 + d.n_heads * d.v_dim], model.config.layer_norm_epsilon,
                             model.dtype)


def _decay_packed(model, i: int, li: int, h: torch.Tensor, meta: PackedMeta):
    p = model.p
    d = model.config.blocks[i - 1].decay
    keep = meta.k is not None
    proj = OF.linear(h, p[f"{i}.attn.in.weight"])
    o = rec_ops.decay_scan(rec_ops.decay_prepare(proj, d, pos=meta.pos), d, meta.cu_seqlens, meta.k[li] if keep else None,
                           meta.seq_slot if keep else None)
    return OF.linear(_decay_branch(model, i, d, proj, o), p[f"{i}.attn.o.weight"])


def _decay_decode(model, i: int, li: int, h: torch.Tensor, k_caches, cache_lens, slots):
    p = model.p
    d = model.config.blocks[i - 1].decay
    proj = OF.linear(h, p[f"{i}.attn.in.weight"])
    o = rec_ops.decay_step(rec_ops.decay_prepare(proj, d, cache_lens=cache_lens, slots=slots), d, k_caches[li], slots)
    return OF.linear(_decay_branch(model, i, d, proj, o), p[f"{i}.attn.o.weight"])


def _parallel_split(b, proj: torch.Tensor):
    """The fused projection row of a `parallel` block as two views: [window attention q | k | v] and [decay q | k | v | gate]."""
    from realhf_b200.models.sharding import wattn_sections
    nl = sum(wattn_sections(b.wattn))
    return proj[:, :nl], proj[:, nl:]


def _parallel_packed(model, i: int, li: int, h: torch.Tensor, meta: PackedMeta):
    """Both branches of a `parallel` block on the packed batch -> (left output, right output), each after its own projection."""
    c, p = model.config, model.p
    b = c.blocks[i - 1]
    w, d = b.wattn, b.decay
    keep = meta.k is not None
    left, right = _parallel_split(b, OF.linear(h, p[f"{i}.attn.in.weight"]))
    if w.rotary is not None:
        attn_ops.rotate_qk_(left, w, pos=meta.pos)
    v_n = attn_ops.value_norm_store(left, w, c.layer_norm_epsilon, meta.k[li] if keep else None, meta.v[li] if keep else None, meta.tok_slot,
                                    meta.pos, meta.remain)
    o = attn_ops.sink_window_attention(left, v_n, w, None, None, meta.pos, meta.cu_seqlens, meta.max_seqlen)
    y_l = OF.linear(o, p[f"{i}.attn.o.weight"])
    s = rec_ops.decay_scan(rec_ops.decay_prepare(right, d, pos=meta.pos), d, meta.cu_seqlens, meta.m[li] if keep else None,
                           meta.seq_slot if keep else None)
    return y_l, OF.linear(_decay_branch(model, i, d, right, s), p[f"{i}.attn.o2.weight"])


def _parallel_decode(model, i: int, li: int, h: torch.Tensor, k_caches, v_caches, m_caches, cache_lens, slots):
    c, p = model.config, model.p
    b = c.blocks[i - 1]
    w, d = b.wattn, b.decay
    left, right = _parallel_split(b, OF.linear(h, p[f"{i}.attn.in.weight"]))
    if w.rotary is not None:
        attn_ops.rotate_qk_(left, w, cache_lens=cache_lens, slots=slots)
    o = attn_ops.sink_window_decode_attention(left, w, None, None, k_caches[li], v_caches[li], cache_lens, slots, c.layer_norm_epsilon)
    y_l = OF.linear(o, p[f"{i}.attn.o.weight"])
    s = rec_ops.decay_step(rec_ops.decay_prepare(right, d, cache_lens=cache_lens, slots=slots), d, m_caches[li], slots)
    return y_l, OF.linear(_decay_branch(model, i, d, right, s), p[f"{i}.attn.o2.weight"])


@dataclasses.dataclass
class PendingBranch:
    """A branch output of a "layer" stack that is still owed to the stream: x += mult * scale * LN(a y + b y2) * w.  The kernel that
    computes the next norm (the next block's, the final one) adds it on the way."""
    y: torch.Tensor
    w: torch.Tensor
    scale: Optional[torch.Tensor]
    y2: Optional[torch.Tensor] = None
    a: float = 1.0
    b: float = 1.0


def _add_pending(model, x: torch.Tensor, pb: PendingBranch, next_w: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    c = model.config
    return OF.residual_add_centred_norm_(x, pb.y, pb.w, c.layer_norm_epsilon, pb.scale, c.residual_mult, pb.y2, pb.a, pb.b, next_w, model.dtype)


def _finish_layer_block(model, i: int, b, x: torch.Tensor, y, defer: bool = False) -> Optional[PendingBranch]:
    """"layer" stacks: x += mult * ls * LN_post(mixer output), then the feed-forward sublayer likewise.  `y` is the mixer's output,
    or the pair of branch outputs of a `parallel` block (summed with `branch_scales` inside the norm kernel).  With `defer` the
    block's last branch is returned instead of added."""
    p = model.p
    y, y2 = y if isinstance(y, tuple) else (y, None)
    sa, sb = b.branch_scales if y2 is not None else (1.0, 1.0)
    pb = PendingBranch(y, p[f"{i}.attn.ln_post.weight"], p.get(f"{i}.attn.ls.weight"), y2, sa, sb)
    if b.mlp is not None:
        h = _add_pending(model, x, pb, p[f"{i}.mlp.ln.weight"])
        pb = PendingBranch(_mlp(model, i, h, b.mlp), p[f"{i}.mlp.ln_post.weight"], p.get(f"{i}.mlp.ls.weight"))
    if defer:
        return pb
    _add_pending(model, x, pb)
    return None


def _first_layer_norm(model, i: int, x: torch.Tensor, pending) -> torch.Tensor:
    """Input of block i's mixer in a "layer" stack; a branch the previous block left pending is added by the same kernel."""
    w = model.p[f"{i}.attn.ln.weight"]
    if isinstance(pending, PendingBranch):
        return _add_pending(model, x, pending, w)
    return OF.centred_norm(settle(model, x, pending), w, model.config.layer_norm_epsilon, model.dtype)


def norm_offset(c) -> float:
    """What is added to a stored norm weight: 1 for weights stored around zero (`layer_norm_type` "gemma")."""
    return 1.0 if c.layer_norm_type == "gemma" else 0.0


def loop_inject(model, i: int, x: torch.Tensor, x0: torch.Tensor) -> torch.Tensor:
    """Start of a pass of the loop.  Mode "linear": x <- W_in [x; x0] (x0 = the embedding output), back on the residual stream's
    dtype; mode "add": x <- x + x0 in place."""
    if model.config.loop.inject_mode == "add":
        return OF.residual_add_norm_(x, x0, None, 1, model.config.layer_norm_epsilon)
    cat = OF.concat_cast(x, x0, model.dtype)
    w = model.p[f"{i}.loop_in.weight"]
    return OF.linear_f32(cat, w) if x.dtype == torch.float32 else OF.linear(cat, w).to(x.dtype)


def plain_prenorm(c) -> bool:
    """One RMSNorm per sublayer and nothing else around it: a sublayer's residual add can wait for the next norm kernel."""
    return c.norm_groups == 1 and not c.sandwich_norm and not c.conv_taps


def first_norm(model, i: int, x: torch.Tensor, pending: Optional[torch.Tensor]) -> torch.Tensor:
    """Input of block i's mixer in a plain pre-norm stack; a branch output still owed to the stream is added in the same kernel."""
    w, eps, off = model.p[f"{i}.attn.ln.weight"], model.config.layer_norm_epsilon, norm_offset(model.config)
    if pending is not None:
        return OF.add_rms_norm_(x, pending, w, eps, model.dtype, off)
    return OF.sublayer_input(x, w, 1, eps, None, None, model.dtype, w_offset=off)


def settle(model, x: torch.Tensor, pending: Optional[torch.Tensor]) -> torch.Tensor:
    """Add a branch output that a block left pending (the caller needs the stream itself)."""
    if isinstance(pending, PendingBranch):
        _add_pending(model, x, pending)
        return x
    if pending is not None:
        OF.residual_add_norm_(x, pending, None, 1, model.config.layer_norm_epsilon)
    return x


def _finish_block(model, i: int, b, x: torch.Tensor, y: torch.Tensor, defer: bool = False) -> Optional[torch.Tensor]:
    """x += mixer output y, then the feed-forward sublayer (same code for packed and one-token batches: neither has a state).  In
    a plain pre-norm stack the add is fused into the feed-forward's norm, and with `defer` the block's last branch output is
    returned instead of added: the next block's first norm (or the final norm) adds it."""
    c, p = model.config, model.p
    G, eps = c.norm_groups, c.layer_norm_epsilon
    post = p.get(f"{i}.attn.ln_post.weight")
    if b.mlp is None:
        if defer and post is None:
            return y
        OF.residual_add_norm_(x, y, post, G, eps)
        return None
    if post is None and G == 1:
        h = OF.add_rms_norm_(x, y, p[f"{i}.mlp.ln.weight"], eps, model.dtype, norm_offset(c))
    else:
        OF.residual_add_norm_(x, y, post, G, eps)
        h = OF.sublayer_input(x, p[f"{i}.mlp.ln.weight"], G, eps, None, None, model.dtype, w_offset=norm_offset(c))
    y2 = _mlp(model, i, h, b.mlp)
    post2 = p.get(f"{i}.mlp.ln_post.weight")
    if defer and post2 is None:
        return y2
    OF.residual_add_norm_(x, y2, post2, G, eps)
    return None


def block_packed(model, i: int, li: int, x: torch.Tensor, meta: PackedMeta, pending: Optional[torch.Tensor] = None, defer: bool = False):
    """Block i (1-based layer index; li = index among this stage's block runs) on the packed batch; x [T, H] is updated in place.
    Returns (x, pending): `pending` is a branch output not yet added to x (only with `defer`, in plain pre-norm stacks), which the
    caller hands to the next block (`pending=`) or settles."""
    c, p = model.config, model.p
    b = c.blocks[i - 1]
    a = b.attn
    G, eps = c.norm_groups, c.layer_norm_epsilon
    keep = meta.k is not None
    if c.layer_norm_type == "layer":
        h = _first_layer_norm(model, i, x, pending)
        mixer = {"window_attention": _window_attention_packed, "delta": _delta_packed, "mlstm": _mlstm_packed, "latent_attention": _latent_rope_packed,
                 "decay": _decay_packed, "parallel": _parallel_packed}[b.mixer]
        return x, _finish_layer_block(model, i, b, x, mixer(model, i, li, h, meta), defer)
    if b.mixer != "latent_attention" or a.rotated:
        defer = defer and plain_prenorm(c)
        h = first_norm(model, i, x, pending) if plain_prenorm(c) else OF.sublayer_input(settle(model, x, pending), p[f"{i}.attn.ln.weight"], G, eps,
                                                                                       None, None, model.dtype, w_offset=norm_offset(c))
        mixer = {"window_attention": _window_attention_packed, "delta": _delta_packed, "mlstm": _mlstm_packed,
                 "latent_attention": _latent_rope_packed}[b.mixer]
        return x, _finish_block(model, i, b, x, mixer(model, i, li, h, meta), defer)
    settle(model, x, pending)
    conv = meta.v[li] if keep and c.conv_taps else None
    h = OF.sublayer_input(x, p[f"{i}.attn.ln.weight"], G, eps, p.get(f"{i}.attn.canon.weight"), meta.pos, model.dtype,
                          conv[0] if conv is not None else None, meta.tok_slot, meta.remain)
    qc = OF.linear(h, p[f"{i}.attn.q_dkv.weight"])
    n_q = a.n_heads * a.qk_dim
    if a.kv_from is None:
        lat = attn_ops.latent_norm_store(qc, n_q, p[f"{i}.attn.dkv_ln.weight"], eps, meta.k[li] if keep else None, meta.tok_slot, meta.pos,
                                         meta.remain)
        meta.latents[i - 1] = lat
    else:
        lat = meta.latents[a.kv_from]
    kv = OF.linear(lat, p[f"{i}.attn.ukv.weight"])
    o = attn_ops.latent_window_attention(qc, kv, meta.pos, a.n_heads, a.qk_dim, a.v_dim, a.scale, a.window, meta.cu_seqlens, meta.max_seqlen)
    y = OF.linear(o, p[f"{i}.attn.o.weight"])
    OF.residual_add_norm_(x, y, p.get(f"{i}.attn.ln_post.weight"), G, eps)
    if b.mlp is not None:
        h = OF.sublayer_input(x, p[f"{i}.mlp.ln.weight"], G, eps, p.get(f"{i}.mlp.canon.weight"), meta.pos, model.dtype,
                              conv[1] if conv is not None else None, meta.tok_slot, meta.remain)
        OF.residual_add_norm_(x, _mlp(model, i, h, b.mlp), p.get(f"{i}.mlp.ln_post.weight"), G, eps)
    return x, None


def _mixer_decode(model, b, i: int, li: int, h: torch.Tensor, k_caches, v_caches, m_caches, cache_lens, slots):
    if b.mixer == "window_attention":
        return _window_attention_decode(model, i, li, h, k_caches, v_caches, cache_lens, slots)
    if b.mixer == "mlstm":
        return _mlstm_decode(model, i, li, h, k_caches, v_caches, slots)
    if b.mixer == "latent_attention":
        return _latent_rope_decode(model, i, li, h, k_caches, cache_lens, slots)
    if b.mixer == "decay":
        return _decay_decode(model, i, li, h, k_caches, cache_lens, slots)
    if b.mixer == "parallel":
        return _parallel_decode(model, i, li, h, k_caches, v_caches, m_caches, cache_lens, slots)
    return _delta_decode(model, i, li, h, k_caches, v_caches, slots)


def block_decode(model, i: int, li: int, x: torch.Tensor, k_caches: List[torch.Tensor], v_caches: List[torch.Tensor],
                 cache_lens: torch.Tensor, slots: Optional[torch.Tensor], pending: Optional[torch.Tensor] = None, defer: bool = False,
                 m_caches: Optional[List[Optional[torch.Tensor]]] = None):
    """Block i for one new token per row; x [B, H] is updated in place.  Row b lives in state slot slots[b] (None: slot b).
    Returns (x, pending) as `block_packed` does."""
    c, p = model.config, model.p
    b = c.blocks[i - 1]
    a = b.attn
    G, eps = c.norm_groups, c.layer_norm_epsilon
    if c.layer_norm_type == "layer":
        h = _first_layer_norm(model, i, x, pending)
        return x, _finish_layer_block(model, i, b, x, _mixer_decode(model, b, i, li, h, k_caches, v_caches, m_caches, cache_lens, slots), defer)
    if b.mixer != "latent_attention" or a.rotated:
        defer = defer and plain_prenorm(c)
        h = first_norm(model, i, x, pending) if plain_prenorm(c) else OF.sublayer_input_step(settle(model, x, pending), p[f"{i}.attn.ln.weight"], G,
                                                                                            eps, None, None, slots, model.dtype,
                                                                                            w_offset=norm_offset(c))
        return x, _finish_block(model, i, b, x, _mixer_decode(model, b, i, li, h, k_caches, v_caches, m_caches, cache_lens, slots), defer)
    settle(model, x, pending)
    conv = v_caches[li] if c.conv_taps else None
    h = OF.sublayer_input_step(x, p[f"{i}.attn.ln.weight"], G, eps, p.get(f"{i}.attn.canon.weight"),
                               conv[0] if conv is not None else None, slots, model.dtype)
    qc = OF.linear(h, p[f"{i}.attn.q_dkv.weight"])
    o = attn_ops.latent_decode_attention(qc, p[f"{i}.attn.dkv_ln.weight"] if a.kv_from is None else None, p[f"{i}.attn.ukv.weight"],
                                         k_caches[li], cache_lens, slots, a.n_heads, a.qk_dim, a.v_dim, a.scale, a.window, eps)
    y = OF.linear(o, p[f"{i}.attn.o.weight"])
    OF.residual_add_norm_(x, y, p.get(f"{i}.attn.ln_post.weight"), G, eps)
    if b.mlp is not None:
        h = OF.sublayer_input_step(x, p[f"{i}.mlp.ln.weight"], G, eps, p.get(f"{i}.mlp.canon.weight"),
                                   conv[1] if conv is not None else None, slots, model.dtype)
        OF.residual_add_norm_(x, _mlp(model, i, h, b.mlp), p.get(f"{i}.mlp.ln_post.weight"), G, eps)
    return x, None


def final_norm(model, x: torch.Tensor, pending: Optional[torch.Tensor] = None) -> torch.Tensor:
    c = model.config
    w = model.p[f"{c.n_layers}.ln_f.weight"]
    if c.layer_norm_type == "layer":
        if isinstance(pending, PendingBranch):
            return _add_pending(model, x, pending, w)
        return OF.centred_norm(x, w, c.layer_norm_epsilon, model.dtype)
    if pending is not None and plain_prenorm(c):
        return OF.add_rms_norm_(x, pending, w, c.layer_norm_epsilon, model.dtype, norm_offset(c))
    return OF.sublayer_input(settle(model, x, pending), w, c.norm_groups, c.layer_norm_epsilon, None, None, model.dtype, w_offset=norm_offset(c))


def ring_rows(cfg, block: int, max_len: int) -> int:
    """Rows of the latent ring of 0-based block `block` (which projects its own latent): the largest window among the blocks
    that read it, or max_len when one of them sees the whole prefix."""
    need = 0
    for j, b in enumerate(cfg.blocks):
        if b.mixer != "latent_attention":
            continue
        if j == block or b.attn.kv_from == block:
            if b.attn.window is None:
                return max_len
            need = max(need, b.attn.window)
    return max(1, min(need, max_len))
