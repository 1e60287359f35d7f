"""Recurrent mixers in packed (prefill) and one-token (decode) form: the gated delta rule (`DeltaRuleConfig`, below), the
matrix-memory LSTM (`MLSTMConfig`) and linear attention with a fixed decay per head (`DecayConfig`), each introduced by a comment
block further down.

Per head, with a matrix state S [d, dv] in fp32:   S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
(the output is read after the update, so it contains what this token just wrote).  Everything that enters the recurrence is fp32.

The stages, each = PyTorch reference (CPU tensors, also the numerics oracle of the kernel tests) + sm_100a kernel (`csrc/delta.cu`):

  delta_prepare(_step)   the fused projection output `proj` [T, ld] = [q (G x d) | k (G x d) | v (H x dv) | gate (H x dv) | beta
                         logits (H) | decay inputs (H) | padding] -> fp32 `u` [T, C + 2H] = [q | k | v | beta | g]:  causal depthwise
                         convolution + SiLU over the first C = 2 G d + H dv channels (inputs before a sequence's first token are zero; the packed
                         form leaves the last taps - 1 raw inputs of every sequence in `conv_state` [n_slots, taps - 1, C] fp32,
                         oldest first; the step form reads and shifts it), q and k scaled to unit length per head (q also by
                         d^-1/2), beta = sigmoid, g = exp(-exp(A_log) softplus(a + dt_bias)).
  delta_rule_scan / _step  the recurrence over each sequence from S = 0 (leaving S in `s_state` [n_slots, H, d, dv] fp32), or one
                         token per row against `s_state`, updated in place.  o [T, H, dv] fp32.
  gated_head_norm        o / rms(o) * w * silu(gate) per head -> [T, H * dv] in the model dtype.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from realhf_b200.ops import lib, use_native


def _offsets(d):
    nqk, nv, H = d.n_kv_heads * d.qk_dim, d.n_heads * d.v_dim, d.n_heads
    C = 2 * nqk + nv
    return nqk, nv, H, C


def _finish_prepare(y, proj, d, A_log, dt_bias):
    """y [T, C] fp32 = convolved channels -> u [T, C + 2H]."""
    nqk, nv, H, C = _offsets(d)
    T = y.shape[0]
    y = y * torch.sigmoid(y)
    q = y[:, :nqk].view(T, d.n_kv_heads, d.qk_dim)
    k = y[:, nqk:2 * nqk].view(T, d.n_kv_heads, d.qk_dim)
    q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + d.unit_eps) * d.qk_dim ** -0.5
    k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + d.unit_eps)
    beta = torch.sigmoid(proj[:, C + nv:C + nv + H].float())
    g = torch.exp(-torch.exp(A_log.float()) * F.softplus(proj[:, C + nv + H:C + nv + 2 * H].float() + dt_bias.float()))
    return torch.cat([q.reshape(T, nqk), k.reshape(T, nqk), y[:, 2 * nqk:], beta, g], -1).contiguous()


def delta_prepare_ref(proj, conv_w, A_log, dt_bias, d, pos, conv_state, tok_slot, remain):
    nqk, nv, H, C = _offsets(d)
    taps = d.conv_taps
    x = proj[:, :C].float()
    cw = conv_w.float()
    y = x * cw[:, taps - 1]
    for back in range(1, taps):
        prev = torch.zeros_like(x)
        prev[back:] = x[:-back]
        y = y + torch.where((pos.long() >= back).unsqueeze(-1), prev, torch.zeros_like(prev)) * cw[:, taps - 1 - back]
    if conv_state is not None and taps > 1:
        keep = (remain < taps - 1) & (tok_slot >= 0)
        conv_state[tok_slot[keep].long(), (taps - 2 - remain[keep]).long()] = x[keep]
    return _finish_prepare(y, proj, d, A_log, dt_bias)


def delta_prepare(proj, conv_w, A_log, dt_bias, d, pos, conv_state=None, tok_slot=None, remain=None):
    if use_native(proj) and d.conv_taps <= 8:
        nqk, nv, H, C = _offsets(d)
        u = torch.empty(proj.shape[0], C + 2 * H, dtype=torch.float32, device=proj.device)
        keep = conv_state is not None and d.conv_taps > 1
        lib().delta_prepare(proj, conv_w, A_log, dt_bias, u, pos, conv_state if keep else None, tok_slot if keep else None,
                            remain if keep else None, None, d.n_heads, d.n_kv_heads, d.qk_dim, d.v_dim, d.conv_taps, d.unit_eps)
        return u
    return delta_prepare_ref(proj, conv_w, A_log, dt_bias, d, pos, conv_state, tok_slot, remain)


def delta_prepare_step_ref(proj, conv_w, A_log, dt_bias, d, conv_state, slots):
    nqk, nv, H, C = _offsets(d)
    taps = d.conv_taps
    x = proj[:, :C].float()
    cw = conv_w.float()
    y = x * cw[:, taps - 1]
    if taps > 1:
        idx = slots.long() if slots is not None else torch.arange(proj.shape[0], device=proj.device)
        st = conv_state[idx]                                               # [B, taps - 1, C], oldest first
        y = y + (st * cw[:, :taps - 1].t().unsqueeze(0)).sum(1)
        conv_state[idx] = torch.cat([st[:, 1:], x.unsqueeze(1)], 1)
    return _finish_prepare(y, proj, d, A_log, dt_bias)


def delta_prepare_step(proj, conv_w, A_log, dt_bias, d, conv_state, slots):
    if use_native(proj) and d.conv_taps <= 8:
        nqk, nv, H, C = _offsets(d)
        u = torch.empty(proj.shape[0], C + 2 * H, dtype=torch.float32, device=proj.device)
        lib().delta_prepare(proj, conv_w, A_log, dt_bias, u, None, conv_state if d.conv_taps > 1 else None, None, None, slots,
                            d.n_heads, d.n_kv_heads, d.qk_dim, d.v_dim, d.conv_taps, d.unit_eps)
        return u
    return delta_prepare_step_ref(proj, conv_w, A_log, dt_bias, d, conv_state, slots)


def _split_u(u, d):
    nqk, nv, H, C = _offsets(d)
    T = u.shape[0]
    return (u[:, :nqk].view(T, d.n_kv_heads, d.qk_dim), u[:, nqk:2 * nqk].view(T, d.n_kv_heads, d.qk_dim),
            u[:, 2 * nqk:C].view(T, H, d.v_dim), u[:, C:C + H], u[:, C + H:C + 2 * H])


def _delta_token(S, q, k, v, beta, g):
    """S [H, d, dv]; q, k [H, d]; v [H, dv]; beta, g [H] -> (S', o [H, dv])."""
    S = S * g.view(-1, 1, 1)
    w = beta.view(-1, 1) * (v - torch.einsum("hdv,hd->hv", S, k))
    S = S + k.unsqueeze(-1) * w.unsqueeze(1)
    return S, torch.einsum("hdv,hd->hv", S, q)


def delta_rule_scan_ref(u, d, cu_seqlens, s_state, slots):
    q, k, v, beta, g = _split_u(u, d)
    rep = d.n_heads // d.n_kv_heads
    q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)
    o = torch.zeros(u.shape[0], d.n_heads, d.v_dim, dtype=torch.float32, device=u.device)
    cu = cu_seqlens.tolist()
    for b in range(len(cu) - 1):
        S = torch.zeros(d.n_heads, d.qk_dim, d.v_dim, dtype=torch.float32, device=u.device)
        for t in range(cu[b], cu[b + 1]):
            S, o[t] = _delta_token(S, q[t], k[t], v[t], beta[t], g[t])
        if s_state is not None and slots is not None and int(slots[b]) >= 0 and cu[b + 1] > cu[b]:
            s_state[int(slots[b])] = S
    return o


def delta_rule_scan(u, d, cu_seqlens, s_state=None, slots=None):
    """u [T, C + 2H] fp32 (see `delta_prepare`), sequences given by cu_seqlens, each from S = 0.  Returns o [T, H, dv] fp32; with
    `s_state` and `slots` [n_seqs] int32, sequence b's final state is left in s_state[slots[b]] (slots[b] < 0: dropped)."""
    if use_native(u) and d.qk_dim <= 512:
        o = torch.empty(u.shape[0], d.n_heads, d.v_dim, dtype=torch.float32, device=u.device)
        lib().delta_rule_scan(u, o, cu_seqlens, s_state, slots if s_state is not None else None, d.n_heads, d.n_kv_heads, d.qk_dim, d.v_dim)
        return o
    return delta_rule_scan_ref(u, d, cu_seqlens, s_state, slots)


def delta_rule_step_ref(u, d, s_state, slots):
    q, k, v, beta, g = _split_u(u, d)
    rep = d.n_heads // d.n_kv_heads
    q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)
    o = torch.zeros(u.shape[0], d.n_heads, d.v_dim, dtype=torch.float32, device=u.device)
    for b in range(u.shape[0]):
        s = int(slots[b]) if slots is not None else b
        s_state[s], o[b] = _delta_token(s_state[s], q[b], k[b], v[b], beta[b], g[b])
    return o


def delta_rule_step(u, d, s_state, slots):
    """One token per row: s_state[slots[b]] (slots None: row b is slot b) is updated in place.  Returns o [B, H, dv] fp32."""
    if use_native(u) and d.qk_dim <= 512:
        o = torch.empty(u.shape[0], d.n_heads, d.v_dim, dtype=torch.float32, device=u.device)
        lib().delta_rule_step(u, o, s_state, slots, d.n_heads, d.n_kv_heads, d.qk_dim, d.v_dim)
        return o
    return delta_rule_step_ref(u, d, s_state, slots)


def gated_head_norm_ref(o, w, gate, eps, out_dtype):
    T, H, dv = o.shape
    n = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    gt = gate.float().view(T, H, dv)
    return (n * gt * torch.sigmoid(gt)).reshape(T, H * dv).to(out_dtype)


def gated_head_norm(o, w, gate, eps: float, out_dtype):
    """o [T, H, dv] fp32, w [dv], gate [T, H * dv] (a column slice of the projection output; unit column stride)."""
    if use_native(o):
        out = torch.empty(o.shape[0], o.shape[1] * o.shape[2], dtype=out_dtype, device=o.device)
        lib().gated_head_norm(o, w, gate, out, eps)
        return out
    return gated_head_norm_ref(o, w, gate, eps, out_dtype)


# ------------------------------------------------------------------------------------------------ matrix-memory LSTM
# (`MLSTMConfig`).  The fused projection output `proj` [T, ld] = [q (H x d) | k (H x d) | v (H x dv) | output gate (H x dv) | input
# gate logits (H) | forget gate logits (H) | padding]; `gate_bias` [2H] = the two gates' biases.  Per head, all fp32:
#   i = cap tanh((x_i + b_i) / cap),  f = logsigmoid(cap tanh((x_f + b_f) / cap)),  m' = max(f + m, i)   (m starts at 0)
#   S <- exp(f + m - m') S + exp(i - m') k v^T,   n likewise with k alone,   o = S^T (q d^-1/2) / (max(|n . q d^-1/2|, exp(-m')) + 1e-6)
# n is stored as column dv of the state, so `state` is [n_slots, H, d, dv + 1] and `m_state` [n_slots, H].  `mlstm_scan` returns
# the raw rows [S^T q | n . q] and m per token; `mlstm_out` applies the denominator, the per-head RMS norm (no weight), the
# full-width weight and the sigmoid output gate.


def _mlstm_offsets(c):
    nq, nv = c.n_heads * c.qk_dim, c.n_heads * c.v_dim
    return nq, 2 * nq, 2 * nq + nv, 2 * nq + 2 * nv        # k, v, output gate, gate logits


def _mlstm_ref(proj, gate_bias, c, seqs, state, m_state, slot_of, load_state):
    T = proj.shape[0]
    H, d, dv, cap = c.n_heads, c.qk_dim, c.v_dim, float(c.gate_cap)
    ok, ov, _, oif = _mlstm_offsets(c)
    q = proj[:, :ok].float().view(T, H, d) * (d ** -0.5)
    k = proj[:, ok:ov].float().view(T, H, d)
    v = torch.cat([proj[:, ov:ov + H * dv].float().view(T, H, dv), torch.ones(T, H, 1, device=proj.device)], -1)
    b = gate_bias.float()
    ig = cap * torch.tanh((proj[:, oif:oif + H].float() + b[:H]) / cap)
    fg = F.logsigmoid(cap * torch.tanh((proj[:, oif + H:oif + 2 * H].float() + b[H:]) / cap))
    o = torch.empty(T, H, dv + 1, dtype=torch.float32, device=proj.device)
    mo = torch.empty(T, H, dtype=torch.float32, device=proj.device)
    for n, (s0, e0) in enumerate(seqs):
        if e0 == s0:
            continue
        sl = slot_of(n)
        if load_state:
            S, m = state[sl].clone(), m_state[sl].clone()
        else:
            S = torch.zeros(H, d, dv + 1, dtype=torch.float32, device=proj.device)
            m = torch.zeros(H, dtype=torch.float32, device=proj.device)
        for t in range(s0, e0):
            mn = torch.maximum(fg[t] + m, ig[t])
            dec, inp = torch.exp(fg[t] + m - mn), torch.exp(ig[t] - mn)
            S = dec[:, None, None] * S + (inp[:, None] * k[t])[:, :, None] * v[t][:, None, :]
            m = mn
            o[t] = torch.einsum("hdv,hd->hv", S, q[t])
            mo[t] = m
        if state is not None:
            state[sl] = S
            m_state[sl] = m
    return o, mo


def mlstm_scan(proj, gate_bias, c, cu_seqlens, state=None, m_state=None, seq_slot=None, load_state: bool = False):
    """Packed recurrence over every sequence, from zero (or, with `load_state`, from the slot's state); the final state is left in
    state[seq_slot[n]] when `state` is given.  Returns (o [T, H, dv + 1] fp32, m [T, H] fp32)."""
    T = proj.shape[0]
    H, d, dv = c.n_heads, c.qk_dim, c.v_dim
    if use_native(proj) and d <= 1024:
        o = torch.empty(T, H, dv + 1, dtype=torch.float32, device=proj.device)
        mo = torch.empty(T, H, dtype=torch.float32, device=proj.device)
        lib().mlstm_scan(proj, gate_bias, o, mo, cu_seqlens, state, m_state, seq_slot if state is not None else None, H, d, dv,
                         float(c.gate_cap), bool(load_state))
        return o, mo
    cu = cu_seqlens.tolist()
    return _mlstm_ref(proj, gate_bias, c, list(zip(cu[:-1], cu[1:])), state, m_state,
                      lambda n: int(seq_slot[n]) if seq_slot is not None else n, load_state)


def mlstm_step(proj, gate_bias, c, state, m_state, slots=None):
    """One token per row against state[slots[b]] (slots None: row b is slot b), updated in place.  Returns (o, m) as `mlstm_scan`."""
    B = proj.shape[0]
    H, d, dv = c.n_heads, c.qk_dim, c.v_dim
    if use_native(proj) and d <= 1024:
        o = torch.empty(B, H, dv + 1, dtype=torch.float32, device=proj.device)
        mo = torch.empty(B, H, dtype=torch.float32, device=proj.device)
        lib().mlstm_scan(proj, gate_bias, o, mo, None, state, m_state, slots, H, d, dv, float(c.gate_cap), True)
        return o, mo
    return _mlstm_ref(proj, gate_bias, c, [(b, b + 1) for b in range(B)], state, m_state,
                      lambda n: int(slots[n]) if slots is not None else n, True)


def mlstm_out(o, m, w, gate, eps: float, out_dtype):
    """o [T, H, dv + 1] fp32 raw rows, m [T, H]: h = o[..., :dv] / (max(|o[..., dv]|, exp(-m)) + 1e-6); h / rms(h) per head; times
    w [H * dv] and sigmoid(gate [T, >= H * dv]) -> [T, H * dv] in out_dtype."""
    T, H, dvx = o.shape
    dv = dvx - 1
    if use_native(o):
        out = torch.empty(T, H * dv, dtype=out_dtype, device=o.device)
        lib().mlstm_out(o, m, w, gate, out, eps)
        return out
    den = torch.maximum(o[..., dv].abs(), torch.exp(-m)) + 1e-6
    h = o[..., :dv] / den.unsqueeze(-1)
    h = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps)
    return (h.reshape(T, H * dv) * w.float() * torch.sigmoid(gate[:, : H * dv].float())).to(out_dtype)


# ------------------------------------------------------------------------------------------------ decayed linear attention
# (`DecayConfig`: retention, lightning attention).  Per head, with a matrix state S [d, dv] in fp32 and a constant decay g_h:
#   S_t = g_h S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t          (no softmax, no denominator)
# The stages, each = PyTorch reference + sm_100a kernel (`csrc/decay.cu`):
#   decay_prepare   the projection row [q (H d) | k (H d) | v (H dv) | gate (H dv)] -> fp32 `u` [T, 2 H d + H dv] = [q | k | v]: SiLU on
#                   all three (`act`), or the rotation of q and k by the position (angles and products in fp32) and `k_scale` on k
#   decay_scan      the recurrence over every packed sequence from S = 0, or one token per row against the slots' states
#   decay_out       the output norm (per head without a weight, or over all heads with one), times silu / sigmoid of the gate


def decay_table(d, device) -> torch.Tensor:
    """fp32 [H] decays on `device` (cached on the config object)."""
    hit = getattr(d, "_decay_dev", None)
    if hit is None or hit.device != torch.device(device):
        hit = torch.tensor(d.decay, dtype=torch.float64).float().to(device)
        d._decay_dev = hit
    return hit


def _rotate_heads_ref(x, p, rot, inv_freq):
    """x [T, H, d] fp32: the first rot.dims dimensions of every head turn by p * f_i; pairs (i, i + dims / 2) or (2i, 2i + 1)."""
    n = rot.dims
    ang = p.float().unsqueeze(-1) * inv_freq                 # fp32 product, as the kernels form it
    cs, sn = torch.cos(ang).unsqueeze(1), torch.sin(ang).unsqueeze(1)
    out = x.clone()
    if rot.interleaved:
        a, b = x[..., 0:n:2], x[..., 1:n:2]
        out[..., 0:n:2] = a * cs - b * sn
        out[..., 1:n:2] = b * cs + a * sn
    else:
        a, b = x[..., : n // 2], x[..., n // 2:n]
        out[..., : n // 2] = a * cs - b * sn
        out[..., n // 2:n] = b * cs + a * sn
    return out


def decay_prepare(proj, d, pos=None, cache_lens=None, slots=None):
    """proj [T, >= d.width] (a view with its own row stride is fine) -> fp32 u [T, 2 H d + H dv].  Packed form: `pos` [T] int32; step
    form (`pos` None): row b's position is cache_lens[slots[b]] (slots None: cache_lens[b])."""
    from realhf_b200.ops.attention import rotary_table
    T = proj.shape[0]
    H, dk, dv = d.n_heads, d.qk_dim, d.v_dim
    nq, nv = H * dk, H * dv
    inv_freq = rotary_table(d.rotary, proj.device)[0] if d.rotary is not None else None
    if use_native(proj):
        u = torch.empty(T, 2 * nq + nv, dtype=torch.float32, device=proj.device)
        lib().decay_prepare(proj, u, pos, cache_lens if pos is None else None, slots if pos is None else None, inv_freq, H, dk, dv,
                            d.rotary.dims if d.rotary is not None else 0, bool(d.rotary.interleaved) if d.rotary is not None else False,
                            d.act == "silu", float(d.k_scale))
        return u
    x = proj[:, : 2 * nq + nv].float()
    if d.act == "silu":
        x = F.silu(x)
    q, k, v = x[:, :nq].reshape(T, H, dk), x[:, nq:2 * nq].reshape(T, H, dk), x[:, 2 * nq:]
    if d.rotary is not None:
        if pos is None:
            idx = slots.long() if slots is not None else torch.arange(T, device=proj.device)
            p = cache_lens[idx]
        else:
            p = pos
        q, k = _rotate_heads_ref(q, p, d.rotary, inv_freq), _rotate_heads_ref(k, p, d.rotary, inv_freq)
    k = k * torch.tensor(d.k_scale, dtype=torch.float32)
    return torch.cat([q.reshape(T, nq), k.reshape(T, nq), v], -1)


def _decay_ref(u, d, seqs, state, slot_of, load_state):
    T = u.shape[0]
    H, dk, dv = d.n_heads, d.qk_dim, d.v_dim
    nq = H * dk
    q, k, v = u[:, :nq].view(T, H, dk), u[:, nq:2 * nq].view(T, H, dk), u[:, 2 * nq:].view(T, H, dv)
    g = decay_table(d, u.device).view(H, 1, 1)
    o = torch.empty(T, H, dv, dtype=torch.float32, device=u.device)
    for n, (s0, e0) in enumerate(seqs):
        if e0 == s0:
            continue
        sl = slot_of(n)
        S = state[sl].clone() if load_state else torch.zeros(H, dk, dv, dtype=torch.float32, device=u.device)
        for t in range(s0, e0):
            S = g * S + k[t][:, :, None] * v[t][:, None, :]
            o[t] = torch.einsum("hdv,hd->hv", S, q[t])
        if state is not None:
            state[sl] = S
    return o


def decay_scan(u, d, cu_seqlens, state=None, seq_slot=None, load_state: bool = False):
    """Packed recurrence over every sequence from S = 0 (or, with `load_state`, from the slot's state); the final state is left in
    state[seq_slot[n]] ([n_slots, H, d, dv] fp32) when `state` is given.  Returns o [T, H, dv] fp32."""
    T = u.shape[0]
    if use_native(u) and d.qk_dim <= 1024:
        o = torch.empty(T, d.n_heads, d.v_dim, dtype=torch.float32, device=u.device)
        lib().decay_scan(u, decay_table(d, u.device), o, cu_seqlens, state, seq_slot if state is not None else None, d.n_heads, d.qk_dim,
                         d.v_dim, bool(load_state))
        return o
    cu = cu_seqlens.tolist()
    return _decay_ref(u, d, list(zip(cu[:-1], cu[1:])), state, lambda n: int(seq_slot[n]) if seq_slot is not None else n, load_state)


def decay_step(u, d, state, slots=None):
    """One token per row against state[slots[b]] (slots None: row b is slot b), updated in place.  Returns o [B, H, dv] fp32."""
    B = u.shape[0]
    if use_native(u) and d.qk_dim <= 1024:
        o = torch.empty(B, d.n_heads, d.v_dim, dtype=torch.float32, device=u.device)
        lib().decay_scan(u, decay_table(d, u.device), o, None, state, slots, d.n_heads, d.qk_dim, d.v_dim, True)
        return o
    return _decay_ref(u, d, [(b, b + 1) for b in range(B)], state, lambda n: int(slots[n]) if slots is not None else n, True)


def decay_out(o, d, w, gate, eps: float, out_dtype):
    """o [T, H, dv] fp32 -> [T, H * dv] in out_dtype: o / rms(o) per head (`out_norm` "head") or over all heads times w [H * dv]
    ("full"), then times silu(gate) or sigmoid(gate) (`gate` [T, >= H * dv], any row stride)."""
    T, H, dv = o.shape
    if use_native(o):
        out = torch.empty(T, H * dv, dtype=out_dtype, device=o.device)
        lib().decay_out(o, w if d.out_norm == "full" else None, gate, out, eps, d.out_norm == "full", d.gate == "silu")
        return out
    if d.out_norm == "full":
        h = o.reshape(T, H * dv)
        h = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    else:
        h = (o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps)).reshape(T, H * dv)
    g = gate[:, : H * dv].float()
    return (h * (F.silu(g) if d.gate == "silu" else torch.sigmoid(g))).to(out_dtype)
