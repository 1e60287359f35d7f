"""Attention entry points: packed varlen causal attention (train / inference / prefill) and
single-token decode attention over a dense KV cache.

CUDA tensors: decode runs the split-KV sm_100a kernel in `csrc/attn_decode.cu` (with fused RoPE and
in-place KV append); varlen forward runs `csrc/attn_fwd_tcgen05.cu` and backward `csrc/attn_bwd_tcgen05.cu`
(TMA + tcgen05 + TMEM; head dim 64 / 128, validated on B200 against the fp32 reference and the library kernel:
`profiles/attention_validation.log`).  The flash-attn library kernel is only the fallback for what the own
kernels do not cover (attention dropout, other head dims) and the A/B arm: `REAL_ATTN=flash` /
`REAL_ATTN_BWD=flash` select it explicitly; both produce / consume the same LSE layout.
CPU tensors: plain PyTorch reference (also the numerics oracle for the tests).
"""

from __future__ import annotations

import math
from typing import Optional

import torch

import os

from realhf_b200.ops import lib, use_native


def attn_impl() -> str:
    """`tcgen05` (own forward kernel, default) or `flash` (library kernel, A/B runs only)."""
    return os.environ.get("REAL_ATTN", "tcgen05")


def _own_fwd_ok(hd: int, dropout_p: float) -> bool:
    return attn_impl() == "tcgen05" and hd in (64, 128) and dropout_p == 0.0


def _own_bwd_ok(hd: int, dropout_p: float) -> bool:
    """`REAL_ATTN_BWD=tcgen05`: own backward (`csrc/attn_bwd_tcgen05.cu`), independent of the forward switch (both produce /
    consume the same LSE layout).  Default; `REAL_ATTN_BWD=flash` selects the library kernel."""
    return os.environ.get("REAL_ATTN_BWD", "tcgen05") == "tcgen05" and hd in (64, 128) and dropout_p == 0.0


def varlen_attention_ref(q, k, v, cu_seqlens, scale: float, causal: bool = True, sliding_window: Optional[int] = None):
    """q [T,nq,hd], k/v [T,nkv,hd] packed; fp32 math; returns [T,nq,hd] in q.dtype."""
    T, nq, hd = q.shape
    nkv = k.shape[1]
    rep = nq // nkv
    out = torch.empty_like(q)
    cu = cu_seqlens.tolist()
    for i in range(len(cu) - 1):
        s, e = cu[i], cu[i + 1]
        if e == s:
            continue
        qi = q[s:e].float().transpose(0, 1)                          # [nq, L, hd]
        ki = k[s:e].float().transpose(0, 1).repeat_interleave(rep, 0)
        vi = v[s:e].float().transpose(0, 1).repeat_interleave(rep, 0)
        att = (qi @ ki.transpose(1, 2)) * scale
        L = e - s
        if causal:
            idx = torch.arange(L, device=q.device)
            mask = idx[None, :] > idx[:, None]
            if sliding_window:
                mask |= idx[None, :] <= idx[:, None] - sliding_window
            att = att.masked_fill(mask, float("-inf"))
        out[s:e] = (torch.softmax(att, dim=-1) @ vi).transpose(0, 1).to(q.dtype)
    return out


def varlen_attention(q, k, v, cu_seqlens, max_seqlen: int, scale: Optional[float] = None, causal: bool = True,
                     dropout_p: float = 0.0):
    """Packed variable-length causal attention with GQA.  q [T,nq,hd]; k,v [T,nkv,hd]."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if use_native(q) and q.dtype in (torch.bfloat16, torch.float16):
        from flash_attn import flash_attn_varlen_func
        cu = cu_seqlens.int()
        if _own_fwd_ok(q.shape[-1], dropout_p) and not torch.is_grad_enabled() and all(
                t.stride(-1) == 1 and t.stride(1) == t.shape[-1] for t in (q, k, v)):
            return lib().attn_fwd(q, k, v, cu, max_seqlen, scale, causal)[0]
        return flash_attn_varlen_func(q, k, v, cu, cu, max_seqlen, max_seqlen, dropout_p=dropout_p,
                                      softmax_scale=scale, causal=causal)
    return varlen_attention_ref(q, k, v, cu_seqlens, scale, causal)


class _PackedQKVAttention(torch.autograd.Function):
    """Varlen attention on the fused projection output qkv [T, (nq + 2 nkv) * hd] (q heads | k heads | v heads).

    Slicing q / k / v out of `qkv` in autograd costs three zero-filled [T, 3H] buffers, three slice copies and two adds per
    layer in the backward pass (0.5 GB each at 20k tokens: ~3% of a 7B PPO step).  Here the backward kernel writes dq / dk / dv
    straight into views of ONE gradient buffer that is returned as d(qkv)."""

    @staticmethod
    def forward(ctx, qkv, cu, max_seqlen, nq, nkv, hd, scale, causal, dropout_p):
        from flash_attn.flash_attn_interface import _wrapped_flash_attn_varlen_forward
        T = qkv.shape[0]
        q = qkv[:, : nq * hd].view(T, nq, hd)
        k = qkv[:, nq * hd:(nq + nkv) * hd].view(T, nkv, hd)
        v = qkv[:, (nq + nkv) * hd:].view(T, nkv, hd)
        if _own_fwd_ok(hd, dropout_p):
            out, lse = lib().attn_fwd(q, k, v, cu, max_seqlen, scale, causal)
            ctx.save_for_backward(qkv, out, lse, cu, torch.empty(2, dtype=torch.int64, device=qkv.device))
            ctx.meta = (max_seqlen, nq, nkv, hd, scale, causal, dropout_p)
            return out
        out, lse, _, rng = _wrapped_flash_attn_varlen_forward(q, k, v, cu, cu, max_seqlen, max_seqlen, dropout_p, scale, causal=causal,
                                                              window_size_left=-1, window_size_right=-1, softcap=0.0, alibi_slopes=None,
                                                              return_softmax=False, block_table=None)
        ctx.save_for_backward(qkv, out, lse, cu, rng)
        ctx.meta = (max_seqlen, nq, nkv, hd, scale, causal, dropout_p)
        return out

    @staticmethod
    def backward(ctx, dout):
        from flash_attn.flash_attn_interface import _wrapped_flash_attn_varlen_backward
        qkv, out, lse, cu, rng = ctx.saved_tensors
        max_seqlen, nq, nkv, hd, scale, causal, dropout_p = ctx.meta
        T = qkv.shape[0]
        q = qkv[:, : nq * hd].view(T, nq, hd)
        k = qkv[:, nq * hd:(nq + nkv) * hd].view(T, nkv, hd)
        v = qkv[:, (nq + nkv) * hd:].view(T, nkv, hd)
        dqkv = torch.empty_like(qkv)
        dq = dqkv[:, : nq * hd].view(T, nq, hd)
        dk = dqkv[:, nq * hd:(nq + nkv) * hd].view(T, nkv, hd)
        dv = dqkv[:, (nq + nkv) * hd:].view(T, nkv, hd)
        if _own_bwd_ok(hd, dropout_p):
            lib().attn_bwd(dout.contiguous().view(T, nq, hd), q, k, v, out.view(T, nq, hd), lse, dq, dk, dv, cu, max_seqlen, scale, causal)
            return dqkv, None, None, None, None, None, None, None, None
        _wrapped_flash_attn_varlen_backward(dout.contiguous(), q, k, v, out, lse, dq, dk, dv, cu, cu, max_seqlen, max_seqlen, dropout_p,
                                            scale, causal, -1, -1, 0.0, None, False, rng_state=rng)
        return dqkv, None, None, None, None, None, None, None, None


def varlen_attention_qkv(qkv, cu_seqlens, max_seqlen: int, nq: int, nkv: int, hd: int, scale: Optional[float] = None,
                         causal: bool = True, dropout_p: float = 0.0):
    """Packed varlen attention taking the fused [T, (nq + 2 nkv) * hd] projection; returns [T, nq, hd]."""
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    T = qkv.shape[0]
    if use_native(qkv) and qkv.dtype in (torch.bfloat16, torch.float16) and qkv.stride(-1) == 1 and hd % 8 == 0:
        return _PackedQKVAttention.apply(qkv, cu_seqlens.int(), max_seqlen, nq, nkv, hd, scale, causal, dropout_p)
    q = qkv[:, : nq * hd].view(T, nq, hd)
    k = qkv[:, nq * hd:(nq + nkv) * hd].view(T, nkv, hd)
    v = qkv[:, (nq + nkv) * hd:].view(T, nkv, hd)
    return varlen_attention(q, k, v, cu_seqlens, max_seqlen, scale, causal, dropout_p)


def decode_attention_ref(q, k_cache, v_cache, cache_lens, scale: float):
    """q [B,nq,hd]; caches [B,S,nkv,hd]; cache_lens [B] = number of valid positions (incl. the new token)."""
    B, nq, hd = q.shape
    nkv = k_cache.shape[2]
    rep = nq // nkv
    S = k_cache.shape[1]
    kk = k_cache.float().permute(0, 2, 1, 3).repeat_interleave(rep, 1)   # [B,nq,S,hd]
    vv = v_cache.float().permute(0, 2, 1, 3).repeat_interleave(rep, 1)
    att = torch.einsum("bhd,bhsd->bhs", q.float(), kk) * scale
    mask = torch.arange(S, device=q.device)[None, :] >= cache_lens[:, None].to(q.device)
    att = att.masked_fill(mask[:, None, :], float("-inf"))
    return torch.einsum("bhs,bhsd->bhd", torch.softmax(att, -1), vv).to(q.dtype)


def decode_attention(qkv, k_cache, v_cache, cache_lens, n_q: int, n_kv: int, hd: int, scale: Optional[float] = None,
                     cos=None, sin=None, rot_dim: Optional[int] = None, interleaved: bool = False):
    """One decode step for B sequences.

    qkv: [B, (n_q+2*n_kv)*hd] fused projection of the new token.  `cache_lens[b]` is the number of tokens
    already in the cache (= position of the new token).  The op applies RoPE to q and k (if cos/sin given),
    writes the new k,v at position cache_lens[b] of the caches *in place*, and returns attention over
    positions [0, cache_lens[b]] as [B, n_q*hd].  Does not advance cache_lens.
    """
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    B = qkv.shape[0]
    if use_native(qkv) and qkv.dtype in (torch.bfloat16, torch.float16) and hd in (64, 128) \
            and k_cache.dtype == qkv.dtype:
        return lib().decode_attention(qkv, k_cache, v_cache, cache_lens.int(), n_q, n_kv, hd, scale, cos, sin,
                                      rot_dim or hd, interleaved)
    # reference path
    from realhf_b200.ops.functional import rope_ref
    x = qkv
    if cos is not None:
        x = rope_ref(qkv, cos, sin, cache_lens, n_q + n_kv, hd, rot_dim or hd, interleaved)
    q = x[:, : n_q * hd].reshape(B, n_q, hd)
    k = x[:, n_q * hd:(n_q + n_kv) * hd].reshape(B, n_kv, hd)
    v = x[:, (n_q + n_kv) * hd:].reshape(B, n_kv, hd)
    idx = torch.arange(B, device=qkv.device)
    pos = cache_lens.long()
    k_cache[idx, pos] = k.to(k_cache.dtype)
    v_cache[idx, pos] = v.to(v_cache.dtype)
    return decode_attention_ref(q, k_cache, v_cache, cache_lens + 1, scale).reshape(B, n_q * hd)


# ------------------------------------------------------------------------------------------------ latent attention
# Keys and values are up-projections of one cached low-rank latent per token; no positional rotation; optional sliding window.
# The latent cache of a slot is a ring of R rows: position p lives in row p % R (R >= the largest window that reads it, or the
# whole sequence length when some reader has no window).


def latent_norm_store_ref(qc, n_q, w_ln, eps, cache, tok_slot, pos, remain):
    c = qc[:, n_q:].float()
    c = c * torch.rsqrt(c.pow(2).mean(-1, keepdim=True) + eps) * w_ln.float()
    c = c.to(qc.dtype)
    if cache is not None:
        keep = (tok_slot >= 0) & (remain < cache.shape[1])
        cache[tok_slot[keep].long(), (pos[keep] % cache.shape[1]).long()] = c[keep].to(cache.dtype)
    return c


def latent_norm_store(qc, n_q: int, w_ln, eps: float, cache, tok_slot, pos, remain):
    """Packed prefill: c = RMSNorm(qc[:, n_q:]) * w_ln (one group, fp32 math) -> [T, rank] in qc's dtype, also written to
    cache[tok_slot[t], pos[t] % R] for the tokens with tok_slot >= 0 that are among the last R of their sequence
    (`remain[t]` < R: earlier positions would overwrite ring rows that later ones own)."""
    if use_native(qc):
        return lib().latent_norm_store(qc, n_q, w_ln, eps, cache, tok_slot if cache is not None else None, pos,
                                       remain if cache is not None else None)
    return latent_norm_store_ref(qc, n_q, w_ln, eps, cache, tok_slot, pos, remain)


def latent_window_attention_ref(q, kv, pos, n_heads, qk, vd, scale, window):
    """q [T, >= n_heads*qk] (leading columns used), kv [T, n_heads*(qk+vd)] = [keys | values] head by head, pos [T]."""
    T = q.shape[0]
    qh = q[:, : n_heads * qk].float().reshape(T, n_heads, qk)
    kh = kv[:, : n_heads * qk].float().reshape(T, n_heads, qk)
    vh = kv[:, n_heads * qk:].float().reshape(T, n_heads, vd)
    att = torch.einsum("ihd,jhd->hij", qh, kh) * scale
    idx = torch.arange(T, device=q.device)
    dist = idx[:, None] - idx[None, :]
    ok = (dist >= 0) & (dist <= pos.long()[:, None])
    if window is not None:
        ok &= dist < window
    att = att.masked_fill(~ok[None], float("-inf"))
    return torch.einsum("hij,jhd->ihd", torch.softmax(att, -1), vh).reshape(T, n_heads * vd).to(q.dtype)


def _tcgen05_window_ok(q, kv, n_heads, qk, vd) -> bool:
    """The tcgen05 varlen kernel takes 16-bit operands with equal query / value head dims of 64 or 128 and 16-byte aligned rows."""
    return (os.environ.get("REAL_LATENT_ATTN", "tcgen05") == "tcgen05" and q.dtype in (torch.bfloat16, torch.float16) and qk == vd
            and qk in (64, 128) and q.stride(1) == 1 and kv.stride(1) == 1 and q.stride(0) % 8 == 0 and kv.stride(0) % 8 == 0
            and q.data_ptr() % 16 == 0 and kv.data_ptr() % 16 == 0)


def latent_window_attention(q, kv, pos, n_heads: int, qk: int, vd: int, scale: float, window: Optional[int], cu_seqlens=None,
                            max_seqlen: Optional[int] = None):
    """Packed prefill attention: token t attends the tokens t - d of its own sequence with 0 <= d <= pos[t] and d < window.
    Scores and softmax are fp32.  Returns [T, n_heads * vd] in q's dtype.  CUDA: 16-bit operands with equal head dims of 64 / 128
    run the tcgen05 varlen kernel with its sliding-window mask (needs `cu_seqlens`, `max_seqlen`; the softmax weights are rounded
    to the operand type for the P V product on the tensor cores, like the V operand itself); every other shape, and fp32, runs
    the CUDA-core kernel of `csrc/latent_attn.cu`, which keeps the weights and the sum in fp32."""
    if use_native(q):
        if cu_seqlens is not None and max_seqlen is not None and _tcgen05_window_ok(q, kv, n_heads, qk, vd):
            T = q.shape[0]
            qv = q[:, : n_heads * qk].view(T, n_heads, qk)
            kk = kv[:, : n_heads * qk].view(T, n_heads, qk)
            vv = kv[:, n_heads * qk:].view(T, n_heads, vd)
            out = lib().attn_fwd_window(qv, kk, vv, cu_seqlens, max_seqlen, scale, True, window if window is not None else 0)[0]
            return out.view(T, n_heads * vd)
        if vd <= 256 and (16 * qk + 32 * (qk + 1) + 32 * vd + 512) * 4 <= 200 * 1024:
            return lib().latent_window_attention(q, kv, pos, n_heads, qk, vd, scale, window if window is not None else 0)
        # head dims beyond the kernel's shared-memory tiles: the reference formula on the device, sequence by sequence
        out = torch.empty(q.shape[0], n_heads * vd, dtype=q.dtype, device=q.device)
        starts = torch.nonzero(pos == 0).flatten().tolist() + [q.shape[0]]
        for a, b in zip(starts[:-1], starts[1:]):
            out[a:b] = latent_window_attention_ref(q[a:b], kv[a:b], pos[a:b], n_heads, qk, vd, scale, window)
        return out
    return latent_window_attention_ref(q, kv, pos, n_heads, qk, vd, scale, window)


def _absorbed_projections(w_ukv, n_heads: int, qk: int, vd: int, scale: float):
    """fp32 per-head forms of the fused [key | value] up-projection for decode: W_uk * scale as [H, qk, rank] (queries go INTO the
    latent space) and W_uv^T as [H, rank, vd] (latent sums come out of it).  Cached on the weight tensor."""
    from realhf_b200.ops.functional import cached_on

    def build(w):
        rank, n_q = w.shape[1], n_heads * qk
        wk = (w[:n_q].reshape(n_heads, qk, rank).float() * scale).contiguous()
        wv = w[n_q:].reshape(n_heads, vd, rank).float().transpose(1, 2).contiguous()
        return wk, wv
    return cached_on(w_ukv, f"_absorbed_{n_heads}_{qk}_{vd}_{float(scale)!r}", build)


def latent_decode_attention_ref(qc, w_ln, w_ukv, cache, cache_lens, slots, n_heads, qk, vd, scale, window, eps):
    B = qc.shape[0]
    n_q = n_heads * qk
    R = cache.shape[1]
    idx = slots.long() if slots is not None else torch.arange(B, device=qc.device)
    pos = cache_lens[idx].long()
    if w_ln is not None:
        c = qc[:, n_q:].float()
        c = c * torch.rsqrt(c.pow(2).mean(-1, keepdim=True) + eps) * w_ln.float()
        cache[idx, pos % R] = c.to(cache.dtype)
    wk = w_ukv[:n_q].float().reshape(n_heads, qk, -1)
    wv = w_ukv[n_q:].float().reshape(n_heads, vd, -1)
    out = torch.empty(B, n_heads * vd, dtype=torch.float32, device=qc.device)
    for b in range(B):
        p = int(pos[b])
        lo = 0 if window is None else max(0, p - window + 1)
        rows = torch.arange(lo, p + 1, device=qc.device) % R
        cw = cache[idx[b], rows].float()                                  # [n, rank]
        qa = torch.einsum("hd,hdr->hr", qc[b, :n_q].float().reshape(n_heads, qk), wk)   # queries absorbed into the latent space
        pr = torch.softmax((qa @ cw.t()) * scale, -1)                     # [h, n]
        out[b] = torch.einsum("hr,hvr->hv", pr @ cw, wv).reshape(-1)
    return out.to(qc.dtype)


def latent_decode_attention(qc, w_ln, w_ukv, cache, cache_lens, slots, n_heads: int, qk: int, vd: int, scale: float,
                            window: Optional[int], eps: float):
    """One decode step of latent attention for B rows.  qc [B, n_heads*qk (+ rank)] is the fused query | latent projection of
    the new token, whose position is cache_lens[slot].  With `w_ln` the row's latent is normalised and written to the cache
    first (a block that projects its own latent); without, the cache already holds it (a block that reads another block's).
    Keys and values are never formed: the query is multiplied into the latent space (q W_uk), scores and the weighted sum run
    over the cached latents of the window, and W_uv is applied to the result.  Does not advance cache_lens."""
    if use_native(qc):
        rank, R, B = cache.shape[2], cache.shape[1], qc.shape[0]
        if rank > 512:  # beyond both kernels' register / shared-memory tiles: the reference formula on the device
            return latent_decode_attention_ref(qc, w_ln, w_ukv, cache, cache_lens, slots, n_heads, qk, vd, scale, window, eps)
        if os.environ.get("REAL_LATENT_DECODE", "split") == "fused":
            # one launch per (row, head): small problems / A-B runs
            return lib().latent_decode_attention(qc, w_ln, w_ukv, cache, cache_lens, slots, n_heads, qk, vd, scale,
                                                 window if window is not None else 0, eps)
        n_q = n_heads * qk
        if w_ln is not None:
            lib().latent_append(qc, n_q, w_ln, cache, cache_lens, slots, eps)
        wk, wv = _absorbed_projections(w_ukv, n_heads, qk, vd, scale)
        qa = torch.bmm(qc[:, :n_q].reshape(B, n_heads, qk).transpose(0, 1).float(), wk)           # [H, B, rank] fp32
        # enough CTAs to fill the GPU (three fit an SM): split the keys when rows x head tiles are few; a split is at least two
        # 32-key tiles
        ctas = B * ((n_heads + 15) // 16)
        splits = max(1, min((3 * 148 + ctas - 1) // ctas, R // 64, 32))
        o = lib().latent_decode_core(qa, cache, cache_lens, slots, window if window is not None else 0, splits)
        return torch.bmm(o, wv).transpose(0, 1).reshape(B, n_heads * vd).to(qc.dtype)
    return latent_decode_attention_ref(qc, w_ln, w_ukv, cache, cache_lens, slots, n_heads, qk, vd, scale, window, eps)


# ------------------------------------------------------------------------------------------------ window attention with a sink
# (`WindowAttentionConfig`): grouped key / value heads, no rotation; per-head temperature, linear distance penalty, sliding window
# that keeps the first tokens, sink logit in the denominator, sigmoid output gate.  Scores, weights and the value norm are fp32.
# The projection output `qkvg` [T, ld] holds [q (H x d) | k (G x d) | v (G x dv) | gate logits (H, padded)] per row.
# Caches: k_cache [n_slots, G, rows, d], v_cache [n_slots, G, rows, dv]; position p of a sequence lives in row p when
# p < keep_first, else in row keep_first + (p - keep_first) % (rows - keep_first).


def cache_row(pos, keep_first: int, rows: int):
    ring = max(rows - keep_first, 1)
    if isinstance(pos, torch.Tensor):
        return torch.where(pos < keep_first, pos, keep_first + (pos - keep_first) % ring)
    return pos if pos < keep_first else keep_first + (pos - keep_first) % ring


def head_slopes(n_heads: int, slope_base: Optional[float], device) -> torch.Tensor:
    """fp32 [n_heads]: 2^(-slope_base (h + 1) / n_heads), zeros without a distance term."""
    if slope_base is None:
        return torch.zeros(n_heads, dtype=torch.float32, device=device)
    return torch.exp2(-slope_base * torch.arange(1, n_heads + 1, dtype=torch.float32, device=device) / n_heads)


def _wa_offsets(a):
    nq, nk, nv = a.n_heads * a.qk_dim, a.n_kv_heads * a.qk_dim, a.n_kv_heads * a.v_dim
    return nq, nq + nk, nq + nk + nv


def value_norm_store_ref(qkvg, a, eps, k_cache, v_cache, tok_slot, pos, remain):
    T = qkvg.shape[0]
    oq, ok_, ov = _wa_offsets(a)
    v = qkvg[:, ok_:ov].float().view(T, a.n_kv_heads, a.v_dim)
    if a.value_norm:
        v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)
    v = v.to(qkvg.dtype)
    if k_cache is not None:
        rows = k_cache.shape[2]
        ring = rows - a.keep_first
        keep = (tok_slot >= 0) & ((pos < a.keep_first) | (remain < ring))
        r = cache_row(pos.long(), a.keep_first, rows)[keep]
        s = tok_slot[keep].long()
        k_cache[s, :, r] = qkvg[keep, oq:ok_].view(-1, a.n_kv_heads, a.qk_dim)
        v_cache[s, :, r] = v[keep]
    return v.reshape(T, a.n_kv_heads * a.v_dim)


def value_norm_store(qkvg, a, eps: float, k_cache, v_cache, tok_slot, pos, remain):
    """Packed prefill: the value heads of `qkvg`, each divided by its root mean square (fp32; `a.value_norm`), as [T, G * dv] in
    the model dtype; with caches, also writes every token's key and normalised value that a later decode step can still see
    (the first `keep_first` positions and the last `rows - keep_first` of each sequence) into its slot."""
    if use_native(qkvg):
        T = qkvg.shape[0]
        out = torch.empty(T, a.n_kv_heads * a.v_dim, dtype=qkvg.dtype, device=qkvg.device)
        lib().value_norm_store(qkvg, out, k_cache, v_cache, tok_slot if k_cache is not None else None, pos,
                               remain if k_cache is not None else None, a.n_heads, a.n_kv_heads, a.qk_dim, a.v_dim, a.keep_first,
                               bool(a.value_norm), eps)
        return out
    return value_norm_store_ref(qkvg, a, eps, k_cache, v_cache, tok_slot, pos, remain)


def rotate_qk_(qkv, a, pos=None, cache_lens=None, slots=None):
    """In place: the (n_heads + n_kv_heads) query / key heads at the start of every row of `qkv` [T, ld] are rotated by the row's
    position over the first `a.rotary.dims` dimensions (angle = position * f_i as an fp32 product, exact sin / cos; the rotated
    values are stored in the tensor's dtype).  Packed form: `pos` [T] int32; step form (`pos` None): row b's position is
    cache_lens[slots[b]] (slots None: cache_lens[b]).  Keys are therefore cached rotated."""
    rot = a.rotary
    inv_freq = rotary_table(rot, qkv.device)[0]
    n_h = a.n_heads + a.n_kv_heads
    if use_native(qkv):
        lib().rotate_heads_(qkv, pos, cache_lens if pos is None else None, slots if pos is None else None, inv_freq, n_h, a.qk_dim, rot.dims,
                            bool(rot.interleaved))
        return qkv
    from realhf_b200.ops.recurrent import _rotate_heads_ref
    T = qkv.shape[0]
    if pos is None:
        idx = slots.long() if slots is not None else torch.arange(T, device=qkv.device)
        pos = cache_lens[idx]
    x = qkv[:, : n_h * a.qk_dim].float().reshape(T, n_h, a.qk_dim)
    qkv[:, : n_h * a.qk_dim] = _rotate_heads_ref(x, pos, rot, inv_freq).reshape(T, -1).to(qkv.dtype)
    return qkv


def _sink_softmax_pv(s, ok, sink_h, v):
    """fp32 scores s [Lq, Lk], visibility ok, sink logit (tensor scalar or None) -> softmax-with-sink weights @ v."""
    s = s.masked_fill(~ok, float("-inf"))
    mx = s.max(-1, keepdim=True).values
    if sink_h is not None:
        mx = torch.maximum(mx, sink_h)
    mx = torch.where(torch.isfinite(mx), mx, torch.zeros_like(mx))
    e = torch.exp(s - mx)
    den = e.sum(-1, keepdim=True)
    if sink_h is not None:
        den = den + torch.exp(sink_h - mx)
    return (e / den) @ v


def sink_window_attention_ref(qkvg, v_n, a, temp, sink, cu_seqlens):
    T = qkvg.shape[0]
    H, G, d, dv = a.n_heads, a.n_kv_heads, a.qk_dim, a.v_dim
    oq, ok_, ov = _wa_offsets(a)
    q = qkvg[:, :oq].float().view(T, H, d)
    k = qkvg[:, oq:ok_].float().view(T, G, d)
    v = v_n.float().view(T, G, dv)
    gate = torch.sigmoid(qkvg[:, ov:ov + H].float()) if a.out_gate else None
    slopes = head_slopes(H, a.slope_base, qkvg.device)
    out = torch.zeros(T, H, dv, dtype=torch.float32, device=qkvg.device)
    cu = cu_seqlens.tolist()
    for b in range(len(cu) - 1):
        s0, e0 = cu[b], cu[b + 1]
        if e0 == s0:
            continue
        L = e0 - s0
        i = torch.arange(L, device=qkvg.device).unsqueeze(1)
        j = torch.arange(L, device=qkvg.device).unsqueeze(0)
        ok = j <= i
        if a.window is not None:
            ok = ok & ((i - j < a.window) | (j < a.keep_first))
        dist = (i - j).float()
        for h in range(H):
            g = h // (H // G)
            sc = (q[s0:e0, h] @ k[s0:e0, g].T) * a.scale
            if temp is not None:
                sc = sc * temp[h].float()
            sc = sc - slopes[h] * dist
            out[s0:e0, h] = _sink_softmax_pv(sc, ok, sink[h].float() if sink is not None else None, v[s0:e0, g])
    if gate is not None:
        out = out * gate.unsqueeze(-1)
    return out.reshape(T, H * dv).to(qkvg.dtype)


def _sink_tc_ok(qkvg, v_n, a) -> bool:
    """The tcgen05 form takes 16-bit operands with equal query / value head size of 64 or 128 (softmax statistics in fp32, the
    weights rounded to the operand type for the P.V product); `REAL_WINDOW_ATTN=simt` selects the all-fp32 CUDA-core kernel."""
    return (os.environ.get("REAL_WINDOW_ATTN", "tcgen05") == "tcgen05" and qkvg.dtype in (torch.bfloat16, torch.float16)
            and a.qk_dim == a.v_dim and a.qk_dim in (64, 128) and qkvg.stride(0) % 8 == 0 and qkvg.data_ptr() % 16 == 0
            and (a.n_heads * a.qk_dim) % 8 == 0 and v_n.data_ptr() % 16 == 0)


def sink_window_attention(qkvg, v_n, a, temp, sink, pos, cu_seqlens, max_seqlen=None):
    """Packed causal attention of a window-attention block over the batch's own keys (every sequence starts at position 0):
    softmax_j(q_i . k_j * scale * temp_h - slope_h (i - j)) with the sink logit in the denominator, over j <= i with
    i - j < window or j < keep_first; head h's output times sigmoid(gate logit h).  Returns [T, H * dv] in the model dtype."""
    if use_native(qkvg) and a.qk_dim <= 512 and a.v_dim <= 256:     # (larger heads: the PyTorch form, on the device)
        T = qkvg.shape[0]
        out = torch.empty(T, a.n_heads * a.v_dim, dtype=qkvg.dtype, device=qkvg.device)
        if max_seqlen is None:
            max_seqlen = int((cu_seqlens[1:] - cu_seqlens[:-1]).max())
        if _sink_tc_ok(qkvg, v_n, a):
            lib().sink_window_attention_tc(qkvg, v_n, out, temp, sink, cu_seqlens, max_seqlen, a.n_heads, a.n_kv_heads, a.qk_dim, a.scale,
                                           a.window if a.window is not None else -1, a.keep_first,
                                           a.slope_base if a.slope_base is not None else -1.0, bool(a.out_gate))
            return out
        lib().sink_window_attention(qkvg, v_n, out, temp, sink, cu_seqlens, max_seqlen, a.n_heads, a.n_kv_heads, a.qk_dim, a.v_dim, a.scale,
                                    a.window if a.window is not None else -1, a.keep_first,
                                    a.slope_base if a.slope_base is not None else -1.0, bool(a.out_gate))
        return out
    return sink_window_attention_ref(qkvg, v_n, a, temp, sink, cu_seqlens)


def sink_window_decode_attention_ref(qkvg, a, temp, sink, k_cache, v_cache, cache_lens, slots, eps):
    B = qkvg.shape[0]
    H, G, d, dv = a.n_heads, a.n_kv_heads, a.qk_dim, a.v_dim
    oq, ok_, ov = _wa_offsets(a)
    rows = k_cache.shape[2]
    slopes = head_slopes(H, a.slope_base, qkvg.device)
    out = torch.zeros(B, H, dv, dtype=torch.float32, device=qkvg.device)
    for b in range(B):
        s = int(slots[b]) if slots is not None else b
        n = int(cache_lens[s])                                     # the new token's position
        v_new = qkvg[b, ok_:ov].float().view(G, dv)
        if a.value_norm:
            v_new = v_new * torch.rsqrt(v_new.pow(2).mean(-1, keepdim=True) + eps)
        r = cache_row(n, a.keep_first, rows)
        k_cache[s, :, r] = qkvg[b, oq:ok_].view(G, d)
        v_cache[s, :, r] = v_new.to(v_cache.dtype)
        j = torch.arange(n + 1, device=qkvg.device)
        if a.window is not None:
            j = j[(n - j < a.window) | (j < a.keep_first)]
        rj = cache_row(j, a.keep_first, rows)
        kk = k_cache[s][:, rj].float()                             # [G, n_keys, d]
        vv = v_cache[s][:, rj].float()
        q = qkvg[b, :oq].float().view(H, d)
        for h in range(H):
            g = h // (H // G)
            sc = (kk[g] @ q[h]) * a.scale
            if temp is not None:
                sc = sc * temp[h].float()
            sc = (sc - slopes[h] * (n - j).float()).unsqueeze(0)
            out[b, h] = _sink_softmax_pv(sc, torch.ones_like(sc, dtype=torch.bool), sink[h].float() if sink is not None else None, vv[g])[0]
        if a.out_gate:
            out[b] = out[b] * torch.sigmoid(qkvg[b, ov:ov + H].float()).unsqueeze(-1)
    return out.reshape(B, H * dv).to(qkvg.dtype)


def sink_window_decode_attention(qkvg, a, temp, sink, k_cache, v_cache, cache_lens, slots, eps: float):
    """One new token per row against the caches of its slot (slots None: row b is slot b).  The row's key and normalised value
    are appended in place at the row of position cache_lens[slot] (cache_lens itself is not changed), then the token attends to
    every cached position its window and `keep_first` allow, itself included.  Returns [B, H * dv] in the model dtype."""
    if use_native(qkvg) and a.v_dim <= 256:
        B = qkvg.shape[0]
        out = torch.empty(B, a.n_heads * a.v_dim, dtype=qkvg.dtype, device=qkvg.device)
        lib().sink_window_decode_attention(qkvg, out, temp, sink, k_cache, v_cache, cache_lens, slots, a.n_heads, a.n_kv_heads, a.qk_dim,
                                           a.v_dim, a.scale, a.window if a.window is not None else -1, a.keep_first,
                                           a.slope_base if a.slope_base is not None else -1.0, bool(a.out_gate), bool(a.value_norm), eps)
        return out
    return sink_window_decode_attention_ref(qkvg, a, temp, sink, k_cache, v_cache, cache_lens, slots, eps)


# ------------------------------------------------------------------------------------------------ differential window attention
# (`WindowAttentionConfig` with n_maps = 2).  The projection row holds [q (H x 2 x d) | k (G x 2 x d) | v (G x dv)]; the query heads are
# stored grouped by key head and map, (g, map, head within the group), so that the kernels see 2H query heads over 2G key heads with
# the ordinary grouping, two consecutive key heads sharing a value head.  Caches: k [n_slots, 2G, rows, d], v [n_slots, G, rows, dv].


def diff_lambda(w_lambda, diff: float):
    """fp32 [1] on the weight's device: exp(lq1 . lk1) - exp(lq2 . lk2) + diff from the [4, d] parameter (lq1, lk1, lq2, lk2)."""
    from realhf_b200.ops.functional import cached_on

    def build(w):
        f = w.float()
        return (torch.exp((f[0] * f[1]).sum()) - torch.exp((f[2] * f[3]).sum()) + diff).reshape(1).contiguous()
    return cached_on(w_lambda, f"_lambda_{float(diff)!r}", build)


def _diff_view(a):
    """The kernels' view of a differential block: every (head, map) is a head."""
    import copy
    v = copy.copy(a)
    v.n_heads, v.n_kv_heads, v.n_maps = a.n_heads * 2, a.n_kv_heads * 2, 1
    return v


def _qk_head_norm_ref(qkv, wq, wk, nq, nk, d, eps):
    T = qkv.shape[0]
    x = qkv[:, : (nq + nk) * d].float().view(T, nq + nk, d)
    x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    w = torch.cat([wq.float().expand(nq, d), wk.float().expand(nk, d)], 0)
    qkv[:, : (nq + nk) * d] = (x * w).reshape(T, -1).to(qkv.dtype)


def _diff_combine_ref(att, lam, H, G, dv, diff, eps, out_dtype):
    T = att.shape[0]
    per = H // G
    x = att.float().view(T, G, 2, per, dv)
    o = (x[:, :, 0] - lam.float() * x[:, :, 1]).reshape(T, H, dv)
    o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps) * (1.0 - diff)
    return o.reshape(T, H * dv).to(out_dtype)


def diff_window_attention(qkv, a, wq, wk, w_lambda, eps: float, k_cache, v_cache, tok_slot, pos, remain, cu_seqlens, max_seqlen=None):
    """Packed differential attention of a block's own tokens (sequences start at position 0).  `qkv` is normalised IN PLACE
    (query / key heads); with caches, the rows a later decode step can still see are stored.  Returns [T, H * dv] in qkv's dtype."""
    H, G, d, dv = a.n_heads, a.n_kv_heads, a.qk_dim, a.v_dim
    T = qkv.shape[0]
    lam = diff_lambda(w_lambda, a.diff)
    av = _diff_view(a)
    win = a.window if a.window is not None else -1
    if use_native(qkv) and d <= 512 and dv <= 256:
        lib().qk_head_norm_(qkv, wq, wk, 2 * H, 2 * G, d, eps)
        v_n = torch.empty(T, G * dv, dtype=qkv.dtype, device=qkv.device)
        lib().value_norm_store(qkv, v_n, k_cache, v_cache, tok_slot if k_cache is not None else None, pos,
                               remain if k_cache is not None else None, 2 * H, 2 * G, d, dv, a.keep_first, False, eps, 2)
        if max_seqlen is None:
            max_seqlen = int((cu_seqlens[1:] - cu_seqlens[:-1]).max())
        if _sink_tc_ok(qkv, v_n, av):
            # 16-bit operands, head size 64 / 128: the tcgen05 kernel; both maps' weighted sums come back in the operand type
            att = torch.empty(T, 2 * H * dv, dtype=qkv.dtype, device=qkv.device)
            lib().sink_window_attention_tc(qkv, v_n, att, None, None, cu_seqlens, max_seqlen, 2 * H, 2 * G, d, a.scale, win, a.keep_first, -1.0, False, 2)
        else:
            att = torch.empty(T, 2 * H * dv, dtype=torch.float32, device=qkv.device)
            lib().sink_window_attention(qkv, v_n, att, None, None, cu_seqlens, max_seqlen, 2 * H, 2 * G, d, dv, a.scale, win, a.keep_first, -1.0, False, 2)
        out = torch.empty(T, H * dv, dtype=qkv.dtype, device=qkv.device)
        lib().diff_combine(att, lam, out, H, G, dv, a.diff, eps)
        return out
    _qk_head_norm_ref(qkv, wq, wk, 2 * H, 2 * G, d, eps)
    oq, ok_ = 2 * H * d, 2 * (H + G) * d
    if k_cache is not None:
        rows = k_cache.shape[2]
        keep = (tok_slot >= 0) & ((pos < a.keep_first) | (remain < rows - a.keep_first))
        r = cache_row(pos.long(), a.keep_first, rows)[keep]
        s = tok_slot[keep].long()
        k_cache[s, :, r] = qkv[keep, oq:ok_].view(-1, 2 * G, d)
        v_cache[s, :, r] = qkv[keep, ok_:ok_ + G * dv].view(-1, G, dv)
    q = qkv[:, :oq].float().view(T, 2 * H, d)
    k = qkv[:, oq:ok_].float().view(T, 2 * G, d)
    v = qkv[:, ok_:ok_ + G * dv].float().view(T, G, dv)
    att = torch.zeros(T, 2 * H, dv, dtype=torch.float32, device=qkv.device)
    cu = cu_seqlens.tolist()
    for b in range(len(cu) - 1):
        s0, e0 = cu[b], cu[b + 1]
        L = e0 - s0
        if L == 0:
            continue
        i = torch.arange(L, device=qkv.device).unsqueeze(1)
        j = torch.arange(L, device=qkv.device).unsqueeze(0)
        ok = j <= i
        if a.window is not None:
            ok = ok & ((i - j < a.window) | (j < a.keep_first))
        for h in range(2 * H):
            g = h // (H // G)
            sc = (q[s0:e0, h] @ k[s0:e0, g].T) * a.scale
            att[s0:e0, h] = _sink_softmax_pv(sc, ok, None, v[s0:e0, g // 2])
    return _diff_combine_ref(att.reshape(T, -1), lam, H, G, dv, a.diff, eps, qkv.dtype)


def diff_window_decode_attention(qkv, a, wq, wk, w_lambda, eps: float, k_cache, v_cache, cache_lens, slots):
    """One new token per row: normalises the row's query / key heads in place, appends key and value at the row of position
    cache_lens[slot] and attends to the window (both maps), then combines.  Returns [B, H * dv]."""
    H, G, d, dv = a.n_heads, a.n_kv_heads, a.qk_dim, a.v_dim
    B = qkv.shape[0]
    lam = diff_lambda(w_lambda, a.diff)
    if use_native(qkv) and dv <= 256:
        lib().qk_head_norm_(qkv, wq, wk, 2 * H, 2 * G, d, eps)
        fast = qkv.dtype != torch.float32 and d == dv and d in (64, 128) and (H // G) in (1, 2, 4, 8)    # the streaming 16-bit kernel
        att = torch.empty(B, 2 * H * dv, dtype=qkv.dtype if fast else torch.float32, device=qkv.device)
        lib().sink_window_decode_attention(qkv, att, None, None, k_cache, v_cache, cache_lens, slots, 2 * H, 2 * G, d, dv, a.scale,
                                           a.window if a.window is not None else -1, a.keep_first, -1.0, False, False, eps, 2)
        out = torch.empty(B, H * dv, dtype=qkv.dtype, device=qkv.device)
        lib().diff_combine(att, lam, out, H, G, dv, a.diff, eps)
        return out
    _qk_head_norm_ref(qkv, wq, wk, 2 * H, 2 * G, d, eps)
    oq, ok_ = 2 * H * d, 2 * (H + G) * d
    rows = k_cache.shape[2]
    att = torch.zeros(B, 2 * H, dv, dtype=torch.float32, device=qkv.device)
    for b in range(B):
        s = int(slots[b]) if slots is not None else b
        n = int(cache_lens[s])
        r = cache_row(n, a.keep_first, rows)
        k_cache[s, :, r] = qkv[b, oq:ok_].view(2 * G, d)
        v_cache[s, :, r] = qkv[b, ok_:ok_ + G * dv].view(G, dv)
        j = torch.arange(n + 1, device=qkv.device)
        if a.window is not None:
            j = j[(n - j < a.window) | (j < a.keep_first)]
        rj = cache_row(j, a.keep_first, rows)
        kk = k_cache[s][:, rj].float()
        vv = v_cache[s][:, rj].float()
        q = qkv[b, :oq].float().view(2 * H, d)
        for h in range(2 * H):
            g = h // (H // G)
            att[b, h] = torch.softmax((kk[g] @ q[h]) * a.scale, -1) @ vv[g // 2]
    return _diff_combine_ref(att.reshape(B, -1), lam, H, G, dv, a.diff, eps, qkv.dtype)


# ------------------------------------------------------------------------------------------------ rotated latent attention
# (`LatentAttentionConfig` with rot_dim / q_rank / sink / out_gate).  The input projection row is
# [query latent (q_rank) | latent (kv_rank) | rotated key part (rot_dim) | gate logits (H x dv)]; a cache row is [c | k_rot].

_ROPE_TABLES: dict = {}


def rotary_table(rot, device):
    """(fp32 frequencies [dims / 2] on `device`, rounded once from double precision; factor on cos / sin)."""
    key = (rot.dims, rot.base, rot.factor, rot.original, rot.fast, rot.slow, str(device))
    hit = _ROPE_TABLES.get(key)
    if hit is None:
        f, m = rot.frequencies()
        hit = _ROPE_TABLES[key] = (torch.tensor(f, dtype=torch.float64).float().to(device), float(m))
    return hit


def _rotate_ref(x, pos, inv_freq, mscale):
    """x [N, ..., rot] fp32, pos [N]: interleaved pairs turn by pos * f_i (fp32)."""
    ang = pos.float().unsqueeze(-1) * inv_freq
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [inv_freq.numel()]
    cs, sn = (torch.cos(ang) * mscale).view(shape), (torch.sin(ang) * mscale).view(shape)
    u, v = x[..., 0::2], x[..., 1::2]
    return torch.stack([u * cs - v * sn, v * cs + u * sn], -1).flatten(-2)


def latent_rope_prepare(proj, a, wq, wc, eps: float, pos, cache, tok_slot=None, remain=None, cache_lens=None, slots=None, want_lat=True):
    """From the input projection: cq = RMSNorm(query latent) * wq ([T, q_rank], None without a query latent) and the row
    [c | k_rot] = [RMSNorm(latent) * wc | rotate(key part)] ([T, kv_rank + rot_dim], with `want_lat`), also written to the ring
    cache.  Packed form (`pos` [T]): the tokens with tok_slot >= 0 among the last R of their sequence are stored; step form
    (`pos` None): row b's position is cache_lens[slot], and its row is stored."""
    T = proj.shape[0]
    qr, r, rot = a.q_rank or 0, a.kv_rank, a.rot_dim
    inv_freq, ms = rotary_table(a.rotary, proj.device) if rot else (torch.zeros(1, device=proj.device), 1.0)
    if use_native(proj):
        cq = torch.empty(T, qr, dtype=proj.dtype, device=proj.device) if qr else None
        lat = torch.empty(T, r + rot, dtype=proj.dtype, device=proj.device) if want_lat else None
        lib().latent_rope_prepare(proj, wq if qr else None, wc, inv_freq, ms, pos, cache_lens if pos is None else None,
                                  slots if pos is None else None, tok_slot if (cache is not None and pos is not None) else None,
                                  remain if (cache is not None and pos is not None) else None, cq, lat, cache, qr, r, rot, eps)
        return cq, lat
    cq = None
    if qr:
        x = proj[:, :qr].float()
        cq = (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * wq.float()).to(proj.dtype)
    c = proj[:, qr:qr + r].float()
    c = c * torch.rsqrt(c.pow(2).mean(-1, keepdim=True) + eps) * wc.float()
    if pos is None:
        idx = slots.long() if slots is not None else torch.arange(T, device=proj.device)
        p = cache_lens[idx]
    else:
        p = pos
    parts = [c]
    if rot:
        parts.append(_rotate_ref(proj[:, qr + r:qr + r + rot].float(), p, inv_freq, ms))
    lat = torch.cat(parts, -1).to(proj.dtype)
    if cache is not None:
        R = cache.shape[1]
        if pos is None:
            cache[idx, (p % R).long()] = lat
        else:
            keep = (tok_slot >= 0) & (remain < R)
            cache[tok_slot[keep].long(), (pos[keep] % R).long()] = lat[keep]
    return cq, lat


def latent_rope_attention(q, kv, lat, a, sink, pos, cu_seqlens, max_seqlen=None):
    """Packed causal attention: q [T, H (d + rot)] (rotated here), kv [T, H d | H dv] the up-projected unrotated keys and values,
    lat [T, kv_rank + rot] whose last rot columns are the rotated key part of every head.  The softmax denominator holds
    exp(sink_h) when `sink` is given.  Returns [T, H * dv] in q's dtype."""
    T = q.shape[0]
    H, d, rot, dv, r = a.n_heads, a.qk_dim, a.rot_dim, a.v_dim, a.kv_rank
    dq = d + rot
    inv_freq, ms = rotary_table(a.rotary, q.device) if rot else (torch.zeros(1, device=q.device), 1.0)
    if use_native(q) and dq <= 512 and dv <= 256:
        qk = torch.empty(T, 2 * H * dq, dtype=q.dtype, device=q.device)
        lib().latent_rope_assemble(q, kv, lat, pos, inv_freq, ms, qk, H, d, rot, r)
        out = torch.empty(T, H * dv, dtype=q.dtype, device=q.device)
        if max_seqlen is None:
            max_seqlen = int((cu_seqlens[1:] - cu_seqlens[:-1]).max())
        vv = kv[:, H * d:]
        if (os.environ.get("REAL_WINDOW_ATTN", "tcgen05") == "tcgen05" and q.dtype in (torch.bfloat16, torch.float16) and dq == dv and dq in (64, 128)
                and kv.stride(0) % 8 == 0 and (H * d) % 8 == 0 and vv.data_ptr() % 16 == 0):
            lib().sink_window_attention_tc(qk, vv, out, None, sink, cu_seqlens, max_seqlen, H, H, dq, a.scale, -1, 0, -1.0, False, 1)
        else:
            lib().sink_window_attention(qk, vv, out, None, sink, cu_seqlens, max_seqlen, H, H, dq, dv, a.scale, -1, 0, -1.0, False, 1)
        return out
    qh = q.float().view(T, H, dq)
    if rot:
        qh = torch.cat([qh[..., :d], _rotate_ref(qh[..., d:], pos, inv_freq, ms).to(q.dtype).float()], -1)
    kh = torch.cat([kv[:, : H * d].float().view(T, H, d), lat[:, r:].float().unsqueeze(1).expand(T, H, rot)], -1)
    vh = kv[:, H * d:].float().view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=torch.float32, device=q.device)
    cu = cu_seqlens.tolist()
    for b in range(len(cu) - 1):
        s0, e0 = cu[b], cu[b + 1]
        L = e0 - s0
        if L == 0:
            continue
        ok = torch.arange(L, device=q.device).unsqueeze(0) <= torch.arange(L, device=q.device).unsqueeze(1)
        for h in range(H):
            sc = (qh[s0:e0, h] @ kh[s0:e0, h].T) * a.scale
            out[s0:e0, h] = _sink_softmax_pv(sc, ok, sink[h].float() if sink is not None else None, vh[s0:e0, h])
    return out.reshape(T, H * dv).to(q.dtype)


def latent_rope_decode_attention(q, a, w_ukv, sink, cache, cache_lens, slots):
    """One new token per row against the cached rows [c | k_rot] of its slot (the row of the new token is already stored).  Keys
    and values are never formed: score_j = scale (q_nope W_uk) . c_j + scale rotate(q_rot) . k_rot_j, the weighted sum of the cached
    latents comes back through W_uv.  Returns [B, H * dv] in q's dtype."""
    B = q.shape[0]
    H, d, rot, dv, r = a.n_heads, a.qk_dim, a.rot_dim, a.v_dim, a.kv_rank
    dq = d + rot
    inv_freq, ms = rotary_table(a.rotary, q.device) if rot else (torch.zeros(1, device=q.device), 1.0)
    wk, wv = _absorbed_projections(w_ukv, H, d, dv, a.scale)
    R = cache.shape[1]
    if use_native(q) and r + rot <= 512:
        from realhf_b200.ops.functional import cached_on
        qa = torch.empty(H, B, r + rot, dtype=torch.float32, device=q.device)
        qa[:, :, :r] = torch.bmm(q.view(B, H, dq)[:, :, :d].transpose(0, 1).float(), wk)
        if rot:
            lib().latent_query_rope(q, cache_lens, slots, inv_freq, ms, a.scale, qa, d, rot)
        ctas = B * ((H + 15) // 16)
        splits = max(1, min((3 * 148 + ctas - 1) // ctas, R // 64, 32))
        sk = cached_on(sink, "_f32", lambda w: w.float().contiguous()) if sink is not None else None
        o = lib().latent_decode_core(qa, cache, cache_lens, slots, 0, splits, sk)
        return torch.bmm(o[:, :, :r], wv).transpose(0, 1).reshape(B, H * dv).to(q.dtype)
    idx = slots.long() if slots is not None else torch.arange(B, device=q.device)
    pos = cache_lens[idx]
    qh = q.float().view(B, H, dq)
    qa = torch.einsum("bhd,hdr->bhr", qh[..., :d], wk)
    if rot:
        qa = torch.cat([qa, _rotate_ref(qh[..., d:], pos, inv_freq, ms) * a.scale], -1)
    out = torch.empty(B, H * dv, dtype=torch.float32, device=q.device)
    for b in range(B):
        p = int(pos[b])
        cw = cache[idx[b], torch.arange(0, p + 1, device=q.device) % R].float()
        sc = qa[b] @ cw.t()
        pr = _sink_softmax_pv(sc, torch.ones_like(sc, dtype=torch.bool), sink.float().unsqueeze(-1) if sink is not None else None, cw[:, :r])
        out[b] = torch.einsum("hr,hrv->hv", pr, wv).reshape(-1)
    return out.to(q.dtype)


def sigmoid_gate_(x, gate):
    """x[t, c] *= sigmoid(gate[t, c]) in place (fp32 inside); gate may be a column slice of a wider projection."""
    if use_native(x):
        lib().sigmoid_gate_(x, gate)
        return x
    x.copy_((x.float() * torch.sigmoid(gate[:, : x.shape[1]].float())).to(x.dtype))
    return x
