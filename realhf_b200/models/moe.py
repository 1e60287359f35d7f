"""Mixture-of-experts MLP: router, token permutation, grouped expert GEMMs, expert parallelism.

Parity: `realhf/impl/model/modules/moe/{router,experts,token_dispatcher,layer}.py` and `utils/moe.py`
(top-k softmax routing, aux load-balancing loss, z-loss, capacity-factor token dropping, sinkhorn).
Beyond the reference: real **expert parallelism** — with `ep_group` set, experts are partitioned across
ranks and tokens travel by all-to-all (`dispatch -> grouped GEMM -> combine`); the reference's
"AlltoAll" dispatcher never leaves the rank (token_dispatcher.py:17-27).
"""

from __future__ import annotations

import os
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn.functional as F

from realhf_b200.ops import functional as OF
from realhf_b200.parallel import tp as TP

MOE_STATS: Dict[str, List[torch.Tensor]] = {"aux_loss": [], "z_loss": []}


def pop_moe_losses() -> Dict[str, torch.Tensor]:
    out = {k: (torch.stack(v).sum() if v else None) for k, v in MOE_STATS.items()}
    for v in MOE_STATS.values():
        v.clear()
    return out


def sinkhorn(cost: torch.Tensor, tol: float = 1e-4, max_iter: int = 100) -> torch.Tensor:
    cost = torch.exp(cost.float())
    d0 = torch.ones(cost.size(0), device=cost.device)
    d1 = torch.ones(cost.size(1), device=cost.device)
    eps, err, it = 1e-8, 1e9, 0
    while err > tol and it < max_iter:
        d0 = (1.0 / d0.size(0)) / (torch.sum(d1.unsqueeze(0) * cost, 1) + eps)
        d1_new = (1.0 / d1.size(0)) / (torch.sum(d0.unsqueeze(1) * cost, 0) + eps)
        err = torch.mean(torch.abs(d1 - d1_new)).item()
        d1, it = d1_new, it + 1
    return d1 * cost * d0.unsqueeze(1)


def route(h: torch.Tensor, w_router: torch.Tensor, mcfg, training: bool, bias: Optional[torch.Tensor] = None,
          correction: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """h [T,H] -> (probs [T,k] fp32 normalised over the chosen experts, expert ids [T,k]).  Logits (+ `bias`) are fp32.
    routing_type "softmax_all": the scores are the softmax over all router outputs, `correction` is added to them for the
    choice only, and the weights are the chosen scores themselves (divided by their sum only with `renormalize`)."""
    if training and mcfg.input_jitter_eps > 0:
        h = h * torch.empty_like(h).uniform_(1 - mcfg.input_jitter_eps, 1 + mcfg.input_jitter_eps)
    logits = F.linear(h.float(), w_router.float(), bias.float() if bias is not None else None)
    if training and mcfg.z_loss_coeff > 0:
        MOE_STATS["z_loss"].append(torch.logsumexp(logits, -1).square().mean() * mcfg.z_loss_coeff)
    if mcfg.routing_type == "sinkhorn" and training:
        with torch.no_grad():
            _, idx = torch.topk(sinkhorn(logits), mcfg.top_k, dim=-1)
        probs = torch.sigmoid(logits).gather(-1, idx) if mcfg.top_k == 1 else torch.softmax(logits, -1).gather(-1, idx)
        return probs, idx
    if mcfg.routing_type in ("softmax_all", "sigmoid"):
        if bias is None and _native_route(h, w_router, mcfg):
            return softmax_all_route(h, w_router, correction, mcfg)[:2]
        full = torch.sigmoid(logits) if mcfg.routing_type == "sigmoid" else torch.softmax(logits, dim=-1)
        idx = torch.topk(full + correction.float() if correction is not None else full, mcfg.top_k, dim=-1).indices
        probs = full.gather(-1, idx)
        return (probs / probs.sum(-1, keepdim=True) if mcfg.renormalize else probs), idx
    if mcfg.routing_type == "none":  # the k largest logits, weighted by the softmax over those k alone
        top, idx = torch.topk(logits, mcfg.top_k, dim=-1)
        return torch.softmax(top, dim=-1), idx
    full = torch.softmax(logits, dim=-1)
    probs, idx = torch.topk(full, mcfg.top_k, dim=-1)
    probs = probs / probs.sum(-1, keepdim=True)
    if training and mcfg.routing_type == "aux_loss" and mcfg.aux_loss_coeff > 0:
        E = logits.shape[-1]
        frac_tokens = F.one_hot(idx, E).float().sum(1).mean(0)     # share of assignments per expert
        frac_probs = full.mean(0)
        MOE_STATS["aux_loss"].append((frac_tokens * frac_probs).sum() * E * mcfg.aux_loss_coeff / mcfg.top_k)
    return probs, idx


def _native_route(h: torch.Tensor, w_router: torch.Tensor, mcfg) -> bool:
    """The fused routing / combination kernels: inference on CUDA, up to 64 router outputs, up to 8 choices."""
    from realhf_b200.ops import native_built
    return (h.is_cuda and not torch.is_grad_enabled() and native_built() and h.dim() == 2 and h.stride(1) == 1 and w_router.shape[0] <= 64
            and mcfg.top_k <= min(8, w_router.shape[0]) and h.dtype in (torch.float32, torch.bfloat16, torch.float16))


def softmax_all_route(h: torch.Tensor, w_router: torch.Tensor, correction: Optional[torch.Tensor], mcfg,
                      w_gate: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """One kernel for routing_type "softmax_all" / "sigmoid" (inference): fp32 logits W h, scores = softmax over all outputs (or the
    sigmoid of every output), the top_k largest of score + correction, their scores as weights; with `w_gate` [1, H] also
    sigmoid(w_gate . h) per token ([T] fp32)."""
    from realhf_b200.ops import lib
    probs, idx, gate = lib().softmax_router(h, w_router.contiguous(), correction.contiguous() if correction is not None else None,
                                            w_gate.contiguous().view(-1) if w_gate is not None else None, mcfg.top_k, bool(mcfg.renormalize),
                                            mcfg.routing_type == "sigmoid")
    return probs, idx, (gate if w_gate is not None else None)


def _apply_capacity(probs, idx, n_experts: int, mcfg):
    """Zero the routing weight of assignments beyond each expert's capacity."""
    if mcfg.capacity_factor is None:
        return probs
    T, k = idx.shape
    cap = int(mcfg.capacity_factor * T * k / n_experts + 0.999)
    flat_e = idx.reshape(-1)
    if mcfg.token_drop_policy == "position":
        order = torch.arange(T * k, device=idx.device)
    else:
        order = torch.argsort(probs.reshape(-1), descending=True, stable=True)
    e_sorted = flat_e[order]
    onehot = F.one_hot(e_sorted, n_experts)
    rank_in_e = (onehot.cumsum(0) * onehot).sum(-1) - 1
    keep_sorted = rank_in_e < cap
    keep = torch.empty_like(keep_sorted)
    keep[order] = keep_sorted
    return probs * keep.view(T, k).to(probs.dtype)


def _count_experts(flat_e: torch.Tensor, n_experts: int) -> torch.Tensor:
    """Assignments per expert without a host sync (`torch.bincount` reads its input's maximum back to size the output, which also
    makes it illegal inside CUDA-graph capture)."""
    return torch.zeros(n_experts, dtype=torch.long, device=flat_e.device).scatter_add_(0, flat_e, torch.ones_like(flat_e))


def grouped_mlp_device(x_sorted: torch.Tensor, counts_dev: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, act: str):
    """Expert MLP over tokens sorted by expert with the counts left on the DEVICE: two grouped tcgen05 GEMM launches and the
    gated activation, no `tokens_per_expert.cpu()` (reference: moe/experts.py:186) and no per-expert Python loop."""
    from realhf_b200.ops import gemm as G
    offsets = torch.zeros(counts_dev.numel() + 1, dtype=torch.int32, device=x_sorted.device)
    offsets[1:] = counts_dev.cumsum(0)
    h = G.grouped_linear(x_sorted, w_gate_up, offsets)
    return G.grouped_linear(_expert_act(h, act), w_down, offsets)


def _use_grouped_kernel(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor) -> bool:
    if not x.is_cuda or OF.gemm_impl() is None:
        return False
    from realhf_b200.ops import gemm as G
    return G.grouped_supported(x, w_gate_up) and G.grouped_supported(x, w_down)


def grouped_mlp(x_sorted: torch.Tensor, counts: List[int], w_gate_up: torch.Tensor, w_down: torch.Tensor, act: str):
    """Tokens sorted by expert; expert e owns rows [sum(counts[:e]), +counts[e]).  w_gate_up [E,2F,H], w_down [E,H,F].  Counts beyond
    the E weight slices belong to identity experts: their rows pass through."""
    outs, off = [], 0
    for e, n in enumerate(counts):
        if n == 0:
            continue
        xe = x_sorted[off: off + n]
        outs.append(OF.linear(_expert_act(OF.linear(xe, w_gate_up[e]), act), w_down[e]) if e < w_gate_up.shape[0] else xe)
        off += n
    if not outs:
        return x_sorted.new_zeros(0, w_down.shape[1])
    return torch.cat(outs, 0)


def _scaled_rows(h: torch.Tensor, tok: torch.Tensor, w_sorted: torch.Tensor) -> torch.Tensor:
    """h[tok] * w (the routing weight on the expert's input): the product in fp32, stored in h's dtype."""
    return (h.index_select(0, tok).float() * w_sorted.float().unsqueeze(-1)).to(h.dtype)


def moe_forward(model, i: int, h: torch.Tensor, mcfg=None, clamp: Optional[Tuple[float, float]] = None) -> torch.Tensor:
    """MoE MLP of block i on normalised hidden states h ([T, H], or [T/t, H] under sequence parallelism).  `mcfg`: the block's own
    MoE config in a heterogeneous stack (default: the model-wide one).  With `fp32_residual` the experts' outputs are combined
    in fp32 and the result stays fp32.  `clamp` = (limit, alpha): the experts are clamped gated units, y = g sigmoid(alpha g) (u + 1)
    with g = min(gate, limit), u = clamp(up, +-limit), instead of units gated by the model's activation.  With `mcfg.scale_input`
    an assignment's routing weight multiplies the expert's input row and the outputs are summed unweighted."""
    c, ctx = model.config, model.ctx
    mcfg = mcfg if mcfg is not None else c.moe
    E, k = mcfg.num_experts, mcfg.top_k
    act = c.activation_function if clamp is None else ("clamped", float(clamp[0]), float(clamp[1]))
    if mcfg.scale_input or not mcfg.shared_gate:
        assert mcfg.routing_type in ("softmax_all", "sigmoid") and ctx.tp_size == 1, "scale_input / ungated shared experts: single-rank stacks"
    w_gu, w_dn = model.p[f"{i}.mlp.experts.gate_up.weight"], model.p[f"{i}.mlp.experts.down.weight"]
    ep = mcfg.expert_parallel and ctx.tp_size > 1
    sp = model.sequence_parallel
    if ep and sp:
        pass  # tokens stay sharded: they travel to the experts' owners by all-to-all
    elif sp:
        h = TP.gather_from_sp(h, ctx)
    else:
        h = TP.copy_to_tp(h, ctx)
    T, H = h.shape
    gate_sh = None
    fused = (mcfg.routing_type in ("softmax_all", "sigmoid") and model.p.get(f"{i}.mlp.router.bias") is None and not ep and ctx.tp_size == 1
             and mcfg.capacity_factor is None and _native_route(h, model.p[f"{i}.mlp.router.weight"], mcfg))
    if fused:       # routing, the shared expert's gate and (below) the weighted sum of the experts' outputs: one kernel each
        probs, idx, gate_sh = softmax_all_route(h, model.p[f"{i}.mlp.router.weight"], model.p.get(f"{i}.mlp.router.correction"), mcfg,
                                                model.p[f"{i}.mlp.shared.sg.weight"] if mcfg.shared_ff and mcfg.shared_gate else None)
    else:
        probs, idx = route(h, model.p[f"{i}.mlp.router.weight"], mcfg, model.training, model.p.get(f"{i}.mlp.router.bias"),
                           model.p.get(f"{i}.mlp.router.correction"))
    n_id = mcfg.identity_experts            # router outputs E .. E + n_id - 1: the expert's output is its input
    if n_id or mcfg.shared_ff:
        assert not ep and ctx.tp_size == 1 and mcfg.capacity_factor is None, "identity / shared experts: single-rank stacks"
    if fused and T * k <= 1024 and mcfg.use_grouped_gemm and _use_grouped_kernel(h, w_gu, w_dn):
        # a decode-sized batch: every assignment's place in the order sorted by expert and the experts' row offsets come from a
        # counting kernel instead of a sort; rows of identity experts lie behind the last offset and never enter the GEMMs
        from realhf_b200.ops import gemm as G, lib
        back, offsets = lib().moe_dispatch(idx, E, E + n_id)
        hid = G.grouped_linear(lib().moe_gather(h, back, k, probs if mcfg.scale_input else None), w_gu, offsets)
        y_sorted = G.grouped_linear(_expert_act(hid, act), w_dn, offsets)
        out = torch.empty(T, H, dtype=torch.float32 if c.fp32_residual else h.dtype, device=h.device)
        lib().moe_combine(y_sorted, h, back, probs, idx, _shared_mlp(model, i, h, mcfg, act) if mcfg.shared_ff else None, gate_sh, out, E,
                          bool(mcfg.scale_input))
        return out
    probs = _apply_capacity(probs, idx, E, mcfg)
    flat_e = idx.reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    tok = torch.arange(T, device=h.device).repeat_interleave(k)[order]
    w_sorted = probs.reshape(-1)[order]
    if mcfg.scale_input:
        assert not ep and not n_id, "scale_input: local experts, no identity experts"
        if fused:      # one kernel: every assignment's token row times its weight, written at its place in the sorted order
            from realhf_b200.ops import lib
            back = torch.empty_like(order).scatter_(0, order, torch.arange(order.numel(), device=order.device))
            x_scaled = lib().moe_gather(h, back, k, probs.float().contiguous())
        else:
            x_scaled = _scaled_rows(h, tok, w_sorted)
        w_sorted = torch.ones_like(w_sorted)
    if ep and sp:
        from realhf_b200.parallel import ep as EP
        x_sorted = h.index_select(0, tok)
        fep = None
        if h.is_cuda and h.dtype in (torch.bfloat16, torch.float16) and _use_grouped_kernel(x_sorted, w_gu, w_dn) \
                and os.environ.get("REAL_EP_FUSED", "1") == "1":
            fep = EP.fused_ep_for(ctx, E, H, h.dtype, h.device)
        if fep is not None and x_sorted.shape[0] <= fep.max_rows:
            # device-driven peer-store dispatch / combine around the grouped GEMMs (csrc/ep.cu): no host sync in this layer
            y_sorted = EP.dispatch_compute_combine_fused(x_sorted, flat_e[order], E, w_gu, w_dn, c.activation_function, fep)
        else:
            y_sorted = EP.dispatch_compute_combine(x_sorted, flat_e[order], E, w_gu, w_dn, c.activation_function, ctx.tp_group)
        return torch.zeros(T, H, dtype=y_sorted.dtype, device=h.device).index_add_(0, tok, y_sorted * w_sorted.to(y_sorted.dtype).unsqueeze(-1))
    if ep and not torch.is_grad_enabled() and _use_grouped_kernel(h, w_gu, w_dn):
        # replicated tokens, sync-free (CUDA-graph capturable: the decode path): every rank sorts ALL assignments, the grouped GEMM
        # is pointed at the row range of MY experts through device-side offsets (rows of other experts are never touched), the
        # foreign rows are masked out and the partial outputs are all-reduced.  Inference only: the untouched rows hold
        # uninitialised memory, which `torch.where` discards in the forward pass but which would leak into the gradients
        # (0 * NaN in the routing-weight gradient, garbage dgrad rows scattered back into dh); training without SP takes the
        # compacting path below
        e_local = E // ctx.tp_size
        lo = ctx.tp_rank * e_local
        e_sorted = flat_e[order]
        offs = torch.zeros(E + 1, dtype=torch.int32, device=h.device)
        offs[1:] = _count_experts(flat_e, E).cumsum(0)
        from realhf_b200.ops import gemm as G
        x_sorted = h.index_select(0, tok)
        my_offs = offs[lo: lo + e_local + 1].contiguous()
        hid = G.grouped_linear(x_sorted, w_gu, my_offs)
        y_sorted = G.grouped_linear(OF.gated_act(hid, c.activation_function), w_dn, my_offs)
        mine = ((e_sorted >= lo) & (e_sorted < lo + e_local)).unsqueeze(-1)
        contrib = torch.where(mine, y_sorted * w_sorted.to(y_sorted.dtype).unsqueeze(-1), torch.zeros((), dtype=y_sorted.dtype, device=h.device))
        out = torch.zeros(T, H, dtype=h.dtype, device=h.device).index_add_(0, tok, contrib.to(h.dtype))
        return TP.reduce_from_tp(out, ctx)
    if ep:
        # replicated tokens: keep only the assignments of my experts, all-reduce the partial outputs
        e_local = E // ctx.tp_size
        lo = ctx.tp_rank * e_local
        e_sorted = flat_e[order]
        mine = (e_sorted >= lo) & (e_sorted < lo + e_local)
        sel = torch.nonzero(mine).squeeze(-1)
        x_sorted = h.index_select(0, tok[sel])
        counts = torch.bincount(e_sorted[sel] - lo, minlength=e_local).tolist()
        y_sorted = grouped_mlp(x_sorted, counts, w_gu, w_dn, c.activation_function)
        out = torch.zeros(T, H, dtype=h.dtype, device=h.device).index_add_(
            0, tok[sel], (y_sorted * w_sorted[sel].to(y_sorted.dtype).unsqueeze(-1)).to(h.dtype))
        return TP.reduce_from_tp(out, ctx)
    x_sorted = x_scaled if mcfg.scale_input else h.index_select(0, tok)
    grouped = mcfg.use_grouped_gemm and _use_grouped_kernel(x_sorted, w_gu, w_dn)   # use_grouped_gemm=False: one GEMM pair per expert
    if not grouped and h.is_cuda and torch.cuda.is_current_stream_capturing():
        # operands the grouped kernel does not take (fp32) inside a CUDA-graph capture, where the per-expert loop's host read of
        # the counts is illegal: every expert runs on every row (decode batches are small) and the routing weight, zero for
        # the experts a row did not choose, selects; summed in expert order
        gate = torch.zeros(T, E + n_id, dtype=torch.float32, device=h.device).scatter_(1, idx, probs.float())
        out = torch.zeros(T, H, dtype=torch.float32 if c.fp32_residual else h.dtype, device=h.device)
        for e in range(E):
            if mcfg.scale_input:       # expert(w h) where chosen (w > 0), nothing elsewhere
                y = OF.linear(_expert_act(OF.linear((h.float() * gate[:, e: e + 1]).to(h.dtype), w_gu[e]), act), w_dn[e])
                out += (y.float() * (gate[:, e: e + 1] > 0)).to(out.dtype)
                continue
            y = OF.linear(OF.gated_act(OF.linear(h, w_gu[e]), c.activation_function), w_dn[e])
            out += (y.float() * gate[:, e: e + 1]).to(out.dtype)
        if n_id:
            out += (h.float() * gate[:, E:].sum(1, keepdim=True)).to(out.dtype)
        return _add_shared(model, i, h, mcfg, out, act)
    if grouped:
        # the device-side offsets end at expert E: rows of identity experts (sorted last) are not touched by the GEMMs and pass through
        y_sorted = grouped_mlp_device(x_sorted, _count_experts(flat_e, E + n_id)[:E], w_gu, w_dn, act)
        if n_id and not fused:
            y_sorted = torch.where((flat_e[order] >= E).unsqueeze(-1), x_sorted, y_sorted)
    else:
        counts = torch.bincount(flat_e, minlength=E + n_id).tolist()
        y_sorted = grouped_mlp(x_sorted, counts, w_gu, w_dn, act)
    if fused:
        from realhf_b200.ops import lib
        if not mcfg.scale_input:
            back = torch.empty_like(order).scatter_(0, order, torch.arange(order.numel(), device=order.device))
        out = torch.empty(T, H, dtype=torch.float32 if c.fp32_residual else h.dtype, device=h.device)
        lib().moe_combine(y_sorted.contiguous(), h, back, probs.float().contiguous(), idx,
                          _shared_mlp(model, i, h, mcfg, act) if mcfg.shared_ff else None, gate_sh, out, E, bool(mcfg.scale_input))
        return out
    if c.fp32_residual:
        # fp32 combine in a fixed order (an atomic index_add_ would make the sum depend on the run): rows back to (token, choice)
        # order, then the sum over the k choices
        back = torch.empty_like(order).scatter_(0, order, torch.arange(order.numel(), device=order.device))
        out = (y_sorted.float() * w_sorted.unsqueeze(-1)).index_select(0, back).view(T, k, H).sum(1)
    else:
        out = torch.zeros(T, H, dtype=y_sorted.dtype, device=h.device).index_add_(0, tok, y_sorted * w_sorted.to(y_sorted.dtype).unsqueeze(-1))
    if ctx.tp_size > 1:  # experts are F-sharded over TP: partial sums
        out = TP.reduce_scatter_to_sp(out, ctx) if sp else TP.reduce_from_tp(out, ctx)
    return _add_shared(model, i, h, mcfg, out, act)


def _expert_act(hid: torch.Tensor, act) -> torch.Tensor:
    """The experts' gated activation on the fused [.., 2F] gate | up rows: the named activation, or ("clamped", limit, alpha)."""
    if isinstance(act, tuple):
        return OF.clamped_glu(hid, act[1], act[2])
    return OF.gated_act(hid, act)


def _add_shared(model, i: int, h: torch.Tensor, mcfg, out: torch.Tensor, act=None) -> torch.Tensor:
    """out += shared expert(h) * sigmoid(w_sg . h): an expert every token uses, scaled by one learned gate value per token (fp32;
    `shared_gate` False: added unscaled)."""
    if not mcfg.shared_ff:
        return out
    y = _shared_mlp(model, i, h, mcfg, act).float()
    if mcfg.shared_gate:
        y = y * torch.sigmoid(F.linear(h.float(), model.p[f"{i}.mlp.shared.sg.weight"].float()))
    return out + y.to(out.dtype)


def _shared_mlp(model, i: int, h: torch.Tensor, mcfg=None, act=None) -> torch.Tensor:
    p = model.p
    if isinstance(act, tuple):     # clamped unit with the shared expert's own limit
        limit = mcfg.shared_limit if mcfg is not None and mcfg.shared_limit is not None else act[1]
        return OF.linear(OF.clamped_gated_linear(h, p[f"{i}.mlp.shared.gate_up.weight"], limit, act[2]), p[f"{i}.mlp.shared.down.weight"])
    return OF.linear(OF.gated_linear(h, p[f"{i}.mlp.shared.gate_up.weight"], model.config.activation_function), p[f"{i}.mlp.shared.down.weight"])
