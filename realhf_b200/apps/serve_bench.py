"""Prefill / decode throughput of a heterogeneous-stack design next to the closest homogeneous model of equal size, and the
roofline position of its kernels next to the like kernels of that model.  Reached through `bench.py --serve-bench rapodra`,
`--serve-bench tizodra`, `--serve-bench defilorn` or `--serve-bench buvesun` (the default workload of bench.py is unaffected).
Buvesun is also timed beside a Defilorn of equal size, the closest heterogeneous stack (window attention, a matrix-state mixer, routed
feed-forwards with a shared expert).

Both models run through `models.generation`: prefill = `prefill_into_state` (the packed prefill `generate` performs) into a
standing decode state, decode = the CUDA-graph loop of `generate` with the sampler in the graph; random weights, bf16.  Timing: CUDA events, >= 3 warm-up calls, weights + state far larger than L2 per call for
the model-level numbers; the kernel table flushes L2 (a 256 MB write) between timed launches.  One JSON line per result.
"""

from __future__ import annotations

import json
import os
from typing import Callable, Dict, List

import torch


SIZES = {
    # name: width, heads, qk dim, v dim, latent rank, window, dense ff, experts, expert ff, top, vocab
    "1b-like": dict(width=2048, heads=16, dim=128, vdim=128, rank=512, window=1024, ff=8192, experts=8, eff=2048, top=2, vocab=32000),
    "7b-like": dict(width=4096, heads=32, dim=128, vdim=128, rank=512, window=2048, ff=11008, experts=8, eff=2816, top=2, vocab=32000),
}


def rapodra_config(s: dict, n_layers: int = 4) -> dict:
    mixer = lambda **k: dict(dict(dim=s["dim"], heads=s["heads"], kv_rank=s["rank"], vdim=s["vdim"], scale=s["dim"] ** -0.5,
                                  mask=dict(size=s["window"])), **k)
    dense = dict(kind="dense", ff=s["ff"], limit=7.0)
    moe = dict(kind="moe", expert=dict(ff=s["eff"]), router=dict(experts=s["experts"], top=s["top"]))
    layers = []
    for i in range(n_layers):
        layers.append(dict(type="latent_attention", mixer=mixer(**({"kv_from": i - 1} if i % 2 else {})), mlp=moe if i % 2 else dense))
    return dict(architecture="Rapodra", canon=dict(taps=4), layers=layers, logit_softcap=30.0, norm=dict(eps=1e-5, groups=8),
                vocab=s["vocab"], width=s["width"])


TIZODRA_SIZES = {
    # name: width, query heads, kv heads, qk dim, v dim, window, kept first tokens, conv taps, ff, vocab
    "1b-like": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, window=512, keep=64, conv=4, ff=8192, vocab=32000),
    "7b-like": dict(width=4096, heads=32, kv_heads=8, dim=128, vdim=128, window=1024, keep=64, conv=4, ff=11008, vocab=32000),
}


def tizodra_config(s: dict, n_layers: int = 4) -> dict:
    """Delta blocks outside, window-attention blocks inside a loop of one pass (so the re-injection projection is on the path)."""
    att = dict(type="attention", mixer=dict(dim=s["dim"], heads=s["heads"], kv_heads=s["kv_heads"], vdim=s["vdim"], scale=s["dim"] ** -0.5,
                                            mask=dict(size=s["window"], keep_first=s["keep"])), mlp=dict(kind="dense", ff=s["ff"]))
    dlt = dict(type="delta", mixer=dict(conv=s["conv"], dim=s["dim"], heads=s["heads"], kv_heads=s["kv_heads"], vdim=s["vdim"]),
               mlp=dict(kind="dense", ff=s["ff"]))
    layers = [dlt if i in (0, n_layers - 1) else att for i in range(n_layers)]
    return dict(architecture="Tizodra", layers=layers, logit_scale=0.7, loop=dict(start=1, stop=max(2, n_layers - 1), times=1),
                norm=dict(eps=1e-5), vocab=s["vocab"], width=s["width"])


DEFILORN_SIZES = {
    # name: width, heads, kv heads (differential attention), head sizes (attention: two maps of `dim` per head), window, latent ranks,
    # unrotated / rotated query-key dims of the latent attention, dense ff, experts, expert ff, top, identity experts, shared ff, vocab
    "1b-like": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, window=512, kv_rank=448, q_rank=768, nope=64, rot=64, ff=8192,
                    experts=8, eff=2048, top=2, identity=1, sff=2048, vocab=32000),
    "7b-like": dict(width=4096, heads=32, kv_heads=8, dim=128, vdim=128, window=1024, kv_rank=448, q_rank=1536, nope=64, rot=64, ff=11008,
                    experts=8, eff=2816, top=2, identity=1, sff=2816, vocab=32000),
}


def defilorn_config(s: dict, n_layers: int = 4) -> dict:
    """Differential attention, matrix-memory LSTM, rotated latent attention in turn; dense and mixture-of-experts feed-forwards alternate."""
    dense = dict(kind="dense", ff=s["ff"])
    moe = dict(kind="moe", expert=dict(ff=s["eff"]), router=dict(experts=s["experts"], identity=s["identity"], top=s["top"]), shared=dict(ff=s["sff"]))
    att = dict(type="attention", mixer=dict(diff=0.6, dim=s["dim"], heads=s["heads"], kv_heads=s["kv_heads"], vdim=s["vdim"], scale=s["dim"] ** -0.5,
                                            mask=dict(size=s["window"])))
    mls = dict(type="mlstm", mixer=dict(dim=s["dim"], gate_cap=15.0, heads=s["heads"], vdim=s["vdim"]))
    lat = dict(type="latent_attention", mixer=dict(dim=s["nope"], heads=s["heads"], kv_rank=s["kv_rank"], q_rank=s["q_rank"], rot_dim=s["rot"],
                                                   vdim=s["vdim"], scale=(s["nope"] + s["rot"]) ** -0.5,
                                                   rot=dict(base=1e6, dims=s["rot"], scaling=dict(factor=8.0, fast=32.0, original=2048, slow=1.0))))
    kinds = [att, mls, lat]
    layers = [dict(kinds[i % 3], mlp=moe if i % 2 else dense) for i in range(n_layers)]
    return dict(architecture="Defilorn", layers=layers, loop=dict(start=0, stop=min(2, n_layers), times=1), norm=dict(eps=1e-5), vocab=s["vocab"],
                width=s["width"])


BUVESUN_SIZES = {
    # the Defilorn sizes (so that a Defilorn of equal size can be built beside it) plus: heads of the decayed linear attention,
    # rotated dimensions, clamp limits
    "1b-like": dict(DEFILORN_SIZES["1b-like"], r_heads=16, rot_dims=64, limit=7.0),
    "7b-like": dict(DEFILORN_SIZES["7b-like"], r_heads=32, rot_dims=64, limit=7.0),
}


def buvesun_config(s: dict, n_layers: int = 4) -> dict:
    """Parallel blocks (window attention beside lightning attention) and retention blocks in turn, every block with a routed
    feed-forward and a shared expert; the first two blocks in a loop of one pass (so the re-injection projection is on the path)."""
    H = s["r_heads"]
    decay = [1.0 - 2.0 ** (-4.0 - 4.0 * h / max(H - 1, 1)) for h in range(H)]
    moe = dict(kind="moe", expert=dict(ff=s["eff"], limit=s["limit"]), router=dict(experts=s["experts"], top=s["top"]),
               shared=dict(ff=s["sff"], limit=s["limit"]))
    par = dict(type="parallel", mlp=moe,
               mixer=dict(left=dict(dim=s["dim"], heads=s["heads"], kv_heads=s["kv_heads"], vdim=s["vdim"], scale=s["dim"] ** -0.5,
                                    mask=dict(size=s["window"]), rot=dict(base=5e5, dims=s["rot_dims"])), left_scale=0.6,
                          right=dict(decay=decay, dim=s["dim"], heads=H, vdim=s["vdim"]), right_scale=1.1))
    ret = dict(type="retention", mlp=moe, mixer=dict(decay=decay, dim=s["dim"], heads=H, vdim=s["vdim"], rot=dict(base=1e5, dims=s["dim"])))
    layers = [par if i % 2 == 0 else ret for i in range(n_layers)]
    return dict(architecture="Buvesun", embedding=dict(scale=2.0), layers=layers, loop=dict(start=0, stop=min(2, n_layers), times=1),
                norm=dict(eps=1e-5), residual_mult=0.7, vocab=s["vocab"], width=s["width"])


def _hetero_model(design: str, s: dict, n_layers: int, dev):
    from realhf_b200.models import hf_io
    from realhf_b200.models.real_model import ReaLModel
    cfg = {"rapodra": rapodra_config, "tizodra": tizodra_config, "defilorn": defilorn_config, "buvesun": buvesun_config}[design](s, n_layers)
    m = ReaLModel(hf_io.family(design).config_from_dict(cfg, False), dtype=torch.bfloat16, device=dev).init_random_fast()
    for p in m.parameters():
        p.requires_grad_(False)
    return m.eval()


def _models(s: dict, n_layers: int, dev, design: str = "rapodra"):
    from realhf_b200.api.model import ReaLModelConfig
    from realhf_b200.models import hf_io
    from realhf_b200.models.real_model import ReaLModel
    new = _hetero_model(design, s, n_layers, dev)
    lc = ReaLModelConfig(n_layers=n_layers, n_kv_heads=s.get("kv_heads", s["heads"]), n_q_heads=s["heads"], hidden_dim=s["width"], intermediate_dim=s["ff"],
                         vocab_size=s["vocab"], head_dim=s["dim"], n_positions=8192, embd_pdrop=0.0, resid_pdrop=0.0, attn_pdrop=0.0,
                         activation_function="silu", scale_attn_by_inverse_layer_idx=False, use_attention_bias=False,
                         use_attn_proj_bias=False, use_mlp_bias=False, layer_norm_type="rms", mlp_type="llama", apply_rotary=True)
    old = ReaLModel(lc, dtype=torch.bfloat16, device=dev).init_random_fast()
    for m in (new, old):
        for p in m.parameters():
            p.requires_grad_(False)
        m.eval()
    return new, old


def _time(fn: Callable[[], None], iters: int, warmup: int = 3, flush: torch.Tensor = None) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    tot = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        tot += a.elapsed_time(b)
    return tot / iters


def model_numbers(name: str, s: dict, n_layers: int, batch: int, prompt_len: int, new_tokens: int, dev, design: str = "rapodra") -> List[dict]:
    from realhf_b200.api.model import GenerationHyperparameters
    from realhf_b200.models import generation as gen
    os.environ["REAL_GEN_TIMING"] = "1"
    out = []
    new, old = _models(s, n_layers, dev, design)
    g = GenerationHyperparameters(max_new_tokens=new_tokens, min_new_tokens=new_tokens, greedy=True, use_cuda_graph=True)
    ids = torch.randint(3, s["vocab"], (batch * prompt_len,), device=dev)
    cu = torch.arange(0, batch + 1, device=dev, dtype=torch.int32) * prompt_len
    arms = [(design, new), ("llama-equal-size", old)]
    if design == "buvesun":
        arms.insert(1, ("defilorn-equal-size", _hetero_model("defilorn", s, n_layers, dev)))
    for label, m in arms:
        # prefill: the packed prefill into a standing decode state (`prefill_into_state`, what `generate` calls), so that the
        # number is the model's and not the caching allocator's (a fresh multi-GB state per `generate` call can fall into
        # cudaMalloc inside the timed region); decode: the CUDA-graph loop of `generate`
        st = gen.DecodeState(m, batch, prompt_len + new_tokens)
        pre, dec = [], []
        with torch.no_grad():
            for it in range(7):
                st.free_slots = list(range(batch))
                slots = st.alloc(batch)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                gen.prefill_into_state(m, st, slots, ids, cu, prompt_len)
                b.record()
                torch.cuda.synchronize()
                if it >= 2:
                    pre.append(a.elapsed_time(b))
        del st
        for it in range(4):
            gen.generate(m, ids, cu, g, eos_id=None, pad_id=0)
            if it:                                     # first call: lazy initialisation
                dec.append(gen.LAST_TIMING["ms_per_decode_step"])
        pre_ms, dec_ms = sorted(pre)[len(pre) // 2], sorted(dec)[len(dec) // 2]
        out.append(dict(bench="serve", size=name, model=label, layers=n_layers, batch=batch, prompt_len=prompt_len, new_tokens=new_tokens,
                        prefill_ms=round(pre_ms, 3), prefill_tokens_per_s=round(batch * prompt_len / pre_ms * 1e3),
                        decode_ms_per_step=round(dec_ms, 4), decode_tokens_per_s=round(batch / dec_ms * 1e3), dtype="bf16", data="synthetic",
                        params=sum(p.numel() for p in m.parameters())))
    del new, old, arms, m
    torch.cuda.empty_cache()
    return out


def kernel_numbers(name: str, s: dict, batch: int, prompt_len: int, ctx: int, dev, peaks: Dict[str, float]) -> List[dict]:
    """Each kernel of the new design and the like kernel of the LLaMA path on the same problem size: time, algorithmic bytes and
    FLOPs, and the fraction of the measured roofline (the slower of bytes / copy bandwidth and FLOPs / GEMM throughput)."""
    from realhf_b200.models.hetero_block import packed_meta
    from realhf_b200.ops import attention as A
    from realhf_b200.ops import functional as OF
    bf = torch.bfloat16
    W, H, qk, vd, rank, win = s["width"], s["heads"], s["dim"], s["vdim"], s["rank"], s["window"]
    T = batch * prompt_len
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []

    def add(kernel, like, ms, nbytes, flops):
        floor_ms = max(nbytes / (peaks["hbm_gbs"] * 1e9), flops / (peaks["bf16_tflops"] * 1e12)) * 1e3
        rows.append(dict(bench="kernel", size=name, kernel=kernel, like=like, ms=round(ms, 4), gbytes=round(nbytes / 1e9, 4),
                         gflop=round(flops / 1e9, 2), roofline_ms=round(floor_ms, 4), frac_of_measured_roofline=round(floor_ms / ms, 4)))

    cu = torch.arange(0, batch + 1, device=dev, dtype=torch.int32) * prompt_len
    meta = packed_meta(cu, T)
    x32 = torch.randn(T, W, device=dev)
    xb = x32.to(bf)
    w = torch.ones(W, device=dev, dtype=bf)
    cw = torch.randn(W, 4, device=dev).to(bf) * 0.1
    add("sublayer_input (grouped norm + conv, prefill)", False, _time(lambda: OF.sublayer_input(x32, w, 8, 1e-5, cw, meta.pos, bf), 10, flush=flush),
        T * W * 6, 0)
    add("residual_add_norm_ (prefill)", False, _time(lambda: OF.residual_add_norm_(x32, xb, w, 8, 1e-5), 10, flush=flush), T * W * 10, 0)
    add("add_rmsnorm (llama, prefill)", True, _time(lambda: OF.add_rmsnorm(xb, xb, w, 1e-5), 10, flush=flush), T * W * 8, 0)
    # attention, prefill: windowed, so the useful FLOPs are those of the visible (query, key) pairs
    q = torch.randn(T, H * qk + rank, device=dev).to(bf)
    kv = torch.randn(T, H * (qk + vd), device=dev).to(bf)
    pairs = batch * sum(min(p + 1, win) for p in range(prompt_len))
    add("latent_window_attention (prefill, tcgen05 kernel with window)", False,
        _time(lambda: A.latent_window_attention(q, kv, meta.pos, H, qk, vd, qk ** -0.5, win, cu, prompt_len), 5, flush=flush),
        T * H * (2 * qk + 2 * vd) * 2, 2.0 * pairs * H * (qk + vd))
    add("latent_window_attention (prefill, CUDA-core kernel: fp32 and other head shapes)", False,
        _time(lambda: A.latent_window_attention(q, kv, meta.pos, H, qk, vd, qk ** -0.5, win), 2, warmup=1, flush=flush),
        T * H * (2 * qk + 2 * vd) * 2, 2.0 * pairs * H * (qk + vd))
    qkv = torch.randn(T, 3 * H * qk, device=dev).to(bf)
    full_pairs = batch * prompt_len * (prompt_len + 1) // 2
    add("varlen attention tcgen05 (llama, prefill, full causal)", True,
        _time(lambda: A.varlen_attention_qkv(qkv, cu, prompt_len, H, H, qk, None, True), 5, flush=flush), T * H * qk * 4 * 2, 4.0 * full_pairs * H * qk)
    # attention, decode at context `ctx`
    keys = min(ctx + 1, win)
    R = min(win, ctx + 64)
    cache = torch.randn(batch, R, rank, device=dev).to(bf)
    lens = torch.full((batch,), ctx, dtype=torch.int32, device=dev)
    qc = torch.randn(batch, H * qk + rank, device=dev).to(bf)
    w_ukv = (torch.randn(H * (qk + vd), rank, device=dev) * rank ** -0.5).to(bf)
    w_ln = torch.ones(rank, device=dev, dtype=bf)
    add(f"latent_decode_attention (ctx {ctx}, {keys} keys)", False,
        _time(lambda: A.latent_decode_attention(qc, w_ln, w_ukv, cache, lens, None, H, qk, vd, qk ** -0.5, win, 1e-5), 10, flush=flush),
        batch * keys * rank * 2 + H * (qk + vd) * rank * 2, 2.0 * batch * H * (keys * 2 * rank + (qk + vd) * rank))
    kc = torch.zeros(batch, H, ctx + 64, qk, device=dev, dtype=bf).permute(0, 2, 1, 3)
    vc = torch.zeros(batch, H, ctx + 64, qk, device=dev, dtype=bf).permute(0, 2, 1, 3)
    qkv1 = torch.randn(batch, 3 * H * qk, device=dev).to(bf)
    cos, sin = OF.rope_tables(ctx + 64, qk, 10000.0, dev)
    add(f"decode_attention (llama, ctx {ctx}, all {ctx + 1} keys)", True,
        _time(lambda: A.decode_attention(qkv1, kc, vc, lens, H, H, qk, None, cos, sin), 10, flush=flush),
        batch * (ctx + 1) * H * qk * 2 * 2, 4.0 * batch * H * (ctx + 1) * qk)
    xs = torch.randn(batch, W, device=dev)
    st = torch.zeros(batch, 3, W, device=dev)
    add("sublayer_input_step (decode)", False, _time(lambda: OF.sublayer_input_step(xs, w, 8, 1e-5, cw, st, None, bf), 10, flush=flush),
        batch * W * (6 + 24), 0)
    gu = torch.randn(T, 2 * s["ff"], device=dev).to(bf)
    add("clamped_glu (prefill)", False, _time(lambda: OF.clamped_glu(gu, 7.0, 1.702), 10, flush=flush), T * s["ff"] * 6, 0)
    add("gated_act silu (llama, prefill)", True, _time(lambda: OF.gated_act(gu, "silu"), 10, flush=flush), T * s["ff"] * 6, 0)
    return rows


def tizodra_kernel_numbers(name: str, s: dict, batch: int, prompt_len: int, ctx: int, dev, peaks: Dict[str, float]) -> List[dict]:
    """The Tizodra kernels next to the like kernels of the LLaMA path (same token count, heads and head sizes).  Attention FLOPs
    count the visible (query, key) pairs only; the delta rule has no like kernel: its floor is the fp32 FMA work (the design keeps
    the recurrence in fp32, so the bf16 tensor-core figure is not its roofline) or its bytes, whichever is slower."""
    from realhf_b200.api.model import DeltaRuleConfig, WindowAttentionConfig
    from realhf_b200.models.hetero_block import packed_meta
    from realhf_b200.ops import attention as A
    from realhf_b200.ops import functional as OF
    from realhf_b200.ops import recurrent as RC
    bf = torch.bfloat16
    W, H, G, d, dv, win, keep, taps, FF = s["width"], s["heads"], s["kv_heads"], s["dim"], s["vdim"], s["window"], s["keep"], s["conv"], s["ff"]
    T = batch * prompt_len
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    fp32_tflops = 148 * 128 * 2 * 1.9e9 / 1e12          # 148 SMs x 128 fp32 lanes x 2 flop x ~1.9 GHz
    rows = []

    def add(kernel, like, ms, nbytes, flops, simt_fp32=False):
        peak = fp32_tflops if simt_fp32 else peaks["bf16_tflops"]
        floor_ms = max(nbytes / (peaks["hbm_gbs"] * 1e9), flops / (peak * 1e12)) * 1e3
        rows.append(dict(bench="kernel", size=name, kernel=kernel, like=like, ms=round(ms, 4), gbytes=round(nbytes / 1e9, 4),
                         gflop=round(flops / 1e9, 2), roofline_ms=round(floor_ms, 4), frac_of_measured_roofline=round(floor_ms / ms, 4),
                         flop_peak="fp32 CUDA cores (nominal)" if simt_fp32 else "bf16 tensor (measured)"))

    cu = torch.arange(0, batch + 1, device=dev, dtype=torch.int32) * prompt_len
    meta = packed_meta(cu, T, torch.arange(batch, dtype=torch.int32, device=dev), None, prompt_len)
    x32 = torch.randn(T, W, device=dev)
    xb = x32.to(bf)
    w = torch.ones(W, device=dev, dtype=bf)
    # ---- row-wise
    wte = torch.randn(s["vocab"], W, device=dev).to(bf)
    ids = torch.randint(0, s["vocab"], (T,), device=dev)
    add("embed_sinusoid (prefill)", False, _time(lambda: OF.embed_sinusoid(ids, wte, meta.pos), 10, flush=flush), T * W * 6, 0)
    add("embedding lookup (llama, prefill)", True, _time(lambda: torch.nn.functional.embedding(ids, wte), 10, flush=flush), T * W * 4, 0)
    add("sublayer_input (RMSNorm of the fp32 stream, prefill)", False, _time(lambda: OF.sublayer_input(x32, w, 1, 1e-5, None, None, bf), 10, flush=flush),
        T * W * 6, 0)
    add("residual_add_norm_ (fp32 stream += branch, prefill)", False, _time(lambda: OF.residual_add_norm_(x32, xb, None, 1, 1e-5), 10, flush=flush),
        T * W * 10, 0)
    add("add_rmsnorm (llama, prefill)", True, _time(lambda: OF.add_rmsnorm(xb, xb, w, 1e-5), 10, flush=flush), T * W * 8, 0)
    up = torch.randn(T, FF, device=dev).to(bf)
    add("relu2 (prefill)", False, _time(lambda: OF.relu2(up), 10, flush=flush), T * FF * 4, 0)
    gu = torch.randn(T, 2 * FF, device=dev).to(bf)
    add("gated_act silu (llama, prefill)", True, _time(lambda: OF.gated_act(gu, "silu"), 10, flush=flush), T * FF * 6, 0)
    # ---- window attention
    a = WindowAttentionConfig(n_heads=H, n_kv_heads=G, qk_dim=d, v_dim=dv, scale=d ** -0.5, window=win, keep_first=keep)
    ld = H * d + G * (d + dv) + (H + 7) // 8 * 8
    qkvg = torch.randn(T, ld, device=dev).to(bf)
    temp = torch.ones(H, device=dev, dtype=bf)
    sink = torch.zeros(H, device=dev, dtype=bf)
    S = prompt_len + 64
    rows_c = a.cache_rows(S)
    kc = torch.zeros(batch, G, rows_c, d, device=dev, dtype=bf)
    vc = torch.zeros(batch, G, rows_c, dv, device=dev, dtype=bf)
    add("value_norm_store (prefill: value norm + cache fill)", False,
        _time(lambda: A.value_norm_store(qkvg, a, 1e-5, kc, vc, meta.tok_slot, meta.pos, meta.remain), 10, flush=flush),
        T * G * (d + 3 * dv) * 2, 0)
    v_n = A.value_norm_store(qkvg, a, 1e-5, None, None, meta.tok_slot, meta.pos, meta.remain)
    pairs = batch * sum(min(p + 1, win) + max(0, min(keep, p + 1 - win)) for p in range(prompt_len))
    add("sink_window_attention (prefill)", False,
        _time(lambda: A.sink_window_attention(qkvg, v_n, a, temp, sink, meta.pos, cu, prompt_len), 3, warmup=1, flush=flush),
        T * (H * (d + dv) + G * (d + dv)) * 2, 2.0 * pairs * H * (d + dv))
    qkv = torch.randn(T, (H + 2 * G) * d, device=dev).to(bf)
    full_pairs = batch * prompt_len * (prompt_len + 1) // 2
    add("varlen attention tcgen05 (llama, prefill, full causal)", True,
        _time(lambda: A.varlen_attention_qkv(qkv, cu, prompt_len, H, G, d, None, True), 5, flush=flush), T * (2 * H + 2 * G) * d * 2,
        4.0 * full_pairs * H * d)
    keys = min(ctx + 1, win) + max(0, min(keep, ctx + 1 - win))
    rows_d = a.cache_rows(ctx + 64)
    kc = torch.randn(batch, G, rows_d, d, device=dev).to(bf)
    vc = torch.randn(batch, G, rows_d, dv, device=dev).to(bf)
    lens = torch.full((batch,), ctx, dtype=torch.int32, device=dev)
    q1 = torch.randn(batch, ld, device=dev).to(bf)
    add(f"sink_window_decode_attention (ctx {ctx}, {keys} keys)", False,
        _time(lambda: A.sink_window_decode_attention(q1, a, temp, sink, kc, vc, lens, None, 1e-5), 10, flush=flush),
        batch * keys * G * (d + dv) * 2, 2.0 * batch * H * keys * (d + dv))
    kl = torch.zeros(batch, G, ctx + 64, d, device=dev, dtype=bf).permute(0, 2, 1, 3)
    vl = torch.zeros(batch, G, ctx + 64, d, device=dev, dtype=bf).permute(0, 2, 1, 3)
    qkv1 = torch.randn(batch, (H + 2 * G) * d, device=dev).to(bf)
    cos, sin = OF.rope_tables(ctx + 64, d, 10000.0, dev)
    add(f"decode_attention (llama, ctx {ctx}, all {ctx + 1} keys)", True,
        _time(lambda: A.decode_attention(qkv1, kl, vl, lens, H, G, d, None, cos, sin), 10, flush=flush),
        batch * (ctx + 1) * G * d * 2 * 2, 4.0 * batch * H * (ctx + 1) * d)
    # ---- delta rule
    dl = DeltaRuleConfig(n_heads=H, n_kv_heads=G, qk_dim=d, v_dim=dv, conv_taps=taps)
    C = dl.conv_channels
    ldp = C + H * dv + (2 * H + 7) // 8 * 8
    proj = torch.randn(T, ldp, device=dev).to(bf)
    conv_w = (torch.randn(C, taps, device=dev) * 0.5).to(bf)
    A_log = torch.zeros(H, device=dev, dtype=bf)
    dtb = torch.zeros(H, device=dev, dtype=bf)
    conv_state = torch.zeros(batch, taps - 1, C, device=dev)
    s_state = torch.zeros(batch, H, d, dv, device=dev)
    add("delta_prepare (prefill: conv + SiLU + unit norms + gates)", False,
        _time(lambda: RC.delta_prepare(proj, conv_w, A_log, dtb, dl, meta.pos, conv_state, meta.tok_slot, meta.remain), 10, flush=flush),
        T * (C + 2 * H) * (2 + 4), T * C * 2.0 * taps, simt_fp32=True)
    u = RC.delta_prepare(proj, conv_w, A_log, dtb, dl, meta.pos, conv_state, meta.tok_slot, meta.remain)
    add("delta_rule_scan (prefill, fp32 recurrence)", False,
        _time(lambda: RC.delta_rule_scan(u, dl, cu, s_state, meta.seq_slot), 3, warmup=1, flush=flush),
        T * (C + 2 * H + H * dv) * 4, T * H * 8.0 * d * dv, simt_fp32=True)
    o = RC.delta_rule_scan(u, dl, cu, s_state, meta.seq_slot)
    add("gated_head_norm (prefill)", False, _time(lambda: RC.gated_head_norm(o, torch.ones(dv, device=dev, dtype=bf), proj[:, C:C + H * dv], 1e-5, bf),
                                                  10, flush=flush), T * H * dv * 8, 0)
    p1 = torch.randn(batch, ldp, device=dev).to(bf)
    add("delta_prepare_step (decode)", False, _time(lambda: RC.delta_prepare_step(p1, conv_w, A_log, dtb, dl, conv_state, None), 10, flush=flush),
        batch * (C * (2 + 4 + 8 * (taps - 1)) + C * taps * 2 / batch), 0)
    u1 = RC.delta_prepare_step(p1, conv_w, A_log, dtb, dl, conv_state, None)
    add("delta_rule_step (decode: state read + write)", False, _time(lambda: RC.delta_rule_step(u1, dl, s_state, None), 10, flush=flush),
        batch * H * d * dv * 8, batch * H * 8.0 * d * dv, simt_fp32=True)
    return rows


def defilorn_kernel_numbers(name: str, s: dict, batch: int, prompt_len: int, ctx: int, dev, peaks: Dict[str, float]) -> List[dict]:
    """The Defilorn kernels next to the like kernels of the framework's other models at the same token count and head sizes: LLaMA's
    attention and row kernels, Tizodra's delta rule for the matrix-memory LSTM.  Attention FLOPs count the visible (query, key) pairs;
    the fp32 recurrences are held against the nominal fp32 CUDA-core rate or their bytes, whichever is slower."""
    from realhf_b200.api.model import DeltaRuleConfig
    from realhf_b200.models import hf_io
    from realhf_b200.models.hetero_block import packed_meta
    from realhf_b200.ops import attention as A
    from realhf_b200.ops import functional as OF
    from realhf_b200.ops import recurrent as RC
    bf = torch.bfloat16
    rc = hf_io.family("defilorn").config_from_dict(defilorn_config(s, 3), False)
    wa, ml, la = rc.blocks[0].wattn, rc.blocks[1].mlstm, rc.blocks[2].attn
    W, H, G, d, dv, win, FF = s["width"], s["heads"], s["kv_heads"], s["dim"], s["vdim"], s["window"], s["ff"]
    T = batch * prompt_len
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    fp32_tflops = 148 * 128 * 2 * 1.9e9 / 1e12
    rows = []

    def add(kernel, like, ms, nbytes, flops, simt_fp32=False):
        peak = fp32_tflops if simt_fp32 else peaks["bf16_tflops"]
        floor_ms = max(nbytes / (peaks["hbm_gbs"] * 1e9), flops / (peak * 1e12)) * 1e3
        rows.append(dict(bench="kernel", size=name, kernel=kernel, like=like, ms=round(ms, 4), gbytes=round(nbytes / 1e9, 4),
                         gflop=round(flops / 1e9, 2), roofline_ms=round(floor_ms, 4), frac_of_measured_roofline=round(floor_ms / ms, 4),
                         flop_peak="fp32 CUDA cores (nominal)" if simt_fp32 else "bf16 tensor (measured)"))

    cu = torch.arange(0, batch + 1, device=dev, dtype=torch.int32) * prompt_len
    slots = torch.arange(batch, dtype=torch.int32, device=dev)
    meta = packed_meta(cu, T, slots, None, prompt_len)
    x32 = torch.randn(T, W, device=dev)
    xb = x32.to(bf)
    w = torch.zeros(W, device=dev, dtype=bf)
    # ---- row-wise
    add("add_rms_norm_ (fp32 stream += branch, norm with 1 + w, prefill)", False, _time(lambda: OF.add_rms_norm_(x32, xb, w, 1e-5, bf, 1.0), 10, flush=flush),
        T * W * 12, 0)
    add("add_rmsnorm (llama, prefill)", True, _time(lambda: OF.add_rmsnorm(xb, xb, w, 1e-5), 10, flush=flush), T * W * 8, 0)
    gu = torch.randn(T, 2 * FF, device=dev).to(bf)
    add("gated_act gelu_tanh (prefill, stand-alone; the prefill path has it in the GEMM epilogue)", False, _time(lambda: OF.gated_act(gu, "gelu_tanh"), 10, flush=flush), T * FF * 6, 0)
    add("gated_act silu (llama, prefill)", True, _time(lambda: OF.gated_act(gu, "silu"), 10, flush=flush), T * FF * 6, 0)
    # ---- differential window attention
    ld = 2 * H * d + 2 * G * d + G * dv
    qkv = torch.randn(T, ld, device=dev).to(bf)
    wn = torch.ones(d, device=dev, dtype=bf)
    lamw = (torch.randn(4, d, device=dev) * 0.1).to(bf)
    rows_c = wa.cache_rows(prompt_len + 64)
    kc = torch.zeros(batch, 2 * G, rows_c, d, device=dev, dtype=bf)
    vc = torch.zeros(batch, G, rows_c, dv, device=dev, dtype=bf)
    from realhf_b200.ops import lib
    add("qk_head_norm_ (prefill)", False, _time(lambda: lib().qk_head_norm_(qkv, wn, wn, 2 * H, 2 * G, d, 1e-5), 10, flush=flush), T * (2 * H + 2 * G) * d * 4, 0)
    pairs = batch * sum(min(p + 1, win) for p in range(prompt_len))
    add("diff_window_attention (prefill: norms + cache fill + both maps + combine)", False,
        _time(lambda: A.diff_window_attention(qkv, wa, wn, wn, lamw, 1e-5, kc, vc, meta.tok_slot, meta.pos, meta.remain, cu, prompt_len), 3, warmup=1, flush=flush),
        T * (ld + H * dv) * 2, 2.0 * pairs * 2 * H * (d + dv))
    qkv_l = torch.randn(T, (H + 2 * G) * d, device=dev).to(bf)
    full_pairs = batch * prompt_len * (prompt_len + 1) // 2
    add("varlen attention tcgen05 (llama, prefill, full causal)", True,
        _time(lambda: A.varlen_attention_qkv(qkv_l, cu, prompt_len, H, G, d, None, True), 5, flush=flush), T * (2 * H + 2 * G) * d * 2, 4.0 * full_pairs * H * d)
    keys = min(ctx + 1, win)
    rows_d = wa.cache_rows(ctx + 64)
    kc = torch.randn(batch, 2 * G, rows_d, d, device=dev).to(bf)
    vc = torch.randn(batch, G, rows_d, dv, device=dev).to(bf)
    lens = torch.full((batch,), ctx, dtype=torch.int32, device=dev)
    q1 = torch.randn(batch, ld, device=dev).to(bf)
    add(f"diff_window_decode_attention (ctx {ctx}, {keys} keys, both maps)", False,
        _time(lambda: A.diff_window_decode_attention(q1, wa, wn, wn, lamw, 1e-5, kc, vc, lens, None), 10, flush=flush),
        batch * keys * G * (2 * d + dv) * 2, 2.0 * batch * 2 * H * keys * (d + dv))
    kl = torch.zeros(batch, G, ctx + 64, d, device=dev, dtype=bf).permute(0, 2, 1, 3)
    vl = torch.zeros(batch, G, ctx + 64, d, device=dev, dtype=bf).permute(0, 2, 1, 3)
    qkv1 = torch.randn(batch, (H + 2 * G) * d, device=dev).to(bf)
    cos, sin = OF.rope_tables(ctx + 64, d, 10000.0, dev)
    add(f"decode_attention (llama, ctx {ctx}, all {ctx + 1} keys)", True,
        _time(lambda: A.decode_attention(qkv1, kl, vl, lens, H, G, d, None, cos, sin), 10, flush=flush),
        batch * (ctx + 1) * G * d * 2 * 2, 4.0 * batch * H * (ctx + 1) * d)
    # ---- rotated latent attention
    r, rot, dn, qr = la.kv_rank, la.rot_dim, la.qk_dim, la.q_rank
    dq = dn + rot
    proj = torch.randn(T, qr + r + rot + H * dv, device=dev).to(bf)
    wq, wc = torch.ones(qr, device=dev, dtype=bf), torch.ones(r, device=dev, dtype=bf)
    cache = torch.zeros(batch, prompt_len + 64, r + rot, device=dev, dtype=bf)
    add("latent_rope_prepare (prefill: two norms + rotation + cache fill)", False,
        _time(lambda: A.latent_rope_prepare(proj, la, wq, wc, 1e-5, meta.pos, cache, meta.tok_slot, meta.remain), 10, flush=flush),
        T * (qr + r + rot) * 2 * 2 + T * (r + rot) * 2, 0)
    cq, latent = A.latent_rope_prepare(proj, la, wq, wc, 1e-5, meta.pos, cache, meta.tok_slot, meta.remain)
    q = torch.randn(T, H * dq, device=dev).to(bf)
    kv = torch.randn(T, H * (dn + dv), device=dev).to(bf)
    sink = torch.zeros(H, device=dev, dtype=bf)
    add("latent_rope_attention (prefill: rotate + assemble + causal attention with a sink)", False,
        _time(lambda: A.latent_rope_attention(q, kv, latent, la, sink, meta.pos, cu, prompt_len), 3, warmup=1, flush=flush),
        T * H * (dq + dn + 2 * dv) * 2 + T * 2 * H * dq * 2 * 2, 2.0 * full_pairs * H * (dq + dv))
    o = torch.randn(T, H * dv, device=dev).to(bf)
    add("sigmoid_gate_ (prefill)", False, _time(lambda: A.sigmoid_gate_(o, proj[:, qr + r + rot:]), 10, flush=flush), T * H * dv * 6, 0)
    cache = torch.randn(batch, ctx + 64, r + rot, device=dev).to(bf)
    w_ukv = (torch.randn(H * (dn + dv), r, device=dev) * r ** -0.5).to(bf)
    q1l = torch.randn(batch, H * dq, device=dev).to(bf)
    add(f"latent_rope_decode_attention (ctx {ctx}, all {ctx + 1} keys)", False,
        _time(lambda: A.latent_rope_decode_attention(q1l, la, w_ukv, sink, cache, lens, None), 10, flush=flush),
        batch * (ctx + 1) * (r + rot) * 2 + H * (dn + dv) * r * 4, 2.0 * batch * H * ((ctx + 1) * (2 * r + rot) + (dn + dv) * r))
    # ---- matrix-memory LSTM next to the delta rule
    ldm = 2 * H * d + 2 * H * dv + (2 * H + 7) // 8 * 8
    pm = (torch.randn(T, ldm, device=dev) * 0.5).to(bf)
    gb = torch.zeros(2 * H, device=dev, dtype=bf)
    S = torch.zeros(batch, H, d, dv + 1, device=dev)
    M = torch.zeros(batch, H, device=dev)
    add("mlstm_scan (prefill, fp32 recurrence)", False, _time(lambda: RC.mlstm_scan(pm, gb, ml, cu, S, M, slots), 3, warmup=1, flush=flush),
        T * (2 * H * d + H * dv) * 2 + T * H * (dv + 2) * 4, T * H * 6.0 * d * (dv + 1), simt_fp32=True)
    dl = DeltaRuleConfig(n_heads=H, n_kv_heads=H, qk_dim=d, v_dim=dv, conv_taps=1)
    u = torch.randn(T, dl.conv_channels + 2 * H, device=dev) * 0.1
    u[:, -2 * H:] = 0.5
    s_state = torch.zeros(batch, H, d, dv, device=dev)
    add("delta_rule_scan (tizodra, prefill, fp32 recurrence)", True, _time(lambda: RC.delta_rule_scan(u, dl, cu, s_state, slots), 3, warmup=1, flush=flush),
        T * (dl.conv_channels + 2 * H + H * dv) * 4, T * H * 8.0 * d * dv, simt_fp32=True)
    om, mm = RC.mlstm_scan(pm, gb, ml, cu, S, M, slots)
    wo = torch.ones(H * dv, device=dev, dtype=bf)
    add("mlstm_out (prefill: denominator + head norm + weight + gate)", False,
        _time(lambda: RC.mlstm_out(om, mm, wo, pm[:, 2 * H * d + H * dv:], 1e-5, bf), 10, flush=flush), T * H * dv * 8, 0)
    od = torch.randn(T, H, dv, device=dev)
    add("gated_head_norm (tizodra, prefill)", True,
        _time(lambda: RC.gated_head_norm(od, torch.ones(dv, device=dev, dtype=bf), pm[:, 2 * H * d + H * dv:2 * H * d + 2 * H * dv], 1e-5, bf), 10, flush=flush),
        T * H * dv * 8, 0)
    p1 = (torch.randn(batch, ldm, device=dev) * 0.5).to(bf)
    add("mlstm_step (decode: state read + write)", False, _time(lambda: RC.mlstm_step(p1, gb, ml, S, M, None), 10, flush=flush),
        batch * H * d * (dv + 1) * 8, batch * H * 6.0 * d * (dv + 1), simt_fp32=True)
    u1 = torch.randn(batch, dl.conv_channels + 2 * H, device=dev) * 0.1
    add("delta_rule_step (tizodra, decode: state read + write)", True, _time(lambda: RC.delta_rule_step(u1, dl, s_state, None), 10, flush=flush),
        batch * H * d * dv * 8, batch * H * 8.0 * d * dv, simt_fp32=True)
    return rows


def buvesun_kernel_numbers(name: str, s: dict, batch: int, prompt_len: int, ctx: int, dev, peaks: Dict[str, float]) -> List[dict]:
    """The Buvesun kernels next to the like kernels of the closest models at the same token count and head sizes: Defilorn's
    matrix-memory LSTM and fused add + norm, its router and combination, LLaMA's rotation and attention.  Attention FLOPs count the
    visible (query, key) pairs; the fp32 recurrences are held against the nominal fp32 CUDA-core rate or their bytes, whichever is
    slower."""
    from realhf_b200.models import hf_io
    from realhf_b200.models.hetero_block import packed_meta
    from realhf_b200.ops import attention as A
    from realhf_b200.ops import functional as OF
    from realhf_b200.ops import lib
    from realhf_b200.ops import recurrent as RC
    bf = torch.bfloat16
    rc = hf_io.family("buvesun").config_from_dict(buvesun_config(s, 2), False)
    wa, lt, rt = rc.blocks[0].wattn, rc.blocks[0].decay, rc.blocks[1].decay
    ml = hf_io.family("defilorn").config_from_dict(defilorn_config(s, 3), False).blocks[1].mlstm
    W, H, G, d, dv, win, HR = s["width"], s["heads"], s["kv_heads"], s["dim"], s["vdim"], s["window"], s["r_heads"]
    T = batch * prompt_len
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    fp32_tflops = 148 * 128 * 2 * 1.9e9 / 1e12
    rows = []

    def add(kernel, like, ms, nbytes, flops, simt_fp32=False):
        peak = fp32_tflops if simt_fp32 else peaks["bf16_tflops"]
        floor_ms = max(nbytes / (peaks["hbm_gbs"] * 1e9), flops / (peak * 1e12)) * 1e3
        rows.append(dict(bench="kernel", size=name, kernel=kernel, like=like, ms=round(ms, 4), gbytes=round(nbytes / 1e9, 4),
                         gflop=round(flops / 1e9, 2), roofline_ms=round(floor_ms, 4), frac_of_measured_roofline=round(floor_ms / ms, 4),
                         flop_peak="fp32 CUDA cores (nominal)" if simt_fp32 else "bf16 tensor (measured)"))

    cu = torch.arange(0, batch + 1, device=dev, dtype=torch.int32) * prompt_len
    slots = torch.arange(batch, dtype=torch.int32, device=dev)
    meta = packed_meta(cu, T, slots, None, prompt_len)
    x32 = torch.randn(T, W, device=dev)
    xb, yb = x32.to(bf), torch.randn(T, W, device=dev).to(bf)
    w = torch.ones(W, device=dev, dtype=bf)
    # ---- row-wise
    add("centred_norm (LayerNorm of the fp32 stream, prefill)", False, _time(lambda: OF.centred_norm(x32, w, 1e-5, bf), 10, flush=flush), T * W * 6, 0)
    add("residual_add_centred_norm_ (two branches, output norm, layer scale, add, next norm; prefill)", False,
        _time(lambda: OF.residual_add_centred_norm_(x32, xb, w, 1e-5, w, 0.7, yb, 0.6, 1.1, w, bf), 10, flush=flush), T * W * 14, 0)
    add("add_rms_norm_ (defilorn: fp32 stream += branch, next norm; prefill)", True, _time(lambda: OF.add_rms_norm_(x32, xb, w, 1e-5, bf, 1.0), 10, flush=flush),
        T * W * 12, 0)
    add("add_rmsnorm (llama, prefill)", True, _time(lambda: OF.add_rmsnorm(xb, xb, w, 1e-5), 10, flush=flush), T * W * 8, 0)
    # ---- window attention with rotation
    ld = H * d + G * (d + dv)
    proj = torch.randn(T, ld + lt.width, device=dev).to(bf)
    left, right = proj[:, :ld], proj[:, ld:]
    add("rotate_heads_ (prefill: q and k in place, fp32 angles)", False, _time(lambda: A.rotate_qk_(left, wa, pos=meta.pos), 10, flush=flush),
        T * (H + G) * wa.rotary.dims * 4, 0)
    qkv_l = torch.randn(T, (H + 2 * G) * d, device=dev).to(bf)
    cos, sin = OF.rope_tables(prompt_len + 64, d, 10000.0, dev)
    add("apply_rope (llama, prefill: q and k, table look-up)", True,
        _time(lambda: OF.apply_rope(qkv_l[:, :(H + G) * d], cos, sin, meta.pos, H + G, d), 10, flush=flush), T * (H + G) * d * 4, 0)
    rows_c = wa.cache_rows(prompt_len + 64)
    kc = torch.zeros(batch, G, rows_c, d, device=dev, dtype=bf)
    vc = torch.zeros(batch, G, rows_c, dv, device=dev, dtype=bf)
    add("value_norm_store (prefill: cache fill)", False,
        _time(lambda: A.value_norm_store(left, wa, 1e-5, kc, vc, meta.tok_slot, meta.pos, meta.remain), 10, flush=flush), T * G * (d + 3 * dv) * 2, 0)
    v_n = A.value_norm_store(left, wa, 1e-5, None, None, meta.tok_slot, meta.pos, meta.remain)
    pairs = batch * sum(min(p + 1, win) for p in range(prompt_len))
    add("sink_window_attention (prefill, tcgen05, window)", False,
        _time(lambda: A.sink_window_attention(left, v_n, wa, None, None, meta.pos, cu, prompt_len), 3, warmup=1, flush=flush),
        T * (H * (d + dv) + G * (d + dv)) * 2, 2.0 * pairs * H * (d + dv))
    full_pairs = batch * prompt_len * (prompt_len + 1) // 2
    add("varlen attention tcgen05 (llama, prefill, full causal)", True,
        _time(lambda: A.varlen_attention_qkv(qkv_l, cu, prompt_len, H, G, d, None, True), 5, flush=flush), T * (2 * H + 2 * G) * d * 2,
        4.0 * full_pairs * H * d)
    keys = min(ctx + 1, win)
    rows_d = wa.cache_rows(ctx + 64)
    kc = torch.randn(batch, G, rows_d, d, device=dev).to(bf)
    vc = torch.randn(batch, G, rows_d, dv, device=dev).to(bf)
    lens = torch.full((batch,), ctx, dtype=torch.int32, device=dev)
    q1 = torch.randn(batch, ld, device=dev).to(bf)
    add(f"sink_window_decode_attention (ctx {ctx}, {keys} keys)", False,
        _time(lambda: A.sink_window_decode_attention(q1, wa, None, None, kc, vc, lens, None, 1e-5), 10, flush=flush),
        batch * keys * G * (d + dv) * 2, 2.0 * batch * H * keys * (d + dv))
    kl = torch.zeros(batch, G, ctx + 64, d, device=dev, dtype=bf).permute(0, 2, 1, 3)
    vl = torch.zeros(batch, G, ctx + 64, d, device=dev, dtype=bf).permute(0, 2, 1, 3)
    qkv1 = torch.randn(batch, (H + 2 * G) * d, device=dev).to(bf)
    cos2, sin2 = OF.rope_tables(ctx + 64, d, 10000.0, dev)
    add(f"decode_attention (llama, ctx {ctx}, all {ctx + 1} keys)", True,
        _time(lambda: A.decode_attention(qkv1, kl, vl, lens, H, G, d, None, cos2, sin2), 10, flush=flush),
        batch * (ctx + 1) * G * d * 2 * 2, 4.0 * batch * H * (ctx + 1) * d)
    # ---- decayed linear attention next to the matrix-memory LSTM
    nu = 2 * HR * d + HR * dv
    S = torch.zeros(batch, HR, d, dv, device=dev)
    for label, dc, src in (("retention: rotation + key factor", rt, torch.randn(T, rt.width, device=dev).mul(0.5).to(bf)),
                           ("lightning: SiLU", lt, right)):
        add(f"decay_prepare (prefill, {label})", False, _time(lambda: RC.decay_prepare(src, dc, pos=meta.pos), 10, flush=flush), T * nu * 6, 0)
    u = RC.decay_prepare(right, lt, pos=meta.pos)
    add("decay_scan (prefill, fp32 recurrence)", False, _time(lambda: RC.decay_scan(u, lt, cu, S, slots), 3, warmup=1, flush=flush),
        T * nu * 4 + T * HR * dv * 4, T * HR * 5.0 * d * dv, simt_fp32=True)
    ldm = 2 * HR * d + 2 * HR * dv + (2 * HR + 7) // 8 * 8
    pm = (torch.randn(T, ldm, device=dev) * 0.5).to(bf)
    gb = torch.zeros(2 * HR, device=dev, dtype=bf)
    Sm = torch.zeros(batch, HR, d, dv + 1, device=dev)
    Mm = torch.zeros(batch, HR, device=dev)
    import dataclasses
    ml = dataclasses.replace(ml, n_heads=HR)
    add("mlstm_scan (defilorn, prefill, fp32 recurrence)", True, _time(lambda: RC.mlstm_scan(pm, gb, ml, cu, Sm, Mm, slots), 3, warmup=1, flush=flush),
        T * (2 * HR * d + HR * dv) * 2 + T * HR * (dv + 2) * 4, T * HR * 6.0 * d * (dv + 1), simt_fp32=True)
    o = RC.decay_scan(u, lt, cu, S, slots)
    wo = torch.ones(HR * dv, device=dev, dtype=bf)
    gate = right[:, nu:]
    add("decay_out (prefill, full-width norm + weight + sigmoid gate)", False, _time(lambda: RC.decay_out(o, lt, wo, gate, 1e-5, bf), 10, flush=flush),
        T * HR * dv * 8, 0)
    add("decay_out (prefill, per-head norm + SiLU gate)", False, _time(lambda: RC.decay_out(o, rt, None, gate, 1e-5, bf), 10, flush=flush),
        T * HR * dv * 8, 0)
    om, mm = RC.mlstm_scan(pm, gb, ml, cu, Sm, Mm, slots)
    add("mlstm_out (defilorn, prefill)", True, _time(lambda: RC.mlstm_out(om, mm, wo, pm[:, 2 * HR * d + HR * dv:], 1e-5, bf), 10, flush=flush),
        T * HR * dv * 8, 0)
    u1 = torch.randn(batch, nu, device=dev) * 0.1
    add("decay_step (decode: state read + write)", False, _time(lambda: RC.decay_step(u1, lt, S, None), 10, flush=flush),
        batch * HR * d * dv * 8, batch * HR * 5.0 * d * dv, simt_fp32=True)
    p1 = (torch.randn(batch, ldm, device=dev) * 0.5).to(bf)
    add("mlstm_step (defilorn, decode: state read + write)", True, _time(lambda: RC.mlstm_step(p1, gb, ml, Sm, Mm, None), 10, flush=flush),
        batch * HR * d * (dv + 1) * 8, batch * HR * 6.0 * d * (dv + 1), simt_fp32=True)
    # ---- routing
    E, k = s["experts"], s["top"]
    wr = (torch.randn(E, W, device=dev) * W ** -0.5).to(bf)
    add("softmax_router (sigmoid scores, prefill)", False, _time(lambda: lib().softmax_router(xb, wr, None, None, k, False, True), 10, flush=flush),
        T * W * 2, 2.0 * T * W * E)
    add("softmax_router (defilorn: softmax scores, prefill)", True, _time(lambda: lib().softmax_router(xb, wr, None, None, k, False, False), 10, flush=flush),
        T * W * 2, 2.0 * T * W * E)
    xd = xb[:batch]
    probs, idx, _ = lib().softmax_router(xd, wr, None, None, k, False, True)
    row, _ = lib().moe_dispatch(idx, E, E)
    add("moe_gather (decode, rows times their routing weight)", False, _time(lambda: lib().moe_gather(xd, row, k, probs), 10, flush=flush),
        batch * k * W * 4, 0)
    add("moe_gather (defilorn, decode, plain copy)", True, _time(lambda: lib().moe_gather(xd, row, k), 10, flush=flush), batch * k * W * 4, 0)
    return rows


def run(design: str, sizes: List[str] = None, n_layers: int = 4) -> List[dict]:
    assert design in ("rapodra", "tizodra", "defilorn", "buvesun")
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    peaks = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")
    pk = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        with open(pk) as f:
            d = json.load(f)
        if "hbm_gbs" in d and "bf16_tflops" in d:
            peaks = dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]), source="measured")
    results = [dict(bench="peaks", **peaks)]
    table = {"rapodra": SIZES, "tizodra": TIZODRA_SIZES, "defilorn": DEFILORN_SIZES, "buvesun": BUVESUN_SIZES}[design]
    for name in sizes or list(table):
        s = table[name]
        results += model_numbers(name, s, n_layers, batch=32, prompt_len=1024, new_tokens=33, dev=dev, design=design)
        kn = {"rapodra": kernel_numbers, "tizodra": tizodra_kernel_numbers, "defilorn": defilorn_kernel_numbers,
              "buvesun": buvesun_kernel_numbers}[design]
        results += kn(name, s, batch=32, prompt_len=1024, ctx=2048, dev=dev, peaks=peaks)
    for r in results:
        print(json.dumps(r), flush=True)
    return results
