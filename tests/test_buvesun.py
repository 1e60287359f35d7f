"""Buvesun (heterogeneous "layer" stack: bias-free LayerNorm around every sublayer with layer scale and a residual factor,
retention, sliding-window attention with partial interleaved rotation beside lightning attention, sigmoid-routed clamped experts
whose weight scales the expert's input, a shared expert, a looped range of blocks with the embedding output projected back in)
against the plain float64 implementation in `buvesun_oracle.py`.

Every test body runs on the CPU (the op layer's PyTorch references, part of the default suite) and, marked `gpu`, on CUDA (the
sm_100a kernels) in fp32 and bf16.  Configurations are small and made here; none is a released model's."""

import copy
import json
import os
import subprocess
import sys

import pytest
import torch

import buvesun_oracle as O
from realhf_b200.api.model import GenerationHyperparameters
from realhf_b200.models import generation as gen
from realhf_b200.models import hf_io
from realhf_b200.models.real_model import ReaLModel

CPU = pytest.param("cpu", torch.float32, id="cpu-f32")
GPU32 = pytest.param("cuda", torch.float32, id="cuda-f32", marks=pytest.mark.gpu)
GPU16 = pytest.param("cuda", torch.bfloat16, id="cuda-bf16", marks=pytest.mark.gpu)
ALL = [CPU, GPU32, GPU16]
EXACT = [CPU, GPU32]


def tol(dtype):
    return 2e-4 if dtype == torch.float32 else 0.15


def row_errs(got, want):
    """Per row: root mean square of the difference (mean removed) over the last dim, relative to the spread of `want`."""
    d = got.double().cpu() - want.double()
    d = d - d.mean(-1, keepdim=True)
    return (d.pow(2).mean(-1).sqrt() / want.double().std(-1).clamp_min(1e-6)).reshape(-1)


def model_ok(errs, dtype):
    errs = torch.cat([e.reshape(-1) for e in errs]) if isinstance(errs, (list, tuple)) else errs
    if dtype == torch.float32:
        return float(errs.max()) < tol(dtype)
    return float((errs > tol(dtype)).float().mean()) <= 0.05


def build(cfg: dict, w: dict, device, dtype) -> ReaLModel:
    fam = hf_io.family("buvesun")
    rc = fam.config_from_dict(cfg, False)
    m = ReaLModel(rc, dtype=dtype, device=device).instantiate(init="empty")
    m.load_state_dict(fam.sd_from_hf(w, rc))
    for p in m.parameters():
        p.requires_grad_(False)
    return m.eval()


def toks(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def packed_logits(m, seqs, trace=None):
    dev = m.device
    ids = torch.tensor([x for s in seqs for x in s], device=dev)
    cu = torch.tensor([0] + [len(s) for s in seqs], device=dev).cumsum(0).int()
    with torch.no_grad():
        if trace is not None:
            return m._forward_hetero(ids, cu, None, None, max(len(s) for s in seqs), trace=trace).logits
        return m(input_ids=ids, cu_seqlens=cu).logits


def decoded_logits(m, seq, cut, max_len=None):
    """The first `cut` tokens as a prompt, the rest one by one through the state: logits of every position."""
    sess = gen.StepSession(m, max_len=max_len or len(seq) + 1, n_slots=2)
    rows = [sess.logits(sess.prefill([("a", seq[:cut])]))]
    rows += [sess.logits(sess.decode([("a", t)])) for t in seq[cut:]]
    return torch.cat(rows)


# ------------------------------------------------------------------------------------------------ configurations

def moe(experts=4, top=2, ff=16, limit=1.5, shared=24, shared_limit=2.5):
    f = dict(expert=dict(ff=ff, limit=limit), kind="moe", router=dict(experts=experts, top=top))
    if shared:
        f["shared"] = dict(ff=shared, limit=shared_limit)
    return f


def ret(heads=3, dim=8, vdim=12, rot=4, base=10000.0, decay=None, mlp=None):
    m = dict(decay=decay or [1.0 - 2.0 ** (-2 - h) for h in range(heads)], dim=dim, heads=heads, vdim=vdim)
    if rot:
        m["rot"] = dict(base=base, dims=rot)
    return dict(type="retention", mixer=m, mlp=mlp)


def par(heads=4, kv_heads=2, dim=12, vdim=8, window=5, rot=6, base=500.0, scale=None, r_heads=2, r_dim=8, r_vdim=12, r_decay=None,
        left_scale=0.7, right_scale=1.2, mlp=None):
    left = dict(dim=dim, heads=heads, kv_heads=kv_heads, scale=scale or dim ** -0.5, vdim=vdim)
    if window is not None:
        left["mask"] = dict(size=window)
    if rot:
        left["rot"] = dict(base=base, dims=rot)
    right = dict(decay=r_decay or [0.6 + 0.39 * h / max(r_heads - 1, 1) for h in range(r_heads)], dim=r_dim, heads=r_heads, vdim=r_vdim)
    return dict(type="parallel", mixer=dict(left=left, left_scale=left_scale, right=right, right_scale=right_scale), mlp=mlp)


def model_cfg(layers, loop=None, width=32, vocab=96, eps=1e-5, embed_scale=2.0, mult=0.6):
    c = dict(architecture="Buvesun", embedding=dict(scale=embed_scale), layers=layers, norm=dict(eps=eps), residual_mult=mult, vocab=vocab,
             width=width)
    if loop:
        c["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
    return c


CONFIGS = {
    # both mixers, blocks with and without a feed-forward, a loop over the last two layers
    "mixed": lambda: model_cfg([par(mlp=moe()), ret(mlp=None), par(mlp=moe(experts=3, top=3, shared=None)), ret(mlp=moe(top=1))], (2, 4, 2)),
    # every count that can be 1 is 1: one head, one expert, one pass, window 1, factors 1
    "ones": lambda: model_cfg([par(heads=1, kv_heads=1, window=1, r_heads=1, left_scale=1.0, right_scale=1.0, mlp=moe(experts=1, top=1, shared=8)),
                               ret(heads=1, mlp=None)], (1, 2, 1), width=16, vocab=40, embed_scale=1.0, mult=1.0),
    # sizes that are not multiples of four, heads = kv heads, no window, rotation over all dimensions, the whole stack looped three times
    "odd": lambda: model_cfg([ret(heads=3, dim=10, vdim=7, rot=10, mlp=moe(experts=5, top=4, ff=12, shared=None)),
                              par(heads=3, kv_heads=3, dim=6, vdim=10, window=None, rot=6, r_heads=3, r_dim=33, r_vdim=5, mlp=None)], (0, 2, 3),
                             width=24, vocab=50),
    # no loop, no rotation; wide heads (the matrix state split over several lanes), a window longer than the prompts
    "wide": lambda: model_cfg([ret(heads=1, dim=72, vdim=40, rot=0, mlp=moe(ff=32)),
                               par(heads=6, kv_heads=2, dim=16, vdim=24, window=200, rot=0, r_heads=2, r_dim=130, r_vdim=36, mlp=moe(top=2, shared=16))],
                              None, width=40, vocab=64),
}


def one_layer(layer, width=32, vocab=64, **kw):
    return model_cfg([layer], None, width=width, vocab=vocab, **kw)


MECHANISMS = {
    "retention-small": lambda: one_layer(ret()),
    "retention-33x7": lambda: one_layer(ret(heads=3, dim=33, vdim=7, rot=32)),
    "retention-130x40": lambda: one_layer(ret(heads=1, dim=130, vdim=40, rot=64, base=1e5)),
    "retention-64x64-full-rotation": lambda: one_layer(ret(heads=2, dim=64, vdim=64, rot=64)),
    "parallel-small": lambda: one_layer(par()),
    "parallel-window1": lambda: one_layer(par(heads=2, kv_heads=1, dim=20, vdim=24, window=1, rot=20)),
    "parallel-nowindow": lambda: one_layer(par(heads=6, kv_heads=2, dim=16, vdim=40, window=None, rot=8)),
    "parallel-odd": lambda: one_layer(par(heads=3, kv_heads=3, dim=7, vdim=9, window=33, rot=2, r_heads=1, r_dim=5, r_vdim=3)),
    "parallel-left-only": lambda: one_layer(par(right_scale=0.0)),
    "parallel-right-only": lambda: one_layer(par(left_scale=0.0)),
    "moe-ff": lambda: one_layer(ret(mlp=moe(experts=6, top=3, ff=8, shared=16))),
    "moe-top1-noshared": lambda: one_layer(ret(mlp=moe(experts=3, top=1, ff=8, shared=None))),
    "moe-all-chosen": lambda: one_layer(ret(mlp=moe(experts=4, top=4, ff=8, shared=8, limit=0.5, shared_limit=0.25))),
    "plain-residual": lambda: one_layer(ret(mlp=moe()), embed_scale=1.0, mult=1.0),
}


@pytest.mark.parametrize("device,dtype", ALL)
@pytest.mark.parametrize("name", list(MECHANISMS))
def test_mechanism_alone_prompt_then_decoding(device, dtype, name):
    """A one-layer model: packed prompts of unequal lengths (1 and 2 tokens among them) against the oracle, then the prompts'
    continuation token by token through the state the prefill left, in shuffled slots."""
    cfg = MECHANISMS[name]()
    w = O.random_checkpoint(cfg, 11)
    m = build(cfg, w, device, dtype)
    V = cfg["vocab"]
    seqs = [toks(n, V, 20 + n) for n in (1, 2, 37, 9)]
    more = 14
    full = [s + toks(more, V, 90 + len(s)) for s in seqs]
    want = [O.forward(cfg, w, s) for s in full]
    got = packed_logits(m, seqs)
    off, errs = 0, []
    for s, wl in zip(seqs, want):
        errs.append(row_errs(got[off:off + len(s)], wl[:len(s)]))
        off += len(s)
    sess = gen.StepSession(m, max_len=64, n_slots=6)
    sess.state.free_slots = [4, 1, 5, 0, 2, 3]
    h = sess.prefill(list(enumerate(seqs)))
    errs.append(row_errs(sess.logits(h[-1:]), want[-1][len(seqs[-1]) - 1][None]))
    for k in range(more):
        hh = sess.decode([(i, full[i][len(seqs[i]) + k]) for i in range(len(seqs))])
        lg = sess.logits(hh)
        errs += [row_errs(lg[i:i + 1], want[i][len(seqs[i]) + k][None]) for i in range(len(seqs))]
    assert model_ok(errs, dtype), float(torch.cat(errs).max())


TC_SHAPES = {
    "window-64-150": lambda: one_layer(par(heads=4, kv_heads=2, dim=64, vdim=64, window=150, rot=32, r_heads=2, r_dim=64, r_vdim=64), width=64),
    "window-128-128": lambda: one_layer(par(heads=2, kv_heads=2, dim=128, vdim=128, window=128, rot=128, base=1e5, r_heads=1, r_dim=128, r_vdim=128),
                                        width=64),
    "nowindow-64-rep4": lambda: one_layer(par(heads=4, kv_heads=1, dim=64, vdim=64, window=None, rot=16, r_heads=1, r_dim=32, r_vdim=64), width=64),
}


@pytest.mark.parametrize("device,dtype", [CPU, GPU32, GPU16])
@pytest.mark.parametrize("name", list(TC_SHAPES))
def test_head_shapes_of_the_tensor_core_and_streaming_kernels(device, dtype, name):
    """Head sizes 64 / 128 with equal query and value size: in 16 bit the prompts run the tcgen05 window kernel on the rotated
    queries and keys and decoding the streaming kernel; sequences of 1, 130 and 300 tokens cross the 128-key tiles and the window."""
    cfg = TC_SHAPES[name]()
    w = O.random_checkpoint(cfg, 21)
    m = build(cfg, w, device, dtype)
    V = cfg["vocab"]
    seqs = [toks(n, V, 20 + n) for n in (1, 130, 300)]
    more = 6
    full = [s + toks(more, V, 90 + len(s)) for s in seqs]
    want = [O.forward(cfg, w, s) for s in full]
    sess = gen.StepSession(m, max_len=320, n_slots=3)
    h = sess.prefill(list(enumerate(seqs)))
    lg = sess.logits(h)
    off, errs = 0, []
    for s, wl in zip(seqs, want):
        errs.append(row_errs(lg[off:off + len(s)], wl[:len(s)]))
        off += len(s)
    for k in range(more):
        lg = sess.logits(sess.decode([(i, full[i][len(seqs[i]) + k]) for i in range(3)]))
        errs += [row_errs(lg[i:i + 1], want[i][len(seqs[i]) + k][None]) for i in range(3)]
    assert model_ok(errs, dtype), float(torch.cat(errs).max())


# ------------------------------------------------------------------------------------------------ edges, made to show


@pytest.mark.parametrize("device,dtype", EXACT)
@pytest.mark.parametrize("mode", ["prompt", "decode"])
def test_window_edge_one_token_off_changes_the_output(device, dtype, mode):
    """The window branch alone (right factor 0), window 6, sharp scores (large scale): every query puts nearly all its weight on one
    key, so a window one token too long or too short picks another key for some query and the logits move by far more than the
    tolerance.  The oracle is first shown to be that sensitive (window 5 and 7 differ); prompt and decoding forms are then held
    against it.  Decoding runs 34 tokens past the ring's size, so rows of the ring are overwritten several times."""
    cfg = one_layer(par(heads=2, kv_heads=1, dim=8, vdim=12, window=6, rot=4, scale=6.0, right_scale=0.0))
    w = O.random_checkpoint(cfg, 5)
    seq = toks(40, cfg["vocab"], 77)
    want = O.forward(cfg, w, seq)
    for other in (5, 7):
        c2 = copy.deepcopy(cfg)
        c2["layers"][0]["mixer"]["left"]["mask"]["size"] = other
        assert float(row_errs(O.forward(c2, w, seq)[8:], want[8:]).max()) > 0.05
    m = build(cfg, w, device, dtype)
    got = packed_logits(m, [seq]) if mode == "prompt" else decoded_logits(m, seq, 3, max_len=48)
    assert float(row_errs(got, want).max()) < tol(dtype)


@pytest.mark.parametrize("device,dtype", EXACT)
@pytest.mark.parametrize("mode", ["prompt", "decode"])
def test_token_outside_the_window_is_invisible_and_inside_visible(device, dtype, mode):
    """The window branch alone over 30 tokens with window 9: changing the token 9 back from the last one (just outside) leaves the
    last logits as they were, changing the token 8 back (just inside) moves them; in the oracle and equally here."""
    cfg = one_layer(par(heads=2, kv_heads=2, dim=8, vdim=8, window=9, rot=8, right_scale=0.0), vocab=32)
    w = O.random_checkpoint(cfg, 15)
    seq = toks(30, 32, 3)
    m = build(cfg, w, device, dtype)

    def last(s):
        return (packed_logits(m, [s]) if mode == "prompt" else decoded_logits(m, s, 12))[-1:]
    base = last(seq)
    assert float(row_errs(base, O.forward(cfg, w, seq)[-1:]).max()) < tol(dtype)
    for back, seen in ((9, False), (8, True)):
        s2 = list(seq)
        s2[-1 - back] = (s2[-1 - back] + 5) % 32
        moved = float(row_errs(last(s2), base.double().cpu()).max())
        assert (moved > 1e-2) if seen else (moved < 1e-6), (back, moved)


@pytest.mark.parametrize("device,dtype", EXACT)
@pytest.mark.parametrize("layer", ["retention", "lightning"])
@pytest.mark.parametrize("mode", ["prompt", "decode"])
def test_first_token_reaches_the_last_one_through_the_matrix_state(device, dtype, layer, mode):
    """300 tokens, decays of 0.999 and 1 - 2^-12: the first token's k v^T is still in the state at the end, so changing token 0
    moves the last logits (in the oracle by more than 1e-3, and equally here, in a prompt and through 40 decoded tokens); a fast
    head (decay 0.5) beside them forgets."""
    if layer == "retention":
        cfg = one_layer(ret(heads=3, dim=8, vdim=12, rot=8, base=100.0, decay=[0.999, 1.0 - 2.0 ** -12, 0.5]), vocab=32)
    else:
        cfg = one_layer(par(left_scale=0.0, r_heads=3, r_decay=[0.999, 1.0 - 2.0 ** -12, 0.5]), vocab=32)
    w = O.random_checkpoint(cfg, 9)
    seq = toks(300, 32, 5)
    m = build(cfg, w, device, dtype)

    def last(s):
        return (packed_logits(m, [s]) if mode == "prompt" else decoded_logits(m, s, 260))[-1:]
    base = O.forward(cfg, w, seq)[-1:]
    assert float(row_errs(last(seq), base).max()) < tol(dtype)
    s2 = list(seq)
    s2[0] = (s2[0] + 7) % 32
    want = O.forward(cfg, w, s2)[-1:]
    assert float(row_errs(want, base).max()) > 1e-3          # the oracle sees the first token
    assert float(row_errs(last(s2), want).max()) < tol(dtype)


@pytest.mark.parametrize("device,dtype", EXACT)
def test_rotation_layouts_and_far_positions(device, dtype):
    """Half and interleaved layouts over part of a head, positions up to 3000: the ops against the oracle's float64 rotation."""
    from realhf_b200.api.model import DecayConfig, RotaryConfig, WindowAttentionConfig
    from realhf_b200.ops import attention as A
    from realhf_b200.ops import recurrent as R
    g = torch.Generator().manual_seed(1)
    pos = torch.tensor([0, 1, 2, 63, 64, 500, 2999], dtype=torch.int32)
    H, d, dv, dims = 2, 12, 4, 8
    proj = torch.randn(7, 2 * H * d + 2 * H * dv, generator=g)
    dc = DecayConfig(n_heads=H, qk_dim=d, v_dim=dv, decay=[0.9, 0.8], rotary=RotaryConfig(dims=dims, base=1e4, interleaved=False), k_scale=0.25)
    u = R.decay_prepare(proj.to(device), dc, pos=pos.to(device)).double().cpu()
    q = O.rotate(proj[:, :H * d].double().view(7, H, d), pos, dims, 1e4, False).reshape(7, -1)
    k = O.rotate(proj[:, H * d:2 * H * d].double().view(7, H, d), pos, dims, 1e4, False).reshape(7, -1) * 0.25
    want = torch.cat([q, k, proj[:, 2 * H * d:2 * H * d + H * dv].double()], -1)
    assert float((u - want).abs().max()) < 2e-3 and float((u[:3] - want[:3]).abs().max()) < 2e-6      # fp32 angles at position 3000
    wa = WindowAttentionConfig(n_heads=3, n_kv_heads=1, qk_dim=d, v_dim=dv, scale=1.0, window=4, qkv_bias=False, value_norm=False, head_temp=False,
                               slope_base=None, sink=False, out_gate=False, rotary=RotaryConfig(dims=dims, base=300.0, interleaved=True))
    x = torch.randn(7, 4 * d + dv, generator=g)
    got = A.rotate_qk_(x.clone().to(device), wa, pos=pos.to(device)).double().cpu()
    want = O.rotate(x[:, :4 * d].double().view(7, 4, d), pos, dims, 300.0, True).reshape(7, -1)
    assert float((got[:, :4 * d] - want).abs().max()) < 2e-3 and float((got[:3, :4 * d] - want[:3]).abs().max()) < 2e-6
    assert torch.equal(got[:, 4 * d:], x[:, 4 * d:].double())                                       # the values are not touched
    # the step form reads the position from the slots' lengths
    lens = torch.tensor([5, 2999, 64], dtype=torch.int32, device=device)
    slots = torch.tensor([1, 2, 1, 0, 2, 2, 0], dtype=torch.int32, device=device)
    got2 = A.rotate_qk_(x.clone().to(device), wa, cache_lens=lens, slots=slots).double().cpu()
    want2 = O.rotate(x[:, :4 * d].double().view(7, 4, d), lens.cpu()[slots.cpu().long()], dims, 300.0, True).reshape(7, -1)
    assert float((got2[:, :4 * d] - want2).abs().max()) < 2e-3


@pytest.mark.parametrize("device,dtype", EXACT)
def test_routing_weight_scales_the_input_not_the_output(device, dtype):
    """One expert chosen of three, a router made decisive: with the expert's clamp active, expert(s h) differs from s expert(h); the
    framework follows the oracle (input scaling), and an oracle with the weight on the output is far away."""
    cfg = one_layer(ret(mlp=moe(experts=3, top=1, ff=8, limit=0.4, shared=None)))
    w = O.random_checkpoint(cfg, 4)
    seq = toks(12, cfg["vocab"], 8)
    want = O.forward(cfg, w, seq)
    orig = O.feed_forward

    def on_output(h, sd, f):
        scores = torch.sigmoid(h @ sd["router"].T)
        top = torch.topk(scores, 1, dim=-1)
        return torch.cat([top.values[t] * O.expert(h[t:t + 1], O.sub(sd, f"e{int(top.indices[t, 0])}."), f["expert"]["limit"]) for t in range(h.shape[0])])
    O.feed_forward = on_output
    try:
        other = O.forward(cfg, w, seq)
    finally:
        O.feed_forward = orig
    assert float(row_errs(other, want).max()) > 0.02
    m = build(cfg, w, device, dtype)
    assert float(row_errs(packed_logits(m, [seq]), want).max()) < tol(dtype)
    assert float(row_errs(decoded_logits(m, seq, 2), want).max()) < tol(dtype)


@pytest.mark.parametrize("device,dtype", EXACT)
def test_long_decoding_through_both_states_and_the_ring(device, dtype):
    """400 tokens, token by token from a 2-token prompt: the matrix states (decays up to 1 - 2^-10) and a ring of 7 rows that is
    overwritten 57 times, against the whole-sequence oracle."""
    cfg = model_cfg([par(window=7, r_decay=[0.97, 1.0 - 2.0 ** -10]), ret(decay=[0.9, 0.99, 1.0 - 2.0 ** -10])], None, vocab=32)
    w = O.random_checkpoint(cfg, 2)
    seq = toks(400, 32, 1)
    m = build(cfg, w, device, dtype)
    assert float(row_errs(decoded_logits(m, seq, 2), O.forward(cfg, w, seq)).max()) < tol(dtype)


# ------------------------------------------------------------------------------------------------ whole models


@pytest.mark.parametrize("device,dtype", ALL)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_packed_forward_matches_oracle_layer_by_layer(device, dtype, name):
    cfg = CONFIGS[name]()
    w = O.random_checkpoint(cfg, 7)
    m = build(cfg, w, device, dtype)
    seqs = [toks(n, cfg["vocab"], 30 + n) for n in (23, 1, 6)]
    trace = []
    got = packed_logits(m, seqs, trace=trace)
    off, errs = 0, []
    for s in seqs:
        wtr = []
        want = O.forward(cfg, w, s, layers_out=wtr)
        errs.append(row_errs(got[off:off + len(s)], want))
        assert len(trace) == len(wtr)
        if dtype == torch.float32:
            for a, b in zip(trace, wtr):
                assert float((a[off:off + len(s)].double().cpu() - b).abs().max()) < 1e-4 * max(1.0, float(b.abs().max()))
        off += len(s)
    assert model_ok(errs, dtype), float(torch.cat(errs).max())


@pytest.mark.parametrize("device,dtype", ALL)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_session_prefill_decode_batches_and_slot_reuse(device, dtype, name):
    """Unequal requests prefilled together, decoded together for 60+ steps while short ones end; new requests then take the freed
    slots (stale caches and states in them) and are checked from their first token on."""
    cfg = CONFIGS[name]()
    w = O.random_checkpoint(cfg, 8)
    m = build(cfg, w, device, dtype)
    V = cfg["vocab"]
    plan = {"a": (1, 64), "b": (2, 20), "c": (17, 70), "d": (9, 5)}          # prompt length, decoded tokens
    full = {r: toks(p + n, V, 40 + p) for r, (p, n) in plan.items()}
    want = {r: O.forward(cfg, w, s) for r, s in full.items()}
    sess = gen.StepSession(m, max_len=96, n_slots=4)
    errs = []
    h = sess.prefill([(r, full[r][:plan[r][0]]) for r in plan])
    off = 0
    for r in plan:
        p = plan[r][0]
        errs.append(row_errs(sess.logits(h[off:off + p]), want[r][:p]))
        off += p
    live = dict(plan)
    late = {}
    for k in range(70):
        batch = [r for r in live if k < live[r][1]]
        if not batch:
            break
        lg = sess.logits(sess.decode([(r, full[r][live[r][0] + k]) for r in batch]))
        errs += [row_errs(lg[j:j + 1], want[r][live[r][0] + k][None]) for j, r in enumerate(batch)]
        done = [r for r in batch if k + 1 == live[r][1]]
        if done:
            sess.release(done)
        if k == 25:                 # "b" and "d" have ended: two new requests reuse their slots while "a" and "c" go on
            late = {"e": (5, 30), "f": (1, 30)}
            for r, (p, n) in late.items():
                full[r] = toks(p + n, V, 70 + p)
                want[r] = O.forward(cfg, w, full[r])
            h = sess.prefill([(r, full[r][:late[r][0]]) for r in late])
            errs.append(row_errs(sess.logits(h[:5]), want["e"][:5]))
        for r in list(late):
            j = k - 25
            if k > 25 and j - 1 < late[r][1]:
                lg = sess.logits(sess.decode([(r, full[r][late[r][0] + j - 1])]))
                errs.append(row_errs(lg, want[r][late[r][0] + j - 1][None]))
    assert model_ok(errs, dtype), float(torch.cat(errs).max())


@pytest.mark.parametrize("device,dtype", EXACT)
def test_batched_equals_alone_and_prefill_equals_decoding(device, dtype):
    cfg = CONFIGS["mixed"]()
    w = O.random_checkpoint(cfg, 12)
    m = build(cfg, w, device, dtype)
    V = cfg["vocab"]
    seqs = [toks(n, V, 60 + n) for n in (30, 3, 11)]
    together = packed_logits(m, seqs)
    off = 0
    for s in seqs:
        alone = packed_logits(m, [s])
        assert float((together[off:off + len(s)] - alone).abs().max()) < 1e-4
        off += len(s)
    for cut in (1, 2, 7):
        assert float((decoded_logits(m, seqs[0], cut, max_len=40) - together[:30]).abs().max()) < 2e-4


@pytest.mark.parametrize("device,dtype", EXACT)
def test_session_grows_and_keeps_live_state(device, dtype):
    """More requests than slots: the state is re-allocated with twice the slots, the live requests' caches and matrix states move."""
    cfg = CONFIGS["mixed"]()
    w = O.random_checkpoint(cfg, 14)
    m = build(cfg, w, device, dtype)
    V = cfg["vocab"]
    full = {r: toks(12 + r, V, 80 + r) for r in range(5)}
    want = {r: O.forward(cfg, w, s) for r, s in full.items()}
    sess = gen.StepSession(m, max_len=32, n_slots=2)
    sess.prefill([(r, full[r][:6]) for r in (0, 1)])
    sess.decode([(0, full[0][6]), (1, full[1][6])])
    sess.prefill([(r, full[r][:7]) for r in (2, 3, 4)])
    errs = []
    for k in range(7, 12):
        lg = sess.logits(sess.decode([(r, full[r][k]) for r in range(5)]))
        errs += [row_errs(lg[r:r + 1], want[r][k][None]) for r in range(5)]
    assert model_ok(errs, dtype), float(torch.cat(errs).max())


@pytest.mark.parametrize("device,dtype", EXACT)
def test_greedy_generation_through_generate_and_inflight_batcher(device, dtype):
    cfg = CONFIGS["mixed"]()
    w = O.random_checkpoint(cfg, 6)
    m = build(cfg, w, device, dtype)
    V, n_new = cfg["vocab"], 10
    prompts = [toks(n, V, 50 + n) for n in (5, 1, 14)]
    want = [O.greedy(cfg, w, p, n_new) for p in prompts]
    g = GenerationHyperparameters(max_new_tokens=n_new, min_new_tokens=n_new, greedy=True, use_cuda_graph=(device == "cuda"))
    ids = torch.tensor([x for p in prompts for x in p], device=device)
    cu = torch.tensor([0] + [len(p) for p in prompts], device=device).cumsum(0).int()
    out, _ = gen.generate(m, ids, cu, g, eos_id=None, pad_id=0)
    assert out.tokens.tolist() == want
    ib = gen.InflightBatchingGenerator(m, g, eos_id=None, pad_id=0, n_slots=2, max_prompt_len=16)
    res = ib.generate([torch.tensor(p, device=device) for p in prompts])
    assert [r[0] for r in res] == want


def write_checkpoint(d, cfg, w):
    from safetensors.torch import save_file
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous().bfloat16() for k, v in w.items()}, os.path.join(d, "model.safetensors"))


def test_checkpoint_roundtrip_and_family_detection(tmp_path):
    for name in ("mixed", "odd"):
        cfg = CONFIGS[name]()
        w = O.random_checkpoint(cfg, 8)
        d = str(tmp_path / name)
        write_checkpoint(d, cfg, w)
        assert hf_io.family_of_path(d) == "buvesun"
        m = hf_io.from_hf("buvesun", d, dtype=torch.float32, device="cpu")
        fam = hf_io.family("buvesun")
        assert fam.config_to_dict(m.config) == cfg
        assert sum(p.numel() for p in w.values()) == m.config.n_params()
        back = fam.sd_to_hf(m.state_dict(), m.config)
        assert set(back) == set(w) and all(torch.equal(back[k].float(), w[k]) for k in w)
        seq = toks(20, cfg["vocab"], 3)
        assert float(row_errs(packed_logits(m.eval(), [seq]), O.forward(cfg, w, seq)).max()) < 2e-4


@pytest.mark.parametrize("device", ["cpu", pytest.param("cuda:0", marks=pytest.mark.gpu)])
def test_trace_replay_command(tmp_path, device):
    """`bin/trace_run` on a checkpoint directory: two requests prefilled in one step, decoded together, one ends early."""
    import numpy as np
    cfg = CONFIGS["mixed"]()
    w = O.random_checkpoint(cfg, 13)
    d = str(tmp_path / "ckpt")
    write_checkpoint(d, cfg, w)
    V = cfg["vocab"]
    a, b = toks(9, V, 1), toks(4, V, 2)
    steps = [dict(step=0, entries=[dict(id="a", tokens=a[:6], want=[0, 5]), dict(id="b", tokens=b[:2], want=[1])], end=[]),
             dict(step=1, entries=[dict(id="a", tokens=a[6:7], want=[]), dict(id="b", tokens=b[2:3], want=[0])], end=[]),
             dict(step=2, entries=[dict(id="a", tokens=a[7:8], want=[0]), dict(id="b", tokens=b[3:4], want=[0])], end=["b"]),
             dict(step=3, entries=[dict(id="a", tokens=a[8:9], want=[0])], end=["a"])]
    out = str(tmp_path / "out")
    exe = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "trace_run")
    r = subprocess.run([sys.executable, exe, "--model", d, "--dtype", "float32", "--out", out, "--max-tokens", "32", "--device", device],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=1500)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == [f"done {i}" for i in range(4)]
    wa, wb = O.forward(cfg, w, a), O.forward(cfg, w, b)
    want = {0: torch.stack([wa[0], wa[5], wb[1]]), 1: wb[2][None], 2: torch.stack([wa[7], wb[3]]), 3: wa[8][None]}
    for s, wl in want.items():
        got = torch.from_numpy(np.fromfile(os.path.join(out, f"{s}.f32"), dtype="<f4").reshape(-1, V))
        assert float(row_errs(got, wl).max()) < 2e-4


# ------------------------------------------------------------------------------------------------ kernels against plain torch


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,W", [(1, 16), (5, 100), (37, 2050), (300, 4096)])
def test_centred_norm_kernel_against_plain_torch(dtype, T, W):
    """LayerNorm without a bias, alone and fused with the scaled residual add of one or two branch outputs and the next norm."""
    from realhf_b200.ops import functional as OF
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(T + W)
    x = (torch.randn(T, W, generator=g) * 3 + 5).to(dev)               # a large mean: the variance must come from the deviations
    y, y2 = (torch.randn(T, W, generator=g).to(dtype).to(dev) for _ in range(2))
    ws = [(1 + 0.3 * torch.randn(W, generator=g)).to(dtype).to(dev) for _ in range(3)]

    def ln(v, w):
        v = v.double()
        d = v - v.mean(-1, keepdim=True)
        return d / torch.sqrt(d.pow(2).mean(-1, keepdim=True) + 1e-5) * w.double()
    tol_ = 1e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(OF.centred_norm(x, ws[0], 1e-5, dtype).double(), ln(x, ws[0]), atol=tol_, rtol=tol_)
    for two in (False, True):
        res = x.clone()
        out = OF.residual_add_centred_norm_(res, y, ws[0], 1e-5, ws[1], 0.6, y2 if two else None, 0.7, 1.3, ws[2], dtype)
        br = 0.7 * y.double() + (1.3 * y2.double() if two else 0.0)
        want = x.double() + 0.6 * ln(br, ws[0]) * ws[1].double()
        assert torch.allclose(res.double(), want, atol=1e-5, rtol=1e-5)
        assert torch.allclose(out.double(), ln(want, ws[2]), atol=tol_, rtol=tol_)
    res = x.clone()
    assert OF.residual_add_centred_norm_(res, y, ws[0], 1e-5) is None
    assert torch.allclose(res.double(), x.double() + ln(y, ws[0]), atol=1e-5, rtol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("H,d,dv", [(1, 8, 12), (3, 33, 7), (2, 64, 64), (2, 128, 128), (1, 130, 40), (1, 260, 20)])
def test_decay_scan_and_output_kernels_against_plain_torch(H, d, dv):
    """The recurrence from zero over packed sequences (one empty), then continued token by token from the slots; the per-head and
    the full-width output norms with both gates."""
    from realhf_b200.api.model import DecayConfig
    from realhf_b200.ops import recurrent as R
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(H * 1000 + d)
    lens = [1, 0, 19, 2, 40]
    T = sum(lens)
    dc = DecayConfig(n_heads=H, qk_dim=d, v_dim=dv, decay=[0.999, 0.9, 0.5][:H])
    u = torch.randn(T + 3, 2 * H * d + H * dv, generator=g) * 0.5
    cu = torch.tensor([0] + lens).cumsum(0).int()
    slots = torch.tensor([3, 0, 4, 1, 2], dtype=torch.int32)
    state = torch.randn(6, H, d, dv, generator=g)                    # stale contents: the prompt form starts from zero
    want_o, want_S = [], {}
    for n, (a, b) in enumerate(zip(cu[:-1].tolist(), cu[1:].tolist())):
        q, k, v = u[a:b, :H * d].double().view(-1, H, d), u[a:b, H * d:2 * H * d].double().view(-1, H, d), u[a:b, 2 * H * d:].double().view(-1, H, dv)
        o, S = O.decayed_state_scan(q, k, v, dc.decay)
        want_o.append(o)
        want_S[int(slots[n])] = S
    st = state.clone().to(dev)
    o = R.decay_scan(u[:T].to(dev), dc, cu.to(dev), st, slots.to(dev))
    assert torch.allclose(o.double().cpu(), torch.cat(want_o), atol=1e-4, rtol=1e-4)
    for s, S in want_S.items():
        if s != 0:                                                    # (slot 0 belongs to the empty sequence: untouched)
            assert torch.allclose(st[s].double().cpu(), S, atol=1e-4, rtol=1e-4)
    assert torch.equal(st[0].cpu(), state[0]) and torch.equal(st[5].cpu(), state[5])
    rows = torch.tensor([4, 2, 3], dtype=torch.int32)                 # one more token for three of the sequences
    us = u[T:T + 3]
    o2 = R.decay_step(us.to(dev), dc, st, rows.to(dev))
    for j, s in enumerate(rows.tolist()):
        q, k, v = us[j:j + 1, :H * d].double().view(1, H, d), us[j:j + 1, H * d:2 * H * d].double().view(1, H, d), us[j:j + 1, 2 * H * d:].double().view(1, H, dv)
        wo, wS = O.decayed_state_scan(q, k, v, dc.decay, want_S[s])
        assert torch.allclose(o2[j].double().cpu(), wo[0], atol=1e-4, rtol=1e-4)
        assert torch.allclose(st[s].double().cpu(), wS, atol=1e-4, rtol=1e-4)
    gate = torch.randn(T, H * dv + 5, generator=g)
    w = 1 + 0.2 * torch.randn(H * dv, generator=g)
    for out_norm, gk in (("head", "silu"), ("full", "sigmoid")):
        dc2 = DecayConfig(n_heads=H, qk_dim=d, v_dim=dv, decay=dc.decay, out_norm=out_norm, gate=gk)
        got = R.decay_out(o, dc2, w.to(dev), gate.to(dev)[:, 2:2 + H * dv], 1e-5, torch.float32).double().cpu()
        od = torch.cat(want_o)
        gd = gate[:, 2:2 + H * dv].double()
        n_ = O.rms(od, 1e-5).reshape(T, -1) if out_norm == "head" else O.rms(od.reshape(T, -1), 1e-5) * w.double()
        want = n_ * (gd * torch.sigmoid(gd) if gk == "silu" else torch.sigmoid(gd))
        assert torch.allclose(got, want, atol=1e-4, rtol=1e-4)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,K,R,k", [(1, 64, 1, 1), (5, 100, 9, 2), (300, 2048, 33, 3)])
def test_sigmoid_router_scaled_gather_and_unit_combine(dtype, T, K, R, k):
    from realhf_b200.ops import lib
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(T * 131 + R)
    x = torch.randn(T, K, generator=g).to(dtype).to(dev)
    w = (torch.randn(R, K, generator=g) * K ** -0.5 * 3).to(dtype).to(dev)
    probs, idx, _ = lib().softmax_router(x, w, None, None, k, False, True)
    s = torch.sigmoid(x.double() @ w.double().T)
    assert torch.allclose(s.gather(1, idx), torch.topk(s, k, -1).values, atol=1e-5, rtol=0)
    assert torch.allclose(probs.double(), s.gather(1, idx), atol=1e-5, rtol=1e-5)
    if T * k <= 1024:
        row, _ = lib().moe_dispatch(idx, R, R)
        xs = lib().moe_gather(x, row, k, probs)
        want = (x.double().repeat_interleave(k, 0) * probs.double().reshape(-1, 1))
        assert torch.allclose(xs[row].double(), want, atol=1e-6 if dtype == torch.float32 else 2e-2, rtol=1e-2)
        y = torch.randn(T * k, K, generator=g).to(dtype).to(dev)
        ysh = torch.randn(T, K, generator=g).to(dtype).to(dev)
        out = torch.empty(T, K, dtype=torch.float32, device=dev)
        lib().moe_combine(y, x, row, probs, idx, ysh, None, out, R, True)
        assert torch.allclose(out.double(), y.double()[row].view(T, k, K).sum(1) + ysh.double(), atol=1e-5, rtol=1e-5)
