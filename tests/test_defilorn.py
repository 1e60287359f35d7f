"""Defilorn (heterogeneous stack: differential window attention with query / key norms, latent attention with a rotated shared key
part, YaRN-rescaled frequencies, a sink and an output gate, the matrix-memory LSTM, gated feed-forwards, a mixture of experts with
identity and shared experts, a looped range of blocks with the embedding added back) against the plain float64 implementation in
`defilorn_oracle.py`.

Every test body runs on the CPU (the op layer's PyTorch references, part of the default suite) and, marked `gpu`, on CUDA (the
sm_100a kernels) in fp32 and bf16.  Configurations are small and made here; none is a released model's."""

import copy
import json
import math
import os
import subprocess
import sys

import pytest
import torch

import defilorn_oracle as O
from realhf_b200.api.model import GenerationHyperparameters
from realhf_b200.models import generation as gen
from realhf_b200.models import hf_io
from realhf_b200.models.real_model import ReaLModel

CPU = pytest.param("cpu", torch.float32, id="cpu-f32")
GPU32 = pytest.param("cuda", torch.float32, id="cuda-f32", marks=pytest.mark.gpu)
GPU16 = pytest.param("cuda", torch.bfloat16, id="cuda-bf16", marks=pytest.mark.gpu)
ALL = [CPU, GPU32, GPU16]
EXACT = [CPU, GPU32]
F64 = torch.float64


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
    fam = hf_io.family("defilorn")
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


# ------------------------------------------------------------------------------------------------ configurations

def lat(heads=2, dim=8, rot=4, vdim=12, kv_rank=16, q_rank=24, scaling=True, base=10000.0, mlp=None, scale=None):
    r = dict(base=base, dims=rot)
    if scaling:
        r["scaling"] = dict(factor=4.0, fast=32.0, original=16, slow=1.0)
    return dict(type="latent_attention", mlp=mlp,
                mixer=dict(dim=dim, heads=heads, kv_rank=kv_rank, q_rank=q_rank, rot=r, rot_dim=rot, scale=scale or (dim + rot) ** -0.5, vdim=vdim))


def att(heads=4, kv_heads=2, dim=8, vdim=12, window=5, diff=0.5, mlp=None, scale=None):
    m = dict(diff=diff, dim=dim, heads=heads, kv_heads=kv_heads, scale=scale or dim ** -0.5, vdim=vdim)
    if window is not None:
        m["mask"] = dict(size=window)
    return dict(type="attention", mixer=m, mlp=mlp)


def mls(heads=2, dim=8, vdim=12, cap=15.0, mlp=None):
    return dict(type="mlstm", mixer=dict(dim=dim, gate_cap=cap, heads=heads, vdim=vdim), mlp=mlp)


def dense(ff=48):
    return dict(ff=ff, kind="dense")


def moe(experts=4, identity=1, top=2, ff=16, shared=24):
    f = dict(expert=dict(ff=ff), kind="moe", router=dict(experts=experts, identity=identity, top=top))
    if shared:
        f["shared"] = dict(ff=shared)
    return f


def model_cfg(layers, loop=None, width=32, vocab=96, eps=1e-5):
    c = dict(architecture="Defilorn", layers=layers, norm=dict(eps=eps), vocab=vocab, width=width)
    if loop:
        c["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
    return c


CONFIGS = {
    # all three mixers, both feed-forwards, a loop over the first two layers
    "mixed": lambda: model_cfg([att(mlp=moe()), mls(mlp=dense()), lat(mlp=moe(experts=3, identity=2, top=3, shared=None)), mls(mlp=None)], (0, 2, 2)),
    # every count that can be 1 is 1: one head, one expert, one pass, window 1, no identity expert
    "ones": lambda: model_cfg([att(heads=1, kv_heads=1, window=1, mlp=moe(experts=1, identity=0, top=1, shared=8)), mls(heads=1, mlp=None),
                               lat(heads=1, scaling=False, mlp=dense(8))], (1, 2, 1), width=16, vocab=40),
    # sizes that are not multiples of four, heads = kv heads, no window, a loop over the whole stack run three times
    "odd": lambda: model_cfg([lat(heads=3, dim=10, rot=6, vdim=7, kv_rank=9, q_rank=11, mlp=dense(20)),
                              att(heads=3, kv_heads=3, dim=6, vdim=10, window=None, diff=0.3, mlp=None),
                              mls(heads=3, dim=33, vdim=5, cap=4.0, mlp=moe(experts=5, identity=3, top=4, ff=12, shared=None))], (0, 3, 3), width=24, vocab=50),
    # no loop; wide heads (the matrix state split over several lanes), a window longer than the prompts
    "wide": lambda: model_cfg([mls(heads=1, dim=72, vdim=40, mlp=dense(32)), att(heads=6, kv_heads=2, dim=16, vdim=24, window=200, diff=0.7, mlp=dense(32)),
                               lat(heads=4, dim=16, rot=16, vdim=16, kv_rank=24, q_rank=8, base=500.0, mlp=None)], None, width=40, vocab=64),
}


# ------------------------------------------------------------------------------------------------ each mechanism alone (one-layer models)


def one_layer(layer, width=32, vocab=64):
    return model_cfg([layer], None, width=width, vocab=vocab)


MECHANISMS = {
    "mlstm-small": lambda: one_layer(mls(heads=2, dim=8, vdim=12)),
    "mlstm-33x7": lambda: one_layer(mls(heads=3, dim=33, vdim=7, cap=3.0)),
    "mlstm-130x40": lambda: one_layer(mls(heads=1, dim=130, vdim=40)),
    "mlstm-64x64": lambda: one_layer(mls(heads=2, dim=64, vdim=64)),
    "diff-window5": lambda: one_layer(att(heads=4, kv_heads=2, dim=8, vdim=12, window=5)),
    "diff-window1": lambda: one_layer(att(heads=2, kv_heads=1, dim=20, vdim=24, window=1, diff=0.2)),
    "diff-nowindow": lambda: one_layer(att(heads=6, kv_heads=2, dim=16, vdim=40, window=None, diff=0.8)),
    "diff-odd": lambda: one_layer(att(heads=3, kv_heads=3, dim=7, vdim=9, window=33)),
    "latent-small": lambda: one_layer(lat()),
    "latent-odd": lambda: one_layer(lat(heads=3, dim=10, rot=6, vdim=7, kv_rank=9, q_rank=11, scaling=False)),
    "latent-64": lambda: one_layer(lat(heads=2, dim=32, rot=32, vdim=64, kv_rank=40, q_rank=32, base=1e6)),
    "dense-ff": lambda: one_layer(mls(mlp=dense(40))),
    "moe-ff": lambda: one_layer(mls(mlp=moe(experts=6, identity=2, top=3, ff=8, shared=16))),
    "moe-top1-noshared": lambda: one_layer(mls(mlp=moe(experts=3, identity=0, top=1, ff=8, shared=None))),
    "moe-all-chosen": lambda: one_layer(mls(mlp=moe(experts=2, identity=2, top=4, ff=8, shared=8))),
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
    want = [O.forward(cfg, w, s)[0] for s in full]
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
    "diff-64-window150": lambda: one_layer(att(heads=4, kv_heads=2, dim=64, vdim=64, window=150), width=64),
    "diff-128-window128": lambda: one_layer(att(heads=2, kv_heads=2, dim=128, vdim=128, window=128, diff=0.3), width=64),
    "diff-64-nowindow-rep4": lambda: one_layer(att(heads=4, kv_heads=1, dim=64, vdim=64, window=None), width=64),
    "latent-32+32-64": lambda: one_layer(lat(heads=3, dim=32, rot=32, vdim=64, kv_rank=48, q_rank=40, base=1e4), width=64),
    "latent-64+64-128": lambda: one_layer(lat(heads=2, dim=64, rot=64, vdim=128, kv_rank=72, q_rank=64, base=1e6), width=64),
}


@pytest.mark.parametrize("device,dtype", [CPU, GPU32, GPU16])
@pytest.mark.parametrize("name", list(TC_SHAPES))
def test_head_shapes_of_the_tensor_core_and_streaming_kernels(device, dtype, name):
    """Head sizes 64 / 128 with equal query and value size: in 16 bit the prompts run the tcgen05 kernel (two maps sharing a value
    head, or the sink) and decoding the streaming kernel; sequences of 1, 130 and 300 tokens cross the 128-key tiles and the window."""
    cfg = TC_SHAPES[name]()
    w = O.random_checkpoint(cfg, 21)
    m = build(cfg, w, device, dtype)
    V = cfg["vocab"]
    seqs = [toks(n, V, 20 + n) for n in (1, 130, 300)]
    more = 6
    full = [s + toks(more, V, 90 + len(s)) for s in seqs]
    want = [O.forward(cfg, w, s)[0] for s in full]
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


def _boost(w, name, rows, factor):
    w[name] = w[name].clone()
    w[name][rows] *= factor


@pytest.mark.parametrize("device,dtype", EXACT)
@pytest.mark.parametrize("mode", ["prompt", "decode"])
def test_window_edge_one_token_off_changes_the_output(device, dtype, mode):
    """Differential attention with a window of 6: scores are made sharp (large scale), so every query puts nearly all its weight on
    one key; a window that is one token too long or too short picks another key for some query and the logits move by far more
    than the tolerance.  Prompt and decoding forms are both held against the oracle, and the oracle itself is shown to be
    sensitive: its output with window 5 or 7 differs."""
    cfg = one_layer(att(heads=2, kv_heads=1, dim=8, vdim=12, window=6, scale=6.0))
    w = O.random_checkpoint(cfg, 5)
    seq = toks(40, cfg["vocab"], 77)
    want = O.forward(cfg, w, seq)[0]
    for other in (5, 7):
        c2 = copy.deepcopy(cfg)
        c2["layers"][0]["mixer"]["mask"]["size"] = other
        assert float(row_errs(O.forward(c2, w, seq)[0][8:], want[8:]).max()) > 0.05
    m = build(cfg, w, device, dtype)
    if mode == "prompt":
        got = packed_logits(m, [seq])
    else:
        sess = gen.StepSession(m, max_len=48, n_slots=2)
        rows = [sess.logits(sess.prefill([("a", seq[:3])]))]
        rows += [sess.logits(sess.decode([("a", t)])) for t in seq[3:]]
        got = torch.cat(rows)
    assert float(row_errs(got, want).max()) < tol(dtype)


@pytest.mark.parametrize("device,dtype", EXACT)
@pytest.mark.parametrize("mode", ["prompt", "decode"])
def test_far_key_and_first_token_reach_the_last_query_through_latent_attention(device, dtype, mode):
    """Latent attention over 300 tokens with nearly flat weights (a small score scale, the sink far below): every key carries about
    1 / 300 of the output, so changing token 0 or a token 250 back moves the last logits by a few thousandths, far above the
    tolerance; in the oracle and equally here, also through decoding with the cache."""
    cfg = one_layer(lat(heads=2, dim=8, rot=8, vdim=12, kv_rank=16, q_rank=16, scale=0.02, base=100.0), vocab=32)
    w = O.random_checkpoint(cfg, 9)
    w["l0.mix.sink"] = torch.full((2,), -30.0)
    w["l0.mix.uv"] = w["l0.mix.uv"] * 4
    seq = toks(300, 32, 5)
    m = build(cfg, w, device, dtype)

    def last(s):
        if mode == "prompt":
            return packed_logits(m, [s])[-1:]
        sess = gen.StepSession(m, max_len=320, n_slots=1)
        sess.prefill([("a", s[:260])])
        for t in s[260:-1]:
            sess.decode([("a", t)])
        return sess.logits(sess.decode([("a", s[-1])]))
    base = O.forward(cfg, w, seq)[0][-1:]
    assert float(row_errs(last(seq), base).max()) < tol(dtype)
    for where in (0, 49):
        s2 = list(seq)
        s2[where] = (s2[where] + 7) % 32
        want = O.forward(cfg, w, s2)[0][-1:]
        assert float(row_errs(want, base).max()) > 1e-3          # the oracle sees the far token
        assert float(row_errs(last(s2), want).max()) < tol(dtype)


@pytest.mark.parametrize("device,dtype", EXACT)
def test_sink_takes_weight_once_and_only_in_the_denominator(device, dtype):
    """One token: the only key has weight 1 / (1 + exp(sink - score)).  A large sink silences the mixer, a very negative one leaves
    plain softmax; both against the oracle."""
    cfg = one_layer(lat(heads=2))
    for sink in (8.0, -30.0, 0.0):
        w = O.random_checkpoint(cfg, 3)
        w["l0.mix.sink"] = torch.full((2,), sink)
        m = build(cfg, w, device, dtype)
        seq = toks(6, cfg["vocab"], 2)
        want, tr = O.forward(cfg, w, seq)
        got_tr = []
        got = packed_logits(m, [seq], trace=got_tr)
        assert float(row_errs(got, want).max()) < tol(dtype)
        x0 = w["embed"].double()[torch.tensor(seq)]
        moved = float((tr[0] - x0)[0].abs().max())              # what the mixer added at the first token
        assert (moved < 2e-3) if sink == 8.0 else (moved > 1e-2)


@pytest.mark.parametrize("device,dtype", EXACT)
def test_rotation_far_positions_and_rescaled_frequencies(device, dtype):
    """Positions up to 2000 with YaRN-rescaled and plain frequencies: the rotated key part against the oracle's float64 rotation."""
    from realhf_b200.api.model import LatentAttentionConfig, RotaryConfig
    from realhf_b200.ops import attention as A
    for scaling in (None, dict(factor=8.0, fast=32.0, original=64, slow=1.0)):
        rot = dict(base=10000.0, dims=12)
        if scaling:
            rot["scaling"] = scaling
        rc = RotaryConfig(dims=12, base=10000.0, factor=scaling["factor"] if scaling else None, original=scaling["original"] if scaling else 0)
        a = LatentAttentionConfig(n_heads=1, qk_dim=4, v_dim=4, kv_rank=8, scale=1.0, rot_dim=12, rotary=rc, q_rank=None)
        f_want, mult = O.yarn_frequencies(rot)
        f_got, mult_got = rc.frequencies()
        assert torch.allclose(torch.tensor(f_got, dtype=F64), f_want, rtol=1e-12) and abs(mult - mult_got) < 1e-12
        g = torch.Generator().manual_seed(1)
        pos = torch.tensor([0, 1, 2, 63, 64, 500, 1999], dtype=torch.int32)
        proj = torch.randn(7, 8 + 12, generator=g)
        wc = torch.ones(8)
        _, latent = A.latent_rope_prepare(proj.to(device), a, None, wc.to(device), 1e-5, pos.to(device), None)
        want = O.rotate(proj[:, 8:].double(), pos, rot)
        assert float((latent[:, 8:].double().cpu() - want).abs().max()) < 2e-3          # fp32 angles at position 2000
        assert float((latent[:3, 8:].double().cpu() - want[:3]).abs().max()) < 2e-6
        c = proj[:, :8].double()
        assert float((latent[:, :8].double().cpu() - O.rms(c, 1e-5)).abs().max()) < 1e-5


@pytest.mark.parametrize("device,dtype", EXACT)
def test_router_correction_decides_the_choice_but_not_the_weight(device, dtype):
    """A correction that lifts the weakest expert into the chosen set: the choice follows score + correction, the weight is the bare
    score, and an identity expert passes its input through."""
    cfg = one_layer(mls(mlp=moe(experts=3, identity=1, top=1, ff=8, shared=None)))
    w = O.random_checkpoint(cfg, 4)
    for e in range(4):
        w["l0.mlp.correction"] = torch.zeros(4)
        w["l0.mlp.correction"][e] = 5.0
        m = build(cfg, w, device, dtype)
        seq = toks(12, cfg["vocab"], 8)
        assert float(row_errs(packed_logits(m, [seq]), O.forward(cfg, w, seq)[0]).max()) < tol(dtype)


@pytest.mark.parametrize("device,dtype", EXACT)
def test_mlstm_long_decoding_keeps_the_state_stable(device, dtype):
    """400 tokens through the recurrent state (forget gates near 1, input gates large: the running maximum grows and the stored
    state stays bounded), token by token from a 2-token prompt, against the whole-sequence oracle."""
    cfg = one_layer(mls(heads=2, dim=12, vdim=8, cap=6.0), vocab=32)
    w = O.random_checkpoint(cfg, 2)
    w["l0.mix.f.b"] = torch.full((2,), 6.0)
    w["l0.mix.i.b"] = torch.full((2,), 3.0)
    seq = toks(400, 32, 1)
    want = O.forward(cfg, w, seq)[0]
    m = build(cfg, w, device, dtype)
    sess = gen.StepSession(m, max_len=400, n_slots=1)
    rows = [sess.logits(sess.prefill([("a", seq[:2])]))]
    rows += [sess.logits(sess.decode([("a", t)])) for t in seq[2:]]
    assert float(row_errs(torch.cat(rows), want).max()) < tol(dtype)
    assert float(sess.state.k[0].abs().max()) < 1e4


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
        want, wtr = O.forward(cfg, w, s)
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
    want = {r: O.forward(cfg, w, s)[0] for r, s in full.items()}
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
                want[r] = O.forward(cfg, w, full[r])[0]
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
        sess = gen.StepSession(m, max_len=40, n_slots=2)
        rows = [sess.logits(sess.prefill([("x", seqs[0][:cut])]))]
        rows += [sess.logits(sess.decode([("x", t)])) for t in seqs[0][cut:]]
        assert float((torch.cat(rows) - together[:30]).abs().max()) < 2e-4


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
        assert hf_io.family_of_path(d) == "defilorn"
        m = hf_io.from_hf("defilorn", d, dtype=torch.float32, device="cpu")
        fam = hf_io.family("defilorn")
        assert fam.config_to_dict(m.config) == cfg
        assert sum(p.numel() for p in w.values()) == m.config.n_params()          # (the fused tensors' padding rows not counted)
        back = fam.sd_to_hf(m.state_dict(), m.config)
        assert set(back) == set(w) and all(torch.equal(back[k].float(), w[k]) for k in w)
        seq = toks(20, cfg["vocab"], 3)
        assert float(row_errs(packed_logits(m.eval(), [seq]), O.forward(cfg, w, seq)[0]).max()) < 2e-4


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
    wa, wb = O.forward(cfg, w, a)[0], O.forward(cfg, w, b)[0]
    want = {0: torch.stack([wa[0], wa[5], wb[1]]), 1: wb[2][None], 2: torch.stack([wa[7], wb[3]]), 3: wa[8][None]}
    for s, wl in want.items():
        got = torch.from_numpy(np.fromfile(os.path.join(out, f"{s}.f32"), dtype="<f4").reshape(-1, V))
        assert float(row_errs(got, wl).max()) < 2e-4


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,K,R,k,with_gate", [(1, 64, 1, 1, False), (5, 100, 9, 2, True), (37, 256, 64, 8, True), (300, 2048, 33, 3, False)])
def test_router_and_combine_kernels_against_plain_torch(dtype, T, K, R, k, with_gate):
    """Routing by the softmax over all outputs (correction for the choice only) and the weighted sum of expert rows, identity
    rows and the gated shared output, each one kernel, against the same arithmetic in fp64."""
    from realhf_b200.ops import lib
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(T * 131 + R)
    x = torch.randn(T, K, generator=g).to(dtype).to(dev)
    w = (torch.randn(R, K, generator=g) * K ** -0.5 * 3).to(dtype).to(dev)
    corr = (torch.randn(R, generator=g) * 0.3).to(dtype).to(dev)
    u = torch.randn(1, K, generator=g).mul(K ** -0.5).to(dtype).to(dev) if with_gate else None
    for c, renorm in ((corr, False), (None, True)):
        probs, idx, gate = lib().softmax_router(x, w, c, u.view(-1) if with_gate else None, k, renorm)
        s = torch.softmax(x.double() @ w.double().T, -1)
        choice = s + (c.double() if c is not None else 0.0)
        want_idx = torch.topk(choice, k, -1).indices
        # a close call between two choice scores may go either way: compare the chosen scores, and the sets where they are apart
        got_choice = choice.gather(1, idx)
        assert torch.allclose(got_choice, choice.gather(1, want_idx), atol=1e-5, rtol=0)
        want_p = s.gather(1, idx)
        if renorm:
            want_p = want_p / want_p.sum(-1, keepdim=True)
        assert torch.allclose(probs.double(), want_p, atol=1e-5, rtol=1e-5)
        if with_gate:
            assert torch.allclose(gate.double(), torch.sigmoid(x.double() @ u.double().view(-1)), atol=1e-5)
    # combination: E real experts, outputs >= E are identity experts
    H, E = K, max(R - 2, 1)
    order = torch.argsort(idx.reshape(-1), stable=True)
    back = torch.empty_like(order).scatter_(0, order, torch.arange(order.numel(), device=dev))
    y = torch.randn(T * k, H, generator=g).to(dtype).to(dev)
    ysh = torch.randn(T, H, generator=g).to(dtype).to(dev) if with_gate else None
    if T * k <= 1024:       # the counting kernel gives the same places as the stable sort, and the offsets of the real experts
        row, offsets = lib().moe_dispatch(idx, E, R)
        assert torch.equal(row, back)
        counts = torch.bincount(idx.reshape(-1), minlength=R)[:E]
        assert offsets.tolist() == [0] + counts.cumsum(0).tolist()
        xs = lib().moe_gather(x, row, k)
        assert torch.equal(xs[row], x.repeat_interleave(k, 0))
    for out_dtype in (torch.float32, dtype):
        out = torch.empty(T, H, dtype=out_dtype, device=dev)
        lib().moe_combine(y, x, back, probs, idx, ysh, gate if with_gate else None, out, E)
        rows = y.double()[back].view(T, k, H)
        rows = torch.where((idx >= E).unsqueeze(-1), x.double().unsqueeze(1), rows)
        want = (rows * probs.double().unsqueeze(-1)).sum(1)
        if with_gate:
            want = want + ysh.double() * gate.double().unsqueeze(-1)
        tol_ = 1e-5 if out_dtype == torch.float32 else 2e-2
        assert torch.allclose(out.double(), want, atol=tol_, rtol=tol_)
