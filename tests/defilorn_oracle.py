"""Plain, slow implementation of the Defilorn design in float64, one function per mechanism, on the checkpoint's own tensor names.

It shares no code with the package: whole sequences, dense score matrices, token-by-token recurrences.  `forward(cfg, sd, tokens)`
returns the logits of every position and the residual stream after every layer run.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

F64 = torch.float64


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def lin(w: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    return x @ w.to(F64).T


def yarn_frequencies(rot: dict) -> Tuple[torch.Tensor, float]:
    """Per-pair frequencies and the factor on cos / sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def dim_of(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, pos: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [L, ..., dims]: pairs (2i, 2i + 1) of the last axis turn by pos * f_i."""
    f, mult = yarn_frequencies(rot)
    ang = pos.to(F64)[:, None] * f[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [f.numel()]
    cos, sin = (torch.cos(ang) * mult).view(shape), (torch.sin(ang) * mult).view(shape)
    u, v = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = u * cos - v * sin
    out[..., 1::2] = v * cos + u * sin
    return out


def latent_attention(m: dict, P: Dict[str, torch.Tensor], h: torch.Tensor, eps: float) -> torch.Tensor:
    L = h.shape[0]
    H, d, r, dv, kr = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    pos = torch.arange(L)
    cq = rms(lin(P["dq"], h), eps) * P["dq.norm"].to(F64)
    q = lin(P["uq"], cq).view(L, H, d + r)
    ckr = lin(P["dkv"], h)
    c = rms(ckr[:, :kr], eps) * P["dkv.norm"].to(F64)
    k_rot = rotate(ckr[:, kr:], pos, m["rot"])                      # [L, r], one for all heads
    q_rot = rotate(q[..., d:], pos, m["rot"])
    k_n = lin(P["uk"], c).view(L, H, d)
    v = lin(P["uv"], c).view(L, H, dv)
    s = (torch.einsum("ihd,jhd->hij", q[..., :d], k_n) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * float(m["scale"])
    i, j = pos[:, None], pos[None, :]
    s = s.masked_fill(~(j <= i)[None], float("-inf"))
    sink = P["sink"].to(F64).view(H, 1, 1)
    mx = torch.maximum(s.max(-1, keepdim=True).values, sink)
    e = torch.exp(s - mx)
    w = e / (e.sum(-1, keepdim=True) + torch.exp(sink - mx))
    o = torch.einsum("hij,jhd->ihd", w, v).reshape(L, H * dv)
    return lin(P["o"], o * torch.sigmoid(lin(P["g"], h)))


def diff_attention(m: dict, P: Dict[str, torch.Tensor], h: torch.Tensor, eps: float) -> torch.Tensor:
    L = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    diff = float(m["diff"])
    q = rms(lin(P["q"], h).view(L, H, 2, d), eps) * P["q.norm"].to(F64)
    k = rms(lin(P["k"], h).view(L, G, 2, d), eps) * P["k.norm"].to(F64)
    v = lin(P["v"], h).view(L, G, dv)
    pos = torch.arange(L)
    i, j = pos[:, None], pos[None, :]
    ok = (j <= i)
    if m.get("mask"):
        ok = ok & (i - j < int(m["mask"]["size"]))
    lam = math.exp(float((P["lq1"].to(F64) * P["lk1"].to(F64)).sum())) - math.exp(float((P["lq2"].to(F64) * P["lk2"].to(F64)).sum())) + diff
    out = torch.empty(L, H, dv, dtype=F64)
    for hh in range(H):
        g = hh // (H // G)
        a = []
        for mp in range(2):
            s = (q[:, hh, mp] @ k[:, g, mp].T) * float(m["scale"])
            a.append(torch.softmax(s.masked_fill(~ok, float("-inf")), -1) @ v[:, g])
        out[:, hh] = rms(a[0] - lam * a[1], eps) * (1.0 - diff)
    return lin(P["o"], out.reshape(L, H * dv))


def mlstm(m: dict, P: Dict[str, torch.Tensor], h: torch.Tensor, eps: float) -> torch.Tensor:
    L = h.shape[0]
    H, d, dv, cap = int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["gate_cap"])
    q = lin(P["q"], h).view(L, H, d) * d ** -0.5
    k = lin(P["k"], h).view(L, H, d)
    v = lin(P["v"], h).view(L, H, dv)
    ig = cap * torch.tanh((lin(P["i"], h) + P["i.b"].to(F64)) / cap)
    fg = torch.nn.functional.logsigmoid(cap * torch.tanh((lin(P["f"], h) + P["f.b"].to(F64)) / cap))
    out = torch.empty(L, H, dv, dtype=F64)
    for hh in range(H):
        S = torch.zeros(d, dv, dtype=F64)
        n = torch.zeros(d, dtype=F64)
        mm = 0.0
        for t in range(L):
            i_t, f_t = float(ig[t, hh]), float(fg[t, hh])
            m_new = max(f_t + mm, i_t)
            S = math.exp(f_t + mm - m_new) * S + math.exp(i_t - m_new) * torch.outer(k[t, hh], v[t, hh])
            n = math.exp(f_t + mm - m_new) * n + math.exp(i_t - m_new) * k[t, hh]
            mm = m_new
            den = max(abs(float(n @ q[t, hh])), math.exp(-mm)) + 1e-6
            out[t, hh] = (S.T @ q[t, hh]) / den
    o = rms(out, eps).reshape(L, H * dv) * P["norm"].to(F64) * torch.sigmoid(lin(P["g"], h))
    return lin(P["o"], o)


def glu(P: Dict[str, torch.Tensor], prefix: str, h: torch.Tensor, act) -> torch.Tensor:
    return lin(P[prefix + "down"], act(lin(P[prefix + "gate"], h)) * lin(P[prefix + "up"], h))


def moe(f: dict, P: Dict[str, torch.Tensor], h: torch.Tensor) -> torch.Tensor:
    E, ident, top = int(f["router"]["experts"]), int(f["router"].get("identity", 0)), int(f["router"]["top"])
    s = torch.softmax(lin(P["router"], h), -1)                       # [L, E + ident]
    choice = s + (P["correction"].to(F64) if "correction" in P else 0.0)
    idx = torch.topk(choice, top, dim=-1).indices
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in idx[t].tolist():
            y = h[t] if e >= E else glu(P, f"e{e}.", h[t:t + 1], silu)[0]
            out[t] += s[t, e] * y
    if f.get("shared"):
        out = out + glu(P, "shared.", h, silu) * torch.sigmoid(lin(P["shared.sg"], h))
    return out


def sub(sd: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in sd.items() if k.startswith(prefix)}


def layer_runs(cfg: dict) -> List[Tuple[int, bool]]:
    """(layer, this run opens a pass after the first) in execution order."""
    n, lp = len(cfg["layers"]), cfg.get("loop")
    if not lp:
        return [(i, False) for i in range(n)]
    runs = [(i, False) for i in range(lp["start"])]
    for p in range(lp["times"]):
        runs += [(i, p > 0 and i == lp["start"]) for i in range(lp["start"], lp["stop"])]
    return runs + [(i, False) for i in range(lp["stop"], n)]


def forward(cfg: dict, sd: Dict[str, torch.Tensor], tokens: List[int]) -> Tuple[torch.Tensor, List[torch.Tensor]]:
    eps = float(cfg["norm"]["eps"])
    x0 = sd["embed"].to(F64)[torch.tensor(tokens)]
    x = x0.clone()
    trace = []
    for i, opens in layer_runs(cfg):
        lay = cfg["layers"][i]
        if opens:
            x = x + x0
        h = rms(x, eps) * (1.0 + sd[f"l{i}.norm1"].to(F64))
        P = sub(sd, f"l{i}.mix.")
        fn = {"latent_attention": latent_attention, "attention": diff_attention, "mlstm": mlstm}[lay["type"]]
        x = x + fn(lay["mixer"], P, h, eps)
        f = lay.get("mlp")
        if f:
            h = rms(x, eps) * (1.0 + sd[f"l{i}.norm2"].to(F64))
            Pm = sub(sd, f"l{i}.mlp.")
            x = x + (glu(Pm, "", h, gelu_tanh) if f["kind"] == "dense" else moe(f, Pm, h))
        trace.append(x.clone())
    h = rms(x, eps) * (1.0 + sd["final.norm"].to(F64))
    return lin(sd["head"], h), trace


# ------------------------------------------------------------------------------------------------ helpers of the tests


def tensor_shapes(cfg: dict) -> Dict[str, Tuple[int, ...]]:
    """Name -> shape of every tensor of a checkpoint with this config."""
    W, V = int(cfg["width"]), int(cfg["vocab"])
    out: Dict[str, Tuple[int, ...]] = {"embed": (V, W), "head": (V, W), "final.norm": (W,)}
    for i, lay in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lay["mixer"]
        out[p + "norm1"] = (W,)
        if lay["type"] == "latent_attention":
            H, d, r, dv, kr, qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            out.update({p + "mix.dq": (qr, W), p + "mix.dq.norm": (qr,), p + "mix.uq": (H * (d + r), qr), p + "mix.dkv": (kr + r, W),
                        p + "mix.dkv.norm": (kr,), p + "mix.uk": (H * d, kr), p + "mix.uv": (H * dv, kr), p + "mix.sink": (H,),
                        p + "mix.g": (H * dv, W), p + "mix.o": (W, H * dv)})
        elif lay["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * 2 * d, W), p + "mix.k": (G * 2 * d, W), p + "mix.v": (G * dv, W), p + "mix.q.norm": (d,),
                        p + "mix.k.norm": (d,), p + "mix.lq1": (d,), p + "mix.lk1": (d,), p + "mix.lq2": (d,), p + "mix.lk2": (d,),
                        p + "mix.o": (W, H * dv)})
        else:
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * d, W), p + "mix.k": (H * d, W), p + "mix.v": (H * dv, W), p + "mix.g": (H * dv, W),
                        p + "mix.o": (W, H * dv), p + "mix.norm": (H * dv,), p + "mix.i": (H, W), p + "mix.i.b": (H,), p + "mix.f": (H, W),
                        p + "mix.f.b": (H,)})
        f = lay.get("mlp")
        if not f:
            continue
        out[p + "norm2"] = (W,)
        if f["kind"] == "dense":
            out.update({p + "mlp.gate": (f["ff"], W), p + "mlp.up": (f["ff"], W), p + "mlp.down": (W, f["ff"])})
        else:
            E, I, F = f["router"]["experts"], f["router"].get("identity", 0), f["expert"]["ff"]
            for e in range(E):
                out.update({f"{p}mlp.e{e}.gate": (F, W), f"{p}mlp.e{e}.up": (F, W), f"{p}mlp.e{e}.down": (W, F)})
            out.update({p + "mlp.router": (E + I, W), p + "mlp.correction": (E + I,)})
            if f.get("shared"):
                Fs = f["shared"]["ff"]
                out.update({p + "mlp.shared.gate": (Fs, W), p + "mlp.shared.up": (Fs, W), p + "mlp.shared.down": (W, Fs), p + "mlp.shared.sg": (1, W)})
    return out


def random_checkpoint(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """Random weights, every value exactly representable in bfloat16 (so that both serving types read the same numbers)."""
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if name.endswith(("norm1", "norm2", "final.norm")) or name.endswith(".norm") and len(shape) == 1:
            t = 0.2 * torch.randn(shape, generator=g) + (1.0 if name.endswith(("q.norm", "k.norm", "dq.norm", "dkv.norm", "mix.norm")) else 0.0)
        elif last == "sink":
            t = torch.randn(shape, generator=g)
        elif last == "correction":
            t = 0.05 * torch.randn(shape, generator=g)
        elif name.endswith("i.b"):
            t = torch.randn(shape, generator=g)
        elif name.endswith("f.b"):
            t = 2.0 + torch.randn(shape, generator=g)
        elif last in ("lq1", "lk1", "lq2", "lk2"):
            t = 0.4 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * (1.3 / math.sqrt(shape[-1]))
        sd[name] = t.bfloat16().float()
    return sd


def greedy(cfg: dict, sd: Dict[str, torch.Tensor], prompt: List[int], n_new: int) -> List[int]:
    seq, out = list(prompt), []
    for _ in range(n_new):
        nxt = int(forward(cfg, sd, seq)[0][-1].argmax())
        out.append(nxt)
        seq.append(nxt)
    return out
