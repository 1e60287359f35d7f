"""A plain, slow statement of the Buvesun design in PyTorch (float64 by default), one function per mechanism.  It shares no
code with the framework: the tests compare the framework's kernels, caches and schedulers against it.

Inputs are the checkpoint's own names (`embed`, `loop.in`, `l<i>.norm1`, `l<i>.mix.q`, ...) and the `config.json` dict.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def layer_norm(x, w, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rotate(x, pos, dims: int, base: float, interleaved: bool):
    """x [T, heads, d]: the first `dims` dimensions of every head turn by pos * base^(-2i / dims); pair (i, i + dims/2) in the
    half layout, (2i, 2i + 1) in the interleaved one."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    ang = pos.to(x.dtype)[:, None] * f[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    if interleaved:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    else:
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * c - v * s
        out[..., half:dims] = v * c + u * s
    return out


def decayed_state_scan(q, k, v, decay: List[float], state: Optional[torch.Tensor] = None):
    """q, k [T, H, d], v [T, H, dv]: S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.  Returns (o [T, H, dv], final S)."""
    T, H, d = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, d, dv, dtype=q.dtype) if state is None else state.clone()
    g = torch.tensor(decay, dtype=q.dtype)[:, None, None]
    o = torch.zeros(T, H, dv, dtype=q.dtype)
    for t in range(T):
        S = g * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return o, S


def retention(h, w: Dict[str, torch.Tensor], m: dict, eps: float, pos, state=None):
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).view(T, H, d)
    k = (h @ w["k"].T).view(T, H, d)
    v = (h @ w["v"].T).view(T, H, dv)
    rot = m.get("rot")
    if rot:
        q = rotate(q, pos, rot["dims"], rot["base"], interleaved=False)
        k = rotate(k, pos, rot["dims"], rot["base"], interleaved=False)
    k = k * d ** -0.5
    o, S = decayed_state_scan(q, k, v, m["decay"], state)
    o = rms(o, eps).reshape(T, H * dv)
    g = h @ w["g"].T
    return (o * g * torch.sigmoid(g)) @ w["o"].T, S


def window_attention(h, w, m: dict, pos, past_k=None, past_v=None):
    """Grouped-query softmax attention over the keys j with 0 <= i - j < mask.size (all j <= i without a mask).  `past_k`, `past_v`:
    rotated keys / values of earlier tokens of the sequence.  Returns (output, all keys, all values)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).view(T, H, d)
    k = (h @ w["k"].T).view(T, G, d)
    v = (h @ w["v"].T).view(T, G, dv)
    rot = m.get("rot")
    if rot:
        q = rotate(q, pos, rot["dims"], rot["base"], interleaved=True)
        k = rotate(k, pos, rot["dims"], rot["base"], interleaved=True)
    if past_k is not None:
        k, v = torch.cat([past_k, k], 0), torch.cat([past_v, v], 0)
    n_past = k.shape[0] - T
    size = m["mask"]["size"] if m.get("mask") else None
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        i = n_past + t
        lo = 0 if size is None else max(0, i - size + 1)
        for hh in range(H):
            g = hh // (H // G)
            s = (k[lo:i + 1, g] @ q[t, hh]) * m["scale"]
            out[t, hh] = torch.softmax(s, 0) @ v[lo:i + 1, g]
    return out.reshape(T, H * dv) @ w["o"].T, k, v


def lightning(h, w, m: dict, eps: float, state=None):
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    silu = torch.nn.functional.silu
    q = silu(h @ w["q"].T).view(T, H, d)
    k = silu(h @ w["k"].T).view(T, H, d)
    v = silu(h @ w["v"].T).view(T, H, dv)
    o, S = decayed_state_scan(q, k, v, m["decay"], state)
    o = rms(o.reshape(T, H * dv), eps) * w["norm"]
    return (o * torch.sigmoid(h @ w["g"].T)) @ w["o"].T, S


def expert(h, w, limit: float):
    g = (h @ w["gate"].T).clamp(max=limit)
    u = (h @ w["up"].T).clamp(min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w["down"].T


def sub(sd: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in sd.items() if k.startswith(prefix)}


def feed_forward(h, sd, f: dict):
    """Routed experts (sigmoid scores, the `top` largest, the score scales the expert's INPUT) plus the shared expert."""
    r = f["router"]
    scores = torch.sigmoid(h @ sd["router"].T)
    top = torch.topk(scores, r["top"], dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for s, e in zip(top.values[t], top.indices[t]):
            out[t] += expert(s * h[t:t + 1], sub(sd, f"e{int(e)}."), f["expert"]["limit"])[0]
    if f.get("shared"):
        out = out + expert(h, sub(sd, "shared."), f["shared"]["limit"])
    return out


class Sequence:
    """One sequence's caches: per layer run the keys / values of the window mixer and the matrix states."""

    def __init__(self):
        self.n = 0
        self.runs: Dict[int, dict] = {}


def forward(cfg: dict, sd: Dict[str, torch.Tensor], tokens: List[int], seq: Optional[Sequence] = None, dtype=torch.float64,
            layers_out: Optional[list] = None):
    """Logits [len(tokens), vocab] of `tokens` appended to `seq` (a fresh sequence when None)."""
    sd = {k: v.to(dtype) if v.is_floating_point() else v for k, v in sd.items()}
    seq = seq if seq is not None else Sequence()
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    T = len(tokens)
    pos = torch.arange(seq.n, seq.n + T)
    x = sd["embed"][torch.tensor(tokens)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    x0 = x
    lp = cfg.get("loop")
    order = []
    L = len(cfg["layers"])
    if lp:
        order += [(i, False) for i in range(lp["start"])]
        for _ in range(lp["times"]):
            order += [(i, i == lp["start"]) for i in range(lp["start"], lp["stop"])]
        order += [(i, False) for i in range(lp["stop"], L)]
    else:
        order = [(i, False) for i in range(L)]
    for run, (i, starts) in enumerate(order):
        lay = cfg["layers"][i]
        w = sub(sd, f"l{i}.")
        st = seq.runs.setdefault(run, {})
        if starts:
            x = torch.cat([x, x0], -1) @ sd["loop.in"].T
        h = layer_norm(x, w["norm1"], eps)
        m = lay["mixer"]
        if lay["type"] == "retention":
            y, st["S"] = retention(h, sub(w, "mix."), m, eps, pos, st.get("S"))
        elif lay["type"] == "parallel":
            a, st["k"], st["v"] = window_attention(h, sub(w, "mix.left."), m["left"], pos, st.get("k"), st.get("v"))
            b, st["S"] = lightning(h, sub(w, "mix.right."), m["right"], eps, st.get("S"))
            y = m["left_scale"] * a + m["right_scale"] * b
        else:
            raise ValueError(lay["type"])
        x = x + mult * (layer_norm(y, w["norm1b"], eps) * w["ls1"])
        if lay.get("mlp") is not None:
            h = layer_norm(x, w["norm2"], eps)
            y = feed_forward(h, sub(w, "mlp."), lay["mlp"])
            x = x + mult * (layer_norm(y, w["norm2b"], eps) * w["ls2"])
        if layers_out is not None:
            layers_out.append(x.clone())
    seq.n += T
    return layer_norm(x, sd["final.norm"], eps) @ sd["head"].T


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    W, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, W), "head": (V, W), "final.norm": (W,)}
    if cfg.get("loop"):
        out["loop.in"] = (W, 2 * W)
    for i, lay in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lay["mixer"]
        out.update({p + "norm1": (W,), p + "norm1b": (W,), p + "ls1": (W,)})
        if lay["type"] == "retention":
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * d, W), p + "mix.k": (H * d, W), p + "mix.v": (H * dv, W), p + "mix.g": (H * dv, W), p + "mix.o": (W, H * dv)})
        else:
            a, b = m["left"], m["right"]
            H, G, d, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            out.update({p + "mix.left.q": (H * d, W), p + "mix.left.k": (G * d, W), p + "mix.left.v": (G * dv, W), p + "mix.left.o": (W, H * dv)})
            H, d, dv = b["heads"], b["dim"], b["vdim"]
            out.update({p + "mix.right.q": (H * d, W), p + "mix.right.k": (H * d, W), p + "mix.right.v": (H * dv, W), p + "mix.right.g": (H * dv, W),
                        p + "mix.right.o": (W, H * dv), p + "mix.right.norm": (H * dv,)})
        f = lay.get("mlp")
        if f is not None:
            out.update({p + "norm2": (W,), p + "norm2b": (W,), p + "ls2": (W,), p + "mlp.router": (f["router"]["experts"], W)})
            F = f["expert"]["ff"]
            for e in range(f["router"]["experts"]):
                out.update({f"{p}mlp.e{e}.gate": (F, W), f"{p}mlp.e{e}.up": (F, W), f"{p}mlp.e{e}.down": (W, F)})
            if f.get("shared"):
                Fs = f["shared"]["ff"]
                out.update({p + "mlp.shared.gate": (Fs, W), p + "mlp.shared.up": (Fs, W), p + "mlp.shared.down": (W, Fs)})
    return out


def random_checkpoint(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """Random weights, every value exactly representable in bfloat16 (so that both serving types read the same numbers)."""
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for name, shape in tensor_shapes(cfg).items():
        if len(shape) == 1:                                   # norm weights and layer scales: around 1, never near 0
            t = 1.0 + 0.25 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        elif name.endswith("mlp.router"):
            t = torch.randn(shape, generator=g) * (3.0 / math.sqrt(shape[-1]))
        else:
            t = torch.randn(shape, generator=g) * (1.3 / math.sqrt(shape[-1]))
        sd[name] = t.bfloat16().float()
    return sd


def greedy(cfg: dict, sd: Dict[str, torch.Tensor], prompt: List[int], n_new: int) -> List[int]:
    seq, out = list(prompt), []
    for _ in range(n_new):
        nxt = int(forward(cfg, sd, seq)[-1].argmax())
        out.append(nxt)
        seq.append(nxt)
    return out
