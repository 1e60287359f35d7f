"""Buvesun checkpoints <-> ReaLModel.

A Buvesun checkpoint is `config.json` + `model.safetensors`.  The config lists the layers one by one (`layers[i]` = mixer type
`retention` or `parallel`, the mixer's sizes, a routed feed-forward or null) and a `loop`: a range of layers that runs several
times with the same weights, each pass with its own cache / state, the embedding output mixed back in by a projection before
every pass.  The model is a heterogeneous stack (`ReaLModelConfig.blocks`) of mechanisms the config classes offer to any family:

  * `layer_norm_type="layer"`: bias-free LayerNorm before AND after every sublayer (`sandwich_norm`), a learned vector on every
    branch output (`layer_scale`), a constant on every residual add (`residual_mult`), an fp32 residual stream, a constant on
    the embedding output (`embed_scale`);
  * `DecayConfig`: linear attention with a fixed decay per head.  Mixer `retention` = rotated q / k (half layout), k times
    dim^(-1/2), per-head RMS norm, SiLU gate; the right branch of `parallel` = SiLU on q, k, v, one RMS norm with a weight over
    the concatenated heads, sigmoid gate;
  * `WindowAttentionConfig` with `rotary` (interleaved, partial) and a sliding window: the left branch of `parallel`;
  * mixer `parallel`: both branches read the same input, `branch_scales` weigh their outputs;
  * `BlockMLPConfig(kind="moe", limit=..)` with `ReaLMoEConfig(routing_type="sigmoid", scale_input=True)`: clamped gated experts,
    sigmoid scores, the weight on the expert's input, an ungated shared expert with its own clamp limit;
  * `LoopConfig(inject_mode="linear")`.

There is no `transformers` class for it: the config is read as a plain dict.  The gate slope of the experts (1.702) is fixed by
the design.

Checkpoint names -> framework names (layer i of the checkpoint is block i + 1 here):
  embed / head / final.norm                  0.wte.weight / {L+1}.head.weight / {L}.ln_f.weight
  loop.in                                    {loop.start+1}.loop_in.weight
  l<i>.norm1, norm1b, ls1                    attn.ln.weight, attn.ln_post.weight, attn.ls.weight
  l<i>.norm2, norm2b, ls2                    mlp.ln.weight, mlp.ln_post.weight, mlp.ls.weight
  mlp.e<j>.gate, up / down                   mlp.experts.gate_up.weight [E, 2F, W] / mlp.experts.down.weight [E, W, F]
  mlp.router / shared.gate, up / down        mlp.router.weight / mlp.shared.gate_up.weight / mlp.shared.down.weight
  retention: mix.q, k, v, g / o              attn.in.weight (sections [q | k | v | g]) / attn.o.weight
  parallel:  mix.left.q, k, v, mix.right.q, k, v, g   attn.in.weight (sections [left q | k | v | right q | k | v | g])
             mix.left.o / right.o / right.norm        attn.o.weight / attn.o2.weight / attn.o_norm.weight
"""

from __future__ import annotations

from typing import Dict, List

import torch

from realhf_b200.api.model import (BlockConfig, BlockMLPConfig, DecayConfig, LoopConfig, ReaLModelConfig, ReaLMoEConfig, RotaryConfig,
                                   WindowAttentionConfig, register_hf_family)

EXPERT_ALPHA = 1.702     # y = g * sigmoid(1.702 g) * (u + 1)


def _rotary(rot, interleaved: bool):
    return RotaryConfig(dims=int(rot["dims"]), base=float(rot["base"]), interleaved=interleaved) if rot else None


def _mlp_from_dict(i: int, f):
    if f is None:
        return None
    if f.get("kind", "moe") != "moe":
        raise ValueError(f"Buvesun layer {i}: unknown feed-forward kind `{f['kind']}`")
    r, sh = f["router"], f.get("shared")
    moe = ReaLMoEConfig(num_experts=int(r["experts"]), top_k=int(r["top"]), routing_type="sigmoid", aux_loss_coeff=0.0, renormalize=False,
                        scale_input=True, shared_ff=int(sh["ff"]) if sh else None, shared_gate=False,
                        shared_limit=float(sh["limit"]) if sh else None)
    return BlockMLPConfig(kind="moe", ff=int(f["expert"]["ff"]), limit=float(f["expert"]["limit"]), alpha=EXPERT_ALPHA, moe=moe)


def config_from_dict(d: dict, is_critic: bool = False) -> ReaLModelConfig:
    blocks: List[BlockConfig] = []
    for i, lay in enumerate(d["layers"]):
        m = lay["mixer"]
        mlp = _mlp_from_dict(i, lay.get("mlp"))
        if lay["type"] == "retention":
            dc = DecayConfig(n_heads=int(m["heads"]), qk_dim=int(m["dim"]), v_dim=int(m["vdim"]), decay=list(m["decay"]), act="none",
                             rotary=_rotary(m.get("rot"), False), k_scale=float(m["dim"]) ** -0.5, out_norm="head", gate="silu")
            blocks.append(BlockConfig(mixer="decay", decay=dc, mlp=mlp))
        elif lay["type"] == "parallel":
            l, r = m["left"], m["right"]
            mask = l.get("mask")
            w = WindowAttentionConfig(n_heads=int(l["heads"]), n_kv_heads=int(l["kv_heads"]), qk_dim=int(l["dim"]), v_dim=int(l["vdim"]),
                                      scale=float(l["scale"]), window=int(mask["size"]) if mask else None, keep_first=0, qkv_bias=False,
                                      value_norm=False, head_temp=False, slope_base=None, sink=False, out_gate=False,
                                      rotary=_rotary(l.get("rot"), True))
            dc = DecayConfig(n_heads=int(r["heads"]), qk_dim=int(r["dim"]), v_dim=int(r["vdim"]), decay=list(r["decay"]), act="silu",
                             rotary=None, k_scale=1.0, out_norm="full", gate="sigmoid")
            blocks.append(BlockConfig(mixer="parallel", wattn=w, decay=dc, mlp=mlp,
                                      branch_scales=(float(m.get("left_scale", 1.0)), float(m.get("right_scale", 1.0)))))
        else:
            raise ValueError(f"Buvesun layer {i}: unknown mixer type `{lay['type']}`")
    lp = d.get("loop")
    loop = LoopConfig(start=int(lp["start"]), stop=int(lp["stop"]), times=int(lp["times"]), inject=True, inject_mode="linear") if lp else None
    first = blocks[0].wattn or blocks[0].decay
    ffs = [b.mlp.ff for b in blocks if b.mlp is not None]
    emb = d.get("embedding") or {}
    return ReaLModelConfig(
        n_layers=len(blocks), n_kv_heads=getattr(first, "n_kv_heads", first.n_heads), n_q_heads=first.n_heads, hidden_dim=int(d["width"]),
        intermediate_dim=max(ffs) if ffs else 0, vocab_size=int(d["vocab"]), head_dim=first.qk_dim, n_positions=None, embd_pdrop=0.0,
        resid_pdrop=0.0, attn_pdrop=0.0, layer_norm_epsilon=float(d["norm"]["eps"]), activation_function="silu",
        scale_attn_by_inverse_layer_idx=False, scale_attn_weights=True, use_attention_bias=False, use_attn_proj_bias=False,
        use_mlp_bias=False, layer_norm_type="layer", mlp_type=None, apply_rotary=False, tied_embedding=False, is_critic=is_critic,
        blocks=blocks, norm_groups=1, sandwich_norm=True, conv_taps=0, fp32_residual=True, loop=loop,
        embed_scale=float(emb["scale"]) if "scale" in emb else None, residual_mult=float(d.get("residual_mult", 1.0)), layer_scale=True)


def _rot_to_dict(r):
    return dict(base=r.base, dims=r.dims)


def _mlp_to_dict(f):
    if f is None:
        return None
    mo = f.moe
    out = dict(expert=dict(ff=f.ff, limit=f.limit), kind="moe", router=dict(experts=mo.num_experts, top=mo.top_k))
    if mo.shared_ff:
        out["shared"] = dict(ff=mo.shared_ff, limit=mo.shared_limit if mo.shared_limit is not None else f.limit)
    return out


def config_to_dict(cfg: ReaLModelConfig) -> dict:
    layers = []
    for b in cfg.blocks:
        d = b.decay
        if b.mixer == "decay":
            m = dict(decay=list(d.decay), dim=d.qk_dim, heads=d.n_heads, vdim=d.v_dim)
            if d.rotary is not None:
                m["rot"] = _rot_to_dict(d.rotary)
            layers.append(dict(mixer=m, mlp=_mlp_to_dict(b.mlp), type="retention"))
        else:
            w = b.wattn
            left = dict(dim=w.qk_dim, heads=w.n_heads, kv_heads=w.n_kv_heads, scale=w.scale, vdim=w.v_dim)
            if w.window is not None:
                left["mask"] = dict(size=w.window)
            if w.rotary is not None:
                left["rot"] = _rot_to_dict(w.rotary)
            right = dict(decay=list(d.decay), dim=d.qk_dim, heads=d.n_heads, vdim=d.v_dim)
            layers.append(dict(mixer=dict(left=left, left_scale=b.branch_scales[0], right=right, right_scale=b.branch_scales[1]),
                               mlp=_mlp_to_dict(b.mlp), type="parallel"))
    out = dict(architecture="Buvesun", layers=layers, norm=dict(eps=cfg.layer_norm_epsilon), residual_mult=cfg.residual_mult,
               vocab=cfg.vocab_size, width=cfg.hidden_dim)
    if cfg.embed_scale is not None:
        out["embedding"] = dict(scale=cfg.embed_scale)
    if cfg.loop is not None:
        out["loop"] = dict(start=cfg.loop.start, stop=cfg.loop.stop, times=cfg.loop.times)
    return out


_LEFT = ("left.q", "left.k", "left.v")
_RIGHT = ("q", "k", "v", "g")


def _sd_from_ckpt(sd: Dict[str, torch.Tensor], cfg: ReaLModelConfig) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    L = cfg.n_layers
    if "embed" in sd:
        out["0.wte.weight"] = sd["embed"]
    if "head" in sd:
        out[f"{L + 1}.head.weight"] = sd["head"]
    if "final.norm" in sd:
        out[f"{L}.ln_f.weight"] = sd["final.norm"]
    if cfg.loop is not None and "loop.in" in sd:
        out[f"{cfg.loop.start + 1}.loop_in.weight"] = sd["loop.in"]
    for i, b in enumerate(cfg.blocks):
        cp, rp = f"l{i}.", f"{i + 1}."
        if cp + "norm1" not in sd:
            continue
        out[rp + "attn.ln.weight"] = sd[cp + "norm1"]
        out[rp + "attn.ln_post.weight"] = sd[cp + "norm1b"]
        out[rp + "attn.ls.weight"] = sd[cp + "ls1"]
        if b.mixer == "decay":
            out[rp + "attn.in.weight"] = torch.cat([sd[f"{cp}mix.{n}"] for n in _RIGHT], 0)
            out[rp + "attn.o.weight"] = sd[cp + "mix.o"]
        else:
            out[rp + "attn.in.weight"] = torch.cat([sd[f"{cp}mix.{n}"] for n in _LEFT] + [sd[f"{cp}mix.right.{n}"] for n in _RIGHT], 0)
            out[rp + "attn.o.weight"] = sd[cp + "mix.left.o"]
            out[rp + "attn.o2.weight"] = sd[cp + "mix.right.o"]
            out[rp + "attn.o_norm.weight"] = sd[cp + "mix.right.norm"]
        f = b.mlp
        if f is None:
            continue
        out[rp + "mlp.ln.weight"] = sd[cp + "norm2"]
        out[rp + "mlp.ln_post.weight"] = sd[cp + "norm2b"]
        out[rp + "mlp.ls.weight"] = sd[cp + "ls2"]
        E = f.moe.num_experts
        out[rp + "mlp.router.weight"] = sd[cp + "mlp.router"]
        out[rp + "mlp.experts.gate_up.weight"] = torch.stack([torch.cat([sd[f"{cp}mlp.e{e}.gate"], sd[f"{cp}mlp.e{e}.up"]], 0) for e in range(E)], 0)
        out[rp + "mlp.experts.down.weight"] = torch.stack([sd[f"{cp}mlp.e{e}.down"] for e in range(E)], 0)
        if f.moe.shared_ff:
            out[rp + "mlp.shared.gate_up.weight"] = torch.cat([sd[cp + "mlp.shared.gate"], sd[cp + "mlp.shared.up"]], 0)
            out[rp + "mlp.shared.down.weight"] = sd[cp + "mlp.shared.down"]
    return out


def _split(v: torch.Tensor, sizes):
    out, off = [], 0
    for n in sizes:
        out.append(v[off:off + n])
        off += n
    return out


def _sd_to_ckpt(sd: Dict[str, torch.Tensor], cfg: ReaLModelConfig) -> Dict[str, torch.Tensor]:
    from realhf_b200.models.sharding import decay_sections, wattn_sections
    out: Dict[str, torch.Tensor] = {}
    L = cfg.n_layers
    plain = {"attn.ln.weight": "norm1", "attn.ln_post.weight": "norm1b", "attn.ls.weight": "ls1", "mlp.ln.weight": "norm2",
             "mlp.ln_post.weight": "norm2b", "mlp.ls.weight": "ls2", "mlp.router.weight": "mlp.router", "mlp.shared.down.weight": "mlp.shared.down"}
    for k, v in sd.items():
        li, name = k.split(".", 1)
        li = int(li)
        if li == 0:
            out["embed"] = v
        elif li == L + 1:
            out["head"] = v
        elif name == "ln_f.weight":
            out["final.norm"] = v
        elif name == "loop_in.weight":
            out["loop.in"] = v
        else:
            cp, b = f"l{li - 1}.", cfg.blocks[li - 1]
            par = b.mixer == "parallel"
            if name in plain:
                out[cp + plain[name]] = v
            elif name == "attn.in.weight":
                parts = _split(v, (wattn_sections(b.wattn) if par else ()) + decay_sections(b.decay))
                names = [f"mix.{n}" for n in _LEFT] + [f"mix.right.{n}" for n in _RIGHT] if par else [f"mix.{n}" for n in _RIGHT]
                for n, t in zip(names, parts):
                    out[cp + n] = t
            elif name == "attn.o.weight":
                out[cp + ("mix.left.o" if par else "mix.o")] = v
            elif name == "attn.o2.weight":
                out[cp + "mix.right.o"] = v
            elif name == "attn.o_norm.weight":
                out[cp + "mix.right.norm"] = v
            elif name == "mlp.shared.gate_up.weight":
                F = b.mlp.moe.shared_ff
                out[cp + "mlp.shared.gate"], out[cp + "mlp.shared.up"] = v[:F], v[F:]
            elif name == "mlp.experts.gate_up.weight":
                for e in range(v.shape[0]):
                    out[f"{cp}mlp.e{e}.gate"], out[f"{cp}mlp.e{e}.up"] = v[e, :b.mlp.ff], v[e, b.mlp.ff:]
            elif name == "mlp.experts.down.weight":
                for e in range(v.shape[0]):
                    out[f"{cp}mlp.e{e}.down"] = v[e]
            else:
                raise KeyError(k)
    return {k: v.contiguous() for k, v in out.items()}


def _block_names(cfg: ReaLModelConfig, i: int) -> List[str]:
    b, cp = cfg.blocks[i], f"l{i}."
    names = [cp + n for n in ("norm1", "norm1b", "ls1")]
    if b.mixer == "decay":
        names += [cp + "mix." + n for n in _RIGHT + ("o",)]
    else:
        names += [cp + "mix." + n for n in _LEFT + ("left.o",)] + [cp + "mix.right." + n for n in _RIGHT + ("o", "norm")]
    f = b.mlp
    if f is not None:
        names += [cp + n for n in ("norm2", "norm2b", "ls2", "mlp.router")]
        names += [f"{cp}mlp.e{e}.{n}" for e in range(f.moe.num_experts) for n in ("gate", "up", "down")]
        if f.moe.shared_ff:
            names += [cp + "mlp.shared." + n for n in ("gate", "up", "down")]
    if cfg.loop is not None and i == cfg.loop.start:
        names.append("loop.in")
    if i == cfg.n_layers - 1:
        names.append("final.norm")
    return names


def make_test_config() -> ReaLModelConfig:
    moe = dict(kind="moe", expert=dict(ff=16, limit=1.5), router=dict(experts=4, top=2), shared=dict(ff=24, limit=2.5))
    ret = dict(type="retention", mlp=moe, mixer=dict(decay=[0.9, 0.97, 0.995], dim=8, heads=3, vdim=12, rot=dict(base=10000.0, dims=4)))
    par = dict(type="parallel", mlp=None,
               mixer=dict(left=dict(dim=12, heads=4, kv_heads=2, vdim=8, scale=0.3, mask=dict(size=5), rot=dict(base=500.0, dims=6)),
                          left_scale=0.7, right=dict(decay=[0.8, 0.99], dim=8, heads=2, vdim=12), right_scale=1.2))
    return config_from_dict(dict(layers=[par, ret, par], loop=dict(start=1, stop=3, times=2), norm=dict(eps=1e-5), vocab=96, width=32,
                                 embedding=dict(scale=2.0), residual_mult=0.6))


register_hf_family(
    "buvesun", "Buvesun", lambda hf, is_critic=False: config_from_dict(hf if isinstance(hf, dict) else hf.to_dict(), is_critic),
    config_to_dict, _sd_from_ckpt, _sd_to_ckpt, lambda cfg: ["embed"], _block_names, lambda cfg: ["head"],
    make_test_config=make_test_config, config_from_dict=config_from_dict, config_to_dict=config_to_dict, weight_file="model.safetensors")
