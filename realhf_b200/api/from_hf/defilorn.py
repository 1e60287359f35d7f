"""Defilorn checkpoints <-> ReaLModel.

A Defilorn checkpoint is `config.json` + `model.safetensors`.  The config lists the layers one by one (`layers[i]` = mixer type
`latent_attention`, `attention` or `mlstm`, the mixer's sizes, a feed-forward or null) and a `loop`: a range of layers that runs
several times with the same weights, each pass with its own cache / state, the embedding output added back to the stream before
every pass but the first.  The model is a heterogeneous stack (`ReaLModelConfig.blocks`) of mechanisms the config classes offer
to any family:

  * pre-norm RMSNorm sublayers whose weights are stored around zero (`layer_norm_type="gemma"`: the factor is 1 + w), an fp32
    residual stream, no positions in the embedding;
  * `LatentAttentionConfig` in its rotated form: queries through a normalised latent, one cached latent per token plus one
    rotated key part shared by the heads (interleaved rotation with YaRN-rescaled frequencies: `RotaryConfig`), causal softmax
    with a sink logit, an element-wise sigmoid output gate;
  * `WindowAttentionConfig` with `n_maps = 2` (differential attention), `qk_norm` and a sliding window, grouped key / value heads;
  * `MLSTMConfig`: the matrix-memory LSTM;
  * `BlockMLPConfig(kind="glu", act="gelu_tanh")` and `kind="moe"` with `ReaLMoEConfig(routing_type="softmax_all")`: scores over
    all experts with a correction term for the choice only, unnormalised weights, identity experts and a gated shared expert;
  * `LoopConfig(inject_mode="add")`.

There is no `transformers` class for it: the config is read as a plain dict.

Checkpoint names -> framework names (layer i of the checkpoint is block i + 1 here):
  embed / head / final.norm                  0.wte.weight / {L+1}.head.weight / {L}.ln_f.weight
  l<i>.norm1 / norm2                         attn.ln.weight / mlp.ln.weight
  dense:  mlp.gate, up / down                mlp.gate_up.weight / mlp.down.weight
  moe:    mlp.e<j>.gate, up / down           mlp.experts.gate_up.weight [E, 2F, W] / mlp.experts.down.weight [E, W, F]
          mlp.router / correction            mlp.router.weight / mlp.router.correction
          mlp.shared.gate, up / down / sg    mlp.shared.gate_up.weight / mlp.shared.down.weight / mlp.shared.sg.weight
  latent_attention: mix.dq, dkv, g           attn.in.weight      (sections [query latent | latent, rotated key part | gate])
          mix.dq.norm / uq / dkv.norm        attn.q_ln.weight / attn.uq.weight / attn.dkv_ln.weight
          mix.uk, uv / sink / o              attn.ukv.weight / attn.sink.weight / attn.o.weight
  attention: mix.q, k, v                     attn.qkvg.weight    (sections [q | k | v]; the query heads, stored (head, map) in the
                                             checkpoint, are regrouped to (key head, map, head within the group))
          mix.q.norm / k.norm                attn.q_norm.weight / attn.k_norm.weight
          mix.lq1, lk1, lq2, lk2 / o         attn.lambda.weight [4, dim] / attn.o.weight
  mlstm:  mix.q, k, v, g, i, f               attn.in.weight      (sections [q | k | v | g | i, f padded to 8 rows])
          mix.i.b, f.b / norm / o            attn.gate_bias.weight [2H] / attn.o_norm.weight / attn.o.weight
"""

from __future__ import annotations

from typing import Dict, List

import torch

from realhf_b200.api.model import (BlockConfig, BlockMLPConfig, LatentAttentionConfig, LoopConfig, MLSTMConfig, ReaLModelConfig, ReaLMoEConfig,
                                   RotaryConfig, WindowAttentionConfig, register_hf_family)


def _mlp_from_dict(i: int, f) -> BlockMLPConfig:
    if f is None:
        return None
    if f["kind"] == "dense":
        return BlockMLPConfig(kind="glu", ff=int(f["ff"]), act="gelu_tanh")
    if f["kind"] == "moe":
        r, sh = f["router"], f.get("shared")
        moe = ReaLMoEConfig(num_experts=int(r["experts"]), top_k=int(r["top"]), routing_type="softmax_all", aux_loss_coeff=0.0,
                            score_correction=True, renormalize=False, identity_experts=int(r.get("identity", 0)),
                            shared_ff=int(sh["ff"]) if sh else None)
        return BlockMLPConfig(kind="moe", ff=int(f["expert"]["ff"]), moe=moe)
    raise ValueError(f"Defilorn layer {i}: unknown feed-forward kind `{f['kind']}`")


def config_from_dict(d: dict, is_critic: bool = False) -> ReaLModelConfig:
    blocks: List[BlockConfig] = []
    for i, lay in enumerate(d["layers"]):
        m = lay["mixer"]
        mlp = _mlp_from_dict(i, lay.get("mlp"))
        if lay["type"] == "latent_attention":
            rot = m.get("rot")
            rotary = None
            if rot:
                sc = rot.get("scaling")
                rotary = RotaryConfig(dims=int(rot["dims"]), base=float(rot["base"]), interleaved=True,
                                      factor=float(sc["factor"]) if sc else None, original=int(sc["original"]) if sc else 0,
                                      fast=float(sc["fast"]) if sc else 32.0, slow=float(sc["slow"]) if sc else 1.0)
            a = LatentAttentionConfig(n_heads=int(m["heads"]), qk_dim=int(m["dim"]), v_dim=int(m["vdim"]), kv_rank=int(m["kv_rank"]),
                                      scale=float(m["scale"]), rot_dim=int(m.get("rot_dim", 0)), rotary=rotary, q_rank=int(m["q_rank"]),
                                      sink=True, out_gate=True)
            blocks.append(BlockConfig(mixer="latent_attention", attn=a, mlp=mlp))
        elif lay["type"] == "attention":
            mask = m.get("mask")
            w = WindowAttentionConfig(n_heads=int(m["heads"]), n_kv_heads=int(m["kv_heads"]), qk_dim=int(m["dim"]), v_dim=int(m["vdim"]),
                                      scale=float(m["scale"]), window=int(mask["size"]) if mask else None, keep_first=0, qkv_bias=False,
                                      value_norm=False, head_temp=False, slope_base=None, sink=False, out_gate=False, qk_norm=True, n_maps=2,
                                      diff=float(m["diff"]))
            blocks.append(BlockConfig(mixer="window_attention", wattn=w, mlp=mlp))
        elif lay["type"] == "mlstm":
            ml = MLSTMConfig(n_heads=int(m["heads"]), qk_dim=int(m["dim"]), v_dim=int(m["vdim"]), gate_cap=float(m["gate_cap"]))
            blocks.append(BlockConfig(mixer="mlstm", mlstm=ml, mlp=mlp))
        else:
            raise ValueError(f"Defilorn layer {i}: unknown mixer type `{lay['type']}`")
    lp = d.get("loop")
    loop = LoopConfig(start=int(lp["start"]), stop=int(lp["stop"]), times=int(lp["times"]), inject=True, inject_mode="add") if lp else None
    heads = [(b.attn or b.wattn or b.mlstm) for b in blocks]
    ffs = [b.mlp.ff for b in blocks if b.mlp is not None]
    return ReaLModelConfig(
        n_layers=len(blocks), n_kv_heads=getattr(heads[0], "n_kv_heads", heads[0].n_heads), n_q_heads=heads[0].n_heads,
        hidden_dim=int(d["width"]), intermediate_dim=max(ffs) if ffs else 0, vocab_size=int(d["vocab"]), head_dim=heads[0].qk_dim,
        n_positions=None, embd_pdrop=0.0, resid_pdrop=0.0, attn_pdrop=0.0, layer_norm_epsilon=float(d["norm"]["eps"]),
        activation_function="silu", scale_attn_by_inverse_layer_idx=False, scale_attn_weights=True, use_attention_bias=False,
        use_attn_proj_bias=False, use_mlp_bias=False, layer_norm_type="gemma", mlp_type=None, apply_rotary=False, tied_embedding=False,
        is_critic=is_critic, blocks=blocks, norm_groups=1, sandwich_norm=False, conv_taps=0, fp32_residual=True, loop=loop)


def _mlp_to_dict(f):
    if f is None:
        return None
    if f.kind == "glu":
        return dict(ff=f.ff, kind="dense")
    mo = f.moe
    out = dict(expert=dict(ff=f.ff), kind="moe", router=dict(experts=mo.num_experts, identity=mo.identity_experts, top=mo.top_k))
    if mo.shared_ff:
        out["shared"] = dict(ff=mo.shared_ff)
    return out


def config_to_dict(cfg: ReaLModelConfig) -> dict:
    layers = []
    for b in cfg.blocks:
        f = _mlp_to_dict(b.mlp)
        if b.mixer == "latent_attention":
            a = b.attn
            m = dict(dim=a.qk_dim, heads=a.n_heads, kv_rank=a.kv_rank, q_rank=a.q_rank, rot_dim=a.rot_dim, scale=a.scale, vdim=a.v_dim)
            if a.rotary is not None:
                r = a.rotary
                m["rot"] = dict(base=r.base, dims=r.dims)
                if r.factor is not None:
                    m["rot"]["scaling"] = dict(factor=r.factor, fast=r.fast, original=r.original, slow=r.slow)
            layers.append(dict(mixer=m, mlp=f, type="latent_attention"))
        elif b.mixer == "window_attention":
            w = b.wattn
            m = dict(diff=w.diff, dim=w.qk_dim, heads=w.n_heads, kv_heads=w.n_kv_heads, scale=w.scale, vdim=w.v_dim)
            if w.window is not None:
                m["mask"] = dict(size=w.window)
            layers.append(dict(mixer=m, mlp=f, type="attention"))
        else:
            ml = b.mlstm
            layers.append(dict(mixer=dict(dim=ml.qk_dim, gate_cap=ml.gate_cap, heads=ml.n_heads, vdim=ml.v_dim), mlp=f, type="mlstm"))
    out = dict(architecture="Defilorn", layers=layers, norm=dict(eps=cfg.layer_norm_epsilon), vocab=cfg.vocab_size, width=cfg.hidden_dim)
    if cfg.loop is not None:
        out["loop"] = dict(start=cfg.loop.start, stop=cfg.loop.stop, times=cfg.loop.times)
    return out


def _pad_rows(t: torch.Tensor, rows: int) -> torch.Tensor:
    if t.shape[0] == rows:
        return t
    return torch.cat([t, torch.zeros(rows - t.shape[0], *t.shape[1:], dtype=t.dtype)], 0)


def _regroup_queries(q: torch.Tensor, w: WindowAttentionConfig, inverse: bool = False) -> torch.Tensor:
    """Query rows (head, map, dim) <-> (key head, map, head within the group, dim)."""
    G, per, d = w.n_kv_heads, w.n_heads // w.n_kv_heads, w.qk_dim
    if inverse:
        return q.reshape(G, 2, per, d, -1).permute(0, 2, 1, 3, 4).reshape(q.shape)
    return q.reshape(G, per, 2, d, -1).permute(0, 2, 1, 3, 4).reshape(q.shape)


def _sd_from_ckpt(sd: Dict[str, torch.Tensor], cfg: ReaLModelConfig) -> Dict[str, torch.Tensor]:
    from realhf_b200.models.sharding import mlstm_sections
    out: Dict[str, torch.Tensor] = {}
    L = cfg.n_layers
    if "embed" in sd:
        out["0.wte.weight"] = sd["embed"]
    if "head" in sd:
        out[f"{L + 1}.head.weight"] = sd["head"]
    if "final.norm" in sd:
        out[f"{L}.ln_f.weight"] = sd["final.norm"]
    for i, b in enumerate(cfg.blocks):
        cp, rp = f"l{i}.", f"{i + 1}."
        if cp + "norm1" not in sd:
            continue
        out[rp + "attn.ln.weight"] = sd[cp + "norm1"]
        if b.mixer == "latent_attention":
            out[rp + "attn.in.weight"] = torch.cat([sd[cp + "mix.dq"], sd[cp + "mix.dkv"], sd[cp + "mix.g"]], 0)
            out[rp + "attn.q_ln.weight"] = sd[cp + "mix.dq.norm"]
            out[rp + "attn.uq.weight"] = sd[cp + "mix.uq"]
            out[rp + "attn.dkv_ln.weight"] = sd[cp + "mix.dkv.norm"]
            out[rp + "attn.ukv.weight"] = torch.cat([sd[cp + "mix.uk"], sd[cp + "mix.uv"]], 0)
            out[rp + "attn.sink.weight"] = sd[cp + "mix.sink"]
        elif b.mixer == "window_attention":
            out[rp + "attn.qkvg.weight"] = torch.cat([_regroup_queries(sd[cp + "mix.q"], b.wattn), sd[cp + "mix.k"], sd[cp + "mix.v"]], 0)
            out[rp + "attn.q_norm.weight"] = sd[cp + "mix.q.norm"]
            out[rp + "attn.k_norm.weight"] = sd[cp + "mix.k.norm"]
            out[rp + "attn.lambda.weight"] = torch.stack([sd[cp + "mix.lq1"], sd[cp + "mix.lk1"], sd[cp + "mix.lq2"], sd[cp + "mix.lk2"]], 0)
        else:
            sec = mlstm_sections(b.mlstm)
            gates = _pad_rows(torch.cat([sd[cp + "mix.i"], sd[cp + "mix.f"]], 0), sec[4])
            out[rp + "attn.in.weight"] = torch.cat([sd[cp + "mix.q"], sd[cp + "mix.k"], sd[cp + "mix.v"], sd[cp + "mix.g"], gates], 0)
            out[rp + "attn.gate_bias.weight"] = torch.cat([sd[cp + "mix.i.b"], sd[cp + "mix.f.b"]], 0)
            out[rp + "attn.o_norm.weight"] = sd[cp + "mix.norm"]
        out[rp + "attn.o.weight"] = sd[cp + "mix.o"]
        f = b.mlp
        if f is None:
            continue
        out[rp + "mlp.ln.weight"] = sd[cp + "norm2"]
        if f.kind == "glu":
            out[rp + "mlp.gate_up.weight"] = torch.cat([sd[cp + "mlp.gate"], sd[cp + "mlp.up"]], 0)
            out[rp + "mlp.down.weight"] = sd[cp + "mlp.down"]
        else:
            E = f.moe.num_experts
            out[rp + "mlp.router.weight"] = sd[cp + "mlp.router"]
            out[rp + "mlp.router.correction"] = sd[cp + "mlp.correction"]
            out[rp + "mlp.experts.gate_up.weight"] = torch.stack([torch.cat([sd[f"{cp}mlp.e{e}.gate"], sd[f"{cp}mlp.e{e}.up"]], 0) for e in range(E)], 0)
            out[rp + "mlp.experts.down.weight"] = torch.stack([sd[f"{cp}mlp.e{e}.down"] for e in range(E)], 0)
            if f.moe.shared_ff:
                out[rp + "mlp.shared.gate_up.weight"] = torch.cat([sd[cp + "mlp.shared.gate"], sd[cp + "mlp.shared.up"]], 0)
                out[rp + "mlp.shared.down.weight"] = sd[cp + "mlp.shared.down"]
                out[rp + "mlp.shared.sg.weight"] = sd[cp + "mlp.shared.sg"]
    return out


def _sd_to_ckpt(sd: Dict[str, torch.Tensor], cfg: ReaLModelConfig) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    L = cfg.n_layers
    plain = {"attn.ln.weight": "norm1", "mlp.ln.weight": "norm2", "attn.o.weight": "mix.o", "attn.q_ln.weight": "mix.dq.norm",
             "attn.uq.weight": "mix.uq", "attn.dkv_ln.weight": "mix.dkv.norm", "attn.sink.weight": "mix.sink",
             "attn.q_norm.weight": "mix.q.norm", "attn.k_norm.weight": "mix.k.norm", "attn.o_norm.weight": "mix.norm",
             "mlp.down.weight": "mlp.down", "mlp.router.weight": "mlp.router", "mlp.router.correction": "mlp.correction",
             "mlp.shared.down.weight": "mlp.shared.down", "mlp.shared.sg.weight": "mlp.shared.sg"}
    for k, v in sd.items():
        li, name = k.split(".", 1)
        li = int(li)
        if li == 0:
            out["embed"] = v
        elif li == L + 1:
            out["head"] = v
        elif name == "ln_f.weight":
            out["final.norm"] = v
        else:
            cp, b = f"l{li - 1}.", cfg.blocks[li - 1]
            if name in plain:
                out[cp + plain[name]] = v
            elif name == "attn.in.weight" and b.mixer == "latent_attention":
                a = b.attn
                out[cp + "mix.dq"], out[cp + "mix.dkv"], out[cp + "mix.g"] = v[:a.q_rank], v[a.q_rank:a.q_rank + a.cache_width], v[a.q_rank + a.cache_width:]
            elif name == "attn.ukv.weight":
                n = b.attn.n_heads * b.attn.qk_dim
                out[cp + "mix.uk"], out[cp + "mix.uv"] = v[:n], v[n:]
            elif name == "attn.qkvg.weight":
                w = b.wattn
                nq, nk = 2 * w.n_heads * w.qk_dim, 2 * w.n_kv_heads * w.qk_dim
                out[cp + "mix.q"], out[cp + "mix.k"], out[cp + "mix.v"] = _regroup_queries(v[:nq], w, inverse=True), v[nq:nq + nk], v[nq + nk:]
            elif name == "attn.lambda.weight":
                out[cp + "mix.lq1"], out[cp + "mix.lk1"], out[cp + "mix.lq2"], out[cp + "mix.lk2"] = v[0], v[1], v[2], v[3]
            elif name == "attn.in.weight":
                m = b.mlstm
                nq, nv, H = m.n_heads * m.qk_dim, m.n_heads * m.v_dim, m.n_heads
                out[cp + "mix.q"], out[cp + "mix.k"], out[cp + "mix.v"], out[cp + "mix.g"] = v[:nq], v[nq:2 * nq], v[2 * nq:2 * nq + nv], v[2 * nq + nv:2 * nq + 2 * nv]
                o0 = 2 * nq + 2 * nv
                out[cp + "mix.i"], out[cp + "mix.f"] = v[o0:o0 + H], v[o0 + H:o0 + 2 * H]
            elif name == "attn.gate_bias.weight":
                H = b.mlstm.n_heads
                out[cp + "mix.i.b"], out[cp + "mix.f.b"] = v[:H], v[H:]
            elif name == "mlp.gate_up.weight":
                out[cp + "mlp.gate"], out[cp + "mlp.up"] = v[:b.mlp.ff], v[b.mlp.ff:]
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
    names = [cp + "norm1", cp + "mix.o"]
    if b.mixer == "latent_attention":
        names += [cp + "mix." + n for n in ("dq", "dq.norm", "uq", "dkv", "dkv.norm", "uk", "uv", "sink", "g")]
    elif b.mixer == "window_attention":
        names += [cp + "mix." + n for n in ("q", "k", "v", "q.norm", "k.norm", "lq1", "lk1", "lq2", "lk2")]
    else:
        names += [cp + "mix." + n for n in ("q", "k", "v", "g", "i", "i.b", "f", "f.b", "norm")]
    f = b.mlp
    if f is not None:
        names.append(cp + "norm2")
        if f.kind == "glu":
            names += [cp + "mlp." + n for n in ("gate", "up", "down")]
        else:
            names += [f"{cp}mlp.e{e}.{n}" for e in range(f.moe.num_experts) for n in ("gate", "up", "down")]
            names += [cp + "mlp.router", cp + "mlp.correction"]
            if f.moe.shared_ff:
                names += [cp + "mlp.shared." + n for n in ("gate", "up", "down", "sg")]
    if i == cfg.n_layers - 1:
        names.append("final.norm")
    return names


def make_test_config() -> ReaLModelConfig:
    lat = dict(type="latent_attention", mlp=dict(kind="dense", ff=48),
               mixer=dict(dim=8, heads=2, kv_rank=16, q_rank=24, rot_dim=4, scale=0.3, vdim=12,
                          rot=dict(base=10000.0, dims=4, scaling=dict(factor=4.0, fast=32.0, original=64, slow=1.0))))
    att = dict(type="attention", mixer=dict(diff=0.5, dim=8, heads=4, kv_heads=2, vdim=12, scale=0.35, mask=dict(size=5)),
               mlp=dict(kind="moe", expert=dict(ff=16), router=dict(experts=4, identity=1, top=2), shared=dict(ff=24)))
    mls = dict(type="mlstm", mixer=dict(dim=8, gate_cap=15.0, heads=2, vdim=12), mlp=None)
    return config_from_dict(dict(layers=[att, mls, lat], loop=dict(start=0, stop=2, times=2), norm=dict(eps=1e-5), vocab=96, width=32))


register_hf_family(
    "defilorn", "Defilorn", lambda hf, is_critic=False: config_from_dict(hf if isinstance(hf, dict) else hf.to_dict(), is_critic),
    config_to_dict, _sd_from_ckpt, _sd_to_ckpt, lambda cfg: ["embed"], _block_names, lambda cfg: ["head"],
    make_test_config=make_test_config, config_from_dict=config_from_dict, config_to_dict=config_to_dict, weight_file="model.safetensors")
