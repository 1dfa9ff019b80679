"""Zobasun: a decoder-only stack that mixes latent-attention layers (some of which read an earlier layer's cache) with
gated-linear-recurrence layers, post-normalised, with an optional clamped gated feed-forward per layer.

``config.json``:
  architecture, vocab, width, embedding.scale, norm.eps,
  layers[i] = {type: "latent_attention" | "rglru", mixer: {...}, mlp: null | {kind: "dense", ff, limit}}
    latent_attention mixer: heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot: {base, dims}, optional kv_from
    rglru mixer:            width, blocks, conv
Tensors (``model.safetensors``, linear weights [out, in]): embed, head, final.norm, and per layer ``l<i>.``:
  norm1, norm2, mix.{dq, dq.norm, uq, dkv, dkv.norm, uk, uv, o} or mix.{y, y.b, x, x.b, conv, conv.b, ra, ra.b, ri, ri.b, lam, o},
  mlp.{gate, up, down}.
This file only maps those names and keys onto the mechanisms of ``layers``; it holds no arithmetic."""
from __future__ import annotations

import os

import torch

from ..checkpoint import read_safetensors
from ..layers import ClampedGatedMLP, GatedLinearRecurrence, LatentAttention, LayerStackModel
from . import register_model

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def build_zobasun(config: dict, tensors: dict, dtype=torch.bfloat16, device="cuda") -> LayerStackModel:
    """``tensors``: name -> CPU tensor as stored.  Everything is moved to ``device`` in ``dtype`` once, here."""
    dtype = _DTYPES[dtype]

    def t(name):
        try:
            return tensors[name].to(device=device, dtype=dtype).contiguous()
        except KeyError:
            raise KeyError(f"checkpoint has no tensor {name!r}") from None

    eps = float(config["norm"]["eps"])
    layers = []
    for i, lc in enumerate(config["layers"]):
        p, m = f"l{i}.", lc["mixer"]
        if lc["type"] == "latent_attention":
            own = "kv_from" not in m
            if not own:
                src = config["layers"][m["kv_from"]]["mixer"]
                if (src.get("kv_rank"), src.get("rot_dim"), src.get("rot")) != (m["kv_rank"], m["rot_dim"], m["rot"]) \
                        or "kv_from" in src:
                    raise ValueError(f"layer {i}: kv_from must name a layer with its own, equally shaped latent cache")
            mixer = LatentAttention(
                i, heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"], vdim=m["vdim"], lat=m["kv_rank"],
                rot_dims=m["rot"]["dims"], rot_base=m["rot"]["base"], scale=m["scale"], eps=eps,
                w_dq=t(p + "mix.dq"), w_dq_norm=t(p + "mix.dq.norm"), w_uq=t(p + "mix.uq"), w_uk=t(p + "mix.uk"),
                w_uv=t(p + "mix.uv"), w_o=t(p + "mix.o"), w_dkv=t(p + "mix.dkv") if own else None,
                w_dkv_norm=t(p + "mix.dkv.norm") if own else None, kv_source=None if own else int(m["kv_from"]))
        elif lc["type"] == "rglru":
            mixer = GatedLinearRecurrence(
                i, channels=m["width"], blocks=m["blocks"], taps=m["conv"], w_y=t(p + "mix.y"), b_y=t(p + "mix.y.b"),
                w_x=t(p + "mix.x"), b_x=t(p + "mix.x.b"), conv_w=t(p + "mix.conv"), conv_b=t(p + "mix.conv.b"),
                w_ra=t(p + "mix.ra"), b_ra=t(p + "mix.ra.b"), w_ri=t(p + "mix.ri"), b_ri=t(p + "mix.ri.b"),
                lam=t(p + "mix.lam"), w_o=t(p + "mix.o"))
        else:
            raise ValueError(f"layer {i}: unknown mixer type {lc['type']!r}")
        mlp = None
        if lc.get("mlp") is not None:
            f = lc["mlp"]
            if f.get("kind", "dense") != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {f['kind']!r}")
            mlp = ClampedGatedMLP(w_gate=t(p + "mlp.gate"), w_up=t(p + "mlp.up"), w_down=t(p + "mlp.down"), limit=f["limit"])
        layers.append({"mixer": mixer, "post1": t(p + "norm1"), "mlp": mlp, "post2": t(p + "norm2") if mlp else None})
    return LayerStackModel(vocab=int(config["vocab"]), width=int(config["width"]), dtype=dtype, embed=t("embed"),
                           embed_scale=config["embedding"]["scale"], layers=layers, final_norm=t("final.norm"),
                           head=t("head"), eps=eps, norm_offset=1.0)


@register_model("Zobasun")
def _load(model_dir, config, dtype="bfloat16", device="cuda", **_):
    return build_zobasun(config, read_safetensors(os.path.join(model_dir, "model.safetensors")), dtype, device)
