"""Nililix: a decoder-only stack of windowed grouped-query attention layers (short convolutions on q, k and v, partial
interleaved rotation with scaled frequencies, a softmax sink and an output gate per head), each followed by a squared-ReLU
or a routed-expert feed-forward, with a norm before and after every sublayer, a residual multiplier, a block of layers
that is run several times with a step vector per pass, and soft-capped logits.

``config.json``:
  architecture, vocab, width, norm.eps, residual_mult, logit_softcap, loop: {start, stop, times},
  layers[i] = {type: "attention", mixer: {...}, mlp: null | {kind: "dense", ff} | {kind: "moe", expert: {ff}, router: {...}}}
    mixer:  heads, kv_heads, dim, vdim, conv (taps), scale, mask: {size}, rot: {base, dims, scaling: {factor, low, high, original}}
    router: experts, top, groups: {count, keep}
Tensors (``model.safetensors``, linear weights [out, in]): embed, head, final.norm, loop.step [times, width], and per layer
``l<i>.``: norm1, norm1b, norm2, norm2b, mix.{q, k, v, q.conv, k.conv, v.conv, sink, g, o}, and mlp.{up, down} or
mlp.{router, correction, e<j>.gate, e<j>.up, e<j>.down}.
This file only maps those names and keys onto the mechanisms of ``layers``; it holds no arithmetic."""
from __future__ import annotations

import os

import torch

from ..checkpoint import read_safetensors
from ..layers import LayerStackModel, RoutedExpertsMLP, SquaredReluMLP, WindowedAttention
from . import register_model

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def build_nililix(config: dict, tensors: dict, dtype=torch.bfloat16, device="cuda") -> LayerStackModel:
    """``tensors``: name -> CPU tensor as stored.  Everything is moved to ``device`` in ``dtype`` once, here."""
    dtype = _DTYPES[dtype]

    def t(name, optional=False):
        if name not in tensors:
            if optional:
                return None
            raise KeyError(f"checkpoint has no tensor {name!r}")
        return tensors[name].to(device=device, dtype=dtype).contiguous()

    layers = []
    for i, lc in enumerate(config["layers"]):
        p, m = f"l{i}.", lc["mixer"]
        if lc["type"] != "attention":
            raise ValueError(f"layer {i}: unknown mixer type {lc['type']!r}")
        rot = m.get("rot") or {}
        sc = rot.get("scaling")
        mixer = WindowedAttention(
            i, heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]),
            vdim=int(m.get("vdim", m["dim"])), taps=int(m.get("conv", 1)), scale=m["scale"],
            window=int((m.get("mask") or {}).get("size", 0)), rot_dims=int(rot.get("dims", 0)), rot_base=rot.get("base", 10000.0),
            rot_scaling=(sc["factor"], sc["low"], sc["high"], sc["original"]) if sc else None,
            w_q=t(p + "mix.q"), w_k=t(p + "mix.k"), w_v=t(p + "mix.v"), conv_q=t(p + "mix.q.conv"), conv_k=t(p + "mix.k.conv"),
            conv_v=t(p + "mix.v.conv"), w_o=t(p + "mix.o"), sink=t(p + "mix.sink", optional=True), w_g=t(p + "mix.g", optional=True))
        mlp, f = None, lc.get("mlp")
        if f is not None:
            kind = f.get("kind", "dense")
            if kind == "dense":
                mlp = SquaredReluMLP(w_up=t(p + "mlp.up"), w_down=t(p + "mlp.down"))
            elif kind == "moe":
                r = f["router"]
                gr = r.get("groups") or {}
                ex = range(int(r["experts"]))
                mlp = RoutedExpertsMLP(
                    w_router=t(p + "mlp.router"), correction=t(p + "mlp.correction", optional=True),
                    w_gate=torch.stack([t(f"{p}mlp.e{j}.gate") for j in ex]), w_up=torch.stack([t(f"{p}mlp.e{j}.up") for j in ex]),
                    w_down=torch.stack([t(f"{p}mlp.e{j}.down") for j in ex]), top=r["top"], groups=gr.get("count", 1),
                    keep=gr.get("keep", gr.get("count", 1)))
            else:
                raise ValueError(f"layer {i}: unknown feed-forward kind {kind!r}")
        layers.append({"mixer": mixer, "pre1": t(p + "norm1"), "post1": t(p + "norm1b"), "mlp": mlp,
                       "pre2": t(p + "norm2") if mlp else None, "post2": t(p + "norm2b") if mlp else None})
    lp = config.get("loop")
    looped = bool(lp) and lp["stop"] > lp["start"]
    return LayerStackModel(vocab=int(config["vocab"]), width=int(config["width"]), dtype=dtype, embed=t("embed"), layers=layers,
                           final_norm=t("final.norm"), head=t("head"), eps=float(config["norm"]["eps"]),
                           residual_mult=config.get("residual_mult", 1.0),
                           loop=(lp["start"], lp["stop"], lp.get("times", 1)) if looped else None,
                           loop_step=t("loop.step", optional=True) if looped else None,
                           logit_cap=config.get("logit_softcap") or 0.0)


@register_model("Nililix")
def _load(model_dir, config, dtype="bfloat16", device="cuda", **_):
    return build_nililix(config, read_safetensors(os.path.join(model_dir, "model.safetensors")), dtype, device)
