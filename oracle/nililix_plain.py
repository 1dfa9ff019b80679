"""Plain float64 restatement of the Nililix design (windowed grouped-query attention with short convolutions, a
softmax sink and per-head output gates; squared-ReLU and routed-expert feed-forwards; sandwich-normalised layers; a
looped block of layers), written from the equations and sharing no code with the product path.  Slow on purpose: whole
sequences at once, explicit loops over positions and heads, no cache, nothing carried between calls.  Test
infrastructure only.

Notation: h [T, W] is one sequence, positions 0..T-1; ``P`` maps tensor names ('l3.mix.q', ...) to float64 tensors;
linear weights are [out, in] and applied as W x; ``cfg`` is the parsed configuration."""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def short_conv(u, w):
    """u [T, C], w [C, taps]: tap j weighs the input ``taps - 1 - j`` positions back (the last tap the current one); inputs
    before position 0 are zero."""
    T, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            back = taps - 1 - j
            if t - back >= 0:
                y[t] += w[:, j] * u[t - back]
    return y


def rotary_frequencies(dims, base, scaling=None):
    """f_i = base^(-2i/dims); with ``scaling`` long wavelengths are slowed by ``factor``, short ones kept, and the
    band between original/low and original/high is blended linearly in original/wavelength."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling:
            factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wavelength = 2.0 * math.pi / f
            if wavelength < orig / high:
                pass
            elif wavelength > orig / low:
                f = f / factor
            else:
                keep = (orig / wavelength - low) / (high - low)       # 0 at the slow end of the band, 1 at the fast end
                f = f * (keep + (1.0 - keep) / factor)
        out.append(f)
    return out


def rotate_interleaved(v, freqs):
    """v [T, heads, d]: the pair (2i, 2i+1) at position p is turned by p * freqs[i]; dimensions past 2 len(freqs) pass."""
    out = v.clone()
    for p in range(v.shape[0]):
        for i, f in enumerate(freqs):
            c, s = math.cos(p * f), math.sin(p * f)
            a, b = v[p, :, 2 * i].clone(), v[p, :, 2 * i + 1].clone()
            out[p, :, 2 * i] = a * c - b * s
            out[p, :, 2 * i + 1] = b * c + a * s
    return out


def windowed_sink_attention(q, k, v, scale, window, sink):
    """q [T, H, d], k [T, G, d], v [T, G, dv], sink [H] or None.  Position i sees j with 0 <= i - j < window; the softmax
    denominator holds one more term exp(sink_h) that carries no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        for i in range(T):
            lo = max(0, i - window + 1) if window else 0
            s = (k[lo:i + 1, g] @ q[i, hd]) * scale
            sk = -math.inf if sink is None else float(sink[hd])
            m = max(float(s.max()), sk)
            e = torch.exp(s - m)
            out[i, hd] = (e @ v[lo:i + 1, g]) / (e.sum() + math.exp(sk - m))
    return out


def attention_mixer(h, P, pre, mc):
    T = h.shape[0]
    H, G, d, dv = mc["heads"], mc["kv_heads"], mc["dim"], mc["vdim"]
    q = short_conv(h @ P[pre + "q"].T, P[pre + "q.conv"]).view(T, H, d)
    k = short_conv(h @ P[pre + "k"].T, P[pre + "k.conv"]).view(T, G, d)
    v = short_conv(h @ P[pre + "v"].T, P[pre + "v.conv"]).view(T, G, dv)
    rot = mc.get("rot")
    if rot:
        fr = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        q, k = rotate_interleaved(q, fr), rotate_interleaved(k, fr)
    window = (mc.get("mask") or {}).get("size", 0)
    o = windowed_sink_attention(q, k, v, mc["scale"], window, P.get(pre + "sink"))
    if pre + "g" in P:
        o = o * torch.sigmoid(h @ P[pre + "g"].T)[:, :, None]       # one gate per token and head
    return o.reshape(T, H * dv) @ P[pre + "o"].T


def relu2_mlp(h, P, pre):
    return torch.relu(h @ P[pre + "up"].T) ** 2 @ P[pre + "down"].T


def route(h, P, pre, rc):
    """-> per token (expert ids, weights).  Choice = sigmoid(logit) + correction, restricted to the groups whose two
    best choices sum highest; the weights are the plain sigmoids of the chosen experts."""
    E, top = rc["experts"], rc["top"]
    gr = rc.get("groups") or {"count": 1, "keep": 1}
    s = torch.sigmoid(h @ P[pre + "router"].T)
    choice = s + P[pre + "correction"]
    per = E // gr["count"]
    picks = []
    for t in range(h.shape[0]):
        c = choice[t].clone()
        gscore = [float(torch.sort(c[g * per:(g + 1) * per], descending=True).values[:2].sum()) for g in range(gr["count"])]
        kept = sorted(range(gr["count"]), key=lambda g: (-gscore[g], g))[:gr["keep"]]
        for g in range(gr["count"]):
            if g not in kept:
                c[g * per:(g + 1) * per] = -math.inf
        ids = sorted(range(E), key=lambda e: (-float(c[e]), e))[:top]
        picks.append((ids, [float(s[t, e]) for e in ids]))
    return picks


def moe_mlp(h, P, pre, fc):
    out = torch.zeros_like(h)
    for t, (ids, ws) in enumerate(route(h, P, pre, fc["router"])):
        for e, w in zip(ids, ws):
            a = P[f"{pre}e{e}.gate"] @ h[t]
            y = P[f"{pre}e{e}.down"] @ (a * torch.sigmoid(a) * (P[f"{pre}e{e}.up"] @ h[t]))
            out[t] += w * y
    return out


def layer(x, P, i, lc, cfg):
    m, eps, pre = cfg["residual_mult"], cfg["norm"]["eps"], f"l{i}."
    if lc["type"] != "attention":
        raise ValueError(lc["type"])
    x = x + m * rms_norm(attention_mixer(rms_norm(x, P[pre + "norm1"], eps), P, pre + "mix.", lc["mixer"]), P[pre + "norm1b"], eps)
    fc = lc.get("mlp")
    if fc:
        hin = rms_norm(x, P[pre + "norm2"], eps)
        f = relu2_mlp(hin, P, pre + "mlp.") if fc["kind"] == "dense" else moe_mlp(hin, P, pre + "mlp.", fc)
        x = x + m * rms_norm(f, P[pre + "norm2b"], eps)
    return x


def layer_runs(cfg):
    """[(layer index, pass number, first of its pass)] in execution order."""
    n, lp = len(cfg["layers"]), cfg.get("loop")
    if not lp or lp["stop"] <= lp["start"]:
        return [(i, 0, False) for i in range(n)]
    runs = [(i, 0, False) for i in range(lp["start"])]
    for t in range(lp["times"]):
        runs += [(i, t, i == lp["start"]) for i in range(lp["start"], lp["stop"])]
    return runs + [(i, 0, False) for i in range(lp["stop"], n)]


def forward(tokens, P, cfg, trace=None):
    """-> logits [T, vocab]; ``trace`` (a list) receives the residual stream after every layer run."""
    x = P["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, t, first in layer_runs(cfg):
        if first:
            x = x + P["loop.step"][t]
        x = layer(x, P, i, cfg["layers"][i], cfg)
        if trace is not None:
            trace.append(x.clone())
    z = rms_norm(x, P["final.norm"], cfg["norm"]["eps"]) @ P["head"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(z / cap) if cap else z


def random_nililix(layers, *, width=48, vocab=61, eps=1e-5, residual_mult=0.8, logit_softcap=20.0, loop=None, seed=0,
                   dtype=torch.bfloat16, spaced_corrections=False):
    """A small random model.  ``layers``: list of dicts {heads, kv_heads, dim, vdim, conv, [window], [rot_dims], [rot_base],
    [scaling], [scale], [sink], [gate], mlp: None | ("dense", ff) | ("moe", ff, experts, top, groups, keep)}.  ``loop`` =
    (start, stop, times).  Returns (config, tensors) in the checkpoint's naming; values are rounded to ``dtype`` so that
    product and oracle start from the same numbers.

    ``spaced_corrections``: the routers' corrections are 2.5 * 2^k in shuffled order instead of random numbers of the
    scores' size, so that neither an expert's nor a group's rank can hang on a score (every sum of two corrections differs
    from every other by more than two scores can): the choice is then the same for every token, and a run in reduced
    precision can be compared position by position without a close call deciding which experts ran."""
    g = torch.Generator().manual_seed(seed)

    def n(*shape, std=None, mean=0.0):
        std = std if std is not None else shape[-1] ** -0.5
        return (torch.randn(*shape, generator=g) * std + mean).to(dtype)

    cfg_layers, t = [], {"embed": n(vocab, width, std=1.0), "head": n(vocab, width, std=3.0 * width ** -0.5),
                         "final.norm": n(width, std=0.2, mean=1.0)}
    for i, l in enumerate(layers):
        p = f"l{i}."
        H, G, d, dv, taps = l["heads"], l["kv_heads"], l["dim"], l["vdim"], l["conv"]
        m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "conv": taps, "scale": l.get("scale", d ** -0.5)}
        if l.get("window"):
            m["mask"] = {"size": l["window"]}
        if l.get("rot_dims"):
            m["rot"] = {"base": l.get("rot_base", 10000.0), "dims": l["rot_dims"]}
            if l.get("scaling"):
                m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), l["scaling"]))
        for k in ("norm1", "norm1b"):
            t[p + k] = n(width, std=0.2, mean=1.0)
        t.update({p + "mix.q": n(H * d, width, std=2.0 * width ** -0.5), p + "mix.k": n(G * d, width, std=2.0 * width ** -0.5),
                  p + "mix.v": n(G * dv, width), p + "mix.q.conv": n(H * d, taps, std=0.6), p + "mix.k.conv": n(G * d, taps, std=0.6),
                  p + "mix.v.conv": n(G * dv, taps, std=0.6), p + "mix.o": n(width, H * dv)})
        if l.get("sink", True):
            t[p + "mix.sink"] = n(H, std=2.0)
        if l.get("gate", True):
            t[p + "mix.g"] = n(H, width, std=2.0 * width ** -0.5)
        mlp = None
        if l.get("mlp"):
            for k in ("norm2", "norm2b"):
                t[p + k] = n(width, std=0.2, mean=1.0)
            if l["mlp"][0] == "dense":
                ff = l["mlp"][1]
                mlp = {"kind": "dense", "ff": ff}
                t.update({p + "mlp.up": n(ff, width, std=2.0 * width ** -0.5), p + "mlp.down": n(width, ff)})
            else:
                _, ff, E, top, groups, keep = l["mlp"]
                mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": E, "top": top, "groups": {"count": groups, "keep": keep}}}
                # corrections of the size of the scores themselves, some negative: the choice differs from the plain top-k
                t.update({p + "mlp.router": n(E, width, std=3.0 * width ** -0.5), p + "mlp.correction": n(E, std=0.5, mean=-0.3)})
                if spaced_corrections:
                    t[p + "mlp.correction"] = (2.5 * 2.0 ** torch.randperm(E, generator=g).double()).to(dtype)
                for e in range(E):
                    t.update({f"{p}mlp.e{e}.gate": n(ff, width, std=2.0 * width ** -0.5),
                              f"{p}mlp.e{e}.up": n(ff, width, std=2.0 * width ** -0.5), f"{p}mlp.e{e}.down": n(width, ff)})
        cfg_layers.append({"type": "attention", "mixer": m, "mlp": mlp})
    config = {"architecture": "Nililix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": residual_mult,
              "logit_softcap": logit_softcap, "layers": cfg_layers}
    if loop:
        config["loop"] = dict(zip(("start", "stop", "times"), loop))
        t["loop.step"] = n(loop[2], width, std=0.5)
    return config, t


def nililix_forward(config, tensors, tokens, return_layers=False):
    """Logits [T, vocab] (float64) of one whole sequence; with ``return_layers`` also the residual stream after every
    layer run."""
    P = {k: v.to(F64) for k, v in tensors.items()}
    trace = []
    with torch.no_grad():
        z = forward(tokens, P, config, trace)
    return (z, trace) if return_layers else z
