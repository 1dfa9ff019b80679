"""Plain float64 restatement of the sequence mixers served in-flight (latent attention, gated linear recurrence,
clamped gated feed-forward, post-normalised layer stack), written from the equations and sharing no code with the
product path.  Slow on purpose: whole sequences at once, explicit loops over time, per-head keys and values
materialised, no cache, no state carried between calls.  Test infrastructure only.

Notation: h [T, W] is the residual stream of one sequence, positions 0..T-1; weights are [out, in] and applied as W x."""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_norm(x, w=None, eps=1e-6, offset=0.0):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * (w + offset)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_pairs(v, positions, base, dims):
    """v [T, ..., d]: pairs (2i, 2i+1), i < dims/2, turned by positions * base^(-2i/dims); the rest untouched."""
    out = v.clone()
    for i in range(dims // 2):
        ang = positions.to(F64) * (float(base) ** (-2.0 * i / dims))
        shape = [-1] + [1] * (v.dim() - 2)
        c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
        a, b = v[..., 2 * i], v[..., 2 * i + 1]
        out[..., 2 * i] = a * c - b * s
        out[..., 2 * i + 1] = b * c + a * s
    return out


def latent_cache_entries(h, w_dkv, w_norm, lat, rot_dims, rot_base, eps):
    """-> (c [T, lat] normalised latent, k_rot [T, rot_dim] rotated shared key part)."""
    kv = h @ w_dkv.T
    pos = torch.arange(h.shape[0])
    return rms_norm(kv[:, :lat], w_norm, eps), rotate_pairs(kv[:, lat:], pos, rot_base, rot_dims)


def latent_attention(h, c, k_rot, *, heads, dim, rot_dim, vdim, rot_dims, rot_base, scale, eps, w_dq, w_dq_norm, w_uq, w_uk,
                     w_uv, w_o):
    """Causal attention of h's queries over the per-head keys / values made from (c, k_rot)."""
    T = h.shape[0]
    pos = torch.arange(T)
    q = (rms_norm(h @ w_dq.T, w_dq_norm, eps) @ w_uq.T).view(T, heads, dim + rot_dim)
    q_rot = rotate_pairs(q[..., dim:], pos, rot_base, rot_dims)
    k = (c @ w_uk.T).view(T, heads, dim)
    v = (c @ w_uv.T).view(T, heads, vdim)
    out = torch.zeros(T, heads, vdim, dtype=F64)
    for hd in range(heads):
        for i in range(T):          # position i sees 0..i
            s = (k[: i + 1, hd] @ q[i, hd, :dim] + k_rot[: i + 1] @ q_rot[i, hd]) * scale
            p = torch.softmax(s, 0)
            out[i, hd] = p @ v[: i + 1, hd]
    return out.reshape(T, heads * vdim) @ w_o.T


def causal_conv(x, w, b):
    """x [T, C], w [C, taps] (last column = current position), zeros before the start."""
    T, taps = x.shape[0], w.shape[1]
    out = torch.zeros_like(x)
    for t in range(T):
        for k in range(taps):
            src = t - (taps - 1 - k)
            if src >= 0:
                out[t] += w[:, k] * x[src]
        out[t] += b
    return out


def gated_linear_recurrence(h, *, channels, blocks, w_y, b_y, w_x, b_x, conv_w, conv_b, w_ra, b_ra, w_ri, b_ri, lam, w_o,
                            decay_scale=8.0):
    T, bw = h.shape[0], channels // blocks
    y = gelu_tanh(h @ w_y.T + b_y)
    u = causal_conv(h @ w_x.T + b_x, conv_w, conv_b)
    S = torch.zeros(channels, dtype=F64)
    out = torch.zeros(T, channels, dtype=F64)
    for t in range(T):
        r = torch.cat([torch.sigmoid(w_ra[b] @ u[t, b * bw:(b + 1) * bw] + b_ra[b]) for b in range(blocks)])
        i = torch.cat([torch.sigmoid(w_ri[b] @ u[t, b * bw:(b + 1) * bw] + b_ri[b]) for b in range(blocks)])
        a = torch.exp(-decay_scale * r * torch.log1p(torch.exp(lam)))
        S = a * S + torch.sqrt(1.0 - a * a) * i * u[t]
        out[t] = S * y[t]
    return out @ w_o.T


def clamped_gated_mlp(h, w_gate, w_up, w_down, limit, alpha=1.702, up_shift=1.0):
    g = torch.clamp(h @ w_gate.T, max=limit)
    u = torch.clamp(h @ w_up.T, -limit, limit)
    return (g * torch.sigmoid(alpha * g) * (u + up_shift)) @ w_down.T


def zobasun_forward(config, tensors, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence run whole.  ``tensors``: name -> tensor (any float type; used in float64)."""
    W = {k: v.to(F64) for k, v in tensors.items()}
    eps = config["norm"]["eps"]
    x = W["embed"][torch.tensor(list(tokens))] * config["embedding"]["scale"]
    caches, per_layer = {}, []
    for i, lc in enumerate(config["layers"]):
        p, m = f"l{i}.", lc["mixer"]
        if lc["type"] == "latent_attention":
            if "kv_from" in m:
                c, k_rot = caches[m["kv_from"]]
            else:
                c, k_rot = caches[i] = latent_cache_entries(x, W[p + "mix.dkv"], W[p + "mix.dkv.norm"], m["kv_rank"],
                                                            m["rot"]["dims"], m["rot"]["base"], eps)
            o = latent_attention(x, c, k_rot, heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"], vdim=m["vdim"],
                                 rot_dims=m["rot"]["dims"], rot_base=m["rot"]["base"], scale=m["scale"], eps=eps,
                                 w_dq=W[p + "mix.dq"], w_dq_norm=W[p + "mix.dq.norm"], w_uq=W[p + "mix.uq"],
                                 w_uk=W[p + "mix.uk"], w_uv=W[p + "mix.uv"], w_o=W[p + "mix.o"])
        else:
            o = gated_linear_recurrence(x, channels=m["width"], blocks=m["blocks"], w_y=W[p + "mix.y"], b_y=W[p + "mix.y.b"],
                                        w_x=W[p + "mix.x"], b_x=W[p + "mix.x.b"], conv_w=W[p + "mix.conv"],
                                        conv_b=W[p + "mix.conv.b"], w_ra=W[p + "mix.ra"], b_ra=W[p + "mix.ra.b"],
                                        w_ri=W[p + "mix.ri"], b_ri=W[p + "mix.ri.b"], lam=W[p + "mix.lam"], w_o=W[p + "mix.o"])
        x = x + rms_norm(o, W[p + "norm1"], eps, 1.0)
        if lc.get("mlp") is not None:
            f = clamped_gated_mlp(x, W[p + "mlp.gate"], W[p + "mlp.up"], W[p + "mlp.down"], lc["mlp"]["limit"])
            x = x + rms_norm(f, W[p + "norm2"], eps, 1.0)
        per_layer.append(x.clone())
    logits = rms_norm(x, W["final.norm"], eps, 1.0) @ W["head"].T
    return (logits, per_layer) if return_layers else logits


def random_zobasun(layers, *, width=48, vocab=61, embed_scale=3.0, eps=1e-5, seed=0, dtype=torch.bfloat16):
    """A small random model.  ``layers``: list of dicts, each {"type": "latent_attention", heads, dim, rot_dim, vdim, kv_rank,
    q_rank, [kv_from], [rot_base], [scale], mlp: None | (ff, limit)} or {"type": "rglru", width, blocks, conv, mlp: ...}.
    Returns (config, tensors) in the checkpoint's naming; values are rounded to ``dtype`` so that product and oracle
    start from the same numbers."""
    g = torch.Generator().manual_seed(seed)

    def n(*shape, std=None, mean=0.0):
        std = std if std is not None else shape[-1] ** -0.5
        return (torch.randn(*shape, generator=g) * std + mean).to(dtype)

    cfg_layers, t = [], {"embed": n(vocab, width, std=1.0), "head": n(vocab, width), "final.norm": n(width, std=0.2)}
    for i, l in enumerate(layers):
        p = f"l{i}."
        mlp = None if l.get("mlp") is None else {"kind": "dense", "ff": l["mlp"][0], "limit": l["mlp"][1]}
        t[p + "norm1"] = n(width, std=0.2)
        if l["type"] == "latent_attention":
            H, dn, dr, dv, R, Q = l["heads"], l["dim"], l["rot_dim"], l["vdim"], l["kv_rank"], l["q_rank"]
            m = {"heads": H, "dim": dn, "rot_dim": dr, "vdim": dv, "kv_rank": R, "q_rank": Q,
                 "scale": l.get("scale", (dn + dr) ** -0.5), "rot": {"base": l.get("rot_base", 10000.0), "dims": dr}}
            t.update({p + "mix.dq": n(Q, width), p + "mix.dq.norm": n(Q, std=0.2, mean=1.0), p + "mix.uq": n(H * (dn + dr), Q),
                      p + "mix.uk": n(H * dn, R), p + "mix.uv": n(H * dv, R), p + "mix.o": n(width, H * dv)})
            if "kv_from" in l:
                m["kv_from"] = l["kv_from"]
            else:
                t.update({p + "mix.dkv": n(R + dr, width), p + "mix.dkv.norm": n(R, std=0.2, mean=1.0)})
        else:
            C, nb, taps = l["width"], l["blocks"], l["conv"]
            m = {"width": C, "blocks": nb, "conv": taps}
            bw = C // nb
            t.update({p + "mix.y": n(C, width), p + "mix.y.b": n(C, std=0.2), p + "mix.x": n(C, width),
                      p + "mix.x.b": n(C, std=0.2), p + "mix.conv": n(C, taps, std=0.5), p + "mix.conv.b": n(C, std=0.2),
                      p + "mix.ra": n(nb, bw, bw), p + "mix.ra.b": n(nb, bw, std=0.3), p + "mix.ri": n(nb, bw, bw),
                      p + "mix.ri.b": n(nb, bw, std=0.3), p + "mix.lam": n(C, std=1.5, mean=-1.0), p + "mix.o": n(width, C)})
        if mlp is not None:
            t.update({p + "norm2": n(width, std=0.2), p + "mlp.gate": n(mlp["ff"], width, std=2.0 * width ** -0.5),
                      p + "mlp.up": n(mlp["ff"], width, std=2.0 * width ** -0.5), p + "mlp.down": n(width, mlp["ff"])})
        cfg_layers.append({"type": l["type"], "mixer": m, "mlp": mlp})
    config = {"architecture": "Zobasun", "vocab": vocab, "width": width, "embedding": {"scale": embed_scale},
              "norm": {"eps": eps}, "layers": cfg_layers}
    return config, t
