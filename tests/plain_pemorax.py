"""The Pemorax architecture restated from its equations: float64, no paging, no slots, no kernels, one function
per mechanism.  It shares no code with the engine; the tests hold the engine against it.

Notation: ``x`` the stream ``[T, D]``, weights ``[out, in]`` applied as ``W v``, ``N(v) = v / sqrt(mean(v^2) +
eps)`` over the last axis, positions from 0.  Functions that carry something from one portion of a sequence to
the next take and return it (``tail``, ``state``), so the tests can also cut a sequence and hand it over.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def unit_rms(v, eps):
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def rms_norm(v, w, eps):
    return unit_rms(v, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def short_conv(u, w, tail=None):
    """y_t = sum_j w[:, j] u_(t - taps + 1 + j) per channel; ``u [T, C]``, ``w [C, taps]``; ``tail`` = the taps-1
    rows ahead of u (all 0 when u opens a sequence).  Returns (y, the new tail)."""
    taps = w.shape[1]
    if tail is None:
        tail = torch.zeros((taps - 1, u.shape[1]), dtype=u.dtype)
    ext = torch.cat([tail, u])
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + w[:, j] * ext[j:j + u.shape[0]]
    return y, ext[ext.shape[0] - (taps - 1):]


def frequencies(rot):
    """(f_i for i < dims/2, the factor on cos and sin) with the frequency scaling if the layer has one."""
    dims, base = rot["dims"], rot["base"]
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    where = lambda t: dims * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo, hi = max(math.floor(where(sc["fast"])), 0), min(math.ceil(where(sc["slow"])), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / sc["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def rotate(x, positions, rot, interleaved):
    """x ``[T, heads, dim]``: the first rot.dims dimensions of every head turn by position * f_i, pairs
    (2i, 2i+1) when interleaved, else (i, i + dims/2)."""
    if not rot or not rot.get("dims"):
        return x
    dims = rot["dims"]
    f, mag = frequencies(rot)
    ang = positions.to(F64)[:, None] * f[None, :]
    c, s = (torch.cos(ang) * mag)[:, None, :], (torch.sin(ang) * mag)[:, None, :]
    out = x.clone()
    if interleaved:
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2], out[..., 1:dims:2] = a * c - b * s, b * c + a * s
    else:
        a, b = x[..., :dims // 2], x[..., dims // 2:dims]
        out[..., :dims // 2], out[..., dims // 2:dims] = a * c - b * s, b * c + a * s
    return out


def visible(n_queries, first_position, mask):
    """[queries, keys] booleans: key j for the query at p iff j <= p and (p - j < size or j < keep_first)."""
    p = torch.arange(first_position, first_position + n_queries)[:, None]
    j = torch.arange(first_position + n_queries)[None, :]
    see = j <= p
    if mask:
        see = see & ((p - j < mask["size"]) | (j < mask.get("keep_first", 0)))
    return see


def sink_attention(q, k, v, m, first_position=0):
    """q ``[Tq, H, dim]`` (the last Tq positions), k ``[T, G, dim]``, v ``[T, G, vdim]`` -> ``[Tq, H * vdim]``:
    scores scaled, capped, masked; weights exp(s_j) / (1 + sum exp(s))."""
    heads, groups = q.shape[1], k.shape[1]
    see = visible(q.shape[0], first_position, m.get("mask"))
    out = []
    for h in range(heads):
        g = h // (heads // groups)
        s = (q[:, h] @ k[:, g].T) * m["scale"]
        if m.get("softcap"):
            s = m["softcap"] * torch.tanh(s / m["softcap"])
        e = torch.where(see, torch.exp(s), torch.zeros_like(s))
        out.append((e / (1.0 + e.sum(-1, keepdim=True))) @ v[:, g])
    return torch.cat(out, dim=-1)


def left_mixer(h, w, p, m):
    """The attention branch over a whole sequence ``h [T, D]``."""
    t = h.shape[0]
    pos = torch.arange(t)
    proj = {}
    for x in ("q", "k", "v"):
        u = h @ w[f"{p}.{x}"].T
        proj[x] = short_conv(u, w[f"{p}.{x}.conv"])[0] if m.get("conv", 0) >= 1 else u
    q = rotate(proj["q"].view(t, m["heads"], m["dim"]), pos, m.get("rot"), True)
    k = rotate(proj["k"].view(t, m["kv_heads"], m["dim"]), pos, m.get("rot"), True)
    v = proj["v"].view(t, m["kv_heads"], m["vdim"])
    o = sink_attention(q, k, v, m) * torch.sigmoid(h @ w[f"{p}.g"].T)
    return o @ w[f"{p}.o"].T


def retention_scan(q, k, v, decay, state=None):
    """q, k ``[T, H, dim]``, v ``[T, H, vdim]``: S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.  Returns
    (o ``[T, H, vdim]``, the last state ``[H, dim, vdim]``)."""
    t, heads, dim = q.shape
    s = torch.zeros((heads, dim, v.shape[2]), dtype=q.dtype) if state is None else state.clone()
    g = torch.tensor(decay, dtype=q.dtype)[:, None, None]
    out = []
    for i in range(t):
        s = g * s + k[i][:, :, None] * v[i][:, None, :]
        out.append(torch.einsum("hdv,hd->hv", s, q[i]))
    return torch.stack(out), s


def right_mixer(h, w, p, m, eps):
    """The retention branch over a whole sequence."""
    t = h.shape[0]
    pos = torch.arange(t)
    q = rotate((h @ w[f"{p}.q"].T).view(t, m["heads"], m["dim"]), pos, m.get("rot"), False)
    k = rotate((h @ w[f"{p}.k"].T).view(t, m["heads"], m["dim"]), pos, m.get("rot"), False) * m["dim"] ** -0.5
    v = (h @ w[f"{p}.v"].T).view(t, m["heads"], m["vdim"])
    o, _ = retention_scan(q, k, v, m["decay"])
    o = unit_rms(o, eps).reshape(t, -1) * silu(h @ w[f"{p}.g"].T)
    return o @ w[f"{p}.o"].T


def side_by_side(h, w, p, mixer, eps):
    a = rms_norm(left_mixer(h, w, f"{p}.left", fill_left(mixer["left"])), w[f"{p}.left.out"], eps)
    b = rms_norm(right_mixer(h, w, f"{p}.right", fill_right(mixer["right"]), eps), w[f"{p}.right.out"], eps)
    return 0.5 * (a + b)


def dense_ff(h, w, p):
    return gelu_tanh(h @ w[f"{p}.up"].T) @ w[f"{p}.down"].T


def route(z, top):
    """The ``top`` largest logits of every row (lowest index first among equals) and the softmax over them alone."""
    order = torch.sort(z, dim=-1, descending=True, stable=True).indices[:, :top]
    return order, torch.softmax(torch.gather(z, 1, order), dim=-1)


def routed_ff(h, w, p, mlp):
    z = h @ w[f"{p}.router"].T + w[f"{p}.router.b"]
    chosen, weight = route(z, mlp["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c, wt in zip(chosen[t].tolist(), weight[t]):
            e = f"{p}.e{c}"
            out[t] += wt * (w[f"{e}.down"] @ (silu(w[f"{e}.gate"] @ h[t]) * (w[f"{e}.up"] @ h[t])))
    return out


def fill_left(m):
    """The defaults a configuration may leave out."""
    m = dict(m)
    m.setdefault("kv_heads", m["heads"]), m.setdefault("vdim", m["dim"])
    if m.get("scale") is None:
        m["scale"] = m["dim"] ** -0.5
    return m


def fill_right(m):
    m = dict(m)
    m.setdefault("vdim", m["dim"])
    return m


def forward(cfg, w, tokens, layers_out=None):
    """Logits ``[T, vocab]`` of a whole sequence; ``layers_out`` (a list) takes the stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        x = x + rms_norm(side_by_side(rms_norm(x, w[f"{p}.norm1"], eps), w, f"{p}.mix", layer["mixer"], eps), w[f"{p}.norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms_norm(x, w[f"{p}.norm2"], eps)
            y = dense_ff(h, w, f"{p}.mlp") if mlp["kind"] == "dense" else routed_ff(h, w, f"{p}.mlp", mlp)
            x = x + rms_norm(y, w[f"{p}.norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T
