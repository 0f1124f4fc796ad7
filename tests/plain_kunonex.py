"""A plain, slow restatement of the Kunonex design, one function per mechanism,
in whatever floating type its inputs have (the tests use float64).  It shares
no code with the engine: no paging, no state slots, no kernels; a whole
sequence goes in and every position's logits come out.

Notation: ``T`` tokens, ``D`` the model width, weights ``[out, in]`` applied
as ``x @ W.T``.  ``w`` maps tensor names to tensors, ``cfg`` is the parsed
config.json (a dict).
"""
from __future__ import annotations

import math

import torch


# ------------------------------------------------------------------- small pieces
def unit_rms(x, eps):
    """Every row divided by the root of (its mean square + eps)."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def layer_norm(x, weight, eps):
    """(x - mean) / sqrt(mean squared deviation + eps) * weight; no bias."""
    mu = x.mean(-1, keepdim=True)
    d = x - mu
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * weight


def sinusoid_positions(positions, width, dtype):
    """Entry 2i = sin(p * 10000^(-2i/width)), entry 2i+1 = cos of the same angle."""
    i = torch.arange(0, width, 2, dtype=torch.float64)
    angle = positions.to(torch.float64)[:, None] * torch.pow(torch.tensor(10000.0, dtype=torch.float64), -i / width)[None, :]
    out = torch.empty((positions.numel(), width), dtype=torch.float64)
    out[:, 0::2] = torch.sin(angle)[:, :out[:, 0::2].shape[1]]
    out[:, 1::2] = torch.cos(angle)[:, :out[:, 1::2].shape[1]]
    return out.to(dtype)


def embed(w, tokens, positions, eps):
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x = x + sinusoid_positions(positions, x.shape[1], x.dtype)
    return layer_norm(x, w["embed.norm"], eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def token_shift(h, mu, before=None):
    """h_t + (h_{t-1} - h_t) * mu, with ``before`` (zeros when None) ahead of the first row."""
    first = torch.zeros_like(h[:1]) if before is None else before.reshape(1, -1)
    prev = torch.cat([first, h[:-1]], 0)
    return h + (prev - h) * mu


# ------------------------------------------------------------------- feed-forward
def poly_norm(z, coeff, eps):
    """a N(z) + b N(z^2) + c N(z^3) + e, N = unit_rms over the row, powers element by element."""
    a, b, c, e = (coeff[i] for i in range(4))
    return a * unit_rms(z, eps) + b * unit_rms(z * z, eps) + c * unit_rms(z * z * z, eps) + e


def dense_ff(h, w, p, eps):
    z = h @ w[f"{p}.up"].T + w[f"{p}.up.b"]
    return poly_norm(z, w[f"{p}.act"], eps) @ w[f"{p}.down"].T + w[f"{p}.down.b"]


# ------------------------------------------------------------------- mixers
def mingru(h, w, p, state=None):
    """z = sigmoid(W_z h + b_z); u = W_x h + b_x; candidate = u + 1/2 (u >= 0) or sigmoid(u) (u < 0);
    S_t = (1 - z_t) S_{t-1} + z_t candidate_t; out_t = W_o (S_t * silu(W_g h_t)).  Returns (out, last S)."""
    z = torch.sigmoid(h @ w[f"{p}.z"].T + w[f"{p}.z.b"])
    u = h @ w[f"{p}.x"].T + w[f"{p}.x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    g = h @ w[f"{p}.g"].T
    s = torch.zeros_like(z[0]) if state is None else state
    rows = []
    for t in range(h.shape[0]):
        s = (1.0 - z[t]) * s + z[t] * cand[t]
        rows.append(s * (g[t] * torch.sigmoid(g[t])))
    return torch.stack(rows) @ w[f"{p}.o"].T, s


def latent_attention(h, w, p, m, eps):
    """Queries and keys/values through latents; causal softmax over all earlier positions; a sigmoid
    gate per head on the input.  ``m`` is the mixer's entry of the config."""
    t = h.shape[0]
    heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
    cq = unit_rms(h @ w[f"{p}.dq"].T, eps) * w[f"{p}.dq.norm"]
    q = (cq @ w[f"{p}.uq"].T).view(t, heads, dim)
    c = unit_rms(h @ w[f"{p}.dkv"].T, eps) * w[f"{p}.dkv.norm"]
    k = (c @ w[f"{p}.uk"].T).view(t, heads, dim)
    v = (c @ w[f"{p}.uv"].T).view(t, heads, vdim)
    s = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    hidden = torch.arange(t)[None, :] > torch.arange(t)[:, None]
    s = s.masked_fill(hidden[None], float("-inf"))
    o = torch.einsum("hij,jhd->ihd", torch.softmax(s, -1), v)
    o = o * torch.sigmoid(h @ w[f"{p}.g"].T)[:, :, None]
    return o.reshape(t, heads * vdim) @ w[f"{p}.o"].T


# ------------------------------------------------------------------- the model
def layer_runs(cfg):
    """The order in which layers run: (layer index, pass number or None); the looped stretch repeats."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, None) for i in range(start)]
    for t in range(times):
        runs += [(i, t) for i in range(start, stop)]
    return runs + [(i, None) for i in range(stop, n)]


def forward(cfg, w, tokens, keep_layers=False):
    """Logits ``[T, vocab]`` of one whole sequence (and the stream after every layer run)."""
    eps = cfg["norm"]["eps"]
    t = len(tokens)
    dtype = w["embed"].dtype
    x0 = embed(w, tokens, torch.arange(t), eps)
    x = x0
    loop = cfg.get("loop")
    after = []
    for i, nth in layer_runs(cfg):
        if nth is not None and i == loop["start"]:
            x = torch.cat([x, x0], -1) @ w["loop.in"].T + w["loop.step"][nth]
        layer = cfg["layers"][i]
        p = f"l{i}"
        h = layer_norm(x, w[f"{p}.norm1"], eps)
        hm = token_shift(h, w[f"{p}.shift"])
        if layer["type"] == "mingru":
            y, _ = mingru(hm, w, f"{p}.mix")
        elif layer["type"] == "latent_attention":
            y = latent_attention(hm, w, f"{p}.mix", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp"):
            y = y + dense_ff(h, w, f"{p}.mlp", eps)
        x = x + y
        after.append(x)
    logits = layer_norm(x, w["final.norm"], eps) @ w["head"].T * cfg["logit_scale"]
    return (logits, torch.stack(after)) if keep_layers else logits
