"""A plain, slow implementation of the Pedotar decoder from its equations: one function per
mechanism, whole sequences at a time, double precision, loops where a loop is the clearest way to
say it.  It shares nothing with the engine (no part, no kernel, no cache): the tests compare the
engine with it.

A model is (config dict, {tensor name: torch tensor}).  Tensor names: `embed`, `final.norm[.b]`,
and per layer i `l<i>.norm1[.b]`, `l<i>.norm1b[.b]`, `l<i>.norm2[.b]`, `l<i>.norm2b[.b]`,
`l<i>.mix.*`, `l<i>.mlp.{gate,up,down}`.
"""
import math

import torch

F = torch.float64


# ----------------------------------------------------------------------------- small pieces
def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rotate_halves(x, positions, dims, base):
    """x [T, ..., n]: the first `dims` of the last axis turn, i with i + dims/2, by position * base^(-2i/dims)."""
    out = x.clone()
    half = dims // 2
    for i in range(half):
        f = base ** (-2.0 * i / dims)
        ang = positions.to(F) * f
        c, s = torch.cos(ang), torch.sin(ang)
        while c.dim() < x.dim() - 1:
            c, s = c.unsqueeze(-1), s.unsqueeze(-1)
        u, v = x[..., i], x[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


# ----------------------------------------------------------------------------- mixers (one sequence, positions 0..T-1)
def mamba1(h, w, p, m):
    """Selective scan, token by token.  h [T, width]; w(name) -> tensor of this mixer."""
    T = h.shape[0]
    inner, N, taps, R = m["inner"], m["state"], m["conv"], m["dt_rank"]
    xz = h @ w("in").T
    x, z = xz[:, :inner], xz[:, inner:]
    conv_w, conv_b = w("conv"), w("conv.b")
    xc = torch.zeros_like(x)
    for t in range(T):
        acc = conv_b.clone()
        for k in range(taps):                       # tap taps-1 is the current token's
            src = t - (taps - 1 - k)
            if src >= 0:
                acc = acc + conv_w[:, k] * x[src]
        xc[t] = acc
    xc = silu(xc)
    proj = xc @ w("x").T
    dt_in, B, C = proj[:, :R], proj[:, R:R + N], proj[:, R + N:R + 2 * N]
    dt = softplus(dt_in @ w("dt").T + w("dt.b"))
    A = -torch.exp(w("A_log"))
    S = torch.zeros((inner, N), dtype=F)
    y = torch.zeros((T, inner), dtype=F)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * xc[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + w("D") * xc[t]
    return (y * silu(z)) @ w("o").T


def latent_attention(h, w, p, m, eps):
    """Keys and values expanded from a cached latent; one rotated key part shared by the heads."""
    T = h.shape[0]
    H, dim, rd, vd, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    q = (h @ w("q").T).view(T, H, dim + rd)
    qn, qr = q[..., :dim], rotate_halves(q[..., dim:], pos, m["rot"]["dims"], m["rot"]["base"])
    dkv = h @ w("dkv").T
    c = rms_norm(dkv[:, :rank], w("dkv.norm"), eps)
    kr = rotate_halves(dkv[:, rank:], pos, m["rot"]["dims"], m["rot"]["base"])
    kn = (c @ w("uk").T).view(T, H, dim)
    v = (c @ w("uv").T).view(T, H, vd)
    out = torch.zeros((T, H, vd), dtype=F)
    for hh in range(H):
        s = (qn[:, hh] @ kn[:, hh].T + qr[:, hh] @ kr.T) * m["scale"]
        s = s.masked_fill(pos[None, :] > pos[:, None], -math.inf)
        out[:, hh] = torch.softmax(s, -1) @ v[:, hh]
    return out.reshape(T, H * vd) @ w("o").T


def chunked_attention(h, w, p, m, eps):
    """Grouped-query attention inside chunks of `mask.size` positions, normalised q and k, no
    positions in the scores, the heads' softmax weights mixed by a matrix before they meet the values."""
    T = h.shape[0]
    H, G, dim, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    size = m["mask"]["size"]
    pos = torch.arange(T)
    q = rms_norm((h @ w("q").T).view(T, H, dim), w("q.norm"), eps)
    k = rms_norm((h @ w("k").T).view(T, G, dim), w("k.norm"), eps)
    v = (h @ w("v").T).view(T, G, vd)
    per = H // G
    seen = (pos[None, :] <= pos[:, None]) & ((pos[None, :] // size) == (pos[:, None] // size))
    P = torch.zeros((H, T, T), dtype=F)
    for hh in range(H):
        s = (q[:, hh] @ k[:, hh // per].T) * m["scale"]
        P[hh] = torch.softmax(s.masked_fill(~seen, -math.inf), -1)
    mixed = torch.einsum("hg,gij->hij", w("talk"), P)
    out = torch.zeros((T, H, vd), dtype=F)
    for hh in range(H):
        out[:, hh] = mixed[hh] @ v[:, hh // per]
    return out.reshape(T, H * vd) @ w("o").T


def dense_mlp(h, w):
    return (silu(h @ w("gate").T) * (h @ w("up").T)) @ w("down").T


MIXERS = {"mamba1": lambda h, w, p, m, eps: mamba1(h, w, p, m), "latent_attention": latent_attention, "attention": chunked_attention}


# ----------------------------------------------------------------------------- the model
def executed_layers(cfg):
    """[(layer index, first of its pass?)] in the order they run; the looped span repeats."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = loop["start"], loop["stop"], loop["times"]
    out = [(i, False) for i in range(a)]
    for r in range(times):
        out += [(i, r > 0 and i == a) for i in range(a, b)]
    out += [(i, False) for i in range(b, n)]
    return out


def forward(cfg, tensors, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence (float64), and optionally the stream after every layer run."""
    t64 = {k: v.to(F) for k, v in tensors.items() if v.dtype.is_floating_point}
    eps = cfg["norm"]["eps"]
    x0 = t64["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x = x0.clone()
    trail = []
    for i, readd in executed_layers(cfg):
        L = cfg["layers"][i]
        pre = f"l{i}."
        if readd:
            x = x + x0
        def ln(name, v):
            return layer_norm(v, t64[pre + name], t64[pre + name + ".b"], eps)
        mix = MIXERS[L["type"]](ln("norm1", x), lambda n: t64[pre + "mix." + n], None, L["mixer"], eps)
        x = x + ln("norm1b", mix)
        if L.get("mlp") is not None:
            x = x + ln("norm2b", dense_mlp(ln("norm2", x), lambda n: t64[pre + "mlp." + n]))
        trail.append(x.clone())
    xn = layer_norm(x, t64["final.norm"], t64["final.norm.b"], eps)
    logits = xn @ t64["embed"].T
    return (logits, torch.stack(trail)) if return_layers else logits
