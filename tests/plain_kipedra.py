"""A plain, slow implementation of the Kipedra decoder from its equations: one function per mechanism, whole sequences
at a time, double precision, loops where a loop is the clearest way to say it.  It shares nothing with the engine (no
part, no kernel, no cache): the tests compare the engine with it.

A model is (config dict, {tensor name: torch tensor}).  Tensor names: `embed`, `final.norm`, and per layer i
`l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*`, `l<i>.mlp.*`.
"""
import math

import torch

F = torch.float64


# ----------------------------------------------------------------------------- small pieces
def zero_centred_rms_norm(x, w, eps):
    """The weight is stored as its distance from one."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * (1.0 + w)


def plain_rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def causal_conv(u, taps_w):
    """u [T, C], taps_w [C, taps]: y[t] = sum_j taps_w[:, j] * u[t - taps + 1 + j], zeros before the start."""
    T, taps = u.shape[0], taps_w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            src = t - taps + 1 + j
            if src >= 0:
                y[t] = y[t] + taps_w[:, j] * u[src]
    return y


def rotate_neighbours(x, positions, dims, base):
    """x [T, heads, n]: of the last axis' first `dims` entries, 2i turns with 2i+1 by position * base^(-2i/dims)."""
    out = x.clone()
    for i in range(dims // 2):
        ang = positions.to(F) * base ** (-2.0 * i / dims)
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        a, b = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = a * c - b * s
        out[..., 2 * i + 1] = b * c + a * s
    return out


# ----------------------------------------------------------------------------- mixers (one sequence, positions 0..T-1)
def gated_delta(h, w, m, eps):
    """The gated delta rule, token by token.  h [T, width]; w(name) -> tensor of this mixer."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w("q").T, w("q.conv"))).view(T, G, dk)
    k = silu(causal_conv(h @ w("k").T, w("k.conv"))).view(T, G, dk)
    v = silu(causal_conv(h @ w("v").T, w("v.conv"))).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w("b").T)                                          # [T, H]
    decay = torch.exp(-torch.exp(w("A_log")) * softplus(h @ w("a").T + w("dt_bias")))    # [T, H]
    gate = silu(h @ w("g").T).view(T, H, dv)
    o = torch.zeros((T, H, dv), dtype=F)
    for head in range(H):
        kv = head // (H // G)
        S = torch.zeros((dk, dv), dtype=F)
        for t in range(T):
            S = decay[t, head] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, kv])
            S = S + torch.outer(k[t, kv], u)
            o[t, head] = S.T @ q[t, kv]
    o = plain_rms_norm(o, w("norm"), eps) * gate
    return o.reshape(T, H * dv) @ w("o").T


def windowed_attention(h, w, m):
    """Grouped-query attention with biases, a short convolution on q, k and v, a partial rotation of neighbours and a
    sliding window."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = causal_conv(h @ w("q").T + w("q.b"), w("q.conv")).view(T, H, dk)
    k = causal_conv(h @ w("k").T + w("k.b"), w("k.conv")).view(T, G, dk)
    v = causal_conv(h @ w("v").T + w("v.b"), w("v.conv")).view(T, G, dv)
    q = rotate_neighbours(q, pos, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_neighbours(k, pos, m["rot"]["dims"], m["rot"]["base"])
    span = m["mask"]["size"]
    out = torch.zeros((T, H, dv), dtype=F)
    for head in range(H):
        kv = head // (H // G)
        for t in range(T):
            lo = max(0, t - span + 1)
            s = (k[lo:t + 1, kv] @ q[t, head]) * m["scale"]
            p = torch.softmax(s, dim=0)
            out[t, head] = p @ v[lo:t + 1, kv]
    return out.reshape(T, H * dv) @ w("o").T


# ----------------------------------------------------------------------------- feed-forwards
def gated_dense(h, w):
    return (gelu_tanh(h @ w("gate").T) * (h @ w("up").T)) @ w("down").T


def routed_experts(h, w, mlp, forced=None):
    """Each token's `top` experts by sigmoid score plus a correction; the weights are the plain scores, normalised and
    scaled.  forced [T, top]: use these experts instead of the router's choice (for comparing beyond a near-tie)."""
    r = mlp["router"]
    s = torch.sigmoid(h @ w("router").T)
    chosen = torch.topk(s + w("correction"), r["top"], dim=-1).indices if forced is None else forced
    picked = torch.gather(s, 1, chosen)
    weights = picked / (picked.sum(-1, keepdim=True) + 1e-20) * r["scale"]
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(r["top"]):
            e = int(chosen[t, j])
            a = torch.relu(h[t] @ w(f"e{e}.up").T) ** 2
            y[t] = y[t] + weights[t, j] * (a @ w(f"e{e}.down").T)
    return y, chosen


# ----------------------------------------------------------------------------- the model
def execution_order(cfg):
    n = len(cfg["layers"])
    lp = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    return list(range(lp["start"])) + list(range(lp["start"], lp["stop"])) * lp["times"] + list(range(lp["stop"], n))


def forward(cfg, weights, tokens, forced=None, streams=None):
    """Logits [T, vocab] (float64) of one sequence.  forced: {executed position: [T, top] experts}.  streams: a list that
    receives the residual stream after every executed layer."""
    W = {k: v.to(F) for k, v in weights.items()}
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    chosen = {}
    for p, i in enumerate(execution_order(cfg)):
        L = cfg["layers"][i]
        mix = lambda name, i=i: W[f"l{i}.mix.{name}"]
        mlp = lambda name, i=i: W[f"l{i}.mlp.{name}"]
        h1 = zero_centred_rms_norm(x, W[f"l{i}.norm1"], eps)
        if L["type"] == "delta":
            y = gated_delta(h1, mix, L["mixer"], eps)
        elif L["type"] == "attention":
            y = windowed_attention(h1, mix, L["mixer"])
        else:
            raise ValueError(L["type"])
        if L.get("mlp") is not None:
            h2 = zero_centred_rms_norm(x, W[f"l{i}.norm2"], eps)
            if L["mlp"]["kind"] == "dense":
                y = y + gated_dense(h2, mlp)
            else:
                f, chosen[p] = routed_experts(h2, mlp, L["mlp"], None if forced is None else forced.get(p))
                y = y + f
        x = x + mult * y
        if streams is not None:
            streams.append(x.clone())
    logits = zero_centred_rms_norm(x, W["final.norm"], eps) @ W["embed"].T
    forward.chosen = chosen
    return logits
