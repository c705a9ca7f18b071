"""Plain, slow Desalix in float64 on the CPU: the oracle of the tests.  One function per
mechanism, written from the design's equations; nothing here is shared with the package.

Notation: x [T, W] the residual stream, h a sublayer's input, p the position of a token in its
sequence (from 0), H query heads, G key/value heads, d the size of a query or key head, dv of a
value head."""
import math

import torch

F = torch.float64
ROUTING_MARGINS = None  # a list: moe() appends (token, gap between the last chosen and the next score)


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scalar_norm(x, g, eps):
    """RMS norm whose gain is one number."""
    return rms(x, eps) * g


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def turn_halves(x, pos, base, dims, sign=1.0):
    """x [T, heads, n]: dimension i < dims/2 is paired with i + dims/2; the pair (u, v) at position
    p becomes (u cos a - v sin a, v cos a + u sin a), a = sign * p * base^(-2i/dims); dimensions
    from dims on pass."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    a = sign * pos.to(F)[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


def visible(i, j, size):
    """Whether the query at position i sees the key at position j: j <= i, and with chunks of
    ``size`` positions (counted from 0) both in the same chunk."""
    return j <= i and (not size or i // size == j // size)


def sink_softmax_attention(q, k, v, pos_q, pos_k, scale, size, sink):
    """q [Tq, H, d], k [Tk, G, d], v [Tk, G, dv], sink [H] -> [Tq, H, dv]: weights
    exp(s_j) / (exp(sink_h) + sum_j exp(s_j)) over the visible keys, s_j = (q . k_j) * scale."""
    Tq, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(Tq, H, v.shape[2], dtype=F)
    for t in range(Tq):
        seen = [n for n, j in enumerate(pos_k) if visible(int(pos_q[t]), int(j), size)]
        for h in range(H):
            g = h // (H // G)
            s = (k[seen, g] @ q[t, h]) * scale
            m = max(float(s.max()) if len(seen) else -math.inf, float(sink[h]))
            e = torch.exp(s - m)
            out[t, h] = (e / (e.sum() + math.exp(float(sink[h]) - m))) @ v[seen, g]
    return out


def attention_parts(h, W, p, m, eps, pos):
    """(q, k, v) of the tokens at positions ``pos`` as they are used and cached: heads normed,
    queries and keys turned on their first rot.dims dimensions, values normed and turned over all
    of theirs."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = scalar_free_head_norm((h @ W[p + "q"].T).view(T, H, d), W[p + "q.norm"], eps)
    k = scalar_free_head_norm((h @ W[p + "k"].T).view(T, G, d), W[p + "k.norm"], eps)
    v = rms((h @ W[p + "v"].T).view(T, G, dv), eps)
    rot = m.get("rot")
    if rot:
        if rot.get("dims"):
            q = turn_halves(q, pos, rot["base"], rot["dims"])
            k = turn_halves(k, pos, rot["base"], rot["dims"])
        v = turn_halves(v, pos, rot["base"], dv)
    return q, k, v


def scalar_free_head_norm(x, w, eps):
    """Per head: RMS norm over the head's dimensions times a weight of that size (plain, shared by
    the heads)."""
    return rms(x, eps) * w


def attention(h, W, p, m, eps, pos=None):
    T = h.shape[0]
    pos = torch.arange(T) if pos is None else pos
    q, k, v = attention_parts(h, W, p, m, eps, pos)
    size = (m.get("mask") or {}).get("size") or 0
    o = sink_softmax_attention(q, k, v, pos, pos, m["scale"], size, W[p + "sink"])
    rot = m.get("rot")
    if rot:
        o = turn_halves(o, pos, rot["base"], m["vdim"], sign=-1.0)
    return o.reshape(T, -1) @ W[p + "o"].T


def clamped_glu(a, W, p, limit, alpha=1.702):
    g = torch.clamp(a @ W[p + "gate"].T, max=limit)
    u = torch.clamp(a @ W[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(alpha * g) * (u + 1)) @ W[p + "down"].T


def route(z, top):
    """Scores sigmoid(z) [E]; the ``top`` largest (the lower index first among equals) with their
    scores as weights."""
    s = torch.sigmoid(z)
    order = sorted(range(len(s)), key=lambda e: (-float(s[e]), e))
    return order[:top], s


def moe(h, W, p, mlp):
    out = torch.zeros_like(h)
    top = mlp["router"]["top"]
    for t in range(h.shape[0]):
        chosen, s = route(W[p + "router"] @ h[t], top)
        if ROUTING_MARGINS is not None and top < len(s):
            rest = max(float(s[e]) for e in range(len(s)) if e not in chosen)
            ROUTING_MARGINS.append((t, float(s[chosen[-1]]) - rest))
        for e in chosen:
            out[t] += clamped_glu(s[e] * h[t], W, f"{p}e{e}.", mlp["expert"]["limit"])
    if mlp.get("shared"):
        out = out + clamped_glu(h, W, p + "shared.", mlp["shared"]["limit"])
    return out


def layer_runs(config):
    """[(layer, t)]: the layers in the order they run; t is the number of the pass over the
    repeated run that begins there, else None."""
    L = len(config["layers"])
    loop = config.get("loop")
    if not loop or loop["start"] == loop["stop"]:
        return [(i, None) for i in range(L)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], L)]


def forward(config, weights, ids, trace=None):
    """Logits [T, vocab] of one sequence; ``trace`` (a list) receives the stream after every layer run."""
    W = {k: v.to(F) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x0 = W["embed"][torch.tensor(ids)] * (config.get("embedding") or {}).get("scale", 1.0)
    x = x0.clone()
    for i, t in layer_runs(config):
        e, p = config["layers"][i], f"l{i}."
        if t is not None:
            if t > 0:
                x = x + x0
            x = x + W["loop.step"][t]
        a = attention(scalar_norm(x, W[p + "norm1"], eps), W, p + "mix.", e["mixer"], eps)
        x = x + scalar_norm(a, W[p + "norm1b"], eps) * W[p + "ls1"]
        if e.get("mlp") is not None:
            f = moe(scalar_norm(x, W[p + "norm2"], eps), W, p + "mlp.", e["mlp"])
            x = x + scalar_norm(f, W[p + "norm2b"], eps) * W[p + "ls2"]
        if trace is not None:
            trace.append(x.clone())
    return scalar_norm(x, W["final.norm"], eps) @ W["head"].T


def greedy(config, weights, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(forward(config, weights, ids)[-1].argmax()))
    return ids[len(prompt):]
