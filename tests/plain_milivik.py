"""Plain, slow Milivik in float64 on the CPU: the oracle of the tests.  One function per
mechanism, written from the design's equations; nothing here is shared with the package.

Notation: x [T, W] the residual stream, h a sublayer's input (the stream itself), p the position
of a token in its sequence (from 0), H query heads, G key/value heads, d the size of a query or
key head (its unrotated part in the latent mixer), r the rotated part, dv the size of a value head.
A layer is x <- x + N1(mixer(x)); x <- x + N2(ffn(x)) with N(y) = y / sqrt(mean(y^2) + eps) * (1 + w)."""
import math

import torch

F = torch.float64
ROUTING_MARGINS = None  # a list: route() appends (token, how far its choice of groups and experts was from another one)


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_plain(x, w, eps):
    return rms(x, eps) * w


def norm_one_plus(x, w, eps):
    """The stream's norms store their gain around zero."""
    return rms(x, eps) * (1.0 + w)


def silu(z):
    return z * torch.sigmoid(z)


# ------------------------------------------------------------------------------- rotation
def yarn_table(rot):
    """(frequencies [dims/2], magnitude) of a rotation with slowed frequencies.  f_i = base^(-2i/dims);
    with ``scaling``: n(t) = dims * ln(original / (2 pi t)) / (2 ln base), lo = max(floor(n(fast)), 0),
    hi = min(ceil(n(slow)), dims - 1), ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
    f_i <- f_i / factor * ramp_i + f_i * (1 - ramp_i); cos and sin times 0.1 ln(factor) + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return torch.tensor(f, dtype=F), 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])
    n = lambda t: dims * math.log(orig / (2 * math.pi * t)) / (2 * math.log(base))
    lo = max(math.floor(n(float(sc["fast"]))), 0)
    hi = min(math.ceil(n(float(sc["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1 - ramp))
    return torch.tensor(out, dtype=F), 0.1 * math.log(factor) + 1.0


def turn_halves(x, pos, freq, mag):
    """x [T, ..., dims]: dimension i < dims/2 is paired with i + dims/2; the pair (u, v) at position p
    becomes (u c - v s, v c + u s) with c = mag cos(p f_i), s = mag sin(p f_i)."""
    half = freq.shape[0]
    a = pos.to(F)[:, None] * freq[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = (mag * torch.cos(a)).view(shape), (mag * torch.sin(a)).view(shape)
    u, v = x[..., :half], x[..., half:2 * half]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., 2 * half:]], -1)


# ------------------------------------------------------------------------------- attention cores
def softmax_attention(q, k, v, pos_q, pos_k, scale, window):
    """q [Tq, H, d], k [Tk, H, d], v [Tk, H, dv] (one key and value head per query head) -> [Tq, H, dv].
    The query at position i sees the keys at j with 0 <= i - j (< window when there is one)."""
    dist = pos_q.to(torch.int64)[:, None] - pos_k.to(torch.int64)[None, :]
    seen = dist >= 0
    if window:
        seen &= dist < window
    s = torch.einsum("thd,jhd->htj", q, k) * scale
    s = s.masked_fill(~seen[None], -math.inf)
    return torch.einsum("htj,jhv->thv", torch.softmax(s, -1), v)


# ------------------------------------------------------------------------------- latent attention
def latent_cached(h, W, p, m, eps, pos):
    """What a token leaves behind: the normed latent c [T, kv_rank] and the turned shared key part [T, r]."""
    R, r = m["kv_rank"], m["rot_dim"]
    down = h @ W[p + "dkv"].T
    c = norm_plain(down[:, :R], W[p + "dkv.norm"], eps)
    kr = down[:, R:R + r]
    if m.get("rot"):
        freq, mag = yarn_table(m["rot"])
        kr = turn_halves(kr, pos, freq, mag)
    return c, kr


def latent_attention(h, W, p, m, eps, pos, past=None):
    """The mixer on tokens at positions ``pos`` after ``past`` = (c, kr, positions) of earlier tokens.
    Returns (output [T, W], (c, kr, positions) including these tokens)."""
    T = h.shape[0]
    H, d, r, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = norm_plain(h @ W[p + "dq"].T, W[p + "dq.norm"], eps)
    q = (cq @ W[p + "uq"].T).view(T, H, d + r)
    q_plain, q_rot = q[..., :d], q[..., d:]
    if m.get("rot"):
        freq, mag = yarn_table(m["rot"])
        q_rot = turn_halves(q_rot, pos, freq, mag)
    c, kr = latent_cached(h, W, p, m, eps, pos)
    if past is not None:
        c, kr, pos_k = torch.cat([past[0], c]), torch.cat([past[1], kr]), torch.cat([past[2], pos])
    else:
        pos_k = pos
    Tk = c.shape[0]
    k_plain = (c @ W[p + "uk"].T).view(Tk, H, d)
    v = (c @ W[p + "uv"].T).view(Tk, H, dv)
    k = torch.cat([k_plain, kr[:, None, :].expand(Tk, H, r)], -1)
    o = softmax_attention(torch.cat([q_plain, q_rot], -1), k, v, pos, pos_k, m["scale"],
                          int((m.get("mask") or {}).get("size") or 0))
    o = o.reshape(T, H * dv) * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T, (c, kr, pos_k)


# ------------------------------------------------------------------------------- differential attention
def query_temperature(pos, qt):
    """1 + coef * ln(floor((p + 1) / every) + 1)."""
    if not qt:
        return torch.ones(pos.shape[0], dtype=F)
    return 1.0 + float(qt["coef"]) * torch.log(torch.floor((pos.to(F) + 1) / int(qt["every"])) + 1.0)


def diff_lambda(W, p, diff):
    return math.exp(float((W[p + "lq1"] * W[p + "lk1"]).sum())) - math.exp(float((W[p + "lq2"] * W[p + "lk2"]).sum())) + diff


def diff_attention(h, W, p, m, eps, pos, past=None, window=0):
    """Two softmax maps over the same values, o = a1 - lambda a2, each head divided by its root mean
    square and scaled by 1 - diff, a gate per head.  ``past`` = (k, v, positions).  Every earlier key
    is seen (the design has no window here; ``window`` serves tests of a mixer that is given one)."""
    T = h.shape[0]
    H, G, d, dv, diff = m["heads"], m["kv_heads"], m["dim"], m["vdim"], float(m["diff"])
    q = norm_plain((h @ W[p + "q"].T).view(T, H, 2, d), W[p + "q.norm"], eps)
    k = norm_plain((h @ W[p + "k"].T).view(T, G, 2, d), W[p + "k.norm"], eps)
    v = (h @ W[p + "v"].T).view(T, G, dv)
    q = q * query_temperature(pos, m.get("q_temp")).view(T, 1, 1, 1)
    if past is not None:
        k, v, pos_k = torch.cat([past[0], k]), torch.cat([past[1], v]), torch.cat([past[2], pos])
    else:
        pos_k = pos
    group = H // G
    kk = k.repeat_interleave(group, dim=1)  # query head a uses key/value head a // group
    vv = v.repeat_interleave(group, dim=1)
    a1 = softmax_attention(q[:, :, 0], kk[:, :, 0], vv, pos, pos_k, m["scale"], window)
    a2 = softmax_attention(q[:, :, 1], kk[:, :, 1], vv, pos, pos_k, m["scale"], window)
    o = rms(a1 - diff_lambda(W, p, diff) * a2, eps) * (1.0 - diff)
    o = o * torch.sigmoid(h @ W[p + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ W[p + "o"].T, (k, v, pos_k)


# ------------------------------------------------------------------------------- feed-forwards
def glu(h, W, p):
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def route(h, W, p, r):
    """(experts [T, top], weights [T, top]): sigmoid scores; a group's score is the sum of its two
    largest; experts of the best ``keep`` groups only; weights s / (sum s + 1e-20) * scale."""
    s = torch.sigmoid(h @ W[p + "router"].T)
    T, E = s.shape
    groups = r.get("groups") or {"count": 1, "keep": 1}
    n, keep, top = int(groups["count"]), int(groups["keep"]), int(r["top"])
    per = E // n
    gs = s.view(T, n, per).topk(min(2, per), dim=-1).values.sum(-1)
    open_groups = gs.topk(keep, dim=-1).indices
    allowed = torch.zeros(T, n, dtype=torch.bool)
    allowed.scatter_(1, open_groups, True)
    masked = torch.where(allowed[:, :, None].expand(T, n, per).reshape(T, E), s, torch.full_like(s, -1.0))
    best = masked.topk(min(top + 1, E), dim=-1)
    if ROUTING_MARGINS is not None:
        gap = (best.values[:, top - 1] - best.values[:, top]) if E > top else torch.full((T,), 1.0, dtype=F)
        gsort = gs.sort(-1, descending=True).values
        ggap = (gsort[:, keep - 1] - gsort[:, keep]) if n > keep else torch.full((T,), 1.0, dtype=F)
        ROUTING_MARGINS.extend(enumerate(torch.minimum(gap, ggap).tolist()))
    ids, w = best.indices[:, :top], best.values[:, :top]
    return ids, w / (w.sum(-1, keepdim=True) + 1e-20) * float(r.get("scale", 1.0))


def moe(h, W, p, mlp):
    ids, w = route(h, W, p, mlp["router"])
    out = torch.zeros(h.shape[0], W[p + "e0.down"].shape[0], dtype=F)
    for t in range(h.shape[0]):
        for e, a in zip(ids[t].tolist(), w[t]):
            out[t] += a * glu(h[t:t + 1], W, f"{p}e{e}.")[0]
    if mlp.get("shared"):
        out = out + glu(h, W, p + "shared.") * torch.sigmoid(h @ W[p + "shared.sg"].T)
    return out


def feed_forward(h, W, p, mlp):
    return glu(h, W, p) if mlp.get("kind", "dense") == "dense" else moe(h, W, p, mlp)


# ------------------------------------------------------------------------------- the model
def forward(cfg, W, tokens, pos=None, past=None, layer_trace=None):
    """Logits [T, vocab] of ``tokens`` (one sequence) at positions ``pos`` (default 0..T-1) after
    ``past`` (a list with one entry per layer, as returned).  Returns (logits, past)."""
    W = {k: v.to(F) for k, v in W.items()}
    T = len(tokens)
    pos = torch.arange(T) if pos is None else pos
    eps = float(cfg["norm"]["eps"])
    x = W["embed"][torch.as_tensor(tokens)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    new_past = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        mix = {"latent_attention": latent_attention, "attention": diff_attention}[layer["type"]]
        y, kept = mix(x, W, p + "mix.", layer["mixer"], eps, pos, past[i] if past is not None else None)
        new_past.append(kept)
        x = x + norm_one_plus(y, W[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + norm_one_plus(feed_forward(x, W, p + "mlp.", layer["mlp"]), W[p + "norm2"], eps)
        if layer_trace is not None:
            layer_trace.append(x.clone())
    logits = norm_one_plus(x, W["final.norm"], eps) @ W["embed"].T * float(cfg.get("logit_scale", 1.0))
    return logits, new_past


def tensor_shapes(cfg):
    """name -> shape of every tensor of a model with this configuration."""
    Wd, out = int(cfg["width"]), {}
    out["embed"] = (int(cfg["vocab"]), Wd)
    out["final.norm"] = (Wd,)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = (Wd,)
        if layer["type"] == "latent_attention":
            H, d, r, dv, R, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            out.update({p + "mix.dq": (Q, Wd), p + "mix.dq.norm": (Q,), p + "mix.uq": (H * (d + r), Q),
                        p + "mix.dkv": (R + r, Wd), p + "mix.dkv.norm": (R,), p + "mix.uk": (H * d, R),
                        p + "mix.uv": (H * dv, R), p + "mix.g": (H * dv, Wd), p + "mix.o": (Wd, H * dv)})
        else:
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * 2 * d, Wd), p + "mix.k": (G * 2 * d, Wd), p + "mix.v": (G * dv, Wd),
                        p + "mix.q.norm": (d,), p + "mix.k.norm": (d,), p + "mix.g": (H, Wd), p + "mix.o": (Wd, H * dv)})
            for n in ("lq1", "lk1", "lq2", "lk2"):
                out[p + "mix." + n] = (d,)
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        out[p + "norm2"] = (Wd,)
        unit = lambda q, ff: {q + "gate": (ff, Wd), q + "up": (ff, Wd), q + "down": (Wd, ff)}
        if mlp.get("kind", "dense") == "dense":
            out.update(unit(p + "mlp.", mlp["ff"]))
        else:
            for e in range(mlp["router"]["experts"]):
                out.update(unit(f"{p}mlp.e{e}.", mlp["expert"]["ff"]))
            out[p + "mlp.router"] = (mlp["router"]["experts"], Wd)
            if mlp.get("shared"):
                out.update(unit(p + "mlp.shared.", mlp["shared"]["ff"]))
                out[p + "mlp.shared.sg"] = (1, Wd)
    return out
