"""Plain statement of the Zebivik decoder: 64-bit, whole sequences, one function per mechanism.

Written from the design's equations and sharing no code with the engine.  `w` maps tensor names to
64-bit tensors, `cfg` is the parsed config.json.  Notation: T tokens, width W, m the residual multiplier.

  norm          n(x) = tanh(alpha x) g + b                         (no mean, no variance)
  layer         x <- x + m n1b(mixer(n1(x)));  x <- x + m n2b(ff(n2(x)))
  rotation      pairs (i, i + d/2) of the first d elements of a head, angle p f_i, f_i = base^(-2i/d), f_i rescaled
                by wavelength bands (kept / divided by `factor` / blended in between)
  attention     q, k, v, o with biases; s_ij = scale q_i.k_j, j <= i; softmax; head h times sigmoid((G x)_h); O
  linear attn   q, k, v = silu(Q x), silu(K x), silu(V x); S_t = d_h S_{t-1} + k_t v_t^T; o_t = S_t^T q_t;
                out = O (rms(o) g sigmoid(Gt x))
  parallel      a * attention(x) + b * linear_attention(x)
  gated lru     y = gelu(Y x + by); u = conv(X x + bx); r, i = sigmoid(block-diagonal products of u + bias);
                a = exp(-8 r softplus(lam)); S_t = a S_{t-1} + sqrt(1 - a^2) i u; out = O (S y)
  dense ff      g = min(Gt x, L); u = clamp(Up x, -L, L); Dn (g sigmoid(1.702 g) (u + 1))
  experts       s = softmax(R x); choice c = s + corr; groups of neighbours ranked by their largest c, the best
                `keep` groups stay; the `top` largest c among them; weights s / (sum s + 1e-20) * scale;
                sum of w_e Dn_e(silu(Gt_e x) Up_e x) + shared(x)
  output        cap tanh((H n(x)) / cap)
"""
from __future__ import annotations

import math

import torch

DECAY_RATE = 8.0          # log a = -DECAY_RATE * r * softplus(lam)
GATE_SHARPNESS = 1.702
RENORM_EPS = 1e-20


def dyt(x, w, prefix):
    return torch.tanh(w[prefix + ".alpha"] * x) * w[prefix] + w[prefix + ".b"]


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(x):
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def frequencies(rot):
    """The rotation's angular frequencies, one per pair, after the rescaling by wavelength."""
    d = int(rot["dims"])
    out = []
    sc = rot.get("scaling")
    for i in range(d // 2):
        f = float(rot["base"]) ** (-2.0 * i / d)
        if sc:
            lam = 2.0 * math.pi / f
            orig, lo, hi, fac = float(sc["original"]), float(sc["low"]), float(sc["high"]), float(sc["factor"])
            if lam < orig / hi:
                pass
            elif lam > orig / lo:
                f = f / fac
            else:
                s = (orig / lam - lo) / (hi - lo)
                f = (1.0 - s) * f / fac + s * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float64)


def rotate_half(x, positions, rot):
    """x [T, heads, dim]: the first rot.dims elements of each head are rotated, pairs (i, i + dims/2)."""
    d = int(rot["dims"])
    ang = positions.to(torch.float64)[:, None] * frequencies(rot)[None, :]          # [T, d/2]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., : d // 2], x[..., d // 2: d]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., d:]], dim=-1)


def softmax_attention(w, p, m, h, positions):
    """The left mixer: grouped-query causal softmax attention with an output gate per head."""
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, dv)
    if m.get("rot"):
        q, k = rotate_half(q, positions, m["rot"]), rotate_half(k, positions, m["rot"])
    gate = torch.sigmoid(h @ w[p + "g"].T)                                          # [T, H]
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for i in range(H):
        j = i // (H // G)
        s = (q[:, i] @ k[:, j].T) * float(m["scale"])
        s = s.masked_fill(~mask, float("-inf"))
        out[:, i] = torch.softmax(s, dim=-1) @ v[:, j]
    out = out * gate[:, :, None]
    return out.reshape(T, H * dv) @ w[p + "o"].T + w[p + "o.b"]


def decayed_linear_attention(w, p, m, h, eps):
    """The right mixer: a matrix state per head with a constant decay."""
    T = h.shape[0]
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(h @ w[p + "q"].T).view(T, H, d)
    k = silu(h @ w[p + "k"].T).view(T, H, d)
    v = silu(h @ w[p + "v"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for i in range(H):
        S = torch.zeros(d, dv, dtype=h.dtype)
        for t in range(T):
            S = float(m["decay"][i]) * S + torch.outer(k[t, i], v[t, i])
            out[t, i] = S.T @ q[t, i]
    o = rms(out.reshape(T, H * dv), eps) * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def parallel_mixer(w, p, m, h, positions, eps):
    return (float(m["left_scale"]) * softmax_attention(w, p + "left.", m["left"], h, positions)
            + float(m["right_scale"]) * decayed_linear_attention(w, p + "right.", m["right"], h, eps))


def causal_conv(x, kernel, bias):
    """x [T, C], kernel [C, taps] (its last column multiplies the current token), zeros before the start."""
    T, taps = x.shape[0], kernel.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, x.shape[1], dtype=x.dtype), x])
    out = bias.expand(T, -1).clone()
    for j in range(taps):
        out = out + padded[j: j + T] * kernel[:, j]
    return out


def block_diagonal(u, mats, bias):
    """u [T, C] cut into len(mats) equal parts; part b is multiplied by mats[b] ([out, in]) and shifted by bias[b]."""
    B, n = mats.shape[0], mats.shape[1]
    parts = u.view(u.shape[0], B, n)
    return (torch.einsum("tbi,boi->tbo", parts, mats) + bias).reshape(u.shape[0], B * n)


def gated_linear_recurrence(w, p, m, h):
    y = gelu_tanh(h @ w[p + "y"].T + w[p + "y.b"])
    u = causal_conv(h @ w[p + "x"].T + w[p + "x.b"], w[p + "conv"], w[p + "conv.b"])
    r = torch.sigmoid(block_diagonal(u, w[p + "ra"], w[p + "ra.b"]))
    i = torch.sigmoid(block_diagonal(u, w[p + "ri"], w[p + "ri.b"]))
    a = torch.exp(-DECAY_RATE * r * softplus(w[p + "lam"]))
    b = torch.sqrt(1.0 - a * a) * i * u
    S = torch.zeros(u.shape[1], dtype=h.dtype)
    out = torch.zeros_like(u)
    for t in range(u.shape[0]):
        S = a[t] * S + b[t]
        out[t] = S
    return (out * y) @ w[p + "o"].T


def dense_ff(w, p, f, h):
    L = float(f["limit"])
    g = torch.clamp(h @ w[p + "gate"].T, max=L)
    u = torch.clamp(h @ w[p + "up"].T, min=-L, max=L)
    return (g * torch.sigmoid(GATE_SHARPNESS * g) * (u + 1.0)) @ w[p + "down"].T


def glu_expert(w, p, h):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(scores, correction, top, groups, scale):
    """scores [T, E] (softmax) -> (chosen [T, top], weights [T, top]); ties go to the lower index."""
    T, E = scores.shape
    choice = scores + correction
    if groups:
        count, keep = int(groups["count"]), int(groups["keep"])
        best = choice.view(T, count, E // count).max(-1).values                   # [T, count]
        order = torch.sort(best, dim=-1, descending=True, stable=True).indices[:, :keep]
        allowed = torch.zeros(T, count, dtype=torch.bool)
        allowed.scatter_(1, order, True)
        allowed = allowed[:, :, None].expand(T, count, E // count).reshape(T, E)
        choice = choice.masked_fill(~allowed, float("-inf"))
    chosen = torch.sort(choice, dim=-1, descending=True, stable=True).indices[:, :top]
    s = torch.gather(scores, 1, chosen)
    return chosen, s / (s.sum(-1, keepdim=True) + RENORM_EPS) * scale


def routing_margin(w, p, f, h):
    """Smallest gap, per token, between a choice score that wins (an expert or a group) and the best that loses."""
    r = f["router"]
    E, top = int(r["experts"]), int(r["top"])
    choice = torch.softmax(h @ w[p + "router"].T, dim=-1) + w[p + "correction"]
    T = h.shape[0]
    margin = torch.full((T,), float("inf"), dtype=torch.float64)
    g = r.get("groups")
    if g:
        count, keep = int(g["count"]), int(g["keep"])
        best = torch.sort(choice.view(T, count, E // count).max(-1).values, dim=-1, descending=True).values
        if keep < count:
            margin = torch.minimum(margin, best[:, keep - 1] - best[:, keep])
        order = torch.sort(choice.view(T, count, E // count).max(-1).values, dim=-1, descending=True).indices[:, :keep]
        allowed = torch.zeros(T, count, dtype=torch.bool).scatter_(1, order, True)
        choice = choice.masked_fill(~allowed[:, :, None].expand(T, count, E // count).reshape(T, E), float("-inf"))
    ranked = torch.sort(choice, dim=-1, descending=True).values
    if top < E and bool(torch.isfinite(ranked[:, top]).all()):
        margin = torch.minimum(margin, ranked[:, top - 1] - ranked[:, top])
    return margin


def experts_ff(w, p, f, h):
    r = f["router"]
    scores = torch.softmax(h @ w[p + "router"].T, dim=-1)
    chosen, weights = route(scores, w[p + "correction"], int(r["top"]), r.get("groups"), float(r["scale"]))
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, wt in zip(chosen[t].tolist(), weights[t]):
            out[t] += wt * glu_expert(w, f"{p}e{e}.", h[t: t + 1])[0]
    if f.get("shared"):
        out = out + glu_expert(w, p + "shared.", h)
    return out


def feed_forward(w, p, f, h):
    return dense_ff(w, p, f, h) if f["kind"] == "dense" else experts_ff(w, p, f, h)


def forward(w, cfg, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence; `layers_out` collects the stream after every layer."""
    eps, m = float(cfg["norm"]["eps"]), float(cfg["residual_mult"])
    positions = torch.arange(len(tokens))
    x = dyt(w["embed"][torch.tensor(tokens)], w, "embed.norm")
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = dyt(x, w, p + "norm1")
        if layer["type"] == "parallel":
            y = parallel_mixer(w, p + "mix.", layer["mixer"], h, positions, eps)
        else:
            y = gated_linear_recurrence(w, p + "mix.", layer["mixer"], h)
        x = x + m * dyt(y, w, p + "norm1b")
        if layer.get("mlp"):
            y = feed_forward(w, p + "mlp.", layer["mlp"], dyt(x, w, p + "norm2"))
            x = x + m * dyt(y, w, p + "norm2b")
        if layers_out is not None:
            layers_out.append(x.clone())
    logits = dyt(x, w, "final.norm") @ w["head"].T
    cap = float(cfg.get("logit_softcap") or 0.0)
    return cap * torch.tanh(logits / cap) if cap > 0 else logits
