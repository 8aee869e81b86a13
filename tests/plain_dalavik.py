"""Plain statement of the Dalavik decoder: 64-bit, whole sequences, one function per mechanism.

Written from the design's equations and sharing no code with the engine.  `w` maps tensor names
to 64-bit tensors, `cfg` is the parsed config.json.  Notation: T tokens, width W, positions from 0.

  layer         x <- x + gn(mixer(x), n1);  x <- x + gn(ff(x), n2);  x <- x + side(x, tok)
                (the norm sits on each sublayer's OUTPUT; the sublayers read x as it is)
  gn(y, g)      y cut into `groups` equal parts, each part / sqrt(mean(part^2) + eps), the whole times g
  side          e = S[tok][i dim : (i + 1) dim] for layer i;  u = P (gelu_tanh(G x) * e);  u / rms(u) * g
  latent attn   cq = rms(Dq h) gq;  q = Uq cq = [qa | qr] per head;  [c' | r] = Dkv h;  c = rms(c') gc;
                qr, r rotated in neighbouring pairs;  k_a = Uk c, v = Uv c per head;
                s_ij = scale (qa_i . ka_j + qr_i . r_j), j <= i;  softmax;  out = O [p v]
                a layer with `kv_from` j takes c and the rotated r of layer j
  attention     q = Q h + bq, k = K h + bk, v = V h + bv;  q, k normed per head with a weight;
                q_i *= 1 + coef ln(floor((i + 1) / every) + 1);
                s = scale q.k;  s <- cap tanh(s / cap);  s <- s - r1 ln(1 + r2 (i - j));
                s_h <- sum_g M[h, g] s_g;  p = exp(s) / (exp(sink) + sum_j exp(s));  out = O [p v]
  feed-forward  Dn (relu(Gt h) * (Up h))
  output        E gn(x, final)
"""
from __future__ import annotations

import math

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def group_norm(y, g, eps, groups):
    """Each of `groups` equal consecutive parts of the last axis divided by its own root mean square."""
    T, W = y.shape
    parts = y.reshape(T, groups, W // groups)
    return rms(parts, eps).reshape(T, W) * g


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_pairs(x, positions, base, dims):
    """x [T, ..., n]: the first `dims` elements of the last axis turn in pairs (2i, 2i + 1) by
    positions * base^(-2i / dims); the rest pass."""
    out = x.clone()
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64)
    a = positions.to(torch.float64)[:, None] * f[None, :]                  # [T, half]
    while a.dim() < x.dim():
        a = a.unsqueeze(1)
    cos, sin = torch.cos(a), torch.sin(a)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def latent_cache(w, p, m, h, positions, eps):
    """What a latent layer keeps per token: the normed latent c [T, rank] and the rotated shared key part [T, rot_dim]."""
    rank = int(m["kv_rank"])
    down = h @ w[p + "dkv"].T
    c = rms(down[:, :rank], eps) * w[p + "dkv.norm"]
    r = rotate_pairs(down[:, rank:], positions, float(m["rot"]["base"]), int(m["rot"]["dims"]))
    return c, r


def causal_softmax(s, sink=None):
    """s [H, T, T]; position i reads j <= i; `sink` [H] joins the denominator only."""
    T = s.shape[-1]
    seen = torch.tril(torch.ones(T, T, dtype=torch.bool))
    s = s.masked_fill(~seen, -math.inf)
    top = s.max(-1, keepdim=True).values
    if sink is not None:
        top = torch.maximum(top, sink[:, None, None])
    e = torch.exp(s - top)
    total = e.sum(-1, keepdim=True)
    if sink is not None:
        total = total + torch.exp(sink[:, None, None] - top)
    return e / total


def latent_attention(w, p, m, h, positions, eps, kept):
    """`kept` = (c, r) of the layer whose cache this one reads."""
    H, d, dr, dv = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"])
    T = h.shape[0]
    cq = rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).reshape(T, H, d + dr)
    qa = q[..., :d]
    qr = rotate_pairs(q[..., d:], positions, float(m["rot"]["base"]), int(m["rot"]["dims"]))
    c, r = kept
    ka = (c @ w[p + "uk"].T).reshape(T, H, d)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    s = (torch.einsum("ihd,jhd->hij", qa, ka) + torch.einsum("ihd,jd->hij", qr, r)) * float(m["scale"])
    prob = causal_softmax(s)
    o = torch.einsum("hij,jhd->ihd", prob, v).reshape(T, H * dv)
    return o @ w[p + "o"].T


def query_temperature(positions, q_temp):
    if not q_temp:
        return torch.ones(positions.shape[0], dtype=torch.float64)
    steps = torch.floor((positions.to(torch.float64) + 1.0) / float(q_temp["every"]))
    return 1.0 + float(q_temp["coef"]) * torch.log(steps + 1.0)


def mixed_heads_attention(w, p, m, h, positions, eps):
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, dv)
    q = rms(q, eps) * w[p + "q.norm"]
    k = rms(k, eps) * w[p + "k.norm"]
    q = q * query_temperature(positions, m.get("q_temp"))[:, None, None]
    per = H // G
    kh, vh = k.repeat_interleave(per, dim=1), v.repeat_interleave(per, dim=1)     # head h reads kv head h // per
    s = torch.einsum("ihd,jhd->hij", q, kh) * float(m["scale"])
    cap = float(m.get("softcap") or 0.0)
    if cap > 0:
        s = cap * torch.tanh(s / cap)
    pos = positions.to(torch.float64)
    dist = (pos[:, None] - pos[None, :]).clamp(min=0.0)                            # i - j where it is seen
    s = s - w[p + "r1"][:, None, None] * torch.log1p(w[p + "r2"][:, None, None] * dist[None])
    s = torch.einsum("hg,gij->hij", w[p + "talk"], s)
    prob = causal_softmax(s, w[p + "sink"])
    o = torch.einsum("hij,jhd->ihd", prob, vh).reshape(T, H * dv)
    return o @ w[p + "o"].T


def dense_ff(w, p, h):
    return (torch.relu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def token_side(w, cfg, i, x, tokens):
    dim = int(cfg["token_side"]["dim"])
    p = f"l{i}.side."
    e = w["side.embed"][torch.tensor(tokens)][:, i * dim:(i + 1) * dim]
    u = (gelu_tanh(x @ w[p + "gate"].T) * e) @ w[p + "proj"].T
    return rms(u, float(cfg["norm"]["eps"])) * w[p + "norm"]


def forward(w, cfg, tokens, keep_layers=False):
    """Logits [T, vocab] of a whole sequence (and the stream after every layer, if asked)."""
    eps, groups = float(cfg["norm"]["eps"]), int(cfg["norm"].get("groups", 1))
    positions = torch.arange(len(tokens))
    x = w["embed"][torch.tensor(tokens)]
    kept, after = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        if layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = latent_cache(w, p, m, x, positions, eps)
                src = i
            y = latent_attention(w, p, m, x, positions, eps, kept[int(src)])
        elif layer["type"] == "attention":
            y = mixed_heads_attention(w, p, m, x, positions, eps)
        else:
            raise ValueError(layer["type"])
        x = x + group_norm(y, w[f"l{i}.norm1"], eps, groups)
        if layer.get("mlp") is not None:
            x = x + group_norm(dense_ff(w, f"l{i}.mlp.", x), w[f"l{i}.norm2"], eps, groups)
        if cfg.get("token_side") is not None:
            x = x + token_side(w, cfg, i, x, tokens)
        after.append(x)
    logits = group_norm(x, w["final.norm"], eps, groups) @ w["embed"].T
    return (logits, after) if keep_layers else logits
