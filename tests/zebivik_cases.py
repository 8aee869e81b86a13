"""Small Zebivik configurations for the tests, their model folders and plain logits."""
from __future__ import annotations

import os
import random
from typing import Dict, List

import torch

import plain_zebivik as plain


def softmax_branch(heads, kv_heads, dim, vdim, scale, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        base, dims, scaling = rot
        m["rot"] = {"base": base, "dims": dims}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return m


def linear_branch(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def parallel(left, right, left_scale, right_scale):
    return {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}


def rglru(width, blocks, conv):
    return {"width": width, "blocks": blocks, "conv": conv}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff, scale, groups=None, shared=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    m = {"kind": "moe", "router": router, "expert": {"ff": ff}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


def layer(mixer, mlp):
    return {"type": "parallel" if "left" in mixer else "rglru", "mixer": mixer, "mlp": mlp}


def model(vocab, width, eps, mult, layers, softcap=None):
    c = {"architecture": "Zebivik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult, "layers": layers}
    if softcap is not None:
        c["logit_softcap"] = softcap
    return c


# K: odd sizes, exact kernels only.  Groups of five heads, values narrower than keys, a rotation of part of a head with
# rescaled frequencies whose three bands are all met (short, blended and long wavelengths), a linear attention of three
# heads with a state of 10 x 6 and decays from none to almost one; recurrences of 3 blocks with 5 taps and of one block
# with one tap; a layer without feed-forward; experts in three groups of which two stay, and experts without groups,
# without a shared expert, all of them chosen.
CONFIG_K = model(203, 72, 1e-5, 0.7, [
    layer(parallel(softmax_branch(5, 1, 12, 10, 0.3, rot=(50.0, 8, (4.0, 1.0, 3.0, 40.0))), linear_branch(3, 10, 6, (0.0, 0.8, 0.995)), 0.9, 1.3),
          moe(6, 2, 20, 2.0, groups=(3, 2), shared=12)),
    layer(rglru(60, 3, 5), dense(40, 0.8)),
    layer(rglru(24, 1, 1), None),
    layer(parallel(softmax_branch(4, 4, 6, 14, 0.5), linear_branch(1, 4, 20, (1.0,)), 1.0, 0.25), moe(3, 3, 16, 0.5)),
], softcap=6.0)
# L: the sizes the tensor-core kernels take: heads of 64 with values of 64 (tcgen05 prefill and cluster decode attention) and
# heads of 128 with values of 64 (the exact kernel under bfloat16 products), a full rotation without rescaling and a partial one
# with it, linear attention states of 64 x 64 and 128 x 32, a recurrence of 256 channels in 2 blocks; experts of 64 (the grouped
# tcgen05 product) in four groups of which one stays; no cap on the logits; the multiplier one.
CONFIG_L = model(1000, 256, 1e-6, 1.0, [
    layer(rglru(256, 2, 4), dense(512, 7.0)),
    layer(parallel(softmax_branch(8, 2, 64, 64, 0.125, rot=(10000.0, 64, None)), linear_branch(4, 64, 64, (0.5, 0.9, 0.99, 0.999)), 1.0, 1.0),
          moe(8, 2, 64, 1.0, groups=(4, 1), shared=128)),
    layer(parallel(softmax_branch(2, 1, 128, 64, 0.09, rot=(500000.0, 32, (6.0, 1.0, 3.0, 64.0))), linear_branch(2, 128, 32, (0.97, 0.6)), 0.5, 2.0),
          moe(4, 1, 128, 2.5)),
    layer(rglru(128, 2, 3), moe(6, 6, 64, 1.0, shared=64)),
])
# M: sizes that are multiples of nothing, and everything another model makes plural is one: one head, one kv head, one
# linear head, one block, one expert, one group; two taps; a rotation of a single pair.
CONFIG_M = model(101, 50, 3e-6, 0.3, [
    layer(parallel(softmax_branch(1, 1, 7, 9, 1.0, rot=(3.0, 2, None)), linear_branch(1, 5, 3, (0.9,)), 2.0, 2.0), moe(1, 1, 11, 1.0, groups=(1, 1), shared=7)),
    layer(rglru(35, 1, 2), dense(13, 100.0)),
], softcap=30.0)
# N: recurrences only: the model has no pages at all, only state slots.
CONFIG_N = model(150, 64, 1e-5, 0.4, [
    layer(rglru(64, 2, 4), moe(4, 2, 32, 1.25, groups=(2, 1))),
    layer(rglru(96, 3, 2), dense(64, 1.0)),
])
# P: heads of 128 with values of 128 (the tcgen05 prefill attention and the decode attention with its input stage inside at
# their widest), half of each head rotated with rescaled frequencies, groups of four heads; a dense unit of 64-row blocks (the
# clamped unit inside the tensor-core product).
CONFIG_P = model(500, 128, 2e-6, 0.6, [
    layer(parallel(softmax_branch(4, 1, 128, 128, 0.088, rot=(30000.0, 64, (4.0, 1.0, 2.0, 256.0))), linear_branch(2, 16, 64, (0.9, 0.998)), 1.1, 0.6),
          dense(128, 1.25)),
    layer(rglru(128, 2, 4), dense(192, 0.7)),
], softcap=12.0)
CASES = {"P": (CONFIG_P, 45, 16), "K": (CONFIG_K, 41, 4), "L": (CONFIG_L, 42, 16), "M": (CONFIG_M, 43, 8), "N": (CONFIG_N, 44, 16)}     # config, seed, page size

_FOLDERS: Dict[tuple, str] = {}
_PLAIN: Dict[tuple, "Plain"] = {}


def _sharpen(name: str, t: torch.Tensor) -> torch.Tensor:
    """Random weights as the initialisers give them hide some faults: routers that barely prefer an expert, corrections
    that never change the order, norms in their linear range, recurrences that forget within a few tokens.  Spread them."""
    n = t.numel()
    if name.endswith(".router"):
        return t.float() * 8.0
    if name.endswith(".correction"):                # of the size of the scores' gaps: the ranking differs from the scores' order
        return torch.linspace(-0.15, 0.15, n).flip(0).view(t.shape)
    if name.endswith(".alpha"):                     # tanh well into its bend
        return torch.full_like(t.float(), 0.9 if "norm1b" in name or "norm2b" in name else 0.6)
    if name.endswith(".lam"):                       # decays from a few tokens to hundreds
        return torch.linspace(-6.0, 1.0, n).view(t.shape)
    if name.endswith((".ra", ".ri")):               # gates that depend on the input
        return t.float() * 4.0
    if name.endswith(".left.g"):
        return t.float() * 6.0
    if name.endswith((".left.q", ".left.k")):       # a softmax that picks few keys, wherever they lie
        return t.float() * 2.0
    if name == "embed":
        return t.float() * 4.0
    if name == "head":
        return t.float() * 6.0
    return t


def folder(tmp_root: str, name: str, dtype: torch.dtype) -> str:
    """The model folder of a case (weights stored in `dtype`), written once per test session."""
    from inferloop_b200.weights import write_random_model, write_safetensors
    from inferloop_b200.weights.safetensors_io import SafetensorsFile
    key = (name, dtype)
    if key not in _FOLDERS:
        config, seed, _ = CASES[name]
        path = os.path.join(tmp_root, f"zebivik-{name}-{str(dtype).split('.')[-1]}")
        write_random_model(path, config, seed, dtype, prefix="")
        f = SafetensorsFile(os.path.join(path, "model.safetensors"))
        tensors = [(n, f.tensor(n).clone()) for n in f.names()]
        f.close()
        tensors = [(n, _sharpen(n, t).to(t.dtype)) for n, t in tensors]
        write_safetensors(os.path.join(path, "model.safetensors"), tensors, metadata={"format": "pt"})
        _FOLDERS[key] = path
    return _FOLDERS[key]


class Plain:
    def __init__(self, config: dict, weights: Dict[str, torch.Tensor]) -> None:
        self.config = config
        self.w = {k: v.double() for k, v in weights.items()}

    def forward(self, tokens, trace=None) -> torch.Tensor:
        return plain.forward(self.w, self.config, list(tokens), trace)

    def least_margin(self, tokens, first: int = 0) -> float:
        """The smallest routing margin over the positions from `first` on, in every routed layer."""
        cfg, w = self.config, self.w
        eps, m = float(cfg["norm"]["eps"]), float(cfg["residual_mult"])
        positions = torch.arange(len(tokens))
        x = plain.dyt(w["embed"][torch.tensor(list(tokens))], w, "embed.norm")
        least = 1.0
        for i, layer_cfg in enumerate(cfg["layers"]):
            p = f"l{i}."
            h = plain.dyt(x, w, p + "norm1")
            if layer_cfg["type"] == "parallel":
                y = plain.parallel_mixer(w, p + "mix.", layer_cfg["mixer"], h, positions, eps)
            else:
                y = plain.gated_linear_recurrence(w, p + "mix.", layer_cfg["mixer"], h)
            x = x + m * plain.dyt(y, w, p + "norm1b")
            f = layer_cfg.get("mlp")
            if f:
                h = plain.dyt(x, w, p + "norm2")
                if f["kind"] == "moe":
                    least = min(least, float(plain.routing_margin(w, p + "mlp.", f, h)[first:].min()))
                x = x + m * plain.dyt(plain.feed_forward(w, p + "mlp.", f, h), w, p + "norm2b")
        return least


def plain_model(tmp_root: str, name: str, dtype: torch.dtype) -> Plain:
    from inferloop_b200.weights.safetensors_io import SafetensorsFile
    key = (name, dtype)
    if key not in _PLAIN:
        path = folder(tmp_root, name, dtype)
        f = SafetensorsFile(os.path.join(path, "model.safetensors"))
        weights = {n: f.tensor(n).clone() for n in f.names()}
        f.close()
        _PLAIN[key] = Plain(CASES[name][0], weights)
    return _PLAIN[key]


def decided_tokens(model: Plain, n: int, vocab: int, seed: int, margin: float, chunk: int = 12) -> List[int]:
    """`n` random tokens whose routing decisions, in the plain model, all have at least this margin, so that no
    comparison rests on a close call.  The sequence grows by chunks; a position's decisions depend on the tokens
    up to it alone, so a chunk whose positions are not all decided is drawn again and the ones before it stay."""
    rng = random.Random(seed)
    tokens: List[int] = []
    failed = 0
    while len(tokens) < n:
        size = max(1, chunk >> (failed // 3))
        more = [rng.randrange(vocab) for _ in range(min(size, n - len(tokens)))]
        if model.least_margin(tokens + more, len(tokens)) >= margin:
            tokens += more
            failed = 0
        else:
            failed += 1
            if failed > 400:
                raise AssertionError("no token sequence with decided routing found")
    return tokens
