"""Small Dalavik configurations for the tests, their model folders and plain logits."""
from __future__ import annotations

import os
from typing import Dict

import torch

import plain_dalavik as plain


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base=10000.0, dims=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim if dims is None else dims}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def attn(heads, kv_heads, dim, vdim, scale, softcap=None, q_temp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap is not None:
        m["softcap"] = softcap
    if q_temp is not None:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return m


def layer(mixer, ff):
    return {"type": "latent_attention" if "kv_rank" in mixer else "attention", "mixer": mixer,
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def model(vocab, width, eps, groups, side, layers):
    c = {"architecture": "Dalavik", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups}, "layers": layers}
    if side is not None:
        c["token_side"] = {"dim": side}
    return c


# P: odd sizes, exact kernels only.  Three norm groups; a rotated part of which only four of six elements turn; a
# layer that reads the first layer's cache although another latent layer with a cache of its own lies between;
# values wider and narrower than keys; a layer without feed-forward; attention with as many kv heads as heads and
# neither cap nor temperature, and one with groups of two, a cap and a temperature that steps every third position.
CONFIG_P = model(211, 72, 3e-5, 3, 5, [
    layer(latent(3, 8, 6, 10, 20, 18, 0.3, base=50.0, dims=4), 40),
    layer(attn(4, 2, 12, 20, 0.25, softcap=5.0, q_temp=(0.7, 3)), None),
    layer(latent(2, 16, 4, 8, 12, 10, 0.2, base=1000.0), 24),
    layer(latent(5, 4, 6, 6, 9, 18, 0.35, base=50.0, dims=4, kv_from=0), 56),
    layer(attn(3, 3, 10, 6, 0.3), 32),
])
# Q: the sizes the tensor-core kernels take: cache rows of 128 and of 64 elements (kv_rank + rot_dim), heads of 64 and
# 128 in the attention with mixed heads, widths in multiples of 64, a feed-forward whose gate is fused into the product.
CONFIG_Q = model(1000, 256, 1e-6, 2, 32, [
    layer(latent(8, 32, 32, 32, 64, 96, 0.12), 512),
    layer(attn(8, 2, 64, 64, 0.125, softcap=30.0, q_temp=(0.5, 16)), 512),
    layer(latent(4, 64, 32, 64, 128, 96, 0.1, kv_from=0), 256),
    layer(latent(8, 16, 32, 48, 64, 32, 0.15, base=500000.0), None),
    layer(attn(4, 4, 128, 128, 0.09, softcap=20.0, q_temp=(0.25, 64)), 512),
    layer(latent(8, 32, 32, 32, 64, 96, 0.12, kv_from=0), 128),
])
# R: what other models make more than one, here one or absent: one norm group, no side input, one head, one kv head for
# all heads, a temperature that steps at every position, a rotated part of a single pair, a latent as wide as the keys.
CONFIG_R = model(130, 64, 1e-5, 1, None, [
    layer(attn(4, 1, 16, 16, 0.25, q_temp=(1.0, 1)), 48),
    layer(latent(1, 24, 2, 24, 16, 24, 0.2), 48),
    layer(attn(1, 1, 32, 8, 0.2, softcap=2.0), None),
    layer(latent(6, 8, 2, 8, 32, 24, 0.3, kv_from=1), 16),
])
# S: nothing is a multiple of eight: a width of 70 in five norm groups, odd ranks, head sizes, feed-forward and side
# sizes, rows of 11 and 21 cached elements, seven query heads on one kv head.
CONFIG_S = model(97, 70, 2e-5, 5, 3, [
    layer(latent(2, 6, 2, 5, 7, 9, 0.4, base=100.0), 45),
    layer(attn(7, 1, 9, 11, 0.3, softcap=4.0, q_temp=(0.3, 5)), 30),
    layer(latent(3, 5, 2, 7, 11, 9, 0.4, base=100.0, kv_from=0), None),
    layer(latent(1, 10, 6, 3, 5, 15, 0.3), 19),
])
CASES = {"P": (CONFIG_P, 31, 4), "Q": (CONFIG_Q, 32, 16), "R": (CONFIG_R, 33, 8), "S": (CONFIG_S, 34, 4)}   # config, seed, page size

_FOLDERS: Dict[tuple, str] = {}
_PLAIN: Dict[tuple, "Plain"] = {}


def _sharpen(name: str, t: torch.Tensor) -> torch.Tensor:
    """Random weights as the initialisers give them hide some faults: sinks near nothing, head mixing near the
    identity, distance terms too flat to notice a position that is one off, projections so small that every score
    is near zero and every softmax flat.  Spread them out."""
    n = t.numel()
    if name.endswith(".sink"):
        return torch.linspace(-1.0, 2.5, n).view(t.shape)
    if name.endswith(".r1"):
        return torch.linspace(0.2, 1.5, n).view(t.shape)
    if name.endswith(".r2"):
        return torch.linspace(2.0, 0.05, n).view(t.shape)
    if name.endswith(".talk"):
        return (t.float() - torch.eye(t.shape[0])) * 3.0 + torch.eye(t.shape[0])
    if name.endswith((".uq", ".uk", ".q", ".k", ".dkv", ".dq")) or name == "embed":
        return t.float() * 6.0
    if name.endswith(".side.gate"):
        return t.float() * 20.0
    return t


def folder(tmp_root: str, name: str, dtype: torch.dtype) -> str:
    """The model folder of a case (weights stored in `dtype`), written once per test session."""
    from inferloop_b200.weights import write_random_model, write_safetensors
    from inferloop_b200.weights.safetensors_io import SafetensorsFile
    key = (name, dtype)
    if key not in _FOLDERS:
        config, seed, _ = CASES[name]
        path = os.path.join(tmp_root, f"dalavik-{name}-{str(dtype).split('.')[-1]}")
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

    def forward(self, tokens, keep_layers=False):
        return plain.forward(self.w, self.config, list(tokens), keep_layers)


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
