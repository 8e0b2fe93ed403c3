"""A plain, slow restatement of the Vudelix design, one function per mechanism, token by token.

Nothing here is shared with the product path: no caches, no packed batches, no fused projections.  The recurrent
mixer, the dense feed-forward and the RMS norm are the ones of ``hybrid_oracle.py`` (also oracle code).  Added here:

* ``stretched_frequencies``   rotary frequencies, stretched by wavelength
* ``rotate_neighbours``       rotary positions, pair (2i, 2i + 1)
* ``window_attention``        grouped-query attention over a sliding window with unit-RMS q/k and a gate per head
* ``moe_ff``                  sigmoid router, top-k, the score multiplies the expert's input, squared-ReLU experts
* ``token_side``              the gated per-layer token embedding
* ``forward``                 the whole model: pre-norm blocks with a residual multiplier, own output head

``forward`` always runs a whole sequence from its first token, which makes it an oracle for caches and states.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional

import torch

from hybrid_oracle import channel_delta, dense_ff, rms_norm, sub

Tensors = Dict[str, torch.Tensor]


def stretched_frequencies(n: int, base: float, scaling: Optional[Dict[str, float]]) -> List[float]:
    out = []
    for i in range(n // 2):
        f = base ** (-2.0 * i / n)
        if scaling:
            wavelength = 2.0 * math.pi / f
            orig, lo, hi, factor = scaling["original"], scaling["low"], scaling["high"], scaling["factor"]
            if wavelength < orig / hi:
                pass
            elif wavelength > orig / lo:
                f = f / factor
            else:
                s = (orig / wavelength - lo) / (hi - lo)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return out


def rotate_neighbours(x: torch.Tensor, pos: int, freqs: List[float]) -> torch.Tensor:
    out = x.clone()
    for i, f in enumerate(freqs):
        a = pos * f
        u, v = x[2 * i], x[2 * i + 1]
        out[2 * i] = u * math.cos(a) - v * math.sin(a)
        out[2 * i + 1] = v * math.cos(a) + u * math.sin(a)
    return out


def window_attention(h: torch.Tensor, p: Tensors, m: Dict[str, Any], eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    window = (m.get("mask") or {}).get("size", 0)
    rot = m.get("rot") or {}
    freqs = stretched_frequencies(rot["dims"], rot["base"], rot.get("scaling")) if rot else []
    keys: List[torch.Tensor] = []
    vals: List[torch.Tensor] = []
    out = torch.zeros(T, H * V, dtype=h.dtype)
    for t in range(T):
        q = (p["q"] @ h[t]).view(H, D)
        k = (p["k"] @ h[t]).view(G, D)
        keys.append(torch.stack([rms_norm(rotate_neighbours(k[g], t, freqs), None, eps) for g in range(G)]))
        vals.append((p["v"] @ h[t]).view(G, V))
        gate = torch.sigmoid(p["g"] @ h[t])
        first = max(0, t - window + 1) if window else 0
        for hd in range(H):
            g = hd // (H // G)
            qh = rms_norm(rotate_neighbours(q[hd], t, freqs), None, eps)
            s = torch.stack([(qh @ keys[j][g]) * m["scale"] for j in range(first, t + 1)])
            w = torch.softmax(s, 0)
            o = sum(w[j - first] * vals[j][g] for j in range(first, t + 1))
            out[t, hd * V:(hd + 1) * V] = o * gate[hd]
    return out @ p["o"].T


def moe_ff(h: torch.Tensor, p: Tensors, mlp: Dict[str, Any]) -> torch.Tensor:
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    out = torch.zeros(h.shape[0], p["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        score = torch.sigmoid(p["router"] @ h[t])
        chosen = sorted(range(E), key=lambda e: (-float(score[e]), e))[:top]
        for e in chosen:
            a = torch.relu(p[f"e{e}.up"] @ (score[e] * h[t])) ** 2
            out[t] += p[f"e{e}.down"] @ a
    return out


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def token_side(x: torch.Tensor, tokens: List[int], table: torch.Tensor, p: Tensors, layer: int, dim: int, eps: float) -> torch.Tensor:
    y = torch.zeros_like(x)
    for t, tok in enumerate(tokens):
        e = table[tok, layer * dim:(layer + 1) * dim]
        y[t] = rms_norm(p["proj"] @ (gelu_tanh(p["gate"] @ x[t]) * e), p["norm"], eps)
    return y


def forward(cfg: Dict[str, Any], tensors: Tensors, tokens: List[int], dtype: torch.dtype = torch.float64,
            trace: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    side = cfg.get("token_side")
    x = W["embed"][torch.tensor(tokens)]
    for li, spec in enumerate(cfg["layers"]):
        pre = f"l{li}."
        mixer = window_attention if spec["type"] == "attention" else channel_delta
        x = x + mult * mixer(rms_norm(x, W[pre + "norm1"], eps), sub(W, pre + "mix."), spec["mixer"], eps)
        mlp = spec.get("mlp")
        if mlp:
            h = rms_norm(x, W[pre + "norm2"], eps)
            y = moe_ff(h, sub(W, pre + "mlp."), mlp) if mlp["kind"] == "moe" else dense_ff(h, sub(W, pre + "mlp."))
            x = x + mult * y
        if side:
            x = x + mult * token_side(x, tokens, W["side.embed"], sub(W, pre + "side."), li, side["dim"], eps)
        if trace is not None:
            trace.append(x.clone())
    return rms_norm(x, W["final.norm"], eps) @ W["head"].T
