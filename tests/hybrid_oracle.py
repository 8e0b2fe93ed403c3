"""A plain, slow restatement of the Badapel design, one function per mechanism, token by token.

Nothing here is shared with the product path (``mdi_llm_b200.models.hybrid`` and the kernels it calls): no
vectorised scans, no caches, no packed batches.  Every function takes and returns ``float64``/``float32`` torch
tensors on the CPU and loops over time in Python, so what it computes can be read off directly:

* ``layer_norm`` / ``rms_norm``         the two normalisations
* ``rotate_half_pairs``                 rotary positions, pair (i, i + n/2)
* ``latent_attention``                  attention whose keys and values are expanded from a cached latent
* ``gated_linear_attention``            S_t = diag(a_t) S_(t-1) + k_t v_t^T
* ``channel_delta``                     the gated delta rule with per-channel decay and short convolutions
* ``dense_ff``                          erf-GELU feed-forward
* ``forward``                           the whole model (looped span with the re-injection matrix, soft cap)

``forward`` always runs a whole sequence from its first token, which is what makes it an oracle for caches and
states: the product must give the same logits however the tokens were cut into steps.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Tuple

import torch

Tensors = Dict[str, torch.Tensor]


def layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def rotate_half_pairs(x: torch.Tensor, pos: int, n: int, base: float) -> torch.Tensor:
    """Rotate the first ``n`` entries of the vector ``x`` for position ``pos``; the rest pass."""
    out = x.clone()
    half = n // 2
    for i in range(half):
        a = pos * base ** (-2.0 * i / n)
        u, v = x[i], x[i + half]
        out[i] = u * math.cos(a) - v * math.sin(a)
        out[i + half] = v * math.cos(a) + u * math.sin(a)
    return out


def latent_attention(h: torch.Tensor, p: Tensors, m: Dict[str, Any], eps: float) -> torch.Tensor:
    """``h [T, width]`` -> ``[T, width]``; ``p`` holds the mixer's tensors by their short names."""
    T = h.shape[0]
    H, D, R, V, L = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    nrot, base = m["rot"]["dims"], m["rot"]["base"]
    out = torch.zeros(T, H * V, dtype=h.dtype)
    lat: List[torch.Tensor] = []
    kr: List[torch.Tensor] = []
    for t in range(T):
        cq = rms_norm(p["dq"] @ h[t], p["dq.norm"], eps)
        q = (p["uq"] @ cq).view(H, D + R)
        ckv = p["dkv"] @ h[t]
        lat.append(rms_norm(ckv[:L], p["dkv.norm"], eps))
        kr.append(rotate_half_pairs(ckv[L:], t, nrot, base))
        for hd in range(H):
            qn, qr = q[hd, :D], rotate_half_pairs(q[hd, D:], t, nrot, base)
            s = torch.empty(t + 1, dtype=h.dtype)
            vals = []
            for j in range(t + 1):
                kn = p["uk"][hd * D:(hd + 1) * D] @ lat[j]
                vals.append(p["uv"][hd * V:(hd + 1) * V] @ lat[j])
                s[j] = (qn @ kn + qr @ kr[j]) * m["scale"]
            w = torch.softmax(s, 0)
            out[t, hd * V:(hd + 1) * V] = sum(w[j] * vals[j] for j in range(t + 1))
        out[t] = out[t] * torch.sigmoid(p["g"] @ h[t])
    return out @ p["o"].T


def gated_linear_attention(h: torch.Tensor, p: Tensors, m: Dict[str, Any], eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    S = torch.zeros(H, D, V, dtype=h.dtype)
    out = torch.zeros(T, H * V, dtype=h.dtype)
    for t in range(T):
        q = (p["q"] @ h[t]).view(H, D) * D ** -0.5
        k = (p["k"] @ h[t]).view(H, D)
        v = (p["v"] @ h[t]).view(H, V)
        z = (p["a2"] @ (p["a1"] @ h[t]) + p["a2.b"]).view(H, D)
        alpha = torch.sigmoid(z) ** (1.0 / m["tau"])
        for hd in range(H):
            S[hd] = alpha[hd][:, None] * S[hd] + torch.outer(k[hd], v[hd])
            o = S[hd].T @ q[hd]
            out[t, hd * V:(hd + 1) * V] = rms_norm(o, p["norm"], eps)
        out[t] = out[t] * torch.nn.functional.silu(p["g"] @ h[t])
    return out @ p["o"].T


def short_conv_silu(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x [T, C]``, ``w [C, taps]`` (last column multiplies the current token), zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            src = t - (taps - 1 - j)
            if src >= 0:
                y[t] += w[:, j] * x[src]
    return torch.nn.functional.silu(y)


def channel_delta(h: torch.Tensor, p: Tensors, m: Dict[str, Any], eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv_silu(h @ p["q"].T, p["q.conv"]).view(T, G, D)
    k = short_conv_silu(h @ p["k"].T, p["k.conv"]).view(T, G, D)
    v = short_conv_silu(h @ p["v"].T, p["v.conv"]).view(T, H, V)
    S = torch.zeros(H, D, V, dtype=h.dtype)
    out = torch.zeros(T, H * V, dtype=h.dtype)
    for t in range(T):
        beta = torch.sigmoid(p["b"] @ h[t])
        z = (p["a2"] @ (p["a1"] @ h[t]) + p["dt_bias"]).view(H, D)
        gate = torch.sigmoid(p["g2"] @ (p["g1"] @ h[t])).view(H, V)
        for hd in range(H):
            g = hd // (H // G)
            qh = q[t, g] / torch.sqrt((q[t, g] ** 2).sum() + 1e-6) * D ** -0.5
            kh = k[t, g] / torch.sqrt((k[t, g] ** 2).sum() + 1e-6)
            decay = torch.exp(-torch.exp(p["A_log"][hd]) * torch.nn.functional.softplus(z[hd]))
            S[hd] = decay[:, None] * S[hd]
            u = beta[hd] * (v[t, hd] - S[hd].T @ kh)
            S[hd] = S[hd] + torch.outer(kh, u)
            o = S[hd].T @ qh
            out[t, hd * V:(hd + 1) * V] = rms_norm(o, p["norm"], eps) * gate[hd]
    return out @ p["o"].T


def dense_ff(h: torch.Tensor, p: Tensors) -> torch.Tensor:
    a = h @ p["up"].T
    a = 0.5 * a * (1.0 + torch.erf(a / math.sqrt(2.0)))
    return a @ p["down"].T


MIXERS = {"latent_attention": latent_attention, "gla": gated_linear_attention, "channel_delta": channel_delta}


def sub(tensors: Tensors, prefix: str) -> Tensors:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def layer_runs(cfg: Dict[str, Any]) -> List[Tuple[int, bool]]:
    """The order in which layers run, as ``(layer index, first of a pass)``."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, False) for i in range(a)]
    for _ in range(times):
        runs += [(i, i == a) for i in range(a, b)]
    return runs + [(i, False) for i in range(b, n)]


def forward(cfg: Dict[str, Any], tensors: Tensors, tokens: List[int], dtype: torch.dtype = torch.float64,
            trace: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one sequence run from its first token; ``trace`` collects the stream after each run."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = cfg["norm"]["eps"]
    x0 = W["embed"][torch.tensor(tokens)]
    x = x0.clone()
    for li, first in layer_runs(cfg):
        spec = cfg["layers"][li]
        pre = f"l{li}."
        if first:
            x = torch.cat((x, x0), -1) @ W["loop.in"].T
        h = layer_norm(x, W[pre + "norm1"], W[pre + "norm1.b"], eps)
        y = MIXERS[spec["type"]](h, sub(W, pre + "mix."), spec["mixer"], eps)
        x = x + layer_norm(y, W[pre + "norm1b"], W[pre + "norm1b.b"], eps)
        if spec.get("mlp"):
            h = layer_norm(x, W[pre + "norm2"], W[pre + "norm2.b"], eps)
            y = dense_ff(h, sub(W, pre + "mlp."))
            x = x + layer_norm(y, W[pre + "norm2b"], W[pre + "norm2b.b"], eps)
        if trace is not None:
            trace.append(x.clone())
    x = layer_norm(x, W["final.norm"], W["final.norm.b"], eps)
    logits = x @ W["embed"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits
