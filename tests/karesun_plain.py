"""The Karesun design written out plainly and slowly, one function per mechanism.

This is the oracle of the Karesun tests: whole sequences, no cache, no batch, loops over tokens and
heads.  It shares no code with the engine.  Everything is computed in the dtype of the tensors it is
given (tests pass float64).

Notation.  ``x`` is the residual stream ``[T, width]``, token t at position t.

    x_t = E[token_t] * s_E + P[t]
    x <- x + mixer(N1(x));  x <- x + ff(N2(x))           N(y) = y / sqrt(mean(y^2) + eps) * (1 + w)
    logits = head N_final(x)

Mixer (differential attention).  Query head h has two queries ``q1, q2`` (the rows of ``Wq`` go head
by head, a head's first ``dim`` rows are map 1); key/value head ``g = h // (H / G)`` has two keys
``k1, k2`` the same way and one value ``v``.  Token i sees tokens j with ``0 <= i - j < window``.  Per
map ``s = q.k * scale``, ``s <- cap * tanh(s / cap)``, ``p = softmax_j s``, ``a = sum_j p_j v_j``.  With
``lam = exp(lq1.lk1) - exp(lq2.lk2) + lam0``: ``o = a1 - lam a2``, then ``o / sqrt(mean(o^2) + eps) * (1 - lam0)``,
heads side by side, ``Wo``.  A layer with ``kv_from: j`` uses layer j's keys and values.

Feed-forward.  Dense: ``Wdown relu(Wup y)^2``.  Mixture: ``s = softmax(Wr y)`` over all router outputs
(the last ``identity`` of them are identity experts), ``c = s + correction``; the outputs form
``groups.count`` equal runs; the ``groups.keep`` runs with the largest ``max c`` stay; the ``top`` largest ``c``
that stay are chosen; output ``sum_e s_e * router.scale * f_e(y)`` with ``f_e(y) = Wdown (silu(Wgate y) * Wup y)``
or ``y`` itself for an identity expert.
"""

from __future__ import annotations

import math
from typing import Any, Mapping, Optional

import torch


def norm(y: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + eps) * (1.0 + weight)


def embed(tokens, weights: Mapping[str, torch.Tensor], scale: float) -> torch.Tensor:
    rows = [weights["embed"][token] * scale + weights["pos"][position] for position, token in enumerate(tokens)]
    return torch.stack(rows)


def lam_of(weights: Mapping[str, torch.Tensor], prefix: str, lam0: float) -> float:
    first = math.exp(float((weights[f"{prefix}.lq1"] * weights[f"{prefix}.lk1"]).sum()))
    second = math.exp(float((weights[f"{prefix}.lq2"] * weights[f"{prefix}.lk2"]).sum()))
    return first - second + lam0


def one_map(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, cap: Optional[float], window: Optional[int]) -> torch.Tensor:
    """q, k [T, dim], v [T, vdim]: a softmax map token by token."""
    out = []
    for i in range(q.shape[0]):
        first = 0 if window is None else max(0, i - window + 1)
        s = (k[first : i + 1] @ q[i]) * scale
        if cap is not None:
            s = cap * torch.tanh(s / cap)
        p = torch.softmax(s, dim=0)
        out.append(p @ v[first : i + 1])
    return torch.stack(out)


def keys_and_values(y: torch.Tensor, weights: Mapping[str, torch.Tensor], prefix: str, m: Mapping[str, Any]):
    T = y.shape[0]
    k = (y @ weights[f"{prefix}.k"].T).view(T, m["kv_heads"], 2, m["dim"])
    v = (y @ weights[f"{prefix}.v"].T).view(T, m["kv_heads"], m["vdim"])
    return k, v


def differential_attention(y: torch.Tensor, weights: Mapping[str, torch.Tensor], prefix: str, m: Mapping[str, Any], eps: float,
                           k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    T = y.shape[0]
    heads, group = m["heads"], m["heads"] // m["kv_heads"]
    q = (y @ weights[f"{prefix}.q"].T).view(T, heads, 2, m["dim"])
    lam = lam_of(weights, prefix, m["diff"])
    window = m["mask"]["size"] if m.get("mask") else None
    outs = []
    for h in range(heads):
        g = h // group
        a1 = one_map(q[:, h, 0], k[:, g, 0], v[:, g], m["scale"], m.get("softcap"), window)
        a2 = one_map(q[:, h, 1], k[:, g, 1], v[:, g], m["scale"], m.get("softcap"), window)
        o = a1 - lam * a2
        outs.append(o / torch.sqrt((o * o).mean(dim=-1, keepdim=True) + eps) * (1.0 - m["diff"]))
    return torch.cat(outs, dim=-1) @ weights[f"{prefix}.o"].T


def dense_ff(y: torch.Tensor, weights: Mapping[str, torch.Tensor], prefix: str) -> torch.Tensor:
    return torch.relu(y @ weights[f"{prefix}.up"].T) ** 2 @ weights[f"{prefix}.down"].T


def route(y: torch.Tensor, weights: Mapping[str, torch.Tensor], prefix: str, router: Mapping[str, Any]):
    """Per token: the chosen router outputs and their weights."""
    outputs = router["experts"] + router.get("identity", 0)
    groups = router.get("groups") or {"count": 1, "keep": 1}
    per = outputs // groups["count"]
    chosen, mix = [], []
    for t in range(y.shape[0]):
        s = torch.softmax(weights[f"{prefix}.router"] @ y[t], dim=0)
        c = s + weights[f"{prefix}.correction"]
        values = [float(c[g * per : (g + 1) * per].max()) for g in range(groups["count"])]
        kept = sorted(range(groups["count"]), key=lambda g: (-values[g], g))[: groups["keep"]]
        allowed = [e for e in range(outputs) if e // per in kept]
        best = sorted(allowed, key=lambda e: (-float(c[e]), e))[: router["top"]]
        chosen.append(best)
        mix.append([s[e] * router.get("scale", 1.0) for e in best])
    return chosen, mix


def expert(y: torch.Tensor, weights: Mapping[str, torch.Tensor], prefix: str, e: int) -> torch.Tensor:
    gate = weights[f"{prefix}.e{e}.gate"] @ y
    up = weights[f"{prefix}.e{e}.up"] @ y
    return weights[f"{prefix}.e{e}.down"] @ (gate / (1.0 + torch.exp(-gate)) * up)


def expert_mixture(y: torch.Tensor, weights: Mapping[str, torch.Tensor], prefix: str, mlp: Mapping[str, Any]) -> torch.Tensor:
    router = mlp["router"]
    chosen, mix = route(y, weights, prefix, router)
    rows = []
    for t in range(y.shape[0]):
        total = torch.zeros_like(y[t])
        for e, weight in zip(chosen[t], mix[t]):
            total = total + weight * (y[t] if e >= router["experts"] else expert(y[t], weights, prefix, e))
        rows.append(total)
    return torch.stack(rows)


def forward(cfg: Mapping[str, Any], weights: Mapping[str, torch.Tensor], tokens, dtype: torch.dtype = torch.float64,
            residuals: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence."""
    w = {name: t.to(dtype) for name, t in weights.items()}
    eps = cfg["norm"]["eps"]
    x = embed(tokens, w, (cfg.get("embedding") or {}).get("scale", 1.0))
    cached = {}
    for index, entry in enumerate(cfg["layers"]):
        prefix, m = f"l{index}", entry["mixer"]
        y = norm(x, w[f"{prefix}.norm1"], eps)
        if m.get("kv_from") is None:
            cached[index] = keys_and_values(y, w, f"{prefix}.mix", m)
        k, v = cached[index if m.get("kv_from") is None else m["kv_from"]]
        x = x + differential_attention(y, w, f"{prefix}.mix", m, eps, k, v)
        if entry.get("mlp") is not None:
            y = norm(x, w[f"{prefix}.norm2"], eps)
            x = x + (dense_ff(y, w, f"{prefix}.mlp") if entry["mlp"]["kind"] == "dense" else expert_mixture(y, w, f"{prefix}.mlp", entry["mlp"]))
        if residuals is not None:
            residuals.append(x.clone())
    return norm(x, w["final.norm"], eps) @ w["head"].T
