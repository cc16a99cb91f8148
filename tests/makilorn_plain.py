"""The Makilorn design written out plainly and slowly, one function per mechanism.

This is the oracle of the Makilorn tests: whole sequences, no cache, no batch, loops over tokens
where the design is a recurrence.  It shares no code with the engine.  Everything is computed in
the dtype of the tensors it is given (tests pass float64 or float32).

Notation.  ``x`` is the residual stream ``[T, width]``; a layer is

    x <- x + N1(mixer(x));  x <- x + N2(ffn(x))          N(y) = y / sqrt(mean(y^2) + eps) * w

The mixers:

* latent attention: ``q = Wq x``; the latent ``c = N(Wdkv x)`` (``kv_rank`` wide); per head
  ``k = Wuk c``, ``v = Wuv c``; token i sees tokens j with ``0 <= i - j < window``; softmax of
  ``scale * q.k``; ``Wo`` over the heads' results side by side.
* gated delta rule: ``q, k, v`` are projections followed by a causal convolution over time per
  channel and silu; q and k become unit vectors per head (``/ sqrt(sum^2 + 1e-6)``), q times
  ``dim^-1/2``; ``beta = sigmoid(Wb x)``; ``g = exp(-exp(A_log) * softplus(Wa x + dt_bias))``; per
  head ``S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q``; o is divided by its root
  mean square over vdim, times a weight, times ``silu(Wg x)``; then ``Wo``.

The feed-forward is a mixture of experts: the ``top`` largest router logits choose, the softmax
over those logits weighs; an expert is ``Wdown(a * sigmoid(1.702 a) * (b + 1))`` with
``a = min(Wgate x, limit)`` and ``b = clamp(Wup x, -limit, limit)``.
"""

from __future__ import annotations

import math
from typing import Any, Mapping

import torch


def rms_norm(y: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + eps) * weight


def silu(z: torch.Tensor) -> torch.Tensor:
    return z / (1.0 + torch.exp(-z))


def latent_attention(x: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, mixer: Mapping[str, Any], eps: float) -> torch.Tensor:
    heads, dim, vdim = mixer["heads"], mixer["dim"], mixer["vdim"]
    window, scale = mixer["mask"]["size"], mixer["scale"]
    T = x.shape[0]
    q = (x @ w[f"{p}.q"].T).view(T, heads, dim)
    c = rms_norm(x @ w[f"{p}.dkv"].T, w[f"{p}.dkv.norm"], eps)
    k = (c @ w[f"{p}.uk"].T).view(T, heads, dim)
    v = (c @ w[f"{p}.uv"].T).view(T, heads, vdim)
    out = torch.zeros(T, heads, vdim, dtype=x.dtype)
    for i in range(T):
        lo = max(0, i - window + 1)
        for h in range(heads):
            s = (k[lo : i + 1, h] @ q[i, h]) * scale
            s = torch.exp(s - s.max())
            out[i, h] = (s / s.sum()) @ v[lo : i + 1, h]
    return out.reshape(T, heads * vdim) @ w[f"{p}.o"].T


def causal_conv(z: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """z [T, C], taps [C, n]: out[t, c] = sum_j taps[c, n-1-j] z[t-j, c], zeros before the start."""
    T, _ = z.shape
    n = taps.shape[1]
    out = torch.zeros_like(z)
    for t in range(T):
        for j in range(n):
            if t - j >= 0:
                out[t] += taps[:, n - 1 - j] * z[t - j]
    return out


def gated_delta(x: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, mixer: Mapping[str, Any], eps: float) -> torch.Tensor:
    heads, kv_heads, dim, vdim = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    T = x.shape[0]
    q = silu(causal_conv(x @ w[f"{p}.q"].T, w[f"{p}.q.conv"])).view(T, kv_heads, dim)
    k = silu(causal_conv(x @ w[f"{p}.k"].T, w[f"{p}.k.conv"])).view(T, kv_heads, dim)
    v = silu(causal_conv(x @ w[f"{p}.v"].T, w[f"{p}.v.conv"])).view(T, heads, vdim)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(x @ w[f"{p}.b"].T)
    g = torch.exp(-torch.exp(w[f"{p}.A_log"]) * torch.nn.functional.softplus(x @ w[f"{p}.a"].T + w[f"{p}.dt_bias"]))
    gate = silu(x @ w[f"{p}.g"].T).view(T, heads, vdim)
    out = torch.zeros(T, heads, vdim, dtype=x.dtype)
    share = heads // kv_heads
    for h in range(heads):
        S = torch.zeros(dim, vdim, dtype=x.dtype)
        for t in range(T):
            kt, qt = k[t, h // share], q[t, h // share]
            S = g[t, h] * S
            u = beta[t, h] * (v[t, h] - S.T @ kt)
            S = S + torch.outer(kt, u)
            out[t, h] = S.T @ qt
    out = out / torch.sqrt((out * out).mean(-1, keepdim=True) + eps) * w[f"{p}.norm"] * gate
    return out.reshape(T, heads * vdim) @ w[f"{p}.o"].T


def expert_mixture(x: torch.Tensor, w: Mapping[str, torch.Tensor], p: str, mlp: Mapping[str, Any]) -> torch.Tensor:
    experts, top, limit = mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["limit"]
    z = x @ w[f"{p}.router"].T + w[f"{p}.router.b"]
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        chosen = sorted(range(experts), key=lambda e: (-float(z[t, e]), e))[:top]
        weights = torch.softmax(z[t, chosen], dim=0)
        for weight, e in zip(weights, chosen):
            a = torch.clamp(w[f"{p}.e{e}.gate"] @ x[t], max=limit)
            b = torch.clamp(w[f"{p}.e{e}.up"] @ x[t], min=-limit, max=limit)
            out[t] += weight * (w[f"{p}.e{e}.down"] @ (a * torch.sigmoid(1.702 * a) * (b + 1.0)))
    return out


def forward(config: Mapping[str, Any], weights: Mapping[str, torch.Tensor], tokens, *, dtype=torch.float64, layer_outputs=None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one whole sequence; ``layer_outputs`` (a list) gets x after every layer."""
    w = {name: (t.to(dtype) if t.is_floating_point() else t) for name, t in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.as_tensor(list(tokens), dtype=torch.long)]
    for index, layer in enumerate(config["layers"]):
        p = f"l{layer.get('weights_of', index)}"
        if layer["type"] == "latent_attention":
            mixed = latent_attention(x, w, f"{p}.mix", layer["mixer"], eps)
        elif layer["type"] == "delta":
            mixed = gated_delta(x, w, f"{p}.mix", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(mixed, w[f"{p}.norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + rms_norm(expert_mixture(x, w, f"{p}.mlp", layer["mlp"]), w[f"{p}.norm2"], eps)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T
