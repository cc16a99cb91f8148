"""Small Makilorn configurations and weights for the tests.

The weights are drawn so that a fault shows: queries and keys are large enough for the softmax to
pick single keys (a window that is one token off then changes the result by far more than
rounding), decays differ per head, routers spread their logits.  Sizes differ between the
configurations in every respect: heads and query/key heads, key and value widths, taps, windows
that are no multiple of a page, ranks that select each of the attention kernels, a layer without a
feed-forward, layers that run another layer's weights.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Mapping

import torch
from safetensors.torch import save_file


def latent(heads, dim, vdim, rank, window, scale):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "mask": {"size": window}, "scale": scale}}


def delta(heads, kv_heads, dim, vdim, conv):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def moe(experts, top, ff, limit):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}


def layer(mixer, mlp, weights_of=None):
    entry = dict(mixer, mlp=mlp)
    if weights_of is not None:
        entry["weights_of"] = weights_of
    return entry


def config(width, vocab, layers, eps=1e-5):
    return {"architecture": "Makilorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


# name -> (config, seed, page size)
CASES: dict[str, tuple[dict, int, int]] = {
    # rank 40: no tensor-core attention takes it, so bfloat16 runs the fp32-arithmetic kernel too;
    # a layer without feed-forward; two layers on other layers' weights
    "mixed": (config(48, 97, [
        layer(latent(3, 16, 24, 40, 21, 0.45), moe(5, 2, 24, 1.25)),
        layer(delta(4, 2, 32, 24, 3), None),
        layer(latent(3, 16, 24, 40, 21, 0.45), moe(5, 2, 24, 1.25), weights_of=0),
        layer(delta(4, 2, 32, 24, 3), None, weights_of=1),
        layer(delta(1, 1, 16, 40, 2), moe(3, 1, 40, 0.75)),
    ]), 11, 8),
    # rank 64, pages of 16: the tcgen05 prefill and the TMA decode attention in bfloat16
    "rank64": (config(64, 131, [
        layer(latent(2, 32, 16, 64, 37, 0.3), moe(4, 3, 48, 2.0)),
        layer(delta(2, 1, 72, 48, 5), moe(4, 3, 48, 2.0)),
        layer(latent(5, 8, 8, 64, 9, 0.7), None),
    ]), 12, 16),
    # nothing a multiple of 8: rows that start on no 16-byte boundary, the scalar paths of every kernel
    "odd": (config(50, 77, [
        layer(latent(3, 10, 14, 36, 13, 0.4), moe(3, 2, 18, 1.5)),
        layer(delta(3, 1, 20, 12, 3), moe(5, 3, 10, 2.5)),
        layer(delta(2, 2, 36, 6, 4), None),
        layer(latent(3, 10, 14, 36, 13, 0.4), moe(3, 2, 18, 1.5), weights_of=0),
    ]), 14, 16),
    # rank 32, pages of 4: the mma.sync attention pair; a convolution of one tap (no kept inputs);
    # one expert of one; a window of one (a token sees itself alone)
    "rank32": (config(32, 61, [
        layer(delta(3, 3, 8, 8, 1), moe(1, 1, 16, 1.0)),
        layer(latent(1, 24, 40, 32, 1, 0.5), moe(6, 6, 8, 3.0)),
        layer(latent(4, 8, 8, 32, 150, 0.5), None),
    ]), 13, 4),
}


def _normal(generator, shape, std):
    return torch.randn(shape, generator=generator, dtype=torch.float32) * std


def make_weights(cfg: Mapping[str, Any], seed: int) -> dict[str, torch.Tensor]:
    """fp32 tensors whose values are exact in bfloat16 (so that a model folder written in either
    dtype holds the same numbers)."""
    g = torch.Generator().manual_seed(seed)
    width, vocab = cfg["width"], cfg["vocab"]
    w: dict[str, torch.Tensor] = {"embed": _normal(g, (vocab, width), 1.0), "final.norm": 1 + _normal(g, (width,), 0.1),
                                  "head": _normal(g, (vocab, width), width ** -0.5)}
    for index, entry in enumerate(cfg["layers"]):
        if "weights_of" in entry:
            continue
        p, m = f"l{index}", entry["mixer"]
        w[f"{p}.norm1"] = 1 + _normal(g, (width,), 0.1)
        if entry["type"] == "latent_attention":
            heads, dim, vdim, rank = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
            # scores of a few units: the softmax picks single keys, window edges matter
            gain = (3.0 / m["scale"]) ** 0.5
            w[f"{p}.mix.q"] = _normal(g, (heads * dim, width), gain * width ** -0.5 * dim ** -0.25)
            w[f"{p}.mix.dkv"] = _normal(g, (rank, width), width ** -0.5)
            w[f"{p}.mix.dkv.norm"] = 1 + _normal(g, (rank,), 0.1)
            w[f"{p}.mix.uk"] = _normal(g, (heads * dim, rank), gain * rank ** -0.5 * dim ** -0.25)
            w[f"{p}.mix.uv"] = _normal(g, (heads * vdim, rank), rank ** -0.5)
            w[f"{p}.mix.o"] = _normal(g, (width, heads * vdim), (heads * vdim) ** -0.5)
        else:
            heads, kvh, dim, vdim, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            for name, rows in (("q", kvh * dim), ("k", kvh * dim), ("v", heads * vdim)):
                w[f"{p}.mix.{name}"] = _normal(g, (rows, width), width ** -0.5)
                w[f"{p}.mix.{name}.conv"] = _normal(g, (rows, taps), 0.6)
            w[f"{p}.mix.b"] = _normal(g, (heads, width), 2 * width ** -0.5)
            w[f"{p}.mix.a"] = _normal(g, (heads, width), 2 * width ** -0.5)
            w[f"{p}.mix.A_log"] = _normal(g, (heads,), 1.0) - 1.0
            w[f"{p}.mix.dt_bias"] = _normal(g, (heads,), 1.0)
            w[f"{p}.mix.norm"] = 1 + _normal(g, (vdim,), 0.1)
            w[f"{p}.mix.g"] = _normal(g, (heads * vdim, width), width ** -0.5)
            w[f"{p}.mix.o"] = _normal(g, (width, heads * vdim), (heads * vdim) ** -0.5)
        if entry["mlp"] is not None:
            experts, ff = entry["mlp"]["router"]["experts"], entry["mlp"]["expert"]["ff"]
            w[f"{p}.norm2"] = 1 + _normal(g, (width,), 0.1)
            for e in range(experts):
                w[f"{p}.mlp.e{e}.gate"] = _normal(g, (ff, width), 1.5 * width ** -0.5)
                w[f"{p}.mlp.e{e}.up"] = _normal(g, (ff, width), 1.5 * width ** -0.5)
                w[f"{p}.mlp.e{e}.down"] = _normal(g, (width, ff), ff ** -0.5)
            w[f"{p}.mlp.router"] = _normal(g, (experts, width), 2 * width ** -0.5)
            w[f"{p}.mlp.router.b"] = _normal(g, (experts,), 0.5)
    return {name: t.to(torch.bfloat16).to(torch.float32) for name, t in w.items()}


def write_model(cfg: Mapping[str, Any], weights: Mapping[str, torch.Tensor], folder: Path, dtype: torch.dtype = torch.bfloat16) -> Path:
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    save_file({name: t.to(dtype).contiguous() for name, t in weights.items()}, str(folder / "model.safetensors"))
    return folder


def relative_error(got, want) -> float:
    """Largest over the rows of rms(difference, its mean taken off) / rms(wanted row, its mean taken off)."""
    import numpy as np

    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    ref = want - want.mean(-1, keepdims=True)
    return float((np.sqrt((d * d).mean(-1)) / np.sqrt((ref * ref).mean(-1) + 1e-30)).max())
