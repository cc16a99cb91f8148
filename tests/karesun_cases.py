"""Small Karesun configurations and weights for the tests.

The weights are drawn so that a fault shows: queries and keys are large enough for the two softmax
maps to pick single keys (a window one token off, a cap left out or a wrong key/value head then
moves the result by far more than rounding), the vectors behind lambda make it differ from its
constant, corrections are of the size of the scores (so they change the choice, and would change the
weights if they entered them), routers spread their logits.  The configurations differ in every size:
heads and key/value heads (one, several, as many as heads), key and value widths (equal, wider,
narrower, no multiple of 8), windows that are no multiple of a page and one of a single token, a
layer that sees everything, readers of another layer's keys and values with a wider and a narrower
window than the writer's, layers without a feed-forward, mixtures with and without identity experts
and groups, all experts chosen, one expert of one.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Mapping, Optional

import torch
from safetensors.torch import save_file


def attention(heads, kv_heads, dim, vdim, window, scale, softcap, diff, kv_from=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if window is not None:
        mixer["mask"] = {"size": window}
    if softcap is not None:
        mixer["softcap"] = softcap
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return mixer


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, identity, top, ff, scale, groups=None):
    router = {"experts": experts, "identity": identity, "top": top, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "router": router, "expert": {"ff": ff}}


def layer(mixer, mlp):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def config(width, vocab, layers, max_positions=512, eps=1e-5, embed_scale=0.7):
    return {"architecture": "Karesun", "vocab": vocab, "width": width, "max_positions": max_positions, "norm": {"eps": eps},
            "embedding": {"scale": embed_scale}, "layers": layers}


# name -> (config, seed, page size)
CASES: dict[str, tuple[dict, int, int]] = {
    # widths of 16 and 32: the tensor-core kernel in bfloat16; a reader with a wider window than its writer's,
    # one with a far wider window than the prompts; a layer without feed-forward
    "shared": (config(48, 97, [
        layer(attention(4, 2, 16, 32, 21, 0.25, 6.0, 0.3), moe(6, 2, 3, 24, 1.7, groups=(4, 2))),
        layer(attention(4, 2, 16, 32, 37, 0.3, 4.0, 0.6, kv_from=0), dense(40)),
        layer(attention(2, 2, 32, 16, 9, 0.2, None, 0.2), None),
        layer(attention(2, 2, 32, 16, 150, 0.35, 20.0, 0.45, kv_from=2), moe(3, 0, 1, 40, 1.0)),
    ]), 31, 8),
    # nothing a multiple of 8: the 32-bit-arithmetic kernel in both modes; every router output chosen; a window of one
    "odd": (config(50, 77, [
        layer(attention(3, 1, 10, 14, 13, 0.4, 5.0, 0.35), moe(3, 1, 4, 18, 0.9, groups=(1, 1))),
        layer(attention(3, 3, 6, 20, 1, 0.5, 3.0, 0.5), dense(30)),
        layer(attention(3, 1, 10, 14, 30, 0.4, None, 0.1, kv_from=0), None),
    ], embed_scale=2.0), 32, 16),
    # the widest keys and values the tensor-core kernel takes, three query heads a key/value head
    "wide": (config(64, 131, [
        layer(attention(2, 1, 64, 128, 70, 0.15, 8.0, 0.4), dense(96)),
        layer(attention(3, 1, 128, 64, 33, 0.1, 10.0, 0.25), moe(5, 3, 2, 48, 2.5, groups=(2, 1))),
    ], embed_scale=1.0), 33, 16),
    # pages of four; widths 48 and 80 (padded inside the kernel); a layer that sees everything; one expert of one
    "small_pages": (config(32, 61, [
        layer(attention(6, 2, 16, 16, 5, 0.3, 7.0, 0.3), moe(1, 0, 1, 16, 1.3)),
        layer(attention(1, 1, 48, 80, None, 0.2, 5.0, 0.55), dense(24)),
        layer(attention(6, 2, 16, 16, 11, 0.3, 2.0, 0.7, kv_from=0), moe(4, 2, 2, 8, 1.0, groups=(2, 1))),
    ]), 34, 4),
}


def _normal(generator, shape, std):
    return torch.randn(shape, generator=generator, dtype=torch.float32) * std


def make_weights(cfg: Mapping[str, Any], seed: int) -> dict[str, torch.Tensor]:
    """fp32 tensors whose values are exact in bfloat16 (a model folder written in either dtype holds the same numbers)."""
    g = torch.Generator().manual_seed(seed)
    width, vocab = cfg["width"], cfg["vocab"]
    w: dict[str, torch.Tensor] = {
        "embed": _normal(g, (vocab, width), 1.0), "pos": _normal(g, (cfg["max_positions"], width), 0.5),
        "final.norm": _normal(g, (width,), 0.1), "head": _normal(g, (vocab, width), width ** -0.5),
    }
    for index, entry in enumerate(cfg["layers"]):
        p, m = f"l{index}", entry["mixer"]
        heads, kvh, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        w[f"{p}.norm1"] = _normal(g, (width,), 0.1)
        gain = (3.0 / m["scale"]) ** 0.5  # scores of a few units: the softmax picks single keys and the cap bends them
        w[f"{p}.mix.q"] = _normal(g, (heads * 2 * dim, width), gain * width ** -0.5 * dim ** -0.25)
        if m.get("kv_from") is None:
            w[f"{p}.mix.k"] = _normal(g, (kvh * 2 * dim, width), gain * width ** -0.5 * dim ** -0.25)
            w[f"{p}.mix.v"] = _normal(g, (kvh * vdim, width), width ** -0.5)
        for name in ("lq1", "lk1", "lq2", "lk2"):
            w[f"{p}.mix.{name}"] = _normal(g, (dim,), 0.6 * dim ** -0.25)
        w[f"{p}.mix.o"] = _normal(g, (width, heads * vdim), (heads * vdim) ** -0.5)
        mlp = entry["mlp"]
        if mlp is None:
            continue
        w[f"{p}.norm2"] = _normal(g, (width,), 0.1)
        if mlp["kind"] == "dense":
            w[f"{p}.mlp.up"] = _normal(g, (mlp["ff"], width), 1.2 * width ** -0.5)
            w[f"{p}.mlp.down"] = _normal(g, (width, mlp["ff"]), mlp["ff"] ** -0.5)
            continue
        router, ff = mlp["router"], mlp["expert"]["ff"]
        outputs = router["experts"] + router["identity"]
        for e in range(router["experts"]):
            w[f"{p}.mlp.e{e}.gate"] = _normal(g, (ff, width), 1.5 * width ** -0.5)
            w[f"{p}.mlp.e{e}.up"] = _normal(g, (ff, width), 1.5 * width ** -0.5)
            w[f"{p}.mlp.e{e}.down"] = _normal(g, (width, ff), ff ** -0.5)
        w[f"{p}.mlp.router"] = _normal(g, (outputs, width), 2 * width ** -0.5)
        w[f"{p}.mlp.correction"] = _normal(g, (outputs,), 0.5 / outputs)
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
