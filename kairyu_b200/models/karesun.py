"""Karesun: a pre-norm decoder of differential-attention layers with learned positions, whose
``config.json`` lists its layers one by one.

``x = embed[token] * embedding.scale + pos[position]``; a layer is ``x += mixer(norm1(x)); x += ff(norm2(x))``
with RMS norms whose weights are stored around zero (``1 + w``); the mixer is differential attention
(two softmax maps a head over the same values, soft-capped scores, a sliding window, no rotation;
``kairyu_b200/parts/diff_attention.py``); the feed-forward is dense (``down(relu(up x)^2)``), a mixture
of experts routed by scores with groups, a choice correction and identity experts
(``kairyu_b200/parts/moe.py``), or absent.  A layer whose mixer names ``kv_from: j`` has no key and value
projections: it reads the keys and values layer j cached in the same step.  In the spec that is a
``LayerCall`` on layer j's cache slot with ``writes_cache=False``; the slot keeps as many positions as the
widest window among its readers needs.

config.json keys::

    architecture: "Karesun"    vocab, width, max_positions    norm: {eps}    embedding: {scale}
    layers: [ {type: "attention", mixer: {...}, mlp: {...} | null}, ... ]
      mixer: heads, kv_heads, dim, vdim, scale, softcap, diff, mask: {size}, kv_from?: j
      mlp:   kind: "dense", ff
             kind: "moe", expert: {ff}, router: {experts, identity, top, scale, groups: {count, keep}}

Tensors: ``embed``, ``pos``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.{q,k,v,o,lq1,lk1,lq2,lk2}``,
``l<i>.mlp.{up,down}`` or ``l<i>.mlp.{router,correction,e<n>.{gate,up,down}}``, ``final.norm``, ``head``
(matrices stored [out, in]).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional

from kairyu_b200.config.model_config import ConfigError
from kairyu_b200.parts.base import LayerCall, LayerSpec, ModelSpec, PartSpec


@dataclass(frozen=True)
class KaresunLayer:
    mixer: Mapping[str, Any]
    mlp: Optional[Mapping[str, Any]]
    kv_from: Optional[int]


@dataclass(frozen=True)
class KaresunConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    norm_eps: float
    embedding_scale: float
    layers: tuple[KaresunLayer, ...]
    max_position_embeddings: int
    eos_token_ids: tuple[int, ...] = ()
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)


def _get(table: Any, key: str, where: str) -> Any:
    if not isinstance(table, Mapping) or key not in table or table[key] is None:
        raise ConfigError(f"config.json: {where} is missing {key!r}")
    return table[key]


def _size(table: Any, key: str, where: str) -> int:
    value = _get(table, key, where)
    if type(value) is not int or value < 1:
        raise ConfigError(f"config.json: {where}.{key} must be an integer >= 1, got {value!r}")
    return value


def _real(table: Any, key: str, where: str) -> float:
    value = _get(table, key, where)
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, got {value!r}")
    return float(value)


def _parse_mixer(mixer: Any, where: str) -> dict[str, Any]:
    parsed = dict(
        heads=_size(mixer, "heads", where), kv_heads=_size(mixer, "kv_heads", where), dim=_size(mixer, "dim", where),
        vdim=_size(mixer, "vdim", where), scale=_real(mixer, "scale", where), diff=_real(mixer, "diff", where),
        softcap=None, window=None,
    )
    if parsed["heads"] % parsed["kv_heads"]:
        raise ConfigError(f"config.json: {where}: heads={parsed['heads']} is not a multiple of kv_heads={parsed['kv_heads']}")
    if mixer.get("softcap") is not None:
        parsed["softcap"] = _real(mixer, "softcap", where)
        if parsed["softcap"] <= 0.0:
            raise ConfigError(f"config.json: {where}.softcap must be positive, got {parsed['softcap']!r}")
    if mixer.get("mask") is not None:
        parsed["window"] = _size(mixer["mask"], "size", f"{where}.mask")
    return parsed


def _parse_mlp(mlp: Any, where: str) -> Optional[dict[str, Any]]:
    if mlp is None:
        return None
    kind = _get(mlp, "kind", where)
    if kind == "dense":
        return dict(kind="dense", ff=_size(mlp, "ff", where))
    if kind != "moe":
        raise ConfigError(f"config.json: {where}: unknown feed-forward kind {kind!r} (dense, moe)")
    router = _get(mlp, "router", where)
    at = f"{where}.router"
    identity = router.get("identity") or 0
    if type(identity) is not int or identity < 0:
        raise ConfigError(f"config.json: {at}.identity must be an integer >= 0, got {identity!r}")
    groups, keep = 1, 1
    if router.get("groups") is not None:
        groups = _size(router["groups"], "count", f"{at}.groups")
        keep = _size(router["groups"], "keep", f"{at}.groups")
    parsed = dict(
        kind="moe", experts=_size(router, "experts", at), identity=identity, top=_size(router, "top", at),
        route_scale=_real(router, "scale", at) if router.get("scale") is not None else 1.0, groups=groups, keep=keep,
        ff=_size(_get(mlp, "expert", where), "ff", f"{where}.expert"),
    )
    outputs = parsed["experts"] + identity
    if outputs % groups or keep > groups:
        raise ConfigError(f"config.json: {at}: {outputs} router outputs do not form {groups} equal groups of which {keep} stay")
    if parsed["top"] > keep * (outputs // groups):
        raise ConfigError(f"config.json: {at}: top={parsed['top']} of the {keep * (outputs // groups)} outputs that stay")
    return parsed


def parse_karesun(config: Mapping[str, Any]) -> KaresunConfig:
    entries = _get(config, "layers", "the file")
    if not isinstance(entries, list) or not entries:
        raise ConfigError("config.json: layers must be a non-empty list")
    layers: list[KaresunLayer] = []
    for index, entry in enumerate(entries):
        where = f"layers[{index}]"
        kind = _get(entry, "type", where)
        if kind != "attention":
            raise ConfigError(f"config.json: {where}: unknown layer type {kind!r} (attention)")
        mixer = _get(entry, "mixer", where)
        source = mixer.get("kv_from")
        if source is not None:
            if type(source) is not int or not 0 <= source < index:
                raise ConfigError(f"config.json: {where}.mixer.kv_from must name an earlier layer, got {source!r}")
            if layers[source].kv_from is not None:
                raise ConfigError(f"config.json: {where}.mixer.kv_from names layer {source}, which has no keys and values of its own")
        parsed = _parse_mixer(mixer, f"{where}.mixer")
        if source is not None:
            theirs = layers[source].mixer
            for key in ("heads", "kv_heads", "dim", "vdim"):
                if theirs[key] != parsed[key]:
                    raise ConfigError(f"config.json: {where}.mixer.{key}={parsed[key]} differs from layer {source}'s {theirs[key]}, whose keys and values it reads")
        layers.append(KaresunLayer(parsed, _parse_mlp(entry.get("mlp"), f"{where}.mlp"), source))
    eos = config.get("eos_token_id")
    return KaresunConfig(
        architecture="Karesun",
        vocab_size=_size(config, "vocab", "the file"),
        hidden_size=_size(config, "width", "the file"),
        norm_eps=_real(_get(config, "norm", "the file"), "eps", "norm"),
        embedding_scale=_real(config["embedding"], "scale", "embedding") if isinstance(config.get("embedding"), Mapping) and config["embedding"].get("scale") is not None else 1.0,
        layers=tuple(layers),
        max_position_embeddings=_size(config, "max_positions", "the file"),
        eos_token_ids=(eos,) if type(eos) is int else tuple(eos) if isinstance(eos, list) else (),
        raw=dict(config),
    )


def _kept_positions(index: int, config: KaresunConfig) -> Optional[int]:
    """How many positions layer ``index``'s cache slot keeps: the widest window among the layer and
    those that read its keys and values; None (all) if one of them sees everything."""
    windows = [layer.mixer["window"] for at, layer in enumerate(config.layers) if at == index or layer.kv_from == index]
    return None if any(window is None for window in windows) else max(windows)


def _layer_spec(index: int, layer: KaresunLayer, config: KaresunConfig) -> LayerSpec:
    prefix = f"l{index}"
    width, eps = config.hidden_size, config.norm_eps
    m = layer.mixer
    mixer = PartSpec(
        "differential_attention", prefix=f"{prefix}.mix", hidden_size=width, num_heads=m["heads"], num_kv_heads=m["kv_heads"],
        head_dim=m["dim"], value_dim=m["vdim"], scale=m["scale"], softcap=m["softcap"], lam_init=m["diff"], window=m["window"],
        keep=_kept_positions(index, config) if layer.kv_from is None else None, own_kv=layer.kv_from is None, norm_eps=eps,
    )
    ffn = ffn_norm = None
    if layer.mlp is not None:
        f = layer.mlp
        if f["kind"] == "dense":
            ffn = PartSpec("mlp", prefix=f"{prefix}.mlp", hidden_size=width, intermediate_size=f["ff"], activation="relu2")
        else:
            ffn = PartSpec(
                "moe", prefix=f"{prefix}.mlp", hidden_size=width, intermediate_size=f["ff"], num_experts=f["experts"],
                num_identity=f["identity"], top=f["top"], routing="scores", groups=f["groups"], groups_keep=f["keep"],
                route_scale=f["route_scale"], limit=None, alpha=1.0, shift=0.0, router_bias=False,
            )
        ffn_norm = PartSpec("rmsnorm", name=f"{prefix}.norm2", size=width, eps=eps, offset=1.0)
    return LayerSpec(
        prefix=prefix, block="pre_norm", mixer=mixer, ffn=ffn,
        mixer_norm=PartSpec("rmsnorm", name=f"{prefix}.norm1", size=width, eps=eps, offset=1.0), ffn_norm=ffn_norm,
    )


def karesun_spec(config: KaresunConfig) -> ModelSpec:
    specs = tuple(_layer_spec(index, layer, config) for index, layer in enumerate(config.layers))
    # a layer that reads another's keys and values runs on that layer's cache slot without writing it
    schedule = tuple(
        LayerCall(layer=index, cache_slot=index if layer.kv_from is None else layer.kv_from, writes_cache=layer.kv_from is None)
        for index, layer in enumerate(config.layers)
    )
    width = config.hidden_size
    return ModelSpec(
        embedding=PartSpec("token_embedding", name="embed", vocab_size=config.vocab_size, hidden_size=width, scale=config.embedding_scale),
        layers=specs,
        schedule=schedule,
        final_norm=PartSpec("rmsnorm", name="final.norm", size=width, eps=config.norm_eps, offset=1.0),
        head=PartSpec("linear_head", name="head", vocab_size=config.vocab_size, hidden_size=width, tied_to=None),
        vocab_size=config.vocab_size,
        hidden_size=width,
        max_position_embeddings=config.max_position_embeddings,
        embedding_position=PartSpec("learned", name="pos", max_positions=config.max_position_embeddings, hidden_size=width),
    )
