"""Makilorn: a decoder whose layers are listed one by one in ``config.json``.

Each entry of ``layers`` names a mixer (``latent_attention``: windowed attention over one cached
latent row a token, no positions; ``delta``: the gated delta rule, a recurrent state per request)
and a feed-forward (a mixture of experts, or none).  The norms sit on the sub-layers' outputs
(``x += norm1(mixer(x)); x += norm2(ffn(x))``).  An entry with ``weights_of: j`` runs layer j's
weights again with a cache or state of its own: in the spec that is one ``LayerSpec`` named by two
``LayerCall`` entries with different cache slots.

config.json keys::

    architecture: "Makilorn"     vocab, width       norm: {eps}
    layers: [ {type, mixer: {...}, mlp: {...} | null, weights_of?: j}, ... ]
      latent_attention mixer: heads, dim, vdim, kv_rank, scale, mask: {size}
      delta mixer:            heads, kv_heads, dim, vdim, conv
      mlp:                    kind: "moe", router: {experts, top}, expert: {ff, limit}

Tensors: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``
(matrices stored [out, in]).  The design has no positions, hence no length limit of its own; the
engine needs one to size its tables and takes ``max_positions`` if the file gives it, else
``DEFAULT_MAX_POSITIONS``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional

from kairyu_b200.config.model_config import ConfigError
from kairyu_b200.parts.base import LayerCall, LayerSpec, ModelSpec, PartSpec

DEFAULT_MAX_POSITIONS = 131072


@dataclass(frozen=True)
class MakilornLayer:
    kind: str  # "latent_attention" | "delta"
    mixer: Mapping[str, Any]
    mlp: Optional[Mapping[str, Any]]
    weights_of: Optional[int]


@dataclass(frozen=True)
class MakilornConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    norm_eps: float
    layers: tuple[MakilornLayer, ...]
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


def _parse_mixer(kind: str, mixer: Any, where: str) -> dict[str, Any]:
    if kind == "latent_attention":
        window = _size(_get(mixer, "mask", where), "size", f"{where}.mask")
        return dict(
            heads=_size(mixer, "heads", where), dim=_size(mixer, "dim", where), vdim=_size(mixer, "vdim", where),
            kv_rank=_size(mixer, "kv_rank", where), scale=_real(mixer, "scale", where), window=window,
        )
    if kind == "delta":
        parsed = dict(
            heads=_size(mixer, "heads", where), kv_heads=_size(mixer, "kv_heads", where), dim=_size(mixer, "dim", where),
            vdim=_size(mixer, "vdim", where), conv=_size(mixer, "conv", where),
        )
        if parsed["heads"] % parsed["kv_heads"]:
            raise ConfigError(f"config.json: {where}: heads={parsed['heads']} is not a multiple of kv_heads={parsed['kv_heads']}")
        return parsed
    raise ConfigError(f"config.json: {where}: unknown layer type {kind!r} (latent_attention, delta)")


def _parse_mlp(mlp: Any, where: str) -> Optional[dict[str, Any]]:
    if mlp is None:
        return None
    kind = _get(mlp, "kind", where)
    if kind != "moe":
        raise ConfigError(f"config.json: {where}: unknown feed-forward kind {kind!r} (moe)")
    router, expert = _get(mlp, "router", where), _get(mlp, "expert", where)
    parsed = dict(
        experts=_size(router, "experts", f"{where}.router"), top=_size(router, "top", f"{where}.router"),
        ff=_size(expert, "ff", f"{where}.expert"), limit=_real(expert, "limit", f"{where}.expert"),
    )
    if parsed["top"] > parsed["experts"]:
        raise ConfigError(f"config.json: {where}: top={parsed['top']} of {parsed['experts']} experts")
    return parsed


def parse_makilorn(config: Mapping[str, Any]) -> MakilornConfig:
    entries = _get(config, "layers", "the file")
    if not isinstance(entries, list) or not entries:
        raise ConfigError("config.json: layers must be a non-empty list")
    layers = []
    for index, entry in enumerate(entries):
        where = f"layers[{index}]"
        kind = _get(entry, "type", where)
        source = entry.get("weights_of")
        if source is not None and (type(source) is not int or not 0 <= source < len(entries) or source == index):
            raise ConfigError(f"config.json: {where}.weights_of must name another layer, got {source!r}")
        layers.append(MakilornLayer(kind, _parse_mixer(kind, _get(entry, "mixer", where), f"{where}.mixer"),
                                    _parse_mlp(entry.get("mlp"), f"{where}.mlp"), source))
    for index, layer in enumerate(layers):
        if layer.weights_of is None:
            continue
        source = layers[layer.weights_of]
        if source.weights_of is not None:
            raise ConfigError(f"config.json: layers[{index}].weights_of names layer {layer.weights_of}, which has no weights of its own")
        if source.kind != layer.kind or (source.mlp is None) != (layer.mlp is None):
            raise ConfigError(f"config.json: layers[{index}] uses layer {layer.weights_of}'s weights but is of another kind")
    limit = config.get("max_positions", DEFAULT_MAX_POSITIONS)
    if type(limit) is not int or limit < 1:
        raise ConfigError(f"config.json: max_positions must be an integer >= 1, got {limit!r}")
    eos = config.get("eos_token_id")
    return MakilornConfig(
        architecture="Makilorn",
        vocab_size=_size(config, "vocab", "the file"),
        hidden_size=_size(config, "width", "the file"),
        norm_eps=_real(_get(config, "norm", "the file"), "eps", "norm"),
        layers=tuple(layers),
        max_position_embeddings=limit,
        eos_token_ids=(eos,) if type(eos) is int else tuple(eos) if isinstance(eos, list) else (),
        raw=dict(config),
    )


def _layer_spec(index: int, layer: MakilornLayer, config: MakilornConfig) -> LayerSpec:
    """``index``: the layer whose tensors these parts bind (the entry's own, or the one it names)."""
    prefix = f"l{index}"
    width, eps = config.hidden_size, config.norm_eps
    m = layer.mixer
    if layer.kind == "latent_attention":
        mixer = PartSpec(
            "latent_attention", prefix=f"{prefix}.mix", hidden_size=width, num_heads=m["heads"], head_dim=m["dim"],
            value_dim=m["vdim"], kv_rank=m["kv_rank"], scale=m["scale"], window=m["window"], norm_eps=eps,
        )
    else:
        mixer = PartSpec(
            "gated_delta", prefix=f"{prefix}.mix", hidden_size=width, num_heads=m["heads"], num_kv_heads=m["kv_heads"],
            head_dim=m["dim"], value_dim=m["vdim"], conv_taps=m["conv"], norm_eps=eps,
        )
    ffn = ffn_norm = None
    if layer.mlp is not None:
        f = layer.mlp
        ffn = PartSpec(
            "moe", prefix=f"{prefix}.mlp", hidden_size=width, intermediate_size=f["ff"], num_experts=f["experts"],
            top=f["top"], limit=f["limit"], alpha=1.702, router_bias=True,
        )
        ffn_norm = PartSpec("rmsnorm", name=f"{prefix}.norm2", size=width, eps=eps)
    return LayerSpec(
        prefix=prefix, block="output_norm", mixer=mixer, ffn=ffn,
        mixer_norm=PartSpec("rmsnorm", name=f"{prefix}.norm1", size=width, eps=eps), ffn_norm=ffn_norm,
    )


def makilorn_spec(config: MakilornConfig) -> ModelSpec:
    # Layers with weights of their own become LayerSpecs; every entry of the file becomes a call with
    # its own cache slot, naming the LayerSpec whose weights it runs.  An entry that uses another's
    # weights with other constants (a window, a scale) gets parts of its own over the same tensors.
    spec_at: dict[LayerSpec, int] = {}
    specs: list[LayerSpec] = []
    calls: list[LayerCall] = []
    for index, layer in enumerate(config.layers):
        spec = _layer_spec(index if layer.weights_of is None else layer.weights_of, layer, config)
        if spec not in spec_at:
            spec_at[spec] = len(specs)
            specs.append(spec)
        calls.append(LayerCall(layer=spec_at[spec], cache_slot=index))
    schedule = tuple(calls)
    width = config.hidden_size
    return ModelSpec(
        embedding=PartSpec("token_embedding", name="embed", vocab_size=config.vocab_size, hidden_size=width),
        layers=tuple(specs),
        schedule=schedule,
        final_norm=PartSpec("rmsnorm", name="final.norm", size=width, eps=config.norm_eps),
        head=PartSpec("linear_head", name="head", vocab_size=config.vocab_size, hidden_size=width, tied_to=None),
        vocab_size=config.vocab_size,
        hidden_size=width,
        max_position_embeddings=config.max_position_embeddings,
    )
