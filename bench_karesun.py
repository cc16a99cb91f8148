"""``bench.py --design karesun``: prefill and decode throughput of the Karesun design at a few layer
sizes, beside the dense Llama decoder of the same width, layer count, value rows per token and
feed-forward rows per token (random bf16 weights, synthetic tokens).  One JSON line; the default
workload of bench.py and its line are untouched by this option.

Eight layers: a layer with keys and values of its own and a dense feed-forward, then a layer that
reads them and has a mixture of experts, four times.  Measured as ``bench_makilorn.py`` measures: a
2,048-token prompt in one step (median of 5 after 3 warm-up steps) and decode steps at batch 8 and 64
over 2,048-token prompts (CUDA events around ``steps`` replayed steps after ``warmup``; every step
reads its layers' weights and the requests' caches, several times the 126 MB L2).
"""

from __future__ import annotations

import json
import sys

from bench_makilorn import LAYERS, PAGE_SIZE, PROMPT, VOCAB, _decode_ms, _engine, _prefill_ms

# width, query heads, key/value heads, experts with weights, identity experts, experts a token, expert rows
SIZES = {
    "w2048": dict(width=2048, heads=16, kv_heads=4, experts=30, identity=2, top=4, ff=1024),
    "w4096": dict(width=4096, heads=32, kv_heads=8, experts=30, identity=2, top=4, ff=2048),
}
WINDOW = 1024


def karesun_config(size: dict) -> dict:
    mixer = {"heads": size["heads"], "kv_heads": size["kv_heads"], "dim": 64, "vdim": 128, "scale": 64 ** -0.5, "softcap": 50.0,
             "diff": 0.4, "mask": {"size": WINDOW}}
    dense = {"kind": "dense", "ff": size["top"] * size["ff"]}
    mixture = {"kind": "moe", "expert": {"ff": size["ff"]},
               "router": {"experts": size["experts"], "identity": size["identity"], "top": size["top"], "scale": 2.0, "groups": {"count": 4, "keep": 2}}}
    layers = []
    for index in range(LAYERS):
        if index % 2 == 0:
            layers.append({"type": "attention", "mixer": dict(mixer), "mlp": dense})
        else:
            layers.append({"type": "attention", "mixer": dict(mixer, kv_from=index - 1), "mlp": mixture})
    return {"architecture": "Karesun", "vocab": VOCAB, "width": size["width"], "max_positions": 4096, "norm": {"eps": 1e-5},
            "embedding": {"scale": 1.0}, "layers": layers}


def dense_config(size: dict) -> dict:
    return {
        "architectures": ["LlamaForCausalLM"], "hidden_size": size["width"], "num_hidden_layers": LAYERS,
        "num_attention_heads": size["heads"], "num_key_value_heads": size["kv_heads"], "head_dim": 128,
        "intermediate_size": size["top"] * size["ff"], "vocab_size": VOCAB, "rope_theta": 500000.0,
        "max_position_embeddings": 8192, "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "hidden_act": "silu",
    }


def run(args) -> int:
    import torch

    if not torch.cuda.is_available():
        print("bench.py: no CUDA device; kairyu_b200 has no CPU path", file=sys.stderr)
        return 1
    torch.cuda.set_device(0)
    steps, warmup = min(args.steps, 64), max(args.warmup, 3)
    sizes = {}
    launches = 0
    for name, size in SIZES.items():
        entry = {}
        for model, config in (("karesun", karesun_config(size)), ("dense", dense_config(size))):
            engine = _engine(config, 64)
            prefill = _prefill_ms(engine)
            result = {"prefill_ms": prefill, "prefill_tokens_per_s": PROMPT / (prefill / 1e3),
                      "weight_bytes_per_decode_token": engine.model.bytes_streamed_per_step()}
            for batch in (8, 64):
                ms, count = _decode_ms(engine, batch, steps, warmup)
                launches += count
                result[f"decode_b{batch}_ms"] = ms
                result[f"decode_b{batch}_tokens_per_s"] = batch / (ms / 1e3)
            entry[model] = result
            del engine
            torch.cuda.empty_cache()
        for what in ("prefill", "decode_b8", "decode_b64"):
            entry[f"{what}_ratio"] = entry["karesun"][f"{what}_tokens_per_s"] / entry["dense"][f"{what}_tokens_per_s"]
        sizes[name] = dict(size, layers=LAYERS, window=WINDOW, **entry)
    print(json.dumps({
        "metric": "karesun_vs_dense_tokens_per_s", "design": "Karesun", "n_gpus": 1, "steps": steps, "warmup": warmup, "dtype": "bf16",
        "data": "synthetic", "gpu_launches": launches,
        "config": {"prompt_len": PROMPT, "page_size": PAGE_SIZE, "layers": LAYERS, "inputs": "weights and caches larger than L2"},
        "sizes": sizes,
    }))
    return 0
