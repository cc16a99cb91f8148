"""``bench.py --design makilorn``: prefill and decode throughput of the Makilorn design at a few
layer sizes, beside the dense Llama decoder of the same width, layer count and feed-forward rows per
token (random bf16 weights, synthetic tokens).  One JSON line; the default workload of bench.py
and its line are untouched by this option.

Per size and model: a 2,048-token prompt in one step (median of 5 after 3 warm-up steps) and
decode steps at batch 8 and 64 over 2,048-token prompts (CUDA events around ``steps`` replayed
steps after ``warmup``; every step reads its layers' weights and the requests' caches, several
times the 126 MB L2).
"""

from __future__ import annotations

import json
import statistics
import sys

PAGE_SIZE = 16
PROMPT = 2048
VOCAB = 32000

# width, heads, experts, top, expert rows; eight layers: latent, latent, latent, delta, twice
SIZES = {
    "w2048": dict(width=2048, heads=16, experts=32, top=4, ff=1024),
    "w4096": dict(width=4096, heads=32, experts=32, top=4, ff=2048),
}
LAYERS = 8


def makilorn_config(size: dict) -> dict:
    width, heads = size["width"], size["heads"]
    mlp = {"kind": "moe", "router": {"experts": size["experts"], "top": size["top"]}, "expert": {"ff": size["ff"], "limit": 7.0}}
    attention = {"type": "latent_attention", "mlp": mlp,
                 "mixer": {"heads": heads, "dim": 128, "vdim": 128, "kv_rank": 128, "scale": 128 ** -0.5, "mask": {"size": 1024}}}
    recurrent = {"type": "delta", "mlp": mlp, "mixer": {"heads": heads, "kv_heads": heads // 2, "dim": 128, "vdim": 128, "conv": 4}}
    return {"architecture": "Makilorn", "vocab": VOCAB, "width": width, "norm": {"eps": 1e-5},
            "layers": [recurrent if index % 4 == 3 else attention for index in range(LAYERS)]}


def dense_config(size: dict) -> dict:
    return {
        "architectures": ["LlamaForCausalLM"], "hidden_size": size["width"], "num_hidden_layers": LAYERS,
        "num_attention_heads": size["heads"], "num_key_value_heads": max(size["heads"] // 4, 1), "head_dim": 128,
        "intermediate_size": size["top"] * size["ff"], "vocab_size": VOCAB, "rope_theta": 500000.0,
        "max_position_embeddings": 8192, "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "hidden_act": "silu",
    }


def _engine(config: dict, max_batch: int):
    from kairyu_b200.config.engine_config import EngineConfig
    from kairyu_b200.engine.engine import Engine

    per_request = -(-(PROMPT + 256) // PAGE_SIZE)
    options = EngineConfig(dtype="bfloat16", page_size=PAGE_SIZE, num_pages=max_batch * per_request + 1, max_num_batched_tokens=PROMPT,
                           max_num_seqs=max_batch, max_model_len=PROMPT + 256, seed=1)
    return Engine.from_random(config, 1, options)


def _tokens(count: int, seed: int) -> list[int]:
    import torch

    return torch.randint(0, VOCAB, (count,), generator=torch.Generator().manual_seed(seed)).tolist()


def _prefill_ms(engine) -> float:
    import torch

    from kairyu_b200.engine.runner import StepEntry

    tokens = _tokens(PROMPT, 7)
    times = []
    for index in range(8):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        engine.runner.step([StepEntry("prefill", tokens, (PROMPT - 1,))])
        stop.record()
        torch.cuda.synchronize()
        engine.cache.release("prefill")
        if index >= 3:
            times.append(start.elapsed_time(stop))
    return statistics.median(times)


def _decode_ms(engine, batch: int, steps: int, warmup: int) -> tuple[float, int]:
    import torch

    from kairyu_b200.engine.runner import StepEntry

    runner = engine.runner
    names = [f"d{index}" for index in range(batch)]
    for index, name in enumerate(names):
        runner.step([StepEntry(name, _tokens(PROMPT, 100 + index), ())])
    feed = [_tokens(batch, 1000 + step) for step in range(warmup + steps)]

    def one(step: int) -> None:
        runner.step([StepEntry(name, [feed[step][index]], (0,)) for index, name in enumerate(names)])

    for step in range(warmup):
        one(step)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    before = runner.counters["kernel_launches"]
    torch.cuda.synchronize()
    start.record()
    for step in range(warmup, warmup + steps):
        one(step)
    stop.record()
    torch.cuda.synchronize()
    runner.check_errors()
    launches = runner.counters["kernel_launches"] - before
    for name in names:
        engine.cache.release(name)
    return start.elapsed_time(stop) / steps, launches


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
        for model, config in (("makilorn", makilorn_config(size)), ("dense", dense_config(size))):
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
        entry["prefill_ratio"] = entry["makilorn"]["prefill_tokens_per_s"] / entry["dense"]["prefill_tokens_per_s"]
        entry["decode_b8_ratio"] = entry["makilorn"]["decode_b8_tokens_per_s"] / entry["dense"]["decode_b8_tokens_per_s"]
        entry["decode_b64_ratio"] = entry["makilorn"]["decode_b64_tokens_per_s"] / entry["dense"]["decode_b64_tokens_per_s"]
        sizes[name] = dict(size, layers=LAYERS, **entry)
    print(json.dumps({
        "metric": "makilorn_vs_dense_tokens_per_s", "design": "Makilorn", "n_gpus": 1, "steps": steps, "warmup": warmup, "dtype": "bf16",
        "data": "synthetic", "gpu_launches": launches,
        "config": {"prompt_len": PROMPT, "page_size": PAGE_SIZE, "layers": LAYERS, "inputs": "weights and caches larger than L2"},
        "sizes": sizes,
    }))
    return 0
