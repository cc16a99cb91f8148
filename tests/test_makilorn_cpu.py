"""Makilorn without a GPU: the config reader, the spec it builds (run order, weight sharing, cache
groups and state), model folders written and read back, and what the GPU tests' bounds can see."""

import json

import numpy as np
import pytest
import torch

import makilorn_plain as plain
import traces
from makilorn_cases import CASES, config, delta, latent, layer, make_weights, moe, relative_error, write_model

from kairyu_b200.cache import CacheLayout
from kairyu_b200.config.model_config import ConfigError
from kairyu_b200.engine.engine import build_model
from kairyu_b200.parts import PagedKVSpec, StateSpec
from kairyu_b200.registry import architecture_of, supported_architectures
from kairyu_b200.weights.loading import WeightError, load_into


def test_registered_by_its_config_key():
    assert "Makilorn" in supported_architectures()
    assert architecture_of({"architecture": "Makilorn"}).name == "Makilorn"
    assert architecture_of({"architectures": ["LlamaForCausalLM"]}).name == "LlamaForCausalLM"


@pytest.mark.parametrize("name", list(CASES))
def test_spec_run_order_and_cache_needs(name):
    cfg, _, _ = CASES[name]
    model, parsed = build_model(cfg, dtype="float32", device="meta")
    entries = cfg["layers"]
    assert len(model.schedule) == len(entries)
    assert [call.cache_slot for call in model.schedule] == list(range(len(entries)))  # a cache or state per entry
    own = [i for i, entry in enumerate(entries) if "weights_of" not in entry]
    assert len(model.blocks) == len(own)
    for index, (entry, call) in enumerate(zip(entries, model.schedule)):
        assert call.layer == own.index(entry.get("weights_of", index))
    needs = model.cache_slot_specs()
    for index, entry in enumerate(entries):
        m = entry["mixer"]
        if entry["type"] == "latent_attention":
            assert needs[index] == (PagedKVSpec(1, m["kv_rank"], m["mask"]["size"], v_head_dim=0),)
        else:
            wanted = [StateSpec((m["heads"], m["vdim"], m["dim"]), "float32")]
            if m["conv"] > 1:
                wanted.append(StateSpec((m["conv"] - 1, 2 * m["kv_heads"] * m["dim"] + m["heads"] * m["vdim"]), "float32"))
            assert needs[index] == tuple(wanted)
    layout = CacheLayout.from_slot_specs(needs)
    windows = {(e["mixer"]["kv_rank"], e["mixer"]["mask"]["size"]) for e in entries if e["type"] == "latent_attention"}
    assert len(layout.groups) == len(windows)  # layers of one rank and window share pages and a block table
    names = {spec.name for spec in model.tensor_specs()}
    assert names == set(make_weights(cfg, 0))  # shared layers ask for no tensors of their own
    assert parsed.vocab_size == cfg["vocab"] and parsed.hidden_size == cfg["width"]


def test_shared_weights_with_other_constants_get_parts_of_their_own():
    cfg = config(32, 17, [layer(latent(2, 8, 8, 16, 5, 0.5), None), layer(latent(2, 8, 8, 16, 9, 0.5), None, weights_of=0)])
    model, _ = build_model(cfg, dtype="float32", device="meta")
    assert len(model.blocks) == 2 and [call.layer for call in model.schedule] == [0, 1]
    assert {spec.name for spec in model.tensor_specs()} == set(make_weights(cfg, 0))
    assert [block.mixer.window for block in model.blocks] == [5, 9]


@pytest.mark.parametrize("damage, message", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][2].update(weights_of=7), "weights_of"),
    (lambda c: c["layers"][2].update(weights_of=1), "another kind"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_config_errors_name_the_key(damage, message):
    cfg = json.loads(json.dumps(CASES["mixed"][0]))
    damage(cfg)
    with pytest.raises(ConfigError, match=message):
        build_model(cfg, dtype="float32", device="meta")


def test_model_folder_round_trip(tmp_path):
    cfg, seed, _ = CASES["rank32"]
    weights = make_weights(cfg, seed)
    folder = write_model(cfg, weights, tmp_path / "m")
    model, _ = build_model(cfg, dtype="float32", device="cpu")
    load_into(model, folder)
    mixer = model.blocks[1].mixer
    assert torch.equal(mixer.w_in[: mixer.q_size], weights["l1.mix.q"])
    assert torch.equal(mixer.w_absorb[0], weights["l1.mix.uk"][: mixer.head_dim].T)
    ffn = model.blocks[1].ffn
    assert torch.equal(ffn.w_gate_up[3, ffn.intermediate_size :], weights["l1.mlp.e3.up"])
    broken = dict(weights)
    del broken["l0.mix.A_log"]
    broken["l1.mlp.router.b"] = torch.zeros(5)
    with pytest.raises(WeightError) as error:
        load_into(build_model(cfg, dtype="float32", device="cpu")[0], write_model(cfg, broken, tmp_path / "b"))
    assert error.value.missing == ["l0.mix.A_log"] and error.value.wrong_shape[0][0] == "l1.mlp.router.b"


def test_random_weights_through_the_registry(tmp_path):
    from kairyu_b200.weights import write_random_model

    cfg, _, _ = CASES["mixed"]
    folder = write_random_model(cfg, tmp_path / "r", seed=4, dtype="bfloat16")
    model, _ = build_model(json.loads((folder / "config.json").read_text()), dtype="float32", device="cpu")
    load_into(model, folder, strict_unexpected=True)


@pytest.mark.parametrize("name", list(CASES))
def test_the_bounds_see_a_window_that_is_one_token_off(name):
    """What the GPU tests' bounds are for: the plain model with every window one token longer, or
    one shorter, is far beyond the bfloat16 bound at most positions that have a window's edge behind
    them (the weights make the softmax pick single keys)."""
    cfg, seed, _ = CASES[name]
    weights = make_weights(cfg, seed)
    windows = [entry["mixer"]["mask"]["size"] for entry in cfg["layers"] if entry["type"] == "latent_attention"]
    tokens = traces.make_requests(cfg["vocab"], [90], seed=1)["r0"]
    right = plain.forward(cfg, weights, tokens, dtype=torch.float64).numpy()
    for change in (1, -1):
        if not any(max(1, w + change) != w and min(w, w + change) < len(tokens) for w in windows):
            continue  # nothing changes: a window of one cannot shrink, one longer than the prompt has no edge in it
        other = json.loads(json.dumps(cfg))
        for entry in other["layers"]:
            if entry["type"] == "latent_attention":
                entry["mixer"]["mask"]["size"] = max(1, entry["mixer"]["mask"]["size"] + change)
        off = plain.forward(other, weights, tokens, dtype=torch.float64).numpy()
        errors = [relative_error(off[i], right[i]) for i in range(min(windows), len(tokens))]
        assert np.median(errors) > 3 * 5e-2, (change, float(np.median(errors)))  # three times the GPU tests' bfloat16 bound


def test_plain_model_pieces():
    """The oracle's own pieces against each other: the recurrence of one token at a time equals a
    whole sequence's prefix, and a window as long as the sequence equals no window."""
    cfg = config(24, 19, [layer(delta(2, 1, 8, 12, 3), moe(3, 2, 8, 1.0)), layer(latent(2, 8, 8, 16, 6, 0.5), None)])
    weights = make_weights(cfg, 5)
    tokens = traces.make_requests(19, [20], seed=2)["r0"]
    whole = plain.forward(cfg, weights, tokens)
    for cut in (1, 7, 19):
        assert torch.allclose(plain.forward(cfg, weights, tokens[:cut]), whole[:cut], atol=1e-9)  # causal
    long_window = json.loads(json.dumps(cfg))
    long_window["layers"][1]["mixer"]["mask"]["size"] = 20
    longer = json.loads(json.dumps(cfg))
    longer["layers"][1]["mixer"]["mask"]["size"] = 500
    assert torch.allclose(plain.forward(long_window, weights, tokens), plain.forward(longer, weights, tokens), atol=1e-9)
    assert not torch.allclose(plain.forward(cfg, weights, tokens), plain.forward(longer, weights, tokens), atol=1e-3)


# ---------------------------------------------------------------------------- the engine on the CPU
# The kernels replaced by their torch statements (makilorn_torch_kernels.py): the cache manager's
# windowed groups and state slots, the step function, the scheduler and the command line as this
# design drives them, in 32-bit.  The same workloads run on the GPU with the kernels.

SHORT = [33, 12, 40, 9, 2, 1, 27]


def cpu_runner(folder, *, page_size, num_pages, max_requests=4):
    from kairyu_b200.cache import CacheManager, CacheStorage
    from kairyu_b200.engine.engine import load_model
    from kairyu_b200.engine.runner import ModelRunner

    model, _ = load_model(folder, dtype="float32", device="cpu")
    layout = CacheLayout.from_slot_specs(model.cache_slot_specs())
    cache = CacheManager(layout, num_pages=num_pages, page_size=page_size, max_requests=max_requests)
    storage = CacheStorage(layout, num_pages=num_pages, page_size=page_size, max_requests=max_requests, dtype=model.dtype, device="cpu")
    return ModelRunner(model, cache, storage, max_model_len=512, decode_mode="eager", check_tables=True, debug_poison=True)


@pytest.mark.parametrize("name", ["mixed", "rank32"])
def test_every_cut_on_the_cpu(name, tmp_path, monkeypatch):
    import makilorn_torch_kernels

    makilorn_torch_kernels.install(monkeypatch)
    cfg, seed, page_size = CASES[name]
    weights = make_weights(cfg, seed)
    folder = write_model(cfg, weights, tmp_path / "m")
    requests = traces.make_requests(cfg["vocab"], SHORT, seed=3)
    expected = {n: plain.forward(cfg, weights, t, dtype=torch.float64).numpy() for n, t in requests.items()}
    cuts = {
        "whole": traces.trace_whole(requests),
        "tail": traces.trace_decode_tail(requests, 6),
        "chunks": traces.trace_chunks(requests, sizes=(5, 2, 11, 3)),
        "mixed": traces.trace_mixed(requests, seed=4, max_live=3),
    }
    pool = max(traces.peak_tokens(steps, round_to=page_size) for steps in cuts.values()) // page_size + 1
    runner = cpu_runner(folder, page_size=page_size, num_pages=pool, max_requests=3)  # three slots for seven requests
    for cut, steps in cuts.items():
        result = traces.run_in_process(runner, steps)
        assert len(result) == sum(SHORT)
        worst = max(relative_error(row, expected[n][p]) for (n, p), row in result.items())
        assert worst < 1e-4, (cut, worst)
        assert runner.cache.live_requests == 0


def test_generation_and_the_command_line_on_the_cpu(tmp_path, capsys, monkeypatch):
    """make-random, validate, generate: greedy tokens through the scheduler (a token budget that cuts the
    prompts) equal the plain model's own continuation."""
    import makilorn_torch_kernels
    from safetensors.torch import load_file

    from kairyu_b200.entrypoints import cli

    makilorn_torch_kernels.install(monkeypatch)
    cfg = CASES["mixed"][0]
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    folder = tmp_path / "model"
    cli.main(["make-random", str(tmp_path / "config.json"), str(folder), "--seed", "5", "--dtype", "float32"])
    cli.main(["validate", str(folder)])
    assert "valid: Makilorn, 5 layers" in capsys.readouterr().out
    prompts = [[5, 17, 3, 9], [1], list(range(20, 60))]
    cli.main(["generate", str(folder), "--dtype", "float32", "--device", "cpu", "--temperature", "0", "--max-tokens", "6", "--num-pages", "24",
              "--page-size", "8", "--max-num-seqs", "2", "--max-num-batched-tokens", "16"]
             + [arg for p in prompts for arg in ("--prompt-token-ids", ",".join(map(str, p)))])
    lines = [json.loads(line) for line in capsys.readouterr().out.splitlines() if line.startswith("{")]
    weights = {n: t.float() for n, t in load_file(str(folder / "model.safetensors")).items()}
    for prompt, line in zip(prompts, lines):
        tokens = list(prompt)
        for _ in range(6):
            tokens.append(int(plain.forward(cfg, weights, tokens)[-1].argmax()))
        assert line["outputs"][0]["token_ids"] == tokens[len(prompt):]
