"""Karesun without a GPU: the config reader, the spec it builds (run order, layers that read another
layer's keys and values, cache groups and what they keep), model folders written and read back, what the
GPU tests' bounds can see, and, with the kernels replaced by their torch statements, every cut through
the step function and greedy generation through the scheduler and the command line."""

import json

import numpy as np
import pytest
import torch

import karesun_plain as plain
import traces
from karesun_cases import CASES, attention, config, dense, layer, make_weights, moe, relative_error, write_model

from kairyu_b200.cache import CacheLayout
from kairyu_b200.config.model_config import ConfigError
from kairyu_b200.engine.engine import build_model
from kairyu_b200.parts import PagedKVSpec
from kairyu_b200.registry import architecture_of, supported_architectures
from kairyu_b200.weights.loading import WeightError, load_into


def test_registered_by_its_config_key():
    assert "Karesun" in supported_architectures()
    assert architecture_of({"architecture": "Karesun"}).name == "Karesun"


@pytest.mark.parametrize("name", list(CASES))
def test_spec_run_order_and_cache_needs(name):
    cfg, _, _ = CASES[name]
    model, parsed = build_model(cfg, dtype="float32", device="meta")
    entries = cfg["layers"]
    assert len(model.schedule) == len(entries) == len(model.blocks)
    needs = model.cache_slot_specs()
    for index, (entry, call) in enumerate(zip(entries, model.schedule)):
        m = entry["mixer"]
        source = m.get("kv_from")
        assert call.layer == index
        assert call.cache_slot == (index if source is None else source)
        assert call.writes_cache == (source is None)
        block = model.blocks[index]
        assert (block.ffn is None) == (entry["mlp"] is None)
        assert block.mixer.window == (m["mask"]["size"] if "mask" in m else None)
        if source is not None:
            assert index not in needs and block.mixer.cache_specs() == ()
            continue
        # a slot keeps what the widest window among its readers needs; everything if one of them sees everything
        windows = [e["mixer"].get("mask", {}).get("size") for at, e in enumerate(entries) if at == index or e["mixer"].get("kv_from") == index]
        keep = None if None in windows else max(windows)
        assert needs[index] == (PagedKVSpec(m["kv_heads"], 2 * m["dim"], keep, v_head_dim=m["vdim"]),)
    layout = CacheLayout.from_slot_specs(needs)
    assert len(layout.groups) == len(set(needs.values()))
    assert not layout.states
    names = {spec.name for spec in model.tensor_specs()}
    assert names == set(make_weights(cfg, 0))  # a reader asks for no key and value projections
    assert parsed.vocab_size == cfg["vocab"] and parsed.hidden_size == cfg["width"]
    assert model.spec.max_position_embeddings == cfg["max_positions"]


@pytest.mark.parametrize("damage, message", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c.pop("max_positions"), "max_positions"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "vdim"),
    (lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=3), "equal groups"),
    (lambda c: c["layers"][1]["mixer"].update(kv_from=1), "earlier layer"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "no keys and values of its own"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=0), "differs from layer 0"),
    (lambda c: c["layers"][1]["mlp"].update(kind="gated"), "unknown feed-forward"),
    (lambda c: c["layers"][0]["mixer"].update(softcap=-1.0), "softcap"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_config_errors_name_the_key(damage, message):
    cfg = json.loads(json.dumps(CASES["shared"][0]))
    damage(cfg)
    with pytest.raises(ConfigError, match=message):
        build_model(cfg, dtype="float32", device="meta")


def test_model_folder_round_trip(tmp_path):
    cfg, seed, _ = CASES["shared"]
    weights = make_weights(cfg, seed)
    folder = write_model(cfg, weights, tmp_path / "m")
    model, _ = build_model(cfg, dtype="float32", device="cpu")
    load_into(model, folder)
    writer, reader = model.blocks[0].mixer, model.blocks[1].mixer
    assert torch.equal(writer.w_in[writer.q_size : writer.q_size + writer.k_size], weights["l0.mix.k"])
    assert reader.w_in.shape[0] == reader.q_size and torch.equal(reader.w_in, weights["l1.mix.q"])
    assert writer.lam == pytest.approx(plain.lam_of(weights, "l0.mix", 0.3), rel=1e-6) and abs(writer.lam - 0.3) > 1e-3
    assert torch.equal(model.blocks[0].mixer_norm.weight, 1.0 + weights["l0.norm1"])  # stored around zero, held as 1 + w
    ffn = model.blocks[0].ffn
    assert ffn.w_router.shape[0] == 8 and ffn.w_gate_up.shape[0] == 6  # identity experts have a router row and no weights
    broken = dict(weights)
    del broken["l2.mix.lq2"]
    broken["l0.mlp.correction"] = torch.zeros(6)
    with pytest.raises(WeightError) as error:
        load_into(build_model(cfg, dtype="float32", device="cpu")[0], write_model(cfg, broken, tmp_path / "b"))
    assert error.value.missing == ["l2.mix.lq2"] and error.value.wrong_shape[0][0] == "l0.mlp.correction"


def test_random_weights_through_the_registry(tmp_path):
    from kairyu_b200.weights import write_random_model

    cfg, _, _ = CASES["small_pages"]
    folder = write_random_model(cfg, tmp_path / "r", seed=4, dtype="bfloat16")
    model, _ = build_model(json.loads((folder / "config.json").read_text()), dtype="float32", device="cpu")
    load_into(model, folder, strict_unexpected=True)


def _faults(cfg, weights):
    """Variants of a model that each get one mechanism wrong: (name, config, weights, first position it can show at)."""
    def changed(edit):
        other = json.loads(json.dumps(cfg))
        edit(other)
        return other

    def each_mixer(other, edit):
        for entry in other["layers"]:
            edit(entry["mixer"])

    def window(mixer, change):
        if "mask" in mixer:
            mixer["mask"]["size"] = max(1, mixer["mask"]["size"] + change)

    windows = [e["mixer"]["mask"]["size"] for e in cfg["layers"] if "mask" in e["mixer"]]
    out = []
    for change in (1, -1):
        # Random weights show a window's edge where windows are short (a key of a few tens weighs a few per cent).  Behind
        # long windows they hide it; there the edge is tested with keys made to stand out (test_karesun_gpu.py:
        # test_keys_that_stand_out).
        if any(max(1, w + change) != w for w in windows) and min(windows) <= 30:
            first = min(min(w, w + change) for w in windows if max(1, w + change) != w)  # the first position a changed window shows at
            out.append((f"windows {change:+d}", changed(lambda o: each_mixer(o, lambda m: window(m, change))), weights, first))
    if any("softcap" in e["mixer"] for e in cfg["layers"]):
        out.append(("no cap", changed(lambda o: each_mixer(o, lambda m: m.pop("softcap", None))), weights, 0))
    plain_lambda = {n: (torch.zeros_like(t) if n.rsplit(".", 1)[-1] in ("lq1", "lq2") else t) for n, t in weights.items()}
    out.append(("lambda from its constant alone", cfg, plain_lambda, 0))
    one_map = changed(lambda o: each_mixer(o, lambda m: m.update(diff=0.0)))
    out.append(("another constant in lambda and the scaling", one_map, weights, 0))
    if any(e["mlp"] and e["mlp"]["kind"] == "moe" and e["mlp"]["router"].get("groups", {}).get("count", 1) > 1 for e in cfg["layers"]):
        def no_groups(o):
            for e in o["layers"]:
                if e["mlp"] and e["mlp"]["kind"] == "moe":
                    e["mlp"]["router"].pop("groups", None)
        out.append(("groups ignored", changed(no_groups), weights, 0))
    routers = [e["mlp"]["router"] for e in cfg["layers"] if e["mlp"] and e["mlp"]["kind"] == "moe"]
    if any(r["top"] < r["experts"] + r["identity"] for r in routers):  # where every output is chosen the correction decides nothing
        out.append(("correction ignored", cfg, {n: (torch.zeros_like(t) if n.endswith("correction") else t) for n, t in weights.items()}, 0))
    return out


@pytest.mark.parametrize("name", list(CASES))
def test_the_bounds_see_each_fault(name):
    """What the GPU tests' bounds are for: the plain model with one mechanism wrong (every window one token
    longer or shorter, the cap left out, lambda without its vectors, groups or the correction ignored) is beyond
    the bfloat16 bound at the median position behind the fault's first place, or beyond three times that bound at more
    than a tenth of them: either fails the GPU tests' judgement."""
    cfg, seed, _ = CASES[name]
    weights = make_weights(cfg, seed)
    tokens = traces.make_requests(cfg["vocab"], [90], seed=1)["r0"]
    right = plain.forward(cfg, weights, tokens).numpy()
    for what, other_cfg, other_weights, first in _faults(cfg, weights):
        off = plain.forward(other_cfg, other_weights, tokens).numpy()
        errors = np.array([relative_error(off[i], right[i]) for i in range(first, len(tokens))])
        if what in ("groups ignored", "correction ignored"):
            # a choice that turns at some tokens only: the 32-bit bound sees every one of them (and the router is
            # compared choice by choice in test_karesun_gpu.py: test_mixture_alone)
            assert np.mean(errors > 1e-4) > 0.05, (what, float(np.mean(errors > 1e-4)))
            continue
        assert np.median(errors) > 5e-2 or np.mean(errors >= 3 * 5e-2) > 0.10, (what, float(np.median(errors)))


def test_plain_model_pieces():
    """The oracle's own pieces against each other: a prefix of a sequence gives the whole sequence's rows
    (causal), a window as long as the sequence equals no window, a cap far above the scores equals none, and an
    identity expert alone returns the weighted input."""
    cfg = config(24, 19, [layer(attention(2, 1, 8, 12, 6, 0.5, 3.0, 0.3), moe(2, 1, 2, 8, 1.5)), layer(attention(2, 1, 8, 12, 9, 0.5, None, 0.4, kv_from=0), dense(16))])
    weights = make_weights(cfg, 5)
    tokens = traces.make_requests(19, [20], seed=2)["r0"]
    whole = plain.forward(cfg, weights, tokens)
    for cut in (1, 7, 19):
        assert torch.allclose(plain.forward(cfg, weights, tokens[:cut]), whole[:cut], atol=1e-9)
    def with_mixer(index, **changes):
        other = json.loads(json.dumps(cfg))
        for key, value in changes.items():
            if value is None:
                other["layers"][index]["mixer"].pop(key, None)
            else:
                other["layers"][index]["mixer"][key] = value
        return other
    assert torch.allclose(plain.forward(with_mixer(0, mask={"size": 20}), weights, tokens), plain.forward(with_mixer(0, mask=None), weights, tokens), atol=1e-9)
    assert not torch.allclose(whole, plain.forward(with_mixer(0, mask=None), weights, tokens), atol=1e-3)
    assert torch.allclose(plain.forward(with_mixer(1, softcap=1e6), weights, tokens), whole, atol=1e-6)
    assert not torch.allclose(plain.forward(with_mixer(0, softcap=None), weights, tokens), whole, atol=1e-3)
    y = torch.randn(3, 24, dtype=torch.float64)
    only_identity = {"router": {"experts": 0, "identity": 1, "top": 1, "scale": 2.0}}
    w = {"p.router": torch.randn(1, 24, dtype=torch.float64), "p.correction": torch.zeros(1, dtype=torch.float64)}
    assert torch.allclose(plain.expert_mixture(y, w, "p", only_identity), 2.0 * y)


# ---------------------------------------------------------------------------- the engine on the CPU
# The kernels replaced by their torch statements (karesun_torch_kernels.py): the cache manager's windowed
# groups shared by a writer and its readers, the step function, the scheduler and the command line as this
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


@pytest.mark.parametrize("name", ["shared", "small_pages"])
def test_every_cut_on_the_cpu(name, tmp_path, monkeypatch):
    import karesun_torch_kernels

    karesun_torch_kernels.install(monkeypatch)
    cfg, seed, page_size = CASES[name]
    weights = make_weights(cfg, seed)
    folder = write_model(cfg, weights, tmp_path / "m")
    requests = traces.make_requests(cfg["vocab"], SHORT, seed=3)
    expected = {n: plain.forward(cfg, weights, t).numpy() for n, t in requests.items()}
    cuts = {
        "whole": traces.trace_whole(requests),
        "tail": traces.trace_decode_tail(requests, 6),
        "chunks": traces.trace_chunks(requests, sizes=(5, 2, 11, 3)),
        "mixed": traces.trace_mixed(requests, seed=4, max_live=3),
    }
    pool = max(traces.peak_tokens(steps, round_to=page_size) for steps in cuts.values()) // page_size + 1
    runner = cpu_runner(folder, page_size=page_size, num_pages=pool, max_requests=3)
    for cut, steps in cuts.items():
        result = traces.run_in_process(runner, steps)
        assert len(result) == sum(SHORT)
        worst = max(relative_error(row, expected[n][p]) for (n, p), row in result.items())
        assert worst < 1e-4, (cut, worst)
        assert runner.cache.live_requests == 0


def test_generation_and_the_command_line_on_the_cpu(tmp_path, capsys, monkeypatch):
    """make-random, validate, generate: greedy tokens through the scheduler (a token budget that cuts the
    prompts) equal the plain model's own continuation."""
    import karesun_torch_kernels
    from safetensors.torch import load_file

    from kairyu_b200.entrypoints import cli

    karesun_torch_kernels.install(monkeypatch)
    cfg = CASES["shared"][0]
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    folder = tmp_path / "model"
    cli.main(["make-random", str(tmp_path / "config.json"), str(folder), "--seed", "5", "--dtype", "float32"])
    cli.main(["validate", str(folder)])
    assert "valid: Karesun, 4 layers" in capsys.readouterr().out
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
