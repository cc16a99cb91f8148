"""Karesun on the GPU against the plain implementation in ``karesun_plain.py``: every mechanism alone,
whole prompts against token-by-token decoding, portions down to two tokens, unequal requests in one
batch over a pool so small that pages are used again, keys made to stand out far away, at page borders
and just inside and outside a window, long decoding, and greedy generation through ``LLM.generate``."""

import types

import numpy as np
import pytest
import torch

import karesun_plain as plain
import traces
from karesun_cases import CASES, attention, config, dense, layer, make_weights, moe, relative_error, write_model

pytestmark = pytest.mark.gpu

# rms of the logits' error over rms of the logits, per position
FP32_BOUND = 1e-4
BF16_BOUND = 5e-2
LENGTHS = [70, 45, 101, 38, 64, 83, 9, 55, 2, 1]


def expected_rows(cfg, weights, requests):
    return {name: plain.forward(cfg, weights, tokens).numpy() for name, tokens in requests.items()}


def make_runner(folder, dtype, *, page_size, num_pages, max_requests=4, decode_mode="eager", max_model_len=512):
    from kairyu_b200.cache import CacheLayout, CacheManager, CacheStorage
    from kairyu_b200.engine.engine import load_model
    from kairyu_b200.engine.runner import ModelRunner

    model, _ = load_model(folder, dtype=dtype, device="cuda")
    layout = CacheLayout.from_slot_specs(model.cache_slot_specs())
    cache = CacheManager(layout, num_pages=num_pages, page_size=page_size, max_requests=max_requests)
    storage = CacheStorage(layout, num_pages=num_pages, page_size=page_size, max_requests=max_requests, dtype=model.dtype, device="cuda")
    return ModelRunner(model, cache, storage, max_model_len=max_model_len, decode_mode=decode_mode, max_graph_batch=max_requests,
                       check_tables=True, debug_poison=True)


def beyond(result, expected, bound):
    errors = [(name, position, relative_error(row, expected[name][position])) for (name, position), row in result.items()]
    return [entry for entry in errors if not entry[2] < bound][:12]


def judge(result, expected, dtype, what=""):
    """float32: every position within the bound.  bfloat16: the weights make the softmax maps pick single keys
    and the routers choose among close scores, so that faults show; rounding to bfloat16 then costs a few per
    cent at a typical position and much more where a close call turns.  A fault moves the median position
    beyond the bound or many positions far beyond it (test_karesun_cpu.py: test_the_bounds_see_each_fault), so
    the median is held to BF16_BOUND and few positions may be far off."""
    errors = np.array([relative_error(row, expected[name][position]) for (name, position), row in result.items()])
    if str(dtype).endswith("float32"):
        print(f"[karesun] {what} float32: worst {errors.max():.3e} bound {FP32_BOUND:.1e}")
        assert errors.max() < FP32_BOUND, (what, errors.max(), beyond(result, expected, FP32_BOUND))
    else:
        far = float((errors >= 3 * BF16_BOUND).mean())
        print(f"[karesun] {what} bfloat16: median {np.median(errors):.3e} worst {errors.max():.3e} far off {far:.3f} bound {BF16_BOUND:.1e}")
        assert np.median(errors) < BF16_BOUND and far <= 0.10, (what, np.median(errors), far, beyond(result, expected, 3 * BF16_BOUND))


@pytest.fixture(scope="module", params=list(CASES))
def case(request, tmp_path_factory):
    cfg, seed, page_size = CASES[request.param]
    weights = make_weights(cfg, seed)
    folder = write_model(cfg, weights, tmp_path_factory.mktemp(request.param))
    requests = traces.make_requests(cfg["vocab"], LENGTHS, seed=seed + 100)
    return dict(name=request.param, cfg=cfg, page_size=page_size, weights=weights, folder=folder, requests=requests,
                expected=expected_rows(cfg, weights, requests))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("decode_mode", ["eager", "cuda_graph"])
def test_every_cut_matches_plain(case, dtype, decode_mode):
    """Whole prompts, tails decoded token by token, portions of changing size and mixed batches, one after the
    other on one engine whose pool holds far less than all requests (pages change hands; pages that went back
    are overwritten before the next step)."""
    requests = case["requests"]
    cuts = {
        "whole": traces.trace_whole(requests),
        "tail": traces.trace_decode_tail(requests, 32),
        "chunks": traces.trace_chunks(requests),
        "twos": traces.trace_chunks(requests, sizes=(2,)),
        "mixed": traces.trace_mixed(requests, seed=5),
    }
    pool = max(traces.peak_tokens(steps) for steps in cuts.values()) // case["page_size"] + 1
    total = sum(len(t) for t in requests.values())
    assert pool * case["page_size"] < total
    runner = make_runner(case["folder"], dtype, page_size=case["page_size"], num_pages=pool, decode_mode=decode_mode)
    results = {}
    for cut, steps in cuts.items():
        results[cut] = traces.run_in_process(runner, steps)
        assert len(results[cut]) == total
        judge(results[cut], case["expected"], dtype, f"{case['name']} {decode_mode} {cut}")
        assert runner.cache.live_requests == 0
    if decode_mode == "cuda_graph":
        assert runner.counters["graph_replays"] > 0
    if dtype == "float32":
        # no 32-bit sum depends on the batch or on where a prompt was cut
        for cut in ("tail", "chunks", "twos", "mixed"):
            different = [key for key, row in results["whole"].items() if not np.array_equal(row, results[cut][key])]
            assert not different, (cut, different[:12])


MIXERS = {
    "narrow": attention(2, 1, 16, 32, 19, 0.5, 4.0, 0.3),            # tensor cores in bfloat16
    "no_tensor_cores": attention(3, 3, 24, 40, 19, 0.4, 6.0, 0.45),  # widths that are no multiple of 16
    "widest": attention(2, 2, 128, 128, 50, 0.1, 9.0, 0.5),
    "many_heads_a_group": attention(16, 2, 16, 16, 70, 0.3, 5.0, 0.2),
    "more_than_a_warp_a_group": attention(20, 1, 32, 16, 45, 0.3, None, 0.35),  # 20 rows of a single token's tile
    "window_of_one": attention(2, 1, 32, 64, 1, 0.3, 5.0, 0.3),
    "long_window": attention(4, 4, 64, 32, 131, 0.15, 30.0, 0.6),
    "sees_everything": attention(2, 1, 48, 16, None, 0.2, 7.0, 0.4),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", list(MIXERS))
def test_one_mixer_alone(kind, dtype, tmp_path):
    """A model of one layer without feed-forward, so that the mixer is all that mixes: a prompt of several
    windows' length in one step, then decoding over more than a window."""
    cfg = config(40, 53, [layer(MIXERS[kind], None)])
    weights = make_weights(cfg, 7)
    folder = write_model(cfg, weights, tmp_path / kind)
    tokens = traces.make_requests(53, [230], seed=3)["r0"]
    expected = {"r0": plain.forward(cfg, weights, tokens).numpy()}
    steps = traces.trace_decode_tail({"r0": tokens}, 90)
    runner = make_runner(folder, dtype, page_size=16, num_pages=20, decode_mode="cuda_graph")
    result = traces.run_in_process(runner, steps)
    judge(result, expected, dtype, f"{kind} alone")


def _attention_reference(q, k, v, m, lam, eps, positions):
    """o [len(positions), heads * vdim] by the plain maps, from whole-sequence q [L, H, 2, D], k [L, G, 2, D], v [L, G, DV]."""
    heads, group = q.shape[1], q.shape[1] // k.shape[1]
    window = m["mask"]["size"] if "mask" in m else None
    outs = []
    for h in range(heads):
        g = h // group
        a1 = plain.one_map(q[:, h, 0], k[:, g, 0], v[:, g], m["scale"], m.get("softcap"), window)
        a2 = plain.one_map(q[:, h, 1], k[:, g, 1], v[:, g], m["scale"], m.get("softcap"), window)
        o = a1 - lam * a2
        outs.append(o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * (1.0 - m["diff"]))
    return torch.cat(outs, dim=-1)[positions]


@pytest.mark.parametrize("variant", ["float32 generic", "bfloat16 generic", "bfloat16 tensor cores"])
@pytest.mark.parametrize("window", [40, 700, None])
def test_keys_that_stand_out(variant, window):
    """The attention kernels alone over a 900-token sequence in shuffled pages, with keys made to stand out: among
    keys whose scores are near zero, one key a query is given a score of 18 in one of the two maps, at distances 0
    and 1, at a page's last and first place, just inside and just outside the window, and hundreds of tokens away.
    The same queries run as one prompt and as single tokens."""
    from kairyu_b200 import kernels
    from kairyu_b200.engine.workspace import Workspace

    dtype = torch.float32 if variant.startswith("float32") else torch.bfloat16
    L, H, G, D, DV, page = 900, 4, 2, 32, 48, 16
    m = attention(H, G, D, DV, window, 0.5, 25.0, 0.4)
    lam, eps = 0.83, 1e-5
    gen = torch.Generator().manual_seed(11)
    q = torch.randn(L, H, 2, D, generator=gen) * 0.1
    k = torch.randn(L, G, 2, D, generator=gen) * 0.1
    v = torch.randn(L, G, DV, generator=gen)
    edge = window if window is not None else 512
    distances = [0, 1, 15, 16, 17, edge - 1, edge, edge + 1, 600]
    wanted = []
    for index, distance in enumerate(distances):
        at = 880 - 9 * index  # positions that are no multiple of anything
        if distance > at:
            continue
        u = torch.nn.functional.normalize(torch.randn(D, generator=gen), dim=0) * 6.0
        which = index % 2
        q[at, :, which] = u
        k[at - distance, :, which] = u
        wanted.append(at)
    q, k, v = (t.to(dtype).double() for t in (q, k, v))  # what the kernels are given, exactly
    want = _attention_reference(q, k, v, m, lam, eps, wanted)
    # and that the stand-out keys matter: with the window one shorter the queries at its edge answer otherwise
    if window is not None:
        shorter = attention(H, G, D, DV, window - 1, 0.5, 25.0, 0.4)
        assert (_attention_reference(q, k, v, shorter, lam, eps, wanted) - want).abs().max() > 0.3

    pages = torch.randperm(L // page + 1, generator=gen) + 1
    k_cache = torch.zeros(len(pages) + 1, page, G, 2 * D, dtype=dtype, device="cuda")
    v_cache = torch.zeros(len(pages) + 1, page, G, DV, dtype=dtype, device="cuda")
    for position in range(L):
        k_cache[pages[position // page], position % page] = k[position].reshape(G, 2 * D).to(dtype)
        v_cache[pages[position // page], position % page] = v[position].to(dtype)
    constants = dict(num_q_heads=H, maps=2, scale=0.5, softcap=25.0, window=window or 0, lam=lam, head_norm_eps=eps, out_scale=0.6)
    i32 = dict(dtype=torch.int32, device="cuda")
    bound = 2e-5 if dtype == torch.float32 else 3e-2

    def run(q_rows, positions, row_ids, table, seq_lens, qo_indptr):
        out = torch.zeros(q_rows.shape[0], H * DV, dtype=dtype, device="cuda")
        if variant.endswith("generic"):
            kernels.diff_attention_generic(q_rows, out, k_cache, v_cache, positions=positions, row_ids=row_ids, block_table=table, **constants)
            return out
        rows = len(seq_lens)
        counts = [qo_indptr[r + 1] - qo_indptr[r] for r in range(rows)]
        tile_rows = [r for r in range(rows) if counts[r] > 1 for _ in range(0, counts[r], kernels.DIFF_ATTENTION_TILE)]
        tile_starts = [s for r in range(rows) if counts[r] > 1 for s in range(0, counts[r], kernels.DIFF_ATTENTION_TILE)]
        single = [r for r in range(rows) if counts[r] == 1]
        ctx = types.SimpleNamespace(
            qo_indptr=torch.tensor(qo_indptr, **i32), seq_lens=torch.tensor(seq_lens, **i32),
            tiles={kernels.DIFF_ATTENTION_TILE: (len(tile_rows), torch.tensor(tile_rows or [0], **i32), torch.tensor(tile_starts or [0], **i32))},
            num_decode_rows=len(single), decode_rows=torch.tensor(single or [0], **i32),
            decode_tokens=torch.tensor([qo_indptr[r] for r in single] or [0], **i32), workspace=Workspace("cuda"),
        )
        kernels.diff_attention_mma(q_rows, out, k_cache, v_cache, ctx=ctx, block_table=table, **constants)
        return out

    flat_q = q.reshape(L, H * 2 * D).to(dtype).cuda()
    # one prompt of 900 tokens
    table = pages.to(torch.int32).cuda()[None, :].contiguous()
    got = run(flat_q, torch.arange(L, **i32), torch.zeros(L, **i32), table, [L], [0, L])
    assert (got[wanted].double().cpu() - want).abs().max() < bound
    # a portion that starts in the middle of a page and of a window, beside single tokens of other lengths
    start = 613
    rows_q = torch.cat([flat_q[start:], flat_q[wanted]])
    positions = torch.tensor(list(range(start, L)) + wanted, **i32)
    row_ids = torch.tensor([0] * (L - start) + list(range(1, len(wanted) + 1)), **i32)
    tables = table.repeat(len(wanted) + 1, 1).contiguous()
    indptr = [0, L - start] + [L - start + n + 1 for n in range(len(wanted))]
    got = run(rows_q, positions, row_ids, tables, [L] + [at + 1 for at in wanted], indptr)
    in_portion = [at - start for at in wanted if at >= start]
    assert (got[in_portion].double().cpu() - want[[n for n, at in enumerate(wanted) if at >= start]]).abs().max() < bound
    assert (got[L - start :].double().cpu() - want).abs().max() < bound


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [
    # width, experts, identity, top, ff, scale, groups, tokens
    (40, 5, 2, 3, 24, 1.7, None, 33), (64, 6, 2, 3, 16, 0.5, (4, 2), 3), (72, 4, 0, 2, 40, 1.5, (2, 1), 16),
    (136, 3, 1, 4, 200, 2.0, None, 11), (24, 1, 0, 1, 70, 2.0, None, 130), (96, 13, 3, 5, 96, 1.5, (8, 3), 700),
    (40, 2, 4, 2, 20, 1.0, (3, 1), 300),
])
def test_mixture_alone(sizes, dtype):
    """The part by itself against the plain mixture, and the router kernel's choices and weights one by one.
    Sizes whose rows are whole 16 bytes take, in bfloat16, the few-pairs kernel up to 16 tokens and the library's
    grouped product beyond; the others this package's tiled kernel; float32 always the FMA kernel.  Identity
    experts (none, some, most), groups (none, some kept, one kept) and every output chosen all occur."""
    from kairyu_b200 import kernels
    from kairyu_b200.engine.workspace import Workspace
    from kairyu_b200.parts import FEED_FORWARDS, PartSpec, StepContext

    width, experts, identity, top, ff, scale, groups, tokens = sizes
    mlp = moe(experts, identity, top, ff, scale, groups)
    cfg = config(width, 11, [layer(attention(1, 1, 8, 8, 4, 1.0, None, 0.5), mlp)])
    weights = {name: t for name, t in make_weights(cfg, 3).items() if name.startswith("l0.mlp")}
    count, keep = groups or (1, 1)
    part = FEED_FORWARDS.build(PartSpec("moe", prefix="l0.mlp", hidden_size=width, intermediate_size=ff, num_experts=experts, num_identity=identity,
                                        top=top, routing="scores", groups=count, groups_keep=keep, route_scale=scale, limit=None, alpha=1.0,
                                        shift=0.0, router_bias=False), dtype=dtype, device="cuda", shared={})
    part.load({name: t.to(device="cuda", dtype=dtype) for name, t in weights.items()})
    x = torch.randn(tokens, width, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).float()
    ctx = StepContext(num_tokens=tokens, num_rows=1, dtype=dtype, token_ids=None, positions=None, row_ids=None, qo_indptr=None, seq_lens=None,
                      write_from=None, state_slots=None, block_tables={}, host_qo_indptr=(), host_seq_lens=(), workspace=Workspace("cuda"))
    doubles = {n: t.double() for n, t in weights.items()}
    want = plain.expert_mixture(x.double(), doubles, "l0.mlp", mlp).numpy()
    got = part.forward(x.to(device="cuda", dtype=dtype), ctx).float().cpu().numpy()
    bound = 1e-5 if dtype == torch.float32 else 2e-2
    assert np.abs(got - want).max() < bound * np.abs(want).max()
    # the router alone, from exact 32-bit logits
    logits = (x.double() @ doubles["l0.mlp.router"].T).float().cuda()
    ids = torch.zeros(tokens, top, dtype=torch.int32, device="cuda")
    mix = torch.zeros(tokens, top, dtype=torch.float32, device="cuda")
    kernels.moe_route_scores(logits, weights["l0.mlp.correction"].cuda(), top, ids, mix, groups=count, keep=keep, scale=scale)
    chosen, their = plain.route(x.double(), doubles, "l0.mlp", mlp["router"])
    assert ids.cpu().tolist() == chosen
    assert np.abs(mix.cpu().numpy() - np.array([[float(w) for w in row] for row in their])).max() < 1e-6 * scale


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_small_kernels(dtype):
    """The scaled embedding, learned positions, the ungated feed-forward's activations, the norm with weights stored
    around zero and the page write of keys and values of different widths."""
    from kairyu_b200 import kernels
    from kairyu_b200.engine.workspace import Workspace
    from kairyu_b200.parts import FEED_FORWARDS, NORMS, PartSpec, StepContext

    g = torch.Generator().manual_seed(4)
    tokens, width, vocab, places = 37, 72, 50, 64
    table = torch.randn(vocab, width, generator=g).to(dtype)
    pos_table = torch.randn(places, width, generator=g).to(dtype)
    ids = torch.randint(0, vocab, (tokens,), generator=g, dtype=torch.int32)
    positions = torch.randint(0, places, (tokens,), generator=g, dtype=torch.int32)
    x = torch.zeros(tokens, width, device="cuda")
    kernels.embedding(table.cuda(), ids.cuda(), x, scale=0.37)
    kernels.add_positions(pos_table.cuda(), positions.cuda(), x)
    want = table[ids.long()].double() * np.float32(0.37) + pos_table[positions.long()].double()
    assert (x.cpu().double() - want).abs().max() < 1e-6

    rows = (torch.randn(tokens, 200, generator=g) * 2).to(dtype)
    for kind, fn in (("relu2", lambda z: torch.relu(z) ** 2), ("silu", lambda z: z / (1 + torch.exp(-z))),
                     ("gelu_tanh", lambda z: 0.5 * z * (1 + torch.tanh(np.sqrt(2 / np.pi) * (z + 0.044715 * z ** 3))))):
        out = torch.empty_like(rows, device="cuda")
        kernels.activation(rows.cuda(), out, kind)
        want = fn(rows.double())
        assert ((out.cpu().double() - want).abs() / (1 + want.abs())).max() < (1e-6 if dtype == torch.float32 else 5e-3)  # one rounding at the store

    ctx = StepContext(num_tokens=tokens, num_rows=1, dtype=dtype, token_ids=None, positions=None, row_ids=None, qo_indptr=None, seq_lens=None,
                      write_from=None, state_slots=None, block_tables={}, host_qo_indptr=(), host_seq_lens=(), workspace=Workspace("cuda"))
    norm = NORMS.build(PartSpec("rmsnorm", name="n", size=width, eps=1e-5, offset=1.0), dtype=dtype, device="cuda")
    stored = (torch.randn(width, generator=g) * 0.1).to(torch.bfloat16)
    norm.load({"n": stored.to(dtype).cuda()})
    residual = torch.randn(tokens, width, generator=g)
    got = norm.apply(residual.cuda(), None, ctx)
    assert (got.cpu().double() - plain.norm(residual.double(), stored.double(), 1e-5)).abs().max() < (1e-5 if dtype == torch.float32 else 0.03)

    ffn = FEED_FORWARDS.build(PartSpec("mlp", prefix="f", hidden_size=width, intermediate_size=120, activation="relu2"), dtype=dtype, device="cuda")
    w = {"f.up": (torch.randn(120, width, generator=g) * width ** -0.5).to(torch.bfloat16), "f.down": (torch.randn(width, 120, generator=g) * 120 ** -0.5).to(torch.bfloat16)}
    ffn.load({n: t.to(dtype).cuda() for n, t in w.items()})
    y = torch.randn(tokens, width, generator=g).to(torch.bfloat16)
    got = ffn.forward(y.to(dtype).cuda(), ctx)
    want = plain.dense_ff(y.double(), {n: t.double() for n, t in w.items()}, "f")
    assert (got.cpu().double() - want).abs().max() < (1e-5 if dtype == torch.float32 else 0.03) * want.abs().max()

    page, heads, kw, vw = 8, 3, 20, 12
    packed = torch.randn(tokens, 10 + heads * (kw + vw), generator=g).to(dtype).cuda()
    k_cache = torch.zeros(9, page, heads, kw, dtype=dtype, device="cuda")
    v_cache = torch.zeros(9, page, heads, vw, dtype=dtype, device="cuda")
    block_table = torch.tensor([[3, 1, 7, 5, 2, -1], [4, 6, 8, -1, -1, -1]], dtype=torch.int32, device="cuda")
    row_ids = torch.tensor([0] * 30 + [1] * 7, dtype=torch.int32, device="cuda")
    where = torch.tensor(list(range(5, 35)) + list(range(11, 18)), dtype=torch.int32, device="cuda")
    write_from = torch.tensor([8, 0], dtype=torch.int32, device="cuda")  # row 0 only reads its first page
    kernels.paged_kv_write(packed, 10, 10 + heads * kw, k_cache, v_cache, positions=where, row_ids=row_ids, block_table=block_table, write_from=write_from)
    for t in range(tokens):
        position, row = int(where[t]), int(row_ids[t])
        slot = (int(block_table[row, position // page]), position % page)
        written = position >= int(write_from[row])
        assert torch.equal(k_cache[slot].flatten(), packed[t, 10 : 10 + heads * kw]) == written
        assert torch.equal(v_cache[slot].flatten(), packed[t, 10 + heads * kw :]) == written


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(case, dtype):
    """``LLM.generate`` with a token budget that cuts the prompts into portions and batches them with decoding
    requests; greedy tokens against the plain model's own greedy continuation."""
    from kairyu_b200.entrypoints.llm import LLM
    from kairyu_b200.entrypoints.prompt import TokensPrompt
    from kairyu_b200.sampling.params import SamplingParams

    cfg, weights = case["cfg"], case["weights"]
    prompts = [tokens for tokens in list(case["requests"].values())[:6]]
    new = 12
    llm = LLM(model=str(case["folder"]), dtype=dtype, num_pages=64, page_size=case["page_size"], max_num_batched_tokens=24,
              max_num_seqs=4, max_model_len=256)
    outputs = llm.generate([TokensPrompt(prompt_token_ids=tokens) for tokens in prompts],
                           SamplingParams(temperature=0.0, max_tokens=new, ignore_eos=True), use_tqdm=False)
    for tokens, output in zip(prompts, outputs):
        got = list(output.outputs[0].token_ids)
        assert len(got) == new
        # teacher-forced: at every step the engine's choice is (nearly) the plain model's best given the engine's own history
        logits = plain.forward(cfg, weights, list(tokens) + got).numpy()
        close = []
        for step, token in enumerate(got):
            row = logits[len(tokens) - 1 + step]
            close.append((row.max() - row[token]) / row.std())
        if dtype == "float32":
            assert max(close) <= 1e-4, close
        else:  # bfloat16 may turn a close call: most steps agree
            assert np.mean(np.array(close) <= 0.15) >= 0.8, close


def test_trace_program(case, tmp_path):
    """The same through ``bin/trace_run``: a pool for the trace's peak."""
    steps = traces.trace_mixed(case["requests"], seed=9)
    result = traces.run_program(case["folder"], tmp_path / "out", steps, dtype="float32", max_tokens=traces.peak_tokens(steps), vocab=case["cfg"]["vocab"],
                                extra=["--page-size", str(case["page_size"])])
    worst = max(relative_error(row, case["expected"][name][position]) for (name, position), row in result.items())
    assert worst < FP32_BOUND
