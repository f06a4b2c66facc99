"""The Tapalix design in the engine against the plain implementation of the tests: every
mechanism alone, whole prompts against decoding token by token, portions down to two tokens,
mixed batches with pages and slots that are used again, keys far away and at page borders in
prompts and in decoding, the first tokens of a sequence, long decoding, and greedy generation
through the engine."""

import math

import numpy as np
import pytest
import torch

import helpers
import plain_tapalix as plain
import tapalix_models as tm

pytestmark = pytest.mark.gpu

F32_BOUND = 2e-4          # largest |engine - plain| of a row, relative to max(1, largest |plain|)
BF16_BOUND = 6e-2
# float32 runs the sharpened weights (a wrong key or expert shows); bfloat16 runs the plain random
# weights, whose rounding error stays a few percent of the logits
SHARPEN = {"float32": True, "bfloat16": False}

_folders = {}
_plain = {}


def folder_of(tmp_path_factory, name, **options):
    key = (name, tuple(sorted(options.items())))
    if key not in _folders:
        _folders[key] = tm.write_model(tmp_path_factory.mktemp(f"tapalix_{name}"), name, **options)
    return _folders[key]


def plain_rows(folder, ids):
    key = (str(folder), tuple(ids))
    if key not in _plain:
        _plain[key] = plain.logits_of(folder, ids).numpy()
    return _plain[key]


def runner_for(folder, dtype, num_pages, max_requests=4, page_size=16, **options):
    from from_scratch_inference_engine_b200 import LoadedModel, ModelRunner
    model = LoadedModel.from_pretrained(folder, dtype=dtype, max_positions=num_pages * page_size)
    return ModelRunner(model.model, model.runtime, page_size=page_size, num_pages=num_pages,
                       max_requests=max_requests, max_step_tokens=num_pages * page_size, **options)


def assert_rows(rows, requests, folder, bound):
    """Every row within `bound` of the plain logits.  bfloat16 rounds every product's result:
    there one row in ten may lie beyond the bound, none beyond three times it.  (The bfloat16
    models' routers are drawn narrow and their corrections far apart, so that the choice of experts
    rests on the corrections and no token's choice is a near tie that rounding could turn; the
    float32 models' routers are wide, and every token chooses for itself.)"""
    assert rows
    beyond = 0
    for (key, pos), row in sorted(rows.items()):
        want = plain_rows(folder, requests[key.split("~")[0]])[pos]
        base = max(1.0, float(np.abs(want).max()))
        diff = float(np.abs(row.astype(np.float64) - want).max())
        limit = bound * base * (3.0 if bound == BF16_BOUND else 1.0)
        assert diff <= limit, f"request {key} position {pos}: off by {diff:.3e} (bound {limit:.3e})"
        beyond += diff > bound * base
    assert beyond <= 0.1 * len(rows), f"{beyond} of {len(rows)} rows beyond the bound"


def vocab_of(name):
    return tm.CONFIGS[name]["vocab"]


# ----------------------------------------------------------------- mechanisms, kernel by kernel
def test_layer_norm_with_bias_over_pending_outputs():
    from from_scratch_inference_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(1)
    for width in (36, 256, 1000, 4104):
        base = torch.randn(7, width, generator=g) * 2 + 0.7
        d1, d2 = torch.randn(7, width, generator=g) * 3, torch.randn(7, width, generator=g)
        gain, bias = torch.randn(width, generator=g), torch.randn(width, generator=g)
        for dtype in (torch.float32, torch.bfloat16):
            a, b = d1.to(dtype), d2.to(dtype)
            tolerance = 2e-5 if dtype is torch.float32 else 2e-2
            for deltas in ((), (a,), (a, b)):
                summed = base.double() + sum(d.double() for d in deltas)
                want = plain.layer_norm(summed, gain.double(), bias.double(), 1e-5)
                x = base.clone().cuda()
                out = torch.empty(7, width, device="cuda", dtype=dtype)
                ops.sum_layernorm(x, [d.cuda() for d in deltas], gain.cuda(), bias.cuda(), 1e-5, out)
                assert (x.cpu().double() - summed).abs().max() < 2e-5           # the sum stays 32-bit
                assert (out.cpu().double() - want).abs().max() < tolerance * max(1.0, float(want.abs().max()))
            # chosen rows only, x left as it is; and without a bias
            rows = torch.tensor([5, 0, 3], dtype=torch.int32)
            x = base.clone().cuda()
            some = torch.empty(3, width, device="cuda", dtype=dtype)
            ops.sum_layernorm(x, [a.cuda(), b.cuda()], gain.cuda(), bias.cuda(), 1e-5, some,
                              rows=rows.cuda(), write_x=False)
            assert torch.equal(x.cpu(), base)
            assert torch.equal(some, out[rows.long()])
            bare = ops.sum_layernorm(base.clone().cuda(), [a.cuda()], gain.cuda(), None, 1e-5,
                                     torch.empty(7, width, device="cuda", dtype=dtype))
            want = plain.layer_norm(base.double() + a.double(), gain.double(), None, 1e-5)
            assert (bare.cpu().double() - want).abs().max() < tolerance * max(1.0, float(want.abs().max()))
    # a constant row has no deviations: the result is the bias, whatever the row's size
    x = torch.full((1, 64), 1000.0, device="cuda")
    out = ops.sum_layernorm(x, [], torch.ones(64, device="cuda"), torch.full((64,), 0.25, device="cuda"),
                            1e-6, torch.empty(1, 64, device="cuda"))
    assert float((out - 0.25).abs().max()) < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_stream_beside_embedding_output_cap_and_gate(dtype):
    from from_scratch_inference_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(2)
    for width in (36, 264):
        x, x0 = torch.randn(9, width, generator=g), torch.randn(9, width, generator=g)
        d1, d2 = torch.randn(9, width, generator=g).to(dtype), torch.randn(9, width, generator=g).to(dtype)
        out = torch.empty(9, 2 * width, device="cuda", dtype=dtype)
        ops.settle_concat(x.cuda(), [d1.cuda(), d2.cuda()], x0.cuda(), out)
        want = torch.cat([x.double() + d1.double() + d2.double(), x0.double()], dim=1)
        tolerance = 1e-6 if dtype is torch.float32 else 2e-2
        assert (out.cpu().double() - want).abs().max() < tolerance * 4
        ops.settle_concat(x.cuda(), [], x0.cuda(), out)
        assert (out.cpu().double() - torch.cat([x, x0], dim=1).double()).abs().max() < tolerance * 4
        heads = torch.randn(9, width, generator=g).to(dtype)
        wide = torch.randn(9, width + 24, generator=g).to(dtype).cuda()
        got = ops.sigmoid_gate(heads.clone().cuda(), wide[:, 16:16 + width])
        want = heads.double() * torch.sigmoid(wide[:, 16:16 + width].cpu().double())
        assert (got.cpu().double() - want).abs().max() < tolerance * 4
    z = torch.randn(5, 77, generator=g) * 10
    got = ops.logit_cap(z.clone().cuda(), 2.0, 15.0)
    assert (got.cpu().double() - 15.0 * torch.tanh(z.double() * 2.0 / 15.0)).abs().max() < 1e-5
    assert float(got.abs().max()) <= 15.0
    got = ops.logit_cap(z.clone().cuda(), 0.5, 0.0)
    assert (got.cpu() - z * 0.5).abs().max() < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("stretched", [False, True])
def test_latent_rows_with_pairs_half_a_rotation_apart(dtype, stretched):
    """The latent is normed and the shared key part turned into the token's cache row, the turned
    parts of the queries land behind the columns that the product per head fills; pairs
    (i, i + dims/2), with and without stretched frequencies, only part of the turned columns
    turning; and the same without any turned part."""
    from from_scratch_inference_engine_b200.kernels import ops
    from from_scratch_inference_engine_b200.parts.rope import rotary_table, yarn_rotary_table
    g = torch.Generator().manual_seed(4)
    heads, dim, rope, rank, dims, page, tokens = 3, 10, 8, 20, 6, 4, 70
    rot = {"base": 300.0, "dims": dims, "scaling": tm.scaling(4.0, 32, 2.0, 0.5) if stretched else None}
    table = (yarn_rotary_table(300.0, dims, 128, 4.0, 32, 2.0, 0.5) if stretched
             else rotary_table(300.0, dims, 128))
    table = torch.from_numpy(table).cuda()
    row = rank + rope
    proj = torch.randn(tokens, heads * (dim + rope) + row + 5, generator=g).to(dtype)   # columns behind: a gate's
    gain = torch.randn(rank, generator=g)
    positions = torch.randint(0, 90, (tokens,), generator=g).to(torch.int32)
    slot_of = torch.randperm(20 * page, generator=g)[:tokens].to(torch.int32)
    pages = torch.zeros(20, page * row, dtype=dtype, device="cuda")
    qa = torch.zeros(tokens, heads * row, dtype=dtype, device="cuda")
    ops.latent_prep(proj.cuda(), positions.cuda(), table, slot_of.cuda(), pages, pages.stride(0), page,
                    gain.cuda(), 1e-5, qa, heads, dim, rope, rank, dims,
                    torch.zeros(1, dtype=torch.int32, device="cuda"), half_pairs=True)
    tolerance = 1e-5 if dtype is torch.float32 else 2e-2
    p = proj.double()
    q = p[:, :heads * (dim + rope)].reshape(tokens, heads, dim + rope)
    lat = p[:, heads * (dim + rope):heads * (dim + rope) + rank]
    kr = p[:, heads * (dim + rope) + rank:heads * (dim + rope) + row]
    c = plain.rms_norm(lat, gain.double(), 1e-5)
    kr = plain.turn(kr, positions.tolist(), rot)
    stored = pages.cpu().double().reshape(20, page, row)
    for t in range(tokens):
        at = int(slot_of[t])
        assert (stored[at // page, at % page, :rank] - c[t]).abs().max() < tolerance * 4
        assert (stored[at // page, at % page, rank:] - kr[t]).abs().max() < tolerance * 4
    got = qa.cpu().double().reshape(tokens, heads, row)
    want = plain.turn(q[..., dim:], positions.tolist(), rot)
    assert (got[..., rank:] - want).abs().max() < tolerance * 4
    assert float((want[..., dims:] - q[..., dim + dims:]).abs().max()) == 0.0      # the rest passes unchanged
    # no turned part at all: the cache row is the latent
    proj = torch.randn(tokens, heads * dim + rank, generator=g).to(dtype)
    pages = torch.zeros(20, page * rank, dtype=dtype, device="cuda")
    none = torch.zeros((1, 0), device="cuda")
    ops.latent_prep(proj.cuda(), positions.cuda(), none, slot_of.cuda(), pages, pages.stride(0), page,
                    gain.cuda(), 1e-5, torch.zeros(tokens, heads * rank, dtype=dtype, device="cuda"), heads,
                    dim, 0, rank, 0, torch.zeros(1, dtype=torch.int32, device="cuda"), half_pairs=True)
    c = plain.rms_norm(proj.double()[:, heads * dim:], gain.double(), 1e-5)
    stored = pages.cpu().double().reshape(20, page, rank)
    for t in range(tokens):
        at = int(slot_of[t])
        assert (stored[at // page, at % page] - c[t]).abs().max() < tolerance * 4


@pytest.mark.parametrize("experts,top,groups,keep,width", [
    (15, 4, 3, 2, 64), (6, 2, 6, 3, 40), (8, 3, 1, 1, 36), (64, 6, 8, 3, 256), (5, 5, 1, 1, 20),
    (40, 1, 4, 1, 100), (16, 4, 16, 4, 72)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_router_choice_and_weights(experts, top, groups, keep, width, dtype):
    """Scores, the choice among the kept groups on scores plus a wide correction (most choice
    values are negative: a masked expert at 0 would win), and the weights on the scores without
    it."""
    from from_scratch_inference_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(experts * 7 + top)
    tokens = 57
    y = torch.randn(tokens, width, generator=g).to(dtype)
    w = (torch.randn(experts, width, generator=g) * 4 / math.sqrt(width)).bfloat16().float()
    correction = (torch.randn(experts, generator=g) - 1.5).bfloat16().float()
    ids = torch.zeros(tokens, top, dtype=torch.int32, device="cuda")
    weights = torch.zeros(tokens, top, device="cuda")
    ops.moe_route(y.cuda(), w.cuda(), correction.cuda(), ids, weights, top, groups, keep, 2.5)
    router = {"experts": experts, "top": top, "scale": 2.5}
    if groups > 1:
        router["groups"] = {"count": groups, "keep": keep}
    z = y.double() @ w.double().T
    wrong = 0
    for t in range(tokens):
        chosen, want = plain.route(z[t], correction.double(), router)
        got = ids[t].tolist()
        if sorted(got) != sorted(chosen):
            wrong += 1                         # a near tie in 32-bit against 64-bit
            continue
        assert len(set(got)) == top
        for e, value in zip(got, weights[t].tolist()):
            assert abs(value - want[chosen.index(e)]) < 1e-5 * 2.5
        assert abs(sum(weights[t].tolist()) - 2.5) < 1e-4
    assert wrong <= 1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,experts,top,width,ff", [
    (1, 4, 2, 64, 32), (7, 12, 4, 40, 24), (150, 3, 2, 72, 100), (300, 16, 4, 128, 64), (90, 2, 1, 36, 10)])
def test_experts_products_and_weighted_sum(dtype, tokens, experts, top, width, ff):
    """Pairs sorted by expert, both products over tiles that share an expert (an expert with more
    rows than a tile holds, experts without rows), the activation, the weighted sum with and
    without a shared expert's output - against a loop over tokens and experts."""
    from from_scratch_inference_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(tokens + experts)
    y = torch.randn(tokens, width, generator=g).to(dtype)
    w_gu = (torch.randn(experts, 2 * ff, width, generator=g) / math.sqrt(width)).to(dtype)
    w_d = (torch.randn(experts, width, ff, generator=g) / math.sqrt(ff)).to(dtype)
    # most tokens go to expert 0 (more rows than one tile), the last expert gets none when it can
    ids = torch.stack([torch.randperm(max(experts - 1, top), generator=g)[:top] for _ in range(tokens)])
    ids[: tokens // 2, 0] = 0
    for t in range(tokens):                   # an expert at most once per token
        seen = set()
        for j in range(top):
            e = int(ids[t, j])
            while e in seen:
                e = (e + 1) % experts
            ids[t, j] = e
            seen.add(e)
    weights = torch.rand(tokens, top, generator=g) + 0.1
    shared = torch.randn(tokens, width, generator=g).to(dtype)
    pairs = tokens * top
    lists = ops.moe_align(ids.int().cuda(), pairs, experts,
                          torch.zeros(ops.moe_lists_size(pairs, experts), dtype=torch.int32, device="cuda"))
    offsets, order = lists[0].cpu().tolist(), lists[1].cpu().tolist()
    flat = ids.reshape(-1).tolist()
    assert sorted(order) == list(range(pairs))
    assert offsets[0] == 0 and offsets[-1] == pairs
    for e in range(experts):
        assert all(flat[p] == e for p in order[offsets[e]:offsets[e + 1]])
    act = torch.full((pairs, ff), float("nan"), dtype=dtype, device="cuda")
    ops.moe_product(y.cuda(), w_gu.cuda(), act, lists, pairs, top, True, "silu")
    out = torch.full((pairs, width), float("nan"), dtype=dtype, device="cuda")
    ops.moe_product(act, w_d.cuda(), out, lists, pairs, top, False)
    tolerance = 2e-5 if dtype is torch.float32 else 3e-2
    want_out = torch.zeros(pairs, width, dtype=torch.float64)
    for p in range(pairs):
        e, h = flat[p], y[p // top].double()
        both = w_gu[e].double() @ h
        if dtype is torch.bfloat16:
            both = both.bfloat16().double()
        a = plain.silu(both[:ff]) * both[ff:]
        at = order.index(p)
        assert (act[at].cpu().double() - a).abs().max() < tolerance * max(1.0, float(a.abs().max()))
        want_out[p] = w_d[e].double() @ act[at].cpu().double()
    assert (out.cpu().double() - want_out).abs().max() < tolerance * max(1.0, float(want_out.abs().max()))
    for extra in (None, shared):
        got = ops.moe_combine(out, weights.cuda(), None if extra is None else extra.cuda(),
                              torch.empty(tokens, width, dtype=dtype, device="cuda"), top)
        want = (weights.double()[:, :, None] * out.cpu().double().reshape(tokens, top, width)).sum(1)
        if extra is not None:
            want = want + extra.double()
        assert (got.cpu().double() - want).abs().max() < tolerance * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("tokens,experts,top,width,ff", [(700, 5, 2, 128, 96), (300, 3, 3, 64, 200), (2100, 16, 4, 256, 72)])
def test_experts_through_the_grouped_tensor_core_product(tokens, experts, top, width, ff):
    """The form for many rows per expert: rows gathered into a layout in which every expert starts on
    a multiple of 256 (rows nobody owns are zeros), the grouped form of the tiled product with the
    activation in its epilogue, the weighted sum through each pair's place - against the form over
    tiles of 64 rows, which the test above holds against a loop."""
    from from_scratch_inference_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(tokens)
    dtype = torch.bfloat16
    y = torch.randn(tokens, width, generator=g).to(dtype).cuda()
    w_gu = (torch.randn(experts, 2 * ff, width, generator=g) / math.sqrt(width)).to(dtype).cuda()
    w_d = (torch.randn(experts, width, ff, generator=g) / math.sqrt(ff)).to(dtype).cuda()
    scores = torch.rand(tokens, experts, generator=g)
    scores[:, 0] += 0.5                              # expert 0 gets most tokens: several tiles of 256
    if experts > 3:
        scores[:, experts - 1] = -1.0                # the last expert none
    ids = scores.topk(top, dim=1).indices.int().cuda()
    weights = (torch.rand(tokens, top, generator=g) + 0.1).cuda()
    pairs, tile = tokens * top, ops.GEMM_TILES_ROWS
    compact = ops.moe_align(ids, pairs, experts, torch.zeros(ops.moe_lists_size(pairs, experts), dtype=torch.int32, device="cuda"))
    act = torch.empty(pairs, ff, dtype=dtype, device="cuda")
    ops.moe_product(y, w_gu, act, compact, pairs, top, True, "silu")
    want_out = torch.empty(pairs, width, dtype=dtype, device="cuda")
    ops.moe_product(act, w_d, want_out, compact, pairs, top, False)
    want = ops.moe_combine(want_out, weights, None, torch.empty(tokens, width, dtype=dtype, device="cuda"), top)

    lists = ops.moe_align(ids, pairs, experts,
                          torch.zeros(ops.moe_lists_size(pairs, experts, tile, True), dtype=torch.int32, device="cuda"),
                          tile, True)
    offsets, order, tile_expert, _, meta, place = lists
    used = int(meta.item())
    counts = torch.bincount(ids.reshape(-1).long().cpu(), minlength=experts)
    assert used == int(((counts + tile - 1) // tile).sum())
    order_host, flat = order.cpu().tolist(), ids.reshape(-1).cpu().tolist()
    assert sorted(p for p in order_host[:used * tile] if p >= 0) == list(range(pairs))
    for m in range(used):
        e = int(tile_expert[m])
        assert all(p < 0 or flat[p] == e for p in order_host[m * tile:(m + 1) * tile])
    assert all(order_host[int(place[p])] == p for p in range(0, pairs, 7))
    rows = (pairs // tile + experts) * tile
    x_sorted = ops.moe_gather(y, lists, tile, top, torch.full((rows, width), 5.0, dtype=dtype, device="cuda"))
    for r in range(0, used * tile, 37):
        p = order_host[r]
        assert torch.equal(x_sorted[r], y[p // top] if p >= 0 else torch.zeros_like(x_sorted[r]))
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    act2 = torch.empty(rows, ff, dtype=dtype, device="cuda")
    ops.gemm_tiles_grouped(ops.GroupedTiledWeight(w_gu, True, "silu"), x_sorted, act2, tile_expert, meta, error, 148)
    out2 = torch.empty(rows, width, dtype=dtype, device="cuda")
    ops.gemm_tiles_grouped(ops.GroupedTiledWeight(w_d, False), act2, out2, tile_expert, meta, error, 148)
    assert int(error.item()) == 0
    got = ops.moe_combine(out2, weights, None, torch.empty(tokens, width, dtype=dtype, device="cuda"), top, place=place)
    scale = max(1.0, float(want.float().abs().max()))
    assert float((got.float() - want.float()).abs().max()) < 2e-2 * scale


# ------------------------------------------------------------------- each mechanism in a model
@pytest.mark.parametrize("name", ["rotated", "gated", "experts", "odd", "loop_first", "loop_last"])
def test_whole_prompt_and_token_by_token(tmp_path_factory, name):
    """The prompt in one step against the same tokens one by one: the first tokens of a sequence,
    page borders, every key of the prompt seen again by every decoded token."""
    folder = folder_of(tmp_path_factory, name)
    requests = {"p": helpers.random_ids(vocab_of(name), 70, 11)}
    runner = runner_for(folder, "float32", num_pages=8)
    rows = helpers.run_trace_in_process(runner, helpers.trace_whole(requests))
    assert len(rows) == 70
    assert_rows(rows, requests, folder, F32_BOUND)
    rows = helpers.run_trace_in_process(runner, helpers.trace_tail_by_one(requests, tail=69))
    assert len(rows) == 70
    assert_rows(rows, requests, folder, F32_BOUND)


def test_faults_would_show_in_the_logits(tmp_path_factory):
    """The test models are sharp enough that a pairing of neighbours instead of half-apart
    columns, frequencies that are not stretched, a missing magnitude factor, a gate left out, a
    correction that enters the weights, masked groups at zero, a stream that enters a pass
    without the embedding output, a missing cap or scale move the logits far beyond the bound the
    engine is held to: the comparisons can tell."""
    def moved(name, change, ids_len=60):
        folder = folder_of(tmp_path_factory, name)
        config, weights = plain.load(folder)
        ids = helpers.random_ids(vocab_of(name), ids_len, 11)
        right = plain.forward(config, weights, ids)
        weights = dict(weights)
        change(config, weights)
        wrong = plain.forward(config, weights, ids)
        return float((wrong - right).abs().max()) / max(1.0, float(right.abs().max()))

    def no_stretch(config, weights):
        config["layers"][0]["mixer"]["rot"]["scaling"] = None

    def other_scale(config, weights):
        config["layers"][0]["mixer"]["scale"] *= 1.1

    def no_gate(config, weights):
        weights["l0.mix.g"] = torch.zeros_like(weights["l0.mix.g"])

    def no_correction(config, weights):
        weights["l0.mlp.correction"] = torch.zeros_like(weights["l0.mlp.correction"])

    def no_groups(config, weights):
        config["layers"][0]["mlp"]["router"].pop("groups")

    def no_embedding_beside(config, weights):
        weights["loop.in"] = weights["loop.in"].clone()
        weights["loop.in"][:, weights["loop.in"].shape[1] // 2:] = 0

    def one_pass_less(config, weights):
        config["loop"]["times"] -= 1

    def no_cap(config, weights):
        config["logit_softcap"] = 0.0

    def no_embedding_scale(config, weights):
        config["embedding"]["scale"] = 1.0

    for name, change in (("rotated", no_stretch), ("rotated", other_scale), ("gated", no_gate),
                         ("experts", no_correction), ("experts", no_groups), ("experts", no_embedding_scale),
                         ("loop", no_embedding_beside), ("loop", one_pass_less), ("loop", no_cap)):
        assert moved(name, change) > 50 * F32_BOUND, (name, change.__name__)


@pytest.mark.parametrize("dtype,name,bound", [("float32", "loop", F32_BOUND), ("bfloat16", "wide", BF16_BOUND)])
def test_far_keys_and_page_borders_in_a_long_prompt(tmp_path_factory, dtype, name, bound):
    """A prompt of several hundred tokens, whole and cut inside a page, beside a short request in
    the same step, then decoding: every layer sees keys hundreds of tokens back (the sharpened
    softmax makes single far keys carry the result), tiles of experts fill and overflow; in
    bfloat16 the long portions take the experts' grouped tensor-core product, the short ones the
    tiles of 64 rows."""
    folder = folder_of(tmp_path_factory, name, sharpen=SHARPEN[dtype])
    requests = {"long": helpers.random_ids(vocab_of(name), 331, 3),
                "short": helpers.random_ids(vocab_of(name), 12, 4)}
    runner = runner_for(folder, dtype, num_pages=48)
    steps = [{"step": 0, "end": ["short"], "entries": [
                  {"id": "long", "tokens": requests["long"][:203], "want": [0, 15, 16, 127, 128, 202]},
                  {"id": "short", "tokens": requests["short"], "want": [0, 11]}]},
             {"step": 1, "end": [], "entries": [
                  {"id": "long", "tokens": requests["long"][203:329], "want": [0, 4, 5, 60, 125]}]},
             {"step": 2, "end": [], "entries": [{"id": "long", "tokens": [requests["long"][329]], "want": [0]}]},
             {"step": 3, "end": ["long"], "entries": [{"id": "long", "tokens": [requests["long"][330]], "want": [0]}]}]
    rows = helpers.run_trace_in_process(runner, steps)
    assert len(rows) == 15
    assert_rows(rows, requests, folder, bound)


def test_sizes_that_fit_no_vector_in_bfloat16(tmp_path_factory):
    """Width 36, experts of 10 and 14, vocabulary 61, head sizes 6 and 10, rank 5 and 9: no row
    starts on 16 bytes.  The bfloat16 products and kernels take their plain forms."""
    folder = folder_of(tmp_path_factory, "odd", sharpen=False)
    requests = {"a": helpers.random_ids(vocab_of("odd"), 45, 6), "b": helpers.random_ids(vocab_of("odd"), 19, 7)}
    runner = runner_for(folder, "bfloat16", num_pages=8)
    for steps in (helpers.trace_whole(requests), helpers.trace_mixed(requests, seed=1, max_live=2)):
        rows = helpers.run_trace_in_process(runner, steps)
        assert len(rows) == 64
        assert_rows(rows, requests, folder, BF16_BOUND)


# ---------------------------------------------------------------------------- the whole design
@pytest.mark.parametrize("name", ["loop", "wide"])
@pytest.mark.parametrize("dtype,bound", [("float32", F32_BOUND), ("bfloat16", BF16_BOUND)])
def test_portions_of_every_size(tmp_path_factory, name, dtype, bound):
    folder = folder_of(tmp_path_factory, name, sharpen=SHARPEN[dtype])
    requests = {"a": helpers.random_ids(vocab_of(name), 90, 1),
                "b": helpers.random_ids(vocab_of(name), 37, 2)}
    runner = runner_for(folder, dtype, num_pages=8)
    steps = helpers.trace_portions(requests, seed=3)
    assert min(len(e["tokens"]) for s in steps for e in s["entries"]) <= 2
    rows = helpers.run_trace_in_process(runner, steps)
    assert len(rows) == 127
    assert_rows(rows, requests, folder, bound)


@pytest.mark.parametrize("dtype,bound", [("float32", F32_BOUND), ("bfloat16", BF16_BOUND)])
def test_mixed_batches_reuse_pages_and_slots(tmp_path_factory, dtype, bound):
    """Six unequal requests through two slots and a pool that holds little more than two of
    them: portions of one beside single tokens of another, requests that sit a step out, one
    that is released in the middle and fed again from its first token - every request's rows
    equal what it gives alone."""
    folder = folder_of(tmp_path_factory, "loop", sharpen=SHARPEN[dtype])
    lengths = {"a": 75, "b": 9, "c": 41, "d": 1, "e": 58, "f": 26}
    requests = {k: helpers.random_ids(vocab_of("loop"), n, i + 20)
                for i, (k, n) in enumerate(lengths.items())}
    steps, names = helpers.trace_mixed_with_recompute(requests, seed=5, max_live=2)
    need = helpers.live_tokens_needed(steps, round_to=16)
    runner = runner_for(folder, dtype, num_pages=need // 16, max_requests=2)
    rows = helpers.run_trace_in_process(runner, steps)
    assert len(rows) >= sum(lengths.values())
    assert_rows(rows, names, folder, bound)
    assert runner.cache.slots.num_free == 2
    assert all(free == need // 16 for free in runner.cache.free_pages())


def test_long_decoding_through_graphs_and_without(tmp_path_factory):
    """A short prompt, then 150 tokens one by one; the decode steps replay captured graphs (the
    routed experts launch the same kernels whatever the router says); the same without graphs
    gives the same rows up to the order of the sums."""
    folder = folder_of(tmp_path_factory, "loop")
    requests = {"long": helpers.random_ids(vocab_of("loop"), 157, 9)}
    steps = helpers.trace_tail_by_one(requests, tail=150)
    both = []
    for graphs in (True, False):
        runner = runner_for(folder, "float32", num_pages=12, cuda_graphs=graphs)
        assert runner.cuda_graphs == graphs
        rows = helpers.run_trace_in_process(runner, steps)
        assert_rows(rows, requests, folder, F32_BOUND)
        both.append(rows)
    for key in both[0]:
        assert float(np.abs(both[0][key] - both[1][key]).max()) < \
            F32_BOUND * max(1.0, float(np.abs(both[0][key]).max()))


def test_decode_batch_with_padding(tmp_path_factory):
    """Three requests decode together in a captured batch of four: the padding entry writes no
    page, and its row in the experts' lists disturbs nobody."""
    folder = folder_of(tmp_path_factory, "wide")
    requests = {k: helpers.random_ids(vocab_of("wide"), n, s)
                for k, n, s in (("a", 30, 1), ("b", 22, 2), ("c", 26, 3))}
    runner = runner_for(folder, "float32", num_pages=12)
    steps = [{"step": 0, "end": [], "entries": [
        {"id": k, "tokens": ids[:12], "want": [11]} for k, ids in requests.items()]}]
    for t in range(12, 22):
        steps.append({"step": len(steps), "end": [], "entries": [
            {"id": k, "tokens": [ids[t]], "want": [0]} for k, ids in requests.items()]})
    steps[-1]["end"] = list(requests)
    rows = helpers.run_trace_in_process(runner, steps)
    assert runner._graphs
    assert_rows(rows, requests, folder, F32_BOUND)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(tmp_path_factory, dtype):
    """Requests of unequal length through `Engine` and its scheduler with a small token budget
    (prompts go in portions) and two slots: every generated token is the plain implementation's
    choice; where the plain logits are a near tie the engine may pick either."""
    from from_scratch_inference_engine_b200 import Engine, LoadedModel, SamplingParams
    folder = folder_of(tmp_path_factory, "loop", sharpen=SHARPEN[dtype])
    model = LoadedModel.from_pretrained(folder, dtype=dtype, max_positions=256)
    engine = Engine(model, block_size=16, num_blocks=16, max_batch=2, max_step_tokens=24)
    prompts = [helpers.random_ids(vocab_of("loop"), n, s) for n, s in ((45, 1), (7, 2), (30, 3))]
    ids = [engine.add_request(p, SamplingParams(temperature=0.0), 8) for p in prompts]
    engine.run_until_done()
    config, weights = plain.load(folder)
    slack = 1e-3 if dtype == "float32" else 0.15
    for rid, prompt in zip(ids, prompts):
        seq = list(prompt)
        assert len(engine.output(rid)) == 8
        for token in engine.output(rid):
            logits = plain.forward(config, weights, seq)[-1]
            assert float(logits.max() - logits[token]) <= slack * max(1.0, float(logits.abs().max()))
            seq.append(token)


def test_llm_entry_point_reads_the_design_by_its_name(tmp_path_factory):
    from from_scratch_inference_engine_b200 import LLM, GenerationConfig, load_config
    folder = folder_of(tmp_path_factory, "odd")
    assert type(load_config(folder)).__name__ == "TapalixConfig"
    llm = LLM(folder, block_size=16, num_blocks=8, max_batch=2, dtype="float32", eos_id=-1)
    prompt = helpers.random_ids(vocab_of("odd"), 19, 4)
    got = llm.generate_ids(prompt, GenerationConfig(max_tokens=5))
    assert len(got) == 5
    config, weights = plain.load(folder)
    seq = list(prompt)
    for token in got:
        logits = plain.forward(config, weights, seq)[-1]
        assert float(logits.max() - logits[token]) <= 1e-3 * max(1.0, float(logits.abs().max()))
        seq.append(token)


@pytest.mark.parametrize("dtype,name,bound", [("float32", "loop", F32_BOUND), ("bfloat16", "wide", BF16_BOUND)])
def test_trace_replay_program_runs_the_design(tmp_path_factory, tmp_path, dtype, name, bound):
    """bin/trace_run as a user runs it (a subprocess, steps on standard input, logits in files)
    on a mixed trace of five requests through four slots and a pool for the live tokens only."""
    import json
    import subprocess
    from pathlib import Path
    folder = folder_of(tmp_path_factory, name, sharpen=SHARPEN[dtype])
    vocab = vocab_of(name)
    requests = {key: helpers.random_ids(vocab, n, i)
                for i, (key, n) in enumerate({"a": 90, "b": 40, "c": 70, "d": 33, "e": 64}.items())}
    steps = helpers.trace_mixed(requests, seed=3)
    need = helpers.live_tokens_needed(steps, round_to=64)
    root = Path(__file__).resolve().parent.parent
    text = "".join(json.dumps(step) + "\n" for step in steps)
    done = subprocess.run([str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
                           "--out", str(tmp_path / "out"), "--max-tokens", str(need)],
                          input=text, capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [line for line in done.stdout.splitlines() if line.startswith("done ")] == \
        [f"done {s['step']}" for s in steps]
    outputs = {s["step"]: np.fromfile(tmp_path / "out" / f"{s['step']}.f32", dtype="<f4").reshape(-1, vocab)
               for s in steps if any(e["want"] for e in s["entries"])}
    rows = helpers.collect_rows(steps, outputs)
    assert len(rows) == sum(len(ids) for ids in requests.values())
    assert_rows(rows, requests, folder, bound)
