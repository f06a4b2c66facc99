"""The Kufulix design in the engine against the plain implementation of the tests: every
mechanism alone, whole prompts against decoding token by token, portions down to two tokens,
mixed batches with pages and slots that are used again, keys far away, at page borders and on
either side of a window's or a chunk's edge in prompts and in decoding, the first tokens of a
sequence, long decoding, and greedy generation through the engine."""

import math

import numpy as np
import pytest
import torch

import helpers
import kufulix_models as km
import plain_kufulix as plain

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
        _folders[key] = km.write_model(tmp_path_factory.mktemp(f"kufulix_{name}"), name, **options)
    return _folders[key]


def plain_rows(folder, ids):
    key = (str(folder), tuple(ids))
    if key not in _plain:
        _plain[key] = plain.logits_for(folder, ids)
    return _plain[key]


def runner_for(folder, dtype, num_pages, max_requests=4, page_size=16, **options):
    from from_scratch_inference_engine_b200 import LoadedModel, ModelRunner
    model = LoadedModel.from_pretrained(folder, dtype=dtype, max_positions=num_pages * page_size)
    return ModelRunner(model.model, model.runtime, page_size=page_size, num_pages=num_pages,
                       max_requests=max_requests, max_step_tokens=num_pages * page_size, **options)


def assert_rows(rows, requests, folder, bound):
    """Every row within `bound` of the plain logits.  bfloat16 rounds every product's result:
    there one row in ten may lie beyond the bound, none beyond three times it."""
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
    return km.CONFIGS[name]["vocab"]


def dev(values, dtype=torch.int32):
    return torch.tensor(values, dtype=dtype, device="cuda")


# ----------------------------------------------------------------- mechanisms, kernel by kernel
def test_weighted_sum_of_two_outputs_meets_the_stream_in_32_bit():
    from from_scratch_inference_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(1)
    for width in (36, 256, 1000, 4104):
        base = torch.randn(7, width, generator=g) * 2 + 0.7
        d1, d2 = torch.randn(7, width, generator=g) * 3, torch.randn(7, width, generator=g)
        stored = torch.randn(width, generator=g) * 0.3
        gain = (1.0 + stored).cuda()
        for dtype in (torch.float32, torch.bfloat16):
            a, b = d1.to(dtype), d2.to(dtype)
            tolerance = 2e-5 if dtype is torch.float32 else 2e-2
            for deltas, scales in (((a,), (0.6,)), ((a, b), (0.6, 1.1))):
                summed = base.double() + sum(s * d.double() for s, d in zip(scales, deltas))
                want = plain.one_plus_norm(summed, stored.double(), 1e-5)
                x = base.clone().cuda()
                out = torch.empty(7, width, device="cuda", dtype=dtype)
                ops.scaled_sum_rmsnorm(x, [d.cuda() for d in deltas], scales, gain, 1e-5, out)
                assert (x.cpu().double() - summed).abs().max() < 2e-5           # the sum stays 32-bit
                assert (out.cpu().double() - want).abs().max() < tolerance * max(1.0, float(want.abs().max()))
            rows = torch.tensor([5, 0, 3], dtype=torch.int32)
            x = base.clone().cuda()
            some = torch.empty(3, width, device="cuda", dtype=dtype)
            ops.scaled_sum_rmsnorm(x, [a.cuda(), b.cuda()], (0.6, 1.1), gain, 1e-5, some, rows=rows.cuda(),
                                   write_x=False)
            assert torch.equal(x.cpu(), base)
            assert torch.equal(some, out[rows.long()])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("normed", [True, False])
def test_heads_normed_then_turned_into_the_cache(dtype, normed):
    """q and k of every head divided by their root mean square and multiplied by the gain BEFORE
    the first columns of the head turn by the rescaled frequencies; q in place, k and v into the
    token's slot of its page; a gate column behind q, k, v is left alone."""
    from from_scratch_inference_engine_b200.kernels import ops
    from from_scratch_inference_engine_b200.parts.rope import llama3_rotary_table
    g = torch.Generator().manual_seed(3)
    heads, kv_heads, dim, vdim, dims, page, eps = 3, 2, 12, 10, 8, 4, 1e-3
    rot = {"base": 50.0, "dims": dims, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}}
    tokens = 9
    positions = torch.tensor([40, 0, 1, 17, 5, 63, 2, 33, 8])
    width = (heads + kv_heads) * dim + kv_heads * vdim
    proj = torch.randn(tokens, width + 3, generator=g).to(dtype)
    q_gain, k_gain = torch.randn(dim, generator=g), torch.randn(dim, generator=g)
    table = torch.from_numpy(llama3_rotary_table(50.0, dims, 64, 4.0, 32, 1.0, 4.0)).cuda()
    slots = torch.tensor([7, 2, 30, 12, 5, 21, -1, 0, 19], dtype=torch.int32)
    pages = 8
    # a page holds its keys and then its values, as the engine lays them out
    both = torch.zeros(pages, kv_heads * page * (dim + vdim), device="cuda", dtype=dtype)
    k_pages, v_pages = both[:, :kv_heads * page * dim], both[:, kv_heads * page * dim:]
    work = proj.clone().cuda()
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.norm_rotate_write(work, positions.int().cuda(), table, slots.cuda(), k_pages, v_pages,
                          both.stride(0), page, heads, kv_heads, dim, vdim, dims,
                          q_gain.cuda() if normed else None, k_gain.cuda() if normed else None, eps, error)
    assert int(error.item()) == 0
    q = proj[:, :heads * dim].double().view(tokens, heads, dim)
    k = proj[:, heads * dim:(heads + kv_heads) * dim].double().view(tokens, kv_heads, dim)
    v = proj[:, (heads + kv_heads) * dim:width].double().view(tokens, kv_heads, vdim)
    if normed:
        q = plain.unit_rms(q, eps) * q_gain.double()
        k = plain.unit_rms(k, eps) * k_gain.double()
    q, k = plain.turn(q, positions, rot), plain.turn(k, positions, rot)
    tolerance = 1e-5 if dtype is torch.float32 else 3e-2
    got_q = work[:, :heads * dim].cpu().double().view(tokens, heads, dim)
    assert (got_q - q).abs().max() < tolerance * max(1.0, float(q.abs().max()))
    assert torch.equal(work[:, width:].cpu(), proj[:, width:])
    kp = k_pages.cpu().double().reshape(pages, kv_heads, page, dim)
    vp = v_pages.cpu().double().reshape(pages, kv_heads, page, vdim)
    for t, slot in enumerate(slots.tolist()):
        if slot < 0:
            continue
        assert (kp[slot // page, :, slot % page] - k[t]).abs().max() < tolerance * max(1.0, float(k.abs().max()))
        assert (vp[slot // page, :, slot % page] - v[t]).abs().max() < 1e-6
    assert float(kp.abs().sum(dim=(1, 3)).ne(0).sum()) == 8          # one token had no slot: nothing stored


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gate_per_head(dtype):
    from from_scratch_inference_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(4)
    for heads, vdim in ((3, 10), (8, 64)):
        out = torch.randn(11, heads * vdim, generator=g).to(dtype)
        wide = torch.randn(11, heads + 9, generator=g).to(dtype).cuda()
        got = ops.head_gate(out.clone().cuda(), wide[:, 5:5 + heads], heads, vdim)
        want = out.double().view(11, heads, vdim) * torch.sigmoid(wide[:, 5:5 + heads].cpu().double())[:, :, None]
        tolerance = 1e-6 if dtype is torch.float32 else 2e-2
        assert (got.cpu().double().view(11, heads, vdim) - want).abs().max() < tolerance * 4


def _paged(rows, page_size, order, pages_total):
    """rows [n, kv_heads, width] laid out as pages [kv_head][slot][width] at the given page ids."""
    n, kv_heads, width = rows.shape
    pages = torch.zeros(pages_total, kv_heads, page_size, width, dtype=rows.dtype)
    table = []
    for b in range(-(-n // page_size)):
        chunk = rows[b * page_size:(b + 1) * page_size]
        pages[order[b], :, :chunk.shape[0]] = chunk.transpose(0, 1)
        table.append(order[b])
    return pages, table


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", ["small", "tensor cores"])
@pytest.mark.parametrize("chunk", [37, 64, 100])
def test_attention_inside_chunks_counted_from_the_start_of_the_sequence(dtype, sizes, chunk):
    """Keys in shuffled pages, a request of 300 cached tokens that brings 77 more and one that
    decodes a token at position 260, whole and split over key ranges.  For chosen queries one key
    is made to stand out - the first key of the query's chunk, while the key just before the
    chunk's start would stand out even more - so that a chunk edge one key off, or chunks counted
    from where the portion starts, changes the output by the size of a value."""
    from from_scratch_inference_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(5 + chunk)
    heads, kv_heads, page = 6, 2, 16
    dk, dv = (24, 40) if sizes == "small" else (48, 128)
    forms = ["plain", "mma", "mma_split"] if sizes != "small" and dtype is torch.bfloat16 else ["auto"]
    group = heads // kv_heads
    lengths = [(300, 77), (260, 1)]
    pages_total = sum(-(-(a + b) // page) for a, b in lengths) + 3
    order = torch.randperm(pages_total, generator=g).tolist()
    scale = 0.5
    k_pages = torch.zeros(pages_total, kv_heads * page * dk, dtype=dtype)
    v_pages = torch.zeros(pages_total, kv_heads * page * dv, dtype=dtype)
    tables, qs, want, used = [], [], [], 0
    for cached, new in lengths:
        n = cached + new
        k = torch.randn(n, kv_heads, dk, generator=g).to(dtype)
        q = torch.randn(new, heads, dk, generator=g)
        for qi in sorted({0, new // 3, new - 1}):
            first = (cached + qi) // chunk * chunk                        # the first key of the query's chunk
            q[qi] = 6.0 * k[first, :, None, :].expand(kv_heads, group, dk).reshape(heads, dk).float() / scale
            if first > 0:
                k[first - 1] = 3.0 * k[first]                             # outside: it would win if it were seen
        q = q.to(dtype)
        v = torch.randn(n, kv_heads, dv, generator=g).to(dtype)
        blocks = -(-n // page)
        kp, table = _paged(k, page, order[used:used + blocks], pages_total)
        vp, _ = _paged(v, page, order[used:used + blocks], pages_total)
        used += blocks
        k_pages += kp.reshape(pages_total, -1)
        v_pages += vp.reshape(pages_total, -1)
        tables.append(table)
        qs.append(q)
        want.append(plain.softmax_attention(
            torch.cat([torch.zeros(cached, heads, dk), q.float()]).double(), k.double(), v.double(),
            plain.chunk_mask(n, chunk), scale)[cached:])
    bt = torch.full((2, max(len(t) for t in tables)), -1, dtype=torch.int32)
    for i, t in enumerate(tables):
        bt[i, :len(t)] = torch.tensor(t, dtype=torch.int32)
    q = torch.cat(qs).reshape(-1, heads * dk).cuda()
    tokens = q.shape[0]
    both = torch.cat([k_pages, v_pages], dim=1).cuda()
    keys = kv_heads * page * dk
    expect = torch.cat(want)
    head_scale = torch.full((heads,), scale, device="cuda")
    for nsplit, form in [(n, f) for n in (1, 3) for f in forms]:
        item, row0 = [], []
        for i, (_, new) in enumerate(lengths):
            for r in range(0, new * group, ops.scaled_attention_rows(dtype, dk, dv, False, form)):
                item.append(i)
                row0.append(r)
        out = torch.zeros(tokens, heads * dv, device="cuda", dtype=dtype)
        error = torch.zeros(1, dtype=torch.int32, device="cuda")
        ops.scaled_attention(q, heads * dk, head_scale, both[:, :keys], both[:, keys:], both.stride(0), page,
                             dk, dv, False, bt.cuda(), dev(item), dev(row0), len(item), dev([0, 77]),
                             dev([77, 1]), dev([300, 260]), dev([0, 1]), out, tokens, heads, kv_heads, 0, error,
                             nsplit, torch.empty(nsplit * tokens * heads * dv, device="cuda"),
                             torch.empty(nsplit * tokens * heads * 2, device="cuda"), form=form, chunk=chunk)
        assert int(error.item()) == 0
        got = out.cpu().double().reshape(tokens, heads, dv)
        tolerance = 2e-4 if dtype is torch.float32 else 4e-2
        assert (got - expect).abs().max() < tolerance * max(1.0, float(expect.abs().max())), (nsplit, form)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,vdim,state,groups,taps,parts", [(3, 8, 6, 1, 3, 1), (4, 5, 7, 2, 4, 2),
                                                                (2, 16, 4, 2, 1, 1), (4, 32, 32, 1, 4, 4)])
def test_state_space_steps_carry_state_between_calls(dtype, heads, vdim, state, groups, taps, parts):
    """The convolution with its kept inputs, step sizes and decays, the scan over a state slot and
    the gated norm in parts: two requests in one call, then each continued in a second call (one of
    them by a single token, one by a portion long enough to run chunk-parallel), against the plain
    recurrence over the whole sequences."""
    from from_scratch_inference_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(heads * 100 + vdim)
    inner, gn = heads * vdim, groups * state
    channels = inner + 2 * gn
    width = 2 * inner + 2 * gn + heads
    eps = 1e-5
    m = {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": taps, "norm_groups": parts}
    w = {"p.conv": torch.randn(channels, taps, generator=g) * 0.5, "p.conv.b": torch.randn(channels, generator=g) * 0.1,
         "p.dt_bias": torch.rand(heads, generator=g) * 3 - 2, "p.A_log": torch.linspace(-4.0, 0.5, heads),
         "p.D": 1 + torch.randn(heads, generator=g) * 0.1, "p.norm": 1 + torch.randn(inner, generator=g) * 0.1}
    lengths = [(5, 1), (9, 170)]                                   # (first call, second call) per request
    projections = [torch.randn(a + b, width, generator=g).to(dtype) for a, b in lengths]
    want = []
    for proj in projections:
        eye = dict({k: v.double() for k, v in w.items()},
                   **{"p.in": torch.eye(width, dtype=torch.float64), "p.o": torch.eye(inner, dtype=torch.float64)})
        want.append(plain.state_space(proj.double(), eye, "p.", m, eps))
    matrix = heads * state * vdim
    floats = -(-(matrix + (taps - 1) * channels) // 4) * 4
    slots = torch.full((3, floats), 7.0, device="cuda")              # slot 1 stays untouched
    slots[0].zero_()
    slots[2].zero_()
    f32 = {k: v.float().cuda().contiguous() for k, v in w.items()}
    got = [[], []]
    for call in range(2):
        parts_in = [p[:a] if call == 0 else p[a:] for p, (a, b) in zip(projections, lengths)]
        proj = torch.cat(parts_in).cuda()
        counts = [p.shape[0] for p in parts_in]
        tokens = sum(counts)
        qstart, qlen, slot = dev([0, counts[0]]), dev(counts), dev([2, 0])
        act = torch.empty(tokens, channels + inner, device="cuda")
        decay = torch.empty(tokens, heads, device="cuda")
        ops.ssd_prep(proj, inner, inner + channels, qstart, qlen, slot, 2, slots, matrix, f32["p.conv"],
                     f32["p.conv.b"], f32["p.dt_bias"], f32["p.A_log"], heads, vdim, act, decay,
                     conv_wt=f32["p.conv"].t().contiguous() if call else None)      # both forms of the kernel
        ops.ssd_tails(proj, inner, channels, taps, qstart, qlen, slot, 2, slots, matrix)
        chunks = {}
        if max(counts) > 128:
            item, row0 = [], []
            for i, n in enumerate(counts):
                for r in range(0, n, 64):
                    item.append(i)
                    row0.append(r)
            chunks = dict(seg_item=dev(item), seg_row0=dev(row0), num_segs=len(item), seg_tokens=64,
                          chunk_states=torch.empty(len(item) * (matrix + heads), device="cuda"))
        o = torch.empty(tokens, inner, device="cuda")
        ops.lightning_scan(act, inner + gn, inner, channels, qstart, qlen, slot, 2, slots, None, o, heads,
                           state, vdim, share=heads // groups, decay_tok=decay, **chunks)
        y = ops.ssd_gate_norm(o, act, proj, 0, f32["p.D"], f32["p.norm"],
                              torch.empty(tokens, inner, device="cuda", dtype=dtype), vdim, parts, eps)
        got[0].append(y[:counts[0]].cpu().double())
        got[1].append(y[counts[0]:].cpu().double())
    assert float((slots[1] - 7.0).abs().max()) == 0.0
    tolerance = 3e-4 if dtype is torch.float32 else 3e-2
    for r in range(2):
        have = torch.cat(got[r])
        assert (have - want[r]).abs().max() < tolerance * max(1.0, float(want[r].abs().max())), r


def test_choice_among_groups_by_their_largest_value_with_identity_experts():
    from from_scratch_inference_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(7)
    for routed, real, top, groups, keep in ((8, 6, 3, 4, 2), (6, 3, 2, 3, 2), (12, 12, 4, 1, 1), (16, 12, 4, 4, 3)):
        tokens = 50
        logits = torch.randn(tokens, routed, generator=g) * 3
        correction = torch.randn(routed, generator=g)
        ids = torch.empty(tokens, top, dtype=torch.int32, device="cuda")
        weights = torch.empty(tokens, top, device="cuda")
        ops.moe_route(None, None, correction.cuda(), ids, weights, top, groups, keep, 1.0, "softmax", True,
                      logits=logits.cuda(), group_score="max")
        w = {"r.router": torch.eye(routed, dtype=torch.float64), "r.correction": correction.double()}
        router = {"experts": real, "identity": routed - real, "top": top}
        if groups > 1:
            router["groups"] = {"count": groups, "keep": keep}
        want_ids, want_w = plain.route(logits.double(), w, "r.", router)
        for t in range(tokens):
            have = dict(zip(ids[t].tolist(), weights[t].tolist()))
            assert set(have) == set(want_ids[t].tolist()), t
            for e, value in zip(want_ids[t].tolist(), want_w[t].tolist()):
                assert abs(have[e] - value) < 1e-5
        # the same choice under "top2" sums is another one for some token: the two rules differ
    logits = torch.tensor([[0.0, 0.0, 0.0, 0.0]])
    correction = torch.tensor([0.9, -5.0, 0.5, 0.45])
    ids = torch.empty(1, 1, dtype=torch.int32, device="cuda")
    weights = torch.empty(1, 1, device="cuda")
    for rule, chosen in (("max", 0), ("top2", 2)):
        ops.moe_route(None, None, correction.cuda(), ids, weights, 1, 2, 1, 1.0, "softmax", True,
                      logits=logits.cuda(), group_score=rule)
        assert int(ids.item()) == chosen


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,width,ff,experts,identity,top", [(9, 36, 10, 3, 3, 2), (70, 64, 24, 6, 2, 3),
                                                                   (700, 128, 64, 4, 2, 2)])
def test_experts_without_gates_and_identity_experts(dtype, tokens, width, ff, experts, identity, top):
    """down(relu(up y)^2) over the pairs sorted by expert - the tiles of 64 rows and, for long
    portions in bfloat16, the grouped tensor-core product - and the weighted sum in which a choice
    beyond the experts gives the token's own row."""
    from from_scratch_inference_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(tokens)
    y = torch.randn(tokens, width, generator=g).to(dtype)
    w_up = (torch.randn(experts, ff, width, generator=g) * 0.2).to(dtype)
    w_down = (torch.randn(experts, width, ff, generator=g) * 0.2).to(dtype)
    scores = torch.rand(tokens, experts + identity, generator=g)
    ids = scores.topk(top, dim=1).indices.int()
    weights = torch.rand(tokens, top, generator=g) + 0.1
    want = torch.zeros(tokens, width, dtype=torch.float64)
    for t in range(tokens):
        for e, wt in zip(ids[t].tolist(), weights[t].tolist()):
            if e >= experts:
                want[t] += wt * y[t].double()
            else:
                up = torch.relu(w_up[e].double() @ y[t].double())
                if dtype is torch.bfloat16:
                    up = up.to(torch.bfloat16).double()          # the stored product, then its square
                want[t] += wt * (w_down[e].double() @ (up * up))
    yd, ids_d, weights_d = y.cuda(), ids.cuda(), weights.cuda()
    pairs = tokens * top
    tolerance = 2e-4 if dtype is torch.float32 else 4e-2
    lists = ops.moe_align(ids_d, pairs, experts, torch.zeros(ops.moe_lists_size(pairs, experts), dtype=torch.int32,
                                                             device="cuda"))
    act = torch.zeros(pairs, ff, dtype=dtype, device="cuda")
    ops.moe_product(yd, w_up.cuda(), act, lists, pairs, top, False, "relu2", first=True)
    expert_out = torch.zeros(pairs, width, dtype=dtype, device="cuda")
    ops.moe_product(act, w_down.cuda(), expert_out, lists, pairs, top, False)
    got = ops.moe_combine(expert_out, weights_d, None, torch.empty(tokens, width, dtype=dtype, device="cuda"), top,
                          ids=ids_d, experts=experts, y=yd)
    assert (got.cpu().double() - want).abs().max() < tolerance * max(1.0, float(want.abs().max()))
    if dtype is not torch.bfloat16 or width % 8 or ff % 8:
        return
    tile = ops.GEMM_TILES_ROWS
    lists = ops.moe_align(ids_d, pairs, experts,
                          torch.zeros(ops.moe_lists_size(pairs, experts, tile, True), dtype=torch.int32, device="cuda"),
                          tile, True)
    rows = (pairs // tile + experts) * tile
    x_sorted = ops.moe_gather(yd, lists, tile, top, torch.empty(rows, width, dtype=dtype, device="cuda"))
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    act2 = torch.empty(rows, ff, dtype=dtype, device="cuda")
    ops.gemm_tiles_grouped(ops.GroupedTiledWeight(w_up.cuda(), False, plain_activation="relu2"), x_sorted, act2,
                           lists[2], lists[4], error, 148)
    out2 = torch.empty(rows, width, dtype=dtype, device="cuda")
    ops.gemm_tiles_grouped(ops.GroupedTiledWeight(w_down.cuda(), False), act2, out2, lists[2], lists[4], error, 148)
    assert int(error.item()) == 0
    got = ops.moe_combine(out2, weights_d, None, torch.empty(tokens, width, dtype=dtype, device="cuda"), top,
                          place=lists[5], ids=ids_d, experts=experts, y=yd)
    assert (got.cpu().double() - want).abs().max() < tolerance * max(1.0, float(want.abs().max()))


# ------------------------------------------------------------------- each mechanism in a model
@pytest.mark.parametrize("name", ["window", "chunk", "experts", "plain", "odd"])
def test_whole_prompt_and_token_by_token(tmp_path_factory, name):
    """The prompt in one step against the same tokens one by one: the first tokens of a sequence,
    page borders, windows and chunks that pass over decoded tokens, the state carried from token
    to token."""
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
    """The test models are sharp enough that a window or a chunk one key off, frequencies that are
    not rescaled, a norm of q and k left out, a missing gate, scales swapped, a state-space mixer
    without its convolution's history or with another decay, a correction that enters the weights,
    groups left out, identity experts left out, a gain without its one, a missing cap move the logits far beyond the bound the engine is held to."""
    def moved(name, change, ids_len=60):
        folder = folder_of(tmp_path_factory, name)
        config, weights = plain.load(folder)
        ids = helpers.random_ids(vocab_of(name), ids_len, 11)
        right = plain.forward(config, weights, ids)
        weights = dict(weights)
        change(config, weights)
        wrong = plain.forward(config, weights, ids)
        return float((wrong - right).abs().max()) / max(1.0, float(right.abs().max()))

    def wider_window(config, weights):
        config["layers"][0]["mixer"]["left"]["mask"]["size"] += 1

    def wider_chunk(config, weights):
        config["layers"][0]["mixer"]["mask"]["size"] += 1

    def no_rescaling(config, weights):
        config["layers"][0]["mixer"]["left"]["rot"]["scaling"] = None

    def plain_norm_of_keys(config, weights):
        weights["l0.mix.left.k.norm"] = torch.ones_like(weights["l0.mix.left.k.norm"])

    def no_gate(config, weights):
        weights["l0.mix.g"] = torch.zeros_like(weights["l0.mix.g"])

    def scales_swapped(config, weights):
        mixer = config["layers"][0]["mixer"]
        mixer["left_scale"], mixer["right_scale"] = mixer["right_scale"], mixer["left_scale"]

    def no_history(config, weights):
        weights["l0.mix.right.conv"] = weights["l0.mix.right.conv"].clone()
        weights["l0.mix.right.conv"][:, :-1] = 0

    def other_decay(config, weights):
        weights["l0.mix.right.A_log"] = weights["l0.mix.right.A_log"] + 0.5

    def no_skip(config, weights):
        weights["l0.mix.right.D"] = torch.zeros_like(weights["l0.mix.right.D"])

    def no_correction(config, weights):
        weights["l0.mlp.correction"] = torch.zeros_like(weights["l0.mlp.correction"])

    def no_groups(config, weights):
        config["layers"][0]["mlp"]["router"].pop("groups")

    def identity_as_nothing(config, weights):
        router = config["layers"][0]["mlp"]["router"]
        router["experts"] += router["identity"]
        router["identity"] = 0
        for e in range(router["experts"] - 2, router["experts"]):
            weights[f"l0.mlp.e{e}.up"] = torch.zeros_like(weights["l0.mlp.e0.up"])
            weights[f"l0.mlp.e{e}.down"] = torch.zeros_like(weights["l0.mlp.e0.down"])

    def gain_without_one(config, weights):
        weights["l0.norm1"] = weights["l0.norm1"] - 1.0

    def no_embedding_norm(config, weights):
        weights["embed.norm"] = weights["embed.norm"] + 1.0

    def no_cap(config, weights):
        config["logit_softcap"] = 0.0

    for name, change in (("window", wider_window), ("window", no_rescaling), ("window", plain_norm_of_keys),
                         ("window", scales_swapped), ("window", no_history), ("window", other_decay),
                         ("window", no_skip), ("window", gain_without_one), ("window", no_embedding_norm),
                         ("chunk", wider_chunk), ("chunk", no_gate), ("chunk", no_cap),
                         ("experts", no_correction), ("experts", no_groups), ("experts", identity_as_nothing)):
        assert moved(name, change) > 50 * F32_BOUND, (name, change.__name__)


@pytest.mark.parametrize("dtype,name,bound", [("float32", "shared", F32_BOUND), ("bfloat16", "wide", BF16_BOUND)])
def test_far_keys_page_borders_and_a_long_prompt(tmp_path_factory, dtype, name, bound):
    """A prompt of several hundred tokens, whole and cut inside a page, a window and a chunk,
    beside a short request in the same step, then decoding: the recurrence runs chunk-parallel
    over the long portions and token by token after them, its slow heads remember hundreds of
    tokens, windows and chunks start inside pages that earlier steps filled; in bfloat16 the long
    portions take the experts' grouped tensor-core product, the short ones the tiles of 64 rows."""
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
    """Width 36, heads of 6 and 10 columns, five state columns per head, experts of 10 and 14:
    no row starts on 16 bytes.  The bfloat16 products and kernels take their plain forms."""
    folder = folder_of(tmp_path_factory, "odd", sharpen=False)
    requests = {"a": helpers.random_ids(vocab_of("odd"), 45, 6), "b": helpers.random_ids(vocab_of("odd"), 19, 7)}
    runner = runner_for(folder, "bfloat16", num_pages=8)
    for steps in (helpers.trace_whole(requests), helpers.trace_mixed(requests, seed=1, max_live=2)):
        rows = helpers.run_trace_in_process(runner, steps)
        assert len(rows) == 64
        assert_rows(rows, requests, folder, BF16_BOUND)


# ---------------------------------------------------------------------------- the whole design
@pytest.mark.parametrize("name", ["shared", "wide"])
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
    that is released in the middle and fed again from its first token into a slot whose state
    another request left - every request's rows equal what it gives alone."""
    folder = folder_of(tmp_path_factory, "shared", sharpen=SHARPEN[dtype])
    lengths = {"a": 75, "b": 9, "c": 41, "d": 1, "e": 58, "f": 26}
    requests = {k: helpers.random_ids(vocab_of("shared"), n, i + 20)
                for i, (k, n) in enumerate(lengths.items())}
    steps, names = helpers.trace_mixed_with_recompute(requests, seed=5, max_live=2)
    need = helpers.live_tokens_needed(steps, round_to=16)
    runner = runner_for(folder, dtype, num_pages=need // 16, max_requests=2)
    rows = helpers.run_trace_in_process(runner, steps)
    assert len(rows) >= sum(lengths.values())
    assert_rows(rows, names, folder, bound)
    assert runner.cache.slots.num_free == 2
    assert all(free == need // 16 for free in runner.cache.free_pages())


def test_pages_behind_windows_and_chunks_are_given_back(tmp_path_factory):
    """A request much longer than the pool: every cache group keeps a window's or a chunk's worth
    of pages, so 400 tokens pass through pages for 96."""
    from from_scratch_inference_engine_b200 import LoadedModel, ModelRunner
    folder = folder_of(tmp_path_factory, "shared")
    requests = {"long": helpers.random_ids(vocab_of("shared"), 400, 8)}
    model = LoadedModel.from_pretrained(folder, dtype="float32", max_positions=512)
    runner = ModelRunner(model.model, model.runtime, page_size=16, num_pages=6, max_requests=2,
                         max_step_tokens=64)
    steps, at = [], 0
    for n in [40, 33, 40, 7, 40, 40, 25, 40, 40, 40, 40, 13]:
        steps.append({"step": len(steps), "end": [], "entries": [
            {"id": "long", "tokens": requests["long"][at:at + n], "want": [0, n - 1]}]})
        at += n
    steps.append({"step": len(steps), "end": ["long"], "entries": [
        {"id": "long", "tokens": requests["long"][at:], "want": [0]}]})
    rows = helpers.run_trace_in_process(runner, steps)
    assert_rows(rows, requests, folder, F32_BOUND)
    assert all(free == 6 for free in runner.cache.free_pages())


def test_long_decoding_through_graphs_and_without(tmp_path_factory):
    """A short prompt, then 150 tokens one by one; the decode steps replay captured graphs (state
    and pages are found through slot numbers and block tables on the device); the same without
    graphs gives the same rows up to the order of the sums."""
    folder = folder_of(tmp_path_factory, "shared")
    requests = {"long": helpers.random_ids(vocab_of("shared"), 157, 9)}
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


def test_decode_batch_with_padding_leaves_other_slots_alone(tmp_path_factory):
    """Three requests decode together in a captured batch of four: the padding entry writes no
    page and no state."""
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
    for state in runner.states:
        if state is not None:
            state.fill_(5.0)                     # a request's first step zeroes the slot it got
    rows = helpers.run_trace_in_process(runner, steps)
    assert runner._graphs
    assert_rows(rows, requests, folder, F32_BOUND)
    for state in runner.states:                  # the fourth slot, which no request held, is as it was
        if state is not None:
            assert int((state == 5.0).all(dim=1).sum()) == 1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(tmp_path_factory, dtype):
    """Requests of unequal length through `Engine` and its scheduler with a small token budget
    (prompts go in portions) and two slots: every generated token is the plain implementation's
    choice; where the plain logits are a near tie the engine may pick either."""
    from from_scratch_inference_engine_b200 import Engine, LoadedModel, SamplingParams
    folder = folder_of(tmp_path_factory, "shared", sharpen=SHARPEN[dtype])
    model = LoadedModel.from_pretrained(folder, dtype=dtype, max_positions=256)
    engine = Engine(model, block_size=16, num_blocks=16, max_batch=2, max_step_tokens=24)
    prompts = [helpers.random_ids(vocab_of("shared"), n, s) for n, s in ((45, 1), (7, 2), (30, 3))]
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
    assert type(load_config(folder)).__name__ == "KufulixConfig"
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


@pytest.mark.parametrize("dtype,name,bound", [("float32", "shared", F32_BOUND), ("bfloat16", "wide", BF16_BOUND)])
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


@pytest.mark.parametrize("seed", [1, 2, 3, 5, 8, 13])
def test_configurations_drawn_at_random(tmp_path_factory, seed):
    """Layer orders, sizes, masks, rotations, routers and shared tensors drawn at random (fixed seeds),
    in float32: a whole prompt, portions beside decoded tokens of another request, and a tail token by
    token, against the plain implementation."""
    folder = km.write_random(tmp_path_factory.mktemp(f"kufulix_random{seed}"), seed)
    vocab = km.CONFIGS[f"random{seed}"]["vocab"]
    requests = {"a": helpers.random_ids(vocab, 150, seed), "b": helpers.random_ids(vocab, 41, seed + 1),
                "c": helpers.random_ids(vocab, 67, seed + 2)}
    runner = runner_for(folder, "float32", num_pages=24)
    for steps in (helpers.trace_whole(requests), helpers.trace_mixed(requests, seed=seed, max_live=3),
                  helpers.trace_tail_by_one({"b": requests["b"]}, tail=30)):
        rows = helpers.run_trace_in_process(runner, steps)
        assert_rows(rows, requests, folder, F32_BOUND)
