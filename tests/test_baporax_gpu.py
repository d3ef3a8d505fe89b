"""Baporax through the engine against the plain implementation (``plain_baporax``).

Kernels alone on drawn and on made-up inputs, then whole models through the replay loop (whole
prompts, token-by-token decoding, portions down to two tokens, mixed batches with pages and state
slots used again), then greedy generation through ``LLMEngine`` and its scheduler.
"""

import pytest
import torch

import baporax_cases as C
import plain_baporax as P
import traces

pytestmark = pytest.mark.gpu

_folders: dict = {}
_references: dict = {}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    for name in C.CASES:
        for sharp in (False, True):
            key = (name, sharp)
            if key not in _folders:
                _folders[key] = C.write_case(name, tmp_path_factory.mktemp(f"baporax_{name}_{int(sharp)}"), sharp)
    return _folders


def reference(folder, requests):
    config, weights = P.read_model_folder(folder)
    out = {}
    for rid, tokens in requests.items():
        key = (str(folder), tuple(tokens))
        if key not in _references:
            _references[key] = P.forward(config, weights, tokens)
        out[rid] = _references[key]
    return out


def run_and_check(folder, dtype, builder, lengths, page_size=16, slack=1.0, **kwargs):
    from turboserve_b200.replay import Replayer

    config = C.read_config(folder)
    requests = traces.make_requests(config["vocab"], lengths, seed=11)
    steps, max_tokens = builder(requests, **kwargs)
    replayer = Replayer(folder, dtype, max_tokens, page_size=page_size)
    got = traces.collect(requests, steps, traces.replay(replayer, steps))
    ref = reference(folder, requests)
    for rid in requests:
        C.check(got[rid], ref[rid], dtype, f"{dtype} {builder.__name__} {rid}", slack)
    replayer.manager.check_invariants()
    assert replayer.manager.free_pages() == [g.num_pages for g in replayer.manager.groups]
    return replayer, got


# ---------------------------------------------------------------------------------------------
# each mechanism alone
# ---------------------------------------------------------------------------------------------


def _dev(t, dtype):
    return t.to("cuda", dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_stream_sum_with_two_updates_a_shift_and_two_norms(dtype):
    from turboserve_b200.ops import kernels

    g = torch.Generator().manual_seed(1)
    n, hidden = 37, 200
    res, a, b = (torch.randn(n, hidden, generator=g) for _ in range(3))
    shift, w1, w2 = (torch.randn(hidden, generator=g) * 0.3 for _ in range(3))
    a, b = a.to(dtype).float(), b.to(dtype).float()
    x = res.double() + a.double() + b.double() + shift.double()
    want1 = P.zero_centred_rms_norm(x, w1.double(), 1e-5)
    want2 = P.zero_centred_rms_norm(x, w2.double(), 1e-5)
    residual = res.cuda()
    out1, out2 = torch.empty(n, hidden, device="cuda", dtype=dtype), torch.empty(n, hidden, device="cuda", dtype=dtype)
    kernels.stream_norm(residual, (_dev(a, dtype), _dev(b, dtype)), shift.cuda(), (1 + w1).cuda(), out1, (1 + w2).cuda(), out2, eps=1e-5)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(residual.cpu().double(), x, atol=1e-5)
    assert torch.allclose(out1.cpu().double(), want1, atol=tol, rtol=tol) and torch.allclose(out2.cpu().double(), want2, atol=tol, rtol=tol)
    # selected rows: the residual stays as it is
    rows = torch.tensor([5, 0, 36], dtype=torch.int32, device="cuda")
    before = residual.clone()
    picked = torch.empty(3, hidden, device="cuda", dtype=dtype)
    kernels.stream_norm(residual, (_dev(a, dtype), _dev(b, dtype)), None, (1 + w1).cuda(), picked, eps=1e-5, rows=rows)
    assert torch.equal(residual, before)
    want = P.zero_centred_rms_norm(before.cpu().double()[rows.cpu().long()] + (a + b).double()[rows.cpu().long()], w1.double(), 1e-5)
    assert torch.allclose(picked.cpu().double(), want, atol=tol, rtol=tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_squared_relu_and_row_scale(dtype):
    from turboserve_b200.ops import kernels

    x = torch.randn(19, 77, generator=torch.Generator().manual_seed(2)).to(dtype)
    out = torch.empty_like(x, device="cuda")
    kernels.activation(x.cuda(), out, "relu2")
    want = torch.clamp(x.double(), min=0) ** 2
    assert torch.allclose(out.cpu().double(), want, rtol=1e-6 if dtype == torch.float32 else 1e-2, atol=0)
    rows = torch.randn(5, 33).cuda()
    kept = rows.clone()
    kernels.scale_rows(rows, 0.37, 3)
    assert torch.allclose(rows[:3], kept[:3] * 0.37) and torch.equal(rows[3:], kept[3:])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_short_convolution_in_portions_with_its_tail_kept(dtype, taps):
    """Three requests whose inputs come in portions of 1 to 9 positions, mixed in one batch per step,
    slots in another order than the requests; every output against the convolution of the whole."""
    from turboserve_b200.ops import kernels

    g = torch.Generator().manual_seed(taps)
    channels, first, width = 70, 5, 90
    lengths = [23, 9, 14]
    slots = [2, 0, 3]
    inputs = [torch.randn(n, channels, generator=g).to(dtype) for n in lengths]
    weight = torch.randn(channels, taps, generator=g)
    bias = torch.randn(channels, generator=g)
    want = [P.silu(P.causal_taps(u.double(), weight.double(), bias.double())) for u in inputs]
    tail = torch.zeros(4, taps - 1, channels, device="cuda", dtype=dtype)
    got = [[] for _ in lengths]
    cursors = [0, 0, 0]
    portion = [1, 3, 2, 9, 1, 1, 4, 2]
    step = 0
    while any(c < n for c, n in zip(cursors, lengths)):
        rows, seq_of, starts, live = [], [], [0], []
        for r, n in enumerate(lengths):
            take = min(portion[(step + r) % len(portion)], n - cursors[r])
            if take == 0 or (step + r) % 5 == 4:  # sometimes a request is left out of a step
                continue
            block = torch.zeros(take, width, dtype=dtype)
            block[:, first:first + channels] = inputs[r][cursors[r]:cursors[r] + take]
            rows.append(block)
            seq_of += [len(live)] * take
            starts.append(starts[-1] + take)
            live.append((r, take))
        step += 1
        if not live:
            continue
        x = torch.cat(rows).cuda()
        out = torch.zeros(x.shape[0], channels, device="cuda", dtype=dtype)
        kernels.causal_conv(x, first, weight.cuda(), bias.cuda(), tail, out,
                            torch.tensor(seq_of, dtype=torch.int32, device="cuda"),
                            torch.tensor(starts, dtype=torch.int32, device="cuda"),
                            torch.tensor([slots[r] for r, _ in live], dtype=torch.int32, device="cuda"),
                            x.shape[0], len(live), silu=True)
        for index, (r, take) in enumerate(live):
            got[r].append(out[starts[index]:starts[index + 1]].cpu())
            cursors[r] += take
    tol = 2e-6 if dtype == torch.float32 else 1e-2
    for r in range(3):
        assert torch.allclose(torch.cat(got[r]).double(), want[r], atol=tol, rtol=tol), r
    assert torch.equal(tail[1], torch.zeros_like(tail[1]))  # a slot nobody holds is not touched


def _paged(keys, values, page_size, order_seed):
    """Scatter whole sequences' keys/values into pages in a shuffled order; returns pages and tables."""
    total = sum(-(-k.shape[0] // page_size) for k in keys) + 3
    perm = torch.randperm(total, generator=torch.Generator().manual_seed(order_seed)).tolist()
    k_pages = torch.zeros(total, page_size, *keys[0].shape[1:], dtype=keys[0].dtype)
    v_pages = torch.zeros(total, page_size, *values[0].shape[1:], dtype=values[0].dtype)
    tables = []
    for k, v in zip(keys, values):
        table = []
        for start in range(0, k.shape[0], page_size):
            page = perm.pop()
            n = min(page_size, k.shape[0] - start)
            k_pages[page, :n], v_pages[page, :n] = k[start:start + n], v[start:start + n]
            table.append(page)
        tables.append(table)
    width = max(len(t) for t in tables)
    return k_pages, v_pages, torch.tensor([t + [-1] * (width - len(t)) for t in tables], dtype=torch.int32)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, window, page_size", [
    (6, 2, 16, 40, 24, 16), (2, 2, 24, 32, None, 8), (4, 1, 8, 96, 17, 16), (8, 2, 64, 128, 64, 32), (3, 3, 5, 7, 1, 4)])
def test_differential_attention_kernel(dtype, heads, kv_heads, dim, vdim, window, page_size):
    """Every position of two sequences (150 and 41 tokens) in one batch, pages in shuffled order."""
    from turboserve_b200.ops import kernels

    g = torch.Generator().manual_seed(heads * 100 + dim)
    lengths = [150, 41]
    qs = [torch.randn(n, heads, 2, dim, generator=g).to(dtype) for n in lengths]
    ks = [(torch.randn(n, kv_heads, 2, dim, generator=g) * 1.5).to(dtype) for n in lengths]
    vs = [torch.randn(n, kv_heads, vdim, generator=g).to(dtype) for n in lengths]
    lam, diff, eps, scale = 0.83, 0.35, 1e-5, 0.4
    want = torch.cat([P.differential_maps(q.double(), k.double(), v.double(), scale, window, lam, diff, eps)
                      for q, k, v in zip(qs, ks, vs)]).reshape(sum(lengths), heads * vdim)
    k_pages, v_pages, table = _paged([k.reshape(k.shape[0], kv_heads, 2 * dim) for k in ks], vs, page_size, 7)
    q = torch.cat(qs).reshape(sum(lengths), heads * 2 * dim).cuda()
    out = torch.empty(sum(lengths), heads * vdim, device="cuda", dtype=dtype)
    seq_of = torch.tensor([0] * lengths[0] + [1] * lengths[1], dtype=torch.int32, device="cuda")
    positions = torch.tensor(list(range(lengths[0])) + list(range(lengths[1])), dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    kernels.diff_attention(q, out, k_pages.cuda(), v_pages.cuda(), table.cuda(), seq_of, positions, sum(lengths), heads,
                           kv_heads, dim, vdim, window, scale, lam, eps, 1.0 - diff, status)
    assert int(status.item()) == 0
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol), float((out.cpu().double() - want).abs().max())


@pytest.mark.parametrize("heads, kv_heads, dim, vdim, window, page_size", [
    (6, 2, 16, 48, 24, 16), (2, 2, 32, 32, None, 8), (4, 1, 64, 128, 100, 16), (8, 2, 128, 64, 64, 32), (3, 3, 48, 16, 1, 4)])
def test_differential_attention_on_tensor_cores(heads, kv_heads, dim, vdim, window, page_size):
    """Portions of three requests in one step: one whole (150 positions), one that is the last 70 positions
    of 300 already in the cache, one of a single position at 41; against the plain function on the whole."""
    from turboserve_b200.ops import kernels

    assert kernels.diff_attention_mma_takes(torch.bfloat16, dim, vdim)
    g = torch.Generator().manual_seed(heads * 100 + dim)
    lengths, portions = [150, 300, 42], [150, 70, 1]
    qs = [torch.randn(n, heads, 2, dim, generator=g).bfloat16() for n in lengths]
    ks = [(torch.randn(n, kv_heads, 2, dim, generator=g) * 1.5).bfloat16() for n in lengths]
    vs = [torch.randn(n, kv_heads, vdim, generator=g).bfloat16() for n in lengths]
    lam, diff, eps, scale = 0.83, 0.35, 1e-5, 0.3
    want = torch.cat([P.differential_maps(q.double(), k.double(), v.double(), scale, window, lam, diff, eps)[-p:]
                      for q, k, v, p in zip(qs, ks, vs, portions)]).reshape(sum(portions), heads * vdim)
    k_pages, v_pages, table = _paged([k.reshape(k.shape[0], kv_heads, 2 * dim) for k in ks], vs, page_size, 7)
    q = torch.cat([q[-p:] for q, p in zip(qs, portions)]).reshape(sum(portions), heads * 2 * dim).cuda()
    out = torch.zeros(sum(portions), heads * vdim, device="cuda", dtype=torch.bfloat16)
    starts = torch.tensor([0, 150, 220, 221], dtype=torch.int32, device="cuda")
    contexts = torch.tensor(lengths, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    kernels.diff_attention_mma(q, out, k_pages.cuda(), v_pages.cuda(), table.cuda(), starts, contexts, sum(portions), 3, heads,
                               kv_heads, dim, vdim, window, scale, lam, eps, 1.0 - diff, status)
    assert int(status.item()) == 0
    assert torch.allclose(out.cpu().double(), want, atol=3e-2, rtol=3e-2), float((out.cpu().double() - want).abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_one_key_that_stands_out_at_the_edge_of_the_window_and_far_back(dtype):
    """One key gets a score far above the others in the first map; its value row is unlike all others.
    A query sees it exactly while it lies within the window: the output's first map is then that value
    row, else the mean of ordinary rows. Without a window a key 700 positions back is found."""
    from turboserve_b200.ops import kernels

    heads = kv_heads = 1
    dim, vdim, n, page_size = 16, 32, 720, 16
    special = 9
    g = torch.Generator().manual_seed(5)
    k = torch.randn(n, 1, 2, dim, generator=g) * 0.05
    v = torch.randn(n, 1, vdim, generator=g) * 0.1
    k[special, 0, 0] = 0.0
    k[special, 0, 0, 3] = 40.0
    v[special, 0] = 0.0
    v[special, 0, 11] = 25.0
    q = torch.randn(n, 1, 2, dim, generator=g) * 0.05
    q[:, 0, 0, 3] = 1.0
    k_pages, v_pages, table = _paged([k.reshape(n, 1, 2 * dim).to(dtype)], [v.to(dtype)], page_size, 3)
    for window in (48, None):
        rows = [special, special + 1, special + 46, special + 47, special + 48, special + 49, n - 1]
        out = torch.empty(len(rows), vdim, device="cuda", dtype=dtype)
        kernels.diff_attention(q[rows].reshape(len(rows), 2 * dim).to(dtype).cuda(), out, k_pages.cuda(), v_pages.cuda(),
                               table.cuda(), torch.zeros(len(rows), dtype=torch.int32, device="cuda"),
                               torch.tensor(rows, dtype=torch.int32, device="cuda"), len(rows), 1, 1, dim, vdim, window, 1.0,
                               0.0, 1e-6, 1.0)
        want = P.differential_maps(q.double().to(dtype).double(), k.to(dtype).double(), v.to(dtype).double(), 1.0, window, 0.0, 0.0, 1e-6)[rows, 0]
        assert torch.allclose(out.cpu().double(), want, atol=3e-2, rtol=3e-2)
        peak = out.cpu().float()[:, 11] / out.cpu().float().norm(dim=-1)
        sees = [True, True, True, True, window is None, window is None, window is None]
        for value, inside in zip(peak.tolist(), sees):
            assert (value > 0.99) == inside, (window, peak.tolist())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, groups, vdim, state", [(4, 1, 24, 16), (6, 3, 16, 48), (2, 2, 40, 24), (4, 2, 64, 128), (3, 1, 5, 200)])
def test_state_space_scan_whole_and_in_portions(dtype, heads, groups, vdim, state):
    """Two requests: whole in one step, then again cut into portions of 1 to 40 positions in mixed
    batches with other slots; outputs and final states agree with the plain recurrence."""
    from turboserve_b200.ops import kernels

    g = torch.Generator().manual_seed(state)
    lengths = [90, 33]
    inner = heads * vdim
    width = inner + 2 * groups * state
    xbc = [(torch.randn(n, width, generator=g) * 0.5).to(dtype) for n in lengths]
    dt_raw = [torch.randn(n, heads, generator=g).to(dtype) for n in lengths]
    dt_bias, a_log, d_skip = torch.randn(heads, generator=g) * 0.5, torch.randn(heads, generator=g) * 0.5 - 1.0, torch.randn(heads, generator=g)
    want = []
    for u, raw in zip(xbc, dt_raw):
        u = u.double()
        n = u.shape[0]
        want.append(P.ssd_recurrence(u[:, :inner].reshape(n, heads, vdim), u[:, inner:inner + groups * state].reshape(n, groups, state),
                                     u[:, inner + groups * state:].reshape(n, groups, state),
                                     P.softplus(raw.double() + dt_bias.double()), a_log.double(), d_skip.double(), groups).reshape(n, inner))
    tol = 3e-5 if dtype == torch.float32 else 2e-2

    def run(portions, slots):
        states = torch.zeros(5, heads, vdim, state, device="cuda")
        got = [[] for _ in lengths]
        cursors = [0, 0]
        k = 0
        while any(c < n for c, n in zip(cursors, lengths)):
            pieces, raws, starts, live = [], [], [0], []
            for r, n in enumerate(lengths):
                take = min(portions[(k + r) % len(portions)], n - cursors[r])
                if take:
                    pieces.append(xbc[r][cursors[r]:cursors[r] + take])
                    raws.append(dt_raw[r][cursors[r]:cursors[r] + take])
                    starts.append(starts[-1] + take)
                    live.append((r, take))
            k += 1
            y = torch.zeros(starts[-1], inner, device="cuda")
            kernels.ssd_scan(torch.cat(pieces).cuda(), torch.cat(raws).cuda(), dt_bias.cuda(), a_log.cuda(), d_skip.cuda(), states, y,
                             torch.tensor(starts, dtype=torch.int32, device="cuda"),
                             torch.tensor([slots[r] for r, _ in live], dtype=torch.int32, device="cuda"), len(live), heads, groups,
                             vdim, state)
            for index, (r, take) in enumerate(live):
                got[r].append(y[starts[index]:starts[index + 1]].cpu())
                cursors[r] += take
        return [torch.cat(parts).double() for parts in got], states.cpu()

    whole, whole_states = run([1000], [1, 3])
    cut, cut_states = run([1, 40, 2, 7, 1, 13], [4, 0])
    for r in range(2):
        scale = want[r].abs().max()
        assert (whole[r] - want[r]).abs().max() <= tol * scale and (cut[r] - want[r]).abs().max() <= tol * scale
    assert torch.allclose(whole_states[1], cut_states[4], atol=1e-4, rtol=1e-4) and torch.allclose(whole_states[3], cut_states[0], atol=1e-4, rtol=1e-4)
    assert torch.equal(whole_states[0], torch.zeros_like(whole_states[0]))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("parts", [1, 2, 4])
def test_gated_grouped_norm(dtype, parts):
    from turboserve_b200.ops import kernels

    g = torch.Generator().manual_seed(parts)
    n, inner = 21, 96
    y = torch.randn(n, inner, generator=g)
    z = torch.randn(n, inner + 30, generator=g).to(dtype)
    w = 1 + 0.2 * torch.randn(inner, generator=g)
    v = (y.double() * P.silu(z[:, 10:10 + inner].double())).view(n, parts, inner // parts)
    want = (v / torch.sqrt((v * v).mean(-1, keepdim=True) + 1e-5)).reshape(n, inner) * w.double()
    out = torch.empty(n, inner, device="cuda", dtype=dtype)
    kernels.gated_group_norm(y.cuda(), z.cuda()[:, 10:10 + inner], w.cuda(), out, n, parts, 1e-5)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol)


# ---------------------------------------------------------------------------------------------
# whole models through the replay loop
# ---------------------------------------------------------------------------------------------

LENGTHS = {"X": [1, 7, 33, 100, 150], "Y": [5, 40, 129, 70], "Z": [3, 64, 130, 200], "W": [2, 9, 61, 140], "V": [4, 37, 150, 260]}
MIXED_LENGTHS = [33, 100, 20, 150, 64, 7, 90, 129, 48, 5, 77, 130]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["X", "Y", "Z", "W", "V"])
def test_each_request_alone_and_whole(folders, name, dtype):
    run_and_check(folders[name, False], dtype, traces.whole, LENGTHS[name])


@pytest.mark.parametrize("name", ["X", "Y", "Z"])
def test_the_stream_after_every_layer_run(folders, name):
    """The float32 residual stream after each run of the run order (a looped layer counts each time)."""
    from turboserve_b200.parts.block import ParallelBlock
    from turboserve_b200.replay import Replayer

    folder = folders[name, False]
    config, weights = P.read_model_folder(folder)
    tokens = traces.make_requests(config["vocab"], [45], seed=3)["r0"]
    want: list = []
    P.forward(config, weights, tokens, want)
    replayer = Replayer(folder, "float32", 64)
    got = []
    original = ParallelBlock.forward

    def recording(self, residual, pending, ctx, cache, shift=None):
        out = original(self, residual, pending, ctx, cache, shift=shift)
        stream = residual[:ctx.batch.num_tokens].clone()
        for update in (out if isinstance(out, tuple) else (out,)):
            stream += update.float()
        got.append(stream.cpu().double())
        return out

    ParallelBlock.forward = recording
    try:
        replayer.step([{"id": "a", "tokens": tokens, "want": []}], ["a"])
    finally:
        ParallelBlock.forward = original
    assert len(got) == len(want) == len(P.run_order(config))
    for index, (ours, ref) in enumerate(zip(got, want)):
        assert (ours - ref).abs().max() <= 2e-5 * max(1.0, float(ref.abs().max())), index


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["X", "Y", "Z", "W", "V"])
def test_prompt_then_token_by_token(folders, name, dtype):
    """The last tokens one by one: more of them than the longest window, so it passes over decoded tokens."""
    run_and_check(folders[name, False], dtype, traces.tail_one_by_one, LENGTHS[name], tail=80)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["X", "Y", "Z"])
def test_portions_of_changing_size_down_to_two_tokens(folders, name, dtype):
    run_and_check(folders[name, False], dtype, traces.changing_portions, LENGTHS[name])
    run_and_check(folders[name, False], dtype, traces.changing_portions, LENGTHS[name][-2:], sizes=(2, 2, 3, 2, 1, 2), page_size=8)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["X", "Y", "Z", "W", "V"])
@pytest.mark.parametrize("page_size", [16, 8])
def test_mixed_batches_with_pages_and_slots_used_again(folders, name, dtype, page_size):
    """Twelve requests, four live at a time, unequal portions beside single tokens: four state slots and
    a pool that holds the live requests only, so every slot and page goes to several requests."""
    replayer, _ = run_and_check(folders[name, False], dtype, traces.mixed, MIXED_LENGTHS, page_size=page_size, seed=3)
    assert replayer.manager.slots.num_slots == 4
    for pool, group in zip(replayer.manager.pools, replayer.manager.groups):
        assert pool.num_allocations > group.num_pages


@pytest.mark.parametrize("name", ["X", "Y", "Z"])
def test_sharp_scores_and_slow_decay_in_float32(folders, name):
    """Weights under which single keys stand out and the state remembers hundreds of tokens: windows'
    edges, keys far back (the layer without a window sees 400 positions) and carried state, in prompts,
    in portions, token by token and in mixed batches."""
    folder = folders[name, True]
    lengths = [400, 170]
    run_and_check(folder, "float32", traces.whole, lengths, slack=2.5)
    run_and_check(folder, "float32", traces.tail_one_by_one, lengths, tail=90, slack=2.5)
    run_and_check(folder, "float32", traces.changing_portions, lengths, page_size=8, slack=2.5)
    run_and_check(folder, "float32", traces.mixed, [170, 60, 200, 33, 90, 120], seed=8, slack=2.5)


@pytest.mark.parametrize("name", ["X", "Z"])
def test_sharp_scores_in_bfloat16_token_by_token(folders, name):
    run_and_check(folders[name, True], "bfloat16", traces.tail_one_by_one, [300], tail=100, slack=3.0)
    run_and_check(folders[name, True], "bfloat16", traces.mixed, [170, 60, 200, 33, 90], seed=8, slack=3.0)


@pytest.mark.parametrize("name", ["X", "Y"])
def test_float32_logits_do_not_depend_on_the_cut_at_all(folders, name):
    """Every float32 sum of a position has one order however its request is cut or batched."""
    folder = folders[name, False]
    _, a = run_and_check(folder, "float32", traces.whole, LENGTHS[name])
    _, b = run_and_check(folder, "float32", traces.changing_portions, LENGTHS[name])
    _, c = run_and_check(folder, "float32", traces.mixed, LENGTHS[name], seed=5)
    for rid in a:
        assert torch.equal(a[rid], b[rid]) and torch.equal(a[rid], c[rid]), rid


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(folders, dtype):
    """Positions 0, 1, 2 one by one and two at once: taps that reach before the start, an empty state."""
    from turboserve_b200.replay import Replayer

    for name in C.CASES:
        folder = folders[name, False]
        config, weights = P.read_model_folder(folder)
        tokens = [5, 9, 2]
        ref = P.forward(config, weights, tokens)
        replayer = Replayer(folder, dtype, 64)
        rows = [replayer.step([{"id": "x", "tokens": [t], "want": [0]}], []) for t in tokens]
        C.check(torch.cat(rows), ref, dtype, f"{name} first tokens")
        replayer.step([], ["x"])
        both = replayer.step([{"id": "y", "tokens": tokens[:2], "want": [0, 1]}], ["y"])
        C.check(both, ref[:2], dtype, f"{name} first two tokens")


def test_a_slot_that_is_used_again_starts_empty(folders):
    """A request that follows another in the same state slot gets what it gets alone (float32, same bits)."""
    from turboserve_b200.replay import Replayer

    folder = folders["X", True]
    config = C.read_config(folder)
    requests = traces.make_requests(config["vocab"], [70, 40], seed=9)
    replayer = Replayer(folder, "float32", 128, state_slots=1)
    first = replayer.step([{"id": "a", "tokens": requests["r0"], "want": [69]}], ["a"])
    second = replayer.step([{"id": "b", "tokens": requests["r1"], "want": list(range(40))}], ["b"])
    alone = Replayer(folder, "float32", 128, state_slots=1).step([{"id": "b", "tokens": requests["r1"], "want": list(range(40))}], ["b"])
    assert first is not None and torch.equal(second, alone)


def test_long_decoding(folders):
    """600 tokens one by one after a short prompt: the window passes over decoded tokens many times,
    pages behind it are given back, the state is carried 600 steps."""
    replayer, _ = run_and_check(folders["X", True], "float32", traces.tail_one_by_one, [620], tail=600, slack=2.5, page_size=8)
    assert replayer.manager.num_window_releases > 0


# ---------------------------------------------------------------------------------------------
# generation through the engine's own entry point and scheduler
# ---------------------------------------------------------------------------------------------


def engine_for(folder, dtype, **scheduler):
    from turboserve_b200 import EngineConfig, LLMEngine, SchedulerConfig

    defaults = dict(max_num_seqs=4, max_num_batched_tokens=256, block_size=16, num_blocks=64)
    defaults.update(scheduler)
    return LLMEngine(EngineConfig(model=str(folder), dtype=dtype, scheduler=SchedulerConfig(**defaults)))


def check_greedy_path(config, weights, prompt, generated, dtype):
    """Every generated token is the plain argmax given the tokens before it (in bfloat16: or a token
    whose plain logit lies within the bfloat16 tolerance of the best)."""
    logits = P.forward(config, weights, prompt + generated)
    spread = float((logits - logits.mean(-1, keepdim=True)).pow(2).mean().sqrt())
    slack = (C.FP32_REL if dtype == "float32" else C.BF16_REL) * spread * 4
    for i, token in enumerate(generated):
        row = logits[len(prompt) + i - 1]
        best = int(row.argmax())
        assert token == best or row[best] - row[token] <= slack, (i, token, best, float(row[best] - row[token]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name, lengths, new", [("X", [1, 7, 33, 100, 60, 12], 40), ("Y", [5, 40, 129], 30), ("Z", [3, 70], 24)])
def test_greedy_generation_through_the_engine(folders, name, lengths, new, dtype):
    from turboserve_b200 import SamplingParams

    folder = folders[name, False]
    config, weights = P.read_model_folder(folder)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, config["vocab"], (n,), generator=g).tolist() for n in lengths]
    with engine_for(folder, dtype) as engine:
        outputs = engine.generate(prompts, SamplingParams(max_tokens=new, temperature=0.0, ignore_eos=True))
        assert engine.cache.free_pages() == [g.num_pages for g in engine.cache.groups]
        if dtype == "bfloat16":
            assert engine.runner.num_graph_replays > 0  # decode steps of this model are replayed from graphs
    for prompt, out in zip(prompts, outputs):
        assert out.finished and out.output_tokens == new and out.prompt_tokens == len(prompt)
        check_greedy_path(config, weights, prompt, out.token_ids, dtype)
    if dtype == "float32":
        assert outputs[1].token_ids[:6] == P.greedy(config, weights, prompts[1], 6)


def test_small_budget_and_few_pages_change_no_token(folders):
    """Prompts cut by a token budget of 16, and a pool too small for everyone (requests are preempted,
    their slots zeroed and their prompts computed again): the same tokens in float32."""
    from turboserve_b200 import SamplingParams

    folder = folders["X", False]
    config = C.read_config(folder)
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, config["vocab"], (n,), generator=g).tolist() for n in [5, 40, 129, 33, 64, 18]]
    sampling = SamplingParams(max_tokens=24, temperature=0.0, ignore_eos=True)
    with engine_for(folder, "float32") as engine:
        base = [o.token_ids for o in engine.generate(prompts, sampling)]
    with engine_for(folder, "float32", max_num_batched_tokens=16) as engine:
        chunked = [o.token_ids for o in engine.generate(prompts, sampling)]
    with engine_for(folder, "float32", max_num_batched_tokens=64, num_blocks=14) as engine:
        tight = [o.token_ids for o in engine.generate(prompts, sampling)]
        stats = engine.stats()
        engine.scheduler.check_invariants()
    assert chunked == base and tight == base
    assert stats["num_preemptions"] > 0


def test_bfloat16_with_graphs_steps_launched_ahead_and_preemption_together(folders):
    """A pool too small for everyone, a small token budget, captured graphs and decode steps launched ahead
    of the tokens being read: requests are preempted (their state slots zeroed when they come back) and every
    token still follows the plain logits."""
    from turboserve_b200 import SamplingParams

    folder = folders["X", False]  # its layer without a window keeps every page: the pool runs out
    config, weights = P.read_model_folder(folder)
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, config["vocab"], (n,), generator=g).tolist() for n in [5, 40, 129, 33, 64, 18, 90]]
    sampling = SamplingParams(max_tokens=40, temperature=0.0, ignore_eos=True)
    with engine_for(folder, "bfloat16", max_num_seqs=4, max_num_batched_tokens=64, num_blocks=22) as engine:
        outputs = engine.generate(prompts, sampling)
        stats = engine.stats()
        engine.scheduler.check_invariants()
        assert engine.cache.free_pages() == [g.num_pages for g in engine.cache.groups]
    assert stats["num_preemptions"] > 0 and stats["num_overlapped_steps"] > 0
    for prompt, out in zip(prompts, outputs):
        assert out.output_tokens == 40
        check_greedy_path(config, weights, prompt, out.token_ids, "bfloat16")
