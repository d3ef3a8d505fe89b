"""Filezen through the engine against the plain implementation (``plain_filezen``).

Kernels and parts alone on drawn and on made-up inputs, then whole models through the replay loop (whole
prompts, token-by-token decoding, portions down to two tokens, mixed batches with pages and state slots
used again), then greedy generation through ``LLMEngine`` and its scheduler.
"""

import pytest
import torch

import filezen_cases as C
import plain_filezen as P
import traces

pytestmark = pytest.mark.gpu

_folders: dict = {}
_references: dict = {}


class _Folders(dict):
    """Model folders by ``(case, sharp)`` or ``(case, sharp, dtype)``, written when first asked for. A bfloat16
    comparison gets the folder whose routers are steady (``filezen_cases.steady_routing``)."""

    def __init__(self, factory):
        super().__init__()
        self.factory = factory

    def __missing__(self, key):
        name, sharp = key[0], key[1]
        steady = len(key) > 2 and key[2] == "bfloat16"
        self[key] = C.write_case(name, self.factory.mktemp(f"filezen_{name}_{int(sharp)}_{int(steady)}"), sharp, steady)
        return self[key]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    global _folders
    if not isinstance(_folders, _Folders):
        _folders = _Folders(tmp_path_factory)
    return _folders


def reference(folder, requests):
    config, weights = P.read_model_folder(folder)
    out = {}
    for rid, tokens in requests.items():
        key = (str(folder), tuple(tokens))
        if key not in _references:
            _references[key] = P.logits_of(config, weights, tokens)
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


def _i32(values):
    return torch.tensor(values, dtype=torch.int32, device="cuda")


def _context(query_lens, dtype, starts=None, slots=None, tables=None):
    """A step context for parts that are run alone: one request per entry of ``query_lens``."""
    from turboserve_b200.engine.batch import RequestSlice, StepContext, Workspace, build_step_batch

    starts = starts or [0] * len(query_lens)
    slots = slots or list(range(len(query_lens)))
    tables = tables or [[0]] * len(query_lens)
    slices = [RequestSlice(token_ids=[0] * n, start_position=s, block_tables=[list(t)], state_slot=slot)
              for n, s, slot, t in zip(query_lens, starts, slots, tables)]
    batch = build_step_batch(slices, 1, "cuda")
    return StepContext(batch=batch, workspace=Workspace("cuda"), dtype=dtype, device=torch.device("cuda"),
                       status=torch.zeros(1, dtype=torch.int32, device="cuda"))


# ---------------------------------------------------------------------------------------------
# each mechanism alone
# ---------------------------------------------------------------------------------------------


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_behind_a_sublayer(dtype):
    from turboserve_b200.ops import kernels

    g = torch.Generator().manual_seed(1)
    n, hidden = 29, 200
    res = torch.randn(n, hidden, generator=g)
    update = (torch.randn(n, hidden, generator=g) * 3.0).to(dtype)
    gain = 1 + 0.3 * torch.randn(hidden, generator=g)
    want = res.double() + 0.7 * P.rms_norm(update.double(), gain.double(), 1e-5)
    residual, copy = res.cuda(), torch.zeros(n, hidden, device="cuda", dtype=dtype)
    kernels.norm_add(residual, update.cuda(), gain.cuda(), copy, 1e-5, 0.7, n)
    assert torch.allclose(residual.cpu().double(), want, atol=1e-5)
    assert torch.allclose(copy.cpu().double(), want, atol=1e-5 if dtype == torch.float32 else 3e-2, rtol=1e-2)
    only = torch.zeros(n, hidden, device="cuda", dtype=dtype)
    kernels.norm_add(residual, None, None, only, 0.0, 0.0, n)  # the copy alone
    assert torch.equal(only, residual.to(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, dim, rot_dim, rank, scaling", [(4, 24, 8, 40, (4.0, 64, 16.0, 2.0)), (3, 20, 6, 45, None), (1, 10, 2, 18, None),
                                                                (8, 32, 32, 96, (6.0, 128, 24.0, 1.5))])
def test_latent_rows_are_normed_rotated_and_appended(dtype, heads, dim, rot_dim, rank, scaling):
    """Positions 37..99 of a request whose pages are in no order: the cache rows and the queries' rotated parts."""
    from turboserve_b200.ops import kernels
    from turboserve_b200.parts.rope import scaled_rotary_frequencies

    g = torch.Generator().manual_seed(rank)
    first, n, page_size, eps = 37, 63, 8, 1e-5
    rot = C.rot(3000.0, rot_dim, scaling)
    down = torch.randn(first + n, rank + rot_dim, generator=g).to(dtype)
    weight = 1 + 0.2 * torch.randn(rank, generator=g)
    q = torch.randn(first + n, heads, dim + rot_dim, generator=g).to(dtype)
    sizes = dict(kv_rank=rank, rot_dim=rot_dim, rot=rot)
    latent, shared = P.latent_cache(down.double(), {"dkv": torch.eye(rank + rot_dim, dtype=torch.float64), "dkv.norm": weight.double()}, sizes, eps)
    want_q = torch.cat([q.double()[..., :dim], P.rotate(q.double()[..., dim:], torch.arange(first + n), rot)], dim=-1)
    pages_needed = -(-(first + n) // page_size)
    table = torch.randperm(pages_needed + 3, generator=g)[:pages_needed].tolist()
    pages = torch.zeros(pages_needed + 3, page_size, 1, rank + rot_dim, device="cuda", dtype=dtype)
    freq, amplitude = scaled_rotary_frequencies(rot_dim, 3000.0, rot.get("scaling"))
    proj = q[first:].reshape(n, heads * (dim + rot_dim)).cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    kernels.latent_prepare(proj, down[first:].cuda(), weight.cuda(), freq.cuda(), amplitude, _i32(range(first, first + n)),
                           _i32([0] * n), _i32([table]), pages, n, heads, dim, rot_dim, rank, eps, status)
    assert int(status.item()) == 0
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(proj.cpu().double().reshape(n, heads, -1), want_q[first:], atol=tol, rtol=tol)
    rows = torch.stack([pages[table[p // page_size], p % page_size, 0] for p in range(first, first + n)]).cpu().double()
    assert torch.allclose(rows[:, :rank], latent[first:], atol=tol, rtol=tol) and torch.allclose(rows[:, rank:], shared[first:], atol=tol, rtol=tol)
    assert float(pages[table[0]].abs().max()) == 0.0  # positions before the step are not written


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_products_of_all_heads_in_one_launch(dtype):
    from turboserve_b200.ops import kernels

    g = torch.Generator().manual_seed(3)
    n, heads, k, out_n, in_head, out_head = 70, 5, 20, 45, 26, 50
    x = torch.randn(n, heads * in_head, generator=g).to(dtype)
    w = torch.randn(heads, out_n, k, generator=g).to(dtype)
    want = torch.einsum("thk,hnk->thn", x.double().reshape(n, heads, in_head)[..., :k], w.double())
    out = torch.zeros(n, heads * out_head, device="cuda", dtype=dtype)
    kernels.head_linear(x.cuda(), in_head, w.cuda(), out, out_head, n)
    got = out.cpu().double().reshape(n, heads, out_head)
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    assert torch.allclose(got[..., :out_n], want, atol=tol * 5, rtol=tol) and float(got[..., out_n:].abs().max()) == 0.0


def _latent_pages(rows, page_size, seed):
    total = sum(-(-r.shape[0] // page_size) for r in rows) + 3
    perm = torch.randperm(total, generator=torch.Generator().manual_seed(seed)).tolist()
    pages = torch.zeros(total, page_size, 1, rows[0].shape[1], dtype=rows[0].dtype)
    tables = []
    for r in rows:
        table = []
        for start in range(0, r.shape[0], page_size):
            page = perm.pop()
            n = min(page_size, r.shape[0] - start)
            pages[page, :n, 0] = r[start:start + n]
            table.append(page)
        tables.append(table)
    width = max(len(t) for t in tables)
    return pages, torch.tensor([t + [-1] * (width - len(t)) for t in tables], dtype=torch.int32)


def _latent_reference(q_lat, q_rot, rows, rank, scale, window):
    """[T, heads, rank]: softmax over the window of (q_lat . c + q_rot . r) * scale, times the latents c."""
    scores = torch.einsum("thc,sc->hts", q_lat, rows[:, :rank]) + torch.einsum("thr,sr->hts", q_rot, rows[:, rank:])
    return torch.einsum("hts,sc->thc", P.window_softmax(scores * scale, window), rows[:, :rank])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, rank, rot, window, page_size", [(4, 40, 8, 24, 16), (8, 16, 4, None, 8), (3, 45, 6, 9, 4), (8, 96, 32, 64, 32),
                                                                  (4, 160, 8, 30, 16), (6, 300, 16, 50, 16), (1, 18, 2, 1, 4)])
def test_attention_over_latent_rows(dtype, heads, rank, rot, window, page_size):
    """Every position of two sequences (150 and 41 tokens) in one batch, pages in shuffled order."""
    from turboserve_b200.ops import kernels

    g = torch.Generator().manual_seed(heads * 100 + rank)
    lengths = [150, 41]
    q_lat = [(torch.randn(n, heads, rank, generator=g) * 0.6).to(dtype) for n in lengths]
    q_rot = [torch.randn(n, heads, rot, generator=g).to(dtype) for n in lengths]
    rows = [torch.randn(n, rank + rot, generator=g).to(dtype) for n in lengths]
    scale = 0.3
    want = torch.cat([_latent_reference(a.double(), b.double(), r.double(), rank, scale, window)
                      for a, b, r in zip(q_lat, q_rot, rows)]).reshape(sum(lengths), heads * rank)
    pages, table = _latent_pages(rows, page_size, 7)
    out = torch.empty(sum(lengths), heads * rank, device="cuda", dtype=dtype)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    packed = torch.cat([torch.cat(q_lat), torch.cat(q_rot)], dim=-1).reshape(sum(lengths), heads * (rank + rot))
    kernels.latent_attention(packed.cuda(), out, pages.cuda(), table.cuda(), _i32([0] * lengths[0] + [1] * lengths[1]),
                             _i32(list(range(lengths[0])) + list(range(lengths[1]))), sum(lengths), heads, rank, rot, window, scale, status)
    assert int(status.item()) == 0
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol), float((out.cpu().double() - want).abs().max())


def test_rows_gathered_and_the_softmax_under_the_mask():
    """The two kernels around the matrix products of long portions: the rows of a range of positions from shuffled
    pages (padded with zeros), and the softmax of a stretch of queries under the causal mask and the window."""
    from turboserve_b200.ops import kernels

    g = torch.Generator().manual_seed(8)
    rows = torch.randn(100, 24, generator=g).bfloat16()
    pages, table = _latent_pages([rows], 8, 5)
    got = torch.full((48, 24), 7.0, device="cuda", dtype=torch.bfloat16)
    kernels.latent_gather(pages.cuda(), table.cuda()[0], 31, 43, got, 48)
    assert torch.equal(got[:43].cpu(), rows[31:74]) and float(got[43:].abs().max()) == 0.0
    heads, first_query, first_key, window, keys, scale = 3, 40, 21, 20, 43, 0.7
    queries = 24  # positions 40..63 against keys 21..63
    scores = torch.randn(queries * heads, 48, generator=g) * 3.0
    weights = torch.full((queries * heads, 48), 7.0, device="cuda", dtype=torch.bfloat16)
    kernels.latent_softmax(scores.cuda(), weights, heads, keys, first_query, first_key, window, scale)
    key_position = first_key + torch.arange(48)
    for r in range(queries * heads):
        p = first_query + r // heads
        seen = (key_position <= p) & (key_position > p - window) & (torch.arange(48) < keys)
        want = torch.softmax((scores[r].double() * scale).masked_fill(~seen, float("-inf")), dim=-1)
        assert torch.allclose(weights[r].cpu().double(), want, atol=4e-3, rtol=1e-2), r
        assert float(weights[r].cpu()[~seen].abs().max()) == 0.0


@pytest.mark.parametrize("heads, dim, rot_dim, vdim, rank, window", [(4, 24, 8, 20, 40, 24), (8, 32, 32, 16, 96, 64), (16, 16, 8, 24, 160, 100), (2, 16, 8, 48, 40, 300)])
def test_long_portions_as_matrix_products(heads, dim, rot_dim, vdim, rank, window):
    """The mixer alone in bfloat16: a step brings the second 150 tokens of a request whose first 150 are cached, a single token
    of another at position 70 and 40 tokens of a third; long portions go through matrix products, the rest through the kernel;
    all against the plain function on the whole sequences, and against the kernel alone."""
    from turboserve_b200.cache.storage import RunCache
    from turboserve_b200.config.model_spec import PartSpec
    from turboserve_b200.parts import latent_attention as module
    from turboserve_b200.parts.base import MIXERS

    g = torch.Generator().manual_seed(rank + window)
    width, page_size, eps = 96, 8, 1e-5
    names = {"q": "q", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "o": "o"}
    rot = C.rot(5000.0, rot_dim, (4.0, 64, 16.0, 2.0))
    sizes = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=rank, scale=0.3, mask={"size": window}, rot=rot)
    spec = PartSpec("latent_attention", dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=rank, scale=0.3, window=window,
                                             eps=eps, rot=rot, names=names))
    part = MIXERS.get("latent_attention")(spec, width, torch.bfloat16, "cuda")
    weights = {p.name: ((1.0 if p.role == "gain" else 0.0) + torch.randn(p.shape, generator=g) * 0.2).bfloat16() for p in part.param_specs()}
    part.bind({p.name: weights[p.name].to("cuda", p.device_dtype(torch.bfloat16)) for p in part.param_specs()})
    lengths = [300, 71, 40]
    inputs = [torch.randn(n, width, generator=g).bfloat16() for n in lengths]
    w64 = {k: v.double() for k, v in weights.items()}
    want = [P.latent_attention(h.double(), w64, sizes, eps, P.latent_cache(h.double(), w64, sizes, eps)) for h in inputs]
    tables, next_page = [], 0
    for n in lengths:
        count = -(-n // page_size)
        tables.append(list(range(next_page, next_page + count)))
        next_page += count
    cache = RunCache("paged", group=0, k_pages=torch.zeros(next_page, page_size, 1, rank + rot_dim, device="cuda", dtype=torch.bfloat16),
                     v_pages=torch.zeros(next_page, page_size, 1, 0, device="cuda", dtype=torch.bfloat16))
    first = part.forward(torch.cat([inputs[0][:150], inputs[1][:70]]).cuda(), _context([150, 70], torch.bfloat16, tables=tables[:2]), cache).cpu()
    step = torch.cat([inputs[0][150:], inputs[1][70:], inputs[2]]).cuda()
    second = part.forward(step, _context([150, 1, 40], torch.bfloat16, starts=[150, 70, 0], tables=tables), cache).cpu()
    old = module.PORTION_MIN
    module.PORTION_MIN = 1 << 30
    try:
        by_kernel = part.forward(step, _context([150, 1, 40], torch.bfloat16, starts=[150, 70, 0], tables=tables), cache).cpu()
    finally:
        module.PORTION_MIN = old
    whole = torch.cat([want[0][150:], want[1][70:], want[2]])
    scale = float(whole.abs().max())
    assert (first.double() - torch.cat([want[0][:150], want[1][:70]])).abs().max() <= 4e-2 * scale
    assert (second.double() - whole).abs().max() <= 4e-2 * scale and (by_kernel.double() - whole).abs().max() <= 4e-2 * scale
    assert (second.double() - by_kernel.double()).abs().max() <= 3e-2 * scale


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_one_latent_row_that_stands_out_at_the_edge_of_the_window_and_far_back(dtype):
    """One row gets a score far above the others and a latent unlike all others. A query sees it exactly while
    it lies within the window: the output is then that latent. Without a window a row 700 positions back is found."""
    from turboserve_b200.ops import kernels

    rank, rot, n, page_size, special = 32, 4, 720, 16, 9
    g = torch.Generator().manual_seed(5)
    rows = torch.randn(n, rank + rot, generator=g) * 0.05
    rows[special] = 0.0
    rows[special, rank + 1] = 40.0   # found through the rotated part
    rows[special, 11] = 25.0
    q_lat = torch.randn(n, 1, rank, generator=g) * 0.05
    q_lat[:, 0, 11] = 0.0
    q_rot = torch.zeros(n, 1, rot)
    q_rot[:, 0, 1] = 1.0
    pages, table = _latent_pages([rows.to(dtype)], page_size, 3)
    for window in (48, None):
        picked = [special, special + 1, special + 46, special + 47, special + 48, special + 49, n - 1]
        out = torch.empty(len(picked), rank, device="cuda", dtype=dtype)
        packed = torch.cat([q_lat[picked, 0], q_rot[picked, 0]], dim=-1).to(dtype)
        kernels.latent_attention(packed.cuda(), out, pages.cuda(), table.cuda(), _i32([0] * len(picked)), _i32(picked), len(picked), 1, rank,
                                 rot, window, 1.0)
        want = _latent_reference(q_lat.to(dtype).double(), q_rot.double(), rows.to(dtype).double(), rank, 1.0, window)[picked, 0]
        assert torch.allclose(out.cpu().double(), want, atol=3e-2, rtol=3e-2)
        peak = out.cpu().float()[:, 11] / out.cpu().float().norm(dim=-1)
        sees = [True, True, True, True, window is None, window is None, window is None]
        for value, inside in zip(peak.tolist(), sees):
            assert (value > 0.99) == inside, (window, peak.tolist())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, dim, vdim, dims, scaling", [(3, 16, 24, 8, None), (2, 40, 10, 20, None), (1, 8, 64, 8, (2.0, 32, 8.0, 1.0)),
                                                             (4, 128, 32, 64, None), (2, 200, 12, 100, None), (5, 6, 9, 2, None), (2, 64, 130, 64, None)])
def test_retention_whole_and_in_portions(dtype, heads, dim, vdim, dims, scaling):
    """Two requests: whole in one step, then again cut into portions of 1 to 40 positions in mixed batches with
    other slots; outputs and final states agree with the plain recurrence."""
    from turboserve_b200.ops import kernels
    from turboserve_b200.parts.rope import scaled_rotary_frequencies

    g = torch.Generator().manual_seed(dim)
    lengths = [90, 33]
    rot = C.rot(700.0, dims, scaling)
    width = 2 * heads * dim + heads * vdim + 3
    rows = [(torch.randn(n, width, generator=g) * 0.7).to(dtype) for n in lengths]
    decay = torch.linspace(0.9, 0.995, heads)
    freq, amplitude = scaled_rotary_frequencies(dims, 700.0, rot.get("scaling"))
    k_first, v_first = heads * dim + 3, 2 * heads * dim + 3   # three unused columns between q and k
    want = []
    for u in rows:
        u, n = u.double(), u.shape[0]
        positions = torch.arange(n)
        q = P.rotate(u[:, :heads * dim].reshape(n, heads, dim), positions, rot)
        k = P.rotate(u[:, k_first:k_first + heads * dim].reshape(n, heads, dim), positions, rot) * dim ** -0.5
        want.append(P.decayed_sums(q, k, u[:, v_first:].reshape(n, heads, vdim), decay.double()).reshape(n, heads * vdim))
    tol = 3e-5 if dtype == torch.float32 else 1e-4  # the inputs are exact in both types; all sums are float32

    def run(portions, slots):
        states = torch.zeros(5, heads, vdim, dim, device="cuda")
        got = [[] for _ in lengths]
        cursors = [0, 0]
        k = 0
        while any(c < n for c, n in zip(cursors, lengths)):
            pieces, positions, starts, live = [], [], [0], []
            for r, n in enumerate(lengths):
                take = min(portions[(k + r) % len(portions)], n - cursors[r])
                if take:
                    pieces.append(rows[r][cursors[r]:cursors[r] + take])
                    positions += list(range(cursors[r], cursors[r] + take))
                    starts.append(starts[-1] + take)
                    live.append((r, take))
            k += 1
            y = torch.zeros(starts[-1], heads * vdim, device="cuda")
            scratch = torch.empty(starts[-1] * kernels.retention_scratch_per_token(heads, dim, vdim), device="cuda")
            seq_of = [index for index, (_, take) in enumerate(live) for _ in range(take)]
            kernels.retention_scan(torch.cat(pieces).cuda(), 0, k_first, v_first, decay.cuda(), freq.cuda(), dims, amplitude, dim ** -0.5,
                                   _i32(positions), _i32(seq_of), _i32(starts), _i32([slots[r] for r, _ in live]), states, y, scratch,
                                   starts[-1], len(live), heads, dim, vdim)
            for index, (r, take) in enumerate(live):
                got[r].append(y[starts[index]:starts[index + 1]].cpu())
                cursors[r] += take
        return [torch.cat(parts).double() for parts in got], states.cpu()

    whole, whole_states = run([1000], [1, 3])
    cut, cut_states = run([1, 40, 2, 7, 1, 13], [4, 0])
    for r in range(2):
        scale = want[r].abs().max()
        assert (whole[r] - want[r]).abs().max() <= tol * scale and (cut[r] - want[r]).abs().max() <= tol * scale
        assert torch.equal(whole[r], cut[r])  # one order of every sum, however the request is cut
    assert torch.equal(whole_states[1], cut_states[4]) and torch.equal(whole_states[3], cut_states[0])
    assert torch.equal(whole_states[0], torch.zeros_like(whole_states[0])) and float(whole_states[1].abs().max()) > 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_unit_heads_times_the_gate(dtype):
    from turboserve_b200.ops import kernels

    g = torch.Generator().manual_seed(4)
    n, heads, vdim = 21, 3, 40
    y = torch.randn(n, heads * vdim, generator=g) * 5.0
    gate = torch.randn(n, heads * vdim + 30, generator=g).to(dtype)
    want = (P.rms_norm(y.double().reshape(n, heads, vdim), None, 1e-5).reshape(n, -1) * P.silu(gate[:, 10:10 + heads * vdim].double()))
    out = torch.empty(n, heads * vdim, device="cuda", dtype=dtype)
    kernels.head_norm_gate(y.cuda(), gate.cuda()[:, 10:10 + heads * vdim], out, n, heads, vdim, 1e-5)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol)


@pytest.mark.parametrize("experts, top, groups", [(8, 2, (4, 2)), (20, 3, (5, 2)), (6, 1, None), (4, 4, (2, 2)), (12, 3, (3, 2)), (9, 3, (3, 1)), (64, 6, (8, 3))])
def test_router_chooses_the_plain_experts(experts, top, groups):
    from turboserve_b200.ops import kernels

    g = torch.Generator().manual_seed(experts)
    n, width = 300, 72
    h = torch.randn(n, width, generator=g).bfloat16()
    router = torch.randn(experts, width, generator=g) * 0.3
    sizes = {"experts": experts, "top": top}
    if groups:
        sizes["groups"] = {"count": groups[0], "keep": groups[1]}
    want_ids, want_weights = P.route(h.double(), router.double(), sizes)
    for dtype in (torch.bfloat16, torch.float32):
        chosen = torch.zeros(n, top, dtype=torch.int32, device="cuda")
        weights = torch.zeros(n, top, device="cuda")
        kernels.moe_route(h.to(dtype).cuda(), router.cuda(), chosen, weights, n, top, *(groups or (1, 1)))
        assert torch.equal(chosen.cpu().long(), want_ids)
        assert torch.allclose(weights.cpu().double(), want_weights, atol=2e-6, rtol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts, top, groups, ff, shared, width", [(8, 2, (4, 2), 48, 32, 96), (6, 1, None, 40, None, 100), (4, 4, (2, 2), 24, None, 64),
                                                                     (12, 3, (3, 2), 24, 64, 128)])
def test_experts_for_single_tokens_and_for_portions(dtype, experts, top, groups, ff, shared, width):
    """The same rows as a step of single tokens (pairs in expert order, an expert streamed once for its tokens), as one portion
    of a prompt (one product per expert), mixed, and as a step of very few single tokens (every pair streams its expert):
    all against the plain mixture."""
    from turboserve_b200.config.model_spec import PartSpec
    from turboserve_b200.parts.base import FEED_FORWARDS

    g = torch.Generator().manual_seed(ff)
    n = 57
    names = {"router": "router", "expert": "e{index}.", "shared": "shared.", "gate": "gate", "up": "up", "down": "down"}
    spec = PartSpec("routed_experts", dict(experts=experts, top=top, groups=groups[0] if groups else 1, keep=groups[1] if groups else 1,
                                           intermediate_size=ff, shared=shared, names=names))
    part = FEED_FORWARDS.get("routed_experts")(spec, width, dtype, "cuda")
    weights = {}
    for p in part.param_specs():
        std = 1.0 if p.name == "router" else 0.15
        weights[p.name] = (torch.randn(p.shape, generator=g) * std).bfloat16()
    part.bind({p.name: weights[p.name].to("cuda", p.device_dtype(dtype)) for p in part.param_specs()})
    x = torch.randn(n, width, generator=g).to(dtype)
    mlp = {"router": {"experts": experts, "top": top}, "shared": {"ff": shared} if shared else None}
    if groups:
        mlp["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    want = P.mixture(x.double(), {k: v.double() for k, v in weights.items()}, mlp)
    tol = 2e-5 if dtype == torch.float32 else 4e-2
    scale = float(want.abs().max())
    for query_lens in ([1] * n, [n], [20, 1, 36]):
        out = part.forward(x.cuda(), _context(query_lens, dtype))
        assert (out.cpu().double() - want).abs().max() <= tol * scale, query_lens
    few = max(1, 4 // top)  # so few single tokens that every pair streams its expert alone
    out = part.forward(x[:few].cuda(), _context([1] * few, dtype))
    assert (out.cpu().double() - want[:few]).abs().max() <= tol * scale


# ---------------------------------------------------------------------------------------------
# whole models through the replay loop
# ---------------------------------------------------------------------------------------------

LENGTHS = {"A": [1, 7, 33, 100, 150], "B": [5, 40, 129, 70], "C": [3, 64, 130, 200], "D": [2, 9, 61, 140]}
MIXED_LENGTHS = [33, 100, 20, 150, 64, 7, 90, 129, 48, 5, 77, 130]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_each_request_alone_and_whole(folders, name, dtype):
    run_and_check(folders[name, False, dtype], dtype, traces.whole, LENGTHS[name])


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_the_stream_after_every_layer(folders, name):
    from turboserve_b200.parts.block import OutputNormBlock
    from turboserve_b200.replay import Replayer

    folder = folders[name, False]
    config, weights = P.read_model_folder(folder)
    tokens = traces.make_requests(config["vocab"], [45], seed=3)["r0"]
    _, want = P.forward(config, weights, tokens)
    replayer = Replayer(folder, "float32", 64)
    got = []
    original = OutputNormBlock.forward

    def recording(self, residual, pending, ctx, cache):
        out = original(self, residual, pending, ctx, cache)
        got.append(residual[:ctx.batch.num_tokens].cpu().double())
        return out

    OutputNormBlock.forward = recording
    try:
        replayer.step([{"id": "a", "tokens": tokens, "want": []}], ["a"])
    finally:
        OutputNormBlock.forward = original
    assert len(got) == len(want) == len(config["layers"])
    for index, (ours, ref) in enumerate(zip(got, want)):
        assert (ours - ref).abs().max() <= 2e-5 * max(1.0, float(ref.abs().max())), index


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_prompt_then_token_by_token(folders, name, dtype):
    """The last tokens one by one: more of them than the longest window, so it passes over decoded tokens."""
    run_and_check(folders[name, False, dtype], dtype, traces.tail_one_by_one, LENGTHS[name], tail=80)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_portions_of_changing_size_down_to_two_tokens(folders, name, dtype):
    run_and_check(folders[name, False, dtype], dtype, traces.changing_portions, LENGTHS[name])
    run_and_check(folders[name, False, dtype], dtype, traces.changing_portions, LENGTHS[name][-2:], sizes=(2, 2, 3, 2, 1, 2), page_size=8)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("page_size", [16, 8])
def test_mixed_batches_with_pages_and_slots_used_again(folders, name, dtype, page_size):
    """Twelve requests, four live at a time, unequal portions beside single tokens: four state slots and
    a pool that holds the live requests only, so every slot and page goes to several requests."""
    replayer, _ = run_and_check(folders[name, False, dtype], dtype, traces.mixed, MIXED_LENGTHS, page_size=page_size, seed=3)
    assert replayer.manager.slots.num_slots == 4
    for pool, group in zip(replayer.manager.pools, replayer.manager.groups):
        assert pool.num_allocations > group.num_pages


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_sharp_scores_and_slow_decay_in_float32(folders, name):
    """Weights under which single keys stand out and the state remembers hundreds of tokens: windows' edges,
    keys far back (the layers without a window see 400 positions) and carried state, in prompts, in portions,
    token by token and in mixed batches."""
    folder = folders[name, True]
    lengths = [400, 170]
    run_and_check(folder, "float32", traces.whole, lengths, slack=2.5)
    run_and_check(folder, "float32", traces.tail_one_by_one, lengths, tail=90, slack=2.5)
    run_and_check(folder, "float32", traces.changing_portions, lengths, page_size=8, slack=2.5)
    run_and_check(folder, "float32", traces.mixed, [170, 60, 200, 33, 90, 120], seed=8, slack=2.5)


@pytest.mark.parametrize("name", ["A", "C"])
def test_sharp_scores_in_bfloat16_token_by_token(folders, name):
    run_and_check(folders[name, True, "bfloat16"], "bfloat16", traces.tail_one_by_one, [300], tail=100, slack=3.0)
    run_and_check(folders[name, True, "bfloat16"], "bfloat16", traces.mixed, [170, 60, 200, 33, 90], seed=8, slack=3.0)


def test_the_sharp_weights_do_make_single_rows_and_old_state_count(folders):
    """Under the sharpened weights the logits of a late position change by far more than the tolerance when a row
    just inside the window, or the first token of all (which only the carried state remembers), is another token."""
    folder = folders["A", True]
    config, weights = P.read_model_folder(folder)
    tokens = traces.make_requests(config["vocab"], [300], seed=2)["r0"]
    base = P.logits_of(config, weights, tokens)[-1:]
    for place in (0, 299 - 39):
        changed = list(tokens)
        changed[place] = (changed[place] + 1) % config["vocab"]
        other = P.logits_of(config, weights, changed)[-1:]
        assert float(C.relative_error(other, base).max()) > 20 * C.FP32_REL, place


@pytest.mark.parametrize("name", ["A", "B"])
def test_float32_single_tokens_do_not_depend_on_the_batch_at_all(folders, name):
    """Decoded alone or beside other requests' portions, through other pages and slots: a single token's float32
    logits are the same bits (every sum of such a step has one order)."""
    folder = folders[name, False]
    _, a = run_and_check(folder, "float32", traces.tail_one_by_one, [90, 60, 41], tail=30)
    _, b = run_and_check(folder, "float32", traces.tail_one_by_one, [90, 60, 41], tail=30, page_size=8)
    for rid in a:
        assert torch.equal(a[rid][-29:], b[rid][-29:]), rid


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(folders, dtype):
    """Positions 0, 1, 2 one by one and two at once: windows that reach before the start, an empty state."""
    from turboserve_b200.replay import Replayer

    for name in C.CASES:
        folder = folders[name, False, dtype]
        config, weights = P.read_model_folder(folder)
        tokens = [5, 9, 2]
        ref = P.logits_of(config, weights, tokens)
        replayer = Replayer(folder, dtype, 64)
        rows = [replayer.step([{"id": "x", "tokens": [t], "want": [0]}], []) for t in tokens]
        C.check(torch.cat(rows), ref, dtype, f"{name} first tokens")
        replayer.step([], ["x"])
        both = replayer.step([{"id": "y", "tokens": tokens[:2], "want": [0, 1]}], ["y"])
        C.check(both, ref[:2], dtype, f"{name} first two tokens")


def test_a_slot_that_is_used_again_starts_empty(folders):
    """A request that follows another in the same state slot gets what it gets alone (float32, same bits)."""
    from turboserve_b200.replay import Replayer

    folder = folders["A", True]
    config = C.read_config(folder)
    requests = traces.make_requests(config["vocab"], [70, 40], seed=9)
    replayer = Replayer(folder, "float32", 128, state_slots=1)
    first = replayer.step([{"id": "a", "tokens": requests["r0"], "want": [69]}], ["a"])
    second = replayer.step([{"id": "b", "tokens": requests["r1"], "want": list(range(40))}], ["b"])
    alone = Replayer(folder, "float32", 128, state_slots=1).step([{"id": "b", "tokens": requests["r1"], "want": list(range(40))}], ["b"])
    assert first is not None and torch.equal(second, alone)


def test_long_decoding(folders):
    """600 tokens one by one after a short prompt: the windows pass over decoded tokens many times, pages behind
    them are given back, the state is carried 600 steps."""
    replayer, _ = run_and_check(folders["A", True], "float32", traces.tail_one_by_one, [620], tail=600, slack=2.5, page_size=8)
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
    logits = P.logits_of(config, weights, prompt + generated)
    spread = float((logits - logits.mean(-1, keepdim=True)).pow(2).mean().sqrt())
    slack = (C.FP32_REL if dtype == "float32" else C.BF16_REL) * spread * 4
    for i, token in enumerate(generated):
        row = logits[len(prompt) + i - 1]
        best = int(row.argmax())
        assert token == best or row[best] - row[token] <= slack, (i, token, best, float(row[best] - row[token]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name, lengths, new", [("A", [1, 7, 33, 100, 60, 12], 40), ("B", [5, 40, 129], 30), ("C", [3, 70], 24)])
def test_greedy_generation_through_the_engine(folders, name, lengths, new, dtype):
    from turboserve_b200 import SamplingParams

    folder = folders[name, False, dtype]
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
    """Prompts cut by a token budget of 16, and a pool too small for everyone (requests are preempted, their
    slots zeroed and their prompts computed again): every token still follows the plain logits in float32."""
    from turboserve_b200 import SamplingParams

    folder = folders["B", False]  # its layers without a window keep every page: the pool runs out
    config, weights = P.read_model_folder(folder)
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, config["vocab"], (n,), generator=g).tolist() for n in [5, 40, 129, 33, 64, 18]]
    sampling = SamplingParams(max_tokens=24, temperature=0.0, ignore_eos=True)
    with engine_for(folder, "float32", max_num_batched_tokens=16) as engine:
        chunked = engine.generate(prompts, sampling)
    with engine_for(folder, "float32", max_num_batched_tokens=64, num_blocks=14) as engine:
        tight = engine.generate(prompts, sampling)
        stats = engine.stats()
        engine.scheduler.check_invariants()
    assert stats["num_preemptions"] > 0
    for prompt, a, b in zip(prompts, chunked, tight):
        check_greedy_path(config, weights, prompt, a.token_ids, "float32")
        check_greedy_path(config, weights, prompt, b.token_ids, "float32")


def test_bfloat16_with_graphs_steps_launched_ahead_and_preemption_together(folders):
    from turboserve_b200 import SamplingParams

    folder = folders["B", False, "bfloat16"]
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
