"""The Tupidra decoder in the engine against the plain implementation (``plain_tupidra.py``, float64): each mechanism
alone, whole prompts, token-by-token decoding, portions down to two tokens, unequal batches, pages and slots used again,
keys far away, at page borders and just inside and outside the window and the kept first tokens (in prompts and
decoded), a sink, state carried over hundreds of tokens, long decoding, several shapes, and greedy generation through
the entry point."""

import itertools
import math

import pytest
import torch

import helpers as H
import plain_tupidra as plain
import tupidra_cases as T

pytestmark = pytest.mark.gpu
DTYPES = [pytest.param(torch.float32, id="f32"), pytest.param(torch.bfloat16, id="bf16")]
DEV = "cuda"


def case(tmp_path, name, seed, sharp=None, slow=False):
    cfg = T.CONFIGS[name] if sharp is None else T.sharpen(T.CONFIGS[name], sharp)
    W = T.weights_for(cfg, seed, slow=slow)
    return cfg, W, T.write_model(str(tmp_path), cfg, W)


def requests_for(cfg, lengths, seed):
    return {f"r{i}": H.random_tokens(cfg["vocab"], n, seed + i) for i, n in enumerate(lengths)}


def _i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


def _rel(got, want):
    return float((got.double().cpu() - want).abs().max() / want.abs().max())


# ---- kernels alone ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [54, 256, 5000])
def test_norm_with_several_weights_adds_what_is_pending(dtype, width):
    from llm_pipeline_b200.ops import kernels
    gen = torch.Generator().manual_seed(width)
    n, eps = 7, 1e-5
    res, a, b = (torch.randn(n, width, generator=gen) * s for s in (3.0, 1.0, 0.5))
    bias, w = torch.randn(width, generator=gen), torch.randn(3, width, generator=gen)
    x = res.double() + ((a.double() + bias.double()) + b.double())
    want = torch.cat([plain.rms(x, eps, w[j].double()) for j in range(3)], dim=1)
    residual = res.to(DEV)
    out = torch.empty(n, 3 * width, device=DEV)
    kernels.add_rmsnorm_multi(residual, a.to(DEV), b.to(DEV), bias.to(DEV), w.to(DEV), eps, out)
    assert _rel(out, want) < 1e-5 and _rel(residual, x) < 1e-6
    # chosen rows, one weight, the compute type, and a residual that stays as it is
    residual = res.to(DEV)
    rows = _i32([5, 0, 3])
    typed = torch.empty(3, width, device=DEV, dtype=dtype)
    kernels.add_rmsnorm_multi(residual, a.to(DEV), None, None, w[:1].to(DEV), eps, typed, rows=rows)
    want_rows = plain.rms(res.double() + a.double(), eps, w[0].double())[[5, 0, 3]]
    assert _rel(typed, want_rows) < (1e-5 if dtype == torch.float32 else 1e-2) and torch.equal(residual.cpu(), res)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps", [1, 2, 5])
def test_input_filters_carry_their_last_inputs_from_step_to_step(dtype, taps):
    """Two sublayers' inputs side by side through one convolution beside the identity; two requests in slots that are not
    theirs by number, fed in portions of 1, 2, 3 and more tokens, together and in turns."""
    from llm_pipeline_b200.ops import kernels
    gen = torch.Generator().manual_seed(taps)
    C = 37
    w = torch.randn(2 * C, taps, generator=gen) * 0.5
    xs = {3: torch.randn(23, 2 * C, generator=gen), 1: torch.randn(16, 2 * C, generator=gen)}
    want = {s: plain.input_conv(x.double(), w.double()) for s, x in xs.items()}
    state = torch.full((5, 2 * (taps - 1) * 2 * C + 11), 9.0, device=DEV)      # other requests' slots, which nothing may touch
    state[[3, 1]] = 0.0                                                         # a slot is zeroed when it is handed out
    done, got = {3: 0, 1: 0}, {3: [], 1: []}
    for sizes in [{3: 1}, {3: 2, 1: 5}, {1: 1}, {3: 3, 1: 1}, {3: 1, 1: 2}, {3: 16, 1: 7}]:
        rows = torch.cat([xs[s][done[s]:done[s] + n] for s, n in sizes.items()])
        q_start = _i32([0] + list(itertools.accumulate(sizes.values())))
        positions = _i32([p for s, n in sizes.items() for p in range(done[s], done[s] + n)])
        request = _i32([i for i, n in enumerate(sizes.values()) for _ in range(n)])
        out = torch.empty(2, rows.shape[0], C, device=DEV, dtype=dtype)
        kernels.short_conv(rows.to(DEV), w.to(DEV), None, state, 4, q_start, _i32(list(sizes)), positions, request, None,
                           max(sizes.values()), silu=False, add_input=True, out_typed=out)
        both = torch.cat([out[0], out[1]], dim=1).float().cpu()
        at = 0
        for s, n in sizes.items():
            got[s].append(both[at:at + n])
            at, done[s] = at + n, done[s] + n
    for s in xs:
        assert _rel(torch.cat(got[s]), want[s]) < (1e-5 if dtype == torch.float32 else 1e-2), s
    assert (state[[0, 2, 4]] == 9.0).all() and (state[:, :4] == torch.tensor([9.0, 0.0, 9.0, 0.0, 9.0], device=DEV)[:, None]).all()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [(96, 12), (30, 7), (64, 16), (22, 5), (40, 200), (130, 32), (17, 1), (10, 129)], ids=str)
def test_selective_scan_alone(dtype, sizes):
    """The recurrence on given rows, whole and cut into portions down to one token, in a slot that is not the first; the
    state of other slots and the entries around the piece stay as they are."""
    from llm_pipeline_b200.ops import kernels
    inner, states = sizes
    gen = torch.Generator().manual_seed(inner + states)
    n = 70
    x, raw, z = (torch.randn(n, inner, generator=gen) for _ in range(3))
    bc = torch.randn(n, 3 + 2 * states, generator=gen)
    dt_bias, skip = torch.randn(inner, generator=gen) * 0.5 - 1.0, torch.randn(inner, generator=gen)
    A = -torch.exp(torch.rand(inner, states, generator=gen) * 5.0 - 4.5)
    dt = torch.nn.functional.softplus(raw.double() + dt_bias.double())
    y, last = plain.scan(x.double(), dt, A.double(), bc[:, 3:3 + states].double(), bc[:, 3 + states:].double(), skip.double())
    want = y * plain.silu(z.double())
    xd, rd, zd, bd = x.to(DEV), raw.to(DEV), z.to(DEV), bc.to(DEV)
    for cuts in ((), (1,), (1, 2, 4, 9, 10, 41), tuple(range(1, n))):
        out = torch.empty(n, inner, device=DEV, dtype=dtype)
        offset, entries = 6, 2 * inner * states
        state = torch.full((4, offset + entries + 3), 5.0, device=DEV)
        state[2] = 0.0
        edges = [0] + list(cuts) + [n]
        for lo, hi in zip(edges[:-1], edges[1:]):
            kernels.selective_scan(xd[lo:hi], rd[lo:hi], dt_bias.to(DEV), bd[lo:hi, 3:3 + states], bd[lo:hi, 3 + states:], A.to(DEV),
                                   skip.to(DEV), zd[lo:hi], state, offset, _i32([0, hi - lo]), _i32([2]), _i32(list(range(lo, hi))), out[lo:hi])
        assert _rel(out, want) < (2e-5 if dtype == torch.float32 else 1e-2), cuts
        assert (state[[0, 1, 3]] == 5.0).all() and (state[2, :offset] == 0.0).all() and (state[2, offset + entries:] == 0.0).all()
        kept = state[2, offset:offset + entries].view(2, inner, states)[(n - 1) & 1].cpu()
        assert _rel(kept, last) < 2e-5, cuts


def _window_case(dtype, heads, kv_heads, dim, vdim, n, page, seed, cap, size, keep, plant=None, rows=None, gate=True):
    """Queries, keys and values as they enter the scores, written into shuffled pages; (engine output, plain output) for
    the token rows ``rows`` (all by default), each launched as the portion it is."""
    from llm_pipeline_b200.ops import kernels
    gen = torch.Generator().manual_seed(seed)
    q, k = torch.randn(n, heads, dim, generator=gen), torch.randn(n, kv_heads, dim, generator=gen)
    v, g = torch.randn(n, kv_heads, vdim, generator=gen), torch.randn(n, heads * vdim, generator=gen)
    if plant is not None:
        plant(q, k, v)
    q, k, v = (t.to(torch.bfloat16).float() for t in (q, k, v))
    scale = 1.0 / math.sqrt(dim)
    want = plain.attend_window(q.double(), k.double(), v.double(), scale, cap, size, keep).reshape(n, -1)
    if gate:
        want = want * torch.sigmoid(g.double())
    pages_n = -(-n // page)
    order = torch.randperm(pages_n + 3, generator=gen)[:pages_n]              # the request's pages lie anywhere in the pool
    pages = torch.full((pages_n + 3, kv_heads, page, dim + vdim), float("nan"))  # other pages hold what must never be read
    for t in range(n):
        pages[order[t // page], :, t % page] = torch.cat([k[t], v[t]], dim=-1)
    table = order.to(torch.int32).view(1, -1).clone()
    rows = list(range(n)) if rows is None else rows
    if size is not None:
        # pages that every asked row's window has passed and that hold no kept token are gone, as in the engine
        for p in range(pages_n):
            if p * page >= keep and (p + 1) * page <= min(rows) - size + 1:
                pages[order[p]] = float("nan")
                table[0, p] = -1
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=torch.float32, device=DEV)
    sink = torch.zeros(heads, device=DEV)
    qd, pd = q.reshape(n, -1).to(DEV).to(dtype)[rows].contiguous(), pages.to(DEV).to(dtype)
    gd = g.to(DEV)[rows].contiguous() if gate else None
    out = torch.empty(len(rows), heads * vdim, device=DEV, dtype=dtype)
    kernels.capped_attention(qd, pd, table.to(DEV), torch.zeros(len(rows), dtype=torch.int32, device=DEV), _i32(rows), out, heads, kv_heads,
                             dim, vdim, size or 0, keep, scale, cap or 0.0, slopes=slopes, sink=sink, gate=gd)
    got = out.float().cpu()
    if kernels.capped_mma_supports(dtype, dim, vdim) and rows == list(range(rows[0], rows[0] + len(rows))):
        # the tensor-core kernel on the same portion (tiles of its own size, the last one short); a single row also with the
        # four warps of a block sharing its keys; both must agree with the general kernel's answer
        per = kernels.capped_mma_tokens_per_tile(heads, kv_heads)
        tok0 = torch.arange(0, len(rows), per, dtype=torch.int32, device=DEV)
        for split in ([False, True] if len(rows) == 1 else [False]):
            tensor = torch.empty_like(out)
            kernels.capped_attention_mma(qd, pd, table.to(DEV), _i32([0, len(rows)]), _i32([rows[-1] + 1]), torch.zeros_like(tok0), tok0, tensor,
                                         heads, kv_heads, dim, vdim, size or 0, keep, scale, cap or 0.0, slopes=slopes, sink=sink, gate=gd,
                                         split=split)
            assert not torch.isnan(tensor).any(), "the tensor-core kernel read a row of a page that is gone"
            assert _rel(tensor, want[rows]) < 3e-2, ("tensor cores", split)
    return got, want[rows]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [(4, 2, 16, 24, 12.0, 40, 3), (3, 3, 12, 20, None, None, 0), (6, 1, 48, 48, 8.0, 9, 20), (2, 2, 128, 64, 30.0, 33, 5),
                                   (32, 2, 16, 16, 30.0, 1, 0), (16, 2, 64, 128, 15.0, 50, 2), (3, 1, 10, 14, 25.0, 7, 1), (5, 5, 10, 200, None, 64, 64),
                                   (1, 1, 64, 128, 1.0, 130, 17), (12, 3, 32, 32, 20.0, 70, 6), (40, 2, 16, 64, 10.0, 24, 40)], ids=str)
def test_capped_window_attention_alone(dtype, sizes):
    """Grouped heads, values of another width than keys, capped scores, the distance bias, windows shorter and longer than
    a page, kept first tokens fewer and more than the window, the fixed sink and the gate, over shuffled pages."""
    heads, kv_heads, dim, vdim, cap, size, keep = sizes
    for rows in (None, list(range(150, 200)), [150, 151, 199], [199]):    # a whole prompt; portions and a single row whose old pages are gone
        got, want = _window_case(dtype, heads, kv_heads, dim, vdim, 200, 16, 3, cap, size, keep, rows=rows)
        assert not torch.isnan(got).any(), "a row of a page that is gone, or of another request, was read"
        assert _rel(got, want) < (1e-5 if dtype == torch.float32 else 2e-2), rows


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("size, keep, page", [(40, 3, 16), (16, 16, 16), (33, 0, 8), (5, 9, 16)])
def test_a_key_just_inside_and_just_outside_the_window_and_the_kept_tokens(dtype, size, keep, page):
    """One key holds nearly all of a query's weight (its score stands out by the cap); where it lies just inside the window,
    just outside, among the kept first tokens or right behind them decides the output. In a prompt and for single rows."""
    heads, kv_heads, dim, vdim, n, cap = 2, 1, 32, 16, 120, 60.0
    asked = {100: 100 - size + 1, 101: 101 - size, 102: max(keep - 1, 0), 103: keep, 104: 104, 119: 119 - size + 1}

    def plant(q, k, v):
        for i, j in asked.items():
            q[i] = k[j, 0] * 40.0 / k[j, 0].norm()
            k[j] = k[j] * 4.0 / k[j].norm() * math.sqrt(dim)

    rows = sorted(asked)
    whole, want = _window_case(dtype, heads, kv_heads, dim, vdim, n, page, 7, cap, size, keep, plant=plant, gate=False)
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    assert _rel(whole[rows], want[rows]) < tol
    # the premise, on the plain implementation: with the window one wider or the kept tokens one more, the asked rows differ much
    _, wider = _window_case(dtype, heads, kv_heads, dim, vdim, n, page, 7, cap, size + 1, keep, plant=plant, gate=False, rows=[101])
    assert (wider[0] - want[101]).abs().max() > 0.1
    if 103 - keep >= size:                                  # the first token that is not kept lies outside row 103's window
        _, more = _window_case(dtype, heads, kv_heads, dim, vdim, n, page, 7, cap, size, keep + 1, plant=plant, gate=False, rows=[103])
        assert (more[0] - want[103]).abs().max() > 0.1
    for i in rows:                                          # decoded alone: one row, old pages gone
        got, ref = _window_case(dtype, heads, kv_heads, dim, vdim, n, page, 7, cap, size, keep, plant=plant, rows=[i], gate=False)
        assert _rel(got, ref) < tol, i


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [(3, 16, 8, 32, 8), (4, 16, 16, 48, 16), (3, 10, 6, 20, 6), (20, 16, 32, 128, 32), (2, 24, 8, 32, 4)], ids=str)
def test_latent_rows_rotation_and_attention_with_a_sink_alone(dtype, sizes):
    """The step after the products (norm of the latent, the interleaved rotation with ramped frequencies and scaled cos and
    sin, the row's write) and the attention over the cached rows with a sink in the denominator, whole and in key
    segments, over shuffled pages; then a layer without rows of its own (queries only)."""
    from llm_pipeline_b200.ops import kernels
    from llm_pipeline_b200.parts.position import RotaryPositions
    heads, dim, rot, rank, rot_dims = sizes
    n, page, eps, base = 300, 16, 1e-5, 100.0
    rule = {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}
    gen = torch.Generator().manual_seed(rank)
    q32, dkv = torch.randn(n, heads * (dim + rot), generator=gen), torch.randn(n, rank + rot, generator=gen)
    nw, sink = torch.randn(rank, generator=gen) * 0.3 + 1.0, torch.randn(heads, generator=gen) + 1.0
    pos = torch.arange(n)
    c = plain.rms(dkv[:, :rank].double(), eps, nw.double())
    k_rot = plain.rotate_interleaved(dkv[:, rank:].double(), pos, rot_dims, base, rule)
    q = q32.double().view(n, heads, dim + rot)
    q_rot = plain.rotate_interleaved(q[..., dim:], pos, rot_dims, base, rule)
    inv = torch.tensor(RotaryPositions.ramp_frequencies(rot_dims, base, dict(rule, kind="ramp")), dtype=torch.float64).float().to(DEV)
    cos, sin = torch.empty(n, rot_dims // 2, device=DEV), torch.empty(n, rot_dims // 2, device=DEV)
    kernels.rope_tables(pos.to(torch.int32).to(DEV), inv, 0.1 * math.log(rule["factor"]) + 1.0, cos, sin)
    pages_n = -(-n // page)
    order = torch.randperm(pages_n + 2, generator=gen)[:pages_n]
    pages = torch.full((pages_n + 2, page, rank + rot), float("nan"), device=DEV, dtype=dtype)
    slots = torch.tensor([int(order[t // page]) * page + t % page for t in range(n)], dtype=torch.int32, device=DEV)
    q_out = torch.empty(n, heads * (dim + rot), device=DEV, dtype=dtype)
    kernels.latent_rows_post(q32.to(DEV), dkv.to(DEV), heads, dim, rot, rank, nw.to(DEV), eps, cos, sin, rot_dims, True, q_out, slots, pages)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    written = pages.view(-1, rank + rot)[slots.long()].float().cpu()
    assert _rel(written, torch.cat([c, k_rot], dim=1)) < tol
    got_q = q_out.float().cpu().view(n, heads, dim + rot)
    assert _rel(got_q[..., dim:], q_rot) < tol and _rel(got_q[..., :dim], q[..., :dim]) < tol
    alone = torch.empty_like(q_out)                      # a layer that reads another's rows rotates its queries and writes nothing
    kernels.latent_rows_post(q32.to(DEV), None, heads, dim, rot, rank, None, eps, cos, sin, rot_dims, True, alone, None, None)
    assert torch.equal(alone, q_out)
    # attention over the rows as the cache holds them: every head reads [latent | key part] as keys and the latent as values
    rows = written.double()
    q_lat = torch.randn(n, heads, rank, generator=gen).to(torch.bfloat16)
    q_r = q_out.float().cpu().view(n, heads, dim + rot)[..., dim:].to(torch.bfloat16)
    scale = 3.0 / math.sqrt(rank + rot)
    want = plain.attend_latent(q_lat.double(), q_r.double(), rows[:, None, :rank].expand(n, heads, rank), rows[:, rank:],
                               rows[:, None, :rank].expand(n, heads, rank), scale, sink.double())
    no_sink = plain.attend_latent(q_lat.double(), q_r.double(), rows[:, None, :rank].expand(n, heads, rank), rows[:, rank:],
                                  rows[:, None, :rank].expand(n, heads, rank), scale, torch.full((heads,), -1e9, dtype=torch.float64))
    assert (want - no_sink).abs().max() > 0.05 * want.abs().max()               # the premise: the sink weighs
    table = order.to(torch.int32).view(1, -1).to(DEV)
    ql, qr = q_lat.to(DEV).to(dtype), q_r.to(DEV).to(dtype).contiguous()
    out = torch.empty(n, heads, rank, device=DEV, dtype=dtype)
    positions = pos.to(torch.int32).to(DEV)
    kernels.latent_attention(ql, qr, pages, table, torch.zeros(n, dtype=torch.int32, device=DEV), positions, out, scale, sink=sink.to(DEV))
    assert _rel(out, want) < (2e-5 if dtype == torch.float32 else 2e-2)
    if kernels.latent_mma_supports(dtype, rank, rot, page):
        per = kernels.latent_mma_tokens_per_tile(heads)
        for tail, segments in ((n, 0), (n, -(-n // kernels.LATENT_SEGMENT_KEYS)), (21, 0), (21, -(-n // kernels.LATENT_SEGMENT_KEYS))):
            tok0 = torch.arange(0, tail, per, dtype=torch.int32, device=DEV)
            part = torch.empty(tail, heads, rank, device=DEV, dtype=dtype)
            kernels.latent_attention_mma(ql[n - tail:], qr[n - tail:], pages, table, _i32([0, tail]), _i32([n]), positions[n - tail:].contiguous(),
                                         torch.zeros_like(tok0), tok0, part, scale, segments, sink=sink.to(DEV))
            assert _rel(part, want[n - tail:]) < 2e-2, (tail, segments)


@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_activation_gate_and_row_conversion_alone(dtype):
    from llm_pipeline_b200.ops import kernels
    gen = torch.Generator().manual_seed(5)
    gu = torch.randn(9, 2 * 70, generator=gen) * 3.0
    want = plain.gelu_tanh(gu[:, :70].double()) * gu[:, 70:].double()
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    out = torch.empty(9, 70, device=DEV, dtype=dtype)
    assert _rel(kernels.gated_act(gu.to(DEV), out, "gelu_tanh"), want) < tol
    assert _rel(kernels.gated_act(gu.to(DEV), out, "silu"), plain.silu(gu[:, :70].double()) * gu[:, 70:].double()) < tol
    wide = torch.randn(9, 200, generator=gen)
    x = torch.randn(9, 70, generator=gen).to(dtype)
    assert _rel(kernels.sigmoid_gate(x.to(DEV).clone(), wide.to(DEV)[:, 30:100]), x.double() * torch.sigmoid(wide[:, 30:100].double())) < tol
    assert _rel(kernels.convert_rows(wide.to(DEV)[:, 30:100], torch.empty(9, 70, device=DEV, dtype=dtype)), wide[:, 30:100].double()) < tol


# ---- one layer of each kind ------------------------------------------------------------------------------------------
ONE_LAYER = {
    "scan": T.config([T.mamba(48, 10, 3, conv=3, mlp=T.dense(40))], width=40, vocab=50, taps=3),
    "scan, bare": T.config([T.mamba(33, 9, 2, conv=4)], width=24, vocab=50, taps=2),
    "window": T.config([T.attention(4, 2, 16, 24, size=12, keep=2, mlp=T.dense(40))], width=40, vocab=50, taps=3),
    "window, no filter": T.config([T.attention(2, 1, 24, 16, size=5, keep=7)], width=40, vocab=50, taps=0),
    "latent": T.config([T.latent(3, 16, 8, 24, 32, 20, scaling=T.RAMP, mlp=T.dense(40))], width=40, vocab=50, taps=3),
    "latent twice": T.config([T.latent(2, 8, 4, 8, 12, 6), T.latent(3, 8, 4, 12, 12, 10, kv_from=0, mlp=T.dense(16))], width=32, vocab=50, taps=2),
}


@pytest.mark.parametrize("name", sorted(ONE_LAYER))
def test_one_layer_alone(tmp_path, name):
    cfg = ONE_LAYER[name]
    W = T.weights_for(cfg, 11)
    folder = T.write_model(str(tmp_path), cfg, W)
    requests = requests_for(cfg, [1, 2, 33, 70], 50)
    want = T.oracle(cfg, W, requests)
    runner = H.make_runner(folder, torch.float32, page_size=8, num_pages=24, max_request_tokens=96, max_requests=2)
    T.assert_matches(H.replay(runner, H.cut_whole(requests)), want, torch.float32, f"{name}, whole")
    T.assert_matches(H.replay(runner, H.cut_portions(requests, (2, 5, 1, 16))), want, torch.float32, f"{name}, portions")


# ---- whole models ----------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(T.CONFIGS))
def test_prefill_decoding_portions_and_batches(tmp_path, name, dtype):
    cfg, W, folder = case(tmp_path, name, 3)
    requests = requests_for(cfg, [1, 2, 3, 19, 64, 65, 150], 100)
    want = T.oracle(cfg, W, requests)
    page = 8
    share = 1.0 if dtype == torch.float32 else 0.99     # bfloat16: one position in a hundred may round further
    runner = H.make_runner(folder, dtype, page_size=page, num_pages=2 * (-(-150 // page)) + 6, max_request_tokens=160, max_requests=4)
    T.assert_matches(H.replay(runner, H.cut_whole(requests)), want, dtype, f"{name}: whole prompts", share)
    T.assert_matches(H.replay(runner, H.cut_tail_one_by_one(requests, tail=40)), want, dtype, f"{name}: last tokens one by one", share)
    T.assert_matches(H.replay(runner, H.cut_portions(requests, (1,))), want, dtype, f"{name}: token by token", share)
    T.assert_matches(H.replay(runner, H.cut_portions(requests, (2, 7, 3, 64, 2, 33))), want, dtype, f"{name}: portions", share)
    # unequal requests side by side, four live at most, so the slots and pages of finished ones go to later ones
    got = H.replay(runner, H.cut_mixed(requests, (2, 5, 16, 3, 31), max_live=4, decode_tail=9))
    T.assert_matches(got, want, dtype, f"{name}: mixed batches", share)
    assert runner.cache.num_live == 0                                   # seven requests went through four slots
    assert runner.cache.pages_reused > 0 or all(layer["type"] == "mamba1" for layer in cfg["layers"])


def test_the_same_logits_alone_and_in_a_batch(tmp_path):
    """float32: a request's logits beside others, or cut into portions, are those it has alone, to rounding of sums."""
    cfg, W, folder = case(tmp_path, "mixed", 4)
    requests = requests_for(cfg, [5, 40, 77, 130], 200)
    runner = H.make_runner(folder, torch.float32, page_size=16, num_pages=24, max_request_tokens=144, max_requests=4)
    alone = H.replay(runner, H.cut_whole(requests))
    mixed = H.replay(runner, H.cut_mixed(requests, (3, 2, 17), max_live=4, decode_tail=5))
    for rid in requests:
        assert (alone[rid] - mixed[rid]).abs().max() < 2e-4 * alone[rid].abs().max(), rid


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "attention_first", "wide_heads"])
def test_far_keys_page_borders_window_edges_and_first_tokens_under_a_sharp_softmax(tmp_path, name, dtype):
    """Scores of a wide spread: a query's weight sits on one or two keys, often hundreds of tokens back (latent attention,
    the unwindowed layers) or at a window's far edge or among the kept first tokens, so a key that is lost, off by one or
    read from another request's page changes the logits by its whole value. Prompts as long as many pages, positions
    around every page border, decoded alone and in portions while the windows pass over decoded tokens and pages go back."""
    cfg, W, folder = case(tmp_path, name, 5, sharp=5.0)
    page = 16
    requests = requests_for(cfg, [4 * page, 4 * page + 1, 330, 17], 300)
    want = T.oracle(cfg, W, requests)
    # the premise: in the plain implementation itself the far keys matter (without the first 3 pages the late logits differ much)
    late = plain.forward(cfg, {k: v.double() for k, v in W.items()}, requests["r2"][3 * page:]).float()
    assert T.row_errors(late[-40:], want["r2"][-40:]).median() > 0.03
    runner = H.make_runner(folder, dtype, page_size=page, num_pages=2 * 21 + 4, max_request_tokens=336, max_requests=4)
    share = 1.0 if dtype == torch.float32 else 0.97
    T.assert_matches(H.replay(runner, H.cut_whole(requests)), want, dtype, "sharp: whole", share)
    T.assert_matches(H.replay(runner, H.cut_tail_one_by_one(requests, tail=3 * page + 2)), want, dtype, "sharp: decoding across borders", share)
    T.assert_matches(H.replay(runner, H.cut_portions(requests, (page - 1, 2, page + 1, 2 * page, 3))), want, dtype, "sharp: portions", share)
    T.assert_matches(H.replay(runner, H.cut_mixed(requests, (page, 2, page + 1), max_live=3, decode_tail=page + 3)), want, dtype, "sharp: mixed", share)


def test_a_window_that_passes_gives_its_pages_back_but_for_the_kept_tokens(tmp_path):
    """While a request decodes, the pages its window has passed return to the pool and go to the next request; the page of
    the kept first tokens stays; the logits stay those of the plain implementation."""
    from llm_pipeline_b200.engine import StepEntry
    cfg = T.config([T.attention(4, 2, 16, 24, size=20, keep=3, mlp=T.dense(40)), T.attention(2, 2, 16, 8, size=20, keep=3)], width=40, vocab=50, taps=2)
    cfg = T.sharpen(cfg, 4.0)
    W = T.weights_for(cfg, 21)
    folder = T.write_model(str(tmp_path), cfg, W)
    requests = requests_for(cfg, [150, 90], 70)
    want = T.oracle(cfg, W, requests)
    page = 8
    runner = H.make_runner(folder, torch.float32, page_size=page, num_pages=12, max_request_tokens=160, max_requests=2)   # 12 pages: 96 tokens
    got = {rid: [] for rid in requests}
    for rid, toks in requests.items():
        out = runner.step([StepEntry(rid, toks[:30], list(range(30)))])
        got[rid].append(out.float().cpu())
    for t in range(30, 150):
        live = [rid for rid, toks in requests.items() if t < len(toks)]
        out = runner.step([StepEntry(rid, [requests[rid][t]], [0]) for rid in live])
        for k, rid in enumerate(live):
            got[rid].append(out[k:k + 1].float().cpu())
        if t == 89:
            table = list(runner.cache.block_table("r1", 0))
            assert table[0] >= 0 and all(p < 0 for p in table[1:(90 - 20) // page]) and all(p >= 0 for p in table[(90 - 20) // page + 1:])
            runner.release("r1")
        runner.cache.check()
    assert runner.cache.pages_reused > 0
    T.assert_matches({rid: torch.cat(rows) for rid, rows in got.items()}, want, torch.float32, "windows over decoded tokens")


def test_scan_states_carry_what_was_written_hundreds_of_tokens_back(tmp_path):
    """Decays close to one: what the first tokens wrote into the states still weighs in the logits 300 tokens later, so a
    state that is lost, zeroed at a cut or taken from another slot shows. Checked whole, in portions and in mixed batches."""
    cfg = T.CONFIGS["scan_only"]
    W = T.weights_for(cfg, 12, slow=True)
    folder = T.write_model(str(tmp_path), cfg, W)
    requests = requests_for(cfg, [320, 301, 47], 900)
    want = T.oracle(cfg, W, requests)
    other = list(requests["r0"])
    other[:8] = H.random_tokens(cfg["vocab"], 8, 77)                    # the premise: the first tokens still matter at the end
    changed = plain.forward(cfg, {k: v.double() for k, v in W.items()}, other).float()
    assert T.row_errors(changed[-20:], want["r0"][-20:]).median() > 0.02
    runner = H.make_runner(folder, torch.float32, page_size=16, num_pages=50, max_request_tokens=336, max_requests=3)
    T.assert_matches(H.replay(runner, H.cut_whole(requests)), want, torch.float32, "long memory: whole")
    T.assert_matches(H.replay(runner, H.cut_portions(requests, (2, 63, 1, 130, 5))), want, torch.float32, "long memory: portions")
    T.assert_matches(H.replay(runner, H.cut_mixed(requests, (40, 2, 9), max_live=2, decode_tail=20)), want, torch.float32, "long memory: mixed")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_through_replayed_graphs(tmp_path, dtype):
    """Two requests decode side by side for 220 steps over many pages, the states and the filters' inputs taking turns
    between their two copies, the windows passing: from the third step on a captured graph is replayed."""
    cfg, W, folder = case(tmp_path, "mixed", 6)
    requests = requests_for(cfg, [260, 231], 400)
    want = T.oracle(cfg, W, requests)
    runner = H.make_runner(folder, dtype, page_size=16, num_pages=40, max_request_tokens=272, max_requests=2)
    from llm_pipeline_b200.engine import StepEntry
    rows = {rid: [] for rid in requests}
    out = runner.step([StepEntry(rid, toks[:11], list(range(11))) for rid, toks in requests.items()])
    for k, rid in enumerate(requests):
        rows[rid].append(out[11 * k:11 * (k + 1)].float().cpu())
    for t in range(11, 231):
        out = runner.step([StepEntry(rid, [toks[t]], [0]) for rid, toks in requests.items()])
        for k, rid in enumerate(requests):
            rows[rid].append(out[k:k + 1].float().cpu())
    assert runner.graph_replays > 200
    for rid in requests:
        T.assert_matches({rid: torch.cat(rows[rid])}, {rid: want[rid][:231]}, dtype, f"long decoding of {rid}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(tmp_path, dtype):
    from llm_pipeline_b200.inference import InferenceConfig, InferenceEngine
    cfg, W, folder = case(tmp_path, "attention_first" if dtype == torch.float32 else "mixed", 7)
    engine = InferenceEngine(InferenceConfig(model_path=folder, dtype=dtype, block_size=8, num_blocks=64, max_sequence_length=128,
                                             max_batch_size=4, max_num_batched_tokens=32))
    prompts = [H.random_tokens(cfg["vocab"], n, 600 + n) for n in (1, 7, 30, 45, 12)]       # five requests for four slots
    got = engine.generate(prompts, max_tokens=10, temperature=0.0)
    W64 = {k: v.double() for k, v in W.items()}
    checked = 0
    for prompt, tokens in zip(prompts, got):
        ids = list(prompt)
        for token in tokens:
            logits = plain.forward(cfg, W64, ids)[-1]
            top2 = torch.topk(logits, 2).values
            if dtype == torch.bfloat16 and float(top2[0] - top2[1]) < 0.15:
                break                                                   # a near tie: the two sequences may part here
            assert token == int(logits.argmax()), (len(prompt), len(ids) - len(prompt))
            ids.append(token)
            checked += 1
    assert checked >= (50 if dtype == torch.float32 else 20)
    assert engine.engine.cache.num_live == 0
    info = engine.get_model_info()
    assert info["vocab_size"] == cfg["vocab"] and info["num_layers"] == len(cfg["layers"]) and info["total_parameters"] > 0
