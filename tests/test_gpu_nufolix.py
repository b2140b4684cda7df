"""The Nufolix decoder in the engine against the plain implementation (``plain_nufolix.py``, float64): each mechanism
alone, whole prompts, token-by-token decoding, portions down to two tokens, unequal batches, pages and slots used again,
keys far away and at page and segment borders under sparse attention weights, state carried over hundreds of tokens,
the first tokens, long decoding, several shapes, and greedy generation through the entry point."""

import itertools
import math

import pytest
import torch

import helpers as H
import nufolix_cases as N
import plain_nufolix as plain

pytestmark = pytest.mark.gpu
DTYPES = [pytest.param(torch.float32, id="f32"), pytest.param(torch.bfloat16, id="bf16")]


def case(tmp_path, name, seed, sharp=None, head_bias=-1.0):
    cfg = N.CONFIGS[name] if sharp is None else N.sharpen(N.CONFIGS[name], sharp)
    W = N.weights_for(cfg, seed, head_bias=head_bias)
    return cfg, W, N.write_model(str(tmp_path), cfg, W)


def requests_for(cfg, lengths, seed):
    return {f"r{i}": H.random_tokens(cfg["vocab"], n, seed + i) for i, n in enumerate(lengths)}


def _i32(values, dev="cuda"):
    return torch.tensor(values, dtype=torch.int32, device=dev)


# ---- kernels alone ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
def test_activation_gated_norms_and_weighted_sum_alone(dtype):
    from llm_pipeline_b200.ops import kernels
    torch.manual_seed(1)
    dev = "cuda"
    tol = 1e-5 if dtype == torch.float32 else 2.0 ** -7
    for rows, width in ((5, 104), (3, 37)):
        z = torch.randn(rows, width) * 3
        bias = torch.randn(width)
        act = torch.tensor([0.4, -0.9], dtype=torch.float64)
        out = torch.empty(rows, width, device=dev, dtype=dtype)
        a_pos, a_neg = float(plain.softplus(act[0])), 0.5 + float(plain.softplus(act[1]))
        kernels.xielu(z.to(dev), bias.to(dev), a_pos, a_neg, out)
        want = plain.xielu(z.double() + bias.double(), act)
        assert ((out.float().cpu().double() - want).abs() <= tol * want.abs() + 1e-5).all()
        assert (z + bias > 0).any() and (z + bias < -2).any()                       # both branches, also far below zero
        a, b = torch.randn(rows, width), torch.randn(rows, width)
        got = kernels.scaled_sum(a.to(dev), 1.7, b.to(dev), -0.4, torch.empty(rows, width, device=dev))
        assert (got.cpu().double() - (1.7 * a.double() - 0.4 * b.double())).abs().max() < 1e-6
    # rows normed in equal parts: gate first (y silu(z), then the norm, a weight per column), and gate last (the norm,
    # a weight per column of the part, then sigmoid(z))
    for rows, parts, size in ((4, 1, 48), (6, 3, 20), (2, 5, 7), (3, 2, 520), (2, 1, 2100)):     # the last two: a block per part
        y, g = torch.randn(rows, parts * size) * 2, torch.randn(rows, parts * size)
        w_row, w_part = 1 + 0.3 * torch.randn(parts * size), 1 + 0.3 * torch.randn(size)
        out = torch.empty(rows, parts * size, device=dev, dtype=dtype)
        kernels.gated_group_norm(y.to(dev), g.to(dev), w_row.to(dev), out, size, 1e-5, gate_first=True)
        gated = y.double() * plain.silu(g.double())
        want = plain.rms(gated.view(rows, parts, size), 1e-5).reshape(rows, -1) * w_row.double()
        assert (out.float().cpu().double() - want).abs().max() < (1e-5 if dtype == torch.float32 else 4e-2)
        kernels.gated_group_norm(y.to(dev), g.to(dev), w_part.to(dev), out, size, 1e-5, gate_first=False)
        want = (plain.rms(y.double().view(rows, parts, size), 1e-5) * w_part.double()).reshape(rows, -1) * torch.sigmoid(g.double())
        assert (out.float().cpu().double() - want).abs().max() < (1e-5 if dtype == torch.float32 else 4e-2)


@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_short_convolution_carries_its_last_inputs_from_step_to_step(taps):
    """Two requests in slots that are not theirs by number, fed in portions of 1, 2, 3 and more tokens, together and in
    turns: every output is that of the whole sequence, so the carried inputs are right at every cut."""
    from llm_pipeline_b200.ops import kernels
    gen = torch.Generator().manual_seed(taps)
    dev, C = "cuda", 37
    w, b = torch.randn(C, taps, generator=gen), torch.randn(C, generator=gen)
    xs = {3: torch.randn(23, C, generator=gen), 1: torch.randn(16, C, generator=gen)}
    want = {s: plain.silu(plain.short_convolution(x.double(), w.double(), b.double())) for s, x in xs.items()}
    state = torch.full((5, 2 * (taps - 1) * C + 11), 9.0, device=dev)              # other requests' slots, which nothing may touch
    state[[3, 1]] = 0.0                                                             # a slot is zeroed when it is handed out
    done = {3: 0, 1: 0}
    got = {3: [], 1: []}
    for step, sizes in enumerate([{3: 1}, {3: 2, 1: 5}, {1: 1}, {3: 3, 1: 1}, {3: 1, 1: 2}, {3: 16, 1: 7}]):
        rows = torch.cat([xs[s][done[s]:done[s] + n] for s, n in sizes.items()])
        q_start = _i32([0] + list(itertools.accumulate(sizes.values())))
        positions = _i32([p for s, n in sizes.items() for p in range(done[s], done[s] + n)])
        request = _i32([i for i, n in enumerate(sizes.values()) for _ in range(n)])
        out = torch.empty(rows.shape[0], C, device=dev)
        kernels.short_conv(rows.to(dev), w.to(dev), b.to(dev), state, 4, q_start, _i32(list(sizes)), positions, request, out,
                           max(sizes.values()), silu=True)
        at = 0
        for s, n in sizes.items():
            got[s].append(out[at:at + n].cpu())
            at, done[s] = at + n, done[s] + n
    for s in xs:
        assert done[s] == xs[s].shape[0]
        assert (torch.cat(got[s]).double() - want[s]).abs().max() < 1e-5, s
    assert (state[[0, 2, 4]] == 9.0).all() and (state[:, :4] == torch.tensor([9.0, 0.0, 9.0, 0.0, 9.0], device=dev)[:, None]).all()


def _scan_in_portions(launch, n, cuts, state_entries, offset):
    """Run ``launch(begin, end, state, q_start, slots, positions)`` over [0, n) cut at ``cuts``, in slot 2 of 4."""
    state = torch.full((4, offset + state_entries + 3), 5.0, device="cuda")     # other requests' slots, which nothing may touch
    state[2] = 0.0                                                               # a slot is zeroed when it is handed out
    edges = [0] + list(cuts) + [n]
    for begin, end in zip(edges[:-1], edges[1:]):
        launch(begin, end, state, _i32([0, end - begin]), _i32([2]), _i32(list(range(begin, end))))
    assert (state[[0, 1, 3]] == 5.0).all() and (state[2, :offset] == 0.0).all() and (state[2, offset + state_entries:] == 0.0).all()
    return state


@pytest.mark.parametrize("sizes", [(4, 2, 24, 16), (3, 3, 7, 12), (2, 1, 64, 32), (5, 1, 16, 128), (2, 2, 200, 9), (1, 1, 530, 3),
                                   (2, 1, 128, 64), (3, 1, 1, 5)], ids=str)
def test_state_space_recurrence_alone(sizes):
    """The scan kernel against the recurrence written out, whole and in portions of 1, 2 and more tokens: heads that share a
    group of state channels, state channels more and fewer than value channels, decays from near 0 to near 1."""
    from llm_pipeline_b200.ops import kernels
    heads, groups, state_n, vdim = sizes
    gen = torch.Generator().manual_seed(sum(sizes))
    dev, n = "cuda", 70
    xbc = torch.randn(n, heads * vdim + 2 * groups * state_n, generator=gen)
    dt = torch.randn(n, heads, generator=gen) * 2
    dt_bias, a_log, d_skip = torch.randn(heads, generator=gen), torch.rand(heads, generator=gen) * 6 - 5, torch.randn(heads, generator=gen)
    x = xbc[:, :heads * vdim].double().view(n, heads, vdim)
    B = xbc[:, heads * vdim:heads * vdim + groups * state_n].double().view(n, groups, state_n)
    C = xbc[:, heads * vdim + groups * state_n:].double().view(n, groups, state_n)
    step = plain.softplus(dt.double() + dt_bias.double())
    want = torch.zeros(n, heads, vdim, dtype=torch.float64)
    for h in range(heads):
        g = h // (heads // groups)
        S = torch.zeros(state_n, vdim, dtype=torch.float64)
        for t in range(n):
            S = torch.exp(-torch.exp(a_log[h].double()) * step[t, h]) * S + step[t, h] * torch.outer(B[t, g], x[t, h])
            want[t, h] = S.T @ C[t, g] + d_skip[h].double() * x[t, h]
    for cuts in ((), (1, 3, 4, 20, 21), tuple(range(1, n))):
        y = torch.empty(n, heads * vdim, device=dev)

        def launch(begin, end, state, q_start, slots, positions):
            kernels.ssd_scan(xbc[begin:end].to(dev), dt[begin:end].to(dev), dt_bias.to(dev), a_log.to(dev), d_skip.to(dev), state, 6,
                             q_start, slots, positions, y[begin:end], heads, groups, state_n, vdim)

        _scan_in_portions(launch, n, cuts, 2 * heads * state_n * vdim, 6)
        assert (y.cpu().double() - want.view(n, -1)).abs().max() < 2e-4 * max(1.0, float(want.abs().max())), cuts


@pytest.mark.parametrize("sizes", [(4, 2, 16, 24), (3, 3, 12, 5), (2, 1, 64, 32), (1, 1, 32, 128), (6, 1, 128, 16), (2, 2, 200, 9),
                                   (1, 1, 530, 3), (2, 1, 96, 40), (3, 1, 1, 5)], ids=str)
def test_gated_delta_rule_alone(sizes):
    """Unit vectors, step sizes and decays (the preparing kernel) and the scan against the rule written out, whole and in
    portions: the read-out sees the token's own write, heads share query/key heads, keys wider and narrower than values."""
    from llm_pipeline_b200.ops import kernels
    heads, qk_heads, dim, vdim = sizes
    gen = torch.Generator().manual_seed(sum(sizes))
    dev, n = "cuda", 60
    q0, k0 = torch.randn(n, qk_heads * dim, generator=gen), torch.randn(n, qk_heads * dim, generator=gen)
    v = torch.randn(n, heads * vdim, generator=gen)
    pre, beta0 = torch.randn(n, heads * dim, generator=gen) * 2, torch.randn(n, heads, generator=gen) * 2
    a_log, dt_bias = torch.rand(heads, generator=gen) * 5 - 4.5, torch.randn(heads * dim, generator=gen)
    q = q0.double().view(n, qk_heads, dim)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k0.double().view(n, qk_heads, dim)
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    decay = torch.exp(-torch.exp(a_log.double())[None, :, None] * plain.softplus(pre.double() + dt_bias.double()).view(n, heads, dim))
    beta = torch.sigmoid(beta0.double())
    want = torch.zeros(n, heads, vdim, dtype=torch.float64)
    for h in range(heads):
        g = h // (heads // qk_heads)
        S = torch.zeros(dim, vdim, dtype=torch.float64)
        for t in range(n):
            S = decay[t, h][:, None] * S
            S = S + torch.outer(k[t, g], beta[t, h] * (v[t].double().view(heads, vdim)[h] - S.T @ k[t, g]))
            want[t, h] = S.T @ q[t, g]
    qd, kd, dd, bd = q0.to(dev), k0.to(dev), pre.to(dev), beta0.to(dev)
    kernels.delta_prep(qd, kd, dd, bd, a_log.to(dev), dt_bias.to(dev), heads, qk_heads, dim)
    assert (qd.cpu().double() - q.view(n, -1)).abs().max() < 1e-6 and (kd.cpu().double() - k.view(n, -1)).abs().max() < 1e-6
    assert (dd.cpu().double() - decay.view(n, -1)).abs().max() < 1e-6 and (bd.cpu().double() - beta).abs().max() < 1e-6
    for cuts in ((), (1, 3, 4, 20, 21), tuple(range(1, n))):
        o = torch.empty(n, heads * vdim, device=dev)

        def launch(begin, end, state, q_start, slots, positions):
            kernels.delta_scan(qd[begin:end], kd[begin:end], v[begin:end].to(dev), dd[begin:end], bd[begin:end], state, 2, q_start, slots,
                               positions, o[begin:end], heads, qk_heads, dim, vdim)

        _scan_in_portions(launch, n, cuts, 2 * heads * dim * vdim, 2)
        assert (o.cpu().double() - want.view(n, -1)).abs().max() < 1e-4, cuts


def _sigmoid_attention_case(dtype, heads, kv_heads, dim, vdim, n, page, seed, cap=0.0, plant=None, segments=(1,), bias=-1.0):
    """Queries, keys and values as they enter the scores, written into shuffled pages; (engine outputs, plain output)."""
    from llm_pipeline_b200.ops import kernels
    gen = torch.Generator().manual_seed(seed)
    dev = "cuda"
    q, k = torch.randn(n, heads, dim, generator=gen), torch.randn(n, kv_heads, dim, generator=gen)
    v = torch.randn(n, kv_heads, vdim, generator=gen)
    talk = torch.eye(heads) * 0.6 + torch.randn(heads, heads, generator=gen) * 0.4
    pb = torch.randn(heads, generator=gen) * 0.5 + bias
    if plant is not None:
        plant(q, k, v)
    q, k, v = (t.to(torch.bfloat16).float() for t in (q, k, v))
    scale = 1.0 / math.sqrt(dim)
    kv_of = torch.arange(heads) // (heads // kv_heads)
    s = torch.einsum("ihd,jhd->hij", q.double(), k.double()[:, kv_of]) * scale
    if cap:
        s = cap * torch.tanh(s / cap)
    w = torch.sigmoid(s + pb.double()[:, None, None]) * (torch.arange(n)[None, :] <= torch.arange(n)[:, None]).double()
    want = torch.einsum("hij,jhv->ihv", torch.einsum("hg,gij->hij", talk.double(), w), v.double()[:, kv_of]).reshape(n, -1)
    pages_n = -(-n // page)
    order = torch.randperm(pages_n + 3, generator=gen)[:pages_n]     # the request's pages lie anywhere in the pool
    pages = torch.full((pages_n + 3, kv_heads, page, dim + vdim), 7.0)  # other pages hold garbage
    for t in range(n):
        pages[order[t // page], :, t % page] = torch.cat([k[t], v[t]], dim=-1)
    table = order.to(torch.int32).view(1, -1).to(dev)
    positions = torch.arange(n, dtype=torch.int32, device=dev)
    qd, pd = q.reshape(n, -1).to(dev).to(dtype).contiguous(), pages.to(dev).to(dtype)
    results = {}
    for count in segments:
        out = torch.empty(n, heads * vdim, device=dev, dtype=dtype)
        kernels.sigmoid_attention(qd, pd, table, torch.zeros(n, dtype=torch.int32, device=dev), positions, talk.to(dev), pb.to(dev), out,
                                  heads, kv_heads, dim, vdim, scale, cap, count)
        results[f"{count} segments"] = out.float().cpu()
    if kernels.sigmoid_attention_mma_supports(dtype, heads, kv_heads, dim, vdim):
        # the tensor-core kernel: the whole prompt in tiles of 16 tokens, its keys in one block and in ranges; then only the
        # last 37 tokens as a portion (three tiles, the last one short, the first one starting in the middle of a page)
        rows = kernels.SIGMOID_MMA_ROWS
        ctx_len = torch.tensor([n], dtype=torch.int32, device=dev)
        for tail, count in ((n, 1), (n, -(-n // kernels.SIGMOID_MMA_SEGMENT_KEYS)), (37, 1), (37, -(-n // kernels.SIGMOID_MMA_SEGMENT_KEYS))):
            out = torch.empty(tail, heads * vdim, device=dev, dtype=dtype)
            tok0 = torch.arange(0, tail, rows, dtype=torch.int32, device=dev)
            kernels.sigmoid_attention_mma(qd[n - tail:], pd, table, torch.tensor([0, tail], dtype=torch.int32, device=dev), ctx_len,
                                          positions[n - tail:].contiguous(), torch.zeros_like(tok0), tok0, talk.to(dev), pb.to(dev), out,
                                          heads, kv_heads, dim, vdim, scale, cap, count)
            full = torch.zeros(n, heads * vdim)
            full[n - tail:] = out.float().cpu()
            full[:n - tail] = want[:n - tail].float()
            results[f"tensor cores, last {tail} tokens, {count} key ranges"] = full
    return results, want


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [(4, 2, 16, 24, 0.0), (3, 3, 12, 20, 2.0), (6, 1, 48, 48, 8.0), (2, 2, 128, 64, 0.0), (32, 2, 16, 16, 30.0), (4, 2, 16, 32, 0.0), (6, 3, 96, 64, 5.0),
                                   (16, 4, 128, 128, 3.0), (12, 12, 32, 96, 0.0),
                                   (1, 1, 64, 128, 1.0), (5, 5, 10, 200, 0.0)], ids=str)
def test_sigmoid_attention_alone(dtype, sizes):
    """Weights that are sigmoids of capped scores, mixed across heads, not normalised: grouped heads, values of another
    width than keys, over shuffled pages, with a token's keys in one block and shared among blocks in segments."""
    from llm_pipeline_b200.ops import kernels
    heads, kv_heads, dim, vdim, cap = sizes
    n = kernels.SIGMOID_SEGMENT_KEYS + 90
    results, want = _sigmoid_attention_case(dtype, heads, kv_heads, dim, vdim, n, page=16, seed=3, cap=cap, segments=(1, 2), bias=-3.0)
    for name, got in results.items():
        err = (got.double() - want).abs().max() / want.abs().max()
        assert err < (1e-5 if dtype == torch.float32 else 1e-2), (name, float(err))


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_far_key_holds_all_the_weight(dtype):
    """Every query has a score of about -12 with every key but one, which lies 1 to 1,100 tokens back and gets +12: across
    page borders, across the border of a key segment, the very first key, the query's own. The result is that key's value
    row (through the head mix) to a few parts in a thousand, so a key that is lost or shifted by one shows wholly."""
    from llm_pipeline_b200.ops import kernels
    heads, kv_heads, dim, vdim = 4, 2, 64, 32
    n = kernels.SIGMOID_SEGMENT_KEYS + 170
    target = [(t * 7919) % (t + 1) if t % 3 else (0 if t % 2 else t) for t in range(n)]     # anywhere, the first key, or itself
    for edge in (15, 16, 17, kernels.SIGMOID_SEGMENT_KEYS - 1, kernels.SIGMOID_SEGMENT_KEYS):
        target[n - 1 - (edge % 5)] = n - 1 - (edge % 5) - edge if n - 1 - (edge % 5) - edge >= 0 else 0
    basis = torch.linalg.qr(torch.randn(n, n, generator=torch.Generator().manual_seed(9)))[0][:, :dim]   # nearly orthogonal rows

    def plant(q, k, v):
        directions = torch.nn.functional.normalize(torch.randn(n, dim, generator=torch.Generator().manual_seed(10)), dim=-1)
        k[:] = directions[:, None, :] * 8
        for t in range(n):
            q[t] = directions[target[t]][None, :] * 24                            # score 24 with its key, |.| < about 10 with others

    results, want = _sigmoid_attention_case(dtype, heads, kv_heads, dim, vdim, n, page=16, seed=4, cap=0.0, plant=plant, segments=(1, 2),
                                            bias=-12.0)
    # the premise: dropping the target key changes the plain result by a large part of itself
    assert want.abs().max() > 0.5
    for name, got in results.items():
        err = (got.double() - want).abs().max()
        assert err < (1e-4 if dtype == torch.float32 else 3e-2), (name, float(err))


@pytest.mark.parametrize("dtype", DTYPES)
def test_projection_bias_rotation_and_cache_rows_alone(dtype):
    """The kernel after the q/k/v product against the plain rotation: biases, rotated parts of all, some and none of a key,
    positions far from zero, rows written into the right place of the pages."""
    from llm_pipeline_b200.ops import kernels
    from llm_pipeline_b200.parts.position import RotaryPositions
    torch.manual_seed(5)
    dev, n, page = "cuda", 11, 4
    for heads, kv_heads, dim, vdim, rot in ((3, 1, 24, 40, 8), (4, 2, 16, 16, 16), (2, 2, 40, 8, 0)):
        width = (heads + kv_heads) * dim + kv_heads * vdim
        qkv, bias = torch.randn(n, width), torch.randn(width).to(torch.bfloat16).float()
        positions = torch.arange(1000, 1000 + n)
        full = qkv.double() + bias.double()
        q = full[:, :heads * dim].view(n, heads, dim)
        k = full[:, heads * dim:(heads + kv_heads) * dim].view(n, kv_heads, dim)
        cos = sin = None
        if rot:
            q, k = plain.rotate_half(q, positions, rot, 500.0), plain.rotate_half(k, positions, rot, 500.0)
            part = RotaryPositions("", rot, 500.0)
            cos, sin = torch.empty(n, rot // 2, device=dev), torch.empty(n, rot // 2, device=dev)
            kernels.rope_tables(positions.to(torch.int32).to(dev), part._inv_freq_cpu.to(dev), 1.0, cos, sin)
        pages = torch.zeros(6, kv_heads, page, dim + vdim, device=dev, dtype=dtype)
        slots = torch.tensor([(5 - t // page) * page + t % page for t in range(n)], dtype=torch.int32, device=dev)
        q_out = torch.empty(n, heads * dim, device=dev, dtype=dtype)
        kernels.sig_qkv_post(qkv.to(dev), bias.to(dev), cos, sin, rot, q_out, slots, pages, heads, kv_heads, dim, vdim)
        tol = 3e-4 if dtype == torch.float32 else 4e-2               # float32 angles at positions around 1000
        assert (q_out.float().cpu().double() - q.reshape(n, -1)).abs().max() < tol
        for t in range(n):
            row = pages[5 - t // page, :, t % page].float().cpu().double()
            assert (row[:, :dim] - k[t]).abs().max() < tol
            assert (row[:, dim:] - full[t, (heads + kv_heads) * dim:].view(kv_heads, vdim)).abs().max() < tol


# ---- one layer of each kind ------------------------------------------------------------------------------------------
ONE_LAYER = {
    "state_space": N.config([N.mamba2(3, 16, 24, groups=1, conv=4, norm_groups=1)], width=40, vocab=71),
    "state_space_with_ff": N.config([N.mamba2(4, 8, 12, groups=2, conv=3, norm_groups=2, mlp=N.dense(56))], width=40, vocab=71),
    "side_by_side": N.config([N.parallel(N.left(4, 2, 16, 24, rot_dims=8), N.right(4, 2, 16, 24, conv=3), 0.8, 1.3)], width=40, vocab=71),
    "side_by_side_with_ff": N.config([N.parallel(N.left(2, 2, 24, 8, rot_dims=None, softcap=None), N.right(2, 1, 12, 20, conv=4), 1.2, 0.5,
                                                 mlp=N.dense(64))], width=40, vocab=71, mult=1.1, scale=1.0),
}


@pytest.mark.parametrize("name", sorted(ONE_LAYER))
def test_one_layer_alone(tmp_path, name):
    cfg = ONE_LAYER[name]
    W = N.weights_for(cfg, 11)
    folder = N.write_model(str(tmp_path), cfg, W)
    requests = requests_for(cfg, [1, 2, 33, 70], 50)
    want = N.oracle(cfg, W, requests)
    runner = H.make_runner(folder, torch.float32, page_size=8, num_pages=24, max_request_tokens=96, max_requests=2)
    N.assert_matches(H.replay(runner, H.cut_whole(requests)), want, torch.float32, f"{name}, whole")
    N.assert_matches(H.replay(runner, H.cut_portions(requests, (2, 5, 1, 16))), want, torch.float32, f"{name}, portions")


# ---- whole models ----------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(N.CONFIGS))
def test_prefill_decoding_portions_and_batches(tmp_path, name, dtype):
    cfg, W, folder = case(tmp_path, name, 3)
    requests = requests_for(cfg, [1, 2, 3, 19, 64, 65, 150], 100)
    want = N.oracle(cfg, W, requests)
    page = 8
    share = 1.0 if dtype == torch.float32 else 0.99     # bfloat16: one position in a hundred may round further
    runner = H.make_runner(folder, dtype, page_size=page, num_pages=2 * (-(-150 // page)) + 6, max_request_tokens=160, max_requests=4)
    N.assert_matches(H.replay(runner, H.cut_whole(requests)), want, dtype, f"{name}: whole prompts", share)
    N.assert_matches(H.replay(runner, H.cut_tail_one_by_one(requests, tail=40)), want, dtype, f"{name}: last tokens one by one", share)
    N.assert_matches(H.replay(runner, H.cut_portions(requests, (1,))), want, dtype, f"{name}: token by token", share)
    N.assert_matches(H.replay(runner, H.cut_portions(requests, (2, 7, 3, 64, 2, 33))), want, dtype, f"{name}: portions", share)
    # unequal requests side by side, four live at most, so the slots and pages of finished ones go to later ones
    got = H.replay(runner, H.cut_mixed(requests, (2, 5, 16, 3, 31), max_live=4, decode_tail=9))
    N.assert_matches(got, want, dtype, f"{name}: mixed batches", share)
    assert runner.cache.num_live == 0                                   # seven requests went through four slots
    assert runner.cache.pages_reused > 0 or all(layer["type"] != "parallel" for layer in cfg["layers"])


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
@pytest.mark.parametrize("name", ["mixed", "attention_first"])
def test_far_keys_page_borders_and_first_tokens_under_sparse_weights(tmp_path, name, dtype):
    """Scores of a wide spread under a strongly negative number per head: a query's weight sits on a few keys, often
    hundreds of tokens back, so a key that is lost, off by one or read from another request's page changes the logits by
    its whole value. Prompts as long as many pages, positions around every page border, decoded alone and in portions."""
    cfg, W, folder = case(tmp_path, name, 5, sharp=5.0, head_bias=-9.0)
    page = 16
    requests = requests_for(cfg, [4 * page, 4 * page + 1, 330, 17], 300)
    want = N.oracle(cfg, W, requests)
    # the premise: in the plain implementation itself the far keys matter (without the first 3 pages the late logits differ much)
    late = plain.forward(cfg, {k: v.double() for k, v in W.items()}, requests["r2"][3 * page:]).float()
    assert N.row_errors(late[-40:], want["r2"][-40:]).median() > 0.03
    runner = H.make_runner(folder, dtype, page_size=page, num_pages=2 * 21 + 4, max_request_tokens=336, max_requests=4)
    share = 1.0 if dtype == torch.float32 else 0.97
    N.assert_matches(H.replay(runner, H.cut_whole(requests)), want, dtype, "sparse: whole", share)
    N.assert_matches(H.replay(runner, H.cut_tail_one_by_one(requests, tail=3 * page + 2)), want, dtype, "sparse: decoding across borders", share)
    N.assert_matches(H.replay(runner, H.cut_portions(requests, (page - 1, 2, page + 1, 2 * page, 3))), want, dtype, "sparse: portions", share)
    N.assert_matches(H.replay(runner, H.cut_mixed(requests, (page, 2, page + 1), max_live=3, decode_tail=page + 3)), want, dtype, "sparse: mixed", share)


@pytest.mark.parametrize("dtype", DTYPES)
def test_few_rows_over_long_contexts_take_key_segments(tmp_path, dtype):
    """Contexts of several key segments under sparse weights: decoding steps and short portions share a token's keys among
    blocks whose sums a second kernel adds; positions around the segment borders, and long portions that take one block.
    In float32 the general kernel runs, in bfloat16 the tensor-core kernel with its shorter key ranges."""
    from llm_pipeline_b200.ops import kernels
    cfg, W, folder = case(tmp_path, "attention_first", 8, sharp=5.0, head_bias=-9.0)
    seg = kernels.SIGMOID_SEGMENT_KEYS
    requests = requests_for(cfg, [seg + 40, 2 * seg + 2, 70], 700)
    want = N.oracle(cfg, W, requests)
    runner = H.make_runner(folder, dtype, page_size=16, num_pages=3 * (seg // 16) + 16, max_request_tokens=2 * seg + 16, max_requests=3)
    used = {"general": [], "tensor cores": []}
    general, tensor = kernels.sigmoid_attention, kernels.sigmoid_attention_mma

    def counting_general(*args, **kwargs):
        used["general"].append(args[-1] if len(args) > 14 else kwargs.get("segments", 1))
        return general(*args, **kwargs)

    def counting_tensor(*args, **kwargs):
        used["tensor cores"].append((args[-1] if len(args) > 17 else kwargs.get("segments", 1), kwargs.get("segment_keys", 0)))
        return tensor(*args, **kwargs)

    kernels.sigmoid_attention, kernels.sigmoid_attention_mma = counting_general, counting_tensor
    try:
        N.assert_matches(H.replay(runner, H.cut_tail_one_by_one(requests, tail=50)), want, dtype, "segments: decoding")
        N.assert_matches(H.replay(runner, H.cut_portions(requests, (seg - 3, 2, 5, seg + 7, 3))), want, dtype, "segments: portions")
        N.assert_matches(H.replay(runner, H.cut_mixed(requests, (seg, 2, 9), max_live=3, decode_tail=12)), want, dtype, "segments: mixed")
    finally:
        kernels.sigmoid_attention, kernels.sigmoid_attention_mma = general, tensor
    if dtype == torch.float32:
        assert not used["tensor cores"] and any(n > 1 for n in used["general"]) and any(n == 1 for n in used["general"]), \
            "both forms of the general kernel should have run"
    else:
        assert not used["general"] and any(n > 1 for n, _ in used["tensor cores"]), "the tensor-core kernel should have run with key ranges"
        assert all(keys in (kernels.SIGMOID_MMA_SEGMENT_KEYS, kernels.SIGMOID_MMA_LONG_SEGMENT_KEYS) for _, keys in used["tensor cores"])


def test_recurrent_states_carry_what_was_written_hundreds_of_tokens_back(tmp_path):
    """Decays close to one: what the first tokens wrote into the states still weighs in the logits 300 tokens later, so a
    state that is lost, zeroed at a cut or taken from another slot shows. Checked whole, in portions and in mixed batches."""
    cfg = N.CONFIGS["mixed"]
    W = N.weights_for(cfg, 12)
    for name in W:
        if name.endswith("A_log"):
            W[name] = torch.full_like(W[name], -6.0)                    # a unit step keeps 0.9975 of the state
        if name.endswith("dt_bias"):
            W[name] = (W[name] - 1.0).to(torch.bfloat16).float()
    folder = N.write_model(str(tmp_path), cfg, W)
    requests = requests_for(cfg, [320, 301, 47], 900)
    want = N.oracle(cfg, W, requests)
    other = list(requests["r0"])
    other[:8] = H.random_tokens(cfg["vocab"], 8, 77)                    # the premise: the first tokens still matter at the end
    changed = plain.forward(cfg, {k: v.double() for k, v in W.items()}, other).float()
    assert N.row_errors(changed[-20:], want["r0"][-20:]).median() > 0.02
    runner = H.make_runner(folder, torch.float32, page_size=16, num_pages=50, max_request_tokens=336, max_requests=3)
    N.assert_matches(H.replay(runner, H.cut_whole(requests)), want, torch.float32, "long memory: whole")
    N.assert_matches(H.replay(runner, H.cut_portions(requests, (2, 63, 1, 130, 5))), want, torch.float32, "long memory: portions")
    N.assert_matches(H.replay(runner, H.cut_mixed(requests, (40, 2, 9), max_live=2, decode_tail=20)), want, torch.float32, "long memory: mixed")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_through_replayed_graphs(tmp_path, dtype):
    """Two requests decode side by side for 220 steps over many pages, the states taking turns between their two copies:
    from the third step on a captured graph is replayed."""
    cfg, W, folder = case(tmp_path, "mixed", 6)
    requests = requests_for(cfg, [260, 231], 400)
    want = N.oracle(cfg, W, requests)
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
        N.assert_matches({rid: torch.cat(rows[rid])}, {rid: want[rid][:231]}, dtype, f"long decoding of {rid}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(tmp_path, dtype):
    from llm_pipeline_b200.inference import InferenceConfig, InferenceEngine
    cfg, W, folder = case(tmp_path, "mixed" if dtype == torch.float32 else "attention_first", 7)
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
