"""The kernels behind capped, chunked attention with a token shift and behind routing by scores, each against plain
PyTorch in float32: every attention kernel that has a form for capped scores and chunks of positions (the general
one, both prompt kernels, the decode kernel with heads as rows), the token shift behind an RMS norm with its state
rows, the clamped gate, the stream's addition, the cap on the logits, and the routing inside groups of experts."""
import math

import pytest
import torch

from sandyrt_b200.csrc import ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _paged(keys, values, page_size, seed, dtype=torch.bfloat16):
    """Scatter per-request keys / values [len, Hkv, D] into a poisoned paged cache with shuffled pages."""
    lens = [k.shape[0] for k in keys]
    Hkv, D = keys[0].shape[1], keys[0].shape[2]
    blocks = [-(-n // page_size) for n in lens]
    n_pages = sum(blocks) + 3
    arena = torch.full((n_pages, 2, Hkv, page_size, D), float("nan"), dtype=dtype, device=DEV)
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    table = torch.full((len(keys), max(blocks)), -1, dtype=torch.int32)
    for r, k in enumerate(keys):
        for b in range(blocks[r]):
            page = order.pop()
            table[r, b] = page
            n = min(page_size, lens[r] - b * page_size)
            arena[page, 0, :, :n] = k[b * page_size:b * page_size + n].transpose(0, 1)
            arena[page, 1, :, :n] = values[r][b * page_size:b * page_size + n].transpose(0, 1)
    return arena[:, 0], arena[:, 1], table.to(DEV)


def _want_rows(q, keys, values, positions, H, scale, cap, chunk, window=0):
    """q [n, H*D] float for queries at `positions` of ONE request whose keys / values are [len, Hkv, D]."""
    Hkv, D = keys.shape[1], keys.shape[2]
    out = torch.zeros(q.shape[0], H * D, dtype=torch.float32, device=q.device)
    j = torch.arange(keys.shape[0], device=q.device)
    for r, pos in enumerate(positions):
        see = j <= pos
        if chunk:
            see &= j >= pos - pos % chunk
        if window:
            see &= j > pos - window
        for h in range(H):
            kv = h // (H // Hkv)
            s = (keys[:, kv].float() @ q[r, h * D:(h + 1) * D].float()) * scale
            if cap:
                s = cap * torch.tanh(s / cap)
            s = s.masked_fill(~see, -math.inf)
            out[r, h * D:(h + 1) * D] = torch.softmax(s, 0) @ values[:, kv].float()
    return out


# portions: (keys before the portion, tokens of the portion); the chunks of 24 / 100 / 128 / 210 positions cut through
# the kernels' tiles of 64 and 128 queries and 128 keys, through pages, and through the portions themselves
PORTIONS = [(0, 1), (0, 300), (37, 150), (209, 3), (210, 130), (511, 2)]


@pytest.mark.parametrize("kernel", ["tcgen05", "mma.sync", "general"])
@pytest.mark.parametrize("H,Hkv,D,cap,chunk,window", [
    (4, 2, 64, 18.0, 210, 0), (6, 1, 64, 8.0, 24, 0), (2, 2, 64, 0.0, 128, 0), (3, 1, 64, 30.0, 0, 0), (4, 4, 64, 12.0, 100, 70),
    (2, 1, 96, 15.0, 100, 0), (2, 2, 32, 10.0, 24, 0),
])
def test_prompt_portions_with_capped_scores_in_chunks(kernel, H, Hkv, D, cap, chunk, window):
    if kernel == "tcgen05" and D != 64:
        pytest.skip("the tcgen05 prompt kernel takes heads of 64")
    g = torch.Generator().manual_seed(H * 100 + D + chunk)
    lens = [b + n for b, n in PORTIONS]
    keys = [torch.randn(n, Hkv, D, generator=g).to(torch.bfloat16).to(DEV) for n in lens]
    values = [torch.randn(n, Hkv, D, generator=g).to(torch.bfloat16).to(DEV) for n in lens]
    k_view, v_view, table = _paged(keys, values, 16, seed=D + chunk)
    T = sum(n for _, n in PORTIONS)
    q = (3.0 * torch.randn(T, H * D, generator=g)).to(torch.bfloat16).to(DEV)      # sharp scores: single keys win, the cap bites
    starts = [0]
    for _, n in PORTIONS:
        starts.append(starts[-1] + n)
    q_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
    kv_before = torch.tensor([b for b, _ in PORTIONS], dtype=torch.int32, device=DEV)
    out = torch.full((T, H * D), 9.0, dtype=torch.bfloat16, device=DEV)
    scale = D ** -0.5
    if kernel == "general":
        token_seq = torch.cat([torch.full((n,), r, dtype=torch.int32) for r, (_, n) in enumerate(PORTIONS)]).to(DEV)
        positions = torch.cat([torch.arange(b, b + n, dtype=torch.int32) for b, n in PORTIONS]).to(DEV)
        ops.paged_attention(q, k_view, v_view, table, token_seq, positions, out, n_heads=H, scale=scale, window=window,
                            softcap=cap, chunk=chunk)
    else:
        ops.prefill_attention(q, k_view, v_view, table, q_start, kv_before, out, n_heads=H, max_q_len=max(n for _, n in PORTIONS),
                              scale=scale, window=window, tc=kernel == "tcgen05", softcap=cap, chunk=chunk)
    ops.check_kernel_status(out.device)
    for r, (b, n) in enumerate(PORTIONS):
        want = _want_rows(q[starts[r]:starts[r + 1]], keys[r], values[r], list(range(b, b + n)), H, scale, cap, chunk, window)
        got = out[starts[r]:starts[r + 1]].float()
        assert torch.allclose(got, want, atol=3e-2, rtol=3e-2), (r, float((got - want).abs().max()))


@pytest.mark.parametrize("H,Hkv,D,cap,chunk,splits", [(5, 1, 80, 18.0, 210, 3), (4, 2, 64, 8.0, 24, 1), (8, 1, 128, 0.0, 100, 4),
                                                      (5, 5, 16, 30.0, 0, 2), (12, 2, 48, 6.0, 7, 1)])
def test_single_tokens_with_capped_scores_in_chunks(H, Hkv, D, cap, chunk, splits):
    """Decoded tokens at the first and the last position of a chunk, one behind an edge, and far into a long request."""
    g = torch.Generator().manual_seed(H * 10 + D)
    lens = [1, 24, 25, 100, 101, 210, 211, 419, 420, 421, 777]
    keys = [torch.randn(n, Hkv, D, generator=g).to(torch.bfloat16).to(DEV) for n in lens]
    values = [torch.randn(n, Hkv, D, generator=g).to(torch.bfloat16).to(DEV) for n in lens]
    k_view, v_view, table = _paged(keys, values, 16, seed=D)
    T = len(lens)
    q = (3.0 * torch.randn(T, H * D, generator=g)).to(torch.bfloat16).to(DEV)
    token_seq = torch.arange(T, dtype=torch.int32, device=DEV)
    positions = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    scale = D ** -0.5
    for which in ("heads as rows", "general"):
        out = torch.full((T, H * D), 9.0, dtype=torch.bfloat16, device=DEV)
        if which == "general":
            ops.paged_attention(q, k_view, v_view, table, token_seq, positions, out, n_heads=H, scale=scale, softcap=cap, chunk=chunk)
        else:
            ops.decode_attention_shared(q, k_view, v_view, table, token_seq, positions, out, n_heads=H, scale=scale, splits=splits,
                                        softcap=cap, chunk=chunk)
        ops.check_kernel_status(out.device)
        for t in range(T):
            want = _want_rows(q[t:t + 1], keys[t], values[t], [lens[t] - 1], H, scale, cap, chunk)
            assert torch.allclose(out[t:t + 1].float(), want, atol=3e-2, rtol=3e-2), (which, t, float((out[t:t + 1].float() - want).abs().max()))


def test_general_kernel_in_float32():
    g = torch.Generator().manual_seed(5)
    H, Hkv, D, cap, chunk = 3, 1, 48, 9.0, 37
    n = 150
    keys = [torch.randn(n, Hkv, D, generator=g).to(DEV)]
    values = [torch.randn(n, Hkv, D, generator=g).to(DEV)]
    k_view, v_view, table = _paged(keys, values, 8, seed=1, dtype=torch.float32)
    q = (3.0 * torch.randn(n, H * D, generator=g)).to(DEV)
    out = torch.empty_like(q)
    ops.paged_attention(q, k_view, v_view, table, torch.zeros(n, dtype=torch.int32, device=DEV),
                        torch.arange(n, dtype=torch.int32, device=DEV), out, n_heads=H, scale=D ** -0.5, softcap=cap, chunk=chunk)
    want = _want_rows(q, keys[0], values[0], list(range(n)), H, D ** -0.5, cap, chunk)
    assert torch.allclose(out, want, atol=2e-5, rtol=2e-5)


# ---- the token shift behind the norm ----------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("width", [48, 100, 256, 768, 1536, 2304, 5000])
def test_token_shift_behind_the_norm(width, dtype, tol):
    """Two steps: portions of 1, 5, 2 and 1 tokens in slots 3, 0, 5, 1 (a request's first token reads its state row, a
    request of one token writes its row in the same launch), then one more token of each, which reads what the first
    step left."""
    g = torch.Generator().manual_seed(width)
    eps = 1e-5
    gain = (1.0 + 0.2 * torch.randn(width, generator=g)).to(DEV)
    mix = torch.rand(width, generator=g).to(DEV)
    state = torch.randn(6, width + 8, generator=g).to(DEV)
    state0 = state.clone()
    lens, slots = [1, 5, 2, 1], [3, 0, 5, 1]
    norm = lambda x: x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * gain
    for step, lens in enumerate((lens, [1, 1, 1, 1])):
        T = sum(lens)
        x = (2.0 * torch.randn(T, width, generator=g)).to(DEV)
        starts = [0]
        for n in lens:
            starts.append(starts[-1] + n)
        token_seq = torch.cat([torch.full((n,), r, dtype=torch.int32) for r, n in enumerate(lens)]).to(DEV)
        out = torch.full((T, width), 9.0, dtype=dtype, device=DEV)
        before_rows = state.clone()
        ops.rmsnorm_shift(x, gain, mix, state, token_seq, torch.tensor(starts, dtype=torch.int32, device=DEV),
                          torch.tensor(slots, dtype=torch.int32, device=DEV), out, eps=eps)
        h = norm(x)
        for r, n in enumerate(lens):
            prev = torch.cat([before_rows[slots[r], :width][None], h[starts[r]:starts[r + 1] - 1]])
            hr = h[starts[r]:starts[r + 1]]
            want = hr + (prev - hr) * mix
            assert torch.allclose(out[starts[r]:starts[r + 1]].float(), want, atol=tol * 4, rtol=tol), (step, r)
            assert torch.allclose(state[slots[r], :width], hr[-1], atol=1e-5, rtol=1e-5)
        for s in (2, 4):                                                  # rows of no request stay as they were
            assert torch.equal(state[s], state0[s])
        assert torch.equal(state[:, width:], state0[:, width:])       # and so does what lies behind the width


# ---- element-wise ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-6), (torch.bfloat16, 1e-2)])
def test_clamped_gate(dtype, tol):
    g = torch.Generator().manual_seed(2)
    both = (3.0 * torch.randn(77, 2 * 40, generator=g)).to(dtype).to(DEV)
    a, b = both[:, :40], both[:, 40:]
    out = torch.empty(77, 40, dtype=dtype, device=DEV)
    ops.glu_clamped(a, b, out, limit=1.5, alpha=1.702)
    gg = a.float().clamp(max=1.5)
    u = b.float().clamp(-1.5, 1.5)
    want = gg * torch.sigmoid(1.702 * gg) * (u + 1.0)
    assert torch.allclose(out.float(), want, atol=tol, rtol=tol)
    assert float(a.float().min()) < -1.5 and float((out.float() - want).abs().max()) < 0.05       # the gate is cut from above only


def test_stream_addition_and_logit_cap():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(33, 100, generator=g).to(DEV)
    x0 = torch.randn(33, 100, generator=g).to(DEV)
    row = torch.randn(100, generator=g).to(DEV)
    for use0, use_row in ((True, True), (False, True), (True, False)):
        y = x.clone()
        ops.stream_add(y, x0 if use0 else None, row if use_row else None)
        want = x + (x0 if use0 else 0) + (row if use_row else 0)
        assert torch.allclose(y, want, atol=1e-6)
    z = (40.0 * torch.randn(7, 333, generator=g)).to(DEV)
    want = 30.0 * torch.tanh(z / 30.0)
    ops.softcap(z, 30.0)
    assert torch.allclose(z, want, atol=1e-4, rtol=1e-5)


# ---- routing by scores inside groups ----------------------------------------------------------------------------
def _route_plain(logits, correction, top, n_groups, keep, rank, scale, eps):
    s = torch.sigmoid(logits.double())
    c = s + correction.double()
    T, E = c.shape
    per = E // n_groups
    gs = c.view(T, n_groups, per).topk(min(rank, per), -1).values.sum(-1)
    order = gs.argsort(dim=-1, descending=True, stable=True)
    kept = torch.zeros_like(gs, dtype=torch.bool)
    kept.scatter_(1, order[:, :keep], True)
    c_in = c.masked_fill(~kept.repeat_interleave(per, 1), -math.inf)
    chosen = c_in.sort(dim=-1, descending=True, stable=True).indices[:, :top]
    picked = s.gather(1, chosen)
    return chosen, picked / (picked.sum(-1, keepdim=True) + eps) * scale


@pytest.mark.parametrize("T,E,top,n_groups,keep,rank", [(1, 8, 2, 2, 1, 2), (300, 12, 3, 4, 2, 2), (50, 6, 6, 1, 1, 2), (70, 6, 2, 6, 3, 2),
                                                        (200, 64, 8, 8, 3, 2), (40, 256, 8, 8, 4, 2), (90, 9, 2, 3, 1, 1)])
def test_routing_by_scores_in_groups(T, E, top, n_groups, keep, rank):
    g = torch.Generator().manual_seed(E + T)
    logits = (2.0 * torch.randn(T, E, generator=g)).to(DEV)
    for shift in (0.0, -3.0):                                  # with -3 every choice score is negative
        correction = (shift + 0.5 * torch.randn(E, generator=g)).to(DEV)
        r = ops.moe_route_scored(logits, correction, top, n_groups=n_groups, keep_groups=keep, group_rank=rank, weight_scale=2.5,
                                 norm_eps=1e-20)
        chosen, weights = _route_plain(logits, correction, top, n_groups, keep, rank, 2.5, 1e-20)
        got_e = r.expert_of.view(T, top).long()
        got_w = r.weight_of.view(T, top)
        assert torch.equal(got_e.sort(-1).values, chosen.sort(-1).values)
        for t in range(T):
            w = {int(e): float(x) for e, x in zip(chosen[t], weights[t])}
            for e, x in zip(got_e[t].tolist(), got_w[t].tolist()):
                assert abs(x - w[e]) < 1e-5
        # the entries grouped by expert
        counts = torch.bincount(got_e.flatten(), minlength=E)
        assert torch.equal((r.group_start[1:] - r.group_start[:-1]).long(), counts)
