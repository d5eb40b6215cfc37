"""The kernels behind several copies of the stream, attention with a bias by distance and the state-space mixer, each
against plain PyTorch in float32: the bias in every attention kernel that has a form for it (the general one, the
mma.sync prompt kernel, the decode kernel with heads as rows), the per-head unit norm and the factor by position in the
per-token pass, one pass over the streams (write, sum, read with its norm), the short convolution with its tail, the
embedding with its pair table and its kept token, the state-space recurrence in portions and single tokens, the gate
in front of a norm in groups, routing by softmax scores and the combining of identity experts."""
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


def _want_rows(q, keys, values, positions, H, scale, bias):
    """q [n, H*D] for queries at `positions` of ONE request whose keys / values are [len, Hkv, D]; bias [H, n_dist]."""
    Hkv, D = keys.shape[1], keys.shape[2]
    out = torch.zeros(q.shape[0], H * D, dtype=torch.float32, device=q.device)
    j = torch.arange(keys.shape[0], device=q.device)
    for r, pos in enumerate(positions):
        see = j <= pos
        dist = (pos - j).clamp(0, bias.shape[1] - 1)
        for h in range(H):
            s = (keys[:, h // (H // Hkv)].float() @ q[r, h * D:(h + 1) * D].float()) * scale + bias[h][dist]
            out[r, h * D:(h + 1) * D] = torch.softmax(s.masked_fill(~see, -math.inf), 0) @ values[:, h // (H // Hkv)].float()
    return out


PORTIONS = [(0, 1), (0, 300), (37, 150), (209, 3), (210, 130), (511, 2)]


@pytest.mark.parametrize("kernel", ["mma.sync", "general"])
@pytest.mark.parametrize("H,Hkv,D,n_dist", [(4, 2, 64, 203), (6, 1, 48, 17), (2, 2, 96, 1000), (3, 3, 16, 2), (8, 2, 128, 65)])
def test_prompt_portions_with_a_bias_by_distance(kernel, H, Hkv, D, n_dist):
    """The bias decides (it is several units steep, the scores are small): an entry read for the wrong distance, the wrong
    head or past the table's end shows.  Portions start inside pages, tiles and the table's reach."""
    g = torch.Generator().manual_seed(H * 100 + D + n_dist)
    lens = [b + n for b, n in PORTIONS]
    keys = [torch.randn(n, Hkv, D, generator=g).to(torch.bfloat16).to(DEV) for n in lens]
    values = [torch.randn(n, Hkv, D, generator=g).to(torch.bfloat16).to(DEV) for n in lens]
    k_view, v_view, table = _paged(keys, values, 16, seed=D + n_dist)
    T = sum(n for _, n in PORTIONS)
    q = torch.randn(T, H * D, generator=g).to(torch.bfloat16).to(DEV)
    bias = (3.0 * torch.randn(H, n_dist, generator=g)).to(DEV)
    starts = [0]
    for _, n in PORTIONS:
        starts.append(starts[-1] + n)
    q_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
    kv_before = torch.tensor([b for b, _ in PORTIONS], dtype=torch.int32, device=DEV)
    token_seq = torch.cat([torch.full((n,), r, dtype=torch.int32) for r, (_, n) in enumerate(PORTIONS)]).to(DEV)
    positions = torch.cat([torch.arange(b, b + n, dtype=torch.int32) for b, n in PORTIONS]).to(DEV)
    out = torch.zeros_like(q)
    scale = 0.3 / math.sqrt(D)
    if kernel == "general":
        ops.paged_attention(q, k_view, v_view, table, token_seq, positions, out, n_heads=H, scale=scale, dist_bias=bias)
    else:
        ops.prefill_attention(q, k_view, v_view, table, q_start, kv_before, out, n_heads=H, max_q_len=300, scale=scale, tc=False, dist_bias=bias)
    ops.check_kernel_status(torch.device(DEV))
    for r, (b, n) in enumerate(PORTIONS):
        want = _want_rows(q[starts[r]:starts[r + 1]], keys[r], values[r], list(range(b, b + n)), H, scale, bias)
        err = (out[starts[r]:starts[r + 1]].float() - want).abs().max().item()
        assert err < 0.03, f"{kernel}: portion {r} differs by {err}"


@pytest.mark.parametrize("H,Hkv,D,n_dist,splits", [(4, 2, 64, 203, 1), (6, 1, 48, 17, 3), (20, 1, 128, 300, 4), (3, 3, 16, 2, 2), (40, 2, 96, 1000, 7)])
def test_single_tokens_with_a_bias_by_distance(H, Hkv, D, n_dist, splits):
    """The decode kernel with heads as rows: a row's head picks the table's row (heads beyond a tile's sixteen, groups of
    fewer), splits that start anywhere."""
    g = torch.Generator().manual_seed(H + D + n_dist)
    lens = [1, 5, 33, 260, 700]
    keys = [torch.randn(n, Hkv, D, generator=g).to(torch.bfloat16).to(DEV) for n in lens]
    values = [torch.randn(n, Hkv, D, generator=g).to(torch.bfloat16).to(DEV) for n in lens]
    k_view, v_view, table = _paged(keys, values, 16, seed=D)
    q = torch.randn(len(lens), H * D, generator=g).to(torch.bfloat16).to(DEV)
    bias = (3.0 * torch.randn(H, n_dist, generator=g)).to(DEV)
    token_seq = torch.arange(len(lens), dtype=torch.int32, device=DEV)
    positions = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    scale = 0.3 / math.sqrt(D)
    out = torch.zeros_like(q)
    ops.decode_attention_shared(q, k_view, v_view, table, token_seq, positions, out, n_heads=H, scale=scale, splits=splits, dist_bias=bias)
    ops.check_kernel_status(torch.device(DEV))
    general = torch.zeros_like(q)
    ops.paged_attention(q, k_view, v_view, table, token_seq, positions, general, n_heads=H, scale=scale, dist_bias=bias)
    for r, n in enumerate(lens):
        want = _want_rows(q[r:r + 1], keys[r], values[r], [n - 1], H, scale, bias)
        assert (out[r:r + 1].float() - want).abs().max().item() < 0.03, f"heads as rows: request {r}"
        assert (general[r:r + 1].float() - want).abs().max().item() < 0.03, f"general kernel: request {r}"


# ---- one pass over the streams -----------------------------------------------------------------------------------
def _layer_norm(u, gain, eps):
    d = u - u.mean(-1, keepdim=True)
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * gain


@pytest.mark.parametrize("T", [37, 300])
@pytest.mark.parametrize("S,W", [(1, 48), (2, 328), (3, 100), (4, 1024), (8, 64), (2, 2500), (5, 1536), (8, 900), (4, 2048)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_pass_over_the_streams(S, W, dtype, T):
    """Write, sum and read in one launch and each alone; widths that keep the streams in registers and widths beyond; few
    tokens (a row over 1,024 threads) and many (256 threads)."""
    g = torch.Generator().manual_seed(S * 1000 + W)
    X0 = torch.randn(T, S * W, generator=g).to(DEV)
    y, gate = torch.randn(T, W, generator=g).to(DEV), torch.randn(T, W, generator=g).to(DEV)
    gate_bias, gain = torch.randn(W, generator=g).to(DEV), (1 + 0.2 * torch.randn(W, generator=g)).to(DEV)
    mix = (torch.eye(S) + 0.3 * torch.randn(S, S, generator=g)).to(DEV)
    out_w, in_w = torch.randn(S, generator=g).to(DEV), torch.randn(S, generator=g).to(DEV)
    Xs = X0.view(T, S, W).double()
    branch = y.double() * torch.sigmoid(gate.double() + gate_bias.double())
    X1 = torch.einsum("st,nsw->ntw", mix.double(), Xs) + out_w.double()[None, :, None] * branch[:, None, :]
    want_h = _layer_norm(torch.einsum("s,nsw->nw", in_w.double(), X1), gain.double(), 1e-5)
    X = X0.clone()
    h = torch.zeros(T, W, dtype=dtype, device=DEV)
    total = torch.zeros(T, W, device=DEV)
    ops.streams_step(X, S, y=y, gate=gate, gate_bias=gate_bias, mix=mix, out_w=out_w, in_w=in_w, gain=gain, eps=1e-5, h=h, sum_out=total)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert (X.view(T, S, W).double() - X1).abs().max().item() < 1e-4
    assert (total.double() - X1.sum(1)).abs().max().item() < 1e-4
    assert (h.double() - want_h).abs().max().item() < tol * max(1.0, want_h.abs().max().item())
    # the read alone leaves the streams as they are
    X = X0.clone()
    ops.streams_step(X, S, in_w=in_w, gain=gain, eps=1e-5, h=h)
    assert torch.equal(X, X0)
    want0 = _layer_norm(torch.einsum("s,nsw->nw", in_w.double(), Xs), gain.double(), 1e-5)
    assert (h.double() - want0).abs().max().item() < tol * max(1.0, want0.abs().max().item())


@pytest.mark.parametrize("S,W,taps", [(2, 40, 3), (4, 1536, 4), (3, 1000, 1), (8, 300, 8), (1, 2100, 2)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_convolution_inside_the_pass_in_steps_of_single_tokens(S, W, taps, dtype):
    """Five steps of one token for each of three requests: the pass that reads the streams also runs the convolution and
    moves the tails on; the same rows through the convolution's own kernel and conv_tail are the measure."""
    g = torch.Generator().manual_seed(S + W + taps)
    off = 5
    slots = torch.tensor([3, 0, 1], dtype=torch.int32, device=DEV)
    token_seq = torch.arange(3, dtype=torch.int32, device=DEV)
    q_start = torch.arange(4, dtype=torch.int32, device=DEV)
    w = torch.randn(W, taps, generator=g).to(DEV)
    in_w, gain = torch.randn(S, generator=g).to(DEV), (1 + 0.2 * torch.randn(W, generator=g)).to(DEV)
    state_a = torch.zeros(4, off + (taps - 1) * W + 3, device=DEV)
    state_b = state_a.clone()
    for step in range(5):
        X = torch.randn(3, S * W, generator=g).to(DEV)
        h_a, c_a = torch.zeros(3, W, dtype=dtype, device=DEV), torch.zeros(3, W, dtype=dtype, device=DEV)
        ops.streams_step(X.clone(), S, in_w=in_w, gain=gain, eps=1e-5, h=h_a, taps=w, state=state_a, tail_off=off, token_seq=token_seq,
                         seq_slots=slots, conv_out=c_a)
        h_b, c_b = torch.zeros_like(h_a), torch.zeros_like(c_a)
        ops.streams_step(X.clone(), S, in_w=in_w, gain=gain, eps=1e-5, h=h_b)
        ops.canon_conv(h_b, w, state_b, off, token_seq, q_start, slots, c_b)
        if taps > 1:
            ops.conv_tail(h_b, taps, state_b, off, q_start, slots)
        assert torch.equal(h_a, h_b), f"step {step}"
        tol = 1e-5 if dtype == torch.float32 else 0.07
        assert (c_a.float() - c_b.float()).abs().max().item() < tol * max(1.0, c_b.float().abs().max().item()), f"step {step}"
        assert torch.equal(state_a, state_b), f"step {step}: the tails differ"
    assert state_a[2].abs().max().item() == 0.0 and (taps == 1 or state_a[3, off:].abs().max().item() > 0.0)


@pytest.mark.parametrize("taps", [1, 2, 3, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_short_convolution_and_its_tail(taps, dtype):
    """Three requests in one step (a long portion, two tokens, one token) with tails from the step before at an offset in
    their slots; then the tails after the step, and a second step that reads them."""
    g = torch.Generator().manual_seed(taps)
    W, off = 40, 7
    lens1, lens2 = [19, 2, 1], [1, 5, 3]
    slots = torch.tensor([2, 0, 3], dtype=torch.int32, device=DEV)
    w = torch.randn(W, taps, generator=g).to(DEV)
    rows = [torch.randn(a + b, W, generator=g).to(dtype).to(DEV) for a, b in zip(lens1, lens2)]
    state = torch.zeros(4, off + (taps - 1) * W + 5, device=DEV)
    got = [[], [], []]
    for step, lens in enumerate((lens1, lens2)):
        begin = [0, 0, 0] if step == 0 else lens1
        h = torch.cat([rows[r][begin[r]:begin[r] + n] for r, n in enumerate(lens)])
        starts = [0]
        for n in lens:
            starts.append(starts[-1] + n)
        q_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
        token_seq = torch.cat([torch.full((n,), r, dtype=torch.int32) for r, n in enumerate(lens)]).to(DEV)
        out = torch.zeros_like(h)
        ops.canon_conv(h, w, state, off, token_seq, q_start, slots, out)
        if taps > 1:
            ops.conv_tail(h, taps, state, off, q_start, slots)
        for r in range(3):
            got[r].append(out[starts[r]:starts[r + 1]])
    for r in range(3):
        x = rows[r].double()
        want = x.clone()
        for j in range(taps):
            back = taps - 1 - j
            if back < x.shape[0]:
                want[back:] += x[:x.shape[0] - back] * w[:, j].double()
        err = (torch.cat(got[r]).double() - want).abs().max().item()
        assert err < (1e-5 if dtype == torch.float32 else 0.06), f"request {r}: {err}"
    assert state[1].abs().max().item() == 0.0 and state[:, :off].abs().max().item() == 0.0      # no other slot, nothing before the tail


def test_the_embedding_with_its_pair_table():
    """Two steps: portions whose first tokens read the state (or, at position 0, the table's last row), then single tokens
    that keep themselves; multipliers whose products pass 2^31."""
    g = torch.Generator().manual_seed(3)
    V, W, buckets, a, b = 50000, 24, 1021, 2000003, 65537
    wte, big, pos = torch.randn(V, W, generator=g).to(DEV), torch.randn(buckets + 1, W, generator=g).to(DEV), torch.randn(64, W, generator=g).to(DEV)
    seqs = [torch.randint(0, V, (n,), generator=g).tolist() for n in (9, 4)]
    slots = torch.tensor([1, 3], dtype=torch.int32, device=DEV)
    state = torch.zeros(4, 2, dtype=torch.int32, device=DEV)
    got = [[], []]
    for cut in ([(0, 5), (0, 2)], [(5, 6), (2, 3)], [(6, 9), (3, 4)]):
        lens = [e - s for s, e in cut]
        ids = torch.tensor(sum((seqs[r][s:e] for r, (s, e) in enumerate(cut)), []), dtype=torch.int32, device=DEV)
        positions = torch.cat([torch.arange(s, e, dtype=torch.int32) for s, e in cut]).to(DEV)
        token_seq = torch.cat([torch.full((n,), r, dtype=torch.int32) for r, n in enumerate(lens)]).to(DEV)
        q_start = torch.tensor([0, lens[0], lens[0] + lens[1]], dtype=torch.int32, device=DEV)
        out = torch.zeros(sum(lens), W, device=DEV)
        ops.embed_bigram(ids, positions, token_seq, q_start, slots, wte, big, pos, state, out, mul_prev=a, mul_cur=b, keep=max(lens) == 1)
        got[0].append(out[:lens[0]])
        got[1].append(out[lens[0]:])
    for r, ids in enumerate(seqs):
        rows = [buckets] + [(ids[t - 1] * a + ids[t] * b) % buckets for t in range(1, len(ids))]
        want = wte[torch.tensor(ids)] + big[torch.tensor(rows)] + pos[:len(ids)]
        assert (torch.cat(got[r]) - want).abs().max().item() < 1e-5
    assert state[1, 0].item() == seqs[0][-1] and state[3, 0].item() == seqs[1][-1] and state[0].abs().sum().item() == 0


# ---- the state-space mixer ----------------------------------------------------------------------------------------
@pytest.mark.parametrize("H,G,N,P,taps", [(4, 2, 16, 8, 3), (5, 5, 40, 12, 1), (2, 1, 128, 64, 4), (3, 1, 200, 40, 2), (8, 2, 48, 48, 4), (1, 1, 7, 70, 8)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_recurrence_in_portions_and_single_tokens(H, G, N, P, taps, dtype):
    """Two requests walk their tokens in unequal portions (one of them token by token, with steps it sits out), states in
    slots at a pitch larger than they need; a plain loop over whole sequences is the measure.  States of 7 to 200 rows
    take every width of the kernel, values of 70 two column blocks with a ragged edge."""
    g = torch.Generator().manual_seed(H * N + P)
    inner, ch = H * P, H * P + 2 * G * N
    lens = [45, 23]
    cuts = [[17, 1, 9, 2, 16], [1] * 23]
    proj = [(0.7 * torch.randn(n, ch, generator=g)).to(dtype).to(DEV) for n in lens]
    dt_raw = [torch.randn(n, H, generator=g).to(DEV) for n in lens]
    w, cb = (0.5 * torch.randn(ch, taps, generator=g)).to(DEV), (0.2 * torch.randn(ch, generator=g)).to(DEV)
    dt_bias, a_log, d_skip = (torch.randn(H, generator=g) - 1.0).to(DEV), torch.log(0.3 + 2 * torch.rand(H, generator=g)).to(DEV), torch.randn(H, generator=g).to(DEV)
    tail_off = H * P * N
    state = torch.zeros(3, tail_off + (taps - 1) * ch + 3, device=DEV)
    slots_all = [2, 0]
    got = [[], []]
    done = [0, 0]
    step = 0
    while done[0] < lens[0] or done[1] < lens[1]:
        who = [r for r in range(2) if done[r] < lens[r] and not (r == 1 and step % 3 == 2)]
        step += 1
        if not who:
            continue
        n_of = {r: (cuts[0][len(got[0])] if r == 0 else 1) for r in who}
        x = torch.cat([proj[r][done[r]:done[r] + n_of[r]] for r in who])
        raw = torch.cat([dt_raw[r][done[r]:done[r] + n_of[r]] for r in who])
        starts = [0]
        for r in who:
            starts.append(starts[-1] + n_of[r])
        q_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
        token_seq = torch.cat([torch.full((n_of[r],), i, dtype=torch.int32) for i, r in enumerate(who)]).to(DEV)
        slots = torch.tensor([slots_all[r] for r in who], dtype=torch.int32, device=DEV)
        T = starts[-1]
        xbc, dta, out = torch.zeros(T, ch, device=DEV), torch.zeros(T, 2 * H, device=DEV), torch.zeros(T, inner, device=DEV)
        single = max(n_of.values()) == 1            # a step of single tokens keeps its tails itself
        ops.ssm_prepare(x, w, cb, raw, dt_bias, a_log, state, tail_off, token_seq, q_start, slots, xbc, dta, keep=single)
        if taps > 1 and not single:
            ops.conv_tail(x, taps, state, tail_off, q_start, slots)
        ops.ssm_scan(xbc, dta, d_skip, state, q_start, slots, out, n_heads=H, n_groups=G, state_dim=N, v_dim=P)
        for i, r in enumerate(who):
            got[r].append(out[starts[i]:starts[i + 1]])
            done[r] += n_of[r]
    group = torch.arange(H) // (H // G)
    for r in range(2):
        x = proj[r].double().cpu()
        conv = torch.zeros_like(x)
        for j in range(taps):
            back = taps - 1 - j
            conv[back:] += x[:x.shape[0] - back] * w[:, j].double().cpu()
        act = conv + cb.double().cpu()
        act = act * torch.sigmoid(act)
        xs, B, C = act[:, :inner].view(-1, H, P), act[:, inner:inner + G * N].view(-1, G, N), act[:, inner + G * N:].view(-1, G, N)
        dt = torch.nn.functional.softplus(dt_raw[r].double().cpu() + dt_bias.double().cpu())
        decay = torch.exp(-torch.exp(a_log.double().cpu()) * dt)
        S = torch.zeros(H, N, P, dtype=torch.float64)
        want = torch.zeros(lens[r], H, P, dtype=torch.float64)
        for t in range(lens[r]):
            S = decay[t][:, None, None] * S + dt[t][:, None, None] * B[t][group][:, :, None] * xs[t][:, None, :]
            want[t] = torch.einsum("hnp,hn->hp", S, C[t][group]) + d_skip.double().cpu()[:, None] * xs[t]
        err = (torch.cat(got[r]).double().cpu() - want.reshape(lens[r], inner)).abs().max().item()
        assert err < 2e-4 * max(1.0, want.abs().max().item()), f"request {r}: {err}"
        left = state[slots_all[r], :tail_off].view(H, P, N).double().cpu()
        assert (left - S.transpose(1, 2)).abs().max().item() < 2e-4 * max(1.0, S.abs().max().item())
    assert state[1].abs().max().item() == 0.0


@pytest.mark.parametrize("cols,groups", [(384, 2), (40, 8), (100, 1), (1536, 3)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_gate_in_front_of_a_norm_in_groups(cols, groups, dtype):
    g = torch.Generator().manual_seed(cols)
    y = torch.randn(9, cols, generator=g).to(DEV)
    z = torch.randn(9, cols + 5, generator=g).to(dtype).to(DEV)[:, 5:]
    gain = (1 + 0.3 * torch.randn(cols, generator=g)).to(DEV)
    out = torch.zeros(9, cols, dtype=dtype, device=DEV)
    ops.gated_group_norm(y, z, gain, out, groups=groups, eps=1e-5)
    v = (y.double() * (z.double() * torch.sigmoid(z.double()))).view(9, groups, cols // groups)
    want = (v / torch.sqrt((v * v).mean(-1, keepdim=True) + 1e-5)).view(9, cols) * gain.double()
    assert (out.double() - want).abs().max().item() < (1e-5 if dtype == torch.float32 else 3e-2)
    # gating after the norm would be another number
    other = (y.double().view(9, groups, -1) / torch.sqrt((y.double().view(9, groups, -1) ** 2).mean(-1, keepdim=True) + 1e-5)).view(9, cols)
    assert ((other * (z.double() * torch.sigmoid(z.double())) * gain.double()) - want).abs().max().item() > 0.1


# ---- routing by softmax scores ------------------------------------------------------------------------------------
@pytest.mark.parametrize("E,top", [(16, 4), (5, 5), (40, 1), (7, 3)])
def test_routing_by_softmax_scores(E, top):
    """The choice is by score plus correction, the weights are the plain scores (they do not sum to one); equal choice
    scores go to the lower expert."""
    g = torch.Generator().manual_seed(E)
    T = 50
    logits = (2 * torch.randn(T, E, generator=g)).to(DEV)
    corr = (0.2 * torch.randn(E, generator=g)).to(DEV)
    logits[3] = 0.0
    r = ops.moe_route_softmax(logits, corr, top)
    s = torch.softmax(logits.double(), -1)
    ranked = (s + corr.double()).sort(dim=-1, descending=True, stable=True)
    chosen = r.expert_of.view(T, top).cpu()
    assert torch.equal(chosen, ranked.indices[:, :top].cpu().to(torch.int32))
    assert (r.weight_of.view(T, top).double().cpu() - s.cpu().gather(1, chosen.long())).abs().max().item() < 1e-6
    if top < E:
        assert (r.weight_of.view(T, top).sum(-1) < 1.0).all()
    start = r.group_start.cpu()
    assert start[0].item() == 0 and start[E].item() == T * top
    assert torch.equal(r.slot_of_entry[r.entry_of_slot.long()].cpu(), torch.arange(T * top, dtype=torch.int32))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_identity_experts_hand_their_input_on(dtype):
    g = torch.Generator().manual_seed(1)
    T, E, real, top, W = 30, 9, 6, 4, 56
    logits = torch.randn(T, E, generator=g).to(DEV)
    r = ops.moe_route_softmax(logits, None, top)
    h = torch.randn(T, W, generator=g).to(dtype).to(DEV)
    rows = torch.randn(T * top, W, generator=g).to(DEV)
    rows[r.group_start[real].item():] = float("nan")            # slots of identity experts are never computed, never read
    y = torch.ones(T, W, device=DEV)
    ops.moe_combine_identity(r, real, h, rows, y, add=True)
    want = torch.ones(T, W, dtype=torch.float64)
    e, wgt, slot = r.expert_of.view(T, top).cpu(), r.weight_of.view(T, top).double().cpu(), r.slot_of_entry.view(T, top).cpu()
    for t in range(T):
        for j in range(top):
            want[t] += wgt[t, j] * (h[t].double().cpu() if e[t, j] >= real else rows[slot[t, j]].double().cpu())
    assert (e >= real).any() and (e < real).any()
    assert (y.double().cpu() - want).abs().max().item() < 1e-5
