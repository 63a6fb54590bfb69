"""The kernels of the state-carrying mixers and of the head-mixing attention, each against the plain
function of the same mechanism (float64 on the CPU), on sizes the tiny models do not reach, cut into
portions, with slots used again, and with inputs made so that one key stands out at a window's edge."""

import math

import pytest
import torch

import plain_vizalix as pv

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def F():
    from mini_infer_b200.ops import functional
    return functional


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def batch_meta(lengths, slots):
    starts = [0]
    for n in lengths:
        starts.append(starts[-1] + n)
    req = [b for b, n in enumerate(lengths) for _ in range(n)]
    return i32(starts), i32(req), i32(slots)


@pytest.mark.parametrize("taps,C,bias,aligned", [(4, 70, False, False), (2, 33, True, False), (1, 8, True, False),
                                                 (8, 300, False, False), (4, 72, True, True), (3, 1024, False, True)])
def test_causal_conv_in_portions_and_batches(taps, C, bias, aligned):
    """``aligned``: rows, columns and state section start on 16-byte boundaries (the four-channel form)."""
    g = torch.Generator().manual_seed(taps * 100 + C)
    lens = [37, 5, 1, 19]
    ld, col0 = (C + 12, 8) if aligned else (C + 11, 7)
    off = 8 if aligned else 5
    xs = [torch.randn(n, ld, generator=g) for n in lens]
    w = torch.randn(C, taps, generator=g)
    b = torch.randn(C, generator=g) if bias else None
    want = [pv.short_conv_silu(x[:, col0:col0 + C].double(), w.double(), None if b is None else b.double()) for x in xs]
    state = torch.zeros(6, off + (taps - 1) * C, device=DEV)
    slots = [4, 0, 2, 5]
    fed = [0] * 4
    got = [torch.zeros(n, C) for n in lens]
    cuts = [[7, 2, 28], [3, 2], [1], [1, 1, 1, 16]]      # portions of every request, fed round robin
    for r in range(4):
        live = [i for i in range(4) if r < len(cuts[i])]
        ns = [cuts[i][r] for i in live]
        x = torch.cat([xs[i][fed[i]:fed[i] + n] for i, n in zip(live, ns)]).to(DEV)
        qs, req, sl = batch_meta(ns, [slots[i] for i in live])
        out = F().causal_conv_silu(x, col0, C, w.to(DEV), None if b is None else b.to(DEV), state, off, qs, req, sl).cpu()
        o = 0
        for i, n in zip(live, ns):
            got[i][fed[i]:fed[i] + n] = out[o:o + n]
            o += n
            fed[i] += n
    for i in range(4):
        assert torch.allclose(got[i].double(), want[i], atol=2e-6), i
        # the state holds the last taps-1 inputs, oldest first
        tail = torch.zeros(taps - 1, C)
        n = min(taps - 1, lens[i])
        if n:
            tail[taps - 1 - n:] = xs[i][lens[i] - n:, col0:col0 + C]
        assert torch.equal(state[slots[i], off:].cpu().view(taps - 1, C), tail)
    assert float(state[:, :off].abs().max()) == 0.0 and float(state[1].abs().max()) == 0.0


def _delta_inputs(T, H, G, d, e, seed):
    g = torch.Generator().manual_seed(seed)
    qkv = torch.randn(T, 2 * G * d + H * e, generator=g)
    beta_raw = torch.randn(T, H + 3, generator=g) * 2
    a_raw = torch.randn(T, H * d + 2, generator=g)
    a_log = torch.randn(H, generator=g) * 0.5 - 1.0
    dt_bias = torch.randn(H * d, generator=g) - 1.0
    return qkv, beta_raw, a_raw, a_log, dt_bias


def _delta_plain(qkv, beta_raw, a_raw, a_log, dt_bias, H, G, d, e):
    T = qkv.shape[0]
    x = qkv.double()
    q, k, v = x[:, :G * d].view(T, G, d), x[:, G * d:2 * G * d].view(T, G, d), x[:, 2 * G * d:].view(T, H, e)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(beta_raw.double()[:, 3:3 + H])
    a = a_raw.double()[:, 2:2 + H * d] + dt_bias.double()
    decay = torch.exp(-torch.exp(a_log.double())[None, :, None] * pv.softplus(a).view(T, H, d))
    return pv.delta_rule(q, k, v, beta, decay).reshape(T, H * e)


@pytest.mark.parametrize("H,G,d,e", [(4, 2, 8, 16), (2, 1, 72, 40), (1, 1, 130, 33), (3, 3, 64, 64)])
def test_delta_rule_whole_in_portions_and_token_by_token(H, G, d, e):
    T = 90
    ins = _delta_inputs(T, H, G, d, e, H * 7 + d)
    want = _delta_plain(*ins, H, G, d, e)
    qkv, beta_raw, a_raw, a_log, dt_bias = [t.to(DEV) for t in ins]
    size = H * d * e
    for cuts in ([T], [1, 2, 40, 9, 2, 36], [1] * T):
        state = torch.zeros(3, 4 + size, device=DEV)
        outs, lo = [], 0
        for n in cuts:
            qs, _, sl = batch_meta([n], [1])
            outs.append(F().delta_scan(qkv[lo:lo + n].contiguous(), beta_raw[lo:lo + n].contiguous(), 3,
                                       a_raw[lo:lo + n].contiguous(), 2, a_log, dt_bias, state, 4, qs, sl, H, G, d, e,
                                       d ** -0.5))
            lo += n
        got = torch.cat(outs).cpu().double()
        assert float((got - want).abs().max()) <= 3e-5 * float(want.abs().max()), cuts[:3]
        assert float(state[0].abs().max()) == 0.0 and float(state[1, :4].abs().max()) == 0.0
        if cuts == [T]:
            first = got
        else:
            assert torch.equal(got, first)      # the cut changes no bit


def test_delta_rule_keeps_a_far_write():
    """A value written at the first token with no decay is read back hundreds of tokens later by the
    query that matches its key, among writes to other keys."""
    H = G = 1
    d, e, T = 16, 8, 400
    qkv = torch.zeros(T, 2 * d + e)
    g = torch.Generator().manual_seed(1)
    for t in range(T):
        qkv[t, d + 1 + t % (d - 1)] = 1.0                       # keys along other axes
        qkv[t, 2 * d:] = torch.randn(e, generator=g)
    qkv[0, d:2 * d] = 0.0
    qkv[0, d] = 1.0                                             # the first token writes along axis 0
    qkv[:, 0] = 1.0                                             # every query reads axis 0
    beta_raw = torch.full((T, 1), 30.0)                         # write strength 1
    a_raw = torch.full((T, d), -40.0)                           # decay 1
    ins = (qkv, beta_raw, a_raw, torch.zeros(1), torch.zeros(d))
    state = torch.zeros(1, d * e, device=DEV)
    qs, _, sl = batch_meta([T], [0])
    got = F().delta_scan(qkv.to(DEV), beta_raw.to(DEV), 0, a_raw.to(DEV), 0, torch.zeros(1, device=DEV),
                         torch.zeros(d, device=DEV), state, 0, qs, sl, 1, 1, d, e, d ** -0.5).cpu()
    assert torch.allclose(got[-1], qkv[0, 2 * d:] * d ** -0.5, atol=1e-5)
    want = _delta_plain_no_offsets(ins, d, e)
    assert torch.allclose(got.double(), want, atol=1e-5)


def _delta_plain_no_offsets(ins, d, e):
    qkv, beta_raw, a_raw, a_log, dt_bias = ins
    T = qkv.shape[0]
    b = torch.cat([torch.zeros(T, 3), beta_raw], 1)
    a = torch.cat([torch.zeros(T, 2), a_raw], 1)
    return _delta_plain(qkv, b, a, a_log, dt_bias, 1, 1, d, e)


@pytest.mark.parametrize("H,G,N,P", [(4, 2, 12, 8), (6, 1, 70, 36), (1, 1, 130, 64), (8, 4, 16, 33)])
def test_state_space_scan_whole_in_portions_and_batched(H, G, N, P):
    lens = [50, 13, 2]
    g = torch.Generator().manual_seed(N + P)
    seqs = [torch.randn(n, H * P + 2 * G * N, generator=g) for n in lens]
    dts = [torch.randn(n, H + 5, generator=g) for n in lens]
    dt_bias, a_log, dsk = torch.randn(H, generator=g) * 0.5, torch.randn(H, generator=g) * 0.5, torch.randn(H, generator=g)
    want = []
    for x, dt in zip(seqs, dts):
        n = x.shape[0]
        xd = x.double()
        want.append(pv.state_space_scan(xd[:, :H * P].reshape(n, H, P), xd[:, H * P:H * P + G * N].reshape(n, G, N),
                                        xd[:, H * P + G * N:].reshape(n, G, N),
                                        pv.softplus(dt.double()[:, 5:] + dt_bias.double()), torch.exp(a_log.double()),
                                        dsk.double()).reshape(n, H * P))
    size = H * N * P
    state = torch.zeros(4, size + 2, device=DEV)
    slots = [3, 1, 0]
    got = [[] for _ in lens]
    fed = [0, 0, 0]
    # steps: all three together in unequal portions, then what is left of each one by one
    plan = [[20, 13, 1], [2, 0, 1], [28, 0, 0]]
    for step in plan:
        live = [i for i in range(3) if step[i]]
        x = torch.cat([seqs[i][fed[i]:fed[i] + step[i]] for i in live]).to(DEV)
        dt = torch.cat([dts[i][fed[i]:fed[i] + step[i]] for i in live]).to(DEV)
        qs, _, sl = batch_meta([step[i] for i in live], [slots[i] for i in live])
        out = F().ssd_scan(x, dt, 5, dt_bias.to(DEV), a_log.to(DEV), dsk.to(DEV), state, 0, qs, sl, H, G, N, P).cpu()
        o = 0
        for i in live:
            got[i].append(out[o:o + step[i]])
            o += step[i]
            fed[i] += step[i]
    for i in range(3):
        g_i = torch.cat(got[i]).double()
        assert float((g_i - want[i]).abs().max()) <= 3e-5 * float(want[i].abs().max()), i
    assert float(state[2].abs().max()) == 0.0 and float(state[:, size:].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_group_norm_both_orders(dtype):
    g = torch.Generator().manual_seed(0)
    T, n = 9, 96
    y, gate = torch.randn(T, n, generator=g) * 3, torch.randn(T, n + 10, generator=g)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    # the gate first, groups of a third of the row, a weight per column
    w = torch.randn(n, generator=g)
    got = F().gated_group_rmsnorm(y.to(DEV), gate.to(DEV), 4, w.to(DEV), 3, True, 1e-5, dtype).float().cpu()
    z = y.double() * pv.silu(gate.double()[:, 4:4 + n])
    want = (pv.unit_rms(z.view(T, 3, n // 3), 1e-5).reshape(T, n) * w.double())
    assert float((got.double() - want).abs().max()) <= tol * float(want.abs().max())
    # the gate last, one group per head, one weight for all heads
    w = torch.randn(24, generator=g)
    got = F().gated_group_rmsnorm(y.to(DEV), gate.to(DEV), 10, w.to(DEV), 4, False, 1e-6, dtype).float().cpu()
    want = (pv.unit_rms(y.double().view(T, 4, 24), 1e-6) * w.double()).reshape(T, n) * torch.sigmoid(gate.double()[:, 10:])
    assert float((got.double() - want).abs().max()) <= tol * float(want.abs().max())


def test_two_scalar_norms_in_one_kernel_and_the_row_forms():
    g = torch.Generator().manual_seed(0)
    T, H = 7, 50
    hidden, a, b = (torch.randn(T, H, generator=g) for _ in range(3))
    g1, g2 = torch.tensor([1.3]), torch.tensor([-0.7])
    h = hidden.clone().to(DEV)
    o1, o2 = F().add2_rmsnorm_scalar(h, a.to(DEV), b.to(DEV), g1.to(DEV), g2.to(DEV), 1e-5, torch.float32)
    s = (hidden + a + b).double()
    assert torch.allclose(h.cpu().double(), s, atol=1e-6)
    assert torch.allclose(o1.cpu().double(), pv.scalar_norm(s, 1.3, 1e-5), atol=1e-5)
    assert torch.allclose(o2.cpu().double(), pv.scalar_norm(s, -0.7, 1e-5), atol=1e-5)
    rows = i32([5, 0, 5])
    h2 = hidden.clone().to(DEV)
    o, none = F().add2_rmsnorm_scalar(h2, a.to(DEV), None, g1.to(DEV), None, 1e-5, torch.float32, rows)
    assert none is None and torch.equal(h2.cpu(), hidden)
    assert torch.allclose(o.cpu().double(), pv.scalar_norm((hidden + a).double()[[5, 0, 5]], 1.3, 1e-5), atol=1e-5)
    gu = torch.randn(T, 2 * 30, generator=g) * 3
    got = F().geglu_tanh(gu.to(DEV)).cpu().double()
    assert torch.allclose(got, pv.gelu_tanh(gu.double()[:, :30]) * gu.double()[:, 30:], atol=1e-5)
    cat = F().concat_cast(hidden.to(DEV), a.to(DEV), b.to(DEV), a.to(DEV), torch.float32).cpu()
    assert torch.allclose(cat, torch.cat([hidden + a + b, a], 1), atol=1e-6)
    vec = torch.randn(H, generator=g).to(torch.bfloat16)
    out = F().rows_plus_vec(torch.zeros(T, H, device=DEV), b.to(DEV), vec.to(DEV)).cpu()
    assert torch.equal(out, b + vec.float())


# --------------------------------------------------------------------------- #
# attention
# --------------------------------------------------------------------------- #

def paged(k, v, page_size, num_pages, seed, dtype):
    """Scatter ``k [T, G, d]`` and ``v [T, G, e]`` over pages in a shuffled order."""
    T, G, d = k.shape
    e = v.shape[2]
    n = -(-T // page_size)
    order = torch.randperm(num_pages, generator=torch.Generator().manual_seed(seed))[:n].tolist()
    kc = torch.full((num_pages, G, page_size, d), 99.0)
    vc = torch.full((num_pages, G, page_size, e), 99.0)
    for t in range(T):
        kc[order[t // page_size], :, t % page_size] = k[t]
        vc[order[t // page_size], :, t % page_size] = v[t]
    return kc.to(dtype).to(DEV), vc.to(dtype).to(DEV), order


def run_attention(q, k, v, talk, window, scale, cap, cuts, dtype=torch.float32, page_size=8):
    """The kernel over a hand-made paged cache, the sequence's queries cut into steps ``cuts``."""
    T, H, d = q.shape
    kc, vc, order = paged(k, v, page_size, 2 * (-(-T // page_size)) + 3, 5, dtype)
    table = i32([order + [-1] * 4])
    outs, lo = [], 0
    for n in cuts:
        got = F().attention_mix(q[lo:lo + n].to(dtype).to(DEV).contiguous(), kc, vc,
                                None if talk is None else talk.float().to(DEV), table, i32([0, n]), i32([lo + n]), n,
                                window, scale, cap or 0.0)
        outs.append(got.float().cpu())
        lo += n
    return torch.cat(outs)


@pytest.mark.parametrize("H,G,d,e,window", [(4, 2, 16, 8, 9), (6, 3, 24, 40, 64), (1, 1, 20, 96, 1), (5, 1, 8, 8, 17),
                                            (16, 4, 64, 128, 40), (3, 3, 130, 200, 23)])
def test_attention_against_plain_in_any_cut(H, G, d, e, window):
    T = 75
    g = torch.Generator().manual_seed(H * 10 + d)
    q, k, v = torch.randn(T, H, d, generator=g), torch.randn(T, G, d, generator=g), torch.randn(T, G, e, generator=g)
    talk = torch.eye(H) + 0.3 * torch.randn(H, H, generator=g)
    want = pv.mixed_head_attention(q.double(), k.double(), v.double(), 0.2, 4.0, talk.double(), window)
    whole = run_attention(q, k, v, talk, window, 0.2, 4.0, [T])
    assert float((whole.double() - want).abs().max()) <= 2e-5 * float(want.abs().max())
    for cuts in ([1] * T, [3, 2, 17, 1, 1, 33, 2, 16]):
        assert torch.equal(run_attention(q, k, v, talk, window, 0.2, 4.0, cuts), whole)      # no bit moves
    # without cap and mix it is ordinary windowed attention
    want = pv.mixed_head_attention(q.double(), k.double(), v.double(), 0.2, None, None, window)
    got = run_attention(q, k, v, None, window, 0.2, None, [40, 35])
    assert float((got.double() - want).abs().max()) <= 2e-5 * float(want.abs().max())
    # bfloat16 storage
    qb, kb, vb = (t.to(torch.bfloat16).float() for t in (q, k, v))
    want = pv.mixed_head_attention(qb.double(), kb.double(), vb.double(), 0.2, 4.0, talk.double(), window)
    got = run_attention(qb, kb, vb, talk, window, 0.2, 4.0, [T - 1, 1], torch.bfloat16)
    assert float((got.double() - want).abs().max()) <= 1e-2 * float(want.abs().max())


@pytest.mark.parametrize("window", [1, 2, 8, 9, 31, 32, 33, 64, 200])
@pytest.mark.parametrize("decoded", [False, True])
def test_a_key_that_stands_out_at_the_edge_of_the_window(window, decoded):
    """One key matches the last query a thousand times better than all others.  Just inside the window the
    output is its value; just outside it plays no part.  The same in a prompt's portion and decoded alone,
    with keys at page and tile borders."""
    T, H, G, d, e = 260, 2, 1, 8, 4
    g = torch.Generator().manual_seed(window)
    v = torch.randn(T, G, e, generator=g)
    for dist, seen in ((window - 1, True), (window, False)):
        if dist >= T:
            continue
        q = torch.zeros(T, H, d)
        k = torch.randn(T, G, d, generator=g) * 0.01
        q[-1, :, 0] = 40.0
        k[T - 1 - dist, 0, 0] = 1.0
        cuts = [T - 1, 1] if decoded else [T - 5, 5]
        got = run_attention(q, k, v, None, window, 1.0, None, cuts)[-1]
        hit = torch.allclose(got, v[T - 1 - dist, 0].expand(H, e), atol=1e-4)
        assert hit == seen, (window, dist, decoded)
        want = pv.mixed_head_attention(q.double(), k.double(), v.double(), 1.0, None, None, window)[-1]
        assert torch.allclose(got.double(), want, atol=1e-5)


def test_a_far_key_among_hundreds_without_a_window():
    T, H, G, d, e = 700, 4, 2, 16, 16
    g = torch.Generator().manual_seed(3)
    q, k, v = torch.zeros(T, H, d), torch.randn(T, G, d, generator=g) * 0.01, torch.randn(T, G, e, generator=g)
    q[-1, :, 3] = 50.0
    k[2, :, 3] = 1.0
    got = run_attention(q, k, v, None, 0, 1.0, None, [T - 1, 1], page_size=16)[-1]
    assert torch.allclose(got, v[2].repeat_interleave(2, 0), atol=1e-4)


def test_the_mix_couples_heads_of_different_key_value_heads():
    """With a mix that swaps two heads the output of each is the other's attention pattern over its own
    values."""
    T, H, G, d, e = 20, 2, 2, 8, 4
    g = torch.Generator().manual_seed(4)
    q, k, v = torch.randn(T, H, d, generator=g), torch.randn(T, G, d, generator=g), torch.randn(T, G, e, generator=g)
    swap = torch.tensor([[0.0, 1.0], [1.0, 0.0]])
    got = run_attention(q, k, v, swap, 50, 0.5, 3.0, [T])
    want = pv.mixed_head_attention(q.double(), k.double(), v.double(), 0.5, 3.0, swap.double(), 50)
    assert float((got.double() - want).abs().max()) <= 1e-5
    plain = pv.mixed_head_attention(q.double(), k.double(), v.double(), 0.5, 3.0, None, 50)
    assert float((want - plain).abs().max()) > 1e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rotation_and_cache_write(dtype):
    from mini_infer_b200.config import part_class
    T, nh, nkv, dk, dv, ps = 11, 3, 1, 12, 20, 4
    rot = {"base": 100.0, "dims": 8, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 16}}
    g = torch.Generator().manual_seed(0)
    qkv = torch.randn(T, (nh + nkv) * dk + nkv * dv, generator=g)
    positions = torch.arange(100, 100 + T)
    table = part_class("position", "rope_scaled")({"head_dim": dk, "rot_dim": 8, "theta": 100.0, **rot["scaling"]}, "").table(DEV)
    kc = torch.zeros(9, nkv, ps, dk, dtype=dtype, device=DEV)
    vc = torch.zeros(9, nkv, ps, dv, dtype=dtype, device=DEV)
    slots = [8 + t if t != 4 else -1 for t in range(T)]           # one row is not cached
    q = F().rope_store(qkv.to(DEV), i32(positions.tolist()), table, 8, i32(slots), kc, vc, nh, nkv, dk, dv, ps, dtype)
    x = qkv.double()
    want_q = pv.rotate(x[:, :nh * dk].view(T, nh, dk), positions, rot)
    want_k = pv.rotate(x[:, nh * dk:(nh + nkv) * dk].view(T, nkv, dk), positions, rot)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(q.float().cpu().double(), want_q, atol=tol)
    for t in range(T):
        if slots[t] < 0:
            continue
        page, off = divmod(slots[t], ps)
        assert torch.allclose(kc[page, :, off].float().cpu().double(), want_k[t], atol=tol)
        assert torch.allclose(vc[page, :, off].float().cpu().double(), x[t, (nh + nkv) * dk:].view(nkv, dv), atol=tol)
    assert float(kc[:2].abs().max()) == 0.0 and float(kc[3, :, 0].abs().max()) == 0.0      # slot 12 stayed empty
    assert float(kc[5:].abs().max()) == 0.0 and float(vc[5:].abs().max()) == 0.0


def run_attention_tc(q, k, v, talk, window, scale, cap, cuts, page_size=8):
    """The tensor-core form over a hand-made paged cache; portions of one token go through the split form."""
    T, H, d = q.shape
    e = v.shape[2]
    kc, vc, order = paged(k, v, page_size, 2 * (-(-T // page_size)) + 3, 5, torch.bfloat16)
    table = i32([order + [-1] * 4])
    outs, lo = [], 0
    for n in cuts:
        kw = {}
        splits = 1
        if n == 1:
            span = min(window, lo + 1) if window else lo + 1
            splits = F().attention_mix_tc_splits(span)
            kw = dict(splits=splits, part_o=torch.full((splits * H * e,), 7.0, device=DEV),
                      part_ml=torch.full((splits * H * 2,), 7.0, device=DEV))
        got = F().attention_mix_tc(q[lo:lo + n].to(torch.bfloat16).to(DEV).contiguous(), kc, vc,
                                   None if talk is None else talk.float().to(DEV), table, i32([0, n]), i32([lo + n]), n,
                                   window, scale, cap or 0.0, **kw)
        outs.append(got.float().cpu())
        lo += n
    return torch.cat(outs)


@pytest.mark.parametrize("H,G,d,e,window", [(16, 4, 64, 128, 40), (8, 2, 128, 128, 300), (4, 2, 16, 64, 9), (24, 8, 32, 64, 64),
                                            (5, 1, 48, 64, 17), (3, 3, 16, 128, 0),
                                            # more heads than one block finishes: two and three blocks share a query tile
                                            (24, 8, 128, 128, 150), (40, 8, 32, 64, 33), (18, 3, 16, 128, 70)])
def test_attention_on_the_tensor_cores(H, G, d, e, window):
    assert F().attention_mix_tc_supported(H, G, d, e)
    assert not F().attention_mix_tc_supported(4, 2, 20, 64) and not F().attention_mix_tc_supported(4, 2, 32, 96)
    T = 330
    g = torch.Generator().manual_seed(H + d)
    q, k, v = (torch.randn(T, n, s, generator=g).to(torch.bfloat16).float() for n, s in ((H, d), (G, d), (G, e)))
    talk = torch.eye(H) + 0.3 * torch.randn(H, H, generator=g)
    want = pv.mixed_head_attention(q.double(), k.double(), v.double(), d ** -0.5, 6.0, talk.double(), window or T)
    tol = 1.5e-2 * float(want.abs().max())
    for cuts in ([T], [200, 17, 3, 100] + [1] * 10, [310] + [1] * 20):
        got = run_attention_tc(q, k, v, talk, window, d ** -0.5, 6.0, cuts)
        assert float((got.double() - want).abs().max()) <= tol, cuts[:2]
    want = pv.mixed_head_attention(q.double(), k.double(), v.double(), d ** -0.5, None, None, window or T)
    got = run_attention_tc(q, k, v, None, window, d ** -0.5, None, [T - 1, 1])
    assert float((got.double() - want).abs().max()) <= 1.5e-2 * float(want.abs().max())


@pytest.mark.parametrize("window", [1, 15, 16, 17, 128, 129, 257])
@pytest.mark.parametrize("decoded", [False, True])
def test_the_edge_of_the_window_on_the_tensor_cores(window, decoded):
    T, H, G, d, e = 300, 4, 2, 16, 64
    g = torch.Generator().manual_seed(window)
    v = torch.randn(T, G, e, generator=g).to(torch.bfloat16).float()
    for dist, seen in ((window - 1, True), (window, False)):
        q = torch.zeros(T, H, d)
        k = (torch.randn(T, G, d, generator=g) * 0.01).to(torch.bfloat16).float()
        q[-1, :, 0] = 40.0
        k[T - 1 - dist, :, 0] = 1.0
        got = run_attention_tc(q, k, v, None, window, 1.0, None, [T - 1, 1] if decoded else [T - 7, 7])[-1]
        hit = torch.allclose(got, v[T - 1 - dist].repeat_interleave(2, 0), atol=2e-2)
        assert hit == seen, (window, dist, decoded)
