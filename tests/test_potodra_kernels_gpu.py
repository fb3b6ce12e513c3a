"""The kernels that came with the Potodra decoder, each alone against float64 torch arithmetic, at sizes of no model."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TYPES = [torch.float32, torch.bfloat16]


def K():
    from exl3_server_b200.ops import kernels
    return kernels


def tol(dt):
    return 2e-5 if dt == torch.float32 else 2e-2


def close(got, want, dt, what=""):
    got, want = got.double().cpu(), want.double().cpu()
    err = float((got - want).abs().max()) / max(1e-30, float(want.abs().max()))
    assert err <= tol(dt), (what, err)


def step_layout(rows):
    """Packed rows of a step: ``rows`` = [(slot, tokens)]."""
    row_start = torch.tensor([0] + list(torch.tensor([n for _, n in rows]).cumsum(0)), dtype=torch.int32)
    slot_ids = torch.tensor([s for s, _ in rows], dtype=torch.int32)
    return row_start.to(DEV), slot_ids.to(DEV)


@pytest.mark.parametrize("y_dt", TYPES)
@pytest.mark.parametrize("r_dt", TYPES)
@pytest.mark.parametrize("S, W", [(1, 96), (2, 100), (3, 37), (5, 1032), (8, 64), (11, 40), (16, 24)])
def test_hyper_step(S, W, y_dt, r_dt):
    g = torch.Generator().manual_seed(S * 1000 + W)
    k_ = K()
    T = 7
    x0 = torch.randn(T, S, W, generator=g)
    y = torch.randn(T, W, generator=g).to(y_dt)
    mix, w_out, w_in = torch.randn(S, S, generator=g), torch.randn(S, generator=g), torch.randn(S, generator=g)
    nw = (1.0 + 0.2 * torch.randn(W, generator=g)).to(r_dt)
    eps = 1e-5
    x = x0.reshape(T, S * W).clone().to(DEV)
    # a write and the read after it
    _, r = k_.hyper_step(x, S, y.to(DEV), mix.to(DEV), w_out.to(DEV), w_in.to(DEV), nw.to(DEV), eps, r_dt)
    new = torch.einsum("st,jsw->jtw", mix.double(), x0.double()) + w_out.double()[None, :, None] * y.double()[:, None, :]
    u = torch.einsum("s,jsw->jw", w_in.double(), new)
    want_r = u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps) * nw.double()
    close(x.reshape(T, S, W), new, torch.float32, "streams after the write")
    close(r, want_r, r_dt, "the read")
    # a write alone leaves the same streams; a read alone, of some rows, reads them
    x2 = x0.reshape(T, S * W).clone().to(DEV)
    assert k_.hyper_step(x2, S, y.to(DEV), mix.to(DEV), w_out.to(DEV), None, None, 0.0, torch.float32)[1] is None
    assert torch.equal(x2, x)
    rows = torch.tensor([5, 0, 6], dtype=torch.int32, device=DEV)
    _, r3 = k_.hyper_step(x2, S, None, None, None, w_in.to(DEV), nw.to(DEV), eps, r_dt, rows=rows)
    close(r3, want_r[[5, 0, 6]], r_dt, "rows")
    assert torch.equal(x2, x)
    # one row per token standing for S equal streams: the read, and the widened streams
    if S == 1:
        return
    one = torch.randn(T, W, generator=g).to(DEV)
    wide = torch.full((T, S * W), 7.0, device=DEV)
    _, r4 = k_.hyper_step(one, S, None, None, None, w_in.to(DEV), None, eps, r_dt, out=wide)
    u = one.double().cpu() * float(w_in.double().sum())
    close(r4, u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps), r_dt, "equal streams")
    assert torch.equal(wide.reshape(T, S, W), one[:, None, :].expand(T, S, W))


@pytest.mark.parametrize("dt", TYPES)
@pytest.mark.parametrize("H, G, d, dv, window, keep, cap, sinks", [
    (4, 2, 24, 16, 50, 5, 9.0, True), (6, 2, 16, 40, 33, 70, 0.0, True), (2, 1, 64, 64, 192, 64, 15.0, False),
    (3, 3, 16, 8, 7, 1, 4.0, True), (2, 2, 40, 40, 300, 130, 0.0, False), (5, 5, 16, 16, 1, 200, 30.0, True),
    (4, 1, 32, 32, 0, 0, 6.0, True)])
def test_attention_with_a_window_that_keeps_the_first_keys(dt, H, G, d, dv, window, keep, cap, sinks):
    """Queries just before and after the window starts to hide keys, at the kept keys' edge, on page borders and at
    chunk borders; pages between the kept keys and the window are not there (-1), as in a cache that gave them back."""
    g = torch.Generator().manual_seed(4)
    k_ = K()
    page, n_pages, width = 64, 40, 12
    lens = [700, 1, 130, 65]
    perm = torch.randperm(n_pages, generator=g)
    bt = torch.full((len(lens), width), -1, dtype=torch.int32)
    at = 0
    for b, n in enumerate(lens):
        need = (n + page - 1) // page
        bt[b, :need] = perm[at:at + need].int()
        at += need
    kp = torch.randn(n_pages, G, page, d, generator=g).to(dt)
    vp = torch.randn(n_pages, G, page, dv, generator=g).to(dt)
    queries = [(0, 699), (0, 698), (0, 449), (0, 450), (0, 255), (0, 256), (0, 0), (1, 0), (2, 129), (2, 127), (2, 128),
               (3, 64), (3, 63), (0, window), (0, max(window - 1, 0)), (0, window + keep), (0, max(window + keep - 1, 0)),
               (0, keep), (0, window + 64)]
    queries = [(b, min(p, lens[b] - 1)) for b, p in queries]
    T = len(queries)
    q = torch.randn(T, H * d, generator=g).to(dt)
    tok_seq = torch.tensor([b for b, _ in queries], dtype=torch.int32)
    tok_pos = torch.tensor([p for _, p in queries], dtype=torch.int32)
    sink = (2.0 * torch.rand(H, generator=g) - 0.5) if sinks else None
    scale = 0.9 / math.sqrt(d)
    want = torch.zeros(T, H, dv, dtype=torch.float64)
    for t, (b, p) in enumerate(queries):
        js = torch.tensor([j for j in range(p + 1) if window == 0 or p - j < window or j < keep])
        pg = bt[b, js // page].long()
        kk, vv = kp[pg, :, js % page].double(), vp[pg, :, js % page].double()          # [n, G, *]
        for h in range(H):
            s = kk[:, h // (H // G)] @ q[t, h * d:(h + 1) * d].double() * scale
            if cap:
                s = cap * torch.tanh(s / cap)
            m = float(s.max())
            e = torch.exp(s - m)
            want[t, h] = (e / (e.sum() + (math.exp(float(sink[h]) - m) if sinks else 0.0))) @ vv[:, h // (H // G)]
    # what a cache with this window has given back by the time the longest row's last query runs
    gone = bt.clone()
    if window:
        first = max(0, 699 - window + 1) // page
        gone[0, (keep + page - 1) // page:first] = -1
    late = [t for t, (b, p) in enumerate(queries) if b != 0 or p >= 690]
    for split in (256, 64):
        n = (700 + split - 1) // split
        if window:
            n = min(n, (window + split - 2) // split + 1 + (keep + split - 1) // split)
        for table, pick in ((bt, list(range(T))), (gone, late)):
            idx = torch.tensor(pick)
            Tn = len(pick)
            scratch = torch.zeros(k_.attn_tokens_scratch_bytes(Tn, H, dv, n) // 4 + 1, device=DEV)
            out = torch.empty(Tn, H * dv, dtype=dt, device=DEV)
            k_.attn_tokens_ex(q[idx].contiguous().to(DEV), H * d, out, kp.to(DEV), vp.to(DEV), table.to(DEV),
                              tok_pos[idx].to(DEV), tok_seq[idx].to(DEV), Tn, H, G, d, dv, page, window, 0, sinks, scale,
                              split, n, scratch if n > 1 else None, keep_first=keep, softcap=cap,
                              sink_vals=sink.to(DEV) if sinks else None)
            close(out.reshape(Tn, H, dv), want[idx], dt, f"split {split}, {Tn} tokens")
    # two tokens: the merge inside the attention kernel
    scratch = torch.zeros(k_.attn_tokens_scratch_bytes(2, H, dv, n) // 4 + 1, device=DEV)
    out = torch.empty(2, H * dv, dtype=dt, device=DEV)
    k_.attn_tokens_ex(q[:2].to(DEV), H * d, out, kp.to(DEV), vp.to(DEV), gone.to(DEV), tok_pos[:2].to(DEV), tok_seq[:2].to(DEV), 2,
                      H, G, d, dv, page, window, 0, sinks, scale, 64, n, scratch if n > 1 else None, keep_first=keep,
                      softcap=cap, sink_vals=sink.to(DEV) if sinks else None)
    close(out.reshape(2, H, dv), want[:2], dt, "two tokens")


@pytest.mark.parametrize("dt", TYPES)
@pytest.mark.parametrize("H, dk, dv, cap", [(3, 16, 24, 8.0), (1, 8, 40, 20.0), (2, 12, 20, 3.0), (2, 128, 64, 12.0),
                                            (2, 64, 130, 15.0), (1, 200, 8, 5.0)])
@pytest.mark.parametrize("lens", [[5, 1, 9], [150, 3, 64], [600, 2, 257]])
def test_mlstm_scan(dt, H, dk, dv, cap, lens):
    """Rows of few tokens walk in order; with a row of 256 tokens or more the step runs as pieces of 64 tokens side by
    side (the long rows in ten and five pieces, the short one in one)."""
    g = torch.Generator().manual_seed(6)
    k_ = K()
    slots = [4, 0, 6][:len(lens)]
    row_start, slot_ids = step_layout(list(zip(slots, lens)))
    T = sum(lens)
    proj = torch.randn(T, 2 * H * dk + H * dv + 8, generator=g).to(dt)
    q, k, v = proj[:, :H * dk], proj[:, H * dk:2 * H * dk], proj[:, 2 * H * dk + 8:]
    z = (3.0 * torch.randn(T, 2 * H, generator=g))
    S0, n0, m0 = torch.randn(9, H, dk, dv, generator=g), torch.randn(9, H, dk, generator=g), torch.rand(9, H, generator=g)
    S, n, m = S0.transpose(2, 3).contiguous().to(DEV), n0.clone().to(DEV), m0.clone().to(DEV)     # the kernel keeps S column by column
    pd, zd = proj.to(DEV), z.to(DEV)
    need = k_.mlstm_scan_scratch_bytes(len(lens), T, H, dk, dv, max(lens))
    assert (need > 0) == (max(lens) >= 256)
    scratch = torch.full((need // 4 + 4,), float("nan"), device=DEV)[:need // 4] if need else None
    out = k_.mlstm_scan(pd[:, :H * dk], pd[:, H * dk:2 * H * dk], pd[:, 2 * H * dk + 8:], zd[:, :H], zd[:, H:], cap,
                        dk ** -0.5, S, n, m, slot_ids, row_start, len(lens), H, dk, dv, max(lens), scratch=scratch)
    want = torch.zeros(T, H, dv, dtype=torch.float64)
    Sa, na, ma = S0.double().clone(), n0.double().clone(), m0.double().clone()
    qd, kd, vd = (q.double() * dk ** -0.5).reshape(T, H, dk), k.double().reshape(T, H, dk), v.double().reshape(T, H, dv)
    gi = cap * torch.tanh(z[:, :H].double() / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh(z[:, H:].double() / cap))
    t = 0
    for slot, cnt in zip(slots, lens):
        for _ in range(cnt):
            for hd in range(H):
                mn = torch.maximum(gf[t, hd] + ma[slot, hd], gi[t, hd])
                a, b = torch.exp(gf[t, hd] + ma[slot, hd] - mn), torch.exp(gi[t, hd] - mn)
                Sa[slot, hd] = a * Sa[slot, hd] + b * torch.outer(kd[t, hd], vd[t, hd])
                na[slot, hd] = a * na[slot, hd] + b * kd[t, hd]
                ma[slot, hd] = mn
                den = torch.maximum(torch.abs(na[slot, hd] @ qd[t, hd]), torch.exp(-mn)) + 1e-6
                want[t, hd] = Sa[slot, hd].T @ qd[t, hd] / den
            t += 1
    # a division by a normaliser near its floor multiplies rounding: compare where it is not tiny against the largest
    close(out.reshape(T, H, dv), want, torch.float32 if dt == torch.float32 else dt, "outputs")
    close(S.transpose(2, 3), Sa, torch.float32, "matrix states, also of the slots that no row has")
    close(n, na, torch.float32, "normalisers")
    close(m, ma, torch.float32, "maxima")


@pytest.mark.parametrize("dt", TYPES)
@pytest.mark.parametrize("H, G, dk, dv", [(3, 1, 16, 8), (2, 2, 24, 16), (4, 2, 20, 12), (2, 1, 128, 32), (2, 2, 64, 130),
                                          (1, 1, 12, 20)])
@pytest.mark.parametrize("lens", [[5, 1, 9], [150, 3, 64], [600, 2, 257]])
def test_delta_scan(dt, H, G, dk, dv, lens):
    """Rows of few tokens walk in order; with a row of 256 tokens or more the step runs as pieces of 64 tokens side by
    side, joined through the pieces' matrices."""
    g = torch.Generator().manual_seed(8)
    k_ = K()
    slots = [4, 0, 6][:len(lens)]
    row_start, slot_ids = step_layout(list(zip(slots, lens)))
    T = sum(lens)
    q = torch.nn.functional.normalize(torch.randn(T, G, dk, generator=g), dim=-1).reshape(T, G * dk) * dk ** -0.5
    k = torch.nn.functional.normalize(torch.randn(T, G, dk, generator=g), dim=-1).reshape(T, G * dk)
    v = torch.randn(T, H * dv, generator=g)
    zb = (2.0 * torch.randn(T, H + 3, generator=g)).to(dt)
    za = torch.randn(T, H * dk + 5, generator=g).to(dt)
    a_log, dt_bias = torch.log(0.05 + 1.5 * torch.rand(H, generator=g)), 2.0 * torch.rand(H * dk, generator=g) - 2.0
    S0 = torch.randn(9, H, dk, dv, generator=g)
    S = S0.transpose(2, 3).contiguous().to(DEV)           # the kernel keeps S column by column
    qkv = torch.cat([q, k, v], dim=1).to(DEV)
    need = k_.delta_scan_scratch_bytes(len(lens), T, H, dk, dv, max(lens))
    assert (need > 0) == (max(lens) >= 256)          # these sizes are few blocks in order: long rows run as pieces
    assert k_.delta_scan_scratch_bytes(8, 8 * 300, 16, 64, 128, 300) == 0      # many blocks in order: no pieces
    scratch = torch.full((need // 4 + 4,), float("nan"), device=DEV)[:need // 4] if need else None
    out = k_.delta_scan(qkv[:, :G * dk], qkv[:, G * dk:2 * G * dk], qkv[:, 2 * G * dk:], zb.to(DEV)[:, 2:2 + H],
                        za.to(DEV)[:, :H * dk], a_log.to(DEV), dt_bias.to(DEV), S, slot_ids, row_start, len(lens), H, G, dk, dv,
                        max(lens), scratch=scratch)
    want = torch.zeros(T, H, dv, dtype=torch.float64)
    Sa = S0.double().clone()
    qd, kd, vd = q.double().reshape(T, G, dk), k.double().reshape(T, G, dk), v.double().reshape(T, H, dv)
    beta = torch.sigmoid(zb[:, 2:2 + H].double())
    step = torch.nn.functional.softplus(za[:, :H * dk].double() + dt_bias.double()).reshape(T, H, dk)
    decay = torch.exp(-torch.exp(a_log.double())[None, :, None] * step)
    t = 0
    for slot, cnt in zip(slots, lens):
        for _ in range(cnt):
            for hd in range(H):
                gq = hd // (H // G)
                Sh = decay[t, hd][:, None] * Sa[slot, hd]
                u = beta[t, hd] * (vd[t, hd] - Sh.T @ kd[t, gq])
                Sa[slot, hd] = Sh + torch.outer(kd[t, gq], u)
                want[t, hd] = Sa[slot, hd].T @ qd[t, gq]
            t += 1
    close(out.reshape(T, H, dv), want, torch.float32, "outputs")
    close(S.transpose(2, 3), Sa, torch.float32, "states, also of the slots that no row has")


@pytest.mark.parametrize("dt", TYPES)
@pytest.mark.parametrize("G, dk, H, dv, taps", [(1, 16, 3, 8, 3), (2, 24, 2, 16, 2), (2, 20, 4, 12, 5), (1, 12, 1, 20, 1),
                                                 (1, 64, 2, 130, 4), (2, 200, 2, 40, 8)])
def test_conv_prep_in_portions(dt, G, dk, H, dv, taps):
    """Three rows fed in portions of unequal sizes, some shorter than the taps reach back, over several steps: the
    outputs and the kept inputs must be those of the whole rows; other slots' state stays as it was."""
    g = torch.Generator().manual_seed(10)
    k_ = K()
    C = 2 * G * dk + H * dv
    lens = {2: 70, 5: 9, 0: 41}
    x = {s: (torch.randn(n, C + 6, generator=g)).to(dt) for s, n in lens.items()}
    w = [torch.randn(G * dk, taps, generator=g), torch.randn(G * dk, taps, generator=g), torch.randn(H * dv, taps, generator=g)]
    eps, q_scale = 1e-6, dk ** -0.5
    state = torch.zeros(8, C, taps - 1, device=DEV)
    state[7] = 3.0
    got = {s: [] for s in lens}
    cuts = {2: [1, 1, 2, 40, 1, 25], 5: [2, 1, 6, 0, 0, 0], 0: [17, 3, 1, 0, 20, 0]}
    at = {s: 0 for s in lens}
    for step in range(6):
        rows = [(s, cuts[s][step]) for s in lens if cuts[s][step] > 0]
        xs = torch.cat([x[s][at[s]:at[s] + n] for s, n in rows]).to(DEV)
        row_start, slot_ids = step_layout(rows)
        out = k_.conv_prep(xs, 3, 3 + G * dk, 3 + 2 * G * dk, w[0].to(DEV), w[1].to(DEV), w[2].to(DEV), G, dk, H, dv, eps,
                           q_scale, state, slot_ids, row_start, len(rows), max(n for _, n in rows))
        o = 0
        for s, n in rows:
            got[s].append(out[o:o + n].cpu())
            o += n
            at[s] += n
    taps_all = torch.cat(w, dim=0).double()
    for s, n in lens.items():
        xd = x[s][:, 3:3 + C].double()
        y = torch.zeros(n, C, dtype=torch.float64)
        for t in range(n):
            for j in range(taps):
                if t - j >= 0:
                    y[t] += taps_all[:, taps - 1 - j] * xd[t - j]
        y = y * torch.sigmoid(y)
        qk = y[:, :2 * G * dk].reshape(n, 2 * G, dk)
        qk = qk / torch.sqrt((qk * qk).sum(-1, keepdim=True) + eps)
        qk[:, :G] *= q_scale
        want = torch.cat([qk.reshape(n, -1), y[:, 2 * G * dk:]], dim=1)
        close(torch.cat(got[s]), want, torch.float32 if dt == torch.float32 else dt, f"slot {s}")
        if taps > 1:
            close(state[s], xd[n - (taps - 1):].T, torch.float32, f"kept inputs of slot {s}")
    if taps > 1:
        assert float((state[7] - 3.0).abs().max()) == 0.0 and float(state[1].abs().max()) == 0.0


@pytest.mark.parametrize("dt", TYPES)
def test_bounded_gate_squared_relu_and_weighted_sum(dt):
    g = torch.Generator().manual_seed(12)
    k_ = K()
    for T, inner, pad in ((5, 24, 0), (3, 30, 2), (130, 7, 1)):
        gu = (3.0 * torch.randn(T, 2 * inner + pad, generator=g)).to(dt)
        out = k_.clamped_glu(gu.to(DEV)[:, :2 * inner], 1.3, 1.702, dt)
        gd = torch.clamp(gu[:, :inner].double(), max=1.3)
        ud = torch.clamp(gu[:, inner:2 * inner].double(), -1.3, 1.3)
        close(out, gd * torch.sigmoid(1.702 * gd) * (ud + 1.0), dt, f"clamped glu {T} x {inner}")
    z = torch.randn(9, 40, generator=g).to(dt)
    close(k_.activation(z.to(DEV), dt, "relu2"), torch.relu(z.double()) ** 2, dt, "relu squared")
    a, b = torch.randn(11, 50, generator=g).to(dt), torch.randn(11, 50, generator=g).to(dt)
    close(k_.scaled_sum2(a.to(DEV), b.to(DEV), 0.6, -0.5), 0.6 * a.double() - 0.5 * b.double(), torch.float32, "weighted sum")
    a, b = torch.randn(3, 7, generator=g).to(dt), torch.randn(3, 7, generator=g).to(dt)
    close(k_.scaled_sum2(a.to(DEV), b.to(DEV), 1.5, 0.25), 1.5 * a.double() + 0.25 * b.double(), torch.float32, "odd size")


def test_squared_relu_in_the_projection():
    g = torch.Generator().manual_seed(14)
    k_ = K()
    x = torch.randn(5, 96, generator=g).to(torch.bfloat16)
    w = (0.2 * torch.randn(72, 96, generator=g)).to(torch.bfloat16)
    out = k_.gemv_bf16_gelu(x.to(DEV), w.to(DEV), None, torch.float32, relu2=True)
    close(out, torch.relu(x.double() @ w.double().T) ** 2, torch.float32, "relu squared in the epilogue")


@pytest.mark.parametrize("E, groups, keep, top", [(9, 3, 2, 2), (8, 4, 3, 3), (6, 6, 2, 2), (12, 2, 1, 5), (5, 1, 1, 3)])
def test_router_scores_groups_by_their_two_best(E, groups, keep, top):
    g = torch.Generator().manual_seed(16)
    k_ = K()
    T, W = 40, 48
    x = torch.randn(T, W, generator=g)
    wr = torch.randn(E + 1, W, generator=g) * 0.3
    corr = (torch.rand(E, generator=g) - 0.7) * 0.6
    idx, wt, gate = k_.moe_route(x.to(DEV), wr.to(DEV), corr.to(DEV), E, 1, groups, keep, top, 1.0, "sigmoid", "top2")
    z = x.double() @ wr.double().T
    s = torch.sigmoid(z[:, :E])
    c = s + corr.double()
    per = E // groups
    for t in range(T):
        gs = torch.stack([torch.topk(c[t, i * per:(i + 1) * per], min(2, per)).values.sum() for i in range(groups)])
        kept = torch.topk(gs, keep).indices.tolist()
        if keep < groups and float(torch.topk(gs, keep + 1).values[-2:].diff().abs()) < 1e-5:
            continue                                  # a tie between groups: either answer is right
        allowed = torch.tensor([e for e in range(E) if e // per in kept])
        order = allowed[torch.argsort(c[t, allowed], descending=True)][:top]
        assert idx[t].cpu().tolist() == order.tolist(), t
        assert torch.allclose(wt[t].cpu().double(), s[t, order], atol=1e-6)
    assert torch.allclose(gate.cpu().double(), torch.sigmoid(z[:, E]), atol=1e-6)


@pytest.mark.parametrize("nh, nkv, hd", [(4, 2, 64), (3, 3, 64), (8, 1, 64), (4, 2, 128), (5, 1, 128)])
@pytest.mark.parametrize("window, keep, cap, sinks", [(100, 5, 9.0, True), (192, 64, 15.0, True), (24, 70, 0.0, True),
                                                      (130, 128, 30.0, False), (64, 1, 0.0, False), (0, 0, 12.0, True)])
def test_tensor_core_attention_for_prompts_with_every_option(nh, nkv, hd, window, keep, cap, sinks):
    """Whole prompts, portions after earlier context and single rows through the tcgen05 kernel in each of its forms,
    with a window that keeps the first keys (less than a page, a page, more than a page, more than the window), capped
    scores and a sink score per head."""
    from test_kernels_gpu import PagedCase
    k_ = K()
    case = PagedCase(lens=[300, 64, 1, 700, 65, 128, 129], new=[300, 64, 1, 200, 65, 1, 129], nh=nh, nkv=nkv, hd=hd,
                     dtype=torch.bfloat16, seed=hd + nh + window)
    T = case.q.shape[0]
    buf = torch.randn(T, (nh + 2 * nkv) * hd, device=DEV).bfloat16()
    buf[:, :nh * hd] = case.q.reshape(T, nh * hd).to(DEV)
    scale = 1.3 / math.sqrt(hd)
    g = torch.Generator().manual_seed(3)
    sink = (3.0 * torch.rand(nh, generator=g) - 1.0) if sinks else None
    outs, t, G = [], 0, nh // nkv
    for b, (n, m) in enumerate(zip(case.lens, case.new)):
        k = case.k[b].double().repeat_interleave(G, dim=1)
        v = case.v[b].double().repeat_interleave(G, dim=1)
        q = case.q[t:t + m].double()
        s = torch.einsum("qhd,khd->hqk", q, k) * scale
        if cap:
            s = cap * torch.tanh(s / cap)
        qpos, kpos = torch.arange(n - m, n)[:, None], torch.arange(n)[None, :]
        allow = kpos <= qpos
        if window > 0:
            allow &= (kpos > qpos - window) | (kpos < keep)
        s = s.masked_fill(~allow, float("-inf"))
        mx = s.max(dim=-1, keepdim=True).values
        e = torch.exp(s - mx)
        den = e.sum(-1, keepdim=True)
        if sinks:
            den = den + torch.exp(sink.double()[:, None, None] - mx)
        outs.append(torch.einsum("hqk,khd->qhd", e / den, v))
        t += m
    want = torch.cat(outs).reshape(-1, nh * hd)
    tile_seq, tile_q0 = case.tiles(128)
    got = []
    for variant in ((0, 1, 2, 3) if hd == 64 else (0, 1, 3)):
        o = torch.full((T, nh * hd), 3.0, device=DEV, dtype=torch.bfloat16)
        k_.attn_prefill_tc(buf, buf.stride(0), o, case.k_pool, case.v_pool, case.table, case.row_start, case.row_pos0,
                           tile_seq, tile_q0, tile_seq.numel(), nh, nkv, hd, 64, window, scale, variant=variant,
                           sink=sinks, keep_first=keep, softcap=cap, sink_vals=sink.to(DEV) if sinks else None)
        err = float((o.double().cpu() - want).abs().max()) / float(want.abs().max())
        assert err <= 1e-2, (variant, err)
        got.append(o)
    for o in got[1:]:
        assert torch.equal(got[0], o)
    torch.cuda.synchronize()
    assert k_.attn_prefill_tc_status() == 0
