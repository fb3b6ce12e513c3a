"""The kernels that came with the Nibelix decoder, each alone against float64 torch arithmetic, at sizes of no model."""
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
    assert got.shape == want.shape, what
    err = float((got - want).abs().max()) / max(1e-30, float(want.abs().max()))
    assert err <= tol(dt), (what, err)


def tanh_norm(h, w, b, alpha):
    return torch.tanh(alpha.double() * h.double()) * w.double() + b.double()


@pytest.mark.parametrize("dt", TYPES)
@pytest.mark.parametrize("T, H", [(1, 100), (7, 96), (130, 2048), (3, 4100)])
def test_tanh_norm_add(dt, T, H):
    g = torch.Generator().manual_seed(T * 31 + H)
    h = torch.randn(T, H, generator=g).to(DEV)
    a = torch.randn(T, H, generator=g).to(dt).to(DEV)
    b = torch.randn(T, H, generator=g).to(dt).to(DEV)
    sa, sb = torch.rand(H, generator=g).to(DEV) + 0.5, torch.rand(H, generator=g).to(DEV) + 0.5
    norms = [(torch.randn(H, generator=g).to(DEV), torch.randn(H, generator=g).to(DEV),
              torch.tensor([0.5 + 0.4 * i], device=DEV)) for i in range(2)]
    # two sublayers and two norms
    want_h = h.double() + 0.7 * (sa.double() * a.double() + sb.double() * b.double())
    h1 = h.clone()
    outs = K().tanh_norm_add(h1, a, b, sa, sb, 0.7, norms, dt)
    close(h1, want_h, torch.float32, "residual")
    for o, n in zip(outs, norms):
        close(o, tanh_norm(want_h, *n), dt, "norm")
    # one sublayer, no norm
    h2 = h.clone()
    assert K().tanh_norm_add(h2, a, None, sa, None, 1.3, [], torch.float32) == []
    close(h2, h.double() + 1.3 * sa.double() * a.double(), torch.float32)
    # norms only, and of chosen rows
    outs = K().tanh_norm_add(h, None, None, None, None, 1.0, norms[:1], dt)
    close(outs[0], tanh_norm(h, *norms[0]), dt)
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device=DEV)
    outs = K().tanh_norm_add(h, None, None, None, None, 1.0, norms[1:], dt, rows=rows)
    close(outs[0], tanh_norm(h[rows.long()], *norms[1]), dt)


def test_softcap():
    x = torch.linspace(-200, 200, 3000, device=DEV).reshape(3, -1).contiguous()
    want = 25.0 * torch.tanh(x.double() / 25.0)
    close(K().softcap(x, 25.0), want, torch.float32)


@pytest.mark.parametrize("dt", TYPES)
@pytest.mark.parametrize("act", ["silu", "gelu", "gelu_tanh"])
def test_gated_activations(dt, act):
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(9, 2 * 136, generator=g) * 2).to(dt).to(DEV)
    gate, up = x[:, :136].double(), x[:, 136:].double()
    f = {"silu": lambda z: z * torch.sigmoid(z), "gelu": lambda z: 0.5 * z * (1 + torch.erf(z / math.sqrt(2))),
         "gelu_tanh": lambda z: 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))}[act]
    close(K().silu_mul(x, act=act), f(gate) * up, dt, act)


def plain_route(z, corr, groups, keep, top, scale, score):
    """Per token (picks, weights): float64, loops."""
    s = torch.softmax(z, dim=-1) if score == "softmax" else torch.sigmoid(z)
    c = s + corr
    n = z.shape[1]
    per = n // groups
    idx, wt = [], []
    for t in range(z.shape[0]):
        best = sorted(range(groups), key=lambda gi: (-float(c[t, gi * per:(gi + 1) * per].max()), gi))[:keep]
        cand = sorted((e for e in range(n) if e // per in best), key=lambda e: (-float(c[t, e]), e))[:top]
        idx.append(cand)
        wt.append([float(s[t, e]) * scale for e in cand])
    return idx, wt


@pytest.mark.parametrize("dt", TYPES)
@pytest.mark.parametrize("T, W, n, groups, keep, top, score, extra", [
    (1, 96, 8, 1, 1, 2, "softmax", 1), (5, 100, 12, 3, 2, 3, "softmax", 0), (37, 2048, 16, 4, 2, 2, "softmax", 1),
    (9, 520, 40, 8, 3, 6, "sigmoid", 1), (4, 64, 6, 6, 2, 2, "softmax", 0), (3, 72, 5, 1, 1, 5, "softmax", 1),
    (150, 1100, 12, 2, 1, 2, "softmax", 1), (70, 4096, 18, 3, 2, 4, "softmax", 1), (2, 5000, 9, 1, 1, 3, "softmax", 0)])
def test_route(dt, T, W, n, groups, keep, top, score, extra):
    g = torch.Generator().manual_seed(T + W + n)
    x = torch.randn(T, W, generator=g).to(dt).to(DEV)
    wr = (torch.randn(n + extra, W, generator=g) * 2.0 / math.sqrt(W)).to(DEV)
    # corrections well below zero for some outputs: a shut-out output must count as minus infinity, not as zero
    corr = ((torch.rand(n, generator=g) - 0.8) * 0.5).to(DEV)
    idx, wt, gate = K().moe_route(x, wr, corr, n, extra, groups, keep, top, 1.7, score)
    z = x.double().cpu() @ wr.double().cpu().T
    want_idx, want_wt = plain_route(z[:, :n], corr.double().cpu(), groups, keep, top, 1.7, score)
    assert idx.cpu().tolist() == want_idx
    close(wt, torch.tensor(want_wt), torch.float32)
    if extra:
        close(gate, torch.sigmoid(z[:, n]), torch.float32)
    else:
        assert gate is None
    # a token's picks and weights are the same bits whether it comes alone (the few-token form) or among many
    if T > 64:
        idx1, wt1, _ = K().moe_route(x[:3], wr, corr, n, extra, groups, keep, top, 1.7, score)
        assert torch.equal(idx1, idx[:3]) and torch.equal(wt1, wt[:3])


def experts_reference(x, idx, w_up, w_down, act):
    f = {"gelu": lambda z: 0.5 * z * (1 + torch.erf(z / math.sqrt(2))), "silu": lambda z: z * torch.sigmoid(z)}[act]
    T, top = idx.shape
    E = w_up.shape[0]
    y = torch.zeros(T * top, w_down.shape[1], dtype=torch.float64)
    mid = torch.zeros(T * top, w_up.shape[1], dtype=torch.float64)
    for t in range(T):
        for k in range(top):
            e = int(idx[t, k])
            if 0 <= e < E:
                mid[t * top + k] = f(w_up[e].double() @ x[t].double())
                y[t * top + k] = w_down[e].double() @ mid[t * top + k]
    return mid, y


def planned_rows(idx, E):
    return [p for p, e in enumerate(idx.flatten().tolist()) if 0 <= e < E]


@pytest.mark.parametrize("dt", TYPES)
@pytest.mark.parametrize("T, top, E, n_out, W, inner", [(1, 2, 4, 6, 96, 40), (70, 3, 5, 8, 100, 33), (300, 2, 3, 3, 64, 72)])
def test_experts_on_cuda_cores(dt, T, top, E, n_out, W, inner):
    """Picks from E on are identity outputs and -1 is no pick: neither is planned; experts nobody picked; more rows
    of an expert than a tile holds."""
    g = torch.Generator().manual_seed(T + E)
    x = torch.randn(T, W, generator=g).to(dt)
    idx = torch.randint(-1, n_out, (T, top), generator=g, dtype=torch.int32)
    idx[idx == 1] = 0                                         # nobody picks expert 1
    w_up = (torch.randn(E, inner, W, generator=g) / math.sqrt(W)).to(dt)
    w_down = (torch.randn(E, W, inner, generator=g) / math.sqrt(inner)).to(dt)
    want_mid, want_y = experts_reference(x.cpu(), idx, w_up, w_down, "gelu")
    order, plan = K().moe_plan(idx.to(DEV), E)
    rows = planned_rows(idx, E)
    assert int(plan[1]) == len(rows) and sorted(order[:len(rows)].cpu().tolist()) == rows
    mid = K().moe_gemm(x.to(DEV), top, w_up.to(DEV), order, plan, dt, act="gelu")
    close(mid[rows], want_mid[rows], dt, "up")
    y = K().moe_gemm(mid, 1, w_down.to(DEV), order, plan, torch.float32)
    close(y[rows], want_y[rows], dt, "down")


@pytest.mark.parametrize("T, top, E, n_out, W, inner", [(1, 2, 4, 6, 96, 40), (8, 2, 14, 16, 2048, 1408), (5, 7, 7, 7, 104, 24),
                                                        (20, 3, 2, 3, 64, 72)])
def test_experts_of_a_few_rows(T, top, E, n_out, W, inner):
    """The decode-sized product: tiles of a few rows, an expert's matrix read once; an expert with more rows than a
    tile holds (20 tokens on 2 experts)."""
    dt = torch.bfloat16
    g = torch.Generator().manual_seed(T + E + 1)
    x = torch.randn(T, W, generator=g).to(dt)
    idx = torch.randint(0, n_out, (T, top), generator=g, dtype=torch.int32)
    w_up = (torch.randn(E, inner, W, generator=g) / math.sqrt(W)).to(dt)
    w_down = (torch.randn(E, W, inner, generator=g) / math.sqrt(inner)).to(dt)
    want_mid, want_y = experts_reference(x, idx, w_up, w_down, "gelu")
    order, plan = K().moe_plan(idx.to(DEV), E, K().moe_tile_rows("few"))
    rows = planned_rows(idx, E)
    mid = K().moe_gemv(x.to(DEV), top, w_up.to(DEV), order, plan, dt, act="gelu")
    close(mid[rows], want_mid[rows], dt, "up")
    y = K().moe_gemv(mid, 1, w_down.to(DEV), order, plan, torch.float32)
    close(y[rows], want_y[rows], dt, "down")


@pytest.mark.parametrize("T, top, E, n_out, W, inner", [(300, 2, 3, 4, 64, 72), (1100, 3, 9, 10, 200, 328), (513, 1, 2, 2, 520, 264)])
def test_experts_on_tensor_cores(T, top, E, n_out, W, inner):
    """The prompt-sized product: rows gathered into the plan's order, tiles of 128 rows that run into the next
    expert's rows, experts of more and of fewer rows than a tile, widths that are no multiple of the tile's 64 and
    256, an expert nobody picked, identity picks left out; the second product puts every pair back at its place."""
    dt = torch.bfloat16
    g = torch.Generator().manual_seed(T + E + 2)
    x = torch.randn(T, W, generator=g).to(dt)
    idx = torch.randint(0, n_out, (T, top), generator=g, dtype=torch.int32)
    if E > 2:
        idx[idx == 1] = 0
        idx[:40][idx[:40] == 2] = 0                           # expert 2 gets fewer rows than the others
    w_up = (torch.randn(E, inner, W, generator=g) / math.sqrt(W)).to(dt)
    w_down = (torch.randn(E, W, inner, generator=g) / math.sqrt(inner)).to(dt)
    want_mid, want_y = experts_reference(x, idx, w_up, w_down, "gelu")
    order, plan = K().moe_plan(idx.to(DEV), E, K().moe_tile_rows("tc"))
    rows = planned_rows(idx, E)
    n = int(plan[1])
    assert n == len(rows)
    xs = K().moe_gather(x.to(DEV), top, order, plan)
    placed = order[:n].long().cpu()
    assert torch.equal(xs[:n].cpu(), x[placed // top])
    mid = K().moe_gemm_tc(xs, w_up.to(DEV), order, plan, dt, act="gelu")
    close(mid[:n], want_mid[placed], dt, "up")
    y = K().moe_gemm_tc(mid, w_down.to(DEV), order, plan, torch.float32)
    close(y[rows], want_y[rows], dt, "down")
    assert K().moe_tc_status() == 0


@pytest.mark.parametrize("dt", TYPES)
def test_combine(dt):
    g = torch.Generator().manual_seed(8)
    T, top, H, E = 11, 3, 100, 4
    x = torch.randn(T, H, generator=g).to(dt).to(DEV)
    idx = torch.randint(-1, E + 2, (T, top), generator=g, dtype=torch.int32).to(DEV)
    wt = torch.rand(T, top, generator=g).to(DEV)
    y = torch.randn(T * top, H, generator=g).to(DEV)
    shared = torch.randn(T, H, generator=g).to(dt).to(DEV)
    gate = torch.rand(T, generator=g).to(DEV)
    want = torch.zeros(T, H, dtype=torch.float64)
    for t in range(T):
        for k in range(top):
            e = int(idx[t, k])
            if e >= E:
                want[t] += float(wt[t, k]) * x[t].double().cpu()
            elif e >= 0:
                want[t] += float(wt[t, k]) * y[t * top + k].double().cpu()
    close(K().moe_combine(y, idx, wt, x, None, None, E), want, torch.float32, "no shared expert")
    want2 = want + gate.double().cpu()[:, None] * shared.double().cpu()
    close(K().moe_combine(y, idx, wt, x, shared, gate, E), want2, torch.float32, "gated shared expert")
    close(K().moe_combine(None, torch.full_like(idx, E), wt, x, None, None, E),
          wt.double().cpu().sum(1, keepdim=True) * x.double().cpu(), torch.float32, "identity only")


@pytest.mark.parametrize("dt", TYPES)
@pytest.mark.parametrize("heads, dv, a_row, out_row", [(3, 6, 8, 8), (4, 24, 24, 24), (2, 128, 128, 128), (5, 40, 64, 40)])
def test_diff_combine(dt, heads, dv, a_row, out_row):
    g = torch.Generator().manual_seed(heads * dv)
    T, lam, eps, mult = 9, 0.37, 1e-5, 0.7
    a = torch.randn(T, heads * 2 * a_row, generator=g).to(dt).to(DEV)
    gate = torch.randn(T, heads + 3, generator=g).to(dt).to(DEV)[:, 1:1 + heads]
    av = a.double().cpu().view(T, heads, 2, a_row)[..., :dv]
    o = av[:, :, 0] - lam * av[:, :, 1]
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * mult
    want = torch.zeros(T, heads, out_row, dtype=torch.float64)
    want[..., :dv] = o * torch.sigmoid(gate.double().cpu())[..., None]
    got = K().diff_combine(a, a_row, gate, lam, eps, mult, heads, dv, out_row, dt)
    close(got, want.view(T, -1), dt)
    want[..., :dv] = o
    close(K().diff_combine(a, a_row, None, lam, eps, mult, heads, dv, out_row, dt), want.view(T, -1), dt, "no gate")


@pytest.mark.parametrize("dt", TYPES)
@pytest.mark.parametrize("heads, dv", [(1, 2048), (1, 300), (2, 2600), (3, 40)])
def test_norm_over_wide_heads(dt, heads, dv):
    """All heads normed together are one head of many values: a block a head instead of a warp."""
    g = torch.Generator().manual_seed(dv)
    T = 5
    o = torch.randn(T, heads * dv, generator=g).to(DEV) * 3
    w = (1 + 0.2 * torch.randn(heads * dv, generator=g)).to(DEV)
    gate = torch.randn(T, heads * dv, generator=g).to(dt).to(DEV)
    ov = o.double().cpu().view(T, heads, dv)
    want = (ov / torch.sqrt((ov * ov).mean(-1, keepdim=True) + 1e-5)).view(T, -1) * w.double().cpu() * \
        torch.sigmoid(gate.double().cpu())
    close(K().head_norm_gate(o, w, gate, 1e-5, heads, dv, dt, gate_kind="sigmoid"), want, dt)


@pytest.mark.parametrize("dt", TYPES)
def test_scan_with_silu_inputs(dt):
    """The recurrence with one fixed decay per head (one of them exactly 1) whose queries, keys and values go through
    SiLU as they are read; rows that start from a state and rows that start from zero."""
    g = torch.Generator().manual_seed(12)
    H, dk, dv = 3, 12, 20
    rows = [(2, 5), (0, 1), (4, 37)]
    T = sum(n for _, n in rows)
    q = torch.randn(T, H * dk, generator=g).to(dt).to(DEV)
    k = torch.randn(T, H * dk, generator=g).to(dt).to(DEV)
    v = torch.randn(T, H * dv, generator=g).to(dt).to(DEV)
    decay = torch.tensor([1.0, 0.9, 0.5], device=DEV)
    state = torch.randn(6, H, dk, dv, generator=g).to(DEV)
    before = state.double().cpu()
    slot_ids = torch.tensor([s for s, _ in rows], dtype=torch.int32, device=DEV)
    starts = [0]
    for _, n in rows:
        starts.append(starts[-1] + n)
    row_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
    got = K().linear_scan(1, q, k, v, state, slot_ids, row_start, len(rows), H, dk, dv, max(n for _, n in rows),
                          decay=decay, in_act="silu")
    silu = lambda z: z * torch.sigmoid(z)
    qd, kd, vd = (silu(t.double().cpu()) for t in (q, k, v))
    want = torch.zeros(T, H, dv, dtype=torch.float64)
    for (slot, n), t0 in zip(rows, starts):
        S = before[slot].clone()
        for t in range(t0, t0 + n):
            S = decay.double().cpu()[:, None, None] * S + kd[t].view(H, dk, 1) * vd[t].view(H, 1, dv)
            want[t] = torch.einsum("hkv,hk->hv", S, qd[t].view(H, dk))
        close(state[slot], S, torch.float32, "state")
    close(got, want.view(T, -1), torch.float32 if dt == torch.float32 else dt)
    assert torch.equal(state[1].double().cpu(), before[1])          # a slot of no row stays as it was


@pytest.mark.parametrize("dt, x_dt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                      (torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("H, G, d, dv, rot", [(4, 2, 24, 16, 12), (3, 3, 10, 6, 10), (2, 1, 64, 128, 0), (8, 2, 32, 64, 32),
                                              (4, 4, 64, 128, 32)])
def test_maps_prep(dt, x_dt, H, G, d, dv, rot):
    """Rotation of part of every map, the queries widened to a head per map, keys and values at their places in the
    pages (two sequences, the second starting in the middle of a page); the projection in the queries' type or in
    float32 (as steps of few tokens leave it)."""
    g = torch.Generator().manual_seed(H * d)
    row, v_row, page = (2 * d + 7) // 8 * 8, (dv + 7) // 8 * 8, 16
    seqs = [(0, 0, 5), (1, 29, 6)]                            # (sequence, first position, tokens)
    tok_seq = torch.tensor([s for s, _, n in seqs for _ in range(n)], dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor([p + i for _, p, n in seqs for i in range(n)], dtype=torch.int32, device=DEV)
    T = len(tok_pos)
    block_table = torch.tensor([[3, 1, -1], [0, 4, 2]], dtype=torch.int32, device=DEV)
    ld = H * 2 * d + G * 2 * d + G * dv + 8
    x = torch.randn(T, ld, generator=g).to(x_dt).to(DEV)
    k_pool = torch.zeros(5, G, page, row, dtype=dt, device=DEV)
    v_pool = torch.zeros(5, G, page, v_row, dtype=dt, device=DEV)
    inv = torch.tensor([300.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64) if rot else None
    table = K().rotary_table(inv).to(DEV) if rot else None
    q_off, k_off = 0, H * 2 * d
    v_off = k_off + G * 2 * d
    q = K().maps_prep(x, q_off, k_off, v_off, H, G, 2, d, dv, rot, table, tok_pos, tok_seq, block_table, page, dt,
                      k_pool, v_pool)

    def rotated(m, pos):                                      # m [..., d] at positions pos [T]
        out = m.clone()
        if rot:
            a = pos.double()[:, None] * inv[None, :]
            c, s = a.cos()[:, None, :], a.sin()[:, None, :]
            u, w_ = m[..., :rot // 2], m[..., rot // 2:rot]
            out[..., :rot // 2], out[..., rot // 2:rot] = u * c - w_ * s, w_ * c + u * s
        return out
    xd, pos = x.double().cpu(), tok_pos.cpu()
    qm = rotated(xd[:, :H * 2 * d].reshape(T, H * 2, d), pos)
    km = rotated(xd[:, k_off:v_off].reshape(T, G * 2, d), pos)
    want_q = torch.zeros(T, H * 2, row, dtype=torch.float64)
    for m in range(2):
        want_q[:, m::2, m * d:(m + 1) * d] = qm[:, m::2]
    close(q.view(T, H * 2, row), want_q, dt, "queries")
    for t in range(T):
        pg = int(block_table[int(tok_seq[t]), int(pos[t]) // page])
        slot = int(pos[t]) % page
        want_k = torch.zeros(G, row, dtype=torch.float64)
        want_k[:, :2 * d] = km[t].reshape(G, 2 * d)
        close(k_pool[pg, :, slot], want_k, dt, ("key", t))
        want_v = torch.zeros(G, v_row, dtype=torch.float64)
        want_v[:, :dv] = xd[t, v_off:v_off + G * dv].reshape(G, dv)
        close(v_pool[pg, :, slot], want_v, dt, ("value", t))
