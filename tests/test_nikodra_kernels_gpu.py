"""The kernels that came with the Nikodra decoder, each alone against float64 torch arithmetic, at sizes of no model."""
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


def step_layout(rows, g):
    """Packed rows of a step: ``rows`` = [(slot, first position, tokens)]."""
    tok_seq = torch.tensor([b for b, (_, _, n) in enumerate(rows) for _ in range(n)], dtype=torch.int32)
    tok_pos = torch.tensor([p0 + i for _, p0, n in rows for i in range(n)], dtype=torch.int32)
    row_start = torch.tensor([0] + list(torch.tensor([n for _, _, n in rows]).cumsum(0)), dtype=torch.int32)
    slot_ids = torch.tensor([s for s, _, _ in rows], dtype=torch.int32)
    return tok_seq.to(DEV), tok_pos.to(DEV), row_start.to(DEV), slot_ids.to(DEV)


@pytest.mark.parametrize("dt", TYPES)
def test_embed_hashed(dt):
    g = torch.Generator().manual_seed(1)
    V, H, buckets, mp, mc = 50, 40, 11, 131, 19
    table = torch.randn(V, H, generator=g).to(dt).to(DEV)
    extra = torch.randn(buckets + 1, H, generator=g).to(dt).to(DEV)
    rows = [(3, 0, 5), (0, 7, 1), (5, 2, 4), (1, 0, 1)]
    tok_seq, tok_pos, row_start, slot_ids = step_layout(rows, g)
    ids = torch.randint(0, V, (int(row_start[-1]),), generator=g, dtype=torch.int32)
    last = torch.randint(0, V, (7,), generator=g, dtype=torch.int32)
    state = last.clone().to(DEV)
    got = K().embed_hashed(ids.to(DEV), tok_pos, tok_seq, row_start, slot_ids, table, extra, buckets, mp, mc, state)
    want = torch.zeros(len(ids), H, dtype=torch.float64)
    t = 0
    for slot, p0, n in rows:
        for i in range(n):
            prev = int(last[slot]) if i == 0 else int(ids[t - 1])
            r = buckets if p0 + i == 0 else (prev * mp + int(ids[t]) * mc) % buckets
            want[t] = table[int(ids[t])].double().cpu() + extra[r].double().cpu()
            t += 1
    close(got, want, torch.float32)
    after = last.clone()
    t = 0
    for slot, _, n in rows:
        t += n
        after[slot] = ids[t - 1]
    assert torch.equal(state.cpu(), after)


def rotate_ref(x, pos, f, factor, rot, interleaved):
    a = pos.double()[:, None] * f[None, :]
    c, s = (a.cos() * factor)[:, None, :], (a.sin() * factor)[:, None, :]
    out = x.clone()
    if interleaved:
        u, v = x[..., 0:rot:2], x[..., 1:rot:2]
        out[..., 0:rot:2], out[..., 1:rot:2] = u * c - v * s, v * c + u * s
    else:
        u, v = x[..., :rot // 2], x[..., rot // 2:rot]
        out[..., :rot // 2], out[..., rot // 2:rot] = u * c - v * s, v * c + u * s
    return out


@pytest.mark.parametrize("dt", TYPES)
@pytest.mark.parametrize("aligned", [False, True])
@pytest.mark.parametrize("H, G, d, dv, norm, rot, layout, mix", [
    (4, 2, 24, 16, 2, 24, 1, True), (3, 1, 10, 6, 1, 0, 0, False), (6, 3, 16, 40, 2, 8, 1, False),
    (2, 2, 64, 128, 0, 32, 0, True), (5, 5, 10, 12, 2, 6, 1, True), (8, 1, 40, 40, 2, 40, 1, True)])
def test_qk_prep_into_the_cache(dt, aligned, H, G, d, dv, norm, rot, layout, mix):
    """``aligned``: offsets and pitches in multiples of 8, which the 16-byte form of the kernel takes where the head
    sizes allow it; otherwise odd offsets, which only the general form takes."""
    g = torch.Generator().manual_seed(2)
    k_ = K()
    page, n_pages = 64, 6
    dp, dvp = (d + 7) // 8 * 8, (dv + 7) // 8 * 8
    rows = [(0, 60, 9), (1, 0, 3), (2, 130, 1)]
    tok_seq, tok_pos, row_start, slot_ids = step_layout(rows, g)
    T = int(row_start[-1])
    off = 8 if aligned else 5
    ld = off + (H + G) * d + G * dv + 3
    if aligned:
        ld = (ld + 7) // 8 * 8
    so = 8 if aligned else 2                              # where the mixed-in values start in their rows
    x = torch.randn(T, ld, generator=g).to(dt).to(DEV)
    qw, kw = (1 + 0.3 * torch.randn(d, generator=g)).to(DEV), (1 + 0.3 * torch.randn(d, generator=g)).to(DEV)
    f = torch.tensor([100.0 ** (-2.0 * i / max(rot, 1)) for i in range(rot // 2)], dtype=torch.float64) * 0.37
    table = k_.rotary_table(f).to(DEV) if rot else None
    factor = 1.14
    lam = torch.tensor([0.35], device=DEV)
    src = torch.randn(T, (G * dv + 16 + 7) // 8 * 8, generator=g).to(dt).to(DEV)
    bt = torch.tensor([[4, 1, -1], [0, -1, -1], [3, 5, 2]], dtype=torch.int32, device=DEV)
    kp = torch.full((n_pages, G, page, dp), 7.0, dtype=dt, device=DEV)
    vp = torch.full((n_pages, G, page, dvp), 7.0, dtype=dt, device=DEV)
    q, none = k_.qk_prep(x, off, off + H * d, off + (H + G) * d, H, G, d, dv, dp, dvp, norm, qw if norm == 2 else None,
                         kw if norm == 2 else None, 1e-5, rot, layout, table, factor, 1.0,
                         (lam, src[:, so:so + G * dv]) if mix else None, tok_pos, tok_seq, bt, page, dt, kp, vp)
    assert none is None
    xd = x.double().cpu()
    qr = xd[:, off:off + H * d].reshape(T, H, d)
    kr = xd[:, off + H * d:off + (H + G) * d].reshape(T, G, d)
    vr = xd[:, off + (H + G) * d:off + (H + G) * d + G * dv].reshape(T, G, dv)

    def nrm(a, w):
        if norm == 0:
            return a
        a = a / torch.sqrt((a * a).mean(-1, keepdim=True) + 1e-5)
        return a * w.double().cpu() if norm == 2 else a
    qr, kr = nrm(qr, qw), nrm(kr, kw)
    if rot:
        qr = rotate_ref(qr, tok_pos.cpu(), f, factor, rot, layout == 1)
        kr = rotate_ref(kr, tok_pos.cpu(), f, factor, rot, layout == 1)
    if mix:
        vr = 0.65 * vr + 0.35 * src[:, so:so + G * dv].double().cpu().reshape(T, G, dv)
    want_q = torch.zeros(T, H, dp, dtype=torch.float64)
    want_q[..., :d] = qr
    close(q.reshape(T, H, dp), want_q, dt, "q")
    want_k, want_v = torch.full(kp.shape, 7.0, dtype=torch.float64), torch.full(vp.shape, 7.0, dtype=torch.float64)
    for t in range(T):
        p = int(tok_pos[t])
        pg = int(bt[int(tok_seq[t]), p // page])
        want_k[pg, :, p % page, :] = 0
        want_v[pg, :, p % page, :] = 0
        want_k[pg, :, p % page, :d] = kr[t]
        want_v[pg, :, p % page, :dv] = vr[t]
    close(kp, want_k, dt, "keys, and no other place of the pool")
    close(vp, want_v, dt, "values, and no other place of the pool")


def test_qk_prep_without_a_cache_keeps_float32():
    g = torch.Generator().manual_seed(3)
    k_ = K()
    H, d, T = 3, 12, 7
    x = torch.randn(T, 2 * H * d + 9, generator=g).to(torch.bfloat16).to(DEV)
    pos = torch.tensor([0, 1, 2, 900, 901, 5, 6], dtype=torch.int32, device=DEV)
    seq = torch.zeros(T, dtype=torch.int32, device=DEV)
    f = torch.tensor([50.0 ** (-2.0 * i / 8) for i in range(4)], dtype=torch.float64)
    q, k = k_.qk_prep(x, 0, H * d, -1, H, H, d, 0, d, 0, 0, None, None, 1e-5, 8, 0, k_.rotary_table(f).to(DEV), 1.0,
                      d ** -0.5, None, pos, seq, None, 0, torch.float32, None, None, k_dtype=torch.float32)
    assert q.dtype == torch.float32 and k.dtype == torch.float32
    xd = x.double().cpu()
    close(q.reshape(T, H, d), rotate_ref(xd[:, :H * d].reshape(T, H, d), pos.cpu(), f, 1.0, 8, False), torch.float32)
    close(k.reshape(T, H, d), rotate_ref(xd[:, H * d:2 * H * d].reshape(T, H, d), pos.cpu(), f, 1.0, 8, False) * d ** -0.5,
          torch.float32)


@pytest.mark.parametrize("dt", TYPES)
@pytest.mark.parametrize("H, G, d, dv, chunk, sink", [
    (4, 2, 24, 16, 0, True), (6, 2, 16, 40, 50, True), (2, 1, 128, 64, 128, True), (3, 1, 16, 8, 7, False),
    (8, 2, 64, 128, 0, True), (4, 4, 40, 40, 150, True), (5, 5, 16, 16, 0, False)])
def test_attention_with_sink_blocks_and_values_of_another_width(dt, H, G, d, dv, chunk, sink):
    g = torch.Generator().manual_seed(4)
    k_ = K()
    page, n_pages, width = 64, 40, 12
    lens = [700, 1, 130, 65]                              # the last query of each row and some before it
    perm = torch.randperm(n_pages, generator=g)
    bt = torch.full((len(lens), width), -1, dtype=torch.int32)
    at = 0
    for b, n in enumerate(lens):
        need = (n + page - 1) // page
        bt[b, :need] = perm[at:at + need].int()
        at += need
    kp = (torch.randn(n_pages, G, page, d, generator=g) * 1.0).to(dt)
    vp = torch.randn(n_pages, G, page, dv, generator=g).to(dt)
    queries = [(0, 699), (0, 698), (0, 449), (0, 450), (0, 255), (0, 256), (0, 0), (1, 0), (2, 129), (2, 127), (2, 128), (3, 64), (3, 63)]
    T = len(queries)
    q = torch.randn(T, H * d, generator=g).to(dt)
    tok_seq = torch.tensor([b for b, _ in queries], dtype=torch.int32)
    tok_pos = torch.tensor([p for _, p in queries], dtype=torch.int32)
    scale = 0.9 / math.sqrt(d)
    want = torch.zeros(T, H, dv, dtype=torch.float64)
    for t, (b, p) in enumerate(queries):
        lo = p // chunk * chunk if chunk else 0
        js = torch.arange(lo, p + 1)
        pg = bt[b, js // page].long()
        kk, vv = kp[pg, :, js % page].double(), vp[pg, :, js % page].double()          # [n, G, *]
        for h in range(H):
            s = kk[:, h // (H // G)] @ q[t, h * d:(h + 1) * d].double() * scale
            m = max(float(s.max()), 0.0) if sink else float(s.max())
            e = torch.exp(s - m)
            want[t, h] = (e / (e.sum() + (math.exp(-m) if sink else 0.0))) @ vv[:, h // (H // G)]
    for split in (256, 64):
        n = (700 + split - 1) // split
        if chunk:
            n = min(n, (chunk + split - 2) // split + 1)
        scratch = torch.zeros(k_.attn_tokens_scratch_bytes(T, H, dv, n) // 4 + 1, device=DEV)
        out = torch.empty(T, H * dv, dtype=dt, device=DEV)
        k_.attn_tokens_ex(q.to(DEV), H * d, out, kp.to(DEV), vp.to(DEV), bt.to(DEV), tok_pos.to(DEV), tok_seq.to(DEV), T, H, G,
                          d, dv, page, 0, chunk, sink, scale, split, n, scratch if n > 1 else None)
        close(out.reshape(T, H, dv), want, dt, f"split {split}")
    # fewer tokens: the merge inside the attention kernel
    n = 3 if not chunk else min(3, (chunk + 254) // 256 + 1)
    scratch = torch.zeros(k_.attn_tokens_scratch_bytes(2, H, dv, n) // 4 + 1, device=DEV)
    out = torch.empty(2, H * dv, dtype=dt, device=DEV)
    k_.attn_tokens_ex(q[:2].to(DEV), H * d, out, kp.to(DEV), vp.to(DEV), bt.to(DEV), tok_pos[:2].to(DEV), tok_seq[:2].to(DEV), 2,
                      H, G, d, dv, page, 0, chunk, sink, scale, 256, n, scratch)
    close(out.reshape(2, H, dv), want[:2], dt, "two tokens")


@pytest.mark.parametrize("dt", TYPES)
def test_token_shift(dt):
    g = torch.Generator().manual_seed(5)
    rows = [(2, 0, 4), (0, 9, 1), (4, 3, 6)]
    tok_seq, tok_pos, row_start, slot_ids = step_layout(rows, g)
    T, W = int(row_start[-1]), 40
    h = torch.randn(T, W, generator=g).to(dt)
    mu = torch.rand(5, W, generator=g)
    prev = torch.randn(6, W, generator=g)
    state = prev.clone().to(DEV)
    got = K().token_shift(h.to(DEV), mu.to(DEV), state, tok_seq, row_start, slot_ids, dt)
    want = torch.zeros(5, T, W, dtype=torch.float64)
    after = prev.clone()
    t = 0
    for slot, _, n in rows:
        for i in range(n):
            before = prev[slot].double() if i == 0 else h[t - 1].double()
            want[:, t] = h[t].double()[None] + (before - h[t].double())[None] * mu.double()
            t += 1
        after[slot] = h[t - 1].float()
    close(got, want, dt)
    assert torch.equal(state.cpu(), after)


@pytest.mark.parametrize("rk_dt", TYPES)
@pytest.mark.parametrize("mode, H, dk, dv", [(0, 3, 16, 16), (1, 3, 16, 24), (1, 2, 12, 20), (0, 2, 14, 14),
                                               (1, 2, 64, 128), (0, 2, 64, 64)])
@pytest.mark.parametrize("lens", [[5, 1, 9], [300, 3, 129, 128, 64, 65]])
def test_linear_scan(rk_dt, mode, H, dk, dv, lens):
    g = torch.Generator().manual_seed(6)
    k_ = K()
    slots = [4, 0, 6, 2, 7, 1][:len(lens)]
    rows = [(s, 0, n) for s, n in zip(slots, lens)]
    tok_seq, tok_pos, row_start, slot_ids = step_layout(rows, g)
    T = int(row_start[-1])
    r = torch.randn(T, H * dk + 8, generator=g).to(rk_dt)
    k = (torch.randn(T, H * dk, generator=g) * 0.5).to(rk_dt)
    v = torch.randn(T, H * dv + 16, generator=g).to(torch.bfloat16)
    wraw = torch.randn(T, H * dk, generator=g).to(rk_dt) - 1.0
    w0 = torch.randn(H * dk, generator=g) - 1.5
    u = torch.randn(H, dk, generator=g)
    decay = torch.tensor([0.9, 0.97, 0.999][:H])
    state0 = torch.randn(9, H, dk, dv, generator=g)
    state = state0.clone().to(DEV)
    max_new = max(lens)
    need = k_.linear_scan_scratch_bytes(len(lens), T, H, dk, dv, max_new)
    assert (need > 0) == (max_new > 128)
    scratch = torch.zeros(need // 4 + 1, device=DEV) if need else None
    rv, vv = r[:, 3:3 + H * dk], v[:, 8:8 + H * dv]
    out = k_.linear_scan(mode, r.to(DEV)[:, 3:3 + H * dk], k.to(DEV), v.to(DEV)[:, 8:8 + H * dv], state, slot_ids, row_start, len(lens), H, dk, dv,
                         max_new, wraw=wraw.to(DEV) if mode == 0 else None, w0=w0.to(DEV) if mode == 0 else None,
                         u=u.to(DEV) if mode == 0 else None, decay=decay.to(DEV) if mode == 1 else None, scratch=scratch)
    want = torch.zeros(T, H, dv, dtype=torch.float64)
    after = state0.double().clone()
    w = torch.exp(-torch.exp(wraw.double() + w0.double()[None])).reshape(T, H, dk)
    rd, kd, vd = rv.double().reshape(T, H, dk), k.double().reshape(T, H, dk), vv.double().reshape(T, H, dv)
    t = 0
    for slot, _, n in rows:
        for _ in range(n):
            for hd in range(H):
                S = after[slot, hd]
                kv = torch.outer(kd[t, hd], vd[t, hd])
                if mode == 0:
                    want[t, hd] = (S + u[hd].double()[:, None] * kv).T @ rd[t, hd]
                    after[slot, hd] = w[t, hd][:, None] * S + kv
                else:
                    after[slot, hd] = float(decay[hd]) * S + kv
                    want[t, hd] = after[slot, hd].T @ rd[t, hd]
            t += 1
    close(out.reshape(T, H, dv), want, torch.float32, "outputs")
    close(state, after, torch.float32, "states, also of the slots that no row has")


@pytest.mark.parametrize("dt", TYPES)
def test_head_norm_gate_normed_sum_and_activations(dt):
    g = torch.Generator().manual_seed(7)
    k_ = K()
    T, H, dv = 9, 3, 20
    o = torch.randn(T, H * dv, generator=g) * 3
    w = 1 + 0.2 * torch.randn(H * dv, generator=g)
    gate = torch.randn(T, H * dv + 8, generator=g).to(dt)
    gv = gate[:, 4:4 + H * dv]
    got = k_.head_norm_gate(o.to(DEV), w.to(DEV), gate.to(DEV)[:, 4:4 + H * dv], 1e-5, H, dv, dt)
    x = o.double().reshape(T, H, dv)
    x = (x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5)).reshape(T, -1) * w.double()
    close(got, x * gv.double() * torch.sigmoid(gv.double()), dt)
    got = k_.head_norm_gate(o.to(DEV), None, None, 1e-5, H, dv, torch.float32)
    close(got, x / w.double(), torch.float32)
    a, b = torch.randn(T, 100, generator=g).to(dt), (torch.randn(T, 100, generator=g) * 5).to(dt)
    wa, wb = torch.randn(100, generator=g), torch.randn(100, generator=g)
    n = lambda z: z.double() / torch.sqrt((z.double() ** 2).mean(-1, keepdim=True) + 1e-6)
    close(k_.normed_sum2(a.to(DEV), b.to(DEV), wa.to(DEV), wb.to(DEV), 1e-6, 0.5), 0.5 * (n(a) * wa.double() + n(b) * wb.double()),
          torch.float32)
    for shape in ((7, 33), (5, 64)):
        z = (torch.randn(shape, generator=g) * 3).to(dt)
        zd = z.double()
        close(k_.activation(z.to(DEV), dt, "gelu"), 0.5 * zd * (1 + torch.erf(zd / math.sqrt(2))), dt)
        close(k_.activation(z.to(DEV), dt, "gelu_tanh"),
              0.5 * zd * (1 + torch.tanh(math.sqrt(2 / math.pi) * (zd + 0.044715 * zd ** 3))), dt)
        close(k_.activation(z.to(DEV), torch.float32, "tanh"), torch.tanh(zd), torch.float32)


@pytest.mark.parametrize("y_dt", TYPES)
@pytest.mark.parametrize("H", [96, 2304])
def test_norm_add_norm(y_dt, H):
    """The norm on a sublayer's output, the residual sum and the next input norm in one kernel; rows longer than a
    thread keeps in registers too."""
    g = torch.Generator().manual_seed(8)
    T = 5
    h = torch.randn(T, H, generator=g)
    y = (torch.randn(T, H, generator=g) * 4).to(y_dt)
    w, w2 = 0.5 + 0.1 * torch.randn(H, generator=g), 1 + 0.1 * torch.randn(H, generator=g)
    hd = h.clone().to(DEV)
    for x_dt in TYPES:
        hd = h.clone().to(DEV)
        x = K().norm_add_norm(hd, y.to(DEV), w.to(DEV), 1e-5, w2.to(DEV), 2e-6, x_dt)
        yd = y.double()
        want_h = h.double() + yd / torch.sqrt((yd * yd).mean(-1, keepdim=True) + 1e-5) * w.double()
        close(hd, want_h, torch.float32, "residual")
        close(x, want_h / torch.sqrt((want_h * want_h).mean(-1, keepdim=True) + 2e-6) * w2.double(), x_dt, "next norm")


def test_gelu_in_the_projection():
    g = torch.Generator().manual_seed(9)
    M, N, Kd = 5, 72, 128
    x = torch.randn(M, Kd, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, Kd, generator=g) * 0.2).to(torch.bfloat16)
    z = x.double() @ w.double().T
    for tanh in (False, True):
        got = K().gemv_bf16_gelu(x.to(DEV), w.to(DEV), None, torch.float32, tanh=tanh)
        want = 0.5 * z * (1 + (torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)) if tanh else torch.erf(z / math.sqrt(2))))
        close(got, want, torch.float32)


@pytest.mark.parametrize("H, G, d, chunk, sink", [(4, 2, 64, 0, True), (8, 1, 128, 100, True), (6, 2, 64, 200, False),
                                                   (4, 4, 128, 0, True)])
def test_tensor_core_attention_for_single_tokens_with_sink_and_blocks(H, G, d, chunk, sink):
    """The decode kernel's three ways of ending a row (one chunk; chunks merged through scratch; chunks merged inside
    a block or a cluster) all count the sink, and its key range starts at the block's edge."""
    g = torch.Generator().manual_seed(10)
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
    kp = torch.randn(n_pages, G, page, d, generator=g).to(torch.bfloat16)
    vp = torch.randn(n_pages, G, page, d, generator=g).to(torch.bfloat16)
    queries = [(0, 699), (1, 0), (2, 129), (3, 64)]
    T = len(queries)
    q = torch.randn(T, H * d, generator=g).to(torch.bfloat16)
    tok_seq = torch.tensor([b for b, _ in queries], dtype=torch.int32)
    tok_pos = torch.tensor([p for _, p in queries], dtype=torch.int32)
    scale = 0.9 / math.sqrt(d)
    want = torch.zeros(T, H, d, dtype=torch.float64)
    for t, (b, p) in enumerate(queries):
        lo = p // chunk * chunk if chunk else 0
        js = torch.arange(lo, p + 1)
        pg = bt[b, js // page].long()
        kk, vv = kp[pg, :, js % page].double(), vp[pg, :, js % page].double()
        for h in range(H):
            s = kk[:, h // (H // G)] @ q[t, h * d:(h + 1) * d].double() * scale
            m = max(float(s.max()), 0.0) if sink else float(s.max())
            e = torch.exp(s - m)
            want[t, h] = (e / (e.sum() + (math.exp(-m) if sink else 0.0))) @ vv[:, h // (H // G)]
    for split, in_block in ((1024, 0), (256, 0), (256, 1), (128, 2)):
        n = (700 + split - 1) // split
        if chunk:
            n = min(n, (chunk + split - 2) // split + 1)
        if in_block and not 1 < n <= 4 * in_block:
            continue
        scratch = torch.zeros(k_.attn_tokens_scratch_bytes(T, H, d, n) // 4 + 1, device=DEV) if n > 1 and not in_block else None
        out = torch.empty(T, H * d, dtype=torch.bfloat16, device=DEV)
        k_.attn_decode(q.to(DEV), H * d, out, kp.to(DEV), vp.to(DEV), bt.to(DEV), tok_pos.to(DEV), tok_seq.to(DEV), T, H, G, d,
                       page, 0, scale, split, n, scratch, in_block=in_block, chunk=chunk, sink=sink)
        close(out.reshape(T, H, d), want, torch.bfloat16, f"split {split} in_block {in_block}")
    assert k_.attn_decode_status() == 0
