"""The Rigitar decoder's kernels alone, each against plain float32/float64 torch arithmetic of the same operation, at
sizes other than any model's: attention over latent rows (tensor cores and CUDA cores, prompts, portions, single tokens,
with and without chunks), the products per head, the step between the joint projection and the rest, the minGRU
recurrence in both forms, the output norm, xIELU alone and as a projection's epilogue."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def K():
    from exl3_server_b200.ops import kernels
    return kernels


def _latent_case(B, H, dk, dv, news, ctxs, dtype, seed):
    """Random pool and queries for B sequences: sequence b brings news[b] tokens that end at position ctxs[b] - 1.
    Pages are dealt out in a scrambled order, so that a wrong page shows."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    pages_seq = [(c + 63) // 64 for c in ctxs]
    width = max(pages_seq)
    n_pages = sum(pages_seq) + 3
    perm = torch.randperm(n_pages, generator=g)
    pool = (torch.randn(n_pages, 1, 64, dk, generator=g) * 0.6).to(dtype).to(DEV)
    bt = torch.full((B, width), -1, dtype=torch.int32)
    at = 0
    for b in range(B):
        bt[b, :pages_seq[b]] = perm[at:at + pages_seq[b]].to(torch.int32)
        at += pages_seq[b]
    T = sum(news)
    q = (torch.randn(T, H * dk, generator=g) * 0.25).to(dtype).to(DEV)
    row_start = torch.tensor([0] + list(torch.tensor(news).cumsum(0)), dtype=torch.int32)
    pos0 = torch.tensor([c - n for c, n in zip(ctxs, news)], dtype=torch.int32)
    tok_seq = torch.cat([torch.full((n,), b, dtype=torch.int32) for b, n in enumerate(news)])
    tok_pos = torch.cat([torch.arange(c - n, c, dtype=torch.int32) for c, n in zip(ctxs, news)])
    return pool, bt.to(DEV), q, row_start.to(DEV), pos0.to(DEV), tok_seq.to(DEV), tok_pos.to(DEV)


def _latent_plain(pool, bt, q, news, ctxs, H, dk, dv, scale, gate=None):
    out = []
    t = 0
    pool64, q64 = pool.double().cpu(), q.double().cpu()
    for b, (n, c) in enumerate(zip(news, ctxs)):
        keys = torch.cat([pool64[int(p), 0] for p in bt[b].cpu() if int(p) >= 0])[:c]       # [c, dk]
        for i in range(n):
            pos = c - n + i
            qq = q64[t].view(H, dk)
            s = (qq @ keys[:pos + 1].T) * scale
            p = torch.softmax(s, dim=-1)
            o = p @ keys[:pos + 1, :dv]
            if gate is not None:
                o = o * gate[t].double().cpu()[:, None]
            out.append(o.reshape(-1))
            t += 1
    return torch.stack(out)


@pytest.mark.parametrize("H, dk, dv, news, ctxs, chunks", [
    (16, 576, 512, [1, 1, 1], [300, 64, 1], (1, 1)),            # single tokens, one chunk
    (16, 576, 512, [1, 1, 1], [700, 65, 129], (2, 6)),          # single tokens, chunks of two pages
    (3, 48, 32, [1, 1], [200, 5], (1, 4)),                      # few heads, narrow rows, chunks of one page
    (40, 176, 128, [1, 1], [130, 257], (2, 3)),                 # more rows than one tile takes
    (5, 160, 96, [70, 3, 1, 129], [70, 3, 1, 129], (1, 1)),     # prompts from position 0, unequal
    (8, 128, 96, [33, 2], [200, 66], (1, 1)),                   # portions after earlier context
    (4, 336, 256, [150], [400], (3, 3)),                        # a portion, its keys in chunks
    (2, 592, 512, [40], [40], (1, 1)),                          # the widest rows
])
def test_attention_over_latent_rows_on_the_tensor_cores(H, dk, dv, news, ctxs, chunks):
    k = K()
    B, T = len(news), sum(news)
    pool, bt, q, row_start, pos0, _, _ = _latent_case(B, H, dk, dv, news, ctxs, torch.bfloat16, seed=H * dk + T)
    assert k.attn_latent_supported(torch.bfloat16, dk, dv, 64)
    per, n = chunks
    gate = torch.rand(T, H, device=DEV) + 0.25
    out = torch.empty(T, H * dv, dtype=torch.bfloat16, device=DEV)
    scratch = torch.zeros(max(1, k.attn_latent_scratch_bytes(T, H, dv, n) // 4), device=DEV) if n > 1 else None
    k.attn_latent(q, out, pool, bt, row_start, pos0, B, T, max(news), H, dk, dv, 64, 0.11, per, n, scratch, gate)
    want = _latent_plain(pool, bt, q, news, ctxs, H, dk, dv, 0.11, gate)
    err = float((out.double().cpu() - want).abs().max() / want.abs().max())
    assert err <= 2e-2, err


@pytest.mark.parametrize("dtype, tol", [(torch.float32, 2e-6), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("H, dk, dv, news, ctxs", [
    (3, 48, 32, [1, 1], [300, 5]),
    (8, 176, 128, [40, 2, 1], [90, 300, 1]),
    (2, 576, 512, [1, 9], [520, 70]),
    (5, 304, 288, [3], [260]),
    (2, 832, 768, [1, 5], [130, 70]),                  # rows wider than anything the tensor-core kernel takes
])
def test_attention_over_latent_rows_on_the_cuda_cores(H, dk, dv, news, ctxs, dtype, tol):
    k = K()
    B, T = len(news), sum(news)
    pool, bt, q, _, _, tok_seq, tok_pos = _latent_case(B, H, dk, dv, news, ctxs, dtype, seed=H + dk)
    out = torch.empty(T, H * dv, dtype=dtype, device=DEV)
    n = (max(ctxs) + 255) // 256
    scratch = torch.zeros(max(1, k.attn_tokens_scratch_bytes(T, H, dv, n) // 4), device=DEV) if n > 1 else None
    k.attn_tokens_kv(q, q.stride(0), out, pool, pool, bt, tok_pos, tok_seq, T, H, 1, dk, dv, dk, 64, 0, 0.13, 256, n, scratch)
    want = _latent_plain(pool, bt, q, news, ctxs, H, dk, dv, 0.13)
    err = float((out.double().cpu() - want).abs().max() / want.abs().max())
    assert err <= tol, err


@pytest.mark.parametrize("dtype, tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("T, H, Kf, N, rot_dim, rot", [(1, 3, 24, 40, 8, 8), (9, 16, 128, 512, 64, 64), (70, 2, 10, 36, 6, 4),
                                                      (5, 4, 520, 48, 0, 0)])
def test_products_per_head_with_the_rotated_tail(T, H, Kf, N, rot_dim, rot, dtype, tol):
    k = K()
    g = torch.Generator().manual_seed(T * H + N)
    hq, pad = Kf + rot_dim, (N + 15) // 16 * 16
    row = (pad + rot_dim + 15) // 16 * 16
    x = torch.randn(T, H * hq, generator=g).to(dtype).to(DEV)
    w = (torch.randn(H, Kf, N, generator=g) * 0.2).to(dtype).to(DEV)
    pos = torch.randint(0, 5000, (T,), generator=g).to(torch.int32).to(DEV)
    mul = (torch.rand(T, H, generator=g) + 0.5).to(DEV)
    out = torch.full((T, H * row), 7.0, dtype=dtype, device=DEV)
    freq = torch.tensor([300.0 ** (-2.0 * i / max(1, rot)) for i in range(rot // 2)], dtype=torch.float64)
    table = k.rotary_table(freq).to(DEV) if rot else None
    k.head_gemm(x, H * hq, hq, w, out, H * row, row, T, H, Kf, N, mul=mul, rot_dim=rot_dim, rot=rot, inv_freq=table,
                tok_pos=pos, tail_off=pad)
    x64, w64 = x.double().cpu().view(T, H, hq), w.double().cpu()
    want = torch.zeros(T, H, row, dtype=torch.float64)
    want[:, :, :N] = torch.einsum("thk,hkn->thn", x64[:, :, :Kf], w64) * mul.double().cpu()[:, :, None]
    if rot_dim:
        tail = x64[:, :, Kf:].clone()
        a = pos.double().cpu()[:, None] * freq[None, :]
        u, v = tail[:, :, :rot // 2].clone(), tail[:, :, rot // 2:rot].clone()
        tail[:, :, :rot // 2] = u * a.cos()[:, None] - v * a.sin()[:, None]
        tail[:, :, rot // 2:rot] = v * a.cos()[:, None] + u * a.sin()[:, None]
        want[:, :, pad:pad + rot_dim] = tail
    got = out.double().cpu().view(T, H, row)
    if row == N:                                   # nothing behind the products: the kernel writes no tail
        want = want[:, :, :N]
    err = float((got - want).abs().max() / want.abs().max())
    assert err <= tol, err


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width, news", [(50, [1, 1, 1]), (96, [5, 130, 1, 64]), (2048, [700]), (130, [129, 257, 33])])
def test_mingru_recurrence_in_both_forms(width, news, dtype):
    k = K()
    g = torch.Generator().manual_seed(width + sum(news))
    B, T = len(news), sum(news)
    zug = (torch.randn(T, 3 * width, generator=g) * 1.5).to(dtype).to(DEV)
    slots = torch.randperm(B + 2, generator=g)[:B].to(torch.int32).to(DEV)
    state = torch.randn(B + 3, width, generator=g).to(DEV)
    before = state.clone()
    row_start = torch.tensor([0] + list(torch.tensor(news).cumsum(0)), dtype=torch.int32, device=DEV)
    need = k.mingru_scratch_bytes(B, T, width, max(news))
    assert (need > 0) == (max(news) > 128)
    scratch = torch.zeros(need // 4, device=DEV) if need else None
    y = k.mingru_scan(zug, state, slots, row_start, B, width, max(news), dtype, scratch)
    z64, t = zug.double().cpu(), 0
    want = torch.zeros(T, width, dtype=torch.float64)
    final = before.double().cpu()
    for b, n in enumerate(news):
        S = final[int(slots[b])].clone()
        for _ in range(n):
            a, u, gg = z64[t, :width], z64[t, width:2 * width], z64[t, 2 * width:]
            z = torch.sigmoid(a)
            S = (1 - z) * S + z * torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
            want[t] = S * gg * torch.sigmoid(gg)
            t += 1
        final[int(slots[b])] = S
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert float((y.double().cpu() - want).abs().max() / want.abs().max()) <= tol
    assert float((state.double().cpu() - final).abs().max()) <= 1e-5         # the state is float32 in both; untouched rows too


@pytest.mark.parametrize("ydt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T, H", [(1, 100), (7, 2048), (3, 9000), (300, 328)])
def test_output_norm_with_the_residual_sum(T, H, ydt):
    k = K()
    g = torch.Generator().manual_seed(T + H)
    h = torch.randn(T, H, generator=g).to(DEV)
    y = (torch.randn(T, H, generator=g) * 3).to(ydt).to(DEV)
    w = (1 + 0.2 * torch.randn(H, generator=g)).to(torch.bfloat16).to(DEV)
    want = h.double().cpu() + y.double().cpu() / torch.sqrt((y.double().cpu() ** 2).mean(-1, keepdim=True) + 1e-5) * w.double().cpu()
    x = k.norm_add(h, y, w, 1e-5, torch.bfloat16)
    assert float((h.double().cpu() - want).abs().max()) <= 1e-5
    assert torch.equal(x, h.to(torch.bfloat16))
    assert k.norm_add(h, None, None, 1e-5, None) is None
    assert torch.equal(k.norm_add(h, None, None, 1e-5, torch.bfloat16), h.to(torch.bfloat16))


def _xielu64(z, p, q):
    sp = lambda v: math.log1p(math.exp(v))
    return torch.where(z > 0, sp(p) * z * z + z / 2, (0.5 + sp(q)) * (torch.expm1(torch.clamp(z, max=0.0)) - z) + z / 2)


@pytest.mark.parametrize("zdt, odt, tol", [(torch.float32, torch.float32, 2e-6), (torch.float32, torch.bfloat16, 5e-3),
                                           (torch.bfloat16, torch.bfloat16, 5e-3)])
@pytest.mark.parametrize("n", [5, 4096, 100003])
def test_xielu(n, zdt, odt, tol):
    k = K()
    g = torch.Generator().manual_seed(n)
    z = torch.cat([torch.randn(n - 4, generator=g) * 3, torch.tensor([0.0, -1e-4, -0.2499, -30.0])]).to(zdt).to(DEV)
    pq = torch.tensor([0.3, -0.7], dtype=torch.bfloat16, device=DEV)
    want = _xielu64(z.double().cpu(), float(pq[0]), float(pq[1]))
    got = k.xielu(z, pq, odt).double().cpu()
    # the two terms of the negative branch cancel near z = -1.6: the error is measured against the terms' size
    assert float(((got - want).abs() / (want.abs() + z.double().cpu().abs() + 1e-3)).max()) <= tol


@pytest.mark.parametrize("M, N, Kf", [(1, 392, 328), (8, 5632, 2048), (16, 70, 88)])
def test_xielu_as_a_projection_epilogue(M, N, Kf):
    k = K()
    g = torch.Generator().manual_seed(M + N)
    x = torch.randn(M, Kf, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, Kf, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    sp = lambda v: math.log1p(math.exp(v))
    got = k.gemv_bf16_act(x, w, None, torch.float32, sp(0.3), 0.5 + sp(-0.7)).double().cpu()
    want = _xielu64(x.double().cpu() @ w.double().cpu().T, 0.3, -0.7)
    assert float((got - want).abs().max() / want.abs().max()) <= 1e-5


def test_step_between_the_joint_projection_and_the_rest():
    """Both latent norms, the rotation of the shared key part, the cache write at the token's page and place, the gates."""
    k = K()
    g = torch.Generator().manual_seed(5)
    T, q_rank, kv_rank, rot_dim, rot, H = 6, 20, 36, 10, 6, 3
    rank_pad, row = 48, 64
    lda = 80
    a = torch.randn(T, lda, generator=g).to(DEV)
    wq = (1 + 0.1 * torch.randn(q_rank, generator=g)).to(DEV)
    wkv = (1 + 0.1 * torch.randn(kv_rank, generator=g)).to(DEV)
    freq = torch.tensor([700.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64)
    pos = torch.tensor([0, 63, 64, 65, 130, 7], dtype=torch.int32, device=DEV)
    seq = torch.tensor([0, 0, 0, 0, 0, 1], dtype=torch.int32, device=DEV)
    bt = torch.tensor([[4, 2, 5], [1, -1, -1]], dtype=torch.int32, device=DEV)
    pool = torch.full((7, 1, 64, row), 9.0, device=DEV)
    cq, gate = k.latent_prep(a, 0, q_rank, wq, q_rank, kv_rank, rot_dim, wkv, q_rank + kv_rank + rot_dim, H, 1e-6,
                             k.rotary_table(freq).to(DEV), rot, pos, seq, bt, 64, pool, row, rank_pad, torch.float32)
    a64 = a.double().cpu()
    rms = lambda v: v / torch.sqrt((v * v).mean(-1, keepdim=True) + 1e-6)
    assert float((cq.double().cpu() - rms(a64[:, :q_rank]) * wq.double().cpu()).abs().max()) <= 1e-5
    assert float((gate.double().cpu() - torch.sigmoid(a64[:, 66:69])).abs().max()) <= 1e-6
    c = rms(a64[:, q_rank:q_rank + kv_rank]) * wkv.double().cpu()
    tail = a64[:, 56:66].clone()
    ang = pos.double().cpu()[:, None] * freq[None, :]
    u, v = tail[:, :3].clone(), tail[:, 3:6].clone()
    tail[:, :3], tail[:, 3:6] = u * ang.cos() - v * ang.sin(), v * ang.cos() + u * ang.sin()
    untouched = pool.clone().cpu()
    for t in range(T):
        page = int(bt[int(seq[t]), int(pos[t]) // 64])
        got = pool[page, 0, int(pos[t]) % 64].double().cpu()
        want = torch.zeros(row, dtype=torch.float64)
        want[:kv_rank], want[rank_pad:rank_pad + rot_dim] = c[t], tail[t]
        assert float((got - want).abs().max()) <= 1e-5, t
        untouched[page, 0, int(pos[t]) % 64] = pool[page, 0, int(pos[t]) % 64].cpu()
    assert torch.equal(untouched, pool.cpu())                    # no other row was written
