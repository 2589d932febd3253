"""Each CUDA kernel alone against a plain float32 torch restatement of the same operation, at
sizes other than the engine's tiny models (odd widths, several head sizes, page sizes, windows,
kv splits).  The references below are written here, from the formulas, and share nothing with
the engine."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def ops():
    from mini_sglang_b200 import ops as o
    return o


def tol(dtype):
    return dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=2e-5, atol=2e-5)


# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,V", [(1, 64, 50), (37, 120, 333), (300, 4096, 1000)])
def test_embedding(dtype, T, H, V):
    g = torch.Generator(device="cpu").manual_seed(0)
    table = torch.randn(V, H, generator=g).to(dtype).to(DEV)
    ids = torch.randint(0, V, (T,), generator=g, dtype=torch.int32).to(DEV)
    out = ops().embedding(ids, table)
    assert out.dtype == torch.float32
    torch.testing.assert_close(out, table[ids.long()].float(), rtol=0, atol=0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,H", [(1, 16), (5, 120), (33, 4096), (3, 12288 + 8)])
def test_rmsnorm_modes(dtype, wdtype, rows, H):
    g = torch.Generator(device="cpu").manual_seed(1)
    x = torch.randn(rows, H, generator=g).to(dtype).to(DEV)
    res = torch.randn(rows, H, generator=g).to(DEV)
    w = (1 + 0.1 * torch.randn(H, generator=g)).to(wdtype).to(DEV)
    eps = 1e-5

    def ref(v):
        return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * w.float())

    o = ops()
    # residual only
    y = o.rmsnorm(w, eps, residual=res, out_dtype=dtype)
    torch.testing.assert_close(y.float(), ref(res).to(dtype).float(), **tol(dtype))
    # sum fused, stream updated in place
    res2 = res.clone()
    y = o.rmsnorm(w, eps, x=x, residual=res2, residual_out=res2, out_dtype=dtype)
    v = res + x.float()
    torch.testing.assert_close(res2, v, rtol=0, atol=0)
    torch.testing.assert_close(y.float(), ref(v).to(dtype).float(), **tol(dtype))
    # plain norm of an activation
    y = o.rmsnorm(w, eps, x=x, out_dtype=dtype)
    torch.testing.assert_close(y.float(), ref(x.float()).to(dtype).float(), **tol(dtype))
    # gather of rows, stream untouched
    idx = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEV)
    y = o.rmsnorm(w, eps, x=x, residual=res, rows=idx, out_dtype=dtype)
    torch.testing.assert_close(y.float(), ref(v)[idx.long()].to(dtype).float(), **tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,I", [(1, 8), (7, 100), (65, 12288)])
def test_swiglu(dtype, T, I):
    g = torch.Generator(device="cpu").manual_seed(2)
    gu = (2 * torch.randn(T, 2 * I, generator=g)).to(dtype).to(DEV)
    out = ops().swiglu(gu)
    a, b = gu[:, :I].float(), gu[:, I:].float()
    ref = (a / (1 + torch.exp(-a)) * b).to(dtype)
    torch.testing.assert_close(out.float(), ref.float(), **tol(dtype))


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(16, 32), (48, 96), (6144, 4096), (4096, 12288), (1008, 160)])
def test_small_m_gemm(M, N, K):
    g = torch.Generator(device="cpu").manual_seed(M * 1000 + N)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) / K ** 0.5).to(torch.bfloat16).to(DEV)
    b = torch.randn(N, generator=g).to(torch.bfloat16).to(DEV)
    o = ops()
    o.SMALL_M_MAX = 16            # the kernel takes up to 16 rows; the engine uses it up to 8
    assert o._small_m_ok(x, w, b)
    ref = x.float() @ w.float().T
    y = o.linear(x, w)
    assert y.dtype == torch.bfloat16
    torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)
    y32 = o.linear(x, w, b, out_dtype=torch.float32)
    assert y32.dtype == torch.float32
    torch.testing.assert_close(y32, ref + b.float(), rtol=2e-3, atol=2e-3)
    # a view with a row stride (rows picked out of a wider buffer)
    wide = torch.randn(M, K + 64, generator=g).to(torch.bfloat16).to(DEV)
    torch.testing.assert_close(o.linear(wide[:, :K], w).float(), wide[:, :K].float() @ w.float().T, rtol=2e-2, atol=2e-2)
    # fused SwiGLU: rows [0, N/2) are the gate, [N/2, N) the up projection
    if (N // 2) % 8 == 0:
        z = o.linear_swiglu(x, w)
        gate, up = ref[:, :N // 2], ref[:, N // 2:]
        torch.testing.assert_close(z.float(), gate / (1 + torch.exp(-gate)) * up, rtol=2e-2, atol=2e-2)
    # the library path gives the same numbers (17 rows are past the kernel's limit)
    x17 = torch.randn(17, K, generator=g).to(torch.bfloat16).to(DEV)
    assert not o._small_m_ok(x17, w, None)
    torch.testing.assert_close(o.linear(x17[:M], w).float(), o.linear(x17, w)[:M].float(), rtol=2e-2, atol=2e-2)
    o.SMALL_M_MAX = 8


@pytest.mark.parametrize("M,N,K", [(1, 16, 8), (128, 256, 64), (129, 24, 72), (300, 520, 200), (700, 1040, 328),
                                   (1500, 6144, 4096), (2048, 4096, 12288), (257, 264, 4104)])
@pytest.mark.parametrize("ctas", [1, 2])
def test_tcgen05_gemm(M, N, K, ctas, monkeypatch):
    """The tcgen05 GEMM alone, on single SMs and on pairs of them: tiles that end inside the matrices in all
    three directions, a bias, a row stride, and SwiGLU in the epilogue, against float32 products of the same
    bfloat16 operands."""
    o = ops()
    monkeypatch.setattr(o, "TC_GEMM", "all")
    monkeypatch.setattr(o, "TC_GEMM_CTAS", ctas)
    monkeypatch.setattr(o, "TC_GEMM_MIN_M", 1)
    g = torch.Generator(device="cpu").manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) / K ** 0.5).to(torch.bfloat16).to(DEV)
    b = torch.randn(N, generator=g).to(torch.bfloat16).to(DEV)
    ref = x.float() @ w.float().T
    y = o._tc_gemm(x, w, None, 0)
    assert y is not None and y.dtype == torch.bfloat16 and y.shape == (M, N)
    torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(o._tc_gemm(x, w, b, 0).float(), ref + b.float(), rtol=2e-2, atol=2e-2)
    wide = torch.randn(M, K + 64, generator=g).to(torch.bfloat16).to(DEV)
    torch.testing.assert_close(o._tc_gemm(wide[:, :K], w, None, 0).float(), wide[:, :K].float() @ w.float().T, rtol=2e-2, atol=2e-2)
    if (N // 2) % 8 == 0:
        z = o._tc_gemm(x, w, None, 1)
        gate, up = ref[:, :N // 2], ref[:, N // 2:]
        assert z.shape == (M, N // 2)
        torch.testing.assert_close(z.float(), gate / (1 + torch.exp(-gate)) * up, rtol=2e-2, atol=2e-2)
        # the engine's entry point takes it from TC_GEMM_MIN_M rows on, and else the library product and the activation kernel
        torch.testing.assert_close(o.linear_swiglu(x, w).float(), z.float(), rtol=0, atol=0)
        monkeypatch.setattr(o, "TC_GEMM", "0")
        torch.testing.assert_close(o.linear_swiglu(x, w).float(), z.float(), rtol=3e-2, atol=3e-2)
    o.check_kernel_status()


@pytest.mark.parametrize("M,N,K,splits", [(9, 256, 512, 0), (16, 6144, 4096, 0), (64, 528, 1032, 3), (100, 1040, 4104, 8),
                                          (200, 4096, 12288, 0), (33, 264, 576, 2), (48, 272, 640, 1)])
def test_tcgen05_gemm_split_k(M, N, K, splits, monkeypatch):
    """The pair kernel with K cut into ranges (few tokens, so too few output tiles to fill the GPU) and the kernel that adds
    the ranges' partial sums: the count of ranges chosen by the library or given, tiles that end inside the matrices, a bias,
    SwiGLU after the sum; against float32 products of the same bfloat16 operands, and the same bits on a second run."""
    o = ops()
    monkeypatch.setattr(o, "MID_GEMM", True)
    monkeypatch.setattr(o, "MID_GEMM_SPLITS", splits)
    g = torch.Generator(device="cpu").manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) / K ** 0.5).to(torch.bfloat16).to(DEV)
    b = torch.randn(N, generator=g).to(torch.bfloat16).to(DEV)
    ref = x.float() @ w.float().T
    before = o.LAUNCHES
    y = o._tc_gemm_mid(x, w, None, 0)
    assert y is not None and y.dtype == torch.bfloat16 and y.shape == (M, N)
    if splits > 1:
        assert o.LAUNCHES - before == 2                      # the product and the sum of the ranges
    torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)
    assert torch.equal(y, o._tc_gemm_mid(x, w, None, 0))
    torch.testing.assert_close(o._tc_gemm_mid(x, w, b, 0).float(), ref + b.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(o.linear(x, w, b).float(), ref + b.float(), rtol=2e-2, atol=2e-2)      # the engine's entry point
    if (N // 2) % 8 == 0:
        z = o._tc_gemm_mid(x, w, None, 1)
        gate, up = ref[:, :N // 2], ref[:, N // 2:]
        assert z.shape == (M, N // 2)
        torch.testing.assert_close(z.float(), gate / (1 + torch.exp(-gate)) * up, rtol=2e-2, atol=2e-2)
        assert torch.equal(o.linear_swiglu(x, w), z)
        monkeypatch.setattr(o, "MID_GEMM", False)                    # the library product and the activation kernel
        torch.testing.assert_close(o.linear_swiglu(x, w).float(), z.float(), rtol=3e-2, atol=3e-2)
    else:
        assert o._tc_gemm_mid(x, w, None, 1) is None                 # refused, not computed wrongly
    o.check_kernel_status()


# ---------------------------------------------------------------------------------------
def rope_table(max_pos, rot, theta):
    idx = torch.arange(0, rot, 2, dtype=torch.float32)
    inv = 1.0 / (theta ** (idx / rot))
    fr = torch.arange(max_pos, dtype=torch.float32)[:, None] * inv[None, :]
    return torch.cat((fr.cos(), fr.sin()), -1)


@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_q,n_kv,d,rot,P,norm,wdtype", [
    (4, 2, 16, 16, 1, True, torch.bfloat16),
    (6, 2, 32, 32, 4, True, torch.float32),
    (15, 3, 48, 48, 16, True, torch.bfloat16),
    (8, 1, 128, 64, 16, False, torch.bfloat16),       # partial rotation, no norm
    (2, 2, 256, 256, 8, True, torch.float32),
    (3, 1, 80, 0, 2, True, torch.bfloat16),           # no rotation at all
    (8, 2, 128, 128, 16, True, torch.bfloat16),
    (5, 5, 64, 64, 3, True, torch.float32),
    (2, 1, 128, 0, 16, False, torch.bfloat16),
])
def test_qknorm_rope_kvwrite(dtype, n_q, n_kv, d, rot, P, norm, wdtype, interleaved):
    if interleaved and rot == 0:
        pytest.skip("no rotation: nothing to pair")
    g = torch.Generator(device="cpu").manual_seed(3)
    T, max_pos, eps = 19, 300, 1e-6
    pages = -(-T // P) + 3
    qkv = torch.randn(T, (n_q + 2 * n_kv) * d, generator=g).to(dtype)
    pos = torch.randint(0, max_pos, (T,), generator=g, dtype=torch.int32)
    loc = torch.randperm(pages * P - P, generator=g)[:T].to(torch.int32) + P      # never the dump page
    qw = (1 + 0.1 * torch.randn(d, generator=g)).to(wdtype) if norm else None
    kw = (1 + 0.1 * torch.randn(d, generator=g)).to(wdtype) if norm else None
    table = rope_table(max_pos, rot, 10000.0) if rot else None
    kc = torch.zeros(pages, n_kv, P, d, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    cu = lambda t: None if t is None else t.to(DEV)
    q = ops().qknorm_rope_kvwrite(cu(qkv), cu(pos), n_q, n_kv, d, q_weight=cu(qw), k_weight=cu(kw), eps=eps,
                                  rope_table=cu(table), out_loc=cu(loc), k_cache=kc, v_cache=vc, page_size=P,
                                  interleaved=interleaved)
    # reference
    x = qkv.float()
    qr = x[:, :n_q * d].reshape(T, n_q, d)
    kr = x[:, n_q * d:(n_q + n_kv) * d].reshape(T, n_kv, d)
    vr = x[:, (n_q + n_kv) * d:].reshape(T, n_kv, d)
    if norm:
        qr = qr * torch.rsqrt(qr.pow(2).mean(-1, keepdim=True) + eps) * qw.float()
        kr = kr * torch.rsqrt(kr.pow(2).mean(-1, keepdim=True) + eps) * kw.float()
    if rot:
        cs = table[pos.long()]
        c, s = cs[:, None, :rot // 2], cs[:, None, rot // 2:]

        def rope(t):
            if interleaved:                       # neighbours 2 p, 2 p + 1 with angle p
                a, b, rest = t[..., 0:rot:2], t[..., 1:rot:2], t[..., rot:]
                return torch.cat((torch.stack((a * c - b * s, a * s + b * c), -1).flatten(-2), rest), -1)
            a, b, rest = t[..., :rot // 2], t[..., rot // 2:rot], t[..., rot:]
            return torch.cat((a * c - b * s, a * s + b * c, rest), -1)
        qr, kr = rope(qr), rope(kr)
    torch.testing.assert_close(q.float().cpu(), qr.to(dtype).float(), **tol(dtype))
    pg, off = (loc // P).long(), (loc % P).long()
    torch.testing.assert_close(kc.cpu()[pg, :, off, :].float(), kr.to(dtype).float(), **tol(dtype))
    torch.testing.assert_close(vc.cpu()[pg, :, off, :].float(), vr.to(dtype).float(), rtol=0, atol=0)
    # nothing else was written
    mask = torch.ones(pages, P, dtype=torch.bool)
    mask[pg, off] = False
    assert kc.cpu().permute(0, 2, 1, 3)[mask].abs().sum() == 0


# ---------------------------------------------------------------------------------------
def test_sampling_greedy_and_race():
    import plain_qwen3 as P
    g = torch.Generator(device="cpu").manual_seed(4)
    N, V = 6, 333
    logits = (3 * torch.randn(N, V, generator=g)).float()
    logits[1, 77] = logits[1, 5] = logits[1].max() + 1          # tie: lowest index wins
    temps = torch.tensor([0.0, 0.0, 0.7, 1.0, 0.0, 1.3])
    keys = torch.tensor([11, 12, 13, 14, 15, 16], dtype=torch.int32)
    steps = torch.tensor([0, 1, 2, 3, 4, 5], dtype=torch.int32)
    seed = 1234567890123
    out = ops().sample(logits.to(DEV), temps.to(DEV), keys.to(DEV), steps.to(DEV), seed).cpu()
    noise = torch.stack([P.exponential_noise(seed, int(k), int(s), V) for k, s in zip(keys, steps)])
    ref = P.sample_with_noise(logits, temps, noise)
    assert out.tolist() == ref.tolist()
    assert out[1].item() == 5
    # all-greedy fast path
    out2 = ops().sample(logits.to(DEV), None, None, None, seed).cpu()
    want2 = logits.argmax(-1).tolist()
    want2[1] = 5                                                 # the tie goes to the lowest index, whatever torch's argmax picks
    assert out2.tolist() == want2
    # a request's draw does not depend on its row in the batch
    out3 = ops().sample(logits[[3, 2]].to(DEV), temps[[3, 2]].to(DEV), keys[[3, 2]].to(DEV), steps[[3, 2]].to(DEV), seed).cpu()
    assert out3.tolist() == [out[3].item(), out[2].item()]


def test_sampling_distribution():
    # chi-square of 4000 draws on a small vocabulary against softmax(logits / T)
    V, n = 12, 4000
    logits = torch.linspace(-1.5, 1.5, V).repeat(n, 1)
    T = 0.8
    temps = torch.full((n,), T)
    keys = torch.arange(n, dtype=torch.int32)
    steps = torch.zeros(n, dtype=torch.int32)
    out = ops().sample(logits.to(DEV), temps.to(DEV), keys.to(DEV), steps.to(DEV), 99).cpu()
    p = torch.softmax(logits[0] / T, -1)
    counts = torch.bincount(out.long(), minlength=V).float()
    chi2 = ((counts - n * p) ** 2 / (n * p)).sum().item()
    assert chi2 < 40.0, chi2          # 11 degrees of freedom: P(chi2 > 40) < 1e-4


# ---------------------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------------------
def attention_reference(q, K, V, q_lens, kv_lens, scale, window):
    """q [T, n_q, d]; K, V: per request dense [L, n_kv, d] float32."""
    T, n_q, d = q.shape
    out = torch.zeros(T, n_q, d)
    t = 0
    for r, (ql, L) in enumerate(zip(q_lens, kv_lens)):
        n_kv = K[r].shape[1]
        G = n_q // n_kv
        pos = torch.arange(L)
        for j in range(ql):
            p = L - ql + j
            ok = pos <= p
            if window:
                ok &= pos > p - window
            for h in range(n_q):
                s = (K[r][:, h // G] @ q[t + j, h]) * scale
                s = s.masked_fill(~ok, float("-inf"))
                out[t + j, h] = torch.softmax(s, -1) @ V[r][:, h // G]
        t += ql
    return out


def run_attention_case(dtype, n_q, n_kv, d, P, q_lens, kv_lens, window=None, force_split=None, seed=0,
                       spike=False, order=None, even_blocks=None, max_pieces=8):
    from mini_sglang_b200.config import PartSpec
    from mini_sglang_b200.parts import BuildEnv, GroupContext, KVCacheView, StepContext, Workspace
    from mini_sglang_b200.parts.attention import PagedAttention

    g = torch.Generator(device="cpu").manual_seed(seed)
    B, T = len(q_lens), sum(q_lens)
    pages_per = [-(-L // P) for L in kv_lens]
    n_pages = sum(pages_per) + 1
    perm = (torch.randperm(n_pages - 1, generator=g) + 1).tolist()          # scattered pages, never page 0
    maxp = max(pages_per)
    bt = torch.zeros(B, maxp, dtype=torch.int32)
    kc = torch.full((n_pages, n_kv, P, d), float("nan")).to(dtype)            # unwritten slots are poison
    vc = torch.full((n_pages, n_kv, P, d), float("nan")).to(dtype)
    kc[0] = 0
    vc[0] = 0
    Ks, Vs = [], []
    for r, L in enumerate(kv_lens):
        pg = [perm.pop() for _ in range(pages_per[r])]
        bt[r, :len(pg)] = torch.tensor(pg, dtype=torch.int32)
        k = torch.randn(L, n_kv, d, generator=g).to(dtype)
        v = torch.randn(L, n_kv, d, generator=g).to(dtype)
        if spike and L > 40:
            k[3] *= 6.0            # a far key that must dominate if (and only if) it is read
        for i in range(L):
            kc[pg[i // P], :, i % P] = k[i]
            vc[pg[i // P], :, i % P] = v[i]
        Ks.append(k.float())
        Vs.append(v.float())
    q = torch.randn(T, n_q, d, generator=g).to(dtype)
    if spike:
        t = 0
        for r, (ql, L) in enumerate(zip(q_lens, kv_lens)):
            if L > 40:
                q[t + ql - 1] = (Ks[r][3].repeat_interleave(n_q // n_kv, 0) * 0.5).to(dtype)
            t += ql
    scale = d ** -0.5
    ref = attention_reference(q.float(), Ks, Vs, q_lens, kv_lens, scale, window)

    env = BuildEnv(dtype=dtype, device=torch.device(DEV))
    mixer = PagedAttention(PartSpec("paged_attention", {"hidden_size": 32, "num_heads": n_q, "num_kv_heads": n_kv,
                                                        "head_dim": d, "scale": scale, "window": window}), "x", env)
    q_start = [0]
    for n in q_lens:
        q_start.append(q_start[-1] + n)
    token_req = [r for r, n in enumerate(q_lens) for _ in range(n)]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    nsplit, max_split = None, 1
    if force_split:
        nsplit, max_split = i32([force_split] * B), force_split
    even = None
    if even_blocks:          # the keys dealt out evenly over even_blocks blocks per kv head (decode only)
        from mini_sglang_b200.engine.step import pack_even_cut, plan_even_cut
        cut = plan_even_cut(kv_lens, window, even_blocks, max_pieces)
        nsplit, max_split = i32(cut[5].tolist()), max_pieces
        even = torch.from_numpy(pack_even_cut(cut, B, even_blocks)).to(DEV)
    grp = GroupContext(block_table=bt.to(DEV), out_loc=i32([0] * T), nsplit=nsplit, max_split=max_split, window=window,
                       order=i32(list(order)) if order is not None else None, even=even, even_nb=even_blocks or 0)
    uniform = all(n == 1 for n in q_lens)
    ctx = StepContext(T=T, B=B, page_size=P, input_ids=i32([0] * T), positions=i32([0] * T), q_start=i32(q_start),
                      kv_len=i32(kv_lens), token_req=i32(token_req), slots=i32([0] * B), groups=[grp],
                      host_q_lens=list(q_lens), host_kv_lens=list(kv_lens), host_slots=[0] * B,
                      uniform_decode=uniform, workspace=Workspace(torch.device(DEV)))
    out = torch.full((T, n_q, d), float("nan"), dtype=dtype, device=DEV)
    mixer.attend(q.to(DEV), out, ctx, KVCacheView(kc.to(DEV), vc.to(DEV), grp, P))
    torch.cuda.synchronize()
    return out.float().cpu(), ref


ATT_TOL = {torch.float32: dict(rtol=1e-4, atol=2e-5), torch.bfloat16: dict(rtol=2e-2, atol=2e-2)}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_q,n_kv,d,P", [(4, 2, 16, 1), (6, 2, 32, 4), (15, 3, 48, 16), (8, 2, 64, 8),
                                          (32, 8, 128, 16), (4, 4, 128, 16), (40, 2, 64, 16), (2, 1, 256, 32),
                                          (3, 1, 72, 4), (8, 8, 80, 16)])
def test_attention_mixed_batch(dtype, n_q, n_kv, d, P):
    # portions of prompts (with and without earlier context), single decoded tokens, one long context
    q_lens = [5, 1, 70, 1, 2, 33]
    kv_lens = [5, 200, 131, 64, 65, 33 + 128]
    out, ref = run_attention_case(dtype, n_q, n_kv, d, P, q_lens, kv_lens, seed=d)
    torch.testing.assert_close(out, ref.to(dtype).float(), **ATT_TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("force_split", [None, 2, 5])
@pytest.mark.parametrize("order", [None, "longest first", "any"])
def test_attention_decode_batch_with_splits(dtype, force_split, order):
    """Single decoded tokens of requests of very different lengths; the blocks take the requests in index order, by
    falling length (what a decode step asks for) or in any other order: which block computes a request changes nothing."""
    from mini_sglang_b200.engine.step import decode_order
    kv_lens = [1, 63, 64, 65, 700, 1500, 300, 129]
    if order == "longest first":
        order = decode_order(kv_lens, [force_split or 1] * len(kv_lens), None, len(kv_lens)).tolist()
        assert order[:4] == [5, 4, 6, 7] and sorted(order) == list(range(8))
    elif order == "any":
        order = [3, 0, 7, 5, 1, 6, 2, 4]
    out, ref = run_attention_case(dtype, 32, 8, 128, 16, [1] * len(kv_lens), kv_lens, force_split=force_split,
                                  seed=7, spike=True, order=order)
    torch.testing.assert_close(out, ref.to(dtype).float(), **ATT_TOL[dtype])


@pytest.mark.parametrize("n_q,n_kv,d,P", [(32, 8, 128, 16), (8, 2, 64, 8), (16, 1, 32, 4), (6, 2, 96, 16)])
@pytest.mark.parametrize("blocks,max_pieces", [(1, 1), (3, 8), (7, 8), (74, 32), (7, 2)])
@pytest.mark.parametrize("window", [None, 600])
def test_attention_decode_even_cut(n_q, n_kv, d, P, blocks, max_pieces, window):
    """Single decoded tokens of requests of very different lengths with the keys of all of them dealt out evenly over
    a fixed number of blocks: a block takes the end of one request, whole short ones and the start of the next; requests
    in several blocks are merged from their pieces.  A far key stands out in every long request (it must be read once)."""
    from mini_sglang_b200.engine.step import plan_even_cut
    kv_lens = [1, 63, 64, 65, 700, 1500, 300, 129, 16, 17, 1025]
    if d not in (32, 64, 96, 128):
        pytest.skip("no transposed decode kernel for this head size")
    cut = plan_even_cut(kv_lens, window, blocks, max_pieces)
    assert cut[5].max() <= max_pieces and (window is not None or blocks == 1 or max_pieces == 1 or cut[5].max() > 1)
    out, ref = run_attention_case(torch.bfloat16, n_q, n_kv, d, P, [1] * len(kv_lens), kv_lens, window=window, seed=11,
                                  spike=window is None, even_blocks=blocks, max_pieces=max_pieces)
    torch.testing.assert_close(out, ref.to(torch.bfloat16).float(), **ATT_TOL[torch.bfloat16])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [1, 7, 64, 100])
def test_attention_window(dtype, window):
    q_lens = [1, 40, 3, 1]
    kv_lens = [300, 140, 65, 5]
    out, ref = run_attention_case(dtype, 6, 2, 32, 4, q_lens, kv_lens, window=window, force_split=3, seed=9)
    torch.testing.assert_close(out, ref.to(dtype).float(), **ATT_TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_far_key_and_page_edges(dtype):
    # one score stands out: the last query of every long request is aligned with key 3, hundreds of
    # keys back, in another page and another key tile; a kernel that skips or mis-addresses far keys
    # cannot pass within tolerance
    q_lens = [17, 1, 16, 1]
    kv_lens = [17 + 480, 1023, 16 + 16 * 7, 1025]
    out, ref = run_attention_case(dtype, 8, 2, 64, 16, q_lens, kv_lens, seed=11, spike=True)
    torch.testing.assert_close(out, ref.to(dtype).float(), **ATT_TOL[dtype])


@pytest.mark.parametrize("version", [1, 2])
@pytest.mark.parametrize("n_q,n_kv,P,window", [(32, 8, 16, None), (8, 8, 8, None), (16, 1, 64, None), (12, 4, 256, None),
                                               (32, 8, 4, None), (4, 2, 1, None), (6, 2, 16, 100), (8, 2, 32, 300)])
def test_attention_tcgen05_kernels(version, n_q, n_kv, P, window, monkeypatch):
    """The two tcgen05 prefill kernels (one query tile per block; two in ping-pong) at head size 128: page sizes
    that TMA fetches and two that it cannot (4 and 1: rows gathered, one-tile kernel), groups of 1, 3, 4 and 16 heads,
    prompts that start at an offset, end inside a key tile or fill only part of a query tile, windows, and a far
    key that must dominate.  Unwritten cache slots hold NaN."""
    from mini_sglang_b200 import ops
    monkeypatch.setattr(ops, "TC_VERSION", version)
    q_lens = [300, 33, 1, 130, 64, 17]
    kv_lens = [300, 33 + 700, 90, 130 + 129, 64 + 1024, 17 + 480]
    out, ref = run_attention_case(torch.bfloat16, n_q, n_kv, 128, P, q_lens, kv_lens, window=window, seed=3 + P, spike=True)
    ops.check_kernel_status()
    torch.testing.assert_close(out, ref.to(torch.bfloat16).float(), **ATT_TOL[torch.bfloat16])


def test_attention_split_requests_never_reach_the_whole_range_kernels():
    """kv splits asked for a request of 5 and of 12 tokens at head size 128: the tcgen05 kernels take whole key
    ranges, so these requests must go to the kernel that writes split partials (else the merge would read what
    nobody wrote)."""
    out, ref = run_attention_case(torch.bfloat16, 32, 8, 128, 16, [5, 1, 12, 1], [3000, 2000, 2500, 700], force_split=4, seed=21)
    torch.testing.assert_close(out, ref.to(torch.bfloat16).float(), **ATT_TOL[torch.bfloat16])


def test_status_words_reach_the_host_as_errors():
    """The kernels with bounded waits report a wait that ran out through status words on the device, which the
    step function polls.  Here the failure is made on the host (a word set by a copy, no kernel gives up): the
    next poll must raise, for the attention word and for the GEMM word, and a cleared word must not."""
    o = ops()
    st = o._status_tensor(DEV)
    o.check_kernel_status()                       # clean to begin with
    for word, what in ((0, "attention"), (2, "GEMM")):
        st[word] = 1
        o.poll_status()
        with pytest.raises(o.KernelError, match=what):
            o.raise_if_failed(wait=True)
        with pytest.raises(o.KernelError, match=what):
            o.check_kernel_status()
        st[word] = 0
        o.check_kernel_status()
    # raise_if_failed() without wait never blocks: it looks only at a poll that has already arrived
    st[0] = 1
    o.poll_status()
    torch.cuda.synchronize()
    with pytest.raises(o.KernelError):
        o.raise_if_failed()
    st[0] = 0
    o.check_kernel_status()
