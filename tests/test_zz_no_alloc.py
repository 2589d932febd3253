"""The allocation-free decode attention entry point (csrc/attention_noalloc.h).

Some callers of the kernel library cannot allocate device memory when they call it: the process
gave all of its memory budget away at start-up, or its request path must not touch the allocator
because cudaMalloc / cudaFree can stall the whole device.  For them the library carries the scratch
memory of the split-KV decode attention inside itself.  This test calls that entry point through
its exported C symbol, exactly as such a caller would (raw pointers and a stream, nothing from
torch's allocator inside the call), and checks it against the regular entry point fed with
scratch from the caller and against the attention formula written out in float32 -- twice in a row
with different inputs, because the built-in scratch keeps whatever the previous call left there.  Collected last on purpose (file name), so a run
that stops at the first failure has been through every other test before.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

c_void_p, c_int, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


def _libs(d):
    from mini_sglang_b200.csrc import build
    new = build.attention_noalloc_library(d)
    new.msgl_attention_decode_noalloc.argtypes = [c_void_p] * 8 + [c_int] * 8 + [c_float, c_int, c_void_p]
    new.msgl_attention_decode_noalloc.restype = c_int
    new.msgl_attention_noalloc_capacity_floats.restype = ctypes.c_ulonglong
    return new


def _case(seed, B, n_q, n_kv, d, P, dtype, max_split):
    g = torch.Generator().manual_seed(seed)
    kv_lens = torch.randint(1, 900, (B,), generator=g).tolist()
    kv_lens[0] = 1500
    pages_per = [-(-L // P) for L in kv_lens]
    n_pages = sum(pages_per) + 1
    perm = (torch.randperm(n_pages - 1, generator=g) + 1).tolist()
    bt = torch.zeros(B, max(pages_per), dtype=torch.int32)
    for r, n in enumerate(pages_per):
        bt[r, :n] = torch.tensor([perm.pop() for _ in range(n)], dtype=torch.int32)
    kc = torch.randn(n_pages, n_kv, P, d, generator=g).to(dtype).cuda()
    vc = torch.randn(n_pages, n_kv, P, d, generator=g).to(dtype).cuda()
    q = torch.randn(B, n_q, d, generator=g).to(dtype).cuda()
    nsplit = torch.tensor([max(1, min(max_split, L // 128)) for L in kv_lens], dtype=torch.int32).cuda()
    return dict(q=q, kc=kc, vc=vc, bt=bt.cuda(), kv_len=torch.tensor(kv_lens, dtype=torch.int32).cuda(),
                q_start=torch.arange(B + 1, dtype=torch.int32).cuda(), nsplit=nsplit)


def _regular(c, n_kv, P, max_split, scale):
    """The existing entry point, with scratch that the caller allocates."""
    from mini_sglang_b200 import ops
    q = c["q"]
    B, n_q, d = q.shape
    out = torch.empty_like(q)
    part_o = torch.empty(max_split * B * n_q * d, dtype=torch.float32, device="cuda")
    part_ml = torch.empty(max_split * B * n_q * 2, dtype=torch.float32, device="cuda")
    variant = ops.VARIANT_MMA_DECODE if ops.mma_supported(d, q.dtype) else ops.VARIANT_SIMT
    ops.attention(q, out, c["kc"], c["vc"], q_start=c["q_start"], kv_len=c["kv_len"], block_table=c["bt"],
                  nsplit=c["nsplit"], part_o=part_o, part_ml=part_ml, n_kv=n_kv, page_size=P, window=0,
                  max_split=max_split, scale=scale, qlen_min=1, qlen_max=1, uniform_decode=True, variant=variant,
                  grid_x=B)
    ops.attention_combine(part_o, part_ml, None, c["nsplit"], out, max_split)
    return out


def _restated(c, n_kv, P, scale):
    """The same attention written out in float32 with torch: every request's keys gathered from its pages, the new
    token attending to all of them.  Shares nothing with either entry point."""
    q, kc, vc = c["q"].float(), c["kc"].float(), c["vc"].float()
    B, n_q, d = q.shape
    group = n_q // n_kv
    out = torch.empty_like(q)
    for r in range(B):
        L = int(c["kv_len"][r])
        pages = c["bt"][r, : -(-L // P)].long()
        k = kc[pages].permute(1, 0, 2, 3).reshape(n_kv, -1, d)[:, :L]          # [kv head, key, d]
        v = vc[pages].permute(1, 0, 2, 3).reshape(n_kv, -1, d)[:, :L]
        for h in range(n_q):
            p = torch.softmax((k[h // group] @ q[r, h]) * scale, dim=0)
            out[r, h] = p @ v[h // group]
    return out


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_no_alloc_entry_point_matches_the_regular_one_twice_in_a_row(dtype):
    B, n_q, n_kv, d, P, max_split = 6, 32, 8, 128, 16, 4
    scale = d ** -0.5
    lib = _libs(d)
    assert lib.msgl_attention_noalloc_capacity_floats() == 4 * 1024 * 1024
    stream = torch.cuda.current_stream().cuda_stream
    for seed in (1, 2):                                  # the second call finds the first call's leftovers
        c = _case(seed, B, n_q, n_kv, d, P, dtype, max_split)
        want = _regular(c, n_kv, P, max_split, scale)
        out = torch.full_like(c["q"], float("nan"))
        before = torch.cuda.memory_allocated()
        rc = lib.msgl_attention_decode_noalloc(
            c["q"].data_ptr(), out.data_ptr(), c["kc"].data_ptr(), c["vc"].data_ptr(), c["q_start"].data_ptr(),
            c["kv_len"].data_ptr(), c["bt"].data_ptr(), c["nsplit"].data_ptr(), B, n_q, n_kv, d, P, c["bt"].stride(0), 0,
            max_split, scale, 1 if dtype == torch.bfloat16 else 0, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        tol = dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=2e-5)
        torch.testing.assert_close(out.float(), want.float(), **tol)
        # and against the formula itself, so that a fault the two entry points had in common would show
        torch.testing.assert_close(out.float(), _restated(c, n_kv, P, scale), **tol)


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    lib = _libs(128)
    # 16 splits * 1024 requests * 32 heads * 130 floats is far beyond the built-in 4 Mi floats
    rc = lib.msgl_attention_decode_noalloc(None, None, None, None, None, None, None, 1, 1024, 32, 8, 128, 16, 1, 0, 16,
                                           0.1, 1, None)
    assert rc == 5
