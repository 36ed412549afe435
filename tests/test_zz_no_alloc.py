"""The allocation-free grouped GEMM entry point against the regular one.

`b200_moe_grouped_gemm_noalloc` exists for hosts that cannot hand the library any scratch
memory (no allocator, or allocation forbidden at that moment); it keeps its token-tile table in
a fixed device array inside the library.  Both entry points run the same GEMM kernel, so their
outputs must be bit-identical.  The array is shared and keeps stale entries from earlier calls,
hence two calls in a row with different routings (the second needs fewer tiles than the first).
This file sorts last on purpose: a failure here cannot hide any other test.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _case(T, E, k, H, I, seed):
    g = torch.Generator().manual_seed(seed)
    hidden = torch.randn(T, H, generator=g).to(BF).cuda()
    gate_up = (torch.randn(E, 2 * I, H, generator=g) * 0.05).to(BF).cuda()
    down = (torch.randn(E, H, I, generator=g) * 0.05).to(BF).cuda()
    sel = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).cuda()
    rw = torch.rand(T, k, generator=g)
    rw = (rw / rw.sum(-1, keepdim=True)).to(BF).cuda()
    return hidden, gate_up, down, sel, rw


def _noalloc(lib_mod, x, w, row_scale, cu_seqlens, n_out, mode):
    out = torch.empty((x.shape[0], n_out), device=x.device, dtype=BF)
    rc = lib_mod.load().b200_moe_grouped_gemm_noalloc(
        x.data_ptr(), w.data_ptr(), lib_mod.ptr(row_scale), out.data_ptr(), cu_seqlens.data_ptr(), x.shape[0],
        w.shape[0], n_out, x.shape[1], out.stride(0), mode, lib_mod.current_stream())
    assert rc == 0, f"b200_moe_grouped_gemm_noalloc returned {rc}"
    return out


def test_noalloc_grouped_gemm_matches_regular_entry_point_twice():
    from vexact_b200 import _lib
    from vexact_b200.fused_moe import _grouped_gemm, _permute

    for (T, E, k, H, I, seed) in [(300, 32, 4, 512, 256, 1), (40, 32, 4, 512, 256, 2)]:
        hidden, gate_up, down, sel, rw = _case(T, E, k, H, I, seed)
        plan = _permute(sel, rw, hidden, E)
        h_ref = _grouped_gemm(plan["x_perm"], gate_up, plan["row_scale"], plan, I, mode=1)
        y_ref = _grouped_gemm(h_ref, down, None, plan, H, mode=0)
        h = _noalloc(_lib, plan["x_perm"], gate_up, plan["row_scale"], plan["cu_seqlens"], I, mode=1)
        y = _noalloc(_lib, h, down, None, plan["cu_seqlens"], H, mode=0)
        torch.cuda.synchronize()
        assert torch.equal(h, h_ref), "fc1 (+SwiGLU) differs between the two entry points"
        assert torch.equal(y, y_ref), "fc2 differs between the two entry points"
    assert _lib.read_status()[0] == 0


def test_noalloc_rejects_sizes_beyond_its_fixed_table():
    from vexact_b200 import _lib

    lib = _lib.load()
    x = torch.zeros((8, 64), device="cuda", dtype=BF)
    cu = torch.zeros(2050, device="cuda", dtype=torch.int32)
    # too many groups, and too many rows for the 4095-tile table: both refused with -2, nothing launched
    assert lib.b200_moe_grouped_gemm_noalloc(x.data_ptr(), x.data_ptr(), None, x.data_ptr(), cu.data_ptr(), 8, 2049,
                                             64, 64, 64, 0, _lib.current_stream()) == -2
    assert lib.b200_moe_grouped_gemm_noalloc(x.data_ptr(), x.data_ptr(), None, x.data_ptr(), cu.data_ptr(),
                                             64 * 5000, 8, 64, 64, 64, 0, _lib.current_stream()) == -2
    assert lib.b200_moe_grouped_gemm_noalloc(None, None, None, None, None, 8, 8, 64, 64, 64, 0, None) == -1


def test_noalloc_clips_an_inconsistent_cu_seqlens_and_reports_it():
    """cu_seqlens is caller data: groups that overrun x_rows, start below zero or decrease must never
    turn into stores outside `out`.  `out` sits between two canary pads larger than any overrun fed in,
    so even a wrong clip would only write memory this test owns."""
    from vexact_b200 import _lib

    rows, K, N, G, pad = 128, 64, 128, 4, 64
    g = torch.Generator().manual_seed(5)
    x = torch.randn(rows, K, generator=g).to(BF).cuda()
    w = (torch.randn(G, N, K, generator=g) * 0.1).to(BF).cuda()
    cases = {
        "overrun": ([0, 32, 64, 96, 160], [0, 32, 64, 96, 128], 3),      # last group runs 32 rows past x_rows
        "decreasing": ([0, 64, 32, 96, 128], None, 1),                   # group 1 (64 -> 32) dropped
        "negative": ([-16, 32, 64, 96, 128], [0, 32, 64, 96, 128], 0),   # group 0 clipped to rows 0..32
    }
    for name, (bad, clipped, bad_group) in cases.items():
        buf = torch.full((pad + rows + pad, N), 7.0, device="cuda", dtype=BF)
        out = buf[pad:pad + rows]
        out.zero_()
        cu = torch.tensor(bad, dtype=torch.int32, device="cuda")
        rc = _lib.load().b200_moe_grouped_gemm_noalloc(x.data_ptr(), w.data_ptr(), None, out.data_ptr(), cu.data_ptr(),
                                                       rows, G, N, K, N, 0, _lib.current_stream())
        assert rc == 0
        torch.cuda.synchronize()
        status = _lib.read_status()
        assert status[0] == 2 and status[1] == bad_group, f"{name}: status {status}"
        assert bool((buf[:pad] == 7.0).all()) and bool((buf[pad + rows:] == 7.0).all()), f"{name}: canary overwritten"
        if clipped is not None:
            # same bits as a call that was handed the clipped table in the first place
            ref = _noalloc(_lib, x, w, None, torch.tensor(clipped, dtype=torch.int32, device="cuda"), N, 0)
            torch.cuda.synchronize()
            assert _lib.read_status()[0] == 0
            assert torch.equal(out, ref), f"{name}: rows differ from a call with the clipped table"
        else:
            # group 1 is dropped; groups 0 (rows 0..64) and 2 (rows 32..96) overlap on rows 32..64, so only
            # the rows a single group owns have a defined value
            for gi, a, b in [(0, 0, 32), (2, 64, 96), (3, 96, 128)]:
                torch.testing.assert_close(out[a:b].float(), x[a:b].float() @ w[gi].float().t(), rtol=2 ** -6,
                                           atol=1e-2)
