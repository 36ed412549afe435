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
