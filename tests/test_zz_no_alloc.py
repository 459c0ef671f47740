"""The allocation-free RMSNorm-backward entry point (``b200_rmsnorm_bwd_noalloc``), called through
its exported C symbol the way a caller that must not allocate would use it: every buffer it
touches is created up front, then the function runs twice in a row on different data and must
reproduce the regular entry point (which takes its scratch from the caller) both times.

Collected last on purpose: a failure here leaves the rest of a stop-at-first-failure run intact.
"""
import ctypes

import pytest
import torch

from create_llm_by_cupy_b200.ops import native

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


@pytest.mark.parametrize("M,H,with_add", [(777, 2048, True), (64, 4096, False), (50, 100, True)])
def test_noalloc_matches_regular_entry_point_twice(M, H, with_add):
    lib = native.lib()
    native.status_tensor()
    fn = lib.b200_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    dev = "cuda"
    stream = native.stream_ptr()
    rows = lib.b200_rmsnorm_bwd_partial_rows(M)
    # everything is allocated before the calls under test
    gamma = (torch.randn(H, device=dev) * 0.1 + 1).to(torch.bfloat16)
    sets = []
    for seed in (0, 1):
        g = torch.Generator(device=dev).manual_seed(seed)
        x = torch.randn(M, H, device=dev, generator=g).to(torch.bfloat16)
        dy = torch.randn(M, H, device=dev, generator=g).to(torch.bfloat16)
        add = torch.randn(M, H, device=dev, generator=g).to(torch.bfloat16) if with_add else None
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
        sets.append((x, dy, add, rstd))
    partial = torch.empty(rows, H, dtype=torch.float32, device=dev)
    ref_dx, ref_dg = torch.empty(M, H, dtype=torch.bfloat16, device=dev), torch.empty(H, dtype=torch.bfloat16, device=dev)
    out_dx, out_dg = torch.empty_like(ref_dx), torch.empty_like(ref_dg)
    kept = [tuple(torch.empty_like(t) for t in (ref_dx, ref_dg, out_dx, out_dg)) for _ in sets]
    import gc
    gc.collect()                              # garbage of earlier tests must not be freed in the middle of the measurement
    # Warm the entry point once: under lazy module loading the first call on a device may load the module
    # that holds the built-in scratch array (that is when the driver materialises its 4.75 MiB).
    x0, dy0, add0, rstd0 = sets[0]
    assert fn(_ptr(dy0), _ptr(x0), _ptr(gamma), _ptr(rstd0), _ptr(add0), _ptr(out_dx), _ptr(out_dg), M, H, 0, stream) == 0
    assert lib.b200_rmsnorm_bwd(_ptr(dy0), _ptr(x0), _ptr(gamma), _ptr(rstd0), _ptr(add0), _ptr(ref_dx), _ptr(ref_dg),
                                _ptr(partial), M, H, 0, stream) == 0
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    # torch's counter only sees torch's own allocator; the driver's free-byte count also sees a raw
    # cudaMalloc made inside the library
    free_before = torch.cuda.mem_get_info()[0]
    for i, (x, dy, add, rstd) in enumerate(sets):      # two calls in a row share the built-in scratch
        rc = lib.b200_rmsnorm_bwd(_ptr(dy), _ptr(x), _ptr(gamma), _ptr(rstd), _ptr(add), _ptr(ref_dx), _ptr(ref_dg),
                                  _ptr(partial), M, H, 0, stream)
        assert rc == 0
        rc = fn(_ptr(dy), _ptr(x), _ptr(gamma), _ptr(rstd), _ptr(add), _ptr(out_dx), _ptr(out_dg), M, H, 0, stream)
        assert rc == 0
        for dst, src in zip(kept[i], (ref_dx, ref_dg, out_dx, out_dg)):
            dst.copy_(src)                    # into buffers made beforehand: nothing is allocated in this loop
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before, "device memory was allocated or freed during the calls"
    assert torch.cuda.memory_allocated() == before
    for r_dx, r_dg, o_dx, o_dg in kept:
        scale = r_dx.float().abs().max().item()
        assert (o_dx.float() - r_dx.float()).abs().max().item() <= 2e-2 + 2e-2 * scale
        gscale = r_dg.float().abs().max().item()
        assert (o_dg.float() - r_dg.float()).abs().max().item() <= 2e-2 + 2e-2 * gscale


def test_noalloc_rejects_sizes_beyond_its_scratch():
    lib = native.lib()
    H = 4096 + 8
    z = torch.zeros(4, H, dtype=torch.bfloat16, device="cuda")
    r = torch.ones(4, device="cuda")
    g = torch.ones(H, dtype=torch.bfloat16, device="cuda")
    rc = lib.b200_rmsnorm_bwd_noalloc(_ptr(z), _ptr(z), _ptr(g), _ptr(r), _ptr(None), _ptr(z.clone()), _ptr(g.clone()),
                                      4, H, 0, native.stream_ptr())
    assert rc != 0
    torch.cuda.synchronize()
