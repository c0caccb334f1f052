"""GPU: the allocation-free force / virial entry point against the regular one.

mb_edge_geometry_bwd_static serves callers that bind the C ABI from an engine which owns all device memory
itself and may not (or cannot) allocate inside its per-step force callback: it keeps its scratch in a fixed
array inside the library.  It must give the same forces-gradient and strain-gradient as mb_edge_geometry_bwd,
call after call, although every call reuses the same scratch array with the previous call's contents in it.
This file sorts last on purpose, so a run that stops at the first failure has executed every other test."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(seed):
    from matris_b200 import ops, workloads
    from matris_b200.graph import build_batched_graph
    crystals = workloads.random_crystals(3, seed=seed)
    g = build_batched_graph([c.numbers for c in crystals], [c.cart for c in crystals], [c.lattice for c in crystals])
    vec, length, unit = ops.edge_geometry_fwd(g.cart32, g.lattice32, g.atom_struct, g.center, g.neighbor, g.image)
    gen = torch.Generator().manual_seed(seed)
    dlen = torch.randn(g.n_edges, generator=gen).cuda()
    dunit = torch.randn(g.n_edges, 3, generator=gen).cuda()
    return g, vec, length, unit, dlen, dunit


def _static(g, vec, length, unit, dlen, dunit):
    """Call the entry point through the C ABI; also report whether the device's free memory moved during the call."""
    from matris_b200 import _lib
    dcart = torch.full((g.n_atoms, 3), float("nan"), device="cuda")
    dstrain = torch.full((g.n_struct, 9), float("nan"), device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    status = _lib.load().mb_edge_geometry_bwd_static(
        g.n_atoms, g.n_struct, g.n_edges, g.edge_ptr.data_ptr(), g.atom_ptr.data_ptr(), g.rev.data_ptr(),
        vec.data_ptr(), length.data_ptr(), unit.data_ptr(), dlen.data_ptr(), dunit.data_ptr(), dcart.data_ptr(),
        dstrain.data_ptr(), st)
    torch.cuda.synchronize()
    return status, dcart, dstrain.view(-1, 3, 3), torch.cuda.mem_get_info()[0] - free_before


def test_static_scratch_entry_matches_regular_entry_twice_in_a_row():
    from matris_b200 import ops
    for seed in (31, 32):  # two calls in a row; the second finds the first call's values in the scratch array
        g, vec, length, unit, dlen, dunit = _inputs(seed)
        ref_dcart, ref_dstrain, _ = ops.edge_geometry_bwd(g.n_atoms, g.n_struct, g.edge_ptr, g.atom_ptr, g.rev, vec,
                                                          length, unit, dlen, dunit)
        if seed == 31:  # the very first call on the device does the one-time address look-up
            _static(g, vec, length, unit, dlen, dunit)
        status, dcart, dstrain, free_delta = _static(g, vec, length, unit, dlen, dunit)
        assert status == 0
        assert free_delta == 0, "the entry point must not allocate or free device memory"
        # same kernels, same summation order: the tolerance of the geometry tests (1e-4 relative) is far above this
        assert torch.isfinite(dcart).all() and torch.isfinite(dstrain).all()
        np.testing.assert_allclose(dcart.cpu().numpy(), ref_dcart.cpu().numpy(), rtol=1e-4, atol=1e-5)
        np.testing.assert_allclose(dstrain.cpu().numpy(), ref_dstrain.cpu().numpy(), rtol=1e-4, atol=1e-4)
        assert torch.equal(dcart, ref_dcart) and torch.equal(dstrain, ref_dstrain)


def test_static_scratch_entry_rejects_oversized_problems():
    from matris_b200 import _lib
    g, vec, length, unit, dlen, dunit = _inputs(33)
    lib = _lib.load()
    too_many_edges = (1 << 19) + 1
    dummy = torch.zeros(16, device="cuda")
    status = lib.mb_edge_geometry_bwd_static(g.n_atoms, g.n_struct, too_many_edges, g.edge_ptr.data_ptr(),
                                             g.atom_ptr.data_ptr(), g.rev.data_ptr(), vec.data_ptr(),
                                             length.data_ptr(), unit.data_ptr(), dlen.data_ptr(), dunit.data_ptr(),
                                             dummy.data_ptr(), dummy.data_ptr(), None)
    assert status == 6 and b"capacity" in lib.mb_status_string(status)
    status = lib.mb_edge_geometry_bwd_static((1 << 15) + 1, g.n_struct, g.n_edges, g.edge_ptr.data_ptr(),
                                             g.atom_ptr.data_ptr(), g.rev.data_ptr(), vec.data_ptr(),
                                             length.data_ptr(), unit.data_ptr(), dlen.data_ptr(), dunit.data_ptr(),
                                             dummy.data_ptr(), dummy.data_ptr(), None)
    assert status == 6
