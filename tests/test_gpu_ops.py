"""GPU: every kernel behind the C ABI against plain PyTorch (CPU, float64 where the
formula allows) evaluations of the reference's expressions (oracle.model)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from functools import partial

import gpu_util
from gpu_util import dev

# feature tensors: the bound scales with the reference's magnitude
report = partial(gpu_util.report, scaled=True)

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from matris_b200 import ops as o
    return o


def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).float()


# ---------------------------------------------------------------- GEMM
# Split-operand tensor-core cores: 3xTF32 carries 22 mantissa bits per operand pair and sits at the float32 rounding
# floor; 3xBF16 (the default) carries 16, so one GEMM output differs from float64 by about 2^-16 sqrt(K) |a| |w|.
# The bounds below are relative to the largest output (report(..., scaled=True)).
TOL_TF32, TOL_BF16 = 1e-5, 6e-5

@pytest.mark.parametrize("n_rows", [1, 77, 128, 1000])
def test_gemm_plain_and_bias_act(ops, n_rows):
    x, W, b = rnd(n_rows, 256, seed=1), rnd(256, 256, seed=2, scale=0.1), rnd(256, seed=3)
    y = ops.linear(dev(x), dev(W), bias=dev(b), out_act=1)
    report(f"gemm bias+silu R={n_rows}", y, F.silu(F.linear(x.double(), W.double(), b.double())), TOL_BF16)
    y = ops.linear(dev(x), dev(W), in_act=1)
    report(f"gemm silu-on-load R={n_rows}", y, F.linear(F.silu(x.double()), W.double()), TOL_BF16)


def test_gemm_gathered_concat_four_segments(ops):
    R, n1, n2 = 700, 90, 40
    e, node, atom = rnd(R, 128, seed=4), rnd(n1, 128, seed=5), rnd(n2, 128, seed=6)
    g = torch.Generator().manual_seed(0)
    tgt, src, ctr = (torch.randint(0, n1, (R,), generator=g), torch.randint(0, n1, (R,), generator=g),
                     torch.randint(0, n2, (R,), generator=g))
    W, b = rnd(256, 512, seed=7, scale=0.05), rnd(256, seed=8)
    out = torch.empty(R, 256, device="cuda")
    de, dn, da = dev(e), dev(node), dev(atom)
    srcs = [ops.S(de), ops.S(da, dev(ctr, torch.int32)), ops.S(dn, dev(tgt, torch.int32)), ops.S(dn, dev(src, torch.int32))]
    dW, db = dev(W), dev(b)
    ops.gemm(R, [ops.B(srcs, dW, w_row=128 * j, bias=db, bias_off=128 * j, out=out, out_col=128 * j) for j in (0, 1)])
    x = torch.cat([e, atom[ctr], node[tgt], node[src]], 1).double()
    report("gemm gather-cat K=512", out, F.linear(x, W.double(), b.double()), TOL_BF16)


def test_gemm_gate_residual_scale(ops):
    R = 300
    x, W, z, res, rw = rnd(R, 128, seed=1), rnd(128, 128, seed=2, scale=0.1), rnd(R, 128, seed=3), rnd(R, 128, seed=4), rnd(128, seed=5)
    y = ops.linear(dev(x), dev(W), gate=dev(z), scale=0.5)
    zz = z.double().requires_grad_(True)
    (sg,) = torch.autograd.grad(F.silu(zz).sum(), zz)
    report("gemm * silu'(gate) * 0.5", y, F.linear(x.double(), W.double()) * sg * 0.5, TOL_BF16)
    y = ops.linear(dev(x), dev(W), res=dev(res), res_w=dev(rw))
    report("gemm + w*res", y, F.linear(x.double(), W.double()) + rw.double() * res.double(), TOL_BF16)


def test_gemm_scatter_modes(ops):
    R, n = 900, 37
    x, W = rnd(R, 256, seed=1), rnd(128, 256, seed=2, scale=0.1)
    idx = torch.randint(0, n, (R,), generator=torch.Generator().manual_seed(1))
    base = rnd(n, 128, seed=3)
    out = dev(base.clone())
    dx = dev(x)
    ops.gemm(R, [ops.B([ops.S(dx, None, 0), ops.S(dx, None, 128)], dev(W), out=out, out_idx=dev(idx, torch.int32),
                       mode=ops.OUT_ATOMIC)])
    want = base.double().index_add_(0, idx, F.linear(x.double(), W.double()))
    report("gemm atomic scatter-add", out, want, 1e-4)
    base2 = rnd(R, 128, seed=4)
    out2 = dev(base2.clone())
    ops.gemm(R, [ops.B([ops.S(dx, None, 0), ops.S(dx, None, 128)], dev(W), out=out2, mode=ops.OUT_ADD)])
    report("gemm accumulate", out2, base2.double() + F.linear(x.double(), W.double()), TOL_BF16)


def test_gemm_large_mixed_direct_and_gathered_sources(ops):
    """Many tiles per CTA of the persistent kernel with a mix of un-indexed and gathered A sources, a ragged last
    tile and a column offset, against the fp32 SIMT core."""
    R, n1 = 20000 + 37, 700
    x, node = rnd(R, 256, seed=21) * 2, rnd(n1, 128, seed=22) * 2
    g = torch.Generator().manual_seed(3)
    idx = torch.randint(0, n1, (R,), generator=g)
    W, b = rnd(256, 384, seed=23, scale=0.2), rnd(256, seed=24)
    dx, dn, dW, db, di = dev(x), dev(node), dev(W), dev(b), dev(idx, torch.int32)
    outs = {}
    for mode in ("simt", "tcgen05", "tcgen05_tf32"):
        ops.set_gemm_mode(mode)
        out = torch.zeros(R, 256, device="cuda")
        srcs = [ops.S(dx, None, 128, 1), ops.S(dn, di), ops.S(dx, None, 0)]
        ops.gemm(R, [ops.B(srcs, dW, w_row=128 * j, bias=db, bias_off=128 * j, out=out, out_col=128 * j) for j in (0, 1)])
        assert ops.gemm_status() == 0
        outs[mode] = out.cpu()
    ops.set_gemm_mode("tcgen05")
    report("tcgen05 3xBF16 (direct + gathered A, 157 tiles) vs simt", outs["tcgen05"], outs["simt"], TOL_BF16)
    report("tcgen05 3xTF32 (direct + gathered A, 157 tiles) vs simt", outs["tcgen05_tf32"], outs["simt"], TOL_TF32)


@pytest.mark.parametrize("n_rows", [100, 148 * 128 + 77, 148 * 128 * 3 + 5])
def test_gemm_column_blocks_sharing_one_a_operand(ops, n_rows):
    """The shape of the gated MLP's input gradient: every column block reads the same K = 256 rows (the persistent
    kernel then converts them once per row tile), one block stored with a residual, three scattered with atomics to
    different targets; one, several and an odd number of row tiles per CTA, ragged last tile.  And K = 128 with two
    column blocks, which shares the operand in the 3xTF32 form too.  Against the fp32 SIMT core."""
    R, n1 = n_rows, 997
    x, W = rnd(R, 256, seed=31), rnd(512, 256, seed=32, scale=0.1)
    res, rw = rnd(R, 128, seed=33), rnd(128, seed=34)
    g = torch.Generator().manual_seed(R)
    idx = [dev(torch.randint(0, n1, (R,), generator=g), torch.int32) for _ in range(3)]
    dx, dW, dres, drw = dev(x), dev(W), dev(res), dev(rw)
    outs = {}
    for mode in ("simt", "tcgen05", "tcgen05_tf32"):
        ops.set_gemm_mode(mode)
        edge = torch.empty(R, 128, device="cuda")
        acc = [torch.zeros(n1, 128, device="cuda") for _ in range(2)]
        srcs = [ops.S(dx, None, 0), ops.S(dx, None, 128)]
        ops.gemm(R, [ops.B(srcs, dW, w_row=0, out=edge, res=dres, res_w=drw),
                     ops.B(srcs, dW, w_row=128, out=acc[0], out_idx=idx[0], mode=ops.OUT_ATOMIC),
                     ops.B(srcs, dW, w_row=256, out=acc[1], out_idx=idx[1], mode=ops.OUT_ATOMIC),
                     ops.B(srcs, dW, w_row=384, out=acc[1], out_idx=idx[2], mode=ops.OUT_ATOMIC)])
        y = ops.linear(dx[:, :128].contiguous(), dW[:256, :128].contiguous(), out_act=1)
        assert ops.gemm_status() == 0
        outs[mode] = [edge.cpu(), acc[0].cpu(), acc[1].cpu(), y.cpu()]
    ops.set_gemm_mode("tcgen05")
    # the scatter targets sum about R / 997 rows each: the bound scales with the largest sum
    for i, name in enumerate(("stored block + residual", "scatter 1", "scatter 2 + 3", "K = 128, two blocks, SiLU")):
        report(f"shared A R={R}: 3xBF16 vs simt, {name}", outs["tcgen05"][i], outs["simt"][i], TOL_BF16)
        report(f"shared A R={R}: 3xTF32 vs simt, {name}", outs["tcgen05_tf32"][i], outs["simt"][i], TOL_TF32)
    want = F.linear(x.double(), W[:128].double()) + rw.double() * res.double()
    report(f"shared A R={R}: 3xBF16 vs float64, stored block", outs["tcgen05"][0], want, TOL_BF16)


def test_status_word_copy_in_stream_order(ops):
    flag = torch.full((1,), 7, dtype=torch.int32).pin_memory()
    x, W = dev(rnd(300, 128, seed=1)), dev(rnd(128, 128, seed=2))
    ops.linear(x, W)
    ops.gemm_status_async(flag)
    torch.cuda.synchronize()
    assert int(flag[0]) == 0 and ops.gemm_status() == 0


def test_tensor_core_gemm_matches_fp32_simt(ops):
    """The tensor-core cores (3xBF16 and 3xTF32, persistent and one-tile) against the exact-fp32 SIMT core on the same
    descriptors, all epilogue paths."""
    R, n1 = 5000, 300
    e, node = rnd(R, 128, seed=4) * 3, rnd(n1, 128, seed=5) * 3
    g = torch.Generator().manual_seed(0)
    tgt, src = torch.randint(0, n1, (R,), generator=g), torch.randint(0, n1, (R,), generator=g)
    W, b, z, res, rw = rnd(256, 384, seed=7, scale=0.2), rnd(256, seed=8), rnd(R, 256, seed=9), rnd(R, 256, seed=10), rnd(128, seed=11)
    de, dn, dW, db, dz, dres, drw = dev(e), dev(node), dev(W), dev(b), dev(z), dev(res), dev(rw)
    it, is_ = dev(tgt, torch.int32), dev(src, torch.int32)
    outs = {}
    for mode in ("simt", "tcgen05", "tcgen05_tile", "tcgen05_tf32"):
        ops.set_gemm_mode(mode)
        out = torch.zeros(R, 256, device="cuda")
        acc = torch.zeros(n1, 128, device="cuda")
        srcs = [ops.S(de, None, 0, 1), ops.S(dn, it), ops.S(dn, is_)]
        ops.gemm(R, [ops.B(srcs, dW, w_row=128 * j, bias=db, bias_off=128 * j, gate=dz, gate_col=128 * j, res=dres,
                           res_col=128 * j, res_w=drw, out=out, out_col=128 * j, scale=0.5) for j in (0, 1)])
        ops.gemm(R, [ops.B(srcs, dW, out=acc, out_idx=it, mode=ops.OUT_ATOMIC)])
        assert ops.gemm_status() == 0
        outs[mode] = (out.cpu(), acc.cpu())
    ops.set_gemm_mode("tcgen05")
    report("tcgen05 3xBF16 vs simt: fused epilogue", outs["tcgen05"][0], outs["simt"][0], TOL_BF16)
    report("tcgen05 3xBF16 vs simt: atomic scatter", outs["tcgen05"][1], outs["simt"][1], TOL_BF16)
    report("tcgen05 3xTF32 vs simt: fused epilogue", outs["tcgen05_tf32"][0], outs["simt"][0], TOL_TF32)
    report("tcgen05 3xTF32 vs simt: atomic scatter", outs["tcgen05_tf32"][1], outs["simt"][1], TOL_TF32)
    report("tcgen05_tile vs simt: fused epilogue", outs["tcgen05_tile"][0], outs["simt"][0], 1e-5)
    report("tcgen05_tile vs simt: atomic scatter", outs["tcgen05_tile"][1], outs["simt"][1], 1e-5)
    x = torch.cat([torch.nn.functional.silu(e), node[tgt], node[src]], 1).double()
    want = torch.nn.functional.linear(x, W.double(), b.double())
    zz = z.double().requires_grad_(True)
    (sg,) = torch.autograd.grad(torch.nn.functional.silu(zz).sum(), zz)
    want = (want * sg + torch.cat([rw, rw]).double() * res.double()) * 0.5
    report("tcgen05 3xBF16 vs float64", outs["tcgen05"][0], want, TOL_BF16)
    report("tcgen05 3xTF32 vs float64", outs["tcgen05_tf32"][0], want, TOL_TF32)


# ---------------------------------------------------------------- fused gated MLP
def _gated_weights(k, seed):
    from types import SimpleNamespace
    w1, b1 = rnd(256, k, seed=seed, scale=k ** -0.5), rnd(256, seed=seed + 1, scale=0.1)
    w2, b2 = rnd(256, 128, seed=seed + 2, scale=128 ** -0.5), rnd(256, seed=seed + 3, scale=0.1)
    nc, ng = 1 + 0.1 * rnd(128, seed=seed + 4), 1 + 0.1 * rnd(128, seed=seed + 5)
    host = SimpleNamespace(w1=w1, b1=b1, w2=w2, b2=b2, nc=nc, ng=ng)
    device = SimpleNamespace(**{k_: dev(v) for k_, v in vars(host).items()})
    return host, device


def _gated_ref(hp, x):
    """GatedMLP.forward (matris/model/functions.py:300-311) in float64 on the concatenated input x."""
    x = x.double()
    z1 = F.linear(x, hp.w1.double(), hp.b1.double())
    a = F.silu(z1)
    z2 = torch.cat([F.linear(a[:, :128], hp.w2[:128].double(), hp.b2[:128].double()),
                    F.linear(a[:, 128:], hp.w2[128:].double(), hp.b2[128:].double())], 1)
    return z1, z2, _gate_ref(z2, hp.nc.double(), hp.ng.double())


@pytest.mark.parametrize("n_rows", [1, 127, 128, 129, 1000, 148 * 128 + 77, 148 * 128 * 2 + 5])
def test_gated_mlp_fwd_row_counts(ops, n_rows):
    """One to many tiles per CTA, ragged last tiles, K = 384, all outputs requested, against float64."""
    hp, dp = _gated_weights(384, seed=31)
    x = rnd(n_rows, 384, seed=32)
    res, rw = rnd(n_rows, 128, seed=33), rnd(128, seed=34)
    dx = dev(x)
    z1, z2, h, out2 = ops.gated_mlp_fwd(dp, n_rows, [ops.S(dx, None, 128 * s) for s in range(3)], res=dev(res),
                                        res_w=dev(rw))
    assert ops.gemm_status() == 0
    r1, r2, rh = _gated_ref(hp, x)
    report(f"gated_mlp_fwd z1 R={n_rows}", z1, r1, TOL_BF16)
    report(f"gated_mlp_fwd z2 R={n_rows}", z2, r2, TOL_BF16)
    report(f"gated_mlp_fwd h R={n_rows}", h, rh, TOL_BF16)
    report(f"gated_mlp_fwd out2 R={n_rows}", out2, rh + rw.double() * res.double(), TOL_BF16)


@pytest.mark.parametrize("k", [128, 256, 384, 512])
def test_gated_mlp_fwd_gathered_sources_and_output_subsets(ops, k):
    """Gathered and direct K segments (one of them through SiLU on load), and every combination of optional outputs:
    without z1 / z2 (the no-save path), h only, out2 only."""
    R, n1 = 3000 + 19, 211
    hp, dp = _gated_weights(k, seed=41)
    edge, node = rnd(R, 128, seed=42), rnd(n1, 128, seed=43)
    g = torch.Generator().manual_seed(k)
    idx = [torch.randint(0, n1, (R,), generator=g) for _ in range(3)]
    de, dn = dev(edge), dev(node)
    parts, srcs = [F.silu(edge)], [ops.S(de, None, 0, 1)]
    for s in range(k // 128 - 1):
        parts.append(node[idx[s]])
        srcs.append(ops.S(dn, dev(idx[s], torch.int32)))
    x = torch.cat(parts, 1)
    res, rw = rnd(R, 128, seed=44), rnd(128, seed=45)
    r1, r2, rh = _gated_ref(hp, x)
    z1, z2, h, out2 = ops.gated_mlp_fwd(dp, R, srcs, save=False)
    assert z1 is None and z2 is None and out2 is None
    report(f"gated_mlp_fwd K={k} h (no save)", h, rh, TOL_BF16)
    z1, z2, h, out2 = ops.gated_mlp_fwd(dp, R, srcs, want_h=False, res=dev(res), res_w=None, save=True)
    assert h is None
    report(f"gated_mlp_fwd K={k} out2 only (unit residual weight)", out2, rh + res.double(), TOL_BF16)
    report(f"gated_mlp_fwd K={k} z1", z1, r1, TOL_BF16)
    report(f"gated_mlp_fwd K={k} z2", z2, r2, TOL_BF16)
    assert ops.gemm_status() == 0


def test_gated_mlp_fwd_fused_equals_composed(ops):
    """The fused kernel against the same result composed from the separate kernels on the exact-fp32 SIMT core."""
    R, n1 = 9000 + 3, 500
    hp, dp = _gated_weights(512, seed=51)
    edge, node = rnd(R, 128, seed=52) * 2, rnd(n1, 128, seed=53) * 2
    g = torch.Generator().manual_seed(9)
    idx = [dev(torch.randint(0, n1, (R,), generator=g), torch.int32) for _ in range(3)]
    de, dn = dev(edge), dev(node)
    srcs = [ops.S(de)] + [ops.S(dn, i) for i in idx]
    res, rw = dev(rnd(R, 128, seed=54)), dev(rnd(128, seed=55))
    outs = {}
    for mode in ("simt", "tcgen05_tile", "tcgen05", "tcgen05_tf32"):
        ops.set_gemm_mode(mode)
        outs[mode] = [t.cpu() for t in ops.gated_mlp_fwd(dp, R, srcs, res=res, res_w=rw)]
        assert ops.gemm_status() == 0
    ops.set_gemm_mode("tcgen05")
    for i, name in enumerate(("z1", "z2", "h", "out2")):
        report(f"gated_mlp_fwd fused 3xBF16 vs simt-composed {name}", outs["tcgen05"][i], outs["simt"][i], TOL_BF16)
        report(f"gated_mlp_fwd 3xTF32-composed vs simt-composed {name}", outs["tcgen05_tf32"][i], outs["simt"][i], TOL_TF32)
        report(f"gated_mlp_fwd 3xTF32-composed vs tile-composed {name}", outs["tcgen05_tf32"][i], outs["tcgen05_tile"][i],
               TOL_TF32)


def _ffn_weights(k, seed, bias=True):
    from types import SimpleNamespace
    host = SimpleNamespace(w1=rnd(128, k, seed=seed, scale=k ** -0.5), w2=rnd(128, 128, seed=seed + 2, scale=128 ** -0.5),
                           b1=rnd(128, seed=seed + 1, scale=0.1) if bias else None,
                           b2=rnd(128, seed=seed + 3, scale=0.1) if bias else None)
    device = SimpleNamespace(**{k_: None if v is None else dev(v) for k_, v in vars(host).items()})
    return host, device


def _ffn_ref(hp, x):
    """node_FFN / edge_FFN (matris/model/interaction_block.py:197-210) in float64."""
    z1 = F.linear(x.double(), hp.w1.double(), None if hp.b1 is None else hp.b1.double())
    return z1, F.linear(F.silu(z1), hp.w2.double(), None if hp.b2 is None else hp.b2.double())


@pytest.mark.parametrize("n_rows", [1, 127, 129, 1000, 148 * 128 + 77, 148 * 128 * 3 + 5])
def test_ffn_fwd_row_counts(ops, n_rows):
    """The plain two-layer form of the fused kernel: one, an even and an odd number of tiles per CTA, ragged last
    tiles, every output requested, against float64."""
    hp, dp = _ffn_weights(128, seed=61)
    x, res, rw = rnd(n_rows, 128, seed=62), rnd(n_rows, 128, seed=63), rnd(128, seed=64)
    z1, y, out2 = ops.ffn_fwd(dp, dev(x), res=dev(res), res_w=dev(rw))
    assert ops.gemm_status() == 0
    r1, ry = _ffn_ref(hp, x)
    report(f"ffn_fwd z1 R={n_rows}", z1, r1, TOL_BF16)
    report(f"ffn_fwd y R={n_rows}", y, ry, TOL_BF16)
    report(f"ffn_fwd out2 R={n_rows}", out2, ry + rw.double() * res.double(), TOL_BF16)


@pytest.mark.parametrize("k,bias", [(128, False), (256, True), (512, True)])
def test_ffn_fwd_output_subsets_and_modes(ops, k, bias):
    """Without z1 (the no-save path), y only, out2 only with a unit residual weight, wider inputs, no biases; and the
    same result composed from two GEMM launches in the other GEMM modes."""
    R = 5000 + 13
    hp, dp = _ffn_weights(k, seed=71, bias=bias)
    x, res = rnd(R, k, seed=72), rnd(R, 128, seed=73)
    dx, dres = dev(x), dev(res)
    r1, ry = _ffn_ref(hp, x)
    z1, y, out2 = ops.ffn_fwd(dp, dx, save=False)
    assert z1 is None and out2 is None
    report(f"ffn_fwd K={k} y (no save)", y, ry, TOL_BF16)
    z1, y, out2 = ops.ffn_fwd(dp, dx, want_y=False, res=dres, save=True)
    assert y is None
    report(f"ffn_fwd K={k} out2 only", out2, ry + res.double(), TOL_BF16)
    report(f"ffn_fwd K={k} z1", z1, r1, TOL_BF16)
    assert ops.gemm_status() == 0
    try:
        for mode, tol in (("simt", 2e-6), ("tcgen05_tile", 1e-5), ("tcgen05_tf32", TOL_TF32)):
            ops.set_gemm_mode(mode)
            z1, y, out2 = ops.ffn_fwd(dp, dx, res=dres, save=False)
            report(f"ffn_fwd K={k} composed in mode {mode}: y", y, ry, tol)
            report(f"ffn_fwd K={k} composed in mode {mode}: out2", out2, ry + res.double(), tol)
            report(f"ffn_fwd K={k} composed in mode {mode}: z1", z1, r1, tol)
            assert ops.gemm_status() == 0
    finally:
        ops.set_gemm_mode("tcgen05")


def test_bounded_wait_expiry_sets_status_and_clears(ops):
    """The failure path of the tensor-core kernels: a wait that runs out raises the status word, nothing hangs, and
    the next kernel runs normally.  The wait is made to run out by a self-test kernel that waits (a few polls) on a
    barrier nothing arrives at."""
    assert ops.gemm_status() == 0
    ops.selftest_wait_expiry()
    flag = torch.zeros(1, dtype=torch.int32).pin_memory()
    ops.gemm_status_async(flag)
    torch.cuda.synchronize()
    assert int(flag[0]) == 1
    ops.gemm_status_clear()
    x, W = rnd(300, 128, seed=1), rnd(128, 128, seed=2)
    y = ops.linear(dev(x), dev(W))
    report("gemm after an expired wait", y, F.linear(x.double(), W.double()), 2e-5)
    assert ops.gemm_status() == 0
    ops.selftest_wait_expiry()
    assert ops.gemm_status() == 1 and ops.gemm_status() == 0  # the synchronous read clears the word


def test_timed_mma_rate_is_plausible(ops):
    tf32, ms = ops.mma_rate("tf32", 4000)
    bf16, _ = ops.mma_rate("bf16", 4000)
    print(f"tcgen05.mma issue rate: tf32 {tf32:.0f} TFLOP/s, bf16 {bf16:.0f} TFLOP/s ({ms:.2f} ms)")
    assert 300 < tf32 < 1400 and 1.7 < bf16 / tf32 < 2.3
    assert ops.gemm_status() == 0


# ---------------------------------------------------------------- row-wise
def _gate_ref(z, wc, wg):
    c = F.rms_norm(z[:, :128], (128,), wc, torch.finfo(torch.float32).eps)
    g = F.rms_norm(z[:, 128:], (128,), wg, torch.finfo(torch.float32).eps)
    return F.silu(c) * torch.sigmoid(g)


def test_gate_fwd_bwd(ops):
    R = 333
    z, wc, wg, dh, res, rw = rnd(R, 256, seed=1), 1 + 0.1 * rnd(128, seed=2), 1 + 0.1 * rnd(128, seed=3), rnd(R, 128, seed=4), rnd(R, 128, seed=5), rnd(128, seed=6)
    h, out2 = ops.gate_fwd(dev(z), dev(wc), dev(wg), res=dev(res), res_w=dev(rw))
    zz = z.double().requires_grad_(True)
    ref = _gate_ref(zz, wc.double(), wg.double())
    report("gate_fwd h", h, ref, 2e-6)
    report("gate_fwd h + w*res", out2, ref + rw.double() * res.double(), 2e-6)
    (dz_ref,) = torch.autograd.grad(ref, zz, dh.double())
    report("gate_bwd dz", ops.gate_bwd(dev(z), dev(wc), dev(wg), dev(dh)), dz_ref, 5e-6)


def _csr(seg, n):
    order = torch.argsort(seg, stable=True)
    ptr = torch.zeros(n + 1, dtype=torch.int64)
    ptr[1:] = torch.cumsum(torch.bincount(seg, minlength=n), 0)
    return order, ptr


@pytest.mark.parametrize("with_emap", [False, True])
def test_seg_attn_fwd_bwd(ops, with_emap):
    from oracle.model import segment_softmax, segment_sum
    R, Nn = 500, 40
    g = torch.Generator().manual_seed(3)
    tgt = torch.sort(torch.randint(0, Nn - 2, (R,), generator=g))[0]  # grouped by target; last nodes empty
    src = torch.randint(0, Nn - 1, (R,), generator=g)
    perm, sptr = _csr(src, Nn)
    _, tptr = _csr(tgt, Nn)
    Ne = 120 if with_emap else R
    emap = torch.randint(0, Ne, (R,), generator=g) if with_emap else None
    logits, h = rnd(Ne, 256, seed=1), rnd(R, 128, seed=2)
    i32 = torch.int32
    d = dict(tgt=dev(tgt, i32), src=dev(src, i32), tptr=dev(tptr, i32), sptr=dev(sptr, i32), perm=dev(perm, i32),
             emap=None if emap is None else dev(emap, i32), lg=dev(logits), h=dev(h))
    agg_t, agg_s, stats = ops.seg_attn_fwd(Nn, d["tptr"], d["sptr"], d["perm"], d["emap"], d["lg"], d["h"])
    L = logits.double().requires_grad_(True)
    H = h.double().requires_grad_(True)
    lg_rows = L[emap] if with_emap else L
    a_s, a_t = segment_softmax(lg_rows[:, :128], src), segment_softmax(lg_rows[:, 128:], tgt)
    ref_s, ref_t = segment_sum(a_s * H, src, Nn), segment_sum(a_t * H, tgt, Nn)
    report("seg_attn_fwd agg_t", agg_t, ref_t, 5e-6)
    report("seg_attn_fwd agg_s", agg_s, ref_s, 5e-6)
    dt, ds, dh_in = rnd(Nn, 128, seed=5), rnd(Nn, 128, seed=6), rnd(Ne if with_emap else R, 128, seed=7)
    scale = 0.5 if with_emap else 1.0
    extra = (dh_in.double()[emap] if with_emap else dh_in.double()) * scale
    loss = (ref_t * dt.double()).sum() + (ref_s * ds.double()).sum() + (H * extra).sum()
    dL, dH = torch.autograd.grad(loss, [L, H])
    dh, dlg = ops.seg_attn_bwd(d["tgt"], d["src"], d["emap"], d["lg"], d["h"], agg_t, agg_s, stats, dev(dt), dev(ds),
                               dev(dh_in), d["emap"], scale)
    report("seg_attn_bwd dh", dh, dH, 1e-5)
    # the same call with the gated MLP's tail adjoint applied to the row gradient in registers: dz2 instead of dh
    z2, wc, wg = rnd(R, 256, seed=8), 1 + 0.1 * rnd(128, seed=9), 1 + 0.1 * rnd(128, seed=10)
    dz2, dlg2 = ops.seg_attn_bwd(d["tgt"], d["src"], d["emap"], d["lg"], d["h"], agg_t, agg_s, stats, dev(dt), dev(ds),
                                 dev(dh_in), d["emap"], scale, gate=(dev(z2), dev(wc), dev(wg)))
    report("seg_attn_bwd with the gate adjoint: dz2", dz2, ops.gate_bwd(dev(z2), dev(wc), dev(wg), dh), 1e-6)
    assert torch.equal(dlg2, dlg)
    if with_emap:  # per-row logits gradients are summed over rows sharing a logits row
        dlg_sum = torch.zeros(Ne, 256, dtype=torch.float64).index_add_(0, emap, dlg.cpu().double())
        report("seg_attn_bwd dlogits (summed)", dlg_sum, dL, 2e-5)
    else:
        report("seg_attn_bwd dlogits", dlg, dL, 1e-5)


@pytest.mark.parametrize("line", [False, True])
def test_seg_smooth_sum_fwd_bwd(ops, line):
    R, Nn = 400, 30
    g = torch.Generator().manual_seed(9)
    i32 = torch.int32
    h, dagg, dh0 = rnd(R, 128, seed=2), rnd(Nn, 128, seed=3), rnd(R, 128, seed=4)
    if line:
        tgt = torch.sort(torch.randint(0, Nn, (R,), generator=g))[0]
        src = torch.randint(0, Nn, (R,), generator=g)
        env = rnd(Nn, 128, seed=1)
        u2d = rev = emap = None
    else:  # atom graph: rows = directed edges in pairs, emap = bond of each edge
        nb = R // 2
        tgt = torch.sort(torch.randint(0, Nn, (R,), generator=g))[0]
        src = torch.randint(0, Nn, (R,), generator=g)
        pairing = torch.randperm(R, generator=g).view(nb, 2)
        emap = torch.empty(R, dtype=torch.int64)
        emap[pairing[:, 0]] = torch.arange(nb)
        emap[pairing[:, 1]] = torch.arange(nb)
        u2d, rev = pairing[:, 0].clone(), torch.empty(R, dtype=torch.int64)
        rev[pairing[:, 0]], rev[pairing[:, 1]] = pairing[:, 1], pairing[:, 0]
        env = rnd(nb, 128, seed=1)
    perm, sptr = _csr(src, Nn)
    _, tptr = _csr(tgt, Nn)
    E, H = env.double().requires_grad_(True), h.double().requires_grad_(True)
    s = E[src] * E[tgt] if line else E[emap]
    ref = torch.zeros(Nn, 128, dtype=torch.float64).index_add_(0, tgt, H * s)
    d_tgt, d_src = dev(tgt, i32), dev(src, i32)
    d_emap = None if line else dev(emap, i32)
    agg = ops.seg_smooth_sum_fwd(Nn, dev(tptr, i32), d_emap, d_src if line else None, dev(env), dev(h))
    report(f"seg_smooth_sum_fwd line={line}", agg, ref, 1e-5)
    dE, dH = torch.autograd.grad((ref * dagg.double()).sum(), [E, H])
    dh = dev(dh0.clone())
    ops.seg_smooth_sum_bwd_rows(d_tgt, d_src if line else None, d_emap, dev(env), dev(dagg), dh, accumulate=True)
    report(f"seg_smooth_sum_bwd_rows line={line}", dh, dh0.double() + dH, 1e-5)
    z2, wc, wg = rnd(len(tgt), 256, seed=8), 1 + 0.1 * rnd(128, seed=9), 1 + 0.1 * rnd(128, seed=10)
    dh_in = dev(dh0.clone())
    dz2 = ops.seg_smooth_sum_bwd_rows(d_tgt, d_src if line else None, d_emap, dev(env), dev(dagg), dh_in, accumulate=True,
                                      gate=(dev(z2), dev(wc), dev(wg)))
    report(f"seg_smooth_sum_bwd_rows with the gate adjoint line={line}", dz2, ops.gate_bwd(dev(z2), dev(wc), dev(wg), dh), 1e-6)
    assert torch.equal(dh_in.cpu(), dh0), "with a gate the incoming dh is read, not written"
    denv = ops.seg_smooth_sum_bwd_env(env.shape[0], dev(tptr, i32), dev(sptr, i32) if line else None, dev(perm, i32),
                                      d_tgt, d_src, None if line else dev(u2d, i32), None if line else dev(rev, i32),
                                      dev(env), dev(h), dev(dagg))
    report(f"seg_smooth_sum_bwd_env line={line}", denv, dE, 2e-5)
    if not line:
        # smoothed rows h * s as a tensor (the edge update of use_smoothed_for_delta_edge) and its adjoints
        hs = ops.mul_rows_gather(dev(h), dev(env), d_emap)
        report("mul_rows_gather", hs, (H * s).detach(), 1e-6)
        drow = rnd(R, 128, seed=9)
        E2, H2 = env.double().requires_grad_(True), h.double().requires_grad_(True)
        hs2 = H2 * E2[emap]
        both = (torch.zeros(Nn, 128, dtype=torch.float64).index_add_(0, tgt, hs2) * dagg.double()).sum() \
            + (hs2 * drow.double()).sum()
        dE2, _ = torch.autograd.grad(both, [E2, H2])
        denv2 = ops.seg_smooth_sum_bwd_env(env.shape[0], dev(tptr, i32), None, dev(perm, i32), d_tgt, d_src,
                                           dev(u2d, i32), dev(rev, i32), dev(env), dev(h), dev(dagg), drow=dev(drow))
        report("seg_smooth_sum_bwd_env with a per-row gradient", denv2, dE2, 2e-5)


def test_pair_mean_scale_small_linear_norms(ops):
    nb = 150
    g = torch.Generator().manual_seed(2)
    pairing = torch.randperm(2 * nb, generator=g).view(nb, 2)
    rev = torch.empty(2 * nb, dtype=torch.int64)
    rev[pairing[:, 0]], rev[pairing[:, 1]] = pairing[:, 1], pairing[:, 0]
    y, res, w = rnd(2 * nb, 128, seed=1), rnd(nb, 128, seed=2), rnd(128, seed=3)
    out = ops.pair_mean_res(nb, dev(pairing[:, 0], torch.int32), dev(rev, torch.int32), dev(y), dev(res), dev(w))
    report("pair_mean_res", out, 0.5 * (y[pairing[:, 0]] + y[pairing[:, 1]]).double() + w.double() * res.double(), 3e-6)
    x = rnd(500, 128, seed=4)
    report("scale_rows", ops.scale_rows(dev(x), dev(w)), x * w, 1e-7)
    base = rnd(500, 128, seed=12)
    acc = dev(base.clone())
    ops.scale_rows(dev(x), dev(w), acc, accumulate=True)
    report("scale_rows accumulate", acc, base + x * w, 2e-6)
    for k in (7, 16):
        xs, W, dy = rnd(500, k, seed=5), rnd(128, k, seed=6), rnd(500, 128, seed=7)
        report(f"small_linear_fwd k={k}", ops.small_linear_fwd(dev(xs), dev(W)), F.linear(xs.double(), W.double()), 5e-6)
        report(f"small_linear_bwd k={k}", ops.small_linear_bwd(dev(dy), dev(W)), dy.double() @ W.double(), 3e-5)
        dx = dev(xs.clone())
        ops.small_linear_bwd(dev(dy), dev(W), dx, accumulate=True)
        report(f"small_linear_bwd acc k={k}", dx, xs.double() + dy.double() @ W.double(), 3e-5)
    x, lw, lb, dy = rnd(300, 128, seed=8) * 3 + 1, 1 + 0.1 * rnd(128, seed=9), 0.1 * rnd(128, seed=10), rnd(300, 128, seed=11)
    X = x.double().requires_grad_(True)
    ref = F.layer_norm(X, (128,), lw.double(), lb.double(), 1e-5)
    report("layernorm_fwd", ops.layernorm_fwd(dev(x), dev(lw), dev(lb)), ref, 3e-6)
    report("layernorm_bwd", ops.layernorm_bwd(dev(x), dev(lw), dev(dy)), torch.autograd.grad(ref, X, dy.double())[0], 5e-6)
    X = x.double().requires_grad_(True)
    ref = F.rms_norm(X, (128,), lw.double(), torch.finfo(torch.float32).eps)
    report("rmsnorm_fwd", ops.rmsnorm_fwd(dev(x), dev(lw)), ref, 3e-6)
    report("rmsnorm_bwd", ops.rmsnorm_bwd(dev(x), dev(lw), dev(dy)), torch.autograd.grad(ref, X, dy.double())[0], 5e-6)


def test_silu_bwd_matches_reference_formula(ops):
    """grad * sigmoid(x) * (1 + x * (1 - sigmoid(x)))  (the reference's fused SiLU backward)."""
    z, dy = rnd(257, 128, seed=1) * 4, rnd(257, 128, seed=2)
    s = torch.sigmoid(z.double())
    report("silu_bwd", ops.silu_bwd(dev(dy), dev(z)), dy.double() * s * (1 + z.double() * (1 - s)), 1e-6)


def test_heads_embedding_segment_sum(ops):
    n = 200
    z, w, b = rnd(n, 256, seed=1), rnd(256, seed=2), rnd(1, seed=3)
    report("head_dot_fwd |.| k=256", ops.head_dot_fwd(dev(z), dev(w), dev(b), True),
           (F.silu(z.double()) @ w.double() + b.double()).abs(), 2e-5)
    z1 = z[:, :128].contiguous()
    Z = z1.double().requires_grad_(True)
    seg = torch.sort(torch.randint(0, 5, (n,), generator=torch.Generator().manual_seed(0)))[0]
    seed = rnd(5, seed=4)
    e = F.silu(Z) @ w[:128].double() + b.double()
    (dz,) = torch.autograd.grad((e * seed.double()[seg]).sum(), Z)
    report("head_dot_bwd seeded", ops.head_dot_bwd(dev(z1), dev(w[:128].contiguous()), dev(seed), dev(seg, torch.int32)), dz, 1e-5)
    _, ptr = _csr(seg, 5)
    x = rnd(n, seed=5)
    report("segment_sum_scalar", ops.segment_sum_scalar(5, dev(ptr, torch.int32), dev(x)),
           torch.zeros(5, dtype=torch.float64).index_add_(0, seg, x.double()), 1e-5)
    table, idx = rnd(94, 128, seed=6), torch.randint(1, 95, (n,), generator=torch.Generator().manual_seed(1))
    report("embedding", ops.embedding(dev(idx, torch.int32), -1, dev(table)), table[idx - 1], 0.0)


# ---------------------------------------------------------------- geometry and bases
def test_bessel_fwd_bwd(ops):
    from oracle.model import bessel
    nb = 400
    g = torch.Generator().manual_seed(4)
    length = torch.rand(2 * nb, generator=g) * 5.2 + 0.8          # 0.8 .. 6.0 (beyond the 4 A cutoff too)
    u2d = torch.randperm(2 * nb, generator=g)[:nb]
    fa = torch.pi * torch.arange(1, 8).float() * (1 + 0.02 * rnd(7, seed=1))
    fb = torch.pi * torch.arange(1, 8).float() * (1 + 0.02 * rnd(7, seed=2))
    ra, rb = ops.bessel_fwd(dev(u2d, torch.int32), dev(length), dev(fa), 6.0, dev(fb), 4.0, 8)
    Ld = length.double().requires_grad_(True)
    ref_a, ref_b = bessel(Ld[u2d], fa.double(), 6.0, 8), bessel(Ld[u2d], fb.double(), 4.0, 8)
    report("bessel_fwd rc=6", ra, ref_a, 3e-6)
    report("bessel_fwd rc=4", rb, ref_b, 3e-6)
    da, db = rnd(nb, 7, seed=3), rnd(nb, 7, seed=4)
    (dl,) = torch.autograd.grad((ref_a * da.double()).sum() + (ref_b * db.double()).sum(), Ld)
    report("bessel_bwd dlen", ops.bessel_bwd(dev(u2d, torch.int32), dev(length), dev(fa), 6.0, dev(fb), 4.0, 8, dev(da), dev(db)),
           dl, 3e-5)


def test_angle_basis_fwd_bwd(ops):
    from oracle.model import spherical_basis
    ne, nt = 60, 900
    g = torch.Generator().manual_seed(5)
    v = torch.randn(ne, 3, generator=g)
    unit = (v / v.norm(dim=1, keepdim=True)).float()
    lg = torch.zeros(nt, 5, dtype=torch.int64)
    lg[:, 2], lg[:, 4] = torch.randint(0, ne, (nt,), generator=g), torch.randint(0, ne, (nt,), generator=g)
    lg[:5, 4] = lg[:5, 2]                                         # collinear (theta = 0) rows
    factor = float(np.sqrt(np.float32(2.0 / 216.0)))
    basis = ops.angle_basis_fwd(dev(lg, torch.int32), dev(unit), factor, 6.0)
    U = unit.double().requires_grad_(True)
    ua, ub = U[lg[:, 2]], U[lg[:, 4]]
    theta = torch.acos((ua * ub).sum(1) * (1 - 1e-6))
    ref = spherical_basis(torch.norm(ub.detach(), dim=1), theta, torch.tensor(factor, dtype=torch.float64), 6.0)
    report("angle_basis_fwd", basis, ref, 2e-6)
    db = rnd(nt, 16, seed=1)
    (dU,) = torch.autograd.grad((ref * db.double()).sum(), U)
    # float32 evaluation of d cos(acos x)/dx loses digits near |x| -> 1 exactly as the reference's autograd does
    report("angle_basis_bwd dunit", ops.angle_basis_bwd(dev(lg, torch.int32), dev(unit), factor, 6.0, dev(db)), dU, 2e-3, rel=True)


def test_gaussian_fwd_bwd(ops):
    from oracle.model import gaussian
    nb = 400
    g = torch.Generator().manual_seed(4)
    length = torch.rand(2 * nb, generator=g) * 5.2 + 0.8
    u2d = torch.randperm(2 * nb, generator=g)[:nb]
    oa, ob = torch.linspace(0.0, 6.0, 7), torch.linspace(0.0, 4.0, 7)
    ca, cb = (-0.5 / (2.0 * (o[1] - o[0])).item() ** 2 for o in (oa, ob))
    ra, rb = ops.gaussian_fwd(dev(u2d, torch.int32), dev(length), dev(oa), ca, dev(ob), cb)
    Ld = length.double().requires_grad_(True)
    ref_a, ref_b = gaussian(Ld[u2d], oa.double()), gaussian(Ld[u2d], ob.double())
    report("gaussian_fwd rc=6", ra, ref_a, 2e-6)
    report("gaussian_fwd rc=4", rb, ref_b, 2e-6)
    da, db = rnd(nb, 7, seed=3), rnd(nb, 7, seed=4)
    (dl,) = torch.autograd.grad((ref_a * da.double()).sum() + (ref_b * db.double()).sum(), Ld)
    report("gaussian_bwd dlen", ops.gaussian_bwd(dev(u2d, torch.int32), dev(length), dev(oa), ca, dev(ob), cb, dev(da), dev(db)),
           dl, 1e-5)


def test_fourier_basis_fwd_bwd(ops):
    from oracle.model import fourier_basis
    ne, nt = 60, 900
    g = torch.Generator().manual_seed(5)
    v = torch.randn(ne, 3, generator=g)
    unit = (v / v.norm(dim=1, keepdim=True)).float()
    lg = torch.zeros(nt, 5, dtype=torch.int64)
    lg[:, 2], lg[:, 4] = torch.randint(0, ne, (nt,), generator=g), torch.randint(0, ne, (nt,), generator=g)
    lg[:5, 4] = lg[:5, 2]                                         # collinear (theta = 0) rows
    freq = torch.arange(1, 4).float() * (1 + 0.02 * rnd(3, seed=1))
    basis = ops.fourier_basis_fwd(dev(lg, torch.int32), dev(unit), dev(freq))
    U = unit.double().requires_grad_(True)
    x = (U[lg[:, 2]] * U[lg[:, 4]]).sum(1) * (1 - 1e-6)
    theta = torch.acos(x)
    ref = fourier_basis(theta, freq.double())
    # theta = acos(x) is ill-conditioned in float32 where |x| -> 1 (one ulp of x moves theta by percents there: the
    # reference's own float32 result has the same spread), so values are compared away from collinearity and the
    # collinear rows are checked for finiteness and the constant first column
    ok = (x.detach().abs() < 0.999)
    assert 5 <= int((~ok).sum()) < 60
    report("fourier_basis_fwd", basis.cpu()[ok], ref[ok], 2e-6)
    assert torch.isfinite(basis).all()
    report("fourier_basis_fwd constant column", basis[:, 0], ref[:, 0], 1e-7)
    db = rnd(nt, 7, seed=1)
    db[~ok] = 0.0
    (dU,) = torch.autograd.grad((ref * db.double()).sum(), U)
    report("fourier_basis_bwd dunit", ops.fourier_basis_bwd(dev(lg, torch.int32), dev(unit), dev(freq), dev(db)), dU, 2e-4, rel=True)


def test_edge_geometry_fwd_bwd(ops):
    from matris_b200.graph import build_batched_graph
    from matris_b200 import workloads
    crystals = workloads.random_crystals(3, seed=2)
    g = build_batched_graph([c.numbers for c in crystals], [c.cart for c in crystals], [c.lattice for c in crystals])
    vec, length, unit = ops.edge_geometry_fwd(g.cart32, g.lattice32, g.atom_struct, g.center, g.neighbor, g.image)
    cart = g.cart32.cpu().double().requires_grad_(True)
    lat = g.lattice32.cpu().double()
    strain = torch.zeros(g.n_struct, 3, 3, dtype=torch.float64, requires_grad=True)
    sym = 0.5 * (strain + strain.transpose(1, 2))
    seg = g.atom_struct.cpu().long()
    pos = cart + torch.einsum("be,bec->bc", cart, sym[seg])
    latt = lat + lat @ sym
    c, n, im = g.center.cpu().long(), g.neighbor.cpu().long(), g.image.cpu().double()
    v = pos[c] - (pos[n] + torch.einsum("ek,ekc->ec", im, latt[seg[c]]))
    d = v.norm(dim=1)
    report("edge_geometry_fwd vec", vec, v, 5e-6)
    report("edge_geometry_fwd len", length, d, 5e-6)
    report("edge_geometry_fwd unit", unit, v / d[:, None], 1e-6)
    dl, du = rnd(g.n_edges, seed=1), rnd(g.n_edges, 3, seed=2)
    gc, gs = torch.autograd.grad((d * dl.double()).sum() + ((v / d[:, None]) * du.double()).sum(), [cart, strain])
    dcart, dstrain, _ = ops.edge_geometry_bwd(g.n_atoms, g.n_struct, g.edge_ptr, g.atom_ptr, g.rev, vec, length, unit,
                                              dev(dl), dev(du))
    report("edge_geometry_bwd dcart", dcart, gc, 2e-4)
    report("edge_geometry_bwd dstrain", dstrain, gs, 2e-3)
