"""Kernel micro-benchmark: one `mb_gemm` or `mb_gated_mlp_fwd` launch shape, timed with CUDA events.

    python -m matris_b200.bench_gemm K N [act] [gate] [rows] [mode] [scatter]
    python -m matris_b200.bench_gemm gated K [rows] [save] [res] [gather]
    python -m matris_b200.bench_gemm ffn K [rows] [save] [res]

ffn: the plain two-layer form of the fused kernel (K -> 128 -> 128, `ops.ffn_fwd`); save: also write z1 (default 1);
res: write out2 = y + res_w * res instead of y (default 1).
gated: the fused gated-MLP forward (K -> 256 -> 2 x 128 -> 128); save: also write z1 / z2 (default 1); res: also
write out2 = h + res_w * res (default 1); gather: 1 = K segments 1.. are gathered from a table of rows/6 rows through
random indices (default 0: all segments read row r).

K: reduction width (a multiple of 128: K/128 concatenated sources), N: output width (a multiple of 128: N/128 column
blocks), act: SiLU on load, gate: SiLU' gate in the epilogue, rows: default 151,552 (8 tiles per SM on 148 SMs),
mode: tcgen05 (persistent 3xBF16 kernel, default) | tcgen05_tf32 | tcgen05_tile | simt; scatter: 0 plain store (default), 1 atomic
scatter-add to rows/5 targets in sorted order (runs of five equal targets), 2 the same targets in random order.
"""
import sys

import torch

from matris_b200 import ops


def gated(argv):
    from types import SimpleNamespace
    K = int(argv[0])
    rows = int(argv[1]) if len(argv) > 1 else 148 * 128 * 8
    save = bool(int(argv[2])) if len(argv) > 2 else True
    with_res = bool(int(argv[3])) if len(argv) > 3 else True
    gather = bool(int(argv[4])) if len(argv) > 4 else False
    torch.manual_seed(0)
    dev = "cuda"
    p = SimpleNamespace(w1=ops.SplitWeight(torch.randn(256, K, device=dev) * K ** -0.5), b1=torch.randn(256, device=dev) * 0.1,
                        w2=ops.SplitWeight(torch.randn(256, 128, device=dev) * 128 ** -0.5),
                        b2=torch.randn(256, device=dev) * 0.1, nc=torch.ones(128, device=dev), ng=torch.ones(128, device=dev))
    x = torch.randn(rows, 128, device=dev)
    srcs = [ops.S(x)]
    if gather:
        table = torch.randn(rows // 6 + 1, 128, device=dev)
        for s_ in range(K // 128 - 1):
            idx = torch.randint(0, table.shape[0], (rows,), device=dev, dtype=torch.int32)
            srcs.append(ops.S(table, idx))
    else:
        more = torch.randn(rows, K - 128, device=dev) if K > 128 else None
        srcs += [ops.S(more, None, 128 * s_) for s_ in range(K // 128 - 1)]
    res = torch.randn(rows, 128, device=dev) if with_res else None
    rw = torch.randn(128, device=dev) if with_res else None

    def launch():
        return ops.gated_mlp_fwd(p, rows, srcs, res=res, res_w=rw, save=save)

    for _ in range(3):
        launch()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    launch()
    e1.record()
    torch.cuda.synchronize()
    assert ops.gemm_status() == 0
    ms = e0.elapsed_time(e1)
    flops = 2.0 * rows * 256 * (K + 128)
    gbytes = 4.0 * rows * (K + 128 * (1 + 4 * save + 2 * with_res)) / 1e9
    print(f"gated rows={rows} K={K} save={int(save)} res={int(with_res)} gather={int(gather)}: {ms:.3f} ms, "
          f"{flops / ms / 1e9:.1f} TFLOP/s fp32-equivalent, {gbytes / ms * 1e3:.0f} GB/s of algorithmic traffic")


def ffn(argv):
    from types import SimpleNamespace
    K = int(argv[0])
    rows = int(argv[1]) if len(argv) > 1 else 148 * 128 * 8
    save = bool(int(argv[2])) if len(argv) > 2 else True
    with_res = bool(int(argv[3])) if len(argv) > 3 else True
    torch.manual_seed(0)
    dev = "cuda"
    p = SimpleNamespace(w1=ops.SplitWeight(torch.randn(128, K, device=dev) * K ** -0.5), b1=torch.randn(128, device=dev) * 0.1,
                        w2=ops.SplitWeight(torch.randn(128, 128, device=dev) * 128 ** -0.5),
                        b2=torch.randn(128, device=dev) * 0.1)
    x = torch.randn(rows, K, device=dev)
    res = torch.randn(rows, 128, device=dev) if with_res else None
    rw = torch.randn(128, device=dev) if with_res else None

    def launch():
        return ops.ffn_fwd(p, x, want_y=not with_res, res=res, res_w=rw, save=save)

    for _ in range(3):
        launch()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    launch()
    e1.record()
    torch.cuda.synchronize()
    assert ops.gemm_status() == 0
    ms = e0.elapsed_time(e1)
    flops = 2.0 * rows * 128 * (K + 128)
    gbytes = 4.0 * rows * (K + 128 * (1 + save + with_res)) / 1e9
    print(f"ffn rows={rows} K={K} save={int(save)} res={int(with_res)}: {ms:.3f} ms, "
          f"{flops / ms / 1e9:.1f} TFLOP/s fp32-equivalent, {gbytes / ms * 1e3:.0f} GB/s of algorithmic traffic")


def main(argv):
    if argv[0] == "gated":
        return gated(argv[1:])
    if argv[0] == "ffn":
        return ffn(argv[1:])
    K, N = int(argv[0]), int(argv[1])
    act = int(argv[2]) if len(argv) > 2 else 0
    gate = int(argv[3]) if len(argv) > 3 else 0
    rows = int(argv[4]) if len(argv) > 4 else 148 * 128 * 8
    mode = argv[5] if len(argv) > 5 else "tcgen05"
    scatter = int(argv[6]) if len(argv) > 6 else 0
    torch.manual_seed(0)
    x = torch.randn(rows, K, device="cuda")
    z = torch.randn(rows, N, device="cuda") if gate else None
    W = ops.SplitWeight((torch.randn(N, K, device="cuda") * 0.1).contiguous())
    out = torch.empty(rows, N, device="cuda")
    out_idx, out_mode = None, ops.OUT_STORE
    if scatter:
        out_idx = (torch.arange(rows, device="cuda") // 5).to(torch.int32)
        if scatter == 2:
            out_idx = out_idx[torch.randperm(rows, device="cuda")].contiguous()
        out = torch.zeros(rows // 5 + 1, N, device="cuda")
        out_mode = ops.OUT_ATOMIC
    ops.set_gemm_mode(mode)

    def launch():
        ops.gemm(rows, [ops.B([ops.S(x, None, 128 * s, act=act) for s in range(K // 128)], W, w_row=128 * j, out=out,
                              out_col=128 * j, gate=z, gate_col=128 * j if gate else 0, out_idx=out_idx, mode=out_mode)
                        for j in range(N // 128)])

    for _ in range(3):
        launch()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    launch()
    e1.record()
    torch.cuda.synchronize()
    assert ops.gemm_status() == 0
    ms = e0.elapsed_time(e1)
    print(f"rows={rows} K={K} N={N} act={act} gate={gate} mode={mode} scatter={scatter}: {ms:.3f} ms, "
          f"{2.0 * rows * K * N / ms / 1e9:.1f} TFLOP/s fp32-equivalent")


if __name__ == "__main__":
    main(sys.argv[1:])
