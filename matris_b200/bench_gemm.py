"""Kernel micro-benchmark: one `mb_gemm` launch shape, timed with CUDA events.

    python -m matris_b200.bench_gemm K N [act] [gate] [rows] [mode] [scatter]

K: reduction width (a multiple of 128: K/128 concatenated sources), N: output width (a multiple of 128: N/128 column
blocks), act: SiLU on load, gate: SiLU' gate in the epilogue, rows: default 151,552 (8 tiles per SM on 148 SMs),
mode: tcgen05 (persistent kernel, default) | tcgen05_tile | simt; scatter: 0 plain store (default), 1 atomic
scatter-add to rows/5 targets in sorted order (runs of five equal targets), 2 the same targets in random order.
"""
import sys

import torch

from matris_b200 import ops


def main(argv):
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
