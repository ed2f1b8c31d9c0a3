"""Time (or expose to a profiler) one operator of the library at a given shape.

    python -m fast_vision_models_b200.opbench conv --n 64 --hw 56 --c 64 --k 256 --r 1 --res --act 1
    python -m fast_vision_models_b200.opbench conv --n 64 --hw 56 --c 64 --k 64 --r 3 --pad 1 --tile 67108864
    python -m fast_vision_models_b200.opbench stem --n 64 --hw 224 --k 64 --r 7 --pad 3
    python -m fast_vision_models_b200.opbench dwconv --n 64 --hw 95 --c 192 --r 3 --pad 1 --act 3
    python -m fast_vision_models_b200.opbench layernorm --n 64 --hw 56 --c 96
    python -m fast_vision_models_b200.opbench gap --n 64 --hw 7 --c 2048        (also: se_scale, maxpool, up_argmax, wbatch)
    python -m fast_vision_models_b200.opbench dual --n 64 --hw 56 --c 64 --k 256 --k2 64 --res     (two 1x1 layers, one launch)

Default: the op is captured 20 times into a CUDA graph over 4 rotating buffer sets (so that inputs do not stay in
L2), the graph is replayed and timed with CUDA events; prints microseconds per launch and the algorithmic GB/s
(bytes of every operand once / time). With `--plain K` the op is simply launched K times, for a profiler that
selects launches itself (`ncu -k regex:... -s 1 -c 1 ... python -m fast_vision_models_b200.opbench ... --plain 3`).
"""
import argparse

import torch

from . import ops


def _cl(t):
    return t.contiguous(memory_format=torch.channels_last)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--groups", type=int, default=1, help="conv: groups (> 1: clfr3.gconv2 path)")
    ap.add_argument("op", choices=["conv", "dual", "stem", "dwconv", "layernorm", "gap", "se_scale", "se_gate", "maxpool", "up_argmax", "wbatch"])
    ap.add_argument("--n", type=int, default=64)
    ap.add_argument("--hw", type=int, nargs="+", default=[56], help="height [width]")
    ap.add_argument("--c", type=int, default=64)
    ap.add_argument("--k", type=int, default=64)
    ap.add_argument("--k2", type=int, default=64, help="dual: output channels of the second layer")
    ap.add_argument("--r", type=int, default=1, help="filter size (square)")
    ap.add_argument("--stride", type=int, default=1)
    ap.add_argument("--pad", type=int, default=0)
    ap.add_argument("--dil", type=int, default=1)
    ap.add_argument("--act", type=int, default=1)
    ap.add_argument("--res", action="store_true")
    ap.add_argument("--tile", type=int, default=0, help="tile code of fvm_conv2d_f16_tile (0 = library's choice)")
    ap.add_argument("--plain", type=int, default=0, help="launch the op this many times and exit (no graph, no timing)")
    a = ap.parse_args()
    dev = torch.device("cuda")
    ops.init(dev)
    H, W = a.hw[0], a.hw[-1]
    N, C, K, R = a.n, a.c, a.k, a.r
    nbuf = 4
    g = torch.Generator(device="cpu").manual_seed(0)

    def rnd(*shape, scale=1.0):
        return (torch.randn(shape, generator=g) * scale).half().to(dev)

    if a.op == "conv":
        P = (H + 2 * a.pad - a.dil * (R - 1) - 1) // a.stride + 1
        Q = (W + 2 * a.pad - a.dil * (R - 1) - 1) // a.stride + 1
        xs = [_cl(rnd(N, C, H, W)) for _ in range(nbuf)]
        w, b = _cl(rnd(K, C, R, R, scale=0.05)), rnd(K, scale=0.1)
        rs = [_cl(rnd(N, K, P, Q)) if a.res else None for _ in range(nbuf)]
        ys = [ops.empty_nhwc(N, K, P, Q, dev) for _ in range(nbuf)]
        nbytes = 2 * (N * H * W * C + K * C * R * R + K + N * P * Q * K * (2 if a.res else 1))
        flops = 2 * N * P * Q * K * C * R * R

        if a.groups > 1:
            from . import fold
            wg = _cl(rnd(K, C // a.groups, R, R, scale=0.05))
            w_sg, gsg, gsk = fold.pack_grouped(wg, a.groups)
            nbytes = 2 * (N * H * W * C + K * (C // a.groups) * R * R + K + N * P * Q * K)
            flops = 2 * N * P * Q * K * (C // a.groups) * R * R

            def launch(i):
                ops.gconv2_packed_into(xs[i], w_sg, b, None, (a.stride, a.stride), (a.pad, a.pad), a.act, gsg, gsk, ys[i])
        else:
            def launch(i):
                ops.conv_fused_into(xs[i], w, b, rs[i], (a.pad, a.pad), (a.stride, a.stride), a.act, ys[i],
                                    dilation=(a.dil, a.dil), tile_n=a.tile)
    elif a.op == "dual":
        # y = act(x . w1^T + b1 + res), z = act(y . w2^T + b2) as one launch (ops.pw_dual)
        K2 = a.k2
        xs = [_cl(rnd(N, C, H, W)) for _ in range(nbuf)]
        w1, b1 = _cl(rnd(K, C, 1, 1, scale=0.08)), rnd(K, scale=0.1)
        w2, b2 = _cl(rnd(K2, K, 1, 1, scale=0.05)), rnd(K2, scale=0.1)
        rs = [_cl(rnd(N, K, H, W)) if a.res else None for _ in range(nbuf)]
        nbytes = 2 * (N * H * W * (C + K * (2 if a.res else 1) + K2) + K * C + K2 * K + K + K2)
        flops = 2 * N * H * W * K * (C + K2)

        def launch(i):
            ops.pw_dual(xs[i], w1, b1, rs[i], a.act, w2, b2, a.act)
    elif a.op == "stem":
        P, Q = (H + 2 * a.pad - R) // 2 + 1, (W + 2 * a.pad - R) // 2 + 1
        xs = [ops.input_nhwc8_split(torch.randn((N, 3, H, W), generator=g).to(dev)) for _ in range(nbuf)]
        w = torch.zeros((K, 8, R, R))
        w[:, :3] = torch.randn((K, 3, R, R), generator=g) * 0.05
        w, b = _cl(w.half().to(dev)), rnd(K, scale=0.1)
        ys = [ops.empty_nhwc(N, K, P, Q, dev) for _ in range(nbuf)]
        nbytes = 2 * (N * H * W * 8 + K * 8 * R * R + K + N * P * Q * K)
        flops = 2 * N * P * Q * K * 3 * R * R

        def launch(i):
            ops.stem_conv_s2(xs[i], w, b, (a.pad, a.pad), a.act, out=ys[i])
    elif a.op == "dwconv":
        P = (H + 2 * a.pad - a.dil * (R - 1) - 1) // a.stride + 1
        Q = (W + 2 * a.pad - a.dil * (R - 1) - 1) // a.stride + 1
        xs = [_cl(rnd(N, C, H, W)) for _ in range(nbuf)]
        w, b = rnd(R, R, C, scale=0.2), rnd(C, scale=0.1)
        nbytes = 2 * (N * H * W * C + R * R * C + C + N * P * Q * C)
        flops = 2 * N * P * Q * C * R * R

        def launch(i):
            ops.dwconv(xs[i], w, b, (a.stride, a.stride), (a.pad, a.pad), a.act, dilation=(a.dil, a.dil))
    elif a.op == "wbatch":
        # squeeze-excite gate folded into per-image 1x1 weights + the project conv on them
        xs = [_cl(rnd(N, C, H, W)) for _ in range(nbuf)]
        w, b, s_ = _cl(rnd(K, C, 1, 1, scale=0.05)), rnd(K, scale=0.1), rnd(N, C, 1, 1)
        rs = [_cl(rnd(N, K, H, W)) if a.res else None for _ in range(nbuf)]
        nbytes = 2 * (N * H * W * C + N * K * C + K + N * H * W * K * (2 if a.res else 1))
        flops = 2 * N * H * W * K * C

        def launch(i):
            ops.conv1x1_wbatch(xs[i], ops.gate_weights(w, s_), b, rs[i], 0)
    else:
        xs = [_cl(rnd(N, C, H, W)) for _ in range(nbuf)]
        flops = 0
        if a.op == "layernorm":
            g_, b_ = torch.ones(C, dtype=torch.float16, device=dev), torch.zeros(C, dtype=torch.float16, device=dev)
            nbytes = 4 * N * H * W * C

            def launch(i):
                ops.layernorm_cl(xs[i], g_, b_, 1e-6)
        elif a.op == "gap":
            nbytes = 2 * (N * H * W * C + N * C)

            def launch(i):
                ops.global_avgpool(xs[i])
        elif a.op == "se_gate":
            # the two small FCs of a squeeze-excite block fed by the fused squeeze: --k = squeeze channels, --hw = slots
            Cs = a.k
            parts = [torch.randn((N, H, C), generator=g).to(dev) for _ in range(nbuf)]
            w1, b1, w2, b2 = rnd(Cs, C, scale=0.05), rnd(Cs, scale=0.1), rnd(C, Cs, scale=0.05), rnd(C, scale=0.1)
            nbytes = 4 * N * H * C + 2 * (2 * C * Cs + C + Cs) + 2 * N * C

            def launch(i):
                ops.se_gate_pooled(parts[i], 100, w1, b1, w2, b2, 3)
        elif a.op == "se_scale":
            s_ = rnd(N, C, 1, 1)
            nbytes = 4 * N * H * W * C

            def launch(i):
                ops.se_scale(xs[i], s_)
        elif a.op == "maxpool":
            P, Q = (H + 2 - 3) // 2 + 1, (W + 2 - 3) // 2 + 1
            nbytes = 2 * (N * H * W * C + N * P * Q * C)

            def launch(i):
                ops.maxpool(xs[i], 3, 2, 1)
        else:       # up_argmax: C score channels (K of them are classes) at H x W -> 8x the size
            nbytes = 2 * N * H * W * C + 4 * N * H * 8 * W * 8

            def launch(i):
                ops.up_argmax(xs[i], H * 8, W * 8, False, K)

    if a.plain > 0:
        for i in range(a.plain):
            launch(i % nbuf)
        torch.cuda.synchronize()
        print(f"{a.op}: launched {a.plain} times, status {ops.last_status()}")
        return

    iters = 20
    for i in range(nbuf):
        launch(i)
    torch.cuda.synchronize()
    graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for i in range(iters):
                launch(i % nbuf)
    graph.replay()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(5):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        e1.synchronize()
        best = min(best, e0.elapsed_time(e1) / iters * 1e3)
    print(f"{a.op} n{N} {H}x{W} c{C} k{K} r{R} s{a.stride} p{a.pad} d{a.dil} act{a.act} res{int(a.res)} tile{a.tile}: "
          f"{best:.1f} us/launch, {nbytes / best / 1e3:.0f} GB/s algorithmic, {flops / best / 1e6:.1f} TFLOP/s, "
          f"status {ops.last_status()}")


if __name__ == "__main__":
    main()
