"""Times every BASELINE configuration of the matmult path on one GPU and prints one JSON line per row.

    python bench.py --configs [--steps K] [--cpu] [--only c1,c3i8,...]
    python -m neurotensor_b200.bench_configs [--steps K] [--only c1,c3i8,...]          # GPU rows only

Rows: c1 (Float32 1024^3), c2 (batched Float16 64x2048^3, transposed-view B), c3i8 (Int8 4096x8192x4096),
c3i32 (Int32 2048^3), c3i16 (Int16 4096^3), f64 (Float64 4096^3 and Complex64 2048^3 on the CUDA-core route), t8192 (Float16 / BFloat16 8192^3), skinny (1 / 2 / 16 / 128 rows x 8192 x 8192), midrows (256 - 512 rows against 2048 - 11008-wide weights), shallowk (8192 x k x 8192 with k = 16 / 256 / 1024), c4 (BFloat16 MLP 8192 x 4096->16384->4096: forward + backward step), c5 (Float16 conv2d
[32,256,56,56] * [256,256,3,3]), sweepN (Float32 N^3).  Inputs are seeded synthetic tensors of the stated shapes
and distributions, resident on the device; time is CUDA events over K launches after 3 warm-ups.  Given a CPU
oracle by its caller (bench.py --configs --cpu), it also times that on a bounded sub-problem of each row (scaled
linearly, stated per row); this package itself never imports it.
"""
import argparse
import json
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from neurotensor_b200 import _lib, api  # noqa: E402


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "measured"
    return 1590.0, 6650.0, "fallback"


def timed(fn, steps, warm=3):
    """(seconds per call, kernels per call).  Calls that take milliseconds are timed as a plain loop.  Short calls
    (the Python wrapper alone costs 10 - 30 us of host time per call, more than many of these kernels run) are
    captured into a CUDA graph, ten calls per graph, and the graph is replayed: the figure is then the time the GPU
    needs per call with the kernels of successive calls back to back, which is what a C or C++ caller of the C ABI
    sees in a loop.  Warm-up and capture run on the same side stream, so the library's per-stream scratch block
    exists before the capture starts."""
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for _ in range(warm):
            fn()
        side.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = _lib.launch_count()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        side.synchronize()
        loop_s = e0.elapsed_time(e1) / steps * 1e-3
        launches = (_lib.launch_count() - l0) // steps
        timed.last_loop_seconds = loop_s
        if loop_s > 0.5e-3:
            return loop_s, launches
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(10):
                    fn()
            for _ in range(2):
                graph.replay()
            side.synchronize()
            replays = max(5, steps // 2)
            e0.record()
            for _ in range(replays):
                graph.replay()
            e1.record()
            side.synchronize()
            graph_s = e0.elapsed_time(e1) / (10 * replays) * 1e-3
            # a graph that caught nothing (work queued on another stream) replays in no time: keep the loop figure then
            return (graph_s if graph_s > 1e-6 else loop_s), launches
        except Exception:
            torch.cuda.synchronize()
            return loop_s, launches


timed.last_loop_seconds = None


def randn(gen, shape, dtype, scale=1.0):
    return (torch.randn(shape, generator=gen, device="cuda") * scale).to(dtype)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--only", default="")
    args = ap.parse_args()
    return run(args.steps, args.only, None)


def run(steps=20, only="", oracle=None):
    """Times the rows named in `only` (all when empty).  `oracle`: the CPU oracle module for the per-row CPU figures, or
    None for GPU rows only."""
    class _Args:
        pass
    args = _Args()
    args.steps, args.cpu = steps, oracle is not None
    only = set(filter(None, only.split(",")))
    tensor_peak, hbm_peak, src = peaks()
    sm_clock_ghz = 1.965
    ffma_peak = 148 * 128 * 2 * sm_clock_ghz / 1e3  # TFLOP/s at the maximum SM clock
    rows = []

    def emit(name, seconds, flops, alg_bytes, bound, launches, note="", cpu=None):
        tf = flops / seconds / 1e12
        gbs = alg_bytes / seconds / 1e9
        peak = {"tensor": tensor_peak, "tensor_i8": 3314.0, "ffma": ffma_peak, "imad": ffma_peak / 2, "dfma": ffma_peak / 2}.get(bound)
        row = {"config": name, "ms": seconds * 1e3, "tflops_or_tops": tf, "algorithmic_GBps": gbs, "bound": bound,
               "frac_of_peak": (tf / peak) if peak else gbs / hbm_peak, "peak": peak if peak else hbm_peak,
               "peak_source": src if bound.startswith("tensor") or bound == "hbm" else "derived: SMs x lanes x 2 x max clock",
               "launches_per_step": launches, "route": _lib.last_route(), "note": note,
               "ms_python_loop": (timed.last_loop_seconds or seconds) * 1e3}
        if cpu:
            row["cpu_oracle"] = cpu
        rows.append(row)
        print(json.dumps(row), flush=True)

    def cpu_time(fn, scale, what):
        if not args.cpu:
            return None
        fn(oracle)  # warm-up
        t0 = time.perf_counter()
        fn(oracle)
        dt = time.perf_counter() - t0
        return {"seconds_scaled": dt * scale, "sample": what, "threads": oracle.default_threads()}

    gen = torch.Generator(device="cuda").manual_seed(1)
    want = lambda n: not only or n in only

    if want("c1"):
        a, b = randn(gen, (1024, 1024), torch.float32), randn(gen, (1024, 1024), torch.float32)
        c = torch.empty((1024, 1024), device="cuda")
        s, l = timed(lambda: api.gemm(a, b, c), args.steps * 5)
        an, bn = a.cpu().numpy(), b.cpu().numpy()
        emit("c1 Float32 1024^3", s, 2 * 1024 ** 3, 3 * 4 * 1024 ** 2, "ffma", l, "latency-sized problem: 64 CTAs",
             cpu_time(lambda o: o.matmult(an, bn), 1, "full problem"))

    if want("c2"):
        a, bs = randn(gen, (64, 2048, 2048), torch.float16, 0.1), randn(gen, (64, 2048, 2048), torch.float16, 0.1)
        c = torch.empty((64, 2048, 2048), dtype=torch.float16, device="cuda")
        s, l = timed(lambda: api.gemm(a, bs.transpose(-1, -2), c), args.steps)
        an, bn = a[:1].cpu().numpy(), bs[:1].cpu().numpy()
        emit("c2 batched Float16 64x2048^3, B transposed view", s, 64 * 2 * 2048 ** 3, 3 * 64 * 2048 ** 2 * 2, "tensor", l, "",
             cpu_time(lambda o: o.matmult(an, bn, False, True), 64, "1 of 64 items, scaled x64"))
        del a, bs, c

    if want("t8192"):
        # the north-star target shape: one 8192^3 GEMM on 16-bit inputs (32 x 32 pair tiles, 13.8 waves)
        for name, dt in (("Float16", torch.float16), ("BFloat16", torch.bfloat16)):
            a, b = randn(gen, (8192, 8192), dt, 0.1), randn(gen, (8192, 8192), dt, 0.1)
            c = torch.empty((8192, 8192), dtype=dt, device="cuda")
            s, l = timed(lambda: api.gemm(a, b, c), max(5, args.steps // 2))
            emit("target %s 8192^3" % name, s, 2 * 8192 ** 3, 3 * 8192 ** 2 * 2, "tensor", l,
                 "nominal dense peak 2250 TFLOP/s: %.1f %% of it" % (2 * 8192 ** 3 / s / 1e12 / 2250 * 100))
            del a, b, c

    if want("skinny"):
        # memory-bound shapes: few rows against a large weight matrix (the weights are read once from HBM)
        for m in (1, 2, 16, 128):
            for name, dt in (("Float16", torch.float16),):
                a, b = randn(gen, (m, 8192), dt, 0.1), randn(gen, (8192, 8192), dt, 0.1)
                c = torch.empty((m, 8192), dtype=dt, device="cuda")
                s, l = timed(lambda: api.gemm(a, b, c), args.steps)
                emit("skinny %s %dx8192x8192" % (name, m), s, 2 * m * 8192 * 8192, (m * 8192 * 2 + 8192 * 8192) * 2, "hbm", l,
                     "the 134 MB weight matrix is the traffic; it exceeds L2")
                bt = b.t().contiguous()
                s, l = timed(lambda: api.gemm(a, bt, c, transpose_b=True), args.steps)
                emit("skinny %s %dx8192x8192, weights stored [N, K]" % (name, m), s, 2 * m * 8192 * 8192,
                     (m * 8192 * 2 + 8192 * 8192) * 2, "hbm", l)
                del a, b, bt, c

    if want("midrows"):
        # a few hundred rows through a Linear layer: too few 256 x 256 tiles to fill the GPU, so the planner weighs
        # CTA pairs against single-CTA tiles and K slices
        for (m, n, k) in ((256, 8192, 8192), (512, 4096, 4096), (384, 4096, 11008), (256, 2048, 8192)):
            a, b = randn(gen, (m, k), torch.float16, 0.1), randn(gen, (k, n), torch.float16, 0.1)
            c = torch.empty((m, n), dtype=torch.float16, device="cuda")
            s, l = timed(lambda: api.gemm(a, b, c), args.steps)
            emit("midrows Float16 %dx%dx%d" % (m, k, n), s, 2 * m * n * k, (m * k + k * n + m * n) * 2, "tensor", l)
            del a, b, c

    if want("shallowk"):
        # weight-gradient shapes of a small batch: dW[8192, 8192] = X[k, 8192]^T . G[k, 8192]; writing C is the traffic
        for k in (16, 256, 1024):
            x, gr = randn(gen, (k, 8192), torch.float16, 0.1), randn(gen, (k, 8192), torch.float16, 0.1)
            c = torch.empty((8192, 8192), dtype=torch.float16, device="cuda")
            s, l = timed(lambda: api.gemm(x, gr, c, transpose_a=True), args.steps)
            emit("shallowk Float16 8192x%dx8192 (A transposed view)" % k, s, 2 * 8192 * 8192 * k,
                 (8192 * 8192 + 2 * k * 8192) * 2, "hbm" if k <= 256 else "tensor", l)
            del x, gr, c

    if want("c3i8"):
        a = torch.randint(-8, 8, (4096, 8192), generator=gen, device="cuda", dtype=torch.int8)
        b = torch.randint(-8, 8, (8192, 4096), generator=gen, device="cuda", dtype=torch.int8)
        c = torch.empty((4096, 4096), dtype=torch.int8, device="cuda")
        s, l = timed(lambda: api.gemm(a, b, c), args.steps)
        an, bn = a[:512].cpu().numpy(), b.cpu().numpy()
        emit("c3 Int8 4096x8192x4096 (int8 out, wrap)", s, 2 * 4096 * 8192 * 4096, 2 * 4096 * 8192 + 4096 * 4096, "tensor_i8", l,
             "peak = cuBLAS int8 (torch._int_mm, s32 out) 8192^3 best of 10 measured on this pool: 3314 TOPS",
             cpu_time(lambda o: o.matmult(an, bn), 8, "512 of 4096 rows, scaled x8"))

    if want("f32exact"):
        a, b = randn(gen, (4096, 4096), torch.float32), randn(gen, (4096, 4096), torch.float32)
        c = torch.empty((4096, 4096), device="cuda")
        s, l = timed(lambda: api.gemm(a, b, c, route=_lib.ROUTE_SIMT), args.steps)
        emit("Float32 4096^3 on the bit-exact CUDA-core route", s, 2 * 4096 ** 3, 12 * 4096 ** 2, "ffma", l)
        bt = b.t().contiguous()
        s, l = timed(lambda: api.gemm(a, bt, c, transpose_b=True, route=_lib.ROUTE_SIMT), args.steps)
        emit("Float32 4096^3 CUDA-core route, B transposed", s, 2 * 4096 ** 3, 12 * 4096 ** 2, "ffma", l)
        del a, b, bt, c

    if want("f64"):
        # Float64 and Int64 exist on the CUDA-core route only (bit-exact chains); B200's FP64 rate is 1/2 of FP32 per SM
        a, b = randn(gen, (4096, 4096), torch.float64), randn(gen, (4096, 4096), torch.float64)
        c = torch.empty((4096, 4096), dtype=torch.float64, device="cuda")
        s, l = timed(lambda: api.gemm(a, b, c), args.steps)
        emit("Float64 4096^3 on the CUDA-core route", s, 2 * 4096 ** 3, 3 * 8 * 4096 ** 2, "dfma", l,
             "peak = DFMA at half the FFMA rate (derived)")
        ca = torch.view_as_complex(randn(gen, (2048, 2048, 2), torch.float32).contiguous())
        cb = torch.view_as_complex(randn(gen, (2048, 2048, 2), torch.float32).contiguous())
        cc = torch.empty((2048, 2048), dtype=torch.complex64, device="cuda")
        s, l = timed(lambda: api.gemm(ca, cb, cc), args.steps)
        emit("Complex64 2048^3 (the reference's lane-wise product: two FMA chains per element)", s, 4 * 2048 ** 3,
             3 * 8 * 2048 ** 2, "ffma", l)
        del a, b, c, ca, cb, cc

    if want("c3i32"):
        a = torch.randint(-1000, 1001, (2048, 2048), generator=gen, device="cuda", dtype=torch.int32)
        b = torch.randint(-1000, 1001, (2048, 2048), generator=gen, device="cuda", dtype=torch.int32)
        c = torch.empty((2048, 2048), dtype=torch.int32, device="cuda")
        s, l = timed(lambda: api.gemm(a, b, c), args.steps)
        an, bn = a.cpu().numpy(), b.cpu().numpy()
        emit("c3 Int32 2048^3 (wrap)", s, 2 * 2048 ** 3, 3 * 4 * 2048 ** 2, "imad", l, "peak = IMAD at half the FFMA rate; the default route is 8-bit limb products on tensor cores",
             cpu_time(lambda o: o.matmult(an, bn), 1, "full problem"))

    if want("c3i16"):
        a = torch.randint(-30000, 30001, (4096, 4096), generator=gen, device="cuda", dtype=torch.int16)
        b = torch.randint(-30000, 30001, (4096, 4096), generator=gen, device="cuda", dtype=torch.int16)
        c = torch.empty((4096, 4096), dtype=torch.int16, device="cuda")
        s, l = timed(lambda: api.gemm(a, b, c), args.steps)
        emit("Int16 4096^3 (wrap) on 8-bit limb products", s, 2 * 4096 ** 3, 3 * 2 * 4096 ** 2, "tensor_i8", l,
             "three 8-bit GEMM depths per int16 product: the tensor cores do 3x the listed ops")
        s, l = timed(lambda: api.gemm(a, b, c, route=_lib.ROUTE_SIMT), max(3, args.steps // 4))
        emit("Int16 4096^3 (wrap) on the CUDA-core route", s, 2 * 4096 ** 3, 3 * 2 * 4096 ** 2, "imad", l)
        del a, b, c

    if want("c4"):
        B, D, H = 8192, 4096, 16384
        dt = torch.bfloat16
        x, t = randn(gen, (B, D), dt), randn(gen, (B, D), dt)
        w1, w2 = randn(gen, (D, H), dt, D ** -0.5), randn(gen, (H, D), dt, H ** -0.5)
        b1, b2 = randn(gen, (H,), dt, 0.01), randn(gen, (D,), dt, 0.01)

        def step():
            h, a = api.linear_relu(x, w1, b1)                  # ReLU as a second output of the GEMM epilogue
            y = api.linear(a, w2, b2)
            loss, dy = api.mse(y, t)
            gw2 = api.matmult(a, dy, True, False)
            dh = api.matmult_relu_backward(dy, w2, h, True)    # ReLU mask applied in the GEMM epilogue
            gw1 = api.matmult(x, dh, True, False)          # the input does not track a gradient: no dX GEMM
            api.column_sum(dy), api.column_sum(dh)
            return loss

        s, l = timed(step, max(3, args.steps // 4))
        flops = 5 * 2 * B * D * H
        xn, wn = x[:256].view(torch.int16).cpu().numpy().view("uint16"), w1.view(torch.int16).cpu().numpy().view("uint16")
        emit("c4 BFloat16 MLP 8192x(4096->16384->4096) fwd+bwd step (5 GEMMs, fused ReLU epilogues, + elementwise)", s, flops,
             0, "tensor", l, "GEMM flops only (5 x 1.0995e12); elementwise kernels are inside the time",
             cpu_time(lambda o: o.matmult(xn, wn, bf16=True), 32 * 5, "256 of 8192 rows of one GEMM, scaled x32 x5 GEMMs"))
        # GEMM-only time of the same five contractions
        h = api.linear(x, w1, b1); a = api.relu(h); y = api.linear(a, w2, b2); _, dy = api.mse(y, t)
        da = api.matmult(dy, w2, False, True); dh = api.relu_backward(h, da)

        def gemms():
            api.linear(x, w1, b1); api.linear(a, w2, b2)
            api.matmult(dy, w2, False, True); api.matmult(a, dy, True, False); api.matmult(x, dh, True, False)

        s, l = timed(gemms, max(3, args.steps // 4))
        emit("c4 the five GEMMs alone", s, flops, 0, "tensor", l)
        # the parameter update that turns the step into a train step: Adam over W1, b1, W2, b2 (134 M parameters)
        gw1, gw2 = api.matmult(x, dh, True, False), api.matmult(a, dy, True, False)
        gb1, gb2 = api.column_sum(dh), api.column_sum(dy)
        params = [(w1, gw1), (b1, gb1.to(dt)), (w2, gw2), (b2, gb2.to(dt))]
        state = [(torch.zeros_like(p), torch.zeros_like(p)) for p, _ in params]

        def adam():
            for (p, g), (m, v) in zip(params, state):
                api.adam_step(p, g, m, v, lr=1e-3)

        s, l = timed(adam, args.steps)
        n_par = sum(p.numel() for p, _ in params)
        emit("c4 optimizers::Adam::step over W1, b1, W2, b2 (%d parameters, BFloat16)" % n_par, s, 0, 7 * 2 * n_par, "hbm", l,
             "reads param, grad, m, v and writes param, m, v once each")
        del gw1, gw2, gb1, gb2, params, state
        del x, t, w1, w2, h, a, y, dy, da, dh

    if want("c5"):
        x = randn(gen, (32, 256, 56, 56), torch.float16)
        w = randn(gen, (256, 256, 3, 3), torch.float16, (256 * 9) ** -0.5)
        ws = torch.empty(32 * 2304 * 3136 * 2, dtype=torch.uint8, device="cuda")
        s, l = timed(lambda: api.conv2d(x, w, 1, 1, workspace=ws), args.steps)
        flops = 2 * 256 * 2304 * 32 * 3136
        xn, wn = x[:1].cpu().numpy(), w.cpu().numpy()
        emit("c5 Float16 conv2d [32,256,56,56]*[256,256,3,3] s1 p1", s, flops, (51.4e6 + 1.18e6 + 51.4e6), "tensor", l,
             "channels-last copy + weights reorder + implicit GEMM; NTB200_CONV_EXPLICIT=1 gives im2col + GEMM", cpu_time(lambda o: o.conv2d(xn, wn, 1, 1), 32, "1 of 32 images, scaled x32"))
        s2, l2 = timed(lambda: api.unfold2d(x, (3, 3), 1, 1, 1), args.steps)
        emit("c5 im2col alone (writes the 462 MB column matrix)", s2, 0, 51.4e6 + 462.4e6, "hbm", l2)
        col = api.unfold2d(x, (3, 3), 1, 1, 1)
        out = torch.empty((32, 256, 3136), dtype=torch.float16, device="cuda")
        w2d = w.reshape(256, 2304)
        s3, l3 = timed(lambda: api.gemm(w2d, col, out), args.steps)
        emit("c5 GEMM alone: w[256,2304] x col[32,2304,3136]", s3, flops, 0, "tensor", l3)
        del col, out
        # backward of the same convolution (the step after the C5 forward): image and kernel gradients
        g = randn(gen, (32, 256, 56, 56), torch.float16)
        need = api.lib().ntb200_conv2d_backward_workspace_bytes(api.dtype_code(x), 32, 256, 56, 56, 256, 3, 3, 1, 1, 1, 1, 1, 1)
        wsb = torch.empty(need, dtype=torch.uint8, device="cuda")
        dxb, dwb = torch.empty_like(x), torch.empty_like(w)

        def bwd_image():
            api.check(api.lib().ntb200_conv2d_backward_image(api.dtype_code(x), g.data_ptr(), w.data_ptr(), dxb.data_ptr(),
                                                             wsb.data_ptr(), 32, 256, 56, 56, 256, 3, 3, 1, 1, 1, 1, 1, 1, api._stream()))

        def bwd_kernel():
            api.check(api.lib().ntb200_conv2d_backward_kernel(api.dtype_code(x), x.data_ptr(), g.data_ptr(), dwb.data_ptr(),
                                                              wsb.data_ptr(), 0, 32, 256, 56, 56, 256, 3, 3, 1, 1, 1, 1, 1, 1, api._stream()))

        s4, l4 = timed(bwd_image, args.steps)
        emit("c5 backward, image gradient [32,256,56,56]", s4, flops, 0, "tensor", l4)
        s5, l5 = timed(bwd_kernel, args.steps)
        emit("c5 backward, kernel gradient [256,256,3,3]", s5, flops, 0, "tensor", l5)
        del g, wsb, dxb, dwb
        del x, w, ws

    for n in (512, 1024, 2048, 4096, 8192, 16384):
        if not want("sweep%d" % n) and not (not only):
            continue
        if only and "sweep%d" % n not in only:
            continue
        a, b = randn(gen, (n, n), torch.float32), randn(gen, (n, n), torch.float32)
        c = torch.empty((n, n), device="cuda")
        s, l = timed(lambda: api.gemm(a, b, c), max(2, args.steps // (1 if n <= 4096 else 5)))
        emit("sweep Float32 %d^3" % n, s, 2 * n ** 3, 12 * n * n, "ffma", l)
        del a, b, c
    return 0


if __name__ == "__main__":
    sys.exit(main())
