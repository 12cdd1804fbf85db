"""Tuning run of the tensor-core GEMM's tile shapes (the counterpart of the reference's
tuning/tune_tc2d.sh, which sweeps its 72 instances at 4096^3):

    python -m kuiper_b200.tune_tc [--laps 20] [--json] [--shapes 2048x2048x2048,1024x1024x4096] [--modes auto,wide] [--eager]

For a grid of shapes it times every tile shape the library has (single-CTA 128 x 256, 128 x 128 and
128 x 64, CTA pair 256 x 256, wide pair 512 x 256) and the library's own choice, bf16 -> f32 with
column-major B, as CUDA-graph replays (device time, no host call between launches), and prints
TFLOP/s per shape and mode.  The 8192^3 row is where the relative rates RATE_SINGLE,
RATE_PAIR and RATE_WIDE in csrc/gemm_umma.cu come from; the other rows show what the
rounds-times-cost estimate built on them picks and what that costs against the best mode.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import klas, synth

SHAPES = [(1024, 1024, 1024), (2048, 2048, 2048), (2560, 2048, 4096), (3072, 3072, 3072), (3584, 3072, 4096),
          (4096, 4096, 4096), (8192, 8192, 8192), (8192, 1024, 8192), (1024, 8192, 8192), (8192, 8192, 512),
          (1024, 1024, 4096), (16384, 4096, 4096)]
MODES = ["single", "narrow", "slim", "pair", "wide", "auto"]


def time_ms(graph, laps):
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    graph.replay()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / laps


def capture(fn, laps, stream):
    """`laps` launches of `fn` as one CUDA graph: the replay runs at the device's rate, with no host
    call between launches (at 1024^3 a launch takes less device time than its host call)."""
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        fn()   # warm-up outside the capture
        with torch.cuda.graph(g, stream=stream):
            for _ in range(laps):
                fn()
    torch.cuda.synchronize()
    return g


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--laps", type=int, default=20)
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--shapes", default="", help="comma-separated ROWSxCOLSxSHARED instead of the built-in grid")
    ap.add_argument("--modes", default="", help="with --eager: comma-separated subset of %s" % ",".join(MODES))
    ap.add_argument("--eager", action="store_true",
                    help="plain launches, `laps` per shape and mode, no timing table: what a profiler run wants")
    a = ap.parse_args(argv)
    shapes = [tuple(int(x) for x in sh.split("x")) for sh in a.shapes.split(",") if sh] or SHAPES
    modes = [md for md in a.modes.split(",") if md] or MODES
    if a.eager:
        for m, n, k in shapes:
            A, Bt = synth.gemm_bf16(1, m, n, k, b_col_major=True, device="cuda")
            D = torch.empty((m, n), dtype=torch.float32, device="cuda")
            for mode in modes:
                klas.debug_set("tc_mode", mode)
                klas.debug_set("tc_ksplit", "auto" if mode == "auto" else "off")
                for _ in range(a.laps):
                    klas.gemm_tc(A, Bt, b_col_major=True, D=D)
            torch.cuda.synchronize()
        klas.debug_set("tc_mode", "auto")
        klas.debug_set("tc_ksplit", "auto")
        return 0 if klas.gemm_tc_status() == 0 else 1
    rows = []
    side = torch.cuda.Stream()
    for m, n, k in shapes:
        A, Bt = synth.gemm_bf16(1, m, n, k, b_col_major=True, device="cuda")
        D = torch.empty((m, n), dtype=torch.float32, device="cuda")
        rec = {"rows": m, "cols": n, "shared": k}
        # The modes take turns in short bursts and the median burst counts: under the power cap the
        # clock sags within a second of load, so timing one mode after the other would favour
        # whichever came first.  The knob is read when the launch is recorded, so each graph keeps
        # its mode.
        burst = max(2, a.laps // 2)
        graphs = {}
        for mode in MODES:
            klas.debug_set("tc_mode", mode)
            klas.debug_set("tc_ksplit", "auto" if mode == "auto" else "off")   # forced shapes run unsplit
            graphs[mode] = capture(lambda: klas.gemm_tc(A, Bt, b_col_major=True, D=D), burst, side)
        klas.debug_set("tc_mode", "auto")
        bursts = {mode: [] for mode in MODES}
        for rnd in range(6):
            for mode in MODES:
                ms = time_ms(graphs[mode], burst)
                if rnd > 0:
                    bursts[mode].append(ms)
        for mode in MODES:
            ms = sorted(bursts[mode])[len(bursts[mode]) // 2]
            rec[mode] = 2.0 * m * n * k / ms / 1e9
        klas.gemm_tc_status()
        best = max(MODES[:-1], key=lambda md: rec[md])
        rec["best"], rec["auto_over_best"] = best, rec["auto"] / rec[best]
        plan = klas.gemm_tc_plan(m, k, n, sm_count=torch.cuda.get_device_properties(0).multi_processor_count)
        rec["plan"] = "%s %d" % (plan["kind"], plan["tile_cols"]) + (", K in %d parts" % plan["k_parts"] if plan["k_parts"] > 1 else "") + (
            ", last round cut" if plan["tail_cut"] else "")
        rows.append(rec)
        del graphs, A, Bt, D
    if a.json:
        print(json.dumps(rows))
    else:
        print("%-22s %8s %8s %8s %8s %8s %8s  %-22s %s" % ("rows x cols x shared", *MODES, "best (auto / best)", "auto is"))
        for r in rows:
            print("%-22s %8.0f %8.0f %8.0f %8.0f %8.0f %8.0f  %-22s %s" % ("%d x %d x %d" % (r["rows"], r["cols"], r["shared"]),
                                                                           *(r[md] for md in MODES),
                                                                           "%s (%.2f)" % (r["best"], r["auto_over_best"]), r["plan"]))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
