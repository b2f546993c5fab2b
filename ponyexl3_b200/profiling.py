"""Where a streamed-GEMV launch spends its time: per-CTA wall-clock stamps.

``python -m ponyexl3_b200.build --profile`` builds ``lib/libexl3b200_prof.so`` (the product
sources with -DEXL3_PROFILE); in that build every CTA of ``exl3_gemv`` records the GPU wall clock
at kernel entry, after barrier set-up, after the programmatic-launch wait, at the start of its
main loop, after its last item and at its end.  ``python -m ponyexl3_b200.profiling`` runs a
CUDA-graph train of launches over distinct layers in that build and prints, per launch, how the
launch period divides into those phases.  The stamps cost a few instructions per CTA, so the
numbers are close to, but not the same as, the product build's; bench figures never come from here.
"""

from __future__ import annotations

import argparse
import json
import statistics

import torch

from . import _lib, build


def gemv_timeline(in_features: int, out_features: int, *, k: int = 4, cb: int = 0, rows: int = 1,
                  layers: int = 8, replays: int = 3, pdl: bool = True, dump: str | None = None) -> dict:
    """Stamps of the LAST replay of a graph train of `layers` launches; times in microseconds
    relative to the first CTA entry of the train's second launch."""
    from . import ops

    lib = _lib.load()
    if not hasattr(lib, "exl3_profile_buffer"):
        raise RuntimeError("this is not the timeline build: call _lib.use_library(build.build(profile=True)) first")
    lib.exl3_profile_buffer.argtypes = [_lib.c_void_p, _lib.c_size_t]
    lib.exl3_profile_buffer.restype = None
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(7)
    trs = [torch.randint(-32768, 32767, (in_features // 16, out_features // 16, 16 * k), dtype=torch.int16,
                         device=dev, generator=g) for _ in range(layers)]
    suh = (torch.randint(0, 2, (in_features,), device=dev, generator=g) * 2 - 1).to(torch.float16)
    svh = (torch.randint(0, 2, (out_features,), device=dev, generator=g) * 2 - 1).to(torch.float16)
    x = torch.randn((rows, in_features), device=dev, generator=g).to(torch.float16)
    y = torch.empty((rows, out_features), dtype=torch.float16, device=dev)
    prof = torch.zeros((layers, 512, 16), dtype=torch.int64, device=dev)
    stream = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        ops.gemv(x, trs[0], k, cb, suh, svh, None, pdl=pdl, out=y)
        stream.synchronize()
        lib.exl3_profile_buffer(prof.data_ptr(), layers)      # the captured launches get the slots
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for t in trs:
                ops.gemv(x, t, k, cb, suh, svh, None, pdl=pdl, out=y)
        lib.exl3_profile_buffer(None, 0)
        for _ in range(replays):
            graph.replay()
        stream.synchronize()
    p = prof.cpu().numpy()
    if dump:
        import numpy as np
        np.save(dump, p)
    out = {"shape": f"{in_features}x{out_features}", "k": k, "rows": rows, "launches": []}
    prev_end = None
    for li in range(layers):
        used = p[li][p[li][:, 0] > 0]
        if used.shape[0] == 0:
            continue
        t0 = int(used[:, 0].min())
        col = lambda j: (used[:, j] - t0) / 1e3
        end = int(used[:, 5].max())
        rec = {
            "ctas": int(used.shape[0]), "sms": int(len(set(used[:, 6].tolist()))),
            "entry_spread": float(col(0).max()),
            "dep_wait_done": [float(col(2).min()), float(statistics.median(col(2))), float(col(2).max())],
            "loop_start": [float(col(3).min()), float(statistics.median(col(3))), float(col(3).max())],
            "last_item": [float(col(4).min()), float(statistics.median(col(4))), float(col(4).max())],
            "end": [float(col(5).min()), float(statistics.median(col(5))), float(col(5).max())],
            "loop_us_median": float(statistics.median((used[:, 4] - used[:, 3]) / 1e3)),
            "warp0_wait_kclk_median": float(statistics.median(used[:, 8] / 1e3)),
            "warp0_work_kclk_median": float(statistics.median(used[:, 9] / 1e3)),
            "producer_wait_kclk_median": float(statistics.median(used[:, 10] / 1e3)),
            "period_us": None if prev_end is None else (end - prev_end) / 1e3,
            "first_entry_vs_prev_end": None if prev_end is None else (t0 - prev_end) / 1e3,
        }
        prev_end = end
        out["launches"].append(rec)
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="5120x17408")
    ap.add_argument("--k", type=int, default=4)
    ap.add_argument("--cb", type=int, default=0)
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--dump", default=None, help="write the raw (launch, CTA, word) array to this .npy file")
    args = ap.parse_args()
    _lib.use_library(build.build(profile=True))
    inf, outf = (int(v) for v in args.shape.split("x"))
    r = gemv_timeline(inf, outf, k=args.k, cb=args.cb, rows=args.rows, layers=args.layers, pdl=not args.no_pdl,
                      dump=args.dump)
    for rec in r.pop("launches"):
        print(json.dumps(rec))
    print(json.dumps(r))


if __name__ == "__main__":
    main()
