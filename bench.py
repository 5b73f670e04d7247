#!/usr/bin/env python
"""bench.py — fused Where -> Select -> Sum throughput on 1/2/4/8 B200, with roofline, end-to-end and CPU-baseline figures.

Workload (all N): Where(x => x > 0.5f).Select(x => x * x + 3f).Sum() over 2^30 float32 uniform [0,1) (PCG64 seed 31),
cut into contiguous shards, one per rank; partial sums combined by an NCCL all-reduce ("strong" scaling: the total is
fixed). One step = one pass of that query over every shard. Prints ONE JSON line on rank 0.

  value      elements/s with the shards already resident in HBM (CUDA events, max over ranks)
  roofline   the fused reduce kernel alone: 4 bytes per element / its mean launch duration, against the measured HBM copy peak
  e2e        the same query through the host-buffer call (pinned host shard -> chunked H2D overlapped with the kernels ->
             record back), every step
  cpu_baseline / --impl reference   the reference's CPU SIMD loops (restated in oracle/cpu_simd.cpp) on the host cores
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC = "fused Where->Select->Sum elems/s & % of HBM roofline @1/2/4/8 B200"
UNIT = "elements/s"
THRESHOLD, THRESHOLD_TXT, ADDEND = 0.5, "0.5f", 3.0
WHERE, SELECT = f"x => x > {THRESHOLD_TXT}", "x => x * x + 3f"
SEED = 31
BYTES_PER_ELEM = 4   # algorithmic: one float read per element, nothing written
# DRAM bytes moved per algorithmic byte by the fused reduce kernel, from an ncu capture of it at 2^28 elements
# (dram__bytes_read.sum + dram__bytes_write.sum = 1.073766 GB + 3.3 MB for 1.073742 GB of input); every element is read
# once, so traffic scales with the element count.
TRAFFIC_RATIO = (1.073766e9 + 3.334e6) / 1.073741824e9


def _rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


# The other benchmark configurations of the reference's hot path, measured kernel-only on one GPU (device-resident inputs). Each entry:
# default log2(n), input generator(s), operators, terminal, algorithmic bytes per element as a function of selectivity.
CONFIG_WORKLOADS = {
    "c1-map": dict(log2n=20, gen=lambda n: [_rng(42).random(n, dtype=np.float32)], ops=[("S", "x => x * 2f + 1f")], term="ToArray",
                   bytes=lambda s: 8.0, what="C1 Select(x*2f+1f).ToArray() f32"),
    "c2-sum-f32": dict(log2n=24, gen=lambda n: [_rng(7).standard_normal(n, dtype=np.float32)], ops=[], term="Sum", bytes=lambda s: 4.0,
                       what="C2 Sum f32"),
    "c2-min-f32": dict(log2n=24, gen=lambda n: [_rng(7).standard_normal(n, dtype=np.float32)], ops=[], term="Min", bytes=lambda s: 4.0,
                       what="C2 Min f32"),
    "c2-avg-f32": dict(log2n=24, gen=lambda n: [_rng(7).standard_normal(n, dtype=np.float32)], ops=[], term="Average", bytes=lambda s: 4.0,
                       what="C2 Average f32"),
    "c2-sum-i32": dict(log2n=24, gen=lambda n: [_rng(8).integers(-1000, 1001, n, dtype=np.int32)], ops=[], term="Sum", bytes=lambda s: 4.0,
                       what="C2 Sum i32"),
    "c3-toarray-50": dict(log2n=26, gen=lambda n: [_rng(11).random(n, dtype=np.float32)], ops=[("W", "x => x > 0.5f"), ("S", "x => x * x + 3f")],
                          term="ToArray", bytes=lambda s: 4.0 + 4.0 * s, what="C3 Where(x>0.5f).Select(x*x+3f).ToArray() f32"),
    "c3-toarray-01": dict(log2n=26, gen=lambda n: [_rng(11).random(n, dtype=np.float32)], ops=[("W", "x => x > 0.99f"), ("S", "x => x * x + 3f")],
                          term="ToArray", bytes=lambda s: 4.0 + 4.0 * s, what="C3 Where(x>0.99f)...ToArray() f32"),
    "c3-toarray-99": dict(log2n=26, gen=lambda n: [_rng(11).random(n, dtype=np.float32)], ops=[("W", "x => x > 0.01f"), ("S", "x => x * x + 3f")],
                          term="ToArray", bytes=lambda s: 4.0 + 4.0 * s, what="C3 Where(x>0.01f)...ToArray() f32"),
    "c3-sum": dict(log2n=26, gen=lambda n: [_rng(11).random(n, dtype=np.float32)], ops=[("W", "x => x > 0.5f"), ("S", "x => x * x + 3f")],
                   term="Sum", bytes=lambda s: 4.0, what="C3 Where(x>0.5f).Select(x*x+3f).Sum() f32"),
    "headline-2p28": dict(log2n=28, gen=lambda n: [gen_shard(0, n)], ops=[("W", "x => x > 0.5f"), ("S", "x => x * x + 3f")],
                          term="Sum", bytes=lambda s: 4.0, what="headline Where(x>0.5f).Select(x*x+3f).Sum() f32 2^28"),
    "c4-zipdot": dict(log2n=28, gen=lambda n: [_rng(21).standard_normal(n, dtype=np.float32), _rng(22).standard_normal(n, dtype=np.float32)],
                      ops=[("Z", "(x, y) => x * y")], term="Sum", bytes=lambda s: 8.0, what="C4 a.Zip(b,(x,y)=>x*y).Sum() f32"),
    "c4-i64-where": dict(log2n=28, gen=lambda n: [_rng(23).integers(-2**63, 2**63 - 1, n, dtype=np.int64, endpoint=True)],
                         ops=[("W", "k => (k & 0xF) == 3")], term="ToArray", bytes=lambda s: 8.0 + 8.0 * s,
                         what="C4 keys.Where(k=>(k&0xF)==3).ToArray() i64"),
}


CONFIG_ORDER = ["c1-map", "c2-sum-f32", "c2-min-f32", "c2-avg-f32", "c2-sum-i32", "c3-sum", "c3-toarray-50", "c3-toarray-01",
                "c3-toarray-99", "headline-2p28", "c4-zipdot", "c4-i64-where"]


def _expected(spec_name, host, chk):
    """What the oracle says the configuration's query returns: ('array', ndarray) or ('scalar', value, raw fp64 or None, sum|x| or None)."""
    x = host[0]
    if spec_name == "c1-map":
        return ("array", chk.select_mul_add(x, 2.0, 1.0))
    if spec_name == "c2-sum-f32":
        v, raw = chk.sum_f32(x)
        return ("scalar", v, raw, chk.sum_abs(x))
    if spec_name == "c2-min-f32":
        return ("scalar", chk.min_f32(x), None, None)
    if spec_name == "c2-avg-f32":
        _v, raw = chk.sum_f32(x)
        return ("scalar", chk.average_f32(x), raw / x.size, chk.sum_abs(x) / x.size)
    if spec_name == "c2-sum-i32":
        return ("scalar", chk.sum_i32(x), None, None)
    if spec_name.startswith("c3-toarray"):
        thr = {"50": 0.5, "01": 0.99, "99": 0.01}[spec_name[-2:]]
        return ("array", chk.where_gt_select_sq_add(x, thr, 3.0))
    if spec_name in ("c3-sum", "headline-2p28"):
        v, raw, _cnt = chk.where_gt_select_sq_add_sum(x, 0.5, 3.0)
        return ("scalar", v, raw, raw)                      # every term is positive: sum|x| == sum
    if spec_name == "c4-zipdot":
        v, raw, sum_abs = chk.zip_mul_sum(x, host[1])
        return ("scalar", v, raw, sum_abs)
    if spec_name == "c4-i64-where":
        return ("array", chk.where_mask_eq_i64(x, 0xF, 3))
    raise KeyError(spec_name)


def measure_config(acc, name, steps, warmup, log2n=None, check=True):
    """K launches of one configuration's fused kernel on device-resident input (CUDA events on the launching stream, median),
    then the result of the last launch against the oracle on the same seeded input. Returns a dict for the JSON line."""
    import torch
    from dotcompute_b200 import native as N
    from dotcompute_b200.accelerator import dcb_type
    from dotcompute_b200.linq import CompiledPipeline
    from dotcompute_b200.sharded import finalize_record

    spec = CONFIG_WORKLOADS[name]
    n = 1 << (log2n or spec["log2n"])
    host = spec["gen"](n)
    bufs = [acc.Memory.AllocateAndCopyAsync(h) for h in host]
    kinds = {"S": N.OP_SELECT, "W": N.OP_WHERE, "Z": N.OP_ZIP}
    terms = {"ToArray": N.OP_TOARRAY, "Sum": N.OP_SUM, "Min": N.OP_MIN, "Max": N.OP_MAX, "Average": N.OP_AVERAGE, "Count": N.OP_COUNT}
    terminal = terms[spec["term"]]
    ops = tuple((kinds[k], lam) for k, lam in spec["ops"]) + ((terminal, None),)
    pipe = CompiledPipeline(acc, dcb_type(host[0].dtype), dcb_type(host[1].dtype) if len(host) > 1 else 0, ops)
    out = acc.Memory.AllocateAsync(n, pipe.out_dtype) if spec["term"] == "ToArray" else None
    rec = acc.Memory.AllocateAsync(16, np.int64)
    in0 = C.c_void_p(bufs[0].GetDeviceMemory())
    in1 = C.c_void_p(bufs[1].GetDeviceMemory()) if len(bufs) > 1 else None
    outp = C.c_void_p(out.GetDeviceMemory()) if out else None
    stream = torch.cuda.Stream()
    sh = stream.cuda_stream
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if n * host[0].itemsize * len(host) < (256 << 20) else None

    def step():
        N.check(N.lib().dcb_pipeline_run_async(pipe.handle, in0, in1, n, outp, n if out else 0, C.c_void_p(rec.GetDeviceMemory()), None,
                                               C.c_void_p(sh)), acc.handle)

    with torch.cuda.stream(stream):
        for _ in range(max(warmup, 3)):
            step()
        stream.synchronize()
        l0 = acc.LaunchCount
        times = []
        for _ in range(steps):
            if flush is not None:
                flush.fill_(1)              # inputs smaller than L2 would otherwise be served from it
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream); step(); b.record(stream)
            stream.synchronize()
            times.append(a.elapsed_time(b))
        launches = acc.LaunchCount - l0
    rec_host = rec.ToArray()
    has_where = any(k == "W" for k, _ in spec["ops"])
    count = int(rec_host[N.SLOT_COUNT]) if (has_where or spec["term"] in ("Count", "Average", "Min", "Max")) else n   # a plain map writes no record
    sel = count / n if spec["term"] == "ToArray" else 1.0
    ms = statistics.median(times)
    peak, kind = measured_peak_gbs()
    gbs = n * spec["bytes"](sel) / (ms * 1e-3) / 1e9
    parity = None
    if check:
        import oracle
        want = _expected(name, host, oracle.c_oracle())
        if want[0] == "array":
            got = out.CopyToAsync(count=count) if count else np.empty(0, pipe.out_dtype)
            parity = bool(got.dtype == want[1].dtype and got.size == want[1].size and
                          np.array_equal(got.view(np.uint8), want[1].view(np.uint8)))
        else:
            value = pipe.scalar(finalize_record(rec_host, terminal, pipe.info.out_type))
            _k, exp, raw, sum_abs = want
            parity = bool(value == exp)
            if raw is not None:             # floating reductions: also the tolerance rule against the fp64 value
                parity = parity and bool(abs(float(value) - raw) <= 1e-5 * sum_abs)
    for b in bufs:
        b.Dispose()
    if out:
        out.Dispose()
    rec.Dispose()
    return {"what": spec["what"], "n_elements": n, "ms": ms, "ms_best": min(times), "elements_per_s": n / (ms * 1e-3),
            "bytes_per_element": spec["bytes"](sel), "selectivity": sel, "achieved_gbs": gbs, "frac": gbs / peak, "peak_kind": kind,
            "parity": parity, "gpu_launches": int(launches), "precompiled_kernel": bool(pipe.precompiled),
            "l2": "L2 flushed between launches (256 MiB write)" if flush is not None else "input larger than L2",
            "dtype": str(host[0].dtype)}


def measure_relational(acc, steps=5):
    """OrderBy, GroupBy(Sum) and Join through the C ABI on device-resident keys: K timed calls each (CUDA events), the result
    of the last one against numpy's stable sort / a dictionary pass / a sequential join. Bytes are what the multi-block
    algorithms must move: a radix pass reads the keys twice and moves (key, index) once."""
    import torch
    from dotcompute_b200 import native as N
    out = {}
    peak, _kind = measured_peak_gbs()
    dev = "cuda"

    def timed(fn):
        fn(); torch.cuda.synchronize()
        ts = []
        for _ in range(steps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record(); torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return statistics.median(ts)

    # OrderBy: 2^26 float32 keys, stable argsort + gather
    n = 1 << 26
    x = _rng(41).random(n, dtype=np.float32)
    dx = torch.from_numpy(x).to(dev)
    srt = torch.empty_like(dx)

    def sort_step():   # what OrderBy() runs for 4-byte elements: the elements travel beside their keys, no gather
        N.check(N.lib().dcb_sort_by_key(acc.handle, N.T_F32, C.c_void_p(dx.data_ptr()), n, 0, 4, C.c_void_p(dx.data_ptr()),
                                        C.c_void_p(srt.data_ptr()), C.c_void_p(1)), acc.handle)
    ms = timed(sort_step)
    got = srt.cpu().numpy()
    bytes_per = 16 + 4 * (4 + 8 + 8)                    # prepare (key, value in; bits, value out), four passes
    out["orderby-f32-2p26"] = {"what": "OrderBy() over 2^26 float32: stable 4-pass radix sort of (key, element) pairs", "n_elements": n, "ms": ms,
                               "elements_per_s": n / (ms * 1e-3), "bytes_per_element": bytes_per,
                               "achieved_gbs": n * bytes_per / (ms * 1e-3) / 1e9, "frac": n * bytes_per / (ms * 1e-3) / 1e9 / peak,
                               "parity": bool(np.array_equal(got, np.sort(x, kind="stable")))}
    del dx, srt
    # GroupBy: 2^26 int32 values, key = v % 1000, Sum per key
    v = _rng(42).integers(0, 1_000_000, n, dtype=np.int32)
    k = (v % 1000).astype(np.int32)
    dv, dk = torch.from_numpy(v).to(dev), torch.from_numpy(k).to(dev)
    cap = 4096
    first = torch.empty(cap, dtype=torch.int32, device=dev)
    cnt = torch.empty(cap, dtype=torch.int64, device=dev)
    f64 = torch.empty(cap, dtype=torch.float64, device=dev)
    i64 = torch.empty(cap, dtype=torch.int64, device=dev)
    groups = C.c_int64()

    def group_step():
        N.check(N.lib().dcb_group_aggregate(acc.handle, N.T_I32, C.c_void_p(dk.data_ptr()), N.T_I32, C.c_void_p(dv.data_ptr()), n, N.AGG_SUM, cap,
                                            C.c_void_p(first.data_ptr()), C.c_void_p(cnt.data_ptr()), C.c_void_p(f64.data_ptr()),
                                            C.c_void_p(i64.data_ptr()), C.byref(groups), C.c_void_p(1)), acc.handle)
    ms = timed(group_step)
    g = int(groups.value)
    order = np.unique(k, return_index=True)[1]
    keys_first = k[np.sort(order)]
    sums = np.bincount(k, weights=None, minlength=1000)                      # counts
    want_sum = np.zeros(1000, dtype=np.int64)
    np.add.at(want_sum, k, v.astype(np.int64))
    ok = g == keys_first.size and np.array_equal(k[first.cpu().numpy()[:g].astype(np.int64)], keys_first) and \
        np.array_equal(i64.cpu().numpy()[:g], want_sum[keys_first]) and np.array_equal(cnt.cpu().numpy()[:g], sums[keys_first])
    bytes_per = 12 + 4 + 8                                                   # key -> sortable bits and position, which bits differ, bits and value
    out["groupby-sum-i32-2p26"] = {"what": "GroupBy(v % 1000).Sum() over 2^26 int32 (1000 groups, first-occurrence order; keys that differ "
                                           "in their low bits only index a table, no sort)", "n_elements": n,
                                   "ms": ms, "elements_per_s": n / (ms * 1e-3), "bytes_per_element": bytes_per,
                                   "achieved_gbs": n * bytes_per / (ms * 1e-3) / 1e9, "frac": n * bytes_per / (ms * 1e-3) / 1e9 / peak,
                                   "parity": bool(ok)}
    del dv, dk
    # Join: 2^24 outer keys against 2^20 inner keys (int64), inner join pairs in Enumerable.Join order
    no, ni = 1 << 24, 1 << 20
    ok_ = _rng(43).integers(0, 1 << 21, no, dtype=np.int64)
    ik_ = _rng(44).integers(0, 1 << 21, ni, dtype=np.int64)
    do, di = torch.from_numpy(ok_).to(dev), torch.from_numpy(ik_).to(dev)
    pairs = C.c_int64()
    N.check(N.lib().dcb_join_indices(acc.handle, N.T_I64, C.c_void_p(do.data_ptr()), no, C.c_void_p(di.data_ptr()), ni, N.JOIN_INNER, 0, None, None,
                                     C.byref(pairs), C.c_void_p(1)), acc.handle)
    m = int(pairs.value)
    oo = torch.empty(max(m, 1), dtype=torch.int32, device=dev)
    io = torch.empty(max(m, 1), dtype=torch.int32, device=dev)

    def join_step():
        N.check(N.lib().dcb_join_indices(acc.handle, N.T_I64, C.c_void_p(do.data_ptr()), no, C.c_void_p(di.data_ptr()), ni, N.JOIN_INNER, m,
                                         C.c_void_p(oo.data_ptr()), C.c_void_p(io.data_ptr()), C.byref(pairs), C.c_void_p(1)), acc.handle)
    ms = timed(join_step)
    go, gi = oo.cpu().numpy().astype(np.int64), io.cpu().numpy().astype(np.int64)
    srt_i = np.argsort(ik_, kind="stable")
    lo, hi = np.searchsorted(ik_[srt_i], ok_, "left"), np.searchsorted(ik_[srt_i], ok_, "right")
    want_o = np.repeat(np.arange(no), hi - lo)
    ok = m == int((hi - lo).sum()) and np.array_equal(go, want_o) and bool(np.all(ok_[go] == ik_[gi])) and \
        bool(np.all((np.diff(gi) > 0) | (np.diff(go) > 0)))                  # inner indices ascend inside one outer element
    out["join-inner-i64-2p24x2p20"] = {"what": "Join of 2^24 outer and 2^20 inner int64 keys, pairs in Enumerable.Join order", "n_elements": no,
                                       "pairs": m, "ms": ms, "elements_per_s": no / (ms * 1e-3), "parity": bool(ok)}
    del do, di, oo, io
    # Scan: running sum of 2^26 float32 (fp64 accumulation, each output rounded once)
    x = _rng(45).random(n, dtype=np.float32)
    dx = torch.from_numpy(x).to(dev)
    ds = torch.empty_like(dx)
    ms = timed(lambda: N.check(N.lib().dcb_prefix_sum(acc.handle, N.T_F32, C.c_void_p(dx.data_ptr()), n, 1, C.c_void_p(ds.data_ptr()), C.c_void_p(1)), acc.handle))
    want = np.cumsum(x.astype(np.float64))
    err = float(np.max(np.abs(ds.cpu().numpy().astype(np.float64) - want)))
    out["scan-f32-2p26"] = {"what": "Scan(): inclusive running sum of 2^26 float32 (tile totals, scan of totals, tiles)", "n_elements": n, "ms": ms,
                            "elements_per_s": n / (ms * 1e-3), "bytes_per_element": 12, "achieved_gbs": n * 12 / (ms * 1e-3) / 1e9,
                            "frac": n * 12 / (ms * 1e-3) / 1e9 / peak, "max_abs_error": err,
                            "parity": bool(err <= 1e-5 * float(np.abs(x).astype(np.float64).sum()))}
    return out


def run_config(args) -> int:
    """One of the secondary configurations on its own: one JSON line in the shape of the headline's."""
    from dotcompute_b200 import CudaAccelerator
    acc = CudaAccelerator(0)
    m = measure_config(acc, args.workload, args.steps, args.warmup, args.log2n if args.log2n != 30 else None, not args.no_check)
    print(json.dumps({
        "metric": "kernel elements/s, device-resident (secondary configuration)", "value": m["elements_per_s"], "unit": UNIT, "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": m["ms"], "ms_best": m["ms_best"], "higher_is_better": True,
        "scaling": "n/a", "vs_baseline": None, "dtype": m["dtype"], "data": "synthetic",
        "config": {"workload": m["what"], "n_elements": m["n_elements"], "selectivity": m["selectivity"], "l2": m["l2"]},
        "roofline": {"bound": "hbm", "achieved": m["achieved_gbs"], "peak": measured_peak_gbs()[0], "unit": "GB/s", "frac": m["frac"],
                     "traffic": None, "peak_kind": m["peak_kind"], "bytes_per_element": m["bytes_per_element"]},
        "parity": m["parity"], "gpu_launches": m["gpu_launches"], "precompiled_kernel": m["precompiled_kernel"]}))
    return 0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--log2n", type=int, default=30, help="log2 of the total element count (default 30 = config 5)")
    ap.add_argument("--e2e-steps", type=int, default=0, help="end-to-end steps (default min(steps, 8))")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-check", action="store_true", help="skip the oracle check of the result")
    ap.add_argument("--no-extras", action="store_true", help="skip the ToArray half of config 5 and the other reductions")
    ap.add_argument("--no-configs", action="store_true", help="skip the per-configuration block of the 1-GPU run")
    ap.add_argument("--config-steps", type=int, default=10, help="timed launches per secondary configuration")
    ap.add_argument("--combine", default="fused", choices=["fused", "nccl"],
                    help="multi-GPU exchange of partial sums: inside the reduce kernel over NVLink peer stores (fused) or an NCCL all-reduce")
    ap.add_argument("--no-numa", action="store_true", help="do not bind the process to the GPU's NUMA node")
    ap.add_argument("--no-overlap", action="store_true",
                    help="launch the reduce kernels without programmatic stream serialisation (DCB_OPT_OVERLAP_LAUNCHES off)")
    ap.add_argument("--no-graph", action="store_true",
                    help="enqueue the timed steps one by one instead of replaying them as one captured CUDA graph")
    ap.add_argument("--profile", action="store_true",
                    help="minimal run for a profiler: no clock spin, no e2e, no CPU baseline, no oracle check")
    ap.add_argument("--workload", default="c5-sum", choices=sorted(CONFIG_WORKLOADS) + ["c5-sum"],
                    help="c5-sum (default, the headline) or one of the other benchmark configurations, 1 GPU, kernel-only")
    args = ap.parse_args()
    if args.profile:
        args.no_e2e = args.no_cpu_baseline = args.no_check = args.no_extras = args.no_configs = True
    return args


def gen_shard(start: int, stop: int, out: np.ndarray | None = None) -> np.ndarray:
    """Elements [start, stop) of rng(31).random(float32): PCG64 yields two floats per 64-bit step, so a shard is
    reached by advancing the generator (start must be even). Generated in parallel blocks."""
    assert start % 2 == 0
    n = stop - start
    if out is None:
        out = np.empty(n, dtype=np.float32)
    block = 1 << 24
    jobs = [(o, min(o + block, n)) for o in range(0, n, block)]

    def work(j):
        lo, hi = j
        bg = np.random.PCG64(SEED)
        bg.advance((start + lo) // 2)
        np.random.Generator(bg).random(out=out[lo:hi], dtype=np.float32)

    threads = [threading.Thread(target=lambda js=jobs[i::8]: [work(j) for j in js]) for i in range(8)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    return out


class ClockSampler:
    """nvidia-smi sampling of SM clock and throttle reasons while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_uuid: str | None):
        self.rows = []
        self.proc = None
        cmd = ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50"]
        if gpu_uuid:
            cmd += ["-i", gpu_uuid if gpu_uuid.startswith("GPU-") else "GPU-" + gpu_uuid]
        try:
            self.proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            parts = [p.strip() for p in r.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); smax.append(float(parts[1])); power.append(float(parts[2]))
            except ValueError:
                continue
            for nm, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "reasons": sorted(reasons), "samples": len(sm),
                "window": "0.7 s of the same steps run untimed immediately before, plus the timed region (50 ms sampling)"}


def bind_to_gpu_numa_node(device_index: int) -> str:
    """Restrict this process to the CPUs of the NUMA node the GPU hangs off, before the pinned host shard is allocated and
    filled, so that its pages are local to the GPU's PCIe root (first-touch placement). Returns a note for the JSON line."""
    try:
        import torch
        p = torch.cuda.get_device_properties(device_index)
        bdf = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return "numa node unknown"
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0) & cpus
        if not allowed:
            return f"gpu on numa node {node}, none of its cpus allowed here"
        os.sched_setaffinity(0, allowed)
        return f"bound to numa node {node} ({len(allowed)} cpus)"
    except Exception as exc:   # no sysfs, no permission: leave the placement to the OS
        return f"not bound ({type(exc).__name__})"


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        return 6650.0, "fallback"


def cpu_baseline(n_total: int, time_limit_s: float = 12.0) -> dict:
    """Times the restated CPU SIMD backend on this host: fused Where->Select->Sum over a bounded sample of the same
    seeded workload, all hardware threads; plus the one-thread scalar loop the shipped provider runs today."""
    import oracle
    simd = oracle.cpu_simd()
    n = min(n_total, 1 << 28)
    x = gen_shard(0, n)
    simd.where_select_sum(x, THRESHOLD, ADDEND)          # warm-up, page-in
    t0 = time.perf_counter(); reps = 0
    while True:
        simd.where_select_sum(x, THRESHOLD, ADDEND)
        reps += 1
        dt = time.perf_counter() - t0
        if dt > time_limit_s * 0.6 or reps >= 200:
            break
    simd_eps = n * reps / dt
    t0 = time.perf_counter()
    simd.scalar_where_select_sum(x, THRESHOLD, ADDEND)
    scalar_eps = n / (time.perf_counter() - t0)
    return {"value": simd_eps, "unit": UNIT, "cores": simd.threads, "kind": "port",
            "sample": f"first 2^{int(np.log2(n))} elements of the workload, {reps} passes, {simd.variant} x {simd.threads} threads "
                      f"(restated CPU SIMD backend); the reference itself is C#/.NET and cannot run on this box",
            "scalar_1thread": scalar_eps}


def run_reference(args) -> int:
    """--impl reference: the reference's CPU implementation of the path (restated SIMD loops), all host threads, on the
    same workload: every step is one pass over all 2^log2n elements. Rank 0 alone works; other ranks leave."""
    if int(os.environ.get("RANK", "0")) != 0:
        return 0
    import oracle
    simd = oracle.cpu_simd()
    n = 1 << args.log2n
    x = gen_shard(0, n)
    for _ in range(max(args.warmup, 1)):
        got = simd.where_select_sum(x, THRESHOLD, ADDEND)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        got = simd.where_select_sum(x, THRESHOLD, ADDEND)
    dt = time.perf_counter() - t0
    eps = n * args.steps / dt
    t0 = time.perf_counter()
    m = min(n, 1 << 27)
    simd.scalar_where_select_sum(x[:m], THRESHOLD, ADDEND)
    scalar_eps = m / (time.perf_counter() - t0)
    want, raw, _cnt = oracle.c_oracle().where_gt_select_sq_add_sum(x, THRESHOLD, ADDEND)
    sample = (f"each step = one pass over all 2^{args.log2n} elements of the workload; {simd.variant}, {simd.threads} threads; "
              f"C++ restatement of the reference's CPU SIMD backend (the C#/.NET original cannot run here)")
    line = {
        "impl": "reference", "metric": METRIC, "value": eps, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"C5: Where(x>0.5f).Select(x*x+3f).Sum() over 2^{args.log2n} float32 uniform[0,1) seed 31, contiguous shards",
                   "n_elements": n},
        "cpu_baseline": {"value": eps, "unit": UNIT, "cores": simd.threads, "kind": "port", "sample": sample,
                         "scalar_1thread": scalar_eps,
                         "scalar_1thread_note": "the one-thread scalar loop is what the shipped provider really runs for this query (System.Linq fallback)"},
        "e2e": {"value": eps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        # fp32 lane accumulators, as in the reference's SIMD Sum: its own error, outside the 1e-5 rule the GPU path meets
        "rel_err_vs_fp64": abs(float(got) - raw) / raw,
    }
    print(json.dumps(line))
    return 0


def toarray_block(args, acc, q, pinned, stream, world, rank, device, fused, barrier):
    """Config 5's other half: Where -> Select -> ToArray over the same shards. Each rank compacts its shard; the survivor
    counts are exchanged by the one-warp peer-store kernel behind the compaction (no NCCL, no host round trip), which leaves
    the rank's output offset and the global total in the record. Checked: the rank's output against the oracle on its own
    shard, bit for bit; offset == sum of the lower ranks' counts; total == sum of all counts."""
    import torch
    import torch.distributed as dist
    from dotcompute_b200 import native as N
    import oracle

    n_local = q.local.Length
    pipe = q.pipeline(N.OP_TOARRAY)
    out = acc.Memory.AllocateAsync(max(n_local, 1), np.float32)
    rec = torch.zeros(N.SLOT_NSLOTS, dtype=torch.int64, device=device)
    steps = max(3, min(args.steps, 10))
    with torch.cuda.stream(stream):
        for _ in range(3):
            q.enqueue_compact(out, stream, rec)
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(stream)
        for _ in range(steps):
            q.enqueue_compact(out, stream, rec)
        t1.record(stream)
        barrier()
        ms = t0.elapsed_time(t1) / steps
        # the compaction kernel alone (eventful pass, no exchange), for the roofline fraction of this kernel
        ka, kb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        kms = []
        for _ in range(steps):
            ka.record(stream)
            N.check(N.lib().dcb_pipeline_run_async(pipe.handle, C.c_void_p(q.local.GetDeviceMemory()), None, n_local,
                                                   C.c_void_p(out.GetDeviceMemory()), n_local, C.c_void_p(rec.data_ptr()), None,
                                                   C.c_void_p(stream.cuda_stream)), acc.handle)
            kb.record(stream)
            stream.synchronize()
            kms.append(ka.elapsed_time(kb))
        if fused:                                            # leave the record exchanged, as after a full step
            N.check(N.lib().dcb_peer_exchange_async(acc.handle, C.c_void_p(rec.data_ptr()), pipe.info.out_type,
                                                    C.c_void_p(stream.cuda_stream)), acc.handle)
        stream.synchronize()
    host = rec.cpu().numpy()
    if fused:
        local_count, offset, total = int(host[N.SLOT_LOCAL_COUNT]), int(host[N.SLOT_OFFSET]), int(host[N.SLOT_COUNT])
    else:
        local_count = int(host[N.SLOT_COUNT])
        offset = total = None
    want = oracle.c_oracle().where_gt_select_sq_add(pinned.array, THRESHOLD, ADDEND)
    got = out.CopyToAsync(count=local_count) if local_count else np.empty(0, np.float32)
    data_ok = bool(got.size == want.size and np.array_equal(got.view(np.uint32), want.view(np.uint32)))
    counts = [want.size]
    if world > 1:
        allc = [torch.zeros(1, dtype=torch.int64, device=device) for _ in range(world)]
        dist.all_gather(allc, torch.tensor([want.size], dtype=torch.int64, device=device))
        counts = [int(c.item()) for c in allc]
    if not fused:
        offset, total = sum(counts[:rank]), sum(counts)      # the NCCL route: offsets from the all-gather of counts
    offsets_ok = bool(offset == sum(counts[:rank]) and total == sum(counts))
    t = torch.tensor([ms, statistics.median(kms), 0.0 if data_ok else 1.0, 0.0 if offsets_ok else 1.0], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    out.Dispose()
    ms, kms_med, bad_data, bad_off = (float(v) for v in t)
    n_total = 1 << args.log2n
    s_all = sum(counts) / n_total
    peak, _kind = measured_peak_gbs()
    gbs_gpu = n_local * (4.0 + 4.0 * local_count / max(n_local, 1)) / (kms_med * 1e-3) / 1e9
    return {"workload": f"C5: Where(x>0.5f).Select(x*x+3f).ToArray() over 2^{args.log2n} float32, contiguous shards, output in rank order",
            "ms_per_step": ms, "elements_per_s": n_total / (ms * 1e-3), "steps": steps, "selectivity": s_all,
            "bytes_per_element": 4.0 + 4.0 * s_all, "kernel_ms": kms_med, "kernel_gbs_per_gpu": gbs_gpu, "frac": gbs_gpu / peak,
            "parity": bad_data == 0.0, "offsets_ok": bad_off == 0.0, "total_survivors": int(sum(counts)),
            "offset_rank0": 0, "exchange": ("one-warp peer-store kernel behind the compaction (offset and total in the record)" if fused
                                            else ("none (1 GPU)" if world == 1 else "all-gather of counts (NCCL)"))}


def reductions_parity_block(args, acc, dev, pinned, world, rank, device, ops):
    """Min / Max / Average / Count of the mapped survivors (f32) and Sum over an int32 shard, through the same exchange as
    the headline Sum; every result against the oracle's, combined over the ranks on the host."""
    import torch
    import torch.distributed as dist
    from dotcompute_b200 import native as N
    from dotcompute_b200.sharded import ShardedQuery
    import oracle

    chk = oracle.c_oracle()
    want = chk.where_gt_select_sq_add(pinned.array, THRESHOLD, ADDEND)
    w64 = want.astype(np.float64)
    xi = (pinned.array * np.float32(2001.0)).astype(np.int32) - np.int32(1000)        # ints in [-1000, 1000]
    local = [float(want.min()) if want.size else float("inf"), float(want.max()) if want.size else float("-inf"),
             float(w64.sum()), float(np.abs(w64).sum()), float(want.size), float(xi.astype(np.int64).sum())]
    allv = [local]
    if world > 1:
        allv = [None] * world
        dist.all_gather_object(allv, local)
    g_min, g_max = min(v[0] for v in allv), max(v[1] for v in allv)
    g_sum, g_abs, g_cnt, g_isum = (sum(v[i] for v in allv) for i in (2, 3, 4, 5))
    q = ShardedQuery(acc, dev, ops)
    got_min, got_max, got_avg, got_cnt = q.Min(), q.Max(), q.Average(), q.Count()
    di = acc.Memory.AllocateAndCopyAsync(xi)
    got_isum = ShardedQuery(acc, di, ()).Sum()
    di.Dispose()
    detail = {"min": bool(float(got_min) == g_min), "max": bool(float(got_max) == g_max), "count": bool(int(got_cnt) == int(g_cnt)),
              "average": bool(abs(float(got_avg) - g_sum / g_cnt) <= 1e-5 * g_abs / g_cnt), "sum_i32": bool(int(got_isum) == int(g_isum))}
    ok = torch.tensor([1 if all(detail.values()) else 0], dtype=torch.int32, device=device)
    if world > 1:
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    return bool(int(ok[0])), detail


def main() -> int:
    args = parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.workload != "c5-sum":
        return run_config(args)

    import torch
    import torch.distributed as dist

    from dotcompute_b200 import CudaAccelerator, native as N
    from dotcompute_b200.sharded import ShardedQuery, connect_peers, finalize_record, shard_bounds, _stream_handle

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if rank == 0:
            print(f"bench.py: --gpus {args.gpus} but WORLD_SIZE={world}; launch with torchrun --nproc-per-node {args.gpus}", file=sys.stderr)
        if world == 1 and args.gpus > 1:
            return 2
    torch.cuda.set_device(local_rank)
    device = torch.device(f"cuda:{local_rank}")
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    n_total = 1 << args.log2n
    start, stop = shard_bounds(n_total, world, rank, 4)
    n_local = stop - start
    acc = CudaAccelerator(local_rank)
    if not args.no_overlap:
        # The shards are written once, before the timed region: a query's input never depends on the kernel before it on the
        # stream, so back-to-back queries may overlap their launch and ramp-up with the previous query's tail.
        acc.SetOption(N.OPT_OVERLAP_LAUNCHES, 1)
    numa_note = "not requested" if args.no_numa else bind_to_gpu_numa_node(local_rank)

    # ---- data: pinned host shard (the e2e source), copied once to HBM (the resident source)
    pinned = acc.Memory.AllocatePinned(n_local, np.float32)
    gen_shard(start, stop, pinned.array)
    dev = acc.Memory.AllocateAsync(n_local, np.float32)
    N.check(N.lib().dcb_h2d_async(acc.handle, dev.handle, 0, C.c_void_p(pinned.ptr), n_local * 4, None), acc.handle)
    acc.Synchronize()

    fused = False
    if world > 1 and args.combine == "fused":
        # Every rank must take the same route: agree on whether the peer set-up (CUDA IPC) worked everywhere.
        try:
            ok = connect_peers(acc)
        except Exception as exc:
            print(f"bench.py[{rank}]: peer exchange set-up failed ({exc}); using the NCCL all-reduce", file=sys.stderr)
            ok = False
        flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        fused = bool(int(flag[0]))
        if ok and not fused:
            from dotcompute_b200.sharded import disconnect_peers
            disconnect_peers(acc)
    ops = ((N.OP_WHERE, WHERE), (N.OP_SELECT, SELECT))
    q = ShardedQuery(acc, dev, ops)
    pipe = q.pipeline(N.OP_SUM)
    stream = torch.cuda.Stream(device=device)
    sh = _stream_handle(stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    launches0 = None
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            q.enqueue_reduce(N.OP_SUM, stream)
        barrier()
        # The timed region lasts milliseconds, far less than nvidia-smi's sampling period. So the sampler starts here, the
        # same step is repeated untimed for about 0.7 s (clocks settle under this load), and the timed region follows at
        # once; the clock record covers that window up to the end of the timed region.
        sampler = ClockSampler(str(torch.cuda.get_device_properties(device).uuid)) if (rank == 0 and not args.profile) else None
        # Every rank must run the SAME number of steps (each step ends in a collective), so the length of this untimed
        # run is agreed on first: time one batch, take the slowest rank's figure, derive the count from it.
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(8):
            q.enqueue_reduce(N.OP_SUM, stream)
        e1.record(stream)
        stream.synchronize()
        bt = torch.tensor([max(e0.elapsed_time(e1), 1e-3)], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(bt, op=dist.ReduceOp.MAX)
        n_batches = 0 if args.profile else int(min(max(700.0 / float(bt[0]), 1), 2000))
        for _ in range(n_batches):
            for _ in range(8):
                q.enqueue_reduce(N.OP_SUM, stream)
            stream.synchronize()
        barrier()
        # ---- timed region: K steps, device-resident
        q._setup()

        def run_steps(k_start=None, k_stop=None):
            """K steps: the fused kernel over this rank's shard, then the exchange of the partial. Returns the last record."""
            last, rec = None, None
            for i in range(args.steps):
                slot = q._step % q.RING
                q._step += 1
                rec = q._ring[slot]
                if q._exchange_done[slot] is not None:
                    stream.wait_event(q._exchange_done[slot])
                if k_start is not None:
                    k_start[i].record(stream)
                q.launch_local(N.OP_SUM, stream, rec)           # the fused Where->Select->Sum kernel
                if k_stop is not None:
                    k_stop[i].record(stream)
                last = q.exchange(N.OP_SUM, stream, rec, slot)   # side-stream NVLink exchange (fused) or NCCL all-reduce
            if last is not None:
                stream.wait_event(last)                          # the region ends when the last record is global
            return rec

        t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        graph = None
        if not args.no_graph and (world == 1 or fused):
            # The K steps are captured once as a CUDA graph (kernels, events and the side stream's exchange kernels) and
            # the timed region replays it: no per-launch host work between kernels. All ranks replay, or none does.
            ok = True
            try:
                q._step = 0
                q._exchange_done = [None] * q.RING
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    rec = run_steps()
            except Exception as exc:                             # capture refused: fall back to plain launches
                print(f"bench.py[{rank}]: CUDA graph capture failed ({exc}); timing plain launches", file=sys.stderr)
                ok = False
            flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=device)
            if world > 1:
                dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if int(flag[0]):
                graph.replay()                                   # one untimed replay (graph upload)
            else:
                graph = None
                q._exchange_done = [None] * q.RING
            barrier()
        launches0 = acc.LaunchCount
        if graph is not None:
            with torch.cuda.stream(stream):
                t_begin.record(stream)
                graph.replay()
                t_end.record(stream)
            graph_launches = args.steps * (2 if fused else 1)
        else:
            t_begin.record(stream)
            rec = run_steps()
            t_end.record(stream)
        barrier()
        total_ms = t_begin.elapsed_time(t_end)
        # Second pass of the same K steps, launched one by one with CUDA events around every kernel: the per-launch
        # duration the roofline figure is computed from (events cannot be timed inside a replayed graph).
        k_start = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
        k_stop = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
        q._exchange_done = [None] * q.RING
        rec = run_steps(k_start, k_stop)
        barrier()
        launches = graph_launches if graph is not None else (acc.LaunchCount - launches0) // 2
        clocks = sampler.stop() if sampler else None
        kernel_ms = [a.elapsed_time(b) for a, b in zip(k_start, k_stop)]
        rec_host = rec.cpu().numpy().copy()

    t = torch.tensor([total_ms, statistics.mean(kernel_ms)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, kernel_ms_mean = float(t[0]), float(t[1])
    ms_per_step = total_ms / args.steps
    value = n_total / (ms_per_step * 1e-3)

    res = finalize_record(rec_host, N.OP_SUM, pipe.info.out_type)
    got = np.float32(res.f64)

    # ---- parity of the benchmarked result against the oracle (each rank checks its shard's fp64 partial)
    parity = None
    if not args.no_check:
        import oracle
        chk = oracle.c_oracle()
        _w, raw_local, _c = chk.where_gt_select_sq_add_sum(pinned.array, THRESHOLD, ADDEND)
        tt = torch.tensor([raw_local], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.SUM)
        raw_total = float(tt[0])
        parity = bool(abs(float(got) - raw_total) <= 1e-5 * raw_total)   # all terms are positive: sum|x| == sum

    # ---- end to end: host shard -> device -> result, every step, through dcb_pipeline_run_host
    e2e = None
    if not args.no_e2e:
        e2e_steps = args.e2e_steps or min(args.steps, 8)
        r = N.Result()
        part = torch.zeros(2, dtype=torch.float64, device=device)

        def e2e_step():
            N.check(N.lib().dcb_pipeline_run_host(pipe.handle, C.c_void_p(pinned.ptr), None, n_local, None, 0, C.byref(r)), acc.handle)
            if world > 1:
                part[0] = r.f64
                dist.all_reduce(part, op=dist.ReduceOp.SUM)
                return float(part[0].item())
            return r.f64

        for _ in range(2):
            e2e_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        w0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_val = e2e_step()
        e1.record()
        barrier()
        wall_ms = (time.perf_counter() - w0) * 1e3
        te = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e_ms = float(te[0]) / e2e_steps
        n_chunks = -(-n_local * 4 // (32 << 20))
        e2e = {"value": n_total / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": n_total * 4,
               "d2h_bytes_per_step": 128 * n_chunks * world, "ms_per_step": e2e_ms, "steps": e2e_steps, "wall_ms_per_step": wall_ms / e2e_steps, "host_placement": numa_note,
               "note": "pinned host shard -> 32 MiB chunks through a three-slot staging ring, H2D overlapped with per-chunk kernels -> records D2H; PCIe-bound"}
        if not args.no_extras:
            # The ToArray half end to end: host shard in, compacted host array out (two-slot output ring, D2H of each chunk's
            # survivors one chunk behind the kernels, overlapping the uploads).
            pipe_arr = q.pipeline(N.OP_TOARRAY)
            out_pinned = acc.Memory.AllocatePinned(n_local, np.float32)
            ra = N.Result()

            def e2e_arr_step():
                N.check(N.lib().dcb_pipeline_run_host(pipe_arr.handle, C.c_void_p(pinned.ptr), None, n_local, C.c_void_p(out_pinned.ptr), n_local,
                                                      C.byref(ra)), acc.handle)
                return int(ra.count)

            e2e_arr_step()
            barrier()
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            arr_steps = max(2, min(e2e_steps, 4))
            for _ in range(arr_steps):
                cnt_local = e2e_arr_step()
            a1.record()
            barrier()
            ta = torch.tensor([a0.elapsed_time(a1) / arr_steps, float(cnt_local)], dtype=torch.float64, device=device)
            tmax = ta.clone()
            if world > 1:
                dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
                dist.all_reduce(ta, op=dist.ReduceOp.SUM)
            arr_ok = None
            if not args.no_check:
                import oracle
                want_arr = oracle.c_oracle().where_gt_select_sq_add(pinned.array, THRESHOLD, ADDEND)
                arr_ok = bool(cnt_local == want_arr.size and np.array_equal(out_pinned.array[:cnt_local].view(np.uint32), want_arr.view(np.uint32)))
                okt = torch.tensor([1 if arr_ok else 0], dtype=torch.int32, device=device)
                if world > 1:
                    dist.all_reduce(okt, op=dist.ReduceOp.MIN)
                arr_ok = bool(int(okt[0]))
            e2e["toarray"] = {"value": n_total / (float(tmax[0]) * 1e-3), "unit": UNIT, "ms_per_step": float(tmax[0]), "steps": arr_steps,
                              "h2d_bytes_per_step": n_total * 4, "d2h_bytes_per_step": int(float(ta[1])) * 4 + 128 * n_chunks * world,
                              "parity": arr_ok}
            out_pinned.Dispose()

    # ---- config 5's ToArray half and the other reductions, through the same exchange; the NCCL all-reduce beside it
    toarray = reductions_ok = reductions_detail = nccl_arm = None
    if not args.profile and not args.no_extras:
        toarray = toarray_block(args, acc, q, pinned, stream, world, rank, device, fused, barrier)
        reductions_ok, reductions_detail = reductions_parity_block(args, acc, dev, pinned, world, rank, device, ops)
        if world > 1 and fused:
            from dotcompute_b200.sharded import combine_record
            recn = torch.zeros(N.SLOT_NSLOTS, dtype=torch.int64, device=device)
            with torch.cuda.stream(stream):
                for _ in range(3):
                    q.launch_local(N.OP_SUM, stream, recn)
                    combine_record(recn, N.OP_SUM, pipe.info.out_type)
                barrier()
                n0, n1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                n0.record(stream)
                for _ in range(args.steps):
                    q.launch_local(N.OP_SUM, stream, recn)
                    combine_record(recn, N.OP_SUM, pipe.info.out_type)     # ncclAllReduce of the fp64 partial on the same stream
                n1.record(stream)
                barrier()
            tn = torch.tensor([n0.elapsed_time(n1) / args.steps], dtype=torch.float64, device=device)
            dist.all_reduce(tn, op=dist.ReduceOp.MAX)
            got_n = np.float32(finalize_record(recn.cpu().numpy(), N.OP_SUM, pipe.info.out_type).f64)
            nccl_arm = {"ms_per_step": float(tn[0]), "elements_per_s": n_total / (float(tn[0]) * 1e-3), "result": float(got_n),
                        "same_result_as_peer_exchange": bool(got_n == got),
                        "what": "the same K steps with an NCCL all-reduce of the fp64 partial after every kernel (plain launches)"}

    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        achieved = n_local * BYTES_PER_ELEM / (kernel_ms_mean * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"C5: Where(x>0.5f).Select(x*x+3f).Sum() over 2^{args.log2n} float32 uniform[0,1) seed 31, contiguous shards",
                       "n_elements": n_total, "elements_per_gpu": n_local, "l2": "inputs larger than L2 (shard >= 512 MiB)",
                       "combine": ("none (1 GPU)" if world == 1 else
                                   "one-warp exchange kernel on a side stream: NVLink peer stores of the fp64 partials, fold in rank order, overlapped with the next step's kernel" if fused else
                                   "NCCL all-reduce of one fp64 partial per GPU"),
                       "precompiled_kernel": bool(pipe.precompiled),
                       "launch": ("the K steps are replayed as one CUDA graph" if graph is not None else "K plain launches") +
                                 ("" if args.no_overlap else "; reduce kernels launched with programmatic stream serialisation")},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": n_local * BYTES_PER_ELEM * TRAFFIC_RATIO,
                         "traffic_source": "ncu capture at 2^28 elements scaled by the element count (bytes per launch)",
                         "peak_kind": peak_kind, "kernel": "dcb_reduce_vec (fused Where->Select->Sum)",
                         "timing": "mean of per-launch CUDA-event durations over a second, un-graphed pass of the same K steps",
                         "kernel_ms": kernel_ms_mean, "frac_of_nominal_8TBs": achieved / 8000.0},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "parity": parity,
            "result": float(got),
        }
        if e2e:
            line["e2e"] = e2e
        if toarray is not None:
            line["toarray"] = toarray
            line["reductions_parity"] = reductions_ok
            line["reductions_parity_detail"] = reductions_detail
        if nccl_arm is not None:
            line["combine_nccl"] = nccl_arm
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(n_total)
        if world == 1 and not args.profile and not args.no_configs:
            # Every other benchmark configuration, kernel-only on this GPU, each checked against the oracle.
            q = None
            dev.Dispose()
            cfgs = {}
            for name in CONFIG_ORDER:
                m = measure_config(acc, name, args.config_steps, 3)
                cfgs[name] = {k: m[k] for k in ("what", "n_elements", "ms", "elements_per_s", "bytes_per_element", "selectivity",
                                                 "achieved_gbs", "frac", "parity", "precompiled_kernel", "l2")}
            line["configs"] = cfgs
            line["relational"] = measure_relational(acc)
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
