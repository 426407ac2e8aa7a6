#!/usr/bin/env python
"""Benchmark of the fusedMM_csr hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--scale S] [--impl reference]

One "step" is one fusedMM_csr call over the whole synthetic graph of the workload (default: the
Fruchterman-Reingold message on R-MAT scale 20, K = 256, float32).  Prints ONE JSON line (rank 0).
  value      GFLOP/s of the whole job with inputs resident in HBM (5K flops per edge for FR/t-dist, 4K
             sigmoid, 2K SpMM, K GCN: the reference's own accounting, test/fusedMMtime.cpp:816-828)
  e2e        the same metric through the synchronous C-ABI call with HOST (pinned) buffers: CSR, X(=Y)
             copied in and Z copied out inside the timed region, every step
  roofline   gathered-byte HBM roofline of the main kernel (fused_vec_kernel), from CUDA events
  cpu_baseline  the reference's own CPU code (oracle/_ref) on the host cores, on a row sample
With N > 1 (under torchrun) the rows are cut into N nnz-balanced shards, one per rank, Y is replicated
and the Z shards are exchanged over NCCL inside the timed region ("scaling": "strong").
`--impl reference` times only the reference's CPU implementation, same metric and unit.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402

DEFAULT_WORKLOAD = "c2_fr_rmat20_k256"
METRIC = "fusedMM_csr GFLOP/s"
L2_BYTES = 126 * 1000 * 1000


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
               0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting"}

    def __init__(self, uuid):
        self.samples, self.reasons, self.max_mhz, self._stop, self._thr, self.h = [], set(), None, False, None, None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            u = uuid if str(uuid).startswith("GPU-") else "GPU-" + str(uuid)
            self.h = pynvml.nvmlDeviceGetHandleByUUID(u.encode() if hasattr(u, "encode") else u)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.h = None

    def _once(self):
        try:
            self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
            mask = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
            for bit, name in self.REASONS.items():
                if mask & bit:
                    self.reasons.add(name)
        except Exception:
            pass

    def _run(self):
        while not self._stop:
            self._once()
            time.sleep(0.02)

    def __enter__(self):
        if self.h is not None:
            self._thr = threading.Thread(target=self._run, daemon=True)
            self._thr.start()
        return self

    def __exit__(self, *a):
        self._stop = True
        if self._thr:
            self._thr.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# --------------------------------------------------------------------------------------------------
# CPU side: the reference's own code (oracle/_ref) or, where that is not built, the oracle port
# --------------------------------------------------------------------------------------------------
def cpu_engine():
    from oracle import cpu
    if cpu.reference_available():
        ref = cpu.Reference()
        return "reference", ref.threads(), (lambda *a, **kw: ref.csr(*a, **kw))
    orc = cpu.Oracle()
    return "port", os.cpu_count(), (lambda *a, **kw: orc.csr(*a, zero_first=False, **kw))


def cpu_sample(csr_host, x_host, stride):
    """Every `stride`-th row of the graph (the four-array CSR takes any row subset as it is), with its X
    rows packed; Y stays whole.  int64 indices: the reference has one INDEXTYPE and 32-bit overflows at
    the larger configurations."""
    rp = csr_host["rowptr"]
    pb = np.ascontiguousarray(rp[:-1][::stride]).astype(np.int64)
    pe = np.ascontiguousarray(rp[1:][::stride]).astype(np.int64)
    xs = np.ascontiguousarray(x_host[::stride])
    return pb, pe, xs, int((pe - pb).sum())


def time_cpu(call, cfg, csr_host, x_host, stride, steps, warmup):
    pb, pe, xs, edges = cpu_sample(csr_host, x_host, stride)
    m, k, n = len(pb), cfg["k"], x_host.shape[0]
    z = np.zeros((m, k), x_host.dtype)
    times = []
    for it in range(warmup + steps):
        z[:] = 0
        t0 = time.perf_counter()
        st = call(cfg["msg"], m, n, k, csr_host["val"], csr_host["indx64"], pb, pe, xs, k, x_host, k, 0.0, z, k,
                  sop_kind=cfg["sop"] if cfg["sop"] is not None else 0)
        dt = time.perf_counter() - t0
        assert st == 0
        if it >= warmup:
            times.append(dt)
    return edges, times


def pick_stride(call, cfg, csr_host, x_host, nnz, target_s):
    """Row stride such that one CPU call takes about target_s seconds (calibrated on a small sample)."""
    probe = max(1, nnz // 300_000)
    edges, times = time_cpu(call, cfg, csr_host, x_host, probe, 1, 1)
    rate = edges / max(times[0], 1e-6)
    want_edges = min(nnz, max(200_000, int(rate * target_s)))
    return max(1, nnz // want_edges), rate


def host_copies(csr, x):
    return ({"rowptr": csr.rowptr.cpu().numpy().astype(np.int64), "indx64": csr.indx.cpu().numpy().astype(np.int64),
             "val": csr.val.cpu().numpy()}, x.cpu().numpy())


def measure_e2e(args, api, torch, dist, world, dev, csr, x, tdtype, msg, sop, n, k, nnz, r0, r1, flops_per_edge, barrier):
    """The same call through the synchronous typed entry point with pinned HOST arrays: all copies inside."""
    e2e_steps = args.e2e_steps or max(3, min(args.steps, 8))
    hv = csr.val.cpu().pin_memory()
    hi = csr.indx.cpu().pin_memory()
    hp = csr.rowptr.cpu().pin_memory()
    hx = x.cpu().pin_memory()
    hz = torch.zeros((r1 - r0, k), dtype=tdtype).pin_memory()
    hpb, hpe = hp[:-1], hp[1:]

    def e2e_step():
        st = api.fusedMM_csr(msg, r1 - r0, n, k, 1.0, nnz, n, n, hv, hi, hpb[r0:], hpe[r0:], hx[r0:], k, hx, k, 0.0,
                             hz, k, sop=sop if sop is not None else 0)
        assert st == 0, api.status_string(st)
        return api.call_info()

    # hpb/hpe are views of one pinned tensor, so pntre == pntrb + 1 element and one copy serves both
    for _ in range(2):
        einfo = e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        einfo = e2e_step()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    t = torch.tensor([e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item())
    e2e = {"value": flops_per_edge * nnz / (e2e_ms * 1e-3) * 1e-9, "unit": "GFLOP/s",
           "h2d_bytes_per_step": int(einfo.h2d_bytes), "d2h_bytes_per_step": int(einfo.d2h_bytes),
           "ms_per_step": e2e_ms, "timer": "host clock around the synchronous call (copies + kernels), max over ranks",
           "note": "per rank: its CSR rows' pointers, all column ids, X rows and all of Y in; its Z rows out"}
    e2e_ok = bool(torch.isfinite(hz).all())

    # the same with the graph kept on the device by a plan (inspector/executor split): per step only X(=Y) goes
    # in and Z comes out; reported beside the headline figure, which stays the plain fusedMM_csr call
    plan = api.Plan(hi, hpb[r0:r1], hpe[r0:r1], hv)  # this rank's rows
    hz2 = torch.zeros((r1 - r0, k), dtype=tdtype).pin_memory()

    def plan_step():
        st = plan.csr(msg, n, k, hx[r0:], k, hx, k, 0.0, hz2, k, sop=sop if sop is not None else 0)
        assert st == 0, api.status_string(st)
        return api.call_info()

    pinfo = plan_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        pinfo = plan_step()
    barrier()
    plan_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    plan.close()
    e2e["with_plan"] = {"value": flops_per_edge * nnz / (plan_ms * 1e-3) * 1e-9, "ms_per_step": plan_ms,
                        "h2d_bytes_per_step": int(pinfo.h2d_bytes), "d2h_bytes_per_step": int(pinfo.d2h_bytes),
                        "same_z": bool(torch.equal(hz, hz2))}
    return e2e, e2e_ok


# --------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD)
    ap.add_argument("--scale", type=int, default=None, help="smaller instance of the same graph family")
    ap.add_argument("--dtype", default="f32", choices=["f32", "f64"])
    ap.add_argument("--e2e-steps", type=int, default=None)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-array (end-to-end) leg; e2e is then null")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    import torch
    from fusedmm_b200 import api, messages as M, synth

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    tdtype = torch.float32 if args.dtype == "f32" else torch.float64
    es = 4 if args.dtype == "f32" else 8

    cfgname = args.workload
    base_cfg = synth.CONFIGS[cfgname]
    flops_per_edge = M.FLOPS_PER_EDGE_PER_K[base_cfg["msg"]] * base_cfg["k"]
    config = {"workload": cfgname + (f"@scale{args.scale}" if args.scale else ""),
              "message": hex(base_cfg["msg"]), "k": base_cfg["k"], "index_types": "rowptr int64, colidx int32",
              "l2": "inputs (Y alone is larger than the 126 MB L2) exceed L2; no flush between steps"}

    # ---------------------------------------------------------------- reference arm (CPU only)
    if args.impl == "reference":
        if rank != 0:
            return
        kind, cores, call = cpu_engine()
        dev = "cuda" if torch.cuda.is_available() else "cpu"
        cfg, csr, x = synth.make_config(cfgname, device=dev, dtype=tdtype, scale=args.scale)
        csr_host, x_host = host_copies(csr, x)
        nnz = csr.nnz
        del csr, x
        stride, _ = pick_stride(call, cfg, csr_host, x_host, nnz, target_s=1.5)
        edges, times = time_cpu(call, cfg, csr_host, x_host, stride, args.steps, args.warmup)
        ms = 1e3 * float(np.mean(times))
        value = flops_per_edge * edges / (ms * 1e-3) * 1e-9
        sample = f"every {stride}-th row of the graph ({edges} of {nnz} edges), whole Y"
        config.update({"n": cfg["n"], "nnz": nnz})
        print(json.dumps({
            "impl": "reference", "metric": METRIC, "value": value, "unit": "GFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
            "config": config, "edges_per_s": edges / (ms * 1e-3),
            "cpu_baseline": {"value": value, "unit": "GFLOP/s", "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    # ---------------------------------------------------------------- B200 arm
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    saved_stdout = None
    if world > 1:
        import torch.distributed as dist
        # NCCL writes its version banner straight to file descriptor 1 when the first communicator comes up;
        # stdout carries the JSON line, so descriptor 1 points at stderr until that line is printed
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        dist.init_process_group("nccl", device_id=dev)
    api.lib()

    cfg, csr, x = synth.make_config(cfgname, device=dev, dtype=tdtype, scale=args.scale)
    n, k, nnz, msg, sop = cfg["n"], cfg["k"], csr.nnz, cfg["msg"], cfg["sop"]
    pb_all, pe_all = csr.pntrb.contiguous(), csr.pntre.contiguous()
    rowptr_host = csr.rowptr.cpu().numpy()
    bounds = api.shard_rows(rowptr_host[:-1].copy(), rowptr_host[1:].copy(), world,
                            row_weight=int(os.environ.get("FUSEDMM_BENCH_ROW_WEIGHT", "8")))
    if world > 1:
        config["row_shard_cost"] = "edges + %s per row" % os.environ.get("FUSEDMM_BENCH_ROW_WEIGHT", "8")
    r0, r1 = int(bounds[rank]), int(bounds[rank + 1])
    my_edges = int(rowptr_host[r1] - rowptr_host[r0])
    z = torch.zeros((n, k), dtype=tdtype, device=dev)
    config.update({"n": n, "nnz": nnz, "sop": sop, "row_shards": [int(b) for b in bounds] if world > 1 else None})

    from fusedmm_b200 import dist as fdist
    # everything that is timed runs on one non-default stream: the library enqueues on it (a NULL stream
    # would mean a synchronous call), NCCL follows it, and the CUDA events are recorded on it
    stream = torch.cuda.Stream()
    torch.cuda.synchronize()
    torch.cuda.set_stream(stream)
    # N > 1: the Z exchange is fused into the kernels (stores into the peers' Z over NVLink) when torch's
    # symmetric memory is available on this box, otherwise one NCCL broadcast per row shard follows the kernels
    pz, exchange = None, None
    if world > 1:
        exchange = "nccl broadcast per row shard after the kernels"
        if os.environ.get("FUSEDMM_BENCH_EXCHANGE", "fused") == "fused":
            try:
                pz = fdist.PeerZ(n, k, tdtype, dev, dist)
                z = pz.z
                z.zero_()
                if os.environ.get("FUSEDMM_BENCH_MULTICAST", "1" if pz.use_multicast() else "0") == "1" and pz.multicast:
                    exchange = ("fused: kernels store each finished row once through the NVSwitch multicast mapping of Z "
                                "(multimem.st), one small all-reduce orders the ranks")
                else:
                    exchange = ("fused: kernels store finished rows into every rank's Z (peer memory, one store per peer), "
                                "one small all-reduce orders the ranks")
            except Exception as exc:  # no symmetric memory on this box: keep the NCCL path
                pz = None
                exchange += f" (symmetric memory unavailable: {type(exc).__name__})"
        config["exchange"] = exchange
    peers = mcast = None
    if pz is not None:
        if "multimem" in exchange:
            mcast = pz.multicast_at_row(r0)
        else:
            peers = pz.peers_at_row(r0)

    def step():
        st = api.fusedMM_csr(msg, r1 - r0, n, k, 1.0, nnz, n, n, csr.val, csr.indx, pb_all[r0:], pe_all[r0:],
                             x[r0:], k, x, k, 0.0, z[r0:], k, sop=sop if sop is not None else 0,
                             stream=stream.cuda_stream, z_peers=peers, z_multicast=mcast)
        assert st == 0, api.status_string(st)
        if pz is not None:
            pz.finish_step()
        elif world > 1:
            fdist.exchange_row_shards(z, bounds, dist)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for attempt in range(3):  # a first call may find the split-row scratch too small; it is then enlarged
        for _ in range(args.warmup):
            step()
        barrier()
        status = api.lib().fusedmm_b200_stream_status()
        if status == 0:
            break
    assert status == 0, api.status_string(status)
    uuid = torch.cuda.get_device_properties(dev).uuid
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # a workload whose Y fits in L2 would be timed warm: write a buffer larger than L2 before every timed
    # step and time each step with its own pair of events (the flush stays outside the pairs)
    flush = None
    if n * k * es < 2 * L2_BYTES:
        flush = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=dev)
        config["l2"] = "inputs fit in the 126 MB L2: a 252 MB buffer is written before every timed step (outside the timed spans)"
    with ClockSampler(uuid) as clocks:
        barrier()
        if flush is None:
            e0.record()
            for _ in range(args.steps):
                step()
            e1.record()
            barrier()
            ms_total = e0.elapsed_time(e1)
        else:
            pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                     for _ in range(args.steps)]
            for a, b in pairs:
                flush.fill_(1)
                a.record()
                step()
                b.record()
            barrier()
            ms_total = sum(a.elapsed_time(b) for a, b in pairs)
        # keep the sampler alive over a few more steps when the timed region was very short
        t_end = time.time() + max(0.0, 0.25 - ms_total * 1e-3)
        while time.time() < t_end:
            step()
            torch.cuda.synchronize()
    t = torch.tensor([ms_total], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    value = flops_per_edge * nnz / (ms_step * 1e-3) * 1e-9
    finite = bool(torch.isfinite(z).all())
    if world > 1:  # every rank must hold the same, complete Z: compare a checksum of checksums
        chk = z.double().sum(dim=1).sum().reshape(1)
        lo, hi = chk.clone(), chk.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        finite = finite and bool(lo.item() == hi.item())
        # and it must be what one GPU computes alone (rank 0 recomputes all rows; outside the timed region)
        if rank == 0:
            zfull = torch.empty((n, k), dtype=tdtype, device=dev)
            st = api.fusedMM_csr(msg, n, n, k, 1.0, nnz, n, n, csr.val, csr.indx, pb_all, pe_all, x, k, x, k, 0.0,
                                 zfull, k, sop=sop if sop is not None else 0)
            assert st == 0
            config["exchanged_z_equals_single_gpu_z"] = bool(torch.equal(zfull, z))
            del zfull

    # per-launch CUDA-event times of one synchronous call on this rank's shard
    kms = {"scan": [], "rows": [], "chunks": [], "fixup": [], "main": []}
    launches_per_step = 0
    for _ in range(5):
        if flush is not None:
            flush.fill_(2)
            torch.cuda.synchronize()
        st = api.fusedMM_csr(msg, r1 - r0, n, k, 1.0, nnz, n, n, csr.val, csr.indx, pb_all[r0:], pe_all[r0:], x[r0:],
                             k, x, k, 0.0, z[r0:], k, sop=sop if sop is not None else 0)
        assert st == 0
        info = api.call_info()
        launches_per_step = info.kernel_launches
        for nm in kms:
            kms[nm].append(getattr(info, "ms_" + nm))
    kmed = {nm: float(np.median(v)) for nm, v in kms.items()}
    peak, peak_kind = load_peaks()
    alg_bytes = synth.algorithmic_bytes(msg, my_edges, r1 - r0, k, es, 4, 8)
    # the whole-row launch and the chunk launch of the main kernel run side by side on two streams, so the
    # kernel time is the span that covers both (and the small fix-up launch that follows the chunks)
    main_ms = kmed["main"]
    achieved = alg_bytes / (main_ms * 1e-3) * 1e-9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": None, "peak_kind": peak_kind, "kernel": "fused_vec_kernel: whole-row launch beside split-row chunk launch (+ fix-up), one span",
                "algorithmic_bytes_per_step": alg_bytes, "kernel_ms": kmed,
                "tiling": f"{info.lanes_per_edge} lanes/edge x {info.vectors_per_lane} vec/lane",
                "split_rows": int(info.hub_rows), "row_chunks": int(info.hub_chunks)}
    tr = ROOT / "profiles" / "traffic.json"
    if tr.exists():
        try:
            rec = json.loads(tr.read_text()).get(cfgname)
            if rec:
                roofline["traffic"] = rec["dram_bytes_per_edge"] * my_edges
                roofline["traffic_note"] = rec.get("note")
        except Exception:
            pass

    # ---------------------------------------------------------------- end to end, host buffers
    e2e, e2e_ok = None, True
    if not args.no_e2e:
        e2e, e2e_ok = measure_e2e(args, api, torch, dist, world, dev, csr, x, tdtype, msg, sop, n, k, nnz, r0, r1,
                                  flops_per_edge, barrier)

    # ---------------------------------------------------------------- CPU baseline (rank 0, N = 1)
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu:
        kind, cores, call = cpu_engine()
        csr_host, x_host = host_copies(csr, x)
        stride, _ = pick_stride(call, cfg, csr_host, x_host, nnz, target_s=4.0)
        edges, times = time_cpu(call, cfg, csr_host, x_host, stride, 3, 1)
        tmed = float(np.median(times))
        # parity spot check of the sample against the GPU result
        pbs, pes, xs, _ = cpu_sample(csr_host, x_host, stride)
        zc = np.zeros((len(pbs), k), x_host.dtype)
        call(msg, len(pbs), n, k, csr_host["val"], csr_host["indx64"], pbs, pes, xs, k, x_host, k, 0.0, zc, k,
             sop_kind=sop if sop is not None else 0)
        zg = z[::stride].cpu().numpy()
        scale = np.maximum(np.abs(zc), np.abs(zc).max(axis=1, keepdims=True)).clip(1e-30)
        err = float((np.abs(zg - zc) / scale).max())
        cpu_baseline = {"value": flops_per_edge * edges / tmed * 1e-9, "unit": "GFLOP/s", "cores": cores, "kind": kind,
                        "sample": f"every {stride}-th row ({edges} of {nnz} edges), whole Y; median of 3 calls",
                        "edges_per_s": edges / tmed, "seconds_per_call": tmed,
                        "gpu_vs_cpu_max_rel_err_on_sample": err,
                        "code": "reference general kernel (fusedMM.c) built by oracle/build_ref.sh" if kind == "reference"
                                else "oracle/fusedmm_oracle.c"}

    if rank == 0:
        out = {"metric": METRIC, "value": value, "unit": "GFLOP/s", "n_gpus": world, "steps": args.steps,
               "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
               "vs_baseline": None, "dtype": args.dtype, "data": "synthetic", "config": config,
               "edges_per_s": nnz / (ms_step * 1e-3),
               "effective_gbs": synth.algorithmic_bytes(msg, nnz, n, k, es, 4, 8) / (ms_step * 1e-3) * 1e-9,
               "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "clocks": clocks.summary(),
               "gpu_launches": launches_per_step * args.steps, "finite": finite and e2e_ok}
        sys.stdout.flush()
        if saved_stdout is not None:
            os.dup2(saved_stdout, 1)
        print(json.dumps(out))
        sys.stdout.flush()
    if world > 1:
        # leave without tearing down NCCL and the symmetric-memory mappings rank by rank: every rank has
        # passed the barrier, nothing is in flight, and a plain exit avoids teardown-order hangs
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
