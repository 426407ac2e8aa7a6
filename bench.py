#!/usr/bin/env python
"""Benchmark of the fusedMM_csr hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--dtype f32|f64] [--scale S]
                    [--impl reference] [--no-configs] [--no-e2e] [--no-cpu]

One "step" is one fusedMM_csr call over the whole synthetic graph of the workload.  The default workload is the
largest benchmark configuration that fits one GPU: the sigmoid (Force2Vec) message on R-MAT scale 24, K = 128,
float32, int64 row pointers with int32 column ids.  Prints ONE JSON line (rank 0).
  value      GFLOP/s of the whole job with inputs resident in HBM (4K flops per edge for sigmoid, 5K FR/t-dist,
             2K SpMM, K GCN: the reference's own accounting, test/fusedMMtime.cpp:816-828)
  e2e        the same metric through the synchronous C-ABI call with HOST (pinned) buffers: CSR, X(=Y)
             copied in and Z copied out inside the timed region, every step
  roofline   gathered-byte HBM roofline of the main kernel (fused_vec_kernel), from CUDA events, with the DRAM
             traffic of the same kernels from an ncu capture beside it (profiles/traffic.json)
  cpu_baseline  the reference's optimised OpenMP kernels (oracle/_ref, built by oracle/build_ref_opt.sh) on the
             host cores, on a row sample of the same graph, and the reference's general kernel as a second figure
  configs    (N = 1, default workload only) one compact record per other benchmark configuration, measured in the
             same run: ms, GFLOP/s, edges/s, roofline fraction, clocks, CPU figure, error against the reference
  generic    (same condition) messages outside the four optimised patterns on the FR configuration's graph
With N > 1 (under torchrun) the rows are cut into N cost-balanced shards, one per rank, Y is replicated and the Z
shards are exchanged over NVLink inside the timed region ("scaling": "strong").
`--impl reference` times only the reference's CPU implementation, same metric, unit and config.
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

DEFAULT_WORKLOAD = "c5_sigmoid_rmat24_k128"
# the other benchmark configurations, reported as compact records beside the default one
SIDE_CONFIGS = [("c1_sigmoid_rmat14_k128", "f32"), ("c2_fr_rmat20_k256", "f32"), ("c3_tdist_er4m_k64", "f32"),
                ("c4_spmm_rmat22_k512", "f32"), ("c5_sigmoid_rmat24_k128", "f64")]
METRIC = "fusedMM_csr GFLOP/s"
L2_BYTES = 126 * 1000 * 1000
PEER_GBS = 770.0  # measured peer-copy bandwidth per direction on this pool's NVSwitch boxes


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


def workload_config(cfgname, dtype, scale, n, nnz, sop, k, msg, es):
    """The `config` object, built the same way by both arms so that they can be compared key by key."""
    l2 = ("inputs fit in the 126 MB L2: a 252 MB buffer is written before every timed step (outside the timed spans)"
          if n * k * es < 2 * L2_BYTES else
          "inputs (Y alone is larger than the 126 MB L2) exceed L2; no flush between steps")
    return {"workload": cfgname + (f"@scale{scale}" if scale else ""), "message": hex(msg), "k": k, "value_type": dtype,
            "index_types": "rowptr int64, colidx int32", "n": n, "nnz": nnz, "sop": sop, "l2": l2}


# --------------------------------------------------------------------------------------------------
# CPU side: the reference's own code (oracle/_ref), or the oracle port where that is not built
# --------------------------------------------------------------------------------------------------
class CpuEngine:
    """The fastest build of the reference present: its optimised OpenMP kernels (`reference`, variant
    "optimised"), else its general kernel alone (`reference`, variant "general"), else the oracle port."""

    def __init__(self):
        from oracle import cpu
        self.general = None
        if cpu.reference_opt_available():
            ref = cpu.ReferenceOpt()
            self.kind, self.variant, self.cores = "reference", "optimised", ref.threads()
            self.code = ("reference optimised path: generated OpenMP SIMD kernels behind {s,d}gfusedMM_csr + fusedMM.c "
                         f"-DENABLE_OPT_FUSEDMM, built by oracle/build_ref_opt.sh ({ref.simd}, int64 indices)")
            self.simd = ref.simd
            self.call = lambda *a, **kw: ref.csr(*a, **kw)
            if ref.general_libs:
                self.general = lambda *a, **kw: ref.csr(*a, general=True, **kw)
        elif cpu.reference_available():
            ref = cpu.Reference()
            self.kind, self.variant, self.cores, self.simd = "reference", "general", ref.threads(), "avx2"
            self.code = "reference general kernel (fusedMM.c) built by oracle/build_ref.sh"
            self.call = lambda *a, **kw: ref.csr(*a, **kw)
        else:
            orc = cpu.Oracle()
            self.kind, self.variant, self.cores, self.simd = "port", "oracle", os.cpu_count(), "avx2"
            self.code = "oracle/fusedmm_oracle.c"
            self.call = lambda *a, **kw: orc.csr(*a, zero_first=False, **kw)


def sample_rows(torch, csr, x, stride):
    """Every `stride`-th row of the graph as a compact CSR (built on the device the graph is on, copied to the
    host): int64 indices, the rows' X packed.  Y stays whole and is not copied here."""
    n = csr.n
    rows = torch.arange(0, n, stride, device=csr.rowptr.device)
    pb, pe = csr.rowptr[rows].to(torch.int64), csr.rowptr[rows + 1].to(torch.int64)
    lens = pe - pb
    newptr = torch.zeros(rows.numel() + 1, dtype=torch.int64, device=pb.device)
    torch.cumsum(lens, 0, out=newptr[1:])
    total = int(newptr[-1].item())
    src = torch.repeat_interleave(pb - newptr[:-1], lens) + torch.arange(total, device=pb.device)
    indx = csr.indx[src].to(torch.int64)
    val = csr.val[src]
    xs = x[::stride].contiguous()
    return {"rowptr": newptr.cpu().numpy(), "indx": indx.cpu().numpy(), "val": val.cpu().numpy(),
            "x": xs.cpu().numpy(), "edges": total, "rows": int(rows.numel()), "stride": stride}


def run_cpu(call, cfg, smp, y_host, z=None, beta=0.0):
    k, n, m = cfg["k"], y_host.shape[0], smp["rows"]
    if z is None:
        z = np.zeros((m, k), y_host.dtype)
    rp = smp["rowptr"]
    t0 = time.perf_counter()
    st = call(cfg["msg"], m, n, k, smp["val"], smp["indx"], rp[:-1], rp[1:], smp["x"], k, y_host, k, beta, z, k,
              sop_kind=cfg["sop"] if cfg["sop"] is not None else 0)
    dt = time.perf_counter() - t0
    assert st == 0
    return dt, z


def time_cpu(call, cfg, smp, y_host, steps, warmup):
    times, z = [], None
    for it in range(warmup + steps):
        if z is not None:
            z[:] = 0  # the general kernel accumulates; the optimised ones overwrite (beta = 0)
        dt, z = run_cpu(call, cfg, smp, y_host, z)
        if it >= warmup:
            times.append(dt)
    return times, z


def pick_stride(torch, call, cfg, csr, x, y_host, nnz, target_s):
    """Row stride such that one CPU call takes about target_s seconds (calibrated on a small sample)."""
    def odd(s):  # an even stride favours the vertices of an R-MAT graph whose ids end in zero bits: the heavy ones
        return s + 1 if s > 2 and s % 2 == 0 else s

    probe = odd(max(1, nnz // 400_000))
    smp = sample_rows(torch, csr, x, probe)
    times, _ = time_cpu(call, cfg, smp, y_host, 1, 1)
    rate = smp["edges"] / max(times[0], 1e-6)
    want_edges = min(nnz, max(200_000, int(rate * target_s)))
    return odd(max(1, nnz // want_edges))


def rel_err(z, zref):
    scale = np.maximum(np.abs(zref), np.abs(zref).max(axis=1, keepdims=True)).clip(1e-30)
    return float((np.abs(z.astype(np.float64) - zref) / scale).max()) if z.size else 0.0


def cpu_leg(torch, eng, cfg, csr, x, z_gpu, nnz, flops_per_edge, target_s, steps):
    """Times the CPU code on a row sample and compares the GPU's Z on those rows with the CPU's."""
    y_host = x.cpu().numpy()
    stride = pick_stride(torch, eng.call, cfg, csr, x, y_host, nnz, target_s)
    smp = sample_rows(torch, csr, x, stride)
    times, zc = time_cpu(eng.call, cfg, smp, y_host, steps, 1)
    tmed = float(np.median(times))
    out = {"value": flops_per_edge * smp["edges"] / tmed * 1e-9, "unit": "GFLOP/s", "cores": eng.cores, "kind": eng.kind,
           "variant": eng.variant, "simd": eng.simd, "omp_threads": eng.cores,
           "sample": f"every {stride}-th row ({smp['edges']} of {nnz} edges), whole Y; median of {steps} calls after 1 warm-up",
           "edges_per_s": smp["edges"] / tmed, "seconds_per_call": tmed, "code": eng.code}
    if z_gpu is not None:
        out["gpu_vs_cpu_max_rel_err_on_sample"] = rel_err(z_gpu[::stride].cpu().numpy(), zc.astype(np.float64))
    if eng.general is not None:  # the general (function-pointer) kernel of the reference, on a smaller sample
        gs = sample_rows(torch, csr, x, max(stride * 4, nnz // 2_000_000 or 1))
        gt, zg = time_cpu(eng.general, cfg, gs, y_host, 1, 1)
        out["general_kernel"] = {"value": flops_per_edge * gs["edges"] / gt[0] * 1e-9, "unit": "GFLOP/s",
                                 "sample": f"every {gs['stride']}-th row ({gs['edges']} edges), 1 call after 1 warm-up"}
        if z_gpu is not None:
            out["general_kernel"]["gpu_vs_cpu_max_rel_err_on_sample"] = rel_err(
                z_gpu[::gs["stride"]].cpu().numpy(), zg.astype(np.float64))
    return out


def measure_e2e(args, api, torch, dist, world, dev, csr, x, tdtype, msg, sop, n, k, nnz, r0, r1, flops_per_edge, barrier,
                bounds=None, pz=None):
    """The same call through the synchronous typed entry point with pinned HOST arrays: all copies inside."""
    e2e_steps = args.e2e_steps or (3 if nnz > 200_000_000 else max(3, min(args.steps, 8)))

    def pinned(t):  # straight from the device into pinned memory: no pageable copy in between
        h = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
        h.copy_(t)
        return h

    # every rank of the node holds its own host copy of the inputs: make sure the node has room for all of them
    need = sum(t.numel() * t.element_size() for t in (csr.val, csr.indx, csr.rowptr, x)) + 2 * (r1 - r0) * k * x.element_size()
    try:
        import psutil
        avail = psutil.virtual_memory().available
    except Exception:
        avail = None
    fits = torch.tensor([1.0 if avail is None or need * world < 0.6 * avail else 0.0], device=dev)
    if world > 1:
        dist.all_reduce(fits, op=dist.ReduceOp.MIN)
    if fits.item() == 0.0:
        return {"value": None, "unit": "GFLOP/s", "h2d_bytes_per_step": None, "d2h_bytes_per_step": None,
                "skipped": f"{world} ranks x {need / 2**30:.1f} GiB of pinned host copies do not fit this node's free memory"}, True
    hv, hi, hp, hx = pinned(csr.val), pinned(csr.indx), pinned(csr.rowptr), pinned(x)
    hpb, hpe = hp[:-1], hp[1:]

    # N > 1: the ranks' PCIe links work side by side (fusedmm_b200.dist.HostStep): a rank brings 1/N of Y and its own
    # shard of the graph, one all-gather over NVLink completes Y, its rows of Z go back
    hs = None
    if world > 1 and bounds is not None:
        from fusedmm_b200 import dist as fdist
        uses_val = ((msg >> 4) & 0xF) == 0 and ((msg >> 12) & 0xF) != 0
        hs = fdist.HostStep(n, k, tdtype, dev, dist, bounds, nnz_max=int(hp[r1] - hp[r0]), with_val=uses_val,
                            idx_dtype=csr.indx.dtype, pz=pz)
    za, zb = hs.out_rows() if hs is not None else (r0, r1)
    hz = torch.zeros((zb - za, k), dtype=tdtype, pin_memory=True)
    z_ref = None
    if hs is not None and pz is not None:  # the timed steps left the whole result in every rank's Z: keep this rank's
        z_ref = pz.z[za:zb].clone()        # output rows for the comparison and make the rest of Z garbage
        barrier()
        pz.z.fill_(-12345.0)
        barrier()

    class _Bytes:
        h2d_bytes = d2h_bytes = 0

    def e2e_step():
        if hs is not None:
            st = hs.step(msg, hp, hi, hv if hs._with_val else None, hx, hx, hz, sop=sop if sop is not None else 0,
                         stream=torch.cuda.current_stream().cuda_stream, z_rows_only=True)
            assert st == 0 and api.lib().fusedmm_b200_stream_status() == 0, api.status_string(st)
            b = _Bytes()
            b.h2d_bytes, b.d2h_bytes = hs.h2d_bytes, hs.d2h_bytes
            return b
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
    nbytes = torch.tensor([float(einfo.h2d_bytes), float(einfo.d2h_bytes)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(nbytes, op=dist.ReduceOp.SUM)  # bytes of the whole job, like the metric
    e2e = {"value": flops_per_edge * nnz / (e2e_ms * 1e-3) * 1e-9, "unit": "GFLOP/s",
           "h2d_bytes_per_step": int(nbytes[0].item()), "d2h_bytes_per_step": int(nbytes[1].item()),
           "ms_per_step": e2e_ms, "steps": e2e_steps,
           "timer": "host clock around the synchronous call (copies + kernels), max over ranks",
           "note": "per rank: its CSR rows' pointers, all column ids, X rows and all of Y in; its Z rows out"}
    if hs is not None:
        e2e["note"] = ("fusedmm_b200.dist.HostStep, bytes summed over the ranks: every rank brings 1/N of the rows of Y and the row "
                       "pointers and column ids of its own row shard over its own PCIe link, one in-place all-gather over "
                       "NVLink completes Y on every GPU, the rank's kernels run on device arrays"
                       + (" and store every finished row into the Z of the rank that copies it out, and every rank copies 1/N "
                          "of the rows of Z back to the host" if pz is not None else ", its rows of Z go back to the host"))
    elif world > 1:
        e2e["note"] += ("; with N ranks every rank stages all of Y over its own PCIe link in the same interval, so this "
                        "figure does not scale with N: it is a one-GPU figure")
    e2e_ok = bool(torch.isfinite(hz).all())
    if z_ref is not None:
        same = torch.tensor([1.0 if torch.equal(hz.to(dev), z_ref) else 0.0], device=dev)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        e2e["host_z_equals_device_resident_z_on_every_rank"] = bool(same.item() == 1.0)
        e2e_ok = e2e_ok and e2e["host_z_equals_device_resident_z_on_every_rank"]
        return e2e, e2e_ok

    # the same with the graph kept on the device by a plan (inspector/executor split): per step only X(=Y) goes
    # in and Z comes out; reported beside the headline figure, which stays the plain fusedMM_csr call
    plan = api.Plan(hi, hpb[r0:r1], hpe[r0:r1], hv)  # this rank's rows
    hz2 = torch.zeros((r1 - r0, k), dtype=tdtype, pin_memory=True)

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


def exchange_self_check(api, torch, dist, fdist, dev, rank, world, tdtype, exchange_mode):
    """Multi-GPU parity of the fused exchange on a small graph, in the value type given: one step with beta = 0 and
    one with beta = 1 (Z accumulates everywhere); every rank's Z must equal, bit for bit, what one GPU computes
    alone.  Returns True/False on rank 0 (None elsewhere)."""
    from fusedmm_b200 import messages as M, synth
    cfg, csr, x = synth.make_config("c2_fr_rmat20_k256", device=dev, dtype=tdtype, scale=15)
    n, k, nnz = cfg["n"], cfg["k"], csr.nnz
    rp_host = csr.rowptr.cpu().numpy()
    bounds = api.shard_rows(rp_host[:-1].copy(), rp_host[1:].copy(), world, row_weight=fdist.ROW_WEIGHT)
    r0, r1 = int(bounds[rank]), int(bounds[rank + 1])
    pz = fdist.PeerZ(n, k, tdtype, dev, dist)
    pz.z.fill_(0.25)
    single = torch.full((n, k), 0.25, dtype=tdtype, device=dev)
    use_mc = exchange_mode == "multicast" and pz.multicast
    stream = torch.cuda.Stream()
    ok = True
    for beta in (0.0, 1.0):
        torch.cuda.synchronize()
        dist.barrier()
        with torch.cuda.stream(stream):
            if beta == 0.0:
                assert pz.zero_foreign_empty_rows(csr.rowptr, r0, r1, stream=stream.cuda_stream) == 0
            st = api.fusedMM_csr(cfg["msg"], r1 - r0, n, k, 1.0, nnz, n, n, csr.val, csr.indx, csr.rowptr[r0:-1],
                                 csr.rowptr[r0 + 1:], x[r0:], k, x, k, beta, pz.z[r0:], k, sop=cfg["sop"],
                                 stream=stream.cuda_stream, z_peers=None if use_mc else pz.peers_at_row(r0),
                                 z_multicast=pz.multicast_at_row(r0) if use_mc else None)
            assert st == 0, api.status_string(st)
            pz.finish_step()
        torch.cuda.synchronize()
        dist.barrier()
        st = api.fusedMM_csr(cfg["msg"], n, n, k, 1.0, nnz, n, n, csr.val, csr.indx, csr.rowptr[:-1], csr.rowptr[1:], x, k, x, k,
                             beta, single, k, sop=cfg["sop"])
        assert st == 0
        same = torch.tensor([1.0 if torch.equal(single, pz.z) else 0.0], device=dev)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        ok = ok and bool(same.item() == 1.0)
    return ok if rank == 0 else None


# --------------------------------------------------------------------------------------------------
def bench_gpu(args, ctx, cfgname, dtype, scale, steps, warmup, with_e2e, cpu_target_s, cpu_steps):
    """One workload on the GPU(s): device-resident timing, per-launch times, roofline, and (N = 1) the e2e and
    CPU legs.  Returns the full record (a dict)."""
    torch, api, synth, M, fdist, dist = ctx["torch"], ctx["api"], ctx["synth"], ctx["M"], ctx["fdist"], ctx["dist"]
    rank, world, dev = ctx["rank"], ctx["world"], ctx["dev"]
    tdtype = torch.float32 if dtype == "f32" else torch.float64
    es = 4 if dtype == "f32" else 8
    base_cfg = synth.CONFIGS[cfgname]
    flops_per_edge = M.FLOPS_PER_EDGE_PER_K[base_cfg["msg"]] * base_cfg["k"]

    cfg, csr, x = synth.make_config(cfgname, device=dev, dtype=tdtype, scale=scale)
    n, k, nnz, msg, sop = cfg["n"], cfg["k"], csr.nnz, cfg["msg"], cfg["sop"]
    config = workload_config(cfgname, dtype, scale, n, nnz, sop, k, msg, es)
    run = {}
    pb_all, pe_all = csr.pntrb.contiguous(), csr.pntre.contiguous()
    rowptr_host = csr.rowptr.cpu().numpy()
    row_weight = int(os.environ.get("FUSEDMM_BENCH_ROW_WEIGHT", str(fdist.ROW_WEIGHT)))
    bounds = api.shard_rows(rowptr_host[:-1].copy(), rowptr_host[1:].copy(), world, row_weight=row_weight)
    r0, r1 = int(bounds[rank]), int(bounds[rank + 1])
    my_edges = int(rowptr_host[r1] - rowptr_host[r0])
    nonempty_rows = int((rowptr_host[1:] > rowptr_host[:-1]).sum())
    z = torch.zeros((n, k), dtype=tdtype, device=dev)
    if world > 1:
        run["row_shards"] = [int(b) for b in bounds]
        run["row_shard_cost"] = f"edges + {row_weight} per row"

    # everything that is timed runs on one non-default stream: the library enqueues on it (a NULL stream
    # would mean a synchronous call), NCCL follows it, and the CUDA events are recorded on it
    stream = torch.cuda.Stream()
    torch.cuda.synchronize()
    torch.cuda.set_stream(stream)
    # N > 1: the Z exchange is fused into the kernels (stores into the peers' Z over NVLink) when torch's
    # symmetric memory is available on this box, otherwise one NCCL broadcast per row shard follows the kernels
    pz, exchange, mode = None, None, "nccl"
    if world > 1:
        exchange = "nccl broadcast per row shard after the kernels"
        if os.environ.get("FUSEDMM_BENCH_EXCHANGE", "fused") == "fused":
            try:
                pz = fdist.PeerZ(n, k, tdtype, dev, dist)
                del z
                z = pz.z
                z.zero_()
                if os.environ.get("FUSEDMM_BENCH_MULTICAST", "1" if pz.use_multicast() else "0") == "1" and pz.multicast:
                    mode = "multicast"
                    exchange = ("fused: kernels store each finished row that has edges once through the NVSwitch multicast "
                                "mapping of Z (multimem.st); rows without edges are zeroed locally by every rank; one small "
                                "all-reduce orders the ranks")
                else:
                    mode = "peer"
                    exchange = ("fused: kernels store finished rows that have edges into every rank's Z (peer memory, one "
                                "store per peer); rows without edges are zeroed locally by every rank; one small all-reduce "
                                "orders the ranks")
            except Exception as exc:  # no symmetric memory on this box: keep the NCCL path
                pz = None
                exchange += f" (symmetric memory unavailable: {type(exc).__name__})"
        run["exchange_kind"] = exchange
    peers = mcast = None
    if pz is not None:
        if mode == "multicast":
            mcast = pz.multicast_at_row(r0)
        else:
            peers = pz.peers_at_row(r0)

    def step():
        if pz is not None:  # beta == 0: rows without edges of the other shards become 0 in this rank's copy
            st = pz.zero_foreign_empty_rows(csr.rowptr, r0, r1, stream=stream.cuda_stream)
            assert st == 0, api.status_string(st)
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

    status = 0
    for attempt in range(3):  # a first call may find the split-row scratch too small; it is then enlarged
        for _ in range(warmup):
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
    with ClockSampler(uuid) as clocks:
        barrier()
        if flush is None:
            e0.record()
            for _ in range(steps):
                step()
            e1.record()
            barrier()
            ms_total = e0.elapsed_time(e1)
        else:
            pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                     for _ in range(steps)]
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
    ms_step = float(t.item()) / steps
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
            run["exchanged_z_equals_single_gpu_z"] = bool(torch.equal(zfull, z))
            del zfull

    # per-launch CUDA-event times of one synchronous call on this rank's shard
    kms = {"scan": [], "rows": [], "chunks": [], "fixup": [], "main": []}
    launches_per_step = 0
    zk = z if pz is None else torch.empty((r1 - r0, k), dtype=tdtype, device=dev)  # not into the shared Z: peers read it
    # first with an event after every launch (the breakdown), then with the outer events only: the events between
    # the kernels keep the library from pairing their launches, so only the second set is the real span
    for detail in (1, 0):
        api.set_option("timing_detail", detail)
        for _ in range(5):
            if flush is not None:
                flush.fill_(2)
                torch.cuda.synchronize()
            st = api.fusedMM_csr(msg, r1 - r0, n, k, 1.0, nnz, n, n, csr.val, csr.indx, pb_all[r0:], pe_all[r0:], x[r0:],
                                 k, x, k, 0.0, zk[r0:] if pz is None else zk, k, sop=sop if sop is not None else 0)
            assert st == 0
            info = api.call_info()
            launches_per_step = info.kernel_launches
            for nm in kms:
                if (nm == "main") != bool(detail):
                    kms[nm].append(getattr(info, "ms_" + nm))
    api.set_option("timing_detail", 1)
    kmed = {nm: float(np.median(v)) for nm, v in kms.items()}
    peak, peak_kind = load_peaks()
    alg_bytes = synth.algorithmic_bytes(msg, my_edges, r1 - r0, k, es, 4, 8)
    # the whole-row launch and the chunk launch of the main kernel run side by side on two streams, so the
    # kernel time is the span that covers both (and the small fix-up work that follows the chunks)
    main_ms = kmed["main"]
    achieved = alg_bytes / (main_ms * 1e-3) * 1e-9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": None, "hbm_frac_real": None, "peak_kind": peak_kind,
                "kernel": "fused_vec_kernel: whole-row launch beside split-row chunk launch, one span",
                "algorithmic_bytes_per_step": alg_bytes, "kernel_ms": kmed,
                "tiling": f"{info.lanes_per_edge} lanes/edge x {info.vectors_per_lane} vec/lane",
                "split_rows": int(info.hub_rows), "row_chunks": int(info.hub_chunks)}
    tr = ROOT / "profiles" / "traffic.json"
    if world == 1 and tr.exists():  # a one-GPU capture says nothing about the L2 hit rate of a shard: null at N > 1
        try:
            rec = json.loads(tr.read_text()).get(cfgname + ("" if dtype == "f32" else "_f64"))
            if rec and not scale:
                roofline["traffic"] = rec["dram_bytes_per_edge"] * my_edges
                roofline["hbm_frac_real"] = roofline["traffic"] / (main_ms * 1e-3) * 1e-9 / peak
                roofline["traffic_note"] = rec.get("note")
        except Exception:
            pass
    if world > 1:
        # bytes every GPU must receive per step: the rows that have edges (multicast: this rank's own rows loop back
        # through the switch too; peer stores: only the other ranks' rows arrive)
        own_nonempty = int((rowptr_host[r0 + 1:r1 + 1] > rowptr_host[r0:r1]).sum())
        rows_in = nonempty_rows if mode == "multicast" else nonempty_rows - own_nonempty
        tt = torch.tensor([float(rows_in), kmed["main"]], dtype=torch.float64, device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        z_in = int(tt[0].item()) * k * es
        run["exchange"] = {"z_bytes_in_per_gpu": z_in, "floor_ms": z_in / (PEER_GBS * 1e9) * 1e3,
                           "peer_gbs": PEER_GBS, "kernel_ms": float(tt[1].item()), "step_ms": ms_step,
                           "rows_with_edges": nonempty_rows, "rows": n,
                           "kernel_only_value": flops_per_edge * nnz / (float(tt[1].item()) * 1e-3) * 1e-9,
                           "note": "floor = bytes every GPU must receive / measured peer bandwidth; kernel_ms = slowest "
                                   "rank's kernels alone on its shard (no exchange); kernel_only_value = the metric if "
                                   "the step took kernel_ms"}

    # ---------------------------------------------------------------- end to end, host buffers
    e2e, e2e_ok = None, True
    if with_e2e:
        e2e, e2e_ok = measure_e2e(args, api, torch, dist, world, dev, csr, x, tdtype, msg, sop, n, k, nnz, r0, r1,
                                  flops_per_edge, barrier, bounds=bounds, pz=pz)

    # ---------------------------------------------------------------- CPU baseline (rank 0, N = 1)
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu_baseline = cpu_leg(torch, ctx["cpu"](), cfg, csr, x, z, nnz, flops_per_edge, cpu_target_s, cpu_steps)

    out = {"metric": METRIC, "value": value, "unit": "GFLOP/s", "n_gpus": world, "steps": steps,
           "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
           "vs_baseline": None, "dtype": dtype, "data": "synthetic", "config": config, "run": run,
           "edges_per_s": nnz / (ms_step * 1e-3),
           "effective_gbs": synth.algorithmic_bytes(msg, nnz, n, k, es, 4, 8) / (ms_step * 1e-3) * 1e-9,
           "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "clocks": clocks.summary(),
           "gpu_launches": (launches_per_step + ((r0 > 0) + (r1 < n) if pz is not None else 0)) * steps,
           "finite": finite and e2e_ok}
    torch.cuda.set_stream(torch.cuda.default_stream())
    del csr, x, z, zk, pb_all, pe_all, flush
    if pz is None:
        api.lib().fusedmm_b200_release()
        torch.cuda.empty_cache()
    return out


def bench_generic(ctx, steps=10):
    """Messages outside the four optimised patterns, on the FR configuration's graph (R-MAT scale 20, K = 256): each
    through the kernel built for it at run time (option jit = 2) and through the flag-interpreting kernel (jit = 0),
    and the FR message itself forced down both routes, to be compared with its built-in kernel."""
    torch, api, synth, M, dev = ctx["torch"], ctx["api"], ctx["synth"], ctx["M"], ctx["dev"]
    cfg, csr, x = synth.make_config("c2_fr_rmat20_k256", device=dev)
    n, k, nnz = cfg["n"], cfg["k"], csr.nnz
    pb, pe = csr.pntrb.contiguous(), csr.pntre.contiguous()
    peak, _ = load_peaks()
    stream = torch.cuda.Stream()
    cases = [("fr_message_as_a_generic_one", M.MSG_TDIST, M.SOP_FR, 2),
             ("add_normr_tdist_mul_max", M.VOP_ADD | M.ROP_NORMR | M.SOP_UDEF | M.VSC_MUL | M.AOP_MAX, M.SOP_TDIST, 0),
             ("min_addrhs_copy_vscadd_min", M.VOP_MIN | M.ROP_ADD_RHS | M.SOP_COPY | M.VSC_ADD | M.AOP_MIN, 0, 0),
             ("subl_dot_sigmoid_mul_add", M.VOP_SUBL | M.ROP_DOT | M.SOP_UDEF | M.VSC_MUL | M.AOP_ADD, M.SOP_SIGMOID, 0)]
    out = []

    def timed(msg, sop, z):
        def call():
            st = api.fusedMM_csr(msg, n, n, k, 1.0, nnz, n, n, csr.val, csr.indx, pb, pe, x, k, x, k, 0.0, z, k, sop=sop,
                                 stream=stream.cuda_stream)
            assert st == 0, api.status_string(st)
        with torch.cuda.stream(stream):
            for _ in range(3):
                call()
            jit = api.call_info().jit_kernel
            stream.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            z.zero_()
            e0.record()
            for _ in range(steps):
                call()
            e1.record()
            stream.synchronize()
            ms = e0.elapsed_time(e1) / steps
            z.zero_()
            call()
            stream.synchronize()
        return ms, jit

    try:
        for name, msg, sop, force in cases:
            bytes_ = synth.algorithmic_bytes(msg, nnz, n, k, 4, 4, 8)
            za = torch.zeros((n, k), device=dev)
            zb = torch.zeros((n, k), device=dev)
            api.set_option("force_generic", force)
            api.set_option("jit", 2)
            ms_jit, used = timed(msg, sop, za)
            api.set_option("jit", 0)
            api.set_option("force_generic", 1 if force else 0)
            ms_rt, _ = timed(msg, sop, zb)
            scale = torch.maximum(zb.abs(), zb.abs().amax(dim=1, keepdim=True)).clamp_min(1e-30)
            err = float(((za - zb).abs() / scale).max())
            out.append({"message": name, "imessage": hex(msg), "sop": sop, "ms": ms_jit, "run_time_built_kernel": bool(used),
                        "generic_frac": bytes_ / (ms_jit * 1e-3) * 1e-9 / peak,
                        "flag_interpreting_ms": ms_rt, "flag_interpreting_frac": bytes_ / (ms_rt * 1e-3) * 1e-9 / peak,
                        "max_rel_diff_between_the_two": err, "finite": bool(torch.isfinite(za).all())})
            del za, zb
    finally:
        api.set_option("force_generic", 0)
        api.set_option("jit", 1)
    api.lib().fusedmm_b200_release()
    torch.cuda.empty_cache()
    return {"graph": "c2_fr_rmat20_k256 (R-MAT scale 20, K = 256, float32)", "steps": steps, "jit": api.jit_stats(), "messages": out}


def compact(rec):
    """One side configuration as a short record."""
    cb = rec["cpu_baseline"] or {}
    return {"workload": rec["config"]["workload"], "dtype": rec["dtype"], "nnz": rec["config"]["nnz"], "k": rec["config"]["k"],
            "ms": rec["ms_per_step"], "gflops": rec["value"], "edges_per_s": rec["edges_per_s"],
            "effective_gbs": rec["effective_gbs"], "frac": rec["roofline"]["frac"],
            "hbm_frac_real": rec["roofline"]["hbm_frac_real"], "kernel_ms": rec["roofline"]["kernel_ms"]["main"],
            "steps": rec["steps"], "l2_flushed": rec["config"]["l2"].startswith("inputs fit"),
            "sm_mhz": rec["clocks"]["sm_mhz"], "reasons": rec["clocks"]["reasons"],
            "cpu_gflops": cb.get("value"), "cpu_variant": cb.get("variant"), "cpu_sample": cb.get("sample"),
            "cpu_general_gflops": (cb.get("general_kernel") or {}).get("value"),
            "err": cb.get("gpu_vs_cpu_max_rel_err_on_sample"), "finite": rec["finite"]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=None)
    ap.add_argument("--scale", type=int, default=None, help="smaller instance of the same graph family")
    ap.add_argument("--dtype", default="f32", choices=["f32", "f64"])
    ap.add_argument("--e2e-steps", type=int, default=None)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-array (end-to-end) leg; e2e is then null")
    ap.add_argument("--no-configs", action="store_true", help="skip the records of the other configurations")
    ap.add_argument("--generic-only", action="store_true", help="only the section on messages outside the four patterns")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    default_run = args.workload is None and args.scale is None and args.dtype == "f32"
    cfgname = args.workload or DEFAULT_WORKLOAD

    import torch
    from fusedmm_b200 import api, messages as M, synth

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    tdtype = torch.float32 if args.dtype == "f32" else torch.float64
    es = 4 if args.dtype == "f32" else 8
    base_cfg = synth.CONFIGS[cfgname]
    flops_per_edge = M.FLOPS_PER_EDGE_PER_K[base_cfg["msg"]] * base_cfg["k"]

    # ---------------------------------------------------------------- reference arm (CPU only)
    if args.impl == "reference":
        if rank != 0:
            return
        eng = CpuEngine()
        dev = "cuda" if torch.cuda.is_available() else "cpu"  # the device only generates the synthetic inputs
        cfg, csr, x = synth.make_config(cfgname, device=dev, dtype=tdtype, scale=args.scale)
        nnz = csr.nnz
        config = workload_config(cfgname, args.dtype, args.scale, cfg["n"], nnz, cfg["sop"], cfg["k"], cfg["msg"], es)
        y_host = x.cpu().numpy()
        # each step is one call on a bounded row sample, sized so that warmup + steps stay within about a minute
        target = max(0.3, min(2.0, 45.0 / max(1, args.steps + args.warmup)))
        stride = pick_stride(torch, eng.call, cfg, csr, x, y_host, nnz, target_s=target)
        smp = sample_rows(torch, csr, x, stride)
        del csr, x
        times, _ = time_cpu(eng.call, cfg, smp, y_host, args.steps, args.warmup)
        ms = 1e3 * float(np.mean(times))
        value = flops_per_edge * smp["edges"] / (ms * 1e-3) * 1e-9
        sample = f"every {stride}-th row of the graph ({smp['edges']} of {nnz} edges), whole Y"
        print(json.dumps({
            "impl": "reference", "metric": METRIC, "value": value, "unit": "GFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
            "config": config, "edges_per_s": smp["edges"] / (ms * 1e-3),
            "cpu_baseline": {"value": value, "unit": "GFLOP/s", "cores": eng.cores, "kind": eng.kind, "variant": eng.variant,
                             "simd": eng.simd, "omp_threads": eng.cores, "sample": sample, "code": eng.code},
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
    from fusedmm_b200 import dist as fdist
    cpu_cache = {}

    def cpu():
        if "e" not in cpu_cache:
            cpu_cache["e"] = CpuEngine()
        return cpu_cache["e"]

    ctx = {"torch": torch, "api": api, "synth": synth, "M": M, "fdist": fdist, "dist": dist, "rank": rank, "world": world,
           "dev": dev, "cpu": cpu}
    if args.generic_only:
        print(json.dumps(bench_generic(ctx)))
        return
    big = synth.CONFIGS[cfgname]["graph"][1] >= 22 and not args.scale
    steps = args.steps
    out = bench_gpu(args, ctx, cfgname, args.dtype, args.scale, steps, args.warmup, with_e2e=not args.no_e2e,
                    cpu_target_s=4.0, cpu_steps=3 if not big else 2)

    if world > 1 and os.environ.get("FUSEDMM_BENCH_SELF_CHECK", "1") == "1":
        # parity of the fused exchange beyond the timed message: beta = 0 and beta = 1, float and double (the
        # multicast store of doubles goes through a bit cast), on a small graph
        mode = "multicast" if "multimem" in out["run"].get("exchange_kind", "") else "peer"
        if "fused" in out["run"].get("exchange_kind", ""):
            chk = {}
            for nm, tdt in (("f32", torch.float32), ("f64", torch.float64)):
                chk[nm] = exchange_self_check(api, torch, dist, fdist, dev, rank, world, tdt, mode)
            out["run"]["exchange_self_check_beta0_beta1"] = chk

    if world == 1 and default_run and not args.no_configs:
        recs = []
        for name, dt in SIDE_CONFIGS:
            small = synth.CONFIGS[name]["graph"][1] < 22 or synth.CONFIGS[name]["graph"][0] == "er"
            rec = bench_gpu(args, ctx, name, dt, None, 20 if small else 5, 5 if small else 3, with_e2e=False,
                            cpu_target_s=1.5, cpu_steps=2)
            recs.append(compact(rec))
        out["configs"] = recs
        out["generic"] = bench_generic(ctx)

    if rank == 0:
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
