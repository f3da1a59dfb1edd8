"""Benchmark of the MTP speculative-decode hot path on B200.

python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Prints ONE JSON line (rank 0). Workloads:
  gemv      BASELINE config 1: Q4_K 17408 x 5120 verify GEMV over 3 rows + argmax + greedy acceptance
A "step" is one pass of the hot path over one batch of seeded synthetic input. Inputs larger than L2: the
weight matrix is rotated through enough device copies (> 512 MB) that no step finds its weights in the 126 MB L2.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PEAKS_FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p)); d["_src"] = "measured"; return d
    d = dict(PEAKS_FALLBACK); d["_src"] = "fallback"; return d


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms during the timed region."""
    Q = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, gpu_index):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--id={gpu_index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200"], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.p = None

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except Exception:
            self.p.kill()
        self.f.flush(); self.f.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.f.read().splitlines():
            c = [x.strip() for x in line.split(",")]
            if len(c) < 9:
                continue
            try:
                sm.append(float(c[1])); mx.append(float(c[2]))
            except ValueError:
                continue
            for n, v in zip(names, c[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        self.f.close()
        try:
            os.unlink(self.f.name)
        except OSError:
            pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = sorted(sm)[len(sm) // 2:]   # upper half = samples under load
        return {"sm_mhz": float(np.median(busy)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


# --------------------------------------------------------------------------------------------- workload: gemv
GEMV_N, GEMV_K, GEMV_R = 17408, 5120, 3
GEMV_BYTES = GEMV_N * (GEMV_K // 256) * 144 + GEMV_R * GEMV_K * 4 + GEMV_R * GEMV_N * 4   # 50,405,376 algorithmic bytes


def gemv_cpu(steps, warmup, threads_note=True):
    """The CPU oracle's restatement of the same step (quantise -> W4A8 GEMV -> argmax -> accept) on the host cores."""
    from oracle import orc
    from hipster_b200 import synth
    W = synth.q4k_matrix(GEMV_N, GEMV_K, seed=0); x = synth.activations(GEMV_R, GEMV_K, seed=0)
    drafts = np.array([1, 2], dtype=np.int32)

    def step():
        q, d, s = orc.quantize_x_q8(x)
        y = orc.gemv_q4k_q8(W, q, d, s, GEMV_N, GEMV_K)
        ids, _ = orc.argmax(y)
        return orc.accept(ids, drafts)
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    return dt, orc.lib().orc_num_threads()


def run_gemv(args, rank, local_rank, world):
    import torch
    import torch.distributed as dist
    from hipster_b200 import kernels as K_, synth, lib, check, ptr
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    W_h = synth.q4k_matrix(GEMV_N, GEMV_K, seed=0)
    ncopy = (512 << 20) // W_h.nbytes + 1
    Ws = [torch.from_numpy(W_h).to(dev) for _ in range(ncopy)]
    x_h = torch.from_numpy(synth.activations(GEMV_R, GEMV_K, seed=0)).pin_memory()
    drafts_h = torch.tensor([1, 2], dtype=torch.int32).pin_memory()
    x_d = x_h.to(dev); drafts_d = drafts_h.to(dev)
    xq = K_.XQ8(GEMV_R, GEMV_K, dev)
    y = torch.empty((GEMV_R, GEMV_N), dtype=torch.float32, device=dev)
    out_h = torch.empty(2, dtype=torch.int32).pin_memory()
    it = [0]

    def step_resident():
        K_.quantize_x_q8(x_d, xq)
        K_.gemv_q4k_q8(Ws[it[0] % ncopy], xq, GEMV_N, GEMV_K, y); it[0] += 1
        ids, _ = K_.argmax(y)
        return K_.accept_greedy(ids, drafts_d)

    def step_e2e():
        xd = x_h.to(dev, non_blocking=True); dd = drafts_h.to(dev, non_blocking=True)
        K_.quantize_x_q8(xd, xq)
        K_.gemv_q4k_q8(Ws[it[0] % ncopy], xq, GEMV_N, GEMV_K, y); it[0] += 1
        ids, _ = K_.argmax(y)
        out = K_.accept_greedy(ids, dd)
        out_h.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return out_h

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record(); torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev); dist.all_reduce(t, op=dist.ReduceOp.MAX); ms = float(t.item()); dist.barrier()
        return ms

    sampler = ClockSampler(local_rank) if rank == 0 else None
    ms = timed(step_resident, args.steps, args.warmup)
    ms_e2e = timed(step_e2e, args.steps, args.warmup)
    # dominant kernel alone, CUDA events on the launching stream, weights rotated past L2
    K_.quantize_x_q8(x_d, xq)
    def gemv_only():
        K_.gemv_q4k_q8(Ws[it[0] % ncopy], xq, GEMV_N, GEMV_K, y); it[0] += 1
    n_k = max(args.steps, 50)
    ms_k = timed(gemv_only, n_k, 5) / n_k
    clocks = sampler.stop() if sampler else None
    K_.device_status()
    if rank != 0:
        return None
    pk = peaks()
    rows_per_s = world * GEMV_R * args.steps / (ms / 1e3)
    achieved = GEMV_BYTES / (ms_k / 1e3) / 1e9
    line = {
        "metric": "MTP-spec decode tokens/s (Q4_K); verify-GEMV HBM GB/s vs B200 peak",
        "value": rows_per_s, "unit": "verify rows/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u4 x i8 -> i32, f32 epilogue", "data": "synthetic",
        "config": {"workload": "config1: Q4_K 17408x5120 verify GEMV, 3 rows, argmax + greedy acceptance",
                   "l2": f"weights rotated through {ncopy} device copies ({ncopy * W_h.nbytes >> 20} MiB > L2)", "parallelism": f"replicas x{world}"},
        "e2e": {"value": world * GEMV_R * args.steps / (ms_e2e / 1e3), "unit": "verify rows/s",
                "h2d_bytes_per_step": int(x_h.numel() * 4 + drafts_h.numel() * 4), "d2h_bytes_per_step": 8},
        "gpu_launches": 5 * args.steps,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
                     "traffic": None, "kernel": "k_gemv_q4k_q8<1>", "us_per_launch": ms_k * 1e3, "peak_source": pk["_src"]},
        "clocks": clocks,
    }
    if world == 1 and not args.no_cpu:
        dt, th = gemv_cpu(3, 1)
        line["cpu_baseline"] = {"value": GEMV_R / dt, "unit": "verify rows/s", "cores": th, "kind": "port",
                                "sample": "full config-1 step (quantise, 17408x5120 W4A8 GEMV over 3 rows, argmax, accept), mean of 3"}
    return line


def run_reference(args, rank, world):
    if rank != 0:
        return None
    dt, th = gemv_cpu(max(1, min(args.steps, 10)), max(1, min(args.warmup, 2)))
    v = GEMV_R / dt
    return {"impl": "reference", "metric": "MTP-spec decode tokens/s (Q4_K); verify-GEMV HBM GB/s vs B200 peak", "value": v, "unit": "verify rows/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "u4 x i8 -> i32, f32 epilogue", "data": "synthetic",
            "config": {"workload": "config1: Q4_K 17408x5120 verify GEMV, 3 rows, argmax + greedy acceptance"},
            "cpu_baseline": {"value": v, "unit": "verify rows/s", "cores": th, "kind": "port",
                             "sample": "CPU restatement of the reference's kernels (its HIP kernels cannot be built without ROCm); full config-1 step"},
            "e2e": {"value": v, "unit": "verify rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gemv")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank, local_rank, world = dist_env()
    if args.impl == "reference":
        line = run_reference(args, rank, world)
        if line:
            print(json.dumps(line), flush=True)
        return
    import torch
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    line = run_gemv(args, rank, local_rank, world)
    if line:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
