#!/usr/bin/env python
"""Benchmark of the EGGROLL population-evaluation path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one ES generation of the Int8NativeFormer benchmark configuration
(4 layers, H=512, 8 heads, MLP 4H, seq 256, vocab 256, 40 960 antithetic members per
GPU, DEVICE_MASK=3, ES-AdamW): population evaluation, pair fitness, fitness exchange
(NCCL all-gather when N > 1) and update reconstruction + optimiser step.  The metric
is the reference's own "tok/s": POPULATION_SIZE * SEQ_LEN / generation seconds
(member-token evaluations per second), aggregated over all GPUs.

Prints ONE JSON line on rank 0.  `--impl reference` times the reference's CPU trainer
(full_trained_egg.c, built into oracle/_ref/ref_cpu_gru) on the host cores instead.
"""
import argparse
import importlib.util
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
METRIC = "member_token_evals_per_sec"
UNIT = "member-tokens/s"
WORKLOAD = ("Int8NativeFormer one ES-AdamW generation: L=4 H=512 heads=8 MLP=4H seq=256 vocab=256, "
            "40960 antithetic members per GPU, rank-1 noise mask 3")
C2 = dict(hidden_dim=512, head_dim=64, n_layers=4, seq_len=256, vocab_size=256, device_mask=3)
POP_PER_GPU = 40960
DATA_LEN = 64 << 20
LR = 0.05


def _load(name, path, search=None):
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, path, submodule_search_locations=search)
    m = importlib.util.module_from_spec(spec)
    sys.modules[name] = m
    spec.loader.exec_module(m)
    return m


def load_pkg():
    d = os.path.join(ROOT, "egg.c_b200")
    return _load("egg_c_b200", os.path.join(d, "__init__.py"), [d])


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if not self.proc:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); smax.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        os.unlink(self.path)
        if sm:
            out.update(sm_mhz=float(np.median(sm)), sm_max_mhz=float(max(smax)), reasons=sorted(reasons), samples=len(sm))
        return out


# ----------------------------------------------------------------------------- reference arm (CPU)
def cpu_reference_run(steps, warmup, pairs=None, tokens=None):
    """Times the reference's own CPU trainer functions (full_trained_egg.c: forward_pass x2 per pair,
    compiled unmodified into oracle/_ref/ref_cpu_gru) on all host cores, on a bounded sample."""
    exe = os.path.join(ROOT, "oracle", "_ref", "ref_cpu_gru")
    if not os.path.exists(exe):
        return None
    pkg = load_pkg()
    from egg_c_b200 import synth
    sizes = json.loads(subprocess.run([exe, "--sizes"], check=True, capture_output=True, text=True).stdout)
    cores = os.cpu_count() or 1
    pairs = pairs or min(sizes["population_size"] // 2, max(1, cores))
    tokens = tokens or 1024
    model = synth.uniform_int8(0, sizes["model_bytes"])
    data = synth.zipf_bytes(1, 1 << 20)
    vals = []
    with tempfile.TemporaryDirectory() as td:
        fin, fout = os.path.join(td, "in.bin"), os.path.join(td, "out.bin")
        with open(fin, "wb") as f:
            f.write(np.uint32(0x00C0FFEE).tobytes()); f.write(np.int64(len(data)).tobytes())
            f.write(model.tobytes()); f.write(data.tobytes())
        for i in range(warmup + steps):
            r = subprocess.run([exe, fin, fout, str(pairs), str(tokens)], check=True, capture_output=True, text=True)
            info = json.loads(r.stdout.strip().splitlines()[-1])
            if i >= warmup:
                vals.append(info["member_tokens_per_s"])
    return {"value": float(np.mean(vals)), "unit": UNIT, "cores": int(info["threads"]), "kind": "reference",
            "ms_per_step": 1e3 * 2 * pairs * tokens / float(np.mean(vals)),
            "sample": "full_trained_egg.c forward_pass (GRU+MLP int8 model at its compiled-in H=512 L=4), %d pairs x %d tokens "
                      "= %d member-tokens per step, one OpenMP task per pair" % (pairs, tokens, 2 * pairs * tokens)}


def run_reference_arm(args, rank):
    if rank != 0:
        return
    res = cpu_reference_run(args.steps, max(args.warmup, 0))
    if res is None:
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/ref_cpu_gru is not built"}))
        return
    line = {"metric": METRIC, "value": res["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8/int32",
            "data": "synthetic", "impl": "reference", "config": {"workload": WORKLOAD, "note": "reference CPU path: " + res["sample"]},
            "cpu_baseline": res, "e2e": {"value": res["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


def gru_model_run(pkg, synth, device, tokens=512, reps=2):
    """The model the CPU baseline runs (full_trained_egg.c: GRU + MLP, H 512, 4 layers, population 128) through this
    library's GPU path, so that the two numbers of the JSON line that share a unit also share a model.  Wall clock
    around the blocking C-ABI call (noise generation, token steps, fitness, update, losses D2H)."""
    import time
    gcfg = pkg.default_gru_config()
    ctx = pkg.GruContext(gcfg, device)
    ctx.upload_model(synth.uniform_int8(0, pkg.gru_model_bytes(gcfg)))
    ctx.set_dataset(synth.zipf_bytes(1, 1 << 20))
    ctx.generation(0x00C0FFEE, 0, 32, True)                    # warm-up: graph capture
    n0 = ctx.launch_count()
    t0 = time.perf_counter()
    for r in range(reps):
        ctx.generation(0x00C0FFEE + 1 + r, (r + 1) * gcfg.seq_len, tokens, True)
    dt = (time.perf_counter() - t0) / reps
    launches = (ctx.launch_count() - n0) // reps
    ctx.close()
    return {"value": gcfg.population_size * tokens / dt, "unit": UNIT, "ms_per_generation_sample": dt * 1e3,
            "sample": "%d members x %d tokens per generation (the reference runs 4096 tokens), update included" % (gcfg.population_size, tokens),
            "gpu_launches": int(launches), "timing": "wall clock around the blocking call"}


# ----------------------------------------------------------------------------- our arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--pop", type=int, default=POP_PER_GPU, help="members per GPU (benchmark value: 40960)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--wave", type=int, default=0, help="members per internal wave (0: the library's default)")
    ap.add_argument("--small", action="store_true", help="profiling-sized run: 1024 members, one warm-up step, no end-to-end / CPU legs")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if args.small:
        args.pop, args.no_cpu_baseline = 1024, True

    # libraries (NCCL's version banner, for one) may write to stdout: keep fd 1 for the single JSON line
    real_stdout = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)

    import torch   # device discovery and the process group only; the hot path is the C ABI
    pkg = load_pkg()
    from egg_c_b200 import synth
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: the library has no CPU path")
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    pop = args.pop * world                       # weak scaling: fixed members per GPU
    cfg = pkg.default_config(population_size=pop, **C2)
    ctx = pkg.Context(cfg, local_rank, args.wave)
    model = synth.random_model(cfg, 0, "uniform")
    ctx.upload_model(model)
    data_np = synth.zipf_bytes(1, DATA_LEN)
    data_pinned = torch.from_numpy(data_np).pin_memory()
    data_host = data_pinned.numpy()
    ctx.set_dataset(data_host)
    per = pop // world
    losses_pinned = torch.empty(per, dtype=torch.int32).pin_memory()
    losses_host = losses_pinned.numpy()
    if world > 1:
        ident = [pkg.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ident, src=0)
        ctx.comm_init(ident[0], rank, world)

    def barrier():
        ctx.sync()
        if dist:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if not dist:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    seed0 = 0x00C0FFEE
    step_no = [0]

    def one_step(host_io):
        s = step_no[0]
        step_no[0] += 1
        if host_io:
            return ctx.generation_host(data_host, s, seed0 + s, LR, losses_host)
        return ctx.generation_host(None, s, seed0 + s, LR, None)

    # ---- kernel-resident timing (inputs already in HBM) ----
    n_warm = args.warmup if args.small else max(args.warmup, 3)
    for _ in range(n_warm):
        one_step(False)
    barrier()
    launches0 = ctx.launch_count()
    sampler = ClockSampler(local_rank)
    sampler.start()
    ctx.profile_enable(True)
    ctx.profile_read()
    ctx.timer_start()
    for _ in range(args.steps):
        one_step(False)
    ms_dev = ctx.timer_stop()
    barrier()
    clocks = sampler.stop()
    prof = ctx.profile_read()
    ctx.profile_enable(False)
    launches = ctx.launch_count() - launches0
    ms_dev = max_over_ranks(ms_dev)
    ms_per_step = ms_dev / args.steps
    value = pop * cfg.seq_len / (ms_per_step / 1e3)

    # ---- end to end through host buffers (dataset H2D, losses D2H every step) ----
    e2e_steps = 0 if args.small else args.steps
    ms_e2e = ms_per_step
    if e2e_steps:
        one_step(True)
        barrier()
        ctx.timer_start()
        for _ in range(e2e_steps):
            one_step(True)
        ms_e2e = max_over_ranks(ctx.timer_stop()) / e2e_steps
        barrier()
    e2e_value = pop * cfg.seq_len / (ms_e2e / 1e3)

    # ---- roofline of the dominant kernel class ----
    H, L, S, V = cfg.hidden_dim, cfg.n_layers, cfg.seq_len, cfg.vocab_size
    rows_per_step = per * S
    gemm_ops = {   # algorithmic int8 ops per generation on this rank (2*M*N*K)
        "gemm_gelu": 2.0 * rows_per_step * H * 4 * H * (L + 1),
        "gemm_pre32": 2.0 * rows_per_step * (4 * H * H * (L + 1) + H * H * L),
        "gemm_qkv": 2.0 * rows_per_step * 3 * H * H * L,
        "gemm_head": 2.0 * rows_per_step * H * V,
    }
    hbm_bytes = {  # algorithmic bytes per generation on this rank
        "attention": 4.0 * H * rows_per_step * L,
        "rowwise": 6.0 * H * rows_per_step * (2 * L + 2),
        "aqn": 15.0 * H * rows_per_step * L,
    }
    # DRAM bytes (read + write) per row of one launch, from the ncu captures summarised under profiles/ (262 144-row
    # launches of the same kernels; traffic grows in proportion to the rows of a launch)
    ncu_traffic_per_row = {"attention": (404.110e6 + 116.544e6) / 262144, "rowwise": (543.130e6 + 249.417e6) / 262144,
                           "aqn": (1613.772e6 + 384.940e6) / 262144,
                           "gemm_gelu": (143.689e6 + 484.641e6) / 262144, "gemm_qkv": (142.191e6 + 1560.224e6) / 262144,
                           "gemm_pre32": (675.062e6 + 494.890e6) / 262144}
    peaks = {}
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peaks = json.load(open(pk))
    hbm_peak = peaks.get("hbm_gbs", 6650.0)
    # no int8 figure is measured on this pool: int8 dense peak taken as 2x the measured sustained bf16 GEMM throughput
    tensor_peak = 2.0 * peaks.get("bf16_tflops_sustained", 1400.0)
    peak_src = "measured" if peaks else "fallback"
    rows_per_launch = min(ctx.wave_members(), per) * S
    traffic_src = "ncu dram__bytes_read.sum + dram__bytes_write.sum of a 262144-row launch (profiles/), scaled by rows per launch"

    def class_roofline(k):
        t_ms, n_launch = prof[k]
        if k in gemm_ops:
            achieved = gemm_ops[k] * args.steps / (t_ms / 1e3) / 1e12
            r = {"kernel": k, "bound": "tensor", "achieved": achieved, "peak": tensor_peak, "unit": "TFLOP/s", "frac": achieved / tensor_peak}
        else:
            achieved = hbm_bytes[k] * args.steps / (t_ms / 1e3) / 1e9
            r = {"kernel": k, "bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak}
        r["avg_launch_ms"] = t_ms / max(1, n_launch)
        r["traffic"] = ncu_traffic_per_row[k] * rows_per_launch if k in ncu_traffic_per_row else None
        return r

    per_class = [class_roofline(k) for k in prof if prof[k][1] > 0 and (k in gemm_ops or k in hbm_bytes)]
    # The dominant kernel is the one __global__ function with the largest share of the step: the projection GEMM
    # (gemm_i8_kernel, four epilogue instantiations) counts as one kernel, the row-wise kernels each as their own.
    gemm_keys = [k for k in gemm_ops if k in prof and prof[k][1] > 0]
    gemm_ms = sum(prof[k][0] for k in gemm_keys)
    gemm_launches = sum(prof[k][1] for k in gemm_keys)
    others = [k for k in hbm_bytes if k in prof and prof[k][1] > 0]
    top_other = max(others, key=lambda k: prof[k][0]) if others else None
    if gemm_keys and (top_other is None or gemm_ms >= prof[top_other][0]):
        achieved = sum(gemm_ops[k] for k in gemm_keys) * args.steps / (gemm_ms / 1e3) / 1e12
        known = [k for k in gemm_keys if k in ncu_traffic_per_row]
        roof = {"kernel": "gemm_i8_kernel (all projection epilogues)", "bound": "tensor", "achieved": achieved, "peak": tensor_peak,
                "unit": "TFLOP/s", "frac": achieved / tensor_peak,
                "traffic": (sum(ncu_traffic_per_row[k] * rows_per_launch * prof[k][1] for k in known) / max(1, sum(prof[k][1] for k in known)))
                if known else None,
                "peak_source": "2 x bf16_tflops_sustained of %s MEASURED_PEAKS (no int8 entry); int8 ops" % peak_src,
                "avg_launch_ms": gemm_ms / max(1, gemm_launches), "share_of_step": None,
                "traffic_source": traffic_src + "; launch-weighted mean over the GELU / residual / QKV instantiations"}
    else:
        roof = class_roofline(top_other)
        roof["peak_source"] = "hbm_gbs of %s MEASURED_PEAKS" % peak_src
        roof["traffic_source"] = traffic_src
    total_prof = sum(v[0] for v in prof.values()) or 1.0
    kernel_share = {k: {"ms_per_step": v[0] / args.steps, "launches_per_step": v[1] / args.steps, "share": v[0] / total_prof}
                    for k, v in prof.items() if v[1] > 0}
    roof["share_of_step"] = (gemm_ms if roof["bound"] == "tensor" else prof[top_other][0]) / total_prof
    gemm_total_ms = sum(prof[k][0] for k in gemm_ops if k in prof)
    gemm_tops = sum(gemm_ops.values()) * args.steps / (gemm_total_ms / 1e3) / 1e12 if gemm_total_ms > 0 else None

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            cpu = cpu_reference_run(1, 0)
        except Exception as e:   # the baseline is reported, never allowed to break the bench line
            cpu = {"value": None, "unit": UNIT, "cores": os.cpu_count(), "kind": "reference", "sample": "failed: %s" % e}

    # what the GEMM's own TMA + tcgen05 loop sustains on this GPU with the accumulators dropped (operands in L2)
    mma_loop_tops = None
    if rank == 0 and not args.small:
        try:
            mma_loop_tops = ctx.measure_int8_peak(16384, 2048, 2048, 20)
        except Exception:
            mma_loop_tops = None

    gru = None
    if rank == 0 and world == 1 and not args.small:
        try:
            gru = gru_model_run(pkg, synth, local_rank)
        except Exception as e:
            gru = {"value": None, "unit": UNIT, "sample": "failed: %s" % e}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": n_warm,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8/int32",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "population_size": pop, "members_per_gpu": per, "seq_len": S, "hidden_dim": H,
                       "n_layers": L, "wave_members": ctx.wave_members(), "dataset_bytes": DATA_LEN,
                       "l2_policy": "inputs larger than L2: each wave streams > 2 GB of activations, dataset 64 MiB",
                       "parallelism": "population sharded, pair-aligned; one NCCL all-gather of fitness per generation"},
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e, "h2d_bytes_per_step": int(DATA_LEN),
                    "d2h_bytes_per_step": int(per * 4 + 8)},
            "gpu_launches": int(launches),
            "roofline": roof,
            "rooflines_by_class": per_class,
            "projection_gemms": {"tops": gemm_tops, "frac_of_peak": (gemm_tops / tensor_peak) if gemm_tops else None, "peak": tensor_peak,
                                 "mma_loop_tops_measured": mma_loop_tops,
                                 "frac_of_mma_loop": (gemm_tops / mma_loop_tops) if (gemm_tops and mma_loop_tops) else None},
            "kernels": kernel_share,
            "clocks": clocks,
            "cpu_baseline": cpu,
            "gru_model_gpu": gru,
        }
        real_stdout.write(json.dumps(line) + "\n")
        real_stdout.flush()
    ctx.close()
    if dist:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
