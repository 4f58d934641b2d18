#!/usr/bin/env python
"""Benchmark of the EGGROLL population-evaluation path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c3|c4|c5slice|c5|tok]

Default workload `c2`: one "step" is one ES generation of the Int8NativeFormer benchmark configuration
(4 layers, H=512, 8 heads, MLP 4H, seq 256, vocab 256, 40 960 antithetic members per GPU, DEVICE_MASK=3,
ES-AdamW): population evaluation, pair fitness, fitness exchange (NCCL all-gather when N > 1) and update
reconstruction + optimiser step.  The metric is the reference's own "tok/s": POPULATION_SIZE * SEQ_LEN /
generation seconds (member-token evaluations per second), aggregated over all GPUs.

Other workloads (single GPU, same JSON contract, named in config.workload):
  c3       isolated perturbed projection, W 4096 x 4096, 4096 members x 64 tokens (rows are member-tokens)
  c4       isolated update reconstruction of a 4096 x 4096 weight from 32 768 pairs of int8 fitness, followed by an
           ES-AdamW step and a Muon step (value: pair-weights reconstructed per second is not the headline metric,
           so the line reports member-token-equivalents = pairs*2 per step second and the tensor roofline)
  c5slice  d-eggs-scale shapes (12 layers, H 1024, seq 512, ternary weights, Muon): a slice of the 262 144-member
           population is evaluated, the update runs over all 131 072 pairs
  tok      the reference's tokenizer build at the benchmark shapes: vocabulary 8192 (--vocab), uint32 tokens, 8192 members
           (--pop) per generation; the head takes two passes over 32 column tiles per row
  c5       the same shapes as a whole generation of a FIXED population (--pop-total, default 262 144) sharded over the N
           GPUs of the launch ("scaling": "strong"); a step takes tens of seconds at N = 1, so run it with --steps 1

Prints ONE JSON line on rank 0.  `--impl reference` times the reference's CPU trainer
(full_trained_egg.c, built into oracle/_ref/ref_cpu_gru) on the host cores instead.
"""
import argparse
import importlib.util
import json
import os
import struct
import subprocess
import sys
import tempfile
import zlib

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
METRIC = "member_token_evals_per_sec"
UNIT = "member-tokens/s"
WORKLOAD = ("Int8NativeFormer one ES-AdamW generation: L=4 H=512 heads=8 MLP=4H seq=256 vocab=256, "
            "40960 antithetic members per GPU, rank-1 noise mask 3")
C2 = dict(hidden_dim=512, head_dim=64, n_layers=4, seq_len=256, vocab_size=256, device_mask=3)
C5 = dict(hidden_dim=1024, head_dim=64, n_layers=12, seq_len=512, vocab_size=256, device_mask=15)
POP_PER_GPU = 40960
DATA_LEN = 64 << 20
LR = 0.05
SEED0 = 0x00C0FFEE


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


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def load_peaks():
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peaks = json.load(open(pk)) if os.path.exists(pk) else {}
    src = "measured" if peaks else "fallback"
    # no int8 figure is measured on this pool: int8 dense peak taken as 2x the measured sustained bf16 GEMM throughput
    return {"hbm": peaks.get("hbm_gbs", 6650.0), "tensor": 2.0 * peaks.get("bf16_tflops_sustained", 1400.0), "src": src,
            "tensor_source": "2 x bf16_tflops_sustained of %s MEASURED_PEAKS (no int8 entry); int8 ops" % src,
            "hbm_source": "hbm_gbs of %s MEASURED_PEAKS" % src}


def load_traffic():
    """DRAM bytes per launch from the committed ncu captures (profiles/ncu_dram_traffic.json), per row."""
    p = os.path.join(ROOT, "profiles", "ncu_dram_traffic.json")
    if not os.path.exists(p):
        return {}, None
    j = json.load(open(p))
    rows = float(j["rows_per_captured_launch"])
    per_row = {k: (v["read"] + v["write"]) / rows for k, v in j["bytes_per_launch"].items()}
    src = ("ncu dram__bytes_read.sum + dram__bytes_write.sum of a %d-row launch (profiles/ncu_dram_traffic.json, captured at "
           "commit %s), scaled by rows per launch; not re-measured by this run" % (int(rows), j["taken_at_commit"]))
    return per_row, src


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
def cpu_reference_run(steps, warmup, tokens=None):
    """Times the reference's own CPU trainer (full_trained_egg.c compiled unmodified into oracle/_ref/ref_cpu_gru) on
    all host cores: one generation of its whole population (64 pairs -> forward_pass x2 per pair, then its 25
    update_matrix calls) on a bounded number of tokens per member (the reference runs 4096)."""
    exe = os.path.join(ROOT, "oracle", "_ref", "ref_cpu_gru")
    if not os.path.exists(exe):
        return None
    load_pkg()
    from egg_c_b200 import synth
    sizes = json.loads(subprocess.run([exe, "--sizes"], check=True, capture_output=True, text=True).stdout)
    cores = host_cores()
    pairs = sizes["population_size"] // 2             # the whole population: only then does the driver run the update
    tokens = tokens or max(64, min(1024, 16 * cores))  # about 10-20 s per step at ~5 ms per member-token and core
    model = synth.uniform_int8(0, sizes["model_bytes"])
    data = synth.zipf_bytes(1, 1 << 20)
    env = dict(os.environ, OMP_NUM_THREADS=str(cores))    # torch.distributed.run exports OMP_NUM_THREADS=1
    vals, info = [], None
    with tempfile.TemporaryDirectory() as td:
        fin, fout = os.path.join(td, "in.bin"), os.path.join(td, "out.bin")
        with open(fin, "wb") as f:
            f.write(np.uint32(SEED0).tobytes()); f.write(np.int64(len(data)).tobytes())
            f.write(model.tobytes()); f.write(data.tobytes())
        for i in range(warmup + steps):
            r = subprocess.run([exe, fin, fout, str(pairs), str(tokens)], check=True, capture_output=True, text=True, env=env)
            info = json.loads(r.stdout.strip().splitlines()[-1])
            if i >= warmup:
                vals.append(info["member_tokens_per_s"])
    return {"value": float(np.mean(vals)), "unit": UNIT, "cores": int(info["threads"]), "kind": "reference",
            "ms_per_step": 1e3 * 2 * pairs * tokens / float(np.mean(vals)),
            "eval_s": info["eval_s"], "update_s": info["update_s"],
            "sample": "full_trained_egg.c (GRU+MLP int8 model at its compiled-in H=512 L=4, population 128): one generation = "
                      "forward_pass of all 64 pairs x 2 members on %d tokens (the reference's SEQ_LEN is 4096) + its 25 update_matrix "
                      "calls = %d member-tokens per step, one OpenMP task per pair, %d threads" % (tokens, 2 * pairs * tokens, int(info["threads"]))}


def run_reference_arm(args, rank):
    if rank != 0:
        return
    res = cpu_reference_run(min(args.steps, 3), min(max(args.warmup, 0), 1))
    if res is None:
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/ref_cpu_gru is not built"}))
        return
    line = {"metric": METRIC, "value": res["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": min(args.steps, 3),
            "warmup": min(max(args.warmup, 0), 1),
            "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8/int32",
            "data": "synthetic", "impl": "reference", "config": {"workload": WORKLOAD, "note": "reference CPU path: " + res["sample"]},
            "cpu_baseline": res, "e2e": {"value": res["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


def reference_gpu_kernels_run(members=1024):
    """Member-tokens/s of the reference's own train_sequence_kernel (mgpu.cu:847, built unmodified for sm_100a into
    oracle/_ref/ref_mgpu_c2) on `members` members of the same configuration on the same GPU: CUDA events inside the
    harness around its launches."""
    exe = os.path.join(ROOT, "oracle", "_ref", "ref_mgpu_c2")
    if not os.path.exists(exe):
        return {"value": None, "unit": UNIT, "sample": "oracle/_ref/ref_mgpu_c2 is not built"}
    pkg = load_pkg()
    from egg_c_b200 import synth
    cfg = pkg.default_config(population_size=40960, **C2)
    model = synth.random_model(cfg, 0, "uniform")
    data = synth.zipf_bytes(1, 1 << 22)
    with tempfile.TemporaryDirectory() as td:
        fin, fout = os.path.join(td, "in.bin"), os.path.join(td, "out.bin")
        with open(fin, "wb") as f:
            f.write(struct.pack("<IIqqiifiii", 0x46524745, SEED0, 256, len(data), 0, members, 0.0, 0, 0, 0))
            f.write(struct.pack("<6i", C2["hidden_dim"], C2["n_layers"], C2["seq_len"], 40960, C2["device_mask"], 0))
            f.write(model.tobytes()); f.write(data.tobytes())
        r = subprocess.run([exe, fin, fout], capture_output=True, text=True, timeout=600)
        if r.returncode != 0:
            return {"value": None, "unit": UNIT, "sample": "harness failed: " + (r.stderr or r.stdout)[-200:]}
        info = json.loads(r.stdout.strip().splitlines()[-1])
    return {"value": members * C2["seq_len"] / (info["eval_ms"] / 1e3), "unit": UNIT, "eval_ms": info["eval_ms"],
            "sample": "train_sequence_kernel of the reference (one block per member, dp4a) on %d members x %d tokens, "
                      "same model configuration, same GPU; evaluation only" % (members, C2["seq_len"])}


def gru_model_run(pkg, synth, device, tokens=512, reps=2):
    """The model the CPU baseline runs (full_trained_egg.c: GRU + MLP, H 512, 4 layers, population 128) through this
    library's GPU path, so that the two numbers of the JSON line that share a unit also share a model.  Wall clock
    around the blocking C-ABI call (noise generation, token steps, fitness, update, losses D2H)."""
    import time
    gcfg = pkg.default_gru_config()
    ctx = pkg.GruContext(gcfg, device)
    ctx.upload_model(synth.uniform_int8(0, pkg.gru_model_bytes(gcfg)))
    ctx.set_dataset(synth.zipf_bytes(1, 1 << 20))
    ctx.generation(SEED0, 0, 32, True)                    # warm-up: graph capture
    n0 = ctx.launch_count()
    t0 = time.perf_counter()
    for r in range(reps):
        ctx.generation(SEED0 + 1 + r, (r + 1) * gcfg.seq_len, tokens, True)
    dt = (time.perf_counter() - t0) / reps
    launches = (ctx.launch_count() - n0) // reps
    ctx.close()
    return {"value": gcfg.population_size * tokens / dt, "unit": UNIT, "ms_per_generation_sample": dt * 1e3,
            "sample": "%d members x %d tokens per generation (the reference runs 4096 tokens), update included" % (gcfg.population_size, tokens),
            "gpu_launches": int(launches), "timing": "wall clock around the blocking call"}


def projection_ops_per_member_token(H, L, V):
    return 2.0 * (8 * H * H + 12 * H * H * L + H * V)


def c5_sample_run(pkg, synth, device, members, peaks, mma_loop_tops, steps=2, fused=2):
    """d-eggs-scale shapes on one GPU: `members` members of the 262 144-member population evaluated (the evaluation
    is linear in the members), then the whole Muon update over all 131 072 pairs from a seeded ternary fitness vector.
    Gives the two times that decide how a fixed population of 262 144 scales over 8 GPUs: evaluation shards, the
    update is replicated."""
    pop = 262144
    cfg = pkg.default_config(population_size=pop, use_muon=1, **C5)
    ctx = pkg.Context(cfg, device, members)
    ctx.set_fused_epilogues(fused)           # level: 0 two-kernel, 1 row-owning projections, 2 + norm inside MLP-down
    fused_active = ctx.fused_epilogues_active()
    ctx.upload_model(synth.random_model(cfg, 0, "ternary"))
    ctx.set_dataset(synth.zipf_bytes(1, 1 << 24))
    rng = np.random.default_rng(5)
    ctx.write_fitness(rng.integers(-1, 2, pop // 2).astype(np.int32), 0)
    S = cfg.seq_len
    ctx.eval_chunk(42, 0, 0, members)
    ctx.apply_update(42, 0.5)
    ctx.sync()
    ctx.profile_enable(True)
    ctx.profile_read()
    ev, up = [], []
    for i in range(steps):
        ctx.timer_start(); ctx.eval_chunk(43 + i, (1 + i) * S, 0, members); ev.append(ctx.timer_stop())
        ctx.timer_start(); ctx.apply_update(43 + i, 0.5); up.append(ctx.timer_stop())
    prof = ctx.profile_read()
    ctx.profile_enable(False)
    ctx.close()
    eval_ms, upd_ms = float(np.mean(ev)), float(np.mean(up))
    gemm_ms = sum(prof[k][0] for k in prof if k.startswith("gemm_")) / steps
    ops = projection_ops_per_member_token(cfg.hidden_dim, cfg.n_layers, cfg.vocab_size) * members * S
    tops = ops / (gemm_ms / 1e3) / 1e12 if gemm_ms > 0 else None
    per_gpu_members = pop // 8
    t_eval_8 = eval_ms * per_gpu_members / members
    t_eval_1 = eval_ms * pop / members
    return {"workload": "12 layers, H 1024, 16 heads, seq 512, ternary weight values, Muon; %d of 262144 members evaluated, update over "
                        "all 131072 pairs" % members,
            "adaptive_norms": {0: "two-kernel form", 1: "fused into the projection epilogues (row-owning kernels on pairs of thread blocks)",
                               2: "fused into the projection epilogues (row-owning kernels on pairs of thread blocks), the next mean-abs norm inside MLP-down",
                               3: "fused into the projection epilogues (row-owning kernels on pairs of thread blocks), every mean-abs norm inside the projection before it"}[fused_active],
            "eval_member_tokens_per_s": members * S / (eval_ms / 1e3), "eval_ms": eval_ms, "update_ms": upd_ms,
            # summed over the two side streams the matrices alternate on: two run at a time, so this exceeds its share of update_ms
            "newton_schulz_and_apply_ms_summed_over_streams": prof.get("muon", (0.0, 0))[0] / steps,
            "update_gemm_ms": prof.get("update_gemm", (0.0, 0))[0] / steps,
            "update_operands_ms": prof.get("update_operands", (0.0, 0))[0] / steps,
            "projection_tops": tops, "projection_frac_of_peak": (tops / peaks["tensor"]) if tops else None,
            "projection_frac_of_mma_loop": (tops / mma_loop_tops) if (tops and mma_loop_tops) else None,
            "implied_generation_ms": {"1_gpu": t_eval_1 + upd_ms, "8_gpus": t_eval_8 + upd_ms},
            "implied_8gpu_efficiency_fixed_population": (t_eval_1 + upd_ms) / (8.0 * (t_eval_8 + upd_ms)),
            "implied_8gpu_eval_share": t_eval_8 / (t_eval_8 + upd_ms),
            "kernels_ms": {k: v[0] / steps for k, v in prof.items() if v[1] > 0}}


# ----------------------------------------------------------------------------- isolated workloads (one GPU)
def run_c3(args, pkg, synth, torch, real_stdout, peaks):
    """Isolated perturbed projection at the size BASELINE names: y = clip((x.W + ((x.b) a ns >> 7)) >> 8)."""
    K = N = 4096
    rpm, members = 64, 4096
    rows = rpm * members
    cfg = pkg.default_config(device_mask=3)
    ctx = pkg.Context(cfg, 0, 2)
    g = torch.Generator(device="cuda"); g.manual_seed(3)
    x = torch.empty((rows, K), dtype=torch.int8, device="cuda")
    for r0 in range(0, rows, 16384):
        x[r0:r0 + 16384] = torch.clamp(torch.round(torch.randn((16384, K), generator=g, device="cuda") * 32.0), -127, 127).to(torch.int8)
    w = synth.uniform_int8(0, K * N)
    d_w = torch.from_numpy(w).cuda()
    y = torch.zeros((rows, N), dtype=torch.int8, device="cuda")
    x_host = torch.empty((rows, K), dtype=torch.int8).pin_memory(); x_host.copy_(x)
    y_host = torch.empty((rows, N), dtype=torch.int8).pin_memory()
    torch.cuda.synchronize()

    def step(host):
        if host:
            ctx.perturbed_projection(x_host.numpy(), w, y_host.numpy(), rows, K, N, rpm, 7, 200, 201, 7, 8)
        else:
            ctx.perturbed_projection(x.data_ptr(), d_w.data_ptr(), y.data_ptr(), rows, K, N, rpm, 7, 200, 201, 7, 8, on_device=True)

    n_warm = max(args.warmup, 3)
    for _ in range(n_warm):
        step(False)
    l0 = ctx.launch_count()
    sampler = ClockSampler(0); sampler.start()
    ctx.timer_start()
    for _ in range(args.steps):
        step(False)
    ms = ctx.timer_stop() / args.steps
    clocks = sampler.stop()
    launches = ctx.launch_count() - l0
    step(True)
    ctx.timer_start()
    for _ in range(args.steps):
        step(True)
    ms_e2e = ctx.timer_stop() / args.steps
    ops = 2.0 * rows * K * N
    achieved = ops / (ms / 1e3) / 1e12
    line = {"metric": METRIC, "value": rows / (ms / 1e3), "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": n_warm, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8/int32", "data": "synthetic",
            "config": {"workload": "c3: isolated perturbed int8 projection, W 4096x4096, 4096 members x 64 tokens = 262144 rows, noise in [-3,3], "
                                   ">>8 and clip; the step includes the weight transpose, the pair noise table and the row dots x.b",
                       "l2_policy": "inputs larger than L2 (x 1 GiB, y 1 GiB)"},
            "e2e": {"value": rows / (ms_e2e / 1e3), "unit": UNIT, "ms_per_step": ms_e2e, "h2d_bytes_per_step": int(rows * K + K * N),
                    "d2h_bytes_per_step": int(rows * N)},
            "gpu_launches": int(launches),
            "roofline": {"kernel": "gemm_i8_kernel<EPI_CLIP8> (whole call: transpose + noise + dots + GEMM)", "bound": "tensor", "achieved": achieved,
                         "peak": peaks["tensor"], "unit": "TFLOP/s", "frac": achieved / peaks["tensor"], "traffic": None,
                         "peak_source": peaks["tensor_source"]},
            "clocks": clocks, "cpu_baseline": None}
    real_stdout.write(json.dumps(line) + "\n"); real_stdout.flush()
    ctx.close()


def run_c4(args, pkg, synth, torch, real_stdout, peaks):
    """Isolated update of a 4096 x 4096 weight from 65 536 members (32 768 pairs, int8 rank-normalised fitness, noise in
    [-3, 3] regenerated from the counter hash): one step = the whole ES-AdamW update (operands, vote GEMM, element step)
    followed by the whole Muon update (operands, vote GEMM, momentum, 5 Newton-Schulz iterations, quantised apply)."""
    R = Cn = 4096
    pairs = 32768
    cfg = pkg.default_config(device_mask=3, population_size=2 * pairs, use_muon=1)
    ctx = pkg.Context(cfg, 0, 2)
    rng = np.random.RandomState(2)
    rank = np.argsort(np.argsort(rng.randn(pairs)))
    fit = np.clip(np.round(rank / (pairs - 1) * 254.0 - 127.0), -127, 127).astype(np.int32)
    w0 = synth.uniform_int8(0, R * Cn)
    d_w = torch.from_numpy(w0.copy()).cuda()
    d_adam = torch.zeros(R * Cn * 3, dtype=torch.float32, device="cuda")
    d_muon = torch.zeros(R * Cn * 2, dtype=torch.float32, device="cuda")
    d_fit = torch.from_numpy(fit).cuda()
    fit_host = torch.from_numpy(fit).pin_memory()
    torch.cuda.synchronize()
    seed = [2]

    def step(host):
        if host:
            d_fit.copy_(fit_host, non_blocking=False)
        seed[0] += 1
        n1 = ctx.update_matrix(d_w.data_ptr(), d_adam.data_ptr(), R, Cn, 402, 403, 1000, d_fit.data_ptr(), pairs, seed[0], LR, optimizer=0, split=True)
        n2 = ctx.update_matrix(d_w.data_ptr(), d_muon.data_ptr(), R, Cn, 402, 403, 1000, d_fit.data_ptr(), pairs, seed[0], LR, optimizer=1, split=True)
        return n1 + n2

    n_warm = max(args.warmup, 3)
    for _ in range(n_warm):
        step(False)
    l0 = ctx.launch_count()
    ctx.profile_enable(True); ctx.profile_read()
    sampler = ClockSampler(0); sampler.start()
    ctx.timer_start()
    for _ in range(args.steps):
        step(False)
    ms = ctx.timer_stop() / args.steps
    clocks = sampler.stop()
    prof = ctx.profile_read(); ctx.profile_enable(False)
    launches = ctx.launch_count() - l0
    ctx.timer_start()
    for _ in range(args.steps):
        step(True)
    ms_e2e = ctx.timer_stop() / args.steps
    k = {n: v[0] / args.steps for n, v in prof.items() if v[1] > 0}
    vote_ops = 2.0 * R * Cn * pairs                         # algorithmic ops of ONE reconstruction (two per step)
    gemm_ms = k.get("update_gemm", 0.0) / 2.0
    achieved = vote_ops / (gemm_ms / 1e3) / 1e12 if gemm_ms > 0 else None
    ns_flop = 5.0 * 2 * 2 * float(R) * R * Cn                # 5 iterations x (Gram + product), 2*K*K*L flop each
    line = {"metric": "member_updates_per_sec", "value": 2 * pairs / (ms / 1e3), "unit": "members/s", "n_gpus": 1, "steps": args.steps,
            "warmup": n_warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8/int32 votes, fp32 optimiser", "data": "synthetic",
            "config": {"workload": "c4: isolated update of a 4096x4096 weight, 65536 members = 32768 pairs, int8 rank-normalised fitness (two-digit "
                                   "operand split: executed contraction 65536), noise in [-3,3]; step = ES-AdamW update + Muon update (5 Newton-Schulz)",
                       "l2_policy": "operands (2 x 268 MB) and votes (64 MiB) exceed L2 together"},
            "e2e": {"value": 2 * pairs / (ms_e2e / 1e3), "unit": "members/s", "ms_per_step": ms_e2e, "h2d_bytes_per_step": int(pairs * 4),
                    "d2h_bytes_per_step": 16},
            "gpu_launches": int(launches),
            "roofline": {"kernel": "gemm_i8_kernel<EPI_VOTE> (vote reconstruction)", "bound": "tensor", "achieved": achieved, "peak": peaks["tensor"],
                         "unit": "TFLOP/s", "frac": (achieved / peaks["tensor"]) if achieved else None, "traffic": None,
                         "peak_source": peaks["tensor_source"],
                         "note": "algorithmic ops 2*4096*4096*32768 per reconstruction; the operand split executes twice that"},
            "kernels_ms_per_step": k,
            "newton_schulz": {"ms": k.get("muon", 0.0), "tflops_fp32": ns_flop / (k["muon"] / 1e3) / 1e12 if k.get("muon") else None,
                              "note": "5 iterations of G = X X^T, X <- 0.5 (3I - G) X in fp32 FFMA, plus normalise and quantised apply"},
            "clocks": clocks, "cpu_baseline": None}
    real_stdout.write(json.dumps(line) + "\n"); real_stdout.flush()
    ctx.close()


def run_c5slice(args, pkg, synth, torch, real_stdout, peaks):
    members = 256 if args.small else 2048        # --small: a profiler-sized case (131 072 rows, activations still beyond L2)
    ctx0 = pkg.Context(pkg.default_config(**C2), 0, 2)
    mma = ctx0.measure_int8_peak(16384, 2048, 2048, 20)
    ctx0.close()
    sampler = ClockSampler(0); sampler.start()
    r = c5_sample_run(pkg, synth, 0, members, peaks, mma, steps=max(1, args.steps), fused=0 if args.two_kernel_norm else args.fused_level)
    clocks = sampler.stop()
    S = C5["seq_len"]
    gen_ms = r["eval_ms"] + r["update_ms"]
    line = {"metric": METRIC, "value": members * S / (gen_ms / 1e3), "unit": UNIT, "n_gpus": 1, "steps": max(1, args.steps), "warmup": 1,
            "ms_per_step": gen_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8/int32", "data": "synthetic",
            "config": {"workload": "c5slice: " + r["workload"], "l2_policy": "inputs larger than L2"},
            "e2e": None, "gpu_launches": None,
            "roofline": {"kernel": "gemm_fused_kernel + gemm_i8_kernel (all projection epilogues)", "bound": "tensor", "achieved": r["projection_tops"],
                         "peak": peaks["tensor"], "unit": "TFLOP/s", "frac": r["projection_frac_of_peak"], "traffic": None,
                         "peak_source": peaks["tensor_source"]},
            "c5_sample": r, "clocks": clocks, "cpu_baseline": None}
    real_stdout.write(json.dumps(line) + "\n"); real_stdout.flush()


def run_tok(args, pkg, synth, torch, real_stdout, peaks):
    """One ES-AdamW generation of the benchmark shapes with the tokenizer build's vocabulary (VOCAB_SIZE != 256:
    uint32 tokens, embedding and tied head over V columns, two-pass cross-entropy)."""
    V = args.vocab
    pop = 1024 if args.small else (args.pop if args.pop != POP_PER_GPU else 8192)
    kw = dict(C2); kw["vocab_size"] = V; kw["ntt_mode"] = args.ntt_mode
    cfg = pkg.default_config(population_size=pop, **kw)
    ctx = pkg.Context(cfg, 0, args.wave)
    ctx.set_fused_epilogues(args.fused_level)
    ctx.upload_model(synth.random_model(cfg, 0, "uniform"))
    data = synth.zipf_tokens(1, 1 << 22, V) if V != 256 else synth.zipf_bytes(1, 1 << 22)
    ctx.set_dataset(data)
    S = cfg.seq_len
    steps, warm = max(1, args.steps), max(1, args.warmup)
    for i in range(warm):
        ctx.eval_chunk(SEED0 + i, i * S, 0, pop); ctx.compute_fitness_pairs(0, pop // 2); ctx.apply_update(SEED0 + i, LR)
    ctx.sync()
    ctx.profile_enable(True); ctx.profile_read()
    sampler = ClockSampler(0); sampler.start()
    ev, up = [], []
    for i in range(steps):
        ctx.timer_start(); ctx.eval_chunk(SEED0 + warm + i, (warm + i) * S, 0, pop); ctx.compute_fitness_pairs(0, pop // 2); ev.append(ctx.timer_stop())
        ctx.timer_start(); ctx.apply_update(SEED0 + warm + i, LR); up.append(ctx.timer_stop())
    clocks = sampler.stop()
    prof = ctx.profile_read()
    ctx.profile_enable(False)
    wave = ctx.wave_members()
    ctx.close()
    eval_ms, upd_ms = float(np.mean(ev)), float(np.mean(up))
    gen_ms = eval_ms + upd_ms
    kern = {k: v[0] / steps for k, v in prof.items() if v[1] > 0}
    gemm_ms = sum(v for k, v in kern.items() if k.startswith("gemm_"))
    ops = projection_ops_per_member_token(cfg.hidden_dim, cfg.n_layers, V) * pop * S
    # the head's own stream: int32 logits written by the projection and read once by the cross-entropy pass
    head_bytes = 2.0 * pop * S * V * 4
    head_ms = kern.get("gemm_head", 0.0)
    line = {"metric": METRIC, "value": pop * S / (gen_ms / 1e3), "unit": UNIT, "n_gpus": 1, "steps": steps, "warmup": warm,
            "ms_per_step": gen_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8/int32", "data": "synthetic",
            "config": {"workload": "tok: Int8NativeFormer generation with the tokenizer build's vocabulary: L=4 H=512 seq=256 vocab=%d, uint32 tokens, "
                                   "%d members, rank-1 noise mask 3%s" % (V, pop, (", transformed-window variant NTT_MODE %d" % args.ntt_mode) if args.ntt_mode else ""),
                       "wave_members": wave, "l2_policy": "inputs larger than L2"},
            "e2e": None, "gpu_launches": None,
            "roofline": {"kernel": "head projection (logits epilogue) + head_loss_kernel", "bound": "hbm", "achieved": head_bytes / (head_ms / 1e3) / 1e9 if head_ms else None,
                         "peak": peaks["hbm"], "unit": "GB/s", "frac": (head_bytes / (head_ms / 1e3) / 1e9 / peaks["hbm"]) if head_ms else None,
                         "traffic": None, "peak_source": peaks["hbm_source"],
                         "algorithmic_bytes": "rows x vocab x 4 B written by the projection + the same read by the cross-entropy pass"},
            "eval_ms": eval_ms, "update_ms": upd_ms, "head_ms": head_ms,
            "projection_tops": ops / (gemm_ms / 1e3) / 1e12 if gemm_ms else None,
            "kernels_ms": kern, "clocks": clocks, "cpu_baseline": None}
    real_stdout.write(json.dumps(line) + "\n"); real_stdout.flush()


# ----------------------------------------------------------------------------- our arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--workload", default="c2", choices=["c2", "c3", "c4", "c5slice", "c5", "tok"])
    ap.add_argument("--vocab", type=int, default=8192, help="workload tok: vocabulary size (a multiple of 256)")
    ap.add_argument("--ntt-mode", type=int, default=0, choices=[0, 1, 2, 3], help="workload tok: the reference's NTT_MODE (transformed input window, three more embedding tables)")
    ap.add_argument("--pop-total", type=int, default=262144, help="workload c5: the fixed population that is sharded over the GPUs")
    ap.add_argument("--pop", type=int, default=POP_PER_GPU, help="members per GPU (benchmark value: 40960)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the extra legs of the default line (recurrent model, reference GPU kernels, C5 sample)")
    ap.add_argument("--two-kernel-norm", action="store_true", help="A/B: take the two-kernel form of the adaptive normalisations (int32 pre-activations + requantisation kernels)")
    ap.add_argument("--fused-level", type=int, default=2, choices=[0, 1, 2, 3],
                    help="A/B: 0 two-kernel adaptive norms, 1 row-owning projections, 2 (default) also the next mean-abs norm inside the MLP-down epilogue")
    ap.add_argument("--attention-tc", type=int, nargs="?", const=1, default=None, choices=[0, 1, 2],
                    help="A/B: attention kernel: 0 mma.sync, 1 tcgen05 scores and sums, 2 mma.sync scores + tcgen05 sums (default: the library's)")
    ap.add_argument("--replicated-update", action="store_true", help="N > 1: repeat the whole update on every GPU as the reference does (default: shard it by matrix)")
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
        args.pop, args.no_cpu_baseline, args.no_extras = 1024, True, True

    # libraries (NCCL's version banner, for one) may write to stdout: keep fd 1 for the single JSON line
    real_stdout = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)

    import torch   # device discovery and the process group only; the hot path is the C ABI
    pkg = load_pkg()
    from egg_c_b200 import synth
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: the library has no CPU path")
    peaks = load_peaks()
    if args.workload not in ("c2", "c5"):
        if world > 1:
            if rank == 0:
                raise SystemExit("workload %s is a single-GPU measurement" % args.workload)
            return
        if args.workload == "c3":
            return run_c3(args, pkg, synth, torch, real_stdout, peaks)
        if args.workload == "c4":
            return run_c4(args, pkg, synth, torch, real_stdout, peaks)
        if args.workload == "tok":
            return run_tok(args, pkg, synth, torch, real_stdout, peaks)
        return run_c5slice(args, pkg, synth, torch, real_stdout, peaks)

    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    strong = args.workload == "c5"
    if strong:
        pop = args.pop_total                     # strong scaling: the fixed population of the d-eggs-scale configuration
        cfg = pkg.default_config(population_size=pop, use_muon=1, **C5)
        args.no_extras = True
    else:
        pop = args.pop * world                   # weak scaling: fixed members per GPU
        cfg = pkg.default_config(population_size=pop, **C2)
    ctx = pkg.Context(cfg, local_rank, args.wave)
    ctx.set_fused_epilogues(0 if args.two_kernel_norm else args.fused_level)
    if args.attention_tc is not None:
        ctx.set_attention_tensor_core(args.attention_tc)
    fused_active = ctx.fused_epilogues_active()
    model = synth.random_model(cfg, 0, "ternary" if strong else "uniform")
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
        if not args.replicated_update:
            ctx.set_update_sharding(True)      # every matrix stepped by one rank, new weights broadcast over NVLink

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

    step_no = [0]

    def one_step(host_io):
        s = step_no[0]
        step_no[0] += 1
        if host_io:
            return ctx.generation_host(data_host, s, SEED0 + s, LR, losses_host)
        return ctx.generation_host(None, s, SEED0 + s, LR, None)

    # ---- kernel-resident timing (inputs already in HBM) ----
    n_warm = args.warmup if (args.small or strong) else max(args.warmup, 3)
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

    # ---- replicas: every rank must hold byte-identical weights and optimiser state after the same generations
    # (with the sharded update download_opt_state first collects every matrix's state from its owner) ----
    crc_model = zlib.crc32(ctx.download_model().tobytes())
    crc_opt = zlib.crc32(ctx.download_opt_state().tobytes())
    replicas_identical = None
    if dist:
        t = torch.tensor([crc_model, crc_opt], dtype=torch.int64, device="cuda")
        allc = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(allc, t)
        replicas_identical = all(bool(torch.equal(a, allc[0])) for a in allc)

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
        # two-kernel form: 4H of int32 in, H + H out per row; fused form: the int8 stream in, the normalised row out
        # (level 2: the norm after every MLP block runs inside the MLP-down epilogue, L + 1 launches per wave remain)
        "rowwise": (2.0 if fused_active else 6.0) * H * rows_per_step * ((L + 1) if fused_active == 2 else (2 * L + 2)),
        "aqn": 15.0 * H * rows_per_step * L,
    }
    traffic_per_row, traffic_src = load_traffic()
    hbm_peak, tensor_peak = peaks["hbm"], peaks["tensor"]
    rows_per_launch = min(ctx.wave_members(), per) * S

    def class_roofline(k):
        t_ms, n_launch = prof[k]
        if k in gemm_ops:
            achieved = gemm_ops[k] * args.steps / (t_ms / 1e3) / 1e12
            r = {"kernel": k, "bound": "tensor", "achieved": achieved, "peak": tensor_peak, "unit": "TFLOP/s", "frac": achieved / tensor_peak}
        else:
            achieved = hbm_bytes[k] * args.steps / (t_ms / 1e3) / 1e9
            r = {"kernel": k, "bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak}
            if r["frac"] > 1.0:
                r["note"] = "above the DRAM copy figure: part of this kernel's bytes are served from L2"
        r["avg_launch_ms"] = t_ms / max(1, n_launch)
        r["traffic"] = traffic_per_row[k] * rows_per_launch if k in traffic_per_row else None
        return r

    per_class = [class_roofline(k) for k in prof if prof[k][1] > 0 and (k in gemm_ops or k in hbm_bytes)]
    # The dominant kernel is the one __global__ function with the largest share of the step: the projection GEMM
    # (gemm_i8_kernel, four epilogue instantiations) counts as one kernel, the row-wise kernels each as their own.
    gemm_keys = [k for k in gemm_ops if k in prof and prof[k][1] > 0]
    gemm_ms = sum(prof[k][0] for k in gemm_keys)
    gemm_launches = sum(prof[k][1] for k in gemm_keys)
    others = [k for k in hbm_bytes if k in prof and prof[k][1] > 0]
    top_other = max(others, key=lambda k: prof[k][0]) if others else None

    # what the GEMM's own TMA + tcgen05 loop sustains on this GPU with the accumulators dropped (operands in L2)
    mma_loop_tops = None
    if rank == 0 and not args.small:
        try:
            mma_loop_tops = ctx.measure_int8_peak(16384, 2048, 2048, 20)
        except Exception:
            mma_loop_tops = None

    if gemm_keys and (top_other is None or gemm_ms >= prof[top_other][0]):
        achieved = sum(gemm_ops[k] for k in gemm_keys) * args.steps / (gemm_ms / 1e3) / 1e12
        known = [k for k in gemm_keys if k in traffic_per_row]
        roof = {"kernel": "gemm_fused_kernel + gemm_i8_kernel (all projection epilogues)", "bound": "tensor", "achieved": achieved, "peak": tensor_peak,
                "unit": "TFLOP/s", "frac": achieved / tensor_peak,
                "frac_of_mma_loop_measured": (achieved / mma_loop_tops) if mma_loop_tops else None,
                "mma_loop_tops_measured": mma_loop_tops,
                "traffic": (sum(traffic_per_row[k] * rows_per_launch * prof[k][1] for k in known) / max(1, sum(prof[k][1] for k in known)))
                if known else None,
                "peak_source": peaks["tensor_source"],
                "avg_launch_ms": gemm_ms / max(1, gemm_launches), "share_of_step": None,
                "traffic_source": (traffic_src + "; launch-weighted mean over the projection instantiations") if traffic_src else None}
    else:
        roof = class_roofline(top_other)
        roof["peak_source"] = peaks["hbm_source"]
        roof["traffic_source"] = traffic_src
    total_prof = sum(v[0] for v in prof.values()) or 1.0
    kernel_share = {k: {"ms_per_step": v[0] / args.steps, "launches_per_step": v[1] / args.steps, "share": v[0] / total_prof}
                    for k, v in prof.items() if v[1] > 0}
    roof["share_of_step"] = (gemm_ms if roof["bound"] == "tensor" else prof[top_other][0]) / total_prof
    gemm_total_ms = sum(prof[k][0] for k in gemm_ops if k in prof)
    gemm_tops = sum(gemm_ops.values()) * args.steps / (gemm_total_ms / 1e3) / 1e12 if gemm_total_ms > 0 else None
    step_tops = sum(gemm_ops.values()) / (ms_per_step / 1e3) / 1e12

    wave_members = ctx.wave_members()
    ctx.close()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            cpu = cpu_reference_run(1, 0)
        except Exception as e:   # the baseline is reported, never allowed to break the bench line
            cpu = {"value": None, "unit": UNIT, "cores": host_cores(), "kind": "reference", "sample": "failed: %s" % e}

    gru = ref_gpu = c5 = None
    if rank == 0 and world == 1 and not args.no_extras:
        try:
            gru = gru_model_run(pkg, synth, local_rank)
        except Exception as e:
            gru = {"value": None, "unit": UNIT, "sample": "failed: %s" % e}
        try:
            ref_gpu = reference_gpu_kernels_run()
        except Exception as e:
            ref_gpu = {"value": None, "unit": UNIT, "sample": "failed: %s" % e}
        try:
            c5 = c5_sample_run(pkg, synth, local_rank, 512, peaks, mma_loop_tops)
        except Exception as e:
            c5 = {"workload": "failed: %s" % e}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": n_warm,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": "int8/int32",
            "data": "synthetic",
            "config": {"workload": ("c5: d-eggs-scale generation, L=12 H=1024 heads=16 MLP=4H seq=512 vocab=256, ternary weight values, Muon, "
                                    "fixed population sharded over the GPUs") if strong else WORKLOAD, "population_size": pop, "members_per_gpu": per, "seq_len": S, "hidden_dim": H,
                       "n_layers": L, "wave_members": wave_members, "dataset_bytes": DATA_LEN,
                       "adaptive_norms": {0: "two-kernel form", 1: "fused into the projection epilogues (row-owning kernels)",
                                          2: "fused into the projection epilogues (row-owning kernels), the next mean-abs norm inside MLP-down",
                                          3: "fused into the projection epilogues (row-owning kernels), every mean-abs norm inside the projection before it"}[fused_active],
                       "l2_policy": "inputs larger than L2: each wave streams > 2 GB of activations, dataset 64 MiB",
                       "parallelism": ("population sharded, pair-aligned; one NCCL all-gather of fitness per generation; " +
                                       ("update replicated on every GPU" if (world == 1 or args.replicated_update) else
                                        "update sharded by matrix, new weights by grouped ncclBroadcast"))},
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e, "h2d_bytes_per_step": int(DATA_LEN),
                    "d2h_bytes_per_step": int(per * 4 + 8)},
            "gpu_launches": int(launches),
            "roofline": roof,
            "rooflines_by_class": per_class,
            "projection_gemms": {"tops": gemm_tops, "frac_of_peak": (gemm_tops / tensor_peak) if gemm_tops else None, "peak": tensor_peak,
                                 "mma_loop_tops_measured": mma_loop_tops,
                                 "frac_of_mma_loop": (gemm_tops / mma_loop_tops) if (gemm_tops and mma_loop_tops) else None,
                                 "whole_step_tops": step_tops, "whole_step_frac_of_peak": step_tops / tensor_peak},
            "kernels": kernel_share,
            "clocks": clocks,
            "replicas_identical": replicas_identical,
            "replica_crc32": {"model": crc_model, "optimizer_state": crc_opt},
            "cpu_baseline": cpu,
            "gru_model_gpu": gru,
            "reference_gpu_kernels": ref_gpu,
            "c5_sample": c5,
        }
        real_stdout.write(json.dumps(line) + "\n")
        real_stdout.flush()
    if dist:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
