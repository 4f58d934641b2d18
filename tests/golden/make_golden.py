"""Regenerates the committed golden vectors.

  python tests/golden/make_golden.py kat      (CPU: runs oracle/_ref/ref_kat, the
                                               reference's egg_math.h / ternary_pack.h)
  python tests/golden/make_golden.py mgpu     (on a B200: runs oracle/_ref/ref_mgpu_*, the
                                               reference's own kernels, on seeded cases; the tok_* cases
                                               are its tokenizer build, VOCAB_SIZE 1024 / 512, uint32 tokens;
                                               the ntt* cases its NTT_MODE 1 / 2 / 3 builds)
  python tests/golden/make_golden.py deggs    (on a B200: runs oracle/_ref/ref_deggs_*, the d-eggs
                                               worker's kernels with adaptive-noise overlays)
  python tests/golden/make_golden.py muon     (on a B200: one Muon step of oracle/_ref/ref_mgpu_muon_*, the
                                               reference's cuBLAS Newton-Schulz, with sampled fp32 state)
  python tests/golden/make_golden.py worker   (CPU: oracle/_ref/ref_worker_fitness, lines 635-687 of the
                                               reference's d-eggs/src/worker.cu compiled unmodified)
  python tests/golden/make_golden.py gru      (CPU, minutes: oracle/_ref/ref_cpu_gru, one generation of
                                               full_trained_egg.c at its compiled-in size, 128 x 4096 tokens)
  python tests/golden/make_golden.py generate (on a B200: the d-eggs generate_sequence_kernel through
                                               the same harness binaries)
"""
import json
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "tests"))


def kat():
    ref = os.path.join(os.environ.get("EGG_REFERENCE", "/root/reference"), "d-eggs", "include")
    src = os.path.join(ROOT, "oracle", "ref_kat.cpp")
    for mask in (15, 3):
        exe = "/tmp/ref_kat_mask%d" % mask
        subprocess.run(["g++", "-O1", "-DDEVICE_MASK=%d" % mask, "-I" + ref, "-o", exe, src], check=True)
        out = subprocess.run([exe], check=True, capture_output=True, text=True).stdout
        json.loads(out)
        open(os.path.join(HERE, "rng_kat_mask%d.json" % mask), "w").write(out)
        print("wrote rng_kat_mask%d.json" % mask)


GOLD_STEPS = 4
GOLD_SEED = 0x00C0FFEE
GOLD_LR = 0.5


def mgpu(outdir):
    """Four chained generations (eval -> host fitness -> update) of the reference's own kernels per
    configuration; weights only start to flip after a few AdamW steps."""
    import zlib
    from common import REF_CONFIGS, make_case, run_ref_mgpu
    os.makedirs(outdir, exist_ok=True)
    only = os.environ.get("EGG_GOLDEN_TAGS")       # e.g. "tok_tiny,tok_small": regenerate a subset
    for tag in ("tiny", "small", "muon_tiny", "tok_tiny", "tok_small", "ntt1_tiny", "ntt2_tiny", "ntt3_small"):
        if only and tag not in only.split(","):
            continue
        kw = REF_CONFIGS[tag]
        cfg, ocfg, model0, data = make_case(kw, data_len=50000)
        pop, S = kw["population_size"], kw["seq_len"]
        model, opt = model0.copy(), None
        losses, fits, ups = [], [], []
        for step in range(GOLD_STEPS):
            r = run_ref_mgpu(tag, model, data, GOLD_SEED + step, step * S, 0, pop, lr=GOLD_LR, do_update=True, opt_state=opt)
            losses.append(r["losses"]); fits.append(r["fitness"]); ups.append(r["updates"])
            model, opt = r["model"], r["opt"]
        changed = np.nonzero(model != model0)[0]
        np.savez_compressed(os.path.join(outdir, "ref_mgpu_%s.npz" % tag), losses=np.array(losses), fitness=np.array(fits),
                            updates=np.array(ups, np.uint64), changed_count=np.int64(len(changed)),
                            changed_idx=changed[:2048].astype(np.int64), changed_val=model[changed[:2048]],
                            model_crc=np.uint32(zlib.crc32(model.tobytes())), opt_crc=np.uint32(zlib.crc32(opt.tobytes())),
                            opt_head=opt.view(np.float32)[:768].copy())
        print("wrote", tag, "updates", ups, "changed", len(changed))


DEGGS_GENS = 6
DEGGS_SEED = 42
DEGGS_LR = 0.5


def deggs(outdir):
    """Six generations of the d-eggs worker's kernels per configuration, starting from seeded overlays;
    the seed follows the worker's chain seed = hash_rng(seed, step + 1)."""
    import zlib
    from common import DEGGS_CONFIGS, deggs_initial_scales, load_oracle, make_case, run_ref_deggs
    O = load_oracle()
    os.makedirs(outdir, exist_ok=True)
    for tag in ("tiny", "small"):
        kw = DEGGS_CONFIGS[tag]
        cfg, ocfg, model0, data = make_case(kw, data_len=50000)
        opt0 = np.zeros(O.opt_bytes(ocfg), np.uint8)
        scales0 = deggs_initial_scales(O.scales_bytes(ocfg))
        r = run_ref_deggs(tag, model0, opt0, scales0, data, DEGGS_SEED, 0, DEGGS_GENS, DEGGS_LR)
        assert r["sizes"]["model_bytes"] == len(model0) and r["sizes"]["scales_bytes"] == len(scales0)
        model, opt = r["model"], r["opt"]
        changed = np.nonzero(model != model0)[0]
        np.savez_compressed(os.path.join(outdir, "ref_deggs_%s.npz" % tag), losses=np.array(r["losses"]),
                            updates=np.array(r["updates"], np.uint64), scales_final=r["scales"][-1],
                            scales_crc=np.array([zlib.crc32(x.tobytes()) for x in r["scales"]], np.uint32),
                            changed_count=np.int64(len(changed)), changed_idx=changed[:2048].astype(np.int64),
                            changed_val=model[changed[:2048]], model_crc=np.uint32(zlib.crc32(model.tobytes())),
                            opt_crc=np.uint32(zlib.crc32(opt.tobytes())), sizes=json.dumps(r["sizes"]))
        print("wrote", tag, "updates", r["updates"], "changed", len(changed))


def muon(outdir):
    """One Muon generation (eval -> host fitness -> momentum, cuBLAS Newton-Schulz, quantised apply) of the
    reference's kernels from zero state, then a second one from its own outputs.  The fp32 state is far too large
    to commit: a seeded sample of 8192 floats per generation is kept with its indices, plus CRCs and the changed
    weights."""
    import zlib
    from common import REF_CONFIGS, make_case, run_ref_mgpu
    os.makedirs(outdir, exist_ok=True)
    for tag in ("muon_tiny", "muon_small"):
        kw = REF_CONFIGS[tag]
        cfg, ocfg, model0, data = make_case(kw, data_len=50000)
        pop, S = kw["population_size"], kw["seq_len"]
        model, opt = model0.copy(), None
        rec = {"losses": [], "fitness": [], "updates": [], "sample_val": [], "changed_count": [], "changed_idx": [], "changed_val": [],
               "model_crc": []}
        nfl = None
        for step in range(2):
            r = run_ref_mgpu(tag, model, data, GOLD_SEED + step, step * S, 0, pop, lr=GOLD_LR, do_update=True, opt_state=opt)
            fl = r["opt"].view(np.float32)
            if nfl is None:
                nfl = len(fl)
                idx = np.sort(np.random.default_rng(17).choice(nfl, 8192, replace=False))
            changed = np.nonzero(r["model"] != model)[0]
            rec["losses"].append(r["losses"]); rec["fitness"].append(r["fitness"]); rec["updates"].append(r["updates"])
            rec["sample_val"].append(fl[idx].copy()); rec["changed_count"].append(len(changed))
            ci = np.full(4096, -1, np.int64); ci[:min(4096, len(changed))] = changed[:4096]
            cv = np.zeros(4096, np.int8); cv[:min(4096, len(changed))] = r["model"][changed[:4096]]
            rec["changed_idx"].append(ci); rec["changed_val"].append(cv); rec["model_crc"].append(zlib.crc32(r["model"].tobytes()))
            model, opt = r["model"], r["opt"]
        np.savez_compressed(os.path.join(outdir, "ref_muon_step_%s.npz" % tag), sample_idx=idx,
                            **{k: np.array(v) for k, v in rec.items()})
        print("wrote", tag, "updates", rec["updates"], "changed", rec["changed_count"])


def worker():
    """Per-chunk fitness of the reference worker (worker.cu:635-687 compiled unmodified) on seeded loss vectors,
    for the four combinations of CHUNK_MEAN_FILTER and USE_ADAPTIVE_THRESHOLD."""
    exe = os.path.join(ROOT, "oracle", "_ref", "ref_worker_fitness")
    rng = np.random.default_rng(7)
    cases = []
    shapes = [(64, 0), (4096, 37), (4096, -5), (2, 0), (8192, 3), (10, 100000)]
    vectors = [(rng.integers(10000, 20000, n) + bias * (np.arange(n) % 2)).astype(np.int32) for n, bias in shapes]
    vectors.append(np.full(16, 5, np.int32))                      # all pairs tie: the "|diff| < 0" case
    vectors.append(np.array([7, 9, 9, 7, 8, 8, 100, -100], np.int32))
    for li, losses in enumerate(vectors):
        for mf in (0, 1):
            for ad in (0, 1):
                r = subprocess.run([exe, str(mf), str(ad)], input=" ".join(str(int(x)) for x in losses), capture_output=True, text=True, check=True)
                o = json.loads(r.stdout)
                fit = np.array(o["fitness"], np.int32)
                cases.append(dict(vector=li, mean_filter=mf, adaptive=ad, sum_loss=o["sum_loss"],
                                  fitness_packed=np.packbits((fit + 1).astype(np.uint8)[:, None] >> np.array([1, 0]) & 1).tolist(),
                                  pairs=len(fit)))
    json.dump({"shapes": shapes, "rng_seed": 7, "cases": cases}, open(os.path.join(HERE, "ref_worker_fitness.json"), "w"))
    print("wrote ref_worker_fitness.json:", len(cases), "cases")


def worker_vectors():
    """The loss vectors of worker(), regenerated from the seed (kept out of the fixture to keep it small)."""
    rng = np.random.default_rng(7)
    shapes = [(64, 0), (4096, 37), (4096, -5), (2, 0), (8192, 3), (10, 100000)]
    vectors = [(rng.integers(10000, 20000, n) + bias * (np.arange(n) % 2)).astype(np.int32) for n, bias in shapes]
    vectors.append(np.full(16, 5, np.int32))
    vectors.append(np.array([7, 9, 9, 7, 8, 8, 100, -100], np.int32))
    return vectors


def gru():
    """One generation of full_trained_egg.c at its compiled-in size (H 512, 4 layers, 128 members, 4096 tokens,
    threshold-vote update): losses, fitness, CRCs of the post-update weights and recurrent states, changed weights."""
    import zlib
    from common import load_oracle, run_ref_gru
    sys.path.insert(0, os.path.join(ROOT, "egg.c_b200"))
    import synth
    O = load_oracle()
    gcfg = O.make_gru_config()
    model0 = synth.uniform_int8(0, O.gru_model_bytes(gcfg))
    data = synth.zipf_bytes(1, 1 << 20)
    r = run_ref_gru(model0, data, GOLD_SEED, gcfg.seq_len, steps=1)
    changed = np.nonzero(r["model"] != model0)[0]
    np.savez_compressed(os.path.join(HERE, "ref_cpu_gru_full.npz"), losses=r["losses"][0], fitness=r["fitness"][0],
                        changed_count=np.int64(len(changed)), changed_idx=changed[:4096].astype(np.int64),
                        changed_val=r["model"][changed[:4096]], model_crc=np.uint32(zlib.crc32(r["model"].tobytes())),
                        states_crc=np.uint32(zlib.crc32(r["states"].tobytes())), states_head=r["states"][:2048].copy(),
                        info=json.dumps(r["info"]))
    print("wrote ref_cpu_gru_full.npz: changed", len(changed), r["info"])


GEN_CASES = [  # (tag, seed_len, gen_len, model kind, rng seed, temperature, min_p, presence penalty)
    ("tiny", 6, 10, "init", 1041, 0.6, 0.08, 0.2), ("tiny", 6, 10, "random_all", 7, 1.0, 0.0, 0.0),
    ("tiny", 4, 12, "random_all", 99, 0.9, 0.3, 1.5), ("small", 12, 20, "init", 1041, 0.6, 0.08, 0.2),
    ("small", 12, 20, "random_all", 7, 1.0, 0.0, 0.0), ("small", 1, 31, "random_all", 99, 0.9, 0.3, 1.5),
]


def generate(outdir):
    """Sampled continuations of the d-eggs generate_sequence_kernel for seeded models and byte streams."""
    from common import DEGGS_CONFIGS, make_case, run_ref_generate
    os.makedirs(outdir, exist_ok=True)
    out = []
    for tag, sl, gl, kind, seed, temp, mp, pen in GEN_CASES:
        cfg, ocfg, model, data = make_case(DEGGS_CONFIGS[tag], data_len=50000, model_kind=kind, model_seed=5)
        toks = run_ref_generate(tag, model, data[100:100 + sl], gl, seed, temp, mp, pen)
        out.append(dict(tag=tag, seed_len=sl, gen_len=gl, model_kind=kind, seed=seed, temp=temp, min_p=mp, penalty=pen,
                        tokens=[int(x) for x in toks]))
        print(tag, kind, seed, toks[sl:sl + 10])
    json.dump(out, open(os.path.join(outdir, "ref_generate.json"), "w"), indent=0)


if __name__ == "__main__":
    if sys.argv[1] == "generate":
        generate(sys.argv[2] if len(sys.argv) > 2 else os.path.join(ROOT, "golden_out"))
    elif sys.argv[1] == "kat":
        kat()
    elif sys.argv[1] == "muon":
        muon(sys.argv[2] if len(sys.argv) > 2 else os.path.join(ROOT, "golden_out"))
    elif sys.argv[1] == "worker":
        worker()
    elif sys.argv[1] == "gru":
        gru()
    elif sys.argv[1] == "deggs":
        deggs(sys.argv[2] if len(sys.argv) > 2 else os.path.join(ROOT, "golden_out"))
    else:
        mgpu(sys.argv[2] if len(sys.argv) > 2 else os.path.join(ROOT, "golden_out"))
