"""Regenerates the committed golden vectors.

  python tests/golden/make_golden.py kat      (CPU: runs oracle/_ref/ref_kat, the
                                               reference's egg_math.h / ternary_pack.h)
  python tests/golden/make_golden.py mgpu     (on a B200: runs oracle/_ref/ref_mgpu_*, the
                                               reference's own kernels, on seeded cases)
  python tests/golden/make_golden.py deggs    (on a B200: runs oracle/_ref/ref_deggs_*, the d-eggs
                                               worker's kernels with adaptive-noise overlays)
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
    for tag in ("tiny", "small", "muon_tiny"):
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
    elif sys.argv[1] == "deggs":
        deggs(sys.argv[2] if len(sys.argv) > 2 else os.path.join(ROOT, "golden_out"))
    else:
        mgpu(sys.argv[2] if len(sys.argv) > 2 else os.path.join(ROOT, "golden_out"))
