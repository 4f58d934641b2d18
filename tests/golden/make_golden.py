"""Regenerates the committed golden vectors.

  python tests/golden/make_golden.py kat      (CPU: runs oracle/_ref/ref_kat, the
                                               reference's egg_math.h / ternary_pack.h)
  python tests/golden/make_golden.py mgpu     (on a B200: runs oracle/_ref/ref_mgpu_*, the
                                               reference's own kernels, on seeded cases)
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
    ref = "/root/reference/d-eggs/include"
    src = os.path.join(ROOT, "oracle", "ref_kat.cpp")
    for mask in (15, 3):
        exe = "/tmp/ref_kat_mask%d" % mask
        subprocess.run(["g++", "-O1", "-DDEVICE_MASK=%d" % mask, "-I" + ref, "-o", exe, src], check=True)
        out = subprocess.run([exe], check=True, capture_output=True, text=True).stdout
        json.loads(out)
        open(os.path.join(HERE, "rng_kat_mask%d.json" % mask), "w").write(out)
        print("wrote rng_kat_mask%d.json" % mask)


def mgpu(outdir):
    from common import REF_CONFIGS, make_case, run_ref_mgpu
    os.makedirs(outdir, exist_ok=True)
    for tag in ("tiny", "small", "muon_tiny"):
        kw = REF_CONFIGS[tag]
        cfg, ocfg, model, data = make_case(kw, data_len=50000)
        pop = kw["population_size"]
        r = run_ref_mgpu(tag, model, data, 0x00C0FFEE, 0, 0, pop, lr=0.5, do_update=True)
        changed = np.nonzero(r["model"] != model)[0]
        np.savez_compressed(os.path.join(outdir, "ref_mgpu_%s.npz" % tag), losses=r["losses"], fitness=r["fitness"],
                            updates=np.uint64(r["updates"]), changed_idx=changed.astype(np.int64),
                            changed_val=r["model"][changed], opt_crc=np.uint32(0),
                            opt_sample=r["opt"].view(np.float32)[:: max(1, len(r["opt"]) // 4 // 4096)][:4096])
        print("wrote", tag, r["info"])


if __name__ == "__main__":
    if sys.argv[1] == "kat":
        kat()
    else:
        mgpu(sys.argv[2] if len(sys.argv) > 2 else os.path.join(ROOT, "gpurun_out", "golden"))
