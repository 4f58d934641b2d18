"""Checkpoint files in the reference's format (save_checkpoint / load_model, egg_disk_utils.h:46-81): raw
TransformerModel and AdamModel bytes under the reference's names, "last" symlinks, and a resume that continues
bit-identically."""
import os

import numpy as np
import pytest

from common import REF_CONFIGS, load_pkg, make_case

pytestmark = pytest.mark.gpu


def test_checkpoint_files_and_resume(tmp_path):
    pkg = load_pkg()
    kw = REF_CONFIGS["tiny"]
    cfg, ocfg, model0, data = make_case(kw, data_len=30000)
    pop, S = kw["population_size"], kw["seq_len"]
    a = pkg.Context(cfg, 0, 0)
    a.upload_model(model0)
    a.set_dataset(data)
    for step in range(3):
        a.generation_host(None, step, 1000 + step, 0.5, None)
    d = str(tmp_path / "models")
    a.save_checkpoint(d, 3)
    mp, ap = os.path.join(d, "egg_step-00000003.model.bin"), os.path.join(d, "egg_step-00000003.adam.bin")
    assert np.array_equal(np.fromfile(mp, np.int8), a.download_model())
    assert np.array_equal(np.fromfile(ap, np.uint8), a.download_opt_state())
    lm, la = os.path.join(d, "egg_transformer_last.model.bin"), os.path.join(d, "egg_transformer_last.adam.bin")
    assert os.readlink(lm) == "egg_step-00000003.model.bin" and os.readlink(la) == "egg_step-00000003.adam.bin"
    a.save_checkpoint(d, 4)                                     # the links move on
    assert os.readlink(lm) == "egg_step-00000004.model.bin"

    b = pkg.Context(cfg, 0, 0)
    b.load_checkpoint(mp, ap)
    b.set_dataset(data)
    la_, lb_ = np.zeros(pop, np.int32), np.zeros(pop, np.int32)
    a.generation_host(None, 3, 2000, 0.5, la_)
    b.generation_host(None, 3, 2000, 0.5, lb_)
    assert (la_ == lb_).all()
    assert np.array_equal(a.download_model(), b.download_model())
    assert np.array_equal(a.download_opt_state(), b.download_opt_state())

    bad = str(tmp_path / "short.bin")
    open(bad, "wb").write(b"\0" * 100)
    with pytest.raises(pkg.EggError):
        b.load_checkpoint(bad)
    a.close(); b.close()
