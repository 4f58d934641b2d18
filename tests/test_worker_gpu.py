"""GPU: the worker loop with the library doing the GPU work (egg_worker_engine_from_ctx), against the reference's
coordinator on 127.0.0.1 (oracle/_ref/ref_coordinator_tiny: d-eggs/src/coordinator.cpp unmodified, built with a
stand-in logging header that posts nothing).  After a few steps the weights, the fp32 optimiser state and the
adaptive-noise overlays must be byte-identical to the same library driven directly through the same sequence
(evaluate every chunk, per-chunk fitness filter, one update with the step's learning rate, seed chain)."""
import numpy as np
import pytest

from common import DEGGS_CHUNK, DEGGS_CONFIGS, load_pkg, make_case
from test_worker_cpu import _coordinator, _stop

pytestmark = pytest.mark.gpu
STEPS = 3


def _fresh_ctx(pkg, cfg, model, data):
    ctx = pkg.Context(cfg, 0, 0)
    ctx.upload_model(model)
    ctx.set_dataset(data)
    ctx.upload_scales(np.full(pkg.scales_bytes(cfg), 64, np.int8))       # ADAPTIVE_NOISE_INIT, worker.cu:346
    return ctx


def test_worker_on_gpu_matches_direct_drive(tmp_path):
    pkg = load_pkg()
    kw = DEGGS_CONFIGS["tiny"]
    chunk = DEGGS_CHUNK["tiny"]
    cfg, ocfg, model, data = make_case(kw, data_len=50000)
    pop, S = kw["population_size"], kw["seq_len"]

    # direct drive
    ctx = _fresh_ctx(pkg, cfg, model, data)
    seed, updates = 42, []
    for step in range(STEPS):
        fit = []
        for c in range(pop // chunk):
            ctx.eval_chunk(seed, step * S, c * chunk, chunk)
            f, _ = pkg.deggs_chunk_fitness(ctx.read_losses(0, chunk), 1, 1.2, 1, 0.1)
            fit.append(f)
        ctx.write_fitness(np.concatenate(fit), 0)
        updates.append(ctx.apply_update(seed, pkg.learning_rate(step)))
        seed = pkg.next_seed(seed, step + 1)
    want = (ctx.download_model(), ctx.download_opt_state(), ctx.download_scales())
    ctx.close()
    assert (want[0] != model).any()

    # the same through the worker loop and the coordinator
    proc = _coordinator(tmp_path)
    try:
        ctx = _fresh_ctx(pkg, cfg, model, data)
        eng = pkg.worker_engine_from_ctx(ctx)
        rc, st = pkg.worker_run(pkg.worker_options(population_size=pop, chunk_size=chunk, stop_at_step=STEPS, wait_sleep_ms=10), eng)
        assert rc == 0, pkg.lib().egg_last_error()
        assert st.final_step == STEPS and st.final_seed == seed and st.chunks_done == STEPS * (pop // chunk)
        got = (ctx.download_model(), ctx.download_opt_state(), ctx.download_scales())
        ctx.close()
    finally:
        _stop(proc)
    assert (got[0] == want[0]).all() and (got[1] == want[1]).all() and (got[2] == want[2]).all()
