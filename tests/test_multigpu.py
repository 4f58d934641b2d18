"""2-GPU run through the C ABI: pair-aligned population slices, one NCCL all-gather of fitness per
generation, replicated update.  Every rank must hold byte-identical weights and optimiser state, equal
to the single-GPU generation.  Skipped where fewer than two GPUs are visible."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from common import ROOT, load_pkg, make_case

pytestmark = pytest.mark.gpu
KW = dict(hidden_dim=256, n_layers=2, seq_len=32, population_size=64, device_mask=3)
SEED, LR, STEPS = 4242, 0.5, 3


def _rank_main(rank, world, ident, q, kw=None, shard=False):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    pkg = load_pkg()
    kw = kw or KW
    cfg, ocfg, model, data = make_case(kw, data_len=40000)
    ctx = pkg.Context(cfg, rank, 0)
    ctx.upload_model(model)
    ctx.set_dataset(data)
    ctx.comm_init(ident, rank, world)
    if shard:
        ctx.set_update_sharding(True)
    per = kw["population_size"] // world
    losses = np.zeros(per, np.int32)
    ups = []
    for step in range(STEPS):
        ups.append(ctx.generation_host(None, step, SEED + step, LR, losses))
    if shard:
        # back to the replicated update: the switch collects every parameter's state, so one more generation on
        # every rank must continue exactly where the owners left off
        ctx.set_update_sharding(False)
        ups.append(ctx.generation_host(None, STEPS, SEED + STEPS, LR, losses))
    q.put((rank, ctx.download_model().tobytes(), ctx.download_opt_state().tobytes(), losses.tobytes(), ups))
    ctx.close()


def test_two_gpu_generation_matches_single_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    pkg = load_pkg()
    cfg, ocfg, model, data = make_case(KW, data_len=40000)
    ctx = pkg.Context(cfg, 0, 0)
    ctx.upload_model(model)
    ctx.set_dataset(data)
    pop = KW["population_size"]
    losses = np.zeros(pop, np.int32)
    ups = [ctx.generation_host(None, step, SEED + step, LR, losses) for step in range(STEPS)]
    want_m, want_o = ctx.download_model().tobytes(), ctx.download_opt_state().tobytes()
    ctx.close()
    ident = pkg.nccl_unique_id()
    mpc = mp.get_context("spawn")
    q = mpc.Queue()
    procs = [mpc.Process(target=_rank_main, args=(r, 2, ident, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, mb, ob, lb, u in got:
        assert mb == want_m and ob == want_o, "rank %d diverged from the single-GPU generation" % rank
        assert u == ups
        per = pop // 2
        assert lb == losses[rank * per:(rank + 1) * per].tobytes()


@pytest.mark.parametrize("muon", [0, 1])
def test_sharded_update_matches_replicated_update(muon):
    """Every matrix updated by one rank and broadcast (egg_set_update_sharding): weights, change counts and the
    collected optimiser state must equal the single-GPU generation's byte for byte (AdamW), and with Muon too, where
    each matrix's Newton-Schulz runs on its owner with the same kernels as on one GPU."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    pkg = load_pkg()
    kw = dict(KW, use_muon=muon)
    cfg, ocfg, model, data = make_case(kw, data_len=40000)
    ctx = pkg.Context(cfg, 0, 0)
    ctx.upload_model(model)
    ctx.set_dataset(data)
    pop = kw["population_size"]
    losses = np.zeros(pop, np.int32)
    ups = [ctx.generation_host(None, step, SEED + step, LR, losses) for step in range(STEPS + 1)]
    want_m, want_o = ctx.download_model().tobytes(), ctx.download_opt_state().tobytes()
    with pytest.raises(pkg.EggError):
        ctx.set_update_sharding(True)            # no communicator
    ctx.close()
    ident = pkg.nccl_unique_id()
    mpc = mp.get_context("spawn")
    q = mpc.Queue()
    procs = [mpc.Process(target=_rank_main, args=(r, 2, ident, q, kw, True)) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, mb, ob, lb, u in got:
        assert mb == want_m, "rank %d: weights diverged from the single-GPU generation" % rank
        assert ob == want_o, "rank %d: collected optimiser state differs" % rank
        assert u == ups


def test_one_process_holds_contexts_on_two_gpus():
    """Kernel attributes (dynamic shared-memory limits, cluster occupancy) are per device: a process that evaluates on
    GPU 0 and then on GPU 1 must get the same losses from both, for the row-owning projections on one thread block
    (H 256) and on pairs (H 1024), the default attention and the sampling kernel's attribute path."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    pkg = load_pkg()
    for hidden, seq in ((256, 128), (1024, 128)):
        kw = dict(hidden_dim=hidden, n_layers=1, seq_len=seq, population_size=8, device_mask=3)
        cfg, ocfg, model, data = make_case(kw, data_len=40000, model_kind="random")
        out = []
        for dev in (0, 1):
            ctx = pkg.Context(cfg, dev, 0)
            ctx.upload_model(model)
            ctx.set_dataset(data)
            ctx.eval_chunk(SEED, seq, 0, 8)
            out.append(ctx.read_losses(0, 8))
            ctx.close()
        assert (out[0] == out[1]).all(), (hidden, out)
