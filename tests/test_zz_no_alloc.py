"""The allocation-free reconstruct entry point against the allocating one.

Some callers may not allocate device memory while they work (a worker with a fixed memory budget,
code inside a pool that forbids cudaMalloc, loops that cannot afford cudaMalloc's device-wide
synchronisation).  egg_update_reconstruct_noalloc serves them from a fixed buffer inside the library.
Its votes must equal egg_update_reconstruct's exactly (integer work) and the CPU oracle's, also on a
second call that reuses the buffer with a different shape; the call must leave the amount of free
device memory unchanged, and oversized requests must be refused."""
import numpy as np
import pytest

from common import cfg_pair, load_oracle, load_pkg

pytestmark = pytest.mark.gpu


def test_noalloc_reconstruct_equals_allocating_entry_point_twice():
    import torch
    pkg, O = load_pkg(), load_oracle()
    cfg, ocfg = cfg_pair(device_mask=3, population_size=2 * 1000)
    ctx = pkg.Context(cfg, 0, 2)
    rng = np.random.default_rng(11)
    cases = [  # (pairs, rows_k, cols_n, int8 fitness?)  -- the second call is smaller and ternary: stale bytes must not leak
        (1000, 256, 384, True),
        (300, 128, 256, False),
    ]
    for pairs, rows_k, cols_n, int8fit in cases:
        fit = (rng.integers(-127, 128, pairs) if int8fit else rng.integers(-1, 2, pairs)).astype(np.int32)
        d_fit = torch.from_numpy(fit).cuda()
        want = torch.zeros(rows_k * cols_n, dtype=torch.int32, device="cuda")
        got = torch.full((rows_k * cols_n,), -7, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        ctx.update_reconstruct(d_fit.data_ptr(), pairs, rows_k, cols_n, 402, 403, 1000, 2, want.data_ptr(), on_device=True)
        free_before = torch.cuda.mem_get_info()[0]
        ctx.update_reconstruct_noalloc(d_fit.data_ptr(), pairs, rows_k, cols_n, 402, 403, 1000, 2, int8fit, got.data_ptr())
        assert torch.cuda.mem_get_info()[0] == free_before, "the allocation-free call changed the free device memory"
        assert torch.equal(got, want), "votes differ in %d places" % int((got != want).sum())
        assert int(want.abs().max()) > 0
        oracle_votes = O.vote_matrix(ocfg, fit, rows_k, cols_n, 402, 403, 1000, 2)
        assert (got.cpu().numpy() == oracle_votes).all(), "votes differ from the CPU oracle's"
    # beyond the built-in buffer: (4096 + 4096) * 4096 bytes > 8 MiB
    big_fit = torch.zeros(4096, dtype=torch.int32, device="cuda")
    big_out = torch.zeros(16, dtype=torch.int32, device="cuda")
    with pytest.raises(pkg.EggError) as ei:
        ctx.update_reconstruct_noalloc(big_fit.data_ptr(), 4096, 4096, 4096, 0, 1, 0, 2, False, big_out.data_ptr())
    assert ei.value.code == pkg.EGG_E_INVALID and "scratch" in str(ei.value)
    ctx.close()
