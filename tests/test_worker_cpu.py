"""CPU: the worker loop (egg_worker_run, the counterpart of d-eggs/src/worker.cu:390-717) against the reference's own
coordinator -- d-eggs/src/coordinator.cpp compiled unmodified into oracle/_ref/ref_coordinator_* with a stand-in for
its logging header, so that it posts nothing anywhere -- on 127.0.0.1.  The GPU work is replaced by host-side fakes:
what is tested here is the protocol, the control flow and the fault cases (a worker that goes silent, stale and
duplicate results, a late joiner), all made on the host."""
import os
import socket
import subprocess
import threading
import time

import numpy as np
import pytest

from common import ROOT, load_pkg

POP, CHUNK, SEQ = 128, 32, 16          # oracle/Makefile DEGGS_tiny: CHUNK_SIZE 32, POPULATION_SIZE = 8 * POPULATION_BATCH_SIZE
PORT = 12345                           # fixed in coordinator.cpp:26


def _coordinator(tmp_path, name="ref_coordinator_tiny"):
    exe = os.path.join(ROOT, "oracle", "_ref", name)
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/%s not built" % name)
    for _ in range(100):                # wait for the port to be free (a previous test's coordinator winding down)
        s = socket.socket()
        try:
            s.bind(("127.0.0.1", PORT))
            s.close()
            break
        except OSError:
            s.close()
            time.sleep(0.1)
    proc = subprocess.Popen([exe], cwd=str(tmp_path), stdout=open(os.path.join(str(tmp_path), "coordinator.out"), "w"),
                            stderr=subprocess.STDOUT)
    for _ in range(100):
        try:
            socket.create_connection(("127.0.0.1", PORT), timeout=0.2).close()
            return proc
        except OSError:
            time.sleep(0.05)
    proc.kill()
    pytest.fail("the coordinator did not start listening")


def _stop(proc):
    proc.terminate()
    try:
        proc.wait(timeout=5)
    except Exception:
        proc.kill()


def fake_losses(seed, step, member):
    x = (seed * 2654435761 + step * 40503 + member * 9973) & 0xFFFFFFFF
    x ^= x >> 15
    return 20000 + (x * 2246822519 & 0xFFFFFFFF) % 5000


class FakeEngine:
    """Deterministic stand-in for the GPU: losses are a hash of (seed, step, member); updates are recorded."""

    def __init__(self, pkg, delay=0.0):
        self.pkg = pkg
        self.updates = []               # (seed, lr, fitness array)
        self.evals = []                 # (seed, step, pop_offset)
        self.delay = delay

        def eval_chunk(_self, seed, step, pop_offset, count, out):
            if self.delay:
                time.sleep(self.delay)
            self.evals.append((seed, step, pop_offset))
            for i in range(count):
                out[i] = fake_losses(seed, step, pop_offset + i)
            return 0

        def apply_update(_self, fit, pairs, seed, lr, lr_bias, upd):
            arr = np.ctypeslib.as_array(fit, shape=(pairs,)).copy()
            self.updates.append((seed, lr, arr))
            assert abs(lr_bias - 0.1 * lr) < 1e-7
            upd[0] = 1000 + len(self.updates)
            return 0

        self._cb = (pkg.EVAL_CHUNK_FN(eval_chunk), pkg.APPLY_UPDATE_FN(apply_update))
        self.struct = pkg.WorkerEngine(None, self._cb[0], self._cb[1], pkg.GENERATE_FN())


def expected_fitness(pkg, seed, step):
    parts = []
    for c in range(POP // CHUNK):
        losses = np.array([fake_losses(seed, step, c * CHUNK + i) for i in range(CHUNK)], np.int32)
        fit, _ = pkg.deggs_chunk_fitness(losses, 1, 1.2, 1, 0.1)
        parts.append(fit)
    return np.concatenate(parts)


def test_single_worker_three_steps(tmp_path):
    pkg = load_pkg()
    proc = _coordinator(tmp_path)
    try:
        eng = FakeEngine(pkg)
        rc, st = pkg.worker_run(pkg.worker_options(population_size=POP, chunk_size=CHUNK, stop_at_step=3, wait_sleep_ms=10), eng.struct)
        assert rc == 0, pkg.lib().egg_last_error()
        assert st.final_step == 3 and st.updates_applied == 3 and st.chunks_done == 3 * (POP // CHUNK)
        seed = 42
        for step in range(3):
            useed, lr, fit = eng.updates[step]
            assert useed == seed and lr == pkg.learning_rate(step)
            assert (fit == expected_fitness(pkg, seed, step)).all(), "fitness of step %d as redistributed by the coordinator" % step
            seed = pkg.next_seed(seed, step + 1)                     # worker.cu:542, coordinator.cpp:406
        assert st.final_seed == seed
        assert sorted(e[2] for e in eng.evals if e[1] == 0) == [0, 32, 64, 96]
    finally:
        _stop(proc)
    rows = [l for l in open(os.path.join(str(tmp_path), "coordinator.log")) if l[0].isdigit()]
    assert len(rows) == 3
    want_loss = sum(fake_losses(42, 0, m) for m in range(POP)) / (POP * SEQ * 16.0)      # coordinator.cpp:337
    assert abs(float(rows[0].split(",")[2]) - want_loss) < 1e-3
    assert int(rows[1].split(",")[3]) == 1001 * 1                    # updates_count of the first update, reported once (worker.cu:701)


def test_two_workers_share_the_chunks_and_stay_in_step(tmp_path):
    pkg = load_pkg()
    proc = _coordinator(tmp_path)
    try:
        engines = [FakeEngine(pkg, delay=0.002), FakeEngine(pkg, delay=0.003)]
        out = [None, None]

        def run(i):
            out[i] = pkg.worker_run(pkg.worker_options(population_size=POP, chunk_size=CHUNK, stop_at_step=4, wait_sleep_ms=5), engines[i].struct)

        th = [threading.Thread(target=run, args=(i,)) for i in range(2)]
        [t.start() for t in th]
        [t.join(timeout=60) for t in th]
        for i in range(2):
            rc, st = out[i]
            assert rc == 0 and st.final_step == 4 and st.updates_applied == 4
        assert out[0][1].final_seed == out[1][1].final_seed
        for step in range(4):
            a, b = engines[0].updates[step], engines[1].updates[step]
            assert a[0] == b[0] and (a[2] == b[2]).all()
            assert (a[2] == expected_fitness(pkg, a[0], step)).all()
        done = out[0][1].chunks_done + out[1][1].chunks_done
        assert done >= 4 * (POP // CHUNK) and out[0][1].chunks_done > 0 and out[1][1].chunks_done > 0
    finally:
        _stop(proc)


def test_silent_worker_chunk_is_reassigned_after_the_straggler_timeout(tmp_path):
    """coordinator.cpp:243-254 re-queues a chunk whose result did not arrive in time.  The build used here is the
    reference source with its 90 s constant set to 1.5 s; the worker's result for chunk 1 of step 0 is dropped once on the
    host (before_result hook), as if that worker had gone silent."""
    pkg = load_pkg()
    proc = _coordinator(tmp_path, "ref_coordinator_tiny_fast")
    try:
        eng = FakeEngine(pkg)
        dropped = []

        def hook(_self, step, chunk):
            if step == 0 and chunk == 1 and not dropped:
                dropped.append(1)
                return 1
            return 0

        cb = pkg.BEFORE_RESULT_FN(hook)
        opts = pkg.worker_options(population_size=POP, chunk_size=CHUNK, stop_at_step=1, wait_sleep_ms=50)
        opts.before_result = cb
        t0 = time.time()
        rc, st = pkg.worker_run(opts, eng.struct)
        assert rc == 0 and st.final_step == 1
        assert st.results_dropped == 1 and st.waits > 0 and time.time() - t0 >= 1.4
        assert [e[2] for e in eng.evals if e[1] == 0].count(CHUNK) == 2          # chunk 1 was evaluated twice
        assert (eng.updates[0][2] == expected_fitness(pkg, 42, 0)).all()
    finally:
        _stop(proc)


def _raw_exchange(sock, pkg, msg, payload=b""):
    sock.sendall(pkg.wire_encode(msg) + payload)


def _raw_read(sock, pkg):
    hdr = b""
    while len(hdr) < 10:
        hdr += sock.recv(10 - len(hdr))
    import ctypes as C
    op, total = C.c_int(), C.c_uint32()
    assert pkg.lib().egg_wire_decode_header(hdr, C.byref(op), C.byref(total)) == 0
    body = b""
    while len(body) < total.value:
        body += sock.recv(total.value - len(body))
    m = pkg.WireMsg()
    assert pkg.lib().egg_wire_decode_body(op.value, body, len(body), C.byref(m)) == 0
    return m, body


def test_stale_and_duplicate_results_are_ignored_by_the_coordinator(tmp_path):
    """coordinator.cpp:308 (a result for another step) and :318 (a chunk already completed): raw protocol messages
    built with the library's own encoder.  Only the first valid result of a chunk may reach the redistributed fitness."""
    pkg = load_pkg()
    proc = _coordinator(tmp_path)
    try:
        s = socket.create_connection(("127.0.0.1", PORT))
        plus = pkg.ternary_pack(np.ones(CHUNK // 2, np.int32)).tobytes()
        minus = pkg.ternary_pack(-np.ones(CHUNK // 2, np.int32)).tobytes()

        def result(step, chunk, payload):
            m = pkg.WireMsg(opcode=1, payload_size=len(payload), seed=42, last_step=step, data_position=chunk * CHUNK, updates_count=0, sum_loss=100)
            _raw_exchange(s, pkg, m, payload)

        _raw_exchange(s, pkg, pkg.WireMsg(opcode=0, seed=42, last_step=0))
        resp, _ = _raw_read(s, pkg)
        assert resp.opcode == 2 and resp.payload_size == 0 and resp.data_position == 0
        result(0, 0, plus)
        result(0, 0, minus)             # duplicate of a completed chunk: ignored
        result(7, 1, minus)             # stale / foreign step: ignored
        for c in (1, 2, 3):
            result(0, c, plus)
        time.sleep(0.2)
        _raw_exchange(s, pkg, pkg.WireMsg(opcode=0, seed=42, last_step=0))
        upd, body = _raw_read(s, pkg)
        assert upd.payload_size == pkg.lib().egg_ternary_packed_size(POP // 2) and upd.last_step == 1
        fit = pkg.ternary_unpack(np.frombuffer(body[28:], np.uint8), POP // 2)
        assert (fit == 1).all()
        s.close()
    finally:
        _stop(proc)


def test_late_joiner_catches_up_from_the_fitness_history(tmp_path):
    """coordinator.cpp:185-209: a worker that reports an old step is sent the stored fitness vectors one step at a time."""
    pkg = load_pkg()
    proc = _coordinator(tmp_path)
    try:
        first = FakeEngine(pkg)
        rc, st = pkg.worker_run(pkg.worker_options(population_size=POP, chunk_size=CHUNK, stop_at_step=3, wait_sleep_ms=10), first.struct)
        assert rc == 0 and st.final_step == 3
        late = FakeEngine(pkg)
        rc2, st2 = pkg.worker_run(pkg.worker_options(population_size=POP, chunk_size=CHUNK, stop_at_step=3, wait_sleep_ms=10), late.struct)
        assert rc2 == 0 and st2.final_step == 3 and st2.updates_applied == 3 and st2.chunks_done == 0
        assert st2.final_seed == st.final_seed
        for a, b in zip(first.updates, late.updates):
            assert a[0] == b[0] and a[1] == b[1] and (a[2] == b[2]).all()
    finally:
        _stop(proc)


def test_worker_reports_a_coordinator_that_goes_away(tmp_path):
    pkg = load_pkg()
    proc = _coordinator(tmp_path)
    eng = FakeEngine(pkg, delay=0.01)
    killer = threading.Timer(0.3, lambda: _stop(proc))
    killer.start()
    rc, st = pkg.worker_run(pkg.worker_options(population_size=POP, chunk_size=CHUNK, recv_timeout_ms=2000, wait_sleep_ms=10), eng.struct)
    killer.join()
    assert rc == pkg.EGG_E_STATE
    assert "coordinator" in pkg.lib().egg_last_error().decode()
    # and one that was never there
    rc2, _ = pkg.worker_run(pkg.worker_options(population_size=POP, chunk_size=CHUNK, port=1), eng.struct)
    assert rc2 == pkg.EGG_E_STATE


def test_run_log_has_the_reference_columns(tmp_path):
    pkg = load_pkg()
    cfg = pkg.default_config(hidden_dim=256, n_layers=2, seq_len=32, population_size=64)
    path = os.path.join(str(tmp_path), "run.log")
    log = pkg.RunLog(path, cfg, num_gpus=8, vram_bytes_per_gpu=180 << 30)
    log.record(0, 5.25, 12345, 0.5)
    log.record(1, 5.125, 7, 0.25)
    log.close()
    lines = open(path).read().splitlines()
    assert lines[0] == "=== Training Run ===" and lines[1].startswith("Run Start:")
    assert lines[2] == "Hardware:        8 GPUs, 184320.00 MB VRAM/GPU"
    assert lines[3] == "Model Config:    Hidden=256, Head=64, Layers=2, SeqLen=32"
    i = lines.index("Step,RelTime,Loss,Updates,LR")                  # egg_disk_log.h:139
    r0, r1 = lines[i + 1].split(","), lines[i + 2].split(",")
    assert r0[0] == "0" and r0[2] == "5.2500" and r0[3] == "12345" and r0[4] == "0.500000"      # "%ld,%.4f,%.4f,%llu,%.6f", :222
    assert r1[0] == "1" and r1[2] == "5.1250" and r1[3] == "7" and r1[4] == "0.250000"
    pkg.RunLog(path, cfg).close()                                    # a second run appends after a blank line
    assert open(path).read().count("=== Training Run ===") == 2
